"""Regenerates the golden fixtures of this directory from the reference's own code. Run in a checkout that has the reference tree
mounted and `make -C oracle` done (it builds oracle/_ref/ref_host and oracle/_ref/ref_validate from the reference's sources
against a stub HIP runtime):

    python tests/golden/make_golden.py

Writes
  harness_inputs.json   sha256 of the input tensors the reference harness (tests/gpu/ref_host.cpp) generates per (data mode, shape),
                        its V descale, and the statistics line its fp64 `check` prints for an all-zero output (= statistics of |ref|)
  validate_cases.json   host-contract cases (valid launches and single-field mutations of them) with the verdict and message of the
                        reference's generated validate() (tests/gpu/generated/*_abi.h)
The fixtures travel with the repository; the reference tree and the binaries built from it do not.
"""
from __future__ import annotations

import hashlib
import json
import os
import random
import re
import struct
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402
from tests import contract_cases as CC  # noqa: E402

# B, H, HK, S, SK: the reference's gate shapes that are cheap on the CPU (tools/port_gate.sh:77-78) plus the small B1 H2 S256 case
SHAPES = [(1, 1, 1, 256, 256), (1, 2, 2, 512, 512), (1, 2, 2, 512, 2048), (3, 3, 3, 768, 1280), (1, 4, 4, 300, 512), (2, 8, 4, 700, 640),
          (1, 16, 4, 256, 1024), (1, 2, 2, 256, 1000), (2, 4, 4, 300, 129), (1, 8, 4, 512, 100), (1, 2, 2, 1024, 1088), (1, 4, 4, 77, 1),
          (1, 2, 1, 200, 1337), (1, 2, 2, 256, 256)]
ROWS = 8
LINE = re.compile(r"vendor kernel vs CPU: checked=(\d+) bad=(\d+) worst_err=(\S+) mean_err=(\S+) max\|ref\|=(\S+)")


def harness_inputs():
    out = []
    for mode in ("lcg", "uniform", "normal"):
        for (B, H, HK, S, SK) in SHAPES:
            with tempfile.TemporaryDirectory() as td:
                pre = os.path.join(td, "d")
                txt = O.run_ref_host(mode, B, H, S, SK, HK, rows=ROWS, dump_prefix=pre)
                m = LINE.search(txt)
                sha = {ext: hashlib.sha256(open(pre + "." + ext, "rb").read()).hexdigest() for ext in ("q", "k", "v", "qs", "ks")}
            out.append({"mode": mode, "B": B, "H": H, "HK": HK, "S": S, "SK": SK, "rows": ROWS, "sha256": sha,
                        "zero_output_check": {"checked": int(m.group(1)), "bad": int(m.group(2)), "worst_err": m.group(3), "mean_err": m.group(4),
                                              "max_ref": m.group(5)}})
            print("harness", mode, (B, H, HK, S, SK), m.group(0))
    return out


def validate_cases():
    rnd = random.Random(20260101)
    cases = CC.build_cases(rnd)
    lines = [CC.case_line(c) for c in cases]
    r = subprocess.run([os.path.join(ROOT, "oracle", "_ref", "ref_validate")], input="\n".join(lines) + "\n", capture_output=True, text=True, check=True)
    verdicts = r.stdout.splitlines()
    assert len(verdicts) == len(cases)
    print("validate cases:", len(cases), "valid:", sum(v == "1" for v in verdicts))
    # compact rows: [kernel, B, H, HK, S, SK, splits, mutations, verdict]
    return [[c["kernel"], c["B"], c["H"], c["HK"], c["S"], c["SK"], c["splits"], c["mut"], v] for c, v in zip(cases, verdicts)]


if __name__ == "__main__":
    json.dump(harness_inputs(), open(os.path.join(HERE, "harness_inputs.json"), "w"), indent=1)
    json.dump(validate_cases(), open(os.path.join(HERE, "validate_cases.json"), "w"), separators=(",", ":"))
