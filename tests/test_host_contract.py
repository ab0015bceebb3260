"""The C ABI's host contract against the reference's generated one: struct layout, exported symbols, validate() verdicts and messages
(golden cases produced by the reference's own validate(), tests/golden/make_golden.py), dispatch and grids. No GPU needed."""
import ctypes as C
import json
import os
import re
import subprocess

import pytest

from tests import contract_cases as CC

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CASES = json.load(open(os.path.join(ROOT, "tests", "golden", "validate_cases.json")))


def test_library_loads_and_exports_every_declared_symbol(abi):
    lib = abi.load()
    header = open(os.path.join(ROOT, "include", "fmha_mxfp8_abi.h")).read()
    declared = set(re.findall(r"\b(fmha_mxfp8_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(abi.EXPORTS)
    for name in declared:
        assert getattr(lib, name) is not None, name


def test_kernel_table_matches_the_reference_json(abi):
    """kernel names, kernarg sizes and workgroup sizes of tests/gpu/generated/*_abi.json (656 / 656 / 648 / 36; 512 / 256 / 512 / 256)."""
    lib = abi.load()
    want = [("fmha_fwd_hd128_mxfp8_v3_vs128", 656, 512), ("fmha_fwd_hd128_mxfp8_v3_t128", 656, 256), ("fmha_fwd_hd128_mxfp8_v3_kvsplit", 648, 512),
            ("fmha_fwd_hd128_mxfp8_v3_kvsplit_combine8h", 36, 256)]
    for k, (name, size, wg) in enumerate(want):
        assert lib.fmha_mxfp8_kernel_name(k).decode() == name
        assert lib.fmha_mxfp8_kernarg_size(k) == size == C.sizeof(abi.ARGS_TYPES[k])
        assert lib.fmha_mxfp8_workgroup_size(k) == wg
    assert lib.fmha_mxfp8_kernel_name(4) is None and lib.fmha_mxfp8_kernarg_size(-1) == 0


def test_field_offsets_match_the_hand_abi(abi):
    """crates/amdc/tests/contract_host_truth.rs:192-213."""
    for name, off in CC.OFF.items():
        assert getattr(abi.KvSplitArgs, name).offset == off, name
        if not name.startswith("kvs_"):
            assert getattr(abi.AttnArgs, name).offset == off, name
    for name, off in (("ptr_o", 0), ("ptr_q", 0x10), ("ptr_k", 0x20), ("ptr_v", 0x30), ("ptr_q_descale", 0x200), ("ptr_k_descale", 0x210), ("ptr_v_descale", 0x220)):
        assert getattr(abi.AttnArgs, name).offset == off and getattr(abi.KvSplitArgs, name).offset == off
    for name, off in (("ptr_ohat", 0), ("ptr_lse", 8), ("ptr_out", 0x10), ("rows_total", 0x18), ("d", 0x1C), ("splits", 0x20)):
        assert getattr(abi.CombineArgs, name).offset == off


def _run_case(abi, row):
    kernel, B, H, HK, S, SK, splits, mut, expect = row
    args, sizes, grid, syms = CC.materialize({"kernel": kernel, "B": B, "H": H, "HK": HK, "S": S, "SK": SK, "splits": splits, "mut": mut})
    lib = abi.load()
    buf = C.create_string_buffer(args, len(args))
    bs = abi.BufferSizes(*sizes)
    sy = abi.Symbols(*syms)
    err = C.create_string_buffer(256)
    rc = lib.fmha_mxfp8_validate(kernel, buf, C.byref(bs), abi.grid3(*grid), C.byref(sy), err, 256)
    return ("1" if rc == 0 else "0 " + err.value.decode()), rc


def test_validate_agrees_with_the_reference_on_every_golden_case(abi):
    """Same verdict, same GV-HOST-* code, same message, same first-failure order as the reference's generated validate()."""
    bad = []
    for row in CASES:
        got, rc = _run_case(abi, row)
        if got != row[-1]:
            bad.append((row, got))
        if rc:
            assert abi.ERROR_CLASSES[rc] == got.split(":")[0][2:]
    assert not bad, bad[:5]


@pytest.mark.skipif(not os.path.exists(os.path.join(ROOT, "oracle", "_ref", "ref_validate")), reason="needs the reference tree (oracle/_ref)")
def test_validate_agrees_with_the_live_reference_on_random_cases(abi):
    import random
    rnd = random.Random(7)
    cases = CC.build_cases(rnd)
    rnd.shuffle(cases)
    cases = cases[:600]
    r = subprocess.run([os.path.join(ROOT, "oracle", "_ref", "ref_validate")], input="\n".join(CC.case_line(c) for c in cases) + "\n",
                       capture_output=True, text=True, check=True)
    for c, want in zip(cases, r.stdout.splitlines()):
        got, _ = _run_case(abi, [c["kernel"], c["B"], c["H"], c["HK"], c["S"], c["SK"], c["splits"], c["mut"], want])
        assert got == want, (c, got, want)


def test_dispatch_matches_the_reference_rule(abi, oracle):
    """Known answers (crates/amdgpu-graph/tests/dispatch_rules.rs:7-15) and a sweep against the CPU restatement."""
    from amdgpu_rustdsl_b200 import select_path
    assert select_path(4, 8, 2048, 2048) == ("vs128", 0)
    assert select_path(1, 8, 8192, 8192)[0] == "vs128"
    assert select_path(2, 8, 2048, 2048) == ("vs128", 0)
    assert select_path(4, 8, 512, 512) == ("t128", 0)
    assert select_path(1, 8, 1024, 1024) == ("t128", 0)
    assert select_path(1, 4, 8192, 8192) == ("kvsplit", 2)
    assert select_path(1, 8, 2048, 2048) == ("kvsplit", 4)
    for B in (1, 2, 3, 16):
        for H in (1, 2, 8, 64):
            for S in (1, 77, 256, 300, 2048, 8192):
                for SK in (1, 100, 129, 1337, 2048, 4096, 131072):
                    assert select_path(B, H, S, SK) == oracle.dispatch(B, H, S, SK)


def test_grid_helper(abi):
    """grid() of the generated headers (…_kvsplit_abi.h:234) and the combine grid of the harness (tests/gpu/ref_host.cpp:510-515)."""
    lib = abi.load()
    for kernel, rows in ((0, 256), (1, 128), (2, 256)):
        args, _, grid, syms = CC.materialize({"kernel": kernel, "B": 2, "H": 8, "HK": 4, "S": 700, "SK": 640, "splits": 4, "mut": []})
        g = abi.grid3(0, 0, 0)
        sy = abi.Symbols(*syms)
        assert lib.fmha_mxfp8_grid(kernel, C.create_string_buffer(args, len(args)), C.byref(sy), g) == 0
        assert list(g) == grid == [-(-700 // rows), 8, 2 * (4 if kernel == 2 else 1)]
    args, _, grid, _ = CC.materialize({"kernel": 3, "B": 2, "H": 8, "HK": 4, "S": 700, "SK": 640, "splits": 4, "mut": []})
    g = abi.grid3(0, 0, 0)
    assert lib.fmha_mxfp8_grid(3, C.create_string_buffer(args, len(args)), None, g) == 0
    assert list(g) == grid


def test_python_entry_rejects_bad_shapes_like_the_reference():
    """python/amdgpu_jit/ops.py:101-111: head dim 128, H a power-of-two multiple (<= 16) of HK."""
    import torch
    from amdgpu_rustdsl_b200 import fmha_fwd_mxfp8
    q = torch.zeros(1, 4, 6, 128, dtype=torch.uint8)
    k = torch.zeros(1, 4, 2, 128, dtype=torch.uint8)
    with pytest.raises(ValueError):
        fmha_fwd_mxfp8(q, k, k, q, q, q, q)   # gqa 3 is not a power of two
    q = torch.zeros(1, 4, 2, 64, dtype=torch.uint8)
    with pytest.raises(ValueError):
        fmha_fwd_mxfp8(q, q, q, q, q, q, q)   # head dim 64


def test_launch_refuses_the_unimplemented_v_block_scales(abi):
    """Per-32-key V scales are declared in the pad bytes of the argument block (ext_flags bit 0) but no kernel implements them: the launch
    refuses such a block before it touches the device instead of ignoring the flag."""
    lib = abi.load()
    for kernel in (0, 1, 2):
        args, _, grid, _ = CC.materialize({"kernel": kernel, "B": 1, "H": 2, "HK": 2, "S": 256, "SK": 512, "splits": 2, "mut": []})
        buf = bytearray(args)
        buf[0x058:0x05C] = (abi.FLAG_V_BLOCKSCALE).to_bytes(4, "little")
        g = abi.grid3(*grid)
        raw = (C.c_char * len(buf)).from_buffer(buf)
        assert lib.fmha_mxfp8_launch(kernel, raw, g, None) == 6   # FMHA_MXFP8_E_ARG


def test_workspace_keys_never_mix_devices_or_streams():
    """The kvsplit workspace of the Python entry is per (device, stream): the default stream's handle is 0 on every GPU, so a key
    without the device would hand one GPU's partial buffer to a launch on another."""
    torch = pytest.importorskip("torch")
    from amdgpu_rustdsl_b200 import ops
    keys = {ops._ws_key(name, torch.device("cuda", d), st) for name in ("ohat", "lse") for d in (0, 1, 7) for st in (0, 0x7F001234)}
    assert len(keys) == 2 * 3 * 2
    assert ops._ws_key("ohat", torch.device("cuda", 0), 0) != ops._ws_key("ohat", torch.device("cuda", 1), 0)
