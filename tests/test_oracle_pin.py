"""The CPU oracle against the reference's own code: golden fixtures produced from the reference harness (tests/golden/make_golden.py),
its known-answer tables, and, where the harness binary built from the reference tree is present, live runs of it."""
import hashlib
import json
import os
import re
import tempfile

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(__file__), "golden")
HARNESS = json.load(open(os.path.join(GOLD, "harness_inputs.json")))


def _close(mine: float, printed: str, rel=2e-4):
    """`printed` is a number as the harness prints it: %.4e for the errors, %.4f for max|ref|."""
    want = float(printed)
    absolute = 6e-5 if "e" not in printed else 1e-12
    return abs(mine - want) <= rel * max(abs(want), 1e-30) + absolute


@pytest.mark.parametrize("case", HARNESS, ids=lambda c: f"{c['mode']}-B{c['B']}H{c['H']}HK{c['HK']}S{c['S']}SK{c['SK']}")
def test_generators_and_fp64_oracle_match_the_reference_harness(oracle, case):
    """Inputs: bit-identical to the harness's REF_INPUT_DUMP files (tests/gpu/ref_host.cpp:183-286). Oracle: the statistics of |ref| equal
    what the harness's `check` printed for an all-zero output (ref_host.cpp:438-471), to its printed precision."""
    inp = oracle.generate(case["mode"], case["B"], case["H"], case["S"], case["SK"], case["HK"])
    for ext, arr in (("q", inp.q), ("k", inp.k), ("v", inp.v), ("qs", inp.qs), ("ks", inp.ks)):
        assert hashlib.sha256(arr.tobytes()).hexdigest() == case["sha256"][ext], ext
    rows = case["rows"]
    ref = oracle.reference(inp, rows)
    st = oracle.compare(inp, np.zeros((inp.B, inp.S, inp.H, 128), np.uint16), ref, rows)
    z = case["zero_output_check"]
    assert st.checked == z["checked"] and st.bad == z["bad"]
    assert _close(st.worst_err, z["worst_err"]) and _close(st.mean_err, z["mean_err"]) and _close(st.max_ref, z["max_ref"])


def test_dispatch_known_answers(oracle):
    """crates/amdgpu-graph/tests/dispatch_rules.rs:7-15 and python/tests/test_unit.py:81-88."""
    table = {(4, 8, 2048, 2048): ("vs128", 0), (1, 8, 8192, 8192): ("vs128", 0), (2, 8, 2048, 2048): ("vs128", 0), (4, 8, 512, 512): ("t128", 0),
             (1, 8, 1024, 1024): ("t128", 0), (1, 4, 8192, 8192): ("kvsplit", 2), (1, 8, 2048, 2048): ("kvsplit", 4)}
    for shape, want in table.items():
        assert oracle.dispatch(*shape) == want


def test_e4m3_codec(oracle):
    t = oracle.e4m3_table()
    assert t[0x38] == 1.0 and t[0x7E] == 448.0 and t[0x7F] == 0.0 and t[0xFF] == 0.0 and t[0x01] == 2.0 ** -9 and t[0xB8] == -1.0
    L = oracle.lib()
    for b in range(256):   # every finite byte survives decode -> encode; -0 and the NaN encodings fold to 0
        if (b & 0x7F) == 0x7F:
            continue
        back = L.oracle_e4m3_encode(float(t[b]))
        assert back == b or (t[b] == 0 and back in (0x00,)), hex(b)
    assert L.oracle_e4m3_encode(1e9) == 126 and L.oracle_e4m3_encode(-1e9) == 0x80 | 126
    assert L.oracle_e4m3_encode(1.0625) == 0x38 and L.oracle_e4m3_encode(1.1875) == 0x3A   # ties go to the even byte


def test_bf16_round_trip(oracle):
    x = np.array([0.0, 1.0, -1.0, 0.1, 3.0e-5, 1.00390625, 1.01171875, 65504.0], np.float32)
    b = oracle.f32_to_bf16(x)
    L = oracle.lib()
    L.oracle_f32_to_bf16.restype = np.ctypeslib.ctypes.c_uint16
    L.oracle_f32_to_bf16.argtypes = [np.ctypeslib.ctypes.c_float]
    assert [int(v) for v in b] == [L.oracle_f32_to_bf16(float(v)) for v in x]
    assert np.all(np.abs(oracle.bf16_to_f32(b) - x) <= np.abs(x) * 2.0 ** -8)


@pytest.mark.parametrize("shape,splits", [((1, 2, 2, 256, 256), 0), ((1, 4, 4, 300, 512), 0), ((1, 2, 2, 512, 2048), 0), ((1, 2, 2, 512, 2048), 4),
                                          ((1, 2, 1, 200, 1337), 2)])
def test_recipe_path_error_level(oracle, shape, splits):
    """The CPU restatement of the reference kernels' arithmetic lands at the error level the reference publishes for its kernels on
    normal data (docs/perf-matrix.md:29-53: mean_err 1.74e-3 at SK 512, 1.25e-3 at 1024, ~9e-4 at 2048; bad = 0 everywhere)."""
    B, H, HK, S, SK = shape
    inp = oracle.generate("normal", B, H, S, SK, HK)
    rows = 16
    ref = oracle.reference(inp, rows)
    st = oracle.compare(inp, oracle.recipe_forward(inp, rows, splits), ref, rows)
    assert st.bad == 0
    published = 1.74e-3 * (512.0 / SK) ** 0.47   # the published table follows SK^-0.47 between 512 and 8192
    assert 0.6 * published < st.mean_err < 1.5 * published, (st, published)


def test_recipe_lazy_reference_equals_naive_softmax(oracle):
    """The lazily moved two-word reference changes only the scaling of P, never the result in exact arithmetic
    (crates/amdgpu-codegen/tests/functional_proofs.rs:41-69): the recipe path and the fp64 oracle agree to P's quantisation error
    on data that forces a rollback on every tile (lcg palette data) and on data that almost never does (normal)."""
    for mode, tol in (("lcg", 8e-3), ("normal", 2e-3)):
        inp = oracle.generate(mode, 1, 2, 128, 1024, 2)
        ref = oracle.reference(inp, 8)
        st = oracle.compare(inp, oracle.recipe_forward(inp, 8, 0), ref, 8)
        assert st.mean_err < tol and st.bad <= 2, (mode, st)


def test_combine_restatement_is_exact_for_equal_partials(oracle):
    """epilogue.rs:117-146: merging identical partials with identical log-sum-exp returns the partial; a split with lse = -inf-like
    weight contributes nothing."""
    rng = np.random.default_rng(1)
    rows, splits = 64, 4
    o = rng.standard_normal((1, rows, 128)).astype(np.float32)
    ohat = np.repeat(o, splits, 0)
    lse = np.full((splits, rows), 3.25, np.float32)
    out = oracle.combine_f32(ohat, lse, rows, splits)
    assert np.array_equal(out, oracle.f32_to_bf16(o[0]))
    lse[1:] = -1.0e30
    ohat[1:] = 1.0e3
    out = oracle.combine_f32(ohat, lse, rows, splits)
    assert np.array_equal(out, oracle.f32_to_bf16(o[0]))


@pytest.mark.skipif(not os.path.exists(os.path.join(os.path.dirname(os.path.dirname(__file__)), "oracle", "_ref", "ref_host")),
                    reason="the reference harness binary is only built where the reference tree is mounted")
def test_live_reference_harness_scores_the_oracle_output(oracle):
    """The harness's own `check` scores the oracle's bf16 output: only bf16 rounding is left, and its statistics equal oracle.compare's."""
    for mode, shape in (("normal", (1, 2, 2, 256, 256)), ("lcg", (2, 8, 4, 700, 640)), ("uniform", (1, 2, 1, 200, 1337))):
        B, H, HK, S, SK = shape
        inp = oracle.generate(mode, B, H, S, SK, HK)
        rows = 16
        ref = oracle.reference(inp, rows)
        out = np.zeros((B, S, H, 128), np.uint16)
        out[:, :min(rows, S)] = oracle.f32_to_bf16(ref.astype(np.float32)).transpose(0, 2, 1, 3)
        with tempfile.TemporaryDirectory() as td:
            f = os.path.join(td, "o.bin")
            out.tofile(f)
            txt = oracle.run_ref_host(mode, B, H, S, SK, HK, rows=rows, out_file=f)
        m = re.search(r"vendor kernel vs CPU: checked=(\d+) bad=(\d+) worst_err=(\S+) mean_err=(\S+) max\|ref\|=(\S+)", txt)
        st = oracle.compare(inp, out, ref, rows)
        assert int(m.group(2)) == 0 == st.bad
        assert _close(st.mean_err, m.group(4)) and _close(st.worst_err, m.group(3)) and _close(st.max_ref, m.group(5))
        assert st.mean_err <= 2.0 ** -8 * st.max_ref


def test_row_lists_select_the_same_rows_as_the_prefix_form(oracle):
    """The oracle, the recipe restatement and the gate statistics evaluated on an explicit list of query rows equal the reference's
    "first REF_ROWS rows" form (tests/gpu/ref_host.cpp:438-471) on those rows: the list only lets the GPU tests reach later query tiles."""
    import numpy as np
    inp = oracle.generate("normal", 1, 2, 300, 512, 2)
    rows = oracle.spread_rows(300)
    assert rows[0] == 0 and rows[-1] == 299 and 128 in rows and 256 in rows
    full = oracle.reference(inp, 300)
    some = oracle.reference(inp, rows)
    assert np.array_equal(some, full[:, :, rows])
    assert np.array_equal(oracle.reference(inp, list(range(16))), oracle.reference(inp, 16))
    assert np.array_equal(oracle.reference(inp, rows, causal=True), oracle.reference(inp, 300, causal=True)[:, :, rows])
    rec_full, rec_some = oracle.recipe_forward(inp, 300), oracle.recipe_forward(inp, rows)
    assert np.array_equal(rec_some[:, rows], rec_full[:, rows])
    a, b = oracle.compare(inp, rec_some, some, rows), oracle.compare(inp, rec_full, full[:, :, rows], rows)
    assert (a.checked, a.bad, a.worst_err, a.mean_err) == (b.checked, b.bad, b.worst_err, b.mean_err) and a.checked == len(rows) * 2 * 128
    with pytest.raises(RuntimeError):
        oracle.reference(inp, [300])
