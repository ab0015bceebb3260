"""V with one E8M0 scale per 32 keys and column (extension: the reference's V has one f32 descale per tensor, README.md:40,
crates/amdgpu-stage/src/attention/block3.rs:145): P V then runs as a block-scaled MMA like Q K^T. Checked against the fp64 oracle on the
inputs dequantised with their block scales. The reference has no kernel arithmetic for this mode, so the yardstick of the mean-error
gate is the reference path's error on the same samples quantised its own way (scalar V descale): the P quantisation, which dominates
the error, is the same in both modes."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

GATE_SHAPES = [(1, 1, 256, 256, 1), (1, 2, 512, 512, 1), (2, 4, 1024, 1024, 1), (1, 8, 2048, 2048, 1), (1, 2, 512, 2048, 1), (3, 3, 768, 1280, 1),
               (1, 4, 300, 512, 1), (2, 8, 700, 640, 2), (1, 16, 256, 1024, 4), (1, 2, 256, 1000, 1), (2, 4, 300, 129, 1), (1, 8, 512, 100, 2),
               (1, 2, 1024, 1088, 1), (1, 4, 77, 1, 1), (1, 2, 200, 1337, 2), (4, 8, 2048, 2048, 1)]


def _run(inp, vscale=None, path="auto", splits=None):
    from amdgpu_rustdsl_b200 import fmha_fwd_mxfp8
    d = {n: torch.from_numpy(getattr(inp, n)).cuda() for n in ("q", "k", "v", "qs", "ks")}
    vs = torch.zeros(1024, dtype=torch.float32, device="cuda")
    vs[0] = inp.vdescale
    out = torch.full((inp.B, inp.S, inp.H, 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    ran = fmha_fwd_mxfp8(d["q"], d["k"], d["v"], d["qs"], d["ks"], vs, out, path=path, splits=splits,
                         v_blockscale=torch.from_numpy(vscale).cuda() if vscale is not None else None)
    torch.cuda.synchronize()
    return ran, out.view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.mark.parametrize("shape", GATE_SHAPES, ids=lambda s: "B%dH%dS%dSK%dg%d" % s)
def test_v_block_scales_against_the_oracle(oracle, shape):
    from amdgpu_rustdsl_b200 import device_status
    B, H, S, SK, g = shape
    rows = oracle.spread_rows(S) if S > 256 else 64
    plain = oracle.generate("normal", B, H, S, SK, H // g)
    ref_plain = oracle.reference(plain, rows)
    yard = oracle.compare(plain, oracle.recipe_forward(plain, rows, 0), ref_plain, rows)
    _, out_plain = _run(plain)
    inp = oracle.generate("normal", B, H, S, SK, H // g, v_blockscale=True)
    assert np.array_equal(inp.q, plain.q) and np.array_equal(inp.k, plain.k) and not np.array_equal(inp.v, plain.v)
    ref = oracle.reference(inp, rows)   # dequantises V with its block scales
    ntiles = -(-SK // 128)
    for path, splits in (("auto", None), ("vs128", None), ("kvsplit", 2)):
        if splits and (splits - 1) * (-(-ntiles // splits)) >= ntiles:
            continue
        _, out = _run(inp, inp.vscale, path, splits)
        ours = oracle.compare(inp, out, ref, rows)
        assert ours.bad == 0 and ours.mean_err <= 1.10 * yard.mean_err and ours.worst_err <= 2e-2, (path, splits, ours, yard)
        assert np.isfinite(oracle.bf16_to_f32(out)).all()
    # the reference's mode is untouched by the extension: same bytes as before for the scalar-descale inputs
    _, again = _run(plain)
    assert np.array_equal(again, out_plain)
    assert device_status() == 0
