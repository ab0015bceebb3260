"""The split kernel with the merge of the partials built in (extension; the reference's "last arriver" combine, tests/gpu/ref_host.cpp:489-497,
docs/last-arriver-memory-model.md, which the reference measured and did not adopt): the CTA that stores the last partial of a 128-row block
merges the block with combine8h's arithmetic. The output must be the bytes of the two-kernel form, the arrival counters must be zero again
after every launch, and the oracle's gate must hold."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

# (B, H, S, SK, gqa, splits): the forced-split headline shape, ragged rows and keys, one row block under 128 rows, batches, grouped heads,
# V block scales are covered below
CASES = [(1, 8, 8192, 8192, 1, 8), (1, 4, 300, 1337, 2, 2), (2, 8, 700, 1408, 2, 4), (3, 3, 768, 1280, 1, 2), (1, 2, 512, 2048, 1, 8), (1, 4, 77, 2048, 1, 4),
         (4, 8, 128, 1024, 4, 8)]


def _dev(inp):
    d = {n: torch.from_numpy(getattr(inp, n)).cuda() for n in ("q", "k", "v", "qs", "ks")}
    d["vs"] = torch.zeros(1024, dtype=torch.float32, device="cuda")
    d["vs"][0] = inp.vdescale
    return d


def _run(d, inp, splits, fused, vscale=None):
    from amdgpu_rustdsl_b200 import fmha_fwd_mxfp8
    out = torch.full((inp.B, inp.S, inp.H, 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    ran = fmha_fwd_mxfp8(d["q"], d["k"], d["v"], d["qs"], d["ks"], d["vs"], out, path="kvsplit", splits=splits, fused_combine=fused, v_blockscale=vscale)
    torch.cuda.synchronize()
    assert ran == ("kvsplit", splits)
    return out.view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.mark.parametrize("case", CASES, ids=lambda c: "B%dH%dS%dSK%dg%dx%d" % c)
def test_fused_merge_gives_the_two_kernel_bytes(oracle, case):
    from amdgpu_rustdsl_b200 import device_status, ops
    B, H, S, SK, g, splits = case
    inp = oracle.generate("normal", B, H, S, SK, H // g)
    d = _dev(inp)
    want = _run(d, inp, splits, False)
    for call in range(3):   # the counters are cleared once, when the workspace is made: every later call relies on the one before
        got = _run(d, inp, splits, True)
        assert np.array_equal(got, want), (case, call, int((got != want).sum()))
    key = ops._ws_key("fused_counters", d["q"].device, torch.cuda.current_stream().cuda_stream)
    assert int(ops._workspace[key].view(torch.int32).abs().sum()) == 0
    rows = oracle.spread_rows(S) if S > 256 else min(S, 64)
    ref = oracle.reference(inp, rows)
    ours = oracle.compare(inp, got, ref, rows)
    yard = oracle.compare(inp, oracle.recipe_forward(inp, rows, 0), ref, rows)
    assert ours.bad == 0 and ours.mean_err <= 1.10 * yard.mean_err and ours.worst_err <= 2e-2, (ours, yard)
    assert device_status() == 0


def test_fused_merge_with_v_block_scales(oracle):
    inp = oracle.generate("normal", 1, 4, 640, 2048, 4, v_blockscale=True)
    d = _dev(inp)
    vsc = torch.from_numpy(inp.vscale).cuda()
    want = _run(d, inp, 4, False, vsc)
    assert np.array_equal(_run(d, inp, 4, True, vsc), want)


def test_fused_merge_through_the_one_call_entry(oracle, abi):
    """fmha_mxfp8_auto with the flag: counters behind the f16 partials, cleared by the entry itself, so an uninitialised workspace is fine."""
    lib = abi.load()
    B, H, S, SK, splits = 2, 4, 600, 4096, 8
    inp = oracle.generate("normal", B, H, S, SK)
    d = _dev(inp)
    want = _run(d, inp, splits, False)
    rows_total = B * S * H
    ws_o = torch.full((splits * rows_total * 512,), 0xA5, dtype=torch.uint8, device="cuda")   # garbage where the counters will be
    ws_l = torch.empty(splits * rows_total * 4, dtype=torch.uint8, device="cuda")
    out = torch.zeros(B, S, H, 128, dtype=torch.bfloat16, device="cuda")
    pr = abi.Problem(B=B, H=H, HK=H, S=S, SK=SK, q=d["q"].data_ptr(), k=d["k"].data_ptr(), v=d["v"].data_ptr(), q_descale=d["qs"].data_ptr(),
                     k_descale=d["ks"].data_ptr(), v_descale=d["vs"].data_ptr(), out=out.data_ptr(), q_descale_bytes=d["qs"].numel(),
                     k_descale_bytes=d["ks"].numel(), v_descale_bytes=4096, ws_ohat=ws_o.data_ptr(), ws_lse=ws_l.data_ptr(),
                     ws_ohat_bytes=ws_o.numel(), ws_lse_bytes=ws_l.numel(), v_blockscale=None, flags=abi.FLAG_FUSED_COMBINE)
    err = C.create_string_buffer(256)
    for _ in range(2):
        out.zero_()
        assert lib.fmha_mxfp8_auto(C.byref(pr), abi.KVSPLIT, splits, None, None, None, err, 256) == 0, err.value
        torch.cuda.synchronize()
        assert np.array_equal(out.view(torch.int16).cpu().numpy().view(np.uint16), want)
    # the flag does nothing on an unsplit path
    out.zero_()
    assert lib.fmha_mxfp8_auto(C.byref(pr), abi.VS128, 0, None, None, None, err, 256) == 0, err.value
    torch.cuda.synchronize()
    assert np.isfinite(oracle.bf16_to_f32(out.view(torch.int16).cpu().numpy().view(np.uint16))).all()


def test_fused_merge_refusals(oracle, abi):
    """No counters, f32 partials: refused before anything is launched."""
    from amdgpu_rustdsl_b200 import ops
    lib = abi.load()
    inp = oracle.generate("normal", 1, 2, 256, 1024)
    d = _dev(inp)
    out = torch.zeros(1, 256, 2, 128, dtype=torch.bfloat16, device="cuda")
    rows_total = 256 * 2
    ohat = torch.empty(2 * rows_total * 512, dtype=torch.uint8, device="cuda")
    lse = torch.empty(2 * rows_total * 4, dtype=torch.uint8, device="cuda")
    cnt = torch.zeros(16, dtype=torch.int32, device="cuda")
    for flags, counters in ((abi.FLAG_FUSED_COMBINE, None), (abi.FLAG_FUSED_COMBINE | abi.FLAG_F32_PARTIALS, cnt)):
        a = ops.fill_common(abi.KvSplitArgs(), d["q"], d["k"], d["v"], d["qs"], d["ks"], d["vs"], out, 1, 256, 2, 1024, 2, flags)
        a.ptr_ohat, a.ptr_lse, a.kvs_splits, a.kvs_rows_total = ohat.data_ptr(), lse.data_ptr(), 2, rows_total
        a.ext_ptr_fused_counters = counters.data_ptr() if counters is not None else None
        assert lib.fmha_mxfp8_launch(abi.KVSPLIT, C.byref(a), abi.grid3(1, 2, 2), None) == 6
    torch.cuda.synchronize()
