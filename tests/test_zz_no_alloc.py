"""The kvsplit entry that keeps its partials in the library's fixed device array (fmha_mxfp8_kvsplit_static_scratch), through the C ABI:
same bytes as the regular entry with a caller-owned workspace, on two calls in a row (the array is reused), and a clear refusal past
the array's size. Named to be collected last, so that it also runs after every other test has used the device."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def _problem(abi, inp, q, k, v, qs, ks, vs, out, ws_o=None, ws_l=None):
    return abi.Problem(B=inp.B, H=inp.H, HK=inp.HK, S=inp.S, SK=inp.SK, q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), q_descale=qs.data_ptr(),
                       k_descale=ks.data_ptr(), v_descale=vs.data_ptr(), out=out.data_ptr(), q_descale_bytes=qs.numel(), k_descale_bytes=ks.numel(),
                       v_descale_bytes=4096, ws_ohat=ws_o.data_ptr() if ws_o is not None else None, ws_lse=ws_l.data_ptr() if ws_l is not None else None,
                       ws_ohat_bytes=ws_o.numel() if ws_o is not None else 0, ws_lse_bytes=ws_l.numel() if ws_l is not None else 0, v_blockscale=None, flags=0)


def _bytes(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.mark.parametrize("shape,splits", [((1, 2, 2, 512, 2048), 8), ((1, 8, 4, 1024, 2048), 4), ((2, 4, 4, 300, 1337), 2)],
                         ids=["B1H2S512SK2048x8", "B1H8HK4S1024SK2048x4", "B2H4S300SK1337x2"])
def test_static_scratch_entry_matches_the_workspace_entry_twice(oracle, abi, shape, splits):
    lib = abi.load()
    B, H, HK, S, SK = shape
    inp = oracle.generate("normal", B, H, S, SK, HK)
    dev = "cuda"
    q, k, v, qs, ks = (torch.from_numpy(a).to(dev) for a in (inp.q, inp.k, inp.v, inp.qs, inp.ks))
    vs = torch.zeros(1024, dtype=torch.float32, device=dev)
    vs[0] = inp.vdescale
    rows_total = B * S * H
    assert rows_total * splits <= abi.STATIC_SCRATCH_MAX_ROW_SPLITS
    err = C.create_string_buffer(256)

    # the existing entry, workspace owned by the caller
    ws_o = torch.empty(splits * rows_total * 512, dtype=torch.uint8, device=dev)
    ws_l = torch.empty(splits * rows_total * 4, dtype=torch.uint8, device=dev)
    want_t = torch.full((B, S, H, 128), float("nan"), dtype=torch.bfloat16, device=dev)
    pr = _problem(abi, inp, q, k, v, qs, ks, vs, want_t, ws_o, ws_l)
    assert lib.fmha_mxfp8_auto(C.byref(pr), abi.KVSPLIT, splits, None, None, None, err, 256) == 0, err.value
    torch.cuda.synchronize()
    want = _bytes(want_t)
    assert np.isfinite(oracle.bf16_to_f32(want)).all()

    # the new entry: no workspace in the problem at all, two calls in a row into poisoned outputs
    for call in range(2):
        got_t = torch.full((B, S, H, 128), float("nan"), dtype=torch.bfloat16, device=dev)
        pr2 = _problem(abi, inp, q, k, v, qs, ks, vs, got_t)
        torch.cuda.synchronize()
        free_before, used_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
        rc = lib.fmha_mxfp8_kvsplit_static_scratch(C.byref(pr2), splits, None, err, 256)
        assert rc == 0, (call, err.value)
        torch.cuda.synchronize()
        if call == 1:   # the warmed-up call takes no device memory from the driver or from torch
            assert torch.cuda.mem_get_info()[0] == free_before and torch.cuda.memory_allocated() == used_before
        assert np.array_equal(_bytes(got_t), want), f"call {call} differs from the workspace entry"

    from amdgpu_rustdsl_b200 import device_status
    assert device_status() == 0


def test_static_scratch_entry_refuses_what_does_not_fit(abi):
    lib = abi.load()
    err = C.create_string_buffer(256)
    dummy = torch.zeros(16, dtype=torch.uint8, device="cuda")
    # 8 splits x 16384 rows = 131072 row-splits: twice the array; refused before any launch, so the dummy pointers are never touched
    pr = abi.Problem(B=1, H=8, HK=8, S=2048, SK=2048, q=dummy.data_ptr(), k=dummy.data_ptr(), v=dummy.data_ptr(), q_descale=dummy.data_ptr(),
                     k_descale=dummy.data_ptr(), v_descale=dummy.data_ptr(), out=dummy.data_ptr(), q_descale_bytes=16, k_descale_bytes=16,
                     v_descale_bytes=16, ws_ohat=None, ws_lse=None, ws_ohat_bytes=0, ws_lse_bytes=0, v_blockscale=None, flags=0)
    rc = lib.fmha_mxfp8_kvsplit_static_scratch(C.byref(pr), 8, None, err, 256)
    assert rc == abi.E_EXTENT if hasattr(abi, "E_EXTENT") else rc == 1
    assert b"static scratch too small" in err.value and b"131072" in err.value and b"65536" in err.value
    assert lib.fmha_mxfp8_kvsplit_static_scratch(C.byref(pr), 3, None, err, 256) == 6 and b"splits" in err.value
    assert lib.fmha_mxfp8_kvsplit_static_scratch(None, 4, None, err, 256) == 6
