"""Python entry of the MXFP8 attention forward path: the same call as the reference's ``amdgpu_jit.fmha_fwd_mxfp8``
(python/amdgpu_jit/ops.py:88-143) and ``select_path`` (ops.py:61-66), over the sm_100a kernels behind the C ABI.

PyTorch is used only as the owner of device memory and streams; every launch goes through ``fmha_mxfp8_validate`` +
``fmha_mxfp8_launch`` of the shared library, exactly as the reference goes through the generated ``validate`` + ``launch``.
"""
from __future__ import annotations

import ctypes as C
import math

from . import _abi
from ._abi import COMBINE8H, KVSPLIT, PATH_IDS, PATH_NAMES, T128, VS128, ContractError

D = 128
Q_SLACK_ROWS = 512   # zeroed slack behind the Q scales, in rows of H*4 bytes (tests/gpu/ref_host.cpp:197)
K_SLACK_ROWS = 640   # same for the K scales (ref_host.cpp:197); note the contract counts it in H, not HK


def select_path(B: int, H: int, S: int, SK: int):
    """The MXFP8 prefill dispatch ``mxfp8_prefill_path`` (crates/amdgpu-graph/src/dispatch.rs:494-511): returns (path, splits)."""
    lib = _abi.load()
    path, splits = C.c_int(0), C.c_uint32(0)
    lib.fmha_mxfp8_dispatch(B, H, S, SK, C.byref(path), C.byref(splits))
    return PATH_NAMES[path.value], int(splits.value)


_workspace = {}


def _ws_key(name, device, stream):
    """Workspaces are per (device, stream): stream handle 0 (the default stream) exists on every device."""
    return (name, device.index if device.index is not None else -1, int(stream))


# Calls already made, by their tensors' addresses, shapes and options: the kernels, filled argument blocks and grids they came to. A call
# with the same key (a layer run step after step on the same buffers) replays them without building and validating the blocks again
# (20 us of host time per call without, 8 with; the smallest shapes are host-bound). Entries die with the workspaces they point into.
_calls = {}
_ws_generation = 0


def _ws(name, nbytes, device, stream, zero=False):
    """Grow-only per-device, per-stream workspace for the KV-split partials (the reference's ``_ws``, ops.py:72-85, which frees the old
    buffer with a synchronising ``hipFree``). Here the old buffer goes back to torch's caching allocator, which only orders its reuse
    against torch's own current stream: a split or combine still running on ``stream`` is therefore waited for first."""
    import torch
    key = _ws_key(name, device, stream)
    buf = _workspace.get(key)
    if buf is None or buf.numel() < nbytes:
        global _ws_generation
        _ws_generation += 1   # remembered calls hold the old buffers' addresses
        if buf is not None:
            (torch.cuda.ExternalStream(int(stream), device=device) if stream else torch.cuda.default_stream(device)).synchronize()
        if zero:   # cleared once; its users leave it cleared. The fill runs on torch's current stream: it must be done before `stream` uses it
            buf = _workspace[key] = torch.zeros(nbytes, dtype=torch.uint8, device=device)
            torch.cuda.current_stream(device).synchronize()
        else:
            buf = _workspace[key] = torch.empty(nbytes, dtype=torch.uint8, device=device)
    return buf


def _nbytes(t):
    return t.numel() * t.element_size()


def _check_launch(lib, kernel, args, sizes, grid, syms, stream, check, record=None):
    if record is not None:
        record.append((kernel, args, grid))
    if check:
        err = C.create_string_buffer(256)
        rc = lib.fmha_mxfp8_validate(kernel, C.byref(args), C.byref(sizes), grid, C.byref(syms) if syms is not None else None, err, 256)
        if rc:
            raise ContractError(rc, err.value.decode())
    rc = lib.fmha_mxfp8_launch(kernel, C.byref(args), grid, C.c_void_p(stream))
    if rc:
        raise RuntimeError(f"fmha_mxfp8_launch({lib.fmha_mxfp8_kernel_name(kernel).decode()}) failed with code {rc}")


def fill_common(a, q, k, v, q_scale, k_scale, v_scale, out, B, S, H, SK, HK, flags=0, v_blockscale=None, lse=None):
    """Fills the fields shared by the three attention argument blocks (ops.py:117-121 builds the same dictionary)."""
    a.ptr_o, a.ptr_q, a.ptr_k, a.ptr_v = out.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr()
    a.s_seq_len, a.s_Seqs, a.s_Hs, a.s_Bs = S, H * D, D, S * H * D
    a.s_gqa = H // HK
    a.s_k_Seqs, a.s_k_Hs, a.s_k_Bs = HK * D, D, SK * HK * D
    a.s_kv_seq_len, a.s_q_head_num = SK, H
    a.s_v_Seqs, a.s_v_Hs, a.s_v_Bs = HK * D, D, SK * HK * D
    a.s_o_Seqs, a.s_o_Hs, a.s_o_Bs = H * D * 2, D * 2, S * H * D * 2
    a.ptr_q_descale, a.ptr_k_descale, a.ptr_v_descale = q_scale.data_ptr(), k_scale.data_ptr(), v_scale.data_ptr()
    a.s_descale_q_Bs, a.s_descale_q_Hs = S * H * 4, 4
    a.s_descale_k_Bs, a.s_descale_k_Hs = SK * HK * 4, 4
    a.ext_flags = flags | (_abi.FLAG_V_BLOCKSCALE if v_blockscale is not None else 0)
    a.ext_ptr_v_blockscale = v_blockscale.data_ptr() if v_blockscale is not None else None
    a.ext_ptr_lse = lse.data_ptr() if lse is not None else None
    return a


def fmha_fwd_mxfp8(q, k, v, q_scale, k_scale, v_scale, out, *, path="auto", splits=None, stream=None, check=True, flags=0,
                   v_blockscale=None, lse=None, causal=False, fused_combine=False):
    """MXFP8 attention forward, head dim 128: ``out = softmax2(q k^T) v`` with E8M0 1x32 scales on q and k and a scalar f32 V descale.

    q        [B, S, H, 128]  e4m3 bytes (uint8 or float8_e4m3fn)      k, v  [B, SK, HK, 128]  (H = gqa * HK, gqa a power of two <= 16)
    q_scale  E8M0 bytes [B, S, H, 4] followed by the contract's zeroed slack (512 * H * 4 bytes), as one flat uint8 buffer
    k_scale  E8M0 bytes [B, SK, HK, 4] followed by 640 * H * 4 bytes of slack
    v_scale  f32 buffer of at least 4096 bytes, element 0 is the V descale
    out      [B, S, H, 128]  bf16
    path     "auto" | "vs128" | "t128" | "kvsplit" (splits in {2, 4, 8}).  Returns (path, splits) like the reference.
    fused_combine  extension: on the kvsplit path the split kernel also merges the partials (the CTA that stores a row block's last partial
             does it), so no combine kernel is launched; same bytes as the two-kernel form. Ignored on the unsplit paths. If a launch ever
             fails (``device_status() != 0``), call ``reset_workspaces()`` before the next fused call: the arrival counters may be left non-zero.
    causal   extension (the reference's MXFP8 path has no mask): key k visible to row i when k < min(i + SK - S + 1, SK); needs SK >= S,
             unsplit paths only ("auto" then never picks the split).
    """
    import torch
    lib = _abi.load()
    dev = q.device
    if not q.is_cuda:
        raise ValueError("fmha_fwd_mxfp8: q must be a contiguous CUDA tensor")
    raw_stream = stream if stream is not None else _raw_stream(torch, dev)
    key = (raw_stream, q.data_ptr(), k.data_ptr(), v.data_ptr(), q_scale.data_ptr(), k_scale.data_ptr(), v_scale.data_ptr(), out.data_ptr(), q.shape, k.shape, v.shape,
           out.shape, out.dtype, q_scale.numel(), k_scale.numel(), path, splits, flags, causal, fused_combine, check,
           None if v_blockscale is None else v_blockscale.data_ptr(), None if lse is None else lse.data_ptr(), dev.index)
    hit = _calls.get(key)
    if hit is not None and hit[0] == _ws_generation and q.is_contiguous() and k.is_contiguous() and v.is_contiguous() and out.is_contiguous():
        raw = raw_stream
        if torch.cuda.current_device() == (dev.index or 0):
            for kernel, args, grid in hit[1]:
                rc = lib.fmha_mxfp8_launch(kernel, C.byref(args), grid, C.c_void_p(raw))
                if rc:
                    raise RuntimeError(f"fmha_mxfp8_launch({lib.fmha_mxfp8_kernel_name(kernel).decode()}) failed with code {rc}")
        else:
            with torch.cuda.device(dev):
                for kernel, args, grid in hit[1]:
                    rc = lib.fmha_mxfp8_launch(kernel, C.byref(args), grid, C.c_void_p(raw))
                    if rc:
                        raise RuntimeError(f"fmha_mxfp8_launch({lib.fmha_mxfp8_kernel_name(kernel).decode()}) failed with code {rc}")
        return hit[2]
    B, S, H, d = q.shape
    _, SK, HK, dk = k.shape
    if d != D or dk != D or HK == 0 or H % HK or (H // HK) & (H // HK - 1) or H // HK > 16:
        raise ValueError(f"fmha_fwd_mxfp8: head dim must be 128 and H a power-of-two multiple (<= 16) of HK (q {tuple(q.shape)}, k {tuple(k.shape)})")
    for name, t, shape in (("q", q, (B, S, H, D)), ("k", k, (B, SK, HK, D)), ("v", v, (B, SK, HK, D)), ("out", out, (B, S, H, D))):
        if tuple(t.shape) != shape or not t.is_contiguous() or not t.is_cuda:
            raise ValueError(f"fmha_fwd_mxfp8: {name} must be a contiguous CUDA tensor of shape {shape}")
    if q.element_size() != 1 or k.element_size() != 1 or v.element_size() != 1 or out.dtype != torch.bfloat16:
        raise ValueError("fmha_fwd_mxfp8: q, k, v are 1-byte e4m3 tensors and out is bf16")
    if _nbytes(v_scale) < 4:
        raise ValueError("v_scale: needs at least one f32")
    if fused_combine:
        flags |= _abi.FLAG_FUSED_COMBINE
    if causal:
        flags |= _abi.FLAG_CAUSAL
        if SK < S:
            raise ValueError("fmha_fwd_mxfp8: causal needs SK >= S")
    if path == "auto":
        path, splits = select_path(B, H, S, SK)
        if causal and path == "kvsplit":
            path, splits = "vs128", 0
    elif path == "kvsplit":
        splits = splits or 4
    stream = raw_stream
    # the library works on the current device (status word, SM count, kernel attributes, stream 0): make it the tensors' device
    record = []
    with torch.cuda.device(q.device):
        ran = _launch_path(lib, q, k, v, q_scale, k_scale, v_scale, out, path, splits, stream, check, flags, v_blockscale, lse, B, S, H, SK, HK, record)
    if len(_calls) >= 256:
        _calls.clear()
    _calls[key] = (_ws_generation, record, ran)   # the key holds the stream: the split path's workspaces belong to one
    return ran


def _raw_stream(torch, dev):
    """The handle of torch's current stream on `dev` (what ``torch.cuda.current_stream(dev).cuda_stream`` gives, without building the object)."""
    get = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    return get(dev.index or 0) if get is not None else torch.cuda.current_stream(dev).cuda_stream


def _launch_path(lib, q, k, v, q_scale, k_scale, v_scale, out, path, splits, stream, check, flags, v_blockscale, lse, B, S, H, SK, HK, record=None):
    sizes = _abi.BufferSizes(ptr_q=_nbytes(q), ptr_k=_nbytes(k), ptr_v=_nbytes(v), ptr_o=_nbytes(out), ptr_q_descale=_nbytes(q_scale),
                             ptr_k_descale=_nbytes(k_scale), ptr_v_descale=_nbytes(v_scale))
    syms = _abi.Symbols(B=B, HK=HK, KL=0)
    if path in ("vs128", "t128"):
        rows = 256 if path == "vs128" else 128
        a = fill_common(_abi.AttnArgs(), q, k, v, q_scale, k_scale, v_scale, out, B, S, H, SK, HK, flags & ~_abi.FLAG_FUSED_COMBINE, v_blockscale, lse)
        _check_launch(lib, PATH_IDS[path], a, sizes, _abi.grid3(math.ceil(S / rows), H, B), syms, stream, check, record)
        return path, 0
    if path != "kvsplit" or splits not in (2, 4, 8):
        raise ValueError(f"fmha_fwd_mxfp8: unknown path {path!r} / splits {splits}")
    rows_total = B * S * H
    ohat = _ws("ohat", splits * rows_total * D * 4, q.device, stream)
    lse_ws = _ws("lse", splits * rows_total * 4, q.device, stream)
    a = fill_common(_abi.KvSplitArgs(), q, k, v, q_scale, k_scale, v_scale, out, B, S, H, SK, HK, flags, v_blockscale, None)
    a.ptr_ohat, a.ptr_lse, a.kvs_splits, a.kvs_rows_total = ohat.data_ptr(), lse_ws.data_ptr(), splits, rows_total
    sizes.ptr_ohat, sizes.ptr_lse = splits * rows_total * D * 4, splits * rows_total * 4
    if flags & _abi.FLAG_FUSED_COMBINE:
        a.ext_ptr_fused_counters = _ws("fused_counters", 4 * B * H * math.ceil(S / 128), q.device, stream, zero=True).data_ptr()
    _check_launch(lib, KVSPLIT, a, sizes, _abi.grid3(math.ceil(S / 256), H, B * splits), syms, stream, check, record)
    if flags & _abi.FLAG_FUSED_COMBINE:
        return path, splits
    c = _abi.CombineArgs(ptr_ohat=ohat.data_ptr(), ptr_lse=lse_ws.data_ptr(), ptr_out=out.data_ptr(), rows_total=rows_total, d=D, splits=splits)
    csizes = _abi.BufferSizes(ptr_ohat=sizes.ptr_ohat, ptr_lse=sizes.ptr_lse, ptr_out=_nbytes(out))
    cgrid = max(1, math.ceil(rows_total * D / (256 * 8)))
    _check_launch(lib, COMBINE8H, c, csizes, _abi.grid3(cgrid, 1, 1), None, stream, check, record)
    return path, splits


def reset_workspaces():
    """Drops the cached KV-split workspaces (partials, log-sum-exps, the fused merge's counters) after a synchronise; the next call makes new ones."""
    import torch
    global _ws_generation
    torch.cuda.synchronize()
    _workspace.clear()
    _calls.clear()
    _ws_generation += 1


def device_status() -> int:
    """The library's device status word (0 = no kernel ever gave up a bounded wait). Synchronises the device."""
    lib = _abi.load()
    st = C.c_uint32(0)
    rc = lib.fmha_mxfp8_device_status(C.byref(st))
    if rc:
        raise RuntimeError(f"fmha_mxfp8_device_status failed with code {rc}")
    return int(st.value)


Q_PRESCALE = 1.4426950408889634 / math.sqrt(128.0)   # log2(e) / sqrt(d): the softmax scale the kernels expect folded into Q


def quantize_qk(x, out, out_scales, *, mul=1.0, stream=None):
    """bf16 ``x`` [..., 128] -> e4m3 bytes ``out`` (same shape, uint8) and E8M0 scale bytes at the start of the flat uint8 buffer
    ``out_scales`` (rows * 4 bytes, followed by whatever zeroed slack the caller allocated). The harness's host rule
    (tests/gpu/ref_host.cpp:239-254) on the device; pass ``mul=Q_PRESCALE`` for Q and 1 for K."""
    import torch
    lib = _abi.load()
    rows = x.numel() // D
    if x.dtype != torch.bfloat16 or x.shape[-1] != D or not x.is_contiguous() or not x.is_cuda:
        raise ValueError("quantize_qk: x must be a contiguous CUDA bf16 tensor [..., 128]")
    if out.numel() != x.numel() or out.element_size() != 1 or not out.is_contiguous() or _nbytes(out_scales) < rows * 4:
        raise ValueError("quantize_qk: out must hold one byte per element and out_scales 4 bytes per row")
    if stream is None:
        stream = torch.cuda.current_stream(x.device).cuda_stream
    with torch.cuda.device(x.device):
        rc = lib.fmha_mxfp8_quantize_qk(x.data_ptr(), rows, float(mul), out.data_ptr(), out_scales.data_ptr(), C.c_void_p(stream))
    if rc:
        raise RuntimeError(f"fmha_mxfp8_quantize_qk failed with code {rc}")


def quantize_v(x, out, v_descale, *, stream=None):
    """bf16 ``x`` -> e4m3 bytes ``out`` with one f32 descale written to ``v_descale[0]`` (f32 buffer, the contract asks for >= 4096 bytes)."""
    import torch
    lib = _abi.load()
    if x.dtype != torch.bfloat16 or not x.is_contiguous() or not x.is_cuda or x.numel() % 8:
        raise ValueError("quantize_v: x must be a contiguous CUDA bf16 tensor with a multiple of 8 elements")
    if out.numel() != x.numel() or out.element_size() != 1 or not out.is_contiguous() or _nbytes(v_descale) < 8:
        raise ValueError("quantize_v: out must hold one byte per element and v_descale at least 8 bytes")
    if stream is None:
        stream = torch.cuda.current_stream(x.device).cuda_stream
    with torch.cuda.device(x.device):
        rc = lib.fmha_mxfp8_quantize_v(x.data_ptr(), x.numel(), out.data_ptr(), v_descale.data_ptr(), C.c_void_p(stream))
    if rc:
        raise RuntimeError(f"fmha_mxfp8_quantize_v failed with code {rc}")
