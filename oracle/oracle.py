"""TEST INFRASTRUCTURE ONLY: numpy-facing binding of the CPU oracle (oracle/fmha_oracle.c, built to oracle/_build/liboracle.so).

Imported by tests/, by ``__graft_entry__.smoke()`` and by the CPU-baseline legs of ``bench.py``; never by the product package.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "_build", "liboracle.so")
REF_HOST = os.path.join(HERE, "_ref", "ref_host")   # the reference harness built against the stub HIP runtime, when available
MODES = {"lcg": 0, "uniform": 1, "normal": 2}


class _Shape(C.Structure):
    _fields_ = [("B", C.c_int), ("H", C.c_int), ("HK", C.c_int), ("S", C.c_int), ("SK", C.c_int)]


class _Stats(C.Structure):
    _fields_ = [("checked", C.c_uint64), ("bad", C.c_uint64), ("worst_err", C.c_double), ("mean_err", C.c_double), ("max_ref", C.c_double)]


_lib = None


def build():
    subprocess.run(["make", "-C", HERE, "--no-print-directory"], check=True, stdout=subprocess.DEVNULL)


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB):
            build()
        _lib = C.CDLL(LIB)
        _lib.oracle_e4m3_decode.restype = C.c_double
        _lib.oracle_e4m3_decode.argtypes = [C.c_uint8]
        _lib.oracle_e4m3_encode.restype = C.c_uint8
        _lib.oracle_e4m3_encode.argtypes = [C.c_float]
        for f in ("oracle_q_bytes", "oracle_kv_bytes", "oracle_qs_bytes", "oracle_ks_bytes"):
            getattr(_lib, f).restype = C.c_size_t
            getattr(_lib, f).argtypes = [C.POINTER(_Shape)]
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


@dataclass
class Inputs:
    B: int
    H: int
    HK: int
    S: int
    SK: int
    q: np.ndarray        # uint8 [B,S,H,128]
    k: np.ndarray        # uint8 [B,SK,HK,128]
    v: np.ndarray        # uint8 [B,SK,HK,128]
    qs: np.ndarray       # uint8 flat, [B,S,H,4] + slack
    ks: np.ndarray       # uint8 flat, [B,SK,HK,4] + slack
    vdescale: float
    vscale: np.ndarray | None = None   # extension: uint8 [B,ceil(SK/32),HK,128]

    @property
    def shape(self):
        return _Shape(self.B, self.H, self.HK, self.S, self.SK)


def generate(mode: str, B: int, H: int, S: int, SK: int, HK: int | None = None, v_blockscale: bool = False) -> Inputs:
    """The reference harness's generators (tests/gpu/ref_host.cpp:183-263): mode is "lcg", "uniform" or "normal"."""
    HK = HK or H
    L = lib()
    sh = _Shape(B, H, HK, S, SK)
    q = np.empty(L.oracle_q_bytes(C.byref(sh)), np.uint8)
    k = np.empty(L.oracle_kv_bytes(C.byref(sh)), np.uint8)
    v = np.empty_like(k)
    qs = np.empty(L.oracle_qs_bytes(C.byref(sh)), np.uint8)
    ks = np.empty(L.oracle_ks_bytes(C.byref(sh)), np.uint8)
    vd = C.c_float(0)
    rc = L.oracle_generate(MODES[mode], C.byref(sh), _p(q), _p(k), _p(v), _p(qs), _p(ks), C.byref(vd))
    if rc:
        raise RuntimeError(f"oracle_generate failed: {rc}")
    vscale = None
    if v_blockscale:
        if mode != "normal":
            raise ValueError("V block scales exist only for normal data")
        vscale = np.empty(B * ((SK + 31) // 32) * HK * 128, np.uint8)
        rc = L.oracle_generate_v_blockscaled(C.byref(sh), _p(v), _p(vscale))
        if rc:
            raise RuntimeError(f"oracle_generate_v_blockscaled failed: {rc}")
        vscale = vscale.reshape(B, (SK + 31) // 32, HK, 128)
    return Inputs(B, H, HK, S, SK, q.reshape(B, S, H, 128), k.reshape(B, SK, HK, 128), v.reshape(B, SK, HK, 128), qs, ks, float(vd.value), vscale)


def _row_list(rows):
    """None for "the first n rows" (an int, the reference's REF_ROWS), else the explicit rows as a C int array."""
    if isinstance(rows, (int, np.integer)):
        return None
    a = np.ascontiguousarray(np.asarray(list(rows), dtype=np.int32))
    assert a.ndim == 1 and a.size > 0
    return a


def spread_rows(S: int, extra=()) -> list:
    """Query rows that reach every kind of 128-row tile of a sequence: the first rows, both sides of the first tile edge, a tile in
    the middle, and the last rows (a ragged last tile included)."""
    cand = [0, 1, 31, 32, 126, 127, 128, 129, 255, 256, S // 2 - 1, S // 2, S // 2 + 77, (S // 128) * 128 - 1, (S // 128) * 128, S - 2, S - 1, *extra]
    return sorted({r for r in cand if 0 <= r < S})


def reference(inp: Inputs, rows, causal: bool = False) -> np.ndarray:
    """fp64 oracle (ref_host.cpp:438-471) for the first ``rows`` query rows of every (b,h), or for the rows of a list:
    float64 [B,H,rows_eff,128].
    ``causal``: row i sees the keys below min(i + SK - S + 1, SK) (the mask of the reference's per-tensor sibling family, attn3.rs:298-306)."""
    L = lib()
    sh = inp.shape
    rl = _row_list(rows)
    if rl is not None:
        ref = np.empty((inp.B, inp.H, rl.size, 128), np.float64)
        rc = L.oracle_reference_rows(C.byref(sh), _p(inp.q), _p(inp.k), _p(inp.v), _p(inp.qs), _p(inp.ks), C.c_float(inp.vdescale),
                                     _p(inp.vscale) if not causal else None, _p(rl), C.c_int(rl.size), C.c_int(1 if causal else 0), _p(ref))
        if rc:
            raise RuntimeError(f"oracle_reference_rows failed: {rc}")
        return ref
    re = min(rows, inp.S)
    ref = np.empty((inp.B, inp.H, re, 128), np.float64)
    if causal:
        rc = L.oracle_reference_causal(C.byref(sh), _p(inp.q), _p(inp.k), _p(inp.v), _p(inp.qs), _p(inp.ks), C.c_float(inp.vdescale),
                                       C.c_int(rows), _p(ref))
        if rc:
            raise RuntimeError(f"oracle_reference_causal failed: {rc}")
        return ref
    rc = L.oracle_reference(C.byref(sh), _p(inp.q), _p(inp.k), _p(inp.v), _p(inp.qs), _p(inp.ks), C.c_float(inp.vdescale), _p(inp.vscale),
                            C.c_int(rows), _p(ref))
    if rc:
        raise RuntimeError(f"oracle_reference failed: {rc}")
    return ref


@dataclass
class Stats:
    checked: int
    bad: int
    worst_err: float
    mean_err: float
    max_ref: float


def compare(inp: Inputs, out_bf16: np.ndarray, ref: np.ndarray, rows) -> Stats:
    """The gate statistics of the reference's ``check`` (ref_host.cpp:463-469). ``out_bf16`` is uint16 [B,S,H,128]; ``rows`` as in ``reference``."""
    L = lib()
    out = np.ascontiguousarray(out_bf16, dtype=np.uint16)
    assert out.size == inp.B * inp.S * inp.H * 128
    ref = np.ascontiguousarray(ref, dtype=np.float64)
    st = _Stats()
    sh = inp.shape
    rl = _row_list(rows)
    if rl is not None:
        assert ref.shape[2] == rl.size
        rc = L.oracle_compare_rows(C.byref(sh), _p(out), _p(ref), _p(rl), C.c_int(rl.size), C.byref(st))
        if rc:
            raise RuntimeError(f"oracle_compare_rows failed: {rc}")
    else:
        L.oracle_compare(C.byref(sh), _p(out), _p(ref), C.c_int(rows), C.byref(st))
    return Stats(int(st.checked), int(st.bad), float(st.worst_err), float(st.mean_err), float(st.max_ref))


def recipe_forward(inp: Inputs, rows, splits: int = 0) -> np.ndarray:
    """CPU restatement of the reference kernels' arithmetic ("the reference path" of the gate): uint16 bf16 [B,S,H,128], of which only
    the asked rows (``rows`` as in ``reference``) are filled."""
    L = lib()
    out = np.zeros((inp.B, inp.S, inp.H, 128), np.uint16)
    sh = inp.shape
    rl = _row_list(rows)
    if rl is not None:
        rc = L.oracle_recipe_forward_rows(C.byref(sh), _p(inp.q), _p(inp.k), _p(inp.v), _p(inp.qs), _p(inp.ks), C.c_float(inp.vdescale),
                                          C.c_int(splits), _p(rl), C.c_int(rl.size), _p(out))
        if rc:
            raise RuntimeError(f"oracle_recipe_forward_rows failed: {rc}")
        return out
    rc = L.oracle_recipe_forward(C.byref(sh), _p(inp.q), _p(inp.k), _p(inp.v), _p(inp.qs), _p(inp.ks), C.c_float(inp.vdescale), C.c_int(splits),
                                 C.c_int(rows), _p(out))
    if rc:
        raise RuntimeError(f"oracle_recipe_forward failed: {rc}")
    return out


def combine_f32(ohat: np.ndarray, lse2: np.ndarray, rows_total: int, splits: int) -> np.ndarray:
    """CPU restatement of the combine kernel (crates/amdgpu-tile/src/epilogue.rs:117-146) on f32 partials: uint16 bf16 [rows_total,128]."""
    L = lib()
    ohat = np.ascontiguousarray(ohat, np.float32)
    lse2 = np.ascontiguousarray(lse2, np.float32)
    out = np.empty((rows_total, 128), np.uint16)
    L.oracle_combine_f32(_p(ohat), _p(lse2), C.c_uint32(rows_total), C.c_uint32(splits), _p(out))
    return out


def quantize_rows(x: np.ndarray, mul: float = 1.0):
    """The harness's Q / K rule (ref_host.cpp:239-252) on f32 rows of 128: returns (e4m3 bytes [rows,128], E8M0 bytes [rows,4])."""
    L = lib()
    x = np.ascontiguousarray(x, np.float32).reshape(-1, 128)
    out = np.empty(x.shape, np.uint8)
    scales = np.empty((x.shape[0], 4), np.uint8)
    L.oracle_quantize_rows(_p(x), C.c_long(x.shape[0]), C.c_float(mul), _p(out), _p(scales))
    return out, scales


def quantize_tensor(x: np.ndarray):
    """The harness's V rule (ref_host.cpp:253-258) on an f32 tensor: returns (e4m3 bytes, f32 descale)."""
    L = lib()
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(x.shape, np.uint8)
    vd = C.c_float(0)
    L.oracle_quantize_tensor(_p(x), C.c_size_t(x.size), _p(out), C.byref(vd))
    return out, float(vd.value)


def generate_raw_normal(B: int, H: int, S: int, SK: int, HK: int | None = None):
    """The `normal` generator's unquantised samples as f32: (q [B,S,H,128] with the softmax scale folded in, k, v [B,SK,HK,128])."""
    HK = HK or H
    L = lib()
    sh = _Shape(B, H, HK, S, SK)
    q = np.empty((B, S, H, 128), np.float32)
    k = np.empty((B, SK, HK, 128), np.float32)
    v = np.empty((B, SK, HK, 128), np.float32)
    L.oracle_generate_raw_normal(C.byref(sh), _p(q), _p(k), _p(v))
    return q, k, v


def dispatch(B, H, S, SK):
    L = lib()
    path, splits = C.c_int(0), C.c_uint32(0)
    L.oracle_dispatch(C.c_uint64(B), C.c_uint64(H), C.c_uint64(S), C.c_uint64(SK), C.byref(path), C.byref(splits))
    return ("vs128", "t128", "kvsplit")[path.value], int(splits.value)


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def set_threads(n: int) -> int:
    """Asks for ``n`` OpenMP threads in the oracle's loops (torch.distributed.run exports OMP_NUM_THREADS=1); returns the count in force."""
    L = lib()
    L.oracle_set_threads.restype = C.c_int
    return int(L.oracle_set_threads(C.c_int(int(n))))


def bf16_to_f32(x: np.ndarray) -> np.ndarray:
    return (x.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    u = u + 0x7FFF + ((u >> 16) & 1)
    return (u >> 16).astype(np.uint16)


E4M3_TABLE = None


def e4m3_table() -> np.ndarray:
    global E4M3_TABLE
    if E4M3_TABLE is None:
        L = lib()
        E4M3_TABLE = np.array([L.oracle_e4m3_decode(i) for i in range(256)], np.float64)
    return E4M3_TABLE


def run_ref_host(mode: str, B: int, H: int, S: int, SK: int, HK: int | None = None, rows: int = 64, out_file: str | None = None,
                 dump_prefix: str | None = None, timeout: float = 600.0) -> str:
    """Runs the reference's own harness (built against the stub HIP runtime) and returns its stdout. Raises if it was not built."""
    if not os.path.exists(REF_HOST):
        raise FileNotFoundError(REF_HOST)
    env = dict(os.environ, REF_DATA=mode, REF_B=str(B), REF_H=str(H), REF_S=str(S), REF_SK=str(SK), REF_HK=str(HK or H), REF_ROWS=str(rows))
    if out_file:
        env["HIPSTUB_OUT"] = out_file
    if dump_prefix:
        env["REF_INPUT_DUMP"] = dump_prefix
    r = subprocess.run([REF_HOST, "stub.co"], env=env, capture_output=True, text=True, timeout=timeout)
    return r.stdout
