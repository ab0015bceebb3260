"""ctypes binding of the C ABI in ``include/fmha_mxfp8_abi.h`` (libfmha_mxfp8_b200.so, built in-tree by ``csrc/Makefile``).

The structs repeat the packed kernel-argument blocks of the reference's generated host contract
(tests/gpu/generated/fmha_fwd_hd128_mxfp8_v3_*_abi.h); offsets are asserted at import time against the
reference's JSON twins' values (kernarg sizes 656 / 656 / 648 / 36, tests/hostgen/test_json_kernarg.py:54-57).
There is no fallback: if the shared library is missing, loading raises.
"""
from __future__ import annotations

import ctypes as C
import os

VS128, T128, KVSPLIT, COMBINE8H = 0, 1, 2, 3
PATH_NAMES = {VS128: "vs128", T128: "t128", KVSPLIT: "kvsplit"}
PATH_IDS = {v: k for k, v in PATH_NAMES.items()}
FLAG_V_BLOCKSCALE = 0x1
FLAG_EXACT_REBASE = 0x2
FLAG_CAUSAL = 0x8
FLAG_F32_PARTIALS = 0x10
FLAG_NO_TAIL_SPLIT = 0x20
FLAG_FUSED_COMBINE = 0x40
TRACE_BYTES = 4 * (16384 + 16384 + 256 + 4096 + 2048)
PEER_HANDLE_BYTES, PEER_MAX_GPUS, PEER_PLAN_BYTES = 64, 8, 1152
STATIC_SCRATCH_MAX_ROW_SPLITS = 65536   # FMHA_MXFP8_STATIC_SCRATCH_MAX_ROW_SPLITS

ERROR_CLASSES = {1: "GV-HOST-EXTENT", 2: "GV-HOST-KA-RANGE", 3: "GV-HOST-KA-IS", 4: "GV-HOST-GRID", 5: "GV-HOST-SYM", 6: "ARG", 7: "DEVICE"}


def _pad(n, i):
    return (f"_pad{i}", C.c_uint8 * n)


_COMMON = [
    ("ptr_o", C.c_void_p), _pad(8, 0), ("ptr_q", C.c_void_p), _pad(8, 1), ("ptr_k", C.c_void_p), _pad(8, 2), ("ptr_v", C.c_void_p),
    ("ext_ptr_peer_plan", C.c_void_p), ("ext_ptr_lse", C.c_void_p), ("ext_ptr_v_blockscale", C.c_void_p), _pad(8, "3b"), ("ext_flags", C.c_uint32), _pad(4, "3c"),
    ("s_seq_len", C.c_uint32), _pad(12, 4), ("s_Seqs", C.c_uint32), _pad(28, 5), ("s_Hs", C.c_uint32), _pad(12, 6), ("s_Bs", C.c_uint32), _pad(12, 7),
    ("s_gqa", C.c_uint32), _pad(12, 8), ("s_k_Seqs", C.c_uint32), _pad(12, 9), ("s_k_Hs", C.c_uint32), _pad(12, 10), ("s_k_Bs", C.c_uint32), _pad(44, 11),
    ("s_kv_seq_len", C.c_uint32), _pad(44, 12), ("s_q_head_num", C.c_uint32), _pad(12, 13), ("s_v_Seqs", C.c_uint32), _pad(12, 14),
    ("s_v_Hs", C.c_uint32), _pad(12, 15), ("s_v_Bs", C.c_uint32), _pad(12, 16), ("s_o_Seqs", C.c_uint32), _pad(12, 17), ("s_o_Hs", C.c_uint32), _pad(12, 18),
    ("s_o_Bs", C.c_uint32), _pad(92, 19), ("ptr_q_descale", C.c_void_p), _pad(8, 20), ("ptr_k_descale", C.c_void_p), _pad(8, 21),
    ("ptr_v_descale", C.c_void_p), _pad(8, 22), ("s_descale_q_Bs", C.c_uint32), _pad(12, 23), ("s_descale_q_Hs", C.c_uint32), _pad(12, 24),
    ("s_descale_k_Bs", C.c_uint32), _pad(12, 25), ("s_descale_k_Hs", C.c_uint32),
]


class AttnArgs(C.Structure):
    """vs128 / t128 kernel arguments (656 bytes)."""
    _pack_ = 1
    _fields_ = _COMMON + [_pad(28, 26), ("abi_tail", C.c_uint8 * 16)]


class KvSplitArgs(C.Structure):
    """kvsplit kernel arguments (648 bytes)."""
    _pack_ = 1
    _fields_ = _COMMON + [_pad(12, 26), ("ptr_ohat", C.c_void_p), ("ptr_lse", C.c_void_p), ("kvs_splits", C.c_uint32), ("kvs_rows_total", C.c_uint32)]

    # offset 0x040 is `ext_ptr_fused_counters` in this block (the unsplit kernels' `ext_ptr_lse`)
    ext_ptr_fused_counters = property(lambda self: self.ext_ptr_lse, lambda self, v: setattr(self, "ext_ptr_lse", v))


class CombineArgs(C.Structure):
    """combine kernel arguments (36 bytes)."""
    _pack_ = 1
    _fields_ = [("ptr_ohat", C.c_void_p), ("ptr_lse", C.c_void_p), ("ptr_out", C.c_void_p), ("rows_total", C.c_uint32), ("d", C.c_uint32), ("splits", C.c_uint32)]


class Symbols(C.Structure):
    _fields_ = [("B", C.c_int64), ("HK", C.c_int64), ("KL", C.c_int64)]


class BufferSizes(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("ptr_q", "ptr_k", "ptr_v", "ptr_o", "ptr_q_descale", "ptr_k_descale", "ptr_v_descale", "ptr_ohat", "ptr_lse", "ptr_out")]


class Problem(C.Structure):
    _fields_ = [
        ("B", C.c_uint32), ("H", C.c_uint32), ("HK", C.c_uint32), ("S", C.c_uint32), ("SK", C.c_uint32),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("q_descale", C.c_void_p), ("k_descale", C.c_void_p), ("v_descale", C.c_void_p),
        ("out", C.c_void_p), ("q_descale_bytes", C.c_uint64), ("k_descale_bytes", C.c_uint64), ("v_descale_bytes", C.c_uint64),
        ("ws_ohat", C.c_void_p), ("ws_lse", C.c_void_p), ("ws_ohat_bytes", C.c_uint64), ("ws_lse_bytes", C.c_uint64),
        ("v_blockscale", C.c_void_p), ("flags", C.c_uint32),
    ]


assert C.sizeof(AttnArgs) == 656 and C.sizeof(KvSplitArgs) == 648 and C.sizeof(CombineArgs) == 36
assert AttnArgs.ext_ptr_peer_plan.offset == 0x38 and KvSplitArgs.ext_ptr_peer_plan.offset == 0x38
assert AttnArgs.s_seq_len.offset == 0x60 and AttnArgs.ptr_q_descale.offset == 0x200 and AttnArgs.abi_tail.offset == 0x280
assert KvSplitArgs.ptr_ohat.offset == 0x270 and KvSplitArgs.kvs_rows_total.offset == 0x284

ARGS_TYPES = {VS128: AttnArgs, T128: AttnArgs, KVSPLIT: KvSplitArgs, COMBINE8H: CombineArgs}

LIB_NAME = "libfmha_mxfp8_b200.so"
_lib = None


def lib_path() -> str:
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), LIB_NAME)


def load():
    """Loads the shared library (once). Raises OSError when it has not been built: there is no other implementation to fall back to."""
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not os.path.exists(path):
        raise OSError(f"{path} is missing: build it with `make -C amdgpu_rustdsl_b200/csrc` (or `python -c 'import __graft_entry__ as g; g.build()'`)")
    lib = C.CDLL(path)
    u32x3 = C.POINTER(C.c_uint32)
    lib.fmha_mxfp8_kernel_name.restype = C.c_char_p
    lib.fmha_mxfp8_kernel_name.argtypes = [C.c_int]
    lib.fmha_mxfp8_kernarg_size.restype = C.c_size_t
    lib.fmha_mxfp8_kernarg_size.argtypes = [C.c_int]
    lib.fmha_mxfp8_workgroup_size.restype = C.c_uint
    lib.fmha_mxfp8_workgroup_size.argtypes = [C.c_int]
    lib.fmha_mxfp8_validate.restype = C.c_int
    lib.fmha_mxfp8_validate.argtypes = [C.c_int, C.c_void_p, C.POINTER(BufferSizes), u32x3, C.POINTER(Symbols), C.c_char_p, C.c_size_t]
    lib.fmha_mxfp8_grid.restype = C.c_int
    lib.fmha_mxfp8_grid.argtypes = [C.c_int, C.c_void_p, C.POINTER(Symbols), u32x3]
    lib.fmha_mxfp8_launch.restype = C.c_int
    lib.fmha_mxfp8_launch.argtypes = [C.c_int, C.c_void_p, u32x3, C.c_void_p]
    lib.fmha_mxfp8_dispatch.restype = None
    lib.fmha_mxfp8_dispatch.argtypes = [C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.POINTER(C.c_int), C.POINTER(C.c_uint32)]
    lib.fmha_mxfp8_auto.restype = C.c_int
    lib.fmha_mxfp8_auto.argtypes = [C.POINTER(Problem), C.c_int, C.c_uint32, C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_uint32), C.c_char_p, C.c_size_t]
    lib.fmha_mxfp8_kvsplit_static_scratch.restype = C.c_int
    lib.fmha_mxfp8_kvsplit_static_scratch.argtypes = [C.POINTER(Problem), C.c_uint32, C.c_void_p, C.c_char_p, C.c_size_t]
    lib.fmha_mxfp8_combine_f32.restype = C.c_int
    lib.fmha_mxfp8_combine_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p]
    vpp = C.POINTER(C.c_void_p)
    lib.fmha_mxfp8_peer_alloc.restype = C.c_int
    lib.fmha_mxfp8_peer_alloc.argtypes = [C.c_size_t, vpp, C.c_void_p]
    lib.fmha_mxfp8_peer_open.restype = C.c_int
    lib.fmha_mxfp8_peer_open.argtypes = [C.c_void_p, vpp]
    lib.fmha_mxfp8_peer_close.restype = C.c_int
    lib.fmha_mxfp8_peer_close.argtypes = [C.c_void_p]
    lib.fmha_mxfp8_peer_free.restype = C.c_int
    lib.fmha_mxfp8_peer_free.argtypes = [C.c_void_p]
    lib.fmha_mxfp8_peer_plan_build.restype = C.c_int
    lib.fmha_mxfp8_peer_plan_build.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_int, vpp, vpp, C.c_void_p, C.c_void_p]
    lib.fmha_mxfp8_combine_scatter.restype = C.c_int
    lib.fmha_mxfp8_combine_scatter.argtypes = [C.c_void_p, C.c_int, C.c_void_p, vpp, C.c_uint32, C.c_uint64, C.c_uint32, C.c_uint32, C.c_void_p]
    lib.fmha_mxfp8_peer_barrier.restype = C.c_int
    lib.fmha_mxfp8_peer_barrier.argtypes = [vpp, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p]
    lib.fmha_mxfp8_copy_async.restype = C.c_int
    lib.fmha_mxfp8_copy_async.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
    lib.fmha_mxfp8_quantize_qk.restype = C.c_int
    lib.fmha_mxfp8_quantize_qk.argtypes = [C.c_void_p, C.c_uint64, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.fmha_mxfp8_quantize_v.restype = C.c_int
    lib.fmha_mxfp8_quantize_v.argtypes = [C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.fmha_mxfp8_device_status.restype = C.c_int
    lib.fmha_mxfp8_device_status.argtypes = [C.POINTER(C.c_uint32)]
    lib.fmha_mxfp8_trace_attach.restype = C.c_int
    lib.fmha_mxfp8_trace_attach.argtypes = [C.c_void_p, C.c_size_t]
    lib.fmha_mxfp8_mma_issue_ceiling.restype = C.c_int
    lib.fmha_mxfp8_mma_issue_ceiling.argtypes = [C.c_int, C.c_int, C.c_void_p, C.POINTER(C.c_float)]
    lib.fmha_mxfp8_selftest_bounded_wait.restype = C.c_int
    lib.fmha_mxfp8_selftest_bounded_wait.argtypes = [C.c_uint32, C.c_void_p, C.POINTER(C.c_uint32), C.POINTER(C.c_float)]
    _lib = lib
    return lib


EXPORTS = (
    "fmha_mxfp8_kernel_name", "fmha_mxfp8_kernarg_size", "fmha_mxfp8_workgroup_size", "fmha_mxfp8_validate", "fmha_mxfp8_grid",
    "fmha_mxfp8_launch", "fmha_mxfp8_dispatch", "fmha_mxfp8_auto", "fmha_mxfp8_device_status", "fmha_mxfp8_trace_attach",
    "fmha_mxfp8_mma_issue_ceiling", "fmha_mxfp8_selftest_bounded_wait", "fmha_mxfp8_kvsplit_static_scratch", "fmha_mxfp8_quantize_qk", "fmha_mxfp8_quantize_v", "fmha_mxfp8_combine_f32", "fmha_mxfp8_peer_alloc", "fmha_mxfp8_peer_open", "fmha_mxfp8_peer_close", "fmha_mxfp8_peer_free",
    "fmha_mxfp8_peer_plan_build", "fmha_mxfp8_combine_scatter", "fmha_mxfp8_copy_async", "fmha_mxfp8_peer_barrier",
)


class ContractError(ValueError):
    """A host-contract check failed (the reference's ``ContractError``, python/amdgpu_jit/_kernarg.py:13)."""

    def __init__(self, code: int, message: str):
        super().__init__(message or ERROR_CLASSES.get(code, f"error {code}"))
        self.code = code


def grid3(x, y, z):
    return (C.c_uint32 * 3)(x, y, z)
