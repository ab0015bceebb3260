"""B200 (sm_100a) implementation of the reference's MXFP8 attention forward path `fmha_fwd_hd128_mxfp8_auto`.

`fmha_fwd_mxfp8` / `select_path` mirror python/amdgpu_jit/ops.py of the reference; `_abi` binds the C ABI of
include/fmha_mxfp8_abi.h. The CUDA library is built in-tree (csrc/Makefile); there is no other backend.
"""
from ._abi import ContractError  # noqa: F401
from .ops import Q_PRESCALE, device_status, fmha_fwd_mxfp8, quantize_qk, quantize_v, reset_workspaces, select_path  # noqa: F401
