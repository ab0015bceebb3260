"""Sharding of the MXFP8 attention path over the GPUs of one node, one process per GPU.

The reference has no multi-GPU code; the two shardings below follow from the structure of its path:
  * by (batch x head): the logical blocks of the unsplit kernels are independent (grid y = H, z = B,
    tests/gpu/generated/fmha_fwd_hd128_mxfp8_v3_vs128_abi.h:200-201), so each rank runs the path on its own packed tensors with
    H/world heads. Whole KV-head groups stay on one rank (kv head = head >> log2 gqa, crates/amdgpu-stage/src/components.rs:8-17).
    No collective.
  * by key range: the KV-split algebra with "split = rank" (crates/amdgpu-stage/src/components.rs:58-74,
    crates/amdgpu-tile/src/epilogue.rs:117-146): every rank runs the split kernel over its local keys for all queries, the f32
    partials (O, base-2 LSE) are exchanged once into local memory (an all-to-all of row slices, or an all-gather of whole partials: NCCL on GPUs, gloo in the
    CPU tests), and the combine kernel merges them with splits = world.
`torch.distributed` is the plumbing; the kernels are the library's.
"""
from __future__ import annotations

import math

D = 128


def head_shard(H: int, HK: int, rank: int, world: int):
    """Heads [h0, h1) and KV heads [k0, k1) of `rank`: KV-head groups are dealt out contiguously, as evenly as possible."""
    if H % HK:
        raise ValueError("H must be a multiple of HK")
    gqa = H // HK
    base, extra = divmod(HK, world)
    k0 = rank * base + min(rank, extra)
    k1 = k0 + base + (1 if rank < extra else 0)
    return (k0 * gqa, k1 * gqa), (k0, k1)


def kv_range_shard(SK: int, rank: int, world: int):
    """Keys [lo, hi) of `rank`: 128-key tiles dealt out like the split kernel's ranges (tiles [r*tps, min(ntiles, (r+1)*tps))); every rank
    must own a tile, as the reference demands of every split (tests/gpu/ref_host.cpp:117-120)."""
    ntiles = -(-SK // 128)
    tps = -(-ntiles // world)
    if (world - 1) * tps >= ntiles:
        raise ValueError(f"SK={SK} gives {ntiles} key tiles: too few for {world} ranks")
    lo = rank * tps * 128
    hi = min((rank + 1) * tps * 128, SK)
    return lo, hi


def local_partials(q, k_local, v_local, q_scale, k_scale_local, v_scale, ohat, lse, *, stream=None, check=True):
    """One rank's contribution to a key-range-sharded forward: the split kernel with splits = 1 over the local keys, writing the
    normalised f32 partial O [rows_total,128] and base-2 log-sum-exp [rows_total] of all queries."""
    import ctypes as C
    import torch
    from . import _abi
    from .ops import _check_launch, _nbytes, fill_common
    lib = _abi.load()
    B, S, H, _ = q.shape
    _, SKl, HK, _ = k_local.shape
    if stream is None:
        stream = torch.cuda.current_stream(q.device).cuda_stream
    rows_total = B * S * H
    # f32 partials: these travel between GPUs before they are combined
    a = fill_common(_abi.KvSplitArgs(), q, k_local, v_local, q_scale, k_scale_local, v_scale, ohat, B, S, H, SKl, HK, flags=_abi.FLAG_F32_PARTIALS)
    a.ptr_o = None
    a.ptr_ohat, a.ptr_lse, a.kvs_splits, a.kvs_rows_total = ohat.data_ptr(), lse.data_ptr(), 1, rows_total
    sizes = _abi.BufferSizes(ptr_q=_nbytes(q), ptr_k=_nbytes(k_local), ptr_v=_nbytes(v_local), ptr_o=B * S * H * 256, ptr_q_descale=_nbytes(q_scale),
                             ptr_k_descale=_nbytes(k_scale_local), ptr_v_descale=_nbytes(v_scale), ptr_ohat=_nbytes(ohat), ptr_lse=_nbytes(lse))
    syms = _abi.Symbols(B=B, HK=HK, KL=0)
    with torch.cuda.device(q.device):
        _check_launch(lib, _abi.KVSPLIT, a, sizes, _abi.grid3(math.ceil(S / 256), H, B), syms, stream, check)


def combine_gathered(ohat_all, lse_all, out, world: int, *, stream=None, check=True):
    """The combine kernel over the gathered f32 partials: ohat_all f32 [world, rows_total, 128], lse_all f32 [world, rows_total] -> bf16 out."""
    import ctypes as C
    import torch
    from . import _abi
    lib = _abi.load()
    rows_total = out.numel() // D
    if stream is None:
        stream = torch.cuda.current_stream(out.device).cuda_stream
    if ohat_all.dtype != torch.float32 or lse_all.dtype != torch.float32 or out.dtype != torch.bfloat16:
        raise ValueError("combine_gathered: f32 partials and log-sum-exps, bf16 output")
    if check and (ohat_all.numel() < world * rows_total * D or lse_all.numel() < world * rows_total):
        raise ValueError("combine_gathered: partial buffers smaller than world x rows_total")
    with torch.cuda.device(out.device):
        rc = lib.fmha_mxfp8_combine_f32(ohat_all.data_ptr(), lse_all.data_ptr(), out.data_ptr(), rows_total, world, C.c_void_p(stream))
    if rc:
        raise RuntimeError(f"fmha_mxfp8_combine_f32 failed with code {rc}")


def exchange_partials(ohat, lse, ohat_all, lse_all, group=None):
    """The one exchange step of the key-range sharding: all-gather of every rank's partials into local memory (rank-major, which is the
    [splits][rows_total] layout the combine kernel reads)."""
    import torch.distributed as dist
    # the output as the concatenation along dim 0 (the form every backend accepts; gloo rejects the stacked [world, ...] shape)
    dist.all_gather_into_tensor(ohat_all.view(-1, ohat.shape[-1]), ohat, group=group)
    dist.all_gather_into_tensor(lse_all.view(-1), lse, group=group)


def exchange_row_slices(ohat, lse, ohat_recv, lse_recv, group=None):
    """The cheaper exchange of the key-range sharding: an all-to-all in which rank j receives, from every rank, only the partials of its
    own 1/world slice of the rows: ohat [rows_total,128] -> ohat_recv [world, rows_total/world, 128] (rank-major = the [splits][rows]
    layout the combine kernel reads), likewise the LSEs. (world-1)/world of one partial crosses the links per rank instead of world-1."""
    import torch.distributed as dist
    dist.all_to_all_single(ohat_recv.view(-1, ohat.shape[-1]), ohat, group=group)
    dist.all_to_all_single(lse_recv.view(-1), lse, group=group)


def gather_output_slices(out, out_slice, group=None):
    """Every rank's combined bf16 row slice -> the whole output on every rank."""
    import torch.distributed as dist
    dist.all_gather_into_tensor(out.view(-1, out.shape[-1]), out_slice.view(-1, out.shape[-1]), group=group)


def kv_sharded_workspace(rows_total: int, world: int, device, sliced: bool = True):
    """Workspaces of `fmha_fwd_mxfp8_kv_sharded` for `rows_total` = B*S*H rows: the local partial, and either the row-slice buffers of the
    all-to-all form (rows_total divisible by world) or the gathered partials of the all-gather form."""
    import torch
    ws = {"ohat": torch.empty(rows_total, D, dtype=torch.float32, device=device), "lse": torch.empty(rows_total, dtype=torch.float32, device=device)}
    if sliced and rows_total % world == 0:
        n = rows_total // world
        ws["ohat_recv"] = torch.empty(world, n, D, dtype=torch.float32, device=device)
        ws["lse_recv"] = torch.empty(world, n, dtype=torch.float32, device=device)
        ws["out_slice"] = torch.empty(n, D, dtype=torch.bfloat16, device=device)
    else:
        ws["ohat_all"] = torch.empty(world, rows_total, D, dtype=torch.float32, device=device)
        ws["lse_all"] = torch.empty(world, rows_total, dtype=torch.float32, device=device)
    return ws


def fmha_fwd_mxfp8_kv_sharded(q, k_local, v_local, q_scale, k_scale_local, v_scale, out, ws, group=None):
    """Key-range-sharded forward on every rank of `group`. `ws` from `kv_sharded_workspace`. With row-slice buffers: local partials ->
    all-to-all of row slices -> combine of the own slice -> all-gather of the bf16 slices; else: local partials -> all-gather of the
    partials -> combine of all rows."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    local_partials(q, k_local, v_local, q_scale, k_scale_local, v_scale, ws["ohat"], ws["lse"])
    if "ohat_recv" in ws:
        exchange_row_slices(ws["ohat"], ws["lse"], ws["ohat_recv"], ws["lse_recv"], group)
        combine_gathered(ws["ohat_recv"], ws["lse_recv"], ws["out_slice"], world)
        gather_output_slices(out, ws["out_slice"], group)
        return
    exchange_partials(ws["ohat"], ws["lse"], ws["ohat_all"], ws["lse_all"], group)
    combine_gathered(ws["ohat_all"], ws["lse_all"], out, world)


class KvShardedPlan:
    """Workspaces and schedule of the key-range-sharded forward for one problem size on one rank (`world` = 1 runs the same two
    kernels without an exchange). `forward` runs a step; `timed_stages` runs steps with CUDA events between the stages."""

    def __init__(self, rows_total: int, world: int, device, group=None):
        self.rows_total, self.world, self.device, self.group = rows_total, world, device, group
        self.ws = kv_sharded_workspace(rows_total, world, device, sliced=True)
        self.sliced = "ohat_recv" in self.ws

    def describe(self) -> str:
        if self.world == 1:
            return "one rank: split kernel over all keys + combine (splits = 1), no exchange"
        if self.sliced:
            return "key-range shards: split kernel -> NCCL all-to-all of the f32 partial row slices and their log-sum-exps -> combine of the own slice -> NCCL all-gather of the bf16 slices"
        return "key-range shards: split kernel -> NCCL all-gather of the f32 partials -> combine of all rows"

    def stages(self, q, k_local, v_local, q_scale, k_scale_local, v_scale, out):
        """The step as a list of (name, callable) in stream order."""
        ws, world = self.ws, self.world
        st = [("split_kernel", lambda: local_partials(q, k_local, v_local, q_scale, k_scale_local, v_scale, ws["ohat"], ws["lse"], check=False))]
        if world == 1:
            st.append(("combine", lambda: combine_gathered(ws["ohat"].view(1, self.rows_total, D), ws["lse"].view(1, self.rows_total), out, 1, check=False)))
        elif self.sliced:
            st.append(("exchange_partials", lambda: exchange_row_slices(ws["ohat"], ws["lse"], ws["ohat_recv"], ws["lse_recv"], self.group)))
            st.append(("combine", lambda: combine_gathered(ws["ohat_recv"], ws["lse_recv"], ws["out_slice"], world, check=False)))
            st.append(("gather_output", lambda: gather_output_slices(out, ws["out_slice"], self.group)))
        else:
            st.append(("exchange_partials", lambda: exchange_partials(ws["ohat"], ws["lse"], ws["ohat_all"], ws["lse_all"], self.group)))
            st.append(("combine", lambda: combine_gathered(ws["ohat_all"], ws["lse_all"], out, world, check=False)))
        return st

    def forward(self, q, k_local, v_local, q_scale, k_scale_local, v_scale, out):
        for _, fn in self.stages(q, k_local, v_local, q_scale, k_scale_local, v_scale, out):
            fn()

    def timed_stages(self, q, k_local, v_local, q_scale, k_scale_local, v_scale, out, reps: int = 5):
        """Median over `reps` steps of the time between the CUDA events that bracket each stage on the launching stream (ms). The ranks
        are lined up by a barrier before each step, so that a stage's time is its own and not the wait for a late peer."""
        import statistics
        import torch
        import torch.distributed as dist
        st = self.stages(q, k_local, v_local, q_scale, k_scale_local, v_scale, out)
        acc = {name: [] for name, _ in st}
        for _ in range(reps):
            if self.world > 1:
                dist.barrier(group=self.group)
            torch.cuda.synchronize(self.device)
            evs = [torch.cuda.Event(enable_timing=True) for _ in range(len(st) + 1)]
            evs[0].record()
            for i, (_, fn) in enumerate(st):
                fn()
                evs[i + 1].record()
            torch.cuda.synchronize(self.device)
            for i, (name, _) in enumerate(st):
                acc[name].append(evs[i].elapsed_time(evs[i + 1]))
        return {name: statistics.median(v) for name, v in acc.items()}

    def close(self):
        self.ws = None
