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


def local_partials(q, k_local, v_local, q_scale, k_scale_local, v_scale, ohat, lse, *, stream=None, check=True, peer_plan=None, f32_partials=True):
    """One rank's contribution to a key-range-sharded forward: the split kernel with splits = 1 over the local keys, writing the
    normalised partial O [rows_total,128] (f32, or f16 with ``f32_partials=False``) and base-2 log-sum-exp [rows_total] of all queries.
    With ``peer_plan`` (a device plan built for the same partial format) the rows go to the GPUs that combine them instead."""
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
    a = fill_common(_abi.KvSplitArgs(), q, k_local, v_local, q_scale, k_scale_local, v_scale, ohat, B, S, H, SKl, HK,
                    flags=_abi.FLAG_F32_PARTIALS if f32_partials else 0)
    a.ptr_o = None
    a.ptr_ohat, a.ptr_lse, a.kvs_splits, a.kvs_rows_total = ohat.data_ptr(), lse.data_ptr(), 1, rows_total
    sizes = _abi.BufferSizes(ptr_q=_nbytes(q), ptr_k=_nbytes(k_local), ptr_v=_nbytes(v_local), ptr_o=B * S * H * 256, ptr_q_descale=_nbytes(q_scale),
                             ptr_k_descale=_nbytes(k_scale_local), ptr_v_descale=_nbytes(v_scale), ptr_ohat=_nbytes(ohat), ptr_lse=_nbytes(lse))
    if not f32_partials:
        # the contract sizes ptr_ohat for f32 rows whatever the kernel writes; this helper's f16 buffers hold exactly the f16 rows
        sizes.ptr_ohat = 2 * _nbytes(ohat)
    if peer_plan is not None:
        # the partial rows go to the GPUs that combine them (fmha_mxfp8_peer_plan_build): ohat / lse are not written and only stand in
        # for the contract's pointer fields; their extents are not this launch's concern
        a.ext_ptr_peer_plan = peer_plan
        sizes.ptr_ohat, sizes.ptr_lse = rows_total * 512, rows_total * 4
    syms = _abi.Symbols(B=B, HK=HK, KL=0)
    with torch.cuda.device(q.device):
        _check_launch(lib, _abi.KVSPLIT, a, sizes, _abi.grid3(math.ceil(S / 256), H, B), syms, stream, check)


def combine_gathered(ohat_all, lse_all, out, world: int, *, stream=None, check=True):
    """The combine kernel over the gathered partials: ohat_all f32 or f16 [world, rows_total, 128], lse_all f32 [world, rows_total] -> bf16 out."""
    import ctypes as C
    import torch
    from . import _abi
    lib = _abi.load()
    rows_total = out.numel() // D
    if stream is None:
        stream = torch.cuda.current_stream(out.device).cuda_stream
    if ohat_all.dtype not in (torch.float32, torch.float16) or lse_all.dtype != torch.float32 or out.dtype != torch.bfloat16:
        raise ValueError("combine_gathered: f32 or f16 partials, f32 log-sum-exps, bf16 output")
    if check and (ohat_all.numel() < world * rows_total * D or lse_all.numel() < world * rows_total):
        raise ValueError("combine_gathered: partial buffers smaller than world x rows_total")
    with torch.cuda.device(out.device):
        if ohat_all.dtype == torch.float32:
            rc = lib.fmha_mxfp8_combine_f32(ohat_all.data_ptr(), lse_all.data_ptr(), out.data_ptr(), rows_total, world, C.c_void_p(stream))
        else:   # the reference's own combine8h over f16 partials
            c = _abi.CombineArgs(ptr_ohat=ohat_all.data_ptr(), ptr_lse=lse_all.data_ptr(), ptr_out=out.data_ptr(), rows_total=rows_total, d=D, splits=world)
            rc = lib.fmha_mxfp8_launch(_abi.COMBINE8H, C.byref(c), _abi.grid3(max(1, math.ceil(rows_total * D / (256 * 8))), 1, 1), C.c_void_p(stream))
    if rc:
        raise RuntimeError(f"the combine failed with code {rc}")


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


class PeerBuffers:
    """One device allocation per rank that every process of the node maps (CUDA IPC through the library's fmha_mxfp8_peer_* entries), cut
    into this rank's receive slots for the partials [world][n][128] (f16 or f32), for their log-sum-exps [world][n] f32, and a whole bf16 output
    [rows_total][128] that every rank's combine stores its row slice into. `ptr[r]` is rank r's allocation as mapped here."""

    def __init__(self, rows_total: int, world: int, rank: int, device, group=None, f32_partials: bool = True):
        """Collective over `group`: every rank allocates, the ranks agree that all succeeded, exchange the handles, map each other's
        buffers and agree again. `ok` tells whether the buffers are usable on every rank; a rank never stops half way through the
        collectives, whatever failed locally."""
        import ctypes as C
        import torch
        import torch.distributed as dist
        from . import _abi
        self.lib = lib = _abi.load()
        self.world, self.rank, self.device = world, rank, device
        n = rows_total // world
        self.n = n
        al = lambda x: (x + 255) // 256 * 256   # noqa: E731
        self.f32_partials = f32_partials
        self.off_lse = al(world * n * D * (4 if f32_partials else 2))
        self.off_out = self.off_lse + al(world * n * 4)
        self.off_flags = self.off_out + al(rows_total * D * 2)   # [world] uint32 arrival flags of the barrier between the GPUs (zero at first)
        self.bytes = self.off_flags + 256
        self.own = C.c_void_p()
        handle = (C.c_ubyte * _abi.PEER_HANDLE_BYTES)()
        self.ptr, self.opened, self.error = [None] * world, [], None

        def agree(flag):
            t = torch.tensor([1 if flag else 0], dtype=torch.int32, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group)
            return int(t.item()) == 1

        with torch.cuda.device(device):
            rc = lib.fmha_mxfp8_peer_alloc(self.bytes, C.byref(self.own), handle)
            if rc:
                self.error = f"fmha_mxfp8_peer_alloc failed with code {rc}"
                self.own = None
            self.ok = agree(rc == 0)
            if not self.ok:
                return
            handles = [None] * world
            dist.all_gather_object(handles, bytes(handle), group=group)
            good = True
            for r in range(world):
                if r == rank:
                    self.ptr[r] = self.own.value
                    continue
                hp = (C.c_ubyte * _abi.PEER_HANDLE_BYTES).from_buffer_copy(handles[r])
                q = C.c_void_p()
                rc = lib.fmha_mxfp8_peer_open(hp, C.byref(q))
                if rc:
                    self.error = f"fmha_mxfp8_peer_open(rank {r}) failed with code {rc}"
                    good = False
                    break
                self.ptr[r] = q.value
                self.opened.append(q.value)
            self.ok = agree(good)

    def close(self, group=None):
        """Unmap the peers' buffers, wait for every rank to have done so, free the own one."""
        import ctypes as C
        import torch
        import torch.distributed as dist
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            dist.barrier(group=group)   # no rank is still storing into another's buffer
            for q in self.opened:
                self.lib.fmha_mxfp8_peer_close(C.c_void_p(q))
            self.opened = []
            dist.barrier(group=group)
            if self.own is not None and self.own.value:
                self.lib.fmha_mxfp8_peer_free(self.own)
                self.own = None


class KvShardedPlan:
    """Workspaces and schedule of the key-range-sharded forward for one problem size on one rank (`world` = 1 runs the same two
    kernels without an exchange). `forward` runs a step; `timed_stages` runs steps with CUDA events between the stages.

    transport "peer" (one batch element, S / world a multiple of 128 rows): the split kernel stores each row block of its partial
    (``partials`` "f32", or "f16", the reference's partial format and half the bytes over NVLink; measured no faster) straight into the memory of the GPU that
    combines it, as the block leaves tensor memory (no collective moves partials; the transfer runs under the remaining compute); barrier;
    every GPU's combine stores its bf16 row slice into every GPU's output; barrier.
    transport "nccl": split kernel -> all-to-all of the partial row slices -> combine of the own slice -> all-gather of the bf16 slices
    (or, when the rows do not divide, an all-gather of the whole partials)."""

    def __init__(self, rows_total: int, world: int, device, group=None, transport: str = "auto", B: int = 1, S: int = 0, H: int = 0, partials: str = "f32",
                 barrier: str = "flags", barrier_timeout_s: float = 30.0):
        import torch
        if partials not in ("f16", "f32"):
            raise ValueError("partials: 'f16' or 'f32'")
        self.rows_total, self.world, self.device, self.group = rows_total, world, device, group
        self.f32_partials = partials == "f32"   # of the peer transport; the NCCL exchange moves f32
        if barrier not in ("flags", "nccl"):
            raise ValueError("barrier: 'flags' (arrival flags in the peer buffers) or 'nccl' (an all-reduce of one float)")
        self.flag_barrier, self.arrivals = barrier == "flags", 0
        # how long a rank waits for the others at a flag barrier before it gives up (sets bit 1 of the device status word and goes on): ranks
        # may reach a step seconds apart (data loading), a rank that is gone never arrives
        self.barrier_budget_us = int(min(max(barrier_timeout_s, 0.001), 4000.0) * 1e6)
        self.transport = "none" if world == 1 else "nccl"
        self.peer = None
        if world > 1 and transport in ("auto", "peer"):
            ok = B == 1 and S > 0 and H > 0 and S * H == rows_total and S % world == 0 and (S // world) % 128 == 0
            if ok:
                self._setup_peer(S, H)
            elif transport == "peer":
                raise ValueError("the peer transport needs one batch element and S / world a multiple of 128")
        self.ws = kv_sharded_workspace(rows_total, world, device, sliced=True) if self.transport != "peer" else {
            "ohat": torch.empty(1, dtype=torch.float32, device=device), "lse": torch.empty(1, dtype=torch.float32, device=device)}
        self.sliced = "ohat_recv" in self.ws

    def _setup_peer(self, S, H):
        """All ranks try; the transport is used only if every rank succeeded (a rank that cannot map its peers must not leave the others
        storing into its memory)."""
        import ctypes as C
        import torch
        import torch.distributed as dist
        from . import _abi
        rank = dist.get_rank(self.group)
        self.peer = PeerBuffers(self.rows_total, self.world, rank, self.device, self.group, self.f32_partials)
        good, err = self.peer.ok, self.peer.error
        if good:
            try:
                self.plan_dev = torch.zeros(_abi.PEER_PLAN_BYTES + 128, dtype=torch.uint8, device=self.device)
                self.plan_ptr = (self.plan_dev.data_ptr() + 127) // 128 * 128
                pb = self.peer
                ohat = (C.c_void_p * self.world)(*[pb.ptr[r] for r in range(self.world)])
                lse = (C.c_void_p * self.world)(*[pb.ptr[r] + pb.off_lse for r in range(self.world)])
                with torch.cuda.device(self.device):
                    rc = pb.lib.fmha_mxfp8_peer_plan_build(self.world, rank, H, S, 1 if self.f32_partials else 0, ohat, lse, C.c_void_p(self.plan_ptr), None)
                if rc:
                    raise RuntimeError(f"fmha_mxfp8_peer_plan_build failed with code {rc}")
                self.outs = (C.c_void_p * self.world)(*[pb.ptr[r] + pb.off_out for r in range(self.world)])
                self.flag_arrays = (C.c_void_p * self.world)(*[pb.ptr[r] + pb.off_flags for r in range(self.world)])
                self.flag = torch.zeros(1, dtype=torch.float32, device=self.device)
            except Exception as e:   # noqa: BLE001
                good, err = False, repr(e)
        t = torch.tensor([1 if good else 0], dtype=torch.int32, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.group)
        if int(t.item()) == 1:
            self.transport = "peer"
        else:
            self.peer_error = err or "another rank could not set the peer buffers up"
            self.peer.close(self.group)
            self.peer = None

    def describe(self) -> str:
        if self.world == 1:
            return "one rank: split kernel over all keys + combine (splits = 1), no exchange"
        if self.transport == "peer":
            return (f"key-range shards: the split kernel stores its {'f32' if self.f32_partials else 'f16'} partial row blocks into the combining GPU's memory over NVLink as they leave tensor memory "
                    "-> barrier -> every GPU's combine stores its bf16 row slice into every GPU's output -> barrier (no collective moves data; barrier = "
                    + ("arrival flags in peer memory)" if self.flag_barrier else "NCCL all-reduce of one float)"))
        if self.sliced:
            return "key-range shards: split kernel -> NCCL all-to-all of the f32 partial row slices and their log-sum-exps -> combine of the own slice -> NCCL all-gather of the bf16 slices"
        return "key-range shards: split kernel -> NCCL all-gather of the f32 partials -> combine of all rows"

    def output(self):
        """Peer transport: this rank's whole bf16 output [rows_total, 128] where the combines of all ranks store it (a view of the peer buffer, no
        copy). Valid after `forward(..., out=None)` until the next `forward`; gone after `close`."""
        import torch
        if self.transport != "peer":
            raise ValueError("output(): only the peer transport keeps the output in a buffer of its own")

        class _View:   # the CUDA array interface of the output region; bf16 has no typestr of its own: 16-bit words, viewed as bf16 below
            __cuda_array_interface__ = {"shape": (self.rows_total, D), "typestr": "<i2", "data": (self.peer.own.value + self.peer.off_out, False), "version": 3,
                                        "strides": None}

        return torch.as_tensor(_View(), device=self.device).view(torch.bfloat16)

    def _barrier(self):
        """The ranks line up on the stream (what follows on the stream starts after every rank got here): arrival flags in the peer buffers,
        written and polled by a one-warp kernel per GPU (`fmha_mxfp8_peer_barrier`, bounded wait of `barrier_timeout_s`), or an all-reduce of one float."""
        if self.flag_barrier:
            import ctypes as C
            import torch
            self.arrivals += 1
            with torch.cuda.device(self.device):
                rc = self.peer.lib.fmha_mxfp8_peer_barrier(self.flag_arrays, self.world, self.peer.rank, self.arrivals, self.barrier_budget_us, None,
                                                           C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream))
            if rc:
                raise RuntimeError(f"fmha_mxfp8_peer_barrier failed with code {rc}")
            return
        import torch.distributed as dist
        dist.all_reduce(self.flag, group=self.group)

    def stages(self, q, k_local, v_local, q_scale, k_scale_local, v_scale, out):
        """The step as a list of (name, callable) in stream order. Peer transport: `out` may be None, the result is then `output()` and
        the copy into a tensor of the caller's is left out."""
        ws, world = self.ws, self.world
        if self.transport == "peer":
            import ctypes as C
            import torch
            pb = self.peer
            stream = lambda: C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)   # noqa: E731

            def combine():
                with torch.cuda.device(self.device):
                    rc = pb.lib.fmha_mxfp8_combine_scatter(C.c_void_p(pb.own.value), 1 if self.f32_partials else 0, C.c_void_p(pb.own.value + pb.off_lse), self.outs, world,
                                                           pb.rank * pb.n, pb.n, world, stream())
                if rc:
                    raise RuntimeError(f"fmha_mxfp8_combine_scatter failed with code {rc}")

            def take_output():
                with torch.cuda.device(self.device):
                    rc = pb.lib.fmha_mxfp8_copy_async(C.c_void_p(out.data_ptr()), C.c_void_p(pb.own.value + pb.off_out), self.rows_total * D * 2, stream())
                if rc:
                    raise RuntimeError(f"fmha_mxfp8_copy_async failed with code {rc}")

            st = [("split_kernel_storing_to_peers", lambda: local_partials(q, k_local, v_local, q_scale, k_scale_local, v_scale, ws["ohat"], ws["lse"], check=False,
                                                                          peer_plan=self.plan_ptr, f32_partials=self.f32_partials)),
                  ("barrier", self._barrier), ("combine_storing_to_peers", combine), ("barrier_2", self._barrier)]
            if out is not None:
                st.append(("copy_out", take_output))
            return st
        if out is None:
            raise ValueError("only the peer transport runs without an output tensor")
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
        import torch
        torch.cuda.synchronize(self.device)
        if self.peer is not None:
            self.peer.close(self.group)
            self.peer = None
        self.ws = None
