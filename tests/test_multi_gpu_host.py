"""Host logic of the two shardings, on CPU: two gloo ranks stand in for two GPUs, a float64 numpy partial stands in for the split
kernel, and the oracle's combine and fp64 reference are the checkers. The algebra under test is the reference's KV-split one
(crates/amdgpu-stage/src/components.rs:58-74, crates/amdgpu-tile/src/epilogue.rs:117-146) with split = rank."""
import os
import socket
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from amdgpu_rustdsl_b200 import multi_gpu  # noqa: E402


def test_head_shard_covers_every_head_once():
    for H, HK, world in ((8, 8, 2), (32, 8, 4), (8, 2, 2), (6, 3, 2), (16, 16, 8), (40, 5, 4)):
        seen_h, seen_k = [], []
        for r in range(world):
            (h0, h1), (k0, k1) = multi_gpu.head_shard(H, HK, r, world)
            g = H // HK
            assert (h0, h1) == (k0 * g, k1 * g)      # whole KV-head groups stay together
            seen_h += list(range(h0, h1))
            seen_k += list(range(k0, k1))
        assert seen_h == list(range(H)) and seen_k == list(range(HK))
    with pytest.raises(ValueError):
        multi_gpu.head_shard(6, 4, 0, 2)


def test_kv_range_shard_tiles():
    for SK, world in ((2048, 2), (1337, 2), (65536, 8), (1024, 4), (129, 2)):
        edges = [multi_gpu.kv_range_shard(SK, r, world) for r in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == SK
        for (lo, hi), (lo2, _) in zip(edges, edges[1:]):
            assert hi == lo2 and lo % 128 == 0 and hi > lo
        assert edges[-1][1] > edges[-1][0]
    with pytest.raises(ValueError):
        multi_gpu.kv_range_shard(128, 1, 2)         # one tile cannot feed two ranks
    with pytest.raises(ValueError):
        multi_gpu.kv_range_shard(5 * 128, 3, 4)     # 5 tiles over 4 ranks: tiles per rank 2, rank 3 would be empty


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _dequant(inp, orc):
    tab = orc.e4m3_table()
    B, S, H, SK, HK = inp.B, inp.S, inp.H, inp.SK, inp.HK
    qs = inp.qs[: B * S * H * 4].reshape(B, S, H, 4).astype(np.float64)
    ks = inp.ks[: B * SK * HK * 4].reshape(B, SK, HK, 4).astype(np.float64)
    q = (tab[inp.q].reshape(B, S, H, 4, 32) * (2.0 ** (qs - 127))[..., None]).reshape(B, S, H, 128)
    k = (tab[inp.k].reshape(B, SK, HK, 4, 32) * (2.0 ** (ks - 127))[..., None]).reshape(B, SK, HK, 128)
    return q, k, tab[inp.v]


def _rank_kv(rank, world, port, shape, q_out):
    """One rank of the key-range sharding: local partial over its keys -> exchange_partials (gloo all-gather) -> combine."""
    import torch
    import torch.distributed as dist
    from oracle import oracle as orc
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        B, H, HK, S, SK = shape
        inp = orc.generate("normal", B, H, S, SK, HK)
        q, k, v = _dequant(inp, orc)
        lo, hi = multi_gpu.kv_range_shard(SK, rank, world)
        g = H // HK
        rows_total = B * S * H
        ohat = np.empty((B, S, H, 128), np.float32)
        lse = np.empty((B, S, H), np.float32)
        for b in range(B):
            for h in range(H):
                s = q[b, :, h] @ k[b, lo:hi, h // g].T          # base-2 logits: log2(e)/sqrt(128) is already folded into q
                m = s.max(-1, keepdims=True)
                p = np.exp2(s - m)
                l = p.sum(-1, keepdims=True)
                ohat[b, :, h] = (p @ v[b, lo:hi, h // g]) * inp.vdescale / l
                lse[b, :, h] = (m + np.log2(l))[:, 0]
        t_ohat, t_lse = torch.from_numpy(ohat.reshape(rows_total, 128)), torch.from_numpy(lse.reshape(rows_total))
        ohat_all = torch.empty(world, rows_total, 128)
        lse_all = torch.empty(world, rows_total)
        multi_gpu.exchange_partials(t_ohat, t_lse, ohat_all, lse_all)
        # rank-major layout = [splits][rows_total], what the combine reads
        assert torch.equal(ohat_all[rank], t_ohat) and torch.equal(lse_all[rank], t_lse)
        out = orc.combine_f32(ohat_all.numpy(), lse_all.numpy(), rows_total, world)
        # the all-to-all form: this rank receives and combines only its own slice of the rows, then the bf16 slices are gathered
        n = rows_total // world
        ohat_recv, lse_recv = torch.empty(world, n, 128), torch.empty(world, n)
        multi_gpu.exchange_row_slices(t_ohat, t_lse, ohat_recv, lse_recv)
        assert torch.equal(ohat_recv[rank], t_ohat[rank * n:(rank + 1) * n]) and torch.equal(lse_recv[rank], t_lse[rank * n:(rank + 1) * n])
        mine = orc.combine_f32(ohat_recv.numpy(), lse_recv.numpy(), n, world)
        out_sliced = torch.empty(rows_total, 128)   # gloo has no 16-bit integer gather: the bf16 values as f32
        multi_gpu.gather_output_slices(out_sliced, torch.from_numpy(orc.bf16_to_f32(mine)))
        assert np.array_equal(out_sliced.numpy(), orc.bf16_to_f32(out))      # both exchange forms give the same values
        ref = orc.reference(inp, S)
        st = orc.compare(inp, out.reshape(B, S, H, 128), ref, S)
        q_out.put((rank, st.bad, st.mean_err, st.worst_err, out.tobytes()))
    finally:
        dist.destroy_process_group()


def _slice_heads(inp, hs, ks_, orc):
    (h0, h1), (k0, k1) = hs, ks_
    B, S, SK = inp.B, inp.S, inp.SK
    qs = inp.qs[: B * S * inp.H * 4].reshape(B, S, inp.H, 4)[:, :, h0:h1]
    ks = inp.ks[: B * SK * inp.HK * 4].reshape(B, SK, inp.HK, 4)[:, :, k0:k1]
    pad = np.zeros(1 << 16, np.uint8)     # the kernels' over-read slack behind the scale arrays
    return orc.Inputs(B, h1 - h0, k1 - k0, S, SK, np.ascontiguousarray(inp.q[:, :, h0:h1]), np.ascontiguousarray(inp.k[:, :, k0:k1]),
                      np.ascontiguousarray(inp.v[:, :, k0:k1]), np.concatenate([qs.ravel(), pad]), np.concatenate([ks.ravel(), pad]), inp.vdescale)


def _rank_heads(rank, world, port, shape, q_out):
    """One rank of the head sharding: the path on its own packed head slice; no data-path collective (the gather here only checks)."""
    import torch
    import torch.distributed as dist
    from oracle import oracle as orc
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        B, H, HK, S, SK = shape
        inp = orc.generate("normal", B, H, S, SK, HK)
        hs, ks_ = multi_gpu.head_shard(H, HK, rank, world)
        mine = orc.reference(_slice_heads(inp, hs, ks_, orc), S)          # [B, H_local, S, 128]
        parts = [torch.empty(B, H // world, S, 128, dtype=torch.float64) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(mine))
        full = torch.cat(parts, dim=1).numpy()
        whole = orc.reference(inp, S)
        q_out.put((rank, bool(np.array_equal(full, whole))))
    finally:
        dist.destroy_process_group()


def _spawn(fn, world, shape):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=fn, args=(r, world, port, shape, q_out)) for r in range(world)]
    for p in procs:
        p.start()
    import queue
    import time
    res, deadline = [], time.time() + 240
    while len(res) < world:
        try:
            res.append(q_out.get(timeout=1))
        except queue.Empty:
            assert time.time() < deadline, "ranks timed out"
            assert all(p.exitcode in (None, 0) for p in procs), "a rank failed"   # do not wait for a rank that has died
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    return sorted(res)


@pytest.mark.timeout(300)
def test_kv_range_sharding_two_ranks_gloo():
    res = _spawn(_rank_kv, 2, (1, 4, 2, 48, 640))       # 5 key tiles: ranks own 3 and 2, the last one ragged in tiles
    assert res[0][4] == res[1][4]                       # every rank ends with the same output bytes
    for _, bad, mean_err, worst, _ in res:
        assert bad == 0 and mean_err < 1e-3 and worst < 1e-2     # f32 partials + one bf16 rounding


@pytest.mark.timeout(300)
def test_head_sharding_two_ranks_gloo():
    res = _spawn(_rank_heads, 2, (1, 8, 4, 32, 256))
    assert all(ok for _, ok in res)
