#!/usr/bin/env python
"""Benchmark of the MXFP8 attention forward path (hd128) on B200: TFLOP/s = 4*B*H*Sq*Skv*128 / t, as the reference counts it
(tests/gpu/ref_host.cpp:403).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c1|c2|c3|c4|c5]

One step = one pass of the default path `fmha_fwd_hd128_mxfp8_auto` over one batch of synthetic inputs (the reference harness's
REF_DATA=normal generator). Default workload: BASELINE config 2 (B4 H8 Sq=Skv=2048) on every rank (weak scaling: the (batch x head)
units are independent, no collective). `--workload c4` is the head-sharded B16 H64 S4096 (strong scaling), `--workload c5` the
key-range-sharded Sq 8192 x Skv 131072 with the partial exchange over NCCL, `--workload c3` the forced 8-way KV split on one GPU.
`--impl reference` times the reference's own CPU implementation of the path (its fp64 `check`, built from the reference tree into
oracle/_ref when available, else the CPU restatement in oracle/) on a bounded sample of the same workload.
Prints one JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {  # B, H, HK, Sq, Skv, forced path, splits
    "c1": (1, 2, 2, 256, 256, "auto", None),
    "c2": (4, 8, 8, 2048, 2048, "auto", None),
    "c3": (1, 8, 8, 8192, 8192, "kvsplit", 8),
    "c4": (16, 64, 64, 4096, 4096, "auto", None),
    "c5": (1, 8, 8, 8192, 131072, "kvshard", None),
}
METRIC = "MXFP8 FMHA fwd TFLOP/s (hd128), 4*B*H*Sq*Skv*128 / t"
NOMINAL_MXFP8_TFLOPS = 4500.0
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant (attention) kernel, from the ncu capture summarised in
# profiles/fmha_fwd_mxfp8_kernel_c2.md; only the captured workload has a figure
NCU_DRAM_BYTES_PER_LAUNCH = {"c2": 25.77e6 + 0.01e6}


def flops(B, H, S, SK):
    return 4.0 * B * H * S * SK * 128


def synthetic_inputs(B, H, HK, S, SK, seed):
    """Seeded stand-in for the reference harness's REF_DATA=normal inputs (tests/gpu/ref_host.cpp:214-263), made with torch on the CPU:
    standard-normal Q (pre-multiplied by log2(e)/sqrt(128)), K and V; Q and K quantised to e4m3 with one E8M0 scale per 32 head-dim
    elements, V to e4m3 with one f32 descale. Returns uint8 tensors q [B,S,H,128], k, v [B,SK,HK,128], qs [B*S*H*4], ks [B*SK*HK*4] and the
    V descale."""
    import math
    import torch
    g = torch.Generator().manual_seed(seed)

    def block_quant(x):
        xb = x.view(*x.shape[:-1], 4, 32)
        amax = xb.abs().amax(-1).clamp_min(2.0 ** -100)
        e = torch.floor(torch.log2(amax)) - 8.0          # e4m3 tops out at 1.75 * 2^8
        q = (xb * torch.exp2(-e).unsqueeze(-1)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)
        return q.view(x.shape), (e + 127.0).clamp(0, 254).to(torch.uint8).reshape(-1)

    q, qs = block_quant(torch.randn(B, S, H, 128, generator=g) * (math.log2(math.e) / math.sqrt(128.0)))
    k, ks = block_quant(torch.randn(B, SK, HK, 128, generator=g))
    vf = torch.randn(B, SK, HK, 128, generator=g)
    vd = float(vf.abs().max()) / 448.0
    v = (vf / vd).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)
    return {"q": q, "k": k, "v": v, "qs": qs, "ks": ks}, vd


def measured_peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        return None


class ClockSampler:
    """nvidia-smi sampled every 200 ms during the timed region (reading only)."""
    Q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.p = None
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--id={index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                                      stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.p = None

    def stop(self):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.p.terminate()
        try:
            out, _ = self.p.communicate(timeout=5)
        except Exception:
            self.p.kill()
            out = ""
        sm, mx, reasons, pw = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1])); pw.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "power_w_max": max(pw) if pw else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_sample(workload, rows, use_ref_binary):
    """Times the CPU implementation of the path on `rows` query rows of every (b,h) of the workload. Returns (tflops, seconds, kind, cores)."""
    from oracle import oracle as O
    B, H, HK, S, SK, _, _ = WORKLOADS[workload]
    fl = 4.0 * B * H * min(rows, S) * SK * 128
    if use_ref_binary and os.path.exists(O.REF_HOST):
        # the reference harness generates its inputs in the same process: subtract a run that checks zero rows
        t0 = time.perf_counter(); O.run_ref_host("normal", B, H, S, SK, HK, rows=0, timeout=3000); t_gen = time.perf_counter() - t0
        t0 = time.perf_counter(); O.run_ref_host("normal", B, H, S, SK, HK, rows=rows, timeout=3000); t_all = time.perf_counter() - t0
        dt = max(t_all - t_gen, 1e-6)
        return fl / dt / 1e12, dt, "reference", 1
    inp = O.generate("normal", B, H, S, SK, HK)
    t0 = time.perf_counter()
    O.reference(inp, rows)
    dt = time.perf_counter() - t0
    return fl / dt / 1e12, dt, "port", O.num_threads()


def run_reference_arm(args):
    """The reference's CPU implementation on the host cores. Rank 0 only; other ranks exit at once. Each step is a bounded sample of the
    workload, sized so that warm-up + steps end within about two and a half minutes."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    wl = args.workload
    B, H, HK, S, SK, _, _ = WORKLOADS[wl]
    from oracle import oracle as O
    n = args.warmup + args.steps
    budget = 150.0
    # the reference harness regenerates all inputs in every run (2 x ~2.3 s at config 2), so it is only used for short runs of the small configs
    use_bin = os.path.exists(O.REF_HOST) and wl in ("c1", "c2") and n <= 12 and not args.cpu_rows
    if use_bin:
        rows = S if wl == "c1" else 8
    elif args.cpu_rows:
        rows = args.cpu_rows
    else:
        _, dt8, _, _ = cpu_sample(wl, 8, False)   # calibration
        rows = max(1, min(S, int(8 * (budget / n) / max(dt8, 1e-4) * 0.8)))
    secs = []
    kind, cores = "port", 1
    for i in range(n):
        _, dt, kind, cores = cpu_sample(wl, rows, use_bin)
        if i >= args.warmup:
            secs.append(dt)
    value = flops(B, H, min(rows, S), SK) * len(secs) / sum(secs) / 1e12
    src = "fp64 check of tests/gpu/ref_host.cpp:438-471" + (" (the reference's own binary, stub HIP runtime)" if kind == "reference" else " (CPU restatement, OpenMP)")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1e3 * sum(secs) / len(secs), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64",
            "data": "synthetic (reference harness REF_DATA=normal generator)",
            "config": {"workload": f"{wl}: B{B} H{H} HK{HK} Sq{S} Skv{SK} hd128, non-causal", "sample": f"first {min(rows, S)} query rows of every (batch, head) per step"},
            "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": kind,
                             "sample": f"{min(rows, S)} query rows x {B * H} (batch, head) pairs per step; {src}"},
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def run_quantizer_bench(args):
    """Side bench of the device quantisers in front of the path (not the headline metric): algorithmic GB/s against the measured HBM rate.
    Rows of 128 bf16; per row the Q/K kernel moves 256 + 128 + 4 bytes, the V path 2 x 256 + 128 (a maximum pass and a conversion pass)."""
    import torch
    from amdgpu_rustdsl_b200 import Q_PRESCALE, _abi, quantize_qk, quantize_v
    _abi.load()
    dev = torch.device("cuda", 0)
    rows = args.rows
    g = torch.Generator(device=dev)
    g.manual_seed(1234)
    x = torch.randn(rows, 128, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    out = torch.empty(rows, 128, dtype=torch.uint8, device=dev)
    sc = torch.zeros(rows * 4, dtype=torch.uint8, device=dev)
    vd = torch.zeros(1024, dtype=torch.float32, device=dev)
    peaks = measured_peaks()
    peak = float(peaks["hbm_gbs"]) if peaks else 6650.0
    res = {}
    for name, fn, nbytes in (("quantize_qk", lambda: quantize_qk(x, out, sc, mul=Q_PRESCALE), rows * 388), ("quantize_v", lambda: quantize_v(x, out, vd), rows * 640)):
        for _ in range(max(3, args.warmup)):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        res[name] = {"ms": ms, "gbs": nbytes / (ms * 1e-3) / 1e9, "bytes": nbytes}
    # CPU beside it: the oracle's restatement of the same rule on a sample of the rows (one core)
    from oracle import oracle as O
    n = min(rows, 65536)
    xs = x[:n].float().cpu().numpy()
    t0 = time.perf_counter()
    O.quantize_rows(xs, Q_PRESCALE)
    dt = time.perf_counter() - t0
    line = {"metric": "MXFP8 quantiser (bf16 -> e4m3 + E8M0 per 32) algorithmic GB/s", "value": res["quantize_qk"]["gbs"], "unit": "GB/s", "n_gpus": 1,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": res["quantize_qk"]["ms"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16 -> u8 (e4m3) + u8 (E8M0)", "data": "synthetic (seeded standard-normal bf16)",
            "config": {"workload": f"quantiser: {rows} rows of 128 bf16 ({rows * 256 / 2**20:.0f} MiB in, larger than L2)"},
            "roofline": {"bound": "hbm", "achieved": res["quantize_qk"]["gbs"], "peak": peak, "unit": "GB/s", "frac": res["quantize_qk"]["gbs"] / peak,
                         "traffic": None, "peak_source": "measured HBM copy rate (MEASURED_PEAKS.json)" if peaks else "fallback 6.65 TB/s"},
            "quantize_v": {"ms_per_step": res["quantize_v"]["ms"], "achieved": res["quantize_v"]["gbs"], "frac": res["quantize_v"]["gbs"] / peak},
            "cpu_baseline": {"value": n * 388 / dt / 1e9, "unit": "GB/s", "cores": 1, "kind": "port", "sample": f"oracle_quantize_rows on the first {n} rows"},
            "gpu_launches": args.steps}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--quantizer", action="store_true", help="side bench: the device quantisers in front of the path (not the headline metric)")
    ap.add_argument("--rows", type=int, default=4194304, help="rows of 128 bf16 for --quantizer")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--cpu-rows", type=int, default=0, help="query rows per (b,h) of the CPU baseline sample (0 = default)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--sets", type=int, default=0, help="number of rotating input sets (0 = enough to exceed L2)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.quantizer:
        return run_quantizer_bench(args)

    import torch
    import torch.distributed as dist
    from amdgpu_rustdsl_b200 import _abi, device_status, fmha_fwd_mxfp8, multi_gpu

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _abi.load()

    wl = args.workload
    B, H, HK, S, SK, path, splits = WORKLOADS[wl]
    scaling = "weak"
    if wl == "c4":   # strong scaling: heads dealt out over the ranks
        (h0, h1), (k0, k1) = multi_gpu.head_shard(H, HK, rank, world)
        Hl, HKl, SKl = h1 - h0, k1 - k0, SK
        scaling = "strong"
    elif wl == "c5":   # strong scaling: key range dealt out over the ranks
        lo, hi = multi_gpu.kv_range_shard(SK, rank, world)
        Hl, HKl, SKl = H, HK, hi - lo
        scaling = "strong"
    else:
        Hl, HKl, SKl = H, HK, SK
    total_flops = flops(B, H, S, SK) * (world if scaling == "weak" else 1)

    # ---- synthetic inputs: the reference generator at the rank's local shape (seeded, deterministic); rotated so that the timed loop never
    # re-reads a set that is still in the 126 MB L2
    bytes_per_set = B * S * Hl * 128 * 3 + 2 * B * SKl * HKl * 128
    nsets = args.sets or max(2, min(16, -(-160 * 2 ** 20 // bytes_per_set)))
    if wl in ("c4", "c5"):
        nsets = args.sets or 1   # one set already exceeds L2
    # generate one batch element (and at most 8192 keys) on the CPU and tile it: the arithmetic does not depend on the values repeating
    gen_B = 1 if wl == "c4" else B
    gen_SK = min(SKl, 8192)
    rep, krep = B // gen_B, SKl // gen_SK
    assert gen_B * rep == B and gen_SK * krep == SKl
    gen, vdescale = synthetic_inputs(gen_B, Hl, HKl, S, gen_SK, seed=1234 + rank)
    host = {"q": gen["q"].repeat(rep, 1, 1, 1), "k": gen["k"].repeat(rep, krep, 1, 1), "v": gen["v"].repeat(rep, krep, 1, 1)}
    qs = torch.zeros(B * S * Hl * 4 + 512 * Hl * 4, dtype=torch.uint8)
    qs[: B * S * Hl * 4] = gen["qs"].repeat(rep)
    ks = torch.zeros(B * SKl * HKl * 4 + 640 * Hl * 4, dtype=torch.uint8)
    ks[: B * SKl * HKl * 4] = gen["ks"].view(gen_B, gen_SK * HKl * 4).repeat(rep, krep).reshape(-1)
    host["qs"], host["ks"] = qs, ks
    host = {n: t.contiguous().pin_memory() for n, t in host.items()}
    sets = []
    for _ in range(nsets):
        s = {n: t.to(dev, non_blocking=True) for n, t in host.items()}
        s["vs"] = torch.zeros(1024, dtype=torch.float32, device=dev)
        s["vs"][0] = vdescale
        s["out"] = torch.empty(B, S, Hl, 128, dtype=torch.bfloat16, device=dev)
        sets.append(s)
    out_host = torch.empty(B, S, Hl, 128, dtype=torch.bfloat16).pin_memory()
    rows_total = B * S * Hl
    ws = None
    if wl == "c5":
        ws = multi_gpu.kv_sharded_workspace(rows_total, world, dev)
    torch.cuda.synchronize()

    launches_per_step = 1
    ran = {}

    def step(s):
        if wl == "c5":
            if world > 1:
                multi_gpu.fmha_fwd_mxfp8_kv_sharded(s["q"], s["k"], s["v"], s["qs"], s["ks"], s["vs"], s["out"], ws)
            else:
                multi_gpu.local_partials(s["q"], s["k"], s["v"], s["qs"], s["ks"], s["vs"], ws["ohat"], ws["lse"], check=False)
                multi_gpu.combine_gathered(ws["ohat"].view(1, rows_total, 128), ws["lse"].view(1, rows_total), s["out"], 1, check=False)
            ran["path"] = ("kvshard", world)
        else:
            ran["path"] = fmha_fwd_mxfp8(s["q"], s["k"], s["v"], s["qs"], s["ks"], s["vs"], s["out"], path=path, splits=splits)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, nwarm, nsteps, join=None):
        for i in range(nwarm):
            fn(i)
        if join:
            join()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(nsteps):
            fn(nwarm + i)
        if join:
            join()   # the launching stream waits for the copy streams: the end event covers the last read-back
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    W, K = max(args.warmup, 3), args.steps
    sampler = ClockSampler(local_rank) if rank == 0 else None
    # ---- device-resident timing: inputs already in HBM
    ms_total = timed(lambda i: step(sets[i % nsets]), W, K)
    if ran["path"][0] in ("kvsplit", "kvshard"):
        launches_per_step = 2
    # ---- end to end through the public entry: every step copies its inputs from pinned host memory and reads the result back
    h2d = sum(host[n].numel() for n in ("q", "k", "v", "qs", "ks"))
    d2h = out_host.numel() * 2

    # The steps are pipelined the way a caller with a queue of requests would: one stream copies step i + 1's inputs in and another reads
    # step i - 1's result back while step i computes; every step still pays its own host-to-device and device-to-host copies in the region.
    main = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    ev_in = [torch.cuda.Event() for _ in sets]
    ev_done = [torch.cuda.Event() for _ in sets]
    ev_out = [torch.cuda.Event() for _ in sets]
    out_hosts = [out_host] + [torch.empty_like(out_host).pin_memory() for _ in sets[1:]]

    def e2e_step(i):
        k = i % nsets
        s = sets[k]
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_done[k])      # the set's previous step has consumed its inputs
            for n in ("q", "k", "v", "qs", "ks"):
                s[n].copy_(host[n], non_blocking=True)
            ev_in[k].record(s_in)
        main.wait_event(ev_in[k])
        main.wait_event(ev_out[k])           # the set's previous result has been read back
        step(s)
        ev_done[k].record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done[k])
            out_hosts[k].copy_(s["out"], non_blocking=True)
            ev_out[k].record(s_out)

    def e2e_join():
        main.wait_stream(s_in)
        main.wait_stream(s_out)

    Ke = max(3, min(K, 50))
    ms_e2e = timed(e2e_step, 3, Ke, e2e_join)
    clocks = sampler.stop() if sampler else None
    status = device_status()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    ms_per_step = ms_total / K
    value = total_flops / (ms_per_step * 1e-3) / 1e12
    e2e_value = total_flops / (ms_e2e / Ke * 1e-3) / 1e12
    peaks = measured_peaks()
    # dominant kernel = the attention kernel; its algorithmic FLOPs per launch are this rank's 4*B*H*Sq*Skv*128
    per_gpu_flops = flops(B, Hl, S, SKl)
    achieved = per_gpu_flops / (ms_per_step * 1e-3) / 1e12
    if peaks:
        peak, peak_src = 2.0 * float(peaks["bf16_tflops"]), "2 x measured dense bf16 burst (MEASURED_PEAKS.json): fp8 tensor rate is twice bf16"
    else:
        peak, peak_src = 2.0 * 1590.0, "2 x fallback dense bf16 (1.59 PFLOP/s)"
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get(wl) if world == 1 else None, "traffic_unit": "bytes per launch (ncu, DRAM read + write)",
                "algorithmic_bytes": B * Hl * S * (128 + 4 + 256) + 2 * B * HKl * SKl * 128 + B * HKl * SKl * 4, "peak_source": peak_src,
                "frac_of_nominal_4500": achieved / NOMINAL_MXFP8_TFLOPS, "note": "achieved = 4*B*H*Sq*Skv*128 per launch / mean step time (CUDA events); for kvsplit steps the combine launch is inside the step"}
    # issue-only ceiling of the tensor pipe, measured now: one thread per SM issues M128 N128 K32 fp8 MMAs on resident operands in a tight loop
    try:
        import ctypes as C
        ms = C.c_float(0)
        lib = _abi.load()
        if lib.fmha_mxfp8_probe_mma_peak(9, 8000, 148, None, C.byref(ms)) == 0 and ms.value > 0:
            roofline["mma_issue_ceiling_tflops"] = 148 * 8000 * 4 * 2.0 * 128 * 128 * 32 / (ms.value * 1e-3) / 1e12
    except Exception:
        pass
    line = {"metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": scaling, "vs_baseline": None, "dtype": "fp8-e4m3 x E8M0 block scales (MXFP8), f32 accumulate, bf16 out", "data": "synthetic (seeded standard-normal Q/K/V quantised to MXFP8 on the host, the distribution of the reference harness's REF_DATA=normal)",
            "config": {"workload": f"{wl}: B{B} H{H} HK{HK} Sq{S} Skv{SK} hd128, non-causal" + (f", per rank (x{world} ranks)" if scaling == "weak" and world > 1 else ""),
                       "path": ran["path"][0], "splits": ran["path"][1], "l2": f"{nsets} rotating input/output sets of {bytes_per_set / 2**20:.0f} MiB (> 126 MB L2 in total)",
                       "parallelism": "none" if world == 1 else ("batch x head shards, no collective" if wl != "c5" else "key-range shards + NCCL all-to-all of partial row slices + combine + all-gather of the bf16 slices")},
            "roofline": roofline, "gpu_launches": K * launches_per_step, "device_status": status,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": Ke, "ms_per_step": ms_e2e / Ke},
            "clocks": clocks}
    if not args.no_cpu and world == 1:
        rows = args.cpu_rows
        if not rows:   # about 10-20 s of CPU work: calibrate on 8 rows
            _, dt8, _, _ = cpu_sample(wl, 8, False)
            rows = max(1, min(S, int(8 * 12.0 / max(dt8, 1e-4))))
        v, dt, kind, cores = cpu_sample(wl, rows, False)
        line["cpu_baseline"] = {"value": v, "unit": "TFLOP/s", "cores": cores, "kind": kind, "seconds": dt,
                                "sample": f"fp64 oracle on the first {min(rows, S)} query rows of every (batch, head) of the same workload"}
    else:
        line["cpu_baseline"] = None
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
