#!/usr/bin/env python
"""Benchmark of the MXFP8 attention forward path (hd128) on B200: TFLOP/s = 4*B*H*Sq*Skv*128 / t, as the reference counts it
(tests/gpu/ref_host.cpp:403).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c1|c2|c3|c4|c5] [--no-sharded]

One step = one pass of the default path `fmha_fwd_hd128_mxfp8_auto` over one batch of synthetic inputs. The line's headline (`value`,
`e2e`, `roofline`) is the reference's headline gate shape B4 H8 Sq=Skv=2048 on every rank (weak scaling: (batch x head) units are
independent, no collective). The same line carries a `sharded` object with the two configurations that do shard across the GPUs of a
node, measured at this N: B16 H64 S4096 dealt out by head (no collective) and B1 H8 Sq8192 Skv131072 dealt out by key range (partials
exchanged between the GPUs, then the combine kernel), each with a parity check of a row sample of its output against the CPU oracle.

Timing protocol (after the reference's, tools/port_gate.sh:163-187, docs/perf-matrix.md:9-13: warm-up, then one event pair around a
window of launches, median of 5 windows): every figure is the median of 5 windows; a window is at least K steps, at least 100 steps and
at least 50 ms for the headline (fewer steps for the long sharded configurations, see `config.timing`); each window is bracketed by a
barrier and a device synchronize, timed with CUDA events on the launching stream, and the maximum over the ranks is taken per window.
`--impl reference` times the reference's own CPU implementation of the path (its fp64 `check`: the reference harness built from the
reference tree into oracle/_ref where available, one process per host core; else the OpenMP restatement in oracle/).
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
N_WINDOWS = 5
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the attention kernel on B4 H8 S2048, a constant recorded from an ncu
# capture of that launch (summary under profiles/); the run itself does not measure DRAM traffic
RECORDED_NCU_DRAM_BYTES = {"c2": 25.78e6}
V_DESCALE_FIXED = 6.0 / 448.0   # key-range shards must agree on the V descale without talking: 6 sigma of N(0,1), larger values saturate


def flops(B, H, S, SK):
    return 4.0 * B * H * S * SK * 128


def synthetic_inputs(B, H, HK, S, SK, seed, kv_seed=None, vdescale=None, want_q=True):
    """Seeded stand-in for the reference harness's REF_DATA=normal inputs (tests/gpu/ref_host.cpp:214-263), made with torch on the CPU:
    standard-normal Q (pre-multiplied by log2(e)/sqrt(128)), K and V; Q and K quantised to e4m3 with one E8M0 scale per 32 head-dim
    elements, V to e4m3 with one f32 descale. Returns uint8 tensors q [B,S,H,128], k, v [B,SK,HK,128], qs [B*S*H*4], ks [B*SK*HK*4] and the
    V descale. `kv_seed` draws K and V from a stream of their own (key-range shards share Q and differ in K / V)."""
    import math
    import torch
    g = torch.Generator().manual_seed(seed)

    def block_quant(x):
        xb = x.view(*x.shape[:-1], 4, 32)
        amax = xb.abs().amax(-1).clamp_min(2.0 ** -100)
        e = torch.floor(torch.log2(amax)) - 8.0          # e4m3 tops out at 1.75 * 2^8
        q = (xb * torch.exp2(-e).unsqueeze(-1)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)
        return q.view(x.shape), (e + 127.0).clamp(0, 254).to(torch.uint8).reshape(-1)

    res = {}
    if want_q:
        res["q"], res["qs"] = block_quant(torch.randn(B, S, H, 128, generator=g) * (math.log2(math.e) / math.sqrt(128.0)))
    if kv_seed is not None:
        g = torch.Generator().manual_seed(kv_seed)
    res["k"], res["ks"] = block_quant(torch.randn(B, SK, HK, 128, generator=g))
    vf = torch.randn(B, SK, HK, 128, generator=g)
    vd = float(vf.abs().max()) / 448.0 if vdescale is None else vdescale
    res["v"] = (vf / vd).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)
    return res, vd


def measured_peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        return None


class ClockSampler:
    """nvidia-smi sampled every 50 ms during a timed region (reading only)."""
    Q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.p = None
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--id={index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50"],
                                      stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.p = None

    def stop(self):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
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
        # the first samples precede the load: the median over the samples at or above 300 W, or over all when the load never got there
        loaded = [c for c, p in zip(sm, pw) if p >= 300.0]
        return {"sm_mhz": statistics.median(loaded or sm) if sm else None, "sm_mhz_min": min(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------------------------------------------- CPU legs

def host_cores():
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


def cpu_port_sample(workload, rows):
    """The OpenMP restatement of the reference's fp64 `check` on `rows` query rows of every (b,h). Returns (tflops, seconds, cores)."""
    from oracle import oracle as O
    B, H, HK, S, SK, _, _ = WORKLOADS[workload]
    cores = O.set_threads(host_cores())   # torch.distributed.run exports OMP_NUM_THREADS=1: ask for the host's cores explicitly
    inp = O.generate("normal", B, H, S, SK, HK)
    t0 = time.perf_counter()
    O.reference(inp, rows)
    dt = time.perf_counter() - t0
    return 4.0 * B * H * min(rows, S) * SK * 128 / dt / 1e12, dt, cores


def ref_binary_wall(workload, rows, procs):
    """Wall time of `procs` concurrent runs of the reference's own harness (single-threaded as the reference wrote it), each generating
    the workload's inputs and checking the first `rows` rows of every (b,h) with its fp64 `check`."""
    from oracle import oracle as O
    B, H, HK, S, SK, _, _ = WORKLOADS[workload]
    env = dict(os.environ, REF_DATA="normal", REF_B=str(B), REF_H=str(H), REF_S=str(S), REF_SK=str(SK), REF_HK=str(HK), REF_ROWS=str(rows))
    t0 = time.perf_counter()
    ps = [subprocess.Popen([O.REF_HOST, "stub.co"], env=env, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL) for _ in range(procs)]
    for p in ps:
        p.wait(timeout=3000)
    return time.perf_counter() - t0


def run_reference_arm(args):
    """The reference's CPU implementation of the path on the host cores. Rank 0 only; other ranks exit at once. Each step is a bounded
    sample of the workload, sized so that warm-up + steps end within about two and a half minutes."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    wl = args.workload
    B, H, HK, S, SK, _, _ = WORKLOADS[wl]
    from oracle import oracle as O
    n = args.warmup + args.steps
    budget = 150.0
    cores = host_cores()
    use_bin = os.path.exists(O.REF_HOST) and wl in ("c1", "c2") and not args.cpu_rows
    secs = []
    if use_bin:
        # one harness process per core, all checking the same rows of the same generated inputs: the harness regenerates its inputs in
        # every run, so a run that checks zero rows is timed first and subtracted
        rows = S if wl == "c1" else 16
        t_gen = min(ref_binary_wall(wl, 0, cores) for _ in range(2))
        per_step = max(ref_binary_wall(wl, rows, cores) - t_gen, 1e-3)
        n_eff = max(2, min(n, int(budget / (per_step + t_gen))))
        for i in range(n_eff):
            dt = max(ref_binary_wall(wl, rows, cores) - t_gen, 1e-6)
            if i >= min(args.warmup, n_eff - 1):
                secs.append(dt)
        work = cores * flops(B, H, min(rows, S), SK)
        kind, binary = "reference", "oracle/_ref/ref_host: the reference's tests/gpu/ref_host.cpp built against a stub HIP runtime, %d concurrent single-threaded processes" % cores
    else:
        if args.cpu_rows:
            rows = args.cpu_rows
        else:
            _, dt8, _ = cpu_port_sample(wl, 8)   # calibration
            rows = max(1, min(S, int(8 * (budget / n) / max(dt8, 1e-4) * 0.8)))
        for i in range(n):
            _, dt, cores = cpu_port_sample(wl, rows)
            if i >= args.warmup:
                secs.append(dt)
        work = flops(B, H, min(rows, S), SK)
        kind, binary = "port", "oracle/_build/liboracle.so: OpenMP restatement of the reference's fp64 check (more generous to the CPU than the reference's single-threaded harness)"
    value = work * len(secs) / sum(secs) / 1e12
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1e3 * sum(secs) / len(secs), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64",
            "data": "synthetic (reference harness REF_DATA=normal generator)",
            "config": {"workload": f"{wl}: B{B} H{H} HK{HK} Sq{S} Skv{SK} hd128, non-causal", "sample": f"first {min(rows, S)} query rows of every (batch, head) per step",
                       "timed_steps": len(secs)},
            "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": kind, "binary": binary,
                             "sample": f"{min(rows, S)} query rows x {B * H} (batch, head) pairs per step, fp64 check of tests/gpu/ref_host.cpp:438-471"},
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


# ---------------------------------------------------------------------------------------------------------------- GPU legs

class Runner:
    """One process per GPU. Holds the distributed state and the timing helpers shared by every workload."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        from amdgpu_rustdsl_b200 import _abi
        self.torch, self.dist, self.args = torch, dist, args
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.lib = _abi.load()
        self.peaks = measured_peaks()
        if self.peaks:
            self.peak, self.peak_src = 2.0 * float(self.peaks["bf16_tflops"]), "2 x measured dense bf16 burst (MEASURED_PEAKS.json): the fp8 tensor rate is twice the bf16 rate; no fp8 figure is measured there"
        else:
            self.peak, self.peak_src = 2.0 * 1590.0, "2 x fallback dense bf16 (1.59 PFLOP/s)"
        self.issue_ceiling = None

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, x):
        t = self.torch.tensor([x], dtype=self.torch.float64, device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def windows(self, fn, warm, per_window, join=None, n_windows=N_WINDOWS):
        """`warm` untimed calls, then `n_windows` windows of `per_window` calls each; returns the per-window times in ms (max over ranks)."""
        torch = self.torch
        it = 0
        for _ in range(warm):
            fn(it); it += 1
        if join:
            join()
        res = []
        for _ in range(n_windows):
            self.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(per_window):
                fn(it); it += 1
            if join:
                join()   # the launching stream waits for the copy streams: the end event covers the last read-back
            e1.record()
            self.barrier()
            res.append(self.max_over_ranks(e0.elapsed_time(e1)))
        return res

    def roofline(self, per_gpu_flops, ms_per_step, extra=None):
        achieved = per_gpu_flops / (ms_per_step * 1e-3) / 1e12
        r = {"bound": "tensor", "achieved": achieved, "peak": self.peak, "unit": "TFLOP/s", "frac": achieved / self.peak, "peak_source": self.peak_src,
             "frac_of_nominal_4500": achieved / NOMINAL_MXFP8_TFLOPS}
        if self.issue_ceiling:
            r["mma_issue_ceiling_tflops"] = self.issue_ceiling
            r["frac_of_issue_ceiling"] = achieved / self.issue_ceiling
        if extra:
            r.update(extra)
        return r

    def measure_issue_ceiling(self):
        """Issue-only ceiling of the tensor pipe, measured now: one thread per SM issues M128 N128 K32 fp8 MMAs on resident operands."""
        import ctypes as C
        try:
            ms = C.c_float(0)
            sms = self.torch.cuda.get_device_properties(self.dev).multi_processor_count
            if self.lib.fmha_mxfp8_mma_issue_ceiling(8000, sms, None, C.byref(ms)) == 0 and ms.value > 0:
                self.issue_ceiling = sms * 8000 * 4 * 2.0 * 128 * 128 * 32 / (ms.value * 1e-3) / 1e12
        except Exception:
            self.issue_ceiling = None


def build_sets(R, wl, nsets_arg, pinned_host=True):
    """Device-resident input / output sets of one workload at this rank's local shape, plus the pinned host copies the end-to-end leg
    copies from. Returns a dict."""
    torch = R.torch
    from amdgpu_rustdsl_b200 import multi_gpu
    B, H, HK, S, SK, path, splits = WORKLOADS[wl]
    rank, world, dev = R.rank, R.world, R.dev
    scaling = "weak"
    lo = 0
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
    bytes_per_set = B * S * Hl * 128 * 3 + 2 * B * SKl * HKl * 128
    nsets = nsets_arg or max(2, min(16, -(-160 * 2 ** 20 // bytes_per_set)))
    if wl in ("c4", "c5"):
        nsets = nsets_arg or 1   # one set already exceeds L2
    # generate one batch element (and at most 8192 keys) on the CPU and tile it: the arithmetic does not depend on the values repeating
    gen_B = 1 if wl == "c4" else B
    gen_SK = min(SKl, 8192)
    rep, krep = B // gen_B, SKl // gen_SK
    assert gen_B * rep == B and gen_SK * krep == SKl
    if wl == "c5":   # every rank holds the same Q and the same V descale; K and V are the rank's own
        gen, vdescale = synthetic_inputs(gen_B, Hl, HKl, S, gen_SK, seed=777, kv_seed=1234 + rank, vdescale=V_DESCALE_FIXED)
    else:
        gen, vdescale = synthetic_inputs(gen_B, Hl, HKl, S, gen_SK, seed=1234 + rank)
    qs1 = torch.zeros(gen_B * S * Hl * 4 + 512 * Hl * 4, dtype=torch.uint8)
    qs1[: gen_B * S * Hl * 4] = gen["qs"]
    # batch element(s) as generated, with all of this rank's keys: what the parity check scores against
    first = {"q": gen["q"], "k": gen["k"].repeat(1, krep, 1, 1), "v": gen["v"].repeat(1, krep, 1, 1), "qs": qs1,
             "ks": gen["ks"].view(gen_B, gen_SK * HKl * 4).repeat(1, krep).reshape(-1)}
    qs = torch.zeros(B * S * Hl * 4 + 512 * Hl * 4, dtype=torch.uint8)
    qs[: B * S * Hl * 4] = gen["qs"].repeat(rep)
    ks = torch.zeros(B * SKl * HKl * 4 + 640 * Hl * 4, dtype=torch.uint8)
    ks[: B * SKl * HKl * 4] = first["ks"].view(gen_B, -1).repeat(rep, 1).reshape(-1)
    host = None
    if pinned_host:
        host = {"q": first["q"].repeat(rep, 1, 1, 1), "k": first["k"].repeat(rep, 1, 1, 1), "v": first["v"].repeat(rep, 1, 1, 1), "qs": qs, "ks": ks}
        # one pinned buffer holds the five inputs of a step back to back (256-byte aligned), and every device set mirrors it: a step's
        # inputs then cross PCIe as one copy instead of five
        names, offs, total = ("q", "k", "v", "qs", "ks"), {}, 0
        for n in names:
            offs[n] = total
            total += (host[n].numel() * host[n].element_size() + 255) // 256 * 256
        flat = torch.empty(total, dtype=torch.uint8).pin_memory()
        views = lambda buf: {n: buf[offs[n]: offs[n] + host[n].numel()].view(host[n].shape) for n in names}   # noqa: E731
        hv = views(flat)
        for n in names:
            assert host[n].dtype == torch.uint8
            hv[n].copy_(host[n])
        host = dict(hv, _flat=flat)
    sets = []
    for _ in range(nsets):
        if host is not None:
            dflat = host["_flat"].to(dev, non_blocking=True)
            s = dict(views(dflat), _flat=dflat)
        else:   # the large sharded shapes: upload one batch element and repeat it on the device
            s = {n: first[n].to(dev).repeat(rep, 1, 1, 1).contiguous() for n in ("q", "k", "v")}
            s["qs"], s["ks"] = qs.to(dev), ks.to(dev)
        s["vs"] = torch.zeros(1024, dtype=torch.float32, device=dev)
        s["vs"][0] = vdescale
        s["out"] = torch.empty(B, S, Hl, 128, dtype=torch.bfloat16, device=dev)
        sets.append(s)
    torch.cuda.synchronize()
    return {"wl": wl, "shape": (B, H, HK, S, SK), "local": (Hl, HKl, SKl), "key_lo": lo, "scaling": scaling, "path": path, "splits": splits, "sets": sets,
            "host": host, "first": first, "vdescale": vdescale, "bytes_per_set": bytes_per_set, "gen": (gen_B, gen_SK, rep, krep)}


def make_step(R, W):
    """The callable that runs one step of workload `W` on a set; fills W['ran'] with the (path, splits) it took."""
    from amdgpu_rustdsl_b200 import fmha_fwd_mxfp8, multi_gpu
    wl = W["wl"]
    B, H, HK, S, SK = W["shape"]
    Hl = W["local"][0]
    rows_total = B * S * Hl
    if wl == "c5":
        W["plan"] = multi_gpu.KvShardedPlan(rows_total, R.world, R.dev, transport=R.args.c5_transport, B=B, S=S, H=Hl, partials=R.args.c5_partials, barrier=R.args.c5_barrier)

        if W["plan"].transport == "peer":
            # the result stays where every rank's combine stores it (the plan's own output buffer): no copy into another tensor
            W["out_view"] = W["plan"].output().view(B, S, Hl, 128)

    def step(s):
        if wl == "c5":
            if "out_view" in W:
                s["out"] = W["out_view"]
                W["plan"].forward(s["q"], s["k"], s["v"], s["qs"], s["ks"], s["vs"], None)
            else:
                W["plan"].forward(s["q"], s["k"], s["v"], s["qs"], s["ks"], s["vs"], s["out"])
            W["ran"] = ("kvshard", R.world)
        else:
            W["ran"] = fmha_fwd_mxfp8(s["q"], s["k"], s["v"], s["qs"], s["ks"], s["vs"], s["out"], path=W["path"], splits=W["splits"])
    return step


def window_size(K, ms_guess, min_steps, min_ms):
    return int(max(K, min_steps, -(-min_ms // max(ms_guess, 1e-6))))


def parity_sample(R, W, s):
    """Scores a row sample of the set's output against the fp64 oracle on the inputs this rank actually used (batch element 0; the key-range
    shards rebuild the other ranks' K / V from their seeds), next to the CPU restatement of the reference's kernel arithmetic, with the
    reference's gate statistics (tests/gpu/ref_host.cpp:438-471). Every rank checks; the worst over the ranks is reported."""
    import numpy as np
    torch = R.torch
    from oracle import oracle as O
    O.set_threads(max(1, host_cores() // max(R.world, 1)))
    wl = W["wl"]
    B, H, HK, S, SK = W["shape"]
    Hl, HKl, SKl = W["local"]
    first = W["first"]
    q = first["q"][:1].numpy()
    qs_np = np.concatenate([first["qs"][: S * Hl * 4].numpy(), np.zeros(512 * Hl * 4, np.uint8)])
    if wl == "c5" and R.world > 1:
        gen_B, gen_SK, rep, krep = W["gen"]
        ks_parts, k_parts, v_parts = [], [], []
        for r in range(R.world):
            g, _ = synthetic_inputs(gen_B, Hl, HKl, S, gen_SK, seed=777, kv_seed=1234 + r, vdescale=V_DESCALE_FIXED, want_q=False)
            k_parts.append(g["k"].repeat(1, krep, 1, 1)); v_parts.append(g["v"].repeat(1, krep, 1, 1))
            ks_parts.append(g["ks"].view(gen_B, gen_SK * HKl * 4).repeat(1, krep).reshape(-1))
        k = torch.cat(k_parts, 1)[:1].numpy(); v = torch.cat(v_parts, 1)[:1].numpy()
        ks_np = np.concatenate([torch.cat(ks_parts).numpy(), np.zeros(640 * Hl * 4, np.uint8)])
        SKo = SK
    else:
        k, v = first["k"][:1].numpy(), first["v"][:1].numpy()
        ks_np = np.concatenate([first["ks"][: SKl * HKl * 4].numpy(), np.zeros(640 * Hl * 4, np.uint8)])
        SKo = SKl
    inp = O.Inputs(1, Hl, HKl, S, SKo, np.ascontiguousarray(q), np.ascontiguousarray(k), np.ascontiguousarray(v), qs_np, ks_np, float(W["vdescale"]))
    rows = [r for r in (0, 127, 128, S // 2 + 77, S - 1) if r < S]
    got = s["out"][:1].contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    ref = O.reference(inp, rows)
    ours = O.compare(inp, got, ref, rows)
    theirs = O.compare(inp, O.recipe_forward(inp, rows, 0), ref, rows)
    vals = torch.tensor([ours.mean_err, theirs.mean_err, float(ours.bad), float(theirs.bad), ours.worst_err if np.isfinite(ours.worst_err) else 1e30],
                        dtype=torch.float64, device=R.dev)
    if R.world > 1:
        R.dist.all_reduce(vals, op=R.dist.ReduceOp.MAX)
    m, rm, bad, rbad, worst = (float(x) for x in vals.tolist())
    return {"mean_err": m, "ref_path_mean_err": rm, "bad": int(bad), "ref_path_bad": int(rbad), "worst": worst, "rows": rows,
            "checked_per_rank": ours.checked, "gate_ok": bool(m <= 1.10 * rm and bad <= rbad and worst <= 2e-2),
            "what": "worst over the ranks of: row sample of batch element 0 of the rank's own output vs the fp64 oracle; gate mean <= 1.10 x reference path, bad <= reference path, worst <= 2e-2"}


def run_headline(R, wl):
    """Device-resident timing, end-to-end timing and roofline of one workload as the line's headline."""
    torch, args = R.torch, R.args
    W = build_sets(R, wl, args.sets)
    B, H, HK, S, SK = W["shape"]
    Hl, HKl, SKl = W["local"]
    sets, host = W["sets"], W["host"]
    nsets = len(sets)
    step = make_step(R, W)
    total_flops = flops(B, H, S, SK) * (R.world if W["scaling"] == "weak" else 1)
    Wm, K = max(args.warmup, 3), args.steps

    # a first short window to size the real ones
    for i in range(3):
        step(sets[i % nsets])
    guess = R.windows(lambda i: step(sets[i % nsets]), 0, 5, n_windows=1)[0] / 5
    per_window = window_size(K, guess, 100 if guess < 1.0 else 10, 50.0)
    sampler = ClockSampler(R.local_rank) if R.rank == 0 else None
    win = R.windows(lambda i: step(sets[i % nsets]), Wm, per_window)
    clocks = sampler.stop() if sampler else None
    ms_per_step = statistics.median(win) / per_window
    launches_per_step = 2 if W["ran"][0] in ("kvsplit", "kvshard") else 1

    # ---- end to end through the public entry: every step copies its inputs from pinned host memory and reads the result back.
    # The steps are pipelined the way a caller with a queue of requests would: one stream copies step i + 1's inputs in and another reads
    # step i - 1's result back while step i computes; every step still pays its own host-to-device and device-to-host copies in the region.
    h2d = host["_flat"].numel()
    out_hosts = [torch.empty(B, S, Hl, 128, dtype=torch.bfloat16).pin_memory() for _ in sets]
    d2h = out_hosts[0].numel() * 2
    main = torch.cuda.current_stream(R.dev)
    s_in, s_out = torch.cuda.Stream(R.dev), torch.cuda.Stream(R.dev)
    ev_in = [torch.cuda.Event() for _ in sets]
    ev_done = [torch.cuda.Event() for _ in sets]
    ev_out = [torch.cuda.Event() for _ in sets]

    def e2e_step(i):
        k = i % nsets
        s = sets[k]
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_done[k])      # the set's previous step has consumed its inputs
            s["_flat"].copy_(host["_flat"], non_blocking=True)   # q, k, v and both scale buffers in one copy
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
    e2e_win = R.windows(e2e_step, 3, Ke, e2e_join)
    ms_e2e = statistics.median(e2e_win) / Ke
    host_us = None
    if wl != "c5":
        # host cost of one call of the Python entry (argument block, validate, four tensor-map encodes, launch), no synchronisation inside
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(300):
            step(sets[i % nsets])
        host_us = (time.perf_counter() - t0) / 300 * 1e6
        torch.cuda.synchronize()
    value = total_flops / (ms_per_step * 1e-3) / 1e12
    alg_bytes = B * Hl * S * (128 + 4 + 256) + 2 * B * HKl * SKl * 128 + B * HKl * SKl * 4
    extra = {"traffic": RECORDED_NCU_DRAM_BYTES.get(wl) if R.world == 1 else None,
             "traffic_unit": "bytes per launch: DRAM read + write of an ncu capture of this launch, a recorded constant (output lines still dirty in L2 at kernel end are not in it)",
             "algorithmic_bytes": alg_bytes,
             "note": "achieved = this rank's 4*B*H*Sq*Skv*128 per step / median step time (CUDA events); for kvsplit steps the combine launch is inside the step"}
    res = {"value": value, "ms_per_step": ms_per_step, "scaling": W["scaling"], "ran": W["ran"], "gpu_launches": N_WINDOWS * per_window * launches_per_step,
           "per_window": per_window, "windows_ms": win, "clocks": clocks,
           "roofline": R.roofline(flops(B, Hl, S, SKl), ms_per_step, extra),
           "e2e": {"value": total_flops / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": Ke,
                   "ms_per_step": ms_e2e, "windows_ms": e2e_win},
           "host_us_per_call": host_us, "nsets": nsets, "bytes_per_set": W["bytes_per_set"]}
    if clocks and clocks.get("sm_mhz"):
        res["ms_per_step_x_sm_mhz"] = ms_per_step * clocks["sm_mhz"]
    W["sets"] = None
    return res


def run_sharded(R, wl):
    """One sharded configuration at this N: value, per-GPU roofline fraction, (key-range shards) the split of a step into its stages, and
    the parity of a row sample."""
    torch, args = R.torch, R.args
    W = build_sets(R, wl, 0, pinned_host=False)
    B, H, HK, S, SK = W["shape"]
    Hl, HKl, SKl = W["local"]
    s = W["sets"][0]
    step = make_step(R, W)
    for _ in range(3):
        step(s)
    guess = R.windows(lambda i: step(s), 0, 2, n_windows=1)[0] / 2
    per_window = max(2, min(int(-(-50.0 // guess)), 200))
    sampler = ClockSampler(R.local_rank) if R.rank == 0 else None
    win = R.windows(lambda i: step(s), 1, per_window)
    clocks = sampler.stop() if sampler else None
    ms = statistics.median(win) / per_window
    res = {"workload": f"{wl}: B{B} H{H} HK{HK} Sq{S} Skv{SK}", "per_rank": f"H{Hl} HK{HKl} Skv{SKl}", "value": flops(B, H, S, SK) / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
           "ms_per_step": ms, "per_window": per_window, "windows_ms": win, "scaling": W["scaling"],
           "roofline_frac_per_gpu": flops(B, Hl, S, SKl) / (ms * 1e-3) / 1e12 / R.peak,
           "clocks": clocks, "parallelism": ("heads dealt out over the ranks, no collective" if wl == "c4" else W["plan"].describe() if wl == "c5"
                                             else f"one GPU: {W['ran'][0]} with {W['ran'][1]} splits (f16 partials) + combine")}
    if wl == "c5":
        stages = W["plan"].timed_stages(s["q"], s["k"], s["v"], s["qs"], s["ks"], s["vs"], None if "out_view" in W else s["out"], reps=5)
        res["stages_ms"] = {k: R.max_over_ranks(v) for k, v in stages.items()}
    step(s)
    torch.cuda.synchronize()
    res["parity"] = parity_sample(R, W, s)
    if wl == "c3":
        # the same step with the merge of the partials built into the split kernel (one launch instead of two): same bytes, its own timing
        from amdgpu_rustdsl_b200 import fmha_fwd_mxfp8
        want = s["out"].clone()
        fused = lambda i: fmha_fwd_mxfp8(s["q"], s["k"], s["v"], s["qs"], s["ks"], s["vs"], s["out"], path=W["path"], splits=W["splits"], fused_combine=True)
        for _ in range(3):
            fused(0)
        torch.cuda.synchronize()
        same = bool(torch.equal(s["out"].view(torch.int16), want.view(torch.int16)))
        fwin = R.windows(fused, 1, per_window)
        fms = statistics.median(fwin) / per_window
        res["fused_merge"] = {"ms_per_step": fms, "value": flops(B, H, S, SK) / (fms * 1e-3) / 1e12, "same_bytes_as_two_kernels": same, "windows_ms": fwin}
    if wl == "c5":
        W.pop("out_view", None)
        s.pop("out", None)
        W["plan"].close()
    W["sets"] = None
    del s
    torch.cuda.empty_cache()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--quantizer", action="store_true", help="side bench: the device quantisers in front of the path (not the headline metric)")
    ap.add_argument("--rows", type=int, default=4194304, help="rows of 128 bf16 for --quantizer")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--cpu-rows", type=int, default=0, help="query rows per (b,h) of the CPU baseline sample (0 = default)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-sharded", action="store_true", help="skip the two sharded configurations of the `sharded` object")
    ap.add_argument("--c5-transport", default="auto", choices=["auto", "peer", "nccl"], help="how the key-range shards' partials reach the combining GPU")
    ap.add_argument("--c5-partials", default="f32", choices=["f16", "f32"], help="format of the partial rows the key-range shards store into the combining GPU (peer transport)")
    ap.add_argument("--c5-barrier", default="flags", choices=["flags", "nccl"], help="how the key-range shards' ranks line up between the kernels (peer transport)")
    ap.add_argument("--sets", type=int, default=0, help="number of rotating input sets (0 = enough to exceed L2)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.quantizer:
        return run_quantizer_bench(args)

    from amdgpu_rustdsl_b200 import device_status
    R = Runner(args)
    R.measure_issue_ceiling()
    wl = args.workload
    B, H, HK, S, SK, _, _ = WORKLOADS[wl]
    head = run_headline(R, wl)
    sharded = None
    if wl == "c2" and not args.no_sharded:
        sharded = {}
        for w in ("c4", "c5"):
            try:
                sharded[w] = run_sharded(R, w)
            except Exception as e:   # a failure here must not take the headline with it, and every rank has to reach the next collective
                sharded[w] = {"error": f"{type(e).__name__}: {e}"}
                R.torch.cuda.synchronize()
    if wl == "c2" and not args.no_sharded and R.world == 1:
        # the forced 8-way key split of B1 H8 S8192 on one GPU (split kernel + combine in one window), beside the headline
        try:
            sharded["c3"] = run_sharded(R, "c3")
        except Exception as e:
            sharded["c3"] = {"error": f"{type(e).__name__}: {e}"}
    status = device_status()

    if R.rank != 0:
        if R.world > 1:
            R.dist.destroy_process_group()
        return
    world = R.world
    line = {"metric": METRIC, "value": head["value"], "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": head["scaling"], "vs_baseline": None,
            "dtype": "fp8-e4m3 x E8M0 block scales (MXFP8), f32 accumulate, bf16 out",
            "data": "synthetic (seeded standard-normal Q/K/V quantised to MXFP8 on the host, the distribution of the reference harness's REF_DATA=normal)",
            "config": {"workload": f"{wl}: B{B} H{H} HK{HK} Sq{S} Skv{SK} hd128, non-causal" + (f", per rank (x{world} ranks)" if head["scaling"] == "weak" and world > 1 else ""),
                       "path": head["ran"][0], "splits": head["ran"][1],
                       "l2": f"{head['nsets']} rotating input/output sets of {head['bytes_per_set'] / 2**20:.0f} MiB (> 126 MB L2 in total)",
                       "timing": f"median of {N_WINDOWS} windows of {head['per_window']} steps each (>= --steps, >= 100 steps, >= 50 ms), CUDA events, max over ranks per window",
                       "parallelism": "none" if world == 1 else ("batch x head replicas per rank, no collective" if wl not in ("c4", "c5") else "see sharded")},
            "roofline": head["roofline"], "gpu_launches": head["gpu_launches"], "device_status": status, "e2e": head["e2e"], "clocks": head["clocks"],
            "windows_ms": head["windows_ms"], "ms_per_step_x_sm_mhz": head.get("ms_per_step_x_sm_mhz"), "host_us_per_call": head["host_us_per_call"]}
    if sharded is not None:
        line["sharded"] = sharded
    if not args.no_cpu and world == 1:
        rows = args.cpu_rows
        if not rows:   # about 10-20 s of CPU work: calibrate on 8 rows
            _, dt8, _ = cpu_port_sample(wl, 8)
            rows = max(1, min(S, int(8 * 12.0 / max(dt8, 1e-4))))
        v, dt, cores = cpu_port_sample(wl, rows)
        line["cpu_baseline"] = {"value": v, "unit": "TFLOP/s", "cores": cores, "kind": "port", "seconds": dt,
                                "sample": f"fp64 oracle on the first {min(rows, S)} query rows of every (batch, head) of the same workload"}
    else:
        line["cpu_baseline"] = None
    print(json.dumps(line), flush=True)
    if world > 1:
        R.dist.destroy_process_group()


if __name__ == "__main__":
    main()
