"""A few launches of one shape of the MXFP8 attention path, for capture under a profiler (`ncu ... python -m amdgpu_rustdsl_b200.profile_case ...`).

Inputs are seeded random e4m3 bytes with fixed block scales: the kernels' work does not depend on the values, and a profile needs no
accuracy check. Nothing here is timed; bench.py measures.
"""
from __future__ import annotations

import argparse


def main():
    import torch
    from . import fmha_fwd_mxfp8
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="4,8,2048,2048", help="B,H,S,SK (HK = H)")
    ap.add_argument("--path", default="auto")
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--launches", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--sets", type=int, default=1, help="rotating input sets (use enough to exceed the 126 MB L2 when DRAM figures matter)")
    ap.add_argument("--causal", action="store_true")
    a = ap.parse_args()
    B, H, S, SK = (int(x) for x in a.shape.split(","))
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev)
    g.manual_seed(1)
    sets = []
    for _ in range(a.sets):
        q, k, v = (torch.randint(0, 120, shp, dtype=torch.uint8, device=dev, generator=g) | (torch.randint(0, 2, shp, dtype=torch.uint8, device=dev, generator=g) << 7)
                   for shp in ((B, S, H, 128), (B, SK, H, 128), (B, SK, H, 128)))
        qs = torch.zeros(B * S * H * 4 + 512 * H * 4, dtype=torch.uint8, device=dev)
        qs[: B * S * H * 4] = 118
        ks = torch.zeros(B * SK * H * 4 + 640 * H * 4, dtype=torch.uint8, device=dev)
        ks[: B * SK * H * 4] = 119
        vs = torch.ones(1024, dtype=torch.float32, device=dev)
        out = torch.empty(B, S, H, 128, dtype=torch.bfloat16, device=dev)
        sets.append((q, k, v, qs, ks, vs, out))
    ran = None
    for i in range(a.warmup + a.launches):
        q, k, v, qs, ks, vs, out = sets[i % a.sets]
        ran = fmha_fwd_mxfp8(q, k, v, qs, ks, vs, out, path=a.path, splits=a.splits or None, causal=a.causal)
    torch.cuda.synchronize()
    print(f"profile_case: B{B} H{H} S{S} SK{SK} ran {ran} x {a.launches} (+{a.warmup} warm-up)")


if __name__ == "__main__":
    main()
