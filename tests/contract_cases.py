"""Host-contract test cases: valid launches of the four kernels (as tests/gpu/ref_host.cpp:342-383,516-551 of the reference builds them)
and single mutations of them. Shared by tests/golden/make_golden.py (which asks the reference's generated validate() for the verdicts)
and tests/test_host_contract.py (which replays them through the C ABI)."""
from __future__ import annotations

import struct

OFF = {  # u32 kernel arguments (tests/gpu/generated/fmha_fwd_hd128_mxfp8_v3_kvsplit_abi.h:73-134)
    "s_seq_len": 0x60, "s_Seqs": 0x70, "s_Hs": 0x90, "s_Bs": 0xA0, "s_gqa": 0xB0, "s_k_Seqs": 0xC0, "s_k_Hs": 0xD0, "s_k_Bs": 0xE0,
    "s_kv_seq_len": 0x110, "s_q_head_num": 0x140, "s_v_Seqs": 0x150, "s_v_Hs": 0x160, "s_v_Bs": 0x170, "s_o_Seqs": 0x180, "s_o_Hs": 0x190,
    "s_o_Bs": 0x1A0, "s_descale_q_Bs": 0x230, "s_descale_q_Hs": 0x240, "s_descale_k_Bs": 0x250, "s_descale_k_Hs": 0x260,
    "kvs_splits": 0x280, "kvs_rows_total": 0x284,
}
COMBINE_OFF = {"rows_total": 0x18, "d": 0x1C, "splits": 0x20}
SIZE_NAMES = ["ptr_q", "ptr_k", "ptr_v", "ptr_o", "ptr_q_descale", "ptr_k_descale", "ptr_v_descale", "ptr_ohat", "ptr_lse", "ptr_out"]
KSIZE = {0: 656, 1: 656, 2: 648, 3: 36}
D = 128


def materialize(c):
    """-> (args bytes, sizes[10], grid[3], (B, HK, KL))"""
    k, B, H, HK, S, SK, splits = c["kernel"], c["B"], c["H"], c["HK"], c["S"], c["SK"], c.get("splits", 0)
    a = bytearray(KSIZE[k])
    sizes = [0] * 10
    rows_total = B * S * H
    if k == 3:
        struct.pack_into("<QQQIII", a, 0, 0x1000, 0x2000, 0x3000, rows_total, D, splits)
        sizes[7], sizes[8], sizes[9] = splits * rows_total * 512, splits * rows_total * 4, rows_total * 256
        grid = [max(1, -(-rows_total * D // 2048)), 1, 1]
        offs = COMBINE_OFF
    else:
        for off, p in ((0x0, 0x10000), (0x10, 0x20000), (0x20, 0x30000), (0x30, 0x40000), (0x200, 0x50000), (0x210, 0x60000), (0x220, 0x70000)):
            struct.pack_into("<Q", a, off, p)
        vals = {"s_seq_len": S, "s_Seqs": H * D, "s_Hs": D, "s_Bs": S * H * D, "s_gqa": H // HK, "s_k_Seqs": HK * D, "s_k_Hs": D, "s_k_Bs": SK * HK * D,
                "s_kv_seq_len": SK, "s_q_head_num": H, "s_v_Seqs": HK * D, "s_v_Hs": D, "s_v_Bs": SK * HK * D, "s_o_Seqs": H * D * 2, "s_o_Hs": D * 2,
                "s_o_Bs": S * H * D * 2, "s_descale_q_Bs": S * H * 4, "s_descale_q_Hs": 4, "s_descale_k_Bs": SK * HK * 4, "s_descale_k_Hs": 4}
        for n, v in vals.items():
            struct.pack_into("<I", a, OFF[n], v & 0xFFFFFFFF)
        sizes[0], sizes[1], sizes[2], sizes[3] = B * S * H * D, B * SK * HK * D, B * SK * HK * D, B * S * H * D * 2
        sizes[4] = B * S * H * 4 + 512 * H * 4       # ref_host.cpp:197-198
        sizes[5] = B * SK * HK * 4 + 640 * H * 4
        sizes[6] = 4096
        rows = 128 if k == 1 else 256
        grid = [-(-S // rows), H, B]
        if k == 2:
            struct.pack_into("<QQII", a, 0x270, 0x80000, 0x90000, splits, rows_total)
            sizes[7], sizes[8] = splits * rows_total * D * 4, splits * rows_total * 4
            grid[2] = B * splits
        offs = OFF
    syms = {"B": B, "HK": HK, "KL": 0}
    for kind, key, val in c.get("mut", []):
        if kind == "field":
            struct.pack_into("<I", a, offs[key], val & 0xFFFFFFFF)
        elif kind == "size":
            sizes[SIZE_NAMES.index(key)] += val
        elif kind == "grid":
            grid[key] = val
        elif kind == "sym":
            syms[key] = val
    return bytes(a), sizes, grid, (syms["B"], syms["HK"], syms["KL"])


def case_line(c):
    a, sizes, grid, syms = materialize(c)
    return " ".join([str(c["kernel"]), a.hex()] + [str(x) for x in sizes] + [str(x) for x in grid] + [str(x) for x in syms])


# shapes of the reference's own contract test (crates/amdc/tests/contract_host_truth.rs:124-128) plus gate shapes with GQA / odd sizes
BASE_SHAPES = [(1, 8, 8, 2048, 2048), (4, 8, 8, 2048, 2048), (1, 2, 1, 200, 1337), (2, 8, 4, 700, 640)]


def build_cases(rnd):
    cases = []
    for (B, H, HK, S, SK) in BASE_SHAPES:
        for kernel in (0, 1, 2, 3):
            for splits in ((2, 4, 8) if kernel in (2, 3) else (0,)):
                base = {"kernel": kernel, "B": B, "H": H, "HK": HK, "S": S, "SK": SK, "splits": splits}
                cases.append(dict(base, mut=[]))
                if splits in (2, 8):
                    continue   # the other split counts only as valid launches
                if kernel == 3:
                    for f in COMBINE_OFF:
                        for v in (0, 1, 127, 128, 129):
                            cases.append(dict(base, mut=[["field", f, v]]))
                    for n in ("ptr_ohat", "ptr_lse", "ptr_out"):
                        cases.append(dict(base, mut=[["size", n, -1]]))
                        cases.append(dict(base, mut=[["size", n, 1]]))
                    continue
                names = [n for n in OFF if kernel == 2 or not n.startswith("kvs_")]
                for f in names:
                    a, _, _, _ = materialize(base)
                    cur = struct.unpack_from("<I", a, OFF[f])[0]
                    for v in {0, 1, cur + 1, max(cur - 1, 0), cur * 2, 17, rnd.randrange(1, 1 << 20)}:
                        if v != cur:
                            cases.append(dict(base, mut=[["field", f, v]]))
                for n in SIZE_NAMES[:9 if kernel == 2 else 7]:
                    cases.append(dict(base, mut=[["size", n, -1]]))
                    cases.append(dict(base, mut=[["size", n, 4096]]))
                for axis in range(3):
                    _, _, g, _ = materialize(base)
                    for v in (0, g[axis] + 1, max(g[axis] - 1, 0), g[axis] * 2):
                        if v != g[axis]:
                            cases.append(dict(base, mut=[["grid", axis, v]]))
                for sname, vals in (("HK", (0, HK + 1, HK * 2, 1)), ("B", (0, B + 1)), ("KL", (-1, 5))):
                    for v in vals:
                        cases.append(dict(base, mut=[["sym", sname, v]]))
                # two simultaneous faults: the first failing check in the reference's order must win
                for _ in range(6):
                    f1, f2 = rnd.sample(names, 2)
                    cases.append(dict(base, mut=[["field", f1, rnd.randrange(0, 4096)], ["size", rnd.choice(SIZE_NAMES[:7]), -rnd.randrange(1, 64)],
                                                 ["field", f2, rnd.randrange(0, 1 << 16)]]))
    return cases
