// MXFP8 attention forward, head dim 128, for sm_100a: the bodies of fmha_fwd_hd128_mxfp8_v3_{vs128, t128, kvsplit}.
//
// What one CTA computes (reference: crates/amdgpu-stage/src/attention/attn3.rs:260-755, block3.rs:79-356): for 128 query rows of
// one (batch, head) and a key range [key_lo, key_hi), out = softmax2(q k^T) v with
//   q k^T  : e4m3 x e4m3 with one E8M0 scale per 32 elements of the head dim on both sides (block-scaled tensor-core MMA),
//   softmax: base 2, no extra scale (the host folds log2(e)/sqrt(128) into Q before quantisation, tests/gpu/ref_host.cpp:238),
//            online over 128-key tiles with a lazily moved reference: the reference only moves when a row maximum passes it by
//            more than a threshold, and then O and the row sum are rescaled (crates/amdgpu-tile/src/softmax.rs:179-243);
//            sequences under 4 tiles move the reference on every tile (crates/amdgpu-stage/src/attention/state.rs:73-77),
//   P      : requantised to e4m3 before P V, and the row sum adds the *quantised* P (crates/amdgpu-tile/src/reduce.rs:163-173),
//   out    : O * v_descale / l as bf16 (state.rs:79-82), or for the split kernel the normalised f32 partial plus a base-2
//            log-sum-exp per row (block3.rs:291-356).
//
// Mapping onto the SM (not a translation of the gfx950 wave layout):
//   warps 0-3  softmax + epilogue: thread r owns query row r = TMEM lane r; reads S with tcgen05.ld, writes P (packed e4m3)
//              back into the first 32 columns of the same S buffer with tcgen05.st, rescales O in TMEM when its reference moves.
//   warp  4    MMA issuer: one lane issues tcgen05.mma; S = Q K^T is kind::mxf8f6f4.block_scale with both operands in swizzled
//              shared memory and the E8M0 factors in TMEM (tcgen05.cp); O += P V takes P from TMEM and V (keys x head dim, i.e.
//              MN-major B) from shared memory. S is double buffered so Q K^T of tile j+1 overlaps the softmax of tile j.
//   warp  5    producer: TMA loads of the Q tile and of the K/V tiles into a ring, plus the 4-byte-per-row scale gathers, which
//              a TMA box cannot express, written in the 32x16-byte layout tcgen05.cp expects.
// TMEM columns: S0 [0,128) S1 [128,256) O [256,384) SFQ [384,388) SFK0 [388,392) SFK1 [392,396) SFP [396,400) SFV [400,404).
#include "kernels.h"
#include "ptx_sm100.cuh"

#include <cuda_bf16.h>
#include <cuda_fp8.h>

namespace fmha {
using namespace sm100;

namespace {

constexpr int kRows = 128;          // query rows per CTA tile
constexpr int kKeys = 128;          // keys per tile
constexpr int kStages = 3;          // K/V ring depth
constexpr int kThreads = 192;
constexpr uint32_t kTileBytes = 128 * 128;   // one e4m3 tile
constexpr uint32_t kSfBytes = 512;           // 128 rows x 4 scale bytes

constexpr uint32_t kColS0 = 0, kColS1 = 128, kColO = 256, kColSfQ = 384, kColSfK0 = 388, kColSfK1 = 392;
constexpr uint32_t kTmemCols = 512;

// P = 2^(s - ref + kPOffset): the reference row maximum maps to 2^kPOffset, and the reference is left alone while the running
// maximum stays within kLazyThreshold binades of it, so P <= 2^(5 + 3.5) = 362 < 448 never saturates e4m3.
constexpr float kPOffset = 5.0f;
constexpr float kLazyThreshold = 3.5f;

struct SmemLayout {
    // all tile buffers are 1024-byte aligned (128-byte swizzle atom = 8 rows x 128 B)
    static constexpr uint32_t q = 0;
    static constexpr uint32_t k = q + kTileBytes;
    static constexpr uint32_t v = k + kStages * kTileBytes;
    static constexpr uint32_t sfq = v + kStages * kTileBytes;
    static constexpr uint32_t sfk = sfq + kSfBytes;
    static constexpr uint32_t bars = sfk + kStages * kSfBytes;
    // barriers (8 bytes each): q_full, kv_full[kStages], kv_empty[kStages], s_full[2], p_full[2], o_done
    static constexpr uint32_t n_bars = 1 + 2 * kStages + 2 + 2 + 1;
    static constexpr uint32_t tmem_slot = bars + 8 * n_bars;
    static constexpr uint32_t abort_flag = tmem_slot + 4;
    static constexpr uint32_t total = abort_flag + 4;
};
constexpr uint32_t kSmemBytes = SmemLayout::total + 1024;   // + slack to align the base to 1024

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float lg2_approx(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Two floats -> two e4m3 bytes (round to nearest even, saturating), `a` in the low byte.
__device__ __forceinline__ uint32_t cvt_e4m3x2(float a, float b) {
    return static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3));
}
// Sum of the two e4m3 values of a packed pair, as f32.
__device__ __forceinline__ float sum_e4m3x2(uint32_t pair) {
    const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(pair), __NV_E4M3);
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h));
    return f.x + f.y;
}

}  // namespace

template <bool kSplit>
__global__ void __launch_bounds__(kThreads, 1)
fmha_fwd_mxfp8_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    const uint32_t q_smem = smem_base + SmemLayout::q;
    const uint32_t k_smem = smem_base + SmemLayout::k;
    const uint32_t v_smem = smem_base + SmemLayout::v;
    const uint32_t sfq_smem = smem_base + SmemLayout::sfq;
    const uint32_t sfk_smem = smem_base + SmemLayout::sfk;
    const uint32_t bar0 = smem_base + SmemLayout::bars;
    const uint32_t bar_q_full = bar0;
    auto bar_kv_full = [&](int st) { return bar0 + 8u * (1 + st); };
    auto bar_kv_empty = [&](int st) { return bar0 + 8u * (1 + kStages + st); };
    auto bar_s_full = [&](int b) { return bar0 + 8u * (1 + 2 * kStages + b); };
    auto bar_p_full = [&](int b) { return bar0 + 8u * (3 + 2 * kStages + b); };
    const uint32_t bar_o_done = bar0 + 8u * (5 + 2 * kStages);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + SmemLayout::tmem_slot);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem_gen + SmemLayout::abort_flag);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // ---- which tile: grid = (q tiles of 128 rows, H, B * splits) ----
    const uint32_t row0 = blockIdx.x * kRows;
    const uint32_t head = blockIdx.y;
    uint32_t batch = blockIdx.z, split = 0;
    if (kSplit) {
        batch = blockIdx.z >> p.split_log2;
        split = blockIdx.z & (p.splits - 1u);
    }
    const uint32_t kv_head = head >> p.gqa_shift;   // crates/amdgpu-stage/src/components.rs:8-17
    const uint32_t ntiles_total = (p.SK + kKeys - 1) / kKeys;
    uint32_t key_lo = 0, key_hi = p.SK;
    if (kSplit) {   // tiles [split*tps, min(ntiles, (split+1)*tps)) (components.rs:58-74)
        const uint32_t tps = (ntiles_total + p.splits - 1) / p.splits;
        const uint32_t tile_lo = split * tps;
        const uint32_t tile_hi = min(ntiles_total, tile_lo + tps);
        key_lo = tile_lo * kKeys;
        key_hi = min(tile_hi * kKeys, p.SK);
    }
    const int n_tiles = (key_hi > key_lo) ? static_cast<int>((key_hi - key_lo + kKeys - 1) / kKeys) : 0;
    // the recipe is chosen from the whole sequence's tile count, also in a split (block3.rs:180-184)
    const bool lazy = (ntiles_total >= 4) && !(p.flags & 0x2u);
    const float thr = lazy ? kLazyThreshold : 0.0f;

    // ---- one-time setup ----
    if (threadIdx.x == 0) {
        *abort_flag = 0u;
        mbar_init(bar_q_full, 1);
        for (int st = 0; st < kStages; ++st) {
            mbar_init(bar_kv_full(st), 1);
            mbar_init(bar_kv_empty(st), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_s_full(b), 1);
            mbar_init(bar_p_full(b), kRows);
        }
        mbar_init(bar_o_done, 1);
        fence_mbar_init();
    }
    if (warp == 4) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
        tmem_relinquish();
    }
    if (warp == 5 && lane == 0) {
        prefetch_tmap(&tm_q);
        prefetch_tmap(&tm_k);
        prefetch_tmap(&tm_v);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp == 5) {
        // =========================================================== producer ===========================================================
        {   // Q scale bytes -> [row % 32][row / 32][4] (the layout tcgen05.cp 32x128b.warpx4 spreads over the four lane quadrants)
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint32_t r = row0 + lane + 32 * i;
                r = min(r, p.S - 1u);   // rows past the sequence reuse the last row's scales (block3.rs:110-113)
                const size_t off = static_cast<size_t>(batch) * p.qs_batch_stride + (static_cast<size_t>(r) * p.H + head) * 4u;
                w[i] = *reinterpret_cast<const uint32_t*>(p.q_descale + off);
            }
            *reinterpret_cast<uint4*>(smem_gen + SmemLayout::sfq + lane * 16) = make_uint4(w[0], w[1], w[2], w[3]);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive_expect_tx(bar_q_full, kTileBytes);
                tma_load_4d(q_smem, &tm_q, bar_q_full, 0, static_cast<int>(head), static_cast<int>(row0), static_cast<int>(batch));
            }
        }
        int armed = 0;
        for (int j = 0; j < n_tiles; ++j) {
            const int st = j % kStages;
            if (j >= kStages) {
                if (!mbar_wait(bar_kv_empty(st), ((j / kStages) - 1) & 1, abort_flag)) break;
            }
            const uint32_t key0 = key_lo + j * kKeys;
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t key = key0 + lane + 32 * i;
                if (key < p.SK) {
                    const size_t off = static_cast<size_t>(batch) * p.ks_batch_stride + (static_cast<size_t>(key) * p.HK + kv_head) * 4u;
                    w[i] = *reinterpret_cast<const uint32_t*>(p.k_descale + off);
                } else {
                    w[i] = 0x7F7F7F7Fu;   // keys past the sequence: data is zero-filled by TMA, any finite scale does
                }
            }
            *reinterpret_cast<uint4*>(smem_gen + SmemLayout::sfk + st * kSfBytes + lane * 16) = make_uint4(w[0], w[1], w[2], w[3]);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive_expect_tx(bar_kv_full(st), 2 * kTileBytes);
                tma_load_4d(k_smem + st * kTileBytes, &tm_k, bar_kv_full(st), 0, static_cast<int>(kv_head), static_cast<int>(key0), static_cast<int>(batch));
                tma_load_4d(v_smem + st * kTileBytes, &tm_v, bar_kv_full(st), 0, static_cast<int>(kv_head), static_cast<int>(key0), static_cast<int>(batch));
            }
            armed = j + 1;
        }
        if (*abort_flag != 0u) {
            // leaving early: let the copies already in flight land before the CTA's shared memory is given back
            for (int j = max(0, armed - kStages); j < armed; ++j) {
                const int st = j % kStages;
                const long long t0 = clock64();
                while (!mbar_try_wait(bar_kv_full(st), (j / kStages) & 1) && clock64() - t0 < kWaitBudgetCycles) {}
            }
        }
    } else if (warp == 4) {
        // =========================================================== MMA issuer ===========================================================
        const uint32_t idesc_qk = idesc_mxf8_block_scaled(128, 128, 0, 0, 0, 0);
        const uint32_t idesc_pv = idesc_f8_dense(128, 128, 0, 1);
        const uint32_t t_sfq = tmem + kColSfQ;
        bool ok = mbar_wait(bar_q_full, 0, abort_flag);
        tc_fence_after_sync();
        if (ok && lane == 0) tmem_cp_sf(t_sfq, make_smem_desc(sfq_smem, 0, 128, kSwizzleNone));

        auto issue_pv = [&](int i) -> bool {
            // O (+)= P(i) V(i): P from TMEM (first 32 columns of S[i&1], 8 columns per 32 keys), V tile = 128 keys x 128 B, MN-major
            if (!mbar_wait(bar_p_full(i & 1), (i >> 1) & 1, abort_flag)) return false;
            tc_fence_after_sync();
            if (lane == 0) {
                const int st = i % kStages;
                const uint32_t t_p = tmem + ((i & 1) ? kColS1 : kColS0);
#pragma unroll
                for (int kb = 0; kb < 4; ++kb) {
                    const uint64_t dv = make_smem_desc(v_smem + st * kTileBytes + kb * 4096, 1024, 1024, kSwizzle128B);
                    mma_f8_ts(tmem + kColO, t_p + 8 * kb, dv, idesc_pv, (i > 0 || kb > 0) ? 1u : 0u);
                }
                tc_commit(bar_kv_empty(st));
                tc_commit(bar_o_done);
            }
            __syncwarp();
            return true;
        };

        for (int j = 0; ok && j < n_tiles; ++j) {
            const int st = j % kStages;
            if (!mbar_wait(bar_kv_full(st), (j / kStages) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after_sync();
            if (lane == 0) {
                const uint32_t t_sfk = tmem + ((j & 1) ? kColSfK1 : kColSfK0);
                const uint32_t t_s = tmem + ((j & 1) ? kColS1 : kColS0);
                tmem_cp_sf(t_sfk, make_smem_desc(sfk_smem + st * kSfBytes, 0, 128, kSwizzleNone));
#pragma unroll
                for (int kb = 0; kb < 4; ++kb) {
                    // K-major 128-byte-swizzled tiles: 8-row groups 1024 B apart, 32 head-dim bytes per MMA
                    const uint64_t dq = make_smem_desc(q_smem + kb * 32, 16, 1024, kSwizzle128B);
                    const uint64_t dk = make_smem_desc(k_smem + st * kTileBytes + kb * 32, 16, 1024, kSwizzle128B);
                    const uint32_t id = idesc_qk | (static_cast<uint32_t>(kb) << 29) | (static_cast<uint32_t>(kb) << 4);
                    mma_mxf8_ss(t_s, dq, dk, id, t_sfq + (static_cast<uint32_t>(kb) << 30), t_sfk + (static_cast<uint32_t>(kb) << 30), kb > 0 ? 1u : 0u);
                }
                tc_commit(bar_s_full(j & 1));
            }
            __syncwarp();
            if (j > 0) ok = issue_pv(j - 1);
        }
        if (ok && n_tiles > 0) issue_pv(n_tiles - 1);
    } else {
        // =========================================================== softmax + epilogue ===========================================================
        const uint32_t r = threadIdx.x;                        // query row within the tile = TMEM lane
        const uint32_t lane_base = (static_cast<uint32_t>(warp) * 32u) << 16;
        float ref = -INFINITY;   // the row's reference (log2 units)
        float l = 0.0f;          // running sum of the quantised P
        bool ok = true;
        const bool tracing = (p.trace != nullptr) && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;

        for (int j = 0; j < n_tiles; ++j) {
            if (!mbar_wait(bar_s_full(j & 1), (j >> 1) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after_sync();
            const uint32_t t_s = tmem + ((j & 1) ? kColS1 : kColS0) + lane_base;
            uint32_t s0[32], s1[32], s2[32], s3[32];
            tmem_ld32(t_s + 0, s0);
            tmem_ld32(t_s + 32, s1);
            tmem_ld32(t_s + 64, s2);
            tmem_ld32(t_s + 96, s3);
            tmem_wait_ld();

            const int nvalid = static_cast<int>(min(static_cast<uint32_t>(kKeys), key_hi - (key_lo + j * kKeys)));
            if (nvalid < kKeys) {   // keys past the range: -inf for the maximum, 0 for P (crates/amdgpu-tile/src/reduce.rs:35-49)
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    if (c >= nvalid) s0[c] = 0xFF800000u;
                    if (c + 32 >= nvalid) s1[c] = 0xFF800000u;
                    if (c + 64 >= nvalid) s2[c] = 0xFF800000u;
                    if (c + 96 >= nvalid) s3[c] = 0xFF800000u;
                }
            }
            if (tracing && j == 0) {
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    p.trace[r * 128 + c] = __uint_as_float(s0[c]);
                    p.trace[r * 128 + 32 + c] = __uint_as_float(s1[c]);
                    p.trace[r * 128 + 64 + c] = __uint_as_float(s2[c]);
                    p.trace[r * 128 + 96 + c] = __uint_as_float(s3[c]);
                }
            }
            float mt = -INFINITY;
#pragma unroll
            for (int c = 0; c < 32; ++c) {
                mt = fmaxf(mt, fmaxf(fmaxf(__uint_as_float(s0[c]), __uint_as_float(s1[c])), fmaxf(__uint_as_float(s2[c]), __uint_as_float(s3[c]))));
            }
            // lazily moved reference: only when this tile's maximum passes it by more than the threshold
            const bool move = mt > ref + thr;
            if (__any_sync(0xFFFFFFFFu, move)) {
                float f = 1.0f;
                if (move) {
                    f = ex2_approx(ref - mt);   // 0 on the first tile (ref = -inf)
                    ref = mt;
                    l *= f;
                }
                if (j > 0) {
                    // O must be complete (P V of tile j-1) before it is rescaled; P V of tile j cannot start before this thread's arrive below
                    if (!mbar_wait(bar_o_done, (j - 1) & 1, abort_flag)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t t_o = tmem + kColO + lane_base;
#pragma unroll 1
                    for (int cc = 0; cc < 4; ++cc) {
                        uint32_t o[32];
                        tmem_ld32(t_o + 32 * cc, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * f);
                        tmem_st32(t_o + 32 * cc, o);
                    }
                    tmem_wait_st();
                }
            }
            // P = e4m3(2^(s - ref + offset)), four keys per 32-bit TMEM column; l adds what P V will add
            const float sh = kPOffset - ref;
            uint32_t pw[32];
            float lsum = 0.0f;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                uint32_t lo, hi;
                lo = cvt_e4m3x2(ex2_approx(__uint_as_float(s0[4 * c]) + sh), ex2_approx(__uint_as_float(s0[4 * c + 1]) + sh));
                hi = cvt_e4m3x2(ex2_approx(__uint_as_float(s0[4 * c + 2]) + sh), ex2_approx(__uint_as_float(s0[4 * c + 3]) + sh));
                lsum += sum_e4m3x2(lo) + sum_e4m3x2(hi);
                pw[c] = lo | (hi << 16);
                lo = cvt_e4m3x2(ex2_approx(__uint_as_float(s1[4 * c]) + sh), ex2_approx(__uint_as_float(s1[4 * c + 1]) + sh));
                hi = cvt_e4m3x2(ex2_approx(__uint_as_float(s1[4 * c + 2]) + sh), ex2_approx(__uint_as_float(s1[4 * c + 3]) + sh));
                lsum += sum_e4m3x2(lo) + sum_e4m3x2(hi);
                pw[8 + c] = lo | (hi << 16);
                lo = cvt_e4m3x2(ex2_approx(__uint_as_float(s2[4 * c]) + sh), ex2_approx(__uint_as_float(s2[4 * c + 1]) + sh));
                hi = cvt_e4m3x2(ex2_approx(__uint_as_float(s2[4 * c + 2]) + sh), ex2_approx(__uint_as_float(s2[4 * c + 3]) + sh));
                lsum += sum_e4m3x2(lo) + sum_e4m3x2(hi);
                pw[16 + c] = lo | (hi << 16);
                lo = cvt_e4m3x2(ex2_approx(__uint_as_float(s3[4 * c]) + sh), ex2_approx(__uint_as_float(s3[4 * c + 1]) + sh));
                hi = cvt_e4m3x2(ex2_approx(__uint_as_float(s3[4 * c + 2]) + sh), ex2_approx(__uint_as_float(s3[4 * c + 3]) + sh));
                lsum += sum_e4m3x2(lo) + sum_e4m3x2(hi);
                pw[24 + c] = lo | (hi << 16);
            }
            l += lsum;
            if (tracing && j == 0) {
#pragma unroll
                for (int c = 0; c < 32; ++c) reinterpret_cast<uint32_t*>(p.trace)[32768 + 256 + r * 32 + c] = pw[c];
            }
            tmem_st32(t_s, pw);
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(bar_p_full(j & 1));
        }

        // ---- epilogue: O * v_descale / l ----
        if (ok && n_tiles > 0) ok = mbar_wait(bar_o_done, (n_tiles - 1) & 1, abort_flag);
        tc_fence_after_sync();
        if (ok && n_tiles > 0) {
            const float vd = *p.v_descale;
            const float fin = vd / l;   // crates/amdgpu-stage/src/attention/state.rs:79-82
            const uint32_t row = row0 + r;
            const bool row_ok = row < p.S;   // rows past the sequence are computed on clamped scales and not stored (block3.rs:194)
            const uint32_t t_o = tmem + kColO + lane_base;
            if (tracing) {
                p.trace[32768 + r] = l;
                p.trace[32768 + 128 + r] = ref;
            }
#pragma unroll 1
            for (int cc = 0; cc < 4; ++cc) {
                uint32_t o[32];
                tmem_ld32(t_o + 32 * cc, o);
                tmem_wait_ld();
                if (tracing) {
#pragma unroll
                    for (int c = 0; c < 32; ++c) p.trace[16384 + r * 128 + 32 * cc + c] = __uint_as_float(o[c]);
                }
                if (!row_ok) continue;
                if (kSplit) {
                    const size_t prow = static_cast<size_t>(split) * p.rows_total + (static_cast<size_t>(batch) * p.S + row) * p.H + head;
                    float4* dst = reinterpret_cast<float4*>(p.ohat + prow * 128 + 32 * cc);
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        dst[c] = make_float4(__uint_as_float(o[4 * c]) * fin, __uint_as_float(o[4 * c + 1]) * fin,
                                             __uint_as_float(o[4 * c + 2]) * fin, __uint_as_float(o[4 * c + 3]) * fin);
                    }
                } else {
                    uint8_t* orow = p.o + static_cast<size_t>(batch) * p.o_batch_stride + static_cast<size_t>(row) * p.o_row_stride + head * 256u;
                    uint4* dst = reinterpret_cast<uint4*>(orow + 64 * cc);
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t wv[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(o[8 * c + 2 * e]) * fin, __uint_as_float(o[8 * c + 2 * e + 1]) * fin);
                            wv[e] = *reinterpret_cast<const uint32_t*>(&b2);
                        }
                        dst[c] = make_uint4(wv[0], wv[1], wv[2], wv[3]);
                    }
                }
            }
            if (row_ok) {
                const float lse2 = ref - kPOffset + lg2_approx(l);   // log2 of sum_j 2^(s_j)
                if (kSplit) {
                    const size_t prow = static_cast<size_t>(split) * p.rows_total + (static_cast<size_t>(batch) * p.S + row) * p.H + head;
                    p.lse2[prow] = lse2;
                } else if (p.lse_nat != nullptr) {
                    p.lse_nat[(static_cast<size_t>(batch) * p.H + head) * p.S + row] = lse2 * 0.6931471805599453f;
                }
            }
        }
    }

    // ---- teardown ----
    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag != 0u) atomicOr(p.status, 1u);
    if (warp == 4) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, kTmemCols);
    }
}

cudaError_t launch_attention(const CUtensorMap& tm_q, const CUtensorMap& tm_k, const CUtensorMap& tm_v, const AttnParams& p,
                             uint32_t B, bool split, uint32_t rows_per_cta, cudaStream_t stream) {
    (void)rows_per_cta;   // both logical block heights run as 128-row CTAs
    static bool attr_done[2] = {false, false};
    cudaError_t e;
    if (!attr_done[split ? 1 : 0]) {
        e = split ? cudaFuncSetAttribute(fmha_fwd_mxfp8_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes)
                  : cudaFuncSetAttribute(fmha_fwd_mxfp8_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return e;
        attr_done[split ? 1 : 0] = true;
    }
    dim3 grid((p.S + kRows - 1) / kRows, p.H, B * (split ? p.splits : 1u));
    if (split) {
        fmha_fwd_mxfp8_kernel<true><<<grid, kThreads, kSmemBytes, stream>>>(tm_q, tm_k, tm_v, p);
    } else {
        fmha_fwd_mxfp8_kernel<false><<<grid, kThreads, kSmemBytes, stream>>>(tm_q, tm_k, tm_v, p);
    }
    return cudaGetLastError();
}

}  // namespace fmha
