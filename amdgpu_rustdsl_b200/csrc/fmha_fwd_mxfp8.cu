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
// Mapping onto the SM (not a translation of the gfx950 wave layout), 19 warps:
//   warp  0    Q K^T issuer: one lane issues S[j % 2] = Q K_j^T as kind::mxf8f6f4.block_scale tcgen05.mma, both operands in swizzled
//              shared memory, the E8M0 factors copied to TMEM with tcgen05.cp. Two score tiles are always ahead of the softmax.
//   warp  1    producer: TMA loads of the Q tile and of the K and V tiles into two rings (K is freed after Q K^T, V after P V), plus
//              the 4-byte-per-row scale gathers, which a TMA box cannot express, written in the 32x16-byte layout tcgen05.cp expects.
//   warp  2    P V issuer: O += P_j V_j with P from TMEM and V (keys x head dim, i.e. MN-major B) from shared memory. The B operand
//              is 144 wide: 128 head dims plus 16 columns of a tile of e4m3 ones, so that O[:, 128..143] (= the L columns) holds the
//              row sums of the *quantised* P at no ALU cost (the reference sums P with a matrix instruction too, reduce.rs:163-173).
//              A second issuing thread matters: one thread issues an MMA about every 75 clocks whatever its N.
//   warps 3-18 softmax + epilogue, four warpgroups: warpgroup 2 * half + parity works on key tiles j = parity (mod 2) and on keys
//              [64 half, 64 half + 64) of them. Thread r of a group owns query row r = TMEM lane r. Per tile it reads its 64 scores
//              twice with tcgen05.ld (maximum, then conversion: holding them would need more than the 96 registers that 19 warps
//              leave a thread), exchanges the half-row maximum with the sibling half and the row reference with the group of the
//              previous tile through 8-byte shared-memory slots {value, tile index}, writes P (packed e4m3) with tcgen05.st, and
//              rescales its half of O in TMEM on the rare tiles that move the reference.
// TMEM columns: S0 [0,128) S1 [128,256) O [256,384) L [384,400) P0 [400,432) P1 [432,464) SFQ [464,468) SFK0 [468,472) SFK1 [472,476).
#include "kernels.h"
#include "ptx_sm100.cuh"

#include <cuda_bf16.h>
#include <cuda_fp8.h>

namespace fmha {
using namespace sm100;

namespace {

constexpr int kRows = 128;          // query rows per CTA tile
constexpr int kKeys = 128;          // keys per tile
constexpr int kStages = 5;          // depth of the K ring and of the V ring (freed separately: K after Q K^T, V after P V)
// The three service warps get the lowest warp ids: the warp schedulers favour older warps, and a service warp that polls behind
// two arithmetic-dense softmax warps on its scheduler is otherwise only issued when they stall. Softmax = warps 3-18 (a warp's TMEM lane quadrant is warp % 4, so any four consecutive warps cover the 128 rows).
constexpr int kMmaWarp = 0, kProducerWarp = 1, kPvWarp = 2, kFirstSoftmaxWarp = 3;
constexpr int kThreads = 32 * (3 + 16);   // 19 warps: five on three of the four schedulers, hence 96 registers per thread
constexpr uint32_t kTileBytes = 128 * 128;   // one e4m3 tile
constexpr uint32_t kSfBytes = 512;           // 128 rows x 4 scale bytes

constexpr uint32_t kColS0 = 0, kColS1 = 128, kColO = 256, kColL = 384, kColP0 = 400, kColP1 = 432, kColSfQ = 464, kColSfK0 = 468, kColSfK1 = 472;
constexpr uint32_t kTmemCols = 512;

// P = 2^(s - ref + kPOffset): the row's reference maps to 2^kPOffset.
// Long sequences (>= 4 key tiles): the reference is an integer, ceil(tile maximum), and is left alone while a tile's maximum stays
// within kLazyThreshold binades above it, so P <= 2^(5 + 3.5) = 362 < 448 never saturates e4m3. Integer references make every
// rescale an exact power of two, so the same keys give the same P mantissas whatever the reference: a KV split and the unsplit
// kernel then differ only by f32 summation order.
// Short sequences move the reference to the tile's own maximum on every tile whose maximum is less than kFollowWindow binades
// below it (so every tile's largest P is exactly 2^kPOffset, which is what keeps the error on sharply peaked rows at the level of
// the reference's short-sequence recipe: thr 120/512 vs target 131/512, crates/amdgpu-tile/src/softmax.rs:26-30).
constexpr float kPOffset = 5.0f;
constexpr float kLazyThreshold = 3.5f;
constexpr float kFollowWindow = 11.0f;

struct SmemLayout {
    // all tile buffers are 1024-byte aligned (128-byte swizzle atom = 8 rows x 128 B)
    static constexpr uint32_t q = 0;
    static constexpr uint32_t k = q + kTileBytes;
    static constexpr uint32_t v = k + kStages * kTileBytes;
    // 32 keys x 128 B of e4m3 1.0 behind the V ring: a second MN-major atom of the P V B operand, of which the MMA uses 16 columns,
    // so that O[:, 128..143] accumulates the row sums of P
    static constexpr uint32_t ones = v + kStages * kTileBytes;
    static constexpr uint32_t sfq = ones + 4096;
    static constexpr uint32_t sfk = sfq + kSfBytes;
    static constexpr uint32_t xref = sfk + kStages * kSfBytes;   // [tile parity 2][half 2][row 128] x {reference bits, tile index}
    static constexpr uint32_t xmax = xref + 2 * 2 * 128 * 8;     // [buffer 2][tile parity 2][half 2][row 128] x {half-row maximum bits, tile index}
    static constexpr uint32_t bars = xmax + 2 * 2 * 2 * 128 * 8;
    // barriers (8 bytes each): q_full, k_full[kStages], k_empty[kStages], v_full[kStages], v_empty[kStages], s_full[2], s_free[2], p_full[2], o_done[2]
    static constexpr uint32_t n_bars = 1 + 4 * kStages + 8;
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
__device__ __forceinline__ float max3(float a, float b, float c) {
    float y;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
    return y;
}

// Two floats -> two e4m3 bytes (round to nearest even, saturating), `a` in the low byte.
__device__ __forceinline__ uint32_t cvt_e4m3x2(float a, float b) {
    uint16_t h;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(h) : "f"(b), "f"(a));
    return static_cast<uint32_t>(h);
}

// Four scores -> one 32-bit word of four e4m3 P values, key order = byte order.
__device__ __forceinline__ uint32_t p_word(uint32_t s0, uint32_t s1, uint32_t s2, uint32_t s3, float sh) {
    const uint32_t lo = cvt_e4m3x2(ex2_approx(__uint_as_float(s0) + sh), ex2_approx(__uint_as_float(s1) + sh));
    const uint32_t hi = cvt_e4m3x2(ex2_approx(__uint_as_float(s2) + sh), ex2_approx(__uint_as_float(s3) + sh));
    return lo | (hi << 16);
}

// The long-sequence conversion: the exp2 unit delivers 16 results per clock per SM, a quarter of what the score tiles need at full
// tensor rate, so two of every four P values are produced on the FMA pipe instead, straight as e4m3 bit patterns:
// byte = rne(8 (x + 7)) with x = log2 P, i.e. exponent field = floor(x) + 7 and a mantissa that is linear in the fraction of x
// (the piecewise-linear exp2 the reference uses for all of P, crates/amdgpu-tile/src/reduce.rs:94-113, docs/vendor-spec.md:271-281).
// fma.sat clamps to [0, 1] = bytes 0..256 (so -inf scores give 0), and adding 2^15 leaves rne(256 t) in the low byte of the sum.
// The linear mantissa overestimates 2^frac by 3.97 % on average; kFastBias shifts x so that the two kinds of P values agree on
// average, otherwise mixing them in one row sum would bias the weights.
constexpr float kFastBias = 0.0562f;
__device__ __forceinline__ uint32_t fast_p_bits(uint32_t s, float c) {
    float t;
    asm("fma.rn.sat.f32 %0, %1, 0f3D000000, %2;" : "=f"(t) : "f"(__uint_as_float(s)), "f"(c));   // s / 32 + c
    return __float_as_uint(t + 32768.0f);
}
__device__ __forceinline__ uint32_t p_word_hybrid(uint32_t s0, uint32_t s1, uint32_t s2, uint32_t s3, float sh, float c) {
    const uint32_t lo = cvt_e4m3x2(ex2_approx(__uint_as_float(s0) + sh), ex2_approx(__uint_as_float(s1) + sh));
    const uint32_t hi = __byte_perm(fast_p_bits(s2, c), fast_p_bits(s3, c), 0x0040);
    return __byte_perm(lo, hi, 0x5410);
}

__device__ __forceinline__ void st_shared_v2(uint32_t addr, uint32_t a, uint32_t b) {
    asm volatile("st.volatile.shared.v2.u32 [%0], {%1, %2};" ::"r"(addr), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ uint2 ld_shared_v2(uint32_t addr) {
    uint2 v;
    asm volatile("ld.volatile.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr) : "memory");
    return v;
}

// Time stamps of logical block (0,0,0) for the first 32 key tiles (the analogue of the reference's in-kernel stamp buffer,
// docs/stamps.md): [role 4: softmax group 0, 1, score MMAs, P V MMAs][tile 32][slot 8] 64-bit SM clock values behind the first 37120 words of the trace buffer.
constexpr int kStampBase = 37120;
template <bool kTrace>
__device__ __forceinline__ void stamp_t(float* trace, int role, int tile, int slot) {
    if (kTrace && trace != nullptr && tile < 32) reinterpret_cast<long long*>(trace + kStampBase)[(role * 32 + tile) * 8 + slot] = clock64();
}

// O columns [col, col + 32) of this thread's lane *= f
__device__ __forceinline__ void scale_tmem32(uint32_t taddr, float f) {
    uint32_t o[32];
    tmem_ld32(taddr, o);
    tmem_wait_ld();
#pragma unroll
    for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * f);
    tmem_st32(taddr, o);
}

}  // namespace

// kTrace = false compiles every diagnostic (tile dumps, time stamps) out of the tile loop: the production launches use that variant.
template <bool kSplit, bool kTrace>
__global__ void __maxnreg__(96)
fmha_fwd_mxfp8_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
    auto stamp = [](float* trace, int role, int tile, int slot) { stamp_t<kTrace>(trace, role, tile, slot); };
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    const uint32_t q_smem = smem_base + SmemLayout::q;
    const uint32_t k_smem = smem_base + SmemLayout::k;
    const uint32_t v_smem = smem_base + SmemLayout::v;
    const uint32_t ones_smem = smem_base + SmemLayout::ones;
    const uint32_t sfq_smem = smem_base + SmemLayout::sfq;
    const uint32_t sfk_smem = smem_base + SmemLayout::sfk;
    const uint32_t bar0 = smem_base + SmemLayout::bars;
    const uint32_t bar_q_full = bar0;
    auto bar_k_full = [&](int st) { return bar0 + 8u * (1 + st); };
    auto bar_k_empty = [&](int st) { return bar0 + 8u * (1 + kStages + st); };
    auto bar_v_full = [&](int st) { return bar0 + 8u * (1 + 2 * kStages + st); };
    auto bar_v_empty = [&](int st) { return bar0 + 8u * (1 + 3 * kStages + st); };
    auto bar_s_full = [&](int b) { return bar0 + 8u * (1 + 4 * kStages + b); };
    auto bar_s_free = [&](int b) { return bar0 + 8u * (3 + 4 * kStages + b); };
    auto bar_p_full = [&](int b) { return bar0 + 8u * (5 + 4 * kStages + b); };
    auto bar_o_done = [&](int b) { return bar0 + 8u * (7 + 4 * kStages + b); };
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
    const float thr = lazy ? kLazyThreshold : -kFollowWindow;

    // ---- one-time setup ----
    if (threadIdx.x == 0) {
        *abort_flag = 0u;
        mbar_init(bar_q_full, 1);
        for (int st = 0; st < kStages; ++st) {
            mbar_init(bar_k_full(st), 1);
            mbar_init(bar_k_empty(st), 1);
            mbar_init(bar_v_full(st), 1);
            mbar_init(bar_v_empty(st), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_s_full(b), 1);
            mbar_init(bar_s_free(b), 2 * kRows);
            mbar_init(bar_p_full(b), 2 * kRows);
            mbar_init(bar_o_done(b), 1);
        }
        fence_mbar_init();
    }
    if (threadIdx.x < 512) {
        for (int i = 0; i < 2; ++i) reinterpret_cast<uint32_t*>(smem_gen + SmemLayout::ones)[threadIdx.x + 512 * i] = 0x38383838u;
        // hand-over slots (512 reference slots, then 1024 maximum slots) start with a tile index no tile has
        for (int i = 0; i < 3; ++i) reinterpret_cast<uint2*>(smem_gen + SmemLayout::xref)[threadIdx.x + 512 * i] = make_uint2(0u, 0xFFFFFFFFu);
        fence_proxy_async_smem();
    }
    if (warp == kMmaWarp) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
        tmem_relinquish();
    }
    if (warp == kProducerWarp && lane == 0) {
        prefetch_tmap(&tm_q);
        prefetch_tmap(&tm_k);
        prefetch_tmap(&tm_v);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp == kProducerWarp) {
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
        // K scale words are fetched two tiles ahead into registers, so their global-load latency never sits on the ring's critical path
        auto load_k_scales = [&](int j, uint32_t (&w)[4]) {
            const uint32_t key0 = key_lo + j * kKeys;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t key = key0 + lane + 32 * i;
                w[i] = 0x7F7F7F7Fu;   // keys past the sequence: data is zero-filled by TMA, any finite scale does
                if (j < n_tiles && key < p.SK) {
                    const size_t off = static_cast<size_t>(batch) * p.ks_batch_stride + (static_cast<size_t>(key) * p.HK + kv_head) * 4u;
                    w[i] = __ldg(reinterpret_cast<const uint32_t*>(p.k_descale + off));
                }
            }
        };
        uint32_t wa[4], wb[4];
        load_k_scales(0, wa);
        load_k_scales(1, wb);
        // Event loop over the two rings: the next K tile (with its scales) goes out as soon as Q K^T of the tile that held its stage is
        // done, the next V tile as soon as P V of the tile that held its stage is done; neither waits for the other.
        int k_next = 0, v_next = 0;
        bool ok = true;
        long long t_idle = clock64();
        while (ok && (k_next < n_tiles || v_next < n_tiles)) {
            bool progressed = false;
            if (k_next < n_tiles) {
                const int j = k_next, st = j % kStages;
                bool rdy = j < kStages || mbar_test_wait(bar_k_empty(st), ((j / kStages) - 1) & 1);
                rdy = __shfl_sync(0xFFFFFFFFu, rdy ? 1 : 0, 0) != 0;
                if (rdy) {
                    uint32_t w[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) w[i] = (j & 1) ? wb[i] : wa[i];
                    if (j & 1) load_k_scales(j + 2, wb); else load_k_scales(j + 2, wa);
                    *reinterpret_cast<uint4*>(smem_gen + SmemLayout::sfk + st * kSfBytes + lane * 16) = make_uint4(w[0], w[1], w[2], w[3]);
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        stamp((blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) ? p.trace : nullptr, 2, j, 6);
                        mbar_arrive_expect_tx(bar_k_full(st), kTileBytes);
                        tma_load_4d(k_smem + st * kTileBytes, &tm_k, bar_k_full(st), 0, static_cast<int>(kv_head), static_cast<int>(key_lo + j * kKeys), static_cast<int>(batch));
                    }
                    ++k_next;
                    progressed = true;
                }
            }
            if (v_next < n_tiles) {
                const int j = v_next, st = j % kStages;
                bool rdy = j < kStages || mbar_test_wait(bar_v_empty(st), ((j / kStages) - 1) & 1);
                rdy = __shfl_sync(0xFFFFFFFFu, rdy ? 1 : 0, 0) != 0;
                if (rdy) {
                    if (lane == 0) {
                        stamp((blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) ? p.trace : nullptr, 3, j, 6);
                        mbar_arrive_expect_tx(bar_v_full(st), kTileBytes);
                        tma_load_4d(v_smem + st * kTileBytes, &tm_v, bar_v_full(st), 0, static_cast<int>(kv_head), static_cast<int>(key_lo + j * kKeys), static_cast<int>(batch));
                    }
                    ++v_next;
                    progressed = true;
                }
            }
            if (progressed) {
                t_idle = clock64();
            } else {

                if (*abort_flag != 0u || clock64() - t_idle > kWaitBudgetCycles) {
                    *abort_flag = 1u;
                    ok = false;
                }
            }
        }
        if (*abort_flag != 0u) {
            // leaving early: let the copies already in flight land before the CTA's shared memory is given back
            for (int j = max(0, k_next - kStages); j < k_next; ++j) {
                const long long t0 = clock64();
                while (!mbar_test_wait(bar_k_full(j % kStages), (j / kStages) & 1) && clock64() - t0 < kWaitBudgetCycles) {}
            }
            for (int j = max(0, v_next - kStages); j < v_next; ++j) {
                const long long t0 = clock64();
                while (!mbar_test_wait(bar_v_full(j % kStages), (j / kStages) & 1) && clock64() - t0 < kWaitBudgetCycles) {}
            }
        }
    } else if (warp == kMmaWarp) {
        // =========================================================== MMA issuer: score tiles ===========================================================
        // One lane runs the role. A tcgen05.mma costs its issuing thread about as long as the tensor pipe needs for a 128 x 128 x 32
        // tile, so Q K^T and P V are issued by two different threads (this warp and kPvWarp): their streams share no operand, and the
        // pipe interleaves them. Polls are non-blocking and descriptors are prepared once.
        if (lane == 0) {
            const uint32_t idesc_qk = idesc_mxf8_block_scaled(128, 128, 0, 0, 0, 0);
            const uint32_t t_sfq = tmem + kColSfQ;
            float* mma_trace = (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) ? p.trace : nullptr;
            // K-major 128-byte-swizzled Q / K tiles: 8-row groups 1024 B apart, 32 head-dim bytes (two 16-byte units) per MMA
            const uint64_t dq0 = make_smem_desc(q_smem, 16, 1024, kSwizzle128B);
            const uint64_t dk0 = make_smem_desc(k_smem, 16, 1024, kSwizzle128B);
            const uint64_t dsf0 = make_smem_desc(sfk_smem, 0, 128, kSwizzleNone);

            bool ok = mbar_wait(bar_q_full, 0, abort_flag);
            tc_fence_after_sync();
            if (ok) tmem_cp_sf(t_sfq, make_smem_desc(sfq_smem, 0, 128, kSwizzleNone));

            long long t_idle = clock64();
            for (int j = 0; ok && j < n_tiles;) {
                // S[j&1] = Q K(j)^T: needs the K tile and its scales, and the softmax of tile j-2 to have read S[j&1] out
                const int st = j % kStages;
                if (mbar_test_wait(bar_k_full(st), (j / kStages) & 1) && (j < 2 || mbar_test_wait(bar_s_free(j & 1), ((j >> 1) - 1) & 1))) {
                    tc_fence_after_sync();
                    stamp(mma_trace, 2, j, 2);
                    const uint32_t t_sfk = tmem + ((j & 1) ? kColSfK1 : kColSfK0);
                    const uint32_t t_s = tmem + ((j & 1) ? kColS1 : kColS0);
                    tmem_cp_sf(t_sfk, dsf0 + static_cast<uint64_t>((st * kSfBytes) >> 4));
                    const uint64_t dk = dk0 + static_cast<uint64_t>((st * kTileBytes) >> 4);
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb) {
                        const uint32_t id = idesc_qk | (static_cast<uint32_t>(kb) << 29) | (static_cast<uint32_t>(kb) << 4);
                        mma_mxf8_ss(t_s, dq0 + 2u * kb, dk + 2u * kb, id, t_sfq + (static_cast<uint32_t>(kb) << 30),
                                    t_sfk + (static_cast<uint32_t>(kb) << 30), kb > 0 ? 1u : 0u);
                    }
                    stamp(mma_trace, 2, j, 4);
                    tc_commit(bar_s_full(j & 1));
                    tc_commit(bar_k_empty(st));
                    stamp(mma_trace, 2, j, 5);
                    ++j;
                    t_idle = clock64();
                } else if (*abort_flag != 0u || clock64() - t_idle > kWaitBudgetCycles) {
                    *abort_flag = 1u;
                    ok = false;
                }
            }
        }
        __syncwarp();
    } else if (warp == kPvWarp) {
        // =========================================================== MMA issuer: P V ===========================================================
        if (lane == 0) {
            // P V with N = 144: head dims 0..127 from the V tile, 16 more columns from the tile of ones (O | L are adjacent in TMEM)
            const uint32_t idesc_pv = idesc_f8_dense(128, 144, 0, 1);
            float* mma_trace = (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) ? p.trace : nullptr;
            bool ok = true;
            long long t_idle = clock64();
            for (int i = 0; ok && i < n_tiles;) {
                // O (+)= P(i) V(i) with the row sums riding along: P from TMEM (32 columns, 8 per 32 keys), V tile = 128 keys x 128 B, MN-major
                const int st = i % kStages;
                if (mbar_test_wait(bar_p_full(i & 1), (i >> 1) & 1) && mbar_test_wait(bar_v_full(st), (i / kStages) & 1)) {
                    tc_fence_after_sync();
                    stamp(mma_trace, 3, i, 2);
                    const uint32_t t_p = tmem + ((i & 1) ? kColP1 : kColP0);
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb) {
                        // MN-major B: 8-key groups 1024 B apart; the second 128-byte-wide atom (columns 128..) is the tile of ones
                        const uint32_t v_addr = v_smem + st * kTileBytes + kb * 4096;
                        const uint64_t dv = make_smem_desc(v_addr, ones_smem - v_addr, 1024, kSwizzle128B);
                        mma_f8_ts(tmem + kColO, t_p + 8 * kb, dv, idesc_pv, (i > 0 || kb > 0) ? 1u : 0u);
                    }
                    stamp(mma_trace, 3, i, 3);
                    tc_commit(bar_v_empty(st));
                    tc_commit(bar_o_done(i & 1));
                    stamp(mma_trace, 3, i, 4);
                    ++i;
                    t_idle = clock64();
                } else if (*abort_flag != 0u || clock64() - t_idle > kWaitBudgetCycles) {
                    *abort_flag = 1u;
                    ok = false;
                }
            }
        }
        __syncwarp();
    } else if (warp >= kFirstSoftmaxWarp) {
        // =========================================================== softmax + epilogue ===========================================================
        // Four warpgroups: wg = 2 * half + parity. Parity = which key tiles (j = parity mod 2) and which S / P buffer; half = which 64 key
        // columns of the tile (and, in the epilogue, which 32 head dims together with the parity). Thread r of a group owns query row r.
        const uint32_t st_id = threadIdx.x - 32u * kFirstSoftmaxWarp;
        const uint32_t wg = st_id >> 7;
        const uint32_t par = wg & 1u, half = wg >> 1;
        const uint32_t r = 32u * (static_cast<uint32_t>(warp) & 3u) + static_cast<uint32_t>(lane);   // TMEM lane = 32 * (warp % 4) + lane
        const uint32_t lane_base = (static_cast<uint32_t>(warp & 3) * 32u) << 16;
        const uint32_t xref = smem_base + SmemLayout::xref;   // 8-byte slots, accessed with single 64-bit shared loads / stores
        const uint32_t xmax = smem_base + SmemLayout::xmax;
        const uint32_t t_s = tmem + (par ? kColS1 : kColS0) + lane_base + 64u * half;
        const uint32_t t_p = tmem + (par ? kColP1 : kColP0) + lane_base + 16u * half;
        const uint32_t t_o_half = tmem + kColO + lane_base + 64u * half;
        const uint32_t t_l = tmem + kColL + lane_base;
        float ref = -INFINITY;   // the row's reference (log2 units) after the last tile this thread has seen
        bool ok = true;
        const bool tracing = kTrace && (p.trace != nullptr) && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
        const bool dumping = tracing && !(p.flags & 0x4u);   // flag 0x4: time stamps only, no tile dumps

        // bounded poll of an 8-byte {value, tile index} slot
        auto wait_slot = [&](uint32_t slot, int j, float& out) -> bool {
            uint2 o = ld_shared_v2(slot);
            if (o.y != static_cast<uint32_t>(j)) {
                const long long t0 = clock64();
                while (true) {
                    o = ld_shared_v2(slot);
                    if (o.y == static_cast<uint32_t>(j)) break;
                    if (*abort_flag != 0u || clock64() - t0 > kWaitBudgetCycles) { *abort_flag = 1u; return false; }
                }
            }
            out = __uint_as_float(o.x);
            return true;
        };
        // the reference the row has after tile j: published by both half-row threads that handled tile j, read from the same half
        auto ref_slot = [&](int j) { return xref + 8u * ((static_cast<uint32_t>(j & 1) * 2u + half) * 128u + r); };
        // the half-row maximum of tile j: double buffered over this parity's consecutive tiles
        auto max_slot = [&](int j, uint32_t h) { return xmax + 8u * (((static_cast<uint32_t>((j >> 1) & 1) * 2u + par) * 2u + h) * 128u + r); };

        for (int j = static_cast<int>(par); j < n_tiles; j += 2) {
            const int k = j >> 1;   // this parity's tile counter
            float* st_trace = (tracing && r == 0 && half == 0) ? p.trace : nullptr;
            stamp(st_trace, par, j, 0);
            if (!mbar_wait(bar_s_full(par), k & 1, abort_flag)) { ok = false; break; }
            tc_fence_after_sync();
            stamp(st_trace, par, j, 1);
            // Pass 1 over the 64 scores of this half row, 32 at a time: the maximum only. The scores are read again for the conversion
            // below instead of being kept, which keeps a softmax thread under 96 registers (18 warps share the register file).
            const int nvalid = static_cast<int>(min(static_cast<uint32_t>(kKeys), key_hi - (key_lo + j * kKeys))) - 64 * static_cast<int>(half);
            float mt;
            {
                float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll 1
                for (int ch = 0; ch < 2; ++ch) {
                    uint32_t s[32];
                    tmem_ld32(t_s + 32 * ch, s);
                    tmem_wait_ld();
                    if (nvalid < 64) {   // keys past the range: -inf for the maximum, 0 for P (crates/amdgpu-tile/src/reduce.rs:35-49)
#pragma unroll
                        for (int c = 0; c < 32; ++c) {
                            if (c + 32 * ch >= nvalid) s[c] = 0xFF800000u;
                        }
                    }
                    if (dumping && j == 0) {
#pragma unroll
                        for (int c = 0; c < 32; ++c) p.trace[r * 128 + 64 * half + 32 * ch + c] = __uint_as_float(s[c]);
                    }
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {   // four independent chains of three-input maxima
                        m0 = max3(m0, __uint_as_float(s[c]), __uint_as_float(s[c + 1]));
                        m1 = max3(m1, __uint_as_float(s[c + 2]), __uint_as_float(s[c + 3]));
                        m2 = max3(m2, __uint_as_float(s[c + 4]), __uint_as_float(s[c + 5]));
                        m3 = max3(m3, __uint_as_float(s[c + 6]), __uint_as_float(s[c + 7]));
                    }
                }
                mt = fmaxf(max3(m0, m1, m2), m3);
            }
            stamp(st_trace, par, j, 2);
            // exchange the half-row maxima with the thread that holds the other 64 keys of this row
            st_shared_v2(max_slot(j, half), __float_as_uint(mt), static_cast<uint32_t>(j));
            stamp(st_trace, par, j, 3);
            {
                float other = mt;
                if (!wait_slot(max_slot(j, half ^ 1u), j, other)) ok = false;
                mt = fmaxf(mt, other);
            }
            // take over the row's reference from the threads that handled tile j - 1
            if (ok && j > 0 && !wait_slot(ref_slot(j - 1), j - 1, ref)) ok = false;
            if (!__all_sync(0xFFFFFFFFu, ok)) { ok = false; break; }
            // the reference moves when this tile's maximum passes it by more than the threshold (negative for short sequences: it then
            // also follows the tile maximum down, and f > 1 scales O and L up). Both halves of a row see the same mt and ref.
            const bool move = mt > ref + thr;
            float f = 1.0f;
            if (move) {
                const float nref = lazy ? ceilf(mt) : mt;
                f = ex2_approx(ref - nref);   // 0 on the first tile (ref = -inf); an exact power of two for integer references
                ref = nref;
            }
            st_shared_v2(ref_slot(j), __float_as_uint(ref), static_cast<uint32_t>(j));
            stamp(st_trace, par, j, 4);
            // P V of this parity's previous tile must be done before its P columns are overwritten (and, observed in order, this keeps
            // the phase parity of the other parity's barrier below unambiguous)
            if (k > 0 && !mbar_wait(bar_o_done(par), (k - 1) & 1, abort_flag)) { ok = false; break; }
            stamp(st_trace, par, j, 5);
            if (j > 0 && __any_sync(0xFFFFFFFFu, move)) {
                // O holds P V of all tiles before j once the other parity's last P V is done; P V of tile j cannot start before this thread's arrive below
                if (!mbar_wait(bar_o_done(par ^ 1u), ((j - 1) >> 1) & 1, abort_flag)) { ok = false; break; }
                tc_fence_after_sync();
                scale_tmem32(t_o_half, f);
                scale_tmem32(t_o_half + 32, f);
                if (half == 0) {   // the row sum lives in column 0 of L
                    uint32_t lv;
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(lv) : "r"(t_l) : "memory");
                    tmem_wait_ld();
                    lv = __float_as_uint(__uint_as_float(lv) * f);
                    asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(t_l), "r"(lv) : "memory");
                }
                tmem_wait_st();
            }
            // Pass 2: P = e4m3(2^(s - ref + offset)), four keys per 32-bit TMEM column
            const float sh = kPOffset - ref;
            const float cf = (kPOffset + 7.0f - kFastBias - ref) * 0.03125f;
            uint32_t pw[16];
#pragma unroll
            for (int ch = 0; ch < 2; ++ch) {
                uint32_t s[32];
                tmem_ld32(t_s + 32 * ch, s);
                tmem_wait_ld();
                if (ch == 1) {
                    tc_fence_before_sync();
                    mbar_arrive(bar_s_free(par));   // the score buffer can take tile j + 2 once all 256 threads of this parity are done with it
                }
                if (nvalid < 64) {
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        if (c + 32 * ch >= nvalid) s[c] = 0xFF800000u;
                    }
                }
                if (lazy) {
#pragma unroll
                    for (int c = 0; c < 8; ++c) pw[8 * ch + c] = p_word_hybrid(s[4 * c], s[4 * c + 1], s[4 * c + 2], s[4 * c + 3], sh, cf);
                } else {
#pragma unroll
                    for (int c = 0; c < 8; ++c) pw[8 * ch + c] = p_word(s[4 * c], s[4 * c + 1], s[4 * c + 2], s[4 * c + 3], sh);
                }
            }
            if (dumping && j == 0) {
#pragma unroll
                for (int c = 0; c < 16; ++c) reinterpret_cast<uint32_t*>(p.trace)[32768 + 256 + r * 32 + 16 * half + c] = pw[c];
            }
            stamp(st_trace, par, j, 6);
            tmem_st16(t_p, pw);
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(bar_p_full(par));
            stamp(st_trace, par, j, 7);
        }

        // ---- epilogue: O * v_descale / l; warpgroup wg stores head dims [32 wg, 32 wg + 32) ----
        if (ok && n_tiles > 0) {
            const int last = n_tiles - 1;
            const int mine = ((last & 1) == static_cast<int>(par)) ? last : last - 1;   // this parity's last tile (-1: none)
            if (mine >= 0) ok = mbar_wait(bar_o_done(par), (mine >> 1) & 1, abort_flag);
            const int theirs = ((last & 1) == static_cast<int>(par)) ? last - 1 : last;
            if (ok && theirs >= 0) ok = mbar_wait(bar_o_done(par ^ 1u), (theirs >> 1) & 1, abort_flag);
            if (ok) ok = wait_slot(ref_slot(last), last, ref);
        }
        tc_fence_after_sync();
        if (ok && n_tiles > 0) {
            uint32_t lv;
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(lv) : "r"(t_l) : "memory");
            tmem_wait_ld();
            const float l = __uint_as_float(lv);
            const float vd = *p.v_descale;
            const float fin = vd / l;   // crates/amdgpu-stage/src/attention/state.rs:79-82
            const uint32_t row = row0 + r;
            const bool row_ok = row < p.S;   // rows past the sequence are computed on clamped scales and not stored (block3.rs:194)
            if (tracing && wg == 0) {
                p.trace[32768 + r] = l;
                p.trace[32768 + 128 + r] = ref;
            }
            uint32_t o[32];
            tmem_ld32(tmem + kColO + lane_base + 32u * wg, o);
            tmem_wait_ld();
            if (dumping) {
#pragma unroll
                for (int c = 0; c < 32; ++c) p.trace[16384 + r * 128 + 32 * wg + c] = __uint_as_float(o[c]);
            }
            if (row_ok) {
                if (kSplit) {
                    const size_t prow = static_cast<size_t>(split) * p.rows_total + (static_cast<size_t>(batch) * p.S + row) * p.H + head;
                    float4* dst = reinterpret_cast<float4*>(p.ohat + prow * 128 + 32 * wg);
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        dst[c] = make_float4(__uint_as_float(o[4 * c]) * fin, __uint_as_float(o[4 * c + 1]) * fin,
                                             __uint_as_float(o[4 * c + 2]) * fin, __uint_as_float(o[4 * c + 3]) * fin);
                    }
                } else {
                    uint8_t* orow = p.o + static_cast<size_t>(batch) * p.o_batch_stride + static_cast<size_t>(row) * p.o_row_stride + head * 256u;
                    uint4* dst = reinterpret_cast<uint4*>(orow + 64 * wg);
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
                if (wg == 0) {
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
    }

    // ---- teardown ----
    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag != 0u) atomicOr(p.status, 1u);
    if (warp == kMmaWarp) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, kTmemCols);
    }
}

cudaError_t launch_attention(const CUtensorMap& tm_q, const CUtensorMap& tm_k, const CUtensorMap& tm_v, const AttnParams& p,
                             uint32_t B, bool split, uint32_t rows_per_cta, cudaStream_t stream) {
    (void)rows_per_cta;   // both logical block heights run as 128-row CTAs
    using Kernel = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const AttnParams);
    static const Kernel kernels[4] = {fmha_fwd_mxfp8_kernel<false, false>, fmha_fwd_mxfp8_kernel<true, false>,
                                      fmha_fwd_mxfp8_kernel<false, true>, fmha_fwd_mxfp8_kernel<true, true>};
    static bool attr_done[4] = {false, false, false, false};
    const int which = (split ? 1 : 0) + (p.trace != nullptr ? 2 : 0);
    if (!attr_done[which]) {
        const cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(kernels[which]), cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return e;
        attr_done[which] = true;
    }
    dim3 grid((p.S + kRows - 1) / kRows, p.H, B * (split ? p.splits : 1u));
    kernels[which]<<<grid, kThreads, kSmemBytes, stream>>>(tm_q, tm_k, tm_v, p);
    return cudaGetLastError();
}

}  // namespace fmha
