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
// Mapping onto the SM (not a translation of the gfx950 wave layout): a persistent kernel, one CTA of 16 warps per SM, each CTA walking
// work items (128 query rows of one (batch, head[, split])) with its rings, buffers and barriers running on across items.
// The four service warps run their loops with all 32 lanes in step on warp-uniform values and let an elected lane issue the tcgen05 /
// TMA instructions (operands then stay in uniform registers).
//   warp  0    Q K^T issuer: S[g % 2] = Q K_g^T as kind::mxf8f6f4.block_scale tcgen05.mma, both operands in swizzled shared memory,
//              the E8M0 factors copied to TMEM with tcgen05.cp. Two score tiles are always ahead of the softmax.
//   warp  1    Q / K producer: TMA loads of the Q tile (double buffered across items) and of the K ring, plus the 4-byte-per-row scale
//              gathers (Q, and K for the tiles with an even counter), which a TMA box cannot express, written in the 32x16-byte
//              layout tcgen05.cp expects.
//   warp  2    P V issuer: O += P_g V_g with P from TMEM and V (keys x head dim, i.e. MN-major B) from shared memory. The B operand
//              is 144 wide: 128 head dims plus 16 columns of a tile of e4m3 ones, so that O[:, 128..143] (= the L columns) holds the
//              row sums of the *quantised* P at no ALU cost (the reference sums P with a matrix instruction too, reduce.rs:163-173).
//              It has a thread of its own: the tensor pipe takes MMAs from one thread at its full rate, but a thread that shares its
//              scheduler with softmax warps only gets an instruction in every few clocks.
//   warp  3    V producer: TMA loads of the V ring (K is freed after Q K^T, V after P V, so the two rings run apart), and the K scale
//              gathers of the tiles with an odd counter.
//   warps 4-11 softmax, two warpgroups: warpgroup p works on the tiles with counter g = p (mod 2). Thread r of a group owns query row
//              r = TMEM lane r: it reads the row's 128 scores with one tensor-memory round trip and hands the S buffer back at once,
//              takes the row's reference from the group of the previous tile through an 8-byte shared-memory slot {value, tile
//              counter}, converts in place, writes P (packed e4m3) with tcgen05.st, and rescales O in TMEM on the rare tiles that move
//              the reference.
//   warps 12-15 epilogue, one warpgroup: takes an item's O and row sums out of tensor memory when its last P V is done, hands the
//              columns back (the next item's first P V waits for that), normalises, stages the tile in shared memory and stores it
//              with TMA (bf16 output, or the split kernel's partial), while the softmax warpgroups are on the next item's tiles.
//              Merges the two halves of an item cut between a pair of CTAs; in the fused instantiations merges a row block's partials.
//   Every thread starts with 128 registers; the service warps then keep 56, the softmax warps take 176 and the epilogue warps 104
//   (setmaxnreg: the roles' shares must come out of the CTA's launch allocation).
// TMEM columns: S0 [0,128) S1 [128,256) O [256,384) L [384,400) P0 [400,432) P1 [432,464) SFQ [464,468) SFK0 [468,472) SFK1 [472,476).
#include "kernels.h"
#include "ptx_sm100.cuh"

#include <cuda_bf16.h>

#include <atomic>
#include <mutex>
#include <type_traits>
#include <cuda_fp8.h>

namespace b200mx {
using namespace sm100;

namespace {

constexpr int kRows = 128;          // query rows per CTA tile
constexpr int kKeys = kKeysPerTile; // keys per tile (128)
constexpr int kStages = 4;          // depth of the K ring and of the V ring (freed separately: K after Q K^T, V after P V)
// The four service warps get the lowest warp ids, one per scheduler (scheduler = warp % 4). Softmax = warps 4-19: a warp's TMEM lane
// quadrant is warp % 4, so any four consecutive warps cover the 128 rows.
constexpr int kMmaWarp = 0, kKProducerWarp = 1, kPvWarp = 2, kVProducerWarp = 3, kFirstSoftmaxWarp = 4, kFirstEpilogueWarp = 12;
// A softmax thread owns a whole score row of a tile: 128 scores in registers, read from tensor memory once. 4 service + 8 softmax + 4
// epilogue warps: every scheduler has one service, two softmax and one epilogue warp and 16 K registers to deal out among them.
constexpr int kCols = 128;                  // score columns per softmax thread
constexpr int kThreads = 32 * (4 + 8 + 4);   // 4 service warps, 8 softmax warps, 4 epilogue warps
// The register file (64 K registers) is dealt out unevenly once the roles part: every thread starts with kMaxRegs, the service and the
// epilogue warpgroups give most of theirs back and the two softmax warpgroups take them.
#ifndef MXA_SERVICE_REGS
#define MXA_SERVICE_REGS 56
#define MXA_SOFTMAX_REGS 176
#define MXA_EPILOGUE_REGS 104
#endif
constexpr int kMaxRegs = 128;
constexpr int kServiceRegs = MXA_SERVICE_REGS, kSoftmaxRegs = MXA_SOFTMAX_REGS, kEpilogueRegs = MXA_EPILOGUE_REGS;
// setmaxnreg.inc waits, without a bound, until the CTA's own pool has the registers, and the pool is what the CTA got at launch
// (kThreads x kMaxRegs), not the SM's register file: the roles together must never ask for more than that.
static_assert(kThreads * kMaxRegs <= 65536, "the CTA must fit the register file at launch");
static_assert(4 * kServiceRegs + 8 * kSoftmaxRegs + 4 * kEpilogueRegs <= (kThreads / 32) * kMaxRegs, "the roles' registers come out of the CTA's launch allocation");
static_assert(kServiceRegs % 8 == 0 && kSoftmaxRegs % 8 == 0 && kEpilogueRegs % 8 == 0 && kServiceRegs >= 24 && kEpilogueRegs >= 24 && kSoftmaxRegs <= 256, "register file split");
constexpr uint32_t kTileBytes = 128 * 128;   // one e4m3 tile
constexpr uint32_t kSfBytes = 512;           // 128 rows x 4 scale bytes

constexpr uint32_t kColS0 = 0, kColS1 = 128, kColO = 256, kColL = 384, kColP0 = 400, kColP1 = 432, kColSfQ = 464, kColSfK0 = 468, kColSfK1 = 472,
                   kColSfP = 476, kColSfV = 480;   // V block scales (extension): P's constant factors [476,480), V's factors [480,484) + the ones columns' [484,488)
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
constexpr uint32_t kFlagCausal = 0x8u;   // FMHA_MXFP8_FLAG_CAUSAL: selects the kCausal instantiations
constexpr uint32_t kFlagF32Partials = 0x10u;   // FMHA_MXFP8_FLAG_F32_PARTIALS: the split kernel's partial rows are f32, not f16
constexpr uint32_t kFlagNoTailSplit = 0x20u;   // FMHA_MXFP8_FLAG_NO_TAIL_SPLIT: never cut the last round's items in two

struct SmemLayout {
    // all tile buffers are 1024-byte aligned (128-byte swizzle atom = 8 rows x 128 B)
    static constexpr uint32_t q = 0;
    static constexpr uint32_t k = q + 2 * kTileBytes;   // two Q tiles: the next item's is loaded while the current one is in use
    static constexpr uint32_t v = k + kStages * kTileBytes;
    // 32 keys x 128 B of e4m3 1.0 behind the V ring: a second MN-major atom of the P V B operand, of which the MMA uses 16 columns,
    // so that O[:, 128..143] accumulates the row sums of P
    static constexpr uint32_t ones = v + kStages * kTileBytes;
    // two 16 KB staging tiles (128 rows x 64 bf16, 128-byte swizzle) for the output's TMA stores, one per warpgroup
    static constexpr uint32_t ostage = ones + 4096;
    static constexpr uint32_t sfq = ostage + 2 * 16384;
    static constexpr uint32_t sfk = sfq + 2 * kSfBytes;
    // [tile counter % 4][row 128] x {reference bits, tile counter}. Four slots per row, not two: a softmax warpgroup goes from an item's
    // last tile straight on to the next item's first, which reads no reference, so it may publish tile g while the other group has yet to
    // read what tile g - 2 left for its tile g - 1
    static constexpr uint32_t sfv = sfk + kStages * kSfBytes;    // V block scales of a key tile (extension), same 32 x 16-byte pattern as the K scales
    static constexpr uint32_t sf_one = sfv + kStages * kSfBytes;  // 512 bytes of E8M0 1.0: the factors of P and of the ones columns
    static constexpr uint32_t xref = sf_one + kSfBytes;
    // [item ordinal % 4][row 128]: the row's reference after the item's last tile, for the epilogue warpgroup. Four slots and a write
    // behind the wait for this parity's previous P V: with one-tile items a softmax group is otherwise two items ahead of the epilogue
    static constexpr uint32_t xfin = xref + 4 * 128 * 8;
    static constexpr uint32_t xstat = xfin + 4 * 128 * 4;         // [row 128] x {row sum, reference} of the partner's half item (launches as pairs)
    static constexpr uint32_t xlse = xstat + 128 * 8;             // fused merge: [row 128][split 8] log-sum-exps of the block being merged
    static constexpr uint32_t bars = xlse + 128 * 8 * 4;
    // barriers (8 bytes each): q_full[2], q_empty[2], k_full[kStages], k_empty[kStages], v_full[kStages], v_empty[kStages], s_full[2], s_free[2],
    // p_full[2], o_done[2], o_free, o_full, four unused, peer_rdy, peer_data
    static constexpr uint32_t n_bars = 4 + 4 * kStages + 16;
    static constexpr uint32_t tmem_slot = bars + 8 * n_bars;
    static constexpr uint32_t abort_flag = tmem_slot + 4;
    static constexpr uint32_t last_flag = abort_flag + 4;   // fused merge: "this CTA brought the row block's arrival count to `splits`"
    static constexpr uint32_t total = last_flag + 4;
};
constexpr uint32_t kSmemBytes = SmemLayout::total + 1024;   // + slack to align the base to 1024
static_assert(kSmemBytes <= 227 * 1024, "shared memory budget of one CTA");

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
// fma.sat clamps t = s / 32 + c to [0, 1] = bytes 0..256 (so -inf scores give 0), and adding 2^15 leaves rne(256 t) in the low byte of the
// sum. The additions (this one, and the shift in front of the exp2 of the other two values) are done two at a time (add.f32x2); the
// two-wide fma has no saturating form, so the clamped fma stays one per value.
// The linear mantissa overestimates 2^frac by 3.97 % on average; kFastBias shifts x so that the two kinds of P values agree on
// average, otherwise mixing them in one row sum would bias the weights.
constexpr float kFastBias = 0.0562f;
// Two f32 additions in one instruction (sm_100 has two-wide f32 add / mul / fma on 64-bit register pairs): a += c, b += c.
__device__ __forceinline__ void add2(uint32_t& a, uint32_t& b, float c) {
    unsigned long long p, q;
    asm("mov.b64 %0, {%1, %2};" : "=l"(p) : "r"(a), "r"(b));
    asm("mov.b64 %0, {%1, %1};" : "=l"(q) : "f"(c));
    asm("add.rn.ftz.f32x2 %0, %1, %2;" : "=l"(p) : "l"(p), "l"(q));
    asm("mov.b64 {%0, %1}, %2;" : "=r"(a), "=r"(b) : "l"(p));
}
// a *= c, b *= c in one instruction
__device__ __forceinline__ void mul2(uint32_t& a, uint32_t& b, float c) {
    unsigned long long p, q;
    asm("mov.b64 %0, {%1, %2};" : "=l"(p) : "r"(a), "r"(b));
    asm("mov.b64 %0, {%1, %1};" : "=l"(q) : "f"(c));
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(p) : "l"(p), "l"(q));
    asm("mov.b64 {%0, %1}, %2;" : "=r"(a), "=r"(b) : "l"(p));
}
__device__ __forceinline__ uint32_t fast_p_sat(uint32_t s, float c) {   // s / 32 + c clamped to [0, 1]
    float t;
    asm("fma.rn.sat.f32 %0, %1, 0f3D000000, %2;" : "=f"(t) : "f"(__uint_as_float(s)), "f"(c));
    return __float_as_uint(t);
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

// One unit of work of the persistent kernel: 128 query rows of one (batch, head) against the key range of one split.
struct Item {
    uint32_t row0, head, batch, split, kv_head, key_lo, key_hi;
    uint32_t half;   // 0: the item's whole key range; 1 / 2: its first / second half, to be merged with the other CTA of the cluster
    int n_tiles;
};

template <bool kSplit, bool kCausal, bool kPair>
__device__ __forceinline__ Item decode_item(uint32_t w, const AttnParams& p) {
    // w = (z * H + head) * n_qtiles + q tile: neighbouring CTAs work on neighbouring row blocks of one head, whose K / V they share in L2
    Item it;
    it.half = 0;
    if (kPair && w >= p.tail_base) {   // a unit of the cut last round: half (w - tail_base) % 2 of item tail_base + (w - tail_base) / 2
        it.half = 1u + ((w - p.tail_base) & 1u);
        w = p.tail_base + ((w - p.tail_base) >> 1);
    }
    uint32_t x = w % p.n_qtiles, yz = w / p.n_qtiles;
    constexpr bool causal = kCausal && !kSplit;
    if (causal) {
        // Items in the order of falling work (the row block's visible keys): rank = (n_qtiles - 1 - q tile) * (H * B) + (batch * H + head).
        // The CTAs walk the ranks in rounds of gridDim.x, odd rounds backwards, so that the CTA that got the heaviest item of one round
        // gets the lightest of the next and every CTA ends with about the same number of key tiles.
        const uint32_t round = w / gridDim.x, base = round * gridDim.x;
        uint32_t pos = w - base;
        if (round & 1u) pos = min(gridDim.x, p.n_items - base) - 1u - pos;
        const uint32_t rank = base + pos;
        const uint32_t hb = p.n_items / p.n_qtiles;
        x = p.n_qtiles - 1u - rank / hb;
        yz = rank % hb;
    }
    it.row0 = x * kRows;
    it.head = yz % p.H;
    const uint32_t z = yz / p.H;
    it.batch = z;
    it.split = 0;
    if (kSplit) {
        it.batch = z >> p.split_log2;
        it.split = z & (p.splits - 1u);
    }
    it.kv_head = it.head >> p.gqa_shift;   // crates/amdgpu-stage/src/components.rs:8-17
    const uint32_t ntiles_total = (p.SK + kKeys - 1) / kKeys;
    it.key_lo = 0;
    it.key_hi = p.SK;
    if (kSplit) {   // tiles [split*tps, min(ntiles, (split+1)*tps)) (components.rs:58-74)
        const uint32_t tps = (ntiles_total + p.splits - 1) / p.splits;
        const uint32_t tile_lo = it.split * tps;
        const uint32_t tile_hi = min(ntiles_total, tile_lo + tps);
        it.key_lo = tile_lo * kKeys;
        it.key_hi = min(tile_hi * kKeys, p.SK);
    }
    // causal (crates/amdgpu-stage/src/attention/attn3.rs:298-306): row i sees the keys below min(i + SK - S + 1, SK); the item's last row decides
    if (causal) it.key_hi = min(p.SK, it.row0 + kRows + (p.SK - p.S));
    it.n_tiles = (it.key_hi > it.key_lo) ? static_cast<int>((it.key_hi - it.key_lo + kKeys - 1) / kKeys) : 0;
    if (it.half != 0u) {   // whole tiles [0, ceil(n / 2)) to the first half, the rest (and a ragged end) to the second
        const int first = (it.n_tiles + 1) / 2;
        if (it.half == 1u) {
            it.key_hi = it.key_lo + static_cast<uint32_t>(first) * kKeys;
            it.n_tiles = first;
        } else {
            it.key_lo += static_cast<uint32_t>(first) * kKeys;
            it.n_tiles -= first;
        }
    }
    return it;
}

}  // namespace

// Persistent: gridDim.x CTAs (one per SM) walk the work items w = blockIdx.x, blockIdx.x + gridDim.x, ... The K / V rings, the score and P
// buffers and every barrier run on one tile counter g that keeps counting across items, so the next item's Q, K and V loads and its first
// two score tiles overlap the current item's last tiles and epilogue; only O is single: P V of an item's first tile waits until the
// epilogue of the item before has read O out (o_free).
// kTrace = false compiles every diagnostic (tile dumps, time stamps) out of the tile loop: the production launches use that variant.
// kLazy: the long-sequence softmax recipe. kCausal: the causal mask (never with kSplit).
// kFused: the split kernel with the merge of the partials built into its epilogue (no pairs, no diagnostics, f16 partials, no peer routing).
template <bool kSplit, bool kTrace, bool kLazy, bool kCausal, bool kPair, bool kVbs, bool kFused = false>
__global__ void __maxnreg__(kMaxRegs)
mxfp8_prefill_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o, const AttnParams p) {
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
    auto bar_q_full = [&](int b) { return bar0 + 8u * b; };
    auto bar_q_empty = [&](int b) { return bar0 + 8u * (2 + b); };
    auto bar_k_full = [&](int st) { return bar0 + 8u * (4 + st); };
    auto bar_k_empty = [&](int st) { return bar0 + 8u * (4 + kStages + st); };
    auto bar_v_full = [&](int st) { return bar0 + 8u * (4 + 2 * kStages + st); };
    auto bar_v_empty = [&](int st) { return bar0 + 8u * (4 + 3 * kStages + st); };
    auto bar_s_full = [&](int b) { return bar0 + 8u * (4 + 4 * kStages + b); };
    auto bar_s_free = [&](int b) { return bar0 + 8u * (6 + 4 * kStages + b); };
    auto bar_p_full = [&](int b) { return bar0 + 8u * (8 + 4 * kStages + b); };
    auto bar_o_done = [&](int b) { return bar0 + 8u * (10 + 4 * kStages + b); };
    const uint32_t bar_o_free = bar0 + 8u * (12 + 4 * kStages);
    const uint32_t bar_o_full = bar0 + 8u * (13 + 4 * kStages);
    // pairs: "this CTA's exchange area is free" (one arrival, from the partner with the first half) and "the partner's half item has
    // landed in this CTA's exchange area" (128 arrivals, from the partner with the second half)
    const uint32_t bar_peer_rdy = bar0 + 8u * (18 + 4 * kStages), bar_peer_data = bar0 + 8u * (19 + 4 * kStages);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + SmemLayout::tmem_slot);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem_gen + SmemLayout::abort_flag);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t n_items = p.n_work, stride = gridDim.x;   // the work units this grid walks (whole items, and halves of the last round's)
    // kLazy: the long-sequence recipe, chosen by the launcher from the whole sequence's tile count, also in a split (block3.rs:180-184)
    constexpr bool lazy = kLazy;
    constexpr float thr = lazy ? kLazyThreshold : -kFollowWindow;
    const bool cta_traced = kTrace && p.trace != nullptr && blockIdx.x == 0;   // diagnostics cover the first item of CTA 0 = logical block (0,0,0)

    // Programmatic dependent launch: the next launch in the stream (if it asks for it, as this library's own launches do) may be
    // scheduled while this grid runs; its CTAs become resident as ours exit and do their set-up, then wait below for this grid's end.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // ---- one-time setup ----
    if (threadIdx.x == 0) stamp(cta_traced ? p.trace : nullptr, 2, 30, 0);   // kernel entry
    if (threadIdx.x == 0) {
        *abort_flag = 0u;
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_q_full(b), 2);   // the TMA's expect-tx arrive + the arrive that follows the scale bytes
            mbar_init(bar_q_empty(b), 1);
            mbar_init(bar_s_full(b), 1);
            mbar_init(bar_s_free(b), kRows);
            mbar_init(bar_p_full(b), kRows);
            mbar_init(bar_o_done(b), 1);
        }
        for (int st = 0; st < kStages; ++st) {
            mbar_init(bar_k_full(st), 2);
            mbar_init(bar_k_empty(st), 1);
            mbar_init(bar_v_full(st), kVbs ? 2 : 1);   // with V block scales: the TMA's expect-tx arrive + the arrive that follows the scale bytes
            mbar_init(bar_v_empty(st), 1);
        }
        mbar_init(bar_o_free, kRows);   // the epilogue warpgroup's 128 threads
        mbar_init(bar_o_full, 1);
        mbar_init(bar_peer_rdy, 1);
        mbar_init(bar_peer_data, kRows);
        fence_mbar_init();
    }
    if (kVbs && threadIdx.x >= 256 && threadIdx.x < 384) {
        reinterpret_cast<uint32_t*>(smem_gen + SmemLayout::sf_one)[threadIdx.x - 256] = 0x7F7F7F7Fu;
        fence_proxy_async_smem();
    }
    if (threadIdx.x < 256) {
        for (int i = 0; i < 4; ++i) reinterpret_cast<uint32_t*>(smem_gen + SmemLayout::ones)[threadIdx.x + 256 * i] = 0x38383838u;
        // the 512 reference hand-over slots start with a tile counter no tile has
        reinterpret_cast<uint2*>(smem_gen + SmemLayout::xref)[threadIdx.x] = make_uint2(0u, 0xFFFFFFFFu);
        reinterpret_cast<uint2*>(smem_gen + SmemLayout::xref)[threadIdx.x + 256] = make_uint2(0u, 0xFFFFFFFFu);
        fence_proxy_async_smem();
    }
    if (warp == kMmaWarp) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
        tmem_relinquish();
    }
    if (warp == kKProducerWarp && lane == 0) {
        prefetch_tmap(&tm_q);
        prefetch_tmap(&tm_k);
    }
    if (warp == kVProducerWarp && lane == 0) prefetch_tmap(&tm_v);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    // launched as pairs (the last round's items are cut in two): the partner's barriers must exist before anything can arrive on them
    // Every thread arrives on the cluster's barrier here and waits for it only where it first touches the partner (the epilogue
    // warpgroup, the score MMA warp) or, failing that, at the end; by then the partner has long arrived, so nobody stands still for it.
    constexpr bool paired = kPair;
    bool cluster_joined = !paired;
    if (paired) asm volatile("barrier.cluster.arrive.release;" ::: "memory");
    auto join_cluster = [&]() {
        if (!cluster_joined) {
            asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
            cluster_joined = true;
        }
    };
    // nothing above touches global memory; everything below may read what the previous grid in the stream wrote
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (threadIdx.x == 0) stamp(cta_traced ? p.trace : nullptr, 2, 30, 2);   // setup done

    // The four service roles are single chains of dependent instructions that share their scheduler with four arithmetic-dense softmax
    // warps, so every instruction costs them several clocks: each role is its own warp, waits with blocking mbarrier waits (its
    // conditions are conjunctions, never alternatives) and keeps its per-tile instruction count small.
    // The register file is split unevenly: the kernel starts with kMaxRegs registers in every thread; the four service warps (one
    // warpgroup) give most of theirs back and the softmax warpgroups take them, which lets the compiler keep the whole score row plus
    // enough temporaries to interleave the conversion's dependent chains without spilling (4-6 % on the full machine).
    if (warp < kFirstSoftmaxWarp) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kServiceRegs));
    if (warp == kKProducerWarp || warp == kVProducerWarp) {
        // =========================================================== producers: Q, K, V tiles; Q and K scales ===========================================================
        // Warp 1 issues the Q and K tile copies and gathers the Q scales, warp 3 issues the V tile copies. The K scale bytes (4 per key,
        // strided by the head count, which a TMA box cannot express) are gathered by both: warp 1 takes the tiles with an even counter,
        // warp 3 the odd ones, so that neither warp's per-tile instruction stream is long (a producer that needs more clocks per tile
        // than the softmax sets the pace of the whole CTA). A tile's scales are loaded four tiles (two of the warp's own) ahead into
        // one of two register sets, each use naming its set statically, so that a tile never waits for loads issued behind it. The
        // scale cursor therefore walks the items on its own.
        auto producer = [&](auto is_k_c) {
            constexpr bool kIsK = decltype(is_k_c)::value;
            constexpr uint32_t kPar = kIsK ? 0u : 1u;   // parity of the tile counters whose K scales this warp gathers
            const uint32_t row_step = 32u * p.HK * 4u, tile_step = 4u * row_step;   // bytes between a lane's four keys / between key tiles
            struct ScaleCursor {
                const uint8_t* ptr;   // scale word of this lane's first key of the tile
                int keys_left;        // sequence keys from the tile's first key on (lanes compare against it)
                int tiles_left;       // of the item
                uint32_t w;           // the item
                bool live;
            };
            auto enter_item = [&](ScaleCursor& c) {
                c.live = c.w < n_items;
                if (!c.live) return;
                const Item it = decode_item<kSplit, kCausal, kPair>(c.w, p);
                c.ptr = p.k_descale + static_cast<size_t>(it.batch) * p.ks_batch_stride + (static_cast<size_t>(it.key_lo + lane) * p.HK + it.kv_head) * 4u;
                c.keys_left = static_cast<int>(p.SK - it.key_lo) - lane;
                c.tiles_left = it.n_tiles;
            };
            auto advance = [&](ScaleCursor& c) {
                if (!c.live) return;
                c.ptr += tile_step;
                c.keys_left -= kKeys;
                if (--c.tiles_left == 0) {
                    c.w += stride;
                    enter_item(c);
                }
            };
            // loads the scales of the cursor's tile and moves the cursor to the warp's next tile (two on)
            auto load_and_advance = [&](ScaleCursor& c, uint32_t (&w)[4]) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    w[i] = 0x7F7F7F7Fu;   // keys past the sequence: data is zero-filled by TMA, any finite scale does
                    if (c.live && 32 * i < c.keys_left) w[i] = __ldg(reinterpret_cast<const uint32_t*>(c.ptr + i * row_step));
                }
                advance(c);
                advance(c);
            };
            // Q scale bytes -> [row % 32][row / 32][4] (the layout tcgen05.cp 32x128b.warpx4 spreads over the four lane quadrants)
            auto load_q_scales = [&](const Item& it, uint32_t (&w)[4]) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint32_t r = it.row0 + lane + 32 * i;
                    r = min(r, p.S - 1u);   // rows past the sequence reuse the last row's scales (block3.rs:110-113)
                    const size_t off = static_cast<size_t>(it.batch) * p.qs_batch_stride + (static_cast<size_t>(r) * p.H + it.head) * 4u;
                    w[i] = __ldg(reinterpret_cast<const uint32_t*>(p.q_descale + off));
                }
            };
            // The CTA's first copies (Q tile and first K tile, first V tile of its first item) go out before anything else of the role's set-up.
            if (blockIdx.x < n_items && elect_one_sync()) {
                const Item it = decode_item<kSplit, kCausal, kPair>(blockIdx.x, p);
                if (kIsK) {
                    mbar_arrive_expect_tx(bar_q_full(0), kTileBytes);
                    tma_load_4d(q_smem, &tm_q, bar_q_full(0), 0, static_cast<int>(it.head), static_cast<int>(it.row0), static_cast<int>(it.batch));
                    stamp(cta_traced ? p.trace : nullptr, 2, 0, 6);
                    mbar_arrive_expect_tx(bar_k_full(0), kTileBytes);
                    tma_load_4d(k_smem, &tm_k, bar_k_full(0), 0, static_cast<int>(it.kv_head), static_cast<int>(it.key_lo), static_cast<int>(it.batch));
                } else {
                    stamp(cta_traced ? p.trace : nullptr, 3, 0, 6);
                    mbar_arrive_expect_tx(bar_v_full(0), kTileBytes);
                    tma_load_4d(v_smem, &tm_v, bar_v_full(0), 0, static_cast<int>(it.kv_head), static_cast<int>(it.key_lo), static_cast<int>(it.batch));
                }
            }
            ScaleCursor cs;
            cs.w = blockIdx.x;
            enter_item(cs);
            if (kPar) advance(cs);   // this warp's first tile is the CTA's second
            uint32_t wq[4] = {0u, 0u, 0u, 0u}, w0[4], w1[4];
            if (kIsK && blockIdx.x < n_items) load_q_scales(decode_item<kSplit, kCausal, kPair>(blockIdx.x, p), wq);
            load_and_advance(cs, w0);
            load_and_advance(cs, w1);

            uint32_t g = 0, n = 0, ph = 0, q_issued = 0;   // g: the running tile counter
            int st = 0;
            bool ok = true;
            for (uint32_t w = blockIdx.x; ok && w < n_items; w += stride, ++n) {
                const Item it = decode_item<kSplit, kCausal, kPair>(w, p);
                const uint32_t qb = n & 1u;
                if (kIsK) {
                    // the Q buffer was last used two items ago
                    if (n >= 2) ok = mbar_wait(bar_q_empty(qb), ((n >> 1) - 1u) & 1u, abort_flag);
                    if (!__all_sync(0xFFFFFFFFu, ok)) { ok = false; break; }
                    // the tile copy goes out first: it does not depend on the scale bytes, whose global loads may still be in flight
                    if (n > 0 && elect_one_sync()) {
                        mbar_arrive_expect_tx(bar_q_full(qb), kTileBytes);
                        tma_load_4d(q_smem + qb * kTileBytes, &tm_q, bar_q_full(qb), 0, static_cast<int>(it.head), static_cast<int>(it.row0), static_cast<int>(it.batch));
                    }
                    *reinterpret_cast<uint4*>(smem_gen + SmemLayout::sfq + qb * kSfBytes + lane * 16) = make_uint4(wq[0], wq[1], wq[2], wq[3]);
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (elect_one_sync()) mbar_arrive(bar_q_full(qb));
                    ++q_issued;
                    if (w + stride < n_items) load_q_scales(decode_item<kSplit, kCausal, kPair>(w + stride, p), wq);   // the next item's Q scales, a whole item ahead
                }
                float* k_trace = cta_traced ? p.trace : nullptr;   // stamps are indexed by the running tile counter
                int key = static_cast<int>(it.key_lo);
                for (int j = 0; j < it.n_tiles; ++j, key += kKeys) {
                    uint32_t vsc[4] = {0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu};   // key blocks past the sequence: data is zero-filled, any finite scale does
                    if (kVbs && !kIsK) {   // issued first, used after the waits below
                        const uint32_t nblk = (p.SK + 31u) / 32u, blk0 = static_cast<uint32_t>(key) / 32u;
#pragma unroll
                        for (uint32_t kb = 0; kb < 4u; ++kb) {
                            if (blk0 + kb < nblk)
                                vsc[kb] = __ldg(reinterpret_cast<const uint32_t*>(p.v_blockscale + ((static_cast<size_t>(it.batch) * nblk + blk0 + kb) * p.HK + it.kv_head) * 128u) + lane);
                        }
                    }
                    const bool own_scales = (g & 1u) == kPar;
                    // K: the stage (tile and scale bytes) is free once Q K^T of the tile that held it is done
                    if ((kIsK || own_scales) && g >= static_cast<uint32_t>(kStages)) ok = mbar_wait(bar_k_empty(st), ph ^ 1u, abort_flag);
                    if (!__all_sync(0xFFFFFFFFu, ok)) { ok = false; break; }
                    if (kIsK && g > 0 && elect_one_sync()) {
                        stamp(k_trace, 2, static_cast<int>(g), 6);
                        mbar_arrive_expect_tx(bar_k_full(st), kTileBytes);
                        tma_load_4d(k_smem + st * kTileBytes, &tm_k, bar_k_full(st), 0, static_cast<int>(it.kv_head), key, static_cast<int>(it.batch));
                    }
                    if (own_scales) {
                        uint4* sf_dst = reinterpret_cast<uint4*>(smem_gen + SmemLayout::sfk + st * kSfBytes + lane * 16);
                        auto put_and_refill = [&](uint32_t (&set)[4]) {
                            *sf_dst = make_uint4(set[0], set[1], set[2], set[3]);
                            load_and_advance(cs, set);   // for the tile four ahead
                        };
                        if (g & 2u) put_and_refill(w1); else put_and_refill(w0);
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (elect_one_sync()) mbar_arrive(bar_k_full(st));
                    }
                    if (!kIsK) {
                        // V: the stage is free once P V of the tile that held it is done
                        if (g >= static_cast<uint32_t>(kStages)) ok = mbar_wait(bar_v_empty(st), ph ^ 1u, abort_flag);
                        if (!__all_sync(0xFFFFFFFFu, ok)) { ok = false; break; }
                        if (g > 0 && elect_one_sync()) {
                            stamp(k_trace, 3, static_cast<int>(g), 6);
                            mbar_arrive_expect_tx(bar_v_full(st), kTileBytes);
                            tma_load_4d(v_smem + st * kTileBytes, &tm_v, bar_v_full(st), 0, static_cast<int>(it.kv_head), key, static_cast<int>(it.batch));
                        }
                        if (kVbs) {
                            // V block scales (extension): E8M0 [batch][key / 32][kv head][128 columns]. The tile's four key blocks are four rows of
                            // 128 bytes; lane l holds columns 4l .. 4l+3 of each (vsc, loaded at the top of the iteration), transposes them to
                            // one word per column (byte = key block) and writes word n to [n % 32][n / 32], the layout tcgen05.cp spreads
                            // over the lane quadrants.
                            const uint32_t a0 = __byte_perm(vsc[0], vsc[1], 0x5140), a1 = __byte_perm(vsc[0], vsc[1], 0x7362);
                            const uint32_t b0 = __byte_perm(vsc[2], vsc[3], 0x5140), b1 = __byte_perm(vsc[2], vsc[3], 0x7362);
                            const uint32_t t[4] = {__byte_perm(a0, b0, 0x5410), __byte_perm(a0, b0, 0x7632), __byte_perm(a1, b1, 0x5410), __byte_perm(a1, b1, 0x7632)};
                            uint32_t* sfv_dst = reinterpret_cast<uint32_t*>(smem_gen + SmemLayout::sfv + st * kSfBytes);
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const uint32_t n = 4u * static_cast<uint32_t>(lane) + static_cast<uint32_t>(i);
                                sfv_dst[(n & 31u) * 4u + (n >> 5)] = t[i];
                            }
                            fence_proxy_async_smem();
                            __syncwarp();
                            if (elect_one_sync()) mbar_arrive(bar_v_full(st));
                        }
                    }
                    ++g;
                    if (++st == kStages) { st = 0; ph ^= 1u; }
                }
            }
            if (*abort_flag != 0u) {
                // leaving early: let the copies already in flight land before the CTA's shared memory is given back
                for (uint32_t t = g > static_cast<uint32_t>(kStages) ? g - kStages : 0u; t < g; ++t) {
                    const long long t0 = clock64();
                    while (!mbar_test_wait(kIsK ? bar_k_full(t % kStages) : bar_v_full(t % kStages), (t / kStages) & 1u) && clock64() - t0 < kWaitBudgetCycles) {}
                }
                for (uint32_t m = q_issued > 2u ? q_issued - 2u : 0u; m < q_issued; ++m) {
                    const long long t0 = clock64();
                    while (!mbar_test_wait(bar_q_full(m & 1u), (m >> 1) & 1u) && clock64() - t0 < kWaitBudgetCycles) {}
                }
            }
        };
        if (warp == kKProducerWarp) producer(std::true_type{});
        else producer(std::false_type{});
    } else if (warp == kMmaWarp) {
        // =========================================================== MMA issuer: score tiles ===========================================================
        // The whole warp runs the role in step on warp-uniform values and an elected lane issues: written as `if (lane == 0) { ... }` the
        // role spent 400 clocks per tile on issuing four MMAs and 200 on the commits, because every operand of a tcgen05 instruction then
        // has to be moved over from vector registers; now 120 and 45. Q K^T and P V are issued by two different threads (this warp's and
        // kPvWarp's elected lanes): their streams share no operand, the pipe interleaves them, and neither holds the other up.
        {
            const uint32_t idesc_qk = idesc_mxf8_block_scaled(128, 128, 0, 0, 0, 0);
            const uint32_t t_sfq = tmem + kColSfQ;
            // K-major 128-byte-swizzled Q / K tiles: 8-row groups 1024 B apart, 32 head-dim bytes (two 16-byte units) per MMA
            const uint64_t dq0 = make_smem_desc(q_smem, 16, 1024, kSwizzle128B);
            const uint64_t dk0 = make_smem_desc(k_smem, 16, 1024, kSwizzle128B);
            const uint64_t dsf0 = make_smem_desc(sfk_smem, 0, 128, kSwizzleNone);
            const uint64_t dsfq0 = make_smem_desc(sfq_smem, 0, 128, kSwizzleNone);
            uint32_t g = 0, n = 0, ph = 0;
            int st = 0;
            bool ok = true;
            for (uint32_t w = blockIdx.x; ok && w < n_items; w += stride, ++n) {
                const Item qk_it = decode_item<kSplit, kCausal, kPair>(w, p);
                const int n_tiles = qk_it.n_tiles;
                const uint32_t qb = n & 1u;
                float* mma_trace = cta_traced ? p.trace : nullptr;
                // first half of a cut item: once its last score tile is done the K ring is idle for good, and the partner may push its
                // half there (the commit below arrives on the partner's barrier)
                uint32_t partner_rdy = 0u;
                if (kPair && qk_it.half == 1u) {
                    join_cluster();
                    partner_rdy = map_to_cta(bar_peer_rdy, 1u);
                }
                ok = mbar_wait(bar_q_full(qb), (n >> 1) & 1u, abort_flag);
                if (!ok) break;
                tc_fence_after_sync();
                // issued behind the previous item's MMAs by the same thread, so it cannot overtake their reads of these columns
                if (elect_one_sync()) tmem_cp_sf(t_sfq, dsfq0 + static_cast<uint64_t>((qb * kSfBytes) >> 4));
                const uint64_t dq = dq0 + static_cast<uint64_t>((qb * kTileBytes) >> 4);
                for (int j = 0; j < n_tiles; ++j) {
                    // S[g&1] = Q K(j)^T: needs the K tile and its scales, and the softmax of tile g-2 to have read S[g&1] out
                    ok = mbar_wait(bar_k_full(st), ph, abort_flag);
                    if (ok && g >= 2) ok = mbar_wait(bar_s_free(g & 1u), ((g >> 1) - 1u) & 1u, abort_flag);
                    if (!ok) break;
                    tc_fence_after_sync();
                    if (lane == 0) stamp(mma_trace, 2, static_cast<int>(g), 2);
                    const uint32_t t_sfk = tmem + ((g & 1u) ? kColSfK1 : kColSfK0);
                    const uint32_t t_s = tmem + ((g & 1u) ? kColS1 : kColS0);
                    const uint64_t dk = dk0 + static_cast<uint64_t>((st * kTileBytes) >> 4);
                    if (elect_one_sync()) {
                        tmem_cp_sf(t_sfk, dsf0 + static_cast<uint64_t>((st * kSfBytes) >> 4));
#pragma unroll
                        for (int kb = 0; kb < 4; ++kb) {
                            const uint32_t id = idesc_qk | (static_cast<uint32_t>(kb) << 29) | (static_cast<uint32_t>(kb) << 4);
                            mma_mxf8_ss(t_s, dq + 2u * kb, dk + 2u * kb, id, t_sfq + (static_cast<uint32_t>(kb) << 30),
                                        t_sfk + (static_cast<uint32_t>(kb) << 30), kb > 0 ? 1u : 0u);
                        }
                        stamp(mma_trace, 2, static_cast<int>(g), 4);
                        tc_commit(bar_s_full(g & 1u));
                        tc_commit(bar_k_empty(st));
                        if (j == n_tiles - 1) tc_commit(bar_q_empty(qb));   // the Q buffer can take the item after next
                        if (kPair && partner_rdy != 0u && j == n_tiles - 1) tc_commit(partner_rdy);
                        stamp(mma_trace, 2, static_cast<int>(g), 5);
                    }
                    ++g;
                    if (++st == kStages) { st = 0; ph ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else if (warp == kPvWarp) {
        // =========================================================== MMA issuer: P V ===========================================================
        {
            // P V with N = 144: head dims 0..127 from the V tile, 16 more columns from the tile of ones (O | L are adjacent in TMEM)
            const uint32_t idesc_pv = idesc_f8_dense(128, 144, 0, 1);
            // V block scales (extension): the same MMA as kind::mxf8f6f4.block_scale, P's factors a constant 1.0, V's one E8M0 per 32 keys and column
            const uint32_t idesc_pv_bs = idesc_mxf8_block_scaled(128, 144, 0, 1, 0, 0);
            const uint32_t t_sfp = tmem + kColSfP, t_sfv = tmem + kColSfV;
            if (kVbs && elect_one_sync()) {   // the constant factors, once: P's four columns and the ones columns' (rows 128..143 of the B factors)
                const uint64_t d1 = make_smem_desc(smem_base + SmemLayout::sf_one, 0, 128, kSwizzleNone);
                tmem_cp_sf(t_sfp, d1);
                tmem_cp_sf(t_sfv + 4, d1);
            }
            uint32_t g = 0, n = 0, ph = 0;
            int st = 0;
            bool ok = true;
            for (uint32_t w = blockIdx.x; ok && w < n_items; w += stride, ++n) {
                const int n_tiles = decode_item<kSplit, kCausal, kPair>(w, p).n_tiles;
                float* mma_trace = cta_traced ? p.trace : nullptr;
                // an item's first tile overwrites O and L, which the epilogue of the item before must have read out
                if (n > 0) ok = mbar_wait(bar_o_free, (n - 1u) & 1u, abort_flag);
                for (int i = 0; ok && i < n_tiles; ++i) {
                    // O (+)= P(i) V(i) with the row sums riding along: P from TMEM (32 columns, 8 per 32 keys), V tile = 128 keys x 128 B, MN-major
                    ok = mbar_wait(bar_v_full(st), ph, abort_flag);
                    if (ok) ok = mbar_wait(bar_p_full(g & 1u), (g >> 1) & 1u, abort_flag);
                    if (!ok) break;
                    tc_fence_after_sync();
                    if (lane == 0) stamp(mma_trace, 3, static_cast<int>(g), 2);
                    const uint32_t t_p = tmem + ((g & 1u) ? kColP1 : kColP0);
                    if (elect_one_sync()) {
#pragma unroll
                        for (int kb = 0; kb < 4; ++kb) {
                            // MN-major B: 8-key groups 1024 B apart; the second 128-byte-wide atom (columns 128..) is the tile of ones
                            const uint32_t v_addr = v_smem + st * kTileBytes + kb * 4096;
                            const uint64_t dv = make_smem_desc(v_addr, ones_smem - v_addr, 1024, kSwizzle128B);
                            if (kVbs) {
                                if (kb == 0) tmem_cp_sf(t_sfv, make_smem_desc(smem_base + SmemLayout::sfv + st * kSfBytes, 0, 128, kSwizzleNone));
                                const uint32_t id = idesc_pv_bs | (static_cast<uint32_t>(kb) << 29) | (static_cast<uint32_t>(kb) << 4);
                                mma_mxf8_ts(tmem + kColO, t_p + 8 * kb, dv, id, t_sfp + (static_cast<uint32_t>(kb) << 30), t_sfv + (static_cast<uint32_t>(kb) << 30),
                                            (i > 0 || kb > 0) ? 1u : 0u);
                            } else {
                                mma_f8_ts(tmem + kColO, t_p + 8 * kb, dv, idesc_pv, (i > 0 || kb > 0) ? 1u : 0u);
                            }
                        }
                        stamp(mma_trace, 3, static_cast<int>(g), 3);
                        tc_commit(bar_v_empty(st));
                        tc_commit(bar_o_done(g & 1u));
                        if (i == n_tiles - 1) tc_commit(bar_o_full);   // the item's O and L are complete: over to the epilogue warpgroup
                        stamp(mma_trace, 3, static_cast<int>(g), 4);
                    }
                    ++g;
                    if (++st == kStages) { st = 0; ph ^= 1u; }
                }
            }
        }
        __syncwarp();
    }
    } else if (warp < kFirstEpilogueWarp) {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSoftmaxRegs));
        // =========================================================== softmax ===========================================================
        // Two warpgroups: wg = parity = which tiles (counter g = parity mod 2) and which S / P buffer. Thread r of a group owns query row r.
        const uint32_t st_id = threadIdx.x - 32u * kFirstSoftmaxWarp;
        const uint32_t wg = st_id >> 7;
        const uint32_t par = wg;
        const uint32_t r = 32u * (static_cast<uint32_t>(warp) & 3u) + static_cast<uint32_t>(lane);   // TMEM lane = 32 * (warp % 4) + lane
        const uint32_t lane_base = (static_cast<uint32_t>(warp & 3) * 32u) << 16;
        const uint32_t xref = smem_base + SmemLayout::xref;   // 8-byte slots, accessed with single 64-bit shared loads / stores
        const uint32_t t_s = tmem + (par ? kColS1 : kColS0) + lane_base;
        const uint32_t t_p = tmem + (par ? kColP1 : kColP0) + lane_base;
        const uint32_t t_o_part = tmem + kColO + lane_base;
        const uint32_t t_l = tmem + kColL + lane_base;
        bool ok = true;

        // bounded poll of an 8-byte {value, tile counter} slot
        auto wait_slot = [&](uint32_t slot, uint32_t g, float& out) -> bool {
            uint2 o = ld_shared_v2(slot);
            if (o.y != g) {
                const long long t0 = clock64();
                for (uint32_t spins = 1;; ++spins) {
                    o = ld_shared_v2(slot);
                    if (o.y == g) break;
                    if ((spins & 15u) == 0u && (*abort_flag != 0u || clock64() - t0 > kWaitBudgetCycles)) { *abort_flag = 1u; return false; }
                }
            }
            out = __uint_as_float(o.x);
            return true;
        };
        // the reference the row has after tile g, published by the thread that handled it
        auto ref_slot = [&](uint32_t g) { return xref + 8u * ((g & 3u) * 128u + r); };

        const bool want_fin = kSplit || p.lse_nat != nullptr || cta_traced || kPair;   // does anything read the final reference?
        uint32_t g0 = 0, n = 0;   // tile counter at the item's first tile; ordinal of the item
        for (uint32_t w = blockIdx.x; ok && w < n_items; w += stride, ++n) {
            // the tile count, the number of tiles every row sees in full and the row's own key limit stay live through the tile loop
            int n_tiles, j_full, row_lim;   // row_lim: this row's visible keys, counted from the item's first key
            {
                const Item it = decode_item<kSplit, kCausal, kPair>(w, p);
                n_tiles = it.n_tiles;
                row_lim = static_cast<int>(it.key_hi - it.key_lo);
                int first_lim = row_lim;   // the limit of the item's first row: the tiles below it need no mask
                if (kCausal && !kSplit) {
                    first_lim = min(row_lim, static_cast<int>(it.row0 + 1u + (p.SK - p.S)));
                    row_lim = min(row_lim, static_cast<int>(it.row0 + r + 1u + (p.SK - p.S)));
                }
                j_full = first_lim / kKeys;
            }
            const bool tracing = cta_traced && n == 0;
            const bool dumping = tracing && !(p.flags & 0x4u);   // flag 0x4: time stamps only, no tile dumps
            float ref = -INFINITY;   // the row's reference (log2 units) after the last tile this thread has seen

            // The tile body exists twice: the copy in the loop has no code for keys past the range; an item's ragged last tile, if this parity
            // owns it, runs through a second copy placed behind the loop (with all SMs busy, instruction fetch is scarce enough that even
            // never-executed masking code inside the loop costs 3-4 %; moving the rare rescale out of the loop the same way did not pay).
            auto tile = [&](int j, auto masked_c) {
                uint32_t v[128];   // the row's scores, converted in place below
                float f = 1.0f;    // factor of a rescale
                bool pv_seen = false;   // P V of this parity's previous tile is known to be done
                constexpr bool kMasked = decltype(masked_c)::value;
                const uint32_t g = g0 + static_cast<uint32_t>(j);
                const uint32_t k = g >> 1;   // this parity's tile counter
                float* st_trace = (cta_traced && r == 0) ? p.trace : nullptr;
                stamp(st_trace, par, static_cast<int>(g), 0);
                if (!mbar_wait(bar_s_full(par), k & 1u, abort_flag)) ok = false;   // no divergent exit: a failed wait only clears `ok`, the vote after the tile loop ends the role
                tc_fence_after_sync();
                stamp(st_trace, par, static_cast<int>(g), 1);
                // All 128 scores of the row in registers with one tensor-memory round trip; the score buffer is handed back at once, so
                // that Q K^T of tile g + 2 runs under this tile's conversion. The scores are converted in place further down.
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) tmem_ld32(t_s + 32 * ch, *reinterpret_cast<uint32_t(*)[32]>(&v[32 * ch]));
                pv_seen = k == 0 || mbar_test_wait(bar_o_done(par), (k - 1u) & 1u);   // probed under the tensor-memory round trip
                tmem_wait_ld();
                tc_fence_before_sync();
                mbar_arrive(bar_s_free(par));
                if (kMasked) {   // keys past the range: -inf for the maximum, 0 for P (crates/amdgpu-tile/src/reduce.rs:35-49)
                    const int valid = row_lim - j * kKeys;   // may be <= 0 on the causal diagonal: the row then has no key in this tile
#pragma unroll
                    for (int c = 0; c < 128; ++c) {
                        if (c >= valid) v[c] = 0xFF800000u;
                    }
                }
                if (dumping && j == 0) {
#pragma unroll
                    for (int c = 0; c < 128; ++c) p.trace[r * 128 + c] = __uint_as_float(v[c]);
                }
                float m[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) m[i] = -INFINITY;
#pragma unroll
                for (int c = 0; c < 128; c += 16) {   // eight independent chains of three-input maxima
#pragma unroll
                    for (int i = 0; i < 8; ++i) m[i] = max3(m[i], __uint_as_float(v[c + 2 * i]), __uint_as_float(v[c + 2 * i + 1]));
                }
                const float mt = fmaxf(fmaxf(max3(m[0], m[1], m[2]), max3(m[3], m[4], m[5])), fmaxf(m[6], m[7]));
                stamp(st_trace, par, static_cast<int>(g), 2);
                stamp(st_trace, par, static_cast<int>(g), 3);
                // The hand-over of the row's reference from the thread that handled the item's previous tile is the one dependency that runs
                // from tile to tile across the two groups, so everything that does not need the old reference is computed before the slot is
                // read, and the new reference is published before the rescale factor is worked out.
                const float cand = lazy ? ceilf(mt) : mt;   // where the reference goes if it moves
                const float mt_thr = mt - thr;
                if (ok && j > 0 && !wait_slot(ref_slot(g - 1u), g - 1u, ref)) ok = false;
                // the reference moves when this tile's maximum passes it by more than the threshold (negative for short sequences: it then
                // also follows the tile maximum down, and f > 1 scales O and L up)
                const bool move = mt_thr > ref;
                const float old_ref = ref;
                ref = move ? cand : ref;
                st_shared_v2(ref_slot(g), __float_as_uint(ref), g);
                f = move ? ex2_approx(old_ref - ref) : 1.0f;   // 0 on the first tile (old reference -inf); an exact power of two for integer references
                stamp(st_trace, par, static_cast<int>(g), 4);
                // P V of this parity's previous tile must be done before its P columns are overwritten (and, observed in order, this keeps
                // the phase parity of the other parity's barrier below unambiguous)
                if (!pv_seen && k > 0 && !mbar_wait(bar_o_done(par), (k - 1u) & 1u, abort_flag)) ok = false;
                stamp(st_trace, par, static_cast<int>(g), 5);
                // The item's last tile leaves the row's final reference for the epilogue warpgroup's log-sum-exp: before this thread's arrive
                // on p_full (which the last P V, and through it the epilogue's o_full, come after), and behind the wait above: P V of tile
                // g - 2 is done, so P V of g - 3 is, so the epilogue has taken the item four back out (o_free) and read its slot
                if (want_fin && j == n_tiles - 1) *reinterpret_cast<volatile float*>(smem_gen + SmemLayout::xfin + 4u * ((n & 3u) * 128u + r)) = ref;
                if (__builtin_expect(j > 0 && __any_sync(0xFFFFFFFFu, move), 0)) {
                    // O holds P V of all the item's tiles before j once the other parity's last P V is done; P V of tile j cannot start before this thread's arrive below
                    if (!mbar_wait(bar_o_done(par ^ 1u), ((g - 1u) >> 1) & 1u, abort_flag)) ok = false;
                    tc_fence_after_sync();
    #pragma unroll 1
                    for (int c = 0; c < kCols / 32; ++c) scale_tmem32(t_o_part + 32 * c, f);
                    {   // the row sum lives in column 0 of L
                        uint32_t lv;
                        asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(lv) : "r"(t_l) : "memory");
                        tmem_wait_ld();
                        lv = __float_as_uint(__uint_as_float(lv) * f);
                        asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(t_l), "r"(lv) : "memory");
                    }
                    tmem_wait_st();
                }
                // P = e4m3(2^(s - ref + offset)), four keys per 32-bit TMEM column
                const float sh = kPOffset - ref;
                const float cf = (kPOffset + 7.0f - kFastBias - ref) * 0.03125f;
                uint32_t pw[kCols / 4];
                if (lazy) {
                    // Software pipeline over the 32 words, in place in the score registers: word c's exp2 (two values) and bit-built values
                    // (two) are started kConvDepth words before they are converted and packed, so that a thread always has that many
                    // independent chains in flight without holding more than the score row itself (+2 % on the headline shape over one word
                    // at a time; depths 4, 16 and 32 and scheduling points between the words were slower).
                    constexpr int kConvDepth = 8;
#pragma unroll
                    for (int c = 0; c < 32 + kConvDepth; ++c) {
                        if (c < 32) {
                            add2(v[4 * c], v[4 * c + 1], sh);
                            v[4 * c] = __float_as_uint(ex2_approx(__uint_as_float(v[4 * c])));
                            v[4 * c + 1] = __float_as_uint(ex2_approx(__uint_as_float(v[4 * c + 1])));
                            v[4 * c + 2] = fast_p_sat(v[4 * c + 2], cf);
                            v[4 * c + 3] = fast_p_sat(v[4 * c + 3], cf);
                            add2(v[4 * c + 2], v[4 * c + 3], 32768.0f);
                        }
                        if (c >= kConvDepth) {
                            const int d = c - kConvDepth;
                            const uint32_t lo = cvt_e4m3x2(__uint_as_float(v[4 * d]), __uint_as_float(v[4 * d + 1]));
                            const uint32_t hi = __byte_perm(v[4 * d + 2], v[4 * d + 3], 0x0040);
                            pw[d] = __byte_perm(lo, hi, 0x5410);
                        }
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < 32; ++c) pw[c] = p_word(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3], sh);
                }
                if (dumping && j == 0) {
#pragma unroll
                    for (int c = 0; c < kCols / 4; ++c) reinterpret_cast<uint32_t*>(p.trace)[32768 + 256 + r * 32 + c] = pw[c];
                }
                stamp(st_trace, par, static_cast<int>(g), 6);
                tmem_st32(t_p, pw);
                tmem_wait_st();
                tc_fence_before_sync();
                mbar_arrive(bar_p_full(par));
                stamp(st_trace, par, static_cast<int>(g), 7);
            };
            // tiles [0, j_full) have all their keys for every row; behind them come at most two tiles (a ragged end: one; the causal
            // diagonal: up to two), of which this parity owns at most one
            int j = static_cast<int>((g0 ^ par) & 1u);
            for (; j < j_full; j += 2) tile(j, std::false_type{});
            if (j < n_tiles) tile(j, std::true_type{});
            // a failed wait above only clears `ok`; the warp leaves as one
            if (!__all_sync(0xFFFFFFFFu, ok)) { ok = false; break; }
            g0 += static_cast<uint32_t>(n_tiles);
        }
    } else {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kEpilogueRegs));
        // =========================================================== epilogue ===========================================================
        // One warpgroup, thread r = TMEM lane r = query row r of the item. It takes an item's O and L out of tensor memory as soon as the
        // item's last P V is done (o_full) and hands the columns back (o_free) before it normalises and stores, so that the softmax
        // warpgroups go straight on with the next item's tiles and the next item's first P V only waits for the read-out.
        // O * v_descale / l (crates/amdgpu-stage/src/attention/state.rs:79-82) leaves through the two 16 KB staging tiles (128-byte
        // swizzle: 16-byte chunk c of row r sits at chunk c ^ (r % 8)) and TMA stores, which also drop the rows past the sequence
        // (block3.rs:194); a thread owns a row, so direct stores would touch 32 different lines per instruction.
        const uint32_t r = 32u * (static_cast<uint32_t>(warp) & 3u) + static_cast<uint32_t>(lane);
        const uint32_t lane_base = (static_cast<uint32_t>(warp & 3) * 32u) << 16;
        const uint32_t t_o = tmem + kColO + lane_base, t_l = tmem + kColL + lane_base;
        const uint32_t stg = smem_base + SmemLayout::ostage;
        const bool issuer = threadIdx.x == 32u * kFirstEpilogueWarp;
        const bool want_fin = kSplit || p.lse_nat != nullptr || cta_traced || kPair;
        // Half items (the cut last round; a half item is a CTA's last unit, so its K / V rings are idle once its last P V is done): the CTA
        // with the first half tells its partner when its K ring is free (the commit of its last score tile arrives on the partner's
        // barrier); the partner pushes its unnormalised O (f32), row sums and references there with distributed-shared-memory stores and
        // arrives on the first half's barrier; the first half merges and stores. Both references are integers (long-sequence recipe), so the rescale factors
        // are exact powers of two.
        // exchange area = the K ring (64 KB): row r at r * 512 bytes, its 16-byte chunk c at position c ^ (r % 8) within each group of 8
        const uint32_t xch_row = smem_base + SmemLayout::k + r * 512u;
        const uint32_t xch_stat = smem_base + SmemLayout::xstat + r * 8u;
        static_assert(128u * 512u <= kStages * kTileBytes, "the exchange area is the K ring");
        auto xch_off = [&](int c, int q4) { return static_cast<uint32_t>(c) * 128u + ((static_cast<uint32_t>(q4) ^ (r & 7u)) << 4); };
        constexpr uint32_t kEpiBar = 1u;   // named barrier of the 128 epilogue threads
        const float vd = kVbs ? 1.0f : __ldg(p.v_descale);   // with V block scales the factors are in the MMA and there is no scalar descale
        uint32_t n = 0;
        bool ok = true;
        for (uint32_t w = blockIdx.x; w < n_items; w += stride, ++n) {
            const Item it = decode_item<kSplit, kCausal, kPair>(w, p);
            const bool tracing = cta_traced && n == 0;
            const bool dumping = tracing && !(p.flags & 0x4u);
            float* ep_trace = (cta_traced && r == 0 && n < 6) ? p.trace : nullptr;   // epilogue stamps: P V role's row, tile index 24 + item ordinal, slots 0, 1, 5, 7
            stamp(ep_trace, 3, 24 + static_cast<int>(n), 0);
            ok = mbar_wait(bar_o_full, n & 1u, abort_flag);
            if (issuer && n > 0) bulk_wait_group_read0();   // the previous item's stores have read the staging tiles out
            // one barrier: the staging tiles are free, and the decision to go on is the whole warpgroup's (the named barriers below count
            // all 128 threads, so no warp may leave while a sibling goes on)
            if (!named_bar_all(kEpiBar, 128u, ok)) break;
            tc_fence_after_sync();
            stamp(ep_trace, 3, 24 + static_cast<int>(n), 1);
            uint32_t lv;
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(lv) : "r"(t_l) : "memory");
            const float ref_fin = want_fin ? *reinterpret_cast<volatile float*>(smem_gen + SmemLayout::xfin + 4u * ((n & 3u) * 128u + r)) : 0.0f;
            tmem_wait_ld();
            float l = __uint_as_float(lv);
            float ref_out = ref_fin;
            if (kPair && it.half == 2u) {
                // second half: wait for the partner's exchange area, push O, l and the reference, one arrive per thread on its barrier
                join_cluster();
                ok = mbar_wait_cluster(bar_peer_rdy, 0u, abort_flag);
                if (!named_bar_all(kEpiBar, 128u, ok)) break;
                const uint32_t dst_row = map_to_cta(xch_row, 0u);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t o[32];
                    tmem_ld32(t_o + 32 * c, o);
                    tmem_wait_ld();
                    if (c == 3) {
                        tc_fence_before_sync();
                        mbar_arrive(bar_o_free);
                    }
#pragma unroll
                    for (int q4 = 0; q4 < 8; ++q4) {
                        asm volatile("st.shared::cluster.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst_row + xch_off(c, q4)),
                                     "r"(o[4 * q4]), "r"(o[4 * q4 + 1]), "r"(o[4 * q4 + 2]), "r"(o[4 * q4 + 3]) : "memory");
                    }
                }
                asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(map_to_cta(xch_stat, 0u)), "f"(l), "f"(ref_fin) : "memory");
                mbar_arrive_remote(map_to_cta(bar_peer_data, 0u));
                continue;
            }
            float fa = 1.0f, fb = 0.0f;   // weights of the own and of the partner's half in a merge
            if (kPair && it.half == 1u) {
                join_cluster();
                ok = mbar_wait_cluster(bar_peer_data, 0u, abort_flag);
                if (!named_bar_all(kEpiBar, 128u, ok)) break;
                float2 ps;   // {l, reference} of the partner's half
                asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(ps.x), "=f"(ps.y) : "r"(xch_stat) : "memory");
                ref_out = fmaxf(ref_fin, ps.y);
                fa = ex2_approx(ref_fin - ref_out);
                fb = ex2_approx(ps.y - ref_out);
                l = l * fa + ps.x * fb;
            }
            const float fin = vd / l;
            const uint32_t row = it.row0 + r;
            if (tracing) {
                p.trace[32768 + r] = l;
                p.trace[32768 + 128 + r] = ref_out;
            }
            const bool half_out = !kSplit || kFused || (p.flags & kFlagF32Partials) == 0u;   // 16-bit rows (bf16 output, f16 partial) or f32 partial rows
            if (half_out) {
                // bf16 output, or the split kernel's f16 partial (the reference's partial format, block3.rs:291-356): four 32-column
                // chunks, all staged before the stores go out; O is free after the last read
                // Two chunks are in flight at a time: the read-out of O, which the next item's first P V waits for (o_free), then takes two
                // tensor-memory round trips and the conversion of two chunks instead of four and three (this warpgroup only gets an
                // instruction issued every few dozen clocks while the softmax warps of its scheduler run, so what stands between o_full
                // and o_free is counted in instructions)
                auto process = [&](int c, uint32_t (&o)[32]) {
                    if (dumping) {
#pragma unroll
                        for (int e = 0; e < 32; ++e) p.trace[16384 + r * 128 + 32 * c + e] = __uint_as_float(o[e]);
                    }
                    if (kPair && it.half == 1u) {
#pragma unroll
                        for (int q4 = 0; q4 < 8; ++q4) {
                            float4 pb;
                            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(pb.x), "=f"(pb.y), "=f"(pb.z), "=f"(pb.w)
                                         : "r"(xch_row + xch_off(c, q4)) : "memory");
                            o[4 * q4] = __float_as_uint(__uint_as_float(o[4 * q4]) * fa + pb.x * fb);
                            o[4 * q4 + 1] = __float_as_uint(__uint_as_float(o[4 * q4 + 1]) * fa + pb.y * fb);
                            o[4 * q4 + 2] = __float_as_uint(__uint_as_float(o[4 * q4 + 2]) * fa + pb.z * fb);
                            o[4 * q4 + 3] = __float_as_uint(__uint_as_float(o[4 * q4 + 3]) * fa + pb.w * fb);
                        }
                    }
                    const uint32_t tile_base = stg + (static_cast<uint32_t>(c) >> 1) * 16384u + r * 128u;
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {   // 8 columns = 16 bytes of bf16 per store
                        uint32_t wv[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            mul2(o[8 * q4 + 2 * e], o[8 * q4 + 2 * e + 1], fin);
                            const float a = __uint_as_float(o[8 * q4 + 2 * e]), b = __uint_as_float(o[8 * q4 + 2 * e + 1]);
                            if (kSplit) {
                                asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(wv[e]) : "f"(b), "f"(a));
                            } else {
                                const __nv_bfloat162 b2 = __floats2bfloat162_rn(a, b);
                                wv[e] = *reinterpret_cast<const uint32_t*>(&b2);
                            }
                        }
                        const uint32_t chunk = static_cast<uint32_t>((c & 1) * 4 + q4);
                        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(tile_base + ((chunk ^ (r & 7u)) << 4)),
                                     "r"(wv[0]), "r"(wv[1]), "r"(wv[2]), "r"(wv[3]) : "memory");
                    }
                };
                uint32_t oa[32], ob[32];
                tmem_ld32(t_o, oa);
                tmem_ld32(t_o + 32, ob);
                tmem_wait_ld();
                process(0, oa);
                tmem_ld32(t_o + 64, oa);
                process(1, ob);
                tmem_ld32(t_o + 96, ob);
                tmem_wait_ld();
                tc_fence_before_sync();
                mbar_arrive(bar_o_free);   // O and L are out: the next item's first P V may overwrite them
                stamp(ep_trace, 3, 24 + static_cast<int>(n), 5);
                process(2, oa);
                process(3, ob);
                fence_proxy_async_smem();
                named_bar_sync(kEpiBar, 128u);
                if (issuer) {
                    if (kSplit) {
                        // with a routing plan the rows go to the GPU that combines them (its receive slot of this GPU), else to this launch's own partial buffer
                        const CUtensorMap* omap = &tm_o;
                        int o_row = static_cast<int>(it.row0), o_split = static_cast<int>(it.split);
                        if (!kFused && p.peer != nullptr) {
                            const uint32_t dest = it.row0 / p.peer->dest_rows;
                            omap = &p.peer->maps[dest];
                            o_row = static_cast<int>(it.row0 - dest * p.peer->dest_rows);
                            o_split = static_cast<int>(p.peer->rank);
                        }
                        tma_store_5d(omap, stg, 0, static_cast<int>(it.head), o_row, static_cast<int>(it.batch), o_split);
                        tma_store_5d(omap, stg + 16384u, 64, static_cast<int>(it.head), o_row, static_cast<int>(it.batch), o_split);
                    } else {
                        tma_store_4d(&tm_o, stg, 0, static_cast<int>(it.head), static_cast<int>(it.row0), static_cast<int>(it.batch));
                        tma_store_4d(&tm_o, stg + 16384u, 64, static_cast<int>(it.head), static_cast<int>(it.row0), static_cast<int>(it.batch));
                    }
                    bulk_commit_group();
                }
            } else {
                // f32 partial: four pieces of 32 columns (128 bytes per row), alternating between the two staging tiles; a tile is written
                // again once the store that last used it has read it out. With a routing plan the rows go to the GPU that combines them
                // (its receive slot of this GPU), else to this launch's own partial buffer.
                const CUtensorMap* omap = &tm_o;
                int o_row = static_cast<int>(it.row0), o_split = static_cast<int>(it.split);
                if (kSplit && p.peer != nullptr) {
                    const uint32_t dest = it.row0 / p.peer->dest_rows;
                    omap = &p.peer->maps[dest];
                    o_row = static_cast<int>(it.row0 - dest * p.peer->dest_rows);
                    o_split = static_cast<int>(p.peer->rank);
                }
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t o[32];
                    tmem_ld32(t_o + 32 * c, o);
                    tmem_wait_ld();
                    if (c == 3) {
                        tc_fence_before_sync();
                        mbar_arrive(bar_o_free);
                        stamp(ep_trace, 3, 24 + static_cast<int>(n), 5);
                    }
                    if (kPair && it.half == 1u) {
#pragma unroll
                        for (int q4 = 0; q4 < 8; ++q4) {
                            float4 pb;
                            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(pb.x), "=f"(pb.y), "=f"(pb.z), "=f"(pb.w)
                                         : "r"(xch_row + xch_off(c, q4)) : "memory");
                            o[4 * q4] = __float_as_uint(__uint_as_float(o[4 * q4]) * fa + pb.x * fb);
                            o[4 * q4 + 1] = __float_as_uint(__uint_as_float(o[4 * q4 + 1]) * fa + pb.y * fb);
                            o[4 * q4 + 2] = __float_as_uint(__uint_as_float(o[4 * q4 + 2]) * fa + pb.z * fb);
                            o[4 * q4 + 3] = __float_as_uint(__uint_as_float(o[4 * q4 + 3]) * fa + pb.w * fb);
                        }
                    }
                    if (c >= 2) {   // the store of piece c - 2 (all but the newest group) must have read its tile out
                        if (issuer) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                        named_bar_sync(kEpiBar, 128u);
                    }
                    const uint32_t tile_base = stg + static_cast<uint32_t>(c & 1) * 16384u + r * 128u;
#pragma unroll
                    for (int q4 = 0; q4 < 8; ++q4) {
                        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(tile_base + ((static_cast<uint32_t>(q4) ^ (r & 7u)) << 4)),
                                     "f"(__uint_as_float(o[4 * q4]) * fin), "f"(__uint_as_float(o[4 * q4 + 1]) * fin),
                                     "f"(__uint_as_float(o[4 * q4 + 2]) * fin), "f"(__uint_as_float(o[4 * q4 + 3]) * fin) : "memory");
                    }
                    fence_proxy_async_smem();
                    named_bar_sync(kEpiBar, 128u);
                    if (issuer) {
                        tma_store_5d(omap, stg + static_cast<uint32_t>(c & 1) * 16384u, 32 * c, static_cast<int>(it.head), o_row, static_cast<int>(it.batch), o_split);
                        bulk_commit_group();
                    }
                }
            }
            if (row < p.S && want_fin) {   // rows past the sequence are computed on clamped scales and not stored (block3.rs:194)
                const float lse2 = ref_out - kPOffset + lg2_approx(l);   // log2 of sum_j 2^(s_j)
                if (kSplit && !kFused && p.peer != nullptr) {
                    const uint32_t dest = it.row0 / p.peer->dest_rows, n_rows = p.peer->dest_rows * p.H;
                    p.peer->lse[dest][static_cast<size_t>(p.peer->rank) * n_rows + static_cast<size_t>(row - dest * p.peer->dest_rows) * p.H + it.head] = lse2;
                } else if (kSplit) {
                    const size_t prow = static_cast<size_t>(it.split) * p.rows_total + (static_cast<size_t>(it.batch) * p.S + row) * p.H + it.head;
                    p.lse2[prow] = lse2;
                } else if (p.lse_nat != nullptr) {
                    p.lse_nat[(static_cast<size_t>(it.batch) * p.H + it.head) * p.S + row] = lse2 * 0.6931471805599453f;
                }
            }
            if (kFused) {
                // Fused merge (the reference's last-arriver combine, tests/gpu/ref_host.cpp:489-497, docs/last-arriver-memory-model.md): every
                // CTA that has stored a partial of this 128-row block counts itself in; the one that completes the count merges the block's
                // `splits` partials into the bf16 output, so no combine kernel follows.
                // Writer side: the bulk stores of the partial are performed, every thread's log-sum-exp store is fenced, then one
                // device-scope atomic publishes both. Reader side: the atomic, a fence, copies and loads that bypass L1.
                volatile uint32_t* last_flag = reinterpret_cast<volatile uint32_t*>(smem_gen + SmemLayout::last_flag);
                if (issuer) bulk_wait_group_done0();
                __threadfence();
                named_bar_sync(kEpiBar, 128u);
                if (issuer) {
                    uint32_t* cnt = p.fused_counters + (static_cast<size_t>(it.batch) * p.H + it.head) * p.n_qtiles + it.row0 / kRows;
                    __threadfence();
                    const uint32_t old = atomicAdd(cnt, 1u);
                    const bool last = old + 1u == p.splits;
                    if (last) *cnt = 0u;   // nobody else touches the counter any more in this launch: the next launch finds it zero
                    *last_flag = last ? 1u : 0u;
                }
                named_bar_sync(kEpiBar, 128u);
                if (*last_flag != 0u) {
                    __threadfence();
                    // The block's partial rows (256 bytes each, `splits` per output row) come in through the two staging tiles with
                    // asynchronous 16-byte copies (cp.async: no registers are tied up by loads in flight, which this warpgroup does not
                    // have), 64 rows of 256 bytes per batch (= 64 / splits output rows), two batches in flight. Piece i of a batch = the
                    // partial of split i % splits for output row i / splits, at byte 256 i of the tile; a warp's copy instruction moves two
                    // whole pieces. For the merge a warp shares an output row, 4 columns per lane.
                    const uint32_t rows_pb = 64u >> p.split_log2;
                    const uint32_t rows_valid = min(static_cast<uint32_t>(kRows), p.S - it.row0);
                    const uint32_t n_batches = (rows_valid + rows_pb - 1u) / rows_pb;
                    const size_t head_row0 = (static_cast<size_t>(it.batch) * p.S + it.row0) * p.H + it.head;   // partial row index of the block's first row
                    const uint8_t* part = static_cast<const uint8_t*>(p.ohat);
                    const uint32_t et = threadIdx.x - 32u * kFirstEpilogueWarp;   // 0 .. 127
                    auto issue = [&](uint32_t b) {   // always closes one copy group, also an empty one: two groups are in flight at any time
                        if (b < n_batches) {
                            const uint32_t first = b * rows_pb, pieces = min(rows_pb, rows_valid - first) << p.split_log2;
                            const uint32_t dst = stg + (b & 1u) * 16384u;
#pragma unroll
                            for (uint32_t i = 0; i < 8u; ++i) {
                                const uint32_t c = i * 128u + et, pc = c >> 4, ch = c & 15u;
                                if (pc < pieces) {
                                    const uint32_t row = first + (pc >> p.split_log2), sp = pc & (p.splits - 1u);
                                    const uint8_t* src = part + (static_cast<size_t>(sp) * p.rows_total + head_row0 + static_cast<size_t>(row) * p.H) * 256u + ch * 16u;
                                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + c * 16u), "l"(src) : "memory");
                                }
                            }
                        }
                        asm volatile("cp.async.commit_group;" ::: "memory");
                    };
                    issue(0u);
                    issue(1u);
                    // while the first batches fly: the block's log-sum-exps, thread r those of row r (all loads in flight at once), to shared memory
                    {
                        float lsv[8];
                        const size_t g = head_row0 + static_cast<size_t>(min(r, rows_valid - 1u)) * p.H;
#pragma unroll
                        for (uint32_t sp = 0; sp < 8u; ++sp) lsv[sp] = sp < p.splits ? __ldcg(p.lse2 + static_cast<size_t>(sp) * p.rows_total + g) : 0.0f;
                        float4* dst4 = reinterpret_cast<float4*>(smem_gen + SmemLayout::xlse + r * 32u);
                        dst4[0] = make_float4(lsv[0], lsv[1], lsv[2], lsv[3]);
                        dst4[1] = make_float4(lsv[4], lsv[5], lsv[6], lsv[7]);
                    }
                    const uint32_t tr = static_cast<uint32_t>(warp) & 3u, tc = static_cast<uint32_t>(lane);   // row within a group of 4, 8-byte column chunk
                    for (uint32_t b = 0; b < n_batches; ++b) {
                        const uint32_t first = b * rows_pb, rows_here = min(rows_pb, rows_valid - first);
                        asm volatile("cp.async.wait_group 1;" ::: "memory");   // this thread's copies of batch b have landed
                        named_bar_sync(kEpiBar, 128u);                          // everybody's have (and, the first time, the log-sum-exps are in place)
                        for (uint32_t rg = 0; rg < rows_here; rg += 4u) {
                            const uint32_t rb = rg + tr;   // row within the batch
                            if (rb < rows_here) {
                                const volatile float* ls_row = reinterpret_cast<const volatile float*>(smem_gen + SmemLayout::xlse + (first + rb) * 32u);
                                float m = -1.0e30f, den = 0.0f, acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                                const uint32_t src = stg + (b & 1u) * 16384u + ((rb << p.split_log2) << 8) + tc * 8u;
                                for (uint32_t sp = 0; sp < p.splits; ++sp) {
                                    const float ls = ls_row[sp];
                                    uint2 raw;
                                    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(raw.x), "=r"(raw.y) : "r"(src + sp * 256u) : "memory");
                                    float a, w;
                                    combine_weights(m, den, ls, a, w);
                                    const float2 f01 = combine_h2_to_f2(raw.x), f23 = combine_h2_to_f2(raw.y);
                                    acc[0] = combine_accumulate(acc[0], a, w, f01.x);
                                    acc[1] = combine_accumulate(acc[1], a, w, f01.y);
                                    acc[2] = combine_accumulate(acc[2], a, w, f23.x);
                                    acc[3] = combine_accumulate(acc[3], a, w, f23.y);
                                }
                                const float rd = 1.0f / den;
                                const __nv_bfloat162 b01 = __floats2bfloat162_rn(__fmul_rn(acc[0], rd), __fmul_rn(acc[1], rd));
                                const __nv_bfloat162 b23 = __floats2bfloat162_rn(__fmul_rn(acc[2], rd), __fmul_rn(acc[3], rd));
                                uint8_t* dst = p.o + static_cast<size_t>(it.batch) * p.o_batch_stride + static_cast<size_t>(it.row0 + first + rb) * p.o_row_stride +
                                               static_cast<size_t>(it.head) * 256u + tc * 8u;
                                *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<const uint32_t*>(&b01), *reinterpret_cast<const uint32_t*>(&b23));
                            }
                        }
                        named_bar_sync(kEpiBar, 128u);   // everybody has read this tile out
                        issue(b + 2u);
                    }
                    asm volatile("cp.async.wait_group 0;" ::: "memory");   // (only empty groups are left)
                }
            }
            stamp(ep_trace, 3, 24 + static_cast<int>(n), 7);
        }
        if (issuer) bulk_wait_group_read0();   // the staging tiles have been read out before the CTA gives its shared memory back
    }

    // ---- teardown ----
    tc_fence_before_sync();
    __syncthreads();
    // a pair stays together to the end: the partner may still be reading this CTA's exchange area or arriving on its barrier
    if (paired) {
        join_cluster();
        asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
    }
    if (threadIdx.x == 0) stamp(cta_traced ? p.trace : nullptr, 2, 30, 1);   // all roles done
    if (threadIdx.x == 0 && *abort_flag != 0u) atomicOr(p.status, 1u);
    if (warp == kMmaWarp) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, kTmemCols);
    }
}

cudaError_t launch_attention(const CUtensorMap& tm_q, const CUtensorMap& tm_k, const CUtensorMap& tm_v, const CUtensorMap& tm_o, const AttnParams& p,
                             uint32_t B, bool split, uint32_t rows_per_cta, cudaStream_t stream) {
    (void)rows_per_cta;   // both logical block heights run as 128-row CTAs
    using Kernel = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap, const AttnParams);
    // The instantiations: [causal][recipe][trace][split] (the causal mask has no split form); behind them the variants for launches as pairs
    // of CTAs (long-sequence recipe, no mask): [trace][split]; behind those the variants with V block scales (no mask, no trace):
    // [pair][recipe][split], pairs only with the long-sequence recipe; last the split kernels with the fused merge: [V block scales][recipe].
#define MXA_K(split, trace, lazy, causal, pair, vbs) mxfp8_prefill_kernel<split, trace, lazy, causal, pair, vbs>
    static const Kernel kernels[32] = {
        MXA_K(false, false, false, false, false, false), MXA_K(true, false, false, false, false, false), MXA_K(false, true, false, false, false, false),
        MXA_K(true, true, false, false, false, false),   MXA_K(false, false, true, false, false, false), MXA_K(true, false, true, false, false, false),
        MXA_K(false, true, true, false, false, false),   MXA_K(true, true, true, false, false, false),   MXA_K(false, false, false, true, false, false),
        nullptr,                                         MXA_K(false, true, false, true, false, false),  nullptr,
        MXA_K(false, false, true, true, false, false),   nullptr,                                        MXA_K(false, true, true, true, false, false),
        nullptr,
        MXA_K(false, false, true, false, true, false),   MXA_K(true, false, true, false, true, false),   MXA_K(false, true, true, false, true, false),
        MXA_K(true, true, true, false, true, false),
        MXA_K(false, false, false, false, false, true),  MXA_K(true, false, false, false, false, true),  MXA_K(false, false, true, false, false, true),
        MXA_K(true, false, true, false, false, true),    nullptr,                                        nullptr,
        MXA_K(false, false, true, false, true, true),    MXA_K(true, false, true, false, true, true),
        mxfp8_prefill_kernel<true, false, false, false, false, false, true>, mxfp8_prefill_kernel<true, false, true, false, false, false, true>,
        mxfp8_prefill_kernel<true, false, false, false, false, true, true>,  mxfp8_prefill_kernel<true, false, true, false, false, true, true>};
#undef MXA_K
    constexpr int kKernels = 32;
    constexpr int kMaxDevices = 64;
    // per-device set-up done lazily from whichever thread launches first: plain flags would be a data race, and both steps are idempotent
    static std::atomic<bool> attr_done[kMaxDevices][kKernels];   // the shared-memory attribute is per device
    static std::atomic<int> sm_count[kMaxDevices];
    static std::atomic<int> pair_capacity[kMaxDevices][kKernels];   // -1 = not asked yet (set below on first use)
    static std::once_flag pair_init;
    std::call_once(pair_init, [] {
        for (auto& d : pair_capacity) for (auto& x : d) x.store(-1, std::memory_order_relaxed);
    });
    // the long-sequence recipe from 4 key tiles of the whole sequence on (crates/amdgpu-stage/src/attention/state.rs:73-77), unless the
    // caller asks for the exact one; each recipe is its own instantiation, which halves the code of the tile loop
    const bool lazy_recipe = (p.SK + kKeys - 1) / kKeys >= 4 && !(p.flags & 0x2u);
    const bool causal = (p.flags & kFlagCausal) != 0u;
    if (causal && split) return cudaErrorInvalidValue;
    const bool vbs = p.v_blockscale != nullptr;
    if (vbs && (causal || p.trace != nullptr)) return cudaErrorInvalidValue;   // V block scales: no mask, no diagnostics
    int which = vbs ? 20 + (split ? 1 : 0) + (lazy_recipe ? 2 : 0) : (split ? 1 : 0) + (p.trace != nullptr ? 2 : 0) + (lazy_recipe ? 4 : 0) + (causal ? 8 : 0);
    const bool fused = p.fused_counters != nullptr;
    if (fused && (!split || p.trace != nullptr || p.peer != nullptr || (p.flags & kFlagF32Partials) || p.splits > 8u || p.o == nullptr)) return cudaErrorInvalidValue;
    if (fused) which = 28 + (lazy_recipe ? 1 : 0) + (vbs ? 2 : 0);
    const int which_pair = vbs ? 26 + (split ? 1 : 0) : 16 + (split ? 1 : 0) + (p.trace != nullptr ? 2 : 0);   // only for the long-sequence recipe without a mask
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    auto ensure_attr = [&](int k) -> cudaError_t {
        if (attr_done[dev][k].load(std::memory_order_acquire)) return cudaSuccess;
        const cudaError_t ea = cudaFuncSetAttribute(reinterpret_cast<const void*>(kernels[k]), cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (ea == cudaSuccess) attr_done[dev][k].store(true, std::memory_order_release);
        return ea;
    };
    e = ensure_attr(which);
    if (e != cudaSuccess) return e;
    int sms = sm_count[dev].load(std::memory_order_relaxed);
    if (sms == 0) {
        int n = 0;
        e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return e;
        sms = n > 0 ? n : 1;
        sm_count[dev].store(sms, std::memory_order_relaxed);
    }
    // Persistent launch: one CTA per SM (a CTA takes all of an SM's tensor memory and nearly all of its shared memory), each walking the
    // work units blockIdx.x, blockIdx.x + gridDim.x, ...
    AttnParams q = p;
    q.n_qtiles = (p.S + kRows - 1) / kRows;
    const unsigned long long items = 1ull * q.n_qtiles * p.H * B * (split ? p.splits : 1u);
    if (items == 0 || items > 0x7FFFFFFFull) return cudaErrorInvalidValue;
    q.n_items = static_cast<uint32_t>(items);
    q.n_work = q.n_items;
    q.tail_base = q.n_items;
    q.tail_split = 0u;
    uint32_t ctas = q.n_items < static_cast<uint32_t>(sms) ? q.n_items : static_cast<uint32_t>(sms);
    // The last round. n_items = rounds * grid + tail: when the tail fills at most half of the grid, its items would keep a few CTAs busy
    // for a whole item while the rest idle. They are then cut in two key ranges each, the grid is launched as clusters of two CTAs, and
    // each pair merges its two halves through distributed shared memory (no workspace). Long-sequence recipe only (integer references
    // merge exactly), no causal mask (its items differ in length and are balanced by their order), and only for items of at least
    // kMinTilesForPairs key tiles: a launch as pairs and the merge cost about 7-9 us (measured), which half an item has to outweigh.
    const uint32_t ntiles_total = (p.SK + kKeys - 1) / kKeys;
    uint32_t min_tiles = ntiles_total;
    if (split) {
        const uint32_t tps = (ntiles_total + p.splits - 1) / p.splits;
        min_tiles = ntiles_total - (p.splits - 1u) * tps;   // the last split's share
    }
    const uint32_t even_sms = static_cast<uint32_t>(sms) & ~1u;
    constexpr uint32_t kMinTilesForPairs = 48u;
    if (lazy_recipe && !causal && !fused && min_tiles >= kMinTilesForPairs && even_sms >= 2u && !(p.flags & kFlagNoTailSplit)) {
        const uint32_t rounds = q.n_items / even_sms, tail = q.n_items - rounds * even_sms;
        if (tail > 0u && 2u * tail <= even_sms) {
            const uint32_t grid = rounds > 0u ? even_sms : 2u * tail;
            e = ensure_attr(which_pair);
            if (e != cudaSuccess) return e;
            int max_clusters = pair_capacity[dev][which_pair].load(std::memory_order_relaxed);
            if (max_clusters < 0) {   // how many pairs of CTAs of this kernel the device holds at once (asked once per device and kernel)
                cudaLaunchConfig_t probe = {};
                probe.gridDim = dim3(even_sms, 1, 1);
                probe.blockDim = dim3(kThreads, 1, 1);
                probe.dynamicSmemBytes = kSmemBytes;
                cudaLaunchAttribute pa[1];
                pa[0].id = cudaLaunchAttributeClusterDimension;
                pa[0].val.clusterDim.x = 2; pa[0].val.clusterDim.y = 1; pa[0].val.clusterDim.z = 1;
                probe.attrs = pa;
                probe.numAttrs = 1;
                int n = 0;
                if (cudaOccupancyMaxActiveClusters(&n, reinterpret_cast<const void*>(kernels[which_pair]), &probe) != cudaSuccess) { n = 0; (void)cudaGetLastError(); }
                max_clusters = n;
                pair_capacity[dev][which_pair].store(n, std::memory_order_relaxed);
            }
            if (static_cast<uint32_t>(max_clusters) * 2u >= grid) {
                q.tail_split = 1u;
                q.tail_base = rounds * even_sms;
                q.n_work = q.tail_base + 2u * tail;
                ctas = grid;
                which = which_pair;
            }
        }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // overlap this grid's launch and set-up with the tail of the grid before it
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (q.tail_split != 0u) {
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = 2; attr[1].val.clusterDim.y = 1; attr[1].val.clusterDim.z = 1;
        cfg.numAttrs = 2;
    }
    return cudaLaunchKernelEx(&cfg, kernels[which], tm_q, tm_k, tm_v, tm_o, q);
}

}  // namespace b200mx
