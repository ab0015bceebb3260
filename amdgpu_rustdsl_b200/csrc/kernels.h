// Internal interface between the C-ABI host layer (host_api.cu) and the kernel translation units.
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace b200mx {

// Keys per K / V tile of the attention kernel = rows of the K and V tensor maps' boxes.
constexpr int kKeysPerTile = 128;

constexpr int kMaxPeerGpus = 8;

// Device-resident routing plan of a key-range-sharded launch (peer_exchange.cu): where the rows of this GPU's f32 partial go.
// Destination d combines the query rows [d * dest_rows, (d + 1) * dest_rows); its receive buffer is f32 [source GPU][dest_rows][H][128]
// (maps[d]: the same 5-D map as a local partial, source GPU in the place of the split) and f32 [source GPU][dest_rows * H] (lse[d]).
struct alignas(128) PeerPlan {
    CUtensorMap maps[kMaxPeerGpus];
    float* lse[kMaxPeerGpus];
    uint32_t world, rank, dest_rows, pad;
};

// bf16 output buffers of the GPUs a combine stores its rows to (already advanced to the rows' offset)
struct OutPointers {
    uint8_t* out[kMaxPeerGpus];
    uint32_t n;
};

// Everything one attention launch needs, already decoded from the packed kernel arguments.
struct AttnParams {
    // outputs
    uint8_t* o;            // bf16 [B,S,H,128] (unsplit)
    void* ohat;            // f16 [splits][rows_total][128], or f32 with FMHA_MXFP8_FLAG_F32_PARTIALS (split)
    float* lse2;           // f32 [splits][rows_total], base-2 (split)
    float* lse_nat;        // optional f32 [B,H,S], natural log (unsplit), may be null
    // scale inputs
    const uint8_t* q_descale;   // E8M0 [B,S,H,4]
    const uint8_t* k_descale;   // E8M0 [B,SK,HK,4]
    const float* v_descale;     // one f32
    const uint8_t* v_blockscale;  // extension: E8M0 [B,ceil(SK/32),HK,128], may be null
    uint32_t* fused_counters;     // extension (split kernel, f16 partials): one arrival counter per 128-row block, zero at launch and at exit; the
                                  // CTA that brings a block's count to `splits` merges the block's partials into `o`. Null: the combine is a kernel of its own
    const PeerPlan* peer;         // extension (split kernel, B = 1): store the partial rows to the GPUs that combine them (the plan's maps must be of the launch's partial format); may be null
    // shape
    uint32_t S, SK, H, HK, gqa_shift;
    uint32_t o_row_stride, o_batch_stride;    // bytes
    uint32_t qs_batch_stride, ks_batch_stride;  // bytes
    uint32_t splits, split_log2, rows_total;
    uint32_t flags;
    // work decomposition of the persistent kernel, filled in by launch_attention: n_items work items (128 query rows of one (batch, head
    // [, split])); the CTAs walk work units 0 .. n_work-1. Units below tail_base are whole items. With tail_split the items of the last,
    // partly filled round are cut in two key ranges each: unit tail_base + 2 i + h is half h of item tail_base + i, and the two CTAs of a
    // cluster take the two halves of one item and merge them through distributed shared memory
    uint32_t n_qtiles, n_items, n_work, tail_base, tail_split;
    // diagnostics
    float* trace;          // may be null
    uint32_t* status;      // device status word
};

// rows_per_cta is 128 (t128) or 256 (vs128 / kvsplit): the logical block height of the reference's grids.
// tm_o: the target of the kernel's TMA stores: the bf16 output as a 4-D map with a 128-row x 64-column box (unsplit kernels), or the
// partials as a 5-D map (split kernel): f16 with a 128-row x 64-column box, or f32 with a 128-row x 32-column box
cudaError_t launch_attention(const CUtensorMap& tm_q, const CUtensorMap& tm_k, const CUtensorMap& tm_v, const CUtensorMap& tm_o, const AttnParams& p,
                             uint32_t B, bool split, uint32_t rows_per_cta, cudaStream_t stream);

#ifdef __CUDACC__
// The merge of the split partials, one split at a time, shared by the combine kernel and by the split kernel's fused merge so that both
// give the same bits (crates/amdgpu-tile/src/epilogue.rs:117-146): m' = max(m, lse); a = 2^(m - m'); w = 2^(lse - m');
// den = den a + w; acc = acc a + w v. The products and sums are spelled out so that no two call sites contract them differently.
__device__ __forceinline__ void combine_weights(float& m, float& den, float lse, float& a, float& w) {
    const float mn = fmaxf(m, lse);
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(a) : "f"(m - mn));
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(w) : "f"(lse - mn));
    den = __fmaf_rn(den, a, w);
    m = mn;
}
__device__ __forceinline__ float combine_accumulate(float acc, float a, float w, float v) { return __fmaf_rn(acc, a, __fmul_rn(w, v)); }
__device__ __forceinline__ float2 combine_h2_to_f2(uint32_t h2) {
    float2 f;
    asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\tcvt.f32.f16 %0, lo;\n\tcvt.f32.f16 %1, hi;\n\t}" : "=f"(f.x), "=f"(f.y) : "r"(h2));
    return f;
}
#endif

cudaError_t launch_combine_scatter(const void* ohat, bool f32_partials, const float* lse2, const OutPointers& outs, uint32_t rows, uint32_t splits, cudaStream_t stream);
cudaError_t launch_combine(const void* ohat, bool f32_partials, const float* lse2, uint8_t* out, uint32_t rows_total, uint32_t splits, cudaStream_t stream);

// Quantisers in front of the path (quantize.cu): bf16 -> e4m3 + E8M0 per 32 head-dim elements (Q with `mul` folded in, K), bf16 -> e4m3 +
// one f32 descale (V; `descale` needs 8 bytes: [0] the result, [1] scratch).
cudaError_t launch_quantize_qk(const void* x_bf16, unsigned long long rows, float mul, void* out_e4m3, void* out_scales, cudaStream_t stream);
cudaError_t launch_quantize_v(const void* x_bf16, unsigned long long n_elems, void* out_e4m3, float* descale, cudaStream_t stream);

cudaError_t launch_mma_issue_ceiling(int iters, int ctas, uint32_t* status, cudaStream_t stream);

// wait_selftest.cu: one CTA lets a bounded wait run out (budget in SM cycles) and reports what happened in *word; *ms = kernel time.
cudaError_t run_bounded_wait_selftest(long long budget_cycles, cudaStream_t stream, uint32_t* word, float* ms);

uint32_t* device_status_word();   // address of the per-device status word (device pointer)

}  // namespace b200mx
