// fmha_fwd_hd128_mxfp8_v3_kvsplit_combine8h: merges the per-split partials of the KV-split attention into bf16 O.
//
// Reference: crates/amdgpu-kernels/src/fmha/io.rs:164-185 (kernel), crates/amdgpu-tile/src/epilogue.rs:89-167 (combine_splits).
// Each thread owns 8 or 16 consecutive output elements of one row and walks the splits once with an online maximum:
//   m' = max(m, lse_s); a = 2^(m - m'); w = 2^(lse_s - m'); den = den*a + w; acc_k = acc_k*a + w*Ohat_s[k]; out = acc/den -> bf16.
// Partials are f16 like the reference's (crates/amdgpu-kernels/src/fmha/io.rs:83-85: half-precision Ohat inside an allocation the
// contract sizes for f32, tests/gpu/generated/..._kvsplit_abi.h:196): one thread reads 16 bytes per split and writes one 16-byte store.
// A second instantiation reads f32 partials (two 16-byte loads per split), for partials that were exchanged between GPUs.
// HBM-bound: bytes = splits*rows*(256 + 4) + rows*256 (f16), splits*rows*(512 + 4) + rows*256 (f32).
#include "kernels.h"

#include <cuda_bf16.h>

namespace b200mx {

namespace {

__device__ __forceinline__ uint4 ld_stream_u4(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// kScatter: the bf16 rows go to several output buffers (this GPU's and its peers': the all-gather of the row slices done by the stores).
// kF32: the partial rows are f32 (512 bytes per row; partials that crossed GPUs), else f16 (256 bytes per row, the reference's format).
// One thread owns kE consecutive outputs of a row: 8 with f32 partials (two 16-byte loads per split), 16 with f16 partials (also two
// 16-byte loads per split: the same bytes in flight per thread, which is what keeps HBM busy).
template <bool kF32, bool kScatter = false>
__global__ void __launch_bounds__(256)
kvsplit_combine_kernel(const void* __restrict__ ohat, const float* __restrict__ lse2, uint8_t* __restrict__ out, uint32_t rows_total, uint32_t splits,
                       const OutPointers outs = OutPointers{}) {
    constexpr int kE = kF32 ? 8 : 16;
    constexpr uint32_t kGroupsPerRow = 128 / kE;
    const uint64_t ngroups = static_cast<uint64_t>(rows_total) * kGroupsPerRow;
    for (uint64_t t = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < ngroups; t += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        const uint64_t row = t / kGroupsPerRow;
        float m = -1.0e30f, den = 0.0f;
        float acc[kE];
#pragma unroll
        for (int k = 0; k < kE; ++k) acc[k] = 0.0f;
        // four splits at a time: all their loads are issued before the first is used (the kernel lives on bytes in flight)
        for (uint32_t s0 = 0; s0 < splits; s0 += 4u) {
            uint4 raw[4][2];
            float ls[4];
#pragma unroll
            for (uint32_t i = 0; i < 4u; ++i) {
                const uint32_t s = s0 + i < splits ? s0 + i : splits - 1u;   // a short last batch re-reads the last split (and skips it below)
                ls[i] = __ldg(lse2 + static_cast<uint64_t>(s) * rows_total + row);
                const uint4* src = reinterpret_cast<const uint4*>(ohat) + (static_cast<uint64_t>(s) * ngroups + t) * 2u;
                raw[i][0] = ld_stream_u4(src);
                raw[i][1] = ld_stream_u4(src + 1);
            }
#pragma unroll
            for (uint32_t i = 0; i < 4u; ++i) {
                if (s0 + i >= splits) break;
                float v[kE];
                const uint32_t hw[8] = {raw[i][0].x, raw[i][0].y, raw[i][0].z, raw[i][0].w, raw[i][1].x, raw[i][1].y, raw[i][1].z, raw[i][1].w};
                if constexpr (kF32) {
#pragma unroll
                    for (int k = 0; k < 8; ++k) v[k] = __uint_as_float(hw[k]);
                } else {
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        const float2 f = combine_h2_to_f2(hw[k]);
                        v[2 * k] = f.x;
                        v[2 * k + 1] = f.y;
                    }
                }
                float a, w;
                combine_weights(m, den, ls[i], a, w);
#pragma unroll
                for (int k = 0; k < kE; ++k) acc[k] = combine_accumulate(acc[k], a, w, v[k]);
            }
        }
        const float rd = 1.0f / den;
        uint32_t wv[kE / 2];
#pragma unroll
        for (int e = 0; e < kE / 2; ++e) {
            const __nv_bfloat162 b2 = __floats2bfloat162_rn(__fmul_rn(acc[2 * e], rd), __fmul_rn(acc[2 * e + 1], rd));
            wv[e] = *reinterpret_cast<const uint32_t*>(&b2);
        }
#pragma unroll
        for (int h = 0; h < kE / 8; ++h) {
            const uint4 o4 = make_uint4(wv[4 * h], wv[4 * h + 1], wv[4 * h + 2], wv[4 * h + 3]);
            const uint64_t off = (t * (kE / 8) + h) * 16u;
            if (kScatter) {
                for (uint32_t i = 0; i < outs.n; ++i) *reinterpret_cast<uint4*>(outs.out[i] + off) = o4;
            } else {
                *reinterpret_cast<uint4*>(out + off) = o4;
            }
        }
    }
}

}  // namespace

cudaError_t launch_combine_scatter(const void* ohat, bool f32_partials, const float* lse2, const OutPointers& outs, uint32_t rows, uint32_t splits, cudaStream_t stream) {
    const uint64_t ngroups = static_cast<uint64_t>(rows) * (f32_partials ? 16u : 8u);
    uint64_t blocks = (ngroups + 255u) / 256u;
    const uint64_t cap = 148u * 8u * 4u;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    if (f32_partials) kvsplit_combine_kernel<true, true><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(ohat, lse2, nullptr, rows, splits, outs);
    else kvsplit_combine_kernel<false, true><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(ohat, lse2, nullptr, rows, splits, outs);
    return cudaGetLastError();
}

cudaError_t launch_combine(const void* ohat, bool f32_partials, const float* lse2, uint8_t* out, uint32_t rows_total, uint32_t splits, cudaStream_t stream) {
    const uint64_t ngroups = static_cast<uint64_t>(rows_total) * (f32_partials ? 16u : 8u);
    uint64_t blocks = (ngroups + 255u) / 256u;
    // cap the grid at a few waves of 148 SMs x 8 resident blocks; the grid-stride loop covers the rest
    const uint64_t cap = 148u * 8u * 4u;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    if (f32_partials) kvsplit_combine_kernel<true><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(ohat, lse2, out, rows_total, splits);
    else kvsplit_combine_kernel<false><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(ohat, lse2, out, rows_total, splits);
    return cudaGetLastError();
}

}  // namespace b200mx
