// Device quantisers that produce the path's inputs from bf16 activations: the step in front of the attention kernels.
//
// The reference has no device code for this (its only FMHA quantiser is host code in the test harness, tests/gpu/ref_host.cpp:239-254;
// its device quantiser `quant_mxfp8_bf16_k` serves GEMM operands with 1x128 blocks and another scale rule,
// crates/amdgpu-kernels/src/rows/mxquant.rs:9-11,153). The rule restated here is the harness's:
//   Q, K: per 32 elements of the head dim  E8M0 = clamp(floor(log2 amax) - 8 + 127, 0, 254), elements e4m3(x * 2^-(E8M0 - 127)) rounded
//         to nearest even, saturating at 448; Q is multiplied by log2(e) / sqrt(128) first (`mul`), K by 1;
//   V:    per tensor  descale = amax / 448, elements e4m3(x / descale).
// All arithmetic is f32 with one rounding per operation, in the order written, so that the CPU restatement in the test oracle matches
// bit for bit. Inputs must be finite. Both kernels are pure streaming: 2 bytes in, 1 (+ 1/32) byte out per element.
#include "kernels.h"

#include <cuda_bf16.h>

namespace b200mx {

namespace {

__device__ __forceinline__ uint32_t e4m3x2(float lo, float hi) {
    uint16_t h;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(h) : "f"(hi), "f"(lo));
    return h;
}

// One thread = 8 consecutive elements (16 bytes in, 8 bytes out); 4 threads = one 32-element block; 16 threads = one row of 128.
__global__ void __launch_bounds__(256) quantize_qk_kernel(const uint4* __restrict__ x, unsigned long long rows, float mul,
                                                          uint2* __restrict__ out, uint32_t* __restrict__ scales) {
    const unsigned long long n_threads = rows * 16ull;
    const unsigned lane = threadIdx.x & 31u;
    for (unsigned long long t0 = (static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x) & ~31ull; t0 < n_threads;
         t0 += static_cast<unsigned long long>(gridDim.x) * blockDim.x) {
        const unsigned long long t = t0 + lane;   // whole warps stay in the loop together: the shuffles below need all lanes
        const bool live = t < n_threads;
        float y[8];
        if (live) {
            const uint4 raw = __ldg(x + t);
            const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                y[2 * i] = __fmul_rn(__uint_as_float(w[i] << 16), mul);
                y[2 * i + 1] = __fmul_rn(__uint_as_float(w[i] & 0xFFFF0000u), mul);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) y[i] = 0.0f;
        }
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(y[i]));
        amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
        // floor(log2 amax) of a normal f32 is its exponent field - 127; zero and subnormal maxima end at the lower clamp either way
        int eb = static_cast<int>((__float_as_uint(amax) >> 23) & 0xFFu) - 8;
        eb = eb < 0 ? 0 : (eb > 254 ? 254 : eb);
        // x * 2^(127 - eb) as two exact multiplications by normal powers of two (the exponent 127 - eb lies in [-127, 127]; a value that
        // an intermediate product flushes or rounds is far below the smallest e4m3 step in the end and encodes as zero either way)
        const int sh = 127 - eb, sh1 = sh >> 1, sh2 = sh - sh1;
        const float s1 = __uint_as_float(static_cast<uint32_t>(127 + sh1) << 23), s2 = __uint_as_float(static_cast<uint32_t>(127 + sh2) << 23);
        uint32_t b[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            b[i] = e4m3x2(__fmul_rn(__fmul_rn(y[4 * i], s1), s2), __fmul_rn(__fmul_rn(y[4 * i + 1], s1), s2)) |
                   (e4m3x2(__fmul_rn(__fmul_rn(y[4 * i + 2], s1), s2), __fmul_rn(__fmul_rn(y[4 * i + 3], s1), s2)) << 16);
        }
        if (live) out[t] = make_uint2(b[0], b[1]);
        // the row's four scale bytes: lanes 0, 4, 8, 12 of each 16-lane half hold them
        const uint32_t e1 = __shfl_down_sync(0xFFFFFFFFu, static_cast<uint32_t>(eb), 4);
        const uint32_t e2 = __shfl_down_sync(0xFFFFFFFFu, static_cast<uint32_t>(eb), 8);
        const uint32_t e3 = __shfl_down_sync(0xFFFFFFFFu, static_cast<uint32_t>(eb), 12);
        if (live && (lane & 15u) == 0u) scales[t >> 4] = static_cast<uint32_t>(eb) | (e1 << 8) | (e2 << 16) | (e3 << 24);
    }
}

__global__ void __launch_bounds__(256) amax_kernel(const uint4* __restrict__ x, unsigned long long n_vec, uint32_t* __restrict__ amax_bits) {
    float amax = 0.0f;
    for (unsigned long long t = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x; t < n_vec;
         t += static_cast<unsigned long long>(gridDim.x) * blockDim.x) {
        const uint4 raw = __ldg(x + t);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) amax = fmaxf(amax, fmaxf(fabsf(__uint_as_float(w[i] << 16)), fabsf(__uint_as_float(w[i] & 0xFFFF0000u))));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    if ((threadIdx.x & 31u) == 0u) atomicMax(amax_bits, __float_as_uint(amax));   // non-negative floats order like their bit patterns
}

__global__ void __launch_bounds__(256) quantize_v_kernel(const uint4* __restrict__ x, unsigned long long n_vec, uint2* __restrict__ out,
                                                         float* __restrict__ descale) {
    const float amax = __uint_as_float(reinterpret_cast<const uint32_t*>(descale)[1]);
    const float vd = amax > 0.0f ? __fdiv_rn(amax, 448.0f) : 1.0f;
    if (blockIdx.x == 0 && threadIdx.x == 0) descale[0] = vd;
    for (unsigned long long t = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x; t < n_vec;
         t += static_cast<unsigned long long>(gridDim.x) * blockDim.x) {
        const uint4 raw = __ldg(x + t);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        uint32_t b[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            b[i] = e4m3x2(__fdiv_rn(__uint_as_float(w[2 * i] << 16), vd), __fdiv_rn(__uint_as_float(w[2 * i] & 0xFFFF0000u), vd)) |
                   (e4m3x2(__fdiv_rn(__uint_as_float(w[2 * i + 1] << 16), vd), __fdiv_rn(__uint_as_float(w[2 * i + 1] & 0xFFFF0000u), vd)) << 16);
        }
        out[t] = make_uint2(b[0], b[1]);
    }
}

int grid_for(unsigned long long threads) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const unsigned long long blocks = (threads + 255) / 256, cap = 8ull * static_cast<unsigned long long>(sms);   // grid-stride beyond 8 CTAs per SM
    return static_cast<int>(blocks < cap ? (blocks ? blocks : 1) : cap);
}

}  // namespace

cudaError_t launch_quantize_qk(const void* x_bf16, unsigned long long rows, float mul, void* out_e4m3, void* out_scales, cudaStream_t stream) {
    quantize_qk_kernel<<<grid_for(rows * 16ull), 256, 0, stream>>>(static_cast<const uint4*>(x_bf16), rows, mul, static_cast<uint2*>(out_e4m3),
                                                                   static_cast<uint32_t*>(out_scales));
    return cudaGetLastError();
}

cudaError_t launch_quantize_v(const void* x_bf16, unsigned long long n_elems, void* out_e4m3, float* descale, cudaStream_t stream) {
    cudaError_t e = cudaMemsetAsync(descale, 0, 8, stream);   // [0] the descale, [1] the running maximum's bits
    if (e != cudaSuccess) return e;
    const unsigned long long n_vec = n_elems / 8;
    amax_kernel<<<grid_for(n_vec), 256, 0, stream>>>(static_cast<const uint4*>(x_bf16), n_vec, reinterpret_cast<uint32_t*>(descale) + 1);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    quantize_v_kernel<<<grid_for(n_vec), 256, 0, stream>>>(static_cast<const uint4*>(x_bf16), n_vec, static_cast<uint2*>(out_e4m3), descale);
    return cudaGetLastError();
}

}  // namespace b200mx
