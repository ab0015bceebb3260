// Issue-only ceiling of the sm_100a tensor pipe for the MMA shape the attention kernels use (M128 N128 K32, e4m3):
// every CTA keeps its operands resident (zero-filled shared memory) and one thread issues tcgen05.mma back to back, four dependent
// MMAs per score tile, tiles alternating between two accumulators (the shape of the attention kernel's Q K^T stream).
// The result is a second denominator of the attention kernel's roofline fraction; no data leaves the SM.
#include "kernels.h"
#include "ptx_sm100.cuh"

namespace b200mx {
using namespace sm100;

namespace {

constexpr uint32_t kProbeSmem = 2 * 16384 + 64 + 1024;

__global__ void __launch_bounds__(128, 1) mma_issue_ceiling_kernel(int iters, uint32_t* status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t a_smem = base, b_smem = base + 16384, bar = base + 32768;
    volatile uint32_t* slot = reinterpret_cast<volatile uint32_t*>(gen + 32768 + 16);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(gen + 32768 + 20);

    for (uint32_t i = threadIdx.x; i < 32768 / 16; i += blockDim.x) reinterpret_cast<uint4*>(gen)[i] = make_uint4(0, 0, 0, 0);
    if (threadIdx.x == 0) {
        *abort_flag = 0u;
        mbar_init(bar, 1);
        fence_mbar_init();
    }
    if (threadIdx.x < 32) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(slot)), 256);
        tmem_relinquish();
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *slot;

    if (threadIdx.x == 0) {
        uint64_t da[4], db[4];
#pragma unroll
        for (int kb = 0; kb < 4; ++kb) {
            da[kb] = make_smem_desc(a_smem + kb * 32, 16, 1024, kSwizzle128B);
            db[kb] = make_smem_desc(b_smem + kb * 32, 16, 1024, kSwizzle128B);
        }
        const uint32_t id = idesc_f8_dense(128, 128, 0, 0);
        for (int it = 0; it < iters; it += 2) {
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) mma_f8_ss(tmem, da[kb], db[kb], id, kb > 0);
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) mma_f8_ss(tmem + 128, da[kb], db[kb], id, kb > 0);
        }
        tc_commit(bar);
    }
    __syncwarp();
    const bool ok = mbar_wait(bar, 0, abort_flag);
    tc_fence_after_sync();
    __syncthreads();
    if (threadIdx.x == 0 && !ok) atomicOr(status, 2u);
    if (threadIdx.x < 32) tmem_dealloc(tmem, 256);
}

}  // namespace

cudaError_t launch_mma_issue_ceiling(int iters, int ctas, uint32_t* status, cudaStream_t stream) {
    const cudaError_t e = cudaFuncSetAttribute(mma_issue_ceiling_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kProbeSmem);
    if (e != cudaSuccess) return e;
    mma_issue_ceiling_kernel<<<ctas, 128, kProbeSmem, stream>>>(iters, status);
    return cudaGetLastError();
}

}  // namespace b200mx
