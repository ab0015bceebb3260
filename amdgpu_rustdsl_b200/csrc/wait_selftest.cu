// Self-test of the bounded wait every kernel of this library relies on (ptx_sm100.cuh: mbar_wait): one tiny CTA waits, with a short
// budget given by the caller, on an mbarrier that nothing ever arrives at. The wait has to run out, flag the failure and return false;
// the kernel then records that in a status word of its own and ends normally. Nothing spins without a limit and nothing faults: the
// point is to execute the give-up path once on real hardware and to see that the context is as usable afterwards as before.
// The reference has no bounded waits and no counterpart of this kernel.
#include "kernels.h"
#include "ptx_sm100.cuh"

namespace b200mx {
using namespace sm100;

namespace {

__device__ uint32_t g_selftest_word = 0;   // bit 0: the wait ran out (expected); bit 1: the abort flag was raised (expected); bit 2: the wait claimed success

__global__ void __launch_bounds__(64, 1) bounded_wait_selftest_kernel(long long budget_cycles) {
    __shared__ __align__(8) uint64_t bar_storage;
    __shared__ uint32_t abort_word;
    const uint32_t bar = smem_u32(&bar_storage);
    volatile uint32_t* abort_flag = &abort_word;
    if (threadIdx.x == 0) {
        abort_word = 0u;
        mbar_init(bar, 1);   // one arrival expected, none will come
        fence_mbar_init();
    }
    __syncthreads();
    uint32_t bits = 0u;
    if (threadIdx.x < 32) {
        // warp 0 waits with the short budget and raises the flag when it runs out ...
        const bool ok = mbar_wait(bar, 0u, abort_flag, budget_cycles);
        bits |= ok ? 4u : 1u;
    } else {
        // ... warp 1 waits with the library's normal budget and has to leave because of the flag, as the roles of the attention kernel do
        const bool ok = mbar_wait(bar, 0u, abort_flag);
        bits |= ok ? 4u : (*abort_flag != 0u ? 2u : 0u);
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) atomicOr(&g_selftest_word, bits);
}

}  // namespace

cudaError_t run_bounded_wait_selftest(long long budget_cycles, cudaStream_t stream, uint32_t* word, float* ms) {
    const uint32_t zero = 0u;
    cudaEvent_t e0, e1;
    cudaError_t e = cudaEventCreate(&e0);
    if (e != cudaSuccess) return e;
    e = cudaEventCreate(&e1);
    if (e != cudaSuccess) { cudaEventDestroy(e0); return e; }
    e = cudaMemcpyToSymbolAsync(g_selftest_word, &zero, 4, 0, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) e = cudaEventRecord(e0, stream);
    if (e == cudaSuccess) {
        bounded_wait_selftest_kernel<<<1, 64, 0, stream>>>(budget_cycles);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaEventRecord(e1, stream);
    if (e == cudaSuccess) e = cudaMemcpyFromSymbolAsync(word, g_selftest_word, 4, 0, cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e == cudaSuccess) e = cudaEventElapsedTime(ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return e;
}

}  // namespace b200mx
