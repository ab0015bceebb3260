// Key-range sharding across the GPUs of one node without a collective for the partials: every GPU's split kernel stores the rows of
// its partial (f16, or f32 on request) straight into the memory of the GPU that will combine them (TMA tile stores and plain stores to peer memory over
// NVLink, as the tiles come out of tensor memory, so the transfer runs under the remaining compute), and every GPU's combine kernel
// stores its bf16 row slice into every GPU's output buffer. Between the two kernels, and after the second, the ranks only need a barrier.
// The reference has no multi-GPU code; the algebra is its KV-split one with "split = GPU" (crates/amdgpu-stage/src/components.rs:58-74,
// crates/amdgpu-tile/src/epilogue.rs:117-146).
//
// This file holds the host side: device buffers that other processes of the node can map (CUDA IPC; one process per GPU), and the
// device-resident plan (one tensor map and one log-sum-exp pointer per destination GPU) that the split kernel reads.
// No TMA load ever touches peer memory here, with or without multicast: peers are only written to.
#include "../../include/fmha_mxfp8_abi.h"
#include "kernels.h"

#include <atomic>
#include <cstring>

namespace b200mx {
int encode_partial_map(CUtensorMap* m, void* base, uint64_t seq, uint64_t heads, uint64_t batches, uint64_t splits, bool f32);   // host_api.cu
}

namespace b200mx {
namespace {

struct FlagArrays {
    uint32_t* a[FMHA_MXFP8_PEER_MAX_GPUS];   // a[r]: rank r's arrival flags [world], as mapped into this process
};

// The ranks of a node line up on their streams: thread t of the one warp tells rank t that this rank has arrived (a release store at
// system scope into rank t's flag array, behind a system-scope fence: what this GPU's earlier kernels stored to its peers is performed
// before the flag) and waits, with a clock budget, until rank t's arrival shows in this rank's own array. The arrival numbers only grow
// (one per barrier of a plan), so a peer that is already one barrier further does no harm. Each GPU runs its own launch of this kernel;
// the launches wait for launches on *other* GPUs, never for one another on the same GPU.
__global__ void peer_barrier_kernel(FlagArrays f, uint32_t world, uint32_t rank, uint32_t arrival, long long budget_cycles, uint32_t* status) {
    const uint32_t t = threadIdx.x;
    if (t >= world) return;
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f.a[t] + rank), "r"(arrival) : "memory");
    const uint32_t* mine = f.a[rank] + t;
    const long long t0 = clock64();
    for (;;) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
        if (static_cast<int32_t>(v - arrival) >= 0) break;
        if (clock64() - t0 > budget_cycles) {
            atomicOr(status, 2u);   // bit 1: a barrier between GPUs ran out of time
            break;
        }
    }
    __threadfence_system();
}

}  // namespace
}  // namespace b200mx

extern "C" {

int fmha_mxfp8_peer_barrier(void* const* flag_arrays, uint32_t world, uint32_t rank, uint32_t arrival, uint32_t budget_us, void* status_dev, void* stream) {
    if (!flag_arrays || world < 1 || world > FMHA_MXFP8_PEER_MAX_GPUS || rank >= world || arrival == 0 || budget_us == 0) return FMHA_MXFP8_E_ARG;
    b200mx::FlagArrays f;
    std::memset(&f, 0, sizeof f);
    for (uint32_t r = 0; r < world; ++r) {
        if (!flag_arrays[r] || (reinterpret_cast<uintptr_t>(flag_arrays[r]) & 3u)) return FMHA_MXFP8_E_ARG;
        f.a[r] = static_cast<uint32_t*>(flag_arrays[r]);
    }
    uint32_t* status = status_dev ? static_cast<uint32_t*>(status_dev) : b200mx::device_status_word();
    if (!status) return -static_cast<int>(cudaErrorInvalidSymbol);
    // the budget in SM clocks at the GPU's maximum clock, asked for once per device (the attribute query takes milliseconds)
    static std::atomic<int> khz_of[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return -static_cast<int>(e);
    int khz = (dev >= 0 && dev < 64) ? khz_of[dev].load(std::memory_order_relaxed) : 0;
    if (khz == 0) {
        e = cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev);
        if (e != cudaSuccess || khz <= 0) khz = 2000000;
        if (dev >= 0 && dev < 64) khz_of[dev].store(khz, std::memory_order_relaxed);
    }
    const long long budget_cycles = static_cast<long long>(budget_us) * khz / 1000;
    b200mx::peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(f, world, rank, arrival, budget_cycles, status);
    e = cudaGetLastError();
    return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

int fmha_mxfp8_peer_alloc(size_t bytes, void** dev_ptr, void* handle64) {
    if (!dev_ptr || !handle64 || bytes == 0) return FMHA_MXFP8_E_ARG;
    static_assert(sizeof(cudaIpcMemHandle_t) == FMHA_MXFP8_PEER_HANDLE_BYTES, "IPC handle size");
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) return -static_cast<int>(e);
    e = cudaMemset(p, 0, bytes);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) { cudaFree(p); return -static_cast<int>(e); }
    std::memcpy(handle64, &h, sizeof h);
    *dev_ptr = p;
    return 0;
}

int fmha_mxfp8_peer_open(const void* handle64, void** dev_ptr) {
    if (!handle64 || !dev_ptr) return FMHA_MXFP8_E_ARG;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle64, sizeof h);
    const cudaError_t e = cudaIpcOpenMemHandle(dev_ptr, h, cudaIpcMemLazyEnablePeerAccess);
    return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

int fmha_mxfp8_peer_close(void* dev_ptr) {
    if (!dev_ptr) return FMHA_MXFP8_E_ARG;
    const cudaError_t e = cudaIpcCloseMemHandle(dev_ptr);
    return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

int fmha_mxfp8_peer_free(void* dev_ptr) {
    if (!dev_ptr) return FMHA_MXFP8_E_ARG;
    const cudaError_t e = cudaFree(dev_ptr);
    return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

int fmha_mxfp8_peer_plan_build(uint32_t world, uint32_t rank, uint32_t H, uint32_t S, int f32_partials, void* const* ohat_recv, void* const* lse_recv, void* plan_dev,
                               void* stream) {
    if (world < 2 || world > FMHA_MXFP8_PEER_MAX_GPUS || rank >= world || H == 0 || S == 0 || !ohat_recv || !lse_recv || !plan_dev) return FMHA_MXFP8_E_ARG;
    // a 128-row block of queries must belong to one destination: whole blocks per GPU
    if (S % world != 0 || (S / world) % 128u != 0) return FMHA_MXFP8_E_ARG;
    if (reinterpret_cast<uintptr_t>(plan_dev) & 127u) return FMHA_MXFP8_E_ARG;
    static_assert(sizeof(b200mx::PeerPlan) == FMHA_MXFP8_PEER_PLAN_BYTES, "plan size");
    b200mx::PeerPlan plan;
    std::memset(&plan, 0, sizeof plan);
    plan.world = world;
    plan.rank = rank;
    plan.dest_rows = S / world;
    for (uint32_t d = 0; d < world; ++d) {
        if (!ohat_recv[d] || !lse_recv[d]) return FMHA_MXFP8_E_ARG;
        // destination d's receive buffer: f16 or f32 [source GPU][its S / world query rows][H][128]
        const int r = b200mx::encode_partial_map(&plan.maps[d], ohat_recv[d], plan.dest_rows, H, 1, world, f32_partials != 0);
        if (r) return r;
        plan.lse[d] = static_cast<float*>(lse_recv[d]);
    }
    const cudaError_t e = cudaMemcpyAsync(plan_dev, &plan, sizeof plan, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return -static_cast<int>(e);
    const cudaError_t e2 = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));   // `plan` lives on this stack frame
    return e2 == cudaSuccess ? 0 : -static_cast<int>(e2);
}

int fmha_mxfp8_combine_scatter(const void* ohat, int f32_partials, const void* lse, void* const* outs, uint32_t n_outs, uint64_t row_offset, uint32_t rows,
                               uint32_t splits, void* stream) {
    if (!ohat || !lse || !outs || n_outs == 0 || n_outs > FMHA_MXFP8_PEER_MAX_GPUS || rows == 0 || splits == 0) return FMHA_MXFP8_E_ARG;
    b200mx::OutPointers op;
    std::memset(&op, 0, sizeof op);
    for (uint32_t i = 0; i < n_outs; ++i) {
        if (!outs[i] || (reinterpret_cast<uintptr_t>(outs[i]) & 15u)) return FMHA_MXFP8_E_ARG;
        op.out[i] = static_cast<uint8_t*>(outs[i]) + row_offset * 256u;
    }
    op.n = n_outs;
    const cudaError_t e = b200mx::launch_combine_scatter(ohat, f32_partials != 0, static_cast<const float*>(lse), op, rows, splits, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

int fmha_mxfp8_copy_async(void* dst, const void* src, size_t bytes, void* stream) {
    if (!dst || !src) return FMHA_MXFP8_E_ARG;
    const cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

}  // extern "C"
