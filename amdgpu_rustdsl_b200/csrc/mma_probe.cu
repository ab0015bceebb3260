// Issue-only ceiling of the sm_100a tensor pipe for the MMA shapes the attention kernels use (M128 N128 K32, e4m3):
// every CTA keeps its operands resident (zero-filled shared / tensor memory) and issues tcgen05.mma back to back.
// The result is the denominator of the attention kernels' roofline fraction; no data leaves the SM.
#include "kernels.h"
#include "ptx_sm100.cuh"

namespace fmha {
using namespace sm100;

namespace {

constexpr uint32_t kProbeSmem = 2 * 16384 + 1024 + 64 + 1024;

__global__ void __launch_bounds__(128, 1) mma_probe_kernel(int variant, int iters, uint32_t* status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t a_smem = base, b_smem = base + 16384, sf_smem = base + 32768, bar = base + 32768 + 1024;
    volatile uint32_t* slot = reinterpret_cast<volatile uint32_t*>(gen + 32768 + 1024 + 16);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(gen + 32768 + 1024 + 20);

    for (uint32_t i = threadIdx.x; i < (32768 + 1024) / 16; i += blockDim.x) reinterpret_cast<uint4*>(gen)[i] = make_uint4(0, 0, 0, 0);
    if (threadIdx.x == 0) {
        *abort_flag = 0u;
        mbar_init(bar, variant == 8 ? 2 : 1);
        fence_mbar_init();
    }
    if (threadIdx.x < 32) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(slot)), 512);
        tmem_relinquish();
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *slot;

    // zero the TMEM columns that variants 1 and 2 read as the A operand (columns 256..287)
    {
        uint32_t z[32];
#pragma unroll
        for (int c = 0; c < 32; ++c) z[c] = 0u;
        tmem_st32(tmem + 256 + (((threadIdx.x >> 5) * 32u) << 16), z);
        tmem_wait_st();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();

    if (threadIdx.x == 0) {
        const uint32_t t_sfa = tmem + 384, t_sfb = tmem + 388;
        tmem_cp_sf(t_sfa, make_smem_desc(sf_smem, 0, 128, kSwizzleNone));
        tmem_cp_sf(t_sfb, make_smem_desc(sf_smem + 512, 0, 128, kSwizzleNone));
        const uint32_t id_bs = idesc_mxf8_block_scaled(128, 128, 0, 0, 0, 0);
        const uint32_t id_bs_mn = idesc_mxf8_block_scaled(128, 128, 0, 1, 0, 0);
        const uint32_t id_f8_mn = idesc_f8_dense(128, 128, 0, 1);
        if (variant >= 9 && variant <= 12) {
            // Tight loops with every descriptor prepared up front, to separate the hardware's cost per instruction from loop overhead:
            // 9 = four dependent MMAs per tile, tiles alternate between two accumulators (what the kernels' Q K^T stream does);
            // 10 = the same work with the two accumulators interleaved MMA by MMA (two independent chains in flight);
            // 11 = one accumulator throughout (one long dependent chain, what the P V stream is); 12 = like 9 with N = 144 from tensor memory.
            uint64_t da[4], db[4], dv[4];
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) {
                da[kb] = make_smem_desc(a_smem + kb * 32, 16, 1024, kSwizzle128B);
                db[kb] = make_smem_desc(b_smem + kb * 32, 16, 1024, kSwizzle128B);
                dv[kb] = make_smem_desc(b_smem + (kb & 1) * 4096, 1024, 1024, kSwizzle128B);
            }
            const uint32_t id = idesc_f8_dense(128, 128, 0, 0), id_pv = idesc_f8_dense(128, 144, 0, 1);
            if (variant == 9) {
                for (int it = 0; it < iters; it += 2) {
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb) mma_f8_ss(tmem, da[kb], db[kb], id, kb > 0);
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb) mma_f8_ss(tmem + 128, da[kb], db[kb], id, kb > 0);
                }
            } else if (variant == 10) {
                for (int it = 0; it < iters; it += 2) {
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb) {
                        mma_f8_ss(tmem, da[kb], db[kb], id, kb > 0);
                        mma_f8_ss(tmem + 128, da[kb], db[kb], id, kb > 0);
                    }
                }
            } else if (variant == 11) {
                for (int it = 0; it < iters; ++it) {
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb) mma_f8_ss(tmem, da[kb], db[kb], id, 1u);
                }
            } else {
                for (int it = 0; it < iters; ++it) {
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb) mma_f8_ts(tmem, tmem + 256 + 8 * kb, dv[kb], id_pv, 1u);
                }
            }
        } else
        for (int it = 0; it < iters; ++it) {
            const uint32_t d = tmem + ((it & 1) ? 128u : 0u);
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) {
                if (variant == 0) {
                    const uint64_t da = make_smem_desc(a_smem + kb * 32, 16, 1024, kSwizzle128B);
                    const uint64_t db = make_smem_desc(b_smem + kb * 32, 16, 1024, kSwizzle128B);
                    mma_mxf8_ss(d, da, db, id_bs | (kb << 29) | (kb << 4), t_sfa + (kb << 30), t_sfb + (kb << 30), kb > 0);
                } else if (variant == 1) {
                    const uint64_t db = make_smem_desc(b_smem + kb * 4096, 1024, 1024, kSwizzle128B);
                    mma_mxf8_ts(d, tmem + 256 + 8 * kb, db, id_bs_mn | (kb << 29) | (kb << 4), t_sfa + (kb << 30), t_sfb + (kb << 30), kb > 0);
                } else if (variant == 2) {
                    const uint64_t db = make_smem_desc(b_smem + kb * 4096, 1024, 1024, kSwizzle128B);
                    mma_f8_ts(d, tmem + 256 + 8 * kb, db, id_f8_mn, kb > 0);
                } else if (variant == 3) {   // plain fp8, A from shared memory, B MN-major
                    const uint64_t da = make_smem_desc(a_smem + kb * 32, 16, 1024, kSwizzle128B);
                    const uint64_t db = make_smem_desc(b_smem + kb * 4096, 1024, 1024, kSwizzle128B);
                    mma_f8_ss(d, da, db, id_f8_mn, kb > 0);
                } else if (variant == 4) {   // plain fp8, A from tensor memory, B K-major
                    const uint64_t db = make_smem_desc(b_smem + kb * 32, 16, 1024, kSwizzle128B);
                    mma_f8_ts(d, tmem + 256 + 8 * kb, db, idesc_f8_dense(128, 128, 0, 0), kb > 0);
                } else if (variant == 5) {   // plain fp8, both from shared memory, K-major
                    const uint64_t da = make_smem_desc(a_smem + kb * 32, 16, 1024, kSwizzle128B);
                    const uint64_t db = make_smem_desc(b_smem + kb * 32, 16, 1024, kSwizzle128B);
                    mma_f8_ss(d, da, db, idesc_f8_dense(128, 128, 0, 0), kb > 0);
                } else if (variant == 6) {   // the 16-column row-sum MMA (A from tensor memory, unswizzled K-major B)
                    const uint64_t db = make_smem_desc(b_smem, 128, 256, kSwizzleNone);
                    mma_f8_ts(d, tmem + 256 + 8 * kb, db, idesc_f8_dense(128, 16, 0, 0), kb > 0);
                } else {   // 7 and 8: plain fp8, both from shared memory, N = 256 (B rows wrap inside the 16 KiB tile: timing only)
                    const uint64_t da = make_smem_desc(a_smem + kb * 32, 16, 1024, kSwizzle128B);
                    const uint64_t db = make_smem_desc(a_smem + kb * 32, 16, 1024, kSwizzle128B);
                    mma_f8_ss(tmem, da, db, idesc_f8_dense(128, 256, 0, 0), kb > 0);
                }
            }
        }
        tc_commit(bar);
    } else if (threadIdx.x == 32 && variant == 8) {
        // a second issuing thread, to see whether the issue rate of one thread or the tensor pipe is the limit
        for (int it = 0; it < iters; ++it) {
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) {
                const uint64_t da = make_smem_desc(a_smem + kb * 32, 16, 1024, kSwizzle128B);
                const uint64_t db = make_smem_desc(b_smem + kb * 32, 16, 1024, kSwizzle128B);
                mma_f8_ss(tmem + 256, da, db, idesc_f8_dense(128, 128, 0, 0), kb > 0);
            }
        }
        tc_commit(bar);
    }
    __syncwarp();
    const bool ok = mbar_wait(bar, 0, abort_flag);
    tc_fence_after_sync();
    __syncthreads();
    if (threadIdx.x == 0 && !ok) atomicOr(status, 2u);
    if (threadIdx.x < 32) tmem_dealloc(tmem, 512);
}

}  // namespace

cudaError_t launch_mma_probe(int variant, int iters, int ctas, uint32_t* status, cudaStream_t stream) {
    static bool attr_done = false;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(mma_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kProbeSmem);
        if (e != cudaSuccess) return e;
        attr_done = true;
    }
    mma_probe_kernel<<<ctas, 128, kProbeSmem, stream>>>(variant, iters, status);
    return cudaGetLastError();
}

}  // namespace fmha
