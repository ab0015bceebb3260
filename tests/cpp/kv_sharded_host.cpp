// A host for the key-range-sharded forward written against the C ABI alone: no PyTorch, no NCCL, one process per GPU (fork), the CUDA
// runtime for memory and the library for everything else. It is what a maintainer of the reference would write in the reference's own
// host language (its harness tests/gpu/ref_host.cpp is C++ over the HIP runtime): fill the generated Args of the kvsplit kernel, launch,
// combine. The multi-GPU part has no counterpart in the reference; its algebra is the reference's KV split with "split = GPU"
// (crates/amdgpu-stage/src/components.rs:58-74, crates/amdgpu-tile/src/epilogue.rs:117-146).
//
//   kv_sharded_host <world> [S] [SK] [H]
//
// Every rank holds all queries and its own key range. Rank r: fmha_mxfp8_peer_alloc -> handles through shared memory ->
// fmha_mxfp8_peer_open -> fmha_mxfp8_peer_plan_build -> kvsplit launch with the plan (partial rows go straight to the combining GPU) ->
// fmha_mxfp8_peer_barrier -> fmha_mxfp8_combine_scatter (bf16 rows to every GPU) -> fmha_mxfp8_peer_barrier. Rank 0 then runs the same
// problem on its GPU alone (one kvsplit launch per key range into ohat_all[r], fmha_mxfp8_combine_f32 with splits = world) and compares
// the bytes: both forms run the same kernels on the same numbers, so they must be equal. Prints "KV_SHARDED_HOST_OK ..." and exits 0.
// Test infrastructure: built and run by tests/test_gpu_cpp_host.py on a machine with at least two GPUs.
#include "fmha_mxfp8_abi.h"

#include <cuda_runtime.h>

#include <sys/mman.h>
#include <sys/wait.h>
#include <unistd.h>

#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <new>
#include <cstring>
#include <vector>

namespace {

constexpr int kMaxWorld = FMHA_MXFP8_PEER_MAX_GPUS;

struct Shared {   // one page of memory shared by the processes (mapped before the fork)
    std::atomic<int> arrived[8];   // host barriers: a counter per use
    std::atomic<int> failed;
    unsigned char handle[kMaxWorld][FMHA_MXFP8_PEER_HANDLE_BYTES];
};

void host_barrier(Shared* sh, int which, int world) {
    sh->arrived[which].fetch_add(1);
    while (sh->arrived[which].load() < world && sh->failed.load() == 0) usleep(50);
}

#define CHECK(cond, what)                                                                   \
    do {                                                                                    \
        if (!(cond)) {                                                                      \
            std::fprintf(stderr, "rank %d: %s failed (%s:%d)\n", rank, what, __FILE__, __LINE__); \
            sh->failed.store(1);                                                            \
            return 1;                                                                       \
        }                                                                                   \
    } while (0)

// deterministic bytes: e4m3 values of moderate size (exponent field 4..9), any sign
void fill_e4m3(std::vector<uint8_t>& v, uint64_t seed) {
    uint64_t x = seed * 0x9E3779B97F4A7C15ull + 1;
    for (auto& b : v) {
        x = x * 6364136223846793005ull + 1442695040888963407ull;
        const uint32_t r = static_cast<uint32_t>(x >> 33);
        b = static_cast<uint8_t>(((r & 1u) << 7) | ((4u + (r >> 1) % 6u) << 3) | ((r >> 8) & 7u));
    }
}

struct Dev {   // device copies of one rank's inputs
    void *q = nullptr, *k = nullptr, *v = nullptr, *qs = nullptr, *ks = nullptr, *vs = nullptr;
};

void fill_args(fmha_mxfp8_kvsplit_args& a, const Dev& d, uint32_t S, uint32_t H, uint32_t SKl, void* ohat, void* lse, uint32_t flags) {
    std::memset(&a, 0, sizeof a);
    a.ptr_q = d.q; a.ptr_k = d.k; a.ptr_v = d.v;
    a.s_seq_len = S; a.s_Seqs = H * 128; a.s_Hs = 128; a.s_Bs = S * H * 128;
    a.s_gqa = 1; a.s_k_Seqs = H * 128; a.s_k_Hs = 128; a.s_k_Bs = SKl * H * 128;
    a.s_kv_seq_len = SKl; a.s_q_head_num = H;
    a.s_v_Seqs = H * 128; a.s_v_Hs = 128; a.s_v_Bs = SKl * H * 128;
    a.s_o_Seqs = H * 256; a.s_o_Hs = 256; a.s_o_Bs = S * H * 256;
    a.ptr_q_descale = d.qs; a.ptr_k_descale = d.ks; a.ptr_v_descale = d.vs;
    a.s_descale_q_Bs = S * H * 4; a.s_descale_q_Hs = 4; a.s_descale_k_Bs = SKl * H * 4; a.s_descale_k_Hs = 4;
    a.ext_flags = flags;
    a.ptr_ohat = ohat; a.ptr_lse = lse; a.kvs_splits = 1; a.kvs_rows_total = S * H;
}

int run_rank(int rank, int world, uint32_t S, uint32_t SK, uint32_t H, Shared* sh) {
    CHECK(cudaSetDevice(rank) == cudaSuccess, "cudaSetDevice");
    const uint32_t rows = S * H, n = rows / world, SKl = SK / world;
    // inputs: the same Q on every rank, the rank's own key range
    auto upload = [&](const std::vector<uint8_t>& h, void** dptr) {
        return cudaMalloc(dptr, h.size()) == cudaSuccess && cudaMemcpy(*dptr, h.data(), h.size(), cudaMemcpyHostToDevice) == cudaSuccess;
    };
    auto make_inputs = [&](int r, Dev& d) {   // rank r's view: Q, scales, K/V of key range r
        std::vector<uint8_t> q(size_t(S) * H * 128), k(size_t(SKl) * H * 128), v(size_t(SKl) * H * 128);
        fill_e4m3(q, 11);
        fill_e4m3(k, 100 + r);
        fill_e4m3(v, 200 + r);
        std::vector<uint8_t> qs(size_t(S) * H * 4 + 512 * H * 4, 0), ks(size_t(SKl) * H * 4 + 640 * H * 4, 0);
        std::fill(qs.begin(), qs.begin() + size_t(S) * H * 4, uint8_t(118));   // E8M0 2^-9 on every 32-element block
        std::fill(ks.begin(), ks.begin() + size_t(SKl) * H * 4, uint8_t(119));
        std::vector<float> vs(1024, 0.0f);
        vs[0] = 0.03125f;
        std::vector<uint8_t> vsb(reinterpret_cast<uint8_t*>(vs.data()), reinterpret_cast<uint8_t*>(vs.data()) + 4096);
        return upload(q, &d.q) && upload(k, &d.k) && upload(v, &d.v) && upload(qs, &d.qs) && upload(ks, &d.ks) && upload(vsb, &d.vs);
    };
    Dev mine;
    CHECK(make_inputs(rank, mine), "input upload");

    // the peer buffer: receive slots [world][n][128] f32, log-sum-exps [world][n] f32, the whole bf16 output, the barrier's flags
    auto al = [](size_t x) { return (x + 255) / 256 * 256; };
    const size_t off_lse = al(size_t(world) * n * 512), off_out = off_lse + al(size_t(world) * n * 4), off_flags = off_out + al(size_t(rows) * 256);
    const size_t bytes = off_flags + 256;
    void* own = nullptr;
    CHECK(fmha_mxfp8_peer_alloc(bytes, &own, sh->handle[rank]) == 0, "fmha_mxfp8_peer_alloc");
    host_barrier(sh, 0, world);
    CHECK(sh->failed.load() == 0, "a peer's set-up");
    void* ptr[kMaxWorld] = {};
    for (int r = 0; r < world; ++r) {
        if (r == rank) ptr[r] = own;
        else CHECK(fmha_mxfp8_peer_open(sh->handle[r], &ptr[r]) == 0, "fmha_mxfp8_peer_open");
    }
    void *ohat_recv[kMaxWorld], *lse_recv[kMaxWorld], *outs[kMaxWorld], *flags[kMaxWorld];
    for (int r = 0; r < world; ++r) {
        ohat_recv[r] = ptr[r];
        lse_recv[r] = static_cast<uint8_t*>(ptr[r]) + off_lse;
        outs[r] = static_cast<uint8_t*>(ptr[r]) + off_out;
        flags[r] = static_cast<uint8_t*>(ptr[r]) + off_flags;
    }
    void* plan_raw = nullptr;
    CHECK(cudaMalloc(&plan_raw, FMHA_MXFP8_PEER_PLAN_BYTES + 128) == cudaSuccess, "cudaMalloc(plan)");
    void* plan = reinterpret_cast<void*>((reinterpret_cast<uintptr_t>(plan_raw) + 127) / 128 * 128);
    CHECK(fmha_mxfp8_peer_plan_build(world, rank, H, S, 1, ohat_recv, lse_recv, plan, nullptr) == 0, "fmha_mxfp8_peer_plan_build");
    host_barrier(sh, 1, world);   // every rank has mapped every buffer: stores may begin
    CHECK(sh->failed.load() == 0, "a peer's set-up");

    // the step, twice (the second run reuses the receive slots and the flags)
    fmha_mxfp8_kvsplit_args a;
    void *dummy_o = nullptr, *dummy_l = nullptr;
    CHECK(cudaMalloc(&dummy_o, 256) == cudaSuccess && cudaMalloc(&dummy_l, 256) == cudaSuccess, "cudaMalloc");
    fill_args(a, mine, S, H, SKl, dummy_o, dummy_l, FMHA_MXFP8_FLAG_F32_PARTIALS);
    a.ext_ptr_peer_plan = plan;
    const uint32_t grid[3] = {(S + 255) / 256, H, 1};
    fmha_mxfp8_buffer_sizes sz;
    std::memset(&sz, 0, sizeof sz);
    sz.ptr_q = size_t(S) * H * 128; sz.ptr_k = sz.ptr_v = size_t(SKl) * H * 128; sz.ptr_o = size_t(S) * H * 256;
    sz.ptr_q_descale = size_t(S) * H * 4 + 512 * H * 4; sz.ptr_k_descale = size_t(SKl) * H * 4 + 640 * H * 4; sz.ptr_v_descale = 4096;
    sz.ptr_ohat = size_t(rows) * 512; sz.ptr_lse = size_t(rows) * 4;   // the contract's extents; with a plan the launch writes neither
    fmha_mxfp8_symbols sy{1, static_cast<int64_t>(H), 0};
    char err[256];
    CHECK(fmha_mxfp8_validate(FMHA_MXFP8_KVSPLIT, &a, &sz, grid, &sy, err, sizeof err) == 0, err);
    uint32_t arrival = 0;
    for (int step = 0; step < 2; ++step) {
        CHECK(fmha_mxfp8_launch(FMHA_MXFP8_KVSPLIT, &a, grid, nullptr) == 0, "kvsplit launch");
        CHECK(fmha_mxfp8_peer_barrier(flags, world, rank, ++arrival, 20000000u, nullptr, nullptr) == 0, "fmha_mxfp8_peer_barrier");
        CHECK(fmha_mxfp8_combine_scatter(own, 1, static_cast<uint8_t*>(own) + off_lse, outs, world, uint64_t(rank) * n, n, world, nullptr) == 0,
              "fmha_mxfp8_combine_scatter");
        CHECK(fmha_mxfp8_peer_barrier(flags, world, rank, ++arrival, 20000000u, nullptr, nullptr) == 0, "fmha_mxfp8_peer_barrier");
    }
    CHECK(cudaDeviceSynchronize() == cudaSuccess, "cudaDeviceSynchronize");
    uint32_t status = 1;
    CHECK(fmha_mxfp8_device_status(&status) == 0 && status == 0, "device status (a bounded wait ran out)");
    std::vector<uint16_t> got(size_t(rows) * 128);
    CHECK(cudaMemcpy(got.data(), outs[rank], got.size() * 2, cudaMemcpyDeviceToHost) == cudaSuccess, "copy out");

    int rc = 0;
    if (rank == 0) {
        // the same problem on this GPU alone: one launch per key range into ohat_all[r], one combine over splits = world
        void *ohat_all = nullptr, *lse_all = nullptr, *out1 = nullptr;
        CHECK(cudaMalloc(&ohat_all, size_t(world) * rows * 512) == cudaSuccess && cudaMalloc(&lse_all, size_t(world) * rows * 4) == cudaSuccess &&
                  cudaMalloc(&out1, size_t(rows) * 256) == cudaSuccess, "cudaMalloc(reference form)");
        for (int r = 0; r < world; ++r) {
            Dev d = mine;
            Dev other;
            if (r != 0) {
                CHECK(make_inputs(r, other), "input upload");
                d = other;
            }
            fmha_mxfp8_kvsplit_args b;
            fill_args(b, d, S, H, SKl, static_cast<uint8_t*>(ohat_all) + size_t(r) * rows * 512, static_cast<uint8_t*>(lse_all) + size_t(r) * rows * 4,
                      FMHA_MXFP8_FLAG_F32_PARTIALS);
            CHECK(fmha_mxfp8_launch(FMHA_MXFP8_KVSPLIT, &b, grid, nullptr) == 0, "kvsplit launch (reference form)");
        }
        CHECK(fmha_mxfp8_combine_f32(ohat_all, lse_all, out1, rows, world, nullptr) == 0, "fmha_mxfp8_combine_f32");
        std::vector<uint16_t> want(size_t(rows) * 128);
        CHECK(cudaMemcpy(want.data(), out1, want.size() * 2, cudaMemcpyDeviceToHost) == cudaSuccess, "copy out");
        size_t differ = 0, nonfinite = 0;
        for (size_t i = 0; i < want.size(); ++i) {
            differ += got[i] != want[i];
            nonfinite += (want[i] & 0x7F80u) == 0x7F80u;
        }
        if (differ == 0 && nonfinite == 0)
            std::printf("KV_SHARDED_HOST_OK world=%d S=%u SK=%u H=%u rows=%u bytes_equal=1\n", world, S, SK, H, rows);
        else {
            std::printf("KV_SHARDED_HOST_FAIL differ=%zu nonfinite=%zu of %zu\n", differ, nonfinite, want.size());
            rc = 2;
        }
        std::fflush(stdout);   // the ranks leave through _exit
    }
    // every rank's output must equal rank 0's: compared through the shared page is overkill; each rank checks it is finite and non-zero
    size_t nz = 0;
    for (uint16_t x : got) nz += (x & 0x7FFFu) != 0;
    CHECK(nz > got.size() / 2, "output looks empty");
    host_barrier(sh, 2, world);   // nobody unmaps while a peer may still store
    for (int r = 0; r < world; ++r)
        if (r != rank) fmha_mxfp8_peer_close(ptr[r]);
    host_barrier(sh, 3, world);
    fmha_mxfp8_peer_free(own);
    return rc;
}

}  // namespace

int main(int argc, char** argv) {
    const int world = argc > 1 ? std::atoi(argv[1]) : 2;
    const uint32_t S = argc > 2 ? std::atoi(argv[2]) : 1024, SK = argc > 3 ? std::atoi(argv[3]) : 4096, H = argc > 4 ? std::atoi(argv[4]) : 4;
    if (world < 2 || world > kMaxWorld || S % (128u * world) != 0 || SK % (128u * world) != 0 || H == 0) {
        std::fprintf(stderr, "usage: kv_sharded_host <world 2..8> [S, a multiple of 128 * world] [SK, a multiple of 128 * world] [H]\n");
        return 64;
    }
    Shared* sh = static_cast<Shared*>(mmap(nullptr, sizeof(Shared), PROT_READ | PROT_WRITE, MAP_SHARED | MAP_ANONYMOUS, -1, 0));
    if (sh == MAP_FAILED) return 65;
    new (sh) Shared();
    std::vector<pid_t> kids;
    for (int r = 0; r < world; ++r) {   // fork before anything touches CUDA
        const pid_t p = fork();
        if (p == 0) _exit(run_rank(r, world, S, SK, H, sh));
        kids.push_back(p);
    }
    int worst = 0;
    for (pid_t p : kids) {
        int st = 0;
        waitpid(p, &st, 0);
        const int code = WIFEXITED(st) ? WEXITSTATUS(st) : 99;
        if (code > worst) worst = code;
    }
    return worst;
}
