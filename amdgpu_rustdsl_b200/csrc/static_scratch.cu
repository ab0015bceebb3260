// The KV-split path with its partials in a fixed device array instead of a caller-supplied workspace.
//
// Who needs this: the split kernel and the combine kernel talk to each other through scratch memory (partial outputs, f16 rows in an
// area the contract sizes for f32, and one base-2 log-sum-exp per row and split). The regular entry points make the caller bring that memory. Some callers have nowhere to
// get it from at the moment of the call: a serving loop whose device memory was handed out in full to its own pools at start-up, a
// callback or a thread that must not enter the CUDA allocator because cudaMalloc / cudaFree synchronise the whole device and take
// driver locks, a host runtime that plans all its buffers ahead of time and learns the split count only at dispatch. For them the
// library carries its own scratch: a file-scope __device__ array, which the CUDA module loader places once per device when this
// translation unit is first used, so that the call itself asks no allocator for anything.
//
// Limits and rules, all consequences of the array being one fixed object per device:
//   * size: splits * B * S * H  <=  kMaxRowSplits. Larger problems are refused before anything is launched.
//   * the first call on a device looks the array's address up (cudaGetSymbolAddress, which may load the module), and the first launch of
//     each kernel variant on a device sets that kernel's shared-memory attribute and may load its code. Which variant a call uses
//     depends on the problem: fewer than 512 keys or not (the two softmax recipes), and whether a trace buffer is attached. So make one
//     call of each kind you will use during start-up, outside any stream capture. After that a call only looks up two symbol addresses
//     (this array's is cached; the status word's is asked for by every launch), encodes four tensor maps on the host and launches.
//   * every call on a device uses the same bytes. Two calls that can overlap in time (different streams, or different host threads
//     on streams that are not ordered against each other) race on the partials and both get garbage. Order them.
//   * nothing in the array has to start at zero or survive between calls: each call's split kernel writes every (split, row)
//     partial that the same call's combine kernel reads, on the same stream.
#include "../../include/fmha_mxfp8_abi.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

namespace {

constexpr unsigned long long kMaxRowSplits = FMHA_MXFP8_STATIC_SCRATCH_MAX_ROW_SPLITS;
constexpr unsigned long long kOhatBytes = kMaxRowSplits * 128ull * 4ull;   // f32 [splits][rows_total][128]: 32 MiB
constexpr unsigned long long kLseBytes = kMaxRowSplits * 4ull;             // f32 [splits][rows_total]: 256 KiB

static __device__ __align__(256) unsigned char g_scratch[kOhatBytes + kLseBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
unsigned char* g_scratch_addr[kMaxDevices] = {};   // device address of g_scratch, per device ordinal, filled on first use

int refuse(char* err, size_t cap, int code, const char* msg) {
    if (err && cap) std::snprintf(err, cap, "%s", msg);
    return code;
}

// Address of this device's copy of the array; looked up once per device, with that device current (it is: we ask which one is).
int scratch_for_current_device(unsigned char** out, char* err, size_t cap) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return refuse(err, cap, -static_cast<int>(e), "cudaGetDevice failed");
    if (dev < 0 || dev >= kMaxDevices) return refuse(err, cap, FMHA_MXFP8_E_ARG, "device ordinal beyond the static scratch table");
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_scratch_addr[dev] == nullptr) {
        unsigned char* ptr = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            if (err && cap) std::snprintf(err, cap, "cudaGetSymbolAddress(static scratch) failed: %s", cudaGetErrorString(e));
            return e != cudaSuccess ? -static_cast<int>(e) : FMHA_MXFP8_E_ARG;
        }
        g_scratch_addr[dev] = ptr;
    }
    *out = g_scratch_addr[dev];
    return 0;
}

}  // namespace

extern "C" int fmha_mxfp8_kvsplit_static_scratch(const fmha_mxfp8_problem* prob, uint32_t splits, void* stream, char* err, size_t cap) {
    if (err && cap) err[0] = 0;
    if (!prob) return refuse(err, cap, FMHA_MXFP8_E_ARG, "null problem");
    if (splits == 0) splits = 4;
    if (splits != 2 && splits != 4 && splits != 8) return refuse(err, cap, FMHA_MXFP8_E_ARG, "splits must be 2, 4 or 8");
    const unsigned long long rows_total = 1ull * prob->B * prob->S * prob->H;
    if (rows_total == 0) return refuse(err, cap, FMHA_MXFP8_E_ARG, "empty problem");
    if (rows_total * splits > kMaxRowSplits) {
        if (err && cap) {
            std::snprintf(err, cap, "static scratch too small: splits * B * S * H = %llu exceeds %llu; use fmha_mxfp8_auto with a workspace of your own",
                          rows_total * splits, kMaxRowSplits);
        }
        return FMHA_MXFP8_E_EXTENT;
    }
    unsigned char* scratch = nullptr;
    const int rc = scratch_for_current_device(&scratch, err, cap);
    if (rc) return rc;
    fmha_mxfp8_problem pr = *prob;   // the caller's inputs and output as they are; only the workspace fields are ours
    pr.ws_ohat = scratch;
    pr.ws_lse = scratch + kOhatBytes;
    pr.ws_ohat_bytes = kOhatBytes;
    pr.ws_lse_bytes = kLseBytes;
    return fmha_mxfp8_auto(&pr, FMHA_MXFP8_KVSPLIT, splits, stream, nullptr, nullptr, err, cap);
}
