// Stand-in for the HIP runtime, just large enough to compile the reference's MXFP8 attention harness
// (tests/gpu/ref_host.cpp of the reference tree, together with its generated *_abi.h headers) on a machine
// without ROCm. TEST INFRASTRUCTURE ONLY: device memory is host memory, module loading always succeeds and
// a kernel launch computes nothing. So the harness's own input generators, host-contract validation and
// fp64 `check` run unchanged, which is what the oracle is pinned against.
//
// One hook: when the environment variable HIPSTUB_OUT names a file, the first 656-byte launch (the harness's
// "vendor kernel" slot) copies that file's bytes into the output buffer (kernel argument 0x000). This lets a
// candidate bf16 output be scored by the reference's own `check`.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>

typedef int hipError_t;
#define hipSuccess 0
typedef void* hipModule_t;
typedef void* hipFunction_t;
typedef void* hipStream_t;
typedef void* hipEvent_t;
enum hipMemcpyKind { hipMemcpyHostToDevice = 1, hipMemcpyDeviceToHost = 2, hipMemcpyDeviceToDevice = 3 };

struct dim3 {
    unsigned x, y, z;
    dim3(unsigned x_ = 1, unsigned y_ = 1, unsigned z_ = 1) : x(x_), y(y_), z(z_) {}
};

#define HIP_LAUNCH_PARAM_BUFFER_POINTER ((void*)0x01)
#define HIP_LAUNCH_PARAM_BUFFER_SIZE ((void*)0x02)
#define HIP_LAUNCH_PARAM_END ((void*)0x03)

static inline const char* hipGetErrorString(hipError_t) { return "hipstub"; }
static inline hipError_t hipMalloc(void** p, size_t n) { *p = std::calloc(n ? n : 1, 1); return *p ? hipSuccess : 1; }
static inline hipError_t hipFree(void* p) { std::free(p); return hipSuccess; }
static inline hipError_t hipMemcpy(void* d, const void* s, size_t n, hipMemcpyKind) { std::memcpy(d, s, n); return hipSuccess; }
static inline hipError_t hipMemset(void* d, int v, size_t n) { std::memset(d, v, n); return hipSuccess; }
static inline hipError_t hipDeviceSynchronize() { return hipSuccess; }
static inline hipError_t hipModuleLoad(hipModule_t* m, const char*) { *m = (void*)1; return hipSuccess; }
static inline hipError_t hipModuleGetFunction(hipFunction_t* f, hipModule_t, const char*) { *f = (void*)1; return hipSuccess; }
static inline hipError_t hipEventCreate(hipEvent_t* e) { *e = nullptr; return hipSuccess; }
static inline hipError_t hipEventDestroy(hipEvent_t) { return hipSuccess; }
static inline hipError_t hipEventRecord(hipEvent_t, hipStream_t = nullptr) { return hipSuccess; }
static inline hipError_t hipEventSynchronize(hipEvent_t) { return hipSuccess; }
static inline hipError_t hipEventElapsedTime(float* ms, hipEvent_t, hipEvent_t) { *ms = 1.0f; return hipSuccess; }

static inline hipError_t hipModuleLaunchKernel(hipFunction_t, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, hipStream_t,
                                               void**, void** extra) {
    static bool used = false;
    const char* path = std::getenv("HIPSTUB_OUT");
    if (!path || used || !extra) return hipSuccess;
    unsigned char* args = nullptr;
    size_t sz = 0;
    for (int i = 0; extra[i] != HIP_LAUNCH_PARAM_END; i += 2) {
        if (extra[i] == HIP_LAUNCH_PARAM_BUFFER_POINTER) args = static_cast<unsigned char*>(extra[i + 1]);
        if (extra[i] == HIP_LAUNCH_PARAM_BUFFER_SIZE) sz = *static_cast<size_t*>(extra[i + 1]);
    }
    if (!args || sz != 656) return hipSuccess;
    used = true;
    void* out;
    std::memcpy(&out, args, 8);
    if (FILE* fp = std::fopen(path, "rb")) {
        std::fseek(fp, 0, SEEK_END);
        const long n = std::ftell(fp);
        std::fseek(fp, 0, SEEK_SET);
        if (n > 0 && std::fread(out, 1, (size_t)n, fp) != (size_t)n) std::fprintf(stderr, "hipstub: short read of %s\n", path);
        std::fclose(fp);
    }
    return hipSuccess;
}
