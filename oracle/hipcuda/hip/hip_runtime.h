// TEST INFRASTRUCTURE ONLY. A HIP runtime made of the CUDA runtime and this repository's C ABI, just large enough to build the
// reference's own MXFP8 attention harness (tests/gpu/ref_host.cpp of the reference tree, with its generated *_abi.h headers) so that it
// drives the sm_100a kernels: the reference's input generators, its packed `Args`, its generated validate() / launch() and its fp64
// `check` then score this library's output with no restated code in between.
//   hipMalloc / hipMemcpy / hipMemset / events      -> the CUDA runtime
//   hipModuleLoad                                   -> always succeeds (there is no code object to load)
//   hipModuleGetFunction(name)                      -> a handle that carries the kernel id whose fmha_mxfp8_kernel_name() is `name`;
//                                                      the vendor kernel's name (the harness's comparison slot) maps to vs128
//   hipModuleLaunchKernel(f, grid, block, extra)    -> fmha_mxfp8_launch(kernel id, the HIP_LAUNCH_PARAM_BUFFER_POINTER bytes, the
//                                                      logical grid, stream). The combine kernel's block count travels as grid x.
// Nothing in the product includes this file.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include <cuda_runtime.h>

#include "fmha_mxfp8_abi.h"

typedef cudaError_t hipError_t;
#define hipSuccess cudaSuccess
typedef void* hipModule_t;
typedef void* hipFunction_t;
typedef cudaStream_t hipStream_t;
typedef cudaEvent_t hipEvent_t;
#define hipMemcpyHostToDevice cudaMemcpyHostToDevice
#define hipMemcpyDeviceToHost cudaMemcpyDeviceToHost
#define hipMemcpyDeviceToDevice cudaMemcpyDeviceToDevice
typedef cudaMemcpyKind hipMemcpyKind;

#define HIP_LAUNCH_PARAM_BUFFER_POINTER ((void*)0x01)
#define HIP_LAUNCH_PARAM_BUFFER_SIZE ((void*)0x02)
#define HIP_LAUNCH_PARAM_END ((void*)0x03)

static inline const char* hipGetErrorString(hipError_t e) { return cudaGetErrorString(e); }
static inline hipError_t hipMalloc(void** p, size_t n) { return cudaMalloc(p, n ? n : 1); }
static inline hipError_t hipFree(void* p) { return cudaFree(p); }
static inline hipError_t hipMemcpy(void* d, const void* s, size_t n, hipMemcpyKind k) { return cudaMemcpy(d, s, n, k); }
static inline hipError_t hipMemset(void* d, int v, size_t n) { return cudaMemset(d, v, n); }
static inline hipError_t hipDeviceSynchronize() {
    const cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return e;
    uint32_t st = 0;   // a kernel that gave up a bounded wait is a failed launch for the harness
    if (fmha_mxfp8_device_status(&st) != 0 || st != 0) return cudaErrorLaunchFailure;
    return cudaSuccess;
}
static inline hipError_t hipModuleLoad(hipModule_t* m, const char*) { *m = (void*)1; return hipSuccess; }
static inline hipError_t hipModuleGetFunction(hipFunction_t* f, hipModule_t, const char* name) {
    for (int k = 0; k < 4; ++k) {
        const char* kn = fmha_mxfp8_kernel_name(k);
        if (kn && std::strcmp(kn, name) == 0) { *f = (void*)(intptr_t)(k + 1); return hipSuccess; }
    }
    if (std::strstr(name, "aiter")) { *f = (void*)(intptr_t)(FMHA_MXFP8_VS128 + 1); return hipSuccess; }   // the vendor slot: the 256-row kernel
    std::fprintf(stderr, "hipcuda: no kernel named %s\n", name);
    return cudaErrorInvalidDeviceFunction;
}
static inline hipError_t hipEventCreate(hipEvent_t* e) { return cudaEventCreate(e); }
static inline hipError_t hipEventDestroy(hipEvent_t e) { return cudaEventDestroy(e); }
static inline hipError_t hipEventRecord(hipEvent_t e, hipStream_t s = nullptr) { return cudaEventRecord(e, s); }
static inline hipError_t hipEventSynchronize(hipEvent_t e) { return cudaEventSynchronize(e); }
static inline hipError_t hipEventElapsedTime(float* ms, hipEvent_t a, hipEvent_t b) { return cudaEventElapsedTime(ms, a, b); }

static inline hipError_t hipModuleLaunchKernel(hipFunction_t f, unsigned gx, unsigned gy, unsigned gz, unsigned, unsigned, unsigned, unsigned, hipStream_t stream,
                                               void**, void** extra) {
    const int kernel = (int)(intptr_t)f - 1;
    if (kernel < 0 || kernel > 3 || !extra) return cudaErrorInvalidValue;
    const void* args = nullptr;
    size_t sz = 0;
    for (int i = 0; extra[i] != HIP_LAUNCH_PARAM_END; i += 2) {
        if (extra[i] == HIP_LAUNCH_PARAM_BUFFER_POINTER) args = extra[i + 1];
        if (extra[i] == HIP_LAUNCH_PARAM_BUFFER_SIZE) sz = *static_cast<size_t*>(extra[i + 1]);
    }
    if (!args || sz < fmha_mxfp8_kernarg_size(kernel)) {
        std::fprintf(stderr, "hipcuda: %zu bytes of kernel arguments for %s, which takes %zu\n", sz, fmha_mxfp8_kernel_name(kernel), fmha_mxfp8_kernarg_size(kernel));
        return cudaErrorInvalidValue;
    }
    const uint32_t grid[3] = {gx, gy, gz};
    const int rc = fmha_mxfp8_launch(kernel, args, grid, stream);
    if (rc != 0) {
        std::fprintf(stderr, "hipcuda: fmha_mxfp8_launch(%s) returned %d\n", fmha_mxfp8_kernel_name(kernel), rc);
        return rc < 0 ? (cudaError_t)(-rc) : cudaErrorInvalidValue;
    }
    return hipSuccess;
}
