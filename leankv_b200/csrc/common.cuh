// Shared helpers for the leankv_b200 kernels (sm_100a only).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "leankv_b200.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "leankv_b200 kernels are written for sm_100a"
#endif

namespace leankv {

// Records a failing CUDA call for leankv_last_cuda_error() and maps it to LEANKV_ECUDA.
int note_cuda_error(cudaError_t e, const char* what);

#define LEANKV_CUDA_TRY(expr)                                              \
    do {                                                                   \
        cudaError_t _e = (expr);                                           \
        if (_e != cudaSuccess) return ::leankv::note_cuda_error(_e, #expr); \
    } while (0)

// Number of SMs of the current device (cached per device id).
int sm_count();

// Whether launches carry the programmatic-stream-serialization attribute (default on; the
// environment variable LEANKV_PDL=0 turns it off).
bool pdl_enabled();
// LEANKV_PDL: 0 = never, 1 = every kernel may start early, 2 (default) = only the bandwidth-bound
// GEMV kernels may (their ramp-up is what is worth hiding; small latency-bound kernels run best alone).
int pdl_mode();

// Launch `kernel` on `st`, allowing it to overlap its start-up with the tail of the previous
// kernel in the stream (see pdl_begin()).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel_ex(bool early_ok, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                    cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    const int mode = pdl_mode();
    cfg.numAttrs = (mode == 1 || (mode == 2 && early_ok)) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
// The same for a grid of thread-block clusters of `cluster` CTAs (every grid dimension a multiple of the
// cluster's).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_cluster_kernel_ex(bool early_ok, dim3 cluster, void (*kernel)(KArgs...), dim3 grid,
                                            dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster.x;
    attr[0].val.clusterDim.y = cluster.y;
    attr[0].val.clusterDim.z = cluster.z;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    const int mode = pdl_mode();
    cfg.numAttrs = (mode == 1 || (mode == 2 && early_ok)) ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                 Args&&... args) {
    return launch_kernel_ex(false, kernel, grid, block, smem, st, static_cast<Args&&>(args)...);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// 16-byte streaming load that does not allocate in L1 (weights are read exactly once).
__device__ __forceinline__ uint4 ld_stream_16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// L2-coherent 4-byte load for data written by other CTAs of the same grid.
__device__ __forceinline__ float ld_cg_f32(const float* p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ float4 ld_cg_f32x4(const float* p) {
    float4 v;
    asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(p));
    return v;
}

// Programmatic dependent launch: a kernel first lets the next kernel in the stream start
// launching (its CTAs become resident and run up to their own pdl_wait), then waits until every
// kernel before it has completed and its writes are visible. Nothing that depends on, or is read
// by, an earlier kernel may be touched before pdl_wait(). Both are no-ops for a normal launch.
__device__ __forceinline__ void pdl_begin() {
#ifdef LEANKV_PDL_TRIGGER_FIRST
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
#else
    // wait first: when a dependent starts early, everything before its immediate predecessor is
    // complete and visible, and at most one kernel sits waiting behind the running one
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
#endif
}

__device__ __forceinline__ float2 h2_to_f2(uint32_t packed) {
    return __half22float2(*reinterpret_cast<const __half2*>(&packed));
}

}  // namespace leankv
