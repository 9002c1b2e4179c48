// Shared helpers for the CUDA side of the library: error plumbing and small device utilities.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <string>
#include <utility>

#include "../../include/dabnn_b200.h"

namespace dabnn {

// Thread-local last-error text behind dabnn_last_error().
void set_error(const std::string& msg);
int fail(int code, const std::string& msg);

#define DABNN_CUDA_OK(expr)                                                                   \
    do {                                                                                      \
        cudaError_t _e = (expr);                                                              \
        if (_e != cudaSuccess)                                                                \
            return ::dabnn::fail(DABNN_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(_e)); \
    } while (0)

#define DABNN_REQUIRE(cond, code, msg)                         \
    do {                                                       \
        if (!(cond)) return ::dabnn::fail((code), (msg));      \
    } while (0)

inline int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(DABNN_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
    return DABNN_OK;
}

// Number of SMs of the current device (cached per device).
int sm_count();

// Launches of consecutive layers overlap at their seams: a kernel launched with launch_overlapped may begin while the
// kernel before it in the stream is still draining, runs its set-up (shared memory, tensor memory, barriers, constant
// weights) and then calls grid_dependency_wait(), which returns once everything launched before it has completed and is
// visible.  Only kernels that make that call before they touch activations may be launched this way.
extern int g_overlap_launches;   // 1 (default): on; dabnn_debug_set_launch_overlap
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Lets the kernel that follows in the stream (if it was launched with launch_overlapped) start as soon as every CTA of
// this grid has made the call: its CTAs take the SMs this grid leaves free and run their own set-up while this grid
// still computes; their grid_dependency_wait() still holds them until this grid has completed.  For kernels whose
// whole grid is resident at once (one persistent CTA per SM): a grid with CTAs still waiting for an SM would have to
// share it with the newcomers.
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
template <class... KArgs, class... Args>
inline cudaError_t launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_overlap_launches ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

inline int conv_out_dim(int in, int pad, int dil, int k, int stride) {
    return (in + 2 * pad - (dil * (k - 1) + 1)) / stride + 1;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
// Shared-memory accesses by 32-bit shared address.  A pointer into dynamic shared memory that went through an
// integer round trip (alignment) is a generic pointer to the compiler, and generic loads and stores to shared
// memory cost the shared-memory pipe several times the wavefronts of ld.shared / st.shared.
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
__device__ __forceinline__ void sts128f(uint32_t addr, float x, float y, float z, float w) {
    asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(x), "f"(y), "f"(z), "f"(w) : "memory");
}
__device__ __forceinline__ float lds_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ float4 lds128f(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}

}  // namespace dabnn
