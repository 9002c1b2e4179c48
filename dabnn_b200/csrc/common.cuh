// Shared helpers for the CUDA side of the library: error plumbing and small device utilities.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <string>

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

inline int conv_out_dim(int in, int pad, int dil, int k, int stride) {
    return (in + 2 * pad - (dil * (k - 1) + 1)) / stride + 1;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

}  // namespace dabnn
