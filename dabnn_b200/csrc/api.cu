// Library-wide pieces of the C ABI: error text, version, device queries.
#include <cuda.h>   // CUtensorMap and the encoder's signature (types only)

#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace dabnn {

int g_overlap_launches = 1;
static thread_local std::string g_last_error;

void set_error(const std::string& msg) { g_last_error = msg; }
int fail(int code, const std::string& msg) {
    g_last_error = msg;
    return code;
}

int sm_count() {
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

typedef CUresult (*TensorMapEncode)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static TensorMapEncode tensor_map_encoder() {
    static TensorMapEncode encode = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        cudaFree(nullptr);   // the encoder needs an initialised driver and a current context
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult st;
        if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &fn, 12000, cudaEnableDefault, &st) == cudaSuccess &&
            st == cudaDriverEntryPointSuccess)
            encode = reinterpret_cast<TensorMapEncode>(fn);
        else
            cudaGetLastError();
    });
    return encode;
}

bool make_f32_tensor_map(CUtensorMap_st* map, float* base, int rank, const unsigned long long* dims,
                         const unsigned long long* strides_bytes, const unsigned* box) {
    const TensorMapEncode encode = tensor_map_encoder();
    if (!encode || !base || rank < 2 || rank > 3) return false;
    cuuint64_t d[3], s[2];
    cuuint32_t b[3], e[3] = {1, 1, 1};
    for (int i = 0; i < rank; i++) { d[i] = dims[i]; b[i] = box[i]; }
    for (int i = 0; i + 1 < rank; i++) s[i] = strides_bytes[i];
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, (cuuint32_t)rank, base, d, s, b, e, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool make_u8_tensor_map(CUtensorMap_st* map, const unsigned char* base, int rank, const unsigned long long* dims,
                        const unsigned long long* strides_bytes, const unsigned* box) {
    const TensorMapEncode encode = tensor_map_encoder();
    if (!encode || !base || rank < 2 || rank > 5 || (box[0] != 64 && box[0] != 128)) return false;
    cuuint64_t d[5], s[4];
    cuuint32_t b[5], e[5] = {1, 1, 1, 1, 1};
    for (int i = 0; i < rank; i++) { d[i] = dims[i]; b[i] = box[i]; }
    for (int i = 0; i + 1 < rank; i++) s[i] = strides_bytes[i];
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, (cuuint32_t)rank, const_cast<unsigned char*>(base), d, s, b, e,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, box[0] == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace dabnn

extern "C" const char* dabnn_last_error(void) { return dabnn::g_last_error.c_str(); }
extern "C" int dabnn_debug_set_launch_overlap(int on) {
    dabnn::g_overlap_launches = on != 0;
    return DABNN_OK;
}
extern "C" const char* dabnn_version(void) { return "dabnn_b200 0.1 (sm_100a)"; }
extern "C" int dabnn_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}
