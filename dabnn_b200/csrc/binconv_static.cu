// dabnn_binconv_forward_static: the BinConv operator for callers that are not allowed to allocate.
//
// Some hosts of this library hand every byte of device memory to their own allocator at start-up,
// or call into it from places where cudaMalloc is forbidden or would stall (a serving loop with a
// latency budget, a plugin callback of another runtime).  They cannot provide the workspace that
// dabnn_binconv_forward needs, and they cannot let the library allocate one.  For them the
// intermediate bit tensor lives in a fixed array inside the library's own device image.
//
// The array's name is only a host-side handle: kernels must be given the device address, which
// cudaGetSymbolAddress returns for the device that is current at the time of the call.  The lookup
// is done once per device, by the first call made with that device current, and cached.
#include <mutex>

#include "common.cuh"

namespace {

constexpr size_t kStaticScratchBytes = DABNN_BINCONV_STATIC_BYTES;  // held by every device that loads the library
static __device__ __align__(256) unsigned char g_binconv_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_lock;
void* g_scratch_addr[kMaxDevices];  // device address of g_binconv_scratch, per device ordinal

// Device address of the scratch array on the current device (resolved on first use).
int scratch_for_current_device(void** out) {
    int dev = 0;
    DABNN_CUDA_OK(cudaGetDevice(&dev));
    DABNN_REQUIRE(dev >= 0 && dev < kMaxDevices, DABNN_ERR_ARG, "device ordinal out of range");
    std::lock_guard<std::mutex> guard(g_lock);
    if (!g_scratch_addr[dev]) {
        void* p = nullptr;
        DABNN_CUDA_OK(cudaGetSymbolAddress(&p, g_binconv_scratch));
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return DABNN_OK;
}

}  // namespace

extern "C" int dabnn_binconv_forward_static(const float* in, const uint64_t* weight, size_t weight_words,
                                            float* out, int n, int h, int w, int cin, int cout, int kh, int kw,
                                            int pad_h, int pad_w, int stride_h, int stride_w, int engine,
                                            dabnn_stream_t s) {
    const size_t need = dabnn_binconv_workspace_bytes(n, h, w, cin, kh, kw, pad_h, pad_w, stride_h, stride_w);
    DABNN_REQUIRE(need > 0, DABNN_ERR_SHAPE, "binconv_forward_static: empty problem");
    if (need > kStaticScratchBytes)
        return dabnn::fail(DABNN_ERR_SHAPE, "binconv_forward_static: this shape needs " + std::to_string(need) +
                                                " bytes of scratch, the built-in buffer holds " +
                                                std::to_string(kStaticScratchBytes) +
                                                "; split the batch or use dabnn_binconv_forward with a workspace");
    void* scratch = nullptr;
    const int rc = scratch_for_current_device(&scratch);
    if (rc) return rc;
    // every word of the scratch that the convolution reads is written first by the packing step of
    // this same call, so nothing has to be cleared between calls
    return dabnn_binconv_forward(in, weight, weight_words, out, n, h, w, cin, cout, kh, kw, pad_h, pad_w, stride_h,
                                 stride_w, scratch, kStaticScratchBytes, engine, s);
}
