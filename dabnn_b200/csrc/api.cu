// Library-wide pieces of the C ABI: error text, version, device queries.
#include <mutex>

#include "common.cuh"

namespace dabnn {

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

}  // namespace dabnn

extern "C" const char* dabnn_last_error(void) { return dabnn::g_last_error.c_str(); }
extern "C" const char* dabnn_version(void) { return "dabnn_b200 0.1 (sm_100a)"; }
extern "C" int dabnn_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}
