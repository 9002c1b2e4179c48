// Register-resident peak rate of one contraction instruction: the roofline denominator for the
// binary contraction.  NVIDIA publishes no 1-bit figure for B200, so it is measured: every warp of
// a full-occupancy grid issues the instruction back to back on eight independent accumulators.
#include "bcontract.cuh"

namespace dabnn {

template <int ENGINE>
__global__ void __launch_bounds__(256) engine_peak_kernel(const uint32_t* __restrict__ in, int* out, int iters) {
    uint32_t a0 = in[threadIdx.x], a1 = in[threadIdx.x + 256], a2 = in[threadIdx.x + 512], a3 = in[threadIdx.x + 768];
    const uint32_t b0 = in[threadIdx.x + 1024], b1 = in[threadIdx.x + 1280];
    int d[8][4];
#pragma unroll
    for (int i = 0; i < 8; i++) d[i][0] = d[i][1] = d[i][2] = d[i][3] = i;
    for (int it = 0; it < iters; it++) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
            if (ENGINE == ENG_B1) {
                mma_b1_and(d[i], a0, a1, a2, a3, b0, b1);
            } else if (ENGINE == ENG_IMMA) {
                mma_u8(d[i], a0, a1, a2, a3, b0, b1);
            } else {  // four dependent-free xor+popc+add per slot; a* change so nothing can be hoisted
                d[i][0] += __popc(a0 ^ b0);
                d[i][1] += __popc(a1 ^ b1);
                d[i][2] += __popc(a2 ^ b0);
                d[i][3] += __popc(a3 ^ b1);
                a0 += 0x9e3779b9u; a1 += 0x7f4a7c15u; a2 += 0x85ebca6bu; a3 += 0xc2b2ae35u;
            }
        }
    }
    int s = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) s += d[i][0] + d[i][1] + d[i][2] + d[i][3];
    if (s == 0x7fffffff) out[0] = s;  // keeps the loop alive without a store on the hot path
}

}  // namespace dabnn

using namespace dabnn;

extern "C" int dabnn_measure_engine_peak(int engine, double* bitops_per_second) {
    DABNN_REQUIRE(bitops_per_second, DABNN_ERR_ARG, "null output");
    DABNN_REQUIRE(engine >= DABNN_ENGINE_POPC && engine <= DABNN_ENGINE_IMMA, DABNN_ERR_ARG, "engine must be POPC, B1 or IMMA");
    uint32_t host[2048];
    for (int i = 0; i < 2048; i++) host[i] = (uint32_t)i * 2654435761u;
    uint32_t* in = nullptr;
    int* out = nullptr;
    DABNN_CUDA_OK(cudaMalloc(&in, sizeof(host)));
    if (cudaMalloc(&out, 64) != cudaSuccess) { cudaFree(in); return fail(DABNN_ERR_CUDA, "cudaMalloc failed"); }
    cudaMemcpy(in, host, sizeof(host), cudaMemcpyHostToDevice);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0); cudaEventCreate(&e1);
    const int grid = sm_count() * 4, iters = engine == DABNN_ENGINE_B1 ? 2000 : 8000;
    // bit-ops per thread per iteration per accumulator slot: an MMA is 2*m*n*k shared by 32 lanes
    const double ops = engine == DABNN_ENGINE_B1 ? 2.0 * 16 * 8 * 256 / 32 : engine == DABNN_ENGINE_IMMA ? 2.0 * 16 * 8 * 32 / 32 : 4 * 64.0;
    float best = 1e30f;
    for (int rep = 0; rep < 4; rep++) {  // rep 0 warms up
        cudaEventRecord(e0);
        if (engine == DABNN_ENGINE_B1) engine_peak_kernel<ENG_B1><<<grid, 256>>>(in, out, iters);
        else if (engine == DABNN_ENGINE_IMMA) engine_peak_kernel<ENG_IMMA><<<grid, 256>>>(in, out, iters);
        else engine_peak_kernel<ENG_POPC><<<grid, 256>>>(in, out, iters);
        cudaEventRecord(e1);
        cudaEventSynchronize(e1);
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        if (rep > 0 && ms < best) best = ms;
    }
    const cudaError_t err = cudaGetLastError();
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    cudaFree(in); cudaFree(out);
    if (err != cudaSuccess) return fail(DABNN_ERR_CUDA, cudaGetErrorString(err));
    *bitops_per_second = ops * 8.0 * iters * 256.0 * grid / (best * 1e-3);
    return DABNN_OK;
}
