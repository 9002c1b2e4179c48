// Register-resident peak rate of one contraction instruction: the roofline denominator for the
// binary contraction.  NVIDIA publishes no 1-bit figure for B200, so it is measured: every warp of
// a full-occupancy grid issues the instruction back to back on eight independent accumulators.
#include "bcontract_tc5.cuh"

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

// tcgen05.mma issued back to back by one thread per SM on fixed shared-memory operands
// (M = 128, N = 128, 32 bytes of K per instruction), alternating between two TMEM accumulators.
// KIND 0: kind::i8 (u8 x u8 -> s32), KIND 1: kind::tf32 (-> f32).  A commit + bounded wait closes
// every batch of 64 instructions so that the issue queue cannot run ahead of the timing.
template <int KIND>
__global__ void __launch_bounds__(128, 1) tcgen05_peak_kernel(int batches, int* status) {
    __shared__ __align__(1024) unsigned char ops[2 * 128 * 32];   // A then B, K-major canonical layout, one 32-byte K slice
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t tmem_base_s;
    __shared__ int s_abort;
    const int tid = threadIdx.x, warp = tid >> 5;
    for (int i = tid; i < (int)sizeof(ops) / 4; i += 128) reinterpret_cast<uint32_t*>(ops)[i] = KIND == 0 ? 0x01000101u : 0x3f800000u;
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(256));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    if (tid == 0) {
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::);
        s_abort = 0;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;
    if (tid == 0) {
        // one 32-byte K slice: two 16-byte units 128 B apart, 8-row groups 256 B apart
        auto desc = [](uint32_t saddr) {
            return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)(128 >> 4) << 16) | ((uint64_t)(256 >> 4) << 32) | ((uint64_t)1 << 46);
        };
        const uint64_t ad = desc(smem_u32(ops)), bd = desc(smem_u32(ops) + 128 * 32);
        const uint32_t idesc = KIND == 0 ? ((2u << 4) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24))
                                         : ((1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24));
        for (int b = 0; b < batches; b++) {
            for (int j = 0; j < 64; j++) {
                const uint32_t d_tmem = tmem_base + (j & 1) * 128, accum = (b | (j >> 1)) ? 1u : 0u;
                if (KIND == 0)
                    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                                 "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}\n"
                                 ::"r"(d_tmem), "l"(ad), "l"(bd), "r"(idesc), "r"(accum), "r"(0), "r"(0), "r"(0), "r"(0) : "memory");
                else
                    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}\n"
                                 ::"r"(d_tmem), "l"(ad), "l"(bd), "r"(idesc), "r"(accum), "r"(0), "r"(0), "r"(0), "r"(0) : "memory");
            }
            umma_commit(&bar);
            if (!mbar_wait(&bar, b & 1, &s_abort)) { atomicCAS(status, 0, 1); break; }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256));
}

}  // namespace dabnn

using namespace dabnn;

// seconds per launch of the tcgen05 issue loop (best of three after a warm-up), or < 0 on failure
static double time_tcgen05_peak(int kind, int batches) {
    int* status = nullptr;
    if (cudaMalloc(&status, sizeof(int)) != cudaSuccess) return -1.0;
    cudaMemset(status, 0, sizeof(int));
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0); cudaEventCreate(&e1);
    float best = 1e30f;
    for (int rep = 0; rep < 4; rep++) {
        cudaEventRecord(e0);
        if (kind == 0) tcgen05_peak_kernel<0><<<sm_count(), 128>>>(batches, status);
        else tcgen05_peak_kernel<1><<<sm_count(), 128>>>(batches, status);
        cudaEventRecord(e1);
        cudaEventSynchronize(e1);
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        if (rep > 0 && ms < best) best = ms;
    }
    int h = 0;
    cudaMemcpy(&h, status, sizeof(int), cudaMemcpyDeviceToHost);
    const cudaError_t err = cudaGetLastError();
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    cudaFree(status);
    return (err != cudaSuccess || h != 0) ? -1.0 : best * 1e-3;
}

extern "C" int dabnn_measure_engine_peak(int engine, double* bitops_per_second) {
    DABNN_REQUIRE(bitops_per_second, DABNN_ERR_ARG, "null output");
    DABNN_REQUIRE(engine >= DABNN_ENGINE_POPC && engine <= DABNN_ENGINE_TCGEN05, DABNN_ERR_ARG, "engine must be POPC, B1, IMMA or TCGEN05");
    if (engine == DABNN_ENGINE_TCGEN05) {
        const int batches = 400;
        const double sec = time_tcgen05_peak(0, batches);
        if (sec <= 0.0) return fail(DABNN_ERR_CUDA, "tcgen05 peak kernel failed");
        *bitops_per_second = 2.0 * 128 * 128 * 32 * 64.0 * batches * sm_count() / sec;
        return DABNN_OK;
    }
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

extern "C" int dabnn_measure_tf32_peak(double* flops_per_second) {
    DABNN_REQUIRE(flops_per_second, DABNN_ERR_ARG, "null output");
    const int batches = 400;
    const double sec = time_tcgen05_peak(1, batches);
    if (sec <= 0.0) return fail(DABNN_ERR_CUDA, "tcgen05 peak kernel failed");
    *flops_per_second = 2.0 * 128 * 128 * 8 * 64.0 * batches * sm_count() / sec;
    return DABNN_OK;
}
