// 1x1 float convolution (a plain GEMM: pixels x Cin times Cin x Cout) on tcgen05.mma kind::tf32 with fp32-grade
// accuracy (3xTF32), fed by TMA: no thread gathers an operand.
//
// The tensor core truncates its fp32 operands to tf32, so the raw fp32 tile that a tiled TMA load drops into shared
// memory (128 rows x 32 floats, 128-byte-swizzled: exactly the K-major layout the MMA reads) IS the head x_hi of the
// split x = x_hi + x_lo.  Four converter warps compute the remainders x_lo = x - trunc(x) into a second tile of the same
// layout (same offsets, so the swizzle never has to be undone), for the pixel tile and for the weight tile alike, and
// the MMA warp issues hi*W_hi + hi*W_lo + lo*W_hi per 8-float slice into a TMEM accumulator.
//
// One persistent CTA per SM walks (pixel tile, channel block) pairs, channel blocks innermost so that a pixel tile
// is fetched from HBM once and re-read from L2.  Warps: 0 TMA loads, 1 - 4 converters, 5 MMA issue, 6 - 21 epilogue
// (tcgen05.ld, bias, affine, relu, 128-byte-swizzled staging boxes, TMA tensor stores).  Every wait is bounded; a wait
// that gives up records a code (41 loader, 42 converters, 43 / 44 MMA thread waiting for an accumulator / a stage,
// 45 epilogue), raises the CTA's abort flag, and the CTA frees its tensor memory and returns.
#pragma once
#include "fconv_tc5.cuh"

namespace dabnn {

constexpr int FG_N = 128;                      // largest channel block (the accumulators lie FG_N columns apart)
constexpr int FG_CHUNK = 32;                   // floats of K per stage: one 128-byte row
constexpr int FG_CONVERTERS = 128, FG_EPILOGUE = 512;
constexpr int FG_THREADS = 32 + FG_CONVERTERS + 32 + FG_EPILOGUE;
constexpr int FG_MMA_WARP = 1 + FG_CONVERTERS / 32;
constexpr int FG_EPI_WARP0 = FG_MMA_WARP + 1;
constexpr int FG_ACCS = 4;
constexpr int FG_TILE_BYTES = 128 * 128;       // 128 rows x 32 floats
constexpr int FG_STAGE_BYTES = 4 * FG_TILE_BYTES;   // pixels hi, pixels lo, weights hi, weights lo
constexpr int FG_MAX_STAGES = 3;

// K-major SWIZZLE_128B shared-memory descriptor: rows of 128 bytes, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t fg_desc_sw128(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}

__host__ __device__ inline int fg_smem_bytes(int stages) { return 1024 + stages * FG_STAGE_BYTES + 2 * FG_TILE_BYTES; }

__global__ void __launch_bounds__(FG_THREADS, 1)
    fconv_gemm_kernel(const FconvParams p, const int M, const int stages, const int n_blk, const __grid_constant__ CUtensorMap a_map,
                      const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap wr_map, const __grid_constant__ CUtensorMap out_map) {
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) uint64_t bar_loaded[FG_MAX_STAGES], bar_ready[FG_MAX_STAGES], bar_empty[FG_MAX_STAGES];
    __shared__ __align__(8) uint64_t bar_acc_full[FG_ACCS], bar_acc_empty[FG_ACCS];
    __shared__ uint32_t tmem_base_s;
    __shared__ int s_abort, epi_abort;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    unsigned char* stage0 = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
    unsigned char* stile = stage0 + stages * FG_STAGE_BYTES;
    const volatile int* abort_flag = &s_abort;
    const int K = p.cin, nchunks = K / FG_CHUNK;
    // n_blk: channels per work item (32, 64 or 128: small when there are few pixel tiles, so that every SM gets work)
    const int tiles_m = (M + 127) / 128, nblocks = (p.cout + n_blk - 1) / n_blk;
    const uint32_t w_bytes = (uint32_t)n_blk * 128u;   // a weight tile of a stage
    const int nitems = tiles_m * nblocks;
    constexpr int TMEM_COLS = FG_ACCS * FG_N;

    if (warp == FG_MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    if (tid == 0) {
        for (int i = 0; i < stages; i++) { mbar_init(&bar_loaded[i], 1); mbar_init(&bar_ready[i], FG_CONVERTERS / 32); mbar_init(&bar_empty[i], 1); }
        for (int i = 0; i < FG_ACCS; i++) { mbar_init(&bar_acc_full[i], 1); mbar_init(&bar_acc_empty[i], FG_EPILOGUE / 32); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::);
        s_abort = 0;
        epi_abort = 0;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;
    grid_launch_dependents();
    grid_dependency_wait();

    if (warp == 0) {
        // =========================== TMA loads: one lane ===========================
        if (lane == 0) {
            const uint32_t stage0_addr = smem_u32(stage0);
            uint32_t s = 0, use = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < nitems && ok; item += gridDim.x) {
                const int tile = item / nblocks, nb = item - tile * nblocks;
                for (int c = 0; c < nchunks; c++) {
                    if (use >= 1 && !mbar_wait<32>(&bar_empty[s], (use - 1) & 1, abort_flag)) {
                        atomicCAS(&g_tc5_status, 0, 41);
                        s_abort = 1;
                        ok = false;
                        break;
                    }
                    const uint32_t bar = smem_u32(&bar_loaded[s]), sa = stage0_addr + s * FG_STAGE_BYTES;
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(FG_TILE_BYTES + (p.wgt_rem ? 2u : 1u) * w_bytes) : "memory");
                    // rows beyond M / beyond Cout read as zeros; a load always delivers its whole box
                    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                                 ::"r"(sa), "l"(reinterpret_cast<uint64_t>(&a_map)), "r"(c * FG_CHUNK), "r"(tile * 128), "r"(bar) : "memory");
                    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                                 ::"r"(sa + 2 * FG_TILE_BYTES), "l"(reinterpret_cast<uint64_t>(&w_map)), "r"(c * FG_CHUNK), "r"(nb * n_blk), "r"(bar) : "memory");
                    if (p.wgt_rem)   // the weights' remainders were computed once, ahead of the launch
                        asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                                     ::"r"(sa + 3 * FG_TILE_BYTES), "l"(reinterpret_cast<uint64_t>(&wr_map)), "r"(c * FG_CHUNK), "r"(nb * n_blk), "r"(bar) : "memory");
                    if (++s == (uint32_t)stages) { s = 0; use++; }
                }
            }
        }
    } else if (warp < FG_MMA_WARP) {
        // =========================== converters: the remainders of both tiles ===========================
        const int ct = tid - 32;
        const uint32_t stage0_addr = smem_u32(stage0);
        uint32_t s = 0, par = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < nitems && ok; item += gridDim.x)
            for (int c = 0; c < nchunks; c++) {
                if (!__all_sync(0xffffffffu, mbar_wait<32>(&bar_loaded[s], par, abort_flag))) {
                    atomicCAS(&g_tc5_status, 0, 42);
                    s_abort = 1;
                    ok = false;
                    break;
                }
                const uint32_t sa = stage0_addr + s * FG_STAGE_BYTES;
                // 16-byte unit u of a hi tile -> the same unit of its lo tile (identical layouts)
#pragma unroll
                for (int half = 0; half < (p.wgt_rem ? 1 : 2); half++) {
                    const uint32_t hi0 = sa + half * 2 * FG_TILE_BYTES + ct * 16, lo0 = hi0 + FG_TILE_BYTES;
                    // eight units per thread and tile, their loads issued together (the shared-memory accesses are ordered
                    // as written: one load, one store at a time would pay the load's latency eight times)
                    constexpr int UNITS = FG_TILE_BYTES / 16 / FG_CONVERTERS;
                    float4 v[UNITS];
#pragma unroll
                    for (int j = 0; j < UNITS; j++)
                        if (half == 0 || (uint32_t)(j * FG_CONVERTERS * 16) < w_bytes) v[j] = lds128f(hi0 + j * FG_CONVERTERS * 16);   // a weight tile has n_blk rows
#pragma unroll
                    for (int j = 0; j < UNITS; j++) {
                        if (half == 1 && (uint32_t)(j * FG_CONVERTERS * 16) >= w_bytes) break;
                        uint32_t h, l0, l1, l2, l3;
                        split_tf32(v[j].x, h, l0); split_tf32(v[j].y, h, l1); split_tf32(v[j].z, h, l2); split_tf32(v[j].w, h, l3);
                        sts128(lo0 + j * FG_CONVERTERS * 16, l0, l1, l2, l3);
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_ready[s]);
                if (++s == (uint32_t)stages) { s = 0; par ^= 1u; }
            }
    } else if (warp == FG_MMA_WARP) {
        // =========================== MMA issue: one lane ===========================
        if (lane == 0) {
            const uint32_t idesc_m = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(128 >> 4) << 24);   // D f32, A = B = tf32, K-major, M = 128
            const uint64_t d_stage = fg_desc_sw128(smem_u32(stage0));
            constexpr uint32_t TILE_UNITS = FG_TILE_BYTES >> 4, STAGE_UNITS = FG_STAGE_BYTES >> 4;
            uint32_t s = 0, par = 0;
            bool ok = true;
            int i = 0;
            for (int item = blockIdx.x; item < nitems && ok; item += gridDim.x, i++) {
                const int nb = item % nblocks;
                const int n_mma = (min(n_blk, p.cout - nb * n_blk) + 15) & ~15;   // weight rows beyond Cout read as zeros
                const uint32_t idesc = idesc_m | ((uint32_t)(n_mma >> 3) << 17);
                const int accbuf = i % FG_ACCS, accuse = i / FG_ACCS;
                if (accuse >= 1 && !mbar_wait(&bar_acc_empty[accbuf], (accuse - 1) & 1, abort_flag)) {
                    atomicCAS(&g_tc5_status, 0, 43);
                    s_abort = 1;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + accbuf * FG_N;
                uint32_t accum = 0;
                for (int c = 0; c < nchunks; c++) {
                    if (!mbar_wait(&bar_ready[s], par, abort_flag)) {
                        atomicCAS(&g_tc5_status, 0, 44);
                        s_abort = 1;
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t ah = d_stage + (uint64_t)(s * STAGE_UNITS), al = ah + TILE_UNITS, wh = ah + 2 * TILE_UNITS, wl = ah + 3 * TILE_UNITS;
#pragma unroll
                    for (int j = 0; j < FG_CHUNK / 8; j++) {   // 8 floats = 32 bytes along the swizzled row
                        mma_tf32_ss(d_tmem, ah + 2 * j, wh + 2 * j, idesc, j ? 1u : accum);
                        mma_tf32_ss(d_tmem, ah + 2 * j, wl + 2 * j, idesc, 1u);
                        mma_tf32_ss(d_tmem, al + 2 * j, wh + 2 * j, idesc, 1u);
                    }
                    accum = 1u;
                    umma_commit(&bar_empty[s]);
                    if (++s == (uint32_t)stages) { s = 0; par ^= 1u; }
                }
                if (ok) umma_commit(&bar_acc_full[accbuf]);
            }
        }
    } else {
        // =========================== epilogue: 64 channels at a time through two staging boxes ===========================
        const int ew = warp - FG_EPI_WARP0, et = tid - FG_EPI_WARP0 * 32;
        const int r = (warp & 3) * 32 + lane, hq = ew >> 2;   // TMEM lane quarter of a warp = warp % 4; 16-channel quarter of the block
        const uint32_t stile_addr = smem_u32(stile);
        int i = 0;
        bool alive = true;
        for (int item = blockIdx.x; item < nitems && alive; item += gridDim.x, i++) {
            const int tile = item / nblocks, nb = item - tile * nblocks;
            const int n0 = nb * n_blk, n_this = min(n_blk, p.cout - n0);
            const int accbuf = i % FG_ACCS, accuse = i / FG_ACCS;
            const bool okw = __all_sync(0xffffffffu, mbar_wait<200>(&bar_acc_full[accbuf], accuse & 1, abort_flag));   // warp-uniform
            if (!okw) {
                atomicCAS(&g_tc5_status, 0, 45);
                s_abort = 1;
                epi_abort = 1;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int nblk64 = (n_this + 63) >> 6;
            for (int blk = 0; blk < nblk64; blk++) {
                const int cb = blk * 64, width = min(64, n_this - cb);
                const bool mine = width > hq * 16;
                uint32_t v[16];
                if (okw && mine) {
                    const int c0 = cb + hq * 16;
                    const uint32_t t_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + accbuf * FG_N + c0;
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                                   "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                                 : "r"(t_addr));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int q = 0; q < 4; q++) {   // channel constants four at a time (Cout is a multiple of four)
                        const int ch = min(n0 + c0 + q * 4, p.cout - 4);   // columns beyond Cout are clipped by the store
                        float4 kb = make_float4(0.f, 0.f, 0.f, 0.f), ka = kb, kc = kb;
                        if (p.bias) kb = __ldg(reinterpret_cast<const float4*>(p.bias + ch));
                        if (p.a) { ka = __ldg(reinterpret_cast<const float4*>(p.a + ch)); kc = __ldg(reinterpret_cast<const float4*>(p.b + ch)); }
                        const float b4[4] = {kb.x, kb.y, kb.z, kb.w}, a4[4] = {ka.x, ka.y, ka.z, ka.w}, c4[4] = {kc.x, kc.y, kc.z, kc.w};
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            float f = __uint_as_float(v[q * 4 + e]);
                            if (p.bias) f = __fadd_rn(f, b4[e]);
                            if (p.a) f = __fadd_rn(__fmul_rn(a4[e], f), c4[e]);
                            if (p.relu) f = relu_ref(f);
                            v[q * 4 + e] = __float_as_uint(f);
                        }
                    }
                }
                if (blk == nblk64 - 1 && okw) {   // the accumulator is in registers: the MMA warp may reuse it
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bar_acc_empty[accbuf]);
                }
                if (et == 0 || et == 32) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the previous block's stores have read the boxes
                asm volatile("bar.sync 1, %0;" ::"n"(FG_EPILOGUE) : "memory");
                if (epi_abort) { alive = false; break; }
                if (mine) {
#pragma unroll
                    for (int q = 0; q < 4; q++)
                        sts128(stile_addr + (hq >> 1) * FG_TILE_BYTES + r * 128 + ((((hq & 1) * 4 + q) ^ (r & 7)) << 4), v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the tensor stores below read what was just written
                }
                asm volatile("bar.sync 1, %0;" ::"n"(FG_EPILOGUE) : "memory");
                // one tensor store per 32-channel box: pixels beyond M and channels beyond Cout are clipped
                if (et == 0 || (et == 32 && width > 32)) {
                    const int hb = et >> 5;
                    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                                 ::"l"(reinterpret_cast<uint64_t>(&out_map)), "r"(n0 + cb + hb * 32), "r"(tile * 128), "r"(stile_addr + hb * FG_TILE_BYTES) : "memory");
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
            }
        }
    }

    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // the stores are complete before the CTA winds down
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == FG_MMA_WARP) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS));
    }
}

}  // namespace dabnn
