// Binary convolution on activations kept as {0,1} bytes: TMA feeds tcgen05.mma kind::i8 directly.
//
// The engine in bcontract_tc5.cuh reads packed bits and spends its time expanding them to bytes in shared
// memory with eight producer warps.  Here the layer that produces an activation also writes it as one byte per
// channel (NHWC, 8x the packed size, a quarter of the fp32 copy that is written anyway), and then the pixel
// operand of a convolution tap is a rectangle of that tensor: for a tile of whole output rows,
//
//   A_tap[(row, ow)][c] = x8[img][row * s + ky - pad][ow * s + kx - pad][c]     (zero outside the image),
//
// which is one tiled TMA load per tap and 64-channel group, 64-byte-swizzled, landing in exactly the K-major
// layout tcgen05.mma reads.  Zero fill outside the image is the reference's padding (bit 0).  No thread touches
// the operand: one lane issues the loads, one lane issues the MMAs, the other warps are the epilogue.
//
//   cnt[p][n] = sum_k a_k xor b_k = sum_k a_k * (1 - 2 b_k) + sum_k b_k
//
// with a the activation bits as unsigned bytes {0,1} and the weights stored as signed bytes 1 - 2b = {+1,-1}: the
// MMA (unsigned x signed 8-bit, s32 accumulators) yields the first sum and the epilogue adds the weight row's
// popcount.  A zero-filled tap contributes b_k, the reference's count for a padded position.
//
// Tiles: OW <= 128.  If an image has more than 128 output pixels a tile is `rows` whole output rows of one image
// (rows * OW <= 128), else `imgs` whole images.  The M = 128 rows of the MMA beyond the tile's pixels hold stale
// bytes; their accumulator lanes are never read.  The input's tensor map has five dimensions (c, w, h, image,
// column parity): stride 1 uses parity 0 only; stride 2 views W as (W / 2, parity) and folds the row parity into
// the base address (two tensor maps), so that a tap is still a dense box.
//
// Where the weights are streamed, a unit of work is a pair of pixel tiles (M = 2 x 128) that share every weight
// stage, each with its own accumulator: half the weight bytes per MMA.
//
// Weights: expanded once (bconv_u8_expand_weights_kernel) into per-(channel block, K box) images in the
// SWIZZLE_NONE K-major core-matrix layout, streamed per stage by one bulk copy - or, when a channel block's
// weights are small (the 64-channel layers: 45 KB), loaded once per CTA and kept in shared memory, which takes
// them off the L2 -> shared-memory path that bounds this kernel.
//
// Every wait is bounded; a wait that gives up records a code in a status word, raises the CTA's abort flag,
// and the CTA frees its tensor memory and returns.
#pragma once
#include "bcontract_tc5.cuh"

namespace dabnn {

constexpr int U8_BOX_BYTES = 128 * 64;       // one K box of the pixel operand: 128 rows x 64 bytes
constexpr int U8_ACCS = 4;                   // TMEM accumulators of up to 128 columns
constexpr int U8_EPI_WARPS = 16;
constexpr int U8_EPILOGUE = U8_EPI_WARPS * 32;
constexpr int U8_THREADS = 64 + U8_EPILOGUE;  // warp 0: loads, warp 1: MMA, then the epilogue warps
// Staging tile of a 64-channel block: two boxes of (a tile's pixels, rounded up to 8) x 32 channels of fp32, 128-byte-swizzled.
__host__ __device__ inline int u8_staging_rows(int tile_pixels) { return (tile_pixels + 7) & ~7; }
__host__ __device__ inline int u8_staging_tile_bytes(int tile_pixels) { return 2 * u8_staging_rows(tile_pixels) * 128; }
constexpr int U8_MAX_STILES = 6;             // staging tiles: one being drained and stored, the others being prefetched
constexpr int U8_MAX_SMEM = 227 * 1024;

__device__ int g_u8_status;   // 0 = ok; 21 loader, 22 MMA (accumulator), 23 MMA (stage), 24 epilogue

struct U8Params {
    const unsigned char* w_img;   // expanded weights (bconv_u8_expand_weights_kernel)
    const float *a, *b;           // per-channel affine (both or neither)
    const float* shortcut;        // fp32 [M][N] added after the affine, or null
    float* out;                   // fp32 [M][N] or null
    unsigned char* out_u8;        // {0,1} bytes [M][N] or null
    uint64_t* out_bits;           // packed sign bits [M][N/64] or null
    int B, OH, OW, N;
    int kh, kw, pad_h, pad_w, stride, cw;
    int rows, imgs, tiles_per_img, ntiles;
    int G, stages, wb, nboxes;    // K boxes per stage, ring stages, rows of a weight box image, kh*kw*cw
    int resident;                 // the channel block's weights stay in shared memory (loaded once per CTA)
    int stiles;                   // staging tiles (2 or 3): the shortcut is prefetched stiles - 1 blocks ahead
    int wide;                     // cin % 128 == 0: one TMA load covers two K boxes (128-byte rows, SWIZZLE_128B)
    int pair;                     // two pixel tiles share every weight stage (streamed weights: halves their bytes)
    int lag;                      // tensor stores that may still be reading their staging tile when the next shortcut is fetched
                                  // (0 or 1): the shortcut runs stiles - 1 - lag blocks ahead
    int nbc;                      // output channels per CTA: TC5_MAX_N, or 64 / 32 when there are too few tiles to fill the SMs
                                  // (streamed weights only: a CTA then copies its rows out of every box image)
};

__host__ __device__ inline int u8_weight_rows(int N) { return min(N, TC5_MAX_N); }
__host__ __device__ inline size_t u8_weight_image_bytes(int N, int nboxes) {
    return (size_t)((N + TC5_MAX_N - 1) / TC5_MAX_N) * nboxes * u8_weight_rows(N) * 64;
}
__host__ __device__ inline size_t u8_weight_bytes(int N, int nboxes) {
    return u8_weight_image_bytes(N, nboxes) + (size_t)((N + TC5_MAX_N - 1) / TC5_MAX_N) * TC5_MAX_N * sizeof(int);
}

// grid (nboxes, channel blocks): the image of K box q (= packed word q) of one channel block: wb rows x 64 bytes,
// byte k of row n = 1 - 2 * bit k of the word (+1 or -1 as a signed byte), stored as 8-row x 16-byte core matrices
// ([row / 8][k / 16][row % 8][k % 16]); rows beyond the channel block are zero.
__global__ void __launch_bounds__(256) bconv_u8_expand_weights_kernel(const uint64_t* w, const long long ldw, const int N,
                                                                      const int nboxes, unsigned char* dst) {
    const int q = blockIdx.x, nb = blockIdx.y, wb = u8_weight_rows(N);
    const int n0 = nb * TC5_MAX_N, n_this = min(TC5_MAX_N, N - n0);
    unsigned char* img = dst + ((size_t)nb * nboxes + q) * wb * 64;
    for (int idx = threadIdx.x; idx < wb * 4; idx += blockDim.x) {
        const int row = idx >> 2, unit = idx & 3;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (row < n_this) {
            const uint32_t bits = (uint32_t)(__ldg(w + (long long)(n0 + row) * ldw + q) >> (unit * 16)) & 0xffffu;
            auto signed_bytes = [](uint32_t nibble) {   // four bits -> four bytes, 0 -> 0x01, 1 -> 0xff
                const uint32_t m = (nibble * 0x00204081u) & 0x01010101u;
                return (m * 0xffu) | (m ^ 0x01010101u);
            };
            v.x = signed_bytes(bits & 0xfu); v.y = signed_bytes((bits >> 4) & 0xfu);
            v.z = signed_bytes((bits >> 8) & 0xfu); v.w = signed_bytes((bits >> 12) & 0xfu);
        }
        *reinterpret_cast<uint4*>(img + (row >> 3) * 512 + unit * 128 + (row & 7) * 16) = v;
    }
    if (q == 0 && threadIdx.x < TC5_MAX_N) {
        int pc = 0;
        if ((int)threadIdx.x < n_this)
            for (int k = 0; k < nboxes; k++) pc += __popcll(__ldg(w + (long long)(n0 + threadIdx.x) * ldw + k));
        reinterpret_cast<int*>(dst + u8_weight_image_bytes(N, nboxes))[n0 + threadIdx.x] = pc;
    }
}

// fp32 -> {0,1} bytes (x > 0), 16 elements per thread step
__global__ void __launch_bounds__(256) binarize_u8_kernel(const float* __restrict__ in, unsigned char* __restrict__ out, const size_t n16,
                                                           const size_t count) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) {
        uint32_t wds[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float4 f = __ldg(reinterpret_cast<const float4*>(in) + i * 4 + j);
            wds[j] = (f.x > 0.f ? 1u : 0u) | (f.y > 0.f ? 0x100u : 0u) | (f.z > 0.f ? 0x10000u : 0u) | (f.w > 0.f ? 0x1000000u : 0u);
        }
        reinterpret_cast<uint4*>(out)[i] = make_uint4(wds[0], wds[1], wds[2], wds[3]);
    }
    if (blockIdx.x == 0)   // tail
        for (size_t i = n16 * 16 + threadIdx.x; i < count; i += blockDim.x) out[i] = in[i] > 0.f ? 1 : 0;
}

// K-major SWIZZLE_64B shared-memory descriptor: 8-row groups 512 bytes apart
__device__ __forceinline__ uint64_t umma_desc_sw64(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)1 << 16) | ((uint64_t)(512 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)4 << 61);
}
// K-major SWIZZLE_128B: rows of 128 bytes, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}

template <bool PAIR>   // PAIR: a unit of work is two pixel tiles sharing the weight stages (p.pair)
__global__ void __launch_bounds__(U8_THREADS, 1)
    bconv_u8_kernel(const U8Params p, const __grid_constant__ CUtensorMap in_map0, const __grid_constant__ CUtensorMap in_map1,
                    const __grid_constant__ CUtensorMap out_map, const __grid_constant__ CUtensorMap sc_map) {
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) uint64_t bar_full[8], bar_empty[8], bar_acc_full[U8_ACCS], bar_acc_empty[U8_ACCS], bar_w, sc_full[U8_MAX_STILES];
    __shared__ uint32_t tmem_base_s;
    __shared__ int s_abort, epi_abort;
    __shared__ __align__(16) int popw[TC5_MAX_N];
    __shared__ __align__(16) float chan_a[TC5_MAX_N];
    __shared__ __align__(16) float chan_b[TC5_MAX_N];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.y * p.nbc;
    const int n_this = min(p.nbc, p.N - n0);        // multiple of 16 (host-checked)
    const int n_mma = n_this;
    constexpr int np = PAIR ? 2 : 1;                // pixel tiles per unit of work (they share the unit's weight stages)
    const int nunits = (p.ntiles + np - 1) / np;
    const int a_bytes1 = p.G * U8_BOX_BYTES, a_bytes = np * a_bytes1;   // one tile's boxes of a stage, all of them
    const int gbox_bytes = p.wb * 64, wbox_bytes = min(p.nbc, p.wb) * 64;   // a box image in global / this CTA's rows of it
    const int stage_bytes = a_bytes + (p.resident ? 0 : p.G * wbox_bytes);
    unsigned char* wres = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
    unsigned char* stage0 = wres + (p.resident ? p.nboxes * wbox_bytes : 0);   // a multiple of 1024 bytes further
    const int nst = (p.nboxes + p.G - 1) / p.G;     // stages per tile
    int tmem_cols = 32;
    while (tmem_cols < U8_ACCS * n_mma) tmem_cols <<= 1;
    const volatile int* abort_flag = &s_abort;
    const int ohw = p.OH * p.OW;
    const int box_px = p.rows * p.OW * p.imgs;      // pixels a tile's loads and stores cover
    const int srows = u8_staging_rows(box_px), sbox_bytes = srows * 128, stile_bytes = 2 * sbox_bytes;

    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(tmem_cols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    if (tid == 0) {
        for (int i = 0; i < p.stages; i++) { mbar_init(&bar_full[i], 1); mbar_init(&bar_empty[i], 1); }
        for (int i = 0; i < U8_ACCS; i++) { mbar_init(&bar_acc_full[i], 1); mbar_init(&bar_acc_empty[i], U8_EPI_WARPS); }
        mbar_init(&bar_w, 1);
        for (int i = 0; i < U8_MAX_STILES; i++) mbar_init(&sc_full[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::);
        s_abort = 0;
        epi_abort = 0;
    }
    if (tid < TC5_MAX_N) {
        popw[tid] = tid < n_this ? __ldg(reinterpret_cast<const int*>(p.w_img + u8_weight_image_bytes(p.N, p.nboxes)) + n0 + tid) : 0;
        const bool have = p.a && tid < n_this;
        chan_a[tid] = have ? __ldg(p.a + n0 + tid) : 1.f;
        chan_b[tid] = have ? __ldg(p.b + n0 + tid) : 0.f;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;
    grid_launch_dependents();
    grid_dependency_wait();   // set-up touched constants only; activations come next

    if (warp == 0) {
        // =========================== loads: one lane ===========================
        if (lane == 0) {
            // this CTA's rows of its channel block's box images
            const unsigned char* wsrc = p.w_img + (size_t)(n0 / TC5_MAX_N) * p.nboxes * gbox_bytes + (size_t)(n0 % TC5_MAX_N) * 64;
            const uint32_t stage0_addr = smem_u32(stage0);
            const uint32_t box_tx = (uint32_t)box_px * 64u;   // a load always delivers its whole box (zeros outside the tensor)
            uint32_t s = 0, use = 0;
            bool ok = true;
            if (p.resident) {   // the whole channel block, once
                const uint32_t bytes = (uint32_t)(p.nboxes * wbox_bytes), bar = smem_u32(&bar_w);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(smem_u32(wres)), "l"(wsrc), "r"(bytes), "r"(bar) : "memory");
            }
            for (int unit = blockIdx.x; unit < nunits && ok; unit += gridDim.x) {
                int img0[2], oh0[2];   // a tile past the last one lies outside the tensor: its loads deliver zeros
                for (int t = 0; t < np; t++) {
                    const int tile = unit * np + t, tq = tile / p.tiles_per_img;
                    img0[t] = tq * p.imgs; oh0[t] = (tile - tq * p.tiles_per_img) * p.rows;
                }
                int cg = 0, ky = 0, kx = 0;
                for (int st = 0; st < nst; st++) {
                    if (use >= 1 && !mbar_wait<32>(&bar_empty[s], (use - 1) & 1, abort_flag)) {
                        atomicCAS(&g_u8_status, 0, 21);
                        s_abort = 1;
                        ok = false;
                        break;
                    }
                    const int nb = min(p.G, p.nboxes - st * p.G);
                    const uint32_t bar = smem_u32(&bar_full[s]), sa = stage0_addr + s * stage_bytes;
                    const uint32_t wbytes = p.resident ? 0u : (uint32_t)(nb * wbox_bytes);
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(wbytes + np * nb * box_tx) : "memory");
                    if (!p.resident) {
                        if (wbox_bytes == gbox_bytes) {   // whole box images: the stage's boxes are one run
                            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                         ::"r"(sa + a_bytes), "l"(wsrc + (size_t)st * p.G * gbox_bytes), "r"(wbytes), "r"(bar) : "memory");
                        } else {
                            for (int b = 0; b < nb; b++)
                                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                             ::"r"(sa + a_bytes + b * wbox_bytes), "l"(wsrc + (size_t)(st * p.G + b) * gbox_bytes), "r"((uint32_t)wbox_bytes),
                                               "r"(bar) : "memory");
                        }
                    }
                    const int bstep = p.wide ? 2 : 1;   // a wide load fills two K boxes (16 KB: 128 rows of 128 bytes)
                    for (int b = 0; b < nb; b += bstep) {
                        const int dy = ky - p.pad_h, dx = kx - p.pad_w;
                        int c1 = 0, c2 = dx, c3 = dy;
                        const CUtensorMap* map = &in_map0;
                        if (p.stride == 2) {
                            const int hp = dy & 1, wp = dx & 1;
                            c1 = wp; c2 = (dx - wp) >> 1; c3 = (dy - hp) >> 1;
                            if (hp) map = &in_map1;
                        }
                        for (int t = 0; t < np; t++)
                            asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
                                         ::"r"(sa + t * a_bytes1 + b * U8_BOX_BYTES), "l"(reinterpret_cast<uint64_t>(map)), "r"(cg * 64), "r"(c2),
                                           "r"(oh0[t] + c3), "r"(img0[t]), "r"(c1), "r"(bar) : "memory");
                        if ((cg += bstep) == p.cw) { cg = 0; if (++kx == p.kw) { kx = 0; ky++; } }
                    }
                    if (++s == (uint32_t)p.stages) { s = 0; use++; }
                }
            }
        }
    } else if (warp == 1) {
        // =========================== MMA issue: one lane ===========================
        if (lane == 0) {
            // instruction descriptor: D = s32, A = u8, B = s8, both K-major, N = n_mma, M = 128
            const uint32_t idesc = (2u << 4) | (1u << 10) | ((uint32_t)(n_mma >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
            const uint64_t d_a = p.wide ? umma_desc_sw128(smem_u32(stage0)) : umma_desc_sw64(smem_u32(stage0));
            const uint64_t d_b = p.resident ? umma_desc(smem_u32(wres), 512) : umma_desc(smem_u32(stage0) + a_bytes, 512);
            if (p.resident && !mbar_wait(&bar_w, 0, abort_flag)) {
                atomicCAS(&g_u8_status, 0, 23);
                s_abort = 1;
            }
            uint32_t s = 0, par = 0;
            bool ok = !s_abort;
            int i = 0;   // tiles so far: tile i accumulates in accumulator i % U8_ACCS
            for (int unit = blockIdx.x; unit < nunits && ok; unit += gridDim.x, i += np) {
                for (int t = 0; t < np && ok; t++) {
                    const int accbuf = (i + t) % U8_ACCS, accuse = (i + t) / U8_ACCS;
                    if (accuse >= 1 && !mbar_wait(&bar_acc_empty[accbuf], (accuse - 1) & 1, abort_flag)) {
                        atomicCAS(&g_u8_status, 0, 22);
                        s_abort = 1;
                        ok = false;
                    }
                }
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + (i % U8_ACCS) * n_mma;   // the pair's second accumulator follows the first
                const uint32_t a_step = (uint32_t)(a_bytes1 >> 4);
                uint32_t accum = 0;
                for (int st = 0; st < nst; st++) {
                    if (!mbar_wait(&bar_full[s], par, abort_flag)) {
                        atomicCAS(&g_u8_status, 0, 23);
                        s_abort = 1;
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const int nb = min(p.G, p.nboxes - st * p.G);
                    uint64_t ad = d_a + (uint64_t)(s * (stage_bytes >> 4));
                    uint64_t bd = d_b + (uint64_t)(p.resident ? st * p.G * (wbox_bytes >> 4) : s * (stage_bytes >> 4));
                    // one MMA per 32 bytes of K: 32 bytes along the swizzled row of A, two 16-byte units (256 bytes) of B
                    if (p.wide) {
                        for (int b = 0; b < nb; b += 2) {   // a 128-byte row of A holds the K of two weight boxes
                            const uint64_t bd2 = bd + (uint64_t)(wbox_bytes >> 4);
                            for (int t = 0; t < np; t++) {
                                const uint64_t at = ad + t * a_step;
                                mma_i8_ss(d_tmem + t * n_mma, at, bd, idesc, accum);
                                mma_i8_ss(d_tmem + t * n_mma, at + 2, bd + 16, idesc, 1u);
                                mma_i8_ss(d_tmem + t * n_mma, at + 4, bd2, idesc, 1u);
                                mma_i8_ss(d_tmem + t * n_mma, at + 6, bd2 + 16, idesc, 1u);
                            }
                            bd = bd2 + (uint64_t)(wbox_bytes >> 4);
                            accum = 1u;
                            ad += (2 * U8_BOX_BYTES) >> 4;
                        }
                    } else {
                        for (int b = 0; b < nb; b++) {
                            for (int t = 0; t < np; t++) {
                                const uint64_t at = ad + t * a_step;
                                mma_i8_ss(d_tmem + t * n_mma, at, bd, idesc, accum);
                                mma_i8_ss(d_tmem + t * n_mma, at + 2, bd + 16, idesc, 1u);
                            }
                            accum = 1u;
                            ad += U8_BOX_BYTES >> 4;
                            bd += (uint64_t)(wbox_bytes >> 4);
                        }
                    }
                    umma_commit(&bar_empty[s]);
                    if (++s == (uint32_t)p.stages) { s = 0; par ^= 1u; }
                }
                if (ok)
                    for (int t = 0; t < np; t++) umma_commit(&bar_acc_full[(i + t) % U8_ACCS]);
            }
        }
    } else {
        // =========================== epilogue ===========================
        // Blocks of 64 channels through p.stiles fp32 staging tiles: the shortcut of block k + stiles - 1 is copied into
        // the idle tile with cp.async (one or two blocks ahead: at 60 % of the HBM bandwidth one 32 KB block in flight per
        // SM does not cover the latency) while block k is drained (thread (r, hq): 16 accumulator columns of pixel r), then one
        // TMA tensor store per 32-channel box writes the fp32 result; the {0,1} bytes and the packed sign bits of the result go straight from registers to global
        // memory.
        const int et = tid - 64, ew = warp - 2;
        const int r = (warp & 3) * 32 + lane, hq = ew >> 2;   // TMEM lane quarter of a warp = warp % 4; column quarter 0..3
        const uint32_t sbuf0_addr = smem_u32(stage0 + p.stages * stage_bytes);
        const int nblk = (n_this + 63) >> 6;
        // This CTA's tiles in order: unit u = blockIdx.x + j * gridDim.x holds tiles u * np .. u * np + np - 1.
        const int first_tile = blockIdx.x * np;
        auto next_tile = [&](int tile, int index) {   // the tile after `tile`, which is this CTA's tile number `index`
            return np == 1 ? tile + (int)gridDim.x : ((index & 1) ? tile + 2 * (int)gridDim.x - 1 : tile + 1);
        };
        int my_tiles = 0;
        for (int t = first_tile, k = 0; t < p.ntiles; t = next_tile(t, k++)) my_tiles++;
        const int total_blocks = my_tiles * nblk;
        // first output pixel of a tile and how many of its pixels exist
        auto tile_span = [&](int tile, long long& base, int& nvalid, int& img0, int& oh0) {
            const int tq = tile / p.tiles_per_img;
            img0 = tq * p.imgs; oh0 = (tile - tq * p.tiles_per_img) * p.rows;
            base = ((long long)img0 * p.OH + oh0) * p.OW;
            nvalid = p.imgs > 1 ? min(p.imgs, p.B - img0) * ohw : min(p.rows, p.OH - oh0) * p.OW;
        };
        // The shortcut of block kb + stiles - 1 is fetched into the staging tile that block kb - 1 has left, by one thread and
        // two tiled TMA loads (the tile's layout is the one the tensor store reads, so the sum happens in place).
        int pkb = 0, ptile = first_tile, pti = 0, pblk = 0, pst = 0;
        auto prefetch_next = [&]() {   // thread et == 0 only
            if (p.shortcut && pkb < total_blocks) {
                const int tq = ptile / p.tiles_per_img;
                const int pimg = tq * p.imgs, poh0 = (ptile - tq * p.tiles_per_img) * p.rows;
                const int cb = pblk * 64, boxes = n_this - cb > 32 ? 2 : 1;
                const uint32_t bar = smem_u32(&sc_full[pst]), dst = sbuf0_addr + pst * stile_bytes;
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)(boxes * box_px * 128)) : "memory");
                for (int hb = 0; hb < boxes; hb++)
                    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                                 ::"r"(dst + hb * sbox_bytes), "l"(reinterpret_cast<uint64_t>(&sc_map)), "r"(n0 + cb + hb * 32), "r"(poh0 * p.OW), "r"(pimg),
                                   "r"(bar) : "memory");
            }
            pkb++;
            if (++pst == p.stiles) pst = 0;
            if (++pblk == nblk) {
                pblk = 0;
                ptile = next_tile(ptile, pti++);
            }
        };
        if (et == 0)
            for (int d = 0; d + 1 + p.lag < p.stiles; d++) prefetch_next();
        bool okw = true;
        uint32_t sc_par = 0;
        int tile = first_tile, ti = 0, blk = 0, st_idx = 0, accbuf = 0, accuse = 0, nvalid = 0, img0 = 0, oh0 = 0;
        long long base = 0;
        for (int kb = 0; kb < total_blocks; kb++) {
            if (blk == 0) tile_span(tile, base, nvalid, img0, oh0);
            const int cb = blk * 64;
            const int width = min(64, n_this - cb);
            const uint32_t sb = sbuf0_addr + st_idx * stile_bytes;
            if (et == 0) {
                // the tile the next shortcut goes to is idle once the stores of block kb - 1 - lag have read it
                if (p.lag) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                else asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                prefetch_next();
            }
            if (p.shortcut && okw) {   // the shortcut of block kb has landed in its tile
                okw = __all_sync(0xffffffffu, mbar_wait<100>(&sc_full[st_idx], sc_par, abort_flag));
                if (!okw) {
                    atomicCAS(&g_u8_status, 0, 24);
                    s_abort = 1;
                    epi_abort = 1;
                }
            }
            const bool mine = width > hq * 16;                               // this thread's 16 columns exist
            if (blk == 0 && okw) {
                okw = __all_sync(0xffffffffu, mbar_wait<200>(&bar_acc_full[accbuf], accuse & 1, abort_flag));
                if (!okw) {
                    atomicCAS(&g_u8_status, 0, 24);
                    s_abort = 1;
                    epi_abort = 1;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            }
            if (okw && mine) {
                const int c0 = cb + hq * 16;
                const uint32_t t_row = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + accbuf * n_mma;
                uint32_t v[16];
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                             : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                               "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                             : "r"(t_row + c0));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                // chunk qq (4 channels) of this pixel's row in box hq / 2: srow + ((qq ^ (r & 7)) << 4)
                const uint32_t srow = sb + (hq >> 1) * sbox_bytes + r * 128;
                const bool staged = r < srows;   // the accumulator rows beyond the tile have no staging row
                uint32_t signs = 0;   // bit j: channel c0 + j of this pixel is positive
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const int cl = c0 + q * 4;
                    const int4 pw = *reinterpret_cast<const int4*>(popw + cl);
                    float o[4];
                    o[0] = small_int_to_float(pw.x + (int)v[q * 4 + 0]);
                    o[1] = small_int_to_float(pw.y + (int)v[q * 4 + 1]);
                    o[2] = small_int_to_float(pw.z + (int)v[q * 4 + 2]);
                    o[3] = small_int_to_float(pw.w + (int)v[q * 4 + 3]);
                    if (p.a) {
                        const float4 ca = *reinterpret_cast<const float4*>(chan_a + cl), cbv = *reinterpret_cast<const float4*>(chan_b + cl);
                        o[0] = __fadd_rn(__fmul_rn(ca.x, o[0]), cbv.x); o[1] = __fadd_rn(__fmul_rn(ca.y, o[1]), cbv.y);
                        o[2] = __fadd_rn(__fmul_rn(ca.z, o[2]), cbv.z); o[3] = __fadd_rn(__fmul_rn(ca.w, o[3]), cbv.w);
                    }
                    const uint32_t sa = srow + ((((hq & 1) * 4 + q) ^ (r & 7)) << 4);
                    if (p.shortcut && staged) {
                        const float4 ad = lds128f(sa);
                        o[0] = __fadd_rn(ad.x, o[0]); o[1] = __fadd_rn(ad.y, o[1]);
                        o[2] = __fadd_rn(ad.z, o[2]); o[3] = __fadd_rn(ad.w, o[3]);
                    }
                    if (staged) sts128f(sa, o[0], o[1], o[2], o[3]);
                    signs |= ((o[0] > 0.f ? 1u : 0u) | (o[1] > 0.f ? 2u : 0u) | (o[2] > 0.f ? 4u : 0u) | (o[3] > 0.f ? 8u : 0u)) << (q * 4);
                }
                if (r < nvalid) {
                    const long long row = base + r;
                    if (p.out_bits)   // 16 channels = a quarter of a packed word (a narrow channel block may start inside a word)
                        reinterpret_cast<unsigned short*>(p.out_bits + row * (p.N >> 6) + ((n0 + cb) >> 6))[(((n0 + cb) & 63) >> 4) + hq] = (unsigned short)signs;
                    if (p.out_u8) {
                        uint32_t w8[4];
#pragma unroll
                        for (int q = 0; q < 4; q++) w8[q] = (((signs >> (q * 4)) & 0xfu) * 0x00204081u) & 0x01010101u;
                        *reinterpret_cast<uint4*>(p.out_u8 + row * p.N + n0 + c0) = make_uint4(w8[0], w8[1], w8[2], w8[3]);
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the tensor store below reads what was just written
            }
            if (blk == nblk - 1 && okw) {   // the whole accumulator has been read
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_acc_empty[accbuf]);
            }
            asm volatile("bar.sync 1, %0;" ::"n"(U8_EPILOGUE) : "memory");   // results of block kb are staged (or abort decided)
            if (epi_abort) break;
            // ---- write-out: one tensor store per 32-channel box; pixels beyond the image / batch and channels beyond N are clipped ----
            if (et == 0) {
                if (p.out)
                    for (int hb = 0; hb < (width > 32 ? 2 : 1); hb++)
                        asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];"
                                     ::"l"(reinterpret_cast<uint64_t>(&out_map)), "r"(n0 + cb + hb * 32), "r"(oh0 * p.OW), "r"(img0),
                                       "r"(sb + hb * sbox_bytes) : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
            if (++st_idx == p.stiles) { st_idx = 0; sc_par ^= 1u; }
            if (++blk == nblk) {
                blk = 0;
                tile = next_tile(tile, ti++);
                if (++accbuf == U8_ACCS) { accbuf = 0; accuse++; }
            }
        }
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols));
    }
}

}  // namespace dabnn
