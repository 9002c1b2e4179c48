// 3x3 stride-1 binary convolution on {0,1}-byte activations in which every input byte enters the SM once per tile.
//
// bconv_u8_kernel loads one box of the tile's pixels per tap: nine copies of (nearly) the same bytes, and on the
// deep layers the weights again for every tile; it runs at the rate at which L2 can feed the SMs.  Here a tile's
// input arrives once, as the halo of the tile: (rows + 2) x (OW + 2) pixels x 64 channels, one tiled TMA load per
// 64-channel group (zero fill outside the image = the reference's padding), 64-byte-swizzled, pixel after pixel at a
// pitch of P = OW + 2.  The pixel operand of tap (ky, kx) is then that same buffer read from pixel ky * P + kx on: the
// K-major SWIZZLE_64B descriptor with its start address advanced by (ky * P + kx) * 64 bytes - the swizzle is a
// function of the final shared-memory address, so a start anywhere inside the swizzle atom reads the rows in order.
// Operand row m of the MMA is halo pixel m, i.e. output pixel (m / P, m % P): the two columns m % P >= OW of every
// output row are computed and never read (116 of 128 rows carry pixels for a 56-pixel row, as against 112 before).
//
// Weights as in bconv_u8.cuh (signed bytes 1 - 2b, per (tap, 64-channel group) box images): resident in shared memory
// when a channel block's nine taps fit, else streamed in stages of one window row (three taps) of one channel group,
// and then a unit of work is two pixel tiles that share every weight stage.  The loop order is channel group, window
// row, tile, tap, so a halo buffer is released after its 18 (36 with two tiles: each its own) MMAs and the ring refills
// while the other groups compute.
//
// Small images (7x7: the last stage of a ResNet) go two to a tile.  The pitch is then P = OW + 1: the zero column left of
// a row doubles as the zero column right of the row above, the second image's halo starts (OH + 1) * P pixels after
// the first one's - its top padding row is the first image's bottom padding row - and one zero pixel, written once at
// start-up, stands behind the second halo for the last pixel's lower right tap.  The two images' boxes are two TMA loads
// into one slot; 98 of the MMA's 128 rows carry pixels, and the nine taps of a pixel cost one load instead of nine.
//
// A block whose result also feeds a 2x2 stride-2 average pooling (the downsample shortcut of the next stage: reference
// layers/AvePool.cpp:84) can write the pooled tensor as well: tiles are then an even number of output rows, and after a
// block of 64 channels is staged every thread folds one pooled pixel x four channels out of the staging tile, in the
// reference's tap order, sum first, then the division.
//
// Warps: 0 halo loads, 1 weight loads, 2 MMA issue (one lane each), 3 .. 18 epilogue (as in bconv_u8.cuh, with the
// accumulator row -> pixel mapping above).  Every wait is bounded; a wait that gives up records a code in the
// byte-activation engine's status word (21 halo loader, 25 weight loader, 22 / 23 / 26 MMA thread waiting for an
// accumulator / a halo / a weight stage, 24 epilogue), raises the CTA's abort flag, and the CTA frees its tensor
// memory and returns.
#pragma once
#include "bconv_u8.cuh"

namespace dabnn {

constexpr int HL_THREADS = 96 + U8_EPILOGUE;   // warps 0, 1, 2 + the epilogue warps
constexpr int HL_MAX_HSLOTS = 8, HL_MAX_WSTAGES = 8;   // (more than four weight stages only with narrow channel blocks)

struct HaloParams {
    const unsigned char* w_img;   // expanded weights (bconv_u8_expand_weights_kernel): box (tap * cw + cg)
    const float *a, *b;
    const float* shortcut;
    float* out;
    unsigned char* out_u8;
    uint64_t* out_bits;
    float* pool_out;              // or null: fp32 [B][OH / 2][OW / 2][N], the 2x2 stride-2 average pooling of `out` (OH, OW, rows even)
    int B, OH, OW, N;
    int cw;                       // 64-channel groups of the input
    int P;                        // halo pitch in pixels: OW + 2 (OW + 1 with two images per tile)
    int imgs, img_pitch;          // images per tile (1 or 2) and, with two, the accumulator rows between them: (OH + 1) * P
    int rows, tiles_per_img, ntiles;
    int hslots, halo_stride;      // halo ring: slots and bytes between them (a multiple of 1024)
    int wstages;                  // weight ring stages of three boxes (streamed weights)
    int wb;                       // rows of a weight box image
    int nb;                       // output channels per CTA: TC5_MAX_N, or 64 / 32 when there are too few tiles to fill the SMs
                                  // (streamed weights only: a CTA then copies its rows out of every box image)
    int resident, stiles, pair;
    int lag;                      // tensor stores that may still be reading their staging tile when the next shortcut is fetched (0 or 1):
                                  // the shortcut runs stiles - 1 - lag blocks ahead
};

template <bool PAIR>
__global__ void __launch_bounds__(HL_THREADS, 1)
    bconv_halo_kernel(const HaloParams p, const __grid_constant__ CUtensorMap in_map, const __grid_constant__ CUtensorMap out_map,
                      const __grid_constant__ CUtensorMap sc_map) {
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) uint64_t halo_full[HL_MAX_HSLOTS], halo_empty[HL_MAX_HSLOTS], w_full[HL_MAX_WSTAGES], w_empty[HL_MAX_WSTAGES];
    __shared__ __align__(8) uint64_t bar_acc_full[U8_ACCS], bar_acc_empty[U8_ACCS], bar_w, sc_full[U8_MAX_STILES];
    __shared__ uint32_t tmem_base_s;
    __shared__ int s_abort, epi_abort;
    __shared__ __align__(16) int popw[TC5_MAX_N];
    __shared__ __align__(16) float chan_a[TC5_MAX_N];
    __shared__ __align__(16) float chan_b[TC5_MAX_N];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.y * p.nb;
    const int n_this = min(p.nb, p.N - n0);        // multiple of 16 (host-checked)
    const int n_mma = n_this;
    constexpr int np = PAIR ? 2 : 1;
    const int nunits = (p.ntiles + np - 1) / np;
    const int nboxes = 9 * p.cw, gbox_bytes = p.wb * 64, wbox_bytes = min(p.nb, p.wb) * 64;   // a box image in global / this CTA's rows of it
    unsigned char* halo0 = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
    unsigned char* wbase = halo0 + p.hslots * p.halo_stride;                                   // resident weights or the weight ring
    unsigned char* sbuf0 = wbase + (p.resident ? nboxes * wbox_bytes : p.wstages * 3 * wbox_bytes);   // a multiple of 1024 bytes further
    int tmem_cols = 32;
    while (tmem_cols < U8_ACCS * n_mma) tmem_cols <<= 1;
    const volatile int* abort_flag = &s_abort;
    const int box_px = p.imgs * p.rows * p.OW;      // pixels a tile's stores cover
    const int srows = u8_staging_rows(box_px), sbox_bytes = srows * 128, stile_bytes = 2 * sbox_bytes;
    const uint32_t halo_tx = (uint32_t)(p.imgs * (p.rows + 2) * p.P * 64);

    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(tmem_cols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    if (tid == 0) {
        for (int i = 0; i < p.hslots; i++) { mbar_init(&halo_full[i], 1); mbar_init(&halo_empty[i], 1); }
        for (int i = 0; i < HL_MAX_WSTAGES; i++) { mbar_init(&w_full[i], 1); mbar_init(&w_empty[i], 1); }
        for (int i = 0; i < U8_ACCS; i++) { mbar_init(&bar_acc_full[i], 1); mbar_init(&bar_acc_empty[i], U8_EPI_WARPS); }
        mbar_init(&bar_w, 1);
        for (int i = 0; i < U8_MAX_STILES; i++) mbar_init(&sc_full[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::);
        s_abort = 0;
        epi_abort = 0;
    }
    if (p.imgs == 2 && tid < p.hslots * 4)   // the zero pixel behind the second image's halo (never written again)
        sts128(smem_u32(halo0) + (tid >> 2) * p.halo_stride + (p.img_pitch + (p.rows + 2) * p.P) * 64 + (tid & 3) * 16, 0u, 0u, 0u, 0u);
    if (tid < TC5_MAX_N) {
        popw[tid] = tid < n_this ? __ldg(reinterpret_cast<const int*>(p.w_img + u8_weight_image_bytes(p.N, nboxes)) + n0 + tid) : 0;
        const bool have = p.a && tid < n_this;
        chan_a[tid] = have ? __ldg(p.a + n0 + tid) : 1.f;
        chan_b[tid] = have ? __ldg(p.b + n0 + tid) : 0.f;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;
    // this CTA's rows of its channel block's box images
    const unsigned char* wsrc = p.w_img + (size_t)(n0 / TC5_MAX_N) * nboxes * gbox_bytes + (size_t)(n0 % TC5_MAX_N) * 64;
    grid_launch_dependents();
    if (warp != 1) grid_dependency_wait();   // the weight loader reads constants only and may run ahead of the previous kernel's end

    if (warp == 0) {
        // =========================== halo loads: one lane ===========================
        if (lane == 0) {
            const uint32_t halo0_addr = smem_u32(halo0);
            uint32_t hs = 0, huse = 0;
            bool ok = true;
            for (int unit = blockIdx.x; unit < nunits && ok; unit += gridDim.x) {
                int img[2], oh0[2];   // a tile past the last one lies outside the tensor: its load delivers zeros
                for (int t = 0; t < np; t++) {
                    const int tile = unit * np + t;
                    if (p.imgs == 2) { img[t] = tile * 2; oh0[t] = 0; }
                    else { img[t] = tile / p.tiles_per_img; oh0[t] = (tile - img[t] * p.tiles_per_img) * p.rows; }
                }
                for (int cg = 0; cg < p.cw && ok; cg++)
                    for (int t = 0; t < np; t++) {
                        if (huse >= 1 && !mbar_wait<32>(&halo_empty[hs], (huse - 1) & 1, abort_flag)) {
                            atomicCAS(&g_u8_status, 0, 21);
                            s_abort = 1;
                            ok = false;
                            break;
                        }
                        const uint32_t bar = smem_u32(&halo_full[hs]);
                        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(halo_tx) : "memory");
                        for (int j = 0; j < p.imgs; j++)   // (an image past the last one lies outside the tensor: zeros)
                            asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
                                         ::"r"(halo0_addr + hs * p.halo_stride + j * p.img_pitch * 64), "l"(reinterpret_cast<uint64_t>(&in_map)), "r"(cg * 64), "r"(-1),
                                           "r"(oh0[t] - 1), "r"(img[t] + j), "r"(0), "r"(bar) : "memory");
                        if (++hs == (uint32_t)p.hslots) { hs = 0; huse++; }
                    }
            }
        }
    } else if (warp == 1) {
        // =========================== weight loads: one lane ===========================
        if (lane == 0) {
            if (p.resident) {   // the whole channel block, once
                const uint32_t bytes = (uint32_t)(nboxes * wbox_bytes), bar = smem_u32(&bar_w);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(smem_u32(wbase)), "l"(wsrc), "r"(bytes), "r"(bar) : "memory");
            } else {
                const uint32_t w0_addr = smem_u32(wbase);
                uint32_t ws = 0, wuse = 0;
                bool ok = true;
                for (int unit = blockIdx.x; unit < nunits && ok; unit += gridDim.x)
                    for (int cg = 0; cg < p.cw && ok; cg++)
                        for (int ky = 0; ky < 3; ky++) {
                            if (wuse >= 1 && !mbar_wait<32>(&w_empty[ws], (wuse - 1) & 1, abort_flag)) {
                                atomicCAS(&g_u8_status, 0, 25);
                                s_abort = 1;
                                ok = false;
                                break;
                            }
                            const uint32_t bar = smem_u32(&w_full[ws]), dst = w0_addr + ws * 3 * wbox_bytes;
                            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(3u * wbox_bytes) : "memory");
                            for (int kx = 0; kx < 3; kx++)   // the three taps of window row ky of this channel group
                                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                             ::"r"(dst + kx * wbox_bytes), "l"(wsrc + (size_t)((ky * 3 + kx) * p.cw + cg) * gbox_bytes), "r"((uint32_t)wbox_bytes),
                                               "r"(bar) : "memory");
                            if (++ws == (uint32_t)p.wstages) { ws = 0; wuse++; }
                        }
            }
        }
    } else if (warp == 2) {
        // =========================== MMA issue: one lane ===========================
        if (lane == 0) {
            // instruction descriptor: D = s32, A = u8, B = s8, both K-major, N = n_mma, M = 128
            const uint32_t idesc = (2u << 4) | (1u << 10) | ((uint32_t)(n_mma >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
            const uint64_t d_halo = umma_desc_sw64(smem_u32(halo0));
            const uint64_t d_w = umma_desc(smem_u32(wbase), 512);
            const uint32_t halo_units = (uint32_t)p.halo_stride >> 4, wbox_units = (uint32_t)wbox_bytes >> 4, row_units = (uint32_t)p.P * 4u;
            bool ok = true;
            if (p.resident && !mbar_wait(&bar_w, 0, abort_flag)) {
                atomicCAS(&g_u8_status, 0, 26);
                s_abort = 1;
                ok = false;
            }
            uint32_t hs = 0, hpar = 0, ws = 0, wpar = 0;
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
                uint32_t d_tmem[np];
                for (int t = 0; t < np; t++) d_tmem[t] = tmem_base + ((i + t) % U8_ACCS) * n_mma;
                uint32_t accum = 0;
                for (int cg = 0; cg < p.cw && ok; cg++) {
                    uint32_t slot[np];
                    for (int t = 0; t < np; t++) {   // this group's halo of every tile of the unit
                        if (!mbar_wait(&halo_full[hs], hpar, abort_flag)) {
                            atomicCAS(&g_u8_status, 0, 23);
                            s_abort = 1;
                            ok = false;
                            break;
                        }
                        slot[t] = hs;
                        if (++hs == (uint32_t)p.hslots) { hs = 0; hpar ^= 1u; }
                    }
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    for (int ky = 0; ky < 3; ky++) {
                        uint64_t bd;
                        if (p.resident) {
                            bd = d_w + (uint64_t)((ky * 3 * p.cw + cg) * wbox_units);
                        } else {
                            if (!mbar_wait(&w_full[ws], wpar, abort_flag)) {
                                atomicCAS(&g_u8_status, 0, 26);
                                s_abort = 1;
                                ok = false;
                                break;
                            }
                            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                            bd = d_w + (uint64_t)(ws * 3 * wbox_units);
                        }
                        const uint32_t bstep = p.resident ? (uint32_t)p.cw * wbox_units : wbox_units;   // from tap kx to tap kx + 1
#pragma unroll
                        for (int t = 0; t < np; t++) {
                            // tap (ky, kx): the halo read from pixel ky * P + kx on; 32 bytes of K per MMA
                            const uint64_t ad = d_halo + (uint64_t)(slot[t] * halo_units + ky * row_units);
#pragma unroll
                            for (int kx = 0; kx < 3; kx++) {
                                mma_i8_ss(d_tmem[t], ad + kx * 4, bd + kx * bstep, idesc, kx ? 1u : accum);
                                mma_i8_ss(d_tmem[t], ad + kx * 4 + 2, bd + kx * bstep + 16, idesc, 1u);
                            }
                        }
                        accum = 1u;
                        if (!p.resident) {
                            umma_commit(&w_empty[ws]);
                            if (++ws == (uint32_t)p.wstages) { ws = 0; wpar ^= 1u; }
                        }
                    }
                    if (ok)
                        for (int t = 0; t < np; t++) umma_commit(&halo_empty[slot[t]]);
                }
                if (ok)
                    for (int t = 0; t < np; t++) umma_commit(&bar_acc_full[(i + t) % U8_ACCS]);
            }
        }
    } else {
        // =========================== epilogue ===========================
        // As in bconv_u8.cuh: blocks of 64 channels through p.stiles fp32 staging tiles, the shortcut prefetched by cp.async,
        // one TMA tensor store per 32-channel box, sign bytes and packed bits straight from registers.  Accumulator row r is
        // halo pixel r: output row r / P of the tile, column r % P; it has a pixel when the column is below OW.
        const int et = tid - 96, ew = warp - 3;
        const int r = (warp & 3) * 32 + lane, hq = ew >> 2;   // TMEM lane quarter of a warp = warp % 4; column quarter 0..3
        const int second = (p.imgs == 2 && r >= p.img_pitch) ? 1 : 0, rr = r - second * p.img_pitch;   // which image of the tile
        const int orow = rr / p.P, ocol = rr - orow * p.P;
        const bool has_px = ocol < p.OW && orow < p.rows;
        const int m = (second * p.rows + orow) * p.OW + ocol;   // the pixel's index within the tile (dense), its staging row
        const uint32_t sbuf0_addr = smem_u32(sbuf0);
        const int nblk = (n_this + 63) >> 6;
        const int first_tile = blockIdx.x * np;
        auto next_tile = [&](int tile, int index) {   // the tile after `tile`, which is this CTA's tile number `index`
            return np == 1 ? tile + (int)gridDim.x : ((index & 1) ? tile + 2 * (int)gridDim.x - 1 : tile + 1);
        };
        int my_tiles = 0;
        for (int t = first_tile, k = 0; t < p.ntiles; t = next_tile(t, k++)) my_tiles++;
        const int total_blocks = my_tiles * nblk;
        auto tile_span = [&](int tile, long long& base, int& nvalid, int& img0, int& oh0) {
            if (p.imgs == 2) {   // whole images, the last tile may hold one
                img0 = tile * 2; oh0 = 0;
                base = (long long)img0 * p.OH * p.OW;
                nvalid = max(0, min(2, p.B - img0)) * p.OH * p.OW;
                return;
            }
            img0 = tile / p.tiles_per_img; oh0 = (tile - img0 * p.tiles_per_img) * p.rows;
            base = ((long long)img0 * p.OH + oh0) * p.OW;
            nvalid = min(p.rows, p.OH - oh0) * p.OW;
        };
        // The shortcut of block kb + stiles - 1 is fetched into the staging tile that block kb - 1 has left, by one thread and
        // two tiled TMA loads (the tile's layout is the one the tensor store reads, so the sum happens in place).
        int pkb = 0, ptile = first_tile, pti = 0, pblk = 0, pst = 0;
        auto prefetch_next = [&]() {   // thread et == 0 only
            if (p.shortcut && pkb < total_blocks) {
                const int pimg = p.imgs == 2 ? ptile * 2 : ptile / p.tiles_per_img, poh0 = p.imgs == 2 ? 0 : (ptile - pimg * p.tiles_per_img) * p.rows;
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
            if (et == 0) {   // the tile the next shortcut goes to is idle once the stores of block kb - 1 - lag have read it
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
                const bool valid = has_px && m < nvalid;   // the last tile of an image may have fewer rows
                if (valid) {
                    // chunk qq (4 channels) of this pixel's row in box hq / 2: srow + ((qq ^ (m & 7)) << 4)
                    const uint32_t srow = sb + (hq >> 1) * sbox_bytes + m * 128;
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
                        const uint32_t sa = srow + ((((hq & 1) * 4 + q) ^ (m & 7)) << 4);
                        if (p.shortcut) {
                            const float4 ad = lds128f(sa);
                            o[0] = __fadd_rn(ad.x, o[0]); o[1] = __fadd_rn(ad.y, o[1]);
                            o[2] = __fadd_rn(ad.z, o[2]); o[3] = __fadd_rn(ad.w, o[3]);
                        }
                        sts128f(sa, o[0], o[1], o[2], o[3]);
                        signs |= ((o[0] > 0.f ? 1u : 0u) | (o[1] > 0.f ? 2u : 0u) | (o[2] > 0.f ? 4u : 0u) | (o[3] > 0.f ? 8u : 0u)) << (q * 4);
                    }
                    const long long row = base + m;
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
            // ---- write-out: one tensor store per 32-channel box; pixels beyond the image and channels beyond N are clipped ----
            if (p.pool_out) {
                // 2x2 average pooling of the staged block: task = pooled pixel (prow, pcol) x four channels
                const int pw = p.OW >> 1, q = et & 15, pp = et >> 4;
                const int prow = pp / pw, pcol = pp - prow * pw;
                if (prow < (p.rows >> 1) && (2 * prow + 1) * p.OW < nvalid && q * 4 < width) {
                    const uint32_t box = sb + (q >> 3) * sbox_bytes;
                    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int tap = 0; tap < 4; tap++) {   // the reference's order: (0,0), (0,1), (1,0), (1,1)
                        const int mm = (2 * prow + (tap >> 1)) * p.OW + 2 * pcol + (tap & 1);
                        const float4 t = lds128f(box + mm * 128 + (((q & 7) ^ (mm & 7)) << 4));
                        acc.x = __fadd_rn(acc.x, t.x); acc.y = __fadd_rn(acc.y, t.y); acc.z = __fadd_rn(acc.z, t.z); acc.w = __fadd_rn(acc.w, t.w);
                    }
                    const size_t e = ((((size_t)img0 * (p.OH >> 1) + (oh0 >> 1) + prow) * pw) + pcol) * p.N + n0 + cb + q * 4;
                    *reinterpret_cast<float4*>(p.pool_out + e) =
                        make_float4(__fdiv_rn(acc.x, 4.f), __fdiv_rn(acc.y, 4.f), __fdiv_rn(acc.z, 4.f), __fdiv_rn(acc.w, 4.f));
                }
                asm volatile("bar.sync 1, %0;" ::"n"(U8_EPILOGUE) : "memory");   // the tile has been read: it may be given back
            }
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
    if (warp == 2) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols));
    }
}

}  // namespace dabnn
