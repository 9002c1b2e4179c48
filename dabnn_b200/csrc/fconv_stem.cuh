// Float convolution of a thin input (at most 4 channels, horizontal stride 2: the 7x7 stride-2 stem of a ResNet)
// on tcgen05.mma kind::tf32 with fp32-grade accuracy (3xTF32, see fconv_tc5.cuh), in which NO thread builds the
// im2col operand: the tensor core reads the convolution windows straight out of the input rows.
//
// An input row is kept in shared memory once, zero-padded left and right and with every pixel widened to four
// floats (16 bytes).  The K slice of tap pair (kx = 2j, 2j + 1) of output pixel ox in input row ky is then the
// 32 contiguous bytes at  row(ky) + (2 ox + 2 j) * 16 : consecutive output pixels lie 32 bytes apart, which is
// exactly the row pitch of a K-major SWIZZLE_32B operand (8-row groups of 256 bytes).  So the A operand of slice
// (ky, j) for a whole output row is the shared-memory descriptor {start = row(ky) + j * 32, SBO = 256}; the
// overlap between the windows of neighbouring pixels is overlap between operand rows of different instructions.
// The 32-byte swizzle XORs address bit 4 with address bit 7 of the final shared-memory address, whatever the start
// address, so the rows are stored with that XOR applied and any start offset reads them back in order.
// K = kh * (kw rounded up to even) * 4 per output pixel (224 for 7x7x3, against 147 real products).
// 3xTF32 needs  head x [W_head; W_rem]  and  remainder x W_head.  The fourth float of a pixel (the input has at most
// three channels) carries channel 0's remainder and meets channel 0's weight head there, so the first product brings a
// third of the second along for nothing; the remainders of channels 1 and 2 form a second plane of 8-byte entries,
// read the same way without swizzle (row pitch 16 bytes, the row's second 16 bytes addressed as the "next core matrix"
// 16 bytes on), with half the K.  Per window row of a 7x7 stem: four N = 128 instructions and two N = 64 ones, where
// full-width remainder planes took four of each - the kernel is bound by the operand bytes the tensor core pulls out of
// shared memory and by the shared-memory traffic of the other roles, not by the arithmetic.
//
// A CTA (one per SM) walks consecutive output rows of consecutive images; a tile is one output row (up to 128
// pixels).  Input rows live in a ring of slots (the two planes of the 3xTF32 split each), so a new output row
// converts only the stride_h input rows that entered its window.  Roles, meeting only at mbarriers:
//   * 4 converter warps: thread x loads pixels x and x + 128 of the next input rows straight from global memory
//     (three row jobs in flight per thread), splits each float into its tf32 head and the remainder, and stores the
//     two 16-byte entries; once per tile a warp arrives on the tile's "rows ready" barrier.  The ring has room for the
//     windows of two tiles beyond the one being multiplied; a slot is overwritten only after the tile that last read
//     it has been committed by the tensor core;
//   * 1 MMA warp: one lane issues per slice  head x [W_head; W_rem]  (one N = 128 instruction, the remainder rows of the
//     resident weights follow the head rows) and per two slices  remainder x W_head  into one of four TMEM accumulators,
//     then one commit per tile;
//   * 16 epilogue warps, thread (pixel, 16-channel quarter), in two groups of eight, one per 32-channel box:
//     tcgen05.ld, add the two column halves, bias, affine, relu, park the row in the group's 128-byte-swizzled
//     staging box, one TMA tensor store per box.
// With POOL the 3x3 stride-2 pad-1 max pooling that follows a ResNet stem happens in the same kernel and the stem's own
// output never leaves the SM: a CTA's share is a run of POOLED rows, the stem rows under them arrive in order (the
// first one computed again by the neighbour that shares it).  An epilogue thread meets the same pixel column in every
// row, so it folds the window's rows in registers with the reference's `acc < t ? t : acc` rule; every second stem row
// completes a pooled row, which alone is parked in the staging boxes, folded over its three columns and written out as
// fp32 and as {0,1} sign bytes.  The values are those of the two layers run one after the other (the maximum does not
// depend on the order of the fold; the only freedom is which zero comes out of a window whose maximum is both +0 and
// -0, where the reference's tap order is row-major and this one is column-major).
// Every wait is bounded; a wait that gives up records a code (31 converters, 32 / 33 MMA thread waiting for rows /
// for an accumulator, 34 epilogue), raises the CTA's abort flag, and the CTA frees its tensor memory and returns.
// Inputs must be finite: a non-finite pixel also poisons the output pixel whose zero-weight odd tap covers it.
#pragma once
#include "fconv_tc5.cuh"

namespace dabnn {

constexpr int FS_CONVERTERS = 128, FS_EPILOGUE = 512;
constexpr int FS_MAX_W = 2 * FS_CONVERTERS;   // a converter thread handles two pixels of an input row
constexpr int FS_CONV_WARPS = FS_CONVERTERS / 32;
constexpr int FS_THREADS = FS_CONVERTERS + FS_EPILOGUE + 32;
constexpr int FS_MMA_WARP = (FS_CONVERTERS + FS_EPILOGUE) / 32;
constexpr int FS_ACCS = 4;
constexpr int FS_N = 64;          // channel block of a CTA
constexpr int FS_PREFETCH = 3;    // row jobs whose global loads a converter thread keeps in flight
constexpr int FS_POOL_TASKS = 2;  // POOL: (pooled column, four channels) tasks of an epilogue thread: pw * 8 <= 256 * FS_POOL_TASKS

struct FsGeom {
    int kxp;                      // taps per window row, rounded up to even
    int kpad;                     // kh * kxp * 4: K of the main contraction
    int kxp2, kpad2;              // taps per window row rounded up to a multiple of four; kh * kxp2 * 2: K of the remainder contraction
    int plane_bytes, slot_bytes;  // one padded input row as 16-byte entries; that plane + the plane of 8-byte remainder entries
    int slots;                    // ring of input-row slots: kh + ahead * stride_h
    int ahead;                    // tiles whose windows may be converted beyond the one being multiplied (1 or 2)
    int srows;                    // rows of a staging box (ow rounded up to 8)
    int rows_total;               // rows shared out among the CTAs: n * oh output rows, n * ph pooled rows with POOL
    int ph, pw;                   // POOL: pooled rows and columns per image
};

__host__ __device__ inline int fs_weight_bytes(int kpad) { return 2 * (FS_N / 8) * (kpad / 4) * 128; }
__host__ __device__ inline int fs_weight2_bytes(int kpad2) { return (FS_N / 8) * (kpad2 / 4) * 128; }
__host__ __device__ inline int fs_smem_bytes(const FsGeom& g) {
    return 1024 + g.slots * g.slot_bytes + fs_weight_bytes(g.kpad) + fs_weight2_bytes(g.kpad2) + 1024 + 2 * g.srows * 128;
}
__device__ __forceinline__ void sts64(uint32_t addr, uint32_t x, uint32_t y) {
    asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(x), "r"(y) : "memory");
}
// the reference's max-pool fold (MaxPool.cpp:209-246): keeps the earlier value on ties, never picks a NaN
__device__ __forceinline__ float4 fs_sel(const float4 a, const float4 t) {
    return make_float4(a.x < t.x ? t.x : a.x, a.y < t.y ? t.y : a.y, a.z < t.z ? t.z : a.z, a.w < t.w ? t.w : a.w);
}

// K-major SWIZZLE_32B shared-memory descriptor: rows of 32 bytes, 8-row groups 256 bytes apart
__device__ __forceinline__ uint64_t umma_desc_sw32(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)1 << 16) | ((uint64_t)(256 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)6 << 61);
}
// where the 16-byte entry at byte address a of a SWIZZLE_32B operand is stored
__device__ __forceinline__ uint32_t sw32(uint32_t a) { return a ^ (((a >> 7) & 1u) << 4); }

// The CTA's tiles in order: output row g of the whole batch, its image and row, and which input rows (numbered by a
// running sequence, slot = sequence mod slots) its window covers.  Converters and the MMA thread step identical copies.
struct FsTileIter {
    int t, img, oy;       // tile number within the CTA, image, output row
    int q0, s0;           // sequence number and slot of the window's first input row
    int next_q;           // first sequence number not yet converted when the tile begins
    bool fresh;           // the window shares no row with the previous tile's
    __device__ __forceinline__ void init(int g_begin, int oh) {
        t = 0; img = g_begin / oh; oy = g_begin - img * oh; q0 = 0; s0 = 0; next_q = 0; fresh = true;
    }
    __device__ __forceinline__ void advance(int oh, int kh, int sh, int slots) {
        next_q = q0 + kh;
        t++;
        bool f = sh >= kh;
        if (++oy == oh) { oy = 0; img++; f = true; }
        const int step = f ? kh : sh;
        q0 += step;
        s0 += step;
        while (s0 >= slots) s0 -= slots;
        fresh = f;
    }
    __device__ __forceinline__ int first_new() const { return fresh ? q0 : next_q; }
};

// SLICES: tap pairs per window row (kxp / 2), a compile-time count lets the issue loop unroll.  POOL: see above; the
// result goes to pool_out (fp32 [n][ph][pw][cout]) and, if not null, pool_u8 (its signs as bytes) instead of p.out.
template <int SLICES, bool POOL>
__global__ void __launch_bounds__(FS_THREADS, 1)
    fconv_stem_kernel(const FconvParams p, const FsGeom g, const __grid_constant__ CUtensorMap out_map, float* __restrict__ pool_out,
                      unsigned char* __restrict__ pool_u8) {
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) uint64_t rows_ready[4], tile_done[FS_ACCS], acc_empty[FS_ACCS];
    __shared__ uint32_t tmem_base_s;
    __shared__ int s_abort, epi_abort[2];
    __shared__ __align__(16) float chan_bias[FS_N], chan_a[FS_N], chan_b[FS_N];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.y * FS_N;
    const int n_this = min(FS_N, p.cout - n0);                  // multiple of 16 (host-checked)
    unsigned char* patch = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
    unsigned char* wbase = patch + g.slots * g.slot_bytes;
    const int w_sbo = (g.kpad / 4) * 128, w_half = (FS_N / 8) * w_sbo;
    unsigned char* w2base = wbase + 2 * w_half;                 // the remainder contraction's weights: heads of channels 1 and 2
    const int w2_sbo = (g.kpad2 / 4) * 128;
    unsigned char* stile = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(w2base + (FS_N / 8) * w2_sbo) + 1023) & ~uintptr_t(1023));
    const int sbox_bytes = g.srows * 128;
    const volatile int* abort_flag = &s_abort;
    constexpr int ACC_COLS = 2 * FS_N, TMEM_COLS = FS_ACCS * ACC_COLS;   // 512 columns: all of the tensor memory

    // this CTA's rows: an even share of n * oh output rows - or of n * ph pooled rows, and then the output rows under them
    // (pooled row py covers output rows 2 py - 1 .. 2 py + 1: consecutive pooled rows share one, so the run of output rows
    // is contiguous and starts one row early)
    const int per = g.rows_total / gridDim.x, extra = g.rows_total - per * gridDim.x;
    const int share_begin = blockIdx.x * per + min((int)blockIdx.x, extra);
    const int share = per + ((int)blockIdx.x < extra ? 1 : 0);
    int g_begin = share_begin, ntiles = share;
    if (POOL && share > 0) {
        const int i0 = share_begin / g.ph, py0 = share_begin - i0 * g.ph;
        const int last = share_begin + share - 1, i1 = last / g.ph, py1 = last - i1 * g.ph;
        g_begin = i0 * p.oh + max(0, 2 * py0 - 1);
        ntiles = i1 * p.oh + min(p.oh - 1, 2 * py1 + 1) - g_begin + 1;
    }

    // ---- set-up ----
    if (warp == FS_MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    if (tid == 0) {
        for (int i = 0; i < 4; i++) mbar_init(&rows_ready[i], FS_CONV_WARPS);
        for (int i = 0; i < FS_ACCS; i++) { mbar_init(&tile_done[i], 1); mbar_init(&acc_empty[i], FS_EPILOGUE / 32); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::);
        s_abort = 0;
        epi_abort[0] = epi_abort[1] = 0;
    }
    {   // the padding entries of every slot must read as zero, and nothing the tensor core multiplies may be a stale NaN
        const uint32_t pa = smem_u32(patch);
        for (int i = tid; i < g.slots * g.slot_bytes / 16; i += FS_THREADS) sts128f(pa + i * 16, 0.f, 0.f, 0.f, 0.f);
    }
    if (tid < FS_N) {
        const bool in = tid < n_this;
        chan_bias[tid] = (in && p.bias) ? __ldg(p.bias + n0 + tid) : 0.f;
        chan_a[tid] = (in && p.a) ? __ldg(p.a + n0 + tid) : 1.f;
        chan_b[tid] = (in && p.a) ? __ldg(p.b + n0 + tid) : 0.f;
    }
    // resident weights, K order (ky, kx < kxp, c < 4): element (n, k) -> (n / 8) * w_sbo + (k / 4) * 128 + (n % 8) * 16 + (k % 4) * 4
    // (four elements per thread and step, their loads issued together: the set-up is a fixed cost of every launch)
    for (int idx0 = tid; idx0 < FS_N * g.kpad; idx0 += 4 * FS_THREADS) {
        float v[4];
        int off[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int idx = idx0 + u * FS_THREADS;
            const int n = idx / g.kpad, k = idx - n * g.kpad;
            const int c = k & 3, tap = k >> 2, ky = tap / g.kxp, kx = tap - ky * g.kxp;
            const int cs = c == 3 ? 0 : c;   // the fourth entry of a pixel carries channel 0's remainder: it meets channel 0's head
            v[u] = (idx < FS_N * g.kpad && n < n_this && kx < p.kw && cs < p.cin) ? __ldg(p.wgt + ((size_t)(n0 + n) * p.kh * p.kw + ky * p.kw + kx) * p.cin + cs) : 0.f;
            off[u] = idx < FS_N * g.kpad ? (n >> 3) * w_sbo + (k >> 2) * 128 + (n & 7) * 16 + (k & 3) * 4 : -1;
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            if (off[u] < 0) continue;
            uint32_t hi, lo;
            split_tf32(v[u], hi, lo);
            *reinterpret_cast<uint32_t*>(wbase + off[u]) = hi;
            *reinterpret_cast<uint32_t*>(wbase + w_half + off[u]) = (off[u] & 12) == 12 ? 0u : lo;   // remainder x remainder is dropped
        }
    }
    // the remainder contraction, K order (ky, kx < kxp2, channel 1 or 2): heads of the weights only
    for (int idx0 = tid; idx0 < FS_N * g.kpad2; idx0 += 4 * FS_THREADS) {
        float v[4];
        int off[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int idx = idx0 + u * FS_THREADS;
            const int n = idx / g.kpad2, k = idx - n * g.kpad2;
            const int c = 1 + (k & 1), tap = k >> 1, ky = tap / g.kxp2, kx = tap - ky * g.kxp2;
            v[u] = (idx < FS_N * g.kpad2 && n < n_this && kx < p.kw && c < p.cin) ? __ldg(p.wgt + ((size_t)(n0 + n) * p.kh * p.kw + ky * p.kw + kx) * p.cin + c) : 0.f;
            off[u] = idx < FS_N * g.kpad2 ? (n >> 3) * w2_sbo + (k >> 2) * 128 + (n & 7) * 16 + (k & 3) * 4 : -1;
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            if (off[u] < 0) continue;
            uint32_t hi, lo;
            split_tf32(v[u], hi, lo);
            *reinterpret_cast<uint32_t*>(w2base + off[u]) = hi;
        }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;
    grid_launch_dependents();
    grid_dependency_wait();   // everything above touched constants only; the images and the output buffers come next

    if (tid < FS_CONVERTERS) {
        // =========================== converters: thread = pixel x of an input row ===========================
        const int x = tid;                       // and x + FS_CONVERTERS
        const bool have_px[2] = {x < p.w, x + FS_CONVERTERS < p.w};
        const uint32_t entry0 = smem_u32(patch) + (uint32_t)(x + p.pad_w) * 16u;
        const uint32_t rem0 = smem_u32(patch) + (uint32_t)g.plane_bytes + (uint32_t)(x + p.pad_w) * 8u;
        const long long row_floats = (long long)p.w * p.cin;
        // a cursor over the row jobs (tile by tile, the tile's new rows in order)
        struct Cursor {
            FsTileIter ti;
            int q, slot;   // sequence number of the row and its slot
        };
        auto begin_tile = [&](Cursor& c) {
            c.q = c.ti.first_new();
            c.slot = c.ti.s0 + (c.q - c.ti.q0);
            while (c.slot >= g.slots) c.slot -= g.slots;
        };
        auto next_job = [&](Cursor& c) {
            if (++c.q == c.ti.q0 + p.kh) {
                c.ti.advance(p.oh, p.kh, p.stride_h, g.slots);
                begin_tile(c);
            } else if (++c.slot == g.slots) {
                c.slot = 0;
            }
        };
        auto load = [&](const Cursor& c, float (&v)[8]) {
#pragma unroll
            for (int e = 0; e < 8; e++) v[e] = 0.f;
            if (c.ti.t < ntiles) {
                const int iy = c.ti.oy * p.stride_h - p.pad_h + (c.q - c.ti.q0);
                if ((unsigned)iy < (unsigned)p.h) {
                    const float* src = p.in + ((long long)c.ti.img * p.h + iy) * row_floats + (long long)x * p.cin;
#pragma unroll
                    for (int h = 0; h < 2; h++)
                        if (have_px[h]) {
#pragma unroll
                            for (int ch = 0; ch < 4; ch++)
                                if (ch < p.cin) v[h * 4 + ch] = __ldg(src + (long long)h * FS_CONVERTERS * p.cin + ch);
                        }
                }
            }
        };
        Cursor ld, st;
        ld.ti.init(g_begin, p.oh);
        begin_tile(ld);
        st = ld;
        float pf[FS_PREFETCH][8];
#pragma unroll
        for (int d = 0; d < FS_PREFETCH; d++) { load(ld, pf[d]); next_job(ld); }
        bool ok = true;
        while (st.ti.t < ntiles && ok) {
#pragma unroll
            for (int d = 0; d < FS_PREFETCH; d++) {
                if (st.ti.t >= ntiles || !ok) break;
                const int t = st.ti.t;
                if (st.q == st.ti.first_new()) {
                    // the slots this tile's new rows overwrite were last read by tile t - 1 - ahead (t - 1 when the window starts afresh)
                    const int need = st.ti.fresh ? t - 1 : t - 1 - g.ahead;
                    if (need >= 0 && !__all_sync(0xffffffffu, mbar_wait<100>(&tile_done[need % FS_ACCS], (need / FS_ACCS) & 1, abort_flag))) {
                        atomicCAS(&g_tc5_status, 0, 31);
                        s_abort = 1;
                        ok = false;
                        break;
                    }
                }
#pragma unroll
                for (int h = 0; h < 2; h++)
                    if (have_px[h]) {
                        uint32_t hi[4], lo[4];
#pragma unroll
                        for (int ch = 0; ch < 4; ch++) split_tf32(pf[d][h * 4 + ch], hi[ch], lo[ch]);
                        const uint32_t so = (uint32_t)st.slot * (uint32_t)g.slot_bytes;
                        sts128(sw32(entry0 + so + (uint32_t)h * (FS_CONVERTERS * 16u)), hi[0], hi[1], hi[2], lo[0]);
                        sts64(rem0 + so + (uint32_t)h * (FS_CONVERTERS * 8u), lo[1], lo[2]);
                    }
                if (st.q == st.ti.q0 + p.kh - 1) {   // the tile's window is complete
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&rows_ready[t & 3]);
                }
                next_job(st);
                load(ld, pf[d]);
                next_job(ld);
            }
        }
    } else if (warp == FS_MMA_WARP) {
        // =========================== MMA issue: one lane ===========================
        if (lane == 0) {
            const uint32_t idesc_m = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(128 >> 4) << 24);   // D f32, A = B = tf32, K-major, M = 128
            const uint32_t idesc = idesc_m | ((uint32_t)(n_this >> 3) << 17);
            const bool stacked = n_this == FS_N;
            const uint32_t idesc2 = idesc_m | ((uint32_t)((2 * FS_N) >> 3) << 17);
            const uint64_t d_a = umma_desc_sw32(smem_u32(patch));
            // the remainder plane: 8-byte entries, no swizzle; an operand row is 32 bytes = four taps of two channels, consecutive
            // output pixels lie 16 bytes apart (the row pitch of the plain K-major layout) and the row's second half is the
            // "next core matrix", 16 bytes on
            const uint64_t d_r = umma_desc_kmajor(smem_u32(patch) + g.plane_bytes, 16, 128);
            const uint64_t d_w2 = umma_desc_kmajor(smem_u32(w2base), 128, w2_sbo);
            constexpr int SLICES2 = (SLICES + 1) / 2;
            const uint64_t d_wh = umma_desc_kmajor(smem_u32(wbase), 128, w_sbo), d_wl = umma_desc_kmajor(smem_u32(wbase) + w_half, 128, w_sbo);
            const uint32_t slot_units = (uint32_t)g.slot_bytes >> 4;
            // The issuing thread is one instruction stream and an MMA of this size executes in 50 - 65 cycles: the loop
            // must cost less than that per instruction, so the slices of a window row are unrolled (descriptors advance
            // by constants) and the two forms of the hi product get their own loops.
            FsTileIter it;
            it.init(g_begin, p.oh);
            for (; it.t < ntiles; it.advance(p.oh, p.kh, p.stride_h, g.slots)) {
                const int t = it.t, accbuf = t % FS_ACCS, accuse = t / FS_ACCS;
                if (accuse >= 1 && !mbar_wait(&acc_empty[accbuf], (accuse - 1) & 1, abort_flag)) {
                    atomicCAS(&g_tc5_status, 0, 33);
                    s_abort = 1;
                    break;
                }
                if (!mbar_wait(&rows_ready[t & 3], (t >> 2) & 1, abort_flag)) {   // the issuing thread is the critical path: no sleep between polls
                    atomicCAS(&g_tc5_status, 0, 32);
                    s_abort = 1;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + accbuf * ACC_COLS;
                uint64_t bh = d_wh, bl = d_wl, b2 = d_w2;
                uint32_t accum = 0;
                int slot = it.s0;
                // one slice = eight floats = two 16-byte units per row: 32 bytes of a window row, 256 bytes of the weight layout
                if (stacked) {
                    for (int ky = 0; ky < p.kh; ky++) {
                        const uint64_t ah = d_a + (uint64_t)(slot * slot_units), ar = d_r + (uint64_t)(slot * slot_units);
#pragma unroll
                        for (int j = 0; j < SLICES; j++) mma_tf32_ss(d_tmem, ah + 2 * j, bh + 16 * j, idesc2, j ? 1u : accum);
#pragma unroll
                        for (int j = 0; j < SLICES2; j++) mma_tf32_ss(d_tmem, ar + 2 * j, b2 + 16 * j, idesc, 1u);
                        accum = 1u;
                        bh += 16 * SLICES;
                        b2 += 16 * SLICES2;
                        if (++slot == g.slots) slot = 0;
                    }
                } else {
                    for (int ky = 0; ky < p.kh; ky++) {
                        const uint64_t ah = d_a + (uint64_t)(slot * slot_units), ar = d_r + (uint64_t)(slot * slot_units);
#pragma unroll
                        for (int j = 0; j < SLICES; j++) {
                            mma_tf32_ss(d_tmem, ah + 2 * j, bh + 16 * j, idesc, j ? 1u : accum);
                            mma_tf32_ss(d_tmem + FS_N, ah + 2 * j, bl + 16 * j, idesc, j ? 1u : accum);
                        }
#pragma unroll
                        for (int j = 0; j < SLICES2; j++) mma_tf32_ss(d_tmem, ar + 2 * j, b2 + 16 * j, idesc, 1u);
                        accum = 1u;
                        bh += 16 * SLICES;
                        bl += 16 * SLICES;
                        b2 += 16 * SLICES2;
                        if (++slot == g.slots) slot = 0;
                    }
                }
                umma_commit(&tile_done[accbuf]);   // the accumulator is complete and the window's slots have been read
            }
        }
    } else {
        // =========================== epilogue: two groups of eight warps, one per 32-channel box ===========================
        const int et = tid - FS_CONVERTERS;
        const int r = et & 127, cq = et >> 7;                  // TMEM lane quarter of a warp = warp % 4 = r / 32; 16-channel quarter
        const int h2 = cq >> 1;                                // the 32-channel box this thread works on
        const int ncol = max(0, min(16, n_this - cq * 16));    // 0 or 16 columns for this thread
        const uint32_t sbox = smem_u32(stile) + h2 * sbox_bytes;
        const bool staged = r < g.srows;
        const bool elected = (et & 255) == 0;                  // one thread per box issues its stores
        const int bar_id = 1 + h2;
        // POOL: a thread sees the same pixel column and channels in every tile, so the vertical part of the pooling window
        // - the maximum over the output rows 2 py - 1, 2 py, 2 py + 1 of pooled row py - is a fold in registers, in row order
        // and with the reference's rule; only a completed row goes through shared memory for the three horizontal taps.
        float vmax[16];
#pragma unroll
        for (int e = 0; e < 16; e++) vmax[e] = 0.f;
        int img = g_begin / p.oh, oy = g_begin - img * p.oh;
        for (int t = 0; t < ntiles; t++, oy = oy + 1 == p.oh ? (img++, 0) : oy + 1) {
            const int accbuf = t % FS_ACCS, accuse = t / FS_ACCS;
            const bool okw = __all_sync(0xffffffffu, mbar_wait<200>(&tile_done[accbuf], accuse & 1, abort_flag));   // warp-uniform
            if (!okw) {
                atomicCAS(&g_tc5_status, 0, 34);
                s_abort = 1;
                epi_abort[h2] = 1;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t v[16];   // accumulator columns, then the finished outputs
            if (okw && ncol > 0) {
                const uint32_t t_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + accbuf * ACC_COLS + cq * 16;
#pragma unroll
                for (int half = 0; half < 2; half++) {   // eight columns at a time: the running maxima need the registers
                    uint32_t* y = v + half * 8;
                    uint32_t xx[8];
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                                 : "=r"(y[0]), "=r"(y[1]), "=r"(y[2]), "=r"(y[3]), "=r"(y[4]), "=r"(y[5]), "=r"(y[6]), "=r"(y[7])
                                 : "r"(t_addr + half * 8));
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                                 : "=r"(xx[0]), "=r"(xx[1]), "=r"(xx[2]), "=r"(xx[3]), "=r"(xx[4]), "=r"(xx[5]), "=r"(xx[6]), "=r"(xx[7])
                                 : "r"(t_addr + FS_N + half * 8));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int q = 0; q < 2; q++) {   // the channel constants four at a time: every shared-memory wavefront counts here
                        const int cl = cq * 16 + half * 8 + q * 4;
                        const float4 cbias = *reinterpret_cast<const float4*>(chan_bias + cl), ca = *reinterpret_cast<const float4*>(chan_a + cl),
                                     cb = *reinterpret_cast<const float4*>(chan_b + cl);
                        const float kb[4] = {cbias.x, cbias.y, cbias.z, cbias.w}, ka[4] = {ca.x, ca.y, ca.z, ca.w}, kc[4] = {cb.x, cb.y, cb.z, cb.w};
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            float f = __uint_as_float(y[q * 4 + e]) + __uint_as_float(xx[q * 4 + e]);   // + the hi*lo part
                            if (p.bias) f = __fadd_rn(f, kb[e]);
                            if (p.a) f = __fadd_rn(__fmul_rn(ka[e], f), kc[e]);
                            if (p.relu) f = relu_ref(f);
                            y[q * 4 + e] = __float_as_uint(f);
                        }
                    }
                }
            }
            if (okw) {   // the accumulator is in registers: the MMA warp may reuse it
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[accbuf]);
            }
            if (POOL) {
                // Output row oy is the middle row of pooled row oy / 2 when even, and when odd the last row of pooled row
                // (oy - 1) / 2 and the first of the next: an odd row completes a pooled row (unless it is the CTA's first: that
                // pooled row is the neighbour's), and so does an image's last row.
                const bool odd = (oy & 1) != 0, prelude = odd && t == 0;
                const bool emit = (odd && !prelude) || (!odd && oy == p.oh - 1);
                const bool init = prelude || oy == 0;
                if (okw && ncol > 0) {
#pragma unroll
                    for (int e = 0; e < 16; e++) {
                        const float f = __uint_as_float(v[e]);
                        vmax[e] = init ? f : (vmax[e] < f ? f : vmax[e]);
                    }
                }
                if (!emit) continue;   // (a warp that gave up runs on, idle, to the next barrier and leaves with its group)
                asm volatile("bar.sync %0, 256;" ::"r"(bar_id) : "memory");   // everybody has read the previous completed row
                if (epi_abort[h2]) break;
                if (staged && ncol > 0) {
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const int chunk = (cq & 1) * 4 + q;   // 16-byte chunk of the pixel's 128-byte row in the box
                        sts128f(sbox + r * 128 + ((chunk ^ (r & 7)) << 4), vmax[q * 4], vmax[q * 4 + 1], vmax[q * 4 + 2], vmax[q * 4 + 3]);
                    }
#pragma unroll
                    for (int e = 0; e < 16; e++) vmax[e] = __uint_as_float(v[e]);   // an odd row also opens the next pooled row
                }
                asm volatile("bar.sync %0, 256;" ::"r"(bar_id) : "memory");
#pragma unroll
                for (int i = 0; i < FS_POOL_TASKS; i++) {   // task: pooled column px, four channels
                    const int k = (et & 255) + 256 * i;
                    const int px = k >> 3, q = k & 7;
                    if (k >= g.pw * 8 || h2 * 32 + q * 4 >= n_this) continue;
                    float4 h = make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX);
#pragma unroll
                    for (int dx = -1; dx <= 1; dx++) {   // the reference skips taps outside the image
                        const int ox = 2 * px + dx;
                        if ((unsigned)ox < (unsigned)p.ow) h = fs_sel(h, lds128f(sbox + ox * 128 + ((q ^ (ox & 7)) << 4)));
                    }
                    const size_t e = (((size_t)img * g.ph + (oy >> 1)) * g.pw + px) * p.cout + n0 + h2 * 32 + q * 4;
                    *reinterpret_cast<float4*>(pool_out + e) = h;
                    if (pool_u8)
                        *reinterpret_cast<uint32_t*>(pool_u8 + e) =
                            (h.x > 0.f ? 1u : 0u) | (h.y > 0.f ? 0x100u : 0u) | (h.z > 0.f ? 0x10000u : 0u) | (h.w > 0.f ? 0x1000000u : 0u);
                }
                continue;
            }
            if (elected) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the previous tile's store has read the box
            asm volatile("bar.sync %0, 256;" ::"r"(bar_id) : "memory");
            if (epi_abort[h2]) break;
            if (staged && ncol > 0) {
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const int chunk = (cq & 1) * 4 + q;   // 16-byte chunk of the pixel's 128-byte row in the box
                    sts128(sbox + r * 128 + ((chunk ^ (r & 7)) << 4), v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the tensor store below reads what was just written
            }
            asm volatile("bar.sync %0, 256;" ::"r"(bar_id) : "memory");
            // one tensor store per box; the descriptor is [output row of the batch][pixel][channel]: pixels beyond the row
            // and channels beyond Cout are clipped
            if (elected && n_this > h2 * 32) {
                asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];"
                             ::"l"(reinterpret_cast<uint64_t>(&out_map)), "r"(n0 + h2 * 32), "r"(0), "r"(g_begin + t), "r"(sbox) : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
        }
    }

    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // the stores are complete before the CTA winds down
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == FS_MMA_WARP) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS));
    }
}

}  // namespace dabnn
