// Binary contraction core shared by bgemm and the binary convolutions.
//
//   cnt[p][n] = sum over K bits of  X[p][k] XOR Wt[n][k]        (p: pixel rows, n: output channels)
//
// X rows and Wt rows are streamed K-chunk by K-chunk (16 uint64 words = 1024 bits per stage) into
// shared memory with 8-byte cp.async copies (zero-filled outside the operand, which is exactly the
// reference's "padding = zero word" rule) through a 3-stage pipeline.  Three engines consume the
// same shared-memory tiles and give identical integers:
//
//   POPC  CUDA cores: xor + popc per 64-bit word.
//   B1    mma.sync.m16n8k256 b1 AND-popc.  xor = popc(x) + popc(w) - 2*and; the row popcounts are
//         accumulated from the shared-memory tiles while they are resident.
//   IMMA  mma.sync.m16n8k32 u8: each 32-bit chunk of a row is expanded in registers to {0,1} bytes
//         ((chunk >> t) & 0x01010101), so the int8 tensor-core path computes the same AND count.
//         Both operands use the same bit -> k-slot permutation, which a contraction is blind to.
//
// On B200 the b1 MMA is not a native tensor-core instruction any more (it runs at about 0.4
// Pbit-op/s, the int8 MMA at about 1.1 and CUDA-core popc at about 0.28), which is why IMMA is
// the default engine.
//
// The accumulators are turned into counts and written straight from the MMA fragment layout by an
// epilogue that can also apply the per-channel affine, add the shortcut and emit the sign bits of
// the result (the next layer's packed input).
#pragma once
#include "common.cuh"

namespace dabnn {

constexpr int KC_WORDS = 16;               // uint64 words of K per pipeline stage
constexpr int PITCH32 = KC_WORDS * 2 + 4;  // row pitch in 32-bit units (144 B): 8 rows x 64-bit reads hit 16 distinct banks
constexpr int NSTAGES = 2;                 // two CTAs of 4 warps fit one SM (shared memory and registers)

enum { ENG_POPC = DABNN_ENGINE_POPC, ENG_B1 = DABNN_ENGINE_B1, ENG_IMMA = DABNN_ENGINE_IMMA };

// ---- operand addressing ------------------------------------------------------------------------
// A loader thread owns one pair of K words (w, w+1; w even) of the current chunk for many rows.
// decode() is called once per chunk for each word of the pair, addr() once per row.
struct RowCtx {
    long long base;  // row-major/col-major: element offset of the row; conv: pixel index of image start
    int iy0, ix0;    // conv: top-left input coordinate of the receptive field
    int valid;
};

// rows contiguous: element (row, word) at p[row*ld + word]
struct RowMajorOperand {
    const uint64_t* p;
    long long ld;
    int rows, kwords;
    struct Dec { int word; };
    __device__ bool pairable() const { return (ld & 1) == 0 && (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
    __device__ Dec decode(int word) const { return Dec{word}; }
    __device__ void advance(Dec& d, int words) const { d.word += words; }
    __device__ RowCtx make_row(int row) const { return RowCtx{(long long)row * ld, 0, 0, row < rows}; }
    __device__ const uint64_t* addr(const RowCtx& r, const Dec& d) const { return r.valid ? p + r.base + d.word : nullptr; }
};
// the reference bgemm's `a`: element (row i, word h) at p[h*ld + i]
struct ColMajorOperand {
    const uint64_t* p;
    long long ld;
    int rows, kwords;
    struct Dec { long long off; };
    __device__ bool pairable() const { return false; }
    __device__ Dec decode(int word) const { return Dec{(long long)word * ld}; }
    __device__ void advance(Dec& d, int words) const { d.off += (long long)words * ld; }
    __device__ RowCtx make_row(int row) const { return RowCtx{(long long)row, 0, 0, row < rows}; }
    __device__ const uint64_t* addr(const RowCtx& r, const Dec& d) const { return r.valid ? p + d.off + r.base : nullptr; }
};
// implicit im2col over packed NHWC bits: row = output pixel, word = (ky*kw + kx)*Cw + cw
struct ConvOperand {
    const uint64_t* p;
    int n, H, W, Cw, OH, OW, kh, kw, pad_h, pad_w, stride_h, stride_w;
    int rows, kwords;
    struct Dec { int ky, kx, cw; };
    __device__ bool pairable() const { return (Cw & 1) == 0 && (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
    __device__ Dec decode(int word) const {
        const int tap = word / Cw, ky = tap / kw;
        return Dec{ky, tap - ky * kw, word - tap * Cw};
    }
    // step the decode of word q to word q + words without a division (words is small)
    __device__ void advance(Dec& d, int words) const {
        d.cw += words;
        while (d.cw >= Cw) {
            d.cw -= Cw;
            if (++d.kx == kw) { d.kx = 0; ++d.ky; }
        }
    }
    __device__ RowCtx make_row(int row) const {
        RowCtx r;
        r.valid = row < rows;
        const int img = row / (OH * OW), rem = row - img * (OH * OW);
        const int oy = rem / OW, ox = rem - oy * OW;
        r.base = (long long)img * H * W;
        r.iy0 = oy * stride_h - pad_h;
        r.ix0 = ox * stride_w - pad_w;
        return r;
    }
    __device__ const uint64_t* addr(const RowCtx& r, const Dec& d) const {
        const int y = r.iy0 + d.ky, x = r.ix0 + d.kx;
        if (!r.valid || (unsigned)y >= (unsigned)H || (unsigned)x >= (unsigned)W) return nullptr;
        return p + (r.base + (long long)y * W + x) * Cw + d.cw;
    }
};

// ---- epilogue ------------------------------------------------------------------------------------
struct EpilogueParams {
    float* out;            // fp32 [rows][ld_out] or nullptr
    long long ld_out;
    int accumulate;        // 1: out += cnt (bgemm), 0: out = value
    const float* a;        // per-channel affine (nullptr: none): v = a[n]*cnt + b[n]
    const float* b;
    const float* shortcut; // fp32 [rows][ld_sc] added after the affine, or nullptr
    long long ld_sc;
    uint64_t* bits;        // sign bits of the final value, [rows][ld_bits words], or nullptr
    long long ld_bits;
    // TCGEN05 engine only (not an epilogue matter, but it travels with the launch): the weights already expanded
    // to bytes in the engine's shared-memory stage layout (tc5_expand_weights), or nullptr to expand them per tile
    const unsigned char* w_expanded;
};

__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void mma_b1_and(int* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                           uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k256.row.col.s32.b1.b1.s32.and.popc {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_u8(int* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// exact int -> float for 0 <= v < 2^23 on the FP32 pipe (I2F runs on the quarter-rate XU pipe)
__device__ __forceinline__ float small_int_to_float(int v) {
    return __fsub_rn(__int_as_float(0x4B000000 | v), 8388608.0f);
}

// A CTA has WM x WN warps; every warp owns a 32-pixel x 64-channel sub-tile (2 x 8 MMA tiles).
template <int WM, int WN>
struct TileCfg {
    static constexpr int TM = WM * 32, TN = WN * 64, NT = WM * WN * 32;
    static constexpr int STAGE_U32 = (TM + TN) * PITCH32;
    static constexpr size_t PIPE_BYTES = (size_t)NSTAGES * STAGE_U32 * 4;
    // two sets of pixel-row contexts (current / next tile), one set of channel-row contexts, row popcounts
    static constexpr size_t SMEM_BYTES = PIPE_BYTES + (size_t)(2 * TM + TN) * sizeof(RowCtx) + (size_t)(TM + TN) * sizeof(int) +
                                         (size_t)2 * TN * sizeof(float);
};

// Copies one K chunk of `NROWS` operand rows into a pipeline stage.  Thread t owns word pair
// (t & 7) of the chunk for rows (t >> 3), (t >> 3) + NT/8, ...
template <int NROWS, int NT, class Op>
__device__ __forceinline__ void load_rows(const Op& op, const RowCtx* ctx, uint32_t stage_addr, int w0,
                                          int kwords, int kfill, bool pair_ok, int tid) {
    const int wp = tid & 7, w = w0 + 2 * wp;
    if (w >= kfill) return;
    const bool v0 = w < kwords, v1 = w + 1 < kwords, f1 = w + 1 < kfill;
    const typename Op::Dec d0 = op.decode(v0 ? w : 0), d1 = op.decode(v1 ? w + 1 : 0);
    const uint32_t col = stage_addr + wp * 16;
    if (pair_ok && v1) {
#pragma unroll 4
        for (int r = tid >> 3; r < NROWS; r += NT / 8) {
            const uint64_t* src = op.addr(ctx[r], d0);
            cp_async16(col + r * (PITCH32 * 4), src ? (const void*)src : (const void*)op.p, src ? 16 : 0);
        }
    } else {
#pragma unroll 4
        for (int r = tid >> 3; r < NROWS; r += NT / 8) {
            const RowCtx c = ctx[r];
            const uint64_t* s0 = v0 ? op.addr(c, d0) : nullptr;
            cp_async8(col + r * (PITCH32 * 4), s0 ? (const void*)s0 : (const void*)op.p, s0 ? 8 : 0);
            if (f1) {
                const uint64_t* s1 = v1 ? op.addr(c, d1) : nullptr;
                cp_async8(col + r * (PITCH32 * 4) + 8, s1 ? (const void*)s1 : (const void*)op.p, s1 ? 8 : 0);
            }
        }
    }
}

// Persistent kernel.  CTA (bx, by) owns channel tile `by` and walks pixel tiles bx, bx + gridDim.x,
// ...; each tile is TM pixels x TN channels, each of the 8 warps a 32 x 64 sub-tile.  While a tile
// is being computed and written out, the first K chunk of the next tile is already in flight.
// Two CTAs (16 warps) share an SM; the register budget is 128 per thread.
//
// Accumulator layout (all engines): acc[(mt*8 + nt)*4 + h*2 + q] is pixel row mt*16 + g + 8*h,
// channel nt*8 + 2*tig + q of the warp's sub-tile (g = lane / 4, tig = lane % 4), the fragment
// layout of mma.sync.  The epilogue works straight from these registers: per m-tile it first
// issues all shortcut loads (16 independent 8-byte loads per thread), then converts, applies the
// affine, adds, stores, and ORs the sign bits of a row together across the four lanes of a quad.
//
// FAST = true assumes N % 8 == 0 and 8-byte aligned, even-pitched output / shortcut rows (every
// network layer); FAST = false handles any N and alignment with scalar accesses.
template <int ENGINE, int WM, int WN, bool FAST, class XOp, class WOp>
__global__ void __launch_bounds__(WM* WN * 32, 2)
    bcontract_kernel(const XOp xop, const WOp wop, const EpilogueParams ep, const int M, const int N,
                     const int kwords, const int ntiles_m) {
    using Cfg = TileCfg<WM, WN>;
    constexpr int TM = Cfg::TM, TN = Cfg::TN, NT = Cfg::NT, ROWS = TM + TN;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint32_t* pipe = reinterpret_cast<uint32_t*>(smem_raw);
    RowCtx* xctx = reinterpret_cast<RowCtx*>(smem_raw + Cfg::PIPE_BYTES);  // [2][TM]
    RowCtx* wctx = xctx + 2 * TM;                                           // [TN]
    int* rowpop = reinterpret_cast<int*>(wctx + TN);                        // [TM + TN]
    float* chan_a = reinterpret_cast<float*>(rowpop + ROWS);                // [TN] affine scale
    float* chan_b = chan_a + TN;                                            // [TN] affine shift

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, tig = lane & 3;
    const int wm = warp / WN, wn = warp % WN;
    const int n0 = blockIdx.y * TN;
    int tile = blockIdx.x;
    if (tile >= ntiles_m) return;

    constexpr bool MMA = ENGINE != ENG_POPC;
    // the b1 MMA consumes 4 words per step: its K tail is zero-filled up to a multiple of 4 words
    const int kfill = ENGINE == ENG_B1 ? (kwords + 3) / 4 * 4 : kwords;
    const int nchunks = (kwords + KC_WORDS - 1) / KC_WORDS;
    const bool xpair = xop.pairable(), wpair = wop.pairable();

    for (int r = tid; r < TN; r += NT) {
        wctx[r] = wop.make_row(n0 + r);
        const bool have = ep.a && n0 + r < N;
        chan_a[r] = have ? __ldg(ep.a + n0 + r) : 1.f;
        chan_b[r] = have ? __ldg(ep.b + n0 + r) : 0.f;
    }
    for (int r = tid; r < TM; r += NT) xctx[r] = xop.make_row(tile * TM + r);
    __syncthreads();

    auto issue = [&](int set, int chunk, int stage) {
        const uint32_t st_addr = smem_u32(pipe + stage * Cfg::STAGE_U32);
        load_rows<TM, NT>(xop, xctx + set * TM, st_addr, chunk * KC_WORDS, kwords, kfill, xpair, tid);
        load_rows<TN, NT>(wop, wctx, st_addr + TM * PITCH32 * 4, chunk * KC_WORDS, kwords, kfill, wpair, tid);
    };
    issue(0, 0, 0);
    cp_async_commit();

    const int colbase = n0 + wn * 64 + tig * 2;
    const float* addsrc = ep.shortcut ? ep.shortcut : (ep.accumulate ? ep.out : nullptr);
    const long long ld_add = ep.shortcut ? ep.ld_sc : ep.ld_out;

    constexpr int POPROWS = (ROWS + NT - 1) / NT;
    int item = 0;
    for (int lt = 0; tile < ntiles_m; tile += gridDim.x, lt++) {
        const int next = tile + gridDim.x;
        const bool has_next = next < ntiles_m;
        const int set = lt & 1;
        if (has_next)
            for (int r = tid; r < TM; r += NT) xctx[(set ^ 1) * TM + r] = xop.make_row(next * TM + r);

        int acc[64];
#pragma unroll
        for (int i = 0; i < 64; i++) acc[i] = 0;
        int mypop[POPROWS];
#pragma unroll
        for (int i = 0; i < POPROWS; i++) mypop[i] = 0;

        for (int chunk = 0; chunk < nchunks; chunk++, item++) {
            cp_async_wait<0>();
            __syncthreads();
            if (chunk + 1 < nchunks) issue(set, chunk + 1, (item + 1) & 1);
            else if (has_next) issue(set ^ 1, 0, (item + 1) & 1);
            cp_async_commit();

            const uint32_t* st = pipe + (item & 1) * Cfg::STAGE_U32;
            const uint32_t* Xs = st + (wm * 32 + g) * PITCH32;
            const uint32_t* Ws = st + (TM + wn * 64 + g) * PITCH32;
            const int words = min(KC_WORDS, kwords - chunk * KC_WORDS);

            if (MMA) {  // row popcounts of both operands for the AND engines
#pragma unroll
                for (int i = 0; i < POPROWS; i++) {
                    const int r = tid + i * NT;
                    if (r < ROWS) {
                        const uint2* rp = reinterpret_cast<const uint2*>(st + r * PITCH32);
                        int s = 0;
                        for (int q = 0; q < words; q++) {
                            const uint2 v = rp[q];
                            s += __popc(v.x) + __popc(v.y);
                        }
                        mypop[i] += s;
                    }
                }
            }

            if (ENGINE == ENG_IMMA) {
                const uint32_t M1 = 0x01010101u;
#pragma unroll 1
                for (int wd = 0; wd < words; wd++) {
                    uint2 xa[2][2], wb[8];
#pragma unroll
                    for (int mt = 0; mt < 2; mt++) {
                        xa[mt][0] = *reinterpret_cast<const uint2*>(Xs + (mt * 16) * PITCH32 + wd * 2);
                        xa[mt][1] = *reinterpret_cast<const uint2*>(Xs + (mt * 16 + 8) * PITCH32 + wd * 2);
                    }
#pragma unroll
                    for (int nt = 0; nt < 8; nt++)
                        wb[nt] = *reinterpret_cast<const uint2*>(Ws + (nt * 8) * PITCH32 + wd * 2);
#pragma unroll
                    for (int half = 0; half < 2; half++) {
                        uint32_t af[2][4];
#pragma unroll
                        for (int mt = 0; mt < 2; mt++) {
                            const uint32_t c0 = (half ? xa[mt][0].y : xa[mt][0].x) >> tig;
                            const uint32_t c1 = (half ? xa[mt][1].y : xa[mt][1].x) >> tig;
                            af[mt][0] = c0 & M1;
                            af[mt][1] = c1 & M1;
                            af[mt][2] = (c0 >> 4) & M1;
                            af[mt][3] = (c1 >> 4) & M1;
                        }
#pragma unroll
                        for (int nt = 0; nt < 8; nt++) {
                            const uint32_t c = (half ? wb[nt].y : wb[nt].x) >> tig;
                            const uint32_t b0 = c & M1, b1 = (c >> 4) & M1;
#pragma unroll
                            for (int mt = 0; mt < 2; mt++)
                                mma_u8(&acc[(mt * 8 + nt) * 4], af[mt][0], af[mt][1], af[mt][2], af[mt][3], b0, b1);
                        }
                    }
                }
            } else if (ENGINE == ENG_B1) {
                const int steps = (words + 3) / 4;  // 4 words = 256 bits per MMA; the tail words are zero
#pragma unroll 1
                for (int s = 0; s < steps; s++) {
                    uint2 xa[2][2];
#pragma unroll
                    for (int mt = 0; mt < 2; mt++) {
                        xa[mt][0] = *reinterpret_cast<const uint2*>(Xs + (mt * 16) * PITCH32 + (s * 4 + tig) * 2);
                        xa[mt][1] = *reinterpret_cast<const uint2*>(Xs + (mt * 16 + 8) * PITCH32 + (s * 4 + tig) * 2);
                    }
#pragma unroll
                    for (int nt = 0; nt < 8; nt++) {
                        const uint2 wb = *reinterpret_cast<const uint2*>(Ws + (nt * 8) * PITCH32 + (s * 4 + tig) * 2);
#pragma unroll
                        for (int mt = 0; mt < 2; mt++)
                            mma_b1_and(&acc[(mt * 8 + nt) * 4], xa[mt][0].x, xa[mt][1].x, xa[mt][0].y, xa[mt][1].y, wb.x, wb.y);
                    }
                }
            } else {
                const uint32_t* Wq = st + (TM + wn * 64 + tig * 2) * PITCH32;
#pragma unroll 1
                for (int wd = 0; wd < words; wd++) {
                    unsigned long long xr[2][2];
#pragma unroll
                    for (int mt = 0; mt < 2; mt++) {
                        xr[mt][0] = *reinterpret_cast<const unsigned long long*>(Xs + (mt * 16) * PITCH32 + wd * 2);
                        xr[mt][1] = *reinterpret_cast<const unsigned long long*>(Xs + (mt * 16 + 8) * PITCH32 + wd * 2);
                    }
#pragma unroll
                    for (int nt = 0; nt < 8; nt++)
#pragma unroll
                        for (int q = 0; q < 2; q++) {
                            const unsigned long long wc =
                                *reinterpret_cast<const unsigned long long*>(Wq + (nt * 8 + q) * PITCH32 + wd * 2);
#pragma unroll
                            for (int mt = 0; mt < 2; mt++)
#pragma unroll
                                for (int h = 0; h < 2; h++) acc[(mt * 8 + nt) * 4 + h * 2 + q] += __popcll(xr[mt][h] ^ wc);
                        }
                }
            }
        }

        if (MMA) {
#pragma unroll
            for (int i = 0; i < POPROWS; i++) {
                const int r = tid + i * NT;
                if (r < ROWS) rowpop[r] = mypop[i];
            }
            __syncthreads();
        }

        // ---- epilogue, straight from the accumulator fragments ----
        const int m0 = tile * TM + wm * 32;
        const int* popw = rowpop + TM + wn * 64 + tig * 2;
        const float* cha = chan_a + wn * 64 + tig * 2;
        const float* chb = chan_b + wn * 64 + tig * 2;
#pragma unroll
        for (int mt = 0; mt < 2; mt++) {
            const int rloc = wm * 32 + mt * 16 + g;
            const int row0 = m0 + mt * 16 + g, row1 = row0 + 8;
            const bool ok0 = row0 < M, ok1 = row1 < M;
            float2 ad[2][8];
            if (FAST && addsrc) {
                const float* a0p = addsrc + (long long)row0 * ld_add + colbase;
                const float* a1p = addsrc + (long long)row1 * ld_add + colbase;
#pragma unroll
                for (int nt = 0; nt < 8; nt++) {
                    const bool cok = colbase + nt * 8 < N;
                    ad[0][nt] = (ok0 && cok) ? __ldcs(reinterpret_cast<const float2*>(a0p + nt * 8)) : make_float2(0.f, 0.f);
                    ad[1][nt] = (ok1 && cok) ? __ldcs(reinterpret_cast<const float2*>(a1p + nt * 8)) : make_float2(0.f, 0.f);
                }
            }
            int px[2] = {0, 0};
            if (MMA) { px[0] = rowpop[rloc]; px[1] = rowpop[rloc + 8]; }
            unsigned lo[2] = {0u, 0u}, hi[2] = {0u, 0u};
#pragma unroll
            for (int nt = 0; nt < 8; nt++) {
                const int col = colbase + nt * 8;
                int2 pw = make_int2(0, 0);
                if (MMA) pw = *reinterpret_cast<const int2*>(popw + nt * 8);
                const float2 sa = *reinterpret_cast<const float2*>(cha + nt * 8);
                const float2 sb = *reinterpret_cast<const float2*>(chb + nt * 8);
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const int row = h ? row1 : row0;
                    const bool ok = (h ? ok1 : ok0) && col < N;
                    const int r0 = acc[(mt * 8 + nt) * 4 + h * 2], r1 = acc[(mt * 8 + nt) * 4 + h * 2 + 1];
                    float v0 = small_int_to_float(MMA ? px[h] + pw.x - 2 * r0 : r0);
                    float v1 = small_int_to_float(MMA ? px[h] + pw.y - 2 * r1 : r1);
                    if (ep.a) {
                        v0 = __fadd_rn(__fmul_rn(sa.x, v0), sb.x);
                        v1 = __fadd_rn(__fmul_rn(sa.y, v1), sb.y);
                    }
                    if (FAST) {
                        if (addsrc) { v0 = __fadd_rn(ad[h][nt].x, v0); v1 = __fadd_rn(ad[h][nt].y, v1); }
                        if (ep.out && ok) __stcs(reinterpret_cast<float2*>(ep.out + (long long)row * ep.ld_out + col), make_float2(v0, v1));
                    } else if (ok) {
                        if (addsrc) {
                            v0 = __fadd_rn(addsrc[(long long)row * ld_add + col], v0);
                            if (col + 1 < N) v1 = __fadd_rn(addsrc[(long long)row * ld_add + col + 1], v1);
                        }
                        if (ep.out) {
                            ep.out[(long long)row * ep.ld_out + col] = v0;
                            if (col + 1 < N) ep.out[(long long)row * ep.ld_out + col + 1] = v1;
                        }
                    }
                    const unsigned b2 = (v0 > 0.f ? 1u : 0u) | (v1 > 0.f ? 2u : 0u);
                    if (nt < 4) lo[h] |= b2 << (nt * 8 + tig * 2);
                    else hi[h] |= b2 << ((nt - 4) * 8 + tig * 2);
                }
            }
            if (ep.bits) {  // a quad holds the 64 channels of a row: OR the four lanes together
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    lo[h] |= __shfl_xor_sync(0xffffffffu, lo[h], 1);
                    hi[h] |= __shfl_xor_sync(0xffffffffu, hi[h], 1);
                    lo[h] |= __shfl_xor_sync(0xffffffffu, lo[h], 2);
                    hi[h] |= __shfl_xor_sync(0xffffffffu, hi[h], 2);
                }
                const int wcol = (n0 + wn * 64) >> 6;
                if (tig == 0 && n0 + wn * 64 < N) {
                    if (ok0) ep.bits[(long long)row0 * ep.ld_bits + wcol] = ((unsigned long long)hi[0] << 32) | lo[0];
                    if (ok1) ep.bits[(long long)row1 * ep.ld_bits + wcol] = ((unsigned long long)hi[1] << 32) | lo[1];
                }
            }
        }
    }
    cp_async_wait<0>();
}

// Host-side launcher: picks the tile shape from N and dispatches on the engine.
template <class XOp, class WOp>
int launch_bcontract(int engine, const XOp& xop, const WOp& wop, const EpilogueParams& ep, int M, int N,
                     int kwords, cudaStream_t stream);

}  // namespace dabnn
