// Float convolution on the 5th-generation tensor cores: tcgen05.mma kind::tf32, three products per
// fp32 product (x = hi + lo with hi, lo representable in tf32; hi*hi + hi*lo + lo*hi keeps the error
// below 2^-22 relative), fp32 accumulators in TMEM.
//
// A CTA (one per SM, persistent over pixel tiles) owns one block of up to 64 output channels.  Its
// weights are split into hi / lo once and stay in shared memory for the life of the CTA in the
// K-major canonical layout of UMMA descriptors (8 rows x 16 B core matrices).  Three kinds of warps
// meet only at mbarriers:
//   * 8 producer warps build the pixel operand (implicit im2col), split it and store hi and lo
//     into a ring of 32 KB stages; thread (r, h) owns 16 consecutive k of pixel row r per 32-float
//     K chunk.  Two ways to get at the pixels:
//       ROWS   - a tile is (a 128-pixel segment of) one output row.  The kh input rows under it
//                are copied once into a double-buffered patch in shared memory, out-of-image
//                parts zero-filled, so that the k loop is a table look-up and one shared-memory
//                load per element with no predicate, and every input byte crosses L2 -> SM once
//                per tile instead of once per tap.  With 16-byte-aligned rows a loader warp does
//                the copying, two tiles ahead, with one bulk copy per input row; otherwise the
//                producers do it themselves with 4-byte cp.async, one tile ahead;
//       DIRECT - a tile is 128 consecutive output pixels and elements come straight from global
//                memory through a k -> (offset, ky, kx) table and two per-row validity masks
//                (1x1 convolutions, where nothing is reused, and windows too large to stage).
//   * 1 MMA warp: one lane issues, per 8-float slice, hi*[hi; lo] as one N = 128 instruction (the
//     lo rows of the weights follow the hi rows) and lo*hi (M = 128, K = 8) into one of four TMEM
//     accumulators; the two column halves are added in the epilogue.
//   * 8 epilogue warps: thread (r, half) reads 32 accumulator columns of row r, adds the bias,
//     applies the affine (product and sum rounded separately) and the relu and parks the row in a
//     shared staging tile (two 128-byte-swizzled boxes), which two TMA tensor stores write out.
// Every mbarrier wait is bounded (see bcontract_tc5.cuh): on a time-out the CTA records a code in
// the device status word, raises its abort flag, frees its TMEM and returns.  Named barriers are
// only reached by code paths that every thread of the role takes the same number of times.
#pragma once
#include "bcontract_tc5.cuh"

namespace dabnn {

constexpr int FT_N = 64;                        // channel block (32 when the weights of 64 channels do not fit)
constexpr int FT_CHUNK = 32;                    // floats of K per ring stage (four MMA slices of 8)
constexpr int FT_MAXK = 256;                    // padded K the resident weights may have
constexpr int FT_ACCS = 4;
constexpr int FT_PRODUCERS = 256, FT_EPILOGUE = 256;
constexpr int FT_THREADS = FT_PRODUCERS + FT_EPILOGUE + 64;   // + the MMA warp and the patch loader warp
constexpr int FT_MMA_WARP = (FT_PRODUCERS + FT_EPILOGUE) / 32;
constexpr int FT_HALF_BYTES = 128 * FT_CHUNK * 4;        // hi (or lo) part of a stage: 16 KB
constexpr int FT_STAGE_BYTES = 2 * FT_HALF_BYTES;
constexpr int FT_A_SBO = (FT_CHUNK / 4) * 128;           // 8-row group stride inside a stage
// staging tile: two boxes of 128 pixels x 32 channels in the 128-byte-swizzled layout of TMA tensor copies
// (16-byte chunk q of row r at r * 128 + ((q ^ (r & 7)) << 4)); 1 KB more for its 1024-byte alignment
constexpr int FT_SBOX_BYTES = 128 * 128;
constexpr int FT_STILE_BYTES = 2 * FT_SBOX_BYTES + 1024;
constexpr int FT_MAX_STAGES = 8;
constexpr int FT_DIRECT = 0, FT_ROWS = 1;
constexpr int FT_MAX_PATCH_BYTES = 72 * 1024;            // both patch buffers together

// hi / lo parts of the resident weights of a channel block: K-major canonical layout over the whole padded K
__host__ __device__ inline int ft_weight_bytes(int kpad, int n_blk) { return 2 * (n_blk / 8) * (kpad / 4) * 128; }
// floats per staged input row: the widest segment's window span, up to 3 floats of alignment shift, rounded to 16 bytes
__host__ __device__ inline int ft_patch_pitch(int ow, int stride_w, int kw, int dil_w, int cin) {
    const int seg = ow < 128 ? ow : 128;
    return (((seg - 1) * stride_w + (kw - 1) * dil_w + 1) * cin + 3 + 3) / 4 * 4 + 4;
}
__host__ __device__ inline int ft_smem_bytes(int kpad, int n_blk, int stages, int patch_bytes) {
    return 1024 + ft_weight_bytes(kpad, n_blk) + patch_bytes + stages * FT_STAGE_BYTES + FT_STILE_BYTES;
}

__device__ __forceinline__ uint64_t umma_desc_kmajor(uint32_t saddr, int lbo, int sbo) {
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) | ((uint64_t)((sbo >> 4) & 0x3FFF) << 32) |
           ((uint64_t)1 << 46);
}
__device__ __forceinline__ void mma_tf32_ss(uint32_t d_tmem, uint64_t ad, uint64_t bd, uint32_t idesc, uint32_t accum) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}\n"
                 ::"r"(d_tmem), "l"(ad), "l"(bd), "r"(idesc), "r"(accum), "r"(0), "r"(0), "r"(0), "r"(0) : "memory");
}
// x = hi + lo exactly, hi with its low 13 mantissa bits clear.  The tensor core reads 19 bits of each 32-bit
// container, so lo loses at most 2^-10 of itself, i.e. 2^-20 of x: two instructions instead of two roundings.
__device__ __forceinline__ void split_tf32(float x, uint32_t& hi, uint32_t& lo) {
    hi = __float_as_uint(x) & 0xffffe000u;
    lo = __float_as_uint(x - __uint_as_float(hi));
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(dst), "l"(src));
}
// barrier over the 256 producers that also ORs a flag: every thread gets the same answer
__device__ __forceinline__ bool producers_sync_or(bool mine) {
    uint32_t res;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 q, %1, 0;\n\tbar.red.or.pred p, 2, %2, q;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                 : "=r"(res) : "r"((uint32_t)mine), "n"(FT_PRODUCERS) : "memory");
    return res != 0;
}

// pixel rows of tile t: first flattened output pixel and how many of the 128 operand rows are real
template <int MODE>
__device__ __forceinline__ void ft_tile_rows(int t, int M, int ow, int nseg, long long& rowbase, int& len) {
    if (MODE == FT_ROWS) {
        const int line = t / nseg, seg = t - line * nseg;
        rowbase = (long long)line * ow + seg * 128;
        len = min(128, ow - seg * 128);
    } else {
        rowbase = (long long)t * 128;
        len = (int)min(128ll, (long long)M - rowbase);
    }
}

template <int MODE>
__global__ void __launch_bounds__(FT_THREADS, 1)
    fconv_tc5_kernel(const FconvParams p, const int M, const int K, const int kpad, const int ntiles, const int stages,
                     const int nseg, const int pitch, const int vec16, const int n_blk, const __grid_constant__ CUtensorMap out_map) {
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) uint64_t bar_full[FT_MAX_STAGES], bar_empty[FT_MAX_STAGES], bar_acc_full[FT_ACCS], bar_acc_empty[FT_ACCS];
    __shared__ __align__(8) uint64_t patch_full[2], patch_empty[2];   // ROWS with bulk copies: patch buffer filled / drained
    __shared__ uint32_t tmem_base_s;
    __shared__ int s_abort, epi_abort;
    __shared__ __align__(16) int tab_off[FT_MAXK];   // k -> float offset of (ky, kx, ci): in the patch (ROWS) or the image (DIRECT)
    __shared__ uint32_t tab_yx[FT_MAXK];             // DIRECT: k -> ky | kx << 8; k >= K -> bit 31 (never valid)
    __shared__ __align__(16) float chan_bias[FT_N], chan_a[FT_N], chan_b[FT_N];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.y * n_blk;
    const int n_this = min(n_blk, p.cout - n0);                 // multiple of 16 (host-checked)
    unsigned char* wbase = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
    const int w_sbo = (kpad / 4) * 128, w_half = (n_blk / 8) * w_sbo;
    float* patch0 = reinterpret_cast<float*>(wbase + 2 * w_half);
    const int patch_floats = MODE == FT_ROWS ? p.kh * pitch : 0;        // one buffer
    unsigned char* stage0 = reinterpret_cast<unsigned char*>(patch0 + 2 * patch_floats);
    unsigned char* stile = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(stage0 + stages * FT_STAGE_BYTES) + 1023) & ~uintptr_t(1023));
    const int nchunks = (kpad + FT_CHUNK - 1) / FT_CHUNK;
    const volatile int* abort_flag = &s_abort;
    constexpr int ACC_COLS = 2 * FT_N;                         // hi*hi + lo*hi in the first 64 columns, hi*lo in the others
    constexpr int TMEM_COLS = FT_ACCS * ACC_COLS;              // 512: all of the tensor memory

    // ---- set-up (all threads) ----
    if (warp == FT_MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    if (tid == 0) {
        for (int i = 0; i < stages; i++) { mbar_init(&bar_full[i], FT_PRODUCERS / 32); mbar_init(&bar_empty[i], 1); }
        for (int i = 0; i < FT_ACCS; i++) { mbar_init(&bar_acc_full[i], 1); mbar_init(&bar_acc_empty[i], FT_EPILOGUE / 32); }
        for (int i = 0; i < 2; i++) { mbar_init(&patch_full[i], 1); mbar_init(&patch_empty[i], FT_PRODUCERS / 32); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::);
        s_abort = 0;
        epi_abort = 0;
    }
    for (int k = tid; k < FT_MAXK; k += FT_THREADS) {
        if (k < K) {
            const int tap = k / p.cin, ky = tap / p.kw, kx = tap - ky * p.kw, ci = k - tap * p.cin;
            // ROWS: byte offset inside the patch; DIRECT: float offset inside the image
            tab_off[k] = MODE == FT_ROWS ? (ky * pitch + kx * p.dil_w * p.cin + ci) * 4 : (ky * p.dil_h * p.w + kx * p.dil_w) * p.cin + ci;
            tab_yx[k] = (uint32_t)ky | ((uint32_t)kx << 8);
        } else {   // padded k: the weights there are zero, so any finite pixel value will do - take the window's first
            tab_off[k] = 0;
            tab_yx[k] = MODE == FT_ROWS ? 0u : 0x80000000u;
        }
    }
    if (tid < FT_N) {
        const bool in = tid < n_this;
        chan_bias[tid] = (in && p.bias) ? __ldg(p.bias + n0 + tid) : 0.f;
        chan_a[tid] = (in && p.a) ? __ldg(p.a + n0 + tid) : 1.f;
        chan_b[tid] = (in && p.a) ? __ldg(p.b + n0 + tid) : 0.f;
    }
    // resident weights: element (n, k) -> (n / 8) * w_sbo + (k / 4) * 128 + (n % 8) * 16 + (k % 4) * 4
    for (int idx = tid; idx < n_blk * kpad; idx += FT_THREADS) {
        const int n = idx / kpad, k = idx - n * kpad;
        const float v = (n < n_this && k < K) ? __ldg(p.wgt + (size_t)(n0 + n) * K + k) : 0.f;
        uint32_t hi, lo;
        split_tf32(v, hi, lo);
        const int off = (n >> 3) * w_sbo + (k >> 2) * 128 + (n & 7) * 16 + (k & 3) * 4;
        *reinterpret_cast<uint32_t*>(wbase + off) = hi;
        *reinterpret_cast<uint32_t*>(wbase + w_half + off) = lo;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;

    if (tid < FT_PRODUCERS) {
        // =========================== producers: thread = (pixel row, 8-float half of the chunk) ===========================
        const int r = tid & 127, h = tid >> 7;
        const int roff = (r >> 3) * FT_A_SBO + (r & 7) * 16 + h * 4 * 128;
        uint32_t s = 0, use = 0;   // ring stage to fill next and how often the ring has wrapped
        bool ok = true;
        const uint32_t stage0_addr = smem_u32(stage0);
        // split 16 values and publish them as this thread's share (four 16-byte units) of the next ring stage
        auto emit = [&](const float (&v)[16]) -> bool {
            if (use >= 1 && !__all_sync(0xffffffffu, mbar_wait<100>(&bar_empty[s], (use - 1) & 1, abort_flag))) {   // warp-uniform
                atomicCAS(&g_tc5_status, 0, 11);
                s_abort = 1;
                return false;
            }
            const uint32_t st = stage0_addr + s * FT_STAGE_BYTES + roff;
#pragma unroll
            for (int u = 0; u < 4; u++) {
                uint32_t hi[4], lo[4];
#pragma unroll
                for (int q = 0; q < 4; q++) split_tf32(v[u * 4 + q], hi[q], lo[q]);
                sts128(st + u * 128, hi[0], hi[1], hi[2], hi[3]);
                sts128(st + FT_HALF_BYTES + u * 128, lo[0], lo[1], lo[2], lo[3]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_full[s]);   // one arrival per warp: arrivals on one mbarrier are serialised
            if (++s == (uint32_t)stages) { s = 0; use++; }
            return true;
        };
        if (MODE == FT_ROWS) {
            const int row_floats = p.w * p.cin;
            // copy the kh input rows under tile t into patch buffer b; patch position s of a row is image float
            // s - shift + gx0, with shift chosen so that 16-byte groups of the patch are 16-byte groups of the image
            auto stage_patch = [&](int t, int b) {
                if (t < ntiles) {
                    const int line = t / nseg, seg = t - line * nseg, img = line / p.oh, oy = line - img * p.oh;
                    const int iy0 = oy * p.stride_h - p.pad_h;
                    const int gx0 = (seg * 128 * p.stride_w - p.pad_w) * p.cin;
                    const float* img_rows = p.in + (long long)img * p.h * row_floats;
                    float* buf = patch0 + b * patch_floats;
                    if (vec16) {
                        const int shift = gx0 & 3, groups = pitch >> 2;
                        for (int idx = tid; idx < p.kh * groups; idx += FT_PRODUCERS) {
                            const int ky = idx / groups, j = idx - ky * groups;
                            const int iy = iy0 + ky * p.dil_h, gidx = 4 * j - shift + gx0;
                            float* dst = buf + ky * pitch + 4 * j;
                            if ((unsigned)iy < (unsigned)p.h && gidx >= 0 && gidx + 4 <= row_floats)
                                cp_async16(smem_u32(dst), img_rows + (long long)iy * row_floats + gidx, 16);
                            else
                                *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
                        }
                    } else {
                        for (int idx = tid; idx < p.kh * pitch; idx += FT_PRODUCERS) {
                            const int ky = idx / pitch, s = idx - ky * pitch;
                            const int iy = iy0 + ky * p.dil_h, gidx = s + gx0;
                            if ((unsigned)iy < (unsigned)p.h && gidx >= 0 && gidx < row_floats)
                                cp_async4(smem_u32(buf + idx), img_rows + (long long)iy * row_floats + gidx);
                            else
                                buf[idx] = 0.f;
                        }
                    }
                }
                cp_async_commit();
            };
            const uint32_t patch0_addr = smem_u32(patch0);
            if (vec16) {   // the loader warp fills the patch buffers with bulk copies
                int i = 0;
                for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, i++) {
                    if (!__all_sync(0xffffffffu, mbar_wait<100>(&patch_full[i & 1], (i >> 1) & 1, abort_flag))) {
                        atomicCAS(&g_tc5_status, 0, 16);
                        s_abort = 1;
                        ok = false;
                        break;
                    }
                    const int seg = tile % nseg, len = min(128, p.ow - seg * 128);
                    const int shift = ((seg * 128 * p.stride_w - p.pad_w) * p.cin) & 3;
                    const uint32_t pb = patch0_addr + ((i & 1) * patch_floats + shift + min(r, len - 1) * p.stride_w * p.cin) * 4;
                    for (int c = 0; c < nchunks && ok; c++) {
                        const int k0 = c * FT_CHUNK + h * 16;
                        float v[16];
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            const int4 o = *reinterpret_cast<const int4*>(tab_off + k0 + u * 4);
                            v[u * 4 + 0] = lds_f32(pb + o.x); v[u * 4 + 1] = lds_f32(pb + o.y);
                            v[u * 4 + 2] = lds_f32(pb + o.z); v[u * 4 + 3] = lds_f32(pb + o.w);
                        }
                        ok = emit(v);
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&patch_empty[i & 1]);   // this warp has read its last float of the buffer
                }
            } else {
            stage_patch(blockIdx.x, 0);
            int i = 0;
            for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x, i++) {
                cp_async_wait<0>();                                   // my copies of this tile's patch have landed
                if (producers_sync_or(!ok || *abort_flag)) break;      // everybody's have, and the other buffer is idle
                stage_patch(tile + gridDim.x, (i + 1) & 1);
                const int seg = tile % nseg, len = min(128, p.ow - seg * 128);
                const uint32_t pb = patch0_addr + ((i & 1) * patch_floats + min(r, len - 1) * p.stride_w * p.cin) * 4;
                for (int c = 0; c < nchunks && ok; c++) {
                    const int k0 = c * FT_CHUNK + h * 16;
                    float v[16];
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const int4 o = *reinterpret_cast<const int4*>(tab_off + k0 + u * 4);
                        v[u * 4 + 0] = lds_f32(pb + o.x); v[u * 4 + 1] = lds_f32(pb + o.y);
                        v[u * 4 + 2] = lds_f32(pb + o.z); v[u * 4 + 3] = lds_f32(pb + o.w);
                    }
                    ok = emit(v);
                }
            }
            }
            cp_async_wait<0>();   // nothing of this thread's is in flight when the CTA winds down
        } else {
            const int ohw = p.oh * p.ow;
            // what a thread needs to gather its pixel's row of a tile: the address of tap (0, 0) and, as bit ky / kx of
            // my / mx, whether that tap row / column lies inside the image
            struct PixelCtx { const float* src; uint32_t my, mx; };
            auto make_ctx = [&](int tile) {
                PixelCtx cx{p.in, 0u, 0u};
                const int pm = tile * 128 + r;
                if (tile < ntiles && pm < M) {
                    const int img = pm / ohw, rem = pm - img * ohw, oy = rem / p.ow, ox = rem - oy * p.ow;
                    const int iy0 = oy * p.stride_h - p.pad_h, ix0 = ox * p.stride_w - p.pad_w;
                    cx.src = p.in + (((long long)img * p.h + iy0) * p.w + ix0) * p.cin;
                    for (int ky = 0; ky < p.kh; ky++) cx.my |= ((unsigned)(iy0 + ky * p.dil_h) < (unsigned)p.h ? 1u : 0u) << ky;
                    for (int kx = 0; kx < p.kw; kx++) cx.mx |= ((unsigned)(ix0 + kx * p.dil_w) < (unsigned)p.w ? 1u : 0u) << kx;
                }
                return cx;
            };
            auto gather = [&](const PixelCtx& cx, int c, float (&v)[16]) {
                const int k0 = c * FT_CHUNK + h * 16;
                if (vec16) {   // channels are a multiple of 4 and 16-byte aligned: a unit is four channels of one tap
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const uint32_t yx = tab_yx[k0 + u * 4];
                        const bool valid = ((cx.my >> (yx & 31u)) & (cx.mx >> ((yx >> 8) & 31u)) & 1u) && !(yx >> 31);
                        const float4 t = valid ? __ldg(reinterpret_cast<const float4*>(cx.src + tab_off[k0 + u * 4])) : make_float4(0.f, 0.f, 0.f, 0.f);
                        v[u * 4 + 0] = t.x; v[u * 4 + 1] = t.y; v[u * 4 + 2] = t.z; v[u * 4 + 3] = t.w;
                    }
                } else {
#pragma unroll
                    for (int q = 0; q < 16; q++) {
                        const uint32_t yx = tab_yx[k0 + q];
                        const bool valid = ((cx.my >> (yx & 31u)) & (cx.mx >> ((yx >> 8) & 31u)) & 1u) && !(yx >> 31);
                        v[q] = valid ? __ldg(cx.src + tab_off[k0 + q]) : 0.f;
                    }
                }
            };
            // Loads run two chunks ahead of the expansion (an L2 round trip each), and the cursor they follow crosses
            // tile boundaries, so the first chunks of a tile are in flight while the previous tile is still expanding.
            int ltile = blockIdx.x, lchunk = 0;
            PixelCtx lcx = make_ctx(ltile);
            auto gather_next = [&](float (&v)[16]) {
                gather(lcx, lchunk, v);   // past the last tile the context masks every tap: zeros, no loads
                if (++lchunk == nchunks) { lchunk = 0; ltile += gridDim.x; lcx = make_ctx(ltile); }
            };
            float cur[16], nx1[16], nx2[16];
            gather_next(cur);
            gather_next(nx1);
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
                for (int c = 0; c < nchunks && ok; c++) {
                    gather_next(nx2);
                    ok = emit(cur);
#pragma unroll
                    for (int q = 0; q < 16; q++) { cur[q] = nx1[q]; nx1[q] = nx2[q]; }
                }
            }
        }
    } else if (warp == FT_MMA_WARP) {
        // =========================== MMA issue: one lane ===========================
        if (lane == 0) {
            // instruction descriptor: D = f32, A = B = tf32, both K-major, N = n_this, M = 128
            const uint32_t idesc_m = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(128 >> 4) << 24);
            const uint32_t idesc = idesc_m | ((uint32_t)(n_this >> 3) << 17);
            // The lo rows of the weights follow the hi rows at the same 8-row stride, so with a full channel block one
            // N = 128 instruction computes hi*[hi; lo] - two instructions (10 KB of operand reads) per slice, not three (18 KB).
            const bool stacked = n_this == FT_N;
            const uint32_t idesc2 = idesc_m | ((uint32_t)((2 * FT_N) >> 3) << 17);
            // The issuing thread is a single instruction stream, so its own latency bounds the MMA rate: descriptors
            // are built once and advanced by adding byte offsets >> 4 to their address field (shared-memory addresses
            // stay below 2^18, so the 14-bit field cannot carry), and the ring position is a counter, not a division.
            const uint64_t d_a = umma_desc_kmajor(smem_u32(stage0), 128, FT_A_SBO);
            const uint64_t d_wh = umma_desc_kmajor(smem_u32(wbase), 128, w_sbo), d_wl = umma_desc_kmajor(smem_u32(wbase) + w_half, 128, w_sbo);
            uint32_t s = 0, par = 0;
            bool ok = true;
            int i = 0;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, i++) {
                const int accbuf = i % FT_ACCS, accuse = i / FT_ACCS;
                if (accuse >= 1 && !mbar_wait(&bar_acc_empty[accbuf], (accuse - 1) & 1, abort_flag)) {
                    atomicCAS(&g_tc5_status, 0, 13);
                    s_abort = 1;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + accbuf * ACC_COLS;
                uint64_t bh = d_wh, bl = d_wl;
                uint32_t accum = 0;
                for (int c = 0; c < nchunks; c++) {
                    if (!mbar_wait<32>(&bar_full[s], par, abort_flag)) {
                        atomicCAS(&g_tc5_status, 0, 14);
                        s_abort = 1;
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t ah = d_a + (uint64_t)(s * (FT_STAGE_BYTES >> 4)), al = ah + (FT_HALF_BYTES >> 4);
                    // one 8-float slice = two 16-byte units = 256 bytes of descriptor address; small terms first
                    const int slices = min(FT_CHUNK / 8, (kpad - c * FT_CHUNK) / 8);
#pragma unroll
                    for (int j = 0; j < FT_CHUNK / 8; j++) {
                        if (j < slices) {
                            if (stacked) {
                                mma_tf32_ss(d_tmem, ah + j * 16, bh + j * 16, idesc2, accum);
                            } else {
                                mma_tf32_ss(d_tmem, ah + j * 16, bh + j * 16, idesc, accum);
                                mma_tf32_ss(d_tmem + FT_N, ah + j * 16, bl + j * 16, idesc, accum);
                            }
                            mma_tf32_ss(d_tmem, al + j * 16, bh + j * 16, idesc, 1u);
                            accum = 1u;
                        }
                    }
                    bh += (FT_CHUNK / 4) * 8;
                    bl += (FT_CHUNK / 4) * 8;
                    umma_commit(&bar_empty[s]);
                    if (++s == (uint32_t)stages) { s = 0; par ^= 1u; }
                }
                if (ok) umma_commit(&bar_acc_full[accbuf]);
            }
        }
    } else if (warp == FT_MMA_WARP + 1) {
        // =========================== patch loader (ROWS, 16-byte case): one warp ===========================
        // Two tiles ahead of the producers: zero-fills what lies outside the image, then lane ky issues one
        // bulk copy for input row ky; the copies complete on patch_full[b].  The producers only wait for
        // patch_full and hand the buffer back through patch_empty.
        if (MODE == FT_ROWS && vec16) {
            const int row_floats = p.w * p.cin;
            const uint32_t patch0_addr = smem_u32(patch0);
            auto stage_patch_bulk = [&](int t, int b) {
                if (t >= ntiles) return;
                const int line = t / nseg, seg = t - line * nseg, img = line / p.oh, oy = line - img * p.oh;
                const int iy0 = oy * p.stride_h - p.pad_h;
                const int gx0 = (seg * 128 * p.stride_w - p.pad_w) * p.cin, shift = gx0 & 3, groups = pitch >> 2;
                // patch group j holds image floats 4j - shift + gx0 .. + 3: inside the row for j_lo <= j < j_hi
                const int j_lo = gx0 < shift ? (shift - gx0) >> 2 : 0;
                const int j_hi = max(j_lo, min(groups, (row_floats - gx0 + shift) >> 2));
                const uint32_t buf = patch0_addr + b * patch_floats * 4;
                const int iy = iy0 + lane * p.dil_h;
                const bool row_in = lane < p.kh && (unsigned)iy < (unsigned)p.h;
                const int npad = j_lo + (groups - j_hi);
                for (int idx = lane; idx < p.kh * npad; idx += 32) {   // left and right of the image
                    const int ky = idx / npad, q = idx - ky * npad, j = q < j_lo ? q : j_hi + (q - j_lo);
                    sts128f(buf + (ky * pitch + 4 * j) * 4, 0.f, 0.f, 0.f, 0.f);
                }
                for (int ky = 0; ky < p.kh; ky++)                      // rows above and below the image
                    if ((unsigned)(iy0 + ky * p.dil_h) >= (unsigned)p.h)
                        for (int j = j_lo + lane; j < j_hi; j += 32) sts128f(buf + (ky * pitch + 4 * j) * 4, 0.f, 0.f, 0.f, 0.f);
                const uint32_t bytes = (uint32_t)(j_hi - j_lo) * 16u, bar = smem_u32(&patch_full[b]);
                const uint32_t nrows = __popc(__ballot_sync(0xffffffffu, row_in));
                __syncwarp();
                if (lane == 0) asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(nrows * bytes) : "memory");
                __syncwarp();
                if (row_in && bytes > 0)
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                 ::"r"(buf + (lane * pitch + 4 * j_lo) * 4),
                                   "l"(p.in + ((long long)img * p.h + iy) * row_floats + (4 * j_lo - shift + gx0)), "r"(bytes), "r"(bar) : "memory");
            };
            int i = 0;
            for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x, i++) {
                if (i >= 2 && !__all_sync(0xffffffffu, mbar_wait<100>(&patch_empty[i & 1], ((i >> 1) - 1) & 1, abort_flag))) {
                    atomicCAS(&g_tc5_status, 0, 15);
                    s_abort = 1;
                    break;
                }
                stage_patch_bulk(tile, i & 1);
            }
        }
    } else {
        // =========================== epilogue ===========================
        const int et = tid - FT_PRODUCERS;
        const int r = et & 127, h2 = et >> 7;          // drain role: TMEM lane quarter = warp % 4 = r / 32
        const int ncol = max(0, min(32, n_this - h2 * 32));   // 0, 16 or 32 columns for this thread
        const uint32_t stile_addr = smem_u32(stile);
        int i = 0;
        for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x, i++) {
            const int accbuf = i % FT_ACCS, accuse = i / FT_ACCS;
            long long rowbase;
            int len;
            ft_tile_rows<MODE>(tile, M, p.ow, nseg, rowbase, len);
            const bool okw = __all_sync(0xffffffffu, mbar_wait<500>(&bar_acc_full[accbuf], accuse & 1, abort_flag));   // warp-uniform
            if (!okw) {
                atomicCAS(&g_tc5_status, 0, 12);
                s_abort = 1;
                epi_abort = 1;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (okw && ncol > 0) {
                const uint32_t t_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + accbuf * ACC_COLS + h2 * 32;
                uint32_t v[32], x[32];
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                             : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                               "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                             : "r"(t_addr));
                if (ncol > 16)
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                                 : "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                                   "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                                 : "r"(t_addr + 16));
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                             : "=r"(x[0]), "=r"(x[1]), "=r"(x[2]), "=r"(x[3]), "=r"(x[4]), "=r"(x[5]), "=r"(x[6]), "=r"(x[7]), "=r"(x[8]),
                               "=r"(x[9]), "=r"(x[10]), "=r"(x[11]), "=r"(x[12]), "=r"(x[13]), "=r"(x[14]), "=r"(x[15])
                             : "r"(t_addr + FT_N));
                if (ncol > 16)
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                                 : "=r"(x[16]), "=r"(x[17]), "=r"(x[18]), "=r"(x[19]), "=r"(x[20]), "=r"(x[21]), "=r"(x[22]), "=r"(x[23]),
                                   "=r"(x[24]), "=r"(x[25]), "=r"(x[26]), "=r"(x[27]), "=r"(x[28]), "=r"(x[29]), "=r"(x[30]), "=r"(x[31])
                                 : "r"(t_addr + FT_N + 16));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                const uint32_t srow = stile_addr + h2 * FT_SBOX_BYTES + r * 128;   // chunk q of this row: srow + ((q ^ (r & 7)) << 4)
#pragma unroll
                for (int q = 0; q < 8; q++) {
                    if (q * 4 >= ncol) break;
                    float o[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const int cl = h2 * 32 + q * 4 + e;
                        float f = __uint_as_float(v[q * 4 + e]) + __uint_as_float(x[q * 4 + e]);   // + the hi*lo part
                        if (p.bias) f = __fadd_rn(f, chan_bias[cl]);
                        if (p.a) f = __fadd_rn(__fmul_rn(chan_a[cl], f), chan_b[cl]);
                        if (p.relu) f = relu_ref(f);
                        o[e] = f;
                    }
                    sts128f(srow + ((q ^ (r & 7)) << 4), o[0], o[1], o[2], o[3]);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the bulk store below reads what was just written
            }
            if (okw) {   // the accumulator has been read: the MMA warp may reuse it
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_acc_empty[accbuf]);
            }
            asm volatile("bar.sync 1, %0;" ::"n"(FT_EPILOGUE) : "memory");   // the tile is staged (or abort decided)
            if (epi_abort) break;
            // ---- write-out: one tensor store (shared -> global) per 32-channel box; the descriptor is [line][pixel][channel],
            //      so pixels beyond the row (ROWS) or beyond M (DIRECT) and channels beyond Cout are clipped ----
            if (et == 0 || (et == 128 && n_this > 32)) {
                const int hb = et >> 7;
                int c1, c2;
                if (MODE == FT_ROWS) { c2 = tile / nseg; c1 = (tile - c2 * nseg) * 128; } else { c2 = 0; c1 = tile * 128; }
                asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];"
                             ::"l"(reinterpret_cast<uint64_t>(&out_map)), "r"(n0 + hb * 32), "r"(c1), "r"(c2), "r"(stile_addr + hb * FT_SBOX_BYTES) : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the box has been read: it may be overwritten
            }
            asm volatile("bar.sync 1, %0;" ::"n"(FT_EPILOGUE) : "memory");   // the staging tile may be overwritten
        }
    }

    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // row stores are complete before the CTA winds down
    // ---- drain: everybody is past its last use of the tensor memory ----
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == FT_MMA_WARP) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS));
    }
}

}  // namespace dabnn
