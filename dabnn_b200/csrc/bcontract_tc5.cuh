// Binary contraction on the 5th-generation tensor cores: tcgen05.mma kind::i8 with TMEM accumulators.
//
//   cnt[p][n] = sum_k  x[p][k] XOR w[n][k]  =  popc(w[n]) - sum_k a[p][k] * s[n][k]
//
// with a = x as {0,1} unsigned bytes and s = +1 / -1 signed bytes for weight bit 1 / 0 (check the four
// cases: only (a=1, w=1) adds +1 to the dot product and only (a=1, w=0) adds -1, so popc(w) - dot
// counts exactly the mismatches).  Blackwell's tcgen05.mma has no 1-bit kind and its legacy b1
// mma.sync is emulated, so the int8 kind is the fastest exact route: 8x the operand bytes of 1-bit,
// but those bytes exist only in shared memory - HBM still carries packed bits.
//
// One CTA = 128 threads = one 128-pixel tile; thread r owns pixel row r for everything:
//   * operand production: the thread reads the 64-bit words of its row (implicit im2col: tap by
//     tap, zero word outside the image), expands 16 bits at a time to 16 bytes through a 16-entry
//     nibble table and stores them in the K-major SWIZZLE_NONE canonical layout of UMMA shared-
//     memory descriptors (8 rows x 16 B core matrices); threads r < Ntile do the same for weight
//     row r with the +-1 table.  K advances in chunks of 128 bits (= 4 MMAs of K = 32 bytes), two
//     chunk buffers, so expansion of chunk c+1 overlaps the MMAs of chunk c.
//   * one elected thread issues the MMAs (M = 128, N = Ntile <= 128, K = 32) and commits them to
//     mbarriers; accumulators (s32) live in TMEM, double buffered, so the MMAs of tile t+1 run
//     while tile t is written out.
//   * epilogue: thread r reads row r of the accumulator with tcgen05.ld (32 columns at a time),
//     turns dot products into counts, applies the affine, adds the shortcut and stores fp32 and
//     the sign bits of its own row (no shuffles: a thread holds whole 64-channel words).
//
// CTAs are persistent over pixel tiles.  Every wait on an mbarrier is bounded: after a fixed
// number of polls the CTA records an error code in a device-side status word, stops issuing work,
// frees its TMEM and returns.
#pragma once
#include "bcontract.cuh"

namespace dabnn {

constexpr int TC5_CHUNK_WORDS = 2;                       // 128 bits of K per chunk
constexpr int TC5_CHUNK_BYTES = TC5_CHUNK_WORDS * 64;    // operand bytes per row per chunk
constexpr int TC5_SBO = (TC5_CHUNK_BYTES / 16) * 128;    // byte stride between 8-row groups
constexpr int TC5_LBO = 128;                             // byte stride between 16-byte K units
constexpr int TC5_MAX_N = 128;
constexpr int TC5_DECTAB = 640;                          // words of K with a precomputed tap decode
constexpr uint32_t TC5_SPIN_LIMIT = 1u << 22;

__device__ int g_tc5_status;  // 0 = ok; otherwise the code of the first wait that gave up

__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)((TC5_LBO >> 4) & 0x3FFF) << 16) |
           ((uint64_t)((TC5_SBO >> 4) & 0x3FFF) << 32) | ((uint64_t)1 << 46);  // version 1, no swizzle
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    uint32_t done = 0;
    for (uint32_t it = 0; it < TC5_SPIN_LIMIT && !done; it++)
        asm volatile("{\n\t.reg .pred P1;\n\tmbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n\tselp.b32 %0, 1, 0, P1;\n\t}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done != 0;
}

struct Tc5Smem {
    static constexpr int A_BYTES = 128 * TC5_CHUNK_BYTES;            // 16 KB
    static constexpr int B_BYTES = TC5_MAX_N * TC5_CHUNK_BYTES;      // 16 KB
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int TOTAL = 2 * STAGE_BYTES + 1024 /*alignment slack*/;
};

template <class XOp, class WOp>
__global__ void __launch_bounds__(128, 2)
    bcontract_tc5_kernel(const XOp xop, const WOp wop, const EpilogueParams ep, const int M, const int N,
                         const int kwords, const int ntiles_m) {
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) uint64_t bar_stage[2], bar_acc[2];
    __shared__ uint32_t tmem_base_s, lut_a[16], lut_b[16];
    __shared__ int s_abort;
    __shared__ int popw[TC5_MAX_N];
    __shared__ float chan_a[TC5_MAX_N], chan_b[TC5_MAX_N];
    __shared__ typename XOp::Dec dectab[TC5_DECTAB];

    const int tid = threadIdx.x, warp = tid >> 5;
    const int n0 = blockIdx.y * TC5_MAX_N;
    const int n_this = min(TC5_MAX_N, N - n0);               // multiple of 16 (host-checked)
    unsigned char* stage0 = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
    const int nchunks = (kwords + TC5_CHUNK_WORDS - 1) / TC5_CHUNK_WORDS;
    const int tmem_cols = n_this <= 16 ? 32 : (n_this <= 32 ? 64 : (n_this <= 64 ? 128 : 256));  // 2 accumulators, power of 2

    // ---- set-up ----
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(tmem_cols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    if (tid == 0) {
        for (int i = 0; i < 2; i++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&bar_stage[i])), "r"(1));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&bar_acc[i])), "r"(1));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::);
        s_abort = 0;
    }
    if (tid < 16) {  // nibble -> 4 bytes: bit i of the nibble -> byte i
        uint32_t a = 0, b = 0;
        for (int i = 0; i < 4; i++) {
            const bool on = (tid >> i) & 1;
            a |= (on ? 0x01u : 0x00u) << (8 * i);
            b |= (on ? 0x01u : 0xFFu) << (8 * i);
        }
        lut_a[tid] = a;
        lut_b[tid] = b;
    }
    const bool use_tab = kwords <= TC5_DECTAB;
    if (use_tab)
        for (int q = tid; q < kwords; q += 128) dectab[q] = xop.decode(q);
    const RowCtx wrow = wop.make_row(n0 + tid);   // weight row owned by this thread (valid if tid < n_this)
    if (tid < TC5_MAX_N) {
        int pc = 0;
        if (tid < n_this)
            for (int q = 0; q < kwords; q++) {
                const uint64_t* p = wop.addr(wrow, wop.decode(q));
                pc += p ? __popcll(__ldg(p)) : 0;
            }
        popw[tid] = pc;
        const bool have = ep.a && tid < n_this;
        chan_a[tid] = have ? __ldg(ep.a + n0 + tid) : 1.f;
        chan_b[tid] = have ? __ldg(ep.b + n0 + tid) : 0.f;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;
    // instruction descriptor: D = s32, A = u8, B = s8, both K-major, N = n_this, M = 128
    const uint32_t idesc = (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(n_this >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);

    uint32_t gchunk = 0;   // chunks produced so far by this CTA (stage = gchunk & 1)
    bool aborted = false;

    auto xdecode = [&](int q) { return use_tab ? dectab[q] : xop.decode(q); };
    auto load_words = [&](const RowCtx& xr, int chunk, uint64_t& a0, uint64_t& a1, uint64_t& b0, uint64_t& b1) {
        const int q = chunk * TC5_CHUNK_WORDS;
        a0 = a1 = b0 = b1 = 0;
        if (q < kwords) {
            const uint64_t* p = xop.addr(xr, xdecode(q));
            if (p) a0 = __ldg(p);
            if (tid < n_this) { const uint64_t* w = wop.addr(wrow, wop.decode(q)); if (w) b0 = __ldg(w); }
        }
        if (q + 1 < kwords) {
            const uint64_t* p = xop.addr(xr, xdecode(q + 1));
            if (p) a1 = __ldg(p);
            if (tid < n_this) { const uint64_t* w = wop.addr(wrow, wop.decode(q + 1)); if (w) b1 = __ldg(w); }
        }
    };
    auto expand_row = [&](unsigned char* dst_row, uint64_t w0, uint64_t w1, const uint32_t* lut) {
        // row base already includes (r/8)*SBO + (r%8)*16; 16-byte unit u lives at + u*128
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const uint32_t bits = (uint32_t)((u < 4 ? w0 : w1) >> (16 * (u & 3))) & 0xFFFFu;
            uint4 v;
            v.x = lut[bits & 15];
            v.y = lut[(bits >> 4) & 15];
            v.z = lut[(bits >> 8) & 15];
            v.w = lut[bits >> 12];
            *reinterpret_cast<uint4*>(dst_row + u * 128) = v;
        }
    };

    // Produce all chunks of one tile: expand operands, issue the MMAs into accumulator `accbuf`.
    auto produce = [&](int tile, int accbuf) {
        const RowCtx xr = xop.make_row(tile * 128 + tid);
        uint64_t a0, a1, b0, b1;
        load_words(xr, 0, a0, a1, b0, b1);
        for (int c = 0; c < nchunks && !aborted; c++, gchunk++) {
            const uint32_t s = gchunk & 1;
            uint64_t na0 = 0, na1 = 0, nb0 = 0, nb1 = 0;
            if (c + 1 < nchunks) load_words(xr, c + 1, na0, na1, nb0, nb1);   // in flight during the expansion
            if (gchunk >= 2 && !mbar_wait(smem_u32(&bar_stage[s]), ((gchunk >> 1) - 1) & 1)) {
                atomicCAS(&g_tc5_status, 0, 1);
                s_abort = 1;
            }
            unsigned char* st = stage0 + s * Tc5Smem::STAGE_BYTES;
            const int roff = (tid >> 3) * TC5_SBO + (tid & 7) * 16;
            expand_row(st + roff, a0, a1, lut_a);
            if (tid < n_this) expand_row(st + Tc5Smem::A_BYTES + roff, b0, b1, lut_b);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncthreads();
            aborted = s_abort != 0;
            if (tid == 0 && !aborted) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const int words = min(TC5_CHUNK_WORDS, kwords - c * TC5_CHUNK_WORDS);
                const uint32_t a_addr = smem_u32(st), b_addr = a_addr + Tc5Smem::A_BYTES;
                const uint32_t d_tmem = tmem_base + accbuf * n_this;
                for (int j = 0; j < words * 2; j++) {   // one MMA per 32 bytes of K
                    const uint64_t ad = umma_desc(a_addr + j * 2 * TC5_LBO), bd = umma_desc(b_addr + j * 2 * TC5_LBO);
                    const uint32_t accum = (c > 0 || j > 0) ? 1u : 0u;
                    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                                 "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}\n"
                                 ::"r"(d_tmem), "l"(ad), "l"(bd), "r"(idesc), "r"(accum), "r"(0), "r"(0), "r"(0), "r"(0) : "memory");
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bar_stage[s])) : "memory");
                if (c == nchunks - 1)
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bar_acc[accbuf])) : "memory");
            }
            a0 = na0; a1 = na1; b0 = nb0; b1 = nb1;
        }
    };

    const float* addsrc = ep.shortcut ? ep.shortcut : (ep.accumulate ? ep.out : nullptr);
    const long long ld_add = ep.shortcut ? ep.ld_sc : ep.ld_out;

    auto epilogue = [&](int tile, int accbuf, uint32_t parity) {
        if (!mbar_wait(smem_u32(&bar_acc[accbuf]), parity)) {
            atomicCAS(&g_tc5_status, 0, 2);
            s_abort = 1;
            aborted = true;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int row = tile * 128 + tid;
        const bool row_ok = row < M && !aborted;
        const uint32_t t_row = tmem_base + ((uint32_t)(warp * 32) << 16) + accbuf * n_this;
        for (int c0 = 0; c0 < n_this && !aborted; c0 += 32) {
            const int ncol = min(32, n_this - c0);   // 16 or 32
            float4 add4[8];
            if (addsrc && row_ok) {
                const float4* ap = reinterpret_cast<const float4*>(addsrc + (long long)row * ld_add + n0 + c0);
#pragma unroll
                for (int q = 0; q < 8; q++) add4[q] = q * 4 < ncol ? __ldg(ap + q) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            uint32_t v[32];
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                         : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                           "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                         : "r"(t_row + c0));
            if (ncol > 16)
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                             : "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                               "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                             : "r"(t_row + c0 + 16));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            uint32_t signs = 0;
#pragma unroll
            for (int q = 0; q < 8; q++) {
                if (q * 4 >= ncol) break;
                float o[4];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int cl = c0 + q * 4 + e;
                    const int cnt = popw[cl] - (int)v[q * 4 + e];
                    float f = small_int_to_float(cnt);
                    if (ep.a) f = __fadd_rn(__fmul_rn(chan_a[cl], f), chan_b[cl]);
                    o[e] = f;
                }
                if (addsrc) {
                    o[0] = __fadd_rn(add4[q].x, o[0]); o[1] = __fadd_rn(add4[q].y, o[1]);
                    o[2] = __fadd_rn(add4[q].z, o[2]); o[3] = __fadd_rn(add4[q].w, o[3]);
                }
                if (ep.out && row_ok)
                    *reinterpret_cast<float4*>(ep.out + (long long)row * ep.ld_out + n0 + c0 + q * 4) = make_float4(o[0], o[1], o[2], o[3]);
                signs |= ((o[0] > 0.f ? 1u : 0u) | (o[1] > 0.f ? 2u : 0u) | (o[2] > 0.f ? 4u : 0u) | (o[3] > 0.f ? 8u : 0u)) << (q * 4);
            }
            if (ep.bits && row_ok)   // n0 and c0 are multiples of 32: this is one aligned half word
                reinterpret_cast<uint32_t*>(ep.bits + (long long)row * ep.ld_bits)[(n0 + c0) >> 5] = signs;
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();   // the accumulator buffer may be overwritten by the MMAs of the tile after next
    };

    // ---- persistent tile loop, one tile of look-ahead ----
    int tile = blockIdx.x;
    if (tile < ntiles_m) {
        produce(tile, 0);
        for (int i = 0; tile < ntiles_m; i++, tile += gridDim.x) {
            const int next = tile + gridDim.x;
            if (next < ntiles_m && !aborted) produce(next, (i + 1) & 1);
            epilogue(tile, i & 1, (uint32_t)(i >> 1) & 1);
            if (aborted) break;
        }
    }
    // drain: the last MMAs were waited for by the last epilogue; free the tensor memory
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols));
}

}  // namespace dabnn
