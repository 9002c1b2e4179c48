// Binary contraction on the 5th-generation tensor cores: tcgen05.mma kind::i8 with TMEM accumulators.
//
//   cnt[p][n] = sum_k x[p][k] XOR w[n][k] = popc(x[p]) + popc(w[n]) - 2 * sum_k a[p][k] * b[n][k]
//
// with a, b the bits as {0,1} unsigned bytes.  Blackwell's tcgen05.mma has no 1-bit kind and its
// legacy b1 mma.sync is emulated, so the int8 kind is the fastest exact route: 8x the operand bytes
// of 1-bit, but those bytes exist only in shared memory - HBM and L2 still carry packed bits.
//
// A CTA works on 128-pixel x (up to) 128-channel tiles with three kinds of warps that only meet
// at mbarriers:
//   * 4 producer warps, thread r = pixel row r: read the 64-bit words of the row (implicit im2col,
//     tap by tap, zero word outside the image), expand every 32 bits to 32 bytes with shift+mask
//     pairs ((w >> s) & 0x01010101 - the resulting bit -> K-slot permutation is the same for
//     both operands, and a contraction is blind to it) and store them in the K-major SWIZZLE_NONE
//     canonical layout of UMMA shared-memory descriptors (8 rows x 16 B core matrices).  Threads
//     r < Ntile expand weight row r the same way.  K advances in chunks of 128 bits through a
//     3-deep ring of chunk buffers.  The row popcount is accumulated on the way.
//   * 1 MMA warp: one lane issues, per chunk, four tcgen05.mma (M = 128, N = Ntile, K = 32 bytes)
//     from shared-memory descriptors into one of two TMEM accumulators and commits them to the
//     ring's "empty" barrier, and to the accumulator's "full" barrier after the last chunk.
//   * 4 epilogue warps, thread r = pixel row r: tcgen05.ld the row's accumulator 32 columns at a
//     time, turn AND counts into XOR counts, apply the affine, add the shortcut, store fp32 and
//     the row's sign bits (a thread holds whole 32-channel half words, no shuffles), then release
//     the accumulator.
// CTAs are persistent over pixel tiles; two fit on an SM (2 x 256 TMEM columns, 2 x ~104 KB).
//
// Every wait on an mbarrier is bounded: after a fixed number of polls the CTA records an error
// code in a device-side status word, raises a CTA-wide abort flag that every role checks, frees
// its TMEM and returns.
#pragma once
#include "bcontract.cuh"

namespace dabnn {

constexpr int TC5_CHUNK_WORDS = 2;                       // 128 bits of K per chunk
constexpr int TC5_CHUNK_BYTES = TC5_CHUNK_WORDS * 64;    // operand bytes per row per chunk
constexpr int TC5_SBO = (TC5_CHUNK_BYTES / 16) * 128;    // byte stride between 8-row groups
constexpr int TC5_LBO = 128;                             // byte stride between 16-byte K units
constexpr int TC5_MAX_N = 128;
constexpr int TC5_STAGES = 3;
constexpr int TC5_DECTAB = 640;                          // words of K with a precomputed tap decode
constexpr int TC5_THREADS = 288;                         // 4 producer + 4 epilogue + 1 MMA warp
constexpr uint32_t TC5_SPIN_LIMIT = 1u << 22;

__device__ int g_tc5_status;  // 0 = ok; otherwise the code of the first wait that gave up

__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)((TC5_LBO >> 4) & 0x3FFF) << 16) |
           ((uint64_t)((TC5_SBO >> 4) & 0x3FFF) << 32) | ((uint64_t)1 << 46);  // version 1, no swizzle
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait; gives up (returns false) when the barrier does not flip or the CTA is aborting.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const volatile int* abort_flag) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t it = 0; it < TC5_SPIN_LIMIT; it++) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred P1;\n\tmbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n\tselp.b32 %0, 1, 0, P1;\n\t}"
                     : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
        if ((it & 1023) == 1023 && *abort_flag) return false;
    }
    return false;
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

struct Tc5Smem {
    static constexpr int A_BYTES = 128 * TC5_CHUNK_BYTES;            // 16 KB
    static constexpr int B_BYTES = TC5_MAX_N * TC5_CHUNK_BYTES;      // 16 KB
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int TOTAL = TC5_STAGES * STAGE_BYTES + 1024 /*alignment slack*/;
};

// 32 bits -> 32 bytes {0,1}: output word s holds bits s, s+8, s+16, s+24.  Two 16-byte stores.
__device__ __forceinline__ void expand32(unsigned char* dst_unit0, uint32_t w) {
    const uint32_t M1 = 0x01010101u;
    uint4 lo, hi;
    lo.x = w & M1;        lo.y = (w >> 1) & M1; lo.z = (w >> 2) & M1; lo.w = (w >> 3) & M1;
    hi.x = (w >> 4) & M1; hi.y = (w >> 5) & M1; hi.z = (w >> 6) & M1; hi.w = (w >> 7) & M1;
    *reinterpret_cast<uint4*>(dst_unit0) = lo;
    *reinterpret_cast<uint4*>(dst_unit0 + TC5_LBO) = hi;
}
// one chunk (two 64-bit words) of one operand row: eight 16-byte units at a 128-byte stride
__device__ __forceinline__ void expand_row(unsigned char* row_base, uint64_t w0, uint64_t w1) {
    expand32(row_base + 0 * TC5_LBO, (uint32_t)w0);
    expand32(row_base + 2 * TC5_LBO, (uint32_t)(w0 >> 32));
    expand32(row_base + 4 * TC5_LBO, (uint32_t)w1);
    expand32(row_base + 6 * TC5_LBO, (uint32_t)(w1 >> 32));
}

template <class XOp, class WOp>
__global__ void __launch_bounds__(TC5_THREADS, 2)
    bcontract_tc5_kernel(const XOp xop, const WOp wop, const EpilogueParams ep, const int M, const int N,
                         const int kwords, const int ntiles_m) {
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) uint64_t bar_full[TC5_STAGES], bar_empty[TC5_STAGES], bar_acc_full[2], bar_acc_empty[2];
    __shared__ uint32_t tmem_base_s;
    __shared__ int s_abort;
    __shared__ int popw[TC5_MAX_N], popx[4][128];   // popx: ring over tiles, producers run at most 3 tiles ahead of the epilogue
    __shared__ float chan_a[TC5_MAX_N], chan_b[TC5_MAX_N];
    __shared__ typename XOp::Dec dectab[TC5_DECTAB];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.y * TC5_MAX_N;
    const int n_this = min(TC5_MAX_N, N - n0);               // multiple of 16 (host-checked)
    unsigned char* stage0 = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
    const int nchunks = (kwords + TC5_CHUNK_WORDS - 1) / TC5_CHUNK_WORDS;
    const int tmem_cols = n_this <= 16 ? 32 : (n_this <= 32 ? 64 : (n_this <= 64 ? 128 : 256));  // 2 accumulators, power of 2
    const volatile int* abort_flag = &s_abort;

    // ---- set-up (all threads) ----
    if (warp == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(tmem_cols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    if (tid == 0) {
        for (int i = 0; i < TC5_STAGES; i++) { mbar_init(&bar_full[i], 128); mbar_init(&bar_empty[i], 1); }
        for (int i = 0; i < 2; i++) { mbar_init(&bar_acc_full[i], 1); mbar_init(&bar_acc_empty[i], 128); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::);
        s_abort = 0;
    }
    const bool use_tab = kwords <= TC5_DECTAB;
    if (use_tab)
        for (int q = tid; q < kwords; q += TC5_THREADS) dectab[q] = xop.decode(q);
    const RowCtx wrow = wop.make_row(n0 + (tid & 127));   // weight row owned by producer thread tid (if tid < n_this)
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

    if (warp < 4) {
        // =========================== producers: thread = operand row ===========================
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
        const int roff = (tid >> 3) * TC5_SBO + (tid & 7) * 16;
        uint32_t g = 0;   // chunks produced by this CTA
        bool ok = true;
        int i = 0;
        for (int tile = blockIdx.x; tile < ntiles_m && ok; tile += gridDim.x, i++) {
            const RowCtx xr = xop.make_row(tile * 128 + tid);
            uint64_t a0, a1, b0, b1;
            load_words(xr, 0, a0, a1, b0, b1);
            int px = 0;
            for (int c = 0; c < nchunks; c++, g++) {
                const uint32_t s = g % TC5_STAGES, use = g / TC5_STAGES;
                uint64_t na0 = 0, na1 = 0, nb0 = 0, nb1 = 0;
                if (c + 1 < nchunks) load_words(xr, c + 1, na0, na1, nb0, nb1);   // in flight during the expansion
                if (use >= 1 && !mbar_wait(&bar_empty[s], (use - 1) & 1, abort_flag)) {
                    atomicCAS(&g_tc5_status, 0, 1);
                    s_abort = 1;
                    ok = false;
                    break;
                }
                unsigned char* st = stage0 + s * Tc5Smem::STAGE_BYTES;
                expand_row(st + roff, a0, a1);
                if (tid < n_this) expand_row(st + Tc5Smem::A_BYTES + roff, b0, b1);
                px += __popcll(a0) + __popcll(a1);
                if (c == nchunks - 1) popx[i & 3][tid] = px;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(&bar_full[s]);
                a0 = na0; a1 = na1; b0 = nb0; b1 = nb1;
            }
        }
    } else if (warp == 8) {
        // =========================== MMA issue: one lane ===========================
        if (lane == 0) {
            // instruction descriptor: D = s32, A = u8, B = u8, both K-major, N = n_this, M = 128
            const uint32_t idesc = (2u << 4) | ((uint32_t)(n_this >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
            uint32_t g = 0;
            bool ok = true;
            int i = 0;
            for (int tile = blockIdx.x; tile < ntiles_m && ok; tile += gridDim.x, i++) {
                const int accbuf = i & 1, accuse = i >> 1;
                if (accuse >= 1 && !mbar_wait(&bar_acc_empty[accbuf], (accuse - 1) & 1, abort_flag)) {
                    atomicCAS(&g_tc5_status, 0, 3);
                    s_abort = 1;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + accbuf * n_this;
                for (int c = 0; c < nchunks; c++, g++) {
                    const uint32_t s = g % TC5_STAGES, use = g / TC5_STAGES;
                    if (!mbar_wait(&bar_full[s], use & 1, abort_flag)) {
                        atomicCAS(&g_tc5_status, 0, 4);
                        s_abort = 1;
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = smem_u32(stage0 + s * Tc5Smem::STAGE_BYTES), b_addr = a_addr + Tc5Smem::A_BYTES;
                    const int words = min(TC5_CHUNK_WORDS, kwords - c * TC5_CHUNK_WORDS);
                    for (int j = 0; j < words * 2; j++) {   // one MMA per 32 bytes of K = two 16-byte units
                        const uint64_t ad = umma_desc(a_addr + j * 2 * TC5_LBO), bd = umma_desc(b_addr + j * 2 * TC5_LBO);
                        const uint32_t accum = (c > 0 || j > 0) ? 1u : 0u;
                        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                                     "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}\n"
                                     ::"r"(d_tmem), "l"(ad), "l"(bd), "r"(idesc), "r"(accum), "r"(0), "r"(0), "r"(0), "r"(0) : "memory");
                    }
                    umma_commit(&bar_empty[s]);
                    if (c == nchunks - 1) umma_commit(&bar_acc_full[accbuf]);
                }
            }
        }
    } else {
        // =========================== epilogue: thread = pixel row ===========================
        const int r = tid - 128;                 // row in the tile; TMEM lane quarter = warp % 4
        const float* addsrc = ep.shortcut ? ep.shortcut : (ep.accumulate ? ep.out : nullptr);
        const long long ld_add = ep.shortcut ? ep.ld_sc : ep.ld_out;
        int i = 0;
        for (int tile = blockIdx.x; tile < ntiles_m; tile += gridDim.x, i++) {
            const int accbuf = i & 1, accuse = i >> 1;
            if (!mbar_wait(&bar_acc_full[accbuf], accuse & 1, abort_flag)) {
                atomicCAS(&g_tc5_status, 0, 2);
                s_abort = 1;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int row = tile * 128 + r;
            const bool row_ok = row < M;
            const int px = popx[i & 3][r];
            const uint32_t t_row = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + accbuf * n_this;
            for (int c0 = 0; c0 < n_this; c0 += 32) {
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
                        const int cnt = px + popw[cl] - 2 * (int)v[q * 4 + e];
                        float f = small_int_to_float(cnt);
                        if (ep.a) f = __fadd_rn(__fmul_rn(chan_a[cl], f), chan_b[cl]);
                        o[e] = f;
                    }
                    if (addsrc && row_ok) {
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
            mbar_arrive(&bar_acc_empty[accbuf]);   // the accumulator may be overwritten by the tile after next
        }
    }

    // ---- drain: everybody is past its last use of the tensor memory ----
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 8) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols));
    }
}

}  // namespace dabnn
