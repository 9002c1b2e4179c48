// Binary contraction on the 5th-generation tensor cores: tcgen05.mma kind::i8 with TMEM accumulators.
//
//   cnt[p][n] = sum_k x[p][k] XOR w[n][k] = popc(x[p]) + popc(w[n]) - 2 * sum_k a[p][k] * b[n][k]
//
// with a, b the bits as {0,1} unsigned bytes.  Blackwell's tcgen05.mma has no 1-bit kind and its
// legacy b1 mma.sync is emulated, so the int8 kind is the fastest exact route: 8x the operand bytes
// of 1-bit, but those bytes exist only in shared memory - HBM and L2 still carry packed bits.
//
// A CTA (one per SM, persistent over pixel tiles) works on 128-pixel x (up to) 128-channel tiles
// with three kinds of warps that only meet at mbarriers:
//   * 8 producer warps; thread (r, h) owns half of the 64-bit words of every K chunk of operand row
//     r (chunks of 128 bits through four stages for short K, 256 bits through two stages otherwise:
//     Tc5Cfg).  It reads its words (implicit im2col: tap by tap, zero word outside the image; the tap
//     decode is stepped, not divided), expands every 32 bits to 32 bytes with shift+mask pairs
//     ((w >> s) & 0x01010101 - the resulting bit -> K-slot permutation is the same for both
//     operands, and a contraction is blind to it) and stores them in the K-major SWIZZLE_NONE
//     canonical layout of UMMA shared-memory descriptors (8 rows x 16 B core matrices).  Loads run
//     two chunks ahead of the expansion; a warp arrives once on the stage's "full" barrier.  Row
//     popcounts are accumulated on the way and handed to the epilogue through a small ring.
//     The weights of a stage are expanded the same way by the same threads, or - when the caller
//     has expanded them once for all pixel tiles (tc5_expand_weights_kernel) - arrive as one bulk
//     copy that completes on the same barrier.
//   * 1 MMA warp: one lane issues, per chunk, one tcgen05.mma per 32 bytes of K (M = 128,
//     N = Ntile) from shared-memory descriptors into one of four TMEM accumulators and commits
//     them to the ring's "empty" barrier, and to the accumulator's "full" barrier after the last
//     chunk.
//   * 8 epilogue warps working on blocks of 128 pixels x 64 channels through two fp32 staging
//     tiles in shared memory.  The shortcut (or the previous output, when accumulating) of the
//     next block is copied into the idle tile with cp.async while the current block is handled,
//     so its HBM latency is hidden behind a whole block of work.  Drain: thread (r, half)
//     tcgen05.ld's 32 accumulator columns of row r, turns AND counts into XOR counts, applies the
//     affine, adds the staged shortcut, writes the fp32 result back in place and stores the 32
//     sign bits it now holds.  Write-out: one bulk copy (shared -> global) per pixel row.
//
// Every wait on an mbarrier is bounded: after a fixed number of polls the CTA records an error
// code in a device-side status word, raises a CTA-wide abort flag that every role checks, frees
// its TMEM and returns.
#pragma once
#include <cuda.h>   // CUtensorMap (type only; the encoder is fetched from the driver at run time)

#include "bcontract.cuh"

namespace dabnn {

constexpr int TC5_LBO = 128;                             // byte stride between 16-byte K units
constexpr int TC5_MAX_N = 128;
constexpr int TC5_ACCS = 4;                              // TMEM accumulators (4 x 128 columns = all of TMEM)
constexpr int TC5_POPRING = 12;                          // tiles of row popcounts in flight (> stages + accumulators)
constexpr int TC5_PRODUCERS = 256, TC5_EPILOGUE = 256;
constexpr int TC5_THREADS = TC5_PRODUCERS + TC5_EPILOGUE + 32;
constexpr int TC5_MMA_WARP = (TC5_PRODUCERS + TC5_EPILOGUE) / 32;
constexpr uint32_t TC5_SPIN_LIMIT = 1u << 22;   // polls before a wait gives up (at least 0.1 s)

__device__ int g_tc5_status;  // 0 = ok; otherwise the code of the first wait that gave up

__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, int sbo) {
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)((TC5_LBO >> 4) & 0x3FFF) << 16) |
           ((uint64_t)((sbo >> 4) & 0x3FFF) << 32) | ((uint64_t)1 << 46);  // version 1, no swizzle
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait; gives up (returns false) when the barrier does not flip or the CTA is aborting.
// Every poll is a shared-memory access, and these kernels are bound by the shared-memory pipe: SLEEP_NS > 0
// makes a waiting thread sleep between polls, as long as the role's slack allows (the epilogue is four
// accumulators behind, the producers a ring of stages ahead).
template <int SLEEP_NS = 0>
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const volatile int* abort_flag) {
    const uint32_t addr = smem_u32(bar);
    constexpr uint32_t LIMIT = SLEEP_NS >= 64 ? (1u << 28) / SLEEP_NS : TC5_SPIN_LIMIT;   // at least 0.1 s either way
    for (uint32_t it = 0; it < LIMIT; it++) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred P1;\n\tmbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n\tselp.b32 %0, 1, 0, P1;\n\t}"
                     : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
        if (SLEEP_NS > 0) __nanosleep(SLEEP_NS);
        if ((it & 255u) == 255u && *abort_flag) return false;
    }
    return false;
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mma_i8_ss(uint32_t d_tmem, uint64_t ad, uint64_t bd, uint32_t idesc, uint32_t accum) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}\n"
                 ::"r"(d_tmem), "l"(ad), "l"(bd), "r"(idesc), "r"(accum), "r"(0), "r"(0), "r"(0), "r"(0) : "memory");
}

// Shapes that depend on the K chunk: CW 64-bit words per chunk (a producer thread owns CW / 2 of them) and
// 8 / CW ring stages, 128 KB of stages either way.  Long chunks amortise the per-stage hand-shake (a
// tcgen05.commit alone costs the issuing thread ~270 cycles) over more MMAs; short K keeps short chunks so
// that its few words still spread over several stages.
template <int CW>
struct Tc5Cfg {
    static constexpr int WORDS = CW, WPT = CW / 2, STAGES = 8 / CW;
    static constexpr int CHUNK_BYTES = CW * 64;                      // operand bytes per row per chunk
    static constexpr int SBO = (CHUNK_BYTES / 16) * 128;             // byte stride between 8-row groups
    static constexpr int A_BYTES = 128 * CHUNK_BYTES;
    static constexpr int B_BYTES = TC5_MAX_N * CHUNK_BYTES;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    // Staging tile of a block: two boxes of 128 pixels x 32 channels of fp32 in the 128-byte-swizzled layout of
    // TMA tensor copies: 16-byte chunk q of row r of a box sits at r * 128 + ((q ^ (r & 7)) << 4).  Thread-per-row
    // accesses are then conflict-free, and one tensor store per box writes the block out.
    static constexpr int SBOX_BYTES = 128 * 128;                     // 16 KB
    static constexpr int STILE_BYTES = 2 * SBOX_BYTES;               // 32 KB: 128 pixels x 64 channels of fp32
    static constexpr int TOTAL = STAGES * STAGE_BYTES + 2 * STILE_BYTES + 1024 /*alignment slack*/;
};
__host__ __device__ inline int tc5_chunk_words(int kwords) { return kwords <= 12 ? 2 : 4; }

// 32 bits -> 32 bytes {0,1}: output word s holds bits s, s+8, s+16, s+24.  Two 16-byte stores.
__device__ __forceinline__ void expand32(unsigned char* dst_unit0, uint32_t w) {
    const uint32_t M1 = 0x01010101u;
    uint4 lo, hi;
    lo.x = w & M1;        lo.y = (w >> 1) & M1; lo.z = (w >> 2) & M1; lo.w = (w >> 3) & M1;
    hi.x = (w >> 4) & M1; hi.y = (w >> 5) & M1; hi.z = (w >> 6) & M1; hi.w = (w >> 7) & M1;
    *reinterpret_cast<uint4*>(dst_unit0) = lo;
    *reinterpret_cast<uint4*>(dst_unit0 + TC5_LBO) = hi;
}
// one 64-bit word of one operand row: four 16-byte units at a 128-byte stride
__device__ __forceinline__ void expand_word(unsigned char* dst, uint64_t w) {
    expand32(dst, (uint32_t)w);
    expand32(dst + 2 * TC5_LBO, (uint32_t)(w >> 32));
}
// the same into shared memory, by shared address
__device__ __forceinline__ void expand32_smem(uint32_t dst_unit0, uint32_t w) {
    const uint32_t M1 = 0x01010101u;
    sts128(dst_unit0, w & M1, (w >> 1) & M1, (w >> 2) & M1, (w >> 3) & M1);
    sts128(dst_unit0 + TC5_LBO, (w >> 4) & M1, (w >> 5) & M1, (w >> 6) & M1, (w >> 7) & M1);
}
__device__ __forceinline__ void expand_word_smem(uint32_t dst, uint64_t w) {
    expand32_smem(dst, (uint32_t)w);
    expand32_smem(dst + 2 * TC5_LBO, (uint32_t)(w >> 32));
}

// Weights expanded once instead of once per pixel tile: for every 128-channel block and every K chunk one
// 16 KB image of the stage's weight half, exactly as the producers would write it, so that a stage's weights
// become one bulk copy (global -> shared, completion on the stage's "full" mbarrier) issued by one thread.
// The buffer ends with the popcount of every weight row (one int per channel, padded to whole channel blocks).
__host__ __device__ inline size_t tc5_expanded_image_bytes(int N, int kwords) {
    const int cw = tc5_chunk_words(kwords);
    return (size_t)((N + TC5_MAX_N - 1) / TC5_MAX_N) * ((kwords + cw - 1) / cw) * (TC5_MAX_N * cw * 64);
}
__host__ __device__ inline size_t tc5_expanded_bytes(int N, int kwords) {
    return tc5_expanded_image_bytes(N, kwords) + (size_t)((N + TC5_MAX_N - 1) / TC5_MAX_N) * TC5_MAX_N * sizeof(int);
}
template <int CW, class WOp>
__global__ void __launch_bounds__(256) tc5_expand_weights_kernel(const WOp wop, const int N, const int kwords, unsigned char* dst) {
    using C = Tc5Cfg<CW>;
    const int c = blockIdx.x, nt = blockIdx.y, r = threadIdx.x & 127, h = threadIdx.x >> 7;
    const int n = nt * TC5_MAX_N + r;
    for (int j = 0; j < C::WPT; j++) {
        const int q = c * C::WORDS + C::WPT * h + j;
        uint64_t w = 0;
        if (n < N && q < kwords) {
            const uint64_t* p = wop.addr(wop.make_row(n), wop.decode(q));
            if (p) w = __ldg(p);
        }
        expand_word(dst + ((size_t)nt * gridDim.x + c) * C::B_BYTES + (r >> 3) * C::SBO + (r & 7) * 16 + (C::WPT * h + j) * 4 * TC5_LBO, w);
    }
    if (c == 0 && h == 0) {   // row popcounts, once
        int pc = 0;
        if (n < N) {
            const RowCtx wr = wop.make_row(n);
            typename WOp::Dec d = wop.decode(0);
            for (int q = 0; q < kwords; q++) {
                const uint64_t* p = wop.addr(wr, d);
                pc += p ? __popcll(__ldg(p)) : 0;
                wop.advance(d, 1);
            }
        }
        reinterpret_cast<int*>(dst + tc5_expanded_image_bytes(N, kwords))[n] = pc;
    }
}

template <int CW, class XOp, class WOp>
__global__ void __launch_bounds__(TC5_THREADS, 1)
    bcontract_tc5_kernel(const XOp xop, const WOp wop, const EpilogueParams ep, const int M, const int N,
                         const int kwords, const int ntiles_m, const __grid_constant__ CUtensorMap out_map) {
    using C = Tc5Cfg<CW>;
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) uint64_t bar_full[C::STAGES], bar_empty[C::STAGES], bar_acc_full[TC5_ACCS], bar_acc_empty[TC5_ACCS];
    __shared__ uint32_t tmem_base_s;
    __shared__ int s_abort, epi_abort;
    __shared__ int popw[TC5_MAX_N], popx[TC5_POPRING][2][128];
    __shared__ __align__(16) float chan_a[TC5_MAX_N];   // read as float4 by the write-out
    __shared__ __align__(16) float chan_b[TC5_MAX_N];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.y * TC5_MAX_N;
    const int n_this = min(TC5_MAX_N, N - n0);               // multiple of 16 (host-checked)
    unsigned char* stage0 = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
    const int nchunks = (kwords + C::WORDS - 1) / C::WORDS;
    int tmem_cols = 32;
    while (tmem_cols < TC5_ACCS * n_this) tmem_cols <<= 1;
    const volatile int* abort_flag = &s_abort;
    const bool pre = ep.w_expanded != nullptr;   // stage weights arrive by bulk copy

    // ---- set-up (all threads) ----
    if (warp == TC5_MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(tmem_cols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    if (tid == 0) {
        for (int i = 0; i < C::STAGES; i++) { mbar_init(&bar_full[i], TC5_PRODUCERS / 32 + (pre ? 1 : 0)); mbar_init(&bar_empty[i], 1); }
        for (int i = 0; i < TC5_ACCS; i++) { mbar_init(&bar_acc_full[i], 1); mbar_init(&bar_acc_empty[i], TC5_EPILOGUE / 32); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::);
        s_abort = 0;
        epi_abort = 0;
    }
    if (tid < TC5_MAX_N) {
        int pc = 0;
        if (pre) {
            pc = __ldg(reinterpret_cast<const int*>(ep.w_expanded + tc5_expanded_image_bytes(N, kwords)) + n0 + tid);
        } else if (tid < n_this) {
            const RowCtx wr = wop.make_row(n0 + tid);
            typename WOp::Dec d = wop.decode(0);
            for (int q = 0; q < kwords; q++) {
                const uint64_t* p = wop.addr(wr, d);
                pc += p ? __popcll(__ldg(p)) : 0;
                wop.advance(d, 1);
            }
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

    if (tid < TC5_PRODUCERS) {
        // =========================== producers: thread = (operand row, word of the chunk) ===========================
        const int r = tid & 127, h = tid >> 7;
        const bool has_w = r < n_this && !pre;
        const unsigned char* wsrc = pre ? ep.w_expanded + (size_t)blockIdx.y * nchunks * C::B_BYTES : nullptr;
        const RowCtx wrow = wop.make_row(n0 + r);
        const int roff = (r >> 3) * C::SBO + (r & 7) * 16 + C::WPT * h * 4 * TC5_LBO;
        const uint32_t stage0_addr = smem_u32(stage0);
        uint32_t s = 0, use = 0;   // ring stage to fill next and how often the ring has wrapped
        bool ok = true;
        // The loads run two chunks ahead of the expansion and do not stop at tile boundaries: the cursor below walks
        // (tile, chunk) for the word being *loaded*, so that the first chunks of a tile are already in flight while the
        // last chunks of the tile before are expanded (with a few chunks per tile their latency would otherwise be
        // paid once per tile).
        struct Pair { uint64_t a[C::WPT], b[C::WPT]; };
        int ltile = blockIdx.x, lchunk = 0, qload = C::WPT * h;          // cursor: tile, chunk, first word index
        RowCtx xr = xop.make_row(ltile * 128 + r);
        typename XOp::Dec xd = xop.decode(C::WPT * h);
        typename WOp::Dec wd = wop.decode(C::WPT * h);
        auto load_next = [&](Pair& v) {   // this thread's words of the next chunk
#pragma unroll
            for (int j = 0; j < C::WPT; j++) {
                v.a[j] = 0; v.b[j] = 0;
                if (ltile < ntiles_m && qload + j < kwords) {
                    const uint64_t* p = xop.addr(xr, xd);
                    if (p) v.a[j] = __ldg(p);
                    if (has_w) { const uint64_t* w = wop.addr(wrow, wd); if (w) v.b[j] = __ldg(w); }
                }
                const int adv = j == C::WPT - 1 ? C::WORDS - (C::WPT - 1) : 1;
                xop.advance(xd, adv);
                if (has_w) wop.advance(wd, adv);
            }
            qload += C::WORDS;
            if (++lchunk == nchunks) {   // on to the next tile of this CTA
                lchunk = 0;
                ltile += gridDim.x;
                qload = C::WPT * h;
                xr = xop.make_row(ltile * 128 + r);
                xd = xop.decode(C::WPT * h);
                wd = wop.decode(C::WPT * h);
            }
        };
        Pair v0, v1;   // chunk c and chunk c+1; chunk c+2 is loaded inside the loop
        load_next(v0);
        load_next(v1);
        int i = 0;
        for (int tile = blockIdx.x; tile < ntiles_m && ok; tile += gridDim.x, i++) {
            int px = 0;
            for (int c = 0; c < nchunks; c++) {
                Pair v2;
                load_next(v2);
                if (use >= 1 && !__all_sync(0xffffffffu, mbar_wait<100>(&bar_empty[s], (use - 1) & 1, abort_flag))) {   // warp-uniform
                    atomicCAS(&g_tc5_status, 0, 1);
                    s_abort = 1;
                    ok = false;
                    break;
                }
                if (pre && tid == 0) {   // this stage's weights: one bulk copy that completes on the stage's "full" barrier
                    const uint32_t bytes = (uint32_t)n_this * C::CHUNK_BYTES, bar = smem_u32(&bar_full[s]);
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                 ::"r"(smem_u32(stage0 + s * C::STAGE_BYTES + C::A_BYTES)), "l"(wsrc + (size_t)c * C::B_BYTES),
                                   "r"(bytes), "r"(bar) : "memory");
                }
                const uint32_t st = stage0_addr + s * C::STAGE_BYTES + roff;
#pragma unroll
                for (int j = 0; j < C::WPT; j++) {
                    expand_word_smem(st + j * 4 * TC5_LBO, v0.a[j]);
                    if (has_w) expand_word_smem(st + C::A_BYTES + j * 4 * TC5_LBO, v0.b[j]);
                    px += __popcll(v0.a[j]);
                }
                if (c == nchunks - 1) popx[i % TC5_POPRING][h][r] = px;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_full[s]);   // one arrival per warp: arrivals on one mbarrier are serialised
                if (++s == C::STAGES) { s = 0; use++; }
                v0 = v1; v1 = v2;
            }
        }
    } else if (warp == TC5_MMA_WARP) {
        // =========================== MMA issue: one lane ===========================
        if (lane == 0) {
            // instruction descriptor: D = s32, A = u8, B = u8, both K-major, N = n_this, M = 128
            const uint32_t idesc = (2u << 4) | ((uint32_t)(n_this >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
            // The issuing thread is a single instruction stream, so its own latency bounds the MMA rate: the
            // descriptors are built once and advanced by adding byte offsets >> 4 to their address field
            // (shared-memory addresses stay below 2^18, so the 14-bit field cannot carry).
            const uint64_t d_a = umma_desc(smem_u32(stage0), C::SBO), d_b = d_a + (C::A_BYTES >> 4);
            uint32_t s = 0, par = 0;
            bool ok = true;
            int i = 0;
            for (int tile = blockIdx.x; tile < ntiles_m && ok; tile += gridDim.x, i++) {
                const int accbuf = i % TC5_ACCS, accuse = i / TC5_ACCS;
                if (accuse >= 1 && !mbar_wait(&bar_acc_empty[accbuf], (accuse - 1) & 1, abort_flag)) {
                    atomicCAS(&g_tc5_status, 0, 3);
                    s_abort = 1;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + accbuf * n_this;
                uint32_t accum = 0;
                for (int c = 0; c < nchunks; c++) {
                    if (!mbar_wait<32>(&bar_full[s], par, abort_flag)) {
                        atomicCAS(&g_tc5_status, 0, 4);
                        s_abort = 1;
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t ad = d_a + (uint64_t)(s * (C::STAGE_BYTES >> 4)), bd = d_b + (uint64_t)(s * (C::STAGE_BYTES >> 4));
                    // one MMA per 32 bytes of K = two 16-byte units = 256 bytes of descriptor address
                    const int slices = min(2 * C::WORDS, 2 * (kwords - c * C::WORDS));
#pragma unroll
                    for (int j = 0; j < 2 * C::WORDS; j++) {
                        if (j < slices) {
                            mma_i8_ss(d_tmem, ad + j * 16, bd + j * 16, idesc, accum);
                            accum = 1u;
                        }
                    }
                    umma_commit(&bar_empty[s]);
                    if (++s == C::STAGES) { s = 0; par ^= 1u; }
                }
                if (ok) umma_commit(&bar_acc_full[accbuf]);
            }
        }
    } else {
        // =========================== epilogue ===========================
        // The channels of a tile are handled in blocks of 64.  Per block k (a counter over the
        // whole kernel): [barrier] -> prefetch block k+1's shortcut into the other staging tile
        // with cp.async -> drain: thread (r, h2) reads 32 accumulator columns of row r, converts,
        // applies the affine, adds the staged shortcut, writes the result back in place and stores
        // the 32 sign bits it now holds -> [barrier] -> write-out: one TMA tensor store per 32-channel
        // box, so the fp32 output costs the load/store pipe nothing and the copy engine two requests.
        const int et = tid - TC5_PRODUCERS;
        const int r = et & 127, h2 = et >> 7;          // drain role: TMEM lane quarter = warp % 4 = r / 32
        const uint32_t sbuf0_addr = smem_u32(stage0 + C::STAGES * C::STAGE_BYTES);
        const float* addsrc = ep.shortcut ? ep.shortcut : (ep.accumulate ? ep.out : nullptr);
        const long long ld_add = ep.shortcut ? ep.ld_sc : ep.ld_out;
        const int nblk = (n_this + 63) >> 6;           // 64-channel blocks per tile
        int my_tiles = 0;
        for (int t = blockIdx.x; t < ntiles_m; t += gridDim.x) my_tiles++;
        const int total_blocks = my_tiles * nblk;

        // issue the shortcut copies of block kb into staging tile kb & 1 (one commit group per call)
        auto prefetch = [&](int kb) {
            if (addsrc && kb < total_blocks) {
                const int tile = blockIdx.x + (kb / nblk) * gridDim.x, cb = (kb % nblk) * 64;
                const int width = min(64, n_this - cb);
                const uint32_t sbase = sbuf0_addr + (kb & 1) * C::STILE_BYTES;
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const int it = et + j * TC5_EPILOGUE, rr = it >> 4, c4 = (it & 15) * 4;
                    const int row = tile * 128 + rr;
                    if (row < M && c4 < width)
                        cp_async16(sbase + (c4 >> 5) * C::SBOX_BYTES + rr * 128 + ((((c4 & 31) >> 2) ^ (rr & 7)) << 4),
                                   addsrc + (long long)row * ld_add + n0 + cb + c4, 16);
                }
            }
            cp_async_commit();
        };
        prefetch(0);
        bool okw = true;
        for (int kb = 0; kb < total_blocks; kb++) {
            const int i = kb / nblk, blk = kb % nblk;
            const int tile = blockIdx.x + i * gridDim.x, cb = blk * 64;
            const int width = min(64, n_this - cb);
            const int accbuf = i % TC5_ACCS, accuse = i / TC5_ACCS;
            const uint32_t sb = sbuf0_addr + (kb & 1) * C::STILE_BYTES;
            cp_async_wait<0>();                                               // my copies of block kb have landed
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");    // my row stores of block kb-1 have read their source
            asm volatile("bar.sync 1, %0;" ::"n"(TC5_EPILOGUE) : "memory");   // everybody's have: the other staging tile is idle
            prefetch(kb + 1);
            // ---- drain ----
            const int ncol = max(0, min(32, width - h2 * 32));               // 0, 16 or 32 columns for this thread
            if (blk == 0 && okw) {
                okw = __all_sync(0xffffffffu, mbar_wait<500>(&bar_acc_full[accbuf], accuse & 1, abort_flag));   // warp-uniform
                if (!okw) {
                    atomicCAS(&g_tc5_status, 0, 2);
                    s_abort = 1;
                    epi_abort = 1;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            }
            if (okw && ncol > 0) {
                const int px = popx[i % TC5_POPRING][0][r] + popx[i % TC5_POPRING][1][r];
                const int c0 = cb + h2 * 32;
                const uint32_t t_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + accbuf * n_this + c0;
                uint32_t v[32];
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                             : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                               "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                             : "r"(t_addr));
                if (ncol > 16)
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                                 : "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                                   "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                                 : "r"(t_addr + 16));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                const uint32_t srow = sb + h2 * C::SBOX_BYTES + r * 128;   // chunk q of this row: srow + ((q ^ (r & 7)) << 4)
                uint32_t signs = 0;   // bit j: channel c0 + j of this row is positive
#pragma unroll
                for (int q = 0; q < 8; q++) {
                    if (q * 4 >= ncol) break;
                    float o[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const int cl = c0 + q * 4 + e;
                        float f = small_int_to_float(px + popw[cl] - 2 * (int)v[q * 4 + e]);
                        if (ep.a) f = __fadd_rn(__fmul_rn(chan_a[cl], f), chan_b[cl]);
                        o[e] = f;
                    }
                    if (addsrc) {
                        const float4 ad = lds128f(srow + ((q ^ (r & 7)) << 4));
                        o[0] = __fadd_rn(ad.x, o[0]); o[1] = __fadd_rn(ad.y, o[1]);
                        o[2] = __fadd_rn(ad.z, o[2]); o[3] = __fadd_rn(ad.w, o[3]);
                    }
                    sts128f(srow + ((q ^ (r & 7)) << 4), o[0], o[1], o[2], o[3]);
                    signs |= ((o[0] > 0.f ? 1u : 0u) | (o[1] > 0.f ? 2u : 0u) | (o[2] > 0.f ? 4u : 0u) | (o[3] > 0.f ? 8u : 0u)) << (q * 4);
                }
                // this thread holds 32 consecutive channels of its row: half of one packed word (the low half first)
                const long long row = (long long)tile * 128 + r;
                if (ep.bits && row < M) reinterpret_cast<uint32_t*>(ep.bits + row * ep.ld_bits + ((n0 + cb) >> 6))[h2] = signs;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the bulk store below reads what was just written
            }
            if (blk == nblk - 1 && okw) {   // the whole accumulator has been read
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_acc_empty[accbuf]);
            }
            asm volatile("bar.sync 1, %0;" ::"n"(TC5_EPILOGUE) : "memory");   // results of block kb are staged (or abort decided)
            if (epi_abort) break;
            // ---- write-out: one tensor store (shared -> global, rows beyond M and channels beyond N clipped) per box ----
            if (ep.out && (et == 0 || (et == 128 && width > 32))) {
                const int hb = et >> 7;
                asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                             ::"l"(reinterpret_cast<uint64_t>(&out_map)), "r"(n0 + cb + hb * 32), "r"(tile * 128), "r"(sb + hb * C::SBOX_BYTES) : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
        }
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // the last row stores are complete before the CTA winds down
        cp_async_wait<0>();   // nothing of this thread's is in flight when the CTA winds down
    }

    // ---- drain: everybody is past its last use of the tensor memory ----
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == TC5_MMA_WARP) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols));
    }
}

}  // namespace dabnn
