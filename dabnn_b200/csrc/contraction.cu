// C-ABI entry points built on the binary contraction core: bgemm, bconv, the fused residual
// block and the BinConv operator.
#include <algorithm>

#include "bcontract_tc5.cuh"
#include "kernels.h"

namespace dabnn {

// engine of the calling thread's most recent contraction launch (dabnn_last_engine)
static thread_local int g_last_engine = DABNN_ENGINE_AUTO;

template <int ENGINE, int WM, int WN, bool FAST, class XOp, class WOp>
static int launch_one(const XOp& xop, const WOp& wop, const EpilogueParams& ep, int M, int N, int kwords,
                      cudaStream_t stream) {
    using Cfg = TileCfg<WM, WN>;
    auto kern = bcontract_kernel<ENGINE, WM, WN, FAST, XOp, WOp>;
    static thread_local int configured_device = -1;  // per (instantiation, thread): opt in once per device
    int dev = 0;
    DABNN_CUDA_OK(cudaGetDevice(&dev));
    if (configured_device != dev) {
        DABNN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)Cfg::SMEM_BYTES));
        configured_device = dev;
    }
    // persistent CTAs: two per SM in total, spread over the channel tiles
    const int tiles_m = (M + Cfg::TM - 1) / Cfg::TM, tiles_n = (N + Cfg::TN - 1) / Cfg::TN;
    const int per_n = std::max(1, 2 * sm_count() / tiles_n);
    dim3 grid(std::min(tiles_m, per_n), tiles_n);
    kern<<<grid, Cfg::NT, Cfg::SMEM_BYTES, stream>>>(xop, wop, ep, M, N, kwords, tiles_m);
    return check_launch("bcontract_kernel");
}

template <int ENGINE, class XOp, class WOp>
static int launch_engine(const XOp& xop, const WOp& wop, const EpilogueParams& ep, int M, int N, int kwords,
                         cudaStream_t stream) {
    auto al8 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 7) == 0; };
    const bool fast = N % 8 == 0 && (!ep.out || (ep.ld_out % 2 == 0 && al8(ep.out))) &&
                      (!ep.shortcut || (ep.ld_sc % 2 == 0 && al8(ep.shortcut)));
    const bool narrow = N <= 64;  // 256 x 64 tiles for 64-channel layers, 128 x 128 otherwise
    if (fast)
        return narrow ? launch_one<ENGINE, 8, 1, true>(xop, wop, ep, M, N, kwords, stream)
                      : launch_one<ENGINE, 4, 2, true>(xop, wop, ep, M, N, kwords, stream);
    return narrow ? launch_one<ENGINE, 8, 1, false>(xop, wop, ep, M, N, kwords, stream)
                  : launch_one<ENGINE, 4, 2, false>(xop, wop, ep, M, N, kwords, stream);
}

// tcgen05 engine: persistent warp-specialised CTAs, one per SM (it owns all of the SM's tensor memory)
template <int CW, class XOp, class WOp>
static int launch_tc5_cw(const XOp& xop, const WOp& wop, const EpilogueParams& ep, int M, int N, int kwords,
                         cudaStream_t stream) {
    auto kern = bcontract_tc5_kernel<CW, XOp, WOp>;
    static thread_local int configured_device = -1;
    int dev = 0;
    DABNN_CUDA_OK(cudaGetDevice(&dev));
    if (configured_device != dev) {
        DABNN_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Tc5Cfg<CW>::TOTAL));
        configured_device = dev;
    }
    const int tiles_m = (M + 127) / 128, tiles_n = (N + TC5_MAX_N - 1) / TC5_MAX_N;
    const int per_n = std::max(1, sm_count() / tiles_n);
    dim3 grid(std::min(tiles_m, per_n), tiles_n);
    CUtensorMap out_map{};
    const unsigned long long dims[2] = {(unsigned long long)N, (unsigned long long)M}, strides[1] = {(unsigned long long)ep.ld_out * sizeof(float)};
    const unsigned box[2] = {32, 128};
    if (ep.out && !make_f32_tensor_map(&out_map, ep.out, 2, dims, strides, box)) {
        g_last_engine = DABNN_ENGINE_IMMA;
        return launch_engine<ENG_IMMA>(xop, wop, ep, M, N, kwords, stream);   // no TMA descriptor: the mma.sync engine
    }
    kern<<<grid, TC5_THREADS, Tc5Cfg<CW>::TOTAL, stream>>>(xop, wop, ep, M, N, kwords, tiles_m, out_map);
    return check_launch("bcontract_tc5_kernel");
}
template <class XOp, class WOp>
static int launch_tc5(const XOp& xop, const WOp& wop, const EpilogueParams& ep, int M, int N, int kwords,
                      cudaStream_t stream) {
    return tc5_chunk_words(kwords) == 2 ? launch_tc5_cw<2>(xop, wop, ep, M, N, kwords, stream)
                                        : launch_tc5_cw<4>(xop, wop, ep, M, N, kwords, stream);
}

static bool tc5_eligible(const EpilogueParams& ep, int N) {
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    return N % 16 == 0 && (!ep.out || (ep.ld_out % 4 == 0 && al16(ep.out))) &&
           (!ep.shortcut || (ep.ld_sc % 4 == 0 && al16(ep.shortcut))) && (!ep.bits || N % 64 == 0);
}

template <class XOp, class WOp>
int launch_bcontract(int engine, const XOp& xop, const WOp& wop, const EpilogueParams& ep, int M, int N,
                     int kwords, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return DABNN_OK;
    DABNN_REQUIRE(kwords < (1 << 17), DABNN_ERR_SHAPE, "contraction: K must be below 2^23 bits");
    if (engine == DABNN_ENGINE_AUTO) engine = DABNN_ENGINE_TCGEN05;
    if (engine == DABNN_ENGINE_TCGEN05 && !tc5_eligible(ep, N)) engine = DABNN_ENGINE_IMMA;
    g_last_engine = engine;
    switch (engine) {
        case DABNN_ENGINE_TCGEN05: return launch_tc5(xop, wop, ep, M, N, kwords, stream);
        case DABNN_ENGINE_POPC: return launch_engine<ENG_POPC>(xop, wop, ep, M, N, kwords, stream);
        case DABNN_ENGINE_B1: return launch_engine<ENG_B1>(xop, wop, ep, M, N, kwords, stream);
        case DABNN_ENGINE_IMMA: return launch_engine<ENG_IMMA>(xop, wop, ep, M, N, kwords, stream);
        default: return fail(DABNN_ERR_ARG, "unknown contraction engine");
    }
}

static ConvOperand make_conv_operand(const uint64_t* in, int n, int h, int w, int cw, int kh, int kw,
                                     int pad_h, int pad_w, int stride_h, int stride_w) {
    ConvOperand op;
    op.p = in; op.n = n; op.H = h; op.W = w; op.Cw = cw;
    op.OH = conv_out_dim(h, pad_h, 1, kh, stride_h);
    op.OW = conv_out_dim(w, pad_w, 1, kw, stride_w);
    op.kh = kh; op.kw = kw; op.pad_h = pad_h; op.pad_w = pad_w; op.stride_h = stride_h; op.stride_w = stride_w;
    op.rows = n * op.OH * op.OW;
    op.kwords = kh * kw * cw;
    return op;
}

static int check_conv_args(const void* in, const void* weight, size_t weight_words, int n, int h, int w,
                           int cw, int cout, int kh, int kw, int pad_h, int pad_w, int stride_h,
                           int stride_w) {
    DABNN_REQUIRE(in && weight, DABNN_ERR_ARG, "bconv: null pointer");
    DABNN_REQUIRE(n > 0 && h > 0 && w > 0 && cw > 0 && cout > 0 && kh > 0 && kw > 0 && stride_h > 0 &&
                      stride_w > 0 && pad_h >= 0 && pad_w >= 0,
                  DABNN_ERR_ARG, "bconv: non-positive dimension");
    DABNN_REQUIRE(weight_words % (size_t)cout == 0, DABNN_ERR_SHAPE,
                  "weight.total() % weight.n == 0 is not satisfied!");  // baseline.h:83
    DABNN_REQUIRE(weight_words / cout >= (size_t)kh * kw * cw, DABNN_ERR_SHAPE,
                  "bconv: filter rows shorter than kh*kw*cw words");
    DABNN_REQUIRE(conv_out_dim(h, pad_h, 1, kh, stride_h) > 0 && conv_out_dim(w, pad_w, 1, kw, stride_w) > 0,
                  DABNN_ERR_SHAPE, "bconv: empty output");
    DABNN_REQUIRE((long long)n * h * w < (1ll << 31) / 2, DABNN_ERR_SHAPE, "bconv: too many pixels");
    return DABNN_OK;
}

size_t bconv_expanded_weight_bytes(int cout, int kwords) { return tc5_expanded_bytes(cout, kwords); }

int bconv_expand_weights(const uint64_t* weight, size_t weight_words, int cout, int kwords, unsigned char* dst,
                         cudaStream_t stream) {
    DABNN_REQUIRE(weight && dst && cout > 0 && kwords > 0, DABNN_ERR_ARG, "expand_weights: bad arguments");
    DABNN_REQUIRE(weight_words % (size_t)cout == 0 && weight_words / cout >= (size_t)kwords, DABNN_ERR_SHAPE,
                  "expand_weights: filter rows shorter than kwords");
    DABNN_REQUIRE((reinterpret_cast<uintptr_t>(dst) & 15) == 0, DABNN_ERR_ARG, "expand_weights: dst must be 16-byte aligned");
    RowMajorOperand wop{weight, (long long)(weight_words / cout), cout, kwords};
    const int cw = tc5_chunk_words(kwords);
    dim3 grid((kwords + cw - 1) / cw, (cout + TC5_MAX_N - 1) / TC5_MAX_N);
    if (cw == 2) tc5_expand_weights_kernel<2><<<grid, 256, 0, stream>>>(wop, cout, kwords, dst);
    else tc5_expand_weights_kernel<4><<<grid, 256, 0, stream>>>(wop, cout, kwords, dst);
    return check_launch("tc5_expand_weights_kernel");
}

int bconv_block_impl(const uint64_t* in_bits, const uint64_t* weight, size_t weight_words, const float* a,
                     const float* b, const float* shortcut, float* out_f32, uint64_t* out_bits, int n, int h,
                     int w, int cw, int cout, int kh, int kw, int pad_h, int pad_w, int stride_h,
                     int stride_w, int engine, cudaStream_t stream, const unsigned char* w_expanded) {
    int rc = check_conv_args(in_bits, weight, weight_words, n, h, w, cw, cout, kh, kw, pad_h, pad_w, stride_h,
                             stride_w);
    if (rc) return rc;
    DABNN_REQUIRE((a == nullptr) == (b == nullptr), DABNN_ERR_ARG, "bconv_block: a and b go together");
    DABNN_REQUIRE(out_f32 || out_bits, DABNN_ERR_ARG, "bconv_block: no output requested");
    DABNN_REQUIRE(!out_bits || cout % 64 == 0, DABNN_ERR_SHAPE, "bconv_block: bit output needs cout % 64 == 0");
    const ConvOperand xop = make_conv_operand(in_bits, n, h, w, cw, kh, kw, pad_h, pad_w, stride_h, stride_w);
    RowMajorOperand wop{weight, (long long)(weight_words / cout), cout, xop.kwords};
    EpilogueParams ep{out_f32, cout, 0, a, b, shortcut, cout, out_bits, cout / 64, w_expanded};
    return launch_bcontract(engine, xop, wop, ep, xop.rows, cout, xop.kwords, stream);
}

}  // namespace dabnn

using namespace dabnn;

extern "C" int dabnn_bgemm(int m, int n, int k, const uint64_t* a, int lda, const uint64_t* b, int ldb,
                           float* c, int ldc, int engine, dabnn_stream_t s) {
    DABNN_REQUIRE(m >= 0 && n >= 0 && k >= 0, DABNN_ERR_ARG, "bgemm: negative dimension");
    if (m == 0 || n == 0) return DABNN_OK;
    DABNN_REQUIRE(a && b && c, DABNN_ERR_ARG, "bgemm: null pointer");
    DABNN_REQUIRE(lda >= m && ldb >= k && ldc >= m, DABNN_ERR_SHAPE, "bgemm: leading dimension too small");
    // pixels (reference n) are the row dimension of the contraction, channels (reference m) the columns
    RowMajorOperand xop{b, ldb, n, k};
    ColMajorOperand wop{a, lda, m, k};
    EpilogueParams ep{c, ldc, 1, nullptr, nullptr, nullptr, 0, nullptr, 0};
    return launch_bcontract(engine, xop, wop, ep, n, m, k, static_cast<cudaStream_t>(s));
}

extern "C" int dabnn_bconv(const uint64_t* in, const uint64_t* weight, size_t weight_words, float* out, int n,
                           int h, int w, int cw, int cout, int kh, int kw, int pad_h, int pad_w, int stride_h,
                           int stride_w, int engine, dabnn_stream_t s) {
    DABNN_REQUIRE(out, DABNN_ERR_ARG, "bconv: null output");
    return bconv_block_impl(in, weight, weight_words, nullptr, nullptr, nullptr, out, nullptr, n, h, w, cw,
                            cout, kh, kw, pad_h, pad_w, stride_h, stride_w, engine,
                            static_cast<cudaStream_t>(s));
}

extern "C" int dabnn_bconv_block(const uint64_t* in_bits, const uint64_t* weight, size_t weight_words,
                                 const float* a, const float* b, const float* shortcut, float* out_f32,
                                 uint64_t* out_bits, int n, int h, int w, int cw, int cout, int kh, int kw,
                                 int pad_h, int pad_w, int stride_h, int stride_w, int engine,
                                 dabnn_stream_t s) {
    return bconv_block_impl(in_bits, weight, weight_words, a, b, shortcut, out_f32, out_bits, n, h, w, cw,
                            cout, kh, kw, pad_h, pad_w, stride_h, stride_w, engine,
                            static_cast<cudaStream_t>(s));
}

// ---- BinConv operator ----------------------------------------------------------------------------
// cin % 64 == 0: pack the input once (N*H*W*cin/8 bytes of scratch) and run the implicit-GEMM
// convolution on it.  Any other cin: materialise the reference's fused binarize-im2col rows
// (pixels x ceil(kh*kw*cin/128)*2 words of scratch) and run the packed GEMM, which is what the
// reference does for every cin != 64 (BinConv.cpp:166-182).
extern "C" size_t dabnn_binconv_workspace_bytes(int n, int h, int w, int cin, int kh, int kw, int pad_h,
                                                int pad_w, int stride_h, int stride_w) {
    if (n <= 0 || h <= 0 || w <= 0 || cin <= 0 || kh <= 0 || kw <= 0 || stride_h <= 0 || stride_w <= 0) return 0;
    if (cin % 64 == 0) return (size_t)n * h * w * (cin / 64) * sizeof(uint64_t);
    const int oh = conv_out_dim(h, pad_h, 1, kh, stride_h), ow = conv_out_dim(w, pad_w, 1, kw, stride_w);
    if (oh <= 0 || ow <= 0) return 0;
    const size_t row_words = ((size_t)kh * kw * cin + 127) / 128 * 2;
    return (size_t)n * oh * ow * row_words * sizeof(uint64_t);
}

extern "C" int dabnn_binconv_forward(const float* in, const uint64_t* weight, size_t weight_words, float* out,
                                     int n, int h, int w, int cin, int cout, int kh, int kw, int pad_h,
                                     int pad_w, int stride_h, int stride_w, void* workspace,
                                     size_t workspace_bytes, int engine, dabnn_stream_t s) {
    DABNN_REQUIRE(in && weight && out && workspace, DABNN_ERR_ARG, "binconv_forward: null pointer");
    DABNN_REQUIRE(n > 0 && h > 0 && w > 0 && cin > 0 && cout > 0, DABNN_ERR_ARG, "binconv_forward: bad dims");
    const size_t need = dabnn_binconv_workspace_bytes(n, h, w, cin, kh, kw, pad_h, pad_w, stride_h, stride_w);
    DABNN_REQUIRE(need > 0, DABNN_ERR_SHAPE, "binconv_forward: empty output");
    DABNN_REQUIRE(workspace_bytes >= need, DABNN_ERR_ARG, "binconv_forward: workspace too small");
    DABNN_REQUIRE(weight_words % (size_t)cout == 0, DABNN_ERR_SHAPE,
                  "weight_mat->total() % m == 0 is not satisfied!");  // BinConv.cpp:62
    uint64_t* ws = static_cast<uint64_t*>(workspace);
    if (cin % 64 == 0) {
        // the converter packs cin == 64 filters as kh*kw words and every other cin in 128-bit padded
        // rows (OnnxConverter.cpp:121-156); both are "at least kh*kw*cw words per filter" here
        int rc = dabnn_pack_mat(in, ws, n, h, w, cin, s);
        if (rc) return rc;
        return dabnn_bconv(ws, weight, weight_words, out, n, h, w, cin / 64, cout, kh, kw, pad_h, pad_w,
                           stride_h, stride_w, engine, s);
    }
    const int oh = conv_out_dim(h, pad_h, 1, kh, stride_h), ow = conv_out_dim(w, pad_w, 1, kw, stride_w);
    const int row_words = (int)(((size_t)kh * kw * cin + 127) / 128 * 2);
    DABNN_REQUIRE(weight_words / cout == (size_t)row_words, DABNN_ERR_SHAPE,
                  "binconv_forward: filters must be packed in 128-bit padded rows");
    int rc = dabnn_fused_binarize_im2col(in, ws, n, h, w, cin, kh, kw, pad_h, pad_w, stride_h, stride_w, 1, 1, s);
    if (rc) return rc;
    RowMajorOperand xop{ws, row_words, n * oh * ow, row_words};
    RowMajorOperand wop{weight, row_words, cout, row_words};
    EpilogueParams ep{out, cout, 0, nullptr, nullptr, nullptr, 0, nullptr, 0};
    return launch_bcontract(engine, xop, wop, ep, n * oh * ow, cout, row_words, static_cast<cudaStream_t>(s));
}

int dabnn::contraction_status_word(int** addr) {
    DABNN_CUDA_OK(cudaGetSymbolAddress(reinterpret_cast<void**>(addr), g_tc5_status));
    return DABNN_OK;
}

extern "C" int dabnn_last_engine(void) { return g_last_engine; }

extern "C" int dabnn_debug_raise_engine_status(int which, int code) {
    DABNN_REQUIRE(which >= 0 && which <= 2, DABNN_ERR_ARG, "raise_engine_status: which must be 0, 1 or 2");
    int* word = nullptr;
    const int rc = which == 0 ? contraction_status_word(&word) : which == 1 ? fconv_status_word(&word) : bconv_u8_status_word(&word);
    if (rc) return rc;
    DABNN_CUDA_OK(cudaMemcpy(word, &code, sizeof(int), cudaMemcpyHostToDevice));
    return DABNN_OK;
}

extern "C" int dabnn_engine_status(int* status) {
    DABNN_REQUIRE(status, DABNN_ERR_ARG, "null output");
    DABNN_CUDA_OK(cudaDeviceSynchronize());
    DABNN_CUDA_OK(cudaMemcpyFromSymbol(status, g_tc5_status, sizeof(int)));
    if (*status == 0) {   // the float convolution (codes 11-16) and the byte-activation engine (21-24) keep their own words
        const int rc = fconv_tc5_status(status);
        if (rc) return rc;
    }
    if (*status == 0) return bconv_u8_status(status);
    return DABNN_OK;
}
