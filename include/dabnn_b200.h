/* dabnn_b200 - C ABI of the B200 (sm_100a) binary-neural-network inference library.
 *
 * Drop-in boundary for the hot path of JDAI-CV/dabnn: every entry point below replaces one
 * function (or one class method) of the reference and keeps its operand meaning, memory layout and
 * error behaviour.  "reference <file>:<line>" names the interface being replaced, relative to the
 * reference project root.
 *
 * Conventions
 *  - Tensors are dense NHWC.  Float tensors are fp32.  Bit tensors hold C/64 uint64 words per
 *    pixel; bit i of word j is channel 64*j+i and is 1 iff the value is > 0 (strictly).
 *  - Kernel-level entry points take DEVICE pointers and a CUDA stream (a cudaStream_t passed as
 *    void*, NULL = the legacy default stream).  They only enqueue work: no allocation, no
 *    synchronisation.  The reference processes one image; every entry point here also accepts a
 *    leading batch count n (n = 1 reproduces the reference).
 *  - Every function returns DABNN_OK (0) or an error code; dabnn_last_error() gives the text of
 *    the calling thread's most recent failure.  Where the reference throws (BNN_ASSERT ->
 *    std::runtime_error, reference common/helper.h:69-77), the same condition returns
 *    DABNN_ERR_SHAPE / DABNN_ERR_ARG here and launches nothing.
 *  - There is no CPU fallback: without a CUDA device every compute entry point fails.
 */
#ifndef DABNN_B200_H
#define DABNN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    DABNN_OK = 0,
    DABNN_ERR_ARG = 1,          /* null pointer / nonsensical argument */
    DABNN_ERR_SHAPE = 2,        /* shape or alignment rule of the reference violated */
    DABNN_ERR_IO = 3,           /* file cannot be opened / read (reference: std::invalid_argument) */
    DABNN_ERR_FORMAT = 4,       /* not a .dab buffer, wrong model version */
    DABNN_ERR_UNSUPPORTED = 5,  /* layer type the runtime does not run ("Not supported op") */
    DABNN_ERR_NOT_FOUND = 6,    /* blob name unknown (reference: std::out_of_range "Key ... not found.") */
    DABNN_ERR_CUDA = 7,         /* a CUDA call failed */
    DABNN_ERR_OOM = 8,          /* device arena cannot be allocated */
    DABNN_ERR_STATE = 9,        /* call order violated (run before read, ...) */
    DABNN_ERR_TIMEOUT = 10      /* a bounded wait inside a tensor-core kernel gave up: results are incomplete */
};

/* Which contraction engine computes the XOR-popcount sums.  All give identical integers. */
enum {
    DABNN_ENGINE_AUTO = 0,  /* the fastest eligible one: TCGEN05, else IMMA */
    DABNN_ENGINE_POPC = 1,  /* CUDA cores: xor + popc */
    DABNN_ENGINE_B1 = 2,    /* mma.sync m16n8k256 b1 AND-popc, xor recovered from row/column popcounts */
    DABNN_ENGINE_IMMA = 3,  /* mma.sync m16n8k32 u8 on bits expanded to {0,1} bytes in registers */
    DABNN_ENGINE_TCGEN05 = 4 /* tcgen05.mma kind::i8 (TMEM accumulators) on bits expanded to bytes in shared
                                memory; needs N % 16 == 0 and 16-byte aligned rows, otherwise IMMA is used */
};

typedef void* dabnn_stream_t; /* cudaStream_t */

const char* dabnn_last_error(void);
const char* dabnn_version(void);
/* Number of CUDA devices visible (0 if none / no driver); never fails. */
int dabnn_device_count(void);

/* ---------------------------------------------------------------------------------------------
 * Kernel level.  Device pointers, stream-ordered.
 * ------------------------------------------------------------------------------------------- */

/* reference dabnn/bitpack.h:277 pack_mat (-> :254 pack_mat_64, common/common_bitpack.h:36
 * pack_64_bitfield).  fp32 [n][h][w][c] -> bits [n][h][w][c/64].  Requires c % 64 == 0 and
 * w*c % 64 == 0 (bitpack.h:259,282). */
int dabnn_pack_mat(const float* in, uint64_t* out, int n, int h, int w, int c, dabnn_stream_t s);

/* reference dabnn/bitpack.h:29 pack_64: `size` floats (multiple of 64) -> size/64 words. */
int dabnn_pack_64(const float* in, uint64_t* out, size_t size, dabnn_stream_t s);

/* reference dabnn/pad.h:7 pad on a Bit mat: zero words around the image (a zero word acts as -1
 * in the xnor arithmetic, pad.h:13).  bits [n][h][w][cw] -> [n][h+2ph][w+2pw][cw]. */
int dabnn_pad_bits(const uint64_t* in, uint64_t* out, int n, int h, int w, int cw, int pad_h,
                   int pad_w, dabnn_stream_t s);
/* reference dabnn/pad.h:7 pad on a Float mat with fill value `val`. */
int dabnn_pad_f32(const float* in, float* out, int n, int h, int w, int c, int pad_h, int pad_w,
                  float val, dabnn_stream_t s);

/* reference dabnn/im2col.h:14 im2col.  `elem_bytes` = 4 (float) or 8 (bit words), c = elements per
 * pixel.  in [n][h][w][c] -> col [n][oh*ow][kh*kw*c], zero for out-of-range taps. */
int dabnn_im2col(const void* in, void* col, int elem_bytes, int n, int h, int w, int c, int kh, int kw,
                 int pad_h, int pad_w, int stride_h, int stride_w, int dil_h, int dil_w,
                 dabnn_stream_t s);

/* reference dabnn/fused_binarize_im2col.h:6.  fp32 [n][h][w][c] -> bits
 * [n][oh*ow][ceil(kh*kw*c/128)*2]: taps gathered as floats (0.0f outside), row zero-extended to a
 * multiple of 128 values, sign-packed.  Requires kh*kw*c < 60000 (fused_binarize_im2col.h:15). */
int dabnn_fused_binarize_im2col(const float* in, uint64_t* col, int n, int h, int w, int c, int kh,
                                int kw, int pad_h, int pad_w, int stride_h, int stride_w, int dil_h,
                                int dil_w, dabnn_stream_t s);

/* reference dabnn/bgemm.h:46 bgemm (and :587 bgemm_naive).  Same operand meaning:
 *   A(i,h) = a[h*lda + i], B(h,j) = b[j*ldb + h], C(i,j) = c[j*ldc + i],
 *   C(i,j) += sum_{h<k} popcount(A(i,h) ^ B(h,j)),   i < m, j < n, k in uint64 words.
 * It ACCUMULATES into c like the reference (the caller zeroes c, BinConv.cpp:153). */
int dabnn_bgemm(int m, int n, int k, const uint64_t* a, int lda, const uint64_t* b, int ldb, float* c,
                int ldc, int engine, dabnn_stream_t s);

/* reference common/baseline.h:77 baseline_bconv, and dabnn/bconv.h:855 bconv_3x3 when called with
 * pad 0 on an already padded input.  bits in [n][h][w][cw], weight = cout filters of
 * weight_words/cout words each laid out [kh][kw][cw] (+ optional zero tail), out-of-range tap =
 * zero word.  out fp32 [n][oh][ow][cout] = XOR mismatch counts.  dilation is 1. */
int dabnn_bconv(const uint64_t* in, const uint64_t* weight, size_t weight_words, float* out, int n,
                int h, int w, int cw, int cout, int kh, int kw, int pad_h, int pad_w, int stride_h,
                int stride_w, int engine, dabnn_stream_t s);

/* reference dabnn/layers/BinConv.cpp:144 BinConv::forward_impl: fp32 in [n][h][w][cin] -> fp32
 * mismatch counts [n][oh][ow][cout]; binarisation included.  `weight` is the .dab initializer of
 * the layer (packed by the converter: 9 words per filter for cin == 64, rows padded to 128 bits
 * otherwise).  Needs device scratch of dabnn_binconv_workspace_bytes() bytes (the reference keeps
 * the same intermediates in its "binaized_for_*" / "col_for_*" mats, BinConv.cpp:28-58). */
size_t dabnn_binconv_workspace_bytes(int n, int h, int w, int cin, int kh, int kw, int pad_h, int pad_w,
                                     int stride_h, int stride_w);
int dabnn_binconv_forward(const float* in, const uint64_t* weight, size_t weight_words, float* out,
                          int n, int h, int w, int cin, int cout, int kh, int kw, int pad_h, int pad_w,
                          int stride_h, int stride_w, void* workspace, size_t workspace_bytes,
                          int engine, dabnn_stream_t s);

/* No counterpart in the reference.  dabnn_binconv_forward for callers that can neither pass a
 * workspace nor let the library allocate one: hosts that give all device memory to their own
 * allocator at start-up, or that call from a context where cudaMalloc is off limits (a latency-bound
 * serving loop, another runtime's plugin callback).  The intermediate bit tensor is kept in a fixed
 * array of DABNN_BINCONV_STATIC_BYTES (16 MiB) that is part of the library's device image; every
 * GPU that loads the library holds those 16 MiB until the process exits.  Shapes that need more
 * scratch than that (dabnn_binconv_workspace_bytes) are refused with DABNN_ERR_SHAPE.  The call
 * makes no cudaMalloc / cudaFree and uses no allocating library routine.
 *  - The first call made with a given device current loads the library's device image there (the driver
 *    materialises the 16 MiB array then and may synchronise), looks up the array's device address
 *    (cudaGetSymbolAddress) and caches it: make one warm-up call per device at initialisation, outside any
 *    stream capture; the no-allocation guarantee holds from the second call on.  The cached address does not
 *    survive cudaDeviceReset or a teardown of the device's primary context.
 *  - All calls on a device share the one array.  Nothing in it needs clearing between calls (each
 *    call overwrites what it reads), but two calls whose kernels can overlap on the GPU - different
 *    streams, or different host threads - race on it: serialise them. */
#define DABNN_BINCONV_STATIC_BYTES (16u << 20)
int dabnn_binconv_forward_static(const float* in, const uint64_t* weight, size_t weight_words, float* out,
                                 int n, int h, int w, int cin, int cout, int kh, int kw, int pad_h,
                                 int pad_w, int stride_h, int stride_w, int engine, dabnn_stream_t s);

/* Fused residual block of a binarised network, the sequence the reference runs as four layers
 * (BinConv.cpp:144 -> Affine.cpp:10 -> Add.cpp:7 -> next layer's bitpack.h:277):
 *   cnt = bconv(in_bits, weight);  y = a[c]*cnt + b[c];  if (shortcut) y = y + shortcut;
 *   if (out_f32) store y;  if (out_bits) store sign bits of y.
 * Arithmetic is the unfused sequence's (product rounded, then each sum rounded), so results are
 * bit-identical to calling the pieces one after the other. */
int dabnn_bconv_block(const uint64_t* in_bits, const uint64_t* weight, size_t weight_words,
                      const float* a, const float* b, const float* shortcut, float* out_f32,
                      uint64_t* out_bits, int n, int h, int w, int cw, int cout, int kh, int kw,
                      int pad_h, int pad_w, int stride_h, int stride_w, int engine, dabnn_stream_t s);

/* The same block on activations kept as {0,1} bytes (one byte per channel, NHWC) instead of packed words: the
 * layout in which a convolution tap is a rectangle that the GPU's copy engine loads straight into the tensor
 * cores' operand format.  It replaces the same reference sequence as dabnn_bconv_block, with the reference's
 * pack_mat (bitpack.h:277) becoming dabnn_binarize_u8 (byte = x > 0).  Shapes taken: cin % 64 == 0,
 * cout % 16 == 0, stride 1 or 2 (equal in both directions; even h and w for 2), output rows of at most 128
 * pixels; dabnn_bconv_u8_supported tells.  The weights are the reference's packed filters
 * (cout rows of kh*kw*cin/64 words) expanded once by dabnn_bconv_u8_expand_weights into a buffer of
 * dabnn_bconv_u8_weight_bytes(cout, kh*kw*cin/64) bytes.  Outputs: any of fp32, {0,1} bytes, packed sign bits. */
int dabnn_binarize_u8(const float* in, unsigned char* out, size_t count, dabnn_stream_t s);
int dabnn_bconv_u8_supported(int n, int h, int w, int cin, int cout, int kh, int kw, int pad_h, int pad_w,
                             int stride_h, int stride_w);
size_t dabnn_bconv_u8_weight_bytes(int cout, int kwords);
int dabnn_bconv_u8_expand_weights(const uint64_t* weight, size_t weight_words, int cout, int kwords,
                                  unsigned char* dst, dabnn_stream_t s);
int dabnn_bconv_u8_block(const unsigned char* in_u8, const unsigned char* w_expanded, const float* a, const float* b,
                         const float* shortcut, float* out_f32, unsigned char* out_u8, uint64_t* out_bits, int n,
                         int h, int w, int cin, int cout, int kh, int kw, int pad_h, int pad_w, int stride_h,
                         int stride_w, dabnn_stream_t s);

/* dabnn_bconv_u8_block that also writes the 2x2 stride-2 average pooling of its fp32 result (reference
 * layers/AvePool.cpp:84 ave_pool_fallback on the block's output: the downsample shortcut of the next stage of a
 * ResNet-shaped net), pool_out fp32 [n][oh / 2][ow / 2][cout], bit-identical to dabnn_avepool on out_f32.  Shapes taken:
 * 3x3, stride 1, padding 1, even h and w (dabnn_bconv_u8_block_pooled_supported tells). */
int dabnn_bconv_u8_block_pooled_supported(int n, int h, int w, int cin, int cout, int kh, int kw, int pad_h, int pad_w,
                                          int stride_h, int stride_w);
int dabnn_bconv_u8_block_pooled(const unsigned char* in_u8, const unsigned char* w_expanded, const float* a, const float* b,
                                const float* shortcut, float* out_f32, unsigned char* out_u8, uint64_t* out_bits, float* pool_out,
                                int n, int h, int w, int cin, int cout, int kh, int kw, int pad_h, int pad_w, int stride_h,
                                int stride_w, dabnn_stream_t s);

/* reference dabnn/layers/Affine.cpp:10 affine_inplace: x = a[c]*x + b[c] (in place). */
int dabnn_affine(float* x, const float* a, const float* b, size_t pixels, int c, dabnn_stream_t s);
/* reference dabnn/layers/Add.cpp:7 add_inplace: x += y. */
int dabnn_add(float* x, const float* y, size_t count, dabnn_stream_t s);
/* reference dabnn/layers/Relu.cpp:21: x = max(x, 0). */
int dabnn_relu(float* x, size_t count, dabnn_stream_t s);
/* reference dabnn/layers/PRelu.cpp:6: x < 0 ? x*slope : x; nslope is 1 or c. */
int dabnn_prelu(float* x, const float* slope, int nslope, size_t pixels, int c, dabnn_stream_t s);
/* reference dabnn/layers/MaxPool.cpp:209 max_pool_fallback (-FLT_MAX start, out-of-range skipped). */
int dabnn_maxpool(const float* in, float* out, int n, int h, int w, int c, int kh, int kw, int pad_h,
                  int pad_w, int stride_h, int stride_w, dabnn_stream_t s);
/* reference dabnn/layers/AvePool.cpp:84 ave_pool_fallback (sum of in-range taps / their count). */
int dabnn_avepool(const float* in, float* out, int n, int h, int w, int c, int kh, int kw, int pad_h,
                  int pad_w, int stride_h, int stride_w, dabnn_stream_t s);
/* reference dabnn/layers/Concat.cpp:7: channel concatenation of two float tensors. */
int dabnn_concat(const float* x1, int c1, const float* x2, int c2, float* out, size_t pixels,
                 dabnn_stream_t s);
/* reference dabnn/fconv.h:14,44 fconv (im2col + sgemm, optional per-channel bias); weight
 * [cout][kh][kw][cin].  fp32 accumulation; agrees with the reference to rounding (1e-4 relative). */
int dabnn_fconv(const float* in, const float* weight, const float* bias, float* out, int n, int h,
                int w, int cin, int cout, int kh, int kw, int pad_h, int pad_w, int stride_h,
                int stride_w, int dil_h, int dil_w, dabnn_stream_t s);

/* The stem of a ResNet-shaped network in one kernel, the sequence the reference runs as four layers
 * (dabnn/fconv.h:14 -> layers/Affine.cpp:10 -> layers/Relu.cpp:21 -> layers/MaxPool.cpp:209 with a 3x3 window, stride 2,
 * padding 1):  y = conv(in, weight) (+ bias);  if (a) y = a[c]*y + b[c];  if (relu) y = max(y, 0);  out = maxpool3x3s2p1(y).
 * y itself is never written.  out fp32 [n][ph][pw][cout] with ph = (oh - 1) / 2 + 1; out_u8 (optional) = its signs as
 * {0,1} bytes.  The result is bit-identical to dabnn_fconv + dabnn_affine + dabnn_relu + dabnn_maxpool.  Shapes taken:
 * cin <= 4, horizontal stride 2, no dilation, kw <= 8, output rows of 64 .. 128 pixels, cout % 16 == 0
 * (dabnn_fconv_maxpool_supported tells); anything else returns DABNN_ERR_SHAPE. */
int dabnn_fconv_maxpool_supported(int n, int h, int w, int cin, int cout, int kh, int kw, int pad_h, int pad_w, int stride_h,
                                  int stride_w);
int dabnn_fconv_maxpool(const float* in, const float* weight, const float* bias, const float* a, const float* b, int relu,
                        float* out, unsigned char* out_u8, int n, int h, int w, int cin, int cout, int kh, int kw, int pad_h,
                        int pad_w, int stride_h, int stride_w, dabnn_stream_t s);

/* ---------------------------------------------------------------------------------------------
 * Net level: reference dabnn/net.h:22-66 class bnn::Net.
 * ------------------------------------------------------------------------------------------- */
typedef struct dabnn_net dabnn_net;

/* reference net.h:57 Net::create().  The net lives on the CUDA device current at creation. */
int dabnn_net_create(dabnn_net** out);
void dabnn_net_destroy(dabnn_net* net);
/* reference net.h:59-61 public flags optimize / run_fconv / strict; defaults true/true/true.
 * optimize = 0 selects the CUDA-core popc engine and the layer-by-layer (unfused) plan, like the
 * reference's optimize=false selects its naive kernels.  Must precede read. */
int dabnn_net_set_flags(dabnn_net* net, int optimize, int run_fconv, int strict);
/* Largest batch `run` will be called with (default 1, the reference's only case) and the engine
 * used when optimize != 0.  Must precede read. */
int dabnn_net_configure(dabnn_net* net, int max_batch, int engine);
/* Host inputs reach the device in sub-batches of `images` (default 256) through two staging buffers, the copy
 * of one overlapping the kernels of the one before.  Small sub-batches shorten a single run() (more of the copy
 * is hidden inside it); with pipelined submissions (dabnn_net_submit) the copy of the next submission hides behind
 * the current one anyway, and a sub-batch as large as the batch keeps the kernels at their full-batch
 * efficiency.  Costs 2 * images * H * W * C * 4 bytes of device memory.  Must precede read. */
int dabnn_net_set_host_chunk(dabnn_net* net, int images);
/* reference net.cpp:32 Net::read(path) / net.cpp:46 Net::read_buf(ptr): parse the .dab model,
 * upload the weights and build the execution plan (net.cpp:54 prepare).  Unlike the reference the
 * buffer may be released after the call (weights are copied to the device). */
int dabnn_net_read_file(dabnn_net* net, const char* path);
int dabnn_net_read_buf(dabnn_net* net, const void* buf, size_t len);
/* reference net.cpp:272 Net::run(input): input fp32 NHWC [batch][H][W][C]; in_is_device = 0 for a
 * host pointer (copied to the device inside the call), 1 for a device pointer.  Work is enqueued
 * on the net's stream; dabnn_net_get_blob / dabnn_net_sync make results visible. */
int dabnn_net_run(dabnn_net* net, const float* input, int batch, int in_is_device);
int dabnn_net_sync(dabnn_net* net);
/* reference net.cpp:288 Net::get_blob(name).  dims = {batch, h, w, c}.  With to_host = NULL only
 * dims and *device_ptr are returned; otherwise the blob of the last run is copied to `to_host`
 * (capacity `host_floats`) after synchronising.  In the fused plan (optimize = 1) only blobs that
 * are still materialised exist: network outputs and the outputs of fused groups. */
int dabnn_net_get_blob(dabnn_net* net, const char* name, int dims[4], const float** device_ptr,
                       float* to_host, size_t host_floats);
/* Pipelined serving (no counterpart in the reference, whose run() is synchronous): enqueue run() on a host
 * input (pinned memory for the copies to be asynchronous) followed by the device-to-host copy of blob `blob`
 * into `host_out` (capacity `host_floats`), and return at once with a ticket; dabnn_net_wait(ticket) blocks
 * until that submission's output is in `host_out`.  Submissions execute in order; the host copy of
 * submission k+1 overlaps the kernels of submission k, so keep two or more in flight (at most 8 tickets
 * are live; a ticket is reused by the 8th later submission).  The caller keeps `host_input` and `host_out`
 * untouched until the wait returns. */
int dabnn_net_submit(dabnn_net* net, const float* host_input, int batch, const char* blob, float* host_out,
                     size_t host_floats, int* ticket);
int dabnn_net_wait(dabnn_net* net, int ticket);
/* The packed sign bits that a Binarize layer produced (reference dabnn/layers/Binarize.cpp:9: pack_mat of the
 * input into a Bit mat, bitpack.h:277; the reference's caller casts get_blob()'s Mat to uint64_t*).  `name` is
 * the layer's output; dims = {batch, h, w, c / 64} words.  Same conventions as dabnn_net_get_blob. */
int dabnn_net_get_blob_bits(dabnn_net* net, const char* name, int dims[4], const uint64_t** device_ptr,
                            uint64_t* to_host, size_t host_words);
/* Name of the i-th blob that no layer consumes (network outputs); NULL when i is out of range. */
const char* dabnn_net_output_name(dabnn_net* net, int i);
/* The CUDA stream (cudaStream_t) the net enqueues on. */
dabnn_stream_t dabnn_net_stream(dabnn_net* net);
/* Number of kernels one run() launches and bytes of device memory held by the net. */
int dabnn_net_stats(dabnn_net* net, int* kernels_per_run, size_t* arena_bytes);
/* Per layer-class device time of the last `run` (reference BNN_BENCHMARK, dabnn/layer.cpp:17-31,
 * net.cpp:303 print_time).  Enable before run with dabnn_net_set_profiling(net, 1); fills up to
 * `cap` entries and returns the count through *n. */
int dabnn_net_set_profiling(dabnn_net* net, int on);
int dabnn_net_layer_times(dabnn_net* net, const char** names, float* ms, int cap, int* n);

/* ---------------------------------------------------------------------------------------------
 * Measurement helper: register-resident peak rate (bit-op/s, one op = one xor or one accumulate
 * per bit pair, i.e. 2*m*n*k per MMA) of one contraction instruction on the current device.
 * `engine` as above (POPC / B1 / IMMA / TCGEN05; for TCGEN05 one thread per SM issues 128x128x32
 * kind::i8 instructions on fixed shared-memory operands).  Used as the roofline denominator of the
 * contraction.
 * ------------------------------------------------------------------------------------------- */
int dabnn_measure_engine_peak(int engine, double* bitops_per_second);

/* The same for the float convolution: FLOP/s of tcgen05.mma kind::tf32 (128x128x8 per
 * instruction, one issuing thread per SM).  The float convolution spends three such products per
 * fp32 product (hi*hi + hi*lo + lo*hi), so its fp32-equivalent ceiling is a third of this. */
int dabnn_measure_tf32_peak(double* flops_per_second);

/* Diagnostic for the kernel-level entry points: synchronises the device and returns, through *status, 0 or the
 * code of the first bounded wait that gave up inside a tensor-core kernel and has not been collected yet.  Such
 * a kernel stops issuing work, frees its tensor memory and returns instead of hanging.  Codes: packed-bit
 * contraction 1 producers (a ring stage was never released), 2 epilogue (an accumulator never completed),
 * 3 / 4 MMA thread (accumulator never released / stage never filled); float convolution 11 producers, 12 epilogue, 13 / 14 MMA thread (accumulator /
 * stage), 15 / 16 row loader and its consumers; byte-activation engine 21 loader, 22 / 23 MMA thread
 * (accumulator / stage or resident weights), 24 epilogue.  A Net collects (and clears) the words itself at the
 * end of every run and reports them as DABNN_ERR_TIMEOUT from dabnn_net_wait / _sync / _get_blob. */
int dabnn_engine_status(int* status);

/* Which engine (DABNN_ENGINE_POPC ... DABNN_ENGINE_TCGEN05) the calling thread's most recent dabnn_bgemm /
 * dabnn_bconv / dabnn_bconv_block / dabnn_binconv_forward call actually launched: DABNN_ENGINE_TCGEN05 requests
 * fall back to IMMA for channel counts and alignments the tensor-memory kernel does not take. */
int dabnn_last_engine(void);

/* Tuning hook.  Bits 0..3: 0 keeps 3x3 stride-1 blocks of dabnn_bconv_u8_block on the kernel that loads one box per
 * tap; the default (1) runs them on the kernel that loads a tile's halo once.  Bits 4..6: staging tiles of the halo
 * kernel (0 = the plan's choice), bit 7: whether the latest tensor store may still be reading its tile when the next
 * shortcut is fetched.  Every setting gives identical results. */
int dabnn_debug_set_halo(int mode);

/* Tuning hook: 0 launches every kernel strictly after the one before it; the default (1) lets the hot kernels of a Net
 * begin their set-up while the previous kernel drains (programmatic dependent launch).  Results are identical. */
int dabnn_debug_set_launch_overlap(int on);

/* Test hook: stores `code` in status word `which` (0 packed-bit contraction, 1 float convolution, 2 byte-activation
 * engine) exactly as a kernel whose bounded wait gave up would, so that the reporting path can be exercised
 * without stalling a GPU. */
int dabnn_debug_raise_engine_status(int which, int code);

#ifdef __cplusplus
}
#endif
#endif /* DABNN_B200_H */
