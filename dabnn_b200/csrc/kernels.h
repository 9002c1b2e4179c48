// Internal (C++) declarations shared between the .cu files and the Net runtime.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

struct CUtensorMap_st;

namespace dabnn {

// TMA descriptor of an fp32 tensor for tiled copies of `box` elements per dimension (innermost first) in the
// 128-byte-swizzled shared-memory layout (inner box = 32 floats).  dims[rank], strides_bytes[rank - 1] (the
// innermost stride is one element).  The encoder is a driver entry point fetched once through the runtime - the
// library links no driver stub.  Returns false when the descriptor cannot be made.
bool make_f32_tensor_map(CUtensorMap_st* map, float* base, int rank, const unsigned long long* dims,
                         const unsigned long long* strides_bytes, const unsigned* box);

// The same for a tensor of bytes, up to five dimensions, inner box 64 or 128 bytes, swizzled over that width (the
// layout a K-major SWIZZLE_64B / SWIZZLE_128B shared-memory descriptor of tcgen05.mma reads); elements outside the
// tensor read as zero.
bool make_u8_tensor_map(CUtensorMap_st* map, const unsigned char* base, int rank, const unsigned long long* dims,
                        const unsigned long long* strides_bytes, const unsigned* box);

// Weights of a binary convolution expanded once to the TCGEN05 engine's stage layout (bytes {0,1}, 8x the packed
// size): size of the buffer, and the kernel that fills it.  bconv_block_impl takes the buffer as w_expanded.
size_t bconv_expanded_weight_bytes(int cout, int kwords);
int bconv_expand_weights(const uint64_t* weight, size_t weight_words, int cout, int kwords, unsigned char* dst,
                         cudaStream_t stream);
// bconv + optional affine + optional shortcut + optional sign-bit output (see dabnn_bconv_block).
int bconv_block_impl(const uint64_t* in_bits, const uint64_t* weight, size_t weight_words, const float* a,
                     const float* b, const float* shortcut, float* out_f32, uint64_t* out_bits, int n, int h,
                     int w, int cw, int cout, int kh, int kw, int pad_h, int pad_w, int stride_h,
                     int stride_w, int engine, cudaStream_t stream, const unsigned char* w_expanded = nullptr);

// Byte-activation engine (bconv_u8.cuh): activations as {0,1} bytes in NHWC, fed to the tensor cores by TMA.
// bconv_u8_supported: whether the shape is taken (and its tensor maps can be encoded on this driver).
bool bconv_u8_supported(int n, int h, int w, int cin, int cout, int kh, int kw, int pad_h, int pad_w, int stride_h, int stride_w);
size_t bconv_u8_weight_bytes(int cout, int nboxes);
int bconv_u8_expand_weights(const uint64_t* weight, size_t weight_words, int cout, int nboxes, unsigned char* dst,
                            cudaStream_t stream);
int binarize_u8_impl(const float* in, unsigned char* out, size_t count, cudaStream_t stream);
// pool_out (optional): the 2x2 stride-2 average pooling of the fp32 result, fp32 [n][oh / 2][ow / 2][cout], written by the
// same kernel; bconv_u8_pool_supported tells for which shapes (3x3, stride 1, padding 1, even height and width).
bool bconv_u8_pool_supported(int n, int h, int w, int cin, int cout, int kh, int kw, int pad_h, int pad_w, int stride_h, int stride_w);
int bconv_u8_block_impl(const unsigned char* in_u8, const unsigned char* w_img, const float* a, const float* b,
                        const float* shortcut, float* out_f32, unsigned char* out_u8, uint64_t* out_bits, int n, int h, int w,
                        int cin, int cout, int kh, int kw, int pad_h, int pad_w, int stride_h, int stride_w,
                        cudaStream_t stream, float* pool_out = nullptr);
int bconv_u8_status(int* status);

// Device addresses (on the current device) of the words in which the tensor-core kernels record the code of a
// bounded wait that gave up: the packed-bit contraction, the float convolution, the byte-activation engine.
int contraction_status_word(int** addr);
int fconv_status_word(int** addr);
int bconv_u8_status_word(int** addr);

// Elementwise chain on an fp32 NHWC tensor, in one pass:  v = x;  if (a) v = a[c]*v + b[c];
// if (add) v += add;  if (relu) v = max(v, 0);  optional fp32 store and optional sign-bit store.
int elementwise_chain(const float* x, const float* a, const float* b, const float* add, int relu,
                      float* out_f32, uint64_t* out_bits, size_t pixels, int c, cudaStream_t stream);

// Float convolution with an optional fused per-channel affine and relu applied to the result
// (conv (+bias) -> a*v+b -> max(v,0)); used for the stem and the downsample shortcuts.
int fconv_tc5_status(int* status);
int fconv_impl(const float* in, const float* weight, const float* bias, const float* a, const float* b,
               int relu, float* out, int n, int h, int w, int cin, int cout, int kh, int kw, int pad_h,
               int pad_w, int stride_h, int stride_w, int dil_h, int dil_w, cudaStream_t stream, const float* weight_rem = nullptr);
// weight_rem (optional, 16-byte aligned): the remainders w - trunc_tf32(w) of constant weights, computed once by
// fconv_split_weights; the 1x1 GEMM kernel then loads them by TMA instead of recomputing them for every tile.
// fconv_uses_weight_remainders tells for which convolutions they are read.
int fconv_split_weights(const float* weight, float* rem, size_t count, cudaStream_t stream);
bool fconv_uses_weight_remainders(int cin, int cout, int kh, int kw, int pad_h, int pad_w, int stride_h, int stride_w);

// The same followed by a 3x3 stride-2 pad-1 max pooling, in one kernel, for the shapes fconv_pool_supported accepts (thin
// inputs with horizontal stride 2: a ResNet stem); the convolution's own output is never written.
bool fconv_pool_supported(int n, int h, int w, int cin, int cout, int kh, int kw, int pad_h, int pad_w, int stride_h, int stride_w);
int fconv_pool_impl(const float* in, const float* weight, const float* bias, const float* a, const float* b, int relu, float* pool_out,
                    unsigned char* pool_u8, int n, int h, int w, int cin, int cout, int kh, int kw, int pad_h, int pad_w, int stride_h,
                    int stride_w, cudaStream_t stream);

// Max pooling that also emits the signs of its output (the first binary conv's input), packed and / or as bytes.
int maxpool_impl(const float* in, float* out, uint64_t* out_bits, int n, int h, int w, int c, int kh, int kw,
                 int pad_h, int pad_w, int stride_h, int stride_w, cudaStream_t stream, unsigned char* out_u8 = nullptr);

}  // namespace dabnn
