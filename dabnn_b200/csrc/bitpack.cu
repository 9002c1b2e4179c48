// Sign bit-packing and the data-movement kernels around it (pad, im2col, fused binarize-im2col).
// All are HBM-bound: 16-byte loads/stores, grid sized to a multiple of the SM count.
#include "common.cuh"

namespace dabnn {

// Each thread tests one float4 (4 channels); 8 neighbouring lanes OR their nibbles into one
// 32-bit half word, so a warp turns 512 contiguous input bytes into 16 output bytes per step.
__global__ void __launch_bounds__(256) pack_kernel(const float4* __restrict__ in, uint32_t* __restrict__ out,
                                                   size_t n4) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const int lane = threadIdx.x & 31;
    // n4 is a multiple of 16 (64 floats per word), so whole 8-lane groups are in or out together;
    // round the loop bound up to a warp so that the shuffles stay convergent
    const size_t n4_warp = (n4 + 31) / 32 * 32;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4_warp; i += stride) {
        unsigned nib = 0;
        if (i < n4) {
            const float4 v = __ldg(in + i);
            nib = (v.x > 0.f ? 1u : 0u) | (v.y > 0.f ? 2u : 0u) | (v.z > 0.f ? 4u : 0u) | (v.w > 0.f ? 8u : 0u);
        }
        unsigned word = nib << (4 * (lane & 7));
        word |= __shfl_xor_sync(0xffffffffu, word, 1);
        word |= __shfl_xor_sync(0xffffffffu, word, 2);
        word |= __shfl_xor_sync(0xffffffffu, word, 4);
        if ((lane & 7) == 0 && i < n4) out[i >> 3] = word;
    }
}

// Generic "fill a padded / gathered tensor" kernels work on 8-byte units.
__global__ void pad_kernel(const uint64_t* __restrict__ in, uint64_t* __restrict__ out, int n, int h, int w,
                           int c8, int pad_h, int pad_w, uint64_t fill) {
    const int oh = h + 2 * pad_h, ow = w + 2 * pad_w;
    const size_t total = (size_t)n * oh * ow * c8;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int cc = i % c8;
        size_t p = i / c8;
        const int x = p % ow; p /= ow;
        const int y = p % oh;
        const int img = p / oh;
        const int iy = y - pad_h, ix = x - pad_w;
        uint64_t v = fill;
        if (iy >= 0 && iy < h && ix >= 0 && ix < w) v = __ldg(in + (((size_t)img * h + iy) * w + ix) * c8 + cc);
        out[i] = v;
    }
}
__global__ void pad_kernel_f32(const float* __restrict__ in, float* __restrict__ out, int n, int h, int w, int c,
                               int pad_h, int pad_w, float fill) {
    const int oh = h + 2 * pad_h, ow = w + 2 * pad_w;
    const size_t total = (size_t)n * oh * ow * c;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int cc = i % c;
        size_t p = i / c;
        const int x = p % ow; p /= ow;
        const int y = p % oh;
        const int img = p / oh;
        const int iy = y - pad_h, ix = x - pad_w;
        float v = fill;
        if (iy >= 0 && iy < h && ix >= 0 && ix < w) v = __ldg(in + (((size_t)img * h + iy) * w + ix) * c + cc);
        out[i] = v;
    }
}

// im2col on 4-byte units (a float, or half of a bit word): one thread per output unit.
__global__ void im2col_kernel(const uint32_t* __restrict__ in, uint32_t* __restrict__ col, int n, int h, int w,
                              int c4, int kh, int kw, int pad_h, int pad_w, int stride_h, int stride_w,
                              int dil_h, int dil_w, int oh, int ow) {
    const size_t total = (size_t)n * oh * ow * kh * kw * c4;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int cc = i % c4;
        size_t p = i / c4;
        const int kx = p % kw; p /= kw;
        const int ky = p % kh; p /= kh;
        const int ox = p % ow; p /= ow;
        const int oy = p % oh;
        const int img = p / oh;
        const int y = oy * stride_h - pad_h + ky * dil_h, x = ox * stride_w - pad_w + kx * dil_w;
        uint32_t v = 0;
        if (y >= 0 && y < h && x >= 0 && x < w) v = __ldg(in + (((size_t)img * h + y) * w + x) * c4 + cc);
        col[i] = v;
    }
}

// fused binarize-im2col: one warp per 32 output bits.  Output row = ceil(kh*kw*c/128)*2 words;
// value index q of a row maps to tap q / c, channel q % c; beyond kh*kw*c and outside the image
// the gathered float is 0.0f, whose bit is 0.
__global__ void __launch_bounds__(256) fused_binarize_im2col_kernel(
    const float* __restrict__ in, uint32_t* __restrict__ col, int n, int h, int w, int c, int kh, int kw,
    int pad_h, int pad_w, int stride_h, int stride_w, int dil_h, int dil_w, int oh, int ow, int row_u32) {
    const int lane = threadIdx.x & 31;
    const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const size_t nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
    const size_t total = (size_t)n * oh * ow * row_u32;
    const int len = kh * kw * c;
    for (size_t u = warp; u < total; u += nwarps) {
        const int wi = u % row_u32;
        size_t p = u / row_u32;
        const int ox = p % ow; p /= ow;
        const int oy = p % oh;
        const int img = p / oh;
        const int q = wi * 32 + lane;
        float v = 0.f;
        if (q < len) {
            const int tap = q / c, ch = q - tap * c;
            const int ky = tap / kw, kx = tap - ky * kw;
            const int y = oy * stride_h - pad_h + ky * dil_h, x = ox * stride_w - pad_w + kx * dil_w;
            if (y >= 0 && y < h && x >= 0 && x < w) v = __ldg(in + (((size_t)img * h + y) * w + x) * c + ch);
        }
        const unsigned word = __ballot_sync(0xffffffffu, v > 0.f);
        if (lane == 0) col[u] = word;
    }
}

// The same for c % 4 == 0 and 16-byte aligned input: a thread tests one float4 (four channels of one tap), eight
// lanes OR their nibbles into one 32-bit word by shuffles; all index arithmetic in 32 bits.
__global__ void __launch_bounds__(256) fused_binarize_im2col_vec4_kernel(
    const float* __restrict__ in, uint32_t* __restrict__ col, int n, int h, int w, int c, int kh, int kw,
    int pad_h, int pad_w, int stride_h, int stride_w, int dil_h, int dil_w, int oh, int ow, int row_u32) {
    const uint32_t per_row = (uint32_t)row_u32 * 8u;              // nibbles per output row
    const uint32_t total = (uint32_t)n * oh * ow * per_row;       // a multiple of 32
    const int len = kh * kw * c;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const uint32_t ni = i % per_row;
        uint32_t p = i / per_row;
        const int ox = (int)(p % (uint32_t)ow); p /= (uint32_t)ow;
        const int oy = (int)(p % (uint32_t)oh);
        const int img = (int)(p / (uint32_t)oh);
        const int q = (int)ni * 4;
        unsigned nib = 0;
        if (q < len) {
            const int tap = q / c, ch = q - tap * c;
            const int ky = tap / kw, kx = tap - ky * kw;
            const int y = oy * stride_h - pad_h + ky * dil_h, x = ox * stride_w - pad_w + kx * dil_w;
            if (y >= 0 && y < h && x >= 0 && x < w) {
                const float4 v = __ldg(reinterpret_cast<const float4*>(in + (((size_t)img * h + y) * w + x) * c + ch));
                nib = (v.x > 0.f ? 1u : 0u) | (v.y > 0.f ? 2u : 0u) | (v.z > 0.f ? 4u : 0u) | (v.w > 0.f ? 8u : 0u);
            }
        }
        unsigned word = nib << (4 * (threadIdx.x & 7));
        word |= __shfl_xor_sync(0xffffffffu, word, 1);
        word |= __shfl_xor_sync(0xffffffffu, word, 2);
        word |= __shfl_xor_sync(0xffffffffu, word, 4);
        if ((threadIdx.x & 7) == 0) col[i >> 3] = word;
    }
}

static int grid_for(size_t work_items, int threads) {
    const size_t blocks = (work_items + threads - 1) / threads;
    const size_t cap = (size_t)sm_count() * 16;
    return (int)(blocks < cap ? (blocks ? blocks : 1) : cap);
}

}  // namespace dabnn

using namespace dabnn;

extern "C" int dabnn_pack_64(const float* in, uint64_t* out, size_t size, dabnn_stream_t s) {
    DABNN_REQUIRE(size % 64 == 0, DABNN_ERR_SHAPE, "size % 64 == 0 is not satisfied!");  // bitpack.h:30
    if (size == 0) return DABNN_OK;
    DABNN_REQUIRE(in && out, DABNN_ERR_ARG, "pack: null pointer");
    DABNN_REQUIRE((reinterpret_cast<uintptr_t>(in) & 15) == 0, DABNN_ERR_ARG, "pack: input must be 16-byte aligned");
    const size_t n4 = size / 4;
    pack_kernel<<<grid_for(n4, 256 * 4), 256, 0, static_cast<cudaStream_t>(s)>>>(
        reinterpret_cast<const float4*>(in), reinterpret_cast<uint32_t*>(out), n4);
    return check_launch("pack_kernel");
}

extern "C" int dabnn_pack_mat(const float* in, uint64_t* out, int n, int h, int w, int c, dabnn_stream_t s) {
    DABNN_REQUIRE(n >= 0 && h >= 0 && w >= 0 && c >= 0, DABNN_ERR_ARG, "pack_mat: negative dimension");
    DABNN_REQUIRE(c % 64 == 0, DABNN_ERR_SHAPE, "float_mat.c % 64 == 0 is not satisfied!");  // bitpack.h:282
    DABNN_REQUIRE((size_t)n * h == 0 || ((long long)w * c > 0 && ((long long)w * c) % 64 == 0), DABNN_ERR_SHAPE,
                  "float_mat.w * float_mat.c > 0 && float_mat.w * float_mat.c % 64 == 0 is not satisfied!");
    return dabnn_pack_64(in, out, (size_t)n * h * w * c, s);
}

extern "C" int dabnn_pad_bits(const uint64_t* in, uint64_t* out, int n, int h, int w, int cw, int pad_h,
                              int pad_w, dabnn_stream_t s) {
    DABNN_REQUIRE(in && out, DABNN_ERR_ARG, "pad: null pointer");
    DABNN_REQUIRE(n > 0 && h > 0 && w > 0 && cw > 0 && pad_h >= 0 && pad_w >= 0, DABNN_ERR_ARG, "pad: bad dims");
    const size_t total = (size_t)n * (h + 2 * pad_h) * (w + 2 * pad_w) * cw;
    pad_kernel<<<grid_for(total, 256), 256, 0, static_cast<cudaStream_t>(s)>>>(in, out, n, h, w, cw, pad_h, pad_w, 0ull);
    return check_launch("pad_kernel");
}

extern "C" int dabnn_pad_f32(const float* in, float* out, int n, int h, int w, int c, int pad_h, int pad_w,
                             float val, dabnn_stream_t s) {
    DABNN_REQUIRE(in && out, DABNN_ERR_ARG, "pad: null pointer");
    DABNN_REQUIRE(n > 0 && h > 0 && w > 0 && c > 0 && pad_h >= 0 && pad_w >= 0, DABNN_ERR_ARG, "pad: bad dims");
    const size_t total = (size_t)n * (h + 2 * pad_h) * (w + 2 * pad_w) * c;
    pad_kernel_f32<<<grid_for(total, 256), 256, 0, static_cast<cudaStream_t>(s)>>>(in, out, n, h, w, c, pad_h, pad_w, val);
    return check_launch("pad_kernel_f32");
}

extern "C" int dabnn_im2col(const void* in, void* col, int elem_bytes, int n, int h, int w, int c, int kh,
                            int kw, int pad_h, int pad_w, int stride_h, int stride_w, int dil_h, int dil_w,
                            dabnn_stream_t s) {
    DABNN_REQUIRE(in && col, DABNN_ERR_ARG, "im2col: null pointer");
    DABNN_REQUIRE(elem_bytes == 4 || elem_bytes == 8, DABNN_ERR_ARG, "im2col: elem_bytes must be 4 or 8");
    DABNN_REQUIRE(n > 0 && h > 0 && w > 0 && c > 0 && kh > 0 && kw > 0 && stride_h > 0 && stride_w > 0 &&
                      dil_h > 0 && dil_w > 0 && pad_h >= 0 && pad_w >= 0, DABNN_ERR_ARG, "im2col: bad dims");
    const int oh = conv_out_dim(h, pad_h, dil_h, kh, stride_h), ow = conv_out_dim(w, pad_w, dil_w, kw, stride_w);
    DABNN_REQUIRE(oh > 0 && ow > 0, DABNN_ERR_SHAPE, "im2col: empty output");
    const int c4 = c * (elem_bytes / 4);
    const size_t total = (size_t)n * oh * ow * kh * kw * c4;
    im2col_kernel<<<grid_for(total, 256), 256, 0, static_cast<cudaStream_t>(s)>>>(
        static_cast<const uint32_t*>(in), static_cast<uint32_t*>(col), n, h, w, c4, kh, kw, pad_h, pad_w, stride_h,
        stride_w, dil_h, dil_w, oh, ow);
    return check_launch("im2col_kernel");
}

extern "C" int dabnn_fused_binarize_im2col(const float* in, uint64_t* col, int n, int h, int w, int c, int kh,
                                           int kw, int pad_h, int pad_w, int stride_h, int stride_w, int dil_h,
                                           int dil_w, dabnn_stream_t s) {
    DABNN_REQUIRE(in && col, DABNN_ERR_ARG, "fused_binarize_im2col: null pointer");
    DABNN_REQUIRE(n > 0 && h > 0 && w > 0 && c > 0 && kh > 0 && kw > 0 && stride_h > 0 && stride_w > 0 &&
                      dil_h > 0 && dil_w > 0 && pad_h >= 0 && pad_w >= 0, DABNN_ERR_ARG,
                  "fused_binarize_im2col: bad dims");
    DABNN_REQUIRE((long long)kh * kw * c < 60000, DABNN_ERR_SHAPE,
                  "kernel_h * kernel_w * im.c must be smaller than 60000");  // fused_binarize_im2col.h:15
    const int oh = conv_out_dim(h, pad_h, dil_h, kh, stride_h), ow = conv_out_dim(w, pad_w, dil_w, kw, stride_w);
    DABNN_REQUIRE(oh > 0 && ow > 0, DABNN_ERR_SHAPE, "fused_binarize_im2col: empty output");
    const int row_u32 = (kh * kw * c + 127) / 128 * 4;
    const size_t total = (size_t)n * oh * ow * row_u32;
    if (c % 4 == 0 && (reinterpret_cast<uintptr_t>(in) & 15) == 0 && total * 8 + (size_t)sm_count() * 16 * 256 < (1ull << 32)) {
        fused_binarize_im2col_vec4_kernel<<<grid_for(total * 8, 256), 256, 0, static_cast<cudaStream_t>(s)>>>(
            in, reinterpret_cast<uint32_t*>(col), n, h, w, c, kh, kw, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w,
            oh, ow, row_u32);
        return check_launch("fused_binarize_im2col_vec4_kernel");
    }
    fused_binarize_im2col_kernel<<<grid_for(total * 32, 256), 256, 0, static_cast<cudaStream_t>(s)>>>(
        in, reinterpret_cast<uint32_t*>(col), n, h, w, c, kh, kw, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w,
        oh, ow, row_u32);
    return check_launch("fused_binarize_im2col_kernel");
}
