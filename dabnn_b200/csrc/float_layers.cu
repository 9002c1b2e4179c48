// The bandwidth-bound float layers (Affine, Add, Relu, PRelu, pooling, Concat) and the float
// convolution.  Elementwise kernels move 16 bytes per thread and follow the reference's operation
// order exactly (product and sum rounded separately, no FMA contraction) so that results - and the
// sign bits derived from them - are bit-identical to the reference's x86 build.
#include <cfloat>

#include "common.cuh"
#include "kernels.h"

namespace dabnn {

static int grid_for(size_t work_items, int threads) {
    const size_t blocks = (work_items + threads - 1) / threads;
    const size_t cap = (size_t)sm_count() * 16;
    return (int)(blocks < cap ? (blocks ? blocks : 1) : cap);
}

__device__ __forceinline__ float relu_ref(float v) { return v < 0.f ? 0.f : v; }  // std::max(v, 0.f)

// 16 consecutive lanes hold 4 channels each = one 64-channel word of one pixel.
__device__ __forceinline__ void store_sign_word(uint64_t* bits, size_t word_index, unsigned nib, bool valid) {
    const int sub = threadIdx.x & 15;
    unsigned lo = sub < 8 ? nib << (4 * sub) : 0u, hi = sub >= 8 ? nib << (4 * (sub - 8)) : 0u;
#pragma unroll
    for (int off = 1; off < 16; off <<= 1) {
        lo |= __shfl_xor_sync(0xffffffffu, lo, off);
        hi |= __shfl_xor_sync(0xffffffffu, hi, off);
    }
    if (sub == 0 && valid) bits[word_index] = ((unsigned long long)hi << 32) | lo;
}

// ---- elementwise chain ---------------------------------------------------------------------------
// VEC = 4: c % 4 == 0 and 16-byte aligned pointers; VEC = 1: anything.
template <int VEC>
__global__ void __launch_bounds__(256) chain_kernel(const float* x, const float* __restrict__ a,
                                                    const float* __restrict__ b, const float* __restrict__ add,
                                                    int relu, const float* __restrict__ slope, int nslope,
                                                    float* out, uint64_t* __restrict__ bits,
                                                    size_t total_vec, int c_vec) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const size_t bound = bits ? (total_vec + 31) / 32 * 32 : total_vec;  // keep warps whole for the shuffles
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < bound; i += stride) {
        const bool valid = i < total_vec;
        float v[VEC];
        unsigned nib = 0;
        if (valid) {
            const int ch = (int)(i % c_vec) * VEC;
            if (VEC == 4) {
                const float4 t = *reinterpret_cast<const float4*>(x + i * 4);
                v[0] = t.x; v[1 % VEC] = t.y; v[2 % VEC] = t.z; v[3 % VEC] = t.w;
            } else {
                v[0] = x[i];
            }
            if (a) {
#pragma unroll
                for (int q = 0; q < VEC; q++) v[q] = __fadd_rn(__fmul_rn(__ldg(a + ch + q), v[q]), __ldg(b + ch + q));
            }
            if (add) {
                float t[VEC];
                if (VEC == 4) {
                    const float4 f = __ldg(reinterpret_cast<const float4*>(add + i * 4));
                    t[0] = f.x; t[1 % VEC] = f.y; t[2 % VEC] = f.z; t[3 % VEC] = f.w;
                } else {
                    t[0] = __ldg(add + i);
                }
#pragma unroll
                for (int q = 0; q < VEC; q++) v[q] = __fadd_rn(v[q], t[q]);
            }
            if (relu) {
#pragma unroll
                for (int q = 0; q < VEC; q++) v[q] = relu_ref(v[q]);
            }
            if (slope) {
#pragma unroll
                for (int q = 0; q < VEC; q++)
                    if (v[q] < 0.f) v[q] = __fmul_rn(v[q], __ldg(slope + (nslope == 1 ? 0 : ch + q)));
            }
            if (out) {
                if (VEC == 4)
                    *reinterpret_cast<float4*>(out + i * 4) = make_float4(v[0], v[1 % VEC], v[2 % VEC], v[3 % VEC]);
                else
                    out[i] = v[0];
            }
#pragma unroll
            for (int q = 0; q < VEC; q++) nib |= (v[q] > 0.f ? 1u : 0u) << q;
        }
        if (bits) store_sign_word(bits, i >> 4, nib, valid);  // VEC == 4 and c % 64 == 0 guaranteed by the host
    }
}

static int launch_chain(const float* x, const float* a, const float* b, const float* add, int relu,
                        const float* slope, int nslope, float* out, uint64_t* bits, size_t pixels, int c,
                        cudaStream_t stream) {
    if (pixels == 0 || c == 0) return DABNN_OK;
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const bool vec = c % 4 == 0 && al16(x) && al16(add) && al16(out);
    DABNN_REQUIRE(!bits || (vec && c % 64 == 0), DABNN_ERR_SHAPE, "sign-bit output needs c % 64 == 0");
    const size_t total = pixels * (size_t)c;
    if (vec) {
        chain_kernel<4><<<grid_for(total / 4, 256 * 2), 256, 0, stream>>>(x, a, b, add, relu, slope, nslope, out,
                                                                         bits, total / 4, c / 4);
    } else {
        chain_kernel<1><<<grid_for(total, 256 * 4), 256, 0, stream>>>(x, a, b, add, relu, slope, nslope, out,
                                                                       nullptr, total, c);
    }
    return check_launch("chain_kernel");
}

int elementwise_chain(const float* x, const float* a, const float* b, const float* add, int relu,
                      float* out_f32, uint64_t* out_bits, size_t pixels, int c, cudaStream_t stream) {
    return launch_chain(x, a, b, add, relu, nullptr, 0, out_f32, out_bits, pixels, c, stream);
}

// ---- pooling -------------------------------------------------------------------------------------
template <int VEC, bool IS_MAX>
__global__ void __launch_bounds__(256) pool_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                   uint64_t* __restrict__ bits, int n, int h, int w, int c_vec,
                                                   int kh, int kw, int pad_h, int pad_w, int stride_h,
                                                   int stride_w, int oh, int ow) {
    const size_t total = (size_t)n * oh * ow * c_vec;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const size_t bound = bits ? (total + 31) / 32 * 32 : total;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < bound; i += stride) {
        const bool valid = i < total;
        unsigned nib = 0;
        if (valid) {
            const int cc = i % c_vec;
            size_t p = i / c_vec;
            const int ox = p % ow; p /= ow;
            const int oy = p % oh;
            const int img = p / oh;
            float acc[VEC];
#pragma unroll
            for (int q = 0; q < VEC; q++) acc[q] = IS_MAX ? -FLT_MAX : 0.f;
            int cnt = 0;
            for (int ky = 0; ky < kh; ky++) {
                const int y = oy * stride_h - pad_h + ky;
                if (y < 0 || y >= h) continue;
                for (int kx = 0; kx < kw; kx++) {
                    const int x = ox * stride_w - pad_w + kx;
                    if (x < 0 || x >= w) continue;
                    const float* src = in + ((((size_t)img * h + y) * w + x) * c_vec + cc) * VEC;
                    float t[VEC];
                    if (VEC == 4) {
                        const float4 f = __ldg(reinterpret_cast<const float4*>(src));
                        t[0] = f.x; t[1 % VEC] = f.y; t[2 % VEC] = f.z; t[3 % VEC] = f.w;
                    } else {
                        t[0] = __ldg(src);
                    }
#pragma unroll
                    for (int q = 0; q < VEC; q++) acc[q] = IS_MAX ? (acc[q] < t[q] ? t[q] : acc[q]) : __fadd_rn(acc[q], t[q]);
                    cnt++;
                }
            }
            if (!IS_MAX) {
#pragma unroll
                for (int q = 0; q < VEC; q++) acc[q] = __fdiv_rn(acc[q], (float)cnt);
            }
            if (VEC == 4)
                *reinterpret_cast<float4*>(out + i * 4) = make_float4(acc[0], acc[1 % VEC], acc[2 % VEC], acc[3 % VEC]);
            else
                out[i] = acc[0];
#pragma unroll
            for (int q = 0; q < VEC; q++) nib |= (acc[q] > 0.f ? 1u : 0u) << q;
        }
        if (bits) store_sign_word(bits, i >> 4, nib, valid);
    }
}

template <bool IS_MAX>
static int launch_pool(const float* in, float* out, uint64_t* bits, int n, int h, int w, int c, int kh, int kw,
                       int pad_h, int pad_w, int stride_h, int stride_w, cudaStream_t stream) {
    DABNN_REQUIRE(in && out, DABNN_ERR_ARG, "pool: null pointer");
    DABNN_REQUIRE(n > 0 && h > 0 && w > 0 && c > 0 && kh > 0 && kw > 0 && stride_h > 0 && stride_w > 0 &&
                      pad_h >= 0 && pad_w >= 0, DABNN_ERR_ARG, "pool: bad dims");
    const int oh = (h + 2 * pad_h - kh) / stride_h + 1, ow = (w + 2 * pad_w - kw) / stride_w + 1;
    DABNN_REQUIRE(oh > 0 && ow > 0, DABNN_ERR_SHAPE, "pool: empty output");
    DABNN_REQUIRE(pad_h < kh && pad_w < kw, DABNN_ERR_SHAPE, "pool: padding must be smaller than the kernel");
    const bool vec = c % 4 == 0 && (reinterpret_cast<uintptr_t>(in) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
    DABNN_REQUIRE(!bits || (vec && c % 64 == 0), DABNN_ERR_SHAPE, "sign-bit output needs c % 64 == 0");
    if (vec) {
        const size_t total = (size_t)n * oh * ow * (c / 4);
        pool_kernel<4, IS_MAX><<<grid_for(total, 256), 256, 0, stream>>>(in, out, bits, n, h, w, c / 4, kh, kw, pad_h,
                                                                         pad_w, stride_h, stride_w, oh, ow);
    } else {
        const size_t total = (size_t)n * oh * ow * c;
        pool_kernel<1, IS_MAX><<<grid_for(total, 256), 256, 0, stream>>>(in, out, nullptr, n, h, w, c, kh, kw, pad_h,
                                                                         pad_w, stride_h, stride_w, oh, ow);
    }
    return check_launch("pool_kernel");
}

int maxpool_impl(const float* in, float* out, uint64_t* out_bits, int n, int h, int w, int c, int kh, int kw,
                 int pad_h, int pad_w, int stride_h, int stride_w, cudaStream_t stream) {
    return launch_pool<true>(in, out, out_bits, n, h, w, c, kh, kw, pad_h, pad_w, stride_h, stride_w, stream);
}

// ---- concat --------------------------------------------------------------------------------------
__global__ void concat_kernel(const float* __restrict__ x1, int c1, const float* __restrict__ x2, int c2,
                              float* __restrict__ out, size_t pixels) {
    const int c = c1 + c2;
    const size_t total = pixels * c;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t p = i / c;
        const int ch = i % c;
        out[i] = ch < c1 ? __ldg(x1 + p * c1 + ch) : __ldg(x2 + p * c2 + (ch - c1));
    }
}

// ---- float convolution -----------------------------------------------------------------------------
// Implicit-GEMM on CUDA cores in fp32: C[pixel][cout] = sum_k A[pixel][k] * W[cout][k],
// k = (ky*kw + kx)*cin + ci.  64x64 tile per CTA, 16-deep K slices in shared memory, 4x4 outputs
// per thread.  The epilogue adds the bias and can apply a per-channel affine and a relu.
constexpr int FT = 64, FK = 16;
__global__ void __launch_bounds__(256) fconv_kernel(const float* __restrict__ in, const float* __restrict__ wgt,
                                                    const float* __restrict__ bias, const float* __restrict__ a,
                                                    const float* __restrict__ b, int relu, float* __restrict__ out,
                                                    int n, int h, int w, int cin, int cout, int kh, int kw, int pad_h,
                                                    int pad_w, int stride_h, int stride_w, int dil_h, int dil_w, int oh,
                                                    int ow) {
    __shared__ float As[FK][FT + 4];
    __shared__ float Bs[FK][FT + 4];
    const int K = kh * kw * cin, M = n * oh * ow;
    const int m0 = blockIdx.x * FT, n0 = blockIdx.y * FT;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    // loader: thread -> (tile row = tid / 4, k offsets (tid % 4) * 4 .. +3)
    const int lr = tid >> 2, lk = (tid & 3) * 4;
    const int pm = m0 + lr;
    int img = 0, iy0 = 0, ix0 = 0;
    const bool prow = pm < M;
    if (prow) {
        img = pm / (oh * ow);
        const int rem = pm - img * (oh * ow);
        const int oy = rem / ow, ox = rem - oy * ow;
        iy0 = oy * stride_h - pad_h;
        ix0 = ox * stride_w - pad_w;
    }
    const int wn = n0 + lr;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += FK) {
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const int k = k0 + lk + q;
            float av = 0.f, bv = 0.f;
            if (k < K) {
                if (prow) {
                    const int tap = k / cin, ci = k - tap * cin;
                    const int ky = tap / kw, kx = tap - ky * kw;
                    const int y = iy0 + ky * dil_h, x = ix0 + kx * dil_w;
                    if (y >= 0 && y < h && x >= 0 && x < w) av = __ldg(in + (((size_t)img * h + y) * w + x) * cin + ci);
                }
                if (wn < cout) bv = __ldg(wgt + (size_t)wn * K + k);
            }
            As[lk + q][lr] = av;
            Bs[lk + q][lr] = bv;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < FK; kk++) {
            const float4 av = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
            const float4 bv = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
            const float ar[4] = {av.x, av.y, av.z, av.w}, br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int row = m0 + ty * 4 + i;
        if (row >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int col = n0 + tx * 4 + j;
            if (col >= cout) continue;
            float v = acc[i][j];
            if (bias) v = __fadd_rn(v, __ldg(bias + col));
            if (a) v = __fadd_rn(__fmul_rn(__ldg(a + col), v), __ldg(b + col));
            if (relu) v = relu_ref(v);
            out[(size_t)row * cout + col] = v;
        }
    }
}

int fconv_impl(const float* in, const float* weight, const float* bias, const float* a, const float* b, int relu,
               float* out, int n, int h, int w, int cin, int cout, int kh, int kw, int pad_h, int pad_w,
               int stride_h, int stride_w, int dil_h, int dil_w, cudaStream_t stream) {
    DABNN_REQUIRE(in && weight && out, DABNN_ERR_ARG, "fconv: null pointer");
    DABNN_REQUIRE(n > 0 && h > 0 && w > 0 && cin > 0 && cout > 0 && kh > 0 && kw > 0 && stride_h > 0 &&
                      stride_w > 0 && dil_h > 0 && dil_w > 0 && pad_h >= 0 && pad_w >= 0, DABNN_ERR_ARG,
                  "fconv: bad dims");
    DABNN_REQUIRE((a == nullptr) == (b == nullptr), DABNN_ERR_ARG, "fconv: a and b go together");
    const int oh = conv_out_dim(h, pad_h, dil_h, kh, stride_h), ow = conv_out_dim(w, pad_w, dil_w, kw, stride_w);
    DABNN_REQUIRE(oh > 0 && ow > 0, DABNN_ERR_SHAPE, "fconv: empty output");
    DABNN_REQUIRE((long long)n * oh * ow < (1ll << 31), DABNN_ERR_SHAPE, "fconv: too many output pixels");
    dim3 grid((n * oh * ow + FT - 1) / FT, (cout + FT - 1) / FT);
    fconv_kernel<<<grid, 256, 0, stream>>>(in, weight, bias, a, b, relu, out, n, h, w, cin, cout, kh, kw, pad_h,
                                           pad_w, stride_h, stride_w, dil_h, dil_w, oh, ow);
    return check_launch("fconv_kernel");
}

}  // namespace dabnn

using namespace dabnn;

extern "C" int dabnn_affine(float* x, const float* a, const float* b, size_t pixels, int c, dabnn_stream_t s) {
    DABNN_REQUIRE(x && a && b, DABNN_ERR_ARG, "affine: null pointer");
    return launch_chain(x, a, b, nullptr, 0, nullptr, 0, x, nullptr, pixels, c, static_cast<cudaStream_t>(s));
}
extern "C" int dabnn_add(float* x, const float* y, size_t count, dabnn_stream_t s) {
    DABNN_REQUIRE(x && y, DABNN_ERR_ARG, "add: null pointer");
    const int c = count % 4 == 0 ? 4 : 1;
    return launch_chain(x, nullptr, nullptr, y, 0, nullptr, 0, x, nullptr, count / c, c, static_cast<cudaStream_t>(s));
}
extern "C" int dabnn_relu(float* x, size_t count, dabnn_stream_t s) {
    DABNN_REQUIRE(x, DABNN_ERR_ARG, "relu: null pointer");
    const int c = count % 4 == 0 ? 4 : 1;
    return launch_chain(x, nullptr, nullptr, nullptr, 1, nullptr, 0, x, nullptr, count / c, c, static_cast<cudaStream_t>(s));
}
extern "C" int dabnn_prelu(float* x, const float* slope, int nslope, size_t pixels, int c, dabnn_stream_t s) {
    DABNN_REQUIRE(x && slope, DABNN_ERR_ARG, "prelu: null pointer");
    DABNN_REQUIRE(nslope == 1 || nslope == c, DABNN_ERR_SHAPE, "slope must have size 1 or input.channels");  // PRelu.cpp:7-9
    return launch_chain(x, nullptr, nullptr, nullptr, 0, slope, nslope, x, nullptr, pixels, c, static_cast<cudaStream_t>(s));
}
extern "C" int dabnn_maxpool(const float* in, float* out, int n, int h, int w, int c, int kh, int kw, int pad_h,
                             int pad_w, int stride_h, int stride_w, dabnn_stream_t s) {
    return launch_pool<true>(in, out, nullptr, n, h, w, c, kh, kw, pad_h, pad_w, stride_h, stride_w,
                             static_cast<cudaStream_t>(s));
}
extern "C" int dabnn_avepool(const float* in, float* out, int n, int h, int w, int c, int kh, int kw, int pad_h,
                             int pad_w, int stride_h, int stride_w, dabnn_stream_t s) {
    return launch_pool<false>(in, out, nullptr, n, h, w, c, kh, kw, pad_h, pad_w, stride_h, stride_w,
                              static_cast<cudaStream_t>(s));
}
extern "C" int dabnn_concat(const float* x1, int c1, const float* x2, int c2, float* out, size_t pixels,
                            dabnn_stream_t s) {
    DABNN_REQUIRE(x1 && x2 && out, DABNN_ERR_ARG, "concat: null pointer");
    DABNN_REQUIRE(c1 > 0 && c2 > 0, DABNN_ERR_ARG, "concat: bad dims");
    if (pixels == 0) return DABNN_OK;
    concat_kernel<<<grid_for(pixels * (c1 + c2), 256 * 4), 256, 0, static_cast<cudaStream_t>(s)>>>(x1, c1, x2, c2, out, pixels);
    return check_launch("concat_kernel");
}
extern "C" int dabnn_fconv(const float* in, const float* weight, const float* bias, float* out, int n, int h,
                           int w, int cin, int cout, int kh, int kw, int pad_h, int pad_w, int stride_h,
                           int stride_w, int dil_h, int dil_w, dabnn_stream_t s) {
    return fconv_impl(in, weight, bias, nullptr, nullptr, 0, out, n, h, w, cin, cout, kh, kw, pad_h, pad_w, stride_h,
                      stride_w, dil_h, dil_w, static_cast<cudaStream_t>(s));
}
