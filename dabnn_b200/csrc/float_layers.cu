// The bandwidth-bound float layers (Affine, Add, Relu, PRelu, pooling, Concat) and the float
// convolution.  Elementwise kernels move 16 bytes per thread and follow the reference's operation
// order exactly (product and sum rounded separately, no FMA contraction) so that results - and the
// sign bits derived from them - are bit-identical to the reference's x86 build.
#include <cuda.h>   // CUtensorMap (type only)

#include <cfloat>

#include <algorithm>
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
        if (bits) store_sign_word(bits, (size_t)(i >> 4), nib, valid);  // VEC == 4 and c % 64 == 0 guaranteed by the host
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
// IDX is the type of the flat output index: 32-bit whenever the tensor allows it, because the four
// divisions that turn it into (image, y, x, channel group) cost several times more in 64 bits than the
// nine loads they lead to.
// WIDE: the taps of a window row are loaded eight at a time before they are folded (a separate instantiation: its
// registers would cost the small windows their occupancy).
template <int VEC, bool IS_MAX, typename IDX, bool WIDE = false>
__global__ void __launch_bounds__(256) pool_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                   uint64_t* __restrict__ bits, int n, int h, int w, int c_vec,
                                                   int kh, int kw, int pad_h, int pad_w, int stride_h,
                                                   int stride_w, int oh, int ow) {
    const IDX total = (IDX)n * oh * ow * c_vec;
    const IDX stride = (IDX)gridDim.x * blockDim.x;
    const IDX bound = bits ? (total + 31) / 32 * 32 : total;
    grid_launch_dependents();   // (a grid-stride kernel: blocks that are not resident yet share the SMs with the newcomers, which only wait)
    grid_dependency_wait();
    for (IDX i = (IDX)blockIdx.x * blockDim.x + threadIdx.x; i < bound; i += stride) {
        const bool valid = i < total;
        unsigned nib = 0;
        if (valid) {
            const int cc = (int)(i % (IDX)c_vec);
            IDX p = i / (IDX)c_vec;
            const int ox = (int)(p % (IDX)ow); p /= (IDX)ow;
            const int oy = (int)(p % (IDX)oh);
            const int img = (int)(p / (IDX)oh);
            float acc[VEC];
#pragma unroll
            for (int q = 0; q < VEC; q++) acc[q] = IS_MAX ? -FLT_MAX : 0.f;
            int cnt = 0;
            for (int ky = 0; ky < kh; ky++) {
                const int y = oy * stride_h - pad_h + ky;
                if (y < 0 || y >= h) continue;
                if (!WIDE) {   // small windows: tap by tap
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
                    continue;
                }
                // the taps of a wide window row are loaded eight at a time before they are folded (in the reference's order):
                // the 7x7 head pool would otherwise wait for one load per tap
                for (int kx0 = 0; kx0 < kw; kx0 += 8) {
                    float t[8][VEC];
#pragma unroll
                    for (int u = 0; u < 8; u++) {
                        const int x = ox * stride_w - pad_w + kx0 + u;
                        if (kx0 + u < kw && x >= 0 && x < w) {
                            const float* src = in + ((((size_t)img * h + y) * w + x) * c_vec + cc) * VEC;
                            if (VEC == 4) {
                                const float4 f = __ldg(reinterpret_cast<const float4*>(src));
                                t[u][0] = f.x; t[u][1 % VEC] = f.y; t[u][2 % VEC] = f.z; t[u][3 % VEC] = f.w;
                            } else {
                                t[u][0] = __ldg(src);
                            }
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 8; u++) {
                        const int x = ox * stride_w - pad_w + kx0 + u;
                        if (kx0 + u < kw && x >= 0 && x < w) {
#pragma unroll
                            for (int q = 0; q < VEC; q++) acc[q] = IS_MAX ? (acc[q] < t[u][q] ? t[u][q] : acc[q]) : __fadd_rn(acc[q], t[u][q]);
                            cnt++;
                        }
                    }
                }
            }
            if (!IS_MAX) {
#pragma unroll
                for (int q = 0; q < VEC; q++) acc[q] = __fdiv_rn(acc[q], (float)cnt);
            }
            if (VEC == 4)
                *reinterpret_cast<float4*>(out + (size_t)i * 4) = make_float4(acc[0], acc[1 % VEC], acc[2 % VEC], acc[3 % VEC]);
            else
                out[i] = acc[0];
#pragma unroll
            for (int q = 0; q < VEC; q++) nib |= (acc[q] > 0.f ? 1u : 0u) << q;
        }
        if (bits) store_sign_word(bits, i >> 4, nib, valid);
    }
}

// 3x3 stride-2 pad-1 max pooling, four channels x a 2x2 block of outputs per thread: the four windows share a
// 5x5 input patch, so a thread loads 25 float4 for four outputs instead of 36 (the kernel is bound by the
// L2 -> SM traffic of those loads).  Each output folds its taps in the reference's order (ky, then kx,
// `acc < t ? t : acc` from -FLT_MAX), so ties between -0 and +0 and NaN inputs resolve identically.
__global__ void __launch_bounds__(256) maxpool3s2_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                         uint64_t* __restrict__ bits, unsigned char* __restrict__ out_u8, int n, int h,
                                                         int w, int c_vec, int oh, int ow) {
    const int bh = (oh + 1) / 2, bw = (ow + 1) / 2;
    const uint32_t total = (uint32_t)n * bh * bw * c_vec;
    const uint32_t bound = (total + 31) / 32 * 32;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < bound; i += gridDim.x * blockDim.x) {
        const bool valid = i < total;
        const int cc = valid ? (int)(i % (uint32_t)c_vec) : 0;
        uint32_t p = valid ? i / (uint32_t)c_vec : 0;
        const int bx = (int)(p % (uint32_t)bw); p /= (uint32_t)bw;
        const int by = (int)(p % (uint32_t)bh);
        const int img = (int)(p / (uint32_t)bh);
        float acc[2][2][4];
#pragma unroll
        for (int a = 0; a < 16; a++) (&acc[0][0][0])[a] = -FLT_MAX;
        const int y0 = 4 * by - 1, x0 = 4 * bx - 1;
        if (valid) {
#pragma unroll
            for (int ry = 0; ry < 5; ry++) {
                const int y = y0 + ry;
                if (y < 0 || y >= h) continue;
                float4 t[5];
#pragma unroll
                for (int rx = 0; rx < 5; rx++) {
                    const int x = x0 + rx;
                    t[rx] = (x >= 0 && x < w) ? __ldg(reinterpret_cast<const float4*>(in + ((((size_t)img * h + y) * w + x) * c_vec + cc) * 4))
                                              : make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX);
                }
#pragma unroll
                for (int dy = 0; dy < 2; dy++) {
                    if (ry < 2 * dy || ry > 2 * dy + 2) continue;
#pragma unroll
                    for (int dx = 0; dx < 2; dx++)
#pragma unroll
                        for (int kx = 0; kx < 3; kx++) {
                            const int rx = 2 * dx + kx;
                            if (x0 + rx < 0 || x0 + rx >= w) continue;   // the reference skips taps outside the image
                            const float4 v = t[rx];
                            float* a = acc[dy][dx];
                            a[0] = a[0] < v.x ? v.x : a[0]; a[1] = a[1] < v.y ? v.y : a[1];
                            a[2] = a[2] < v.z ? v.z : a[2]; a[3] = a[3] < v.w ? v.w : a[3];
                        }
                }
            }
        }
#pragma unroll
        for (int dy = 0; dy < 2; dy++)
#pragma unroll
            for (int dx = 0; dx < 2; dx++) {
                const int oy = 2 * by + dy, ox = 2 * bx + dx;
                const bool live = valid && oy < oh && ox < ow;
                const size_t pix = ((size_t)img * oh + oy) * ow + ox;
                const float* a = acc[dy][dx];
                if (live) *reinterpret_cast<float4*>(out + (pix * c_vec + cc) * 4) = make_float4(a[0], a[1], a[2], a[3]);
                if (bits) {
                    const unsigned nib = (a[0] > 0.f ? 1u : 0u) | (a[1] > 0.f ? 2u : 0u) | (a[2] > 0.f ? 4u : 0u) | (a[3] > 0.f ? 8u : 0u);
                    store_sign_word(bits, live ? (pix * c_vec + cc) >> 4 : 0, nib, live);
                }
                if (out_u8 && live)   // the signs as {0,1} bytes, four channels per store
                    reinterpret_cast<uint32_t*>(out_u8)[pix * c_vec + cc] =
                        (a[0] > 0.f ? 1u : 0u) | (a[1] > 0.f ? 0x100u : 0u) | (a[2] > 0.f ? 0x10000u : 0u) | (a[3] > 0.f ? 0x1000000u : 0u);
            }
    }
}

template <bool IS_MAX>
static int launch_pool(const float* in, float* out, uint64_t* bits, int n, int h, int w, int c, int kh, int kw,
                       int pad_h, int pad_w, int stride_h, int stride_w, cudaStream_t stream, unsigned char* out_u8 = nullptr) {
    DABNN_REQUIRE(in && out, DABNN_ERR_ARG, "pool: null pointer");
    DABNN_REQUIRE(n > 0 && h > 0 && w > 0 && c > 0 && kh > 0 && kw > 0 && stride_h > 0 && stride_w > 0 &&
                      pad_h >= 0 && pad_w >= 0, DABNN_ERR_ARG, "pool: bad dims");
    const int oh = (h + 2 * pad_h - kh) / stride_h + 1, ow = (w + 2 * pad_w - kw) / stride_w + 1;
    DABNN_REQUIRE(oh > 0 && ow > 0, DABNN_ERR_SHAPE, "pool: empty output");
    DABNN_REQUIRE(pad_h < kh && pad_w < kw, DABNN_ERR_SHAPE, "pool: padding must be smaller than the kernel");
    const bool vec = c % 4 == 0 && (reinterpret_cast<uintptr_t>(in) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
    DABNN_REQUIRE(!bits || (vec && c % 64 == 0), DABNN_ERR_SHAPE, "sign-bit output needs c % 64 == 0");
    if (vec && IS_MAX && kh == 3 && kw == 3 && stride_h == 2 && stride_w == 2 && pad_h == 1 && pad_w == 1 &&
        (c / 4) % 16 == 0 && (size_t)n * ((oh + 1) / 2) * ((ow + 1) / 2) * (c / 4) < (1ull << 31)) {
        const size_t blocks = (size_t)n * ((oh + 1) / 2) * ((ow + 1) / 2) * (c / 4);
        maxpool3s2_kernel<<<grid_for(blocks, 256), 256, 0, stream>>>(in, out, bits, out_u8, n, h, w, c / 4, oh, ow);
        return check_launch("maxpool3s2_kernel");
    }
    if (vec) {
        const size_t total = (size_t)n * oh * ow * (c / 4);
        if (kw > 4 && total < (1ull << 31))   // wide windows (the 7x7 head pool): a window row's loads in flight together
            launch_overlapped(pool_kernel<4, IS_MAX, uint32_t, true>, grid_for(total, 256), 256, 0, stream, in, out, bits, n, h, w, c / 4, kh, kw, pad_h,
                              pad_w, stride_h, stride_w, oh, ow);
        else if (total + (size_t)grid_for(total, 256) * 256 + 32 < (1ull << 32))   // the grid-stride loop must not wrap either
            launch_overlapped(pool_kernel<4, IS_MAX, uint32_t>, grid_for(total, 256), 256, 0, stream, in, out, bits, n, h, w, c / 4, kh, kw, pad_h,
                              pad_w, stride_h, stride_w, oh, ow);
        else
            pool_kernel<4, IS_MAX, size_t><<<grid_for(total, 256), 256, 0, stream>>>(in, out, bits, n, h, w, c / 4, kh, kw, pad_h,
                                                                                     pad_w, stride_h, stride_w, oh, ow);
    } else {
        const size_t total = (size_t)n * oh * ow * c;
        if (total + (size_t)grid_for(total, 256) * 256 + 32 < (1ull << 32))
            pool_kernel<1, IS_MAX, uint32_t><<<grid_for(total, 256), 256, 0, stream>>>(in, out, nullptr, n, h, w, c, kh, kw, pad_h,
                                                                                       pad_w, stride_h, stride_w, oh, ow);
        else
            pool_kernel<1, IS_MAX, size_t><<<grid_for(total, 256), 256, 0, stream>>>(in, out, nullptr, n, h, w, c, kh, kw, pad_h,
                                                                                     pad_w, stride_h, stride_w, oh, ow);
    }
    const int rc = check_launch("pool_kernel");
    if (rc || !out_u8) return rc;
    return binarize_u8_impl(out, out_u8, (size_t)n * oh * ow * c, stream);   // only the 3x3 / 2 kernel writes the bytes itself
}

int maxpool_impl(const float* in, float* out, uint64_t* out_bits, int n, int h, int w, int c, int kh, int kw,
                 int pad_h, int pad_w, int stride_h, int stride_w, cudaStream_t stream, unsigned char* out_u8) {
    return launch_pool<true>(in, out, out_bits, n, h, w, c, kh, kw, pad_h, pad_w, stride_h, stride_w, stream, out_u8);
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
// Implicit GEMM  C[pixel][cout] = sum_k A[pixel][k] * W[cout][k],  k = (ky*kw + kx)*cin + ci, on the
// tensor cores with fp32-grade accuracy: every fp32 operand is split into a TF32 head and a TF32
// tail (x = hi + lo, 21+ significant bits) and each product is formed as lo*hi + hi*lo + hi*hi
// with mma.sync.m16n8k8 TF32 MMAs accumulating in fp32 ("3xTF32").  The dropped lo*lo term is
// below 2^-22 relative, i.e. the result differs from an fp32 FMA chain by summation order only.
//
// CTA tile 256 pixels x 64 channels, 8 warps of 32 x 64, K slices of 16 staged in shared memory
// (register double buffering).  Weights are split into head and tail once, when a slice is
// stored to shared memory; pixels are split per fragment (each is used by one warp only).  The
// k -> (ky, kx, ci) decomposition comes from a table built once per CTA, so the gather loop has no
// integer division.  The epilogue adds the bias and can apply a per-channel affine (product and
// sum rounded separately, like the Affine layer) and a relu.
constexpr int FTM = 256, FTN = 64, FKC = 16, FPITCH = FKC + 4, FNT = 256, FTABLE = 2048;

__device__ __forceinline__ uint32_t to_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;\n" : "=r"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ void mma_tf32(float* d, const uint32_t* a, const uint32_t* b) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

struct FconvParams {
    const float *in, *wgt, *bias, *a, *b;
    float* out;
    int relu, n, h, w, cin, cout, kh, kw, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w, oh, ow;
    const float* wgt_rem;   // or null: w - trunc_tf32(w) for every weight, computed once by fconv_split_weights (1x1 GEMM kernel)
};

__global__ void __launch_bounds__(FNT, 2) fconv_kernel(const FconvParams p) {
    __shared__ __align__(16) float As[FTM * FPITCH];
    __shared__ __align__(16) uint32_t Bhi[FTN * FPITCH];
    __shared__ __align__(16) uint32_t Blo[FTN * FPITCH];
    __shared__ uint32_t ktab[FTABLE];  // k -> ci << 16 | (kx*dil_w) << 8 | (ky*dil_h)
    const int K = p.kh * p.kw * p.cin, M = p.n * p.oh * p.ow;
    const int h = p.h, w = p.w, cin = p.cin, cout = p.cout;
    const int m0 = blockIdx.x * FTM, n0 = blockIdx.y * FTN;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, tig = lane & 3;
    const bool use_tab = K <= FTABLE && p.cin < 65536 && p.kh * p.dil_h < 256 && p.kw * p.dil_w < 256;
    auto decode = [&](int k) -> uint32_t {
        const int tap = k / cin, ky = tap / p.kw;
        return ((uint32_t)(k - tap * cin) << 16) | ((uint32_t)((tap - ky * p.kw) * p.dil_w) << 8) | (uint32_t)(ky * p.dil_h);
    };
    if (use_tab)
        for (int k = tid; k < K; k += FNT) ktab[k] = decode(k);
    // loader: thread -> k quad (tid & 3) of the slice, pixel rows (tid >> 2) + 64*i, weight row tid >> 2
    const int kq = (tid & 3) * 4, lr = tid >> 2;
    long long abase[4];
    int aiy[4], aix[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int pm = m0 + lr + 64 * i;
        if (pm < M) {
            const int img = pm / (p.oh * p.ow), rem = pm - img * (p.oh * p.ow);
            const int oy = rem / p.ow, ox = rem - oy * p.ow;
            abase[i] = (long long)img * h * w;
            aiy[i] = oy * p.stride_h - p.pad_h;
            aix[i] = ox * p.stride_w - p.pad_w;
        } else {
            abase[i] = 0; aiy[i] = -(1 << 28); aix[i] = 0;   // every tap out of range -> zeros
        }
    }
    const bool vec4 = (cin % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.in) & 15) == 0);
    const bool wvec4 = (K % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.wgt) & 15) == 0);
    const int wrow = n0 + lr;
    float ra[4][4], rb[4];
    __syncthreads();   // ktab

    auto gload = [&](int k0) {
        const int k = k0 + kq;
        uint32_t e[4];
#pragma unroll
        for (int q = 0; q < 4; q++) e[q] = (k + q < K) ? (use_tab ? ktab[k + q] : decode(k + q)) : 0u;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            if (vec4 && k + 3 < K) {   // the four k share one tap: one 16-byte load
                const int y = aiy[i] + (int)(e[0] & 255u), x = aix[i] + (int)((e[0] >> 8) & 255u);
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if ((unsigned)y < (unsigned)h && (unsigned)x < (unsigned)w)
                    v = __ldg(reinterpret_cast<const float4*>(p.in + (abase[i] + (long long)y * w + x) * cin + (e[0] >> 16)));
                ra[i][0] = v.x; ra[i][1] = v.y; ra[i][2] = v.z; ra[i][3] = v.w;
            } else {
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const int y = aiy[i] + (int)(e[q] & 255u), x = aix[i] + (int)((e[q] >> 8) & 255u);
                    float v = 0.f;
                    if (k + q < K && (unsigned)y < (unsigned)h && (unsigned)x < (unsigned)w)
                        v = __ldg(p.in + (abase[i] + (long long)y * w + x) * cin + (e[q] >> 16));
                    ra[i][q] = v;
                }
            }
        }
        if (wvec4 && wrow < cout && k + 3 < K) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(p.wgt + (size_t)wrow * K + k));
            rb[0] = v.x; rb[1] = v.y; rb[2] = v.z; rb[3] = v.w;
        } else {
#pragma unroll
            for (int q = 0; q < 4; q++) rb[q] = (wrow < cout && k + q < K) ? __ldg(p.wgt + (size_t)wrow * K + k + q) : 0.f;
        }
    };
    auto sstore = [&]() {
#pragma unroll
        for (int i = 0; i < 4; i++)
            *reinterpret_cast<float4*>(&As[(lr + 64 * i) * FPITCH + kq]) = make_float4(ra[i][0], ra[i][1], ra[i][2], ra[i][3]);
        uint4 hi, lo;
        hi.x = to_tf32(rb[0]); lo.x = to_tf32(rb[0] - __uint_as_float(hi.x));
        hi.y = to_tf32(rb[1]); lo.y = to_tf32(rb[1] - __uint_as_float(hi.y));
        hi.z = to_tf32(rb[2]); lo.z = to_tf32(rb[2] - __uint_as_float(hi.z));
        hi.w = to_tf32(rb[3]); lo.w = to_tf32(rb[3] - __uint_as_float(hi.w));
        *reinterpret_cast<uint4*>(&Bhi[lr * FPITCH + kq]) = hi;
        *reinterpret_cast<uint4*>(&Blo[lr * FPITCH + kq]) = lo;
    };

    float acc[2][8][4];
#pragma unroll
    for (int i = 0; i < 2; i++)
#pragma unroll
        for (int j = 0; j < 8; j++)
#pragma unroll
            for (int q = 0; q < 4; q++) acc[i][j][q] = 0.f;

    gload(0);
    for (int k0 = 0; k0 < K; k0 += FKC) {
        __syncthreads();   // the previous slice has been consumed
        sstore();
        __syncthreads();
        if (k0 + FKC < K) gload(k0 + FKC);   // overlaps the MMAs below
#pragma unroll
        for (int ks = 0; ks < FKC; ks += 8) {
            uint32_t ahi[2][4], alo[2][4];
#pragma unroll
            for (int mt = 0; mt < 2; mt++) {
                const float* ap = &As[(warp * 32 + mt * 16 + g) * FPITCH + ks + tig];
                const float v[4] = {ap[0], ap[8 * FPITCH], ap[4], ap[8 * FPITCH + 4]};
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    ahi[mt][q] = to_tf32(v[q]);
                    alo[mt][q] = to_tf32(v[q] - __uint_as_float(ahi[mt][q]));
                }
            }
#pragma unroll
            for (int nt = 0; nt < 8; nt++) {
                const int bo = (nt * 8 + g) * FPITCH + ks + tig;
                const uint32_t bhi[2] = {Bhi[bo], Bhi[bo + 4]}, blo[2] = {Blo[bo], Blo[bo + 4]};
#pragma unroll
                for (int mt = 0; mt < 2; mt++) {
                    mma_tf32(acc[mt][nt], alo[mt], bhi);
                    mma_tf32(acc[mt][nt], ahi[mt], blo);
                    mma_tf32(acc[mt][nt], ahi[mt], bhi);
                }
            }
        }
    }
    // epilogue straight from the fragments: thread holds (row g / g+8, cols 2*tig, 2*tig+1) per tile
#pragma unroll
    for (int nt = 0; nt < 8; nt++) {
        const int col = n0 + nt * 8 + tig * 2;
        float bb[2] = {0.f, 0.f}, ca[2] = {1.f, 1.f}, cb[2] = {0.f, 0.f};
#pragma unroll
        for (int q = 0; q < 2; q++)
            if (col + q < cout) {
                if (p.bias) bb[q] = __ldg(p.bias + col + q);
                if (p.a) { ca[q] = __ldg(p.a + col + q); cb[q] = __ldg(p.b + col + q); }
            }
#pragma unroll
        for (int mt = 0; mt < 2; mt++)
#pragma unroll
            for (int hh = 0; hh < 2; hh++) {
                const int row = m0 + warp * 32 + mt * 16 + g + hh * 8;
                if (row >= M) continue;
                float v[2] = {acc[mt][nt][hh * 2], acc[mt][nt][hh * 2 + 1]};
#pragma unroll
                for (int q = 0; q < 2; q++) {
                    if (p.bias) v[q] = __fadd_rn(v[q], bb[q]);
                    if (p.a) v[q] = __fadd_rn(__fmul_rn(ca[q], v[q]), cb[q]);
                    if (p.relu) v[q] = relu_ref(v[q]);
                }
                float* op = p.out + (size_t)row * cout + col;
                if (col + 1 < cout && (cout & 1) == 0) {
                    *reinterpret_cast<float2*>(op) = make_float2(v[0], v[1]);
                } else {
                    if (col < cout) op[0] = v[0];
                    if (col + 1 < cout) op[1] = v[1];
                }
            }
    }
}

}  // namespace dabnn

#include "fconv_tc5.cuh"
#include "fconv_stem.cuh"
#include "fconv_gemm.cuh"

namespace dabnn {

// The window-reading kernel (fconv_stem.cuh) takes thin inputs with horizontal stride 2 whose output rows fill
// most of a 128-row tile: the stem of a ResNet.  Returns false for every other shape.
static bool fconv_stem_plan(const FconvParams& p, FsGeom& g, bool pool = false) {
    if (p.cin > 3 || p.stride_w != 2 || p.dil_h != 1 || p.dil_w != 1 || (p.cout % 16) != 0) return false;
    if (p.ow < 64 || p.ow > 128 || p.w > FS_MAX_W || p.kh > 16 || p.kw > 8) return false;
    if ((reinterpret_cast<uintptr_t>(p.out) & 15) != 0 || (reinterpret_cast<uintptr_t>(p.in) & 3) != 0) return false;
    g.kxp = (p.kw + 1) & ~1;
    g.kpad = p.kh * g.kxp * 4;
    g.kxp2 = (p.kw + 3) & ~3;
    g.kpad2 = p.kh * g.kxp2 * 2;
    // a multiple of four entries: both planes of every slot then start on a 32-byte boundary, so that the 32-byte swizzle
    // pairs up entries of the same plane
    const int entries = (std::max(p.w + 2 * p.pad_w, 2 * (p.ow - 1) + g.kxp2) + 3) & ~3;
    g.plane_bytes = entries * 16;
    g.slot_bytes = g.plane_bytes + entries * 8;
    g.ahead = 2;
    g.slots = p.kh + 2 * std::min(p.stride_h, p.kh);
    g.srows = (p.ow + 7) & ~7;
    g.ph = pool ? (p.oh - 1) / 2 + 1 : 0;     // 3x3 stride 2 pad 1
    g.pw = pool ? (p.ow - 1) / 2 + 1 : 0;
    g.rows_total = pool ? p.n * g.ph : p.n * p.oh;
    if (g.pw * 8 > 256 * FS_POOL_TASKS) return false;
    static thread_local int budget_device = -1, budget = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return false;
    if (dev != budget_device) {
        int optin = 0;
        cudaFuncAttributes fa;
        if (cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return false;
        if (cudaFuncGetAttributes(&fa, fconv_stem_kernel<4, true>) != cudaSuccess) return false;
        budget = optin - (int)fa.sharedSizeBytes;
        if (cudaFuncSetAttribute(fconv_stem_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, budget) != cudaSuccess ||
            cudaFuncSetAttribute(fconv_stem_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, budget) != cudaSuccess ||
            cudaFuncSetAttribute(fconv_stem_kernel<3, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, budget) != cudaSuccess ||
            cudaFuncSetAttribute(fconv_stem_kernel<4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, budget) != cudaSuccess ||
            cudaFuncSetAttribute(fconv_stem_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, budget) != cudaSuccess ||
            cudaFuncSetAttribute(fconv_stem_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, budget) != cudaSuccess ||
            cudaFuncSetAttribute(fconv_stem_kernel<3, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, budget) != cudaSuccess ||
            cudaFuncSetAttribute(fconv_stem_kernel<4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, budget) != cudaSuccess)
            return false;
        budget_device = dev;
    }
    if (fs_smem_bytes(g) > budget) {   // a shorter ring: one tile of look-ahead
        g.ahead = 1;
        g.slots = p.kh + std::min(p.stride_h, p.kh);
    }
    return fs_smem_bytes(g) <= budget;
}

// The tcgen05 kernel takes a convolution whose padded K fits the resident weight block, whose taps
// fit the 32-bit validity masks and whose channel blocks are MMA-sized; everything else runs on the
// mma.sync kernel above.  Windows larger than 1x1 go through the staged-rows variant when both
// patch buffers fit beside at least two ring stages.
struct FconvTc5Plan {
    int mode = -1, stages = 0, pitch = 0, patch_bytes = 0, vec16 = 0, n_blk = FT_N;   // mode < 0: not eligible
};

static FconvTc5Plan fconv_tc5_plan(const FconvParams& p, int kpad) {
    FconvTc5Plan plan;
    if (kpad > FT_MAXK || p.kh > 32 || p.kw > 32 || (p.cout % 16) != 0) return plan;
    if ((reinterpret_cast<uintptr_t>(p.out) & 15) != 0 || (reinterpret_cast<uintptr_t>(p.in) & 3) != 0) return plan;
    if ((long long)(p.kh * p.dil_h) * p.w * p.cin >= (1ll << 31)) return plan;
    static thread_local int budget_device = -1, budget = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return plan;
    if (dev != budget_device) {
        int optin = 0;
        cudaFuncAttributes fa0, fa1;
        if (cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return plan;
        if (cudaFuncGetAttributes(&fa0, fconv_tc5_kernel<FT_DIRECT>) != cudaSuccess) return plan;
        if (cudaFuncGetAttributes(&fa1, fconv_tc5_kernel<FT_ROWS>) != cudaSuccess) return plan;
        budget = optin - (int)std::max(fa0.sharedSizeBytes, fa1.sharedSizeBytes);
        if (cudaFuncSetAttribute(fconv_tc5_kernel<FT_DIRECT>, cudaFuncAttributeMaxDynamicSharedMemorySize, budget) != cudaSuccess) return plan;
        if (cudaFuncSetAttribute(fconv_tc5_kernel<FT_ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, budget) != cudaSuccess) return plan;
        budget_device = dev;
    }
    auto stages_for = [&](int patch_bytes) {
        const int st = (budget - ft_smem_bytes(kpad, plan.n_blk, 0, patch_bytes)) / FT_STAGE_BYTES;
        return st > FT_MAX_STAGES ? FT_MAX_STAGES : st;
    };
    if (stages_for(0) < 2) plan.n_blk = FT_N / 2;   // long K: the weights of 64 channels would leave no room for the ring
    if (p.kh * p.kw > 1) {
        const int pitch = ft_patch_pitch(p.ow, p.stride_w, p.kw, p.dil_w, p.cin);
        const int patch_bytes = 2 * p.kh * pitch * 4;
        if (patch_bytes <= FT_MAX_PATCH_BYTES && stages_for(patch_bytes) >= 2) {
            plan.mode = FT_ROWS;
            plan.stages = stages_for(patch_bytes);
            plan.pitch = pitch;
            plan.patch_bytes = patch_bytes;
            plan.vec16 = ((p.w * p.cin) % 4 == 0 && (reinterpret_cast<uintptr_t>(p.in) & 15) == 0) ? 1 : 0;
            return plan;
        }
    }
    if (stages_for(0) >= 2) {
        plan.mode = FT_DIRECT;
        plan.stages = stages_for(0);
        plan.vec16 = (p.cin % 4 == 0 && (reinterpret_cast<uintptr_t>(p.in) & 15) == 0) ? 1 : 0;
    }
    return plan;
}

// status word of the tcgen05 float convolution (this translation unit has its own copy of the word)
int fconv_tc5_status(int* status) {
    DABNN_CUDA_OK(cudaMemcpyFromSymbol(status, g_tc5_status, sizeof(int)));
    return DABNN_OK;
}

// Float convolution + (bias, affine, relu) + 3x3 stride-2 pad-1 max pooling in one kernel (fconv_stem.cuh with POOL):
// whether the shape is taken, and the launch.  The pooled result is fp32 [n][ph][pw][cout] (+ its signs as bytes).
bool fconv_pool_supported(int n, int h, int w, int cin, int cout, int kh, int kw, int pad_h, int pad_w, int stride_h, int stride_w) {
    if (n <= 0 || h <= 0 || w <= 0 || cin <= 0 || cout <= 0 || kh <= 0 || kw <= 0 || stride_h <= 0 || stride_w <= 0 || pad_h < 0 || pad_w < 0) return false;
    const int oh = conv_out_dim(h, pad_h, 1, kh, stride_h), ow = conv_out_dim(w, pad_w, 1, kw, stride_w);
    if (oh < 2 || ow < 2 || (long long)n * oh * ow >= (1ll << 31)) return false;
    const FconvParams prm{reinterpret_cast<const float*>(uintptr_t(1) << 20), nullptr, nullptr, nullptr, nullptr, reinterpret_cast<float*>(uintptr_t(1) << 20),
                          0, n, h, w, cin, cout, kh, kw, pad_h, pad_w, stride_h, stride_w, 1, 1, oh, ow};
    FsGeom g;
    return fconv_stem_plan(prm, g, true);
}

int fconv_pool_impl(const float* in, const float* weight, const float* bias, const float* a, const float* b, int relu, float* pool_out,
                    unsigned char* pool_u8, int n, int h, int w, int cin, int cout, int kh, int kw, int pad_h, int pad_w, int stride_h,
                    int stride_w, cudaStream_t stream) {
    DABNN_REQUIRE(in && weight && pool_out, DABNN_ERR_ARG, "fconv_pool: null pointer");
    DABNN_REQUIRE((a == nullptr) == (b == nullptr), DABNN_ERR_ARG, "fconv_pool: a and b go together");
    DABNN_REQUIRE(fconv_pool_supported(n, h, w, cin, cout, kh, kw, pad_h, pad_w, stride_h, stride_w), DABNN_ERR_SHAPE,
                  "fconv_pool: shape not taken by the fused convolution + pooling kernel");
    DABNN_REQUIRE(((reinterpret_cast<uintptr_t>(pool_out) | reinterpret_cast<uintptr_t>(pool_u8)) & 15) == 0 && (reinterpret_cast<uintptr_t>(in) & 3) == 0,
                  DABNN_ERR_ARG, "fconv_pool: outputs must be 16-byte aligned");
    const int oh = conv_out_dim(h, pad_h, 1, kh, stride_h), ow = conv_out_dim(w, pad_w, 1, kw, stride_w);
    const FconvParams prm{in, weight, bias, a, b, pool_out, relu, n, h, w, cin, cout, kh, kw, pad_h, pad_w, stride_h, stride_w, 1, 1, oh, ow};
    FsGeom geom;
    DABNN_REQUIRE(fconv_stem_plan(prm, geom, true), DABNN_ERR_SHAPE, "fconv_pool: shape not taken by the fused convolution + pooling kernel");
    const int ny = (cout + FS_N - 1) / FS_N;
    dim3 sgrid(std::min(geom.rows_total, std::max(1, sm_count() / ny)), ny);
    const int smem = fs_smem_bytes(geom);
    const CUtensorMap no_map{};
    switch (geom.kxp / 2) {
        case 1: launch_overlapped(fconv_stem_kernel<1, true>, sgrid, FS_THREADS, smem, stream, prm, geom, no_map, pool_out, pool_u8); break;
        case 2: launch_overlapped(fconv_stem_kernel<2, true>, sgrid, FS_THREADS, smem, stream, prm, geom, no_map, pool_out, pool_u8); break;
        case 3: launch_overlapped(fconv_stem_kernel<3, true>, sgrid, FS_THREADS, smem, stream, prm, geom, no_map, pool_out, pool_u8); break;
        default: launch_overlapped(fconv_stem_kernel<4, true>, sgrid, FS_THREADS, smem, stream, prm, geom, no_map, pool_out, pool_u8); break;
    }
    return check_launch("fconv_stem_kernel (pooled)");
}

int fconv_status_word(int** addr) {
    DABNN_CUDA_OK(cudaGetSymbolAddress(reinterpret_cast<void**>(addr), g_tc5_status));
    return DABNN_OK;
}

// remainders of the 3xTF32 split of constant weights: rem = w - (w with its low 13 mantissa bits cleared)
__global__ void split_weights_kernel(const float* __restrict__ w, float* __restrict__ rem, size_t count) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x) {
        uint32_t hi, lo;
        split_tf32(w[i], hi, lo);
        rem[i] = __uint_as_float(lo);
    }
}

int fconv_split_weights(const float* weight, float* rem, size_t count, cudaStream_t stream) {
    DABNN_REQUIRE(weight && rem, DABNN_ERR_ARG, "fconv_split_weights: null pointer");
    if (!count) return DABNN_OK;
    split_weights_kernel<<<(int)std::min<size_t>((count + 255) / 256, 1024), 256, 0, stream>>>(weight, rem, count);
    return check_launch("split_weights_kernel");
}

bool fconv_uses_weight_remainders(int cin, int cout, int kh, int kw, int pad_h, int pad_w, int stride_h, int stride_w) {
    return kh == 1 && kw == 1 && stride_h == 1 && stride_w == 1 && pad_h == 0 && pad_w == 0 && cin % FG_CHUNK == 0 && cout % 4 == 0;
}

int fconv_impl(const float* in, const float* weight, const float* bias, const float* a, const float* b, int relu,
               float* out, int n, int h, int w, int cin, int cout, int kh, int kw, int pad_h, int pad_w,
               int stride_h, int stride_w, int dil_h, int dil_w, cudaStream_t stream, const float* weight_rem) {
    DABNN_REQUIRE(in && weight && out, DABNN_ERR_ARG, "fconv: null pointer");
    DABNN_REQUIRE(n > 0 && h > 0 && w > 0 && cin > 0 && cout > 0 && kh > 0 && kw > 0 && stride_h > 0 &&
                      stride_w > 0 && dil_h > 0 && dil_w > 0 && pad_h >= 0 && pad_w >= 0, DABNN_ERR_ARG,
                  "fconv: bad dims");
    DABNN_REQUIRE((a == nullptr) == (b == nullptr), DABNN_ERR_ARG, "fconv: a and b go together");
    const int oh = conv_out_dim(h, pad_h, dil_h, kh, stride_h), ow = conv_out_dim(w, pad_w, dil_w, kw, stride_w);
    DABNN_REQUIRE(oh > 0 && ow > 0, DABNN_ERR_SHAPE, "fconv: empty output");
    DABNN_REQUIRE((long long)n * oh * ow < (1ll << 31), DABNN_ERR_SHAPE, "fconv: too many output pixels");
    DABNN_REQUIRE((reinterpret_cast<uintptr_t>(out) & 7) == 0, DABNN_ERR_ARG, "fconv: output must be 8-byte aligned");
    dim3 grid((n * oh * ow + FTM - 1) / FTM, (cout + FTN - 1) / FTN);
    const FconvParams prm{in, weight, bias, a, b, out, relu, n, h, w, cin, cout, kh, kw, pad_h, pad_w,
                          stride_h, stride_w, dil_h, dil_w, oh, ow, (reinterpret_cast<uintptr_t>(weight_rem) & 15) == 0 ? weight_rem : nullptr};
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    if (kh == 1 && kw == 1 && stride_h == 1 && stride_w == 1 && pad_h == 0 && pad_w == 0 && cin % FG_CHUNK == 0 && cout % 4 == 0 &&
        al16(in) && al16(weight) && al16(out) && al16(bias) && al16(a) && al16(b)) {
        // a 1x1 convolution is a GEMM over [pixels][cin]: TMA-fed (fconv_gemm.cuh)
        static thread_local int gemm_device = -1, gemm_stages = 0;
        int dev = 0;
        DABNN_CUDA_OK(cudaGetDevice(&dev));
        if (dev != gemm_device) {
            int optin = 0;
            cudaFuncAttributes fa;
            DABNN_CUDA_OK(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
            DABNN_CUDA_OK(cudaFuncGetAttributes(&fa, fconv_gemm_kernel));
            gemm_stages = FG_MAX_STAGES;
            while (gemm_stages >= 2 && fg_smem_bytes(gemm_stages) > optin - (int)fa.sharedSizeBytes) gemm_stages--;
            if (gemm_stages >= 2)
                DABNN_CUDA_OK(cudaFuncSetAttribute(fconv_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, fg_smem_bytes(gemm_stages)));
            gemm_device = dev;
        }
        const int Mpx = n * oh * ow, tiles_m = (Mpx + 127) / 128;
        // channels per work item: as large as leaves every SM a work item
        int n_blk = FG_N;
        while (n_blk > 32 && tiles_m * ((cout + n_blk - 1) / n_blk) < sm_count()) n_blk >>= 1;
        CUtensorMap a_map, w_map, wr_map{}, o_map;
        const unsigned box[2] = {32, 128}, wbox[2] = {32, (unsigned)n_blk};
        const unsigned long long adims[2] = {(unsigned long long)cin, (unsigned long long)Mpx}, astr[1] = {(unsigned long long)cin * 4};
        const unsigned long long wdims[2] = {(unsigned long long)cin, (unsigned long long)cout};
        const unsigned long long odims[2] = {(unsigned long long)cout, (unsigned long long)Mpx}, ostr[1] = {(unsigned long long)cout * 4};
        if (gemm_stages >= 2 && make_f32_tensor_map(&a_map, const_cast<float*>(in), 2, adims, astr, box) &&
            make_f32_tensor_map(&w_map, const_cast<float*>(weight), 2, wdims, astr, wbox) && make_f32_tensor_map(&o_map, out, 2, odims, ostr, box) &&
            (!prm.wgt_rem || make_f32_tensor_map(&wr_map, const_cast<float*>(prm.wgt_rem), 2, wdims, astr, wbox))) {
            const int items = tiles_m * ((cout + n_blk - 1) / n_blk);
            launch_overlapped(fconv_gemm_kernel, std::min(items, sm_count()), FG_THREADS, fg_smem_bytes(gemm_stages), stream, prm, Mpx, gemm_stages, n_blk, a_map,
                              w_map, wr_map, o_map);
            return check_launch("fconv_gemm_kernel");
        }
    }
    FsGeom geom;
    if (fconv_stem_plan(prm, geom)) {
        const int ny = (cout + FS_N - 1) / FS_N;
        CUtensorMap out_map{};
        const unsigned long long dims[3] = {(unsigned long long)cout, (unsigned long long)ow, (unsigned long long)n * oh};
        const unsigned long long strides[2] = {(unsigned long long)cout * 4, (unsigned long long)ow * cout * 4};
        const unsigned box[3] = {32, (unsigned)geom.srows, 1};
        if (make_f32_tensor_map(&out_map, out, 3, dims, strides, box)) {
            dim3 sgrid(std::min(geom.rows_total, std::max(1, sm_count() / ny)), ny);
            const int smem = fs_smem_bytes(geom);
            switch (geom.kxp / 2) {
                case 1: launch_overlapped(fconv_stem_kernel<1, false>, sgrid, FS_THREADS, smem, stream, prm, geom, out_map, nullptr, nullptr); break;
                case 2: launch_overlapped(fconv_stem_kernel<2, false>, sgrid, FS_THREADS, smem, stream, prm, geom, out_map, nullptr, nullptr); break;
                case 3: launch_overlapped(fconv_stem_kernel<3, false>, sgrid, FS_THREADS, smem, stream, prm, geom, out_map, nullptr, nullptr); break;
                default: launch_overlapped(fconv_stem_kernel<4, false>, sgrid, FS_THREADS, smem, stream, prm, geom, out_map, nullptr, nullptr); break;
            }
            return check_launch("fconv_stem_kernel");
        }
    }
    const int M = n * oh * ow, K = kh * kw * cin, kpad = (K + 7) / 8 * 8;
    const FconvTc5Plan plan = fconv_tc5_plan(prm, kpad);
    if (plan.mode >= 0) {
        const int nseg = (ow + 127) / 128, ny = (cout + plan.n_blk - 1) / plan.n_blk;
        const int ntiles = plan.mode == FT_ROWS ? n * oh * nseg : (M + 127) / 128;
        dim3 tgrid(std::min(ntiles, std::max(1, sm_count() / ny)), ny);
        const int smem = ft_smem_bytes(kpad, plan.n_blk, plan.stages, plan.patch_bytes);
        // output descriptor [line][pixel][channel]: ROWS = (n * oh, ow, cout), DIRECT = (1, M, cout)
        CUtensorMap out_map{};
        const bool rows = plan.mode == FT_ROWS;
        const unsigned long long dims[3] = {(unsigned long long)cout, (unsigned long long)(rows ? ow : M), (unsigned long long)(rows ? n * oh : 1)};
        const unsigned long long strides[2] = {(unsigned long long)cout * 4, (unsigned long long)(rows ? ow : M) * cout * 4};
        const unsigned box[3] = {32, 128, 1};
        if (!make_f32_tensor_map(&out_map, out, 3, dims, strides, box)) {
            fconv_kernel<<<grid, FNT, 0, stream>>>(prm);   // no TMA descriptor: the mma.sync kernel
            return check_launch("fconv_kernel");
        }
        if (plan.mode == FT_ROWS)
            fconv_tc5_kernel<FT_ROWS><<<tgrid, FT_THREADS, smem, stream>>>(prm, M, K, kpad, ntiles, plan.stages, nseg, plan.pitch, plan.vec16, plan.n_blk, out_map);
        else
            fconv_tc5_kernel<FT_DIRECT><<<tgrid, FT_THREADS, smem, stream>>>(prm, M, K, kpad, ntiles, plan.stages, nseg, 0, plan.vec16, plan.n_blk, out_map);
        return check_launch("fconv_tc5_kernel");
    }
    fconv_kernel<<<grid, FNT, 0, stream>>>(prm);
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
extern "C" int dabnn_fconv_maxpool_supported(int n, int h, int w, int cin, int cout, int kh, int kw, int pad_h, int pad_w, int stride_h,
                                             int stride_w) {
    return fconv_pool_supported(n, h, w, cin, cout, kh, kw, pad_h, pad_w, stride_h, stride_w) ? 1 : 0;
}
extern "C" int dabnn_fconv_maxpool(const float* in, const float* weight, const float* bias, const float* a, const float* b, int relu,
                                   float* out, unsigned char* out_u8, int n, int h, int w, int cin, int cout, int kh, int kw, int pad_h,
                                   int pad_w, int stride_h, int stride_w, dabnn_stream_t s) {
    return fconv_pool_impl(in, weight, bias, a, b, relu, out, out_u8, n, h, w, cin, cout, kh, kw, pad_h, pad_w, stride_h, stride_w,
                           static_cast<cudaStream_t>(s));
}
extern "C" int dabnn_fconv(const float* in, const float* weight, const float* bias, float* out, int n, int h,
                           int w, int cin, int cout, int kh, int kw, int pad_h, int pad_w, int stride_h,
                           int stride_w, int dil_h, int dil_w, dabnn_stream_t s) {
    return fconv_impl(in, weight, bias, nullptr, nullptr, 0, out, n, h, w, cin, cout, kh, kw, pad_h, pad_w, stride_h,
                      stride_w, dil_h, dil_w, static_cast<cudaStream_t>(s));
}
