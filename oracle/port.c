/* TEST INFRASTRUCTURE ONLY.
 *
 * Plain-C restatement of the reference's (JDAI-CV/dabnn) portable CPU algorithm for the binary
 * convolution hot path and the float layers around it.  It exists to check the CUDA kernels:
 * only tests/, the smoke check and the CPU-baseline leg of bench.py may build, load or call it.
 * The product library never links or calls anything in this directory.
 *
 * Every function cites the reference file:line it restates (paths relative to the reference
 * project root).  The restatement is pinned by tests/test_oracle.py against the reference's own
 * sources compiled into oracle/_ref/libdabnn_ref.so and against the committed fixtures under
 * tests/golden/ that were generated from that library.
 *
 * Conventions: tensors are dense NHWC (row stride = W*C, the reference's `hstep` for every shape
 * whose rows are already 16-byte multiples, dabnn/mat.h:534,564); bit tensors hold C/64 uint64
 * words per pixel, bit i of word j = channel 64*j+i (common/common_bitpack.h:36-175).
 * Compile with -ffp-contract=off so that a*x+b stays two rounded operations like the reference's
 * stock x86-64 build.
 */
#include <float.h>
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static inline int popcount64(uint64_t x) { /* common/baseline.h:12-19 bitcount */
    return __builtin_popcountll(x);
}

static inline int conv_out_dim(int in, int pad, int dil, int k, int stride) {
    /* dabnn/im2col.h:18-21, common/Shaper.cpp:43-52 */
    return (in + 2 * pad - (dil * (k - 1) + 1)) / stride + 1;
}

/* common/common_bitpack.h:36-175 pack_64_bitfield; dabnn/bitpack.h:29-37 pack_64.
 * bit i of each word = (f[i] > 0), strict: 0, -0 and NaN give 0. */
void port_pack_64(const float *f, uint64_t *out, size_t size) {
    for (size_t i = 0; i < size / 64; i++) {
        uint64_t w = 0;
        for (int b = 0; b < 64; b++) w |= (uint64_t)(f[i * 64 + b] > 0) << b;
        out[i] = w;
    }
}

/* dabnn/bitpack.h:254-293 pack_mat -> pack_mat_64 (requires C % 64 == 0, W*C % 64 == 0). */
int port_pack_mat(const float *in, int n, int h, int w, int c, uint64_t *out) {
    if (c % 64 != 0 || (w * c) % 64 != 0 || w * c <= 0) return 1;
    port_pack_64(in, out, (size_t)n * h * w * c);
    return 0;
}

/* tools/onnx2bnn/OnnxConverter.cpp:121-156 bitpack (offline weight packing) with
 * common/common_bitpack.h:12-34 pack_64_bitset.  `wf` is [O][kh][kw][I] floats.  If I == 64 the
 * whole tensor is packed contiguously; otherwise each filter's kh*kw*I bits are packed in 128-bit
 * chunks with a zero tail.  Returns the number of words written (out may be NULL to size). */
size_t port_pack_weight(const float *wf, int o, int kh, int kw, int i_c, uint64_t *out) {
    const size_t hwc = (size_t)kh * kw * i_c;
    size_t nw = 0;
    if (i_c != 64) {
        for (int n = 0; n < o; n++) {
            for (size_t i = 0; i < hwc; i += 128) {
                size_t eff = hwc - i < 128 ? hwc - i : 128;
                for (int half = 0; half < 2; half++) {
                    size_t e = eff > (size_t)half * 64 ? eff - (size_t)half * 64 : 0;
                    if (e > 64) e = 64;
                    if (out) {
                        uint64_t word = 0;
                        for (size_t b = 0; b < e; b++)
                            word |= (uint64_t)(wf[n * hwc + i + half * 64 + b] > 0) << b;
                        out[nw] = word;
                    }
                    nw++;
                }
            }
        }
    } else {
        size_t total = (size_t)o * hwc;
        for (size_t i = 0; i < total; i += 64) {
            if (out) {
                uint64_t word = 0;
                for (int b = 0; b < 64; b++) word |= (uint64_t)(wf[i + b] > 0) << b;
                out[nw] = word;
            }
            nw++;
        }
    }
    return nw;
}

/* dabnn/pad.h:7-30 pad: fill, then copy the interior row by row.  Bit fill is the zero word
 * (which plays the role of -1 in the xnor arithmetic, pad.h:13). */
void port_pad_bits(const uint64_t *in, int h, int w, int cw, int pad_h, int pad_w, uint64_t *out) {
    const int ow = w + 2 * pad_w, oh = h + 2 * pad_h;
    memset(out, 0, (size_t)oh * ow * cw * sizeof(uint64_t));
    for (int y = 0; y < h; y++)
        memcpy(out + ((size_t)(y + pad_h) * ow + pad_w) * cw, in + (size_t)y * w * cw,
               (size_t)w * cw * sizeof(uint64_t));
}
void port_pad_f32(const float *in, int h, int w, int c, int pad_h, int pad_w, float val, float *out) {
    const int ow = w + 2 * pad_w, oh = h + 2 * pad_h;
    for (size_t i = 0; i < (size_t)oh * ow * c; i++) out[i] = val;
    for (int y = 0; y < h; y++)
        memcpy(out + ((size_t)(y + pad_h) * ow + pad_w) * c, in + (size_t)y * w * c,
               (size_t)w * c * sizeof(float));
}

/* dabnn/im2col.h:14-47 im2col: one row per output pixel, taps in (kh, kw) order, `pix_bytes`
 * (= C * elemsize) bytes per tap, zero bytes for out-of-range taps. */
void port_im2col(const void *in, int h, int w, size_t pix_bytes, int kh, int kw, int ph, int pw,
                 int sh, int sw, int dh, int dw, void *col) {
    const int oh = conv_out_dim(h, ph, dh, kh, sh), ow = conv_out_dim(w, pw, dw, kw, sw);
    char *dst = (char *)col;
    for (int oy = 0; oy < oh; oy++)
        for (int ox = 0; ox < ow; ox++)
            for (int ky = 0; ky < kh; ky++)
                for (int kx = 0; kx < kw; kx++) {
                    const int y = oy * sh - ph + ky * dh, x = ox * sw - pw + kx * dw;
                    if (y < 0 || y >= h || x < 0 || x >= w)
                        memset(dst, 0, pix_bytes);
                    else
                        memcpy(dst, (const char *)in + ((size_t)y * w + x) * pix_bytes, pix_bytes);
                    dst += pix_bytes;
                }
}

/* dabnn/fused_binarize_im2col.h:6-68: gather each output pixel's taps as floats (0.0f for
 * out-of-range taps), zero-extend the row to a multiple of 128 floats, sign-pack it.
 * Output: OH*OW rows of ceil(kh*kw*C/128)*2 words. */
int port_fused_binarize_im2col(const float *in, int h, int w, int c, int kh, int kw, int ph, int pw,
                               int sh, int sw, int dh, int dw, uint64_t *col) {
    const int oh = conv_out_dim(h, ph, dh, kh, sh), ow = conv_out_dim(w, pw, dw, kw, sw);
    const size_t len = (size_t)kh * kw * c, len128 = (len + 127) / 128 * 128;
    if (len >= 60000) return 1; /* fused_binarize_im2col.h:15 */
    float *row = (float *)malloc(len128 * sizeof(float));
    if (!row) return 2;
    for (int oy = 0; oy < oh; oy++)
        for (int ox = 0; ox < ow; ox++) {
            float *p = row;
            for (int ky = 0; ky < kh; ky++)
                for (int kx = 0; kx < kw; kx++) {
                    const int y = oy * sh - ph + ky * dh, x = ox * sw - pw + kx * dw;
                    if (y < 0 || y >= h || x < 0 || x >= w)
                        memset(p, 0, (size_t)c * sizeof(float));
                    else
                        memcpy(p, in + ((size_t)y * w + x) * c, (size_t)c * sizeof(float));
                    p += c;
                }
            memset(p, 0, (len128 - len) * sizeof(float));
            port_pack_64(row, col, len128);
            col += len128 / 64;
        }
    free(row);
    return 0;
}

/* dabnn/bgemm.h:587-597 bgemm_naive (what bgemm.h:46-66 bgemm runs off-ARM), operand macros
 * bgemm.h:22-24: A(i,h) = a[h*lda+i], B(h,j) = b[j*ldb+h], C(i,j) = c[j*ldc+i];
 * C(i,j) += sum_h popcount(A(i,h) ^ B(h,j)), accumulated in float like the reference. */
void port_bgemm(int m, int n, int k, const uint64_t *a, int lda, const uint64_t *b, int ldb, float *c,
                int ldc) {
    for (int i = 0; i < m; i++)
        for (int j = 0; j < n; j++)
            for (int hh = 0; hh < k; hh++)
                c[(size_t)j * ldc + i] +=
                    (float)popcount64(a[(size_t)hh * lda + i] ^ b[(size_t)j * ldb + hh]);
}

/* common/baseline.h:77-116 baseline_bconv: direct binary convolution, out-of-range tap = zero
 * word; filter n starts at weight + n * (weight_words / out_c) (baseline.h:84).
 * out[oy][ox][n] = (float) sum popcount(w ^ x). */
int port_baseline_bconv(const uint64_t *in, int h, int w, int cw, const uint64_t *weight,
                        size_t weight_words, int kh, int kw, int ph, int pw, int sh, int sw, int dh,
                        int dw, int out_c, float *out) {
    if (weight_words % (size_t)out_c != 0) return 1;
    const size_t hwc = weight_words / out_c;
    const int oh = conv_out_dim(h, ph, dh, kh, sh), ow = conv_out_dim(w, pw, dw, kw, sw);
    for (int oy = 0; oy < oh; oy++)
        for (int ox = 0; ox < ow; ox++)
            for (int n = 0; n < out_c; n++) {
                uint32_t acc = 0;
                for (int ky = 0; ky < kh; ky++)
                    for (int kx = 0; kx < kw; kx++) {
                        const int y = oy * sh - ph + ky * dh, x = ox * sw - pw + kx * dw;
                        const int oob = y < 0 || y >= h || x < 0 || x >= w;
                        for (int ci = 0; ci < cw; ci++) {
                            const uint64_t wv = weight[n * hwc + ((size_t)ky * kw + kx) * cw + ci];
                            const uint64_t xv = oob ? 0 : in[((size_t)y * w + x) * cw + ci];
                            acc += (uint32_t)popcount64(wv ^ xv);
                        }
                    }
                out[((size_t)oy * ow + ox) * out_c + n] = (float)acc;
            }
    return 0;
}

/* dabnn/layers/BinConv.cpp:144-191 BinConv::forward_impl with the method chosen off-ARM
 * (BinConv.cpp:80-98): Cin == 64 -> pack_mat + baseline_bconv; otherwise zero the output,
 * fused_binarize_im2col, weights transposed to [k][Cout] (BinConv.cpp:59-76) and bgemm_naive
 * with m = Cout, n = pixels, k = weight_words / Cout (BinConv.cpp:159-164).
 * Input fp32 [H][W][Cin] (one image), output fp32 [OH][OW][Cout] of mismatch counts. */
int port_binconv_forward(const float *in, int h, int w, int cin, const uint64_t *weight,
                         size_t weight_words, int cout, int kh, int kw, int ph, int pw, int sh,
                         int sw, float *out) {
    const int oh = conv_out_dim(h, ph, 1, kh, sh), ow = conv_out_dim(w, pw, 1, kw, sw);
    int rc = 0;
    if (cin == 64) {
        uint64_t *bits = (uint64_t *)malloc((size_t)h * w * sizeof(uint64_t));
        if (!bits) return 2;
        rc = port_pack_mat(in, 1, h, w, cin, bits);
        if (!rc)
            rc = port_baseline_bconv(bits, h, w, 1, weight, weight_words, kh, kw, ph, pw, sh, sw, 1,
                                     1, cout, out);
        free(bits);
        return rc;
    }
    if (weight_words % (size_t)cout != 0) return 1;
    const int k = (int)(weight_words / cout);
    const size_t len128 = ((size_t)kh * kw * cin + 127) / 128 * 128;
    if ((size_t)k != len128 / 64) return 3; /* weights must be packed with the 128-bit row rule */
    uint64_t *col = (uint64_t *)malloc((size_t)oh * ow * k * sizeof(uint64_t));
    uint64_t *wt = (uint64_t *)malloc(weight_words * sizeof(uint64_t));
    if (!col || !wt) { free(col); free(wt); return 2; }
    for (int i = 0; i < k; i++)
        for (int j = 0; j < cout; j++) wt[(size_t)i * cout + j] = weight[(size_t)j * k + i];
    memset(out, 0, (size_t)oh * ow * cout * sizeof(float));
    rc = port_fused_binarize_im2col(in, h, w, cin, kh, kw, ph, pw, sh, sw, 1, 1, col);
    if (!rc) port_bgemm(cout, oh * ow, k, wt, cout, col, k, out, cout);
    free(col);
    free(wt);
    return rc;
}

/* dabnn/layers/Affine.cpp:10-23 affine_inplace: x = a[c]*x + b[c], product rounded, then sum. */
void port_affine(float *x, size_t pixels, int c, const float *a, const float *b) {
    for (size_t p = 0; p < pixels; p++)
        for (int ch = 0; ch < c; ch++) {
            float *v = x + p * c + ch;
            *v = a[ch] * *v + b[ch];
        }
}
/* dabnn/layers/Add.cpp:7-17 add_inplace */
void port_add(float *x, const float *y, size_t n) {
    for (size_t i = 0; i < n; i++) x[i] += y[i];
}
/* dabnn/layers/Relu.cpp:21-26 (non-NEON branch): x = max(x, 0) */
void port_relu(float *x, size_t n) {
    for (size_t i = 0; i < n; i++) x[i] = x[i] < 0.f ? 0.f : x[i]; /* std::max(x, 0.f) keeps NaN */
}
/* dabnn/layers/PRelu.cpp:6-31: x<0 ? x*slope : x; slope scalar (nslope == 1) or per channel */
int port_prelu(float *x, size_t pixels, int c, const float *slope, int nslope) {
    if (nslope != 1 && nslope != c) return 1;
    for (size_t p = 0; p < pixels; p++)
        for (int ch = 0; ch < c; ch++) {
            float *v = x + p * c + ch;
            if (*v < 0) *v = *v * slope[nslope == 1 ? 0 : ch];
        }
    return 0;
}
/* dabnn/layers/MaxPool.cpp:209-246 max_pool_fallback: start at -FLT_MAX, skip out-of-range taps */
void port_maxpool(const float *in, int h, int w, int c, int kh, int kw, int ph, int pw, int sh, int sw,
                  float *out) {
    const int oh = (h + 2 * ph - kh) / sh + 1, ow = (w + 2 * pw - kw) / sw + 1;
    for (int oy = 0; oy < oh; oy++)
        for (int ox = 0; ox < ow; ox++)
            for (int ch = 0; ch < c; ch++) {
                float m = -FLT_MAX;
                for (int ky = 0; ky < kh; ky++)
                    for (int kx = 0; kx < kw; kx++) {
                        const int y = oy * sh - ph + ky, x = ox * sw - pw + kx;
                        if (!(y < 0 || y >= h || x < 0 || x >= w)) {
                            const float v = in[((size_t)y * w + x) * c + ch];
                            m = m < v ? v : m; /* std::max(m, v) */
                        }
                    }
                out[((size_t)oy * ow + ox) * c + ch] = m;
            }
}
/* dabnn/layers/AvePool.cpp:84-123 ave_pool_fallback: sum of in-range taps (in tap order) divided
 * by the number of in-range taps */
void port_avepool(const float *in, int h, int w, int c, int kh, int kw, int ph, int pw, int sh, int sw,
                  float *out) {
    const int oh = (h + 2 * ph - kh) / sh + 1, ow = (w + 2 * pw - kw) / sw + 1;
    for (int oy = 0; oy < oh; oy++)
        for (int ox = 0; ox < ow; ox++)
            for (int ch = 0; ch < c; ch++) {
                size_t cnt = 0;
                float sum = 0;
                for (int ky = 0; ky < kh; ky++)
                    for (int kx = 0; kx < kw; kx++) {
                        const int y = oy * sh - ph + ky, x = ox * sw - pw + kx;
                        if (!(y < 0 || y >= h || x < 0 || x >= w)) {
                            sum += in[((size_t)y * w + x) * c + ch];
                            cnt++;
                        }
                    }
                out[((size_t)oy * ow + ox) * c + ch] = sum / cnt;
            }
}
/* dabnn/layers/Concat.cpp:7-22: per pixel, channels of input 1 then channels of input 2 */
void port_concat(const float *a, int ca, const float *b, int cb, size_t pixels, float *out) {
    for (size_t p = 0; p < pixels; p++) {
        memcpy(out + p * (ca + cb), a + p * ca, (size_t)ca * sizeof(float));
        memcpy(out + p * (ca + cb) + ca, b + p * cb, (size_t)cb * sizeof(float));
    }
}
/* dabnn/fconv.h:14-76 fconv = im2col + (W[Cout x K] * col^T) (+ bias per output channel), weights
 * [Cout][kh][kw][Cin].  The reference multiplies with Eigen 3.3.5's sgemm whose summation order
 * is blocked; this restatement sums each dot product in k order in float (the order of
 * common/baseline.h:37-75 baseline_fconv), so it agrees with fconv only to rounding (the
 * reference's own tests/fconv_test.cpp accepts 1e-5 absolute between the two). */
void port_fconv(const float *in, int h, int w, int c, const float *weight, const float *bias, int kh,
                int kw, int ph, int pw, int sh, int sw, int dh, int dw, int out_c, float *out) {
    const int oh = conv_out_dim(h, ph, dh, kh, sh), ow = conv_out_dim(w, pw, dw, kw, sw);
    for (int oy = 0; oy < oh; oy++)
        for (int ox = 0; ox < ow; ox++)
            for (int n = 0; n < out_c; n++) {
                float acc = 0.f;
                for (int ky = 0; ky < kh; ky++)
                    for (int kx = 0; kx < kw; kx++) {
                        const int y = oy * sh - ph + ky * dh, x = ox * sw - pw + kx * dw;
                        if (y < 0 || y >= h || x < 0 || x >= w) continue;
                        const float *ip = in + ((size_t)y * w + x) * c;
                        const float *wp = weight + (((size_t)n * kh + ky) * kw + kx) * c;
                        for (int ci = 0; ci < c; ci++) acc += wp[ci] * ip[ci];
                    }
                out[((size_t)oy * ow + ox) * out_c + n] = bias ? acc + bias[n] : acc;
            }
}
/* tools/onnx2bnn/OnnxConverter.cpp:583-639 CalculateCoeff: BatchNorm -> Affine coefficients;
 * after a binary conv over K = Cin*kh*kw bits: b += K*a (conv bias folded as b += a*bias), then
 * a *= -2, so that Affine(mismatch count) = a0*(K - 2*mismatches) + b0. */
void port_bn_to_affine(const float *scale, const float *beta, const float *mean, const float *var,
                       float eps, int n, int binary_k, const float *conv_bias, float *a, float *b) {
    for (int i = 0; i < n; i++) {
        const float t = sqrtf(var[i] + eps);
        a[i] = scale[i] / t;
        b[i] = beta[i] - scale[i] * mean[i] / t;
    }
    if (binary_k > 0) {
        for (int i = 0; i < n; i++) b[i] = b[i] + (float)binary_k * a[i];
        if (conv_bias)
            for (int i = 0; i < n; i++) b[i] += a[i] * conv_bias[i];
        for (int i = 0; i < n; i++) a[i] *= -2;
    }
}
