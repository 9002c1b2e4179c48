// TEST INFRASTRUCTURE ONLY.  This file is part of the parity oracle: it is compiled together
// with the *unmodified* reference sources (found at build time under $DABNN_REFERENCE, never
// copied into this repository) into oracle/_ref/libdabnn_ref.so.  Only tests/, the smoke check
// and the CPU-baseline leg of bench.py may load that library; the product (dabnn_b200/) never does.
//
// What is here:
//   1. plain-C entry points around the reference's free functions (pack_mat, pad, im2col,
//      fused_binarize_im2col, bgemm, bgemm_naive, baseline_bconv, bconv_3x3, fconv,
//      baseline_fconv) so that Python/ctypes can call them on numpy buffers;
//   2. definitions of the bnn::Net member functions that normally live in dabnn/net.cpp.
//      net.cpp cannot be compiled here (it needs the FlatBuffers C++ runtime, an empty
//      submodule in the reference checkout), so Net::prepare() below performs the same steps as
//      dabnn/net.cpp:54-270 from an in-memory graph description instead of a flatbuffer.  The
//      layer classes themselves (dabnn/layers/*.cpp, dabnn/layer.cpp, common/Shaper.cpp) are the
//      reference's own translation units, compiled unmodified.
//
// Mat argument order: the reference declares Mat(w, h, c) but every caller passes (H, W, C)
// (dabnn/mat.h:180-187 vs dabnn/net.cpp:64).  The kernel-level wrappers below construct Mats with
// the true (w = W, h = H) so that non-square tensors are handled as the function bodies intend;
// the Net glue mirrors net.cpp literally and is therefore only meaningful for square tensors.

#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include <common/baseline.h>
#include <dabnn/bconv.h>
#include <dabnn/bgemm.h>
#include <dabnn/bitpack.h>
#include <dabnn/fused_binarize_im2col.h>
#include <dabnn/im2col.h>
#include <dabnn/layers/Binarize.h>
#include <dabnn/layers/Concat.h>
#include <dabnn/layers/PRelu.h>
#include <dabnn/layers/Relu.h>
#include <dabnn/net.h>
#include <dabnn/pad.h>

// dabnn/fconv.h defines its two (non-inline) fconv overloads in every TU that includes it; the
// reference's own dabnn/layers/FloatConv.cpp already does, so they are only declared here.
namespace bnn {
void fconv(const Mat &input, const Mat &weight, const int kernel_h, const int kernel_w,
           const int pad_h, const int pad_w, const int stride_h, const int stride_w,
           const int dilation_h, const int dilation_w, const int output_channels, Mat &output);
void fconv(const Mat &input, const Mat &weight, const Mat &bias, const int kernel_h,
           const int kernel_w, const int pad_h, const int pad_w, const int stride_h,
           const int stride_w, const int dilation_h, const int dilation_w,
           const int output_channels, Mat &output);
}  // namespace bnn

namespace {

thread_local std::string g_err;

template <class F>
int guarded(F&& f) {
    try {
        f();
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return 1;
    } catch (const std::string& s) {
        g_err = s;
        return 1;
    } catch (...) {
        g_err = "unknown exception";
        return 1;
    }
}

using bnn::DataType;
using bnn::Mat;

// External dense NHWC view with the true width/height (n = 1).
inline Mat view_f32(const float* p, int h, int w, int c) {
    return Mat(1, w, h, c, const_cast<float*>(p), DataType::Float, false);
}
inline Mat view_bits(const uint64_t* p, int h, int w, int c_bits) {
    return Mat(1, w, h, c_bits, const_cast<uint64_t*>(p), DataType::Bit, false);
}

// ---------------------------------------------------------------------------------------------
// In-memory graph description consumed by the Net glue.
struct GTensor {
    std::string name;
    bool is_bit = false;
    std::vector<uint32_t> shape;
    std::vector<uint64_t> bits;
    std::vector<float> floats;
};
struct GLayer {
    int type = -1;  // numeric values of flatbnn::LayerType, common/dab.fbs:4-5
    std::string name, in0, in1, w, b, out;
    int pad_h = 0, pad_w = 0, stride_h = 1, stride_w = 1, kernel_h = 0, kernel_w = 0;
};
struct Graph {
    std::string input_name;
    uint32_t in_h = 0, in_w = 0, in_c = 0;
    std::vector<GTensor> tensors;
    std::vector<GLayer> layers;
};
struct NetHandle {
    std::shared_ptr<Graph> graph;
    std::shared_ptr<bnn::Net> net;
};

enum LType {
    FpConv2D = 0, AvePoolT, MaxPoolT, ReluT, SoftmaxT, FCT, AddT, ConcatT,
    BinConv2D, AffineT, BinarizeT, SplitT, ShuffleT, PReluT
};

}  // namespace

// ---------------------------------------------------------------------------------------------
// bnn::Net member definitions (stand-ins for dabnn/net.cpp, see file header).
namespace bnn {

void Net::add_mat(const std::string& name, std::shared_ptr<Mat> mat) { mat_map_[name] = mat; }
std::shared_ptr<Mat> Net::get_blob(const std::string& name) { return mat_map_.at(name); }
std::weak_ptr<Net> Net::get_weak() { return shared_from_this(); }
std::shared_ptr<Net> Net::create() {
    struct Enabler : public Net {};
    return std::make_shared<Enabler>();
}
void Net::read_buf(const void* ptr) { read_impl(ptr); }
void Net::read_impl(const void* ptr) {
    model_ = static_cast<const flatbnn::Model*>(ptr);  // really a Graph*, see prepare()
    prepare();
}
void Net::read(const std::string&) { throw std::invalid_argument("oracle glue: read(path) is not available"); }

// Same sequence of steps as dabnn/net.cpp:54-270, driven by a Graph instead of a flatbuffer.
void Net::prepare() {
    BNN_ASSERT(!(strict && !run_fconv), "fconv must be run in strict mode");
    const Graph& g = *reinterpret_cast<const Graph*>(model_);
    {   // net.cpp:59-70
        Shaper::Shape shape{1, g.in_h, g.in_w, g.in_c};
        shaper.AddShape(g.input_name, shape);
        add_mat(g.input_name, std::make_shared<Mat>(shape[1], shape[2], shape[3], DataType::Float));
        input_name_ = g.input_name;
    }
    for (const auto& t : g.tensors) {  // net.cpp:72-138 (non-aarch64 branch)
        Shaper::Shape shape(t.shape.begin(), t.shape.end());
        shaper.AddShape(t.name, shape);
        if (t.is_bit) {
            add_mat(t.name, std::make_shared<Mat>(shape[0], shape[1], shape[2], shape[3],
                                                  const_cast<uint64_t*>(t.bits.data()), DataType::Bit,
                                                  t.bits.size(), false));
        } else if (shape.size() == 4) {
            add_mat(t.name, std::make_shared<Mat>(shape[0], shape[1], shape[2], shape[3],
                                                  const_cast<float*>(t.floats.data()), DataType::Float,
                                                  false));
        } else if (shape.size() == 1) {
            auto buf = std::make_shared<std::vector<float>>(t.floats);
            add_mat(t.name, std::make_shared<Mat>(shape[0], buf->data(), DataType::Float));
            float_bufs_.push_back(buf);
        }
    }
    auto new_output = [&](const std::string& out, const std::string& first_in) {  // ADD_LAYER tail
        const auto& os = shaper[out];
        const auto& im = *mat_map_[first_in];
        add_mat(out, std::make_shared<Mat>(os[1], os[2], os[3], im.data_type, out));
    };
    for (const auto& l : g.layers) {
        const std::vector<int32_t> strides{l.stride_h, l.stride_w}, dil{1, 1},
            pads{l.pad_h, l.pad_w, l.pad_h, l.pad_w}, kernel{l.kernel_h, l.kernel_w};
        switch (l.type) {
            case FpConv2D: {  // net.cpp:145-172
                if (mat_map_.find(l.out) == mat_map_.end()) {
                    shaper.Conv(l.in0, strides, dil, pads, l.w, l.out);
                    new_output(l.out, l.in0);
                }
                if (run_fconv) {
                    if (l.b != "") {
                        layers.push_back(std::make_shared<FloatConv>(get_weak(), l.name, l.in0, l.w, l.b,
                                                                     l.out, pads[0], pads[1], strides[0],
                                                                     strides[1], 1));
                    } else {
                        layers.push_back(std::make_shared<FloatConv>(get_weak(), l.name, l.in0, l.w, l.out,
                                                                     pads[0], pads[1], strides[0],
                                                                     strides[1], 1));
                    }
                }
                break;
            }
            case BinConv2D: {  // net.cpp:173-190
                if (mat_map_.find(l.out) == mat_map_.end()) {
                    shaper.Conv(l.in0, strides, dil, pads, l.w, l.out);
                    new_output(l.out, l.in0);
                }
                layers.push_back(std::make_shared<BinConv>(get_weak(), l.name, l.in0, l.w, l.out, pads[0],
                                                           pads[1], strides[0], strides[1]));
                break;
            }
            case AffineT: {  // net.cpp:191-202 (in-place form)
                add_mat(l.out, mat_map_[l.in0]);
                shaper.Affine(l.in0, l.w, l.b, l.out);
                layers.push_back(std::make_shared<Affine>(get_weak(), l.name, l.in0, l.w, l.b));
                break;
            }
            case AddT: {  // net.cpp:203-214 (in-place form)
                add_mat(l.out, mat_map_[l.in0]);
                shaper.Eltwise(l.in0, l.in1, l.out);
                layers.push_back(std::make_shared<Add>(get_weak(), l.name, l.in0, l.in1));
                break;
            }
            case MaxPoolT: {  // net.cpp:215-223
                if (mat_map_.find(l.out) == mat_map_.end()) {
                    shaper.Pool(l.in0, strides, pads, kernel, l.out);
                    new_output(l.out, l.in0);
                }
                layers.push_back(std::make_shared<MaxPool>(get_weak(), l.name, l.in0, l.out, kernel[0],
                                                           kernel[1], pads[0], pads[1], strides[0],
                                                           strides[1]));
                break;
            }
            case AvePoolT: {  // net.cpp:224-232
                if (mat_map_.find(l.out) == mat_map_.end()) {
                    shaper.Pool(l.in0, strides, pads, kernel, l.out);
                    new_output(l.out, l.in0);
                }
                layers.push_back(std::make_shared<AvePool>(get_weak(), l.name, l.in0, l.out, kernel[0],
                                                           kernel[1], pads[0], pads[1], strides[0],
                                                           strides[1]));
                break;
            }
            case ConcatT: {  // net.cpp:233-240
                if (mat_map_.find(l.out) == mat_map_.end()) {
                    shaper.Concat({l.in0, l.in1}, 3, l.out);
                    new_output(l.out, l.in0);
                }
                layers.push_back(std::make_shared<Concat>(get_weak(), l.name, l.in0, l.in1, l.out));
                break;
            }
            case ReluT: {  // net.cpp:241-247
                add_mat(l.out, mat_map_[l.in0]);
                shaper.Relu(l.in0, l.out);
                layers.push_back(std::make_shared<Relu>(get_weak(), l.name, l.in0));
                break;
            }
            case PReluT: {  // net.cpp:256-261
                add_mat(l.out, mat_map_[l.in0]);
                shaper.Eltwise(l.in0, l.w, l.out);
                layers.push_back(std::make_shared<PRelu>(get_weak(), l.name, l.in0, l.w));
                break;
            }
            default:  // net.cpp:262-266: Softmax / FC / Binarize / Split / Shuffle are not runnable
                throw std::runtime_error("Not supported op " + std::to_string(l.type));
        }
    }
}

void Net::run(void* input) {  // net.cpp:272-286
    BNN_ASSERT(!(strict && !run_fconv), "fconv must be run in strict mode");
    mat_map_[input_name_]->external_memory = true;
    mat_map_[input_name_]->data = input;
    for (const auto& layer : layers) layer->forward();
}

}  // namespace bnn

// ---------------------------------------------------------------------------------------------
extern "C" {

const char* ref_last_error() { return g_err.c_str(); }

// bitpack.h:277 pack_mat (-> pack_mat_64 -> common_bitpack.h:36 pack_64_bitfield)
int ref_pack_mat(const float* in, int h, int w, int c, uint64_t* out) {
    return guarded([&] {
        Mat fm = view_f32(in, h, w, c);
        Mat bm = view_bits(out, h, w, c);
        bnn::pack_mat(fm, bm);
    });
}
// baseline.h:21 baseline_pack_mat
int ref_baseline_pack_mat(const float* in, int h, int w, int c, uint64_t* out) {
    return guarded([&] {
        Mat fm = view_f32(in, h, w, c);
        Mat bm = view_bits(out, h, w, c);
        baseline_pack_mat(fm, bm);
    });
}
// bitpack.h:29 pack_64 on a flat buffer (size must be a multiple of 64)
int ref_pack_64(const float* in, uint64_t* out, size_t size) {
    return guarded([&] { bnn::pack_64(in, out, size); });
}
// common_bitpack.h:12 pack_64_bitset (offline weight packing, tail bits zeroed)
int ref_pack_64_bitset(const float* in, uint64_t* out, size_t eff_bits) {
    return guarded([&] { pack_64_bitset(in, out, eff_bits); });
}
// pad.h:7 pad on a Bit mat
int ref_pad_bits(const uint64_t* in, int h, int w, int c_bits, int pad_h, int pad_w, uint64_t* out) {
    return guarded([&] {
        Mat im = view_bits(in, h, w, c_bits);
        Mat om = view_bits(out, h + 2 * pad_h, w + 2 * pad_w, c_bits);
        bnn::pad(im, pad_h, pad_w, om);
    });
}
// pad.h:7 pad on a Float mat
int ref_pad_f32(const float* in, int h, int w, int c, int pad_h, int pad_w, float val, float* out) {
    return guarded([&] {
        Mat im = view_f32(in, h, w, c);
        Mat om = view_f32(out, h + 2 * pad_h, w + 2 * pad_w, c);
        bnn::pad(im, pad_h, pad_w, om, val);
    });
}
// im2col.h:14 im2col, Float or Bit input; `col` must hold OH*OW*kh*kw*c elements
int ref_im2col(const void* in, int is_bit, int h, int w, int c_elems, int kh, int kw, int ph, int pw,
               int sh, int sw, int dh, int dw, void* col, size_t col_elems) {
    return guarded([&] {
        if (is_bit) {
            Mat im = view_bits(static_cast<const uint64_t*>(in), h, w, c_elems);
            Mat cm(static_cast<int>(col_elems), col, DataType::Bit);
            bnn::im2col(im, kh, kw, ph, pw, sh, sw, dh, dw, cm);
        } else {
            Mat im = view_f32(static_cast<const float*>(in), h, w, c_elems);
            Mat cm(static_cast<int>(col_elems), col, DataType::Float);
            bnn::im2col(im, kh, kw, ph, pw, sh, sw, dh, dw, cm);
        }
    });
}
// fused_binarize_im2col.h:6
int ref_fused_binarize_im2col(const float* in, int h, int w, int c, int kh, int kw, int ph, int pw,
                              int sh, int sw, int dh, int dw, uint64_t* col, size_t col_words) {
    return guarded([&] {
        Mat im = view_f32(in, h, w, c);
        Mat cm(static_cast<int>(col_words), col, DataType::Bit);
        bnn::fused_binarize_im2col(im, kh, kw, ph, pw, sh, sw, dh, dw, cm);
    });
}
// bgemm.h:46 bgemm (== bgemm_naive off-ARM) and bgemm.h:587 bgemm_naive; both accumulate into c
int ref_bgemm(int m, int n, int k, const uint64_t* a, int lda, const uint64_t* b, int ldb, float* c,
              int ldc) {
    return guarded([&] { bgemm(m, n, k, a, lda, b, ldb, c, ldc); });
}
int ref_bgemm_naive(int m, int n, int k, const uint64_t* a, int lda, const uint64_t* b, int ldb,
                    float* c, int ldc) {
    return guarded([&] { bgemm_naive(m, n, k, a, lda, b, ldb, c, ldc); });
}
// baseline.h:77 baseline_bconv; weight = out_c filters of `weight_words / out_c` words each
int ref_baseline_bconv(const uint64_t* in, int h, int w, int c_bits, const uint64_t* weight,
                       size_t weight_words, int kh, int kw, int ph, int pw, int sh, int sw, int dh,
                       int dw, int out_c, float* out) {
    return guarded([&] {
        Mat im = view_bits(in, h, w, c_bits);
        Mat wm(out_c, kw, kh, c_bits, const_cast<uint64_t*>(weight), DataType::Bit, weight_words, false);
        const int oh = (h + 2 * ph - (dh * (kh - 1) + 1)) / sh + 1;
        const int ow = (w + 2 * pw - (dw * (kw - 1) + 1)) / sw + 1;
        Mat om = view_f32(out, oh, ow, out_c);
        bnn::baseline_bconv(im, wm, kh, kw, ph, pw, sh, sw, dh, dw, out_c, om);
    });
}
// bconv.h:855 bconv_3x3 on an already padded Bit input
int ref_bconv_3x3(const uint64_t* padded, int hp, int wp, int c_bits, const uint64_t* weight,
                  size_t weight_words, int out_c, int stride, float* out) {
    return guarded([&] {
        Mat im = view_bits(padded, hp, wp, c_bits);
        Mat wm(out_c, 3, 3, c_bits, const_cast<uint64_t*>(weight), DataType::Bit, weight_words, false);
        const int oh = (hp - 3) / stride + 1, ow = (wp - 3) / stride + 1;
        Mat om = view_f32(out, oh, ow, out_c);
        bnn::bconv_3x3(im, wm, om, stride);
    });
}
// fconv.h:14 / :44 fconv (Eigen GEMM) and baseline.h:37 baseline_fconv (accumulates into out)
int ref_fconv(const float* in, int h, int w, int c, const float* weight, const float* bias, int kh,
              int kw, int ph, int pw, int sh, int sw, int dh, int dw, int out_c, float* out) {
    return guarded([&] {
        Mat im = view_f32(in, h, w, c);
        Mat wm(out_c, kw, kh, c, const_cast<float*>(weight), DataType::Float, false);
        const int oh = (h + 2 * ph - (dh * (kh - 1) + 1)) / sh + 1;
        const int ow = (w + 2 * pw - (dw * (kw - 1) + 1)) / sw + 1;
        Mat om = view_f32(out, oh, ow, out_c);
        if (bias) {
            Mat bm(out_c, const_cast<float*>(bias), DataType::Float);
            bnn::fconv(im, wm, bm, kh, kw, ph, pw, sh, sw, dh, dw, out_c, om);
        } else {
            bnn::fconv(im, wm, kh, kw, ph, pw, sh, sw, dh, dw, out_c, om);
        }
    });
}
int ref_baseline_fconv(const float* in, int h, int w, int c, const float* weight, int kh, int kw,
                       int ph, int pw, int sh, int sw, int dh, int dw, int out_c, float* out) {
    return guarded([&] {
        Mat im = view_f32(in, h, w, c);
        Mat wm(out_c, kw, kh, c, const_cast<float*>(weight), DataType::Float, false);
        const int oh = (h + 2 * ph - (dh * (kh - 1) + 1)) / sh + 1;
        const int ow = (w + 2 * pw - (dw * (kw - 1) + 1)) / sw + 1;
        Mat om = view_f32(out, oh, ow, out_c);
        bnn::baseline_fconv(im, wm, kh, kw, ph, pw, sh, sw, dh, dw, out_c, om);
    });
}

// ---- graph / Net -------------------------------------------------------------------------------
void* ref_graph_new(const char* input_name, int h, int w, int c) {
    auto* g = new std::shared_ptr<Graph>(std::make_shared<Graph>());
    (*g)->input_name = input_name;
    (*g)->in_h = h; (*g)->in_w = w; (*g)->in_c = c;
    return g;
}
void ref_graph_free(void* gp) { delete static_cast<std::shared_ptr<Graph>*>(gp); }
int ref_graph_add_bit_tensor(void* gp, const char* name, const uint32_t* shape4, const uint64_t* data,
                             size_t words) {
    return guarded([&] {
        GTensor t;
        t.name = name; t.is_bit = true;
        t.shape.assign(shape4, shape4 + 4);
        t.bits.assign(data, data + words);
        (*static_cast<std::shared_ptr<Graph>*>(gp))->tensors.push_back(std::move(t));
    });
}
int ref_graph_add_float_tensor(void* gp, const char* name, const uint32_t* shape, int ndim,
                               const float* data) {
    return guarded([&] {
        GTensor t;
        t.name = name;
        t.shape.assign(shape, shape + ndim);
        size_t n = 1;
        for (int i = 0; i < ndim; i++) n *= shape[i];
        t.floats.assign(data, data + n);
        (*static_cast<std::shared_ptr<Graph>*>(gp))->tensors.push_back(std::move(t));
    });
}
// ints = {pad_h, pad_w, stride_h, stride_w, kernel_h, kernel_w}; unused strings may be "".
// `w` doubles as Affine.a / PRelu.slope and `b` as Affine.b / conv bias.
int ref_graph_add_layer(void* gp, int type, const char* name, const char* in0, const char* in1,
                        const char* w, const char* b, const char* out, const int* ints) {
    return guarded([&] {
        GLayer l;
        l.type = type; l.name = name; l.in0 = in0; l.in1 = in1; l.w = w; l.b = b; l.out = out;
        l.pad_h = ints[0]; l.pad_w = ints[1]; l.stride_h = ints[2]; l.stride_w = ints[3];
        l.kernel_h = ints[4]; l.kernel_w = ints[5];
        (*static_cast<std::shared_ptr<Graph>*>(gp))->layers.push_back(std::move(l));
    });
}
void* ref_net_build(void* gp, int optimize) {
    NetHandle* h = nullptr;
    int rc = guarded([&] {
        auto nh = std::make_unique<NetHandle>();
        nh->graph = *static_cast<std::shared_ptr<Graph>*>(gp);
        nh->net = bnn::Net::create();
        nh->net->optimize = optimize != 0;
        nh->net->read_buf(nh->graph.get());
        h = nh.release();
    });
    return rc == 0 ? h : nullptr;
}
void ref_net_free(void* np) { delete static_cast<NetHandle*>(np); }
int ref_net_run(void* np, const float* input) {
    return guarded([&] { static_cast<NetHandle*>(np)->net->run(const_cast<float*>(input)); });
}
// dims = {n, h, w, c(elements or words), is_bit}; *total = Mat::total()
int ref_net_get_blob(void* np, const char* name, const void** data, int* dims, size_t* total) {
    return guarded([&] {
        auto m = static_cast<NetHandle*>(np)->net->get_blob(name);
        *data = m->data;
        dims[0] = m->n; dims[1] = m->h; dims[2] = m->w; dims[3] = m->c;
        dims[4] = m->data_type == DataType::Bit;
        *total = m->total();
    });
}

}  // extern "C"
