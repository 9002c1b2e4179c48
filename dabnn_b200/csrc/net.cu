// Host runtime: the counterpart of the reference's bnn::Net (dabnn/net.h:22-66, dabnn/net.cpp).
//
// read_buf()  parses the .dab model, uploads the initializers, infers blob shapes
//             (reference common/Shaper.cpp) and compiles the layer list into a fixed sequence of
//             kernel launches ("plan") over one device arena.
// run()       copies the input to the device when it is a host pointer and enqueues the plan on
//             the net's stream.
//
// Two plans exist.  optimize = false is the literal layer-by-layer sequence of the reference with
// every blob kept (any blob can be fetched afterwards, Affine/Add/Relu/PRelu alias their first
// input like the reference, common/flatbuffers_helper.h:68-73) and the CUDA-core popc engine.
// optimize = true fuses BinConv + Affine (+ Add) into one kernel that also emits the sign bits the
// next BinConv consumes, fuses FpConv + Affine (+ Relu), lets pooling / elementwise producers emit
// sign bits, and reuses arena memory between blobs whose lifetimes do not overlap.  Both plans run
// the same arithmetic in the same order, so their outputs are bit-identical.
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "common.cuh"
#include "dab_reader.h"
#include "kernels.h"

namespace dabnn {

namespace {

// Last node of every launch plan: collects the status words the tensor-core kernels raise when one of their
// bounded waits gives up (one word per translation unit), clears them, and reports the first code to the host
// through a word of mapped pinned memory that the Net checks after it has synchronised.
__global__ void status_gather_kernel(int* w0, int* w1, int* w2, volatile int* host_word) {
    int code = 0;
    int* words[3] = {w0, w1, w2};
    for (int i = 0; i < 3; i++) {
        const int v = words[i] ? atomicExch(words[i], 0) : 0;
        if (v && !code) code = v;
    }
    if (code) {
        *host_word = code;
        __threadfence_system();
    }
}

struct TensorInfo {
    bool is_bit = false;
    std::vector<uint32_t> shape;
    size_t count = 0;        // elements (floats or words)
    void* dev = nullptr;     // device copy
};

struct Blob {                // one activation buffer (aliases share a Blob)
    int h = 0, w = 0, c = 0; // per image
    int def_op = -1, last_use = -1;
    bool keep = false;       // must survive the run (network output / unfused plan)
    bool need_f32 = true;    // some op reads or exposes the float values
    bool need_bits = false;  // some op reads the sign bits
    bool u8 = false;         // the sign bits are kept as {0,1} bytes (byte-activation engine), not packed words
    bool keep_bits = false;  // the packed bits are a named output of the model (Binarize layer): they survive the run
    size_t f32_off = (size_t)-1, bits_off = (size_t)-1;
    size_t per_image() const { return (size_t)h * w * c; }
};

enum class OpKind { FConv, FConvPool, BConvBlock, BinConvIm2col, Pack, Chain, PRelu, MaxPool, AvePool, Concat };

struct Op {
    OpKind kind;
    std::string cls;  // reference layer class, for per-class timing
    int in = -1, in2 = -1, out = -1;
    int out2 = -1;    // BConvBlock: the blob that holds the 2x2 / 2 average pooling of out, written by the same kernel
    const TensorInfo *w = nullptr, *bias = nullptr, *a = nullptr, *b = nullptr, *slope = nullptr;
    int kh = 0, kw = 0, pad_h = 0, pad_w = 0, stride_h = 1, stride_w = 1;
    int relu = 0;
    bool write_f32 = true, write_bits = false;
    const unsigned char* w_expanded = nullptr;   // BConvBlock: the weights in the TCGEN05 engine's stage layout
    const float* w_rem = nullptr;                // FConv on the 1x1 GEMM kernel: the weights' 3xTF32 remainders, computed at load time
    bool u8 = false;                             // BConvBlock: runs on the byte-activation engine (its input blob is u8)
};

struct Layer {
    LayerType type;
    std::string name, input, input2, weight, bias, a, b, slope, output;
    std::vector<int32_t> pads, strides, dilations, kernel;
};

}  // namespace

struct NetImpl {
    int device = 0;
    cudaStream_t stream = nullptr;
    bool optimize = true, run_fconv = true, strict = true;
    int max_batch = 1, engine = DABNN_ENGINE_AUTO;
    bool loaded = false, profiling = false;

    std::string input_name;
    int in_h = 0, in_w = 0, in_c = 0;
    std::map<std::string, TensorInfo> tensors;
    std::vector<Layer> layers;
    std::map<std::string, int> blob_of;  // blob name -> index in blobs (aliases map to the same index)
    std::vector<Blob> blobs;
    std::vector<Op> plan;
    std::vector<std::string> outputs;

    unsigned char* arena = nullptr;
    size_t arena_bytes = 0, weights_bytes = 0, arena_bytes_extra = 0;
    unsigned char* weights = nullptr;
    unsigned char* expanded = nullptr;   // all binary convolution weights expanded to bytes, once, at load time
    size_t expanded_bytes = 0;
    float* remainders = nullptr;         // 3xTF32 remainders of the 1x1 float convolutions' weights
    size_t remainders_bytes = 0;
    const float* cur_input = nullptr;  // device pointer of the images the plan is currently reading
    int cur_batch = 0;
    int input_blob = -1;
    size_t out_offset = 0;             // first image of the sub-batch being computed (kept blobs are full-batch)

    // host inputs are streamed in sub-batches: copy of sub-batch k+1 overlaps the kernels of k
    int host_chunk = 256;   // images per staging buffer
    size_t chunk_seq = 0;   // sub-batches copied so far, over all runs: sub-batch i uses staging buffer i & 1
    cudaStream_t copy_stream = nullptr;
    float* staging[2] = {nullptr, nullptr};
    cudaEvent_t copied[2] = {nullptr, nullptr}, consumed[2] = {nullptr, nullptr};

    static constexpr int kTickets = 8;
    cudaEvent_t tickets[kTickets] = {};
    int next_ticket = 0;

    std::vector<cudaEvent_t> events;
    std::vector<std::string> time_names;
    std::vector<float> time_ms;

    std::map<std::string, int> bit_names;   // outputs of Binarize layers: blob whose packed sign bits they name
    int* status_words[3] = {nullptr, nullptr, nullptr};   // device addresses of the kernels' status words
    volatile int* status_host = nullptr;                  // mapped pinned word written by status_gather_kernel
    int* status_dev = nullptr;                            // its device-side address
    int check_status();                                   // after a synchronisation: DABNN_OK or DABNN_ERR_TIMEOUT

    ~NetImpl() {
        if (status_host) cudaFreeHost(const_cast<int*>(status_host));
        for (auto& g : graphs) if (g.exec) cudaGraphExecDestroy(g.exec);
        for (auto e : events) cudaEventDestroy(e);
        for (auto e : tickets) if (e) cudaEventDestroy(e);
        for (int i = 0; i < 2; i++) {
            if (copied[i]) cudaEventDestroy(copied[i]);
            if (consumed[i]) cudaEventDestroy(consumed[i]);
            if (staging[i]) cudaFree(staging[i]);
        }
        if (copy_stream) cudaStreamDestroy(copy_stream);
        if (arena) cudaFree(arena);
        if (weights) cudaFree(weights);
        if (expanded) cudaFree(expanded);
        if (remainders) cudaFree(remainders);
        if (stream) cudaStreamDestroy(stream);
    }

    int parse(const uint8_t* buf, size_t len);
    int build();
    int run(const float* input, int batch, bool is_device);
    int run_plan(int batch);
    int run_plan_graphed(int batch);

    // The launch plan of one (sub-batch size, input pointer, output offset) captured as a CUDA graph on its second
    // use: a small batch is bound by the host's launch rate (29 launches for Bi-Real-18), a graph replays them
    // with one call.  Off while profiling (events between launches) and after any capture failure.
    struct PlanGraph {
        int batch;
        const float* input;
        size_t out_offset;
        cudaGraphExec_t exec;
    };
    std::vector<PlanGraph> graphs;
    bool use_graphs = true;
    static constexpr size_t kMaxGraphs = 16;
    // blobs that outlive the run hold the whole batch; everything else is reused per sub-batch
    float* f32(int blob) const {
        if (blob == input_blob) return const_cast<float*>(cur_input);
        const Blob& b = blobs[blob];
        return reinterpret_cast<float*>(arena + b.f32_off) + (b.keep ? out_offset * b.per_image() : 0);
    }
    uint64_t* bits(int blob) const {
        const Blob& b = blobs[blob];
        return reinterpret_cast<uint64_t*>(arena + b.bits_off) + ((b.keep || b.keep_bits) ? out_offset * b.h * b.w * (b.c / 64) : 0);
    }
    unsigned char* bytes(int blob) const {   // the same buffer when the blob keeps its signs as bytes
        const Blob& b = blobs[blob];
        return arena + b.bits_off + (b.keep ? out_offset * b.per_image() : 0);
    }
};

// -------------------------------------------------------------------------------------------------
int NetImpl::parse(const uint8_t* buf, size_t len) {
    DABNN_REQUIRE(buf && len >= 8, DABNN_ERR_FORMAT, "dab: buffer too small");
    try {
        FbBuffer fb(buf, len);
        FbTable model(&fb, fb.read<uint32_t>(0));
        const uint32_t version = model.scalar<uint32_t>(3, 0);
        DABNN_REQUIRE(version == 2, DABNN_ERR_FORMAT,
                      "The model version should be 2, got " + std::to_string(version) + " instead.");  // net.cpp:56
        const auto inputs = model.tables(2);
        DABNN_REQUIRE(!inputs.empty(), DABNN_ERR_FORMAT, "dab: model has no input");
        {   // only the first input is used (net.cpp:59-70)
            const auto shape = inputs[0].vec<uint32_t>(0);
            DABNN_REQUIRE(shape.size() == 4, DABNN_ERR_FORMAT, "dab: input shape must be NHWC");
            DABNN_REQUIRE(shape[1] > 0 && shape[2] > 0 && shape[3] > 0 && shape[1] < (1u << 16) && shape[2] < (1u << 16) &&
                              shape[3] < (1u << 16), DABNN_ERR_FORMAT, "dab: input dimensions must lie in [1, 65535]");
            in_h = shape[1]; in_w = shape[2]; in_c = shape[3];
            input_name = inputs[0].str(1);
        }
        // ---- initializers: one device slab, 256-byte aligned entries ----
        struct Pending { TensorInfo* t; const void* src; size_t bytes, off; };
        std::vector<Pending> pend;
        size_t off = 0;
        for (const auto& t : model.tables(1)) {
            TensorInfo ti;
            ti.is_bit = t.scalar<int8_t>(0, 0) == 1;
            ti.shape = t.vec<uint32_t>(3);
            const std::string name = t.str(4);
            size_t count = 0;
            const void* src = ti.is_bit ? (const void*)t.vec_view<uint64_t>(1, &count)
                                        : (const void*)t.vec_view<float>(2, &count);
            DABNN_REQUIRE(src && count > 0, DABNN_ERR_FORMAT, "dab: tensor " + name + " has no data");
            for (uint32_t d : ti.shape) DABNN_REQUIRE(d > 0, DABNN_ERR_FORMAT, "dab: tensor " + name + " has an empty dimension");
            ti.count = count;
            auto& slot = tensors[name];
            slot = ti;
            const size_t bytes = count * (ti.is_bit ? 8 : 4);
            pend.push_back({&slot, src, bytes, off});
            off += (bytes + 255) / 256 * 256;
        }
        weights_bytes = off;
        if (off) {
            if (cudaMalloc(&weights, off) != cudaSuccess) return fail(DABNN_ERR_OOM, "cannot allocate weights on the device");
            for (auto& p : pend) {
                DABNN_CUDA_OK(cudaMemcpyAsync(weights + p.off, p.src, p.bytes, cudaMemcpyHostToDevice, stream));
                p.t->dev = weights + p.off;
            }
            DABNN_CUDA_OK(cudaStreamSynchronize(stream));  // the caller may free the buffer after read
        }
        // ---- layers ----
        for (const auto& l : model.tables(0)) {
            Layer L;
            L.type = (LayerType)l.scalar<int8_t>(0, 0);
            L.name = l.str(14);
            auto conv = [&](const FbTable& p) {
                L.input = p.str(0); L.weight = p.str(1); L.bias = p.str(2);
                L.pads = p.vec<int32_t>(3); L.strides = p.vec<int32_t>(4); L.dilations = p.vec<int32_t>(5);
                L.output = p.str(6);
            };
            auto pool = [&](const FbTable& p) {
                L.input = p.str(0); L.kernel = p.vec<int32_t>(1); L.pads = p.vec<int32_t>(2);
                L.strides = p.vec<int32_t>(3); L.output = p.str(4);
            };
            FbTable p;
            switch (L.type) {
                case LayerType::FpConv2D: p = l.table(1); break;
                case LayerType::BinConv2D: p = l.table(2); break;
                case LayerType::AvePool: p = l.table(3); break;
                case LayerType::MaxPool: p = l.table(4); break;
                case LayerType::Relu: p = l.table(5); break;
                case LayerType::Softmax: p = l.table(6); break;
                case LayerType::FC: p = l.table(7); break;
                case LayerType::Add: p = l.table(8); break;
                case LayerType::Concat: p = l.table(9); break;
                case LayerType::Affine: p = l.table(10); break;
                case LayerType::Binarize: p = l.table(11); break;
                case LayerType::Split: p = l.table(12); break;
                case LayerType::Shuffle: p = l.table(13); break;
                case LayerType::PRelu: p = l.table(15); break;
                default: return fail(DABNN_ERR_UNSUPPORTED, "Not supported op " + std::to_string((int)L.type));
            }
            DABNN_REQUIRE(p.valid(), DABNN_ERR_FORMAT, "param != nullptr is not satisfied!");  // flatbuffers_helper.h:43
            switch (L.type) {
                case LayerType::FpConv2D: case LayerType::BinConv2D: conv(p); break;
                case LayerType::AvePool: case LayerType::MaxPool: pool(p); break;
                case LayerType::Relu: case LayerType::Softmax: case LayerType::Binarize: case LayerType::Shuffle:
                    L.input = p.str(0); L.output = p.str(1); break;
                case LayerType::FC: L.input = p.str(0); L.weight = p.str(1); L.bias = p.str(2); L.output = p.str(3); break;
                case LayerType::Add: L.input = p.str(0); L.input2 = p.str(1); L.output = p.str(2); break;
                case LayerType::Concat: {
                    const auto ins = p.strings(0);
                    DABNN_REQUIRE(ins.size() == 2, DABNN_ERR_UNSUPPORTED, "concat takes exactly two inputs");
                    DABNN_REQUIRE(p.scalar<int32_t>(1, 0) == 3, DABNN_ERR_SHAPE, "axis == 3 is not satisfied!");  // net.cpp:235
                    L.input = ins[0]; L.input2 = ins[1]; L.output = p.str(2);
                    break;
                }
                case LayerType::Affine: L.input = p.str(0); L.a = p.str(1); L.b = p.str(2); L.output = p.str(3); break;
                case LayerType::PRelu: L.input = p.str(0); L.slope = p.str(1); L.output = p.str(2); break;
                default: L.input = p.str(0); break;
            }
            layers.push_back(std::move(L));
        }
    } catch (const DabError& e) {
        return fail(DABNN_ERR_FORMAT, e.what());
    } catch (const std::exception& e) {   // bad_alloc / length_error from a hostile length field
        return fail(DABNN_ERR_FORMAT, std::string("dab: ") + e.what());
    }
    return DABNN_OK;
}

// -------------------------------------------------------------------------------------------------
int NetImpl::build() {
    DABNN_REQUIRE(!(strict && !run_fconv), DABNN_ERR_STATE, "fconv must be run in strict mode");  // net.cpp:55
    auto new_blob = [&](const std::string& name, int h, int w, int c) {
        Blob b; b.h = h; b.w = w; b.c = c;
        blobs.push_back(b);
        blob_of[name] = (int)blobs.size() - 1;
        return (int)blobs.size() - 1;
    };
    auto find_blob = [&](const std::string& name, int* idx) -> int {
        auto it = blob_of.find(name);
        if (it == blob_of.end()) return fail(DABNN_ERR_NOT_FOUND, "Key " + name + " not found.");  // StrKeyMap.h:59-65
        *idx = it->second;
        return DABNN_OK;
    };
    auto find_tensor = [&](const std::string& name, const TensorInfo** t) -> int {
        auto it = tensors.find(name);
        if (it == tensors.end()) return fail(DABNN_ERR_NOT_FOUND, "Key " + name + " not found.");
        *t = &it->second;
        return DABNN_OK;
    };
    input_blob = new_blob(input_name, in_h, in_w, in_c);

    // ---- 1. literal layer-by-layer op list with reference aliasing -------------------------------
    struct LOp { Op op; LayerType type; };
    std::vector<LOp> lops;
    for (const auto& L : layers) {
        Op op{};
        int rc;
        auto sym2 = [&](const std::vector<int32_t>& v, const char* what, int* a0, int* a1) -> int {
            // pads: 2 values or 4 symmetric ones; strides likewise (net.cpp:148-155)
            DABNN_REQUIRE(v.size() == 2 || (v.size() == 4 && v[0] == v[2] && v[1] == v[3]), DABNN_ERR_SHAPE,
                          std::string(what) + " must have 2 entries or 4 symmetric ones");
            *a0 = v[0]; *a1 = v[1];
            return DABNN_OK;
        };
        switch (L.type) {
            case LayerType::FpConv2D:
            case LayerType::BinConv2D: {
                const bool bin = L.type == LayerType::BinConv2D;
                if ((rc = find_blob(L.input, &op.in))) return rc;
                if ((rc = find_tensor(L.weight, &op.w))) return rc;
                DABNN_REQUIRE(op.w->shape.size() == 4 && op.w->is_bit == bin, DABNN_ERR_FORMAT,
                              "conv weight " + L.weight + " has the wrong type or rank");
                if (!L.bias.empty() && !bin) {
                    if ((rc = find_tensor(L.bias, &op.bias))) return rc;
                    DABNN_REQUIRE(!op.bias->is_bit && op.bias->count == op.w->shape[0], DABNN_ERR_FORMAT,
                                  "conv bias " + L.bias + " must hold one float per output channel");
                }
                if ((rc = sym2(L.pads, "pads", &op.pad_h, &op.pad_w))) return rc;
                if ((rc = sym2(L.strides, "strides", &op.stride_h, &op.stride_w))) return rc;
                DABNN_REQUIRE(op.stride_h > 0 && op.stride_w > 0 && op.pad_h >= 0 && op.pad_w >= 0, DABNN_ERR_SHAPE,
                              "conv: bad pads/strides");
                for (int d : L.dilations) DABNN_REQUIRE(d == 1, DABNN_ERR_UNSUPPORTED, "conv: dilation must be 1");
                const Blob ib = blobs[op.in];
                const int cout = op.w->shape[0];
                op.kh = op.w->shape[1]; op.kw = op.w->shape[2];
                DABNN_REQUIRE(cout > 0 && op.kh > 0 && op.kw > 0 && op.kh < 256 && op.kw < 256, DABNN_ERR_FORMAT,
                              "conv weight " + L.weight + ": output channels and kernel size must be positive (kernel below 256)");
                DABNN_REQUIRE((int)op.w->shape[3] == ib.c, DABNN_ERR_SHAPE, "conv: weight channels != input channels");
                const int oh = conv_out_dim(ib.h, op.pad_h, 1, op.kh, op.stride_h);
                const int ow = conv_out_dim(ib.w, op.pad_w, 1, op.kw, op.stride_w);
                DABNN_REQUIRE(oh > 0 && ow > 0, DABNN_ERR_SHAPE, "conv: empty output");
                op.out = blob_of.count(L.output) ? blob_of[L.output] : new_blob(L.output, oh, ow, cout);
                if (bin) {
                    DABNN_REQUIRE(op.w->count % cout == 0, DABNN_ERR_SHAPE, "weight_mat->total() % m == 0 is not satisfied!");
                    const size_t per = op.w->count / cout;
                    if (ib.c % 64 == 0) {
                        // cin == 64: the reference requires pack_mat (c % 64 == 0) - satisfied
                        DABNN_REQUIRE(per >= (size_t)op.kh * op.kw * (ib.c / 64), DABNN_ERR_SHAPE, "binconv: filter too short");
                        op.kind = OpKind::BConvBlock;
                    } else {
                        DABNN_REQUIRE(per == ((size_t)op.kh * op.kw * ib.c + 127) / 128 * 2, DABNN_ERR_SHAPE,
                                      "binconv: filters must be packed in 128-bit padded rows");
                        op.kind = OpKind::BinConvIm2col;
                    }
                    op.cls = "Bin Conv";
                } else {
                    if (!run_fconv) continue;  // net.cpp:157
                    DABNN_REQUIRE(op.w->count == (size_t)cout * op.kh * op.kw * ib.c, DABNN_ERR_FORMAT, "fconv: weight size");
                    op.kind = OpKind::FConv;
                    op.cls = "Float Conv";
                }
                break;
            }
            case LayerType::Affine: {
                if ((rc = find_blob(L.input, &op.in))) return rc;
                if ((rc = find_tensor(L.a, &op.a))) return rc;
                if ((rc = find_tensor(L.b, &op.b))) return rc;
                DABNN_REQUIRE(!op.a->is_bit && !op.b->is_bit, DABNN_ERR_FORMAT, "affine: coefficients must be float tensors");
                DABNN_REQUIRE((int)op.a->count == blobs[op.in].c && (int)op.b->count == blobs[op.in].c, DABNN_ERR_SHAPE,
                              "affine: coefficient length != channels");
                blob_of[L.output] = op.in;  // in place (ADD_INPLACE_LAYER)
                op.out = op.in; op.kind = OpKind::Chain; op.cls = "Affine";
                break;
            }
            case LayerType::Add: {
                if ((rc = find_blob(L.input, &op.in))) return rc;
                if ((rc = find_blob(L.input2, &op.in2))) return rc;
                const Blob x = blobs[op.in], y = blobs[op.in2];
                DABNN_REQUIRE(x.h == y.h && x.w == y.w && x.c == y.c, DABNN_ERR_SHAPE, "add: shapes differ");
                blob_of[L.output] = op.in;
                op.out = op.in; op.kind = OpKind::Chain; op.cls = "Add";
                break;
            }
            case LayerType::Relu: {
                if ((rc = find_blob(L.input, &op.in))) return rc;
                blob_of[L.output] = op.in;
                op.out = op.in; op.relu = 1; op.kind = OpKind::Chain; op.cls = "Relu";
                break;
            }
            case LayerType::PRelu: {
                if ((rc = find_blob(L.input, &op.in))) return rc;
                if ((rc = find_tensor(L.slope, &op.slope))) return rc;
                DABNN_REQUIRE(!op.slope->is_bit, DABNN_ERR_FORMAT, "prelu: slope must be a float tensor");
                DABNN_REQUIRE(op.slope->count == 1 || (int)op.slope->count == blobs[op.in].c, DABNN_ERR_SHAPE,
                              "slope must have size 1 or input.channels");  // PRelu.cpp:7-9
                blob_of[L.output] = op.in;
                op.out = op.in; op.kind = OpKind::PRelu; op.cls = "PRelu";
                break;
            }
            case LayerType::MaxPool:
            case LayerType::AvePool: {
                if ((rc = find_blob(L.input, &op.in))) return rc;
                DABNN_REQUIRE(L.kernel.size() == 2 && L.pads.size() >= 2 && L.strides.size() >= 2, DABNN_ERR_SHAPE,
                              "pool: kernel_shape/pads/strides");
                op.kh = L.kernel[0]; op.kw = L.kernel[1]; op.pad_h = L.pads[0]; op.pad_w = L.pads[1];
                op.stride_h = L.strides[0]; op.stride_w = L.strides[1];
                const Blob ib = blobs[op.in];
                DABNN_REQUIRE(op.kh > 0 && op.kw > 0 && op.stride_h > 0 && op.stride_w > 0, DABNN_ERR_UNSUPPORTED,
                              "pool: global pooling must be given as an explicit kernel");
                const int oh = (ib.h + 2 * op.pad_h - op.kh) / op.stride_h + 1, ow = (ib.w + 2 * op.pad_w - op.kw) / op.stride_w + 1;
                DABNN_REQUIRE(oh > 0 && ow > 0, DABNN_ERR_SHAPE, "pool: empty output");
                op.out = blob_of.count(L.output) ? blob_of[L.output] : new_blob(L.output, oh, ow, ib.c);
                op.kind = L.type == LayerType::MaxPool ? OpKind::MaxPool : OpKind::AvePool;
                op.cls = L.type == LayerType::MaxPool ? "MaxPool" : "AvePool";
                break;
            }
            case LayerType::Concat: {
                if ((rc = find_blob(L.input, &op.in))) return rc;
                if ((rc = find_blob(L.input2, &op.in2))) return rc;
                const Blob x = blobs[op.in], y = blobs[op.in2];
                DABNN_REQUIRE(x.h == y.h && x.w == y.w, DABNN_ERR_SHAPE, "Wrong input for concat");
                op.out = blob_of.count(L.output) ? blob_of[L.output] : new_blob(L.output, x.h, x.w, x.c + y.c);
                op.kind = OpKind::Concat; op.cls = "Concat";
                break;
            }
            case LayerType::FC: {  // extension: the reference runtime has no FC handler (net.cpp:263)
                if ((rc = find_blob(L.input, &op.in))) return rc;
                if ((rc = find_tensor(L.weight, &op.w))) return rc;
                const Blob ib = blobs[op.in];
                DABNN_REQUIRE(!op.w->is_bit && op.w->shape.size() == 2 && op.w->shape[1] == ib.per_image() &&
                                  op.w->count == (size_t)op.w->shape[0] * ib.per_image(), DABNN_ERR_SHAPE,
                              "fc: weight must be [units][input_size]");
                if (!L.bias.empty()) {
                    if ((rc = find_tensor(L.bias, &op.bias))) return rc;
                    DABNN_REQUIRE(!op.bias->is_bit && op.bias->count == op.w->shape[0], DABNN_ERR_FORMAT,
                                  "fc bias " + L.bias + " must hold one float per unit");
                }
                op.kh = ib.h; op.kw = ib.w;  // a full-size "valid" convolution
                op.out = blob_of.count(L.output) ? blob_of[L.output] : new_blob(L.output, 1, 1, op.w->shape[0]);
                op.kind = OpKind::FConv; op.cls = "FC";
                break;
            }
            case LayerType::Binarize: {  // extension: exposes the sign bits of a blob (Binarize.cpp:9)
                if ((rc = find_blob(L.input, &op.in))) return rc;
                DABNN_REQUIRE(blobs[op.in].c % 64 == 0, DABNN_ERR_SHAPE, "float_mat.c % 64 == 0 is not satisfied!");
                blob_of[L.output] = op.in;
                bit_names[L.output] = op.in;
                blobs[op.in].keep_bits = true;
                op.out = op.in; op.kind = OpKind::Pack; op.cls = "Binarize";
                break;
            }
            default:
                return fail(DABNN_ERR_UNSUPPORTED, std::string("Not supported op ") + layer_type_name(L.type));  // net.cpp:264
        }
        lops.push_back({op, L.type});
    }

    // network outputs: blobs that no op reads
    {
        std::vector<char> read(blobs.size(), 0);
        for (const auto& lo : lops) {
            const Op& o = lo.op;
            if (o.kind == OpKind::Chain || o.kind == OpKind::PRelu || o.kind == OpKind::Pack) {
                if (o.in2 >= 0) read[o.in2] = 1;
            } else {
                if (o.in >= 0) read[o.in] = 1;
                if (o.in2 >= 0) read[o.in2] = 1;
            }
        }
        for (const auto& kv : blob_of)
            if (!read[kv.second] && kv.second != input_blob) blobs[kv.second].keep = true;
        // report the last name given to each output blob (in-place layers rename blobs)
        for (size_t i = 0; i < blobs.size(); i++) {
            if (!blobs[i].keep) continue;
            std::string last;
            for (const auto& L : layers)
                if (!L.output.empty() && blob_of.count(L.output) && blob_of[L.output] == (int)i) last = L.output;
            if (!last.empty()) outputs.push_back(last);
        }
    }

    // ---- 2. plan ------------------------------------------------------------------------------------
    if (!optimize) {
        for (auto& lo : lops) {
            Op o = lo.op;
            if (o.kind == OpKind::BConvBlock) {  // literal: pack_mat, then the convolution
                Op pk{}; pk.kind = OpKind::Pack; pk.in = pk.out = o.in; pk.cls = "Bin Conv";
                plan.push_back(pk);
                blobs[o.in].need_bits = true;
            }
            if (o.kind == OpKind::Pack) blobs[o.in].need_bits = true;
            plan.push_back(o);
        }
        for (auto& b : blobs) b.keep = true;
    } else {
        // which op index consumes each blob, to decide what can be fused
        const int nl = (int)lops.size();
        std::vector<char> used(nl, 0);
        // A block whose Add comes later in the file (Bi-Real's stride-2 blocks: BinConv, Affine, then the
        // downsample branch AvePool / FpConv / Affine, then Add) is held back until that Add, so that the
        // shortcut is added in the block's own epilogue.  Legal when nothing in between touches the block's
        // output or overwrites its input; the sum itself is the same two operands either way.
        Op held{};
        int held_until = -1;
        for (int i = 0; i < nl; i++) {
            if (i == held_until) {
                held.in2 = lops[i].op.in2;
                plan.push_back(held);
                held_until = -1;
                continue;
            }
            if (used[i]) continue;
            Op o = lops[i].op;
            used[i] = 1;
            int j = i + 1;
            auto next_is = [&](LayerType t) {
                return j < nl && !used[j] && lops[j].type == t && lops[j].op.in == o.out &&
                       (lops[j].op.kind == OpKind::Chain);
            };
            if (o.kind == OpKind::BConvBlock) {
                if (next_is(LayerType::Affine)) { o.a = lops[j].op.a; o.b = lops[j].op.b; used[j++] = 1; }
                o.cls = "Bin Conv block";
                if (next_is(LayerType::Add) && lops[j].op.in2 != o.out) {
                    o.in2 = lops[j].op.in2;
                    used[j++] = 1;
                } else if (held_until < 0) {
                    for (int k = j; k < nl; k++) {
                        const Op& q = lops[k].op;
                        if (used[k]) break;
                        if (lops[k].type == LayerType::Add && q.kind == OpKind::Chain && q.in == o.out && q.in2 != o.out) {
                            held = o;
                            held_until = k;
                            used[k] = 1;
                            break;
                        }
                        if (q.in == o.out || q.in2 == o.out || q.out == o.out || q.out == o.in) break;   // not independent
                    }
                    if (held_until >= 0) continue;   // emitted when the loop reaches the Add
                }
            } else if (o.kind == OpKind::FConv && lops[i].type == LayerType::FpConv2D) {
                if (next_is(LayerType::Affine)) { o.a = lops[j].op.a; o.b = lops[j].op.b; used[j++] = 1; }
                if (next_is(LayerType::Relu)) { o.relu = 1; used[j++] = 1; }
                // A ResNet stem: the 3x3 stride-2 pad-1 max pooling that is the convolution's only reader happens in the
                // convolution's epilogue, and the convolution's own output is never materialised.
                if (j < nl && !used[j] && lops[j].type == LayerType::MaxPool && lops[j].op.in == o.out && !blobs[o.out].keep) {
                    const Op& mp = lops[j].op;
                    int readers = 0;
                    for (int k = i + 1; k < nl; k++)
                        if (!used[k] && (lops[k].op.in == o.out || lops[k].op.in2 == o.out || (k != j && lops[k].op.out == o.out))) readers++;
                    const Blob& ib = blobs[o.in];
                    if (readers == 1 && mp.kh == 3 && mp.kw == 3 && mp.stride_h == 2 && mp.stride_w == 2 && mp.pad_h == 1 && mp.pad_w == 1 &&
                        fconv_pool_supported(max_batch, ib.h, ib.w, ib.c, blobs[o.out].c, o.kh, o.kw, o.pad_h, o.pad_w, o.stride_h, o.stride_w)) {
                        o.kind = OpKind::FConvPool;
                        o.out = mp.out;
                        used[j++] = 1;
                    }
                }
            } else if (o.kind == OpKind::Chain) {
                // merge a run of in-place elementwise layers on the same blob, in reference order:
                // affine -> add -> relu is the only order one pass can express
                int stage = lops[i].type == LayerType::Affine ? 0 : lops[i].type == LayerType::Add ? 1 : 2;
                while (j < nl && !used[j] && lops[j].op.kind == OpKind::Chain && lops[j].op.in == o.out) {
                    const int st = lops[j].type == LayerType::Affine ? 0 : lops[j].type == LayerType::Add ? 1 : 2;
                    if (st <= stage || (st == 1 && lops[j].op.in2 == o.out)) break;
                    if (st == 0) { o.a = lops[j].op.a; o.b = lops[j].op.b; }
                    if (st == 1) o.in2 = lops[j].op.in2;
                    if (st == 2) o.relu = 1;
                    stage = st;
                    used[j++] = 1;
                }
                o.cls = "Elementwise";
            }
            plan.push_back(o);
        }
        // sign bits: every blob read by a BConvBlock needs bits; let its producer emit them
        for (auto& o : plan)
            if (o.kind == OpKind::BConvBlock || o.kind == OpKind::Pack) blobs[o.in].need_bits = true;
        // A blob keeps its signs as {0,1} bytes when every reader is a binary convolution that the byte-activation
        // engine takes (the Binarize layer exposes packed words, so a blob it reads stays packed).
        if (engine == DABNN_ENGINE_AUTO || engine == DABNN_ENGINE_TCGEN05) {
            std::vector<char> can(blobs.size(), 1);
            for (auto& o : plan) {
                if (o.kind == OpKind::Pack) can[o.in] = 0;
                if (o.kind == OpKind::BConvBlock &&
                    !bconv_u8_supported(max_batch, blobs[o.in].h, blobs[o.in].w, blobs[o.in].c, blobs[o.out].c, o.kh, o.kw,
                                        o.pad_h, o.pad_w, o.stride_h, o.stride_w))
                    can[o.in] = 0;
            }
            for (size_t i = 0; i < blobs.size(); i++) blobs[i].u8 = blobs[i].need_bits && can[i];
            for (auto& o : plan)
                if (o.kind == OpKind::BConvBlock) o.u8 = blobs[o.in].u8;
        }
        std::vector<Op> with_packs;
        std::vector<char> bits_ready(blobs.size(), 0);
        for (auto& o : plan) {
            if (o.kind == OpKind::BConvBlock && !bits_ready[o.in]) {
                Op pk{}; pk.kind = OpKind::Pack; pk.in = pk.out = o.in; pk.cls = "Binarize";
                with_packs.push_back(pk);
                bits_ready[o.in] = 1;
            }
            if (o.kind == OpKind::Pack) {   // a Binarize layer of the model: skipped when the blob's writer already emitted the bits
                if (bits_ready[o.in]) continue;
                bits_ready[o.in] = 1;
            }
            if (o.out >= 0 && o.kind != OpKind::Pack) {
                bool emits = false;
                if (blobs[o.out].need_bits && blobs[o.out].c % 64 == 0 &&
                    (o.kind == OpKind::BConvBlock || o.kind == OpKind::Chain || o.kind == OpKind::MaxPool || o.kind == OpKind::FConvPool)) {
                    // only the blob's last writer emits the bits: an in-place writer later in the
                    // plan would change the values
                    bool later_writer = false, seen = false;
                    for (auto& q : plan) {
                        if (&q == &o) { seen = true; continue; }
                        if (seen && q.out == o.out && q.kind != OpKind::Pack) later_writer = true;
                    }
                    emits = !later_writer && !blobs[o.out].keep_bits;   // a Binarize layer's bits are packed where the layer stands
                    // bytes are written by the byte-activation engine and the max pool; any other producer is followed by a Pack
                    if (blobs[o.out].u8 && !((o.kind == OpKind::BConvBlock && o.u8) || o.kind == OpKind::MaxPool || o.kind == OpKind::FConvPool)) emits = false;
                    if (o.kind == OpKind::FConvPool && !blobs[o.out].u8) emits = false;   // the fused kernel writes sign bytes, not packed words
                }
                o.write_bits = emits;
                bits_ready[o.out] = emits;
            }
            with_packs.push_back(o);
        }
        plan.swap(with_packs);
        // A 2x2 stride-2 average pooling (the downsample shortcut of a ResNet stage) whose input was last written by a
        // fused binary block that the halo kernel takes is computed in that block's epilogue, from the tile still in
        // shared memory: same four operands in the same order, so the same bits, and the block's output is not re-read.
        for (size_t k = 0; k < plan.size(); k++) {
            const Op& q = plan[k];
            if (q.kind != OpKind::AvePool || q.kh != 2 || q.kw != 2 || q.stride_h != 2 || q.stride_w != 2 || q.pad_h || q.pad_w) continue;
            int writer = -1;
            bool clean = true;
            for (size_t i = 0; i < k; i++) {
                if (plan[i].kind != OpKind::Pack && plan[i].out == q.in) writer = (int)i;
                if (plan[i].in == q.out || plan[i].in2 == q.out || plan[i].out == q.out || plan[i].out2 == q.out) clean = false;
            }
            if (writer < 0 || !clean) continue;
            Op& o = plan[writer];
            const Blob& ib = blobs[o.in];
            if (o.kind != OpKind::BConvBlock || !o.u8 || o.out2 >= 0 ||
                !bconv_u8_pool_supported(max_batch, ib.h, ib.w, ib.c, blobs[o.out].c, o.kh, o.kw, o.pad_h, o.pad_w, o.stride_h, o.stride_w))
                continue;
            o.out2 = q.out;
            plan.erase(plan.begin() + k);
            k--;
        }
    }

    // ---- 3. lifetimes and arena layout ------------------------------------------------------------
    for (int i = 0; i < (int)plan.size(); i++) {
        const Op& o = plan[i];
        auto touch = [&](int b) {
            if (b < 0) return;
            if (blobs[b].def_op < 0) blobs[b].def_op = i;
            blobs[b].last_use = i;
        };
        touch(o.in); touch(o.in2); touch(o.out); touch(o.out2);
    }
    blobs[input_blob].def_op = 0;
    if (blobs[input_blob].last_use < 0) blobs[input_blob].last_use = 0;
    struct Item { int blob; bool is_bits; size_t bytes; int a, b; size_t off; };
    std::vector<Item> items;
    for (int i = 0; i < (int)blobs.size(); i++) {
        const Blob& b = blobs[i];
        if (b.def_op < 0) continue;
        const int last = b.keep ? (int)plan.size() : b.last_use;
        if (i == input_blob && !b.need_bits) continue;   // read in place (device input or staging buffer)
        const size_t fbytes = ((size_t)max_batch * b.per_image() * 4 + 255) / 256 * 256;
        // a kept blob holds the whole batch across sub-batch executions of the plan, so its memory
        // is never shared with another blob
        const int first = b.keep ? 0 : b.def_op;
        if (i != input_blob) items.push_back({i, false, fbytes, first, last, 0});
        if (b.need_bits) {
            const size_t bb = ((size_t)max_batch * b.h * b.w * (b.u8 ? b.c : b.c / 64 * 8) + 255) / 256 * 256;
            items.push_back({i, true, bb, b.keep_bits ? 0 : first, b.keep_bits ? (int)plan.size() : last, 0});
        }
    }
    // BinConvIm2col scratch: one shared region sized for the largest user
    size_t scratch = 0;
    for (const auto& o : plan)
        if (o.kind == OpKind::BinConvIm2col) {
            const Blob& ib = blobs[o.in];
            scratch = std::max(scratch, dabnn_binconv_workspace_bytes(max_batch, ib.h, ib.w, ib.c, o.kh, o.kw, o.pad_h,
                                                                      o.pad_w, o.stride_h, o.stride_w));
        }
    // greedy first-fit by decreasing size; lifetimes [a, b] inclusive
    std::vector<int> order(items.size());
    for (size_t i = 0; i < order.size(); i++) order[i] = (int)i;
    std::sort(order.begin(), order.end(), [&](int x, int y) { return items[x].bytes > items[y].bytes; });
    std::vector<int> placed;
    size_t top = (scratch + 255) / 256 * 256;
    for (int idx : order) {
        Item& it = items[idx];
        std::vector<std::pair<size_t, size_t>> busy;
        for (int p : placed) {
            const Item& q = items[p];
            if (q.a <= it.b && it.a <= q.b) busy.push_back({q.off, q.off + q.bytes});
        }
        std::sort(busy.begin(), busy.end());
        size_t off = (scratch + 255) / 256 * 256;
        for (auto& iv : busy) {
            if (off + it.bytes <= iv.first) break;
            off = std::max(off, iv.second);
        }
        it.off = off;
        top = std::max(top, off + it.bytes);
        placed.push_back(idx);
    }
    for (const auto& it : items) (it.is_bits ? blobs[it.blob].bits_off : blobs[it.blob].f32_off) = it.off;
    arena_bytes = top;
    if (cudaMalloc(&arena, arena_bytes ? arena_bytes : 256) != cudaSuccess) {
        cudaGetLastError();
        return fail(DABNN_ERR_OOM, "cannot allocate a " + std::to_string(arena_bytes) + " byte device arena");
    }
    {   // double-buffered staging for host inputs
        const size_t sb = (size_t)std::min(max_batch, host_chunk) * in_h * in_w * in_c * sizeof(float);
        DABNN_CUDA_OK(cudaStreamCreateWithFlags(&copy_stream, cudaStreamNonBlocking));
        for (int i = 0; i < 2; i++) {
            if (cudaMalloc(&staging[i], sb) != cudaSuccess) {
                cudaGetLastError();
                return fail(DABNN_ERR_OOM, "cannot allocate the input staging buffers");
            }
            DABNN_CUDA_OK(cudaEventCreateWithFlags(&copied[i], cudaEventDisableTiming));
            DABNN_CUDA_OK(cudaEventCreateWithFlags(&consumed[i], cudaEventDisableTiming));
        }
        arena_bytes_extra = 2 * sb;
    }
    if (engine == DABNN_ENGINE_AUTO || engine == DABNN_ENGINE_TCGEN05) {
        // the weights never change: expand them to the tensor-core engine's byte layout once, not once per pixel tile
        std::vector<size_t> offs;
        for (const Op& o : plan) {
            if (o.kind != OpKind::BConvBlock) continue;
            offs.push_back(expanded_bytes);
            const int kwords = o.kh * o.kw * (blobs[o.in].c / 64);
            expanded_bytes += ((o.u8 ? bconv_u8_weight_bytes(blobs[o.out].c, kwords) : bconv_expanded_weight_bytes(blobs[o.out].c, kwords)) + 255) / 256 * 256;
        }
        if (expanded_bytes) {
            if (cudaMalloc(&expanded, expanded_bytes) != cudaSuccess) {
                cudaGetLastError();
                return fail(DABNN_ERR_OOM, "cannot allocate the expanded binary weights");
            }
            size_t k = 0;
            for (Op& o : plan) {
                if (o.kind != OpKind::BConvBlock) continue;
                unsigned char* dst = expanded + offs[k++];
                const int kwords = o.kh * o.kw * (blobs[o.in].c / 64);
                const int rc = o.u8 ? bconv_u8_expand_weights(static_cast<const uint64_t*>(o.w->dev), o.w->count, blobs[o.out].c, kwords, dst, stream)
                                    : bconv_expand_weights(static_cast<const uint64_t*>(o.w->dev), o.w->count, blobs[o.out].c, kwords, dst, stream);
                if (rc) return rc;
                o.w_expanded = dst;
            }
            DABNN_CUDA_OK(cudaStreamSynchronize(stream));
        }
    }
    if (optimize) {
        // 1x1 float convolutions run as a TMA-fed GEMM whose tensor core wants x = head + remainder of both operands: the
        // weights' remainders are constants, computed here once instead of once per pixel tile
        std::vector<size_t> offs;
        for (const Op& o : plan) {
            if (o.kind != OpKind::FConv || !fconv_uses_weight_remainders(blobs[o.in].c, blobs[o.out].c, o.kh, o.kw, o.pad_h, o.pad_w, o.stride_h, o.stride_w)) continue;
            offs.push_back(remainders_bytes);
            remainders_bytes += (o.w->count * sizeof(float) + 255) / 256 * 256;
        }
        if (remainders_bytes) {
            if (cudaMalloc(&remainders, remainders_bytes) != cudaSuccess) {
                cudaGetLastError();
                return fail(DABNN_ERR_OOM, "cannot allocate the float convolutions' weight remainders");
            }
            size_t k = 0;
            for (Op& o : plan) {
                if (o.kind != OpKind::FConv || !fconv_uses_weight_remainders(blobs[o.in].c, blobs[o.out].c, o.kh, o.kw, o.pad_h, o.pad_w, o.stride_h, o.stride_w)) continue;
                float* dst = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(remainders) + offs[k++]);
                const int rc = fconv_split_weights(static_cast<const float*>(o.w->dev), dst, o.w->count, stream);
                if (rc) return rc;
                o.w_rem = dst;
            }
            DABNN_CUDA_OK(cudaStreamSynchronize(stream));
        }
    }
    if (profiling) {
        events.resize(plan.size() + 1);
        for (auto& e : events) DABNN_CUDA_OK(cudaEventCreate(&e));
    }
    {   // where the kernels report a wait that gave up, and the host-visible word run_plan's last launch copies it to
        int rc;
        if ((rc = contraction_status_word(&status_words[0]))) return rc;
        if ((rc = fconv_status_word(&status_words[1]))) return rc;
        if ((rc = bconv_u8_status_word(&status_words[2]))) return rc;
        int* host = nullptr;
        DABNN_CUDA_OK(cudaHostAlloc(&host, 64, cudaHostAllocMapped));
        *host = 0;
        status_host = host;
        DABNN_CUDA_OK(cudaHostGetDevicePointer(&status_dev, host, 0));
    }
    loaded = true;
    return DABNN_OK;
}

int NetImpl::check_status() {
    if (!status_host) return DABNN_OK;
    const int code = *status_host;
    if (!code) return DABNN_OK;
    *status_host = 0;
    return fail(DABNN_ERR_TIMEOUT, "a bounded wait inside a tensor-core kernel gave up (code " + std::to_string(code) +
                                       "): the results of the runs in flight are incomplete");
}

// -------------------------------------------------------------------------------------------------
int NetImpl::run(const float* input, int batch, bool is_device) {
    DABNN_REQUIRE(loaded, DABNN_ERR_STATE, "run: no model has been read");
    DABNN_REQUIRE(input, DABNN_ERR_ARG, "run: null input");
    DABNN_REQUIRE(batch >= 1 && batch <= max_batch, DABNN_ERR_ARG,
                  "run: batch must be between 1 and the configured max_batch");
    DABNN_CUDA_OK(cudaSetDevice(device));
    cur_batch = batch;
    const size_t img_floats = (size_t)in_h * in_w * in_c;
    if (is_device) {
        cur_input = input;
        out_offset = 0;
        return run_plan_graphed(batch);
    }
    // host input: sub-batches through two staging buffers; the copy of sub-batch k+1 is issued
    // before the kernels of sub-batch k so that PCIe transfer and compute overlap
    const int chunk = std::min(max_batch, host_chunk);
    const int nchunks = (batch + chunk - 1) / chunk;
    const size_t seq0 = chunk_seq;
    chunk_seq += nchunks;
    auto issue_copy = [&](int k) -> int {
        const int i0 = k * chunk, cnt = std::min(chunk, batch - i0), sb = (int)((seq0 + k) & 1);
        // the buffer's last reader: sub-batch k - 2 of this run, or the matching sub-batch of the previous run
        // (a wait on an event that was never recorded returns at once)
        DABNN_CUDA_OK(cudaStreamWaitEvent(copy_stream, consumed[sb], 0));
        DABNN_CUDA_OK(cudaMemcpyAsync(staging[sb], input + (size_t)i0 * img_floats, (size_t)cnt * img_floats * sizeof(float),
                                      cudaMemcpyHostToDevice, copy_stream));
        DABNN_CUDA_OK(cudaEventRecord(copied[sb], copy_stream));
        return DABNN_OK;
    };
    // Nothing here waits for the previous run as a whole: its last sub-batches still compute while this
    // run's first copies cross PCIe, which is what lets back-to-back submissions overlap.
    int rc = issue_copy(0);
    for (int k = 0; k < nchunks && rc == DABNN_OK; k++) {
        if (k + 1 < nchunks) rc = issue_copy(k + 1);
        if (rc) break;
        const int i0 = k * chunk, cnt = std::min(chunk, batch - i0), sb = (int)((seq0 + k) & 1);
        DABNN_CUDA_OK(cudaStreamWaitEvent(stream, copied[sb], 0));
        cur_input = staging[sb];
        out_offset = (size_t)i0;
        rc = run_plan_graphed(cnt);
        DABNN_CUDA_OK(cudaEventRecord(consumed[sb], stream));
    }
    out_offset = 0;
    return rc;
}

int NetImpl::run_plan_graphed(int batch) {
    if (!use_graphs || profiling) return run_plan(batch);
    PlanGraph* g = nullptr;
    for (auto& c : graphs)
        if (c.batch == batch && c.input == cur_input && c.out_offset == out_offset) g = &c;
    if (g && g->exec) {
        DABNN_CUDA_OK(cudaGraphLaunch(g->exec, stream));
        return DABNN_OK;
    }
    if (!g) {   // first use of this key: run eagerly (this also performs the kernels' one-time attribute set-up)
        if (graphs.size() >= kMaxGraphs) {   // callers that keep changing pointers: forget the oldest
            if (graphs.front().exec) cudaGraphExecDestroy(graphs.front().exec);
            graphs.erase(graphs.begin());
        }
        graphs.push_back(PlanGraph{batch, cur_input, out_offset, nullptr});
        return run_plan(batch);
    }
    // second use: capture the same launches instead of running them, then replay
    if (cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
        cudaGetLastError();
        use_graphs = false;
        return run_plan(batch);
    }
    const int rc = run_plan(batch);
    cudaGraph_t graph = nullptr;
    const cudaError_t end = cudaStreamEndCapture(stream, &graph);
    if (rc != DABNN_OK || end != cudaSuccess || !graph) {
        cudaGetLastError();
        if (graph) cudaGraphDestroy(graph);
        use_graphs = false;
        return rc != DABNN_OK ? rc : run_plan(batch);
    }
    cudaGraphExec_t exec = nullptr;
    const cudaError_t inst = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (inst != cudaSuccess || !exec) {
        cudaGetLastError();
        use_graphs = false;
        return run_plan(batch);
    }
    g->exec = exec;
    DABNN_CUDA_OK(cudaGraphLaunch(exec, stream));
    return DABNN_OK;
}

int NetImpl::run_plan(int batch) {
    const int eng = optimize ? engine : DABNN_ENGINE_POPC;
    int rc = DABNN_OK;
    for (size_t i = 0; i < plan.size() && rc == DABNN_OK; i++) {
        const Op& o = plan[i];
        if (profiling && !events.empty()) cudaEventRecord(events[i], stream);
        const Blob& ib = blobs[o.in];
        const size_t pixels_in = (size_t)batch * ib.h * ib.w;
        switch (o.kind) {
            case OpKind::Pack:
                rc = ib.u8 ? binarize_u8_impl(f32(o.in), bytes(o.in), pixels_in * ib.c, stream)
                           : dabnn_pack_64(f32(o.in), bits(o.in), pixels_in * ib.c, stream);
                break;
            case OpKind::BConvBlock: {
                const Blob& ob = blobs[o.out];
                if (o.u8) {
                    rc = bconv_u8_block_impl(bytes(o.in), o.w_expanded, o.a ? static_cast<const float*>(o.a->dev) : nullptr,
                                             o.b ? static_cast<const float*>(o.b->dev) : nullptr,
                                             o.in2 >= 0 ? f32(o.in2) : nullptr, f32(o.out),
                                             o.write_bits && ob.u8 ? bytes(o.out) : nullptr,
                                             o.write_bits && !ob.u8 ? bits(o.out) : nullptr, batch, ib.h, ib.w, ib.c, ob.c, o.kh,
                                             o.kw, o.pad_h, o.pad_w, o.stride_h, o.stride_w, stream, o.out2 >= 0 ? f32(o.out2) : nullptr);
                    break;
                }
                rc = bconv_block_impl(bits(o.in), static_cast<const uint64_t*>(o.w->dev), o.w->count,
                                      o.a ? static_cast<const float*>(o.a->dev) : nullptr,
                                      o.b ? static_cast<const float*>(o.b->dev) : nullptr,
                                      o.in2 >= 0 ? f32(o.in2) : nullptr, f32(o.out),
                                      o.write_bits ? bits(o.out) : nullptr, batch, ib.h, ib.w, ib.c / 64, ob.c, o.kh,
                                      o.kw, o.pad_h, o.pad_w, o.stride_h, o.stride_w, eng, stream, o.w_expanded);
                break;
            }
            case OpKind::BinConvIm2col: {
                const Blob& ob = blobs[o.out];
                rc = dabnn_binconv_forward(f32(o.in), static_cast<const uint64_t*>(o.w->dev), o.w->count, f32(o.out),
                                           batch, ib.h, ib.w, ib.c, ob.c, o.kh, o.kw, o.pad_h, o.pad_w, o.stride_h,
                                           o.stride_w, arena, arena_bytes, eng, stream);
                break;
            }
            case OpKind::FConv: {
                const Blob& ob = blobs[o.out];
                rc = fconv_impl(f32(o.in), static_cast<const float*>(o.w->dev),
                                o.bias ? static_cast<const float*>(o.bias->dev) : nullptr,
                                o.a ? static_cast<const float*>(o.a->dev) : nullptr,
                                o.b ? static_cast<const float*>(o.b->dev) : nullptr, o.relu, f32(o.out), batch, ib.h,
                                ib.w, ib.c, ob.c, o.kh, o.kw, o.pad_h, o.pad_w, o.stride_h, o.stride_w, 1, 1, stream, o.w_rem);
                break;
            }
            case OpKind::FConvPool: {
                const Blob& ob = blobs[o.out];
                rc = fconv_pool_impl(f32(o.in), static_cast<const float*>(o.w->dev),
                                     o.bias ? static_cast<const float*>(o.bias->dev) : nullptr,
                                     o.a ? static_cast<const float*>(o.a->dev) : nullptr,
                                     o.b ? static_cast<const float*>(o.b->dev) : nullptr, o.relu, f32(o.out),
                                     o.write_bits && ob.u8 ? bytes(o.out) : nullptr, batch, ib.h, ib.w, ib.c, ob.c, o.kh, o.kw,
                                     o.pad_h, o.pad_w, o.stride_h, o.stride_w, stream);
                break;
            }
            case OpKind::Chain:
                rc = elementwise_chain(f32(o.in), o.a ? static_cast<const float*>(o.a->dev) : nullptr,
                                       o.b ? static_cast<const float*>(o.b->dev) : nullptr,
                                       o.in2 >= 0 ? f32(o.in2) : nullptr, o.relu, f32(o.out),
                                       o.write_bits ? bits(o.out) : nullptr, pixels_in, ib.c, stream);
                break;
            case OpKind::PRelu:
                rc = dabnn_prelu(f32(o.in), static_cast<const float*>(o.slope->dev), (int)o.slope->count, pixels_in,
                                 ib.c, stream);
                break;
            case OpKind::MaxPool:
                rc = maxpool_impl(f32(o.in), f32(o.out), o.write_bits && !blobs[o.out].u8 ? bits(o.out) : nullptr, batch, ib.h,
                                  ib.w, ib.c, o.kh, o.kw, o.pad_h, o.pad_w, o.stride_h, o.stride_w, stream,
                                  o.write_bits && blobs[o.out].u8 ? bytes(o.out) : nullptr);
                break;
            case OpKind::AvePool:
                rc = dabnn_avepool(f32(o.in), f32(o.out), batch, ib.h, ib.w, ib.c, o.kh, o.kw, o.pad_h, o.pad_w,
                                   o.stride_h, o.stride_w, stream);
                break;
            case OpKind::Concat:
                rc = dabnn_concat(f32(o.in), ib.c, f32(o.in2), blobs[o.in2].c, f32(o.out), pixels_in, stream);
                break;
        }
    }
    if (profiling && !events.empty()) cudaEventRecord(events[plan.size()], stream);
    if (rc == DABNN_OK && status_dev) {
        status_gather_kernel<<<1, 1, 0, stream>>>(status_words[0], status_words[1], status_words[2], status_dev);
        rc = check_launch("status_gather_kernel");
    }
    return rc;
}

}  // namespace dabnn

using namespace dabnn;
struct dabnn_net {
    NetImpl impl;
};

extern "C" int dabnn_net_create(dabnn_net** out) {
    DABNN_REQUIRE(out, DABNN_ERR_ARG, "net_create: null pointer");
    *out = nullptr;
    int dev = 0;
    DABNN_CUDA_OK(cudaGetDevice(&dev));
    std::unique_ptr<dabnn_net> n(new dabnn_net());
    n->impl.device = dev;
    DABNN_CUDA_OK(cudaStreamCreateWithFlags(&n->impl.stream, cudaStreamNonBlocking));
    *out = n.release();
    return DABNN_OK;
}
extern "C" void dabnn_net_destroy(dabnn_net* net) { delete net; }

extern "C" int dabnn_net_set_flags(dabnn_net* net, int optimize, int run_fconv, int strict) {
    DABNN_REQUIRE(net, DABNN_ERR_ARG, "null net");
    DABNN_REQUIRE(!net->impl.loaded, DABNN_ERR_STATE, "flags must be set before the model is read");
    net->impl.optimize = optimize != 0; net->impl.run_fconv = run_fconv != 0; net->impl.strict = strict != 0;
    return DABNN_OK;
}
extern "C" int dabnn_net_configure(dabnn_net* net, int max_batch, int engine) {
    DABNN_REQUIRE(net, DABNN_ERR_ARG, "null net");
    DABNN_REQUIRE(!net->impl.loaded, DABNN_ERR_STATE, "configure must precede read");
    DABNN_REQUIRE(max_batch >= 1, DABNN_ERR_ARG, "max_batch must be >= 1");
    DABNN_REQUIRE(engine >= DABNN_ENGINE_AUTO && engine <= DABNN_ENGINE_TCGEN05, DABNN_ERR_ARG, "unknown engine");
    net->impl.max_batch = max_batch; net->impl.engine = engine;
    return DABNN_OK;
}
extern "C" int dabnn_net_set_host_chunk(dabnn_net* net, int images) {
    DABNN_REQUIRE(net, DABNN_ERR_ARG, "null net");
    DABNN_REQUIRE(!net->impl.loaded, DABNN_ERR_STATE, "set_host_chunk must precede read");
    DABNN_REQUIRE(images >= 1, DABNN_ERR_ARG, "host chunk must be >= 1 image");
    net->impl.host_chunk = images;
    return DABNN_OK;
}
extern "C" int dabnn_net_read_buf(dabnn_net* net, const void* buf, size_t len) {
    DABNN_REQUIRE(net, DABNN_ERR_ARG, "null net");
    DABNN_REQUIRE(!net->impl.loaded, DABNN_ERR_STATE, "a model has already been read into this net");
    DABNN_CUDA_OK(cudaSetDevice(net->impl.device));
    try {
        int rc = net->impl.parse(static_cast<const uint8_t*>(buf), len);
        if (rc) return rc;
        return net->impl.build();
    } catch (const std::exception& e) {   // nothing may unwind through the C boundary
        return fail(DABNN_ERR_FORMAT, std::string("read_buf: ") + e.what());
    }
}
extern "C" int dabnn_net_read_file(dabnn_net* net, const char* path) {
    DABNN_REQUIRE(net && path, DABNN_ERR_ARG, "null argument");
    const int fd = open(path, O_RDONLY);
    if (fd == -1) return fail(DABNN_ERR_IO, "Open file error " + std::to_string(errno));  // net.cpp:35
    struct stat st;
    if (fstat(fd, &st) != 0) { close(fd); return fail(DABNN_ERR_IO, "fstat failed, errno = " + std::to_string(errno)); }
    std::vector<uint8_t> data((size_t)st.st_size);
    size_t got = 0;
    while (got < data.size()) {
        const ssize_t r = read(fd, data.data() + got, data.size() - got);
        if (r <= 0) { close(fd); return fail(DABNN_ERR_IO, "read failed, errno = " + std::to_string(errno)); }
        got += (size_t)r;
    }
    close(fd);
    return dabnn_net_read_buf(net, data.data(), data.size());
}
extern "C" int dabnn_net_run(dabnn_net* net, const float* input, int batch, int in_is_device) {
    DABNN_REQUIRE(net, DABNN_ERR_ARG, "null net");
    return net->impl.run(input, batch, in_is_device != 0);
}
extern "C" int dabnn_net_sync(dabnn_net* net) {
    DABNN_REQUIRE(net, DABNN_ERR_ARG, "null net");
    DABNN_CUDA_OK(cudaStreamSynchronize(net->impl.stream));
    return net->impl.check_status();
}
extern "C" int dabnn_net_submit(dabnn_net* net, const float* host_input, int batch, const char* blob, float* host_out,
                                size_t host_floats, int* ticket) {
    DABNN_REQUIRE(net && blob && host_out && ticket, DABNN_ERR_ARG, "null argument");
    NetImpl& n = net->impl;
    DABNN_REQUIRE(n.loaded, DABNN_ERR_STATE, "submit: no model has been read");
    auto it = n.blob_of.find(blob);
    if (it == n.blob_of.end()) return fail(DABNN_ERR_NOT_FOUND, std::string("Key ") + blob + " not found.");
    const Blob& b = n.blobs[it->second];
    DABNN_REQUIRE(b.keep && it->second != n.input_blob, DABNN_ERR_NOT_FOUND, "submit: the blob is not materialised");
    DABNN_REQUIRE(batch >= 1 && host_floats >= (size_t)batch * b.per_image(), DABNN_ERR_ARG, "submit: host buffer too small");
    int rc = n.run(host_input, batch, false);
    if (rc) return rc;
    DABNN_CUDA_OK(cudaMemcpyAsync(host_out, n.f32(it->second), (size_t)batch * b.per_image() * 4, cudaMemcpyDeviceToHost, n.stream));
    const int t = n.next_ticket;
    if (!n.tickets[t]) DABNN_CUDA_OK(cudaEventCreateWithFlags(&n.tickets[t], cudaEventDisableTiming));
    DABNN_CUDA_OK(cudaEventRecord(n.tickets[t], n.stream));
    n.next_ticket = (t + 1) % NetImpl::kTickets;
    *ticket = t;
    return DABNN_OK;
}
extern "C" int dabnn_net_wait(dabnn_net* net, int ticket) {
    DABNN_REQUIRE(net && ticket >= 0 && ticket < NetImpl::kTickets && net->impl.tickets[ticket], DABNN_ERR_ARG, "wait: unknown ticket");
    DABNN_CUDA_OK(cudaEventSynchronize(net->impl.tickets[ticket]));
    return net->impl.check_status();
}
extern "C" int dabnn_net_get_blob(dabnn_net* net, const char* name, int dims[4], const float** device_ptr,
                                  float* to_host, size_t host_floats) {
    DABNN_REQUIRE(net && name, DABNN_ERR_ARG, "null argument");
    NetImpl& n = net->impl;
    DABNN_REQUIRE(n.loaded, DABNN_ERR_STATE, "get_blob: no model has been read");
    auto it = n.blob_of.find(name);
    if (it == n.blob_of.end()) return fail(DABNN_ERR_NOT_FOUND, std::string("Key ") + name + " not found.");
    const Blob& b = n.blobs[it->second];
    if (n.bit_names.count(name))
        return fail(DABNN_ERR_NOT_FOUND, std::string("blob ") + name + " holds packed sign bits (a Binarize output): fetch it with dabnn_net_get_blob_bits");
    if (it->second == n.input_blob)
        return fail(DABNN_ERR_NOT_FOUND, std::string("blob ") + name + " is the caller's input; it is read in place and not kept");
    if (!b.keep)
        return fail(DABNN_ERR_NOT_FOUND, std::string("blob ") + name + " is not materialised in the fused plan; read the model with optimize = 0 to keep every blob");
    const int batch = n.cur_batch > 0 ? n.cur_batch : 1;
    if (dims) { dims[0] = batch; dims[1] = b.h; dims[2] = b.w; dims[3] = b.c; }
    if (device_ptr) *device_ptr = n.f32(it->second);
    if (to_host) {
        const size_t cnt = (size_t)batch * b.per_image();
        DABNN_REQUIRE(host_floats >= cnt, DABNN_ERR_ARG, "get_blob: host buffer too small");
        DABNN_CUDA_OK(cudaMemcpyAsync(to_host, n.f32(it->second), cnt * 4, cudaMemcpyDeviceToHost, n.stream));
        DABNN_CUDA_OK(cudaStreamSynchronize(n.stream));
        return n.check_status();
    }
    return DABNN_OK;
}
extern "C" int dabnn_net_get_blob_bits(dabnn_net* net, const char* name, int dims[4], const uint64_t** device_ptr,
                                       uint64_t* to_host, size_t host_words) {
    DABNN_REQUIRE(net && name, DABNN_ERR_ARG, "null argument");
    NetImpl& n = net->impl;
    DABNN_REQUIRE(n.loaded, DABNN_ERR_STATE, "get_blob_bits: no model has been read");
    auto it = n.bit_names.find(name);
    if (it == n.bit_names.end())
        return fail(DABNN_ERR_NOT_FOUND, std::string("Key ") + name + " not found among the outputs of Binarize layers.");
    const Blob& b = n.blobs[it->second];
    if (!b.keep_bits || !b.need_bits || b.u8 || b.bits_off == (size_t)-1)
        return fail(DABNN_ERR_NOT_FOUND, std::string("blob ") + name + " is consumed inside the fused plan; read the model with optimize = 0 to keep every blob");
    const int batch = n.cur_batch > 0 ? n.cur_batch : 1;
    if (dims) { dims[0] = batch; dims[1] = b.h; dims[2] = b.w; dims[3] = b.c / 64; }
    if (device_ptr) *device_ptr = n.bits(it->second);
    if (to_host) {
        const size_t cnt = (size_t)batch * b.h * b.w * (b.c / 64);
        DABNN_REQUIRE(host_words >= cnt, DABNN_ERR_ARG, "get_blob_bits: host buffer too small");
        DABNN_CUDA_OK(cudaMemcpyAsync(to_host, n.bits(it->second), cnt * 8, cudaMemcpyDeviceToHost, n.stream));
        DABNN_CUDA_OK(cudaStreamSynchronize(n.stream));
        return n.check_status();
    }
    return DABNN_OK;
}
extern "C" const char* dabnn_net_output_name(dabnn_net* net, int i) {
    if (!net || i < 0 || i >= (int)net->impl.outputs.size()) return nullptr;
    return net->impl.outputs[i].c_str();
}
extern "C" dabnn_stream_t dabnn_net_stream(dabnn_net* net) { return net ? net->impl.stream : nullptr; }
extern "C" int dabnn_net_stats(dabnn_net* net, int* kernels_per_run, size_t* arena_bytes) {
    DABNN_REQUIRE(net, DABNN_ERR_ARG, "null net");
    int k = 0;
    for (const auto& o : net->impl.plan) k += o.kind == OpKind::BinConvIm2col ? 2 : 1;
    if (net->impl.status_dev) k += 1;   // the status collector that ends every plan
    if (kernels_per_run) *kernels_per_run = k;
    if (arena_bytes) *arena_bytes = net->impl.arena_bytes + net->impl.weights_bytes + net->impl.arena_bytes_extra + net->impl.expanded_bytes + net->impl.remainders_bytes;
    return DABNN_OK;
}
extern "C" int dabnn_net_set_profiling(dabnn_net* net, int on) {
    DABNN_REQUIRE(net, DABNN_ERR_ARG, "null net");
    NetImpl& n = net->impl;
    n.profiling = on != 0;
    if (n.profiling && n.loaded && n.events.empty()) {
        n.events.resize(n.plan.size() + 1);
        for (auto& e : n.events) DABNN_CUDA_OK(cudaEventCreate(&e));
    }
    return DABNN_OK;
}
extern "C" int dabnn_net_layer_times(dabnn_net* net, const char** names, float* ms, int cap, int* count) {
    DABNN_REQUIRE(net && count, DABNN_ERR_ARG, "null argument");
    NetImpl& n = net->impl;
    DABNN_REQUIRE(n.profiling && !n.events.empty(), DABNN_ERR_STATE, "profiling is off");
    DABNN_CUDA_OK(cudaStreamSynchronize(n.stream));
    std::map<std::string, float> acc;
    for (size_t i = 0; i < n.plan.size(); i++) {
        float t = 0.f;
        DABNN_CUDA_OK(cudaEventElapsedTime(&t, n.events[i], n.events[i + 1]));
        acc[n.plan[i].cls] += t;
    }
    n.time_names.clear(); n.time_ms.clear();
    for (auto& kv : acc) { n.time_names.push_back(kv.first); n.time_ms.push_back(kv.second); }
    *count = (int)n.time_names.size();
    for (int i = 0; i < *count && i < cap; i++) {
        if (names) names[i] = n.time_names[i].c_str();
        if (ms) ms[i] = n.time_ms[i];
    }
    return DABNN_OK;
}
