// Minimal, bounds-checked reader for the FlatBuffers wire format of `.dab` model files
// (reference common/dab.fbs; field slots from the reference's generated accessors,
// common/dab_generated.h).  No FlatBuffers library is needed: a table starts with an int32 that
// points back to its vtable {u16 vtable bytes, u16 table bytes, u16 field offset per slot}; strings,
// vectors and sub-tables are reached through u32 offsets relative to the referring field.
#pragma once
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

namespace dabnn {

struct DabError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

class FbBuffer {
   public:
    FbBuffer(const uint8_t* data, size_t len) : d_(data), n_(len) {}
    template <class T>
    T read(size_t pos) const {
        if (pos + sizeof(T) > n_ || pos + sizeof(T) < pos) throw DabError("dab: read out of bounds");
        T v;
        std::memcpy(&v, d_ + pos, sizeof(T));
        return v;
    }
    const uint8_t* ptr(size_t pos, size_t bytes) const {
        if (pos + bytes > n_ || pos + bytes < pos) throw DabError("dab: vector out of bounds");
        return d_ + pos;
    }
    size_t size() const { return n_; }

   private:
    const uint8_t* d_;
    size_t n_;
};

class FbTable {
   public:
    FbTable() : b_(nullptr), pos_(0), vt_(0), vsize_(0) {}
    FbTable(const FbBuffer* b, size_t pos) : b_(b), pos_(pos) {
        const int32_t so = b->read<int32_t>(pos);
        const long long vt = (long long)pos - so;
        if (vt < 0) throw DabError("dab: vtable out of bounds");
        vt_ = (size_t)vt;
        vsize_ = b->read<uint16_t>(vt_);
    }
    bool valid() const { return b_ != nullptr; }
    // absolute position of field `slot`, 0 when absent
    size_t field(int slot) const {
        const size_t o = 4 + 2 * (size_t)slot;
        if (o + 2 > vsize_) return 0;
        const uint16_t rel = b_->read<uint16_t>(vt_ + o);
        return rel ? pos_ + rel : 0;
    }
    template <class T>
    T scalar(int slot, T dflt) const {
        const size_t p = field(slot);
        return p ? b_->read<T>(p) : dflt;
    }
    size_t indirect(int slot) const {
        const size_t p = field(slot);
        return p ? p + b_->read<uint32_t>(p) : 0;
    }
    std::string str(int slot) const {
        const size_t t = indirect(slot);
        if (!t) return "";
        const uint32_t n = b_->read<uint32_t>(t);
        return std::string(reinterpret_cast<const char*>(b_->ptr(t + 4, n)), n);
    }
    FbTable table(int slot) const {
        const size_t t = indirect(slot);
        return t ? FbTable(b_, t) : FbTable();
    }
    template <class T>
    std::vector<T> vec(int slot) const {
        std::vector<T> out;
        const size_t t = indirect(slot);
        if (!t) return out;
        const uint32_t n = b_->read<uint32_t>(t);
        if (!n) return out;
        const uint8_t* src = b_->ptr(t + 4, (size_t)n * sizeof(T));   // bounds-checked before anything is allocated
        out.resize(n);
        std::memcpy(out.data(), src, (size_t)n * sizeof(T));
        return out;
    }
    // raw view of a scalar vector (pointer into the buffer, element count)
    template <class T>
    const T* vec_view(int slot, size_t* count) const {
        const size_t t = indirect(slot);
        *count = 0;
        if (!t) return nullptr;
        const uint32_t n = b_->read<uint32_t>(t);
        *count = n;
        return reinterpret_cast<const T*>(b_->ptr(t + 4, (size_t)n * sizeof(T)));
    }
    std::vector<FbTable> tables(int slot) const {
        std::vector<FbTable> out;
        const size_t t = indirect(slot);
        if (!t) return out;
        const uint32_t n = b_->read<uint32_t>(t);
        b_->ptr(t + 4, 4 * (size_t)n);   // the offset array lies inside the buffer
        for (uint32_t i = 0; i < n; i++) {
            const size_t p = t + 4 + 4 * (size_t)i;
            out.emplace_back(b_, p + b_->read<uint32_t>(p));
        }
        return out;
    }
    std::vector<std::string> strings(int slot) const {
        std::vector<std::string> out;
        const size_t t = indirect(slot);
        if (!t) return out;
        const uint32_t n = b_->read<uint32_t>(t);
        b_->ptr(t + 4, 4 * (size_t)n);
        for (uint32_t i = 0; i < n; i++) {
            const size_t p = t + 4 + 4 * (size_t)i;
            const size_t s = p + b_->read<uint32_t>(p);
            const uint32_t len = b_->read<uint32_t>(s);
            out.emplace_back(reinterpret_cast<const char*>(b_->ptr(s + 4, len)), len);
        }
        return out;
    }

   private:
    const FbBuffer* b_;
    size_t pos_, vt_;
    uint16_t vsize_;
};

// flatbnn::LayerType, reference common/dab.fbs:4-5
enum class LayerType : int8_t {
    FpConv2D = 0, AvePool, MaxPool, Relu, Softmax, FC, Add, Concat, BinConv2D, Affine, Binarize, Split,
    Shuffle, PRelu
};
inline const char* layer_type_name(LayerType t) {  // reference common/flatbuffers_helper.h:125-158
    static const char* names[] = {"fpconv", "avepool", "maxpool", "relu", "softmax", "fc", "Add",
                                  "concat", "binconv", "affine", "binarize", "split", "shuffle", "prelu"};
    const int i = (int)t;
    return (i >= 0 && i < 14) ? names[i] : "unknown";
}

}  // namespace dabnn
