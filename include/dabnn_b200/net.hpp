// Header-only C++ mirror of the reference's bnn::Net (dabnn/net.h:22-66) over the C ABI of
// libdabnn_b200.so.  Same method names, same public flags, same exception types, so that code
// written against the reference (binaries/run.cpp, benchmark/benchmark_single_model.cpp,
// tests/net_test.cpp) only needs to include this header instead of <dabnn/net.h>.
#pragma once
#include <cstddef>
#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "../dabnn_b200.h"

namespace bnn {

// The slice of the reference's bnn::Mat (dabnn/mat.h:37-155) that callers of Net::get_blob use:
// a dense NHWC fp32 tensor on the host.
class Mat {
   public:
    int n = 0, h = 0, w = 0, c = 0;
    std::vector<float> storage;
    void* data = nullptr;
    size_t total() const { return storage.size(); }
    float& operator[](int i) { return storage[static_cast<size_t>(i)]; }
    const float& operator[](int i) const { return storage[static_cast<size_t>(i)]; }
    template <typename T>
    operator T*() { return reinterpret_cast<T*>(storage.data()); }
};

class Net : public std::enable_shared_from_this<Net> {
   public:
    static std::shared_ptr<Net> create() { return std::shared_ptr<Net>(new Net()); }  // net.h:57
    ~Net() { dabnn_net_destroy(handle_); }
    Net(const Net&) = delete;
    Net& operator=(const Net&) = delete;

    // reference net.h:59-61
    bool optimize = true;
    bool run_fconv = true;
    bool strict = true;
    // extensions: the reference runs one image at a time on one fixed code path
    int max_batch = 1;
    int engine = DABNN_ENGINE_AUTO;

    void read(const std::string& path) {  // net.cpp:32
        configure();
        const int rc = dabnn_net_read_file(handle_, path.c_str());
        if (rc == DABNN_ERR_IO) throw std::invalid_argument(dabnn_last_error());
        check(rc);
    }
    void read_buf(const void* ptr, size_t len) {  // net.cpp:46 (the length makes the parse bounds-checked)
        configure();
        check(dabnn_net_read_buf(handle_, ptr, len));
    }
    void run(void* input, int batch = 1) {  // net.cpp:272: host fp32 NHWC
        check(dabnn_net_run(handle_, static_cast<const float*>(input), batch, 0));
    }
    void run_device(const float* device_input, int batch) {
        check(dabnn_net_run(handle_, device_input, batch, 1));
    }
    std::shared_ptr<Mat> get_blob(const std::string& name) {  // net.cpp:288
        int dims[4];
        int rc = dabnn_net_get_blob(handle_, name.c_str(), dims, nullptr, nullptr, 0);
        if (rc == DABNN_ERR_NOT_FOUND) throw std::out_of_range(dabnn_last_error());
        check(rc);
        auto m = std::make_shared<Mat>();
        m->n = dims[0]; m->h = dims[1]; m->w = dims[2]; m->c = dims[3];
        m->storage.resize(static_cast<size_t>(dims[0]) * dims[1] * dims[2] * dims[3]);
        m->data = m->storage.data();
        check(dabnn_net_get_blob(handle_, name.c_str(), nullptr, nullptr, m->storage.data(), m->storage.size()));
        return m;
    }
    // Output of a Binarize layer (dabnn/layers/Binarize.cpp:9): the packed words, dims {n, h, w, c / 64}.
    std::vector<uint64_t> get_blob_bits(const std::string& name, int dims[4]) {
        int rc = dabnn_net_get_blob_bits(handle_, name.c_str(), dims, nullptr, nullptr, 0);
        if (rc == DABNN_ERR_NOT_FOUND) throw std::out_of_range(dabnn_last_error());
        check(rc);
        std::vector<uint64_t> words(static_cast<size_t>(dims[0]) * dims[1] * dims[2] * dims[3]);
        check(dabnn_net_get_blob_bits(handle_, name.c_str(), nullptr, nullptr, words.data(), words.size()));
        return words;
    }
    dabnn_net* handle() const { return handle_; }

   private:
    Net() { check(dabnn_net_create(&handle_)); }
    void configure() {
        check(dabnn_net_set_flags(handle_, optimize, run_fconv, strict));
        check(dabnn_net_configure(handle_, max_batch, engine));
    }
    static void check(int rc) {
        if (rc != DABNN_OK) throw std::runtime_error(dabnn_last_error());
    }
    dabnn_net* handle_ = nullptr;
};

}  // namespace bnn
