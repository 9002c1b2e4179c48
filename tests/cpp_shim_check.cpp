// Compile-and-link check of the header-only bnn::Net shim (run by tests/test_host.py with g++).
// It exercises the reference's call sequence (binaries/run.cpp:21-55); without a CUDA device
// Net::create() throws std::runtime_error, which is the expected outcome on a CPU-only machine.
#include <dabnn_b200/net.hpp>

#include <cstdio>

int main(int argc, char** argv) {
    try {
        auto net = bnn::Net::create();
        net->optimize = true;
        if (argc > 1) {
            net->read(argv[1]);
            std::vector<float> ones(224 * 224 * 3, 1.f);
            net->run(ones.data());
            auto blob = net->get_blob(argc > 2 ? argv[2] : "fc_out");
            for (size_t i = 0; i < blob->total(); i++) std::printf("%.9g ", (*blob)[static_cast<int>(i)]);
            std::printf("\n");
        }
        std::puts("created");
    } catch (const std::invalid_argument& e) {   // reference net.cpp:35: the model file cannot be opened
        std::printf("invalid_argument: %s\n", e.what());
        return 4;
    } catch (const std::runtime_error& e) {
        std::printf("runtime_error: %s\n", e.what());
        return 3;
    }
    return 0;
}
