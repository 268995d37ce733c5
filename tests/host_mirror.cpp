// Drives the C++ mirror of the reference's operator interface the way the reference's
// main.cpp + layers do: load a bundle, register the quantised tensors, run projections.
//   host_mirror <model.bin> <model.meta.json> <weight key> <x.f16> <out.f16> [M]
// x.f16 holds M*K raw fp16 values; out.f16 receives M*N.  Exit code 0 on success.
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "../adreno-llms_b200/host/nnopt_linear.hpp"

int main(int argc, char** argv) {
    if (argc < 6) return 2;
    const int M = argc > 6 ? atoi(argv[6]) : 1;
    nn_context* ctx = nullptr;
    if (nn_init(0, &ctx) != NN_OK) { fprintf(stderr, "init: %s\n", nn_last_error()); return 3; }
    {
    nnopt::Weights weights;  // must go away before the context, like the reference's Weights and its cl_context
    if (!weights.load(argv[1], argv[2], ctx)) return 4;
    const int registered = weights.register_quantized();
    const std::string key = argv[3];
    if (!weights.has_tensor(key)) return 5;
    const std::vector<int> shape = weights.get_shape(key);
    const std::string dtype = weights.get_dtype(key);
    const int N = shape[0];
    int K = shape[1];
    if (dtype == "q4_packed") K = weights.get_shape(key + ".scale")[1] * 32;
    std::vector<unsigned short> x((size_t)M * K), out((size_t)M * N);
    FILE* f = fopen(argv[4], "rb");
    if (!f || fread(x.data(), 2, x.size(), f) != x.size()) return 6;
    fclose(f);
    nn_buf W = weights.get_buffer(key);
    nn_buf xb = nn_buf_alloc(ctx, x.size() * 2), ob = nn_buf_alloc(ctx, out.size() * 2);
    if (!W || !xb || !ob) return 7;
    nn_buf_write(ctx, xb, 0, x.data(), x.size() * 2);
    if (!nnopt::pytorch_linear(ctx, M, N, K, xb, W, ob)) return 8;
    nn_buf_read(ctx, out.data(), ob, 0, out.size() * 2);
    if (nn_sync(ctx) != NN_OK) return 9;
    f = fopen(argv[5], "wb");
    fwrite(out.data(), 2, out.size(), f);
    fclose(f);
    // a missing key is silent when optional, loud otherwise; both return nullptr
    if (weights.get_buffer("no.such.key", true) != nullptr) return 10;
    printf("registered=%d dtype=%s N=%d K=%d M=%d\n", registered, dtype.c_str(), N, K, M);
    nn_buf_free(ctx, xb);
    nn_buf_free(ctx, ob);
    }
    nn_shutdown(ctx);
    return 0;
}
