// C++ mirror of the reference's linear-operator interface over the nnopt_b200 C ABI.
//
// The reference's layers call free functions from src/utils.h and a Weights object
// (src/models/lfm2-5-350m/src/utils.h:117-142, src/weights.h:13-51).  A port of those
// layers to CUDA keeps its call sites: same names, argument order and bool / nullptr
// error behaviour; `cl_command_queue` becomes `nn_context*` (one in-order stream) and
// `cl_mem` becomes `nn_buf` (a device pointer).  Header-only; link libnnopt_b200.so.
#pragma once
#include <string>
#include <vector>

#include "../../include/nnopt_b200.h"

namespace nnopt {

// out[M,N] = x[M,K] . W[N,K]^T  (utils.h:117-119).  Returns false after printing
// "ERROR: ... (file:line)" on failure, like the reference.
inline bool pytorch_linear(nn_context* queue, int M, int N, int K, nn_buf x, nn_buf W, nn_buf out) {
    return nn_linear(queue, M, N, K, x, W, out) == NN_OK;
}

// utils.h:127,132.  The reference keeps one process-wide registry; here it lives in the
// context, so the context is the first argument.
inline bool nnopt_register_int8_weight(nn_context* ctx, nn_buf W_int8, nn_buf scale_fp16, int N, int K) {
    return nn_register_int8_weight(ctx, W_int8, scale_fp16, N, K) == NN_OK;
}
inline bool nnopt_register_q4_weight(nn_context* ctx, nn_buf W_q4, nn_buf scale_fp16, int N, int K) {
    return nn_register_q4_weight(ctx, W_q4, scale_fp16, N, K) == NN_OK;
}

// utils.h:140-142 (M = 1 in the reference).
inline bool pytorch_linear_silu_gate_fused(nn_context* queue, int N, int K, nn_buf x, nn_buf W3, nn_buf gate_inout) {
    return nn_linear_silu_gate_fused(queue, 1, N, K, x, W3, gate_inout) == NN_OK;
}

// src/models/qwen2-5-0-5b/src/utils.cpp:862-882 and :478-487.
inline bool pytorch_linear_add(nn_context* queue, int M, int N, int K, nn_buf x, nn_buf W, nn_buf residual_inout) {
    return nn_linear_add(queue, M, N, K, x, W, residual_inout) == NN_OK;
}
inline bool fused_gate_up_silu_m1(nn_context* queue, int N, int K, nn_buf x, nn_buf Wg, nn_buf Wu, nn_buf out) {
    return nn_fused_gate_up_silu(queue, 1, N, K, x, Wg, Wu, out) == NN_OK;
}

// src/models/smollm2-135m-instruct/src/layers/attention.cpp:653-722: the three decode projections.
inline bool fused_qkv_gemv_m1(nn_context* queue, int K, nn_buf x, nn_buf Wq, int Nq, nn_buf Wk, int Nk, nn_buf Wv, int Nv,
                              nn_buf q, nn_buf k, nn_buf v) {
    return nn_linear_qkv(queue, 1, K, x, Wq, Nq, Wk, Nk, Wv, Nv, q, k, v) == NN_OK;
}

// src/models/smollm2-135m-instruct/src/layers/lm_head.cpp:36-67 followed by the GPU arg-max of
// src/model.cpp:603-623, as one launch; `logits` may be nullptr (they are then never written).
inline bool lm_head_argmax_m1(nn_context* queue, int vocab, int hidden, nn_buf x, nn_buf W, nn_buf logits, nn_buf token_out) {
    return nn_linear_argmax(queue, vocab, hidden, x, W, logits, token_out) == NN_OK;
}

// RMSNorm::forward (src/models/smollm2-135m-instruct/src/layers/layer_norm.cpp:76-126) and the norm fused
// into the projection that consumes it.
inline bool rmsnorm_forward(nn_context* queue, int rows, int cols, nn_buf x, nn_buf weight, float eps, nn_buf out) {
    return nn_rmsnorm(queue, rows, cols, x, weight, eps, out) == NN_OK;
}
inline bool rmsnorm_qkv_m1(nn_context* queue, int K, nn_buf x, nn_buf norm_weight, float eps, nn_buf Wq, int Nq, nn_buf Wk, int Nk, nn_buf Wv,
                           int Nv, nn_buf q, nn_buf k, nn_buf v) {
    return nn_rmsnorm_linear_qkv(queue, 1, K, x, norm_weight, eps, Wq, Nq, Wk, Nk, Wv, Nv, q, k, v) == NN_OK;
}
inline bool rmsnorm_gate_up_silu_m1(nn_context* queue, int N, int K, nn_buf x, nn_buf norm_weight, float eps, nn_buf Wg, nn_buf Wu, nn_buf out) {
    return nn_rmsnorm_gate_up_silu(queue, 1, N, K, x, norm_weight, eps, Wg, Wu, out) == NN_OK;
}

// class Weights (weights.h:13-51).  load() takes the context the buffers are created in.
class Weights {
public:
    Weights() = default;
    Weights(const Weights&) = delete;
    Weights& operator=(const Weights&) = delete;
    ~Weights() { nn_weights_free(w_); }

    bool load(const std::string& bin_path, const std::string& meta_path, nn_context* ctx) {
        nn_weights_free(w_);
        w_ = nullptr;
        ctx_ = ctx;
        return nn_weights_load(ctx, bin_path.c_str(), meta_path.c_str(), &w_) == NN_OK;
    }
    bool has_tensor(const std::string& key) const { return w_ && nn_weights_has_tensor(w_, key.c_str()) != 0; }
    nn_buf get_buffer(const std::string& key, bool optional = false) {
        return w_ ? nn_weights_get_buffer(w_, key.c_str(), optional ? 1 : 0) : nullptr;
    }
    size_t get_size_bytes(const std::string& key) const { return w_ ? nn_weights_get_size_bytes(w_, key.c_str()) : 0; }
    size_t get_num_elements(const std::string& key) const { return w_ ? nn_weights_get_num_elements(w_, key.c_str()) : 0; }
    std::vector<int> get_shape(const std::string& key) const {
        std::vector<int> s(8);
        const int rank = w_ ? nn_weights_get_shape(w_, key.c_str(), s.data(), 8) : 0;
        s.resize(rank < 8 ? rank : 8);
        return s;
    }
    std::vector<float> get_host_vec(const std::string& key) const {
        std::vector<float> v(get_num_elements(key));
        if (v.empty() || nn_weights_get_host_f32(w_, key.c_str(), v.data(), v.size()) != NN_OK) v.clear();
        return v;
    }
    std::string get_dtype(const std::string& key) const { return w_ ? nn_weights_get_dtype(w_, key.c_str()) : ""; }
    std::vector<std::string> all_keys() const {
        std::vector<std::string> out;
        const int n = w_ ? nn_weights_num_keys(w_) : 0;
        for (int i = 0; i < n; ++i) out.emplace_back(nn_weights_key_at(w_, i));
        return out;
    }
    // The NNOPT_QUANT walk of src/models/lfm2-5-350m/src/main.cpp:527-566.
    int register_quantized() { return (w_ && ctx_) ? nn_weights_register_quantized(ctx_, w_) : 0; }

private:
    nn_weights* w_ = nullptr;
    nn_context* ctx_ = nullptr;
};

}  // namespace nnopt
