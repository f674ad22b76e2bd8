// Batched (n > 1 tokens) path of one MoE block.
#include "common.cuh"

namespace moe {

int batch_reserve(moe_engine* e, int32_t n_tokens) {
    BatchWork& bw = e->bw;
    if (n_tokens <= bw.capacity) return MOE_OK;
    MOE_CUDA(cudaStreamSynchronize(e->stream));
    batch_destroy(e);
    const size_t hb = (size_t)n_tokens * e->dims.hidden * sizeof(float);
    MOE_CUDA(cudaMalloc(&bw.h_a, hb));
    MOE_CUDA(cudaMalloc(&bw.h_b, hb));
    bw.capacity = n_tokens;
    return MOE_OK;
}

void batch_destroy(moe_engine* e) {
    BatchWork& bw = e->bw;
    cudaFree(bw.h_a);
    cudaFree(bw.h_b);
    bw = BatchWork{};
}

// Token-serial walk: every token goes through the decode kernel on its own
// (what the reference does for N tokens, src/engine/qwen35_moe/batched.rs:334-447).
int launch_batched_layer(moe_engine* e, int layer, const float* h_in, int32_t n, float* h_out,
                         const float* logit_bias, const int32_t* forced_idx, int32_t* out_idx, float* out_w) {
    const int H = e->dims.hidden, K = e->dims.top_k;
    for (int t = 0; t < n; ++t) {
        int rc = launch_decode(e, layer, layer + 1, h_in + (size_t)t * H, h_out + (size_t)t * H, logit_bias,
                               forced_idx ? forced_idx + (size_t)t * K : nullptr,
                               out_idx ? out_idx + (size_t)t * K : nullptr, out_w ? out_w + (size_t)t * K : nullptr);
        if (rc) return rc;
    }
    return MOE_OK;
}

}  // namespace moe
