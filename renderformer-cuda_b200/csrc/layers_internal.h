// Internal declarations shared by the layer library sources (not part of the C ABI).
#pragma once
#include <cublas_v2.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "rfk_layers.h"

struct rfk_ctx {
    cublasHandle_t blas = nullptr;
    void* ws = nullptr;      // cuBLAS workspace, set explicitly so capture never allocates
    size_t ws_bytes = 0;
    void* attn_ws = nullptr;  // split workspace of the attention kernel (rfk_ctx_reserve_attention_workspace), else NULL
    size_t attn_ws_bytes = 0;
    int device = 0;
};

namespace rfk_layers {
constexpr float kEpsFp16 = 0.0009765625f;   // 2^-10, the reference's kEpsFp16 (src/kernels/rmsnorm.h:9)
constexpr float kEpsFp32 = 1.1920929e-07f;  // 2^-23, the reference's kEpsFp32 (src/kernels/rmsnorm.h:10)

// rfk_decoder_layer_forward_cached with cache_flags (bit 0: keys arrive rotated and carrying the query norm weight; bit 1:
// the values are shared by the batch elements; see layers.cu); the session calls this form.
int decoder_layer_impl(rfk_ctx* ctx, const rfk_decoder_layer_weights* w, rfk_half* x, const rfk_half* pending_residual,
                       const rfk_half** pending_out, rfk_half* temp, rfk_half* proj_buf, rfk_half* qkv_buf, rfk_half* ffn_buf,
                       rfk_half* window_buf, float* cross_score_buf, float* self_score_buf, const rfk_half* K_cached,
                       const rfk_half* V_cached, int B, int Sq, int Sk, int n_keys, int dim, int num_heads, int ffn_hidden,
                       int patch_h, int patch_w, int window_size, int shift_size, const uint8_t* shift_mask,
                       const rfk_half* q_rope_cos, const rfk_half* q_rope_sin, const rfk_half* k_rope_cos,
                       const rfk_half* k_rope_sin, int cache_flags, rfk_stream_t stream);
}  // namespace rfk_layers
