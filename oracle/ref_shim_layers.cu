// Test infrastructure: extern "C" doors onto the reference engine's src/layers functions
// (residual/cast helpers, linear, sdpa, cached cross-attention, swin attention, SwiGLU FFN,
// the cached decoder layer and the mixed-precision encoder layer). Compiled together with
// the reference's unmodified sources by oracle/Makefile into oracle/_ref/libref_layers.so.
// Not part of the product.
#include "layers/attention.h"
#include "layers/linear.h"
#include "layers/transformer.h"
#include "kernels/rmsnorm.h"
#include <cublas_v2.h>

#define S(s) reinterpret_cast<cudaStream_t>(s)

// Flat, C-visible weight record of one decoder layer (all device pointers; NULL = absent).
struct RefDecoderLayerW {
    const float* query_norm_gamma;
    const float* kv_norm_gamma;
    const half *q_proj_w, *k_proj_w, *v_proj_w, *cross_out_w;
    const float *cross_q_norm, *cross_k_norm;
    const float* self_attn_norm_gamma;
    const half *swin_in_w, *swin_out_w;
    const float *swin_q_norm, *swin_k_norm;
    const float* ffn_norm_gamma;
    const half *w1, *w2, *w3;
};

static rf::DecoderLayerWeights to_ref(const RefDecoderLayerW& w) {
    rf::DecoderLayerWeights d{};
    d.query_norm_gamma = w.query_norm_gamma;
    d.kv_norm_gamma = w.kv_norm_gamma;
    d.cross_attn = rf::CrossAttnWeights{w.q_proj_w, nullptr, w.k_proj_w, nullptr, w.v_proj_w, nullptr,
                                        w.cross_out_w, nullptr, w.cross_q_norm, w.cross_k_norm};
    d.self_attn_norm_gamma = w.self_attn_norm_gamma;
    d.self_attn = rf::SwinAttnWeights{w.swin_in_w, nullptr, w.swin_out_w, nullptr, w.swin_q_norm,
                                      w.swin_k_norm};
    d.ffn_norm_gamma = w.ffn_norm_gamma;
    d.ffn = rf::FFNWeights{w.w1, w.w2, w.w3};
    return d;
}

extern "C" {

void* ref_cublas_create(void) {
    cublasHandle_t h = nullptr;
    if (cublasCreate(&h) != CUBLAS_STATUS_SUCCESS) return nullptr;
    return h;
}
void ref_cublas_destroy(void* h) { if (h) cublasDestroy((cublasHandle_t)h); }

void ref_residual_add(half* y, const half* r, int n, void* s) { rf::residual_add(y, r, n, S(s)); }
void ref_residual_add_f32(float* y, const float* r, int n, void* s) { rf::residual_add_f32(y, r, n, S(s)); }
void ref_residual_add_mixed(float* y, const half* r, int n, void* s) { rf::residual_add_mixed(y, r, n, S(s)); }
void ref_cast_fp32_to_fp16(const float* in, half* out, int n, void* s) { rf::cast_fp32_to_fp16(in, out, n, S(s)); }
void ref_cast_fp16_to_fp32(const half* in, float* out, int n, void* s) { rf::cast_fp16_to_fp32(in, out, n, S(s)); }

// the three launches that the fused residual + RMSNorm + cast kernel replaces
// (src/layers/transformer.cu:216,220-221); tmp32 is the fp32 norm output scratch
void ref_residual_rmsnorm_cast(float* h, const float* r, const float* gamma, float* tmp32,
                               half* y16, int rows, int dim, float eps, void* s) {
    rf::residual_add_f32(h, r, rows * dim, S(s));
    rf::rmsnorm_f32(h, gamma, tmp32, rows, dim, eps, S(s));
    rf::cast_fp32_to_fp16(tmp32, y16, rows * dim, S(s));
}

void ref_linear(void* h, const half* X, const half* W, const half* bias, half* Y, int M, int N,
                int K, void* s) {
    rf::linear((cublasHandle_t)h, X, W, bias, Y, M, N, K, S(s));
}

void ref_sdpa(void* h, const half* Q, const half* K, const half* V, half* O, float* ws,
              const bool* mask, int B, int H, int Sq, int Sk, int D, void* s) {
    rf::sdpa((cublasHandle_t)h, Q, K, V, O, ws, mask, B, H, Sq, Sk, D, S(s));
}

void ref_ffn_swiglu(void* h, const half* w1, const half* w2, const half* w3, const half* x,
                    half* out, half* buf, int M, int dim, int hidden, void* s) {
    rf::FFNWeights w{w1, w2, w3};
    rf::ffn_swiglu((cublasHandle_t)h, w, x, out, buf, M, dim, hidden, S(s));
}

void ref_window_partition(const half* x, half* win, int B, int H, int W, int C, int ws, void* s) {
    rf::window_partition(x, win, B, H, W, C, ws, S(s));
}
void ref_window_reverse(const half* win, half* x, int B, int H, int W, int C, int ws, void* s) {
    rf::window_reverse(win, x, B, H, W, C, ws, S(s));
}
void ref_cyclic_shift_2d(const half* x, half* out, int B, int H, int W, int C, int sh, int sw, void* s) {
    rf::cyclic_shift_2d(x, out, B, H, W, C, sh, sw, S(s));
}

void ref_swin_self_attention(void* h, const RefDecoderLayerW* w, const half* x, half* out,
                             half* window_buf, half* qkv_buf, float* score_buf, half* scratch,
                             int B, int H, int W, int dim, int heads, int ws, int shift,
                             const bool* shift_mask, void* s) {
    rf::SwinAttnWeights sw{w->swin_in_w, nullptr, w->swin_out_w, nullptr, w->swin_q_norm, w->swin_k_norm};
    rf::swin_self_attention((cublasHandle_t)h, sw, x, out, window_buf, qkv_buf, score_buf, scratch,
                            B, H, W, dim, heads, ws, shift, shift_mask, S(s));
}

void ref_cross_attention_cached(void* h, const RefDecoderLayerW* w, const half* q_in, half* out,
                                half* proj_buf, float* score_buf, const half* Kc, const half* Vc,
                                int B, int Sq, int Sk, int dim, int heads, const half* qc,
                                const half* qs, const half* kc, const half* ks, void* s) {
    rf::DecoderLayerWeights d = to_ref(*w);
    rf::cross_attention_cached((cublasHandle_t)h, d.cross_attn, q_in, out, proj_buf, score_buf, Kc,
                               Vc, nullptr, B, Sq, Sk, dim, dim, heads, qc, qs, kc, ks, 0, S(s));
}

void ref_precompute_cross_kv(void* h, const RefDecoderLayerW* w, const half* ctx_normed, half* K,
                             half* V, half* proj_buf, int B, int Sk, int kv_dim, int dim, int heads,
                             void* s) {
    rf::DecoderLayerWeights d = to_ref(*w);
    rf::precompute_cross_kv((cublasHandle_t)h, d.cross_attn, ctx_normed, K, V, proj_buf, B, Sk,
                            kv_dim, dim, heads, S(s));
}

// src/layers/transformer.cu:151-194, called as src/pipeline/render_session.cu:223-233 does
void ref_decoder_layer_forward_cached(void* h, const RefDecoderLayerW* w, half* x, half* temp,
                                      half* proj_buf, half* qkv_buf, half* ffn_buf, half* window_buf,
                                      float* cross_score, float* self_score, const half* Kc,
                                      const half* Vc, int B, int Sq, int Sk, int dim, int heads,
                                      int ffn_hidden, int pH, int pW, int ws, int shift,
                                      const bool* shift_mask, const half* qc, const half* qs,
                                      const half* kc, const half* ks, void* s) {
    rf::DecoderLayerWeights d = to_ref(*w);
    rf::decoder_layer_forward_cached((cublasHandle_t)h, d, x, temp, proj_buf, qkv_buf, ffn_buf,
                                     window_buf, cross_score, self_score, Kc, Vc, nullptr, B, Sq,
                                     Sk, dim, heads, ffn_hidden, pH, pW, ws, shift, shift_mask, qc,
                                     qs, kc, ks, S(s));
}

// src/layers/transformer.cu:196-224 (fp32 hidden state, fp16 sub-layers), flat weight arguments
void ref_encoder_layer_forward_mixed(void* h, const float* query_norm, const half* in_proj_w,
                                     const half* out_proj_w, const float* q_norm, const float* k_norm,
                                     const float* ffn_norm, const half* w1, const half* w2, const half* w3,
                                     float* x, half* temp, half* qkv_buf, half* ffn_buf, float* score_buf,
                                     int B, int S_, int dim, int heads, int ffn_hidden, const half* rc,
                                     const half* rs, void* s) {
    rf::EncoderLayerWeights w{};
    w.query_norm_gamma = query_norm;
    w.attn = rf::MHAWeights{in_proj_w, nullptr, out_proj_w, nullptr, q_norm, k_norm};
    w.ffn_norm_gamma = ffn_norm;
    w.ffn = rf::FFNWeights{w1, w2, w3};
    rf::encoder_layer_forward_mixed((cublasHandle_t)h, w, x, temp, qkv_buf, ffn_buf, score_buf, nullptr, B, S_,
                                    dim, heads, ffn_hidden, rc, rs, S(s));
}

}  // extern "C"
