// Test infrastructure: extern "C" doors onto the reference engine's src/layers functions
// (residual/cast helpers, linear, sdpa, cached cross-attention, swin attention, SwiGLU FFN,
// the cached decoder layer and the mixed-precision encoder layer). Compiled together with
// the reference's unmodified sources by oracle/Makefile into oracle/_ref/libref_layers.so.
// Not part of the product.
#include "layers/attention.h"
#include "layers/dpt.h"
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

// glue operators of the DPT head that src/layers/dpt.h exports
void ref_bilinear_upsample(const half* in, half* out, int N, int C, int H_in, int W_in, int H_out, int W_out, void* s) {
    rf::bilinear_upsample(in, out, N, C, H_in, W_in, H_out, W_out, S(s));
}
void ref_silu_inplace(half* x, int n, void* s) { rf::silu_inplace(x, n, S(s)); }

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

// rf::dpt_forward (src/layers/dpt.cu:322-461) behind a flat weight record. RefDptW has the field order of
// rfk_dpt_weights in include/rfk_layers.h, so a test passes one ctypes structure to both libraries.
struct RefRcuW { const half *conv1_w, *conv1_b, *conv2_w, *conv2_b; };
struct RefFfbW { RefRcuW rcu1, rcu2; const half *out_conv_w, *out_conv_b; int has_resconv1; };
struct RefDptW {
    const half* project_w[4]; const half* project_b[4]; const half* resize_w[4]; const half* resize_b[4];
    const half* layer_rn_w[4]; RefFfbW refinenet[4];
    const half *output_conv1_w, *output_conv1_b, *output_conv2a_w, *output_conv2a_b, *output_conv2b_w, *output_conv2b_b;
    int features_dim, out_dim; int out_channels[4];
};

extern "C" void ref_dpt_forward(void* h, const RefDptW* w, const half* f0, const half* f1, const half* f2, const half* f3,
                                half* out, half* col_buf, int B, int dim, int pH, int pW, int ps, void* s) {
    rf::DPTWeights d{};
    for (int i = 0; i < 4; ++i) {
        d.project_w[i] = w->project_w[i]; d.project_b[i] = w->project_b[i];
        d.resize_w[i] = w->resize_w[i]; d.resize_b[i] = w->resize_b[i];
        d.layer_rn_w[i] = w->layer_rn_w[i];
        const RefFfbW& f = w->refinenet[i];
        d.refinenet[i].rcu1 = rf::RCUWeights{f.rcu1.conv1_w, f.rcu1.conv1_b, f.rcu1.conv2_w, f.rcu1.conv2_b};
        d.refinenet[i].rcu2 = rf::RCUWeights{f.rcu2.conv1_w, f.rcu2.conv1_b, f.rcu2.conv2_w, f.rcu2.conv2_b};
        d.refinenet[i].out_conv_w = f.out_conv_w; d.refinenet[i].out_conv_b = f.out_conv_b;
        d.refinenet[i].has_resconv1 = f.has_resconv1 != 0;
    }
    d.output_conv1_w = w->output_conv1_w; d.output_conv1_b = w->output_conv1_b;
    d.output_conv2a_w = w->output_conv2a_w; d.output_conv2a_b = w->output_conv2a_b;
    d.output_conv2b_w = w->output_conv2b_w; d.output_conv2b_b = w->output_conv2b_b;
    const half* feats[4] = {f0, f1, f2, f3};
    rf::dpt_forward((cublasHandle_t)h, d, feats, out, col_buf, B, dim, pH, pW, ps, w->features_dim, w->out_dim,
                    w->out_channels, S(s));
}

// ---------------------------------------------------------------------------------------
// Per-view decoder pipeline of the reference, composed from the reference's own functions in
// the order of src/pipeline/render_session.cu:189-238 (RenderSession::Impl::render_view) and
// captured as a CUDA graph as :474-495 does. RenderSession itself cannot be used: it needs the
// HDF5 scene reader, compiles the head count in (8 x 128, src/model/config.h:8-9) and ends in
// the DPT convolution head; this composition takes runtime shapes and stops after the decoder
// stack. Two kernels that are file-local in render_session.cu are restated here
// (k_patchify_s :48-59, k_center_pos_from_c2w :73-88).
#include "kernels/coord_transform.h"
#include "kernels/ray_gen.h"
#include "kernels/rope.h"
#include <vector>

namespace {
__global__ void shim_patchify(const half* __restrict__ in, half* __restrict__ out, int H, int W, int C, int ps,
                              int pH, int pW) {
    int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= pH * pW * C * ps * ps) return;
    int p2 = idx % ps, r = idx / ps;
    int p1 = r % ps; r /= ps;
    int c = r % C, patch = r / C;
    int h1 = patch / pW, w1 = patch % pW;
    out[patch * (C * ps * ps) + c * (ps * ps) + p1 * ps + p2] = in[((h1 * ps + p1) * W + w1 * ps + p2) * C + c];
}
__global__ void shim_center_pos(const float* __restrict__ c2w, const float* __restrict__ wc, half* __restrict__ out, int nr) {
    int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= nr) return;
    float vx = wc[0] - c2w[3], vy = wc[1] - c2w[7], vz = wc[2] - c2w[11];
    half hx = __float2half(c2w[0] * vx + c2w[4] * vy + c2w[8] * vz);
    half hy = __float2half(c2w[1] * vx + c2w[5] * vy + c2w[9] * vz);
    half hz = __float2half(c2w[2] * vx + c2w[6] * vy + c2w[10] * vz);
    for (int v = 0; v < 3; ++v) { out[r * 9 + 3 * v] = hx; out[r * 9 + 3 * v + 1] = hy; out[r * 9 + 3 * v + 2] = hz; }
}
__global__ void shim_broadcast_add(half* __restrict__ out, const half* __restrict__ bc, int n, int dim) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __float2half(__half2float(out[i]) + __half2float(bc[i % dim]));
}
}  // namespace

struct RefViewPipeline {
    // configuration
    int N, res, dim, heads, ffn, nr, nf, ps, ws, shift, layers;
    int Se, Se_pad, pH, pW, nP, hd;
    // model / scene (device pointers owned by the caller)
    const half *tri16, *vn16; const float* world_center;
    const float* vt_rope_freqs; const half *ray_enc_w, *ray_enc_b, *ray_map_patch_token; const float* ray_enc_norm;
    const half* const* kvK; const half* const* kvV;  // host arrays [layers]
    const bool* shift_mask; const half *q_cos, *q_sin;
    RefDecoderLayerW w[32];
    // buffers (owned here)
    std::vector<void*> owned;
    float *c2w_gpu, *fov_gpu, *id_c2w, *rays_o; half *vtri, *vvn, *vpos, *k_cos, *k_sin, *rays_d, *ray_pat, *rtok;
    half *temp, *proj, *qkv, *ffnb, *win, *dft[4]; float *score, *self_score;
    std::vector<const half*> K, V;
    cublasHandle_t blas; cudaStream_t stream; float *pin_c2w, *pin_fov;
    cudaGraph_t graph = nullptr; cudaGraphExec_t exec = nullptr; cudaEvent_t e0, e1;
};

static void ref_view_body(RefViewPipeline& d) {
    cudaStream_t s = d.stream;
    const int N = d.N, nr = d.nr, dim = d.dim, nP = d.nP, ps = d.ps;
    cudaMemcpyAsync(d.c2w_gpu, d.pin_c2w, 16 * sizeof(float), cudaMemcpyHostToDevice, s);
    cudaMemcpyAsync(d.vtri, d.tri16, N * 9 * sizeof(half), cudaMemcpyDeviceToDevice, s);
    cudaMemcpyAsync(d.vvn, d.vn16, N * 9 * sizeof(half), cudaMemcpyDeviceToDevice, s);
    rf::world_to_cam(d.c2w_gpu, d.vtri, d.vvn, 1, N, s);
    shim_center_pos<<<(nr + 255) / 256, 256, 0, s>>>(d.c2w_gpu, d.world_center, d.vpos, nr);
    cudaMemcpyAsync(d.vpos + nr * 9, d.vtri, N * 9 * sizeof(half), cudaMemcpyDeviceToDevice, s);
    rf::triangle_rope_freqs(d.vpos, d.vt_rope_freqs, d.k_cos, d.k_sin, 1, d.Se_pad, d.nf, d.hd, s);
    cudaMemcpyAsync(d.fov_gpu, d.pin_fov, sizeof(float), cudaMemcpyHostToDevice, s);
    rf::ray_gen(d.id_c2w, d.fov_gpu, d.rays_o, d.rays_d, 1, d.res, s);
    shim_patchify<<<(nP * 3 * ps * ps + 255) / 256, 256, 0, s>>>(d.rays_d, d.ray_pat, d.res, d.res, 3, ps, d.pH, d.pW);
    rf::linear(d.blas, d.ray_pat, d.ray_enc_w, d.ray_enc_b, d.rtok, nP, dim, 3 * ps * ps, s);
    rf::rmsnorm(d.rtok, d.ray_enc_norm, d.rtok, nP, dim, rf::kEpsFp16, s);
    shim_broadcast_add<<<(nP * dim + 255) / 256, 256, 0, s>>>(d.rtok, d.ray_map_patch_token, nP * dim, dim);
    const int L4 = d.layers / 4 > 0 ? d.layers / 4 : 1;
    for (int i = 0; i < d.layers; ++i) {
        const int cur_shift = (i % 2 == 1) ? d.shift : 0;
        rf::DecoderLayerWeights w = to_ref(d.w[i]);
        rf::decoder_layer_forward_cached(d.blas, w, d.rtok, d.temp, d.proj, d.qkv, d.ffnb, d.win, d.score, d.self_score,
                                         d.K[i], d.V[i], nullptr, 1, nP, d.Se_pad, dim, d.heads, d.ffn, d.pH, d.pW, d.ws,
                                         cur_shift, cur_shift > 0 ? d.shift_mask : nullptr, d.q_cos, d.q_sin, d.k_cos,
                                         d.k_sin, s);
        if ((i + 1) % L4 == 0 && (i + 1) / L4 <= 4)
            cudaMemcpyAsync(d.dft[(i + 1) / L4 - 1], d.rtok, (size_t)nP * dim * sizeof(half), cudaMemcpyDeviceToDevice, s);
    }
}

extern "C" {

// cfg: {N, res, dim, heads, ffn, nr, nf, ps, ws, shift, layers}
void* ref_view_create(const int* cfg, const half* tri16, const half* vn16, const float* world_center,
                      const float* vt_rope_freqs, const half* ray_enc_w, const half* ray_enc_b,
                      const float* ray_enc_norm, const half* ray_map_patch_token, const RefDecoderLayerW* w,
                      const half* const* kvK, const half* const* kvV, const bool* shift_mask, int use_graph) {
    auto* d = new RefViewPipeline();
    d->N = cfg[0]; d->res = cfg[1]; d->dim = cfg[2]; d->heads = cfg[3]; d->ffn = cfg[4]; d->nr = cfg[5]; d->nf = cfg[6];
    d->ps = cfg[7]; d->ws = cfg[8]; d->shift = cfg[9]; d->layers = cfg[10];
    d->Se = d->nr + d->N; d->Se_pad = (d->Se + 7) & ~7; d->pH = d->pW = d->res / d->ps; d->nP = d->pH * d->pW;
    d->hd = d->dim / d->heads;
    d->tri16 = tri16; d->vn16 = vn16; d->world_center = world_center; d->vt_rope_freqs = vt_rope_freqs;
    d->ray_enc_w = ray_enc_w; d->ray_enc_b = ray_enc_b; d->ray_enc_norm = ray_enc_norm;
    d->ray_map_patch_token = ray_map_patch_token; d->shift_mask = shift_mask;
    for (int i = 0; i < d->layers; ++i) { d->w[i] = w[i]; d->K.push_back(kvK[i]); d->V.push_back(kvV[i]); }
    auto alloc = [&](auto** p, size_t bytes) { void* q = nullptr; cudaMalloc(&q, bytes < 256 ? 256 : bytes); d->owned.push_back(q); *p = (decltype(*p))q; };
    const size_t nP = d->nP, dim = d->dim, Sep = d->Se_pad, hd = d->hd, nh = d->heads, ffn = d->ffn, ws = d->ws;
    const size_t nWin = (d->pH / ws) * (d->pW / ws);
    alloc(&d->c2w_gpu, 64); alloc(&d->fov_gpu, 4); alloc(&d->id_c2w, 64); alloc(&d->rays_o, 12);
    alloc(&d->vtri, d->N * 18); alloc(&d->vvn, d->N * 18); alloc(&d->vpos, Sep * 18);
    cudaMemset(d->vpos, 0, Sep * 18);
    alloc(&d->k_cos, Sep * hd * 2); alloc(&d->k_sin, Sep * hd * 2);
    alloc(&d->rays_d, (size_t)d->res * d->res * 6); alloc(&d->ray_pat, nP * 3 * d->ps * d->ps * 2); alloc(&d->rtok, nP * dim * 2);
    alloc(&d->temp, nP * dim * 2);
    // sizes of src/pipeline/render_session.cu:435-444
    const size_t proj_sz = (2 * nP + Sep) * dim, swin_sz = 3 * nP * dim + nWin * nh * ws * ws * ws * ws;
    alloc(&d->proj, (proj_sz > swin_sz ? proj_sz : swin_sz) * 2);
    alloc(&d->qkv, nP * (3 * dim > 2 * ffn ? 3 * dim : 2 * ffn) * 2);
    alloc(&d->ffnb, nP * (dim > ffn ? dim : ffn) * 2);
    alloc(&d->win, nP * dim * 2);
    alloc(&d->score, nh * nP * Sep * 4); alloc(&d->self_score, nWin * nh * ws * ws * ws * ws * 4);
    for (auto& b : d->dft) alloc(&b, nP * dim * 2);
    half *qc, *qs, *ray_pos;
    alloc(&qc, nP * hd * 2); alloc(&qs, nP * hd * 2); alloc(&ray_pos, nP * 18);
    cudaMemset(ray_pos, 0, nP * 18);
    const float id[16] = {1, 0, 0, 0, 0, 1, 0, 0, 0, 0, 1, 0, 0, 0, 0, 1};
    cudaMemcpy(d->id_c2w, id, sizeof(id), cudaMemcpyHostToDevice);
    cublasCreate(&d->blas);
    cudaStreamCreate(&d->stream);
    cublasSetStream(d->blas, d->stream);
    cudaEventCreate(&d->e0); cudaEventCreate(&d->e1);
    cudaHostAlloc(&d->pin_c2w, 64, cudaHostAllocDefault); cudaHostAlloc(&d->pin_fov, 4, cudaHostAllocDefault);
    // query RoPE tables from zero positions (render_session.cu:446-454)
    rf::triangle_rope_freqs(ray_pos, vt_rope_freqs, qc, qs, 1, d->nP, d->nf, d->hd, d->stream);
    d->q_cos = qc; d->q_sin = qs;
    for (int i = 0; i < 16; ++i) d->pin_c2w[i] = id[i];
    d->pin_c2w[11] = 3.0f; *d->pin_fov = 0.7f;
    ref_view_body(*d);  // warm-up: builds the cuDNN attention plan, loads cuBLAS kernels
    cudaStreamSynchronize(d->stream);
    if (use_graph) {
        cudaStreamBeginCapture(d->stream, cudaStreamCaptureModeThreadLocal);
        ref_view_body(*d);
        if (cudaStreamEndCapture(d->stream, &d->graph) != cudaSuccess || !d->graph ||
            cudaGraphInstantiate(&d->exec, d->graph, 0) != cudaSuccess) {
            d->exec = nullptr;  // as the reference: fall back to eager launches
            cudaGetLastError();
        }
    }
    return d;
}

int ref_view_graph_nodes(void* p) {
    auto* d = (RefViewPipeline*)p;
    size_t n = 0;
    if (d->graph) cudaGraphGetNodes(d->graph, nullptr, &n);
    return (int)n;
}

// src/pipeline/render_session.cu:501-513 (render_frame): copy camera, launch, time with events
void ref_view_render(void* p, const float* h_c2w, float fov) {
    auto* d = (RefViewPipeline*)p;
    for (int i = 0; i < 16; ++i) d->pin_c2w[i] = h_c2w[i];
    *d->pin_fov = fov;
    cudaEventRecord(d->e0, d->stream);
    if (d->exec) cudaGraphLaunch(d->exec, d->stream); else ref_view_body(*d);
    cudaEventRecord(d->e1, d->stream);
}
float ref_view_wait(void* p) {
    auto* d = (RefViewPipeline*)p;
    cudaEventSynchronize(d->e1);
    float ms = 0; cudaEventElapsedTime(&ms, d->e0, d->e1);
    return ms;
}
// device pointer of the final token map [nP, dim]
const void* ref_view_result(void* p) { return ((RefViewPipeline*)p)->rtok; }
// device pointers of the four decoder feature taps [nP, dim] (src/pipeline/render_session.cu:235-238)
void ref_view_taps(void* p, const void** out4) {
    auto* d = (RefViewPipeline*)p;
    for (int j = 0; j < 4; ++j) out4[j] = d->dft[j];
}
cudaStream_t ref_view_stream(void* p) { return ((RefViewPipeline*)p)->stream; }
int ref_view_download(void* p, void* h_out, size_t bytes) {
    auto* d = (RefViewPipeline*)p;
    return (int)cudaMemcpyAsync(h_out, d->rtok, bytes, cudaMemcpyDeviceToHost, d->stream) |
           (int)cudaStreamSynchronize(d->stream);
}
void ref_view_destroy(void* p) {
    auto* d = (RefViewPipeline*)p;
    cudaStreamSynchronize(d->stream);
    if (d->exec) cudaGraphExecDestroy(d->exec);
    if (d->graph) cudaGraphDestroy(d->graph);
    for (void* q : d->owned) cudaFree(q);
    cublasDestroy(d->blas); cudaStreamDestroy(d->stream);
    cudaFreeHost(d->pin_c2w); cudaFreeHost(d->pin_fov);
    delete d;
}

}  // extern "C"
