/*
 * rfk_layers.h — C ABI of librfk_layers.so: the launch / fusion boundaries around the
 * rfk kernels (attention and transformer layers), the per-view render session with its
 * CUDA-graph capture, and the hooks a multi-GPU view scheduler needs.
 *
 * The dense contractions stay library calls (cuBLAS GEMMs, as in the reference); every
 * element-wise, normalisation, softmax, rotary and layout step between them is an rfk
 * kernel (include/rfk.h), fused across the boundaries the reference leaves open.
 *
 * Conventions are those of rfk.h (int status, device pointers, stream last). Functions
 * taking an rfk_ctx use its cuBLAS handle and workspace; one rfk_ctx per device and per
 * host thread. Nothing here allocates on the launch path: all device memory is allocated
 * by rfk_ctx_create / rfk_session_create or supplied by the caller, so every call made
 * after creation can be captured in a CUDA graph.
 *
 * "replaces" comments name the reference interface (BANANASJIM/renderformer-cuda, paths
 * relative to that project).
 */
#ifndef RFK_LAYERS_H
#define RFK_LAYERS_H

#include "rfk.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct rfk_ctx rfk_ctx;          /* per-device cuBLAS handle + workspace      */
typedef struct rfk_session rfk_session;  /* per-device, per-scene render session      */

/* Creates the context on the current CUDA device (allocates a 64 MiB cuBLAS workspace).
 * replaces rf::CublasHandle — src/core/cuda_utils.h:50-59 */
int rfk_ctx_create(rfk_ctx** out);
int rfk_ctx_destroy(rfk_ctx* ctx);
/* Gives the context the workspace of rfk_flash_attention_ex's key split (rfk.h; about 21 MB, allocated here,
 * freed by rfk_ctx_destroy): the attention inside the layer functions called with this context then uses it. The
 * workspace is shared by all of them, so their launches must not overlap in time (one stream, or streams ordered
 * by events); rfk_session_create does this for the session's own context. No reference counterpart. */
int rfk_ctx_reserve_attention_workspace(rfk_ctx* ctx);

/* ------------------------------------------------------------- weight records */

/* replaces rf::FFNWeights — src/layers/transformer.h:9-13. If w3 == w1 + hidden*dim (the
 * two matrices stored back to back) the gate and up projections run as one GEMM. */
typedef struct {
    const rfk_half* w1;  /* [hidden, dim] */
    const rfk_half* w2;  /* [dim, hidden] */
    const rfk_half* w3;  /* [hidden, dim] */
} rfk_ffn_weights;

/* replaces rf::MHAWeights and rf::SwinAttnWeights (same fields) —
 * src/layers/attention.h:23-30, 84-91 */
typedef struct {
    const rfk_half* in_proj_w;   /* [3*dim, dim] */
    const rfk_half* in_proj_b;   /* [3*dim] or NULL */
    const rfk_half* out_proj_w;  /* [dim, dim] */
    const rfk_half* out_proj_b;  /* [dim] or NULL */
    const float* q_norm_gamma;   /* [dim] or NULL */
    const float* k_norm_gamma;   /* [dim] or NULL */
} rfk_mha_weights;

/* replaces rf::CrossAttnWeights — src/layers/attention.h:40-51 */
typedef struct {
    const rfk_half* q_proj_w;   const rfk_half* q_proj_b;
    const rfk_half* k_proj_w;   const rfk_half* k_proj_b;
    const rfk_half* v_proj_w;   const rfk_half* v_proj_b;
    const rfk_half* out_proj_w; const rfk_half* out_proj_b;
    const float* q_norm_gamma;  const float* k_norm_gamma;
} rfk_cross_attn_weights;

/* replaces rf::EncoderLayerWeights — src/layers/transformer.h:16-21 */
typedef struct {
    const float* query_norm_gamma;
    rfk_mha_weights attn;
    const float* ffn_norm_gamma;
    rfk_ffn_weights ffn;
} rfk_encoder_layer_weights;

/* replaces rf::DecoderLayerWeights — src/layers/transformer.h:24-32 */
typedef struct {
    const float* query_norm_gamma;
    const float* kv_norm_gamma;
    rfk_cross_attn_weights cross_attn;
    const float* self_attn_norm_gamma;
    rfk_mha_weights self_attn;
    const float* ffn_norm_gamma;
    rfk_ffn_weights ffn;
} rfk_decoder_layer_weights;

/* ------------------------------------------------------------------- layers */

/* Y[M,N] = X[M,K] W[N,K]^T (+ bias[N]); fp16 in/out, fp32 accumulation (cuBLAS).
 * replaces rf::linear — src/layers/linear.h:9, linear.cu:7-25 */
int rfk_linear(rfk_ctx* ctx, const rfk_half* X, const rfk_half* W, const rfk_half* bias,
               rfk_half* Y, int M, int N, int K, rfk_stream_t stream);

/* out[M,dim] = W2 (silu(W1 x) * (W3 x)); buf holds [M, 2*hidden] halves.
 * One or two GEMMs into a gate|up buffer, the SwiGLU gate kernel, one GEMM.
 * replaces rf::ffn_swiglu — src/layers/transformer.h:118, transformer.cu:63-79 */
int rfk_ffn_swiglu(rfk_ctx* ctx, const rfk_ffn_weights* w, const rfk_half* x, rfk_half* out,
                   rfk_half* buf, int M, int dim, int hidden, rfk_stream_t stream);

/* Scaled dot-product attention on [B,H,S,D] fp16 tensors, scale 1/sqrt(D):
 * batched GEMM into fp32 scores, rfk softmax (probabilities written as fp16 over the first
 * half of each score row), batched GEMM. Any Sk is accepted; score rows have a pitch of
 * roundup8(Sk) floats, and roundup8(Sk) must not exceed 8192 (the softmax keeps a row in
 * registers; larger shapes return RFK_EUNSUPPORTED before anything is launched).
 *   workspace: B*H*Sq*roundup8(Sk) floats.
 *   n_keys: keys that take part in the softmax (<= Sk); keys [n_keys, Sk) get probability 0.
 *           n_keys == Sk reproduces the reference, which attends its zero pad keys.
 *   o_bshd != 0: O is written as [B,Sq,H*D] (saves the transpose that follows).
 * replaces the cuBLAS + softmax_cast_fp16 path of rf::sdpa — src/layers/attention.cu:112-165
 * (the reference's first choice, cuDNN fused SDPA, attention.cu:97-110, computes the same
 * function without materialising the scores). mask must be NULL or [B,Sk] bytes. */
int rfk_sdpa(rfk_ctx* ctx, const rfk_half* Q, const rfk_half* K, const rfk_half* V, rfk_half* O,
             float* workspace, const uint8_t* mask, int B, int H, int Sq, int Sk, int n_keys,
             int D, int o_bshd, rfk_stream_t stream);

/* rfk_sdpa for callers that cannot allocate device memory (code running inside a CUDA stream
 * capture, stream host callbacks, plug-in hosts with a fixed memory budget): the fp32 score
 * matrix lives in a 32 MiB array inside the library instead of a caller-supplied workspace,
 * so B*H*Sq*roundup8(Sk) must not exceed 8 Mi (8388608) floats; larger shapes return
 * RFK_ETOOBIG (and roundup8(Sk) > 8192 returns RFK_EUNSUPPORTED, as for rfk_sdpa). The device
 * that is current at the call must be the one ctx was created on (RFK_EINVAL otherwise).
 * The call allocates and frees nothing. The first call on each device looks up
 * the array's device address (cudaGetSymbolAddress, with that device current) and should
 * therefore be made before any stream capture begins; later calls only launch. All calls on
 * a device share the one array: it keeps the previous call's contents (no call depends on
 * them), and two calls whose work overlaps on the GPU (different streams) race on it.
 * This entry point has no counterpart in the reference, whose attention allocates per call. */
int rfk_sdpa_static(rfk_ctx* ctx, const rfk_half* Q, const rfk_half* K, const rfk_half* V,
                    rfk_half* O, int B, int H, int Sq, int Sk, int n_keys, int D, int o_bshd,
                    rfk_stream_t stream);

/* K/V projections of the (normalised) context, K-RMSNorm, [B,H,Sk_pad,D] layout with rows
 * [Sk, Sk_pad) zeroed. proj_buf: 2*B*Sk*dim halves.
 * replaces rf::precompute_cross_kv + the per-head padding copies —
 * src/layers/attention.cu:302-324, src/pipeline/render_session.cu:395-414 */
int rfk_precompute_cross_kv(rfk_ctx* ctx, const rfk_cross_attn_weights* w,
                            const rfk_half* ctx_normed, rfk_half* K_out, rfk_half* V_out,
                            rfk_half* proj_buf, int B, int Sk, int Sk_pad, int kv_dim, int dim,
                            int num_heads, rfk_stream_t stream);

/* Cross-attention of q_in [B*Sq, q_dim] against cached K/V [B,H,Sk,D] (Sk a multiple of 8).
 * proj_buf: (2*B*Sq*dim + max(B*Sq*dim, B*H*Sk*D)) halves (the third region holds the rotated
 * keys and, for shapes the fused Q epilogue does not serve, a [B*Sq, dim] staging copy); score_buf: B*H*Sq*Sk floats, or NULL when the head
 * size is 64 or 128 (rfk_flash_attention then serves the attention and no score matrix exists;
 * with NULL any other head size returns RFK_EINVAL). The same holds for every score buffer below;
 * the swin score buffer may be NULL for 64-token windows of 64-wide heads.
 * Fusions: Q-RMSNorm + transpose + RoPE in one kernel; cached-K copy + RoPE in one kernel;
 * softmax writes fp16 in place; the PV GEMM writes [B,Sq,dim] directly.
 * replaces rf::cross_attention_cached — src/layers/attention.h:70-82, attention.cu:326-373 */
int rfk_cross_attention_cached(rfk_ctx* ctx, const rfk_cross_attn_weights* w,
                               const rfk_half* q_in, rfk_half* out, rfk_half* proj_buf,
                               float* score_buf, const rfk_half* K_cached,
                               const rfk_half* V_cached, int B, int Sq, int Sk, int n_keys,
                               int q_dim, int dim, int num_heads,
                               const rfk_half* q_rope_cos, const rfk_half* q_rope_sin,
                               const rfk_half* k_rope_cos, const rfk_half* k_rope_sin,
                               rfk_stream_t stream);

/* Shifted-window self-attention on an [B,H,W,dim] token map.
 *   window_buf: B*H*W*dim halves; qkv_buf: 3*B*H*W*dim halves; scratch: 3*B*H*W*dim halves;
 *   score_buf: B*nW*heads*ws^4 floats; shift_mask [nW, ws^2, ws^2] bytes (used when shift > 0).
 * If residual_x != NULL the result is added into residual_x (fp16 residual add fused with the
 * window reverse + un-shift) and `out` is not written; otherwise out receives the result.
 * replaces rf::swin_self_attention (+ residual_add) — src/layers/attention.h:95-102,
 * attention.cu:476-576, src/layers/transformer.cu:183-188 */
int rfk_swin_self_attention(rfk_ctx* ctx, const rfk_mha_weights* w, const rfk_half* x,
                            rfk_half* out, rfk_half* residual_x, rfk_half* window_buf,
                            rfk_half* qkv_buf, float* score_buf, rfk_half* scratch, int B, int H,
                            int W, int dim, int num_heads, int window_size, int shift_size,
                            const uint8_t* shift_mask, rfk_stream_t stream);

/* Self-attention with packed QKV projection on [B,S,dim] (encoder). score_buf:
 * B*H*S*S_pad floats (S_pad = S rounded up to 8); qkv_buf: B*S*3*dim halves + 3*B*H*S_pad*D.
 * replaces rf::self_attention — src/layers/attention.h:32-37, attention.cu:170-231 */
int rfk_self_attention(rfk_ctx* ctx, const rfk_mha_weights* w, const rfk_half* x, rfk_half* out,
                       rfk_half* qkv_buf, float* score_buf, int B, int S, int dim, int num_heads,
                       const rfk_half* rope_cos, const rfk_half* rope_sin, rfk_stream_t stream);

/* One decoder layer with cached cross-attention K/V, in place on x [B*Sq, dim] fp16.
 * Buffer minimums (halves unless noted), Mq = B*Sq:
 *   temp Mq*dim; proj_buf max(2*Mq*dim + B*heads*Sk*hd, 3*Mq*dim); qkv_buf Mq*max(3*dim, 2*ffn);
 *   ffn_buf Mq*max(dim, ffn); window_buf Mq*dim; cross_score_buf B*heads*Sq*Sk floats;
 *   self_score_buf B*nW*heads*ws^4 floats.
 * pending_residual: if non-NULL, a sub-layer output of the PREVIOUS layer that has not been
 * added to x yet; it is added by this layer's first fused residual+RMSNorm kernel.
 * On return *pending_out (if pending_out != NULL) names a sub-layer output of this layer that
 * is not yet added to x (the caller passes it to the next layer, or adds it with
 * rfk_residual_add), or is NULL when x is complete: the decoder layer adds its FFN output in the
 * epilogue of the last projection and always returns NULL; the encoder layer defers it.
 * With pending_out == NULL x is complete on return.
 * replaces rf::decoder_layer_forward_cached — src/layers/transformer.h:88-103,
 * transformer.cu:151-194 */
int rfk_decoder_layer_forward_cached(rfk_ctx* ctx, const rfk_decoder_layer_weights* w,
                                     rfk_half* x, const rfk_half* pending_residual,
                                     const rfk_half** pending_out, rfk_half* temp,
                                     rfk_half* proj_buf, rfk_half* qkv_buf, rfk_half* ffn_buf,
                                     rfk_half* window_buf, float* cross_score_buf,
                                     float* self_score_buf, const rfk_half* K_cached,
                                     const rfk_half* V_cached, int B, int Sq, int Sk, int n_keys,
                                     int dim, int num_heads, int ffn_hidden, int patch_h,
                                     int patch_w, int window_size, int shift_size,
                                     const uint8_t* shift_mask, const rfk_half* q_rope_cos,
                                     const rfk_half* q_rope_sin, const rfk_half* k_rope_cos,
                                     const rfk_half* k_rope_sin, rfk_stream_t stream);

/* One encoder layer with an fp32 hidden state and fp16 sub-layers, in place on x [B*S, dim].
 * temp: B*S*dim halves; qkv_buf: as rfk_self_attention, at least B*S*2*ffn halves;
 * ffn_buf: B*S*max(dim, ffn) halves; score_buf: as rfk_self_attention.
 * Same pending-residual protocol as the decoder layer (fp16 sub-layer output added to the
 * fp32 hidden state by the next fused residual+RMSNorm+cast kernel).
 * replaces rf::encoder_layer_forward_mixed — src/layers/transformer.h:48-57,
 * transformer.cu:196-224 */
int rfk_encoder_layer_forward_mixed(rfk_ctx* ctx, const rfk_encoder_layer_weights* w, float* x,
                                    const rfk_half* pending_residual,
                                    const rfk_half** pending_out, rfk_half* temp,
                                    rfk_half* qkv_buf, rfk_half* ffn_buf, float* score_buf, int B,
                                    int S, int dim, int num_heads, int ffn_hidden,
                                    const rfk_half* rope_cos, const rfk_half* rope_sin,
                                    rfk_stream_t stream);

/* ------------------------------------------------------------ DPT image head */

/* replaces rf::RCUWeights / rf::FFBWeights / rf::DPTWeights — src/layers/dpt.h:36-62 (device pointers;
 * convolution weights [Cout, Cin, kH, kW] fp16, biases [Cout] fp16), with the head's shape
 * parameters (rf::Config::dpt_features / dpt_out_dim / dpt_out_channels, src/model/config.h:38-42)
 * carried in the record instead of compiled in. */
typedef struct {
    const rfk_half* conv1_w; const rfk_half* conv1_b;   /* [F, F, 3, 3], [F] */
    const rfk_half* conv2_w; const rfk_half* conv2_b;
} rfk_rcu_weights;
typedef struct {
    rfk_rcu_weights rcu1;        /* used only when has_resconv1 != 0 */
    rfk_rcu_weights rcu2;
    const rfk_half* out_conv_w;  /* [F, F, 1, 1] */
    const rfk_half* out_conv_b;
    int has_resconv1;
} rfk_ffb_weights;
typedef struct {
    const rfk_half* project_w[4];   /* [out_channels[i], dim, 1, 1] */
    const rfk_half* project_b[4];
    const rfk_half* resize_w[4];    /* 0: transposed 4x4 stride 4, 1: transposed 2x2 stride 2, 2: none (NULL), 3: 3x3 stride 2 */
    const rfk_half* resize_b[4];
    const rfk_half* layer_rn_w[4];  /* [features_dim, out_channels[i], 3, 3], no bias */
    rfk_ffb_weights refinenet[4];
    const rfk_half* output_conv1_w;  const rfk_half* output_conv1_b;   /* [F/2, F, 3, 3] */
    const rfk_half* output_conv2a_w; const rfk_half* output_conv2a_b;  /* [32, F/2, 3, 3] */
    const rfk_half* output_conv2b_w; const rfk_half* output_conv2b_b;  /* [out_dim, 32, 1, 1] */
    int features_dim, out_dim;
    int out_channels[4];
} rfk_dpt_weights;

typedef struct rfk_dpt rfk_dpt;  /* a planned head: buffers, cuDNN descriptors and algorithms, the list of steps */

/* Plans the head for B images of patch_h x patch_w tokens of width dim (image patch_h*patch_size x
 * patch_w*patch_size): sizes and allocates every intermediate, creates a cuDNN handle, chooses the
 * convolution algorithms and allocates one workspace. Everything that allocates happens here.
 * replaces the cudaMallocAsync / cudaFreeAsync calls and the lazy plan cache of rf::dpt_forward /
 * rf::conv2d — src/layers/dpt.cu:23-47,130-160,329-337 */
int rfk_dpt_create(rfk_ctx* ctx, const rfk_dpt_weights* w, int B, int dim, int patch_h, int patch_w,
                   int patch_size, rfk_dpt** out);
int rfk_dpt_destroy(rfk_dpt* dpt);
/* features: HOST array of 4 device pointers, the decoder feature taps [B, patch_h*patch_w, dim]
 * fp16. Writes the image [B, out_dim, H, W] fp16 (before the ELU / 10^x - 1 post-process) into the
 * plan's own buffer (rfk_dpt_output) and, if image_out != NULL, copies it there. Launch-only:
 * capturable. cuDNN convolutions for k > 1 and the transposed ones, cuBLAS for 1x1 (as the
 * reference), rfk kernels for permute / bias / SiLU / residual / bilinear upsampling.
 * replaces rf::dpt_forward — src/layers/dpt.h:64-72, src/layers/dpt.cu:322-461 */
int rfk_dpt_forward(rfk_dpt* dpt, const rfk_half* const* features, rfk_half* image_out,
                    rfk_stream_t stream);
const rfk_half* rfk_dpt_output(rfk_dpt* dpt);
int rfk_dpt_num_convolutions(rfk_dpt* dpt);

/* ------------------------------------------------------------ render session */

#define RFK_MAX_LAYERS 32

/* Model record (device pointers): the fields of rf::RenderFormerModel
 * (src/model/renderformer.h:12-44) without the DPT head, with runtime shapes in place of
 * the compile-time rf::Config (src/model/config.h:6-43). */
typedef struct {
    int dim, num_heads, ffn_hidden, num_register_tokens;
    int enc_layers, dec_layers;
    int rope_num_freqs;          /* frequencies per coordinate: 9*nf <= head_dim/2 */
    int patch_size, window_size, shift_size;
    int texture_channels;        /* 13 */
    int vn_pe_num_freqs;         /* 6  */
    const rfk_half* tri_token;   /* [dim] */
    const rfk_half* reg_tokens;  /* [num_register_tokens, dim] */
    const rfk_half* tex_enc_w;   const rfk_half* tex_enc_b;  const float* tex_enc_norm;
    const rfk_half* vn_proj_w;   const rfk_half* vn_proj_b;  const float* vn_enc_norm;
    const float* enc_rope_freqs;
    const rfk_half* ray_map_patch_token;
    const rfk_half* ray_enc_w;   const rfk_half* ray_enc_b;  const float* ray_enc_norm;
    const float* vt_rope_freqs;
    rfk_encoder_layer_weights enc[RFK_MAX_LAYERS];
    rfk_decoder_layer_weights dec[RFK_MAX_LAYERS];
    const rfk_dpt_weights* dpt;  /* HOST pointer, read at rfk_session_create; NULL: the view ends at the token map.
                                    Otherwise the captured view continues through the DPT head and the image
                                    post-process (rf::RenderFormerModel::dpt, src/model/renderformer.h:43-44;
                                    render_session.cu:239-253) */
} rfk_model;

enum {
    RFK_SESSION_PAD_KEYS_ATTEND = 1,  /* reproduce the reference: zero pad keys take part in the
                                         cross-attention softmax (render_session.cu:229-230) */
    RFK_SESSION_NO_GRAPH        = 2   /* launch eagerly instead of replaying a CUDA graph */
};

/* Bytes of the scene state of an n_tris scene: the encoder's cross-attention K/V cache
 * [dec_layers][2][heads][Se_pad][head_dim] fp16 followed by the fp16 triangles, the fp16
 * vertex normals and the fp32 scene centre. This is the blob a view scheduler broadcasts. */
size_t rfk_scene_state_bytes(const rfk_model* model, int n_tris);

/* Creates a session on the current device for `n_tris` triangles at img_res x img_res.
 * scene_state: caller-owned device buffer of rfk_scene_state_bytes() bytes (filled either by
 * rfk_session_encode_scene on this device or by a broadcast from the device that ran it).
 * Allocates every per-view buffer; runs nothing.
 * replaces the allocation half of rf::RenderSession::create — src/pipeline/render_session.cu:258-295,418-462 */
int rfk_session_create(const rfk_model* model, int n_tris, int img_res, void* scene_state,
                       int flags, rfk_session** out);
/* The same with views_per_frame (1..64) views rendered together: a frame is then a batch of that many views of the
 * scene, each with its own camera, that go through the decoder as one batch (rfk_session_render_frames). Throughput
 * mode: the projections see views_per_frame times the rows and the cross-attention that many times the work units,
 * which is what fills all SMs evenly (four views at 512 x 512: 1024 units on 148 SMs instead of 256); a frame's
 * results are the views' results back to back, bit-identical to rendering them one by one. Needs the fused attention
 * route (head size 64, dim % 256 == 0, QK-norm weights present): RFK_EUNSUPPORTED otherwise. No reference counterpart
 * (the reference renders one view at a time, render_session.cu:501-548). */
int rfk_session_create_batched(const rfk_model* model, int n_tris, int img_res, void* scene_state, int flags,
                               int views_per_frame, rfk_session** out);
int rfk_session_views_per_frame(rfk_session* s);
int rfk_session_destroy(rfk_session* s);

/* Scene preprocessing, 12-layer encoder and K/V cache build into the scene state.
 * tri, vn: [n_tris,3,3] fp32 world space; tex: [n_tris, texture_channels] fp16 (first texel
 * of each channel; the last 3 channels are log-encoded here). Synchronises at the end.
 * replaces the compute half of rf::RenderSession::create — render_session.cu:296-416 */
int rfk_session_encode_scene(rfk_session* s, const float* tri, const float* vn,
                             const rfk_half* tex);

/* Builds the per-session constants (query RoPE tables, shift mask), runs one warm-up view and
 * captures the per-view CUDA graph. Call after the scene state is complete on this device.
 * replaces render_session.cu:430-495 */
int rfk_session_finalize(rfk_session* s);

/* Renders one view asynchronously on the session's stream: copies c2w (16 floats, row-major,
 * HOST) and fov (radians) into pinned staging memory and launches the captured graph.
 * The session has two frame slots (pinned camera, graph instance, result buffer each), so the
 * call returns at once unless the frame submitted two calls ago is still running or
 * downloading: the host can stay one frame ahead of the device.
 * replaces rf::RenderSession::render_frame_async — render_session.cu:515-527 */
int rfk_session_render_frame(rfk_session* s, const float* h_c2w, float fov_rad);
/* One frame of a session created with views_per_frame = V: h_c2w [V][16] and fov_rad [V] (HOST). Results, feature
 * taps and images of the frame hold the V views back to back ([V, tokens, dim], [V, channels, res, res]); the download
 * calls copy all of them (bytes >= V times the single-view size). rfk_session_render_frame is this call for V = 1 and
 * returns RFK_EINVAL on a session with V > 1. */
int rfk_session_render_frames(rfk_session* s, const float* h_c2w, const float* fov_rad);
/* Blocks until the last submitted frame is done; *ms (optional) receives its device time.
 * replaces rf::RenderSession::get_frame_result — render_session.cu:539-548 */
int rfk_session_wait(rfk_session* s, float* ms);
/* Device pointer and shape of the last frame's result: the decoder's final token map
 * [(img_res/patch)^2, dim] fp16 (the DPT image head is outside this library). */
int rfk_session_result(rfk_session* s, const rfk_half** tokens, int* n_tokens, int* dim);
/* Device pointers of the 4 decoder feature taps a DPT head consumes (layers at 1/4, 1/2, 3/4
 * and the end of the stack; render_session.cu:235-238), for the LAST submitted frame. Each of
 * the two frame slots has its own set of taps: the pointers stay valid, and their contents
 * untouched, until the second rfk_session_render_frame call after the one that produced them
 * (the same lifetime as the slot's result buffer). The frame must have completed
 * (rfk_session_wait) before a consumer on another stream reads them. */
int rfk_session_feature_taps(rfk_session* s, const rfk_half** taps /* HOST array of 4 */);
/* With a DPT head in the model: device pointer and shape of the last frame's image
 * [channels, img_res, img_res] fp32 after ELU(1e-3) and 10^x - 1 (what rf::RenderSession::
 * download_frame_hwc reads, planar instead of interleaved) — render_session.cu:249-253, 550-559.
 * RFK_EINVAL without a head. rfk_session_download_image copies it to HOST memory (waits for the frame). */
int rfk_session_image(rfk_session* s, const float** image, int* channels, int* img_res);
int rfk_session_download_image(rfk_session* s, float* h_out, size_t bytes);
/* Copies the last frame's token map to HOST memory (waits for the frame).
 * replaces rf::RenderSession::download_frame_hwc — render_session.cu:550-559 */
int rfk_session_download(rfk_session* s, rfk_half* h_out, size_t bytes);
/* Queues the device->host copy of the last submitted frame's token map on the session's copy
 * stream (h_out should be pinned); it runs as soon as that frame is done, overlapping the
 * next frame. rfk_session_drain waits for every submitted frame and copy and returns RFK_EKERNEL if
 * the fused attention kernel has reported a time-out since its error word was last cleared
 * (rfk_flash_attention_error); rfk_session_finalize makes the same check after its warm-up view. */
int rfk_session_download_async(rfk_session* s, rfk_half* h_out, size_t bytes);
int rfk_session_drain(rfk_session* s);
/* Timing marks: mark_begin records a CUDA event on the session's render stream; mark_end
 * records a second one, waits for it (and for the copy stream) and returns the device time
 * between the two in *ms. Brackets a batch of rfk_session_render_frame calls. */
int rfk_session_mark_begin(rfk_session* s);
int rfk_session_mark_end(rfk_session* s, float* ms);
/* Number of nodes in the captured per-view graph (0 when running eagerly). */
int rfk_session_graph_nodes(rfk_session* s);
/* Kernels of librfk.so launched per view (counted while the graph was captured). */
int rfk_session_kernels_per_view(rfk_session* s);

#ifdef __cplusplus
}
#endif
#endif /* RFK_LAYERS_H */
