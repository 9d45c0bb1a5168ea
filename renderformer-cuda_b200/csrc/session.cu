// Per-scene render session: scene encoding (once), per-view front end + decoder stack
// captured as a CUDA graph, double-buffered frame slots so the host can stay one frame
// ahead of the device.
//
// Reference: src/pipeline/render_session.cu (BANANASJIM/renderformer-cuda)
//   :177-254  render_view            (the captured per-view work)
//   :258-416  create: preprocessing, encoder, K/V cache
//   :418-495  create: buffers, constants, warm-up, graph capture
//   :501-559  render_frame / async API / download
// Differences that matter:
//   - the per-view geometry front end is one kernel (rfk_view_geometry) instead of three
//     device-to-device copies and three launches; rays are generated directly as patch tokens;
//   - nothing inside the captured region allocates (the reference's DPT head and attention
//     fall-back call cudaMallocAsync while capturing);
//   - two frame slots (pinned camera + result buffer + graph instance each): frame i+1 can be
//     submitted while frame i renders and frame i-1 downloads;
//   - the query RoPE tables are built from all-zero positions in the reference
//     (render_session.cu:446-454), i.e. cos = 1 and sin = 0 exactly; rotating by them returns
//     the input bit for bit, so the query rotation is skipped;
//   - the DPT convolution head and the image post-process are outside this library: the frame
//     result is the decoder's final token map plus the four feature taps a DPT head reads.
#include "layers_internal.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <vector>

using namespace rfk_layers;

#define TRY(expr)                       \
    do {                                \
        int rc_ = (expr);               \
        if (rc_ != RFK_OK) return rc_;  \
    } while (0)
#define TRY_CUDA(expr)                          \
    do {                                        \
        cudaError_t e_ = (expr);                \
        if (e_ != cudaSuccess) return (int)e_;  \
    } while (0)

namespace {

constexpr int kSlots = 2;

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct StateLayout {
    size_t kv_layer_bytes;  // one K (or V) cache of one layer: [heads, Se_pad, hd] fp16
    size_t kv_off, tri_off, vn_off, center_off, total;
};

StateLayout state_layout(const rfk_model& m, int n_tris) {
    const int Se_pad = (m.num_register_tokens + n_tris + 7) & ~7;
    StateLayout L{};
    L.kv_layer_bytes = (size_t)Se_pad * m.dim * sizeof(__half);
    L.kv_off = 0;
    L.tri_off = align_up(L.kv_off + 2 * (size_t)m.dec_layers * L.kv_layer_bytes, 256);
    L.vn_off = align_up(L.tri_off + (size_t)n_tris * 9 * sizeof(__half), 256);
    L.center_off = align_up(L.vn_off + (size_t)n_tris * 9 * sizeof(__half), 256);
    L.total = align_up(L.center_off + 3 * sizeof(float), 256);
    return L;
}

// last `last_n` channels of each row: v <- half(log10f(float(v) + 1))   (render_session.cu:33-38)
__global__ void log_encode_kernel(__half* data, int N, int C, int last_n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= N * last_n) return;
    const int n = i / last_n, idx = n * C + (C - last_n) + (i % last_n);
    data[idx] = __float2half(log10f(__half2float(data[idx]) + 1.0f));
}

// out = a + b + float(c[i % dim])   (render_session.cu:39-43)
__global__ void add3_bc_kernel(float* out, const float* a, const float* b, const __half* c, long long n, int dim) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = a[i] + b[i] + __half2float(c[i % dim]);
}

inline unsigned blocks_for(long long n) { return (unsigned)((n + 255) / 256); }

// Attention mask of the shifted windows, [windows, ws*ws, ws*ws] bytes. After the cyclic shift
// the token at row y of the shifted map is the token of row (y + shift) mod extent of the
// unshifted one (columns alike). Two tokens of a window may see each other only if both came
// out of the same ws x ws cell of the unshifted map; since a cell is a product of a row band
// and a column band, the test separates per axis. (The reference states the same rule through
// one region number per token, src/pipeline/render_session.cu:99-116.)
std::vector<uint8_t> build_window_mask(int rows, int cols, int ws, int shift) {
    const int win_y = rows / ws, win_x = cols / ws, T = ws * ws;
    const auto band = [ws, shift](int p, int extent) { return ((p + shift) % extent) / ws; };
    std::vector<uint8_t> mask((size_t)win_y * win_x * T * T);
    std::vector<int> by(T), bx(T);
    uint8_t* out = mask.data();
    for (int wy = 0; wy < win_y; ++wy)
        for (int wx = 0; wx < win_x; ++wx) {
            for (int t = 0; t < T; ++t) {
                by[t] = band(wy * ws + t / ws, rows);
                bx[t] = band(wx * ws + t % ws, cols);
            }
            for (int q = 0; q < T; ++q)
                for (int k = 0; k < T; ++k) *out++ = (uint8_t)((by[q] == by[k]) & (bx[q] == bx[k]));
        }
    return mask;
}

}  // namespace

struct rfk_session {
    rfk_model m{};
    int N = 0, res = 0, Se = 0, Se_pad = 0, pH = 0, pW = 0, nP = 0, hd = 0, flags = 0;
    int V = 1;  // views per frame: a frame is V views of the scene rendered together as one batch (see render_view)
    rfk_ctx* ctx = nullptr;
    cudaStream_t stream = nullptr, copy_stream = nullptr, side_stream = nullptr;
    StateLayout L{};
    char* state = nullptr;  // caller-owned scene state
    std::vector<void*> owned;  // device allocations of this session

    // per-view buffers
    float* cam_gpu = nullptr;  // per view [16 c2w | 1 fov | pad to kCamStride]
    float* id_c2w = nullptr;
    rfk_half *vtri = nullptr, *vvn = nullptr, *vpos = nullptr, *k_cos = nullptr, *k_sin = nullptr;
    rfk_half *ray_pat = nullptr, *rtok = nullptr;
    rfk_half *temp = nullptr, *proj = nullptr, *qkv = nullptr, *ffn = nullptr, *win = nullptr;
    float *score = nullptr, *self_score = nullptr;  // only allocated when a materialised attention path can be taken
    rfk_half* k_rot = nullptr;  // [dec_layers][heads][Se_pad][hd]: this view's rotated keys of every layer
    float* q_gamma_all = nullptr;  // [dec_layers][dim]: the cross-attention query norm weights, contiguous
    bool prescale = false;         // the rotation multiplies the keys by those weights (deferred Q-RMSNorm, see layers.cu)
    cudaEvent_t ev_fork = nullptr, ev_rot[RFK_MAX_LAYERS]{};
    uint8_t* shift_mask = nullptr;
    rfk_half* dft[kSlots][4] = {};  // the four decoder feature taps of each frame slot
    rfk_dpt_weights dptw{};          // copy of the model's DPT record (if any)
    rfk_dpt* dpt = nullptr;          // planned image head; null: the view ends at the token map
    float* image[kSlots] = {nullptr, nullptr};  // [out_dim, res, res] fp32 after the post-process
    rfk_half* result[kSlots] = {nullptr, nullptr};

    // frame slots
    float* pin_cam[kSlots] = {nullptr, nullptr};  // pinned [16 c2w | fov]
    cudaGraph_t graph[kSlots] = {nullptr, nullptr};
    cudaGraphExec_t exec[kSlots] = {nullptr, nullptr};
    cudaEvent_t ev_start[kSlots]{}, ev_done[kSlots]{}, ev_dl[kSlots]{};
    bool dl_pending[kSlots] = {false, false};
    cudaEvent_t ev_mark0 = nullptr, ev_mark1 = nullptr;
    long long frames = 0;  // frames submitted so far
    int graph_nodes = 0, kernels_per_view = 0;
    bool finalized = false;

    rfk_half* kvK(int layer) const { return (rfk_half*)(state + L.kv_off + (size_t)(2 * layer) * L.kv_layer_bytes); }
    // rotated keys: [dec_layers][V][heads][Se_pad][hd], so that a layer's keys are one [V * heads, Se_pad, hd] batch
    rfk_half* kRot(int layer, int view = 0) const { return k_rot + ((size_t)layer * V + view) * m.num_heads * Se_pad * hd; }
    rfk_half* kvV(int layer) const { return (rfk_half*)(state + L.kv_off + (size_t)(2 * layer + 1) * L.kv_layer_bytes); }
    rfk_half* tri16() const { return (rfk_half*)(state + L.tri_off); }
    rfk_half* vn16() const { return (rfk_half*)(state + L.vn_off); }
    float* center() const { return (float*)(state + L.center_off); }

    template <typename T> int alloc(T** p, size_t count) {
        void* d = nullptr;
        cudaError_t e = cudaMalloc(&d, std::max<size_t>(count * sizeof(T), 256));
        if (e != cudaSuccess) return (int)e;
        owned.push_back(d);
        *p = (T*)d;
        return RFK_OK;
    }

    int render_view(const float* pinned_cam, rfk_half* result_out, rfk_half* const* taps_out, float* image_out);
};

// The work of one frame = V views; everything here is captured into the graph. The views of a frame go through the
// decoder as one batch: every projection sees V * nP rows, the cross-attention V * heads * nP / 256 units of work (with
// V = 4 at 512 x 512 that is 1024 units on 148 SMs, 6.9 rounds instead of the 1.7 of a single view, whose second,
// partial round leaves 14 % of the machine idle), the window attention V * nW windows. Each view has its own camera,
// geometry, rotary tables and rotated keys; the values of the K/V cache are shared by the batch.
constexpr int kCamStride = 32;  // floats per view in the camera buffers
int rfk_session::render_view(const float* pinned_cam, rfk_half* result_out, rfk_half* const* taps_out, float* image_out) {
    rfk_stream_t s = (rfk_stream_t)stream;
    const int dim = m.dim, nr = m.num_register_tokens, ps = m.patch_size;
    const size_t tri_n = (size_t)N * 9, pos_n = (size_t)Se_pad * 9, tab_n = (size_t)Se_pad * hd;
    const size_t pat_n = (size_t)nP * 3 * ps * ps;
    TRY_CUDA(cudaMemcpyAsync(cam_gpu, pinned_cam, (size_t)V * kCamStride * sizeof(float), cudaMemcpyHostToDevice, stream));
    // world -> camera of triangles and normals, register-token positions, K RoPE tables (per view)
    for (int v = 0; v < V; ++v)
        TRY(rfk_view_geometry(cam_gpu + v * kCamStride, tri16(), vn16(), center(), m.vt_rope_freqs, vtri + v * tri_n, vvn + v * tri_n,
                              vpos + v * pos_n, k_cos + v * tab_n, k_sin + v * tab_n, N, nr, Se_pad, m.rope_num_freqs, hd, s));
    // The rotation of the cached keys by a view's tables is the same for every query and independent of the
    // layers' data flow, so it runs on a second stream (a parallel branch of the graph) while the front end and the
    // first layer's projections run. Two launches per view: layer 0 alone (the first attention waits only for 23 MB of
    // work per view), then all remaining layers at once (one shared table, batch = layers, source stride = a K and a
    // V slab, destination stride = the V views of a layer).
    TRY_CUDA(cudaEventRecord(ev_fork, stream));
    TRY_CUDA(cudaStreamWaitEvent(side_stream, ev_fork, 0));
    {
        const long long slab = (long long)(L.kv_layer_bytes / sizeof(__half));
        const long long rot_slab = (long long)m.num_heads * Se_pad * hd;
        const float* g0 = prescale ? q_gamma_all : nullptr;
        for (int v = 0; v < V; ++v)
            TRY(rfk_rope_one_oop_strided(kvK(0), kRot(0, v), k_cos + v * tab_n, k_sin + v * tab_n, 1, 2 * slab, rot_slab, 0,
                                         m.num_heads, Se_pad, hd, Se_pad, Se_pad, g0, 0, (rfk_stream_t)side_stream));
        TRY_CUDA(cudaEventRecord(ev_rot[0], side_stream));
        if (m.dec_layers > 1) {
            for (int v = 0; v < V; ++v)
                TRY(rfk_rope_one_oop_strided(kvK(1), kRot(1, v), k_cos + v * tab_n, k_sin + v * tab_n, m.dec_layers - 1, 2 * slab,
                                             (long long)V * rot_slab, 0, m.num_heads, Se_pad, hd, Se_pad, Se_pad,
                                             g0 ? g0 + dim : nullptr, dim, (rfk_stream_t)side_stream));
            TRY_CUDA(cudaEventRecord(ev_rot[1], side_stream));
        }
    }
    // camera-space rays (identity pose, as the reference does) written straight as patch tokens
    for (int v = 0; v < V; ++v)
        TRY(rfk_ray_gen_patchify(id_c2w, cam_gpu + v * kCamStride + 16, nullptr, ray_pat + v * pat_n, 1, res, ps, s));
    const int rows = V * nP;
    TRY(rfk_linear(ctx, ray_pat, m.ray_enc_w, m.ray_enc_b, rtok, rows, dim, 3 * ps * ps, s));
    TRY(rfk_rmsnorm(rtok, m.ray_enc_norm, rtok, rows, dim, kEpsFp16, s));
    TRY(rfk_broadcast_add(rtok, m.ray_map_patch_token, (long long)rows * dim, dim, s));

    const int n_keys = (flags & RFK_SESSION_PAD_KEYS_ATTEND) ? Se_pad : Se;
    const rfk_half* pending = nullptr;
    const int L4 = std::max(1, m.dec_layers / 4);
    const int cache_flags = (prescale ? 1 : 0) | (V > 1 ? 2 : 0);  // keys rotated + weighted here; values shared by the views
    for (int i = 0; i < m.dec_layers; ++i) {
        const int shift = (i % 2 == 1) ? m.shift_size : 0;
        const bool tap = ((i + 1) % L4 == 0) && ((i + 1) / L4 <= 4);
        const bool last = i == m.dec_layers - 1;
        const rfk_half* next_pending = nullptr;
        // a tapped (or the last) layer finishes x itself; the others leave their FFN residual
        // to the first kernel of the next layer
        if (i < 2) TRY_CUDA(cudaStreamWaitEvent(stream, ev_rot[i], 0));
        TRY(decoder_layer_impl(ctx, &m.dec[i], rtok, pending, (tap || last) ? nullptr : &next_pending,
                               temp, proj, qkv, ffn, win, score, self_score, kRot(i), kvV(i), V, nP,
                               Se_pad, n_keys, dim, m.num_heads, m.ffn_hidden, pH, pW, m.window_size,
                               shift, shift > 0 ? shift_mask : nullptr, nullptr, nullptr, nullptr, nullptr, cache_flags, s));
        pending = next_pending;
        if (tap)
            TRY_CUDA(cudaMemcpyAsync(taps_out[(i + 1) / L4 - 1], rtok, (size_t)rows * dim * sizeof(rfk_half),
                                     cudaMemcpyDeviceToDevice, stream));
    }
    TRY_CUDA(cudaMemcpyAsync(result_out, rtok, (size_t)rows * dim * sizeof(rfk_half), cudaMemcpyDeviceToDevice, stream));
    if (dpt) {
        // image head over this frame's taps, then ELU(1e-3) -> fp32 -> 10^x - 1 in one kernel (render_session.cu:239-253)
        TRY(rfk_dpt_forward(dpt, taps_out, nullptr, s));
        TRY(rfk_post_elu_pow10(rfk_dpt_output(dpt), image_out, (long long)V * dptw.out_dim * res * res, 1e-3f, s));
    }
    return RFK_OK;
}

extern "C" size_t rfk_scene_state_bytes(const rfk_model* model, int n_tris) {
    if (!model || n_tris <= 0) return 0;
    return state_layout(*model, n_tris).total;
}

static int check_model(const rfk_model* m) {
    if (!m) return RFK_EINVAL;
    if (m->dim <= 0 || m->num_heads <= 0 || m->dim % m->num_heads || m->ffn_hidden <= 0) return RFK_EINVAL;
    if (m->enc_layers < 0 || m->enc_layers > RFK_MAX_LAYERS || m->dec_layers <= 0 || m->dec_layers > RFK_MAX_LAYERS)
        return RFK_EINVAL;
    const int hd = m->dim / m->num_heads;
    if (m->rope_num_freqs <= 0 || 9 * m->rope_num_freqs > hd / 2 || hd % 16) return RFK_EINVAL;
    if (m->patch_size <= 0 || m->window_size <= 0 || m->shift_size < 0 || m->shift_size >= m->window_size)
        return RFK_EINVAL;
    return RFK_OK;
}

extern "C" int rfk_session_create(const rfk_model* model, int n_tris, int img_res, void* scene_state, int flags,
                                  rfk_session** out) {
    return rfk_session_create_batched(model, n_tris, img_res, scene_state, flags, 1, out);
}

extern "C" int rfk_session_create_batched(const rfk_model* model, int n_tris, int img_res, void* scene_state, int flags,
                                          int views_per_frame, rfk_session** out) {
    if (!out || !scene_state || n_tris <= 0 || img_res <= 0 || views_per_frame <= 0 || views_per_frame > 64) return RFK_EINVAL;
    TRY(check_model(model));
    if (img_res % model->patch_size || (img_res / model->patch_size) % model->window_size) return RFK_EINVAL;
    rfk_session* d = new rfk_session();
    d->m = *model;
    if (model->dpt) { d->dptw = *model->dpt; d->m.dpt = &d->dptw; }
    d->N = n_tris; d->res = img_res; d->flags = flags; d->V = views_per_frame;
    d->Se = model->num_register_tokens + n_tris;
    d->Se_pad = (d->Se + 7) & ~7;
    d->pH = d->pW = img_res / model->patch_size;
    d->nP = d->pH * d->pW;
    d->hd = model->dim / model->num_heads;
    d->L = state_layout(*model, n_tris);
    d->state = (char*)scene_state;
    const int dim = model->dim, nh = model->num_heads, ffn = model->ffn_hidden, nP = d->nP, Se_pad = d->Se_pad;
    const int ws = model->window_size, nWin = (d->pH / ws) * (d->pW / ws);
    int rc = rfk_ctx_create(&d->ctx);
    if (!rc) rc = rfk_ctx_reserve_attention_workspace(d->ctx);  // all attention launches of a session are on its one stream
    auto fail = [&](int code) { rfk_session_destroy(d); return code; };
    if (rc) return fail(rc);
    if (cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking) != cudaSuccess) return fail((int)cudaGetLastError());
    if (cudaStreamCreateWithFlags(&d->copy_stream, cudaStreamNonBlocking) != cudaSuccess) return fail((int)cudaGetLastError());
    if (cudaStreamCreateWithFlags(&d->side_stream, cudaStreamNonBlocking) != cudaSuccess) return fail((int)cudaGetLastError());
    if (cudaEventCreateWithFlags(&d->ev_fork, cudaEventDisableTiming) != cudaSuccess) return fail((int)cudaGetLastError());
    for (int i = 0; i < model->dec_layers; ++i)
        if (cudaEventCreateWithFlags(&d->ev_rot[i], cudaEventDisableTiming) != cudaSuccess) return fail((int)cudaGetLastError());
    for (int k = 0; k < kSlots; ++k) {
        if (cudaEventCreate(&d->ev_start[k]) != cudaSuccess || cudaEventCreate(&d->ev_done[k]) != cudaSuccess ||
            cudaEventCreateWithFlags(&d->ev_dl[k], cudaEventDisableTiming) != cudaSuccess)
            return fail((int)cudaGetLastError());
        if (cudaHostAlloc((void**)&d->pin_cam[k], (size_t)views_per_frame * kCamStride * sizeof(float), cudaHostAllocDefault) != cudaSuccess)
            return fail((int)cudaGetLastError());
    }
#define ALLOC(ptr, count)                    \
    if ((rc = d->alloc(&d->ptr, (count)))) return fail(rc)
    const size_t V = (size_t)views_per_frame;
    ALLOC(cam_gpu, V * kCamStride);
    ALLOC(id_c2w, 16);
    ALLOC(vtri, V * n_tris * 9);
    ALLOC(vvn, V * n_tris * 9);
    ALLOC(vpos, V * Se_pad * 9);
    ALLOC(k_cos, V * Se_pad * d->hd);
    ALLOC(k_sin, V * Se_pad * d->hd);
    ALLOC(ray_pat, V * nP * 3 * model->patch_size * model->patch_size);
    ALLOC(rtok, V * nP * dim);
    ALLOC(temp, V * nP * dim);
    ALLOC(proj, V * std::max((size_t)2 * nP * dim + (size_t)nh * Se_pad * d->hd, (size_t)3 * nP * dim));
    ALLOC(qkv, V * nP * std::max(3 * dim, 2 * ffn));
    ALLOC(ffn, V * nP * std::max(dim, ffn));
    ALLOC(win, V * nP * dim);
    ALLOC(k_rot, V * model->dec_layers * nh * Se_pad * d->hd);
    ALLOC(q_gamma_all, (size_t)model->dec_layers * dim);
    {
        // Deferred Q-RMSNorm of the cross-attention (layers.cu): possible when the fused kernels serve the shape and every
        // layer has a norm weight, no query bias and no window-path exclusions; then the key rotation folds the weights in.
        bool ok = d->hd == 64 && dim % 256 == 0 && d->nP % 32 == 0 && d->pH % ws == 0 && dim <= 2048;
        for (int i = 0; i < model->dec_layers && ok; ++i)
            ok = model->dec[i].cross_attn.q_norm_gamma && !model->dec[i].cross_attn.q_proj_b && !model->dec[i].cross_attn.out_proj_b &&
                 (reinterpret_cast<uintptr_t>(model->dec[i].cross_attn.q_norm_gamma) & 15u) == 0;
        d->prescale = ok;
        if (!ok && views_per_frame > 1) return fail(RFK_EUNSUPPORTED);  // a batch of views needs the fused attention route
        for (int i = 0; i < model->dec_layers && ok; ++i)
            if (cudaMemcpy(d->q_gamma_all + (size_t)i * dim, model->dec[i].cross_attn.q_norm_gamma, (size_t)dim * sizeof(float),
                           cudaMemcpyDeviceToDevice) != cudaSuccess)
                return fail((int)cudaGetLastError());
    }
    const bool fused_attention = d->hd == 64 || d->hd == 128;  // rfk_flash_attention serves these
    if (!fused_attention) ALLOC(score, V * nh * nP * Se_pad);
    if (!(ws * ws == 64 && d->hd == 64)) ALLOC(self_score, V * nWin * nh * ws * ws * ws * ws);
    ALLOC(shift_mask, (size_t)nWin * ws * ws * ws * ws);
    for (int k = 0; k < kSlots; ++k)
        for (int j = 0; j < 4; ++j) ALLOC(dft[k][j], V * nP * dim);
    for (int k = 0; k < kSlots; ++k) ALLOC(result[k], V * nP * dim);
    if (model->dpt) {
        for (int k = 0; k < kSlots; ++k) ALLOC(image[k], V * d->dptw.out_dim * img_res * img_res);
        if ((rc = rfk_dpt_create(d->ctx, &d->dptw, views_per_frame, dim, d->pH, d->pW, model->patch_size, &d->dpt))) return fail(rc);
    }
#undef ALLOC
    const float id[16] = {1, 0, 0, 0, 0, 1, 0, 0, 0, 0, 1, 0, 0, 0, 0, 1};
    if (cudaMemcpy(d->id_c2w, id, sizeof(id), cudaMemcpyHostToDevice) != cudaSuccess) return fail((int)cudaGetLastError());
    *out = d;
    return RFK_OK;
}

extern "C" int rfk_session_destroy(rfk_session* d) {
    if (!d) return RFK_OK;
    if (d->stream) cudaStreamSynchronize(d->stream);
    if (d->copy_stream) cudaStreamSynchronize(d->copy_stream);
    if (d->side_stream) cudaStreamSynchronize(d->side_stream);
    if (d->ev_fork) cudaEventDestroy(d->ev_fork);
    for (int i = 0; i < RFK_MAX_LAYERS; ++i)
        if (d->ev_rot[i]) cudaEventDestroy(d->ev_rot[i]);
    for (int k = 0; k < kSlots; ++k) {
        if (d->exec[k]) cudaGraphExecDestroy(d->exec[k]);
        if (d->graph[k]) cudaGraphDestroy(d->graph[k]);
        if (d->pin_cam[k]) cudaFreeHost(d->pin_cam[k]);
        if (d->ev_start[k]) cudaEventDestroy(d->ev_start[k]);
        if (d->ev_done[k]) cudaEventDestroy(d->ev_done[k]);
        if (d->ev_dl[k]) cudaEventDestroy(d->ev_dl[k]);
    }
    if (d->ev_mark0) cudaEventDestroy(d->ev_mark0);
    if (d->ev_mark1) cudaEventDestroy(d->ev_mark1);
    for (void* p : d->owned) cudaFree(p);
    rfk_dpt_destroy(d->dpt);
    if (d->stream) cudaStreamDestroy(d->stream);
    if (d->copy_stream) cudaStreamDestroy(d->copy_stream);
    if (d->side_stream) cudaStreamDestroy(d->side_stream);
    rfk_ctx_destroy(d->ctx);
    delete d;
    return RFK_OK;
}

// Scratch allocations of the one-time scene encoding (freed on every exit path).
struct Scratch {
    std::vector<void*> ptrs;
    ~Scratch() { for (void* p : ptrs) cudaFree(p); }
    template <typename T> int get(T** p, size_t count) {
        void* d = nullptr;
        cudaError_t e = cudaMalloc(&d, std::max<size_t>(count * sizeof(T), 256));
        if (e != cudaSuccess) return (int)e;
        ptrs.push_back(d);
        *p = (T*)d;
        return RFK_OK;
    }
};

extern "C" int rfk_session_encode_scene(rfk_session* d, const float* tri, const float* vn, const rfk_half* tex) {
    if (!d || !tri || !vn || !tex) return RFK_EINVAL;
    const rfk_model& m = d->m;
    const int N = d->N, Se = d->Se, Se_pad = d->Se_pad, dim = m.dim, nh = m.num_heads, hd = d->hd, nr = m.num_register_tokens;
    const int ffn = m.ffn_hidden, C = m.texture_channels;
    const int vn_pe_dim = 9 + 9 * m.vn_pe_num_freqs * 2;
    cudaStream_t st = d->stream;
    rfk_stream_t s = (rfk_stream_t)st;
    Scratch sc;

    // texture: log-encode the last 3 channels (render_session.cu:297-299)
    rfk_half* tex_buf; TRY(sc.get(&tex_buf, (size_t)N * C));
    TRY_CUDA(cudaMemcpyAsync(tex_buf, tex, (size_t)N * C * sizeof(rfk_half), cudaMemcpyDeviceToDevice, st));
    log_encode_kernel<<<blocks_for((long long)N * 3), 256, 0, st>>>((__half*)tex_buf, N, C, 3);
    // fp16 copies of the geometry kept for every view (render_session.cu:301-304)
    TRY(rfk_cast_fp32_to_fp16(tri, d->tri16(), (long long)N * 9, s));
    TRY(rfk_cast_fp32_to_fp16(vn, d->vn16(), (long long)N * 9, s));
    // Scene centre = mean of all 3N fp16 vertices, summed on the host in double precision (the
    // reference's centroid is the same quantity, src/pipeline/render_session.cu:62-70).
    std::vector<__half> h_tri((size_t)N * 9);
    TRY_CUDA(cudaMemcpyAsync(h_tri.data(), d->tri16(), h_tri.size() * sizeof(__half), cudaMemcpyDeviceToHost, st));
    TRY_CUDA(cudaStreamSynchronize(st));
    double axis_sum[3] = {0.0, 0.0, 0.0};
    for (size_t v = 0; v < (size_t)N * 3; ++v)
        for (int a = 0; a < 3; ++a) axis_sum[a] += (double)__half2float(h_tri[v * 3 + a]);
    float c[3];
    for (int a = 0; a < 3; ++a) c[a] = (float)(axis_sum[a] / (3.0 * N));
    TRY_CUDA(cudaMemcpyAsync(d->center(), c, sizeof(c), cudaMemcpyHostToDevice, st));

    // normals: NeRF PE -> linear -> fp32 RMSNorm (render_session.cu:310-318)
    rfk_half *vn_pe, *emb16; float *vn_n, *tex_n, *seq;
    TRY(sc.get(&vn_pe, (size_t)N * vn_pe_dim));
    TRY(sc.get(&emb16, (size_t)N * dim));
    TRY(sc.get(&vn_n, (size_t)N * dim));
    TRY(sc.get(&tex_n, (size_t)N * dim));
    TRY(sc.get(&seq, (size_t)Se * dim));
    TRY(rfk_nerf_pe_f32(vn, vn_pe, 1, N, 9, m.vn_pe_num_freqs, 0.0f, (float)(m.vn_pe_num_freqs - 1), 1, s));
    TRY(rfk_linear(d->ctx, vn_pe, m.vn_proj_w, m.vn_proj_b, emb16, N, dim, vn_pe_dim, s));
    TRY(rfk_cast_fp16_to_fp32(emb16, vn_n, (long long)N * dim, s));
    TRY(rfk_rmsnorm_f32(vn_n, m.vn_enc_norm, vn_n, N, dim, kEpsFp16, s));
    // texture: linear -> fp32 RMSNorm (render_session.cu:321-327)
    TRY(rfk_linear(d->ctx, tex_buf, m.tex_enc_w, m.tex_enc_b, emb16, N, dim, C, s));
    TRY(rfk_cast_fp16_to_fp32(emb16, tex_n, (long long)N * dim, s));
    TRY(rfk_rmsnorm_f32(tex_n, m.tex_enc_norm, tex_n, N, dim, kEpsFp16, s));
    // sequence = [register tokens | texture + normal + triangle token] in fp32 (render_session.cu:330-339)
    TRY(rfk_cast_fp16_to_fp32(m.reg_tokens, seq, (long long)nr * dim, s));
    add3_bc_kernel<<<blocks_for((long long)N * dim), 256, 0, st>>>(seq + (size_t)nr * dim, tex_n, vn_n,
                                                                   (const __half*)m.tri_token, (long long)N * dim, dim);
    // encoder positions: world centroid for the register tokens, then the triangles (render_session.cu:91-97,342-350)
    rfk_half *enc_pos, *enc_cos, *enc_sin;
    TRY(sc.get(&enc_pos, (size_t)Se * 9));
    TRY(sc.get(&enc_cos, (size_t)Se * hd));
    TRY(sc.get(&enc_sin, (size_t)Se * hd));
    std::vector<__half> h_reg((size_t)nr * 9);
    for (int r = 0; r < nr; ++r)
        for (int k = 0; k < 9; ++k) h_reg[(size_t)r * 9 + k] = __float2half(c[k % 3]);
    TRY_CUDA(cudaMemcpyAsync(enc_pos, h_reg.data(), h_reg.size() * sizeof(__half), cudaMemcpyHostToDevice, st));
    TRY_CUDA(cudaMemcpyAsync(enc_pos + (size_t)nr * 9, d->tri16(), (size_t)N * 9 * sizeof(rfk_half), cudaMemcpyDeviceToDevice, st));
    TRY(rfk_triangle_rope_freqs(enc_pos, m.enc_rope_freqs, enc_cos, enc_sin, 1, Se,
                                m.rope_num_freqs, hd, s));
    TRY_CUDA(cudaStreamSynchronize(st));  // h_reg goes out of use

    // encoder (render_session.cu:356-371)
    rfk_half *temp, *qkvb, *ffnb; float* score;
    TRY(sc.get(&temp, (size_t)Se * dim));
    TRY(sc.get(&qkvb, (size_t)Se * std::max(6 * dim, 2 * ffn)));
    TRY(sc.get(&ffnb, (size_t)Se * std::max(dim, ffn)));
    score = nullptr;
    if (!(hd == 64 || hd == 128)) TRY(sc.get(&score, (size_t)nh * Se * Se_pad));
    const rfk_half* pending = nullptr;
    for (int i = 0; i < m.enc_layers; ++i) {
        const rfk_half* next = nullptr;
        TRY(rfk_encoder_layer_forward_mixed(d->ctx, &m.enc[i], seq, pending, i + 1 < m.enc_layers ? &next : nullptr,
                                            temp, qkvb, ffnb, score, 1, Se, dim, nh, ffn,
                                            enc_cos, enc_sin, s));
        pending = next;
    }
    // context in fp16, then per decoder layer: kv-norm, K/V projections, padded head-major cache
    // (render_session.cu:377-416)
    rfk_half *ctx16, *ctx_normed, *kv_proj;
    TRY(sc.get(&ctx16, (size_t)Se * dim));
    TRY(sc.get(&ctx_normed, (size_t)Se * dim));
    TRY(sc.get(&kv_proj, (size_t)2 * Se * dim));
    TRY(rfk_cast_fp32_to_fp16(seq, ctx16, (long long)Se * dim, s));
    for (int i = 0; i < m.dec_layers; ++i) {
        TRY(rfk_rmsnorm(ctx16, m.dec[i].kv_norm_gamma, ctx_normed, Se, dim, kEpsFp16, s));
        TRY(rfk_precompute_cross_kv(d->ctx, &m.dec[i].cross_attn, ctx_normed, d->kvK(i),
                                    d->kvV(i), kv_proj, 1, Se, Se_pad, dim, dim, nh, s));
    }
    TRY_CUDA(cudaStreamSynchronize(st));
    TRY_CUDA(cudaGetLastError());
    return RFK_OK;
}

// The fused attention kernel reports a time-out of one of its bounded waits in a device word instead of hanging;
// frames rendered since the word was last clear are not to be trusted.
static int check_attention_error() {
    int code = 0;
    TRY(rfk_flash_attention_error(&code, 0));
    if (code) return RFK_EKERNEL;
    TRY(rfk_gemm_error(&code, 0));  // the tcgen05 GEMM kernel reports the same way
    return code ? RFK_EKERNEL : RFK_OK;
}

extern "C" int rfk_session_finalize(rfk_session* d) {
    if (!d) return RFK_EINVAL;
    if (d->finalized) return RFK_OK;
    const rfk_model& m = d->m;
    std::vector<uint8_t> mask = build_window_mask(d->pH, d->pW, m.window_size, m.shift_size);
    TRY_CUDA(cudaMemcpy(d->shift_mask, mask.data(), mask.size(), cudaMemcpyHostToDevice));
    // warm-up view (also lets cuBLAS pick and load its kernels before capture)
    float cam[17] = {1, 0, 0, 0, 0, 1, 0, 0, 0, 0, 1, 3, 0, 0, 0, 1, 0.7f};
    for (int k = 0; k < kSlots; ++k)
        for (int v = 0; v < d->V; ++v) memcpy(d->pin_cam[k] + v * kCamStride, cam, sizeof(cam));
    {
        int rc = d->render_view(d->pin_cam[0], d->result[0], d->dft[0], d->image[0]);
        if (rc == RFK_EUNSUPPORTED && d->prescale && d->V == 1) {  // the kernels of the deferred norm cannot run here: separate norm instead
            TRY_CUDA(cudaStreamSynchronize(d->stream));
            TRY_CUDA(cudaStreamSynchronize(d->side_stream));
            d->prescale = false;
            rc = d->render_view(d->pin_cam[0], d->result[0], d->dft[0], d->image[0]);
        }
        TRY(rc);
    }
    TRY_CUDA(cudaStreamSynchronize(d->stream));
    if (!(d->flags & RFK_SESSION_NO_GRAPH)) {
        for (int k = 0; k < kSlots; ++k) {
            const unsigned long long n0 = rfk_launch_count();
            TRY_CUDA(cudaStreamBeginCapture(d->stream, cudaStreamCaptureModeThreadLocal));
            int rc = d->render_view(d->pin_cam[k], d->result[k], d->dft[k], d->image[k]);
            cudaError_t e = cudaStreamEndCapture(d->stream, &d->graph[k]);
            if (rc != RFK_OK) return rc;
            TRY_CUDA(e);
            d->kernels_per_view = (int)(rfk_launch_count() - n0);
            TRY_CUDA(cudaGraphInstantiate(&d->exec[k], d->graph[k], 0));
            size_t nodes = 0;
            TRY_CUDA(cudaGraphGetNodes(d->graph[k], nullptr, &nodes));
            d->graph_nodes = (int)nodes;
        }
    } else {
        const unsigned long long n0 = rfk_launch_count();
        TRY(d->render_view(d->pin_cam[0], d->result[0], d->dft[0], d->image[0]));
        d->kernels_per_view = (int)(rfk_launch_count() - n0);
        TRY_CUDA(cudaStreamSynchronize(d->stream));
    }
    TRY_CUDA(cudaStreamSynchronize(d->stream));
    TRY(check_attention_error());
    d->finalized = true;
    return RFK_OK;
}

extern "C" int rfk_session_render_frames(rfk_session* d, const float* h_c2w, const float* fov_rad) {
    if (!d || !h_c2w || !fov_rad || !d->finalized) return RFK_EINVAL;
    const int k = (int)(d->frames % kSlots);
    // the slot's previous frame (two frames ago) must have left the device, and its download
    // must have finished, before its pinned cameras and result buffer are reused
    if (d->frames >= kSlots) TRY_CUDA(cudaEventSynchronize(d->ev_done[k]));
    if (d->dl_pending[k]) {
        TRY_CUDA(cudaEventSynchronize(d->ev_dl[k]));
        d->dl_pending[k] = false;
    }
    for (int v = 0; v < d->V; ++v) {
        memcpy(d->pin_cam[k] + v * kCamStride, h_c2w + v * 16, 16 * sizeof(float));
        d->pin_cam[k][v * kCamStride + 16] = fov_rad[v];
    }
    TRY_CUDA(cudaEventRecord(d->ev_start[k], d->stream));
    if (d->exec[k]) TRY_CUDA(cudaGraphLaunch(d->exec[k], d->stream));
    else TRY(d->render_view(d->pin_cam[k], d->result[k], d->dft[k], d->image[k]));
    TRY_CUDA(cudaEventRecord(d->ev_done[k], d->stream));
    d->frames++;
    return RFK_OK;
}

extern "C" int rfk_session_render_frame(rfk_session* d, const float* h_c2w, float fov_rad) {
    if (!d || d->V != 1) return RFK_EINVAL;  // a session of V views per frame takes its cameras V at a time
    return rfk_session_render_frames(d, h_c2w, &fov_rad);
}

extern "C" int rfk_session_views_per_frame(rfk_session* d) { return d ? d->V : 0; }

extern "C" int rfk_session_wait(rfk_session* d, float* ms) {
    if (!d || d->frames == 0) return RFK_EINVAL;
    const int k = (int)((d->frames - 1) % kSlots);
    TRY_CUDA(cudaEventSynchronize(d->ev_done[k]));
    if (ms) TRY_CUDA(cudaEventElapsedTime(ms, d->ev_start[k], d->ev_done[k]));
    return RFK_OK;
}

extern "C" int rfk_session_result(rfk_session* d, const rfk_half** tokens, int* n_tokens, int* dim) {
    if (!d || d->frames == 0) return RFK_EINVAL;
    if (tokens) *tokens = d->result[(d->frames - 1) % kSlots];
    if (n_tokens) *n_tokens = d->nP;
    if (dim) *dim = d->m.dim;
    return RFK_OK;
}

extern "C" int rfk_session_feature_taps(rfk_session* d, const rfk_half** taps) {
    if (!d || !taps || d->frames == 0) return RFK_EINVAL;
    const int k = (int)((d->frames - 1) % kSlots);
    for (int j = 0; j < 4; ++j) taps[j] = d->dft[k][j];
    return RFK_OK;
}

extern "C" int rfk_session_image(rfk_session* d, const float** image, int* channels, int* img_res) {
    if (!d || !d->dpt || d->frames == 0) return RFK_EINVAL;
    if (image) *image = d->image[(d->frames - 1) % kSlots];
    if (channels) *channels = d->dptw.out_dim;
    if (img_res) *img_res = d->res;
    return RFK_OK;
}

extern "C" int rfk_session_download_image(rfk_session* d, float* h_out, size_t bytes) {
    if (!d || !d->dpt || !h_out || d->frames == 0) return RFK_EINVAL;
    const size_t need = (size_t)d->V * d->dptw.out_dim * d->res * d->res * sizeof(float);
    if (bytes < need) return RFK_EINVAL;
    const int k = (int)((d->frames - 1) % kSlots);
    TRY_CUDA(cudaStreamWaitEvent(d->copy_stream, d->ev_done[k], 0));
    TRY_CUDA(cudaMemcpyAsync(h_out, d->image[k], need, cudaMemcpyDeviceToHost, d->copy_stream));
    TRY_CUDA(cudaStreamSynchronize(d->copy_stream));
    return RFK_OK;
}

extern "C" int rfk_session_download_async(rfk_session* d, rfk_half* h_out, size_t bytes) {
    if (!d || !h_out || d->frames == 0) return RFK_EINVAL;
    const size_t need = (size_t)d->V * d->nP * d->m.dim * sizeof(rfk_half);
    if (bytes < need) return RFK_EINVAL;
    const int k = (int)((d->frames - 1) % kSlots);
    TRY_CUDA(cudaStreamWaitEvent(d->copy_stream, d->ev_done[k], 0));
    TRY_CUDA(cudaMemcpyAsync(h_out, d->result[k], need, cudaMemcpyDeviceToHost, d->copy_stream));
    TRY_CUDA(cudaEventRecord(d->ev_dl[k], d->copy_stream));
    d->dl_pending[k] = true;
    return RFK_OK;
}

extern "C" int rfk_session_drain(rfk_session* d) {
    if (!d) return RFK_EINVAL;
    TRY_CUDA(cudaStreamSynchronize(d->stream));
    TRY_CUDA(cudaStreamSynchronize(d->copy_stream));
    for (int k = 0; k < kSlots; ++k) d->dl_pending[k] = false;
    return check_attention_error();
}

extern "C" int rfk_session_download(rfk_session* d, rfk_half* h_out, size_t bytes) {
    TRY(rfk_session_download_async(d, h_out, bytes));
    TRY_CUDA(cudaStreamSynchronize(d->copy_stream));
    d->dl_pending[(d->frames - 1) % kSlots] = false;
    return RFK_OK;
}

extern "C" int rfk_session_mark_begin(rfk_session* d) {
    if (!d) return RFK_EINVAL;
    if (!d->ev_mark0) {
        TRY_CUDA(cudaEventCreate(&d->ev_mark0));
        TRY_CUDA(cudaEventCreate(&d->ev_mark1));
    }
    TRY_CUDA(cudaEventRecord(d->ev_mark0, d->stream));
    return RFK_OK;
}

extern "C" int rfk_session_mark_end(rfk_session* d, float* ms) {
    if (!d || !d->ev_mark0) return RFK_EINVAL;
    // downloads are part of the bracketed work: the end mark waits for the copy stream too
    cudaEvent_t dl = nullptr;
    TRY_CUDA(cudaEventCreateWithFlags(&dl, cudaEventDisableTiming));
    cudaError_t e = cudaEventRecord(dl, d->copy_stream);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(d->stream, dl, 0);
    cudaEventDestroy(dl);
    TRY_CUDA(e);
    TRY_CUDA(cudaEventRecord(d->ev_mark1, d->stream));
    TRY_CUDA(cudaEventSynchronize(d->ev_mark1));
    if (ms) TRY_CUDA(cudaEventElapsedTime(ms, d->ev_mark0, d->ev_mark1));
    return RFK_OK;
}

extern "C" int rfk_session_graph_nodes(rfk_session* d) { return d ? d->graph_nodes : 0; }
extern "C" int rfk_session_kernels_per_view(rfk_session* d) { return d ? d->kernels_per_view : 0; }
