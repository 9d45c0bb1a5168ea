// DPT image head: the four decoder feature taps -> [out_dim, H, W] image.
//
// Reference: rf::dpt_forward, src/layers/dpt.cu:322-461 (BANANASJIM/renderformer-cuda), with rf::conv2d (:100-178) and
// rf::conv_transpose2d (:182-236); same operator sequence, same roundings between the operators. What is different:
//   - the head runs channels-last ([N, H, W, C] fp16). The decoder's token maps are already in that layout, so the
//     reference's permute to NCHW is gone; the library's tensor-core convolution kernels take channels-last operands as
//     they are (handed NCHW tensors they convert every operand on the way in and out: 69 conversion launches, 35 % of
//     the head's time when it ran that way); a 1x1 convolution is a row-major GEMM and goes to rfk_linear, i.e. the
//     tcgen05 projection kernel with the bias in its epilogue; the two transposed convolutions (kernel = stride) are that
//     same GEMM followed by a depth-to-space scatter. Only the 3x3 convolutions remain library (cuDNN) calls. Filters
//     are re-laid out once, at plan time.
//   - bias, SiLU and residual adds that follow a convolution are one pass (rfk_bias_act_residual_nhwc), bit-identical
//     to the separate operators; the copy the reference's in-place SiLU forces before a residual unit is gone.
//   - nothing is allocated on the launch path. The reference calls cudaMallocAsync / cudaFreeAsync for every
//     intermediate inside dpt_forward (and so inside its captured graph); here rfk_dpt_create sizes every intermediate
//     once, picks the cuDNN algorithms, allocates one workspace, and records the whole head as a list of steps over
//     fixed buffers. rfk_dpt_forward only walks that list, so it can be captured.
#include "layers_internal.h"

#include <cudnn.h>

#include <algorithm>
#include <functional>
#include <vector>

namespace {

#define DNN_TRY(expr)                                      \
    do {                                                   \
        cudnnStatus_t s_ = (expr);                         \
        if (s_ != CUDNN_STATUS_SUCCESS) return 2000 + (int)s_; \
    } while (0)
#define TRY(expr)                       \
    do {                                \
        int rc_ = (expr);               \
        if (rc_ != RFK_OK) return rc_;  \
    } while (0)

using Step = std::function<int(const rfk_half* const* feats, cudaStream_t st)>;

}  // namespace

struct rfk_dpt {
    rfk_ctx* ctx = nullptr;  // borrowed: cuBLAS handle for the 1x1 convolutions
    cudnnHandle_t dnn = nullptr;
    rfk_dpt_weights w{};
    int B = 0, dim = 0, pH = 0, pW = 0, ps = 0;
    std::vector<void*> owned;
    std::vector<cudnnTensorDescriptor_t> tdescs;
    std::vector<cudnnFilterDescriptor_t> fdescs;
    std::vector<cudnnConvolutionDescriptor_t> cdescs;
    void* workspace = nullptr;
    size_t ws_bytes = 0;
    std::vector<Step> program;
    rfk_half* out = nullptr;  // [B, out_dim, pH*ps, pW*ps]
    int n_convs = 0;

    rfk_half* alloc(size_t halves) {
        void* p = nullptr;
        if (cudaMalloc(&p, std::max<size_t>(halves * sizeof(rfk_half), 256)) != cudaSuccess) return nullptr;
        owned.push_back(p);
        return (rfk_half*)p;
    }
    cudnnTensorDescriptor_t tensor(int n, int c, int h, int w_) {
        cudnnTensorDescriptor_t d = nullptr;
        if (cudnnCreateTensorDescriptor(&d) != CUDNN_STATUS_SUCCESS) return nullptr;
        tdescs.push_back(d);
        if (cudnnSetTensor4dDescriptor(d, CUDNN_TENSOR_NHWC, CUDNN_DATA_HALF, n, c, h, w_) != CUDNN_STATUS_SUCCESS) return nullptr;
        return d;
    }
    cudnnFilterDescriptor_t filter(int k, int c, int r, int s) {
        cudnnFilterDescriptor_t d = nullptr;
        if (cudnnCreateFilterDescriptor(&d) != CUDNN_STATUS_SUCCESS) return nullptr;
        fdescs.push_back(d);
        if (cudnnSetFilter4dDescriptor(d, CUDNN_DATA_HALF, CUDNN_TENSOR_NHWC, k, c, r, s) != CUDNN_STATUS_SUCCESS) return nullptr;
        return d;
    }
    cudnnConvolutionDescriptor_t conv(int pad, int stride) {
        cudnnConvolutionDescriptor_t d = nullptr;
        if (cudnnCreateConvolutionDescriptor(&d) != CUDNN_STATUS_SUCCESS) return nullptr;
        cdescs.push_back(d);
        if (cudnnSetConvolution2dDescriptor(d, pad, pad, stride, stride, 1, 1, CUDNN_CROSS_CORRELATION, CUDNN_DATA_FLOAT) !=
                CUDNN_STATUS_SUCCESS ||
            cudnnSetConvolutionMathType(d, CUDNN_TENSOR_OP_MATH) != CUDNN_STATUS_SUCCESS)
            return nullptr;
        return d;
    }

    // o [B, Ho, Wo, Cout] = conv(in [B, H, W, Cin], weight [Cout, Cin, k, k] as the reference stores it) + bias, then SiLU
    // if silu, then + residual if given. in == nullptr: the step reads feature tap `tap` ([B, pH*pW, dim] is [B, pH, pW, dim]).
    int add_conv(const rfk_half* in, int tap, const rfk_half* weight, const rfk_half* bias, rfk_half* o, int Cin, int H, int W,
                 int Cout, int k, int stride, int pad, bool silu = false, const rfk_half* residual = nullptr) {
        const int Ho = (H + 2 * pad - k) / stride + 1, Wo = (W + 2 * pad - k) / stride + 1;
        const long long rows_out = (long long)B * Ho * Wo;
        ++n_convs;
        rfk_ctx* c = ctx;
        if (k == 1 && stride == 1 && pad == 0) {
            // 1x1: out [B*H*W, Cout] = in [B*H*W, Cin] weight[Cout, Cin]^T (+ bias in the GEMM's epilogue) (src/layers/dpt.cu:112-126)
            const long long M = (long long)B * H * W;
            if (M > 0x7fffffffLL) return RFK_EUNSUPPORTED;
            program.push_back([=](const rfk_half* const* feats, cudaStream_t st) -> int {
                TRY(rfk_linear(c, in ? in : feats[tap], weight, bias, o, (int)M, Cout, Cin, (rfk_stream_t)st));
                if (silu || residual) return rfk_bias_act_residual_nhwc(o, nullptr, residual, rows_out, Cout, silu, (rfk_stream_t)st);
                return RFK_OK;
            });
            return RFK_OK;
        }
        if (!in) return RFK_EINVAL;
        rfk_half* wk = alloc((size_t)Cout * Cin * k * k);  // [Cout, k, k, Cin]
        if (!wk) return (int)cudaErrorMemoryAllocation;
        TRY(rfk_permute_filter(weight, wk, Cout, Cin, k * k, 0, nullptr));
        cudnnTensorDescriptor_t xd = tensor(B, Cin, H, W), yd = tensor(B, Cout, Ho, Wo);
        cudnnFilterDescriptor_t fd = filter(Cout, Cin, k, k);
        cudnnConvolutionDescriptor_t cd = conv(pad, stride);
        if (!xd || !yd || !fd || !cd) return RFK_EINVAL;
        // The library's heuristic picks the algorithm. Measuring the candidates at plan time (cudnnFind...) was tried: no
        // faster in the view (198 against 201 images/s, noise), and under a profiler, whose replays distort the
        // timings, it chose a kernel 25 times slower - a plan must not depend on how it is being observed.
        int returned = 0;
        cudnnConvolutionFwdAlgoPerf_t perf[4];
        DNN_TRY(cudnnGetConvolutionForwardAlgorithm_v7(dnn, xd, fd, cd, yd, 4, &returned, perf));
        if (returned < 1 || perf[0].status != CUDNN_STATUS_SUCCESS) return RFK_EUNSUPPORTED;
        const cudnnConvolutionFwdAlgo_t algo = perf[0].algo;
        size_t ws = 0;
        DNN_TRY(cudnnGetConvolutionForwardWorkspaceSize(dnn, xd, fd, cd, yd, algo, &ws));
        ws_bytes = std::max(ws_bytes, ws);
        rfk_dpt* self = this;
        program.push_back([=](const rfk_half* const*, cudaStream_t st) -> int {
            const float one = 1.0f, zero = 0.0f;
            DNN_TRY(cudnnSetStream(self->dnn, st));
            DNN_TRY(cudnnConvolutionForward(self->dnn, &one, xd, in, fd, wk, cd, algo, self->workspace, ws, &zero, yd, o));
            if (bias || silu || residual) return rfk_bias_act_residual_nhwc(o, bias, residual, rows_out, Cout, silu, (rfk_stream_t)st);
            return RFK_OK;
        });
        return RFK_OK;
    }

    // Transposed convolution with kernel = stride = f and no padding (the head's only kind, src/layers/dpt.cu:182-236,
    // :372-380): every input pixel produces its own f x f block of output pixels, so it is one GEMM with the filter laid
    // out as [(i, j, co), ci] followed by a scatter of the blocks (+ bias).
    int add_conv_transpose(const rfk_half* in, const rfk_half* weight, const rfk_half* bias, rfk_half* o, int Cin, int H, int W,
                           int Cout, int f) {
        ++n_convs;
        const long long M = (long long)B * H * W;
        const long long N = (long long)f * f * Cout;
        if (M > 0x7fffffffLL || N > 0x7fffffffLL) return RFK_EUNSUPPORTED;
        rfk_half* wg = alloc((size_t)N * Cin);
        rfk_half* blocks = alloc((size_t)M * N);
        if (!wg || !blocks) return (int)cudaErrorMemoryAllocation;
        TRY(rfk_permute_filter(weight, wg, Cin, Cout, f * f, 1, nullptr));
        rfk_ctx* c = ctx;
        const int Bn = B;
        program.push_back([=](const rfk_half* const*, cudaStream_t st) -> int {
            TRY(rfk_linear(c, in, wg, nullptr, blocks, (int)M, (int)N, Cin, (rfk_stream_t)st));
            return rfk_depth_to_space_bias_nhwc(blocks, bias, o, Bn, H, W, Cout, f, (rfk_stream_t)st);
        });
        return RFK_OK;
    }

    // residual convolution unit (src/layers/dpt.cu:397-409): *result <- conv2(silu(conv1(silu(x)))) + x; x is left as it was
    int add_rcu(const rfk_rcu_weights& r, const rfk_half* x, int F, int H, int W, rfk_half** result) {
        const long long n = (long long)B * F * H * W;
        rfk_half* t0 = alloc((size_t)n);
        rfk_half* t1 = alloc((size_t)n);
        if (!t0 || !t1) return (int)cudaErrorMemoryAllocation;
        program.push_back([=](const rfk_half* const*, cudaStream_t st) -> int { return rfk_silu(x, t0, n, (rfk_stream_t)st); });
        TRY(add_conv(t0, -1, r.conv1_w, r.conv1_b, t1, F, H, W, F, 3, 1, 1, /*silu=*/true));
        TRY(add_conv(t1, -1, r.conv2_w, r.conv2_b, t0, F, H, W, F, 3, 1, 1, /*silu=*/false, /*residual=*/x));
        *result = t0;
        return RFK_OK;
    }

    // feature fusion block (src/layers/dpt.cu:411-426); returns the [B, th, tw, F] result buffer in *result
    int add_refinenet(int i, rfk_half* path_in, rfk_half* lr, int ph, int pw, int th, int tw, rfk_half** result) {
        const int F = w.features_dim;
        const rfk_ffb_weights& f = w.refinenet[i];
        if (f.has_resconv1) {
            if (!lr) return RFK_EINVAL;
            rfk_half* r1 = nullptr;
            TRY(add_rcu(f.rcu1, lr, F, ph, pw, &r1));
            const long long n = (long long)B * F * ph * pw;
            program.push_back([=](const rfk_half* const*, cudaStream_t st) -> int { return rfk_residual_add(path_in, r1, n, (rfk_stream_t)st); });
        }
        rfk_half* r2 = nullptr;
        TRY(add_rcu(f.rcu2, path_in, F, ph, pw, &r2));
        rfk_half* up = alloc((size_t)B * F * th * tw);
        rfk_half* res = alloc((size_t)B * F * th * tw);
        if (!up || !res) return (int)cudaErrorMemoryAllocation;
        const int Bn = B;
        program.push_back([=](const rfk_half* const*, cudaStream_t st) -> int {
            return rfk_bilinear_upsample_nhwc(r2, up, Bn, ph, pw, th, tw, F, (rfk_stream_t)st);
        });
        TRY(add_conv(up, -1, f.out_conv_w, f.out_conv_b, res, F, th, tw, F, 1, 1, 0));
        *result = res;
        return RFK_OK;
    }

    int build() {
        const int S = pH * pW, F = w.features_dim;
        rfk_half* resized[4];
        int rh[4], rw[4];
        for (int i = 0; i < 4; ++i) {
            const int C = w.out_channels[i];
            rfk_half* projected = alloc((size_t)B * C * S);
            if (!projected) return (int)cudaErrorMemoryAllocation;
            TRY(add_conv(nullptr, i, w.project_w[i], w.project_b[i], projected, dim, pH, pW, C, 1, 1, 0));  // straight off the token map
            if (i == 0 || i == 1) {  // x4 / x2 transposed convolution, kernel = stride
                const int f = i == 0 ? 4 : 2;
                rh[i] = pH * f; rw[i] = pW * f;
                resized[i] = alloc((size_t)B * C * rh[i] * rw[i]);
                if (!resized[i]) return (int)cudaErrorMemoryAllocation;
                TRY(add_conv_transpose(projected, w.resize_w[i], w.resize_b[i], resized[i], C, pH, pW, C, f));
            } else if (i == 2) {
                rh[i] = pH; rw[i] = pW;
                resized[i] = projected;
            } else {  // stride-2 3x3
                rh[i] = (pH + 1) / 2; rw[i] = (pW + 1) / 2;
                resized[i] = alloc((size_t)B * C * rh[i] * rw[i]);
                if (!resized[i]) return (int)cudaErrorMemoryAllocation;
                TRY(add_conv(projected, -1, w.resize_w[i], w.resize_b[i], resized[i], C, pH, pW, C, 3, 2, 1));
            }
        }
        rfk_half* layer_rn[4];
        for (int i = 0; i < 4; ++i) {
            layer_rn[i] = alloc((size_t)B * F * rh[i] * rw[i]);
            if (!layer_rn[i]) return (int)cudaErrorMemoryAllocation;
            TRY(add_conv(resized[i], -1, w.layer_rn_w[i], nullptr, layer_rn[i], w.out_channels[i], rh[i], rw[i], F, 3, 1, 1));
        }
        rfk_half *path4, *path3, *path2, *path1;
        TRY(add_refinenet(3, layer_rn[3], nullptr, rh[3], rw[3], rh[2], rw[2], &path4));
        TRY(add_refinenet(2, path4, layer_rn[2], rh[2], rw[2], rh[1], rw[1], &path3));
        TRY(add_refinenet(1, path3, layer_rn[1], rh[1], rw[1], rh[0], rw[0], &path2));
        const int oh = rh[0] * 2, ow = rw[0] * 2;
        TRY(add_refinenet(0, path2, layer_rn[0], rh[0], rw[0], oh, ow, &path1));
        // output head (src/layers/dpt.cu:440-460)
        const int fh = F / 2, full_h = pH * ps, full_w = pW * ps;
        rfk_half* oc1 = alloc((size_t)B * fh * oh * ow);
        rfk_half* oc1_up = alloc((size_t)B * fh * full_h * full_w);
        rfk_half* oc2a = alloc((size_t)B * 32 * full_h * full_w);
        rfk_half* oc2b = alloc((size_t)B * w.out_dim * full_h * full_w);  // [B, H, W, out_dim]
        out = alloc((size_t)B * w.out_dim * full_h * full_w);            // [B, out_dim, H, W]
        if (!oc1 || !oc1_up || !oc2a || !oc2b || !out) return (int)cudaErrorMemoryAllocation;
        TRY(add_conv(path1, -1, w.output_conv1_w, w.output_conv1_b, oc1, F, oh, ow, fh, 3, 1, 1));
        const int Bn = B;
        const rfk_half* oc2a_in = oc1_up;
        if (oh == full_h && ow == full_w) {
            // With patch size 8 the fusion path already is at full resolution: an align_corners resample onto the same
            // grid has weights exactly 1 and 0, i.e. it is the identity (for finite values), and is not run.
            oc2a_in = oc1;
        } else {
            program.push_back([=](const rfk_half* const*, cudaStream_t st) -> int {
                return rfk_bilinear_upsample_nhwc(oc1, oc1_up, Bn, oh, ow, full_h, full_w, fh, (rfk_stream_t)st);
            });
        }
        TRY(add_conv(oc2a_in, -1, w.output_conv2a_w, w.output_conv2a_b, oc2a, fh, full_h, full_w, 32, 3, 1, 1, /*silu=*/true));
        rfk_half* image = out;
        const int od = w.out_dim;
        const long long HWf = (long long)full_h * full_w;
        const rfk_half *w2b = w.output_conv2b_w, *b2b = w.output_conv2b_b;
        if (od <= 4) {  // 1x1 to the colour channels + bias, written planar, in one launch
            ++n_convs;
            program.push_back([=](const rfk_half* const*, cudaStream_t st) -> int {
                return rfk_pointwise_conv_to_planar(oc2a, w2b, b2b, image, Bn, HWf, 32, od, (rfk_stream_t)st);
            });
        } else {
            TRY(add_conv(oc2a, -1, w2b, b2b, oc2b, 32, full_h, full_w, od, 1, 1, 0));
            program.push_back([=](const rfk_half* const*, cudaStream_t st) -> int {  // the interface's image is planar
                return rfk_permute_nhwc_to_nchw(oc2b, image, Bn, HWf, od, (rfk_stream_t)st);
            });
        }
        if (ws_bytes) {
            if (cudaMalloc(&workspace, ws_bytes) != cudaSuccess) return (int)cudaErrorMemoryAllocation;
            owned.push_back(workspace);
        }
        // the filter re-layouts above ran on the default stream: they must be complete before the first forward
        return (int)cudaDeviceSynchronize();
    }
};

extern "C" int rfk_dpt_destroy(rfk_dpt* d) {
    if (!d) return RFK_OK;
    for (auto t : d->tdescs) cudnnDestroyTensorDescriptor(t);
    for (auto f : d->fdescs) cudnnDestroyFilterDescriptor(f);
    for (auto c : d->cdescs) cudnnDestroyConvolutionDescriptor(c);
    for (void* p : d->owned) cudaFree(p);
    if (d->dnn) cudnnDestroy(d->dnn);
    delete d;
    return RFK_OK;
}

extern "C" int rfk_dpt_create(rfk_ctx* ctx, const rfk_dpt_weights* w, int B, int dim, int patch_h, int patch_w, int patch_size,
                              rfk_dpt** out) {
    if (!ctx || !w || !out || B <= 0 || dim <= 0 || patch_h <= 0 || patch_w <= 0 || patch_size <= 0) return RFK_EINVAL;
    if (w->features_dim <= 0 || w->features_dim % 2 || w->out_dim <= 0) return RFK_EINVAL;
    // the channels-last element-wise kernels move 8 channels per access
    if (w->features_dim % 16 || dim % 8) return RFK_EUNSUPPORTED;
    for (int i = 0; i < 4; ++i)
        if (w->out_channels[i] % 8) return RFK_EUNSUPPORTED;
    for (int i = 0; i < 4; ++i)
        if (w->out_channels[i] <= 0 || !w->project_w[i] || !w->layer_rn_w[i] || (i != 2 && !w->resize_w[i])) return RFK_EINVAL;
    rfk_dpt* d = new rfk_dpt();
    d->ctx = ctx; d->w = *w; d->B = B; d->dim = dim; d->pH = patch_h; d->pW = patch_w; d->ps = patch_size;
    if (cudnnCreate(&d->dnn) != CUDNN_STATUS_SUCCESS) { delete d; return 2000; }
    const int rc = d->build();
    if (rc != RFK_OK) { rfk_dpt_destroy(d); return rc; }
    *out = d;
    return RFK_OK;
}

extern "C" int rfk_dpt_forward(rfk_dpt* d, const rfk_half* const* features, rfk_half* image_out, rfk_stream_t stream) {
    if (!d || !features) return RFK_EINVAL;
    for (int i = 0; i < 4; ++i)
        if (!features[i]) return RFK_EINVAL;
    cudaStream_t st = (cudaStream_t)stream;
    for (const Step& s : d->program) TRY(s(features, st));
    if (image_out && image_out != d->out) {
        const size_t bytes = (size_t)d->B * d->w.out_dim * d->pH * d->ps * d->pW * d->ps * sizeof(rfk_half);
        cudaError_t e = cudaMemcpyAsync(image_out, d->out, bytes, cudaMemcpyDeviceToDevice, st);
        if (e != cudaSuccess) return (int)e;
    }
    return RFK_OK;
}

extern "C" const rfk_half* rfk_dpt_output(rfk_dpt* d) { return d ? d->out : nullptr; }
extern "C" int rfk_dpt_num_convolutions(rfk_dpt* d) { return d ? d->n_convs : 0; }
