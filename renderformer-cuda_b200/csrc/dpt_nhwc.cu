// Channels-last companions of the DPT head's element-wise operators.
//
// The head (csrc/dpt.cu) keeps its activations as [N, H, W, C] fp16: the decoder's token maps already are
// ([S, dim] = [pH, pW, dim]), the tensor-core convolution kernels of the library want that layout (given NCHW
// tensors they convert every operand on the way in and out: 35 % of the head's time), and a 1x1 convolution is then
// a plain row-major GEMM that the tcgen05 projection kernel serves. Every operator here works on rows of C
// contiguous channels with C % 8 == 0, one thread per 8 channels (one 128-bit access per operand).
//
// Arithmetic and roundings are those of the reference's NCHW operators applied one after the other
// (BANANASJIM/renderformer-cuda, src/layers/dpt.cu: add_bias_nchw_kernel :88-96, silu_inplace :289-298,
// residual_add via src/layers/transformer.cu, bilinear_upsample :240-277): where two of them are fused here the
// intermediate is still rounded to fp16, so the values are bit-identical to the unfused sequence.
#include "common.cuh"
#include "dpt_math.cuh"

namespace rfk {

// x[r, c] = act(half(x[r, c] + bias[c])) (+ residual[r, c]); bias / residual may be null; act: 0 none, 1 SiLU.
template <bool BIAS, bool SILU, bool RES>
__global__ void __launch_bounds__(256)
bias_act_residual_nhwc_kernel(__half* __restrict__ x, const __half* __restrict__ bias, const __half* __restrict__ res,
                              long long chunks, int c8 /* C / 8 */) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= chunks) return;
    float f[8];
    load8(x + i * 8, f);
    if (BIAS) {
        float b[8];
        load8(bias + (int)((unsigned)i % (unsigned)c8) * 8, b);  // chunks < 2^32 (checked by the launcher)
#pragma unroll
        for (int k = 0; k < 8; ++k) f[k] = __half2float(__float2half(f[k] + b[k]));
    }
    if (SILU) {
#pragma unroll
        for (int k = 0; k < 8; ++k) f[k] = silu_sfu(f[k]);
        if (RES) {
#pragma unroll
            for (int k = 0; k < 8; ++k) f[k] = __half2float(__float2half(f[k]));
        }
    }
    if (RES) {
        float r[8];
        load8(res + i * 8, r);
#pragma unroll
        for (int k = 0; k < 8; ++k) f[k] += r[k];
    }
    store8(x + i * 8, f);
}

__global__ void __launch_bounds__(256)
silu_nhwc_kernel(const __half* __restrict__ x, __half* __restrict__ y, long long chunks) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= chunks) return;
    float f[8];
    load8(x + i * 8, f);
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] = silu_sfu(f[k]);
    store8(y + i * 8, f);
}

// out[n, ho, wo, :] from in[n, :, :, :], align_corners = true; a thread owns 8 channels of one output pixel, so the
// source coordinates and the two weights are computed once per 8 outputs and every access is 16 bytes. Grid: x over
// (wo, channel chunk) of one output row, y = ho, z = n: the row arithmetic is uniform over a CTA and the only
// division left is a 32-bit one (with one thread per flat 64-bit index the three divisions cost more than the loads).
__global__ void __launch_bounds__(256)
bilinear_upsample_nhwc_kernel(const __half* __restrict__ in, __half* __restrict__ out, int H_in, int W_in, int H_out, int W_out,
                              int c8) {
    const unsigned idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (unsigned)W_out * (unsigned)c8) return;
    const int w_out = (int)(idx / (unsigned)c8), cc = (int)(idx % (unsigned)c8);
    const int h_out = blockIdx.y;
    const long long n = blockIdx.z;
    const float h_scale = (H_out > 1) ? (float)(H_in - 1) / (H_out - 1) : 0.0f;
    const float w_scale = (W_out > 1) ? (float)(W_in - 1) / (W_out - 1) : 0.0f;
    const float h_in_f = h_out * h_scale, w_in_f = w_out * w_scale;
    const int h0 = (int)h_in_f, w0 = (int)w_in_f;
    const int h1 = min(h0 + 1, H_in - 1), w1 = min(w0 + 1, W_in - 1);
    const float hf = h_in_f - h0, wf = w_in_f - w0;
    const long long C = (long long)c8 * 8;
    const __half* base = in + n * H_in * W_in * C + cc * 8;
    float v00[8], v01[8], v10[8], v11[8], o[8];
    unpack8(ldg_half8(base + ((long long)h0 * W_in + w0) * C), v00);
    unpack8(ldg_half8(base + ((long long)h0 * W_in + w1) * C), v01);
    unpack8(ldg_half8(base + ((long long)h1 * W_in + w0) * C), v10);
    unpack8(ldg_half8(base + ((long long)h1 * W_in + w1) * C), v11);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = bilerp_ref(v00[k], v01[k], v10[k], v11[k], hf, wf);
    store8(out + ((n * H_out + h_out) * W_out) * C + (long long)idx * 8, o);
}

// A transposed convolution whose stride equals its kernel size f, as GEMM + this scatter: in [N*H*W, f*f*C] holds, for
// every input pixel, the f x f output pixels it produces (column (i*f + j)*C + c); out [N, H*f, W*f, C] (+ bias[c]).
__global__ void __launch_bounds__(256)
depth_to_space_bias_nhwc_kernel(const __half* __restrict__ in, const __half* __restrict__ bias, __half* __restrict__ out,
                                long long chunks, int H, int W, int c8, int f) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // over the OUTPUT, 8 channels each
    if (i >= chunks) return;
    const int cc = (int)(i % c8);
    long long p = i / c8;
    const int wo = (int)(p % (W * f));
    p /= (W * f);
    const int ho = (int)(p % (H * f));
    const long long n = p / (H * f);
    const int h = ho / f, di = ho % f, w = wo / f, dj = wo % f;
    const long long src = (((n * H + h) * W + w) * (f * f) + (di * f + dj)) * c8 + cc;
    float v[8];
    load8(in + src * 8, v);
    if (bias) {
        float b[8];
        load8(bias + cc * 8, b);
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] += b[k];
    }
    store8(out + i * 8, v);
}

// [N, HW, C] -> [N, C, HW] for small C (the head's last layer: C = 3): one thread per output element
__global__ void __launch_bounds__(256)
permute_nhwc_to_nchw_kernel(const __half* __restrict__ in, __half* __restrict__ out, long long total, long long HW, int C) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long hw = i % HW;
    const long long nc = i / HW;
    const int c = (int)(nc % C);
    const long long n = nc / C;
    out[i] = in[(n * HW + hw) * C + c];
}

// The head's last layer: a 1x1 convolution to a few channels (C_out <= 4: the image's colour channels) + bias, written
// planar. in [N*HW, C_in] channels-last, w [C_out, C_in], out [N, C_out, HW]; one thread per pixel: the pixel's C_in
// values are read once (16 bytes at a time) and every output plane is written with consecutive threads on consecutive
// pixels. fp32 accumulation over the channels in order, the product rounded to fp16 before the bias is added (as a
// convolution followed by the bias kernel does).
template <int COUT>
__global__ void __launch_bounds__(256)
pointwise_to_planar_kernel(const __half* __restrict__ in, const __half* __restrict__ w, const __half* __restrict__ bias,
                           __half* __restrict__ out, long long HW, long long total, int c_in) {
    extern __shared__ float sw[];  // [COUT][c_in]
    for (int i = threadIdx.x; i < COUT * c_in; i += blockDim.x) sw[i] = __half2float(w[i]);
    __syncthreads();
    const long long p = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= total) return;
    float acc[COUT];
#pragma unroll
    for (int o = 0; o < COUT; ++o) acc[o] = 0.0f;
    const __half* px = in + p * c_in;
    for (int c = 0; c < c_in; c += 8) {
        float v[8];
        load8(px + c, v);
#pragma unroll
        for (int o = 0; o < COUT; ++o)
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[o] = fmaf(v[k], sw[o * c_in + c + k], acc[o]);
    }
    const long long n = p / HW, hw = p % HW;
#pragma unroll
    for (int o = 0; o < COUT; ++o) {
        float r = __half2float(__float2half(acc[o]));
        if (bias) r += __half2float(bias[o]);
        out[(n * COUT + o) * HW + hw] = __float2half(r);
    }
}

// One-off weight layouts (at plan time): mode 0: [K, C, RS] -> [K, RS, C] (filter for channels-last convolutions);
// mode 1: transposed-convolution filter [Cin = K, Cout = C, RS = f*f] -> GEMM weight [(p * Cout + co)][ci].
__global__ void __launch_bounds__(256)
permute_filter_kernel(const __half* __restrict__ w, __half* __restrict__ out, int K, int C, int RS, int mode) {
    const long long total = (long long)K * C * RS;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int p = (int)(i % RS);
    const int c = (int)((i / RS) % C);
    const int k = (int)(i / ((long long)RS * C));
    const long long dst = mode == 0 ? ((long long)k * RS + p) * C + c : ((long long)p * C + c) * K + k;
    out[dst] = w[i];
}

template <bool BIAS, bool SILU, bool RES>
static int launch_bar(__half* x, const __half* bias, const __half* res, long long chunks, int c8, cudaStream_t st) {
    bias_act_residual_nhwc_kernel<BIAS, SILU, RES><<<(unsigned)ceil_div(chunks, 256), 256, 0, st>>>(x, bias, res, chunks, c8);
    return launch_status();
}

}  // namespace rfk

using namespace rfk;

extern "C" int rfk_bias_act_residual_nhwc(rfk_half* x, const rfk_half* bias, const rfk_half* residual, long long rows, int C,
                                          int silu, rfk_stream_t stream) {
    if (!x || rows < 0 || C <= 0) return RFK_EINVAL;
    if (rows == 0) return RFK_OK;
    if (C % 8 || !aligned16(x) || (bias && !aligned16(bias)) || (residual && !aligned16(residual))) return RFK_EUNSUPPORTED;
    const long long chunks = rows * (C / 8);
    if (chunks > 0xffffffffLL) return RFK_EUNSUPPORTED;
    __half* px = (__half*)x;
    const __half *pb = (const __half*)bias, *pr = (const __half*)residual;
    cudaStream_t st = as_stream(stream);
    const int c8 = C / 8;
    switch ((bias ? 4 : 0) | (silu ? 2 : 0) | (residual ? 1 : 0)) {
        case 0: return RFK_OK;
        case 1: return launch_bar<false, false, true>(px, pb, pr, chunks, c8, st);
        case 2: return launch_bar<false, true, false>(px, pb, pr, chunks, c8, st);
        case 3: return launch_bar<false, true, true>(px, pb, pr, chunks, c8, st);
        case 4: return launch_bar<true, false, false>(px, pb, pr, chunks, c8, st);
        case 5: return launch_bar<true, false, true>(px, pb, pr, chunks, c8, st);
        case 6: return launch_bar<true, true, false>(px, pb, pr, chunks, c8, st);
        default: return launch_bar<true, true, true>(px, pb, pr, chunks, c8, st);
    }
}

extern "C" int rfk_silu(const rfk_half* x, rfk_half* y, long long n, rfk_stream_t stream) {
    if (!x || !y || n < 0) return RFK_EINVAL;
    if (n == 0) return RFK_OK;
    if (n % 8 || !aligned16(x) || !aligned16(y)) return RFK_EUNSUPPORTED;
    silu_nhwc_kernel<<<(unsigned)ceil_div(n / 8, 256), 256, 0, as_stream(stream)>>>((const __half*)x, (__half*)y, n / 8);
    return launch_status();
}

extern "C" int rfk_bilinear_upsample_nhwc(const rfk_half* in, rfk_half* out, int N, int H_in, int W_in, int H_out, int W_out,
                                          int C, rfk_stream_t stream) {
    if (!in || !out || N < 0 || C <= 0 || H_in <= 0 || W_in <= 0 || H_out <= 0 || W_out <= 0) return RFK_EINVAL;
    if (N == 0) return RFK_OK;
    if (C % 8 || !aligned16(in) || !aligned16(out)) return RFK_EUNSUPPORTED;
    const long long per_row = (long long)W_out * (C / 8);
    if (per_row > 0x7fffffffLL || H_out > 65535 || N > 65535) return RFK_EUNSUPPORTED;
    dim3 grid((unsigned)ceil_div(per_row, 256), (unsigned)H_out, (unsigned)N);
    bilinear_upsample_nhwc_kernel<<<grid, 256, 0, as_stream(stream)>>>((const __half*)in, (__half*)out, H_in, W_in, H_out, W_out,
                                                                      C / 8);
    return launch_status();
}

extern "C" int rfk_depth_to_space_bias_nhwc(const rfk_half* in, const rfk_half* bias, rfk_half* out, int N, int H, int W, int C,
                                            int f, rfk_stream_t stream) {
    if (!in || !out || N < 0 || H <= 0 || W <= 0 || C <= 0 || f <= 0) return RFK_EINVAL;
    if (N == 0) return RFK_OK;
    if (C % 8 || !aligned16(in) || !aligned16(out) || (bias && !aligned16(bias))) return RFK_EUNSUPPORTED;
    const long long chunks = (long long)N * H * f * W * f * (C / 8);
    if (chunks > 0x7fffffffLL * 256) return RFK_EUNSUPPORTED;
    depth_to_space_bias_nhwc_kernel<<<(unsigned)ceil_div(chunks, 256), 256, 0, as_stream(stream)>>>(
        (const __half*)in, (const __half*)bias, (__half*)out, chunks, H, W, C / 8, f);
    return launch_status();
}

extern "C" int rfk_permute_nhwc_to_nchw(const rfk_half* in, rfk_half* out, int N, long long HW, int C, rfk_stream_t stream) {
    if (!in || !out || N < 0 || HW < 0 || C <= 0) return RFK_EINVAL;
    const long long total = (long long)N * HW * C;
    if (total == 0) return RFK_OK;
    if (total > 0x7fffffffLL * 256) return RFK_EUNSUPPORTED;
    permute_nhwc_to_nchw_kernel<<<(unsigned)ceil_div(total, 256), 256, 0, as_stream(stream)>>>((const __half*)in, (__half*)out,
                                                                                               total, HW, C);
    return launch_status();
}

extern "C" int rfk_permute_filter(const rfk_half* w, rfk_half* out, int K, int C, int RS, int mode, rfk_stream_t stream) {
    if (!w || !out || K <= 0 || C <= 0 || RS <= 0 || mode < 0 || mode > 1) return RFK_EINVAL;
    const long long total = (long long)K * C * RS;
    if (total > 0x7fffffffLL * 256) return RFK_EUNSUPPORTED;
    permute_filter_kernel<<<(unsigned)ceil_div(total, 256), 256, 0, as_stream(stream)>>>((const __half*)w, (__half*)out, K, C, RS,
                                                                                         mode);
    return launch_status();
}

extern "C" int rfk_pointwise_conv_to_planar(const rfk_half* in, const rfk_half* weight, const rfk_half* bias, rfk_half* out, int N,
                                            long long HW, int C_in, int C_out, rfk_stream_t stream) {
    if (!in || !weight || !out || N < 0 || HW < 0 || C_in <= 0 || C_out <= 0) return RFK_EINVAL;
    const long long total = (long long)N * HW;
    if (total == 0) return RFK_OK;
    if (C_out > 4 || C_in % 8 || C_in > 2048 || !aligned16(in)) return RFK_EUNSUPPORTED;
    if (total > 0x7fffffffLL * 256) return RFK_EUNSUPPORTED;
    const unsigned grid = (unsigned)ceil_div(total, 256);
    const size_t smem = (size_t)C_out * C_in * sizeof(float);
    cudaStream_t st = as_stream(stream);
    const __half *pi = (const __half*)in, *pw = (const __half*)weight, *pb = (const __half*)bias;
    __half* po = (__half*)out;
    switch (C_out) {
        case 1: pointwise_to_planar_kernel<1><<<grid, 256, smem, st>>>(pi, pw, pb, po, HW, total, C_in); break;
        case 2: pointwise_to_planar_kernel<2><<<grid, 256, smem, st>>>(pi, pw, pb, po, HW, total, C_in); break;
        case 3: pointwise_to_planar_kernel<3><<<grid, 256, smem, st>>>(pi, pw, pb, po, HW, total, C_in); break;
        default: pointwise_to_planar_kernel<4><<<grid, 256, smem, st>>>(pi, pw, pb, po, HW, total, C_in); break;
    }
    return launch_status();
}
