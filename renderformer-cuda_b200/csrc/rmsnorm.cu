// RMSNorm family: plain, and fused with the residual add that precedes it and the
// fp16 cast that follows it.
//
// Reference semantics (BANANASJIM/renderformer-cuda):
//   src/kernels/rmsnorm.cu:17-50,67-90   s = sum x^2 ; r = rsqrtf(s/dim + eps) ; y = (x*r)*gamma
//   src/layers/transformer.cu:9-19       y16 = half(float(y16) + float(r16))
//   src/layers/transformer.cu:21-30      y32 += r32
//   src/layers/transformer.cu:52-61      y32 += float(r16)
//   src/layers/transformer.cu:32-35      out16 = half(in32)
//
// Design: the op is a pure HBM stream (config 1: 3 fp32 row passes + 1 fp16 pass,
// < 1 flop/byte). A row lives in registers between the sum-of-squares and the scaling
// pass, so every byte crosses HBM exactly once. Each lane moves 8 consecutive elements per
// access (128-bit loads/stores for fp16, 2 x 128-bit for fp32).
// A row is spread over W warps of a 128-thread CTA (W = 4 for dim 1024, i.e. one row per
// CTA and one chunk per thread). A first version gave each warp a whole row (32 floats of h
// and of r per lane): ncu showed 30 % DRAM utilisation with every warp stalled on its own
// loads (long-scoreboard 35 cycles/issue), because the whole grid loaded in lock step and
// then stored in lock step, in 1.4 waves. Small CTAs of short-lived threads (32 registers,
// 16 CTAs per SM) retire and get replaced continuously, so loads of new rows overlap the
// stores of finished ones. The W partial sums meet through 16 bytes of shared memory.
#include "common.cuh"

namespace rfk {

template <typename T> struct IsHalf { static constexpr bool value = false; };
template <> struct IsHalf<__half> { static constexpr bool value = true; };

constexpr int kRmsThreads = 128;

// Token (b, h, w) of a [B, H, W] grid -> its row in swin window order (windows of ws x ws over the
// grid shifted by -shift, as the reference's cyclic shift + window_partition produce).
struct WinRows {
    int H, W, ws, shift;
    __device__ __forceinline__ long long operator()(long long token) const {
        const int w = (int)(token % W);
        const long long t = token / W;
        const int h = (int)(t % H);
        const long long b = t / H;
        const int hs = (h + shift) % H, wsft = (w + shift) % W;  // position in the shifted grid
        const int nWw = W / ws, nW = (H / ws) * nWw;
        const int win = (hs / ws) * nWw + wsft / ws, local = (hs % ws) * ws + wsft % ws;
        return (b * nW + win) * (long long)(ws * ws) + local;
    }
};

// TH: hidden-state storage, TR: residual storage, TY: normalised output storage.
// MAP: 0 all operands in token order; 1 y is written in window order; 2 r is read in window order.
// W: warps per row (1, 2 or 4); NCH: 8-element chunks per lane (dim <= NCH * W * 256).
template <typename TH, typename TR, typename TY, int NCH, int W, bool HAS_RES, bool WRITE_H, int MAP = 0>
__global__ void __launch_bounds__(kRmsThreads)
rmsnorm_row_kernel(const TH* x, TH* xw, const TR* __restrict__ r,
                   const float* __restrict__ gamma, TY* y,  // x, xw, y may alias
                   int rows, int dim, float eps, WinRows wr = WinRows{}) {
    constexpr int kWarps = kRmsThreads / 32;
    constexpr int kRowsPerCta = kWarps / W;
    __shared__ float s_part[kWarps];
    pdl_wait();
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int wir = warp % W;  // warp index within its row
    long long row = (long long)blockIdx.x * kRowsPerCta + warp / W;
    const bool live = row < rows;
    if (!live) row = rows - 1;  // idle warps shadow the last row and never store
    const size_t base = (size_t)row * dim;
    const size_t rbase = MAP == 2 ? (size_t)wr(row) * dim : base;
    const size_t ybase = MAP == 1 ? (size_t)wr(row) * dim : base;

    float v[NCH][8];
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
        const int off = (wir * 32 + lane + k * W * 32) * 8;
        if (off < dim) load8(x + base + off, v[k]);
    }
    if (HAS_RES) {
#pragma unroll
        for (int k = 0; k < NCH; ++k) {
            const int off = (wir * 32 + lane + k * W * 32) * 8;
            if (off < dim) {
                float rr[8];
                load8(r + rbase + off, rr);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float s = v[k][i] + rr[i];
                    // an fp16 hidden state is stored, then re-read by the norm
                    v[k][i] = IsHalf<TH>::value ? round_half(s) : s;
                }
                if (WRITE_H && live) store8(xw + base + off, v[k]);
            }
        }
    }
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
        const int off = (wir * 32 + lane + k * W * 32) * 8;
        if (off < dim) {
#pragma unroll
            for (int i = 0; i < 8; ++i) ss = fmaf(v[k][i], v[k][i], ss);
        }
    }
    ss = warp_sum(ss);
    if (W > 1) {
        if (lane == 0) s_part[warp] = ss;
        __syncthreads();
        ss = 0.0f;
#pragma unroll
        for (int i = 0; i < W; ++i) ss += s_part[(warp / W) * W + i];
    }
    const float rinv = rsqrtf(ss * (1.0f / (float)dim) + eps);
    if (!live) return;
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
        const int off = (wir * 32 + lane + k * W * 32) * 8;
        if (off < dim) {
            float g[8], o[8];
            ldg_float8(gamma + off, g);
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = (v[k][i] * rinv) * g[i];
            store8(y + ybase + off, o);
        }
    }
}

// Any dim / any alignment: one CTA per row, scalar accesses, the row is re-read.
template <typename TH, typename TR, typename TY, bool HAS_RES, bool WRITE_H>
__global__ void __launch_bounds__(256)
rmsnorm_generic_kernel(const TH* x, TH* xw, const TR* __restrict__ r,
                       const float* __restrict__ gamma, TY* y, int dim, float eps) {
    __shared__ float red[8];
    const size_t base = (size_t)blockIdx.x * dim;
    auto value = [&](int i) -> float {
        float s = (float)x[base + i];
        if (HAS_RES) {
            s += (float)r[base + i];
            if (IsHalf<TH>::value) s = round_half(s);
        }
        return s;
    };
    float ss = 0.0f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        float s = value(i);
        ss = fmaf(s, s, ss);
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) tot += red[w];
    const float rinv = rsqrtf(tot / (float)dim + eps);
    // every thread re-reads exactly the elements it will overwrite, so y == x is safe
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        float s = value(i);
        if (HAS_RES && WRITE_H) xw[base + i] = (TH)s;
        y[base + i] = (TY)((s * rinv) * gamma[i]);
    }
}

template <typename TH, typename TR, typename TY, bool HAS_RES, bool WRITE_H>
static int launch_variant(const TH* x, TH* xw, const TR* r, const float* gamma, TY* y,
                          int rows, int dim, float eps, cudaStream_t st) {
    const bool vec = (dim % 8 == 0) && dim <= 2048 && aligned16(x) && aligned16(y) &&
                     aligned16(gamma) && (!HAS_RES || aligned16(r)) &&
                     (!WRITE_H || aligned16(xw));
    if (vec) {
#define RFK_RMS_LAUNCH(N, WW)                                                                         \
    launch_pdl(rmsnorm_row_kernel<TH, TR, TY, N, WW, HAS_RES, WRITE_H, 0>,                             \
               dim3(ceil_div(rows, (kRmsThreads / 32) / WW)), dim3(kRmsThreads), 0, st, x, xw, r, gamma, y, \
               rows, dim, eps, WinRows{})
        if (dim <= 256) RFK_RMS_LAUNCH(1, 1);
        else if (dim <= 512) RFK_RMS_LAUNCH(1, 2);
        else if (dim <= 1024) RFK_RMS_LAUNCH(1, 4);
        else RFK_RMS_LAUNCH(2, 4);
#undef RFK_RMS_LAUNCH
    } else {
        rmsnorm_generic_kernel<TH, TR, TY, HAS_RES, WRITE_H><<<rows, 256, 0, st>>>(
            x, xw, r, gamma, y, dim, eps);
    }
    return launch_status();
}

template <typename TH, typename TR, typename TY>
static int launch_rmsnorm(const TH* x, TH* xw, const TR* r, const float* gamma, TY* y,
                          int rows, int dim, float eps, cudaStream_t st) {
    if (!x || !gamma || !y || rows < 0 || dim <= 0) return RFK_EINVAL;
    if (rows == 0) return RFK_OK;
    if (r) return launch_variant<TH, TR, TY, true, true>(x, xw, r, gamma, y, rows, dim, eps, st);
    return launch_variant<TH, TR, TY, false, false>(x, xw, r, gamma, y, rows, dim, eps, st);
}

}  // namespace rfk

using namespace rfk;

extern "C" int rfk_rmsnorm(const rfk_half* x, const float* gamma, rfk_half* y, int rows, int dim,
                           float eps, rfk_stream_t stream) {
    return launch_rmsnorm<__half, __half, __half>((const __half*)x, nullptr, nullptr, gamma,
                                                  (__half*)y, rows, dim, eps, as_stream(stream));
}

extern "C" int rfk_rmsnorm_f32(const float* x, const float* gamma, float* y, int rows, int dim,
                               float eps, rfk_stream_t stream) {
    return launch_rmsnorm<float, float, float>(x, nullptr, nullptr, gamma, y, rows, dim, eps,
                                               as_stream(stream));
}

extern "C" int rfk_rmsnorm_residual_f32_cast16(float* h, const float* r, const float* gamma,
                                               rfk_half* y16, int rows, int dim, float eps,
                                               rfk_stream_t stream) {
    return launch_rmsnorm<float, float, __half>(h, h, r, gamma, (__half*)y16, rows, dim, eps,
                                                as_stream(stream));
}

extern "C" int rfk_rmsnorm_residual_mixed_cast16(float* h, const rfk_half* r, const float* gamma,
                                                 rfk_half* y16, int rows, int dim, float eps,
                                                 rfk_stream_t stream) {
    return launch_rmsnorm<float, __half, __half>(h, h, (const __half*)r, gamma, (__half*)y16, rows,
                                                 dim, eps, as_stream(stream));
}

extern "C" int rfk_rmsnorm_residual_f16_windows(rfk_half* x, const rfk_half* r, const float* gamma,
                                                rfk_half* y, int B, int H, int W, int dim,
                                                int window_size, int shift_size, int windowed_operand,
                                                float eps, rfk_stream_t stream) {
    if (!x || !gamma || !y || B < 0 || H <= 0 || W <= 0 || dim <= 0) return RFK_EINVAL;
    if (window_size <= 0 || H % window_size || W % window_size || shift_size < 0) return RFK_EINVAL;
    if (windowed_operand != 1 && windowed_operand != 2) return RFK_EINVAL;
    if (!r && windowed_operand != 1) return RFK_EINVAL;  // without a residual only the output can be in window order
    if ((const void*)x == (const void*)y || (r && (const void*)r == (const void*)y)) return RFK_EINVAL;
    if (dim % 8 != 0 || dim > 2048 || !aligned16(x) || !aligned16(y) || !aligned16(gamma) || (r && !aligned16(r)))
        return RFK_EUNSUPPORTED;
    const long long rows_ll = (long long)B * H * W;
    if (rows_ll > 0x7fffffffLL) return RFK_EUNSUPPORTED;
    const int rows = (int)rows_ll;
    if (rows == 0) return RFK_OK;
    const WinRows wr{H, W, window_size, shift_size};
    cudaStream_t st = as_stream(stream);
    __half* xh = (__half*)x;
#define RFK_RMS_WIN(N, WW, M)                                                                                   \
    if (r)                                                                                                      \
        launch_pdl(rmsnorm_row_kernel<__half, __half, __half, N, WW, true, true, M>,                             \
                   dim3(ceil_div(rows, (kRmsThreads / 32) / WW)), dim3(kRmsThreads), 0, st, (const __half*)xh, xh, \
                   (const __half*)r, gamma, (__half*)y, rows, dim, eps, wr);                                     \
    else                                                                                                        \
        launch_pdl(rmsnorm_row_kernel<__half, __half, __half, N, WW, false, false, 1>,                           \
                   dim3(ceil_div(rows, (kRmsThreads / 32) / WW)), dim3(kRmsThreads), 0, st, (const __half*)xh, xh, \
                   (const __half*)nullptr, gamma, (__half*)y, rows, dim, eps, wr)
#define RFK_RMS_WIN_DIM(M)                            \
    if (dim <= 256) { RFK_RMS_WIN(1, 1, M); }         \
    else if (dim <= 512) { RFK_RMS_WIN(1, 2, M); }    \
    else if (dim <= 1024) { RFK_RMS_WIN(1, 4, M); }   \
    else { RFK_RMS_WIN(2, 4, M); }
    if (windowed_operand == 1) { RFK_RMS_WIN_DIM(1); } else { RFK_RMS_WIN_DIM(2); }
#undef RFK_RMS_WIN_DIM
#undef RFK_RMS_WIN
    return launch_status();
}

extern "C" int rfk_rmsnorm_residual_f16(rfk_half* x, const rfk_half* r, const float* gamma,
                                        rfk_half* y, int rows, int dim, float eps,
                                        rfk_stream_t stream) {
    if (r && (const void*)x == (const void*)y) return RFK_EINVAL;
    return launch_rmsnorm<__half, __half, __half>((const __half*)x, (__half*)x, (const __half*)r,
                                                  gamma, (__half*)y, rows, dim, eps,
                                                  as_stream(stream));
}
