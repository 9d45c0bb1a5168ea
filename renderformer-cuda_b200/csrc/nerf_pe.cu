// NeRF positional encoding: out = [x, sin(f_k * x_d) (d major, k minor), cos(f_k * x_d)].
//
// Reference semantics (BANANASJIM/renderformer-cuda, src/kernels/nerf_pe.cu):
//   :57-61  f_k = pow(2.0f, min + (max - min) * k / max(nf - 1, 1)), computed on the host
//   :26-45  feature order and the fp16 / fp32 input forms
// The reference wrapper cudaMalloc's, uploads and cudaFree's the frequency table on every
// call (:64-78), which synchronises the device and cannot be captured in a graph. Here the
// table travels in the kernel parameter block (<= 32 floats), so the call is a plain
// asynchronous launch.
//
// Design: output rows are 2*(in_dim*(2nf+1)) bytes (234 B for the 9-D normals, 78 B for
// ray directions), never 16-byte multiples, so the output is treated as one flat fp16
// array and each thread produces 8 consecutive elements with a single 128-bit store.
// sin/cos arguments are reduced to [-pi, pi] with a two-constant Cody-Waite step and
// evaluated on the SFU; accurate sinf/cosf would make the ray-direction case
// (11 M outputs) instruction-bound at ~4x its HBM time.
#include "common.cuh"
#include <cmath>

namespace rfk {

struct FreqTable {
    float f[32];
};

__device__ __forceinline__ float sincos_sel(float val, bool is_cos) {
    if (fabsf(val) < 8192.0f) {
        // k = round(val / 2pi); r = val - k*2pi with 2pi split into hi + lo parts
        const float k = rintf(val * 0.15915494309189535f);
        float r = fmaf(k, -6.2831854820251465f, val);   // 2pi rounded to fp32
        r = fmaf(k, 1.7484555e-7f, r);                  // 2pi - fl(2pi) = -1.7484555e-7
        return is_cos ? __cosf(r) : __sinf(r);
    }
    return is_cos ? cosf(val) : sinf(val);
}

template <typename TI>
__device__ __forceinline__ float pe_element(const TI* __restrict__ in_row, int feat, int in_dim,
                                            int num_freqs, int include_input,
                                            const FreqTable& ft) {
    int enc = feat;
    if (include_input) {
        if (feat < in_dim) return (float)in_row[feat];
        enc -= in_dim;
    }
    const int half_dim = in_dim * num_freqs;
    const bool is_cos = enc >= half_dim;
    const int si = is_cos ? enc - half_dim : enc;
    const int d = si / num_freqs, f = si - d * num_freqs;
    const float val = (float)in_row[d] * ft.f[f];
    return sincos_sel(val, is_cos);
}

template <typename TI>
__global__ void __launch_bounds__(256)
nerf_pe_kernel(const TI* __restrict__ input, __half* __restrict__ output, long long total,
               int in_dim, int num_freqs, int out_dim, int include_input,
               const __grid_constant__ FreqTable ft, int vec) {
    const long long e0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (e0 >= total) return;
    long long row = e0 / out_dim;
    int feat = (int)(e0 - row * out_dim);
    float o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        o[i] = 0.0f;
        if (e0 + i < total) o[i] = pe_element(input + row * in_dim, feat, in_dim, num_freqs,
                                              include_input, ft);
        if (++feat == out_dim) { feat = 0; ++row; }
    }
    if (vec && e0 + 8 <= total) {
        st_half8(output + e0, pack8(o));
    } else {
        for (int i = 0; i < 8 && e0 + i < total; ++i) output[e0 + i] = __float2half(o[i]);
    }
}

template <typename TI>
static int launch_nerf_pe(const TI* input, __half* output, int batch, int seq_len, int in_dim,
                          int num_freqs, float min_exp, float max_exp, int include_input,
                          cudaStream_t st) {
    if (!input || !output || batch < 0 || seq_len < 0 || in_dim <= 0 || num_freqs <= 0)
        return RFK_EINVAL;
    if (num_freqs > 32) return RFK_ETOOBIG;
    const int out_dim = in_dim * num_freqs * 2 + (include_input ? in_dim : 0);
    const long long total = (long long)batch * seq_len * out_dim;
    if (total == 0) return RFK_OK;
    FreqTable ft{};
    for (int i = 0; i < num_freqs; ++i) {
        // same expression, in float, as the reference's host loop
        float e = min_exp + (max_exp - min_exp) * i / std::max(num_freqs - 1, 1);
        ft.f[i] = std::pow(2.0f, e);
    }
    const int vec = aligned16(output);
    nerf_pe_kernel<TI><<<ceil_div((total + 7) / 8, 256), 256, 0, st>>>(
        input, output, total, in_dim, num_freqs, out_dim, include_input ? 1 : 0, ft, vec);
    return launch_status();
}

}  // namespace rfk

using namespace rfk;

extern "C" int rfk_nerf_pe(const rfk_half* input, rfk_half* output, int batch, int seq_len,
                           int in_dim, int num_freqs, float min_freq_exp, float max_freq_exp,
                           int include_input, rfk_stream_t stream) {
    return launch_nerf_pe<__half>((const __half*)input, (__half*)output, batch, seq_len, in_dim,
                                  num_freqs, min_freq_exp, max_freq_exp, include_input,
                                  as_stream(stream));
}

extern "C" int rfk_nerf_pe_f32(const float* input, rfk_half* output, int batch, int seq_len,
                               int in_dim, int num_freqs, float min_freq_exp, float max_freq_exp,
                               int include_input, rfk_stream_t stream) {
    return launch_nerf_pe<float>(input, (__half*)output, batch, seq_len, in_dim, num_freqs,
                                 min_freq_exp, max_freq_exp, include_input, as_stream(stream));
}
