// Element-wise / layout operators of the DPT head (everything in it that is not a convolution).
//
// Reference semantics (BANANASJIM/renderformer-cuda, src/layers/dpt.cu):
//   :240-277  bilinear_upsample, NCHW fp16, align_corners = true:
//             scale = (in - 1) / (out - 1) (0 when out == 1), src = dst * scale, i0 = (int)src,
//             i1 = min(i0 + 1, in - 1), f = src - i0,
//             val = v00*(1-hf)*(1-wf) + v01*(1-hf)*wf + v10*hf*(1-wf) + v11*hf*wf, rounded to fp16
//   :289-298  silu_inplace: x = half(v / (1 + expf(-v)))
//   :88-96    add_bias_nchw_kernel: out[n,c,:] = half(float(out[n,c,:]) + float(bias[c]))
//   :303-318  permute_bsd_to_nchw: out[b,d,h,w] = in[b, h*pW + w, d]
//
// Design. All four are HBM-bound streams over feature maps of up to 256 x 512 x 512 fp16 (134 MB).
// The reference gives every element its own thread with two or three integer divisions and
// 2-byte accesses; here a thread owns 8 consecutive elements of a row (one 128-bit store), the
// row / plane decomposition is done once per thread, and the source rows of the upsample are
// read through the read-only path (each input value is used by up to 2 x 2 x scale^2 outputs, so
// it is served from L1/L2). The interpolation keeps the reference's expression, term for term.
// SiLU uses ex2 + rcp on the special-function unit like the SwiGLU gate (the reference's expf and
// IEEE division would make the kernel instruction-bound); the permute is a 64 x 64 tile
// transpose through shared memory so that both sides move full 128-byte lines.
#include "common.cuh"
#include "dpt_math.cuh"

namespace rfk {

// One thread = 8 consecutive output columns x kUpRows consecutive output rows of one plane: the column
// arithmetic (two int <-> float conversions per column, which run on the 16-per-clock conversion
// unit) is done once and reused for every row, the row arithmetic once per 8 outputs.
constexpr int kUpRows = 4;
__global__ void __launch_bounds__(256)
bilinear_upsample_kernel(const __half* __restrict__ in, __half* __restrict__ out, long long planes, int H_in, int W_in,
                         int H_out, int W_out, int vec) {
    const int cpr = (W_out + 7) / 8;                    // column chunks per output row
    const int rpp = (H_out + kUpRows - 1) / kUpRows;    // row groups per plane
    const long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= planes * rpp * cpr) return;
    const int w0o = (int)(c % cpr) * 8;
    const long long rg = c / cpr;
    const int h_out0 = (int)(rg % rpp) * kUpRows;
    const long long plane = rg / rpp;
    const float h_scale = (H_out > 1) ? (float)(H_in - 1) / (H_out - 1) : 0.0f;
    const float w_scale = (W_out > 1) ? (float)(W_in - 1) / (W_out - 1) : 0.0f;
    int w0[8];
    float wf[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int w_out = min(w0o + i, W_out - 1);
        const float w_in_f = w_out * w_scale;
        w0[i] = (int)w_in_f;
        wf[i] = w_in_f - w0[i];
    }
    const __half* pin = in + plane * H_in * W_in;
#pragma unroll
    for (int r = 0; r < kUpRows; ++r) {
        const int h_out = h_out0 + r;
        if (h_out >= H_out) break;
        const float h_in_f = h_out * h_scale;
        const int h0 = (int)h_in_f;
        const int h1 = min(h0 + 1, H_in - 1);
        const float hf = h_in_f - h0;
        const __half* r0 = pin + (long long)h0 * W_in;
        const __half* r1 = pin + (long long)h1 * W_in;
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int w1 = min(w0[i] + 1, W_in - 1);
            v[i] = bilerp_ref(__half2float(__ldg(r0 + w0[i])), __half2float(__ldg(r0 + w1)),
                              __half2float(__ldg(r1 + w0[i])), __half2float(__ldg(r1 + w1)), hf, wf[i]);
        }
        __half* o = out + (plane * H_out + h_out) * (long long)W_out + w0o;
        if (vec) {
            store8(o, v);
        } else {
            for (int i = 0; i < 8 && w0o + i < W_out; ++i) o[i] = __float2half(v[i]);
        }
    }
}

__global__ void __launch_bounds__(256)
silu_inplace_kernel(__half* x, long long n, int vec) {
    const long long i0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (i0 >= n) return;
    if (vec && i0 + 8 <= n) {
        float f[8];
        load8(x + i0, f);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = silu_sfu(f[i]);
        store8(x + i0, f);
    } else {
        for (long long i = i0; i < n && i < i0 + 8; ++i) x[i] = __float2half(silu_sfu(__half2float(x[i])));
    }
}

// x [planes_total = N*C, HW] += bias[c], c = plane % C; one thread = 8 consecutive pixels of a plane
__global__ void __launch_bounds__(256)
add_bias_nchw_kernel(__half* x, const __half* __restrict__ bias, long long planes, int C, long long HW, int vec) {
    const long long cpp = (HW + 7) / 8;  // chunks per plane
    const long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= planes * cpp) return;
    const long long plane = c / cpp;
    const long long p0 = (c % cpp) * 8;
    const float b = __half2float(__ldg(bias + (int)(plane % C)));
    __half* px = x + plane * HW + p0;
    if (vec) {
        float f[8];
        load8(px, f);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] += b;
        store8(px, f);
    } else {
        for (int i = 0; i < 8 && p0 + i < HW; ++i) px[i] = __float2half(__half2float(px[i]) + b);
    }
}

// in [B, S, D] -> out [B, D, S]: 64 x 64 tiles through shared memory (row pitch 66 halves: the
// column reads of the second phase fall on distinct banks pair-wise)
constexpr int kPermTile = 64;
__global__ void __launch_bounds__(256)
permute_bsd_to_nchw_kernel(const __half* __restrict__ in, __half* __restrict__ out, int S, int D) {
    __shared__ __half tile[kPermTile][kPermTile + 2];
    const int b = blockIdx.z;
    const int s0 = blockIdx.y * kPermTile, d0 = blockIdx.x * kPermTile;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
    const __half* src = in + (long long)b * S * D;
    __half* dst = out + (long long)b * S * D;
    // phase 1: rows of the tile are tokens, a lane reads channels d0 + 2*tx, +1
#pragma unroll
    for (int r = ty; r < kPermTile; r += 8) {
        const int s = s0 + r, d = d0 + 2 * tx;
        __half a = __float2half(0.0f), c = a;
        if (s < S) {
            if (d < D) a = src[(long long)s * D + d];
            if (d + 1 < D) c = src[(long long)s * D + d + 1];
        }
        tile[r][2 * tx] = a;
        tile[r][2 * tx + 1] = c;
    }
    __syncthreads();
    // phase 2: rows of the output are channels, a lane writes tokens s0 + 2*tx, +1
#pragma unroll
    for (int r = ty; r < kPermTile; r += 8) {
        const int d = d0 + r, s = s0 + 2 * tx;
        if (d < D) {
            if (s < S) dst[(long long)d * S + s] = tile[2 * tx][r];
            if (s + 1 < S) dst[(long long)d * S + s + 1] = tile[2 * tx + 1][r];
        }
    }
}

}  // namespace rfk

using namespace rfk;

extern "C" int rfk_bilinear_upsample(const rfk_half* in, rfk_half* out, int N, int C, int H_in, int W_in, int H_out,
                                     int W_out, rfk_stream_t stream) {
    if (!in || !out || N < 0 || C < 0 || H_in <= 0 || W_in <= 0 || H_out <= 0 || W_out <= 0) return RFK_EINVAL;
    const long long planes = (long long)N * C;
    if (planes == 0) return RFK_OK;
    const long long chunks = planes * ((H_out + kUpRows - 1) / kUpRows) * ((W_out + 7) / 8);
    if (chunks > 0x7fffffffLL * 256) return RFK_EUNSUPPORTED;
    const int vec = (W_out % 8 == 0) && aligned16(out);
    bilinear_upsample_kernel<<<(unsigned)ceil_div(chunks, 256), 256, 0, as_stream(stream)>>>(
        (const __half*)in, (__half*)out, planes, H_in, W_in, H_out, W_out, vec);
    return launch_status();
}

extern "C" int rfk_silu_inplace(rfk_half* x, long long n, rfk_stream_t stream) {
    if (!x || n < 0) return RFK_EINVAL;
    if (n == 0) return RFK_OK;
    silu_inplace_kernel<<<(unsigned)ceil_div(ceil_div(n, 8), 256), 256, 0, as_stream(stream)>>>((__half*)x, n,
                                                                                                 aligned16(x));
    return launch_status();
}

extern "C" int rfk_add_bias_nchw(rfk_half* x, const rfk_half* bias, int N, int C, long long HW, rfk_stream_t stream) {
    if (!x || !bias || N < 0 || C <= 0 || HW < 0) return RFK_EINVAL;
    const long long planes = (long long)N * C;
    if (planes == 0 || HW == 0) return RFK_OK;
    const long long chunks = planes * ((HW + 7) / 8);
    const int vec = (HW % 8 == 0) && aligned16(x);
    add_bias_nchw_kernel<<<(unsigned)ceil_div(chunks, 256), 256, 0, as_stream(stream)>>>((__half*)x, (const __half*)bias,
                                                                                         planes, C, HW, vec);
    return launch_status();
}

extern "C" int rfk_permute_bsd_to_nchw(const rfk_half* in, rfk_half* out, int B, int S, int D, rfk_stream_t stream) {
    if (!in || !out || B < 0 || S < 0 || D < 0) return RFK_EINVAL;
    if (B == 0 || S == 0 || D == 0) return RFK_OK;
    if (B > 65535 || ceil_div(S, kPermTile) > 65535) return RFK_EUNSUPPORTED;
    dim3 grid((unsigned)ceil_div(D, kPermTile), (unsigned)ceil_div(S, kPermTile), (unsigned)B);
    permute_bsd_to_nchw_kernel<<<grid, 256, 0, as_stream(stream)>>>((const __half*)in, (__half*)out, S, D);
    return launch_status();
}
