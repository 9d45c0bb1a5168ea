// Activations: SiLU(a)*b (SwiGLU gate), ELU, 10^x - 1, and the fused post-process chain.
//
// Reference semantics (BANANASJIM/renderformer-cuda, src/kernels/activations.cu):
//   :10-13  out = half((a / (1 + expf(-a))) * b)
//   :42-43  y = v > 0 ? v : alpha * (expf(v) - 1)
//   :56     y = powf(10, x) - 1
// and src/pipeline/render_session.cu:249-253 for the elu -> fp32 cast -> pow10 chain.
//
// Design: the SwiGLU gate is the only large tensor here (config 4: three passes over
// [4096,4096] fp16). With the reference's expf + IEEE division the kernel would be
// instruction-bound before it is HBM-bound on B200, so the sigmoid is evaluated as
// rcp.approx(1 + ex2.approx(-a*log2e)) (2 SFU ops per element, error far below the fp16
// rounding of the result) and every thread moves 8 elements per 128-bit access.
// ELU / 10^x-1 run on 0.8 M elements per view: they keep the reference's exact expf/powf
// so their results are bit-identical, and they are vectorised the same way.
#include "common.cuh"

namespace rfk {

__device__ __forceinline__ float silu_fast(float a) {
    // a * sigmoid(a); a -> -inf gives a * rcp(inf) = -0, a -> +inf gives a * 1
    return a * fast_rcp(1.0f + fast_exp2(a * -1.4426950408889634f));
}

template <typename T>
__global__ void __launch_bounds__(256)
silu_mul_kernel(const T* a, const T* __restrict__ b, T* out, long long n, int vec) {
    const long long i0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (i0 >= n) return;
    if (vec && i0 + 8 <= n) {
        float fa[8], fb[8];
        load8(a + i0, fa);
        load8(b + i0, fb);
#pragma unroll
        for (int i = 0; i < 8; ++i) fa[i] = silu_fast(fa[i]) * fb[i];
        store8(out + i0, fa);
    } else {
        for (long long i = i0; i < n && i < i0 + 8; ++i)
            out[i] = (T)(silu_fast((float)a[i]) * (float)b[i]);
    }
}

// gate_up [rows, 2*hidden] -> out [rows, hidden]
__global__ void __launch_bounds__(256)
swiglu_kernel(const __half* gate_up, __half* out, long long rows, int hidden,
              long long out_pitch, int vec) {  // out may alias the gate half of gate_up
    const int cpr = (hidden + 7) / 8;
    const long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= rows * cpr) return;
    const long long row = c / cpr;
    const int j0 = (int)(c % cpr) * 8;
    const __half* g = gate_up + row * 2 * hidden + j0;
    const __half* u = g + hidden;
    __half* o = out + row * out_pitch + j0;
    if (vec) {
        float fg[8], fu[8];
        unpack8(ldcs_half8(g), fg);
        unpack8(ldcs_half8(u), fu);
#pragma unroll
        for (int i = 0; i < 8; ++i) fg[i] = silu_fast(fg[i]) * fu[i];
        store8(o, fg);
    } else {
        for (int i = 0; i < 8 && j0 + i < hidden; ++i)
            o[i] = __float2half(silu_fast(__half2float(g[i])) * __half2float(u[i]));
    }
}

enum { POST_ELU = 0, POST_POW10 = 1, POST_ELU_POW10 = 2 };

__device__ __forceinline__ float elu_ref(float v, float alpha) {
    return v > 0.0f ? v : alpha * (expf(v) - 1.0f);
}

template <int OP, typename TI, typename TO>
__global__ void __launch_bounds__(256)
post_kernel(const TI* x, TO* y, long long n, float alpha, int vec) {
    const long long i0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (i0 >= n) return;
    auto f = [&](float v) -> float {
        if (OP == POST_ELU) return elu_ref(v, alpha);
        if (OP == POST_POW10) return powf(10.0f, v) - 1.0f;
        return powf(10.0f, round_half(elu_ref(v, alpha))) - 1.0f;
    };
    if (vec && i0 + 8 <= n) {
        float v[8];
        load8(x + i0, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = f(v[i]);
        store8(y + i0, v);
    } else {
        for (long long i = i0; i < n && i < i0 + 8; ++i) y[i] = (TO)f((float)x[i]);
    }
}

template <int OP, typename TI, typename TO>
static int launch_post(const TI* x, TO* y, long long n, float alpha, cudaStream_t st) {
    if (!x || !y || n < 0) return RFK_EINVAL;
    if (n == 0) return RFK_OK;
    const int vec = aligned16(x) && aligned16(y);
    post_kernel<OP, TI, TO><<<ceil_div((n + 7) / 8, 256), 256, 0, st>>>(x, y, n, alpha, vec);
    return launch_status();
}

}  // namespace rfk

using namespace rfk;

extern "C" int rfk_fused_silu_mul(const rfk_half* a, const rfk_half* b, rfk_half* out, long long n,
                                  rfk_stream_t stream) {
    if (!a || !b || !out || n < 0) return RFK_EINVAL;
    if (n == 0) return RFK_OK;
    const int vec = aligned16(a) && aligned16(b) && aligned16(out);
    silu_mul_kernel<__half><<<ceil_div((n + 7) / 8, 256), 256, 0, as_stream(stream)>>>(
        (const __half*)a, (const __half*)b, (__half*)out, n, vec);
    return launch_status();
}

extern "C" int rfk_fused_silu_mul_f32(const float* a, const float* b, float* out, long long n,
                                      rfk_stream_t stream) {
    if (!a || !b || !out || n < 0) return RFK_EINVAL;
    if (n == 0) return RFK_OK;
    const int vec = aligned16(a) && aligned16(b) && aligned16(out);
    silu_mul_kernel<float><<<ceil_div((n + 7) / 8, 256), 256, 0, as_stream(stream)>>>(a, b, out, n,
                                                                                      vec);
    return launch_status();
}

extern "C" int rfk_swiglu(const rfk_half* gate_up, rfk_half* out, int rows, int hidden,
                          rfk_stream_t stream) {
    if (!gate_up || !out || rows < 0 || hidden <= 0) return RFK_EINVAL;
    if (rows == 0) return RFK_OK;
    const int vec = hidden % 8 == 0 && aligned16(gate_up) && aligned16(out);
    const long long chunks = (long long)rows * ((hidden + 7) / 8);
    swiglu_kernel<<<ceil_div(chunks, 256), 256, 0, as_stream(stream)>>>(
        (const __half*)gate_up, (__half*)out, rows, hidden, hidden, vec);
    return launch_status();
}

extern "C" int rfk_swiglu_inplace(rfk_half* gate_up, int rows, int hidden, rfk_stream_t stream) {
    if (!gate_up || rows < 0 || hidden <= 0) return RFK_EINVAL;
    if (rows == 0) return RFK_OK;
    const int vec = hidden % 8 == 0 && aligned16(gate_up);
    const long long chunks = (long long)rows * ((hidden + 7) / 8);
    // every thread overwrites exactly the gate elements it has just read
    swiglu_kernel<<<ceil_div(chunks, 256), 256, 0, as_stream(stream)>>>(
        (const __half*)gate_up, (__half*)gate_up, rows, hidden, 2LL * hidden, vec);
    return launch_status();
}

extern "C" int rfk_elu(const rfk_half* x, rfk_half* y, long long n, float alpha,
                       rfk_stream_t stream) {
    return launch_post<POST_ELU>((const __half*)x, (__half*)y, n, alpha, as_stream(stream));
}

extern "C" int rfk_pow10_minus1(const float* x, float* y, long long n, rfk_stream_t stream) {
    return launch_post<POST_POW10>(x, y, n, 0.0f, as_stream(stream));
}

extern "C" int rfk_post_elu_pow10(const rfk_half* x, float* y, long long n, float alpha,
                                  rfk_stream_t stream) {
    return launch_post<POST_ELU_POW10>((const __half*)x, y, n, alpha, as_stream(stream));
}
