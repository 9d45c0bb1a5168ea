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
// ray directions), never 16-byte multiples, and the reference spends one thread, two
// integer divisions and one sinf OR cosf per output element, which makes the op
// instruction-bound (measured: 35 us for the 22 MB ray-direction case on B200 with that
// structure). Here a CTA owns a tile of consecutive rows whose byte size is a multiple of
// 16: each (row, d, k) item is evaluated once with a shared range reduction and one
// sin+cos pair on the SFU, results are staged in shared memory in output order, and the
// tile is then streamed to HBM with 128-bit stores. Index arithmetic uses multiply-high
// reciprocals instead of divisions.
#include "common.cuh"
#include <cmath>

namespace rfk {

struct FreqTable {
    float f[32];
};

// n / d for n*d < 2^32 via one multiply-high (m = ceil(2^32 / d)); d == 1 handled apart.
struct FastDiv {
    unsigned m, d;
    __host__ explicit FastDiv(unsigned dd = 1) : m(dd > 1 ? (unsigned)((0x100000000ULL + dd - 1) / dd) : 0), d(dd) {}
    __device__ __forceinline__ unsigned div(unsigned n) const { return d == 1 ? n : __umulhi(n, m); }
};

// sin and cos of val: Cody-Waite reduction to [-pi, pi] with 2pi = hi + lo, then the SFU.
__device__ __forceinline__ void sincos_fast(float val, float& s, float& c) {
    if (fabsf(val) < 8192.0f) {
        const float k = rintf(val * 0.15915494309189535f);
        float r = fmaf(k, -6.2831854820251465f, val);  // 2pi rounded to fp32
        r = fmaf(k, 1.7484555e-7f, r);                 // fl(2pi) - 2pi
        __sincosf(r, &s, &c);
    } else {
        sincosf(val, &s, &c);
    }
}

constexpr int kPeThreads = 256;

template <typename TI>
__global__ void __launch_bounds__(kPeThreads)
nerf_pe_tile_kernel(const TI* __restrict__ input, __half* __restrict__ output, long long rows,
                    int rows_per_block, int in_dim, int num_freqs, int include_input,
                    const __grid_constant__ FreqTable ft, FastDiv div_in, int vec_out) {
    extern __shared__ __align__(16) __half s_out[];
    const int per_row = in_dim * num_freqs;
    const int off = include_input ? in_dim : 0;
    const int out_dim = 2 * per_row + off;
    const long long r0 = (long long)blockIdx.x * rows_per_block;
    const int nrows = (int)min((long long)rows_per_block, rows - r0);
    const TI* in = input + r0 * in_dim;

    // one (row, input coordinate) pair per step: a single coalesced read of x, then all of its
    // frequencies (two consecutive runs of num_freqs outputs: the sin block and the cos block)
    const unsigned pairs = (unsigned)nrows * in_dim;
    for (unsigned it = threadIdx.x; it < pairs; it += kPeThreads) {
        const unsigned r = div_in.div(it);
        const unsigned d = it - r * in_dim;
        const float x = (float)in[it];
        __half* o = s_out + r * out_dim;
        if (include_input) o[d] = __float2half(x);
        o += off + d * num_freqs;
        for (int k = 0; k < num_freqs; ++k) {
            float s, c;
            sincos_fast(x * ft.f[k], s, c);
            o[k] = __float2half(s);
            o[per_row + k] = __float2half(c);
        }
    }
    __syncthreads();
    const int n_out = nrows * out_dim;
    __half* dst = output + r0 * out_dim;
    if (vec_out) {
        const int nvec = n_out / 8;
        for (int v = threadIdx.x; v < nvec; v += kPeThreads)
            reinterpret_cast<uint4*>(dst)[v] = reinterpret_cast<const uint4*>(s_out)[v];
        for (int e = nvec * 8 + threadIdx.x; e < n_out; e += kPeThreads) dst[e] = s_out[e];
    } else {
        for (int e = threadIdx.x; e < n_out; e += kPeThreads) dst[e] = s_out[e];
    }
}

// The same tile scheme with the number of frequencies known at compile time (loops unrolled, the table
// in registers). DOUBLING: the frequencies are f0 * 2^k exactly (the usual log-spaced bands with integer
// exponents), so only the first angle goes through the sine / cosine units and the others follow from
// sin 2a = 2 sin a cos a, cos 2a = 1 - 2 sin^2 a; the absolute error doubles per step from about 5e-7,
// far below the fp16 rounding of the outputs (5e-4).
template <typename TI, int NF, bool DOUBLING>
__global__ void __launch_bounds__(kPeThreads)
nerf_pe_tile_nf_kernel(const TI* __restrict__ input, __half* __restrict__ output, long long rows,
                       int rows_per_block, int in_dim, int include_input,
                       const __grid_constant__ FreqTable ft, FastDiv div_in, int vec_out) {
    extern __shared__ __align__(16) __half s_out[];
    const int per_row = in_dim * NF;
    const int off = include_input ? in_dim : 0;
    const int out_dim = 2 * per_row + off;
    const long long r0 = (long long)blockIdx.x * rows_per_block;
    const int nrows = (int)min((long long)rows_per_block, rows - r0);
    const TI* in = input + r0 * in_dim;
    float f[NF];
#pragma unroll
    for (int k = 0; k < NF; ++k) f[k] = ft.f[k];
    const unsigned pairs = (unsigned)nrows * in_dim;
    for (unsigned it = threadIdx.x; it < pairs; it += kPeThreads) {
        const unsigned r = div_in.div(it);
        const unsigned d = it - r * in_dim;
        const float x = (float)in[it];
        __half* o = s_out + r * out_dim;
        if (include_input) o[d] = __float2half(x);
        o += off + d * NF;
        if (DOUBLING) {
            float sn, cs;
            sincos_fast(x * f[0], sn, cs);
#pragma unroll
            for (int k = 0; k < NF; ++k) {
                o[k] = __float2half(sn);
                o[per_row + k] = __float2half(cs);
                const float s2 = 2.0f * sn * cs;
                cs = fmaf(-2.0f * sn, sn, 1.0f);
                sn = s2;
            }
        } else {
#pragma unroll
            for (int k = 0; k < NF; ++k) {
                float sn, cs;
                sincos_fast(x * f[k], sn, cs);
                o[k] = __float2half(sn);
                o[per_row + k] = __float2half(cs);
            }
        }
    }
    __syncthreads();
    const int n_out = nrows * out_dim;
    __half* dst = output + r0 * out_dim;
    if (vec_out) {
        const int nvec = n_out / 8;
        for (int v = threadIdx.x; v < nvec; v += kPeThreads)
            __stcs(reinterpret_cast<uint4*>(dst) + v, reinterpret_cast<const uint4*>(s_out)[v]);
        for (int e = nvec * 8 + threadIdx.x; e < n_out; e += kPeThreads) dst[e] = s_out[e];
    } else {
        for (int e = threadIdx.x; e < n_out; e += kPeThreads) dst[e] = s_out[e];
    }
}

constexpr int kPeRowThreads = 128;
// Input width and frequency count both known at compile time: one thread per row. The tile's inputs are
// fetched with coalesced loads into shared memory, each thread then walks its own row with fully unrolled
// loops (no index arithmetic per value), and the tile leaves with 128-bit stores as above.
template <typename TI, int IN_DIM, int NF, bool DOUBLING, bool INCLUDE>
__global__ void __launch_bounds__(kPeRowThreads)
nerf_pe_rows1_kernel(const TI* __restrict__ input, __half* __restrict__ output, long long rows,
                    const __grid_constant__ FreqTable ft, int vec_out) {
    constexpr int PER_ROW = IN_DIM * NF, OFF = INCLUDE ? IN_DIM : 0, OUT_DIM = 2 * PER_ROW + OFF;
    __shared__ __align__(16) __half s_out[kPeRowThreads * OUT_DIM];
    __shared__ TI s_in[kPeRowThreads * IN_DIM];
    const long long r0 = (long long)blockIdx.x * kPeRowThreads;
    const int nrows = (int)min((long long)kPeRowThreads, rows - r0);
    for (int i = threadIdx.x; i < nrows * IN_DIM; i += kPeRowThreads) s_in[i] = input[r0 * IN_DIM + i];
    __syncthreads();
    float f[NF];
#pragma unroll
    for (int k = 0; k < NF; ++k) f[k] = ft.f[k];
    if ((int)threadIdx.x < nrows) {
        __half* o = s_out + threadIdx.x * OUT_DIM;
#pragma unroll
        for (int d = 0; d < IN_DIM; ++d) {
            const float x = (float)s_in[threadIdx.x * IN_DIM + d];
            if (INCLUDE) o[d] = __float2half(x);
            if (DOUBLING) {
                float sn, cs;
                sincos_fast(x * f[0], sn, cs);
#pragma unroll
                for (int k = 0; k < NF; ++k) {
                    o[OFF + d * NF + k] = __float2half(sn);
                    o[OFF + PER_ROW + d * NF + k] = __float2half(cs);
                    const float s2 = 2.0f * sn * cs;
                    cs = fmaf(-2.0f * sn, sn, 1.0f);
                    sn = s2;
                }
            } else {
#pragma unroll
                for (int k = 0; k < NF; ++k) {
                    float sn, cs;
                    sincos_fast(x * f[k], sn, cs);
                    o[OFF + d * NF + k] = __float2half(sn);
                    o[OFF + PER_ROW + d * NF + k] = __float2half(cs);
                }
            }
        }
    }
    __syncthreads();
    const int n_out = nrows * OUT_DIM;
    __half* dst = output + r0 * OUT_DIM;  // kPeRowThreads * OUT_DIM halves per tile: a multiple of 16 bytes
    if (vec_out) {
        const int nvec = n_out / 8;
        for (int v = threadIdx.x; v < nvec; v += kPeRowThreads)
            __stcs(reinterpret_cast<uint4*>(dst) + v, reinterpret_cast<const uint4*>(s_out)[v]);
        for (int e = nvec * 8 + threadIdx.x; e < n_out; e += kPeRowThreads) dst[e] = s_out[e];
    } else {
        for (int e = threadIdx.x; e < n_out; e += kPeRowThreads) dst[e] = s_out[e];
    }
}

// A thread owns two adjacent rows: their 2 * OUT_DIM halves start on a 4-byte boundary whatever the parity
// of OUT_DIM (39 and 117 are odd), so the values leave the registers as packed pairs: half as many
// shared-memory stores as with one row per thread.
template <typename TI, int IN_DIM, int NF, bool DOUBLING, bool INCLUDE>
__global__ void __launch_bounds__(kPeRowThreads)
nerf_pe_rows_kernel(const TI* __restrict__ input, __half* __restrict__ output, long long rows,
                    const __grid_constant__ FreqTable ft, int vec_out) {
    constexpr int PER_ROW = IN_DIM * NF, OFF = INCLUDE ? IN_DIM : 0, OUT_DIM = 2 * PER_ROW + OFF;
    constexpr int kRows = 2 * kPeRowThreads;
    __shared__ __align__(16) __half s_out[kRows * OUT_DIM];
    __shared__ TI s_in[kRows * IN_DIM];
    const long long r0 = (long long)blockIdx.x * kRows;
    const int nrows = (int)min((long long)kRows, rows - r0);
    for (int i = threadIdx.x; i < nrows * IN_DIM; i += kPeRowThreads) s_in[i] = input[r0 * IN_DIM + i];
    __syncthreads();
    float f[NF];
#pragma unroll
    for (int k = 0; k < NF; ++k) f[k] = ft.f[k];
    const int ra = 2 * threadIdx.x;  // rows ra and ra + 1 of the tile
    if (ra < nrows) {
        __half v[2 * OUT_DIM];
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            __half* o = v + rr * OUT_DIM;
            const bool live = ra + rr < nrows;
#pragma unroll
            for (int d = 0; d < IN_DIM; ++d) {
                const float x = live ? (float)s_in[(ra + rr) * IN_DIM + d] : 0.0f;
                if (INCLUDE) o[d] = __float2half(x);
                if (DOUBLING) {
                    float sn, cs;
                    sincos_fast(x * f[0], sn, cs);
#pragma unroll
                    for (int k = 0; k < NF; ++k) {
                        o[OFF + d * NF + k] = __float2half(sn);
                        o[OFF + PER_ROW + d * NF + k] = __float2half(cs);
                        const float s2 = 2.0f * sn * cs;
                        cs = fmaf(-2.0f * sn, sn, 1.0f);
                        sn = s2;
                    }
                } else {
#pragma unroll
                    for (int k = 0; k < NF; ++k) {
                        float sn, cs;
                        sincos_fast(x * f[k], sn, cs);
                        o[OFF + d * NF + k] = __float2half(sn);
                        o[OFF + PER_ROW + d * NF + k] = __float2half(cs);
                    }
                }
            }
        }
        __half2* dst2 = reinterpret_cast<__half2*>(s_out + ra * OUT_DIM);  // ra even: 4-byte aligned
#pragma unroll
        for (int i = 0; i < OUT_DIM; ++i) dst2[i] = __halves2half2(v[2 * i], v[2 * i + 1]);
    }
    __syncthreads();
    const int n_out = nrows * OUT_DIM;
    __half* dst = output + r0 * OUT_DIM;  // kRows * OUT_DIM halves per tile: a multiple of 16 bytes
    if (vec_out) {
        const int nvec = n_out / 8;
        for (int v = threadIdx.x; v < nvec; v += kPeRowThreads)
            __stcs(reinterpret_cast<uint4*>(dst) + v, reinterpret_cast<const uint4*>(s_out)[v]);
        for (int e = nvec * 8 + threadIdx.x; e < n_out; e += kPeRowThreads) dst[e] = s_out[e];
    } else {
        for (int e = threadIdx.x; e < n_out; e += kPeRowThreads) dst[e] = s_out[e];
    }
}

// Rows too wide for a shared-memory tile: one thread per output element.
template <typename TI>
__global__ void __launch_bounds__(256)
nerf_pe_flat_kernel(const TI* __restrict__ input, __half* __restrict__ output, long long total,
                    int in_dim, int num_freqs, int out_dim, int include_input,
                    const __grid_constant__ FreqTable ft) {
    const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= total) return;
    const long long row = e / out_dim;
    int feat = (int)(e - row * out_dim);
    const TI* in_row = input + row * in_dim;
    float o;
    if (include_input && feat < in_dim) {
        o = (float)in_row[feat];
    } else {
        if (include_input) feat -= in_dim;
        const int half_dim = in_dim * num_freqs;
        const bool is_cos = feat >= half_dim;
        const int si = is_cos ? feat - half_dim : feat;
        const int d = si / num_freqs, f = si - d * num_freqs;
        float s, c;
        sincos_fast((float)in_row[d] * ft.f[f], s, c);
        o = is_cos ? c : s;
    }
    output[e] = __float2half(o);
}

template <typename TI>
static int launch_nerf_pe(const TI* input, __half* output, int batch, int seq_len, int in_dim,
                          int num_freqs, float min_exp, float max_exp, int include_input,
                          cudaStream_t st) {
    if (!input || !output || batch < 0 || seq_len < 0 || in_dim <= 0 || num_freqs <= 0)
        return RFK_EINVAL;
    if (num_freqs > 32) return RFK_ETOOBIG;
    const long long out_dim = (long long)in_dim * num_freqs * 2 + (include_input ? in_dim : 0);
    const long long rows = (long long)batch * seq_len;
    if (rows == 0) return RFK_OK;
    FreqTable ft{};
    for (int i = 0; i < num_freqs; ++i) {
        // same expression, in float, as the reference's host loop
        float e = min_exp + (max_exp - min_exp) * i / std::max(num_freqs - 1, 1);
        ft.f[i] = std::pow(2.0f, e);
    }
    if (out_dim <= 3072) {
        // tile rows: a multiple of 8 (so every tile starts 16-byte aligned), ~16 KB of output
        int rpb = (int)std::max(8LL, std::min(256LL, (8192 / out_dim) & ~7LL));
        const size_t smem = (size_t)rpb * out_dim * sizeof(__half);
        const unsigned grid = ceil_div(rows, rpb);
        bool doubling = true;  // exact powers of two apart, and small enough angles for the fast reduction to stay exact
        for (int i = 1; i < num_freqs; ++i) doubling = doubling && ft.f[i] == 2.0f * ft.f[i - 1];
        const int vec = aligned16(output) ? 1 : 0, inc = include_input ? 1 : 0;
#define RFK_PE_NF(NF)                                                                                              \
    do {                                                                                                           \
        if (doubling)                                                                                              \
            nerf_pe_tile_nf_kernel<TI, NF, true><<<grid, kPeThreads, smem, st>>>(input, output, rows, rpb, in_dim, \
                                                                                 inc, ft, FastDiv((unsigned)in_dim), vec); \
        else                                                                                                       \
            nerf_pe_tile_nf_kernel<TI, NF, false><<<grid, kPeThreads, smem, st>>>(input, output, rows, rpb, in_dim, \
                                                                                  inc, ft, FastDiv((unsigned)in_dim), vec); \
    } while (0)
        const unsigned row_grid = ceil_div(rows, 2 * kPeRowThreads), row1_grid = ceil_div(rows, kPeRowThreads);
#define RFK_PE_ROWS1(IN, NF)                                                                                  \
    do {                                                                                                      \
        if (doubling) nerf_pe_rows1_kernel<TI, IN, NF, true, true><<<row1_grid, kPeRowThreads, 0, st>>>(input, output, rows, ft, vec); \
        else nerf_pe_rows1_kernel<TI, IN, NF, false, true><<<row1_grid, kPeRowThreads, 0, st>>>(input, output, rows, ft, vec);         \
    } while (0)
#define RFK_PE_ROWS(IN, NF)                                                                                   \
    do {                                                                                                      \
        if (doubling) nerf_pe_rows_kernel<TI, IN, NF, true, true><<<row_grid, kPeRowThreads, 0, st>>>(input, output, rows, ft, vec); \
        else nerf_pe_rows_kernel<TI, IN, NF, false, true><<<row_grid, kPeRowThreads, 0, st>>>(input, output, rows, ft, vec);         \
    } while (0)
        if (num_freqs == 6 && in_dim == 3 && inc) RFK_PE_ROWS(3, 6);
        else if (num_freqs == 6 && in_dim == 9 && inc) RFK_PE_ROWS1(9, 6);
        else if (num_freqs == 6) RFK_PE_NF(6);
        else if (num_freqs == 4) RFK_PE_NF(4);
        else if (num_freqs == 10) RFK_PE_NF(10);
        else
            nerf_pe_tile_kernel<TI><<<grid, kPeThreads, smem, st>>>(
                input, output, rows, rpb, in_dim, num_freqs, inc, ft, FastDiv((unsigned)in_dim), vec);
#undef RFK_PE_NF
#undef RFK_PE_ROWS
#undef RFK_PE_ROWS1
    } else {
        const long long total = rows * out_dim;
        nerf_pe_flat_kernel<TI><<<ceil_div(total, 256), 256, 0, st>>>(
            input, output, total, in_dim, num_freqs, (int)out_dim, include_input ? 1 : 0, ft);
    }
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
