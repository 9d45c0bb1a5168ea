// Element-wise plumbing and layout shuffles that sit between the GEMMs: residual adds,
// dtype casts, broadcast add, head transposes, swin window gather/scatter, patchify.
//
// Reference semantics (BANANASJIM/renderformer-cuda):
//   src/layers/transformer.cu:9-61      residual_add{,_f32,_mixed}, cast_fp32_to_fp16, cast_fp16_to_fp32
//   src/layers/attention.cu:17-48       transpose_bshd_to_bhsd, transpose_bhsd_to_bsd
//   src/layers/attention.cu:377-472     window_partition, window_reverse, cyclic_shift
//   src/pipeline/render_session.cu:44-59  k_broadcast_add_s, k_patchify_s
//
// Design: the reference moves one 2-byte element per thread. All of these are pure
// copies/adds, so every kernel here moves 8 elements (128 bits for fp16) per thread and
// falls back to a scalar kernel only when the innermost extent is not a multiple of 8
// or a pointer is not 16-byte aligned.
#include "common.cuh"

namespace rfk {

// ----------------------------------------------------------- flat element-wise

enum { EW_ADD_H = 0, EW_ADD_F = 1, EW_ADD_MIXED = 2, EW_CAST_F2H = 3, EW_CAST_H2F = 4 };

template <int OP> struct EwTypes;
template <> struct EwTypes<EW_ADD_H> { using A = __half; using B = __half; };
template <> struct EwTypes<EW_ADD_F> { using A = float; using B = float; };
template <> struct EwTypes<EW_ADD_MIXED> { using A = float; using B = __half; };
template <> struct EwTypes<EW_CAST_F2H> { using A = __half; using B = float; };
template <> struct EwTypes<EW_CAST_H2F> { using A = float; using B = __half; };

// a is the in/out (or out) array, b the second operand (or the cast source)
template <int OP>
__global__ void __launch_bounds__(256)
ew_kernel(typename EwTypes<OP>::A* a, const typename EwTypes<OP>::B* __restrict__ b, long long n,
          int vec) {
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long i0 = t * 8;
    if (i0 >= n) return;
    if (vec && i0 + 8 <= n) {
        float fb[8], fa[8];
        load8(b + i0, fb);
        if (OP == EW_ADD_H || OP == EW_ADD_F || OP == EW_ADD_MIXED) {
            load8(a + i0, fa);
#pragma unroll
            for (int i = 0; i < 8; ++i) fa[i] += fb[i];
            store8(a + i0, fa);
        } else {
            store8(a + i0, fb);
        }
    } else {
        for (long long i = i0; i < n && i < i0 + 8; ++i) {
            if (OP == EW_ADD_H || OP == EW_ADD_F || OP == EW_ADD_MIXED)
                a[i] = (typename EwTypes<OP>::A)((float)a[i] + (float)b[i]);
            else
                a[i] = (typename EwTypes<OP>::A)((float)b[i]);
        }
    }
}

template <int OP>
static int launch_ew(typename EwTypes<OP>::A* a, const typename EwTypes<OP>::B* b, long long n,
                     cudaStream_t st) {
    if (!a || !b || n < 0) return RFK_EINVAL;
    if (n == 0) return RFK_OK;
    const int vec = aligned16(a) && aligned16(b);
    ew_kernel<OP><<<ceil_div((n + 7) / 8, 256), 256, 0, st>>>(a, b, n, vec);
    return launch_status();
}

__global__ void __launch_bounds__(256)
broadcast_add_kernel(__half* out, const __half* __restrict__ bc, long long n, int dim, int vec) {
    const long long i0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (i0 >= n) return;
    if (vec && i0 + 8 <= n) {
        float a[8], b[8];
        load8(out + i0, a);
        unpack8(ldg_half8(bc + (i0 % dim)), b);
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] += b[i];
        store8(out + i0, a);
    } else {
        for (long long i = i0; i < n && i < i0 + 8; ++i)
            out[i] = __float2half(__half2float(out[i]) + __half2float(bc[i % dim]));
    }
}

// ----------------------------------------------------------- row-chunk copies
// All remaining kernels copy rows of `inner` contiguous fp16 values between two index
// spaces. A thread moves one 8-element chunk; MAP turns a destination chunk index into
// source and destination element offsets.

struct TransposeMap {  // [B,S,H,D] -> [B,H,S,D]; forward == 0 inverts it ([B,H,S,D] -> [B,S,H,D])
    int S, H, D, forward;
    __device__ __forceinline__ void operator()(long long chunk, int cpr, size_t& src, size_t& dst) const {
        const int j = (int)(chunk % cpr);
        long long t = chunk / cpr;
        const int h = (int)(t % H); t /= H;
        const int s = (int)(t % S);
        const long long b = t / S;
        const size_t bshd = (((size_t)b * S + s) * H + h) * D + (size_t)j * 8;
        const size_t bhsd = (((size_t)b * H + h) * S + s) * D + (size_t)j * 8;
        src = forward ? bshd : bhsd;
        dst = forward ? bhsd : bshd;
    }
};

struct WindowMap {  // token (b,h,w) <-> window row; gather == 1: windows <- x
    int H, W, C, ws, shift, gather;
    __device__ __forceinline__ void operator()(long long chunk, int cpr, size_t& src, size_t& dst) const {
        const int j = (int)(chunk % cpr);
        long long t = chunk / cpr;          // window-order token index
        const int ws2 = ws * ws, nWw = W / ws, nW = (H / ws) * nWw;
        const int local = (int)(t % ws2); t /= ws2;
        const int win = (int)(t % nW);
        const long long b = t / nW;
        const int hs = (win / nWw) * ws + local / ws;  // position in the shifted image
        const int wsft = (win % nWw) * ws + local % ws;
        // the reference shifts by -shift: shifted[hs][ws] = x[(hs-shift) mod H][(ws-shift) mod W]
        const int h = (hs - shift + H) % H, w = (wsft - shift + W) % W;
        const size_t xo = (((size_t)b * H + h) * W + w) * C + (size_t)j * 8;
        const size_t wo = (((size_t)b * nW + win) * ws2 + local) * C + (size_t)j * 8;
        src = gather ? xo : wo;
        dst = gather ? wo : xo;
    }
};

struct PatchMap {  // [H,W,C] -> [pH*pW, C*ps*ps], element granularity (inner extent 1)
    int H, W, C, ps;
    __device__ __forceinline__ void operator()(long long idx, size_t& src, size_t& dst) const {
        const int pW = W / ps;
        const int p2 = (int)(idx % ps); long long r = idx / ps;
        const int p1 = (int)(r % ps); r /= ps;
        const int c = (int)(r % C);
        const long long patch = r / C;
        const int h1 = (int)(patch / pW), w1 = (int)(patch % pW);
        dst = (size_t)idx;
        src = ((size_t)(h1 * ps + p1) * W + (size_t)w1 * ps + p2) * C + c;
    }
};

template <typename MAP, bool ACCUM>
__global__ void __launch_bounds__(256)
chunk_copy_kernel(const __half* __restrict__ in, __half* out, long long nchunks, int cpr,
                  MAP map) {
    const long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= nchunks) return;
    size_t src, dst;
    map(c, cpr, src, dst);
    if (ACCUM) {
        float a[8], b[8];
        load8(out + dst, a);
        unpack8(ldcs_half8(in + src), b);
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] += b[i];
        store8(out + dst, a);
    } else {
        st_half8(out + dst, ldcs_half8(in + src));
    }
}

// scalar twin: `inner` arbitrary, one element per thread
template <typename MAP, bool ACCUM>
__global__ void __launch_bounds__(256)
elem_copy_kernel(const __half* __restrict__ in, __half* out, long long n, int inner, MAP map) {
    const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n) return;
    // reuse the chunk maps with "chunks" of one row and add the in-row offset
    size_t src, dst;
    map(e / inner, 1, src, dst);
    const int d = (int)(e % inner);
    if (ACCUM)
        out[dst + d] = __float2half(__half2float(out[dst + d]) + __half2float(in[src + d]));
    else
        out[dst + d] = in[src + d];
}

__global__ void __launch_bounds__(256)
patchify_kernel(const __half* __restrict__ in, __half* __restrict__ out, long long n, PatchMap map) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    size_t src, dst;
    map(i, src, dst);
    out[dst] = in[src];
}

template <typename MAP, bool ACCUM>
static int launch_rows(const __half* in, __half* out, long long n_rows, int inner, MAP map,
                       cudaStream_t st) {
    if (n_rows == 0) return RFK_OK;
    if (inner % 8 == 0 && aligned16(in) && aligned16(out)) {
        const int cpr = inner / 8;
        const long long nchunks = n_rows * cpr;
        chunk_copy_kernel<MAP, ACCUM><<<ceil_div(nchunks, 256), 256, 0, st>>>(in, out, nchunks, cpr,
                                                                              map);
    } else {
        const long long n = n_rows * inner;
        elem_copy_kernel<MAP, ACCUM><<<ceil_div(n, 256), 256, 0, st>>>(in, out, n, inner, map);
    }
    return launch_status();
}

}  // namespace rfk

using namespace rfk;

extern "C" int rfk_residual_add(rfk_half* y, const rfk_half* r, long long n, rfk_stream_t s) {
    return launch_ew<EW_ADD_H>((__half*)y, (const __half*)r, n, as_stream(s));
}
extern "C" int rfk_residual_add_f32(float* y, const float* r, long long n, rfk_stream_t s) {
    return launch_ew<EW_ADD_F>(y, r, n, as_stream(s));
}
extern "C" int rfk_residual_add_mixed(float* y, const rfk_half* r, long long n, rfk_stream_t s) {
    return launch_ew<EW_ADD_MIXED>(y, (const __half*)r, n, as_stream(s));
}
extern "C" int rfk_cast_fp32_to_fp16(const float* in, rfk_half* out, long long n, rfk_stream_t s) {
    return launch_ew<EW_CAST_F2H>((__half*)out, in, n, as_stream(s));
}
extern "C" int rfk_cast_fp16_to_fp32(const rfk_half* in, float* out, long long n, rfk_stream_t s) {
    return launch_ew<EW_CAST_H2F>(out, (const __half*)in, n, as_stream(s));
}

extern "C" int rfk_broadcast_add(rfk_half* out, const rfk_half* bc, long long n, int dim,
                                 rfk_stream_t stream) {
    if (!out || !bc || n < 0 || dim <= 0) return RFK_EINVAL;
    if (n == 0) return RFK_OK;
    const int vec = aligned16(out) && aligned16(bc) && dim % 8 == 0;
    broadcast_add_kernel<<<ceil_div((n + 7) / 8, 256), 256, 0, as_stream(stream)>>>(
        (__half*)out, (const __half*)bc, n, dim, vec);
    return launch_status();
}

extern "C" int rfk_transpose_bshd_to_bhsd(const rfk_half* in, rfk_half* out, int batch,
                                          int seq_len, int num_heads, int head_dim,
                                          rfk_stream_t stream) {
    if (!in || !out || batch < 0 || seq_len < 0 || num_heads <= 0 || head_dim <= 0)
        return RFK_EINVAL;
    TransposeMap m{seq_len, num_heads, head_dim, 1};
    return launch_rows<TransposeMap, false>((const __half*)in, (__half*)out,
                                            (long long)batch * seq_len * num_heads, head_dim, m,
                                            as_stream(stream));
}

extern "C" int rfk_transpose_bhsd_to_bsd(const rfk_half* in, rfk_half* out, int batch,
                                         int num_heads, int seq_len, int head_dim,
                                         rfk_stream_t stream) {
    if (!in || !out || batch < 0 || seq_len < 0 || num_heads <= 0 || head_dim <= 0)
        return RFK_EINVAL;
    TransposeMap m{seq_len, num_heads, head_dim, 0};
    return launch_rows<TransposeMap, false>((const __half*)in, (__half*)out,
                                            (long long)batch * seq_len * num_heads, head_dim, m,
                                            as_stream(stream));
}

static int check_window_args(const void* a, const void* b, int B, int H, int W, int C, int ws,
                             int shift) {
    if (!a || !b || B < 0 || H <= 0 || W <= 0 || C <= 0 || ws <= 0) return RFK_EINVAL;
    if (H % ws || W % ws || shift < 0 || shift >= ws) return RFK_EINVAL;
    return RFK_OK;
}

extern "C" int rfk_window_gather(const rfk_half* x, rfk_half* windows, int B, int H, int W, int C,
                                 int ws, int shift, rfk_stream_t stream) {
    int rc = check_window_args(x, windows, B, H, W, C, ws, shift);
    if (rc) return rc;
    WindowMap m{H, W, C, ws, shift, 1};
    return launch_rows<WindowMap, false>((const __half*)x, (__half*)windows, (long long)B * H * W,
                                         C, m, as_stream(stream));
}

extern "C" int rfk_window_scatter(const rfk_half* windows, rfk_half* x, int B, int H, int W, int C,
                                  int ws, int shift, int residual_into, rfk_stream_t stream) {
    int rc = check_window_args(windows, x, B, H, W, C, ws, shift);
    if (rc) return rc;
    WindowMap m{H, W, C, ws, shift, 0};
    if (residual_into)
        return launch_rows<WindowMap, true>((const __half*)windows, (__half*)x,
                                            (long long)B * H * W, C, m, as_stream(stream));
    return launch_rows<WindowMap, false>((const __half*)windows, (__half*)x, (long long)B * H * W,
                                         C, m, as_stream(stream));
}

extern "C" int rfk_patchify(const rfk_half* in, rfk_half* out, int H, int W, int C, int ps,
                            rfk_stream_t stream) {
    if (!in || !out || H <= 0 || W <= 0 || C <= 0 || ps <= 0 || H % ps || W % ps)
        return RFK_EINVAL;
    PatchMap m{H, W, C, ps};
    const long long n = (long long)H * W * C;
    patchify_kernel<<<ceil_div(n, 256), 256, 0, as_stream(stream)>>>((const __half*)in,
                                                                     (__half*)out, n, m);
    return launch_status();
}
