// Row softmax family: fp32 scores -> fp16 probabilities (strided rows, zero-filled
// pad), the in-place fp32 variants, and the masked / swin-window forms.
//
// Reference semantics (BANANASJIM/renderformer-cuda, src/kernels/softmax.cu):
//   :190-235  softmax_cast_fp16: m = max_j x_j over j<cols, l = sum exp(x_j-m),
//             p_j = half(exp(x_j-m)/l); p_j = 0 for cols <= j < out_stride
//   :259-285  masked form: masked-out entries are excluded from m,l and written as 0;
//             mask row = row % mask_rows
//   :7-44, :55-95, :108-153  in-place fp32 forms: masked-out inputs become -FLT_MAX,
//             then a plain softmax; swin mask row = ((bh / heads) % nW, sq)
//
// Design: the reference reads every row twice and evaluates two exponentials per
// element. Here a row is read from HBM once, held in registers (up to 32 floats per
// thread), reduced with warp shuffles (+ one shared-memory hop across the warps of
// a CTA), and each element costs one ex2. Loads are 2 x 128-bit per 8-element
// chunk, fp16 stores are 128-bit. Three tiers by row length:
//   cols <= 256   : a group of 8/16/32 lanes per row, shuffle-only reductions
//   cols <= 8192  : one CTA (128/256 threads) per row, row in registers
//   cols  > 8192  : one 1024-thread CTA per row, three streaming passes
#include "common.cuh"

namespace rfk {

enum { MASK_NONE = 0, MASK_EXCLUDE = 1, MASK_FILL = 2 };

struct MaskMap {
    int swin;       // 0: mask row = row % mask_rows ; 1: swin window mapping
    int mask_rows;  // swin == 0
    int ws2, heads, nW;  // swin == 1
};

__device__ __forceinline__ long long mask_row_of(const MaskMap& mm, long long row) {
    if (!mm.swin) return row % mm.mask_rows;
    const int sq = (int)(row % mm.ws2);
    const long long bh = row / mm.ws2;
    const int w = (int)((bh / mm.heads) % mm.nW);
    return (long long)w * mm.ws2 + sq;
}

constexpr float kLog2e = 1.4426950408889634f;

template <int MASK> __device__ __forceinline__ float masked_value() {
    return MASK == MASK_FILL ? -FLT_MAX : -INFINITY;
}

__device__ __forceinline__ void store_out(__half* p, float v) { *p = __float2half_rn(v); }
__device__ __forceinline__ void store_out(float* p, float v) { *p = v; }

// ------------------------------------------------------------------ tier M
// One CTA per row; thread t owns chunks t, t+T, ... of 8 consecutive columns.
template <typename TOut, int NCH, int MASK>
__global__ void __launch_bounds__(256)
softmax_row_kernel(const float* in, TOut* out, const uint8_t* __restrict__ mask, MaskMap mm,
                   int cols, long long in_stride, long long out_stride, long long out_pitch,
                   float scale_log2e, int vec_in, int vec_out, int vec_mask) {
    __shared__ float s_max[8];
    __shared__ float s_sum[8];
    const int tid = threadIdx.x;
    const int nthreads = blockDim.x;
    const long long row = blockIdx.x;
    const float* ri = in + row * in_stride;
    TOut* ro = out + row * out_pitch;  // out_stride: columns to fill, out_pitch: row pitch
    const uint8_t* rm = nullptr;
    if (MASK != MASK_NONE) rm = mask + mask_row_of(mm, row) * (long long)cols;

    float v[NCH][8];
    float m = -INFINITY;
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
        const int off = (tid + k * nthreads) * 8;
        if (off + 8 <= cols && vec_in) {
            ldcs_float8(ri + off, v[k]);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[k][i] = (off + i < cols) ? ri[off + i] : -INFINITY;
        }
        if (MASK != MASK_NONE) {
            if (off + 8 <= cols && vec_mask) {
                const uint2 mb = __ldg(reinterpret_cast<const uint2*>(rm + off));
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const unsigned w = (i < 4) ? mb.x : mb.y;
                    if (((w >> (8 * (i & 3))) & 0xffu) == 0) v[k][i] = masked_value<MASK>();
                }
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (off + i < cols && rm[off + i] == 0) v[k][i] = masked_value<MASK>();
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) m = fmaxf(m, v[k][i]);
    }
    const int lane = tid & 31, wid = tid >> 5, nwarps = nthreads >> 5;
    m = warp_max(m);
    if (lane == 0) s_max[wid] = m;
    __syncthreads();
    m = s_max[0];
    for (int w = 1; w < nwarps; ++w) m = fmaxf(m, s_max[w]);
    if (m == -INFINITY) m = 0.0f;  // every entry excluded: all exponentials become 0

    float l = 0.0f;
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float e = fast_exp2((v[k][i] - m) * scale_log2e);
            v[k][i] = e;
            l += e;
        }
    }
    l = warp_sum(l);
    if (lane == 0) s_sum[wid] = l;
    __syncthreads();
    l = s_sum[0];
    for (int w = 1; w < nwarps; ++w) l += s_sum[w];
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;

#pragma unroll
    for (int k = 0; k < NCH; ++k) {
        const int off = (tid + k * nthreads) * 8;
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = v[k][i] * inv;  // columns >= cols hold exp2(-inf) = 0
        if (off + 8 <= out_stride && vec_out) {
            store8(ro + off, o);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (off + i < out_stride) store_out(ro + off + i, o[i]);
        }
    }
}

// ------------------------------------------------------------------ tier S
// G lanes per row, each lane owns chunks of 4 consecutive columns.
template <typename TOut, int G, int NCH, int MASK>
__global__ void __launch_bounds__(256)
softmax_small_kernel(const float* in, TOut* out, const uint8_t* __restrict__ mask, MaskMap mm,
                     long long rows, int cols, long long in_stride, long long out_stride,
                     long long out_pitch, float scale_log2e, int vec_in, int vec_out) {
    const long long gid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / G;
    const int gl = threadIdx.x % G;
    const bool live = gid < rows;
    const long long row = live ? gid : rows - 1;  // idle groups shadow the last row, never store
    const float* ri = in + row * in_stride;
    TOut* ro = out + row * out_pitch;  // out_stride: columns to fill, out_pitch: row pitch
    const uint8_t* rm = nullptr;
    if (MASK != MASK_NONE) rm = mask + mask_row_of(mm, row) * (long long)cols;

    float v[NCH][4];
    float m = -INFINITY;
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
        const int off = (gl + k * G) * 4;
        if (off + 4 <= cols && vec_in) {
            const float4 t = *reinterpret_cast<const float4*>(ri + off);
            v[k][0] = t.x; v[k][1] = t.y; v[k][2] = t.z; v[k][3] = t.w;
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) v[k][i] = (off + i < cols) ? ri[off + i] : -INFINITY;
        }
        if (MASK != MASK_NONE) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (off + i < cols && rm[off + i] == 0) v[k][i] = masked_value<MASK>();
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) m = fmaxf(m, v[k][i]);
    }
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (m == -INFINITY) m = 0.0f;
    float l = 0.0f;
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float e = fast_exp2((v[k][i] - m) * scale_log2e);
            v[k][i] = e;
            l += e;
        }
    }
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    if (!live) return;
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
        const int off = (gl + k * G) * 4;
        float o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) o[i] = v[k][i] * inv;
        if (off + 4 <= out_stride && vec_out) {
            if (sizeof(TOut) == 2) {
                __half2 a = __floats2half2_rn(o[0], o[1]);
                __half2 b = __floats2half2_rn(o[2], o[3]);
                uint2 pk;
                pk.x = *reinterpret_cast<unsigned*>(&a);
                pk.y = *reinterpret_cast<unsigned*>(&b);
                *reinterpret_cast<uint2*>(ro + off) = pk;
            } else {
                *reinterpret_cast<float4*>(ro + off) = make_float4(o[0], o[1], o[2], o[3]);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (off + i < out_stride) store_out(ro + off + i, o[i]);
        }
    }
}

// ------------------------------------------------------------------ tier L
// Rows too long for registers: three coalesced streaming passes (the second and third
// normally hit L2: a 64 K-column row is 256 KB).
template <typename TOut, int MASK>
__global__ void __launch_bounds__(1024)
softmax_long_kernel(const float* in, TOut* out, const uint8_t* __restrict__ mask, MaskMap mm,
                    int cols, long long in_stride, long long out_stride, long long out_pitch,
                    float scale_log2e) {
    __shared__ float s_red[32];
    __shared__ float s_bcast;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5, nwarps = blockDim.x >> 5;
    const long long row = blockIdx.x;
    const float* ri = in + row * in_stride;
    TOut* ro = out + row * out_pitch;  // out_stride: columns to fill, out_pitch: row pitch
    const uint8_t* rm = nullptr;
    if (MASK != MASK_NONE) rm = mask + mask_row_of(mm, row) * (long long)cols;
    auto value = [&](int j) -> float {
        float x = ri[j];
        if (MASK != MASK_NONE && rm[j] == 0) x = masked_value<MASK>();
        return x;
    };
    float m = -INFINITY;
    for (int j = tid; j < cols; j += blockDim.x) m = fmaxf(m, value(j));
    m = warp_max(m);
    if (lane == 0) s_red[wid] = m;
    __syncthreads();
    if (wid == 0) {
        float t = lane < nwarps ? s_red[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) s_bcast = t;
    }
    __syncthreads();
    m = s_bcast;
    if (m == -INFINITY) m = 0.0f;
    float l = 0.0f;
    for (int j = tid; j < cols; j += blockDim.x) l += fast_exp2((value(j) - m) * scale_log2e);
    l = warp_sum(l);
    __syncthreads();  // s_red / s_bcast reuse
    if (lane == 0) s_red[wid] = l;
    __syncthreads();
    if (wid == 0) {
        float t = lane < nwarps ? s_red[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) s_bcast = t;
    }
    __syncthreads();
    l = s_bcast;
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    for (int j = tid; j < out_stride; j += blockDim.x) {
        float p = 0.0f;
        if (j < cols) p = fast_exp2((value(j) - m) * scale_log2e) * inv;
        store_out(ro + j, p);
    }
}

template <typename TOut, int MASK>
static int launch_softmax(const float* in, TOut* out, const uint8_t* mask, MaskMap mm,
                          long long rows, int cols, long long in_stride, long long out_stride,
                          float scale, cudaStream_t st, long long out_pitch = 0,
                          bool registers_only = false) {
    if (out_pitch == 0) out_pitch = out_stride;
    if (!in || !out || rows < 0 || cols <= 0 || in_stride < cols || out_stride < cols ||
        (out_pitch != 0 && out_pitch < out_stride))
        return RFK_EINVAL;
    if (MASK != MASK_NONE && !mask) return RFK_EINVAL;
    if (!(scale > 0.0f)) return RFK_EINVAL;
    if (rows == 0) return RFK_OK;
    if (rows > 0x7fffffffLL) return RFK_EUNSUPPORTED;
    const float sl2 = scale * kLog2e;
    const long long span = out_stride > cols ? out_stride : cols;  // columns a row must cover
    constexpr int osz = (int)sizeof(TOut);

    if (span <= 256) {
        const int vec_in = aligned16(in) && (in_stride % 4 == 0);
        const int vec_out = ((reinterpret_cast<uintptr_t>(out) % (4 * osz)) == 0) &&
                            (out_pitch % 4 == 0);
#define RFK_SM_SMALL(G, N)                                                                    \
    softmax_small_kernel<TOut, G, N, MASK><<<ceil_div(rows * G, 256), 256, 0, st>>>(          \
        in, out, mask, mm, rows, cols, in_stride, out_stride, out_pitch, sl2, vec_in, vec_out)
        if (span <= 32) RFK_SM_SMALL(8, 1);
        else if (span <= 64) RFK_SM_SMALL(16, 1);
        else if (span <= 128) RFK_SM_SMALL(32, 1);
        else RFK_SM_SMALL(32, 2);
#undef RFK_SM_SMALL
        return launch_status();
    }
    if (span <= 8192) {
        const int vec_in = aligned16(in) && (in_stride % 4 == 0);
        const int vec_out = aligned16(out) && ((out_pitch * osz) % 16 == 0);
        const int vec_mask = MASK != MASK_NONE && aligned8(mask) && (cols % 8 == 0);
        const int chunks = (int)((span + 7) / 8);
        const int threads = chunks <= 128 ? 128 : 256;
        const int nch = (chunks + threads - 1) / threads;
#define RFK_SM_ROW(N)                                                                         \
    softmax_row_kernel<TOut, N, MASK><<<(unsigned)rows, threads, 0, st>>>(                    \
        in, out, mask, mm, cols, in_stride, out_stride, out_pitch, sl2, vec_in, vec_out, vec_mask)
        switch (nch) {
            case 1: RFK_SM_ROW(1); break;
            case 2: RFK_SM_ROW(2); break;
            case 3: RFK_SM_ROW(3); break;
            default: RFK_SM_ROW(4); break;
        }
#undef RFK_SM_ROW
        return launch_status();
    }
    if (registers_only) return RFK_EUNSUPPORTED;  // the streaming tier re-reads its input
    softmax_long_kernel<TOut, MASK><<<(unsigned)rows, 1024, 0, st>>>(
        in, out, mask, mm, cols, in_stride, out_stride, out_pitch, sl2);
    return launch_status();
}

}  // namespace rfk

using namespace rfk;

extern "C" int rfk_softmax_inplace(float* data, int rows, int cols, rfk_stream_t stream) {
    return launch_softmax<float, MASK_NONE>(data, data, nullptr, MaskMap{}, rows, cols, cols, cols,
                                            1.0f, as_stream(stream));
}

extern "C" int rfk_masked_softmax_inplace(float* data, const uint8_t* mask, int rows, int cols,
                                          int mask_rows, rfk_stream_t stream) {
    if (mask_rows <= 0) return RFK_EINVAL;
    MaskMap mm{0, mask_rows, 0, 0, 0};
    return launch_softmax<float, MASK_FILL>(data, data, mask, mm, rows, cols, cols, cols, 1.0f,
                                            as_stream(stream));
}

extern "C" int rfk_swin_masked_softmax_inplace(float* data, const uint8_t* mask, int BnW,
                                               int num_heads, int ws2, int nW,
                                               rfk_stream_t stream) {
    if (BnW < 0 || num_heads <= 0 || ws2 <= 0 || nW <= 0) return RFK_EINVAL;
    MaskMap mm{1, 0, ws2, num_heads, nW};
    return launch_softmax<float, MASK_FILL>(data, data, mask, mm,
                                            (long long)BnW * num_heads * ws2, ws2, ws2, ws2, 1.0f,
                                            as_stream(stream));
}

extern "C" int rfk_softmax_cast_fp16(const float* in, rfk_half* out, int rows, int cols,
                                     int in_stride, int out_stride, rfk_stream_t stream) {
    return launch_softmax<__half, MASK_NONE>(in, (__half*)out, nullptr, MaskMap{}, rows, cols,
                                             in_stride, out_stride, 1.0f, as_stream(stream));
}

extern "C" int rfk_softmax_cast_fp16_scaled(const float* in, rfk_half* out, int rows, int cols,
                                            int in_stride, int out_stride, float scale,
                                            rfk_stream_t stream) {
    return launch_softmax<__half, MASK_NONE>(in, (__half*)out, nullptr, MaskMap{}, rows, cols,
                                             in_stride, out_stride, scale, as_stream(stream));
}

extern "C" int rfk_softmax_cast_fp16_masked(const float* in, rfk_half* out, const uint8_t* mask,
                                            int rows, int cols, int in_stride, int out_stride,
                                            int mask_rows, rfk_stream_t stream) {
    if (mask_rows <= 0) return RFK_EINVAL;
    MaskMap mm{0, mask_rows, 0, 0, 0};
    return launch_softmax<__half, MASK_EXCLUDE>(in, (__half*)out, mask, mm, rows, cols, in_stride,
                                                out_stride, 1.0f, as_stream(stream));
}

extern "C" int rfk_swin_softmax_cast_fp16(const float* in, rfk_half* out, const uint8_t* mask,
                                          int BnW, int num_heads, int ws2, int nW,
                                          rfk_stream_t stream) {
    if (BnW < 0 || num_heads <= 0 || ws2 <= 0 || nW <= 0) return RFK_EINVAL;
    const long long rows = (long long)BnW * num_heads * ws2;
    if (!mask)
        return launch_softmax<__half, MASK_NONE>(in, (__half*)out, nullptr, MaskMap{}, rows, ws2,
                                                 ws2, ws2, 1.0f, as_stream(stream));
    MaskMap mm{1, 0, ws2, num_heads, nW};
    // the unfused pair fills masked scores with -FLT_MAX before the softmax, keep that rule
    return launch_softmax<__half, MASK_FILL>(in, (__half*)out, mask, mm, rows, ws2, ws2, ws2, 1.0f,
                                             as_stream(stream));
}

extern "C" int rfk_softmax_probs_inplace(float* scores, int rows, int n_valid, int stride,
                                         float scale, rfk_stream_t stream) {
    if (stride < n_valid) return RFK_EINVAL;
    // fp16 row r lives in the first half of fp32 row r: pitch = 2*stride halves. Safe because
    // the register tiers read a whole row before they store any of it.
    return launch_softmax<__half, MASK_NONE>(scores, reinterpret_cast<__half*>(scores), nullptr,
                                             MaskMap{}, rows, n_valid, stride, stride, scale,
                                             as_stream(stream), 2LL * stride, true);
}

extern "C" int rfk_swin_softmax_probs_inplace(float* scores, const uint8_t* mask, int BnW,
                                              int num_heads, int ws2, int nW, rfk_stream_t stream) {
    if (BnW < 0 || num_heads <= 0 || ws2 <= 0 || nW <= 0) return RFK_EINVAL;
    const long long rows = (long long)BnW * num_heads * ws2;
    __half* out = reinterpret_cast<__half*>(scores);
    if (!mask)
        return launch_softmax<__half, MASK_NONE>(scores, out, nullptr, MaskMap{}, rows, ws2, ws2, ws2,
                                                 1.0f, as_stream(stream), 2LL * ws2, true);
    MaskMap mm{1, 0, ws2, num_heads, nW};
    return launch_softmax<__half, MASK_FILL>(scores, out, mask, mm, rows, ws2, ws2, ws2, 1.0f,
                                             as_stream(stream), 2LL * ws2, true);
}
