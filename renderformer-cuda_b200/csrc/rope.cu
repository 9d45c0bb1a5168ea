// Triangle-vertex RoPE: table generation, rotate-half application (in place and out of
// place), and the fused projection epilogue (QK-RMSNorm + BSHD->BHSD transpose + RoPE).
//
// Reference semantics (BANANASJIM/renderformer-cuda, src/kernels/rope.cu):
//   :23-43  tables: l = d mod (hd/2); theta = l < 9*nf ? pos[l / nf] * freq[l mod nf] : 0;
//           cos_d = half(cosf(theta)), sin_d = half(sinf(theta))
//   :75-88  apply: out_d = x_d*c_d + (x_rot*sign)*s_d, rot = d +- hd/2, sign = -1 for d < hd/2
// and src/layers/attention.cu:73-85,184-210,341-361 for the sequence the fused epilogue
// replaces.
//
// Design: the reference assigns one thread per element; both partners of a rotation
// pair are read by two different threads and written in place without ordering. Here
// one thread owns the 8-wide chunk d..d+7 of the first half of a head and the matching
// chunk of the second half, so each element is read once (two 128-bit loads), written
// once, and the in-place update is race-free by construction. The cos/sin chunk is
// loaded once per thread and reused across the heads the thread walks.
#include "common.cuh"

namespace rfk {

// ---------------------------------------------------------------- tables

// thread -> (token, chunk j of the first half); writes both halves (they are equal)
__global__ void __launch_bounds__(256)
rope_table_vec_kernel(const __half* __restrict__ pos, const float* __restrict__ freqs,
                      __half* __restrict__ out_cos, __half* __restrict__ out_sin,
                      long long tokens, int num_freqs, int head_dim) {
    const int cpt = head_dim / 16;  // chunks per token (first half)
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= tokens * cpt) return;
    const long long tok = idx / cpt;
    const int j = (int)(idx % cpt);
    const int freq_dim = 9 * num_freqs;
    float c[8], s[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int l = j * 8 + i;
        float val = 0.0f;
        if (l < freq_dim) {
            const float p = __half2float(pos[tok * 9 + l / num_freqs]);
            val = p * __ldg(freqs + l % num_freqs);
        }
        c[i] = cosf(val);
        s[i] = sinf(val);
    }
    const size_t o = (size_t)tok * head_dim + j * 8;
    const Half8 hc = pack8(c), hs = pack8(s);
    st_half8(out_cos + o, hc);
    st_half8(out_cos + o + head_dim / 2, hc);
    st_half8(out_sin + o, hs);
    st_half8(out_sin + o + head_dim / 2, hs);
}

__global__ void __launch_bounds__(256)
rope_table_generic_kernel(const __half* __restrict__ pos, const float* __restrict__ freqs,
                          __half* __restrict__ out_cos, __half* __restrict__ out_sin,
                          long long tokens, int num_freqs, int head_dim) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= tokens * head_dim) return;
    const long long tok = idx / head_dim;
    const int d = (int)(idx % head_dim);
    const int l = d % (head_dim / 2);
    float val = 0.0f;
    if (l < 9 * num_freqs)
        val = __half2float(pos[tok * 9 + l / num_freqs]) * freqs[l % num_freqs];
    out_cos[idx] = __float2half(cosf(val));
    out_sin[idx] = __float2half(sinf(val));
}

// ---------------------------------------------------------------- apply

// rotate one (lo, hi) chunk pair; c/s are the table chunks at the lo and hi positions
__device__ __forceinline__ void rotate8(float (&lo)[8], float (&hi)[8], const float (&cl)[8],
                                        const float (&sl)[8], const float (&ch)[8],
                                        const float (&sh)[8]) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float x_lo = lo[i], x_hi = hi[i];
        const float rot_lo = x_hi * -1.0f;  // partner of a first-half element, sign -1
        const float rot_hi = x_lo * 1.0f;
        lo[i] = x_lo * cl[i] + rot_lo * sl[i];
        hi[i] = x_hi * ch[i] + rot_hi * sh[i];
    }
}

// T = __half or float data. NT tensors (1 or 2) share the tables. Each thread walks HP heads.
// src/dst are [B,H,src_rows,D] / [B,H,dst_rows,D]; rows s >= seq_len (dst only) are copied.
template <typename T, int NT, int HP>
__global__ void __launch_bounds__(128)
rope_apply_kernel(const T* src0, T* dst0, const T* src1, T* dst1,
                  const __half* __restrict__ cos_vals, const __half* __restrict__ sin_vals,
                  int batch, int num_heads, int seq_len, int rows_total, int head_dim,
                  long long src_rows, long long dst_rows, long long src_bstride, long long dst_bstride,
                  long long tab_bstride, const float* __restrict__ col_scale, long long scale_bstride) {
    pdl_wait();
    pdl_trigger();
    const int cpt = head_dim / 16;
    const int hgroups = num_heads / HP;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total = (long long)batch * hgroups * rows_total * cpt;
    if (idx >= total) return;
    const int j = (int)(idx % cpt);
    long long t = idx / cpt;
    const int s = (int)(t % rows_total);
    t /= rows_total;
    const int hg = (int)(t % hgroups);
    const int b = (int)(t / hgroups);
    const int half_d = head_dim / 2;
    const bool rotate = s < seq_len;

    float cl[8], sl[8], ch[8], sh[8];
    if (rotate) {
        const size_t to = (size_t)b * tab_bstride + (size_t)s * head_dim + j * 8;
        unpack8(ldg_half8(cos_vals + to), cl);
        unpack8(ldg_half8(sin_vals + to), sl);
        unpack8(ldg_half8(cos_vals + to + half_d), ch);
        unpack8(ldg_half8(sin_vals + to + half_d), sh);
    }
#pragma unroll
    for (int hh = 0; hh < HP; ++hh) {
        const int h = hg * HP + hh;
        const size_t so = (size_t)b * src_bstride + ((size_t)h * src_rows + s) * head_dim + j * 8;
        const size_t dofs = (size_t)b * dst_bstride + ((size_t)h * dst_rows + s) * head_dim + j * 8;
#pragma unroll
        for (int tsel = 0; tsel < NT; ++tsel) {
            const T* sp = tsel == 0 ? src0 : src1;
            T* dp = tsel == 0 ? dst0 : dst1;
            float lo[8], hi[8];
            load8(sp + so, lo);
            load8(sp + so + half_d, hi);
            if (rotate) rotate8(lo, hi, cl, sl, ch, sh);
            if (col_scale) {  // per-(head, element) factor applied to the rotated value before the one rounding
                float g0[8], g1[8];
                const float* gs = col_scale + (size_t)b * scale_bstride + (size_t)h * head_dim + j * 8;
                ldg_float8(gs, g0);
                ldg_float8(gs + half_d, g1);
#pragma unroll
                for (int i = 0; i < 8; ++i) { lo[i] *= g0[i]; hi[i] *= g1[i]; }
            }
            store8(dp + dofs, lo);
            store8(dp + dofs + half_d, hi);
        }
    }
}

// head_dim not a multiple of 16 (but even): one thread per rotation pair, scalar accesses.
template <typename T, int NT>
__global__ void __launch_bounds__(256)
rope_apply_generic_kernel(const T* src0, T* dst0, const T* src1, T* dst1,
                          const __half* __restrict__ cos_vals,
                          const __half* __restrict__ sin_vals, int batch, int num_heads,
                          int seq_len, int rows_total, int head_dim, long long src_rows,
                          long long dst_rows, long long src_bstride, long long dst_bstride,
                          long long tab_bstride) {
    const int half_d = head_dim / 2;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total = (long long)batch * num_heads * rows_total * half_d;
    if (idx >= total) return;
    const int d = (int)(idx % half_d);
    long long t = idx / half_d;
    const int s = (int)(t % rows_total);
    t /= rows_total;
    const int h = (int)(t % num_heads);
    const int b = (int)(t / num_heads);
    const size_t so = (size_t)b * src_bstride + ((size_t)h * src_rows + s) * head_dim + d;
    const size_t dofs = (size_t)b * dst_bstride + ((size_t)h * dst_rows + s) * head_dim + d;
#pragma unroll
    for (int tsel = 0; tsel < NT; ++tsel) {
        const T* sp = tsel == 0 ? src0 : src1;
        T* dp = tsel == 0 ? dst0 : dst1;
        float x_lo = (float)sp[so], x_hi = (float)sp[so + half_d];
        float o_lo = x_lo, o_hi = x_hi;
        if (s < seq_len) {
            const size_t to = (size_t)b * tab_bstride + (size_t)s * head_dim + d;
            const float c_lo = __half2float(cos_vals[to]), s_lo = __half2float(sin_vals[to]);
            const float c_hi = __half2float(cos_vals[to + half_d]);
            const float s_hi = __half2float(sin_vals[to + half_d]);
            o_lo = x_lo * c_lo + (x_hi * -1.0f) * s_lo;
            o_hi = x_hi * c_hi + (x_lo * 1.0f) * s_hi;
        }
        dp[dofs] = (T)o_lo;
        dp[dofs + half_d] = (T)o_hi;
    }
}

template <typename T, int NT>
static int launch_rope(const T* src0, T* dst0, const T* src1, T* dst1, const __half* cos_vals,
                       const __half* sin_vals, int batch, int num_heads, int seq_len,
                       int rows_total, int head_dim, long long src_rows, long long dst_rows,
                       cudaStream_t st, long long src_bstride = -1, long long dst_bstride = -1,
                       long long tab_bstride = -1, const float* col_scale = nullptr, long long scale_bstride = 0) {
    // batch strides in elements; by default the tensors and the tables are densely packed
    if (src_bstride < 0) src_bstride = (long long)num_heads * src_rows * head_dim;
    if (dst_bstride < 0) dst_bstride = (long long)num_heads * dst_rows * head_dim;
    if (tab_bstride < 0) tab_bstride = (long long)seq_len * head_dim;
    if (!src0 || !dst0 || (NT == 2 && (!src1 || !dst1)) || !cos_vals || !sin_vals)
        return RFK_EINVAL;
    if (batch < 0 || num_heads <= 0 || seq_len < 0 || head_dim <= 0 || (head_dim & 1))
        return RFK_EINVAL;
    if (rows_total < seq_len || src_rows < rows_total || dst_rows < rows_total) return RFK_EINVAL;
    if (batch == 0 || rows_total == 0) return RFK_OK;
    const bool vec = head_dim % 16 == 0 && aligned16(src0) && aligned16(dst0) &&
                     (NT == 1 || (aligned16(src1) && aligned16(dst1))) && aligned16(cos_vals) &&
                     aligned16(sin_vals) && src_bstride % 8 == 0 && dst_bstride % 8 == 0 &&
                     tab_bstride % 8 == 0 && (!col_scale || (aligned16(col_scale) && scale_bstride % 4 == 0));
    if (col_scale && !vec) return RFK_EUNSUPPORTED;  // the scaled form exists in the vector kernel only
    if (vec) {
        const int cpt = head_dim / 16;
        // One head per thread unless the problem is large: at the benchmark size (47 MB) the
        // kernel lasts ~10 us and is bound by how evenly short-lived CTAs keep loads in
        // flight (ncu: 24 % DRAM utilisation with 2 heads per thread and 1.6 waves of
        // 705 CTAs); walking several heads per thread only pays once there are at least two
        // full waves of threads left (the cos/sin re-reads it saves come from L2 anyway).
        const long long per_head = (long long)batch * rows_total * cpt;
        const long long two_waves = 2LL * kNumSMs * 2048;
        const int hp = (num_heads % 4 == 0 && per_head * (num_heads / 4) >= two_waves) ? 4
                     : (num_heads % 2 == 0 && per_head * (num_heads / 2) >= two_waves) ? 2 : 1;
        const long long total = (long long)batch * (num_heads / hp) * rows_total * cpt;
        const unsigned grid = ceil_div(total, 128);
#define RFK_ROPE(HPV)                                                                         \
    launch_pdl(rope_apply_kernel<T, NT, HPV>, dim3(grid), dim3(128), 0, st, src0, dst0, src1, dst1, \
               cos_vals, sin_vals, batch, num_heads, seq_len, rows_total, head_dim, src_rows,        \
               dst_rows, src_bstride, dst_bstride, tab_bstride, col_scale, scale_bstride)
        if (hp == 4) RFK_ROPE(4);
        else if (hp == 2) RFK_ROPE(2);
        else RFK_ROPE(1);
#undef RFK_ROPE
    } else {
        const long long total = (long long)batch * num_heads * rows_total * (head_dim / 2);
        rope_apply_generic_kernel<T, NT><<<ceil_div(total, 256), 256, 0, st>>>(
            src0, dst0, src1, dst1, cos_vals, sin_vals, batch, num_heads, seq_len, rows_total,
            head_dim, src_rows, dst_rows, src_bstride, dst_bstride, tab_bstride);
    }
    return launch_status();
}

// ------------------------------------------- fused projection epilogue

struct QkvParts {
    const float* gamma[3];
    __half* out[3];
    int use_rope[3];
};

// WPR warps per token row and part, 4 warps per CTA. A thread owns rotation-pair chunks
// p = t + 32 * WPR * k (t = its index within the row's threads) of the dim/16 pairs in the row:
// head h = p / (D/16), chunk j = p % (D/16). With WPR > 1 the sum of squares crosses the warps
// of a row through shared memory; rows past the end are clamped (and not stored) so that every
// thread reaches the barrier.
template <int NPAIR, int WPR>
__global__ void __launch_bounds__(128, NPAIR == 1 ? 8 : 1)
qkv_epilogue_kernel(const __half* __restrict__ x, long long row_stride,
                    const __grid_constant__ QkvParts parts,
                    const __half* __restrict__ cos_vals, const __half* __restrict__ sin_vals,
                    int batch, int seq_len, int num_heads, int head_dim, float eps,
                    long long out_seq_stride) {
    constexpr int RPC = 4 / WPR;  // rows per CTA
    pdl_wait();
    pdl_trigger();
    const int lane = (WPR == 1) ? (threadIdx.x & 31) : (threadIdx.x % (32 * WPR));  // index within the row's threads
    const long long rows = (long long)batch * seq_len;
    long long row = (long long)blockIdx.x * RPC + threadIdx.x / (32 * WPR);
    const bool live = row < rows;
    if (WPR == 1 && !live) return;
    if (!live) row = rows - 1;
    const int part = blockIdx.y;
    const int dim = num_heads * head_dim;
    const int npairs = dim / 16, cpt = head_dim / 16, half_d = head_dim / 2;
    const int b = (int)(row / seq_len), s = (int)(row % seq_len);
    const __half* xr = x + row * row_stride + (long long)part * dim;
    const float* gamma = parts.gamma[part];
    __half* out = parts.out[part];

    // every load of the row is issued before the first use: the row itself (streamed), the norm weights
    // and the rotation tables (both shared by all rows, L2-resident)
    const bool rope = parts.use_rope[part] != 0;
    Half8 xl[NPAIR], xh[NPAIR], cl8[NPAIR], sl8[NPAIR], ch8[NPAIR], sh8[NPAIR];
    float gl[NPAIR][8], gh[NPAIR][8];
#pragma unroll
    for (int k = 0; k < NPAIR; ++k) {
        const int p = lane + 32 * WPR * k;
        if (p < npairs) {
            const int o = (p / cpt) * head_dim + (p % cpt) * 8;
            xl[k] = ldcs_half8(xr + o);
            xh[k] = ldcs_half8(xr + o + half_d);
        }
    }
#pragma unroll
    for (int k = 0; k < NPAIR; ++k) {
        const int p = lane + 32 * WPR * k;
        if (p < npairs) {
            const int o = (p / cpt) * head_dim + (p % cpt) * 8;
            if (gamma) {
                ldg_float8(gamma + o, gl[k]);
                ldg_float8(gamma + o + half_d, gh[k]);
            }
            if (rope) {
                const size_t to = ((size_t)b * seq_len + s) * head_dim + (p % cpt) * 8;
                cl8[k] = ldg_half8(cos_vals + to);
                sl8[k] = ldg_half8(sin_vals + to);
                ch8[k] = ldg_half8(cos_vals + to + half_d);
                sh8[k] = ldg_half8(sin_vals + to + half_d);
            }
        }
    }
    float lo[NPAIR][8], hi[NPAIR][8];
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < NPAIR; ++k) {
        const int p = lane + 32 * WPR * k;
        if (p < npairs) {
            unpack8(xl[k], lo[k]);
            unpack8(xh[k], hi[k]);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                ss = fmaf(lo[k][i], lo[k][i], ss);
                ss = fmaf(hi[k][i], hi[k][i], ss);
            }
        }
    }
    if (gamma) {  // uniform over the CTA
        ss = warp_sum(ss);
        if (WPR > 1) {
            __shared__ float s_part[4];
            const int w = threadIdx.x >> 5;
            if ((threadIdx.x & 31) == 0) s_part[w] = ss;
            __syncthreads();
            const int w0 = (w / WPR) * WPR;
            ss = 0.0f;
#pragma unroll
            for (int i = 0; i < WPR; ++i) ss += s_part[w0 + i];
        }
        const float rinv = rsqrtf(ss / (float)dim + eps);
#pragma unroll
        for (int k = 0; k < NPAIR; ++k) {
            const int p = lane + 32 * WPR * k;
            if (p < npairs) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    // the unfused path stores the normalised value as fp16 before rotating it
                    lo[k][i] = round_half((lo[k][i] * rinv) * gl[k][i]);
                    hi[k][i] = round_half((hi[k][i] * rinv) * gh[k][i]);
                }
            }
        }
    }
#pragma unroll
    for (int k = 0; k < NPAIR; ++k) {
        const int p = lane + 32 * WPR * k;
        if (p < npairs) {
            const int h = p / cpt, j = p % cpt;
            if (rope) {
                float cl[8], sl[8], ch[8], sh[8];
                unpack8(cl8[k], cl);
                unpack8(sl8[k], sl);
                unpack8(ch8[k], ch);
                unpack8(sh8[k], sh);
                rotate8(lo[k], hi[k], cl, sl, ch, sh);
            }
            const size_t oo = (((size_t)b * num_heads + h) * out_seq_stride + s) * head_dim + j * 8;
            if (live) {
                store8(out + oo, lo[k]);
                store8(out + oo + half_d, hi[k]);
            }
        }
    }
}

}  // namespace rfk

using namespace rfk;

extern "C" int rfk_triangle_rope_freqs(const rfk_half* pos, const float* learned_freqs,
                                       rfk_half* out_cos, rfk_half* out_sin, int batch,
                                       int seq_len, int num_freqs, int head_dim,
                                       rfk_stream_t stream) {
    if (!pos || !learned_freqs || !out_cos || !out_sin) return RFK_EINVAL;
    if (batch < 0 || seq_len < 0 || num_freqs <= 0 || head_dim <= 0 || (head_dim & 1))
        return RFK_EINVAL;
    const long long tokens = (long long)batch * seq_len;
    if (tokens == 0) return RFK_OK;
    cudaStream_t st = as_stream(stream);
    if (head_dim % 16 == 0 && aligned16(out_cos) && aligned16(out_sin)) {
        const long long n = tokens * (head_dim / 16);
        rope_table_vec_kernel<<<ceil_div(n, 256), 256, 0, st>>>(
            (const __half*)pos, learned_freqs, (__half*)out_cos, (__half*)out_sin, tokens,
            num_freqs, head_dim);
    } else {
        const long long n = tokens * head_dim;
        rope_table_generic_kernel<<<ceil_div(n, 256), 256, 0, st>>>(
            (const __half*)pos, learned_freqs, (__half*)out_cos, (__half*)out_sin, tokens,
            num_freqs, head_dim);
    }
    return launch_status();
}

extern "C" int rfk_apply_rope(rfk_half* q, rfk_half* k, const rfk_half* c, const rfk_half* s,
                              int batch, int num_heads, int seq_len, int head_dim,
                              rfk_stream_t stream) {
    return launch_rope<__half, 2>((const __half*)q, (__half*)q, (const __half*)k, (__half*)k,
                                  (const __half*)c, (const __half*)s, batch, num_heads, seq_len,
                                  seq_len, head_dim, seq_len, seq_len, as_stream(stream));
}

extern "C" int rfk_apply_rope_one(rfk_half* x, const rfk_half* c, const rfk_half* s, int batch,
                                  int num_heads, int seq_len, int head_dim, rfk_stream_t stream) {
    return launch_rope<__half, 1>((const __half*)x, (__half*)x, nullptr, nullptr, (const __half*)c,
                                  (const __half*)s, batch, num_heads, seq_len, seq_len, head_dim,
                                  seq_len, seq_len, as_stream(stream));
}

extern "C" int rfk_apply_rope_f32(float* q, float* k, const rfk_half* c, const rfk_half* s,
                                  int batch, int num_heads, int seq_len, int head_dim,
                                  rfk_stream_t stream) {
    return launch_rope<float, 2>(q, q, k, k, (const __half*)c, (const __half*)s, batch, num_heads,
                                 seq_len, seq_len, head_dim, seq_len, seq_len, as_stream(stream));
}

extern "C" int rfk_apply_rope_one_f32(float* x, const rfk_half* c, const rfk_half* s, int batch,
                                      int num_heads, int seq_len, int head_dim,
                                      rfk_stream_t stream) {
    return launch_rope<float, 1>(x, x, nullptr, nullptr, (const __half*)c, (const __half*)s, batch,
                                 num_heads, seq_len, seq_len, head_dim, seq_len, seq_len,
                                 as_stream(stream));
}

extern "C" int rfk_rope_one_oop(const rfk_half* src, rfk_half* dst, const rfk_half* c,
                                const rfk_half* s, int batch, int num_heads, int seq_len,
                                int head_dim, int src_seq_stride, int dst_seq_stride,
                                int copy_tail, rfk_stream_t stream) {
    if (src_seq_stride < seq_len || dst_seq_stride < seq_len) return RFK_EINVAL;
    int rows_total = seq_len;
    if (copy_tail) {
        rows_total = dst_seq_stride;
        if (src_seq_stride < rows_total) return RFK_EINVAL;
    }
    return launch_rope<__half, 1>((const __half*)src, (__half*)dst, nullptr, nullptr,
                                  (const __half*)c, (const __half*)s, batch, num_heads, seq_len,
                                  rows_total, head_dim, src_seq_stride, dst_seq_stride,
                                  as_stream(stream));
}

extern "C" int rfk_rope_one_oop_strided(const rfk_half* src, rfk_half* dst, const rfk_half* c,
                                        const rfk_half* s, int batch, long long src_batch_stride,
                                        long long dst_batch_stride, long long table_batch_stride,
                                        int num_heads, int seq_len, int head_dim, int src_seq_stride,
                                        int dst_seq_stride, const float* col_scale,
                                        long long col_scale_batch_stride, rfk_stream_t stream) {
    if (src_seq_stride < seq_len || dst_seq_stride < seq_len) return RFK_EINVAL;
    if (src_batch_stride < 0 || dst_batch_stride < 0 || table_batch_stride < 0 || col_scale_batch_stride < 0) return RFK_EINVAL;
    return launch_rope<__half, 1>((const __half*)src, (__half*)dst, nullptr, nullptr,
                                  (const __half*)c, (const __half*)s, batch, num_heads, seq_len,
                                  seq_len, head_dim, src_seq_stride, dst_seq_stride,
                                  as_stream(stream), src_batch_stride, dst_batch_stride,
                                  table_batch_stride, (const float*)col_scale, col_scale_batch_stride);
}

extern "C" int rfk_qkv_norm_rope_transpose(const rfk_half* x, long long row_stride, int n_parts,
                                           const float* const* gamma, rfk_half* const* out,
                                           const int* use_rope, const rfk_half* cos_vals,
                                           const rfk_half* sin_vals, int batch, int seq_len,
                                           int num_heads, int head_dim, float eps,
                                           int out_seq_stride, rfk_stream_t stream) {
    if (!x || !gamma || !out || !use_rope || n_parts < 1 || n_parts > 3) return RFK_EINVAL;
    if (out_seq_stride == 0) out_seq_stride = seq_len;
    if (out_seq_stride < seq_len) return RFK_EINVAL;
    if (batch < 0 || seq_len < 0 || num_heads <= 0 || head_dim <= 0) return RFK_EINVAL;
    const long long dim = (long long)num_heads * head_dim;
    if (row_stride < dim * n_parts) return RFK_EINVAL;
    if (head_dim % 16 != 0 || dim > 2048 || row_stride % 8 != 0 || !aligned16(x))
        return RFK_EUNSUPPORTED;
    QkvParts parts{};
    for (int p = 0; p < n_parts; ++p) {
        if (!out[p] || !aligned16(out[p])) return RFK_EINVAL;
        if (gamma[p] && !aligned16(gamma[p])) return RFK_EUNSUPPORTED;
        if (use_rope[p] && (!cos_vals || !sin_vals || !aligned16(cos_vals) || !aligned16(sin_vals)))
            return RFK_EINVAL;
        parts.gamma[p] = gamma[p];
        parts.out[p] = (__half*)out[p];
        parts.use_rope[p] = use_rope[p];
    }
    const long long rows = (long long)batch * seq_len;
    if (rows == 0) return RFK_OK;
    cudaStream_t st = as_stream(stream);
    const int npairs = (int)(dim / 16);
    // two warps per row from 64 chunk pairs on (dim 1024: one pair per thread, 64 registers, 8 CTAs per SM)
#define RFK_QKV(N, W)                                                                            \
    launch_pdl(qkv_epilogue_kernel<N, W>, dim3(ceil_div(rows, 4 / W), n_parts), dim3(128), 0, st, \
               (const __half*)x, row_stride, parts, (const __half*)cos_vals, (const __half*)sin_vals, \
               batch, seq_len, num_heads, head_dim, eps, (long long)out_seq_stride)
    if (npairs <= 32) RFK_QKV(1, 1);
    else if (npairs <= 64) RFK_QKV(1, 2);
    else RFK_QKV(2, 2);
#undef RFK_QKV
    return launch_status();
}
