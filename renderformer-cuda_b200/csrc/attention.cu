// Fused scaled-dot-product attention (forward): O = softmax(scale * Q K^T) V without
// materialising the score matrix.
//
// Reference boundary: rf::sdpa (src/layers/attention.cu:89-166 of BANANASJIM/renderformer-cuda),
// which hands this contraction to a cuDNN fused kernel when it can and otherwise runs
// GEMM -> softmax_cast_fp16 -> GEMM over a [B*H, Sq, Sk] fp32 score matrix (1.5 GB per
// decoder layer at 16 x 4096 x 5672). Semantics kept: fp16 operands, fp32 accumulation,
// scale 1/sqrt(D) applied to the scores, probabilities rounded to fp16 before the second
// product, no mask other than "the first n_keys keys take part".
//
// Design (one CTA = 128 queries of one head, 8 warps x 16 query rows):
//   - Q tile loaded once (cp.async) and kept as mma A fragments in registers;
//   - K and V tiles of 64 keys stream through a double-buffered shared-memory ring filled
//     with 16-byte cp.async (zero-filled past the last key row), XOR-swizzled so that the
//     ldmatrix reads are bank-conflict free;
//   - S = Q K^T and O += P V on the tensor cores via mma.sync m16n8k16 (fp16 x fp16 -> fp32);
//     the score tile never leaves registers: its accumulator fragments are rescaled, exponentiated
//     (one ex2 per score, scale folded into the exponent) and re-packed as the A fragments of
//     the second product;
//   - running row maximum / row sum per query are kept per thread quad and combined with two
//     shuffles per tile;
//   - the output tile is normalised, staged through shared memory and written with 128-bit
//     stores, either [B,H,Sq,D] or directly [B,Sq,H*D] (what the output projection reads).
// This is the portable tensor-core path (it also serves head_dim 128 and ragged lengths);
// per layer it replaces 0.72 ms of GEMM + softmax + GEMM and 2.2 GB of score traffic.
#include "common.cuh"

namespace rfk {

constexpr int kAttnBM = 128;      // queries per CTA
constexpr int kAttnBN = 64;       // keys per tile
constexpr int kAttnWarps = 8;
constexpr int kAttnThreads = kAttnWarps * 32;

__device__ __forceinline__ unsigned smem_u32(const void* p) {
    return (unsigned)__cvta_generic_to_shared(p);
}
// 16-byte async copy; src_bytes == 0 zero-fills the destination
__device__ __forceinline__ void cp_async16(void* dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
// D(16x8,f32) += A(16x16,f16,row) * B(16x8,f16,col)
__device__ __forceinline__ void mma_16816(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_half2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&h);
}

// A [rows x HD] fp16 tile in shared memory; 16-byte chunk c of row r lives at chunk c ^ (r & 7).
template <int HD>
__device__ __forceinline__ __half* tile_ptr(__half* base, int row, int chunk) {
    return base + row * HD + ((chunk ^ (row & 7)) << 3);
}

// Copy `rows` x HD halves from global (row pitch `pitch` halves) into a swizzled tile; rows at or
// beyond `valid_rows` are zero-filled.
template <int HD>
__device__ __forceinline__ void load_tile_async(__half* tile, const __half* src, long long pitch, int rows,
                                                int valid_rows, int tid) {
    constexpr int CPR = HD / 8;  // 16-byte chunks per row
    for (int i = tid; i < rows * CPR; i += kAttnThreads) {
        const int r = i / CPR, c = i % CPR;
        const bool ok = r < valid_rows;
        cp_async16(tile_ptr<HD>(tile, r, c), ok ? (const void*)(src + (long long)r * pitch + c * 8) : (const void*)src,
                   ok ? 16 : 0);
    }
}

template <int HD>
__global__ void __launch_bounds__(kAttnThreads)
flash_attention_kernel(const __half* __restrict__ Q, const __half* __restrict__ K, const __half* __restrict__ V,
                       __half* __restrict__ O, int H, int Sq, int Sk, int n_keys, long long kv_head_stride,
                       int o_bshd, float scale_log2e) {
    constexpr int KS = HD / 16;  // k-steps of the QK^T product
    constexpr int NT = HD / 8;   // n-tiles of the PV product (output columns / 8)
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __half* sQ = reinterpret_cast<__half*>(smem_raw);            // [128][HD], reused to stage O
    __half* sK = sQ + kAttnBM * HD;                               // 2 x [64][HD]
    __half* sV = sK + 2 * kAttnBN * HD;                           // 2 x [64][HD]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, tig = lane & 3;
    const int q0 = blockIdx.x * kAttnBM;
    const int bh = blockIdx.y;  // b * H + h
    const __half* Qh = Q + ((long long)bh * Sq + q0) * HD;
    const __half* Kh = K + (long long)bh * kv_head_stride;
    const __half* Vh = V + (long long)bh * kv_head_stride;
    const int n_tiles = (n_keys + kAttnBN - 1) / kAttnBN;

    // prologue: Q tile and the first K/V tile
    load_tile_async<HD>(sQ, Qh, HD, kAttnBM, Sq - q0, tid);
    load_tile_async<HD>(sK, Kh, HD, kAttnBN, Sk, tid);
    load_tile_async<HD>(sV, Vh, HD, kAttnBN, Sk, tid);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();

    // this warp's 16 query rows as A fragments, kept in registers for the whole loop
    unsigned qf[KS][4];
    {
        const int r = warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) ldmatrix_x4(qf[ks], tile_ptr<HD>(sQ, r, ks * 2 + (lane >> 4)));
    }

    float o_acc[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) o_acc[n][0] = o_acc[n][1] = o_acc[n][2] = o_acc[n][3] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY};  // rows g and g+8 of this warp's 16
    float l_run[2] = {0.0f, 0.0f};

    for (int t = 0; t < n_tiles; ++t) {
        const int buf = t & 1;
        // prefetch the next K/V tile into the other buffer (free: tile t-1 was consumed before the
        // barrier that ended the previous iteration)
        if (t + 1 < n_tiles) {
            const int k_next = (t + 1) * kAttnBN;
            load_tile_async<HD>(sK + (buf ^ 1) * kAttnBN * HD, Kh + (long long)k_next * HD, HD, kAttnBN, Sk - k_next, tid);
            load_tile_async<HD>(sV + (buf ^ 1) * kAttnBN * HD, Vh + (long long)k_next * HD, HD, kAttnBN, Sk - k_next, tid);
        }
        cp_async_commit();
        const __half* kt = sK + buf * kAttnBN * HD;
        const __half* vt = sV + buf * kAttnBN * HD;

        // S = Q K^T for 64 keys: 8 n-tiles of 8 keys
        float s[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
            for (int np = 0; np < 4; ++np) {  // pairs of n-tiles
                unsigned kb[4];
                const int key = np * 16 + (lane & 7) + 8 * (lane >> 4);
                ldmatrix_x4(kb, tile_ptr<HD>(const_cast<__half*>(kt), key, ks * 2 + ((lane >> 3) & 1)));
                mma_16816(s[2 * np], qf[ks], kb[0], kb[1]);
                mma_16816(s[2 * np + 1], qf[ks], kb[2], kb[3]);
            }
        }
        // keys at or beyond n_keys do not take part
        const int key_base = t * kAttnBN;
        if (key_base + kAttnBN > n_keys) {
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                const int c = key_base + n * 8 + 2 * tig;
                if (c >= n_keys) s[n][0] = s[n][2] = -INFINITY;
                if (c + 1 >= n_keys) s[n][1] = s[n][3] = -INFINITY;
            }
        }
        // online softmax: rows g (regs 0,1) and g+8 (regs 2,3)
        float mx[2] = {m_run[0], m_run[1]};
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            mx[0] = fmaxf(mx[0], fmaxf(s[n][0], s[n][1]));
            mx[1] = fmaxf(mx[1], fmaxf(s[n][2], s[n][3]));
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        }
        float alpha[2], mc[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            // a row whose keys are all excluded so far keeps m = -inf; use 0 as the reference point then
            const float m_new = mx[r] == -INFINITY ? 0.0f : mx[r];
            alpha[r] = fast_exp2((m_run[r] - m_new) * scale_log2e);  // exp2(-inf) = 0 on the first tile
            m_run[r] = mx[r];
            mc[r] = m_new * scale_log2e;
        }
        float rs[2] = {0.0f, 0.0f};
        unsigned pf[4][4];  // P as A fragments: 4 k-steps of 16 keys
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            const float p0 = fast_exp2(fmaf(s[n][0], scale_log2e, -mc[0]));
            const float p1 = fast_exp2(fmaf(s[n][1], scale_log2e, -mc[0]));
            const float p2 = fast_exp2(fmaf(s[n][2], scale_log2e, -mc[1]));
            const float p3 = fast_exp2(fmaf(s[n][3], scale_log2e, -mc[1]));
            rs[0] += p0 + p1;
            rs[1] += p2 + p3;
            pf[n >> 1][(n & 1) * 2 + 0] = pack_half2(p0, p1);
            pf[n >> 1][(n & 1) * 2 + 1] = pack_half2(p2, p3);
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) l_run[r] = l_run[r] * alpha[r] + rs[r];  // quad partial sums, combined at the end
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            o_acc[n][0] *= alpha[0]; o_acc[n][1] *= alpha[0];
            o_acc[n][2] *= alpha[1]; o_acc[n][3] *= alpha[1];
        }
        // O += P V : k = 64 keys in 4 steps, n = HD output columns in pairs of n-tiles
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
            for (int np = 0; np < NT / 2; ++np) {
                unsigned vb[4];
                const int key = ks * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
                ldmatrix_x4_trans(vb, tile_ptr<HD>(const_cast<__half*>(vt), key, np * 2 + (lane >> 4)));
                mma_16816(o_acc[2 * np], pf[ks], vb[0], vb[1]);
                mma_16816(o_acc[2 * np + 1], pf[ks], vb[2], vb[3]);
            }
        }
        cp_async_wait<0>();  // next tile has landed
        __syncthreads();     // ... for every thread, and everyone is done with this tile's buffers
    }

    // finish: combine the quad's partial row sums, normalise, stage through shared memory
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    const float inv0 = l_run[0] > 0.0f ? 1.0f / l_run[0] : 0.0f;
    const float inv1 = l_run[1] > 0.0f ? 1.0f / l_run[1] : 0.0f;
    // sQ is free: every warp took its fragments before the first barrier of the loop
    __half* sO = sQ;
    {
        const int r0 = warp * 16 + g;
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            const int col = n * 8 + 2 * tig;
            *reinterpret_cast<unsigned*>(tile_ptr<HD>(sO, r0, col >> 3) + (col & 7)) =
                pack_half2(o_acc[n][0] * inv0, o_acc[n][1] * inv0);
            *reinterpret_cast<unsigned*>(tile_ptr<HD>(sO, r0 + 8, col >> 3) + (col & 7)) =
                pack_half2(o_acc[n][2] * inv1, o_acc[n][3] * inv1);
        }
    }
    __syncthreads();
    constexpr int CPR = HD / 8;
    const int b = bh / H, h = bh % H;
    for (int i = tid; i < kAttnBM * CPR; i += kAttnThreads) {
        const int r = i / CPR, c = i % CPR;
        const int q = q0 + r;
        if (q < Sq) {
            const long long off = o_bshd ? (((long long)b * Sq + q) * H + h) * HD + c * 8
                                         : (((long long)bh) * Sq + q) * HD + c * 8;
            *reinterpret_cast<uint4*>(O + off) = *reinterpret_cast<const uint4*>(tile_ptr<HD>(sO, r, c));
        }
    }
}

template <int HD>
static int launch_flash(const __half* Q, const __half* K, const __half* V, __half* O, int B, int H, int Sq, int Sk,
                        int n_keys, long long kv_head_stride, int o_bshd, float scale, cudaStream_t st) {
    const size_t smem = (size_t)(kAttnBM + 4 * kAttnBN) * HD * sizeof(__half);
    if (smem > 48 * 1024) {  // opt in to large dynamic shared memory once per device
        static bool configured[64] = {};
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return (int)e;
        if (dev < 0 || dev >= 64) return RFK_EUNSUPPORTED;
        if (!configured[dev]) {
            e = cudaFuncSetAttribute(flash_attention_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
            configured[dev] = true;
        }
    }
    dim3 grid(ceil_div(Sq, kAttnBM), B * H);
    flash_attention_kernel<HD><<<grid, kAttnThreads, smem, st>>>(Q, K, V, O, H, Sq, Sk, n_keys, kv_head_stride, o_bshd,
                                                                scale * 1.4426950408889634f);
    return launch_status();
}

// ------------------------------------------------------------------ swin window attention
// One CTA = one (window, head): 64 queries x 64 keys x head_dim 64, everything in one pass:
// S = scale Q K^T (mma.sync), optional shifted-window mask, row softmax in registers, P rounded to
// fp16 after normalisation (what the unfused GEMM -> softmax -> GEMM sequence does), O = P V, and
// the output written straight into the [windows * 64, heads * 64] token-major layout the output
// projection reads. Four warps, 16 query rows each; Q, K, V are 8 KB contiguous tiles.
constexpr int kWinTokens = 64, kWinThreads = 128;

// NORMED: Q and K arrive un-normalised (straight from the projection) together with the partial sums of squares of
// their rows (rfk_gemm_f16_heads); the QK-RMSNorm - half((x * rsqrt(mean x^2 + eps)) * gamma), the formula and the
// rounding of the separate kernel - is applied while the tiles are staged into shared memory.
struct WinNorm {
    const float* q_ss; const float* k_ss;      // [rows][tiles] partial sums of squares (rows in window order)
    const float* gamma_q; const float* gamma_k;  // [heads * 64]
    int tiles; float inv_dim, eps;
};

template <bool NORMED>
__global__ void __launch_bounds__(kWinThreads, 8)  // 8 CTAs per SM: the 1024 CTAs of a decoder layer are one wave
window_attention_kernel(const __half* __restrict__ Q, const __half* __restrict__ K, const __half* __restrict__ V,
                        __half* __restrict__ O, const uint8_t* __restrict__ mask, int heads, int nW, float scale_log2e,
                        const WinNorm nrm) {
    constexpr int HD = 64;
    __shared__ __align__(128) __half sQ[kWinTokens * HD];
    __shared__ __align__(128) __half sK[kWinTokens * HD];
    __shared__ __align__(128) __half sV[kWinTokens * HD];
    __shared__ __align__(16) uint8_t sMask[kWinTokens * kWinTokens];  // this window's mask, fetched with the tiles
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, tig = lane & 3;
    pdl_wait();
    pdl_trigger();
    const long long bh = blockIdx.x;
    const int bw = (int)(bh / heads), h = (int)(bh % heads);
    const __half* Qh = Q + bh * (kWinTokens * HD);
    const __half* Kh = K + bh * (kWinTokens * HD);
    const __half* Vh = V + bh * (kWinTokens * HD);
    for (int i = tid; i < kWinTokens * 8; i += kWinThreads) {
        const int r = i >> 3, c = i & 7;
        if (!NORMED) {
            cp_async16(tile_ptr<HD>(sQ, r, c), Qh + r * HD + c * 8, 16);
            cp_async16(tile_ptr<HD>(sK, r, c), Kh + r * HD + c * 8, 16);
        }
        cp_async16(tile_ptr<HD>(sV, r, c), Vh + r * HD + c * 8, 16);
    }
    if (NORMED) {
        // A thread keeps one 8-column chunk (c) of four rows (r0 + 16 k) of both tiles: the weights of its columns are
        // loaded once, and every global load is issued before the first value is needed.
        const int c = tid & 7, r0 = tid >> 3;
        constexpr int kRowsPerThread = kWinTokens * 8 / kWinThreads;  // 4
        Half8 raw[2][kRowsPerThread];
        float ss[2][kRowsPerThread];
        float gq[8], gk[8];
#pragma unroll
        for (int k = 0; k < kRowsPerThread; ++k) {
            const int r = r0 + k * (kWinThreads / 8);
            raw[0][k] = ldg_half8(Qh + r * HD + c * 8);
            raw[1][k] = ldg_half8(Kh + r * HD + c * 8);
            const long long row = (long long)bw * kWinTokens + r;   // token row in window order
            float sq = 0.0f, sk = 0.0f;
            for (int t = 0; t < nrm.tiles; ++t) {
                sq += __ldg(nrm.q_ss + row * nrm.tiles + t);
                sk += __ldg(nrm.k_ss + row * nrm.tiles + t);
            }
            ss[0][k] = sq;
            ss[1][k] = sk;
        }
        ldg_float8(nrm.gamma_q + h * HD + c * 8, gq);
        ldg_float8(nrm.gamma_k + h * HD + c * 8, gk);
#pragma unroll
        for (int k = 0; k < kRowsPerThread; ++k) {
            const int r = r0 + k * (kWinThreads / 8);
#pragma unroll
            for (int which = 0; which < 2; ++which) {
                const float rinv = rsqrtf(ss[which][k] * nrm.inv_dim + nrm.eps);
                float x[8];
                unpack8(raw[which][k], x);
#pragma unroll
                for (int e = 0; e < 8; ++e) x[e] = (x[e] * rinv) * (which ? gk[e] : gq[e]);
                *reinterpret_cast<Half8*>(tile_ptr<HD>(which ? sK : sQ, r, c)) = pack8(x);
            }
        }
    }
    if (mask) {
        const uint8_t* mw = mask + (long long)(bw % nW) * (kWinTokens * kWinTokens);
        for (int i = tid; i < kWinTokens * kWinTokens / 16; i += kWinThreads) cp_async16(sMask + i * 16, mw + i * 16, 16);
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();

    unsigned qf[4][4];
    {
        const int r = warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) ldmatrix_x4(qf[ks], tile_ptr<HD>(sQ, r, ks * 2 + (lane >> 4)));
    }
    float s[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f;
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
        for (int np = 0; np < 4; ++np) {
            unsigned kb[4];
            const int key = np * 16 + (lane & 7) + 8 * (lane >> 4);
            ldmatrix_x4(kb, tile_ptr<HD>(sK, key, ks * 2 + ((lane >> 3) & 1)));
            mma_16816(s[2 * np], qf[ks], kb[0], kb[1]);
            mma_16816(s[2 * np + 1], qf[ks], kb[2], kb[3]);
        }
    }
    // scores in the exponent's units; masked-out pairs get -FLT_MAX (a fully masked row ends up uniform)
    const int q_lo = warp * 16 + g;  // this thread's rows: q_lo (regs 0, 1) and q_lo + 8 (regs 2, 3)
    const uint8_t* m0 = sMask + q_lo * kWinTokens;
    const uint8_t* m1 = m0 + 8 * kWinTokens;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 8; ++n) {
        const int c = n * 8 + 2 * tig;
        s[n][0] *= scale_log2e; s[n][1] *= scale_log2e; s[n][2] *= scale_log2e; s[n][3] *= scale_log2e;
        if (mask) {
            const unsigned a = *reinterpret_cast<const unsigned short*>(m0 + c);
            const unsigned b = *reinterpret_cast<const unsigned short*>(m1 + c);
            if ((a & 0xffu) == 0) s[n][0] = -FLT_MAX;
            if ((a >> 8) == 0) s[n][1] = -FLT_MAX;
            if ((b & 0xffu) == 0) s[n][2] = -FLT_MAX;
            if ((b >> 8) == 0) s[n][3] = -FLT_MAX;
        }
        mx[0] = fmaxf(mx[0], fmaxf(s[n][0], s[n][1]));
        mx[1] = fmaxf(mx[1], fmaxf(s[n][2], s[n][3]));
    }
    float rs[2] = {0.0f, 0.0f};
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    }
#pragma unroll
    for (int n = 0; n < 8; ++n) {
        s[n][0] = fast_exp2(s[n][0] - mx[0]); s[n][1] = fast_exp2(s[n][1] - mx[0]);
        s[n][2] = fast_exp2(s[n][2] - mx[1]); s[n][3] = fast_exp2(s[n][3] - mx[1]);
        rs[0] += s[n][0] + s[n][1];
        rs[1] += s[n][2] + s[n][3];
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
        rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
        rs[r] = 1.0f / rs[r];
    }
    unsigned pf[4][4];  // normalised P as A fragments: 4 k-steps of 16 keys
#pragma unroll
    for (int n = 0; n < 8; ++n) {
        pf[n >> 1][(n & 1) * 2 + 0] = pack_half2(s[n][0] * rs[0], s[n][1] * rs[0]);
        pf[n >> 1][(n & 1) * 2 + 1] = pack_half2(s[n][2] * rs[1], s[n][3] * rs[1]);
    }
    float o_acc[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) o_acc[n][0] = o_acc[n][1] = o_acc[n][2] = o_acc[n][3] = 0.0f;
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
        for (int np = 0; np < 4; ++np) {
            unsigned vb[4];
            const int key = ks * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
            ldmatrix_x4_trans(vb, tile_ptr<HD>(sV, key, np * 2 + (lane >> 4)));
            mma_16816(o_acc[2 * np], pf[ks], vb[0], vb[1]);
            mma_16816(o_acc[2 * np + 1], pf[ks], vb[2], vb[3]);
        }
    }
    // stage this warp's 16 output rows over its own rows of sQ (only this warp read them), then 128-bit stores
    __syncwarp();
#pragma unroll
    for (int n = 0; n < 8; ++n) {
        const int col = n * 8 + 2 * tig;
        *reinterpret_cast<unsigned*>(tile_ptr<HD>(sQ, q_lo, col >> 3) + (col & 7)) = pack_half2(o_acc[n][0], o_acc[n][1]);
        *reinterpret_cast<unsigned*>(tile_ptr<HD>(sQ, q_lo + 8, col >> 3) + (col & 7)) = pack_half2(o_acc[n][2], o_acc[n][3]);
    }
    __syncwarp();
    const long long dim = (long long)heads * HD;
#pragma unroll
    for (int i = lane; i < 16 * 8; i += 32) {
        const int r = warp * 16 + (i >> 3), c = i & 7;
        *reinterpret_cast<uint4*>(O + ((long long)bw * kWinTokens + r) * dim + h * HD + c * 8) =
            *reinterpret_cast<const uint4*>(tile_ptr<HD>(sQ, r, c));
    }
}

// attention_tc.cu
extern std::atomic<int> g_attn_path;
extern std::atomic<int> g_attn_split;
size_t attention_tc_workspace_bytes();
int attention_tc_plan(long long units, int n_tiles, int sms, int* whole_units, int* n_pieces, unsigned short* pieces, int max_pieces);
int launch_attention_tc(const __half* Q, const __half* K, const __half* V, __half* O, int B, int H, int Sq, int Sk,
                        int n_keys, int o_bshd, float scale, cudaStream_t st, const float* row_ss, int ss_tiles,
                        int norm_dim, float norm_eps, void* ws, size_t ws_bytes, int v_shared);

}  // namespace rfk

using namespace rfk;

extern "C" int rfk_flash_attention(const rfk_half* Q, const rfk_half* K, const rfk_half* V, rfk_half* O, int B,
                                   int H, int Sq, int Sk, int n_keys, int D, int o_bshd, float scale,
                                   rfk_stream_t stream) {
    if (!Q || !K || !V || !O || B < 0 || H <= 0 || Sq < 0 || Sk <= 0 || n_keys <= 0 || n_keys > Sk) return RFK_EINVAL;
    if (!(scale > 0.0f)) return RFK_EINVAL;
    if (B == 0 || Sq == 0) return RFK_OK;
    if ((long long)B * H > 65535) return RFK_EUNSUPPORTED;
    if (!aligned16(Q) || !aligned16(K) || !aligned16(V) || !aligned16(O)) return RFK_EUNSUPPORTED;
    cudaStream_t st = as_stream(stream);
    const long long kvs = (long long)Sk * D;
    const int path = g_attn_path.load(std::memory_order_relaxed);
    if (D == 64 && path != 1) {  // tcgen05 kernel; in automatic mode the mma.sync kernel takes over if it cannot run
        const int rc = launch_attention_tc((const __half*)Q, (const __half*)K, (const __half*)V, (__half*)O, B, H, Sq, Sk,
                                           n_keys, o_bshd, scale, st, nullptr, 0, 0, 0.0f, nullptr, 0, 0);
        if (rc != RFK_EUNSUPPORTED || path == 2) return rc;
    }
    if (D == 64)
        return launch_flash<64>((const __half*)Q, (const __half*)K, (const __half*)V, (__half*)O, B, H, Sq, Sk, n_keys, kvs,
                                o_bshd, scale, st);
    if (D == 128)
        return launch_flash<128>((const __half*)Q, (const __half*)K, (const __half*)V, (__half*)O, B, H, Sq, Sk, n_keys, kvs,
                                 o_bshd, scale, st);
    return RFK_EUNSUPPORTED;
}

extern "C" int rfk_flash_attention_ex(const rfk_half* Q, const rfk_half* K, const rfk_half* V, rfk_half* O,
                                      const float* q_row_ss, int ss_tiles, int norm_dim, float eps, void* workspace,
                                      size_t workspace_bytes, int v_shared, int B, int H, int Sq, int Sk, int n_keys, int D,
                                      int o_bshd, float scale, rfk_stream_t stream) {
    if (!Q || !K || !V || !O || B < 0 || H <= 0 || Sq < 0 || Sk <= 0 || n_keys <= 0 || n_keys > Sk || !(scale > 0.0f))
        return RFK_EINVAL;
    if (q_row_ss && (ss_tiles <= 0 || norm_dim <= 0)) return RFK_EINVAL;
    if (workspace && workspace_bytes < attention_tc_workspace_bytes()) return RFK_EINVAL;
    if (B == 0 || Sq == 0) return RFK_OK;
    if (D != 64 || (long long)B * H > 65535 || g_attn_path.load(std::memory_order_relaxed) == 1) return RFK_EUNSUPPORTED;
    if (!aligned16(Q) || !aligned16(K) || !aligned16(V) || !aligned16(O) || !aligned16(workspace)) return RFK_EUNSUPPORTED;
    return launch_attention_tc((const __half*)Q, (const __half*)K, (const __half*)V, (__half*)O, B, H, Sq, Sk, n_keys, o_bshd,
                               scale, as_stream(stream), q_row_ss, ss_tiles, norm_dim, eps, workspace, workspace_bytes, v_shared != 0);
}

extern "C" size_t rfk_flash_attention_workspace_bytes(void) { return attention_tc_workspace_bytes(); }

extern "C" int rfk_flash_attention_plan(long long units, int n_tiles, int sms, int* whole_units, int* n_pieces,
                                        unsigned short* pieces, int max_pieces) {
    return attention_tc_plan(units, n_tiles, sms, whole_units, n_pieces, pieces, max_pieces);
}

extern "C" int rfk_flash_attention_set_split(int on) {
    g_attn_split.store(on ? 1 : 0, std::memory_order_relaxed);
    return RFK_OK;
}

extern "C" int rfk_window_attention(const rfk_half* Q, const rfk_half* K, const rfk_half* V, rfk_half* O,
                                    const uint8_t* mask, int BnW, int num_heads, int window_tokens, int head_dim, int nW,
                                    float scale, rfk_stream_t stream) {
    if (!Q || !K || !V || !O || BnW < 0 || num_heads <= 0 || nW <= 0) return RFK_EINVAL;
    if (window_tokens != kWinTokens || head_dim != 64) return RFK_EUNSUPPORTED;
    if (BnW == 0) return RFK_OK;
    if (!aligned16(Q) || !aligned16(K) || !aligned16(V) || !aligned16(O)) return RFK_EUNSUPPORTED;
    if (mask && !aligned16(mask)) return RFK_EUNSUPPORTED;
    const long long ctas = (long long)BnW * num_heads;
    if (ctas > 0x7fffffffLL) return RFK_EUNSUPPORTED;
    launch_pdl(window_attention_kernel<false>, dim3((unsigned)ctas), dim3(kWinThreads), 0, as_stream(stream),
               (const __half*)Q, (const __half*)K, (const __half*)V, (__half*)O, mask, num_heads, nW,
               scale * 1.4426950408889634f, WinNorm{});
    return launch_status();
}

extern "C" int rfk_window_attention_normed(const rfk_half* Q, const rfk_half* K, const rfk_half* V, rfk_half* O,
                                           const uint8_t* mask, const float* q_row_ss, const float* k_row_ss, int ss_tiles,
                                           const float* gamma_q, const float* gamma_k, int norm_dim, float eps, int BnW,
                                           int num_heads, int window_tokens, int head_dim, int nW, float scale,
                                           rfk_stream_t stream) {
    if (!Q || !K || !V || !O || !q_row_ss || !k_row_ss || !gamma_q || !gamma_k || BnW < 0 || num_heads <= 0 || nW <= 0 ||
        ss_tiles <= 0 || norm_dim <= 0)
        return RFK_EINVAL;
    if (window_tokens != kWinTokens || head_dim != 64) return RFK_EUNSUPPORTED;
    if (BnW == 0) return RFK_OK;
    if (!aligned16(Q) || !aligned16(K) || !aligned16(V) || !aligned16(O) || !aligned16(gamma_q) || !aligned16(gamma_k))
        return RFK_EUNSUPPORTED;
    if (mask && !aligned16(mask)) return RFK_EUNSUPPORTED;
    const long long ctas = (long long)BnW * num_heads;
    if (ctas > 0x7fffffffLL) return RFK_EUNSUPPORTED;
    const WinNorm nrm{q_row_ss, k_row_ss, gamma_q, gamma_k, ss_tiles, 1.0f / (float)norm_dim, eps};
    launch_pdl(window_attention_kernel<true>, dim3((unsigned)ctas), dim3(kWinThreads), 0, as_stream(stream),
               (const __half*)Q, (const __half*)K, (const __half*)V, (__half*)O, mask, num_heads, nW,
               scale * 1.4426950408889634f, nrm);
    return launch_status();
}
