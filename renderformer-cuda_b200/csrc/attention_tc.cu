// Fused attention on the 5th-generation tensor cores (tcgen05 + tensor memory), head_dim 64.
//
// Same function as flash_attention_kernel (attention.cu): O = softmax(scale * Q K^T) V over
// the first n_keys keys, fp16 operands, fp32 accumulation, probabilities rounded to fp16.
// Reference boundary: rf::sdpa, src/layers/attention.cu:89-166 of BANANASJIM/renderformer-cuda.
//
// One CTA = 128 queries of one head, 6 warps with fixed roles:
//   warps 0-3  softmax: thread r owns query row r. The score tile S (128 x 128 fp32) lives in
//              tensor memory, lane = row, so a row's max / sum are thread-local: tcgen05.ld
//              brings 32 columns at a time into registers, no shuffles. P = exp2(...) goes to
//              shared memory as fp16 in the operand layout of the second product; the output
//              accumulator O (128 x 64 fp32, also in tensor memory) is rescaled in place
//              (tcgen05.ld / st) only when some row's running maximum moved.
//   warp 4     producer: streams K and V tiles of 128 keys through a 2-stage shared-memory ring
//              with 16-byte cp.async (zero-filled past the last key row).
//   warp 5     one elected thread issues tcgen05.mma: S = Q K^T (M128 N128 K16 x 4) and
//              O += P V (M128 N64 K16 x 8), and tcgen05.commit onto mbarriers.
// All operand tiles (Q, K, V, P) use one layout: rows of 128 bytes with the 16-byte chunks
// XOR-swizzled by (row & 7), which is both what 16-byte copies write without bank conflicts and
// the tensor core's SWIZZLE_128B canonical layout (K-major for Q, K, P; MN-major for V).
// Tensor memory: 256 columns per CTA (S: 128, O: 64), shared memory 113 KB: two CTAs per SM.
// Every mbarrier wait is bounded; on a time-out the CTA raises an error flag, drains its copies,
// frees its tensor memory and returns.
#include "attention_tc.cuh"
#include "common.cuh"

namespace rfk {

__device__ int g_attn_tc_error = 0;  // first time-out / failure code seen by any CTA since load

namespace tcattn {

constexpr int BM = 128, BN = 128, HD = 64;
constexpr int kThreads = 192;
constexpr int kTileBytes = 128 * 128;          // 128 rows x 128 bytes
constexpr int kTmemCols = 256;                 // S at +0 (128 columns), O at +128 (64 columns)

struct __align__(8) Ctrl {
    uint64_t full[2], empty[2], s_full, s_free, p_full, pv_done;
    uint32_t tmem_base;
    int abort;
};

// Q, K0, K1, V0, V1, P0, P1 and the control block. Two CTAs (plus 1 KB each that the system
// reserves) have to fit the SM's 228 KB, so there is no alignment slack: the dynamic shared
// memory window is declared 1024-byte aligned and the kernel checks it.
constexpr int kSmemBytes = 7 * kTileBytes + 128;
static_assert(sizeof(Ctrl) <= 128, "control block");
static_assert(2 * (kSmemBytes + 1024) <= 228 * 1024, "two CTAs per SM");

enum : int { kErrTimeout = 1, kErrSmemAlign = 2 };

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

__device__ __forceinline__ void cp16(uint32_t dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_wait_all() {
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}
// byte offset of 16-byte chunk `c` of row `r` inside a [128 x 128 B] swizzled tile
__device__ __forceinline__ uint32_t swz(int r, int c) { return (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4)); }

// rows [0, valid) of a [128 x 64] fp16 global tile (row pitch 64 halves) -> swizzled smem tile
__device__ __forceinline__ void load_tile(uint32_t tile, const __half* src, int valid, int t, int nthreads) {
    for (int i = t; i < 128 * 8; i += nthreads) {
        const int r = i >> 3, c = i & 7;
        const bool ok = r < valid;
        cp16(tile + swz(r, c), ok ? (const void*)(src + (size_t)r * HD + c * 8) : (const void*)src, ok ? 16 : 0);
    }
}

__global__ void __launch_bounds__(kThreads, 2)
attention_tc_kernel(const __half* __restrict__ Q, const __half* __restrict__ K, const __half* __restrict__ V,
                    __half* __restrict__ O, int H, int Sq, int Sk, int n_keys, int o_bshd, float scale_log2e) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const uint32_t base = tc::smem_addr(smem_raw);
    if (base & 1023u) {  // swizzled tiles need 1024-byte alignment; uniform over the CTA, nothing allocated yet
        if (threadIdx.x == 0) atomicCAS(&g_attn_tc_error, 0, kErrSmemAlign);
        return;
    }
    const uint32_t sQ = base, sK = base + kTileBytes, sV = base + 3 * kTileBytes, sP = base + 5 * kTileBytes;
    Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem_raw + 7 * kTileBytes);
    volatile int* abort_flag = &ctrl->abort;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int q0 = blockIdx.x * BM;
    const int bh = blockIdx.y;
    const __half* Qh = Q + ((size_t)bh * Sq + q0) * HD;
    const __half* Kh = K + (size_t)bh * Sk * HD;
    const __half* Vh = V + (size_t)bh * Sk * HD;
    const int n_tiles = (n_keys + BN - 1) / BN;

    if (tid == 0) {
        tc::mbar_init(&ctrl->full[0], 1); tc::mbar_init(&ctrl->full[1], 1);
        tc::mbar_init(&ctrl->empty[0], 1); tc::mbar_init(&ctrl->empty[1], 1);
        tc::mbar_init(&ctrl->s_full, 1); tc::mbar_init(&ctrl->s_free, 4);
        tc::mbar_init(&ctrl->p_full, 4); tc::mbar_init(&ctrl->pv_done, 1);
        ctrl->abort = 0;
        tc::fence_barrier_init();
    }
    if (warp == 0) {  // one warp allocates the CTA's tensor memory and later frees it
        tc::tmem_alloc(&ctrl->tmem_base, kTmemCols);
        tc::tmem_relinquish();
    }
    load_tile(sQ, Qh, Sq - q0, tid, kThreads);
    cp_wait_all();
    tc::fence_proxy_async();
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem = ctrl->tmem_base;
    const uint32_t tmem_S = tmem, tmem_O = tmem + 128;

    if (warp == 4) {
        // ------------------------------------------------------------ producer
        for (int j = 0; j < n_tiles; ++j) {
            const int s = j & 1;
            // stage s was last read by the products of tile j - 2 (phase (j >> 1) - 1 of empty[s])
            if (j >= 2 && !__all_sync(0xffffffffu, tc::mbar_wait(&ctrl->empty[s], ((j >> 1) + 1) & 1, abort_flag))) break;
            const int k0 = j * BN;
            load_tile(sK + s * kTileBytes, Kh + (size_t)k0 * HD, Sk - k0, lane, 32);
            load_tile(sV + s * kTileBytes, Vh + (size_t)k0 * HD, Sk - k0, lane, 32);
            cp_wait_all();
            tc::fence_proxy_async();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&ctrl->full[s]);
        }
        cp_wait_all();
    } else if (warp == 5) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_qk = tc::umma_idesc_f16(BM, BN, 0);
            constexpr uint32_t idesc_pv = tc::umma_idesc_f16(BM, HD, 1);
            auto issue_qk = [&](int stage) {
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks)  // 16 head-dim elements = 32 bytes along a row
                    tc::umma_f16(tmem_S, tc::umma_desc_sw128(sQ + ks * 32),
                                 tc::umma_desc_sw128(sK + stage * kTileBytes + ks * 32), idesc_qk, ks > 0);
            };
            bool ok = tc::mbar_wait(&ctrl->full[0], 0, abort_flag);
            if (ok) {
                tc::tc_fence_after();
                issue_qk(0);
                tc::umma_commit(&ctrl->s_full);
            }
            for (int j = 0; ok && j < n_tiles; ++j) {
                const int s = j & 1;
                if (j + 1 < n_tiles) {
                    ok = tc::mbar_wait(&ctrl->full[s ^ 1], ((j + 1) >> 1) & 1, abort_flag) &&
                         tc::mbar_wait(&ctrl->s_free, j & 1, abort_flag);
                    if (!ok) break;
                    tc::tc_fence_after();
                    issue_qk(s ^ 1);
                    tc::umma_commit(&ctrl->s_full);
                }
                ok = tc::mbar_wait(&ctrl->p_full, j & 1, abort_flag);
                if (!ok) break;
                tc::tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < BN / 16; ++ks) {
                    // P: two [128 x 64] K-major sub-tiles, 32 bytes per step inside a sub-tile;
                    // V: MN-major, 16 keys = 16 rows of 128 bytes per step
                    const uint32_t pa = sP + (ks >> 2) * kTileBytes + (ks & 3) * 32;
                    const uint32_t vb = sV + s * kTileBytes + ks * 16 * 128;
                    tc::umma_f16(tmem_O, tc::umma_desc_sw128(pa), tc::umma_desc_sw128(vb), idesc_pv, (j > 0) || (ks > 0));
                }
                tc::umma_commit(&ctrl->empty[s]);
                tc::umma_commit(&ctrl->pv_done);
            }
        }
        __syncwarp();
    }
    else {
        // ------------------------------------------------------------ softmax, warps 0-3
        constexpr unsigned kFull = 0xffffffffu;
        const int r = tid;                                          // query row of this thread = its tensor-memory lane
        const uint32_t lane_off = (uint32_t)(warp * 32) << 16;      // a warp reaches lanes [32 * (warp % 4), +32)
        float m_run = -INFINITY, l_run = 0.0f;
        bool ok = true;
        uint32_t v[32];
        for (int j = 0; j < n_tiles; ++j) {
            ok = __all_sync(kFull, tc::mbar_wait(&ctrl->s_full, j & 1, abort_flag));
            if (!ok) break;
            tc::tc_fence_after();
            const int n_valid = min(BN, n_keys - j * BN);           // real keys among this tile's 128 columns
            // pass 1: row maximum of the raw scores
            float m_tile = -INFINITY;
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
                tc::tmem_ld32(tmem_S + lane_off + ch * 32, v);
                tc::tc_wait_ld();
                if (n_valid >= (ch + 1) * 32) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) m_tile = fmaxf(m_tile, __uint_as_float(v[i]));
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (ch * 32 + i < n_valid) m_tile = fmaxf(m_tile, __uint_as_float(v[i]));
                }
            }
            const float m_new = fmaxf(m_run, m_tile);
            const float alpha = fast_exp2((m_run - m_new) * scale_log2e);  // first tile: exp2(-inf) = 0
            const float mc = m_new * scale_log2e;
            if (j > 0) {
                // O and the P tiles belong to the tensor core until the previous tile's P V is done
                ok = __all_sync(kFull, tc::mbar_wait(&ctrl->pv_done, (j - 1) & 1, abort_flag));
                if (!ok) break;
                tc::tc_fence_after();
                if (__any_sync(kFull, m_new > m_run)) {  // some row's maximum moved: rescale this warp's 32 rows of O
#pragma unroll
                    for (int hc = 0; hc < 2; ++hc) {
                        tc::tmem_ld32(tmem_O + lane_off + hc * 32, v);
                        tc::tc_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                        tc::tmem_st32(tmem_O + lane_off + hc * 32, v);
                    }
                    tc::tc_wait_st();
                }
            }
            l_run *= alpha;
            m_run = m_new;
            // pass 2: P = exp2(scale * log2e * (S - max)) as fp16 into the two K-major sub-tiles of sP
            float l_tile = 0.0f;
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
                tc::tmem_ld32(tmem_S + lane_off + ch * 32, v);
                tc::tc_wait_ld();
                uint32_t pk[16];
                if (n_valid >= (ch + 1) * 32) {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float p0 = fast_exp2(fmaf(__uint_as_float(v[i]), scale_log2e, -mc));
                        const float p1 = fast_exp2(fmaf(__uint_as_float(v[i + 1]), scale_log2e, -mc));
                        l_tile += p0 + p1;
                        pk[i >> 1] = pack_half2(p0, p1);
                    }
                } else {  // last tile: columns at or beyond n_keys contribute nothing
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        float p0 = fast_exp2(fmaf(__uint_as_float(v[i]), scale_log2e, -mc));
                        float p1 = fast_exp2(fmaf(__uint_as_float(v[i + 1]), scale_log2e, -mc));
                        if (ch * 32 + i >= n_valid) p0 = 0.0f;
                        if (ch * 32 + i + 1 >= n_valid) p1 = 0.0f;
                        l_tile += p0 + p1;
                        pk[i >> 1] = pack_half2(p0, p1);
                    }
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int cc = ch * 4 + q;  // 16-byte chunk (8 keys) of the 256-byte P row
                    st_shared_v4(sP + (cc >> 3) * kTileBytes + swz(r, cc & 7), pk[4 * q], pk[4 * q + 1], pk[4 * q + 2],
                                 pk[4 * q + 3]);
                }
            }
            l_run += l_tile;
            tc::tc_fence_before();    // this thread's tensor-memory reads of S and writes of O come before the arrivals
            tc::fence_proxy_async();  // its P values become visible to the tensor core
            __syncwarp();
            if (lane == 0) {
                tc::mbar_arrive(&ctrl->s_free);  // S may be overwritten by the next Q K^T
                tc::mbar_arrive(&ctrl->p_full);  // P (and the rescaled O) are ready for P V
            }
        }
        // ---- epilogue: O / l -> fp16 -> global, one 128-byte row per thread
        if (ok) ok = __all_sync(kFull, tc::mbar_wait(&ctrl->pv_done, (n_tiles - 1) & 1, abort_flag));
        if (ok) {
            tc::tc_fence_after();
            const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
            const int q = q0 + r;
            const int b = bh / H, h = bh % H;
            __half* dst = o_bshd ? O + (((size_t)b * Sq + q) * H + h) * HD : O + ((size_t)bh * Sq + q) * HD;
#pragma unroll
            for (int hc = 0; hc < 2; ++hc) {
                tc::tmem_ld32(tmem_O + lane_off + hc * 32, v);
                tc::tc_wait_ld();
                if (q < Sq) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint4 o;
                        o.x = pack_half2(__uint_as_float(v[8 * c + 0]) * inv, __uint_as_float(v[8 * c + 1]) * inv);
                        o.y = pack_half2(__uint_as_float(v[8 * c + 2]) * inv, __uint_as_float(v[8 * c + 3]) * inv);
                        o.z = pack_half2(__uint_as_float(v[8 * c + 4]) * inv, __uint_as_float(v[8 * c + 5]) * inv);
                        o.w = pack_half2(__uint_as_float(v[8 * c + 6]) * inv, __uint_as_float(v[8 * c + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + hc * 32 + c * 8) = o;
                    }
                }
            }
        }
    }

    // ---- teardown: every path (normal or aborted) arrives here with no divergence inside a warp
    tc::tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc::tc_fence_after();
        tc::tmem_dealloc(tmem, kTmemCols);
    }
    if (tid == 0 && ctrl->abort) atomicCAS(&g_attn_tc_error, 0, kErrTimeout);
}

}  // namespace tcattn

int g_attn_path = 0;  // 0 automatic, 1 mma.sync kernel, 2 tcgen05 kernel (head_dim 64 only)

// Launches the tcgen05 kernel; the caller has validated pointers, alignment and sizes (D == 64).
int launch_attention_tc(const __half* Q, const __half* K, const __half* V, __half* O, int B, int H, int Sq, int Sk,
                        int n_keys, int o_bshd, float scale, cudaStream_t st) {
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return RFK_EUNSUPPORTED;
    if (!configured[dev]) {
        e = cudaFuncSetAttribute(tcattn::attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 tcattn::kSmemBytes);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(tcattn::attention_tc_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return (int)e;
        configured[dev] = true;
    }
    dim3 grid(ceil_div(Sq, tcattn::BM), B * H);
    tcattn::attention_tc_kernel<<<grid, tcattn::kThreads, tcattn::kSmemBytes, st>>>(Q, K, V, O, H, Sq, Sk, n_keys, o_bshd,
                                                                                    scale * 1.4426950408889634f);
    return launch_status();
}

}  // namespace rfk

using namespace rfk;

extern "C" int rfk_flash_attention_set_path(int path) {
    if (path < 0 || path > 2) return RFK_EINVAL;
    g_attn_path = path;
    return RFK_OK;
}

extern "C" int rfk_flash_attention_error(int* code, int clear) {
    if (!code) return RFK_EINVAL;
    cudaError_t e = cudaMemcpyFromSymbol(code, g_attn_tc_error, sizeof(int));
    if (e != cudaSuccess) return (int)e;
    if (clear) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(g_attn_tc_error, &zero, sizeof(int));
        if (e != cudaSuccess) return (int)e;
    }
    return RFK_OK;
}
