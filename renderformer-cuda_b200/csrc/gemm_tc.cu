// Dense projection C = epilogue(A W^T) on the 5th-generation tensor cores (tcgen05 + tensor memory
// + TMA), fp16 operands, fp32 accumulation, with the element-wise step that follows the projection
// in the layer fused into the epilogue:
//   RFK_GEMM_EPI_NONE      C = A W^T (+ bias)                                   rf::linear
//   RFK_GEMM_EPI_RESIDUAL  C = A W^T (+ bias) + R                               rf::linear + rf::residual_add
//   RFK_GEMM_EPI_SWIGLU    C = silu(A Wg^T) * (A Wu^T)                          the two projections and the
//                                                                               gate of rf::ffn_swiglu
// Reference boundary: rf::linear, src/layers/linear.cu:7-25 (one cublasGemmEx + a bias kernel), and
// rf::ffn_swiglu, src/layers/transformer.cu:63-79 (two GEMMs into [M, hidden] buffers, fused_silu_mul,
// a third GEMM) of BANANASJIM/renderformer-cuda.
//
// One persistent CTA per SM walks output tiles of 128 rows x 256 accumulator columns (row-tile index
// fastest, so that the CTAs running together share weight tiles in L2). K is consumed in blocks of
// 64 halves (one 128-byte swizzle row) through a ring of kStages shared-memory stages:
//   warp 0   producer: one thread issues three TMA tile loads per stage (A 128 x 64; two weight boxes
//            of 128 x 64 - rows n0..n0+127 and n0+128..n0+255 of W, or, with the SwiGLU epilogue,
//            the gate rows and the up rows of the same 128 hidden units) that complete on the
//            stage's mbarrier; rows and columns past the end of a tensor arrive as zeros.
//   warp 1   one thread issues tcgen05.mma M128 N256 K16 x 4 per stage into one of two accumulators
//            in tensor memory (2 x 256 columns), then commits the stage's "empty" barrier; after
//            the last K block it commits the accumulator's "full" barrier.
//   warps 2-5 epilogue: a thread owns one output row (= its tensor-memory lane), reads the row in
//            chunks of 32 columns with tcgen05.ld, applies bias / residual / gate in fp32, rounds
//            once to fp16 and writes 64 contiguous bytes per chunk. While they drain accumulator a,
//            the tensor core already fills accumulator a ^ 1 with the CTA's next tile.
// Every mbarrier wait is bounded; on a time-out the CTA raises an error word, waits (bounded) for its
// own copies and products in flight, frees its tensor memory and returns.
#include <cuda.h>  // CUtensorMap and its enums; the encoder itself is looked up at run time
#include <cstdlib>
#include "attention_tc.cuh"
#include "common.cuh"

namespace rfk {

__device__ int g_gemm_tc_error = 0;  // first time-out / failure code seen by any CTA since load

namespace tcgemm {

constexpr int BM = 128, BNACC = 256, BK = 64;
constexpr int kStages = 4;
constexpr int kThreads = 192;                  // warp 0 producer, warp 1 MMA issuer, warps 2-5 epilogue
constexpr int kABytes = BM * BK * 2;           // 16 KB
constexpr int kWBoxBytes = 128 * BK * 2;       // 16 KB, two per stage
constexpr int kStageBytes = kABytes + 2 * kWBoxBytes;
constexpr int kTmemCols = 512;                 // two accumulators of 256 fp32 columns

struct __align__(8) Ctrl {
    uint64_t full[kStages], empty[kStages], acc_full[2], acc_empty[2], drain;
    uint32_t tmem_base;
    int abort;
};
constexpr int kSmemBytes = kStages * kStageBytes + 256;
static_assert(sizeof(Ctrl) <= 256, "control block");
static_assert(kSmemBytes + 1024 <= 227 * 1024, "one CTA per SM");

enum : int { kErrTimeout = 1, kErrSmemAlign = 2 };

// Build with -DRFK_GEMM_TIMELINE to make CTA 0 of the pair kernel record %globaltimer stamps (ns) of its phases
// in a device array that rfk_gemm_timeline() reads back; compiled out otherwise.
#ifdef RFK_GEMM_TIMELINE
__device__ unsigned long long g_timeline[16];
#define RFK_STAMP(i) do { if (blockIdx.x == 0) g_timeline[i] = tc::global_timer_ns(); } while (0)
#else
#define RFK_STAMP(i) do { } while (0)
#endif

// Fourth epilogue of the pair kernel (own entry point, rfk_gemm_f16_heads): the output is stored head-split,
// [part][group][head][seq][64], through a rank-5 tile store, and every row's sum of squares over each 256-column
// tile (of the fp16-rounded values) is written to row_ss[part][row][tile] for the parts selected by ss_mask: the
// statistic of the QK-RMSNorm that follows the projection, so that the consumer can normalise while it loads.
constexpr int kEpiHeads = 3;

struct Params {
    __half* C; long long ldc;
    const __half* R; long long ldr;     // residual (EPI_RESIDUAL), may alias C
    const __half* bias;                 // [N] or null
    int M, N, K;                        // N = output columns
    int tiles_m, tiles_n;
    float* row_ss;                      // kEpiHeads: [parts][M][tiles per part] partial sums of squares, or null
    int seq, heads, ss_mask;            // kEpiHeads: rows per group, heads per part (64 wide), parts that get row_ss
};

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float2 unpack_half2(uint32_t w) {
    return __half22float2(*reinterpret_cast<__half2*>(&w));
}

// Tiled copy global -> shared of one box of a rank-2 tensor map (x innermost, in elements; x * 2 bytes
// is always a multiple of 128 here); the bytes are counted on `bar`.
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const void* tmap, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst_smem), "l"(tmap), "r"(x), "r"(y), "r"(tc::smem_addr(bar)) : "memory");
}

// Epilogue of one thread for one tile: the thread's accumulator row (tensor-memory address t_acc, BN_OUT output
// columns, for SwiGLU the up columns 128 further on) -> bias / residual / gate in fp32 -> fp16 -> global row `row`.
template <int EPI>
__device__ __forceinline__ void epilogue_tile(const Params& p, uint32_t t_acc, int row, int n0) {
    constexpr int BN_OUT = (EPI == RFK_GEMM_EPI_SWIGLU) ? 128 : 256;
    uint32_t v[32];
    const bool row_ok = row < p.M;
    __half* crow = p.C + (size_t)(row_ok ? row : 0) * p.ldc + n0;
    if (EPI == RFK_GEMM_EPI_SWIGLU) {
        uint32_t u[32];
#pragma unroll 1
        for (int c = 0; c < BN_OUT / 32; ++c) {
            tc::tmem_ld32(t_acc + c * 32, v);          // gate columns
            tc::tmem_ld32(t_acc + 128 + c * 32, u);    // up columns of the same hidden units
            tc::tc_wait_ld(v);
            tc::tc_wait_ld(u);
            uint32_t o[16];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                const float g0 = __uint_as_float(v[i]), g1 = __uint_as_float(v[i + 1]);
                // silu(g) * u = g * u / (1 + 2^(-g log2 e))
                const float s0 = g0 * fast_rcp(1.0f + fast_exp2(-1.4426950408889634f * g0));
                const float s1 = g1 * fast_rcp(1.0f + fast_exp2(-1.4426950408889634f * g1));
                o[i >> 1] = pack_half2(s0 * __uint_as_float(u[i]), s1 * __uint_as_float(u[i + 1]));
            }
            if (row_ok) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int col = n0 + c * 32 + q * 8;
                    if (col < p.N)
                        *reinterpret_cast<uint4*>(crow + c * 32 + q * 8) = make_uint4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
                }
            }
        }
    } else {
        const __half* rrow = (EPI == RFK_GEMM_EPI_RESIDUAL) ? p.R + (size_t)(row_ok ? row : 0) * p.ldr + n0 : nullptr;
        // The residual row is read two chunks ahead of its use (each thread reads 64 bytes of its own row per chunk:
        // the latency of these scattered loads, not their volume, is what an un-pipelined epilogue pays 8 times).
        constexpr int kAhead = 2;
        uint4 res[kAhead + 1][4];
        auto load_res = [&](int c) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int col = n0 + c * 32 + q * 8;
                res[c % (kAhead + 1)][q] = (row_ok && c < BN_OUT / 32 && col < p.N)
                                               ? *reinterpret_cast<const uint4*>(rrow + c * 32 + q * 8) : make_uint4(0, 0, 0, 0);
            }
        };
        if (EPI == RFK_GEMM_EPI_RESIDUAL) {
#pragma unroll
            for (int c = 0; c < kAhead; ++c) load_res(c);
        }
#pragma unroll
        for (int c = 0; c < BN_OUT / 32; ++c) {
            if (n0 + c * 32 >= p.N) break;             // uniform over the CTA: the tile's tail lies beyond N
            tc::tmem_ld32(t_acc + c * 32, v);
            if (EPI == RFK_GEMM_EPI_RESIDUAL) load_res(c + kAhead);
            tc::tc_wait_ld(v);
            if (p.bias) {
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    const int col = n0 + c * 32 + i;
                    if (col < p.N) {
                        const float2 b = unpack_half2(__ldg(reinterpret_cast<const uint32_t*>(p.bias + col)));
                        // the unfused path rounds the product to fp16 before the bias is added (linear.cu:15-25)
                        v[i] = __float_as_uint(round_half(__uint_as_float(v[i])) + b.x);
                        v[i + 1] = __float_as_uint(round_half(__uint_as_float(v[i + 1])) + b.y);
                    }
                }
            }
            uint32_t o[16];
            if (EPI == RFK_GEMM_EPI_RESIDUAL) {
                const uint32_t* rw = reinterpret_cast<const uint32_t*>(res[c % (kAhead + 1)]);
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float2 rr = unpack_half2(rw[i]);
                    o[i] = pack_half2(__uint_as_float(v[2 * i]) + rr.x, __uint_as_float(v[2 * i + 1]) + rr.y);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) o[i] = pack_half2(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
            }
            if (row_ok) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int col = n0 + c * 32 + q * 8;
                    if (col < p.N)
                        *reinterpret_cast<uint4*>(crow + c * 32 + q * 8) = make_uint4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
                }
            }
        }
    }
}

// out columns per tile: 256 (plain / residual) or 128 (SwiGLU: 128 gate + 128 up accumulator columns)
template <int EPI>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w0,
               const __grid_constant__ CUtensorMap map_w1, const Params p) {
    constexpr int BN_OUT = (EPI == RFK_GEMM_EPI_SWIGLU) ? 128 : 256;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const uint32_t base = tc::smem_addr(smem_raw);
    if (base & 1023u) {  // uniform over the CTA, nothing allocated yet
        if (threadIdx.x == 0) atomicCAS(&g_gemm_tc_error, 0, kErrSmemAlign);
        return;
    }
    Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem_raw + kStages * kStageBytes);
    volatile int* abort_flag = &ctrl->abort;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int num_kb = (p.K + BK - 1) / BK;
    const int num_tiles = p.tiles_m * p.tiles_n;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) { tc::mbar_init(&ctrl->full[s], 1); tc::mbar_init(&ctrl->empty[s], 1); }
        for (int a = 0; a < 2; ++a) { tc::mbar_init(&ctrl->acc_full[a], 1); tc::mbar_init(&ctrl->acc_empty[a], 4); }
        tc::mbar_init(&ctrl->drain, 1);
        ctrl->abort = 0;
        tc::fence_barrier_init();
    }
    if (warp == 0) {  // one warp allocates the CTA's tensor memory and later frees it
        tc::tmem_alloc(&ctrl->tmem_base, kTmemCols);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem_cta = ctrl->tmem_base;
    pdl_wait();      // set-up above is on-chip only; the operands are another kernel's output
    pdl_trigger();

    if (warp == 0) {
        // ------------------------------------------------------------ producer (one thread)
        if (lane == 0) {
            tc::prefetch_tensormap(&map_a); tc::prefetch_tensormap(&map_w0); tc::prefetch_tensormap(&map_w1);
            int it = 0;       // K blocks issued so far by this CTA, over all of its tiles
            bool ok = true;
            for (int t = blockIdx.x; ok && t < num_tiles; t += gridDim.x) {
                const int m0 = (t % p.tiles_m) * BM, n0 = (t / p.tiles_m) * BN_OUT;
                // second weight box: the next 128 rows of W, or the up-projection rows of the same hidden units
                const int n1 = (EPI == RFK_GEMM_EPI_SWIGLU) ? n0 : n0 + 128;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % kStages;
                    // stage s was last read by the products of K block it - kStages
                    if (it >= kStages && !tc::mbar_wait(&ctrl->empty[s], ((it / kStages) + 1) & 1, abort_flag)) { ok = false; break; }
                    const uint32_t sA = base + s * kStageBytes;
                    tc::mbar_arrive_expect_tx(&ctrl->full[s], kStageBytes);
                    tma_load_2d(sA, &map_a, kb * BK, m0, &ctrl->full[s]);
                    tma_load_2d(sA + kABytes, &map_w0, kb * BK, n0, &ctrl->full[s]);
                    tma_load_2d(sA + kABytes + kWBoxBytes, &map_w1, kb * BK, n1, &ctrl->full[s]);
                }
            }
            if (*abort_flag) {
                // The CTA is giving up: every copy this thread started lands in this CTA's shared memory and counts on a
                // full[] barrier; wait (bounded) for the last copy of each stage before the CTA exits.
                for (int s = 0; s < kStages && s < it; ++s) {
                    const int last = ((it - 1 - s) / kStages) * kStages + s;
                    tc::mbar_wait_drain(&ctrl->full[s], (last / kStages) & 1);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ issuer of the products (one thread)
        if (lane == 0) {
            constexpr uint32_t idesc = tc::umma_idesc_f16(BM, BNACC, 0);  // A and B both K-major
            int it = 0, tl = 0;  // K blocks and tiles consumed so far
            bool ok = true;
            for (int t = blockIdx.x; ok && t < num_tiles; t += gridDim.x, ++tl) {
                const int acc = tl & 1;
                // the epilogue must have drained this accumulator's previous tile (tile tl - 2)
                if (tl >= 2) ok = tc::mbar_wait(&ctrl->acc_empty[acc], ((tl >> 1) + 1) & 1, abort_flag);
                if (!ok) break;
                tc::tc_fence_after();
                const uint32_t d_tmem = tmem_cta + acc * BNACC;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % kStages;
                    ok = tc::mbar_wait(&ctrl->full[s], (it / kStages) & 1, abort_flag);
                    if (!ok) break;
                    tc::tc_fence_after();
                    const uint32_t a_lo = tc::umma_desc_lo(base + s * kStageBytes);
                    const uint32_t b_lo = tc::umma_desc_lo(base + s * kStageBytes + kABytes);
#pragma unroll
                    for (int ks = 0; ks < BK / 16; ++ks)  // 16 halves = 32 bytes along a swizzled row
                        tc::umma_f16_lo(d_tmem, a_lo + ks * 2, b_lo + ks * 2, idesc, (kb > 0) || (ks > 0));
                    tc::umma_commit(&ctrl->empty[s]);     // the stage is free once these products have read it
                }
                if (ok) tc::umma_commit(&ctrl->acc_full[acc]);
            }
            if (*abort_flag) {  // giving up: let this thread's products finish before tensor memory is freed
                tc::umma_commit(&ctrl->drain);
                tc::mbar_wait_drain(&ctrl->drain, 0);
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ epilogue, warps 2-5
        const int lane_grp = warp & 3;                        // a warp reaches tensor-memory lanes [32 * (warp % 4), +32)
        const int r = lane_grp * 32 + lane;                   // row within the tile
        const uint32_t lane_off = (uint32_t)(lane_grp * 32) << 16;
        bool ok = true;
        int tl = 0;
        for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++tl) {
            const int acc = tl & 1;
            const int m0 = (t % p.tiles_m) * BM, n0 = (t / p.tiles_m) * BN_OUT;
            ok = tc::mbar_wait_warp(&ctrl->acc_full[acc], (tl >> 1) & 1, abort_flag);
            if (!ok) break;
            tc::tc_fence_after();
            epilogue_tile<EPI>(p, tmem_cta + lane_off + acc * BNACC, m0 + r, n0);
            // every tcgen05.ld of this warp has completed (wait::ld above): hand the accumulator back
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&ctrl->acc_empty[acc]);
        }
    }

    // ---- teardown: every path (normal or aborted) arrives here with no divergence inside a warp
    tc::tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc::tc_fence_after();
        tc::tmem_dealloc(tmem_cta, kTmemCols);
    }
    if (tid == 0 && ctrl->abort) atomicCAS(&g_gemm_tc_error, 0, kErrTimeout);
}

// ------------------------------------------------------------------------------------------------
// The same product on CTA pairs: a cluster of two CTAs (two SMs of one TPC) owns a tile of 256 rows x 256
// accumulator columns and one thread of the pair's first CTA issues tcgen05.mma.cta_group::2 (M = 256):
// each CTA stages only ITS 128 rows of A and ITS half of the weight tile (128 of the 256 accumulator
// columns' rows; with the SwiGLU epilogue CTA 0 holds the gate rows and CTA 1 the up rows), so a K block
// costs each SM 32 KB of L2 -> shared-memory traffic instead of 48 KB for the same number of products.
// That traffic, not the tensor pipe, bounds the single-CTA kernel above (the same ~510 ns per K block on
// every shape = 14 TB/s over 148 SMs). Both accumulator halves live in the two CTAs' tensor memories at the
// same address; each CTA's epilogue warps drain their own 128 rows.
//   barriers: full[s] in CTA 0 collects both CTAs' copies (one arrive.expect_tx of 64 KB by CTA 0); empty[s] and
//   acc_full[a] exist in both CTAs and are signalled together by one multicast tcgen05.commit;
//   acc_empty[a] in CTA 0 counts the 8 epilogue warps of the pair.
// The copies are ordinary per-CTA TMA loads (no cluster multicast), with the .cta_group::2 form that lets
// CTA 1's copies count on CTA 0's barrier.
namespace pair {

constexpr int kStageBytes = kABytes + kWBoxBytes;   // 32 KB per CTA
// The epilogue goes through shared memory both ways: an epilogue warp owns staging buffers of 32 rows x 64 halves
// (4 KB, the 128-byte-swizzled layout of a TMA box) for its 32 rows of the tile; it writes the finished fp16 values
// of 64 output columns there and one lane issues a TMA tile store, so the global writes are whole 128-byte lines
// issued by the copy engine instead of 16-byte pieces of 32 different rows per store instruction (measured:
// 2.8 us per tile for the register-to-global epilogue, most of it the scattered stores). With the residual
// epilogue the same buffers first receive the residual tile by TMA loads issued before the accumulator is ready
// (one buffer per 64-column unit, so the loads of a whole tile are in flight during its main loop); the sum
// overwrites the residual in place and is stored from there. Plain / SwiGLU: two buffers per warp in turn.
constexpr int kUnitCols = 64;
constexpr int kUnitBytes = 32 * kUnitCols * 2;       // 4 KB
template <int EPI> struct Cfg {
    static constexpr int kUnits = (EPI == RFK_GEMM_EPI_SWIGLU) ? 2 : 4;                    // 64-column units per tile
    static constexpr int kBufsPerWarp = (EPI == RFK_GEMM_EPI_RESIDUAL) ? 4 : 2;
    static constexpr int kStagingBytes = 4 * kBufsPerWarp * kUnitBytes;                      // 4 epilogue warps
    static constexpr int kStages = (EPI == RFK_GEMM_EPI_RESIDUAL) ? 5 : 6;
    static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + 512;
    static_assert(kSmemBytes + 1024 <= 227 * 1024, "one CTA per SM");
};
constexpr int kMaxStages = 6;

struct __align__(8) Ctrl {
    uint64_t full[kMaxStages], empty[kMaxStages], acc_full[2], acc_empty[2], drain;
    uint64_t res_full[4][4];   // residual epilogue: [epilogue warp][unit], completes when that unit's residual box has landed
    uint32_t tmem_base;
    int abort;
};
static_assert(sizeof(Ctrl) <= 512, "control block");

// ---- shared <-> global tile copies used by the epilogue
__device__ __forceinline__ void tma_store_2d(const void* tmap, uint32_t src_smem, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(tmap), "r"(src_smem), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_store_5d(const void* tmap, uint32_t src_smem, int c0, int c1, int c2, int c3, int c4) {
    asm volatile("cp.async.bulk.tensor.5d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5, %6}], [%1];"
                 ::"l"(tmap), "r"(src_smem), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// waits until at most N of this thread's committed store groups still READ their shared-memory source
template <int N> __device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the location `smem_addr` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void remote_arrive(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void remote_arrive_expect_tx(uint32_t cluster_bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.release.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_bar), "r"(bytes) : "memory");
}
// per-CTA tiled copy whose bytes are counted on a barrier that may live in the pair's other CTA
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst_smem, const void* tmap, int x, int y, uint32_t cluster_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst_smem), "l"(tmap), "r"(x), "r"(y), "r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void umma_pair_f16_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %5};\n\t"
        "mov.b64 db, {%2, %5};\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(tc::kDescHiSw128) : "memory");
}
// one arrival on the barrier at this shared-memory offset in BOTH CTAs of the pair when every product issued so far is complete
__device__ __forceinline__ void umma_pair_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(tc::smem_addr(bar)), "h"((uint16_t)3) : "memory");
}
// bounded pause on the abort path: lets copies that were started a moment ago land
__device__ __forceinline__ void drain_pause() {
    const uint64_t t0 = tc::global_timer_ns();
    for (int i = 0; i < 4096 && tc::global_timer_ns() - t0 < 50000; ++i) __nanosleep(256);
}

// Byte offset of 16-byte chunk j (0..7) of row r (0..31) inside a staging buffer (SWIZZLE_128B box layout).
__device__ __forceinline__ uint32_t staged(int r, int j) { return (uint32_t)(r * 128 + ((j ^ (r & 7)) << 4)); }

// Residual epilogue, before the tile's accumulator is waited for: bring the warp's residual rows of the whole tile
// into its four staging buffers. Lane 0 only. The buffers were last read by the TMA stores of the previous tile.
template <int EPI>
__device__ __forceinline__ void epilogue_prefetch_residual(const CUtensorMap* map_r, uint32_t stage_base, uint64_t* res_full,
                                                           int row0, int n0) {
    if (EPI != RFK_GEMM_EPI_RESIDUAL) return;
    bulk_wait_read<0>();
#pragma unroll
    for (int u = 0; u < 4; ++u) {   // units beyond N are loaded too (all zeros): every barrier sees one phase per tile
        tc::mbar_arrive_expect_tx(&res_full[u], kUnitBytes);
        tma_load_2d(stage_base + u * kUnitBytes, map_r, n0 + u * kUnitCols, row0, &res_full[u]);
    }
}

// One epilogue warp, one tile: accumulator rows [lane] -> (bias / residual / gate) -> fp16 -> staging buffer -> TMA store.
// t_acc: tensor-memory address of the thread's accumulator row; row0: global row of the warp's lane 0.
template <int EPI>
__device__ __forceinline__ bool epilogue_tile_staged(const Params& p, const CUtensorMap* map_c, uint32_t t_acc,
                                                     unsigned char* stage_ptr, uint64_t* res_full, uint32_t res_parity,
                                                     int row0, int n0, int lane, volatile int* abort_flag) {
    constexpr int kUnits = Cfg<EPI>::kUnits;
    const uint32_t stage_base = tc::smem_addr(stage_ptr);
    uint32_t v[32];
    float ss = 0.0f;   // kEpiHeads: this row's sum of squares over the tile
#pragma unroll 1
    for (int u = 0; u < kUnits; ++u) {
        const int b = (EPI == RFK_GEMM_EPI_RESIDUAL) ? u : (u & 1);
        unsigned char* buf = stage_ptr + b * kUnitBytes;
        if (EPI == RFK_GEMM_EPI_RESIDUAL) {                 // this unit's residual box has landed (also for units beyond N)
            if (!tc::mbar_wait_warp(&res_full[u], res_parity, abort_flag)) return false;
        }

        if (n0 + u * kUnitCols >= p.N) continue;            // uniform: the tile's tail lies beyond N
        if (EPI != RFK_GEMM_EPI_RESIDUAL) {                 // the store issued two units ago must have read this buffer
            if (lane == 0) bulk_wait_read<1>();
            __syncwarp();
        }
#pragma unroll
        for (int hc = 0; hc < 2; ++hc) {                    // two half units of 32 output columns
            const int c32 = u * 2 + hc;                     // 32-column chunk index within the tile's output
            uint32_t o[16];
            if (EPI == RFK_GEMM_EPI_SWIGLU) {
                uint32_t up[32];
                tc::tmem_ld32(t_acc + c32 * 32, v);          // gate columns
                tc::tmem_ld32(t_acc + 128 + c32 * 32, up);   // up columns of the same hidden units
                tc::tc_wait_ld(v);
                tc::tc_wait_ld(up);
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    const float g0 = __uint_as_float(v[i]), g1 = __uint_as_float(v[i + 1]);
                    // silu(g) * u = g * u / (1 + 2^(-g log2 e))
                    const float s0 = g0 * fast_rcp(1.0f + fast_exp2(-1.4426950408889634f * g0));
                    const float s1 = g1 * fast_rcp(1.0f + fast_exp2(-1.4426950408889634f * g1));
                    o[i >> 1] = pack_half2(s0 * __uint_as_float(up[i]), s1 * __uint_as_float(up[i + 1]));
                }
            } else {
                tc::tmem_ld32(t_acc + c32 * 32, v);
                uint4 res[4];
                if (EPI == RFK_GEMM_EPI_RESIDUAL) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) res[q] = *reinterpret_cast<const uint4*>(buf + staged(lane, hc * 4 + q));
                }
                tc::tc_wait_ld(v);
                if (p.bias) {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const int col = n0 + c32 * 32 + i;
                        if (col < p.N) {
                            const float2 bb = unpack_half2(__ldg(reinterpret_cast<const uint32_t*>(p.bias + col)));
                            // the unfused path rounds the product to fp16 before the bias is added (linear.cu:15-25)
                            v[i] = __float_as_uint(round_half(__uint_as_float(v[i])) + bb.x);
                            v[i + 1] = __float_as_uint(round_half(__uint_as_float(v[i + 1])) + bb.y);
                        }
                    }
                }
                if (EPI == RFK_GEMM_EPI_RESIDUAL) {
                    const uint32_t* rw = reinterpret_cast<const uint32_t*>(res);
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float2 rr = unpack_half2(rw[i]);
                        o[i] = pack_half2(__uint_as_float(v[2 * i]) + rr.x, __uint_as_float(v[2 * i + 1]) + rr.y);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) o[i] = pack_half2(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
                    if (EPI == kEpiHeads) {   // the norm that follows sees the stored fp16 values
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const float2 r2 = unpack_half2(o[i]);
                            ss = fmaf(r2.x, r2.x, ss);
                            ss = fmaf(r2.y, r2.y, ss);
                        }
                    }
                }
            }
#pragma unroll
            for (int q = 0; q < 4; ++q)
                *reinterpret_cast<uint4*>(buf + staged(lane, hc * 4 + q)) = make_uint4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
        }
        tc::fence_proxy_async();                            // the copy engine reads what the threads just wrote
        __syncwarp();
        if (lane == 0) {
            if (EPI == kEpiHeads) {
                const int g = (n0 + u * kUnitCols) / kUnitCols;   // 64-wide head index over all parts
                tma_store_5d(map_c, stage_base + b * kUnitBytes, 0, row0 % p.seq, g % p.heads, row0 / p.seq, g / p.heads);
            } else {
                tma_store_2d(map_c, stage_base + b * kUnitBytes, n0 + u * kUnitCols, row0);   // rows >= M, columns >= N are clipped
            }
            bulk_commit();
        }
    }
    if (EPI == kEpiHeads && p.row_ss) {
        const int dim = p.heads * kUnitCols, part = n0 / dim, row = row0 + lane;
        if (((p.ss_mask >> part) & 1) && row < p.M)
            p.row_ss[((size_t)part * p.M + row) * (dim / 256) + (n0 % dim) / 256] = ss;
    }
    return true;
}

template <int EPI>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w0,
                    const __grid_constant__ CUtensorMap map_w1, const __grid_constant__ CUtensorMap map_c,
                    const __grid_constant__ CUtensorMap map_r, const Params p) {
    constexpr int BN_OUT = (EPI == RFK_GEMM_EPI_SWIGLU) ? 128 : 256;
    constexpr int kStages = Cfg<EPI>::kStages;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const uint32_t base = tc::smem_addr(smem_raw);
    const uint32_t rank = cluster_rank();            // 0: issues the products for the pair; 1: its peer
    unsigned char* staging = smem_raw + kStages * kStageBytes;   // 1024-byte aligned: the stages are 32 KB each
    Ctrl* ctrl = reinterpret_cast<Ctrl*>(staging + Cfg<EPI>::kStagingBytes);
    volatile int* abort_flag = &ctrl->abort;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) RFK_STAMP(0);   // kernel entry
    const int num_kb = (p.K + BK - 1) / BK;
    const int num_tiles = p.tiles_m * p.tiles_n;      // pair tiles: tiles_m counts 256-row blocks
    const int first_tile = blockIdx.x >> 1, tile_step = gridDim.x >> 1;
    const bool aligned = (base & 1023u) == 0;         // the same in both CTAs (same kernel, same shared-memory layout)
    auto wait = [&](uint64_t* bar, uint32_t parity) { return tc::mbar_wait(bar, parity, abort_flag); };

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) { tc::mbar_init(&ctrl->full[s], 1); tc::mbar_init(&ctrl->empty[s], 1); }
        for (int a = 0; a < 2; ++a) { tc::mbar_init(&ctrl->acc_full[a], 1); tc::mbar_init(&ctrl->acc_empty[a], 8); }
        tc::mbar_init(&ctrl->drain, 1);
        for (int w = 0; w < 4; ++w)
            for (int u = 0; u < 4; ++u) tc::mbar_init(&ctrl->res_full[w][u], 1);
        ctrl->abort = 0;
        tc::fence_barrier_init();
    }
    if (warp == 0 && aligned) {  // each CTA allocates its own tensor memory (all 512 columns: both get the same address)
        tc::tmem_alloc(&ctrl->tmem_base, kTmemCols);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before();
    __syncthreads();
    cluster_sync();              // both CTAs' barriers are initialised before either signals the other
    tc::tc_fence_after();
    if (!aligned) {
        if (tid == 0) atomicCAS(&g_gemm_tc_error, 0, kErrSmemAlign);
        return;
    }
    const uint32_t tmem_cta = ctrl->tmem_base;
    pdl_wait();      // set-up above is on-chip only; the operands are another kernel's output
    pdl_trigger();
    if (tid == 0) RFK_STAMP(1);   // prologue done (barriers, tensor memory, cluster barrier)

    if (warp == 0) {
        // ------------------------------------------------------------ producer (one thread per CTA)
        if (lane == 0) {
            const void* map_w = rank == 0 ? (const void*)&map_w0 : (const void*)&map_w1;
            tc::prefetch_tensormap(&map_a); tc::prefetch_tensormap(map_w); tc::prefetch_tensormap(&map_c);
            if (EPI == RFK_GEMM_EPI_RESIDUAL) tc::prefetch_tensormap(&map_r);
            int it = 0;
            bool ok = true;
            for (int t = first_tile; ok && t < num_tiles; t += tile_step) {
                const int m0 = (t % p.tiles_m) * (2 * BM) + (int)rank * BM, n0 = (t / p.tiles_m) * BN_OUT;
                // this CTA's half of the weight tile: rows n0.. (CTA 0) / n0+128.. (CTA 1) of W, or the gate / up rows
                const int nw = (EPI == RFK_GEMM_EPI_SWIGLU || rank == 0) ? n0 : n0 + 128;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % kStages;
                    if (it >= kStages && !wait(&ctrl->empty[s], ((it / kStages) + 1) & 1)) { ok = false; break; }
                    const uint32_t sA = base + s * kStageBytes;
                    const uint32_t full0 = map_to_cta(tc::smem_addr(&ctrl->full[s]), 0);
                    // CTA 0 announces the bytes of both CTAs' copies on its own barrier (one local arrival); CTA 1 only
                    // copies. CTA 1's bytes may land before CTA 0's announcement: the phase still cannot complete before
                    // that arrival, and the transaction count balances once it is made.
                    if (rank == 0) tc::mbar_arrive_expect_tx(&ctrl->full[s], 2 * kStageBytes);
                    tma_load_2d_pair(sA, &map_a, kb * BK, m0, full0);
                    tma_load_2d_pair(sA + kABytes, map_w, kb * BK, nw, full0);
                }
            }
            if (*abort_flag) drain_pause();   // this CTA's copies count on CTA 0's barriers: give them time to land
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ issuer of the pair's products (one thread of CTA 0)
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = tc::umma_idesc_f16(2 * BM, BNACC, 0);
            int it = 0, tl = 0;
            bool ok = true;
            for (int t = first_tile; ok && t < num_tiles; t += tile_step, ++tl) {
                const int acc = tl & 1;
                if (tl >= 2) ok = wait(&ctrl->acc_empty[acc], ((tl >> 1) + 1) & 1);
                if (!ok) break;
                tc::tc_fence_after();
                const uint32_t d_tmem = tmem_cta + acc * BNACC;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % kStages;
                    ok = wait(&ctrl->full[s], (it / kStages) & 1);
                    if (!ok) break;
                    if (it == 0) RFK_STAMP(2);   // first K block has landed
                    tc::tc_fence_after();
                    const uint32_t a_lo = tc::umma_desc_lo(base + s * kStageBytes);
                    const uint32_t b_lo = tc::umma_desc_lo(base + s * kStageBytes + kABytes);
#pragma unroll
                    for (int ks = 0; ks < BK / 16; ++ks)
                        umma_pair_f16_lo(d_tmem, a_lo + ks * 2, b_lo + ks * 2, idesc, (kb > 0) || (ks > 0));
                    umma_pair_commit(&ctrl->empty[s]);
                }
                if (ok) umma_pair_commit(&ctrl->acc_full[acc]);
                if (tl == 0) RFK_STAMP(3);       // all products of the first tile issued
            }
            if (*abort_flag) {
                umma_pair_commit(&ctrl->drain);
                tc::mbar_wait_drain(&ctrl->drain, 0);
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ epilogue, warps 2-5 of both CTAs
        const int lane_grp = warp & 3;                        // a warp reaches tensor-memory lanes [32 * (warp % 4), +32)
        const uint32_t lane_off = (uint32_t)(lane_grp * 32) << 16;
        unsigned char* my_stage = staging + lane_grp * Cfg<EPI>::kBufsPerWarp * kUnitBytes;
        uint64_t* my_res = ctrl->res_full[lane_grp];
        bool ok = true;
        int tl = 0;
        for (int t = first_tile; t < num_tiles; t += tile_step, ++tl) {
            const int acc = tl & 1;
            const int m0 = (t % p.tiles_m) * (2 * BM) + (int)rank * BM, n0 = (t / p.tiles_m) * BN_OUT;
            const int row0 = m0 + lane_grp * 32;
            if (lane == 0) {
                // The residual boxes of the CTA's first tile are asked for only once the first K block has been consumed
                // (first multicast commit): issued at kernel start they delay the first operand tiles by ~0.5 us.
                if (EPI == RFK_GEMM_EPI_RESIDUAL && tl == 0) tc::mbar_wait(&ctrl->empty[0], 0, abort_flag);
                epilogue_prefetch_residual<EPI>(&map_r, tc::smem_addr(my_stage), my_res, row0, n0);
            }
            ok = tc::mbar_wait_warp(&ctrl->acc_full[acc], (tl >> 1) & 1, abort_flag);
            if (!ok) break;
            tc::tc_fence_after();
            if (tl == 0 && warp == 2 && lane == 0) RFK_STAMP(4);   // first tile's accumulator complete
            ok = epilogue_tile_staged<EPI>(p, &map_c, tmem_cta + lane_off + acc * BNACC, my_stage, my_res, tl & 1, row0, n0,
                                           lane, abort_flag);
            if (!ok) break;
            if (tl == 0 && warp == 2 && lane == 0) RFK_STAMP(5);   // its epilogue done (stores issued)
            // every tcgen05.ld of this warp has completed: hand the accumulator back
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) remote_arrive(map_to_cta(tc::smem_addr(&ctrl->acc_empty[acc]), 0));
        }
        // this lane's stores must have left shared memory (and, on an aborted run, its residual loads landed) before
        // the CTA gives the memory up
        if (lane == 0) {
            if (*abort_flag) drain_pause();
            bulk_wait_read<0>();   // the stores themselves complete with the grid; shared memory only has to outlive their reads
        }
        __syncwarp();
    }

    // ---- teardown: neither CTA leaves while the other may still signal its barriers or read its shared memory
    tc::tc_fence_before();
    __syncthreads();
    cluster_sync();
    if (warp == 0) {
        tc::tc_fence_after();
        tc::tmem_dealloc(tmem_cta, kTmemCols);
    }
    if (tid == 0 && ctrl->abort) atomicCAS(&g_gemm_tc_error, 0, kErrTimeout);
    if (tid == 0) RFK_STAMP(6);   // CTA exit
}

}  // namespace pair
}  // namespace tcgemm

// 0 automatic (tcgen05 kernel on CTA pairs when the shape allows), 1 never (callers use their library GEMM), 2 as 0,
// 3 the single-CTA tcgen05 kernel. The
// environment variable RFK_GEMM_PATH sets the initial value, for side-by-side runs of an unchanged program.
static int initial_gemm_path() {
    const char* e = getenv("RFK_GEMM_PATH");
    return (e && e[0] >= '0' && e[0] <= '3' && e[1] == 0) ? e[0] - '0' : 0;
}
std::atomic<int> g_gemm_path{initial_gemm_path()};

namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled, taken from the driver the runtime already has loaded (no link against libcuda)
EncodeTiledFn tensor_map_encoder() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// fp16 matrix [rows][cols] with a row pitch of ld elements; boxes of 128 rows x 64 columns in the
// 128-byte-swizzled layout; elements outside the matrix read as zeros
bool make_map_2d(CUtensorMap* m, const void* base, long long rows, long long cols, long long ld, int box_rows = 128) {
    EncodeTiledFn enc = tensor_map_encoder();
    if (!enc) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int EPI>
int launch_gemm_single(const CUtensorMap& ma, const CUtensorMap& mw0, const CUtensorMap& mw1, tcgemm::Params p, int dev,
                       cudaStream_t st) {
    static std::atomic<bool> configured[64];
    static std::atomic<int> sm_count[64];
    if (!configured[dev].load(std::memory_order_acquire)) {
        cudaError_t e = cudaFuncSetAttribute(tcgemm::gemm_tc_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             tcgemm::kSmemBytes);
        if (e != cudaSuccess) return (int)e;
        int n = 0;
        e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return (int)e;
        sm_count[dev].store(n, std::memory_order_relaxed);
        configured[dev].store(true, std::memory_order_release);
    }
    const int tiles = p.tiles_m * p.tiles_n;
    const int grid = std::min(tiles, std::max(1, sm_count[dev].load(std::memory_order_relaxed)));
    launch_pdl(tcgemm::gemm_tc_kernel<EPI>, dim3(grid), dim3(tcgemm::kThreads), tcgemm::kSmemBytes, st, ma, mw0, mw1, p);
    return launch_status();
}

std::atomic<int> g_pair_clusters[64];  // CTA pairs the device can run at once, per device (0 not asked yet, -1 none)

// CTA-pair kernel: clusters of two; returns RFK_EUNSUPPORTED (nothing launched) when the device cannot co-schedule pairs
template <int EPI>
int launch_gemm_pair(const CUtensorMap& ma, const CUtensorMap& mw0, const CUtensorMap& mw1, tcgemm::Params p, int dev,
                     cudaStream_t st, const CUtensorMap* heads_map = nullptr) {
    // tile maps of the output (stores) and of the residual (loads): boxes of 32 rows x 64 columns, one per epilogue warp
    CUtensorMap mc, mr;
    if (heads_map) mc = *heads_map;
    if ((!heads_map && !make_map_2d(&mc, p.C, p.M, p.N, p.ldc, 32)) ||
        !make_map_2d(&mr, EPI == RFK_GEMM_EPI_RESIDUAL ? (const void*)p.R : (const void*)p.C, p.M, p.N,
                     EPI == RFK_GEMM_EPI_RESIDUAL ? p.ldr : p.ldc, 32))
        return RFK_EUNSUPPORTED;
    constexpr int kSmem = tcgemm::pair::Cfg<EPI>::kSmemBytes;
    std::atomic<int>* max_clusters = g_pair_clusters;   // 0 not asked yet, -1 unavailable
    static std::atomic<bool> configured[64];            // per instantiation of the kernel
    cudaLaunchConfig_t cfg{};
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // see launch_pdl in common.cuh
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.blockDim = dim3(tcgemm::kThreads); cfg.dynamicSmemBytes = kSmem; cfg.stream = st;
    cfg.attrs = attr; cfg.numAttrs = 1;
    int nc = max_clusters[dev].load(std::memory_order_acquire);
    if (nc == 0 || !configured[dev].load(std::memory_order_acquire)) {
        cudaError_t e = cudaFuncSetAttribute(tcgemm::pair::gemm_tc_pair_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             kSmem);
        if (e != cudaSuccess) return (int)e;
        int sms = 0;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return (int)e;
        cfg.gridDim = dim3(2 * std::max(1, sms / 2));
        int n = 0;
        e = cudaOccupancyMaxActiveClusters(&n, tcgemm::pair::gemm_tc_pair_kernel<EPI>, &cfg);
        if (e != cudaSuccess) { cudaGetLastError(); n = 0; }
        nc = n > 0 ? std::min(n, sms / 2) : -1;
        max_clusters[dev].store(nc, std::memory_order_release);
        configured[dev].store(true, std::memory_order_release);
    }
    if (nc < 0) return RFK_EUNSUPPORTED;
    p.tiles_m = (p.M + 2 * tcgemm::BM - 1) / (2 * tcgemm::BM);
    const int tiles = p.tiles_m * p.tiles_n;
    cfg.gridDim = dim3(2 * std::min(tiles, nc));
    cfg.numAttrs = g_pdl_enabled ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, tcgemm::pair::gemm_tc_pair_kernel<EPI>, ma, mw0, mw1, mc, mr, p);
    if (e != cudaSuccess) { cudaGetLastError(); return (int)e; }
    return launch_status();
}

// rank-5 map of a head-split output: [part][group][head][seq][64] halves, boxes of 32 rows x 64 columns
bool make_map_heads(CUtensorMap* m, const void* base, int seq, int heads, long long groups, int parts, long long part_stride) {
    EncodeTiledFn enc = tensor_map_encoder();
    if (!enc) return false;
    const cuuint64_t dims[5] = {64, (cuuint64_t)seq, (cuuint64_t)heads, (cuuint64_t)groups, (cuuint64_t)parts};
    const cuuint64_t strides[4] = {128, (cuuint64_t)seq * 128, (cuuint64_t)heads * seq * 128, (cuuint64_t)part_stride * 2};
    const cuuint32_t box[5] = {64, 32, 1, 1, 1};
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// path 0 / 2: CTA pairs, the single-CTA kernel if pairs are unavailable; path 3: the single-CTA kernel
template <int EPI>
int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mw0, const CUtensorMap& mw1, const tcgemm::Params& p, int dev,
                cudaStream_t st) {
    if (g_gemm_path.load(std::memory_order_relaxed) != 3) {
        const int rc = launch_gemm_pair<EPI>(ma, mw0, mw1, p, dev, st);
        if (rc != RFK_EUNSUPPORTED) return rc;
    }
    return launch_gemm_single<EPI>(ma, mw0, mw1, p, dev, st);
}

}  // namespace
}  // namespace rfk

using namespace rfk;

extern "C" int rfk_gemm_f16(const rfk_half* A, long long lda, const rfk_half* W, long long ldw, const rfk_half* W_up,
                            const rfk_half* bias, const rfk_half* R, long long ldr, rfk_half* C, long long ldc, int M,
                            int N, int K, int epilogue, rfk_stream_t stream) {
    if (!A || !W || !C || M < 0 || N <= 0 || K <= 0) return RFK_EINVAL;
    if (epilogue < RFK_GEMM_EPI_NONE || epilogue > RFK_GEMM_EPI_SWIGLU) return RFK_EINVAL;
    if (epilogue == RFK_GEMM_EPI_SWIGLU && (!W_up || bias)) return RFK_EINVAL;
    if (epilogue == RFK_GEMM_EPI_RESIDUAL && !R) return RFK_EINVAL;
    if (lda < K || ldw < K || ldc < N || (epilogue == RFK_GEMM_EPI_RESIDUAL && ldr < N)) return RFK_EINVAL;
    if (M == 0) return RFK_OK;
    if (g_gemm_path.load(std::memory_order_relaxed) == 1) return RFK_EUNSUPPORTED;
    // TMA needs 16-byte aligned bases and pitches; the epilogue moves 8 halves per access
    if ((lda | ldw | ldc | (epilogue == RFK_GEMM_EPI_RESIDUAL ? ldr : 0)) % 8 != 0 || N % 8 != 0 || K % 8 != 0)
        return RFK_EUNSUPPORTED;
    if (!aligned16(A) || !aligned16(W) || !aligned16(C) || (W_up && !aligned16(W_up)) || (R && !aligned16(R)) ||
        (bias && (reinterpret_cast<uintptr_t>(bias) & 3u)))
        return RFK_EUNSUPPORTED;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return RFK_EUNSUPPORTED;
    CUtensorMap ma, mw0, mw1;
    const bool swiglu = epilogue == RFK_GEMM_EPI_SWIGLU;
    if (!make_map_2d(&ma, A, M, K, lda) || !make_map_2d(&mw0, W, N, K, ldw) ||
        !make_map_2d(&mw1, swiglu ? W_up : W, N, K, ldw))
        return RFK_EUNSUPPORTED;
    tcgemm::Params p{};
    p.C = (__half*)C; p.ldc = ldc; p.R = (const __half*)R; p.ldr = ldr; p.bias = (const __half*)bias;
    p.M = M; p.N = N; p.K = K;
    p.tiles_m = (M + tcgemm::BM - 1) / tcgemm::BM;
    p.tiles_n = (N + (swiglu ? 128 : 256) - 1) / (swiglu ? 128 : 256);
    cudaStream_t st = as_stream(stream);
    switch (epilogue) {
        case RFK_GEMM_EPI_NONE: return launch_gemm<RFK_GEMM_EPI_NONE>(ma, mw0, mw1, p, dev, st);
        case RFK_GEMM_EPI_RESIDUAL: return launch_gemm<RFK_GEMM_EPI_RESIDUAL>(ma, mw0, mw1, p, dev, st);
        default: return launch_gemm<RFK_GEMM_EPI_SWIGLU>(ma, mw0, mw1, p, dev, st);
    }
}

extern "C" int rfk_gemm_f16_heads(const rfk_half* A, long long lda, const rfk_half* W, long long ldw, rfk_half* out,
                                  long long part_stride, float* row_ss, int ss_parts_mask, int M, int N, int K, int seq_len,
                                  int num_heads, rfk_stream_t stream) {
    if (!A || !W || !out || M < 0 || N <= 0 || K <= 0 || seq_len <= 0 || num_heads <= 0 || lda < K || ldw < K) return RFK_EINVAL;
    const int dim = num_heads * 64;
    if (N % dim != 0 || (ss_parts_mask && !row_ss)) return RFK_EINVAL;
    const int parts = N / dim;
    if (parts > 1 && part_stride < (long long)M * dim) return RFK_EINVAL;
    if (M == 0) return RFK_OK;
    const int path = g_gemm_path.load(std::memory_order_relaxed);
    if (path == 1 || path == 3) return RFK_EUNSUPPORTED;   // pair kernel only
    // a 256-column tile must lie inside one part, a 32-row store box inside one group
    if (dim % 256 != 0 || seq_len % 32 != 0 || M % seq_len != 0) return RFK_EUNSUPPORTED;
    if ((lda | ldw | part_stride) % 8 != 0 || K % 8 != 0 || !aligned16(A) || !aligned16(W) || !aligned16(out) ||
        (row_ss && !aligned16(row_ss)))
        return RFK_EUNSUPPORTED;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return RFK_EUNSUPPORTED;
    CUtensorMap ma, mw, mh;
    if (!make_map_2d(&ma, A, M, K, lda) || !make_map_2d(&mw, W, N, K, ldw) ||
        !make_map_heads(&mh, out, seq_len, num_heads, M / seq_len, parts, parts > 1 ? part_stride : (long long)M * dim))
        return RFK_EUNSUPPORTED;
    tcgemm::Params p{};
    p.C = (__half*)out; p.ldc = N; p.M = M; p.N = N; p.K = K;
    p.tiles_m = (M + tcgemm::BM - 1) / tcgemm::BM;
    p.tiles_n = N / 256;
    p.row_ss = row_ss; p.seq = seq_len; p.heads = num_heads; p.ss_mask = ss_parts_mask;
    return launch_gemm_pair<tcgemm::kEpiHeads>(ma, mw, mw, p, dev, as_stream(stream), &mh);
}

extern "C" int rfk_gemm_pair_clusters(void) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    return g_pair_clusters[dev].load(std::memory_order_relaxed);
}

#ifdef RFK_GEMM_TIMELINE
extern "C" int rfk_gemm_timeline(unsigned long long* host_out8) {
    return (int)cudaMemcpyFromSymbol(host_out8, tcgemm::g_timeline, 16 * sizeof(unsigned long long));
}
#endif

extern "C" int rfk_gemm_set_path(int path) {
    if (path < 0 || path > 3) return RFK_EINVAL;
    g_gemm_path.store(path, std::memory_order_relaxed);
    return RFK_OK;
}

extern "C" int rfk_gemm_error(int* code, int clear) {
    if (!code) return RFK_EINVAL;
    cudaError_t e = cudaMemcpyFromSymbol(code, g_gemm_tc_error, sizeof(int));
    if (e != cudaSuccess) return (int)e;
    if (clear) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(g_gemm_tc_error, &zero, sizeof(int));
        if (e != cudaSuccess) return (int)e;
    }
    return RFK_OK;
}
