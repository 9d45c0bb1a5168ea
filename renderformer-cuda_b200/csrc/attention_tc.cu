// Fused attention on the 5th-generation tensor cores (tcgen05 + tensor memory + TMA), head_dim 64.
//
// Same function as flash_attention_kernel (attention.cu): O = softmax(scale * Q K^T) V over
// the first n_keys keys, fp16 operands, fp32 accumulation, probabilities rounded to fp16.
// Reference boundary: rf::sdpa, src/layers/attention.cu:89-166 of BANANASJIM/renderformer-cuda.
//
// One CTA = 256 queries of one head as two blocks of 128 that share the K/V tiles in shared
// memory (every key tile is fetched once per CTA, i.e. half as often as with one block per CTA),
// keys in tiles of 64, 16 warps (13 with a role):
//   warp 8       producer: one thread issues TMA tile loads (both Q blocks once, then K and V tiles
//                through a ring of kStages shared-memory stages); the copies land in the tensor
//                core's 128-byte-swizzled layout and complete on mbarriers, no thread touches the bytes.
//   warps 11-12  one thread per block issues S = Q K^T (tcgen05.mma M128 N64 K16 x 4) into one of
//                the block's three score buffers in tensor memory, as soon as the P V product that
//                read that buffer's previous contents is complete: the softmax warps find their
//                next two tiles ready and never wait for a product.
//   warps 0-7    softmax (block = warp / 4): a thread owns one query row = its tensor-memory lane,
//                so row maximum and row sum are thread-local (no shuffles). The 64 scores come to
//                registers with tcgen05.ld; the common tile exponentiates them against the running
//                reference right away and checks afterwards that this was admissible (the exact path,
//                with the tile's maximum first, runs for the first tile, a padded last tile and a
//                failed check); P = exp2(...) is rounded to fp16 and stored back with
//                tcgen05.st over the first 32 columns of the same score buffer, from where
//   warps 9-10   one thread per block issues O += P V with P as the A operand from tensor memory
//                and V (MN-major) from shared memory: P never passes through shared memory. The
//                output accumulator O (128 x 64 fp32 per block) is rescaled in place only when a
//                row's running maximum has grown by more than 2^8 (the factor cancels in O / l).
// A stage of the ring is free again when both blocks' P V products of its tile are complete
// (kv_empty counts two arrivals). The products have separate issuing threads because one thread's
// instruction stream (8 products, 3 commits and 2-3 waits per tile, all dependent) takes about as
// long as the softmax of a tile; the order between them is kept by mbarriers, not by issue order.
// Tensor memory: all 512 columns (per block S0, S1, S2, O: 64 each); shared memory 32 KB (Q) +
// kStages x 16 KB; one CTA per SM. Every mbarrier wait is bounded; on a time-out the CTA raises an
// error word, frees its tensor memory and returns.
//
// Key split for grids that do not fill the machine. A unit = 256 queries of one head over all keys = one CTA. With few
// units (a 256 x 256 view has 64 of them for 148 SMs) most SMs idle, so when the caller supplies a workspace and the
// estimate below says it pays, the key range of the units is cut into one equal share per SM; a share is one or two
// pieces (it may cross a unit boundary), a piece is one CTA over a range of key tiles. A piece writes its un-normalised
// O, running maximum and sum to the workspace and increments its unit's counter; the CTA that finds the counter
// complete (no CTA ever waits for another) merges the unit's pieces, writes the output and zeroes the counter for the
// next launch. A piece costs about 10 us beyond its tiles (pipeline fill, publishing, merging), which is why grids
// that already fill the SMs once or more are left whole: measured, cutting the last partial round of a 256-unit grid
// gains nothing.
#include <algorithm>
#include <cuda.h>  // CUtensorMap and its enums; the encoder itself is looked up at run time
#define RFK_TC_WAIT_INLINE  // this kernel re-partitions its registers (setmaxnreg)
#include "attention_tc.cuh"
#include "common.cuh"

namespace rfk {

__device__ int g_attn_tc_error = 0;  // first time-out / failure code seen by any CTA since load

namespace tcattn {

constexpr int BM = 128, BN = 64, HD = 64;
constexpr int kBlocks = 2;                     // 128-query blocks per CTA, sharing the K/V ring
constexpr int kThreads = 512;                  // warps 0-7 softmax (block = warp / 4), 8 producer, 9-10 PV, 11-12 QK issuers, 13-15 none
// Registers: the CTA starts with 128 per thread. The two warpgroups that only issue copies and products (warps 8-15)
// hand theirs back down to kRegsIssue and the softmax warpgroups (warps 0-7) grow to kRegsSoftmax, which lets the
// compiler keep both halves of a score tile and their exponentials in flight without reusing registers early
// (measured: 3 % off the kernel's time). 256 * 40 + 256 * 216 = 65536, the register file.
constexpr int kRegsIssue = 40, kRegsSoftmax = 216;
constexpr int kStages = 6;
constexpr int kQBytes = BM * HD * 2;           // 16 KB
constexpr int kKBytes = BN * HD * 2;           // 8 KB; a stage is K then V
constexpr int kStageBytes = 2 * kKBytes;
constexpr int kSBufs = 3;                      // score buffers in tensor memory
constexpr int kTmemCols = 512;                 // per block: S0, S1, S2 at +0, +64, +128; O at +192

struct __align__(8) Ctrl {
    uint64_t q_full, kv_full[kStages], kv_empty[kStages], s_full[kBlocks][kSBufs], p_full[kBlocks][kSBufs],
        pv_done[kBlocks][kSBufs];
    uint64_t drain[2 * kBlocks];  // abort path only, one per issuing thread: completes once that thread's products have finished
    uint32_t tmem_base;
    int abort;
    int merge;  // set by thread 0 of a split unit's last piece: this CTA merges the unit
};

// The shared-memory window is declared 1024-byte aligned (swizzled tiles need it) and the kernel checks it.
constexpr int kSmemBytes = kBlocks * kQBytes + kStages * kStageBytes + 512;
static_assert(sizeof(Ctrl) <= 512, "control block");
static_assert(kSmemBytes + 1024 <= 227 * 1024, "one CTA per SM");

enum : int { kErrTimeout = 1, kErrSmemAlign = 2 };

// A CTA's share of a unit whose keys are split: key tiles [t0, t0 + nt) of unit `unit`; the unit's pieces own the
// workspace slots [first, first + count), this one `slot`.
struct Piece { uint16_t unit, t0, nt, first, count, slot; };
constexpr int kMaxPieces = 320;
struct WorkList {
    int whole_units;  // CTAs [0, whole_units) take the unit of their index over all keys
    int n_pieces;     // CTAs [whole_units, whole_units + n_pieces) take pieces[index - whole_units]
    int q_blocks;     // units per head: ceil(Sq / 256)
    Piece pieces[kMaxPieces];
};
// Workspace: 256 counters (one per split unit, zero between launches), then per slot 256 x {m, l}, then per slot the
// un-normalised output as [16 groups of 4 columns][256 rows] float4 (a warp's 32 rows of one group are contiguous).
constexpr int kUnitRows = kBlocks * BM;
constexpr size_t kWsCounterBytes = 1024;
constexpr size_t kWsMlBytes = (size_t)kMaxPieces * kUnitRows * 2 * sizeof(float);
constexpr size_t kWsOBytes = (size_t)kMaxPieces * kUnitRows * HD * sizeof(float);
constexpr size_t kWsBytes = kWsCounterBytes + kWsMlBytes + kWsOBytes;

__device__ __forceinline__ void regs_release() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsIssue)); }
__device__ __forceinline__ void regs_take() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax)); }
__device__ __forceinline__ void softmax_warps_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }  // warps 0-7 only

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// 2^x for two values on the FMA pipes (no special-function unit): x = n + f with n = round(x),
// 2^f from a polynomial on [-0.5, 0.5] and n added into the exponent field. Degree 3 (the default;
// relative error 7.5e-5, a sixth of the fp16 rounding of the result) or, with -DRFK_ATTN_POLY_DEG=4,
// degree 4 (2.6e-6). Inputs below -125 give a value near 2^-125; the result is only good for inputs
// below 128 (the caller checks the largest it passes).
#ifndef RFK_ATTN_POLY_DEG
#define RFK_ATTN_POLY_DEG 3
#endif
__device__ __forceinline__ float2 exp2_poly(float2 x) {
    constexpr float kMagic = 12582912.0f;  // 1.5 * 2^23: x + kMagic holds round(x) in its low mantissa bits
    x.x = fmaxf(x.x, -125.0f);
    x.y = fmaxf(x.y, -125.0f);
    const float2 t = __fadd2_rn(x, make_float2(kMagic, kMagic));
    const float2 n = __fadd2_rn(t, make_float2(-kMagic, -kMagic));
    const float2 f = __ffma2_rn(n, make_float2(-1.0f, -1.0f), x);
#if RFK_ATTN_POLY_DEG == 3
    float2 p = __ffma2_rn(f, make_float2(0.05517136f, 0.05517136f), make_float2(0.2426111f, 0.2426111f));
    p = __ffma2_rn(p, f, make_float2(0.69326103f, 0.69326103f));
    p = __ffma2_rn(p, f, make_float2(0.99992806f, 0.99992806f));
#else
    float2 p = __ffma2_rn(f, make_float2(0.009570092f, 0.009570092f), make_float2(0.05591786f, 0.05591786f));
    p = __ffma2_rn(p, f, make_float2(0.24024744f, 0.24024744f));
    p = __ffma2_rn(p, f, make_float2(0.6931218f, 0.6931218f));
    p = __ffma2_rn(p, f, make_float2(0.9999993f, 0.9999993f));
#endif
    return make_float2(__uint_as_float(__float_as_uint(p.x) + (__float_as_uint(t.x) << 23)),
                       __uint_as_float(__float_as_uint(p.y) + (__float_as_uint(t.y) << 23)));
}

// 32 raw scores -> 32 probabilities exp2(s * c - mc), packed two fp16 per word into pk[0..16); their
// fp32 sums are added to acc0 / acc1 (two lanes each).
// Packed fp32x2 multiply-adds and adds halve the instruction count around the exponentials. The
// special-function unit (16 exponentials per clock and SM) is the scarcest resource of this kernel,
// so of every four pairs, those selected by kPolyMask take the polynomial path instead.
#ifndef RFK_ATTN_POLY_MASK
#define RFK_ATTN_POLY_MASK 0x1
#endif
constexpr int kPolyMask = RFK_ATTN_POLY_MASK;

#ifndef RFK_ATTN_POLY_PERIOD
#define RFK_ATTN_POLY_PERIOD 4
#endif
__device__ __forceinline__ constexpr bool poly_pair(int pair) { return (kPolyMask >> (pair % RFK_ATTN_POLY_PERIOD)) & 1; }

__device__ __forceinline__ void exp_half(uint32_t (&v)[32], uint32_t* pk /* may alias v */, float c, float mc, float2& acc0,
                                         float2& acc1, float& poly_max) {
    const float2 c2 = make_float2(c, c), nm2 = make_float2(-mc, -mc);
    // three passes over the registers, each a run of independent instructions: exponents, exponentials
    // (back to back, so that one warp alone can keep the special-function unit busy), then sums and packing
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
        const float2 x = __ffma2_rn(make_float2(__uint_as_float(v[i]), __uint_as_float(v[i + 1])), c2, nm2);
        v[i] = __float_as_uint(x.x);
        v[i + 1] = __float_as_uint(x.y);
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        if (poly_pair(i >> 1)) continue;  // this pair takes the polynomial path below
        v[i] = __float_as_uint(fast_exp2(__uint_as_float(v[i])));
    }
    if (kPolyMask) {
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
            if (poly_pair(i >> 1)) {
                // the polynomial path is only good for exponents below 128: the caller checks the largest it was given
                poly_max = fmax3(poly_max, __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
                const float2 p = exp2_poly(make_float2(__uint_as_float(v[i]), __uint_as_float(v[i + 1])));
                v[i] = __float_as_uint(p.x);
                v[i + 1] = __float_as_uint(p.y);
            }
        }
    }
    // four independent chains of packed adds (with two, the adds of a half waited on each other: -3 % with four), the
    // packing written ahead of the adds (the compiler keeps this order; -1 %)
    float2 a2 = make_float2(0.0f, 0.0f), a3 = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
        const float2 p0 = make_float2(__uint_as_float(v[i]), __uint_as_float(v[i + 1]));
        const float2 p1 = make_float2(__uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
        const float2 p2 = make_float2(__uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
        const float2 p3 = make_float2(__uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
        pk[i >> 1] = pack_half2(p0.x, p0.y);
        pk[(i >> 1) + 1] = pack_half2(p1.x, p1.y);
        pk[(i >> 1) + 2] = pack_half2(p2.x, p2.y);
        pk[(i >> 1) + 3] = pack_half2(p3.x, p3.y);
        acc0 = __fadd2_rn(acc0, p0);
        acc1 = __fadd2_rn(acc1, p1);
        a2 = __fadd2_rn(a2, p2);
        a3 = __fadd2_rn(a3, p3);
    }
    acc0 = __fadd2_rn(acc0, a2);
    acc1 = __fadd2_rn(acc1, a3);
}

// 32 fp32 values (as raw words) * inv -> fp16 -> 64 bytes at dst
__device__ __forceinline__ void store_row_half(__half* dst, const uint32_t (&v)[32], float inv) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        uint4 o;
        o.x = pack_half2(__uint_as_float(v[8 * c + 0]) * inv, __uint_as_float(v[8 * c + 1]) * inv);
        o.y = pack_half2(__uint_as_float(v[8 * c + 2]) * inv, __uint_as_float(v[8 * c + 3]) * inv);
        o.z = pack_half2(__uint_as_float(v[8 * c + 4]) * inv, __uint_as_float(v[8 * c + 5]) * inv);
        o.w = pack_half2(__uint_as_float(v[8 * c + 6]) * inv, __uint_as_float(v[8 * c + 7]) * inv);
        *reinterpret_cast<uint4*>(dst + c * 8) = o;
    }
}

__global__ void __launch_bounds__(kThreads, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, __half* __restrict__ O, int H, int Sq, int n_keys,
                    int o_bshd, float scale_log2e_all, const float* __restrict__ row_ss, int ss_tiles, float inv_norm_dim,
                    float norm_eps, unsigned char* __restrict__ ws, int v_heads, const __grid_constant__ WorkList work) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const uint32_t base = tc::smem_addr(smem_raw);
    if (base & 1023u) {  // uniform over the CTA, nothing allocated yet
        if (threadIdx.x == 0) atomicCAS(&g_attn_tc_error, 0, kErrSmemAlign);
        return;
    }
    const uint32_t sQ = base, sKV = base + kBlocks * kQBytes;
    Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem_raw + kBlocks * kQBytes + kStages * kStageBytes);
    volatile int* abort_flag = &ctrl->abort;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // this CTA's work: a whole unit, or a piece of one (n_tiles key tiles from tile t0)
    int unit = blockIdx.x, t0 = 0, n_tiles = (n_keys + BN - 1) / BN, split_count = 1, split_first = 0, split_slot = 0;
    if ((int)blockIdx.x >= work.whole_units) {
        const Piece& pc = work.pieces[blockIdx.x - work.whole_units];
        unit = pc.unit; t0 = pc.t0; n_tiles = pc.nt; split_count = pc.count; split_first = pc.first; split_slot = pc.slot;
    }
    const int q0 = (unit % work.q_blocks) * kUnitRows;
    const int bh = unit / work.q_blocks;

    if (tid == 0) {
        tc::mbar_init(&ctrl->q_full, 1);
        for (int s = 0; s < kStages; ++s) { tc::mbar_init(&ctrl->kv_full[s], 1); tc::mbar_init(&ctrl->kv_empty[s], kBlocks); }
        for (int k = 0; k < kBlocks; ++k)
            for (int b = 0; b < kSBufs; ++b) {
                tc::mbar_init(&ctrl->s_full[k][b], 1); tc::mbar_init(&ctrl->p_full[k][b], 4); tc::mbar_init(&ctrl->pv_done[k][b], 1);
            }
        for (int k = 0; k < 2 * kBlocks; ++k) tc::mbar_init(&ctrl->drain[k], 1);
        ctrl->abort = 0;
        ctrl->merge = 0;
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
    // everything above touched only this CTA's shared and tensor memory; the operands below are another kernel's output
    pdl_wait();
    pdl_trigger();

    // The register hand-over: every warp of a warpgroup executes the same setmaxnreg instruction (warpgroups 2 and 3 the
    // release, 0 and 1 the take), as the first statement of a branch that does not meet the other again before the
    // teardown - placed ahead of the branch, the compiler bound every role by the smaller budget.
    if (warp >= 8) {
    regs_release();
    if (warp == 8) {
        // ------------------------------------------------------------ producer (one thread)
        if (lane == 0) {
            tc::prefetch_tensormap(&map_q); tc::prefetch_tensormap(&map_k); tc::prefetch_tensormap(&map_v);
            tc::mbar_arrive_expect_tx(&ctrl->q_full, kBlocks * kQBytes);
            for (int k = 0; k < kBlocks; ++k) tc::tma_load_3d(sQ + k * kQBytes, &map_q, 0, q0 + k * BM, bh, &ctrl->q_full);
            int issued = 0;
            for (int j = 0; j < n_tiles; ++j) {
                const int s = j % kStages;
                // stage s was last read by the products of tile j - kStages (phase j / kStages - 1 of kv_empty[s])
                if (j >= kStages && !tc::mbar_wait(&ctrl->kv_empty[s], ((j / kStages) + 1) & 1, abort_flag)) break;
                tc::mbar_arrive_expect_tx(&ctrl->kv_full[s], kStageBytes);
                tc::tma_load_3d(sKV + s * kStageBytes, &map_k, 0, (t0 + j) * BN, bh, &ctrl->kv_full[s]);
                tc::tma_load_3d(sKV + s * kStageBytes + kKBytes, &map_v, 0, (t0 + j) * BN, bh % v_heads, &ctrl->kv_full[s]);
                issued = j + 1;
            }
            if (*abort_flag) {
                // The CTA is giving up. Every copy this thread started lands in this CTA's shared memory and counts
                // on a kv_full / q_full barrier: wait (bounded) for the last copy of each stage before the CTA exits.
                tc::mbar_wait_drain(&ctrl->q_full, 0);
                for (int s = 0; s < kStages && s < issued; ++s) {
                    const int last = ((issued - 1 - s) / kStages) * kStages + s;  // last tile loaded into stage s
                    tc::mbar_wait_drain(&ctrl->kv_full[s], (last / kStages) & 1);
                }
            }
        }
        __syncwarp();
    } else if (warp == 9 || warp == 10) {
        const int blk = warp - 9;
        const uint32_t tmem = tmem_cta + blk * 256, tmem_O = tmem + kSBufs * 64;
        // ------------------------------------------------------------ issuer of O += P V (one thread)
        // tile j: score buffer j % kSBufs (its use number j / kSBufs gives the barrier phase), ring stage j % kStages
        if (lane == 0) {
            constexpr uint32_t idesc_pv = tc::umma_idesc_f16(BM, HD, 1);  // B = V tile, MN-major
            const uint32_t v_lo = tc::umma_desc_lo(sKV + kKBytes);
            bool ok = true;
            int buf = 0, buf_par = 0, st = 0;
            for (int j = 0; ok && j < n_tiles; ++j) {
                ok = tc::mbar_wait(&ctrl->p_full[blk][buf], buf_par, abort_flag);
                if (!ok) break;
                tc::tc_fence_after();
                const uint32_t p_tmem = tmem + buf * 64, vt_lo = v_lo + st * (kStageBytes >> 4);
#pragma unroll
                for (int ks = 0; ks < BN / 16; ++ks)  // P: 16 keys = 8 columns; V: 16 keys = 16 rows of 128 bytes
                    tc::umma_f16_ts_lo(tmem_O, p_tmem + ks * 8, vt_lo + ks * (2048 >> 4), idesc_pv, (j > 0) || (ks > 0));
                tc::umma_commit(&ctrl->kv_empty[st]);  // K of this stage was consumed before its scores could be read
                tc::umma_commit(&ctrl->pv_done[blk][buf]);
                if (++buf == kSBufs) { buf = 0; buf_par ^= 1; }
                if (++st == kStages) st = 0;
            }
            if (*abort_flag) {  // giving up: let this thread's products finish before tensor memory is freed
                tc::umma_commit(&ctrl->drain[blk]);
                tc::mbar_wait_drain(&ctrl->drain[blk], 0);
            }
        }
        __syncwarp();
    } else if (warp == 11 || warp == 12) {
        const int blk = warp - 11;
        const uint32_t tmem = tmem_cta + blk * 256;
        // ------------------------------------------------------------ issuer of S = Q K^T (one thread)
        if (lane == 0) {
            constexpr uint32_t idesc_qk = tc::umma_idesc_f16(BM, BN, 0);  // B = K tile, K-major
            const uint32_t q_lo = tc::umma_desc_lo(sQ + blk * kQBytes), k_lo = tc::umma_desc_lo(sKV);
            bool ok = tc::mbar_wait(&ctrl->q_full, 0, abort_flag);
            int buf = 0, buf_par = 0, st = 0, st_par = 0;
            for (int j = 0; ok && j < n_tiles; ++j) {
                ok = tc::mbar_wait(&ctrl->kv_full[st], st_par, abort_flag);
                // the buffer still holds P of tile j - kSBufs until that tile's P V is complete
                if (ok && j >= kSBufs) ok = tc::mbar_wait(&ctrl->pv_done[blk][buf], buf_par ^ 1, abort_flag);
                if (!ok) break;
                tc::tc_fence_after();
                const uint32_t kt_lo = k_lo + st * (kStageBytes >> 4);
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks)  // 16 head-dim elements = 32 bytes along a row
                    tc::umma_f16_lo(tmem + buf * 64, q_lo + ks * 2, kt_lo + ks * 2, idesc_qk, ks > 0);
                tc::umma_commit(&ctrl->s_full[blk][buf]);
                if (++buf == kSBufs) { buf = 0; buf_par ^= 1; }
                if (++st == kStages) { st = 0; st_par ^= 1; }
            }
            if (*abort_flag) {
                tc::umma_commit(&ctrl->drain[kBlocks + blk]);
                tc::mbar_wait_drain(&ctrl->drain[kBlocks + blk], 0);
            }
        }
        __syncwarp();
    }  // warps 13-15 have no role beyond handing their registers back together with warp 12
    } else {
        regs_take();
        // ------------------------------------------------------------ softmax, warps 0-7 (query block = warp / 4)
        constexpr unsigned kFull = 0xffffffffu;
        constexpr float kSumLimit = 256.0f;  // 2^kRescaleThreshold
        constexpr uint32_t kNegInf = 0xff800000u;
        constexpr float kRescaleThreshold = 8.0f;  // in exponent units: P stays below 2^8, well inside fp16
        const int blk = warp >> 2;
        const int r = (warp & 3) * 32 + lane;                       // query row within the block = its tensor-memory lane
        const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;  // a warp reaches lanes [32 * (warp % 4), +32)
        const uint32_t tmem = tmem_cta + blk * 256, tmem_O = tmem + kSBufs * 64;
        const uint32_t tO = tmem_O + lane_off;
        // Queries that arrive un-normalised (rfk_gemm_f16_heads) bring the partial sums of squares of their rows: the
        // RMSNorm's 1 / rms is a per-row factor of the scores, i.e. of this thread's exponent scale (the norm's weight
        // is folded into the keys by the caller). The row statistic spans all heads of the token.
        float scale_log2e = scale_log2e_all;
        if (row_ss) {
            const int q = min(q0 + blk * BM + r, Sq - 1);
            const float* sp = row_ss + ((size_t)(bh / H) * Sq + q) * ss_tiles;
            float ss = 0.0f;
            for (int t = 0; t < ss_tiles; ++t) ss += __ldg(sp + t);
            scale_log2e *= rsqrtf(ss * inv_norm_dim + norm_eps);
        }
        float m_run = -INFINITY, l_run = 0.0f;
        uint32_t va[32], vb[32];
        bool ok = true;
        int buf = 0, buf_par = 0;  // score buffer of tile j and the phase parity of its barriers
        for (int j = 0; j < n_tiles; ++j) {
            const uint32_t tS = tmem + lane_off + buf * 64;
            ok = tc::mbar_wait_warp(&ctrl->s_full[blk][buf], buf_par, abort_flag);
            if (!ok) break;
            tc::tc_fence_after();
            const int n_valid = min(BN, n_keys - (t0 + j) * BN);  // real keys among this tile's 64 columns
            tc::tmem_ld32(tS, va);
            tc::tc_wait_ld(va);
            tc::tmem_ld32(tS + 32, vb);  // in flight during the first half's arithmetic
            if (n_valid != BN) {  // last tile: keys at or beyond n_keys score -inf, i.e. contribute nothing
                tc::tc_wait_ld(vb);
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    if (i >= n_valid) va[i] = kNegInf;
                    if (32 + i >= n_valid) vb[i] = kNegInf;
                }
            }
            // The running maximum only follows a tile's maximum when it would move by more than the threshold; until
            // then the probabilities of the row are scaled by up to 2^threshold, which cancels in O / l. So the common
            // tile leaves the reference where it is, and its exponentials start from the reference already known,
            // without this tile's maximum ahead of them: if afterwards no row's probabilities sum to more than
            // 2^threshold, none of them exceeded it and the tile is done. Otherwise (and for the first and the last
            // tile) the scores are read again, the maximum is taken and the same code runs once more.
            float2 acc0, acc1;
            float m_new = m_run, alpha = 1.0f;
            bool any_move = false, need_max = j == 0 || n_valid != BN;
#pragma unroll 1
            for (;;) {
                acc0 = make_float2(0.0f, 0.0f);
                acc1 = make_float2(0.0f, 0.0f);
                if (need_max) {
                    tc::tc_wait_ld(vb);
                    float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        m0 = fmax3(m0, __uint_as_float(va[i]), __uint_as_float(va[i + 1]));
                        m1 = fmax3(m1, __uint_as_float(va[i + 2]), __uint_as_float(va[i + 3]));
                        m2 = fmax3(m2, __uint_as_float(vb[i]), __uint_as_float(vb[i + 1]));
                        m3 = fmax3(m3, __uint_as_float(vb[i + 2]), __uint_as_float(vb[i + 3]));
                    }
                    const float m_tile = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
                    const bool move = (m_tile - m_run) * scale_log2e > kRescaleThreshold;  // first tile: m_run = -inf
                    m_new = move ? m_tile : m_run;
                    any_move = __any_sync(kFull, move);
                    if (any_move && move) alpha = fast_exp2((m_run - m_new) * scale_log2e);  // first tile: 0
                }
                // P = exp2(scale * log2e * (S - max)), two fp16 per 32-bit column: keys 2i, 2i+1 in column i;
                // the 32 packed words end up in va, which is what the store below takes
                const float mc = m_new * scale_log2e;
                float poly_max = -INFINITY;
                exp_half(va, va, scale_log2e, mc, acc0, acc1, poly_max);
                tc::tc_wait_ld(vb);
                exp_half(vb, va + 16, scale_log2e, mc, acc0, acc1, poly_max);
                if (need_max) break;
                const float sum = (acc0.x + acc0.y) + (acc1.x + acc1.y);
                if (!__any_sync(kFull, !(sum <= kSumLimit) || poly_max > kRescaleThreshold)) break;
                need_max = true;
                tc::tmem_ld32(tS, va);
                tc::tc_wait_ld(va);
                tc::tmem_ld32(tS + 32, vb);
            }
            if (j > 0 && any_move) {  // rescale this warp's 32 rows of O (vb is free here)
                // O belongs to the tensor core until the previous tile's P V is done. Having seen s_full of tile j,
                // P V of tile j - 4 (the previous phase of this barrier) is known complete: the parity is unambiguous.
                const int pbuf = buf == 0 ? kSBufs - 1 : buf - 1, pbuf_par = buf == 0 ? buf_par ^ 1 : buf_par;  // of tile j - 1
                ok = tc::mbar_wait_warp(&ctrl->pv_done[blk][pbuf], pbuf_par, abort_flag);
                if (!ok) break;
                tc::tc_fence_after();
#pragma unroll
                for (int hc = 0; hc < 2; ++hc) {
                    tc::tmem_ld32(tO + hc * 32, vb);
                    tc::tc_wait_ld(vb);
#pragma unroll
                    for (int i = 0; i < 32; ++i) vb[i] = __float_as_uint(__uint_as_float(vb[i]) * alpha);
                    tc::tmem_st32(tO + hc * 32, vb);
                }
            }
            l_run = (any_move ? l_run * alpha : l_run) + ((acc0.x + acc0.y) + (acc1.x + acc1.y));
            m_run = m_new;
            tc::tmem_st32(tS, va);    // P over the first 32 columns of this thread's own lane of S
            tc::tc_wait_st();
            tc::tc_fence_before();    // the writes of P and O come before the arrival
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&ctrl->p_full[blk][buf]);
            if (++buf == kSBufs) { buf = 0; buf_par ^= 1; }
        }
        // ---- epilogue: O / l -> fp16 -> global, one 128-byte row per thread
        if (ok) {  // buf / buf_par have moved on to tile n_tiles: step back to the last tile
            const int lbuf = buf == 0 ? kSBufs - 1 : buf - 1, lbuf_par = buf == 0 ? buf_par ^ 1 : buf_par;
            ok = tc::mbar_wait_warp(&ctrl->pv_done[blk][lbuf], lbuf_par, abort_flag);
        }
        const int q = q0 + blk * BM + r;
        __half* dst = o_bshd ? O + (((size_t)(bh / H) * Sq + q) * H + bh % H) * HD : O + ((size_t)bh * Sq + q) * HD;
        if (split_count == 1) {
            if (ok) {
                tc::tc_fence_after();
                const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
#pragma unroll
                for (int hc = 0; hc < 2; ++hc) {
                    tc::tmem_ld32(tO + hc * 32, va);
                    tc::tc_wait_ld(va);
                    if (q < Sq) store_row_half(dst + hc * 32, va, inv);
                }
            }
        } else {
            // ---- a piece of a split unit: publish (m, l, O), count, and merge if this CTA completes the unit
            float* ws_ml = reinterpret_cast<float*>(ws + kWsCounterBytes);
            float* ws_o = reinterpret_cast<float*>(ws + kWsCounterBytes + kWsMlBytes);
            const int row = blk * BM + r;
            if (ok) {
                tc::tc_fence_after();
                uint4* po = reinterpret_cast<uint4*>(ws_o) + (size_t)split_slot * (HD / 4) * kUnitRows + row;
#pragma unroll
                for (int hc = 0; hc < 2; ++hc) {
                    tc::tmem_ld32(tO + hc * 32, va);
                    tc::tc_wait_ld(va);
#pragma unroll
                    for (int c = 0; c < 8; ++c)
                        __stcg(po + (hc * 8 + c) * kUnitRows, make_uint4(va[4 * c], va[4 * c + 1], va[4 * c + 2], va[4 * c + 3]));
                }
                // the exponent reference in exponent units (the row's own scale applied), so that pieces compare directly
                __stcg(reinterpret_cast<float2*>(ws_ml + ((size_t)split_slot * kUnitRows + row) * 2), make_float2(m_run * scale_log2e, l_run));
                __threadfence();
            }
            softmax_warps_sync();  // every softmax warp comes here, whatever its ok: the barrier cannot be left short
            if (tid == 0) {
                int merge = 0;
                if (!*abort_flag) {
                    int* counter = reinterpret_cast<int*>(ws) + (unit - work.whole_units);
                    merge = atomicAdd(counter, 1) == split_count - 1;
                    if (merge) {
                        *counter = 0;  // every piece of the unit has arrived: ready for the next launch
                        __threadfence();
                    }
                }
                ctrl->merge = merge;
            }
            softmax_warps_sync();
            if (ctrl->merge && ok) {
                float m_all = -INFINITY;
                for (int p = 0; p < split_count; ++p)
                    m_all = fmaxf(m_all, __ldcg(ws_ml + ((size_t)(split_first + p) * kUnitRows + row) * 2));
                float l_all = 0.0f;
                float* acc = reinterpret_cast<float*>(va);  // va, vb: this row's 64 merged outputs
                float* acc2 = reinterpret_cast<float*>(vb);
#pragma unroll
                for (int i = 0; i < 32; ++i) { acc[i] = 0.0f; acc2[i] = 0.0f; }
                for (int p = 0; p < split_count; ++p) {  // in slot order, whichever CTA merges: the sum is reproducible
                    const size_t pr = (size_t)(split_first + p) * kUnitRows + row;
                    const float2 ml = __ldcg(reinterpret_cast<const float2*>(ws_ml + pr * 2));
                    const float w = fast_exp2(ml.x - m_all);
                    l_all += w * ml.y;
                    const float4* src = reinterpret_cast<const float4*>(ws_o) + (size_t)(split_first + p) * (HD / 4) * kUnitRows + row;
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        const float4 a = __ldcg(src + c * kUnitRows), b = __ldcg(src + (8 + c) * kUnitRows);
                        acc[4 * c] += w * a.x; acc[4 * c + 1] += w * a.y; acc[4 * c + 2] += w * a.z; acc[4 * c + 3] += w * a.w;
                        acc2[4 * c] += w * b.x; acc2[4 * c + 1] += w * b.y; acc2[4 * c + 2] += w * b.z; acc2[4 * c + 3] += w * b.w;
                    }
                }
                const float inv = l_all > 0.0f ? 1.0f / l_all : 0.0f;
                if (q < Sq) {
                    store_row_half(dst, va, inv);
                    store_row_half(dst + 32, vb, inv);
                }
            }
        }
    }

    // ---- teardown: every path (normal or aborted) arrives here with no divergence inside a warp
    tc::tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc::tc_fence_after();
        tc::tmem_dealloc(tmem_cta, kTmemCols);
    }
    if (tid == 0 && ctrl->abort) atomicCAS(&g_attn_tc_error, 0, kErrTimeout);
}

}  // namespace tcattn

std::atomic<int> g_attn_path{0};  // 0 automatic, 1 mma.sync kernel, 2 tcgen05 kernel (head_dim 64 only)
std::atomic<int> g_attn_split{1};  // 0: never split keys, even with a workspace (to time both side by side)

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

// fp16 tensor [n_heads][rows][64], contiguous; boxes of box_rows x 64 in the 128-byte-swizzled layout,
// rows past the end of a head read as zeros
bool make_map(CUtensorMap* m, const void* base, long long n_heads, long long rows, int box_rows) {
    EncodeTiledFn enc = tensor_map_encoder();
    if (!enc) return false;
    const cuuint64_t dims[3] = {64, (cuuint64_t)rows, (cuuint64_t)n_heads};
    const cuuint64_t strides[2] = {128, (cuuint64_t)rows * 128};  // bytes, dimensions 1 and 2
    const cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Fills `w` for `units` units of `n_tiles` key tiles each on a device with `sms` SMs (see "Key split" above).
// split = false, or the estimate says it does not pay: every unit whole.
void plan_work(tcattn::WorkList& w, long long units, int n_tiles, int sms, bool split) {
    using tcattn::Piece;
    constexpr int kPieceCostTiles = 12;  // what a piece costs beyond its tiles (fill, publishing, merging), in tile times
    w.whole_units = (int)units;
    w.n_pieces = 0;
    if (!split || sms <= 0 || units <= 0 || units >= sms || units > 256 || n_tiles > 65535) return;  // 256 unit counters
    const long long tiles = units * n_tiles;
    constexpr int kMaxPiecesPerUnit = 8;  // the CTA that merges a unit reads its pieces one after the other
    const int shares = (int)std::min<long long>(std::min(sms, tcattn::kMaxPieces / 2), units * kMaxPiecesPerUnit);
    // whole: one round of n_tiles; split: a share's tiles plus the piece overhead. Cut only for a clear gain.
    if ((tiles + shares - 1) / shares + kPieceCostTiles > (long long)n_tiles * 4 / 5) return;
    Piece* pc = w.pieces;
    int n = 0;
    for (int s = 0; s < shares; ++s) {
        long long b = tiles * s / shares;
        const long long e = tiles * (s + 1) / shares;
        while (b < e) {  // at most twice: a share is shorter than a unit
            const long long u = b / n_tiles, pe = std::min(e, (u + 1) * n_tiles);
            pc[n].unit = (uint16_t)u;
            pc[n].t0 = (uint16_t)(b - u * n_tiles);
            pc[n].nt = (uint16_t)(pe - b);
            pc[n].slot = (uint16_t)n;
            ++n;
            b = pe;
        }
    }
    for (int i = 0; i < n;) {  // pieces of a unit are consecutive here: give each its unit's slot range
        int j = i;
        while (j < n && pc[j].unit == pc[i].unit) ++j;
        for (int k = i; k < j; ++k) { pc[k].first = (uint16_t)i; pc[k].count = (uint16_t)(j - i); }
        i = j;
    }
    // longest first: in-order dispatch then hands the short pieces to the SMs that finish their long ones first
    std::stable_sort(pc, pc + n, [](const Piece& a, const Piece& b) { return a.nt > b.nt; });
    w.whole_units = 0;
    w.n_pieces = n;
}

}  // namespace

size_t attention_tc_workspace_bytes() { return tcattn::kWsBytes; }

// The launcher's plan for a grid, without launching anything (host only: no device is touched).
int attention_tc_plan(long long units, int n_tiles, int sms, int* whole_units, int* n_pieces, unsigned short* pieces, int max_pieces) {
    if (units < 0 || n_tiles <= 0 || sms <= 0 || !whole_units || !n_pieces || max_pieces < 0 || (max_pieces && !pieces)) return RFK_EINVAL;
    tcattn::WorkList w;
    plan_work(w, units, n_tiles, sms, true);
    *whole_units = w.whole_units;
    *n_pieces = w.n_pieces;
    for (int i = 0; i < w.n_pieces && i < max_pieces; ++i) {
        const tcattn::Piece& pc = w.pieces[i];
        const unsigned short rec[6] = {pc.unit, pc.t0, pc.nt, pc.first, pc.count, pc.slot};
        for (int k = 0; k < 6; ++k) pieces[i * 6 + k] = rec[k];
    }
    return RFK_OK;
}

// Launches the tcgen05 kernel; the caller has validated pointers, alignment and sizes (D == 64). v_shared: V is
// [H, Sk, D], one set of values for every batch element (views of one scene). ws (may be NULL):
// attention_tc_workspace_bytes() bytes whose first 1024 are zero, for the key split.
int launch_attention_tc(const __half* Q, const __half* K, const __half* V, __half* O, int B, int H, int Sq, int Sk,
                        int n_keys, int o_bshd, float scale, cudaStream_t st, const float* row_ss, int ss_tiles,
                        int norm_dim, float norm_eps, void* ws, size_t ws_bytes, int v_shared) {
    // per-device "kernel attributes set" marks; setting them twice from racing threads is harmless
    static std::atomic<bool> configured[64];
    static std::atomic<int> sm_count[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return RFK_EUNSUPPORTED;
    if (!configured[dev].load(std::memory_order_acquire)) {
        e = cudaFuncSetAttribute(tcattn::attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 tcattn::kSmemBytes);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(tcattn::attention_tc_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return (int)e;
        int sms = 0;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return (int)e;
        sm_count[dev].store(sms, std::memory_order_relaxed);
        configured[dev].store(true, std::memory_order_release);
    }
    CUtensorMap mq, mk, mv;
    if (!make_map(&mq, Q, (long long)B * H, Sq, tcattn::BM) || !make_map(&mk, K, (long long)B * H, Sk, tcattn::BN) ||
        !make_map(&mv, V, v_shared ? (long long)H : (long long)B * H, Sk, tcattn::BN))
        return RFK_EUNSUPPORTED;
    tcattn::WorkList work;
    work.q_blocks = ceil_div(Sq, tcattn::kUnitRows);
    const long long units = (long long)B * H * work.q_blocks;
    if (units > 0x7fffffffLL) return RFK_EUNSUPPORTED;
    const bool split = ws && ws_bytes >= tcattn::kWsBytes && aligned16(ws) && g_attn_split.load(std::memory_order_relaxed);
    plan_work(work, units, ceil_div(n_keys, tcattn::BN), sm_count[dev].load(std::memory_order_relaxed), split);
    dim3 grid((unsigned)(work.whole_units + work.n_pieces));
    launch_pdl(tcattn::attention_tc_kernel, grid, dim3(tcattn::kThreads), tcattn::kSmemBytes, st, mq, mk, mv, O, H, Sq, n_keys,
               o_bshd, scale * 1.4426950408889634f, row_ss, ss_tiles, norm_dim > 0 ? 1.0f / (float)norm_dim : 0.0f, norm_eps,
               static_cast<unsigned char*>(ws), v_shared ? H : B * H, work);
    return launch_status();
}

}  // namespace rfk

using namespace rfk;

extern "C" int rfk_flash_attention_set_path(int path) {
    if (path < 0 || path > 2) return RFK_EINVAL;
    g_attn_path.store(path, std::memory_order_relaxed);
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
