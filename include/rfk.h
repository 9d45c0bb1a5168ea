/*
 * rfk.h — C ABI of librfk.so: the sm_100a layer-kernel family of a RenderFormer
 * inference engine (RMSNorm with fused residual and fp16 cast, triangle-vertex
 * RoPE, NeRF positional encoding, row softmax, activations, ray generation,
 * world->camera transform) plus the layout helpers that sit between its GEMMs.
 *
 * Conventions
 *   - every entry point returns an int status: RFK_OK (0), a negative RFK_E*
 *     code for a rejected argument, or a positive cudaError_t from the launch;
 *   - all pointers are device pointers unless a comment says otherwise;
 *   - `rfk_half` is an IEEE binary16 stored in 16 bits (the CUDA `half`);
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream);
 *   - no entry point allocates, frees or synchronises unless its comment says
 *     so: every call is asynchronous on `stream` and may be captured in a CUDA
 *     graph;
 *   - in-place aliasing that the reference relies on (y == x for the norms,
 *     out == a for SiLU*b, elu/pow10 in place) is supported where stated.
 *
 * "replaces" comments give the interface of the reference engine
 * (BANANASJIM/renderformer-cuda, paths relative to that project) whose
 * arguments, meaning and numerics the entry point reproduces.
 */
#ifndef RFK_H
#define RFK_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef uint16_t rfk_half;      /* IEEE binary16 bit pattern               */
typedef void*    rfk_stream_t;  /* cudaStream_t                            */

enum {
    RFK_OK          = 0,
    RFK_EINVAL      = -1,  /* null pointer, negative size, unsupported shape */
    RFK_EUNSUPPORTED= -2,  /* shape outside what the kernels implement       */
    RFK_ETOOBIG     = -3,  /* size beyond a documented fixed maximum         */
    RFK_EKERNEL     = -4   /* a kernel gave up on a bounded device-side wait (rfk_flash_attention_error) */
};

/* Library identification: returns a static string "rfk <version> sm_100a". */
const char* rfk_version(void);
/* Human-readable text for a status returned by any entry point. */
const char* rfk_status_string(int status);
/* Number of kernels this library has launched in the calling process so far
 * (host-side counter, incremented per launch; used by benchmarks). */
unsigned long long rfk_launch_count(void);

/* ------------------------------------------------------------------ RMSNorm */

/* y[r,:] = half((float(x[r,:]) * rsqrt(mean(x[r,:]^2) + eps)) * gamma), y may alias x.
 * replaces rf::rmsnorm — src/kernels/rmsnorm.h:13, src/kernels/rmsnorm.cu:8-57 */
int rfk_rmsnorm(const rfk_half* x, const float* gamma, rfk_half* y,
                int rows, int dim, float eps, rfk_stream_t stream);

/* fp32 in / fp32 out variant, y may alias x.
 * replaces rf::rmsnorm_f32 — src/kernels/rmsnorm.h:18, src/kernels/rmsnorm.cu:59-96 */
int rfk_rmsnorm_f32(const float* x, const float* gamma, float* y,
                    int rows, int dim, float eps, rfk_stream_t stream);

/* Fused: h += r (fp32, written back); y16 = half(rmsnorm(h) * gamma).
 * One launch instead of the reference's residual_add_f32 -> rmsnorm_f32 ->
 * cast_fp32_to_fp16 triple (src/layers/transformer.cu:21-30, 32-45;
 * src/kernels/rmsnorm.cu:59-96; sequence at src/layers/transformer.cu:216,220-221).
 * r may be NULL (no residual; h is then not rewritten). */
int rfk_rmsnorm_residual_f32_cast16(float* h, const float* r, const float* gamma,
                                    rfk_half* y16, int rows, int dim, float eps,
                                    rfk_stream_t stream);

/* Same with an fp16 residual (the encoder's fp32 hidden += fp16 sub-layer output).
 * replaces residual_add_mixed -> rmsnorm_f32 -> cast_fp32_to_fp16 —
 * src/layers/transformer.cu:52-61, 216, 220-221 */
int rfk_rmsnorm_residual_mixed_cast16(float* h, const rfk_half* r, const float* gamma,
                                      rfk_half* y16, int rows, int dim, float eps,
                                      rfk_stream_t stream);

/* fp16 hidden state (decoder): x = half(float(x) + float(r)) written back, then
 * y = rmsnorm(x). r may be NULL. y must not alias x when r != NULL.
 * replaces residual_add -> rmsnorm — src/layers/transformer.cu:9-19, 179-182 */
int rfk_rmsnorm_residual_f16(rfk_half* x, const rfk_half* r, const float* gamma,
                             rfk_half* y, int rows, int dim, float eps,
                             rfk_stream_t stream);

/* The same with one operand in swin window order, for the two norms around the window attention of a
 * decoder layer over a [B, H, W] token grid (window_size x window_size windows of the grid shifted by
 * -shift_size). windowed_operand = 1: y is written in window order, i.e. residual add + norm + cyclic
 * shift + window partition in one pass — replaces residual_add -> rmsnorm (src/layers/transformer.cu:
 * 9-19, 179-182) -> cyclic_shift -> window_partition (src/layers/attention.cu:495-506).
 * windowed_operand = 2: r is read in window order, i.e. window reverse + shift back + residual add +
 * norm — replaces window_reverse -> cyclic_shift (src/layers/attention.cu:568-575) -> residual_add ->
 * rmsnorm. r may be NULL only with windowed_operand = 1 (plain norm written in window order, x left
 * untouched); y must alias neither x nor r. dim % 8 == 0 and dim <= 2048
 * (RFK_EUNSUPPORTED otherwise). */
int rfk_rmsnorm_residual_f16_windows(rfk_half* x, const rfk_half* r, const float* gamma,
                                     rfk_half* y, int B, int H, int W, int dim, int window_size,
                                     int shift_size, int windowed_operand, float eps,
                                     rfk_stream_t stream);

/* ----------------------------------------------- residual / cast plumbing */

/* y = half(float(y) + float(r)) — replaces rf::residual_add, src/layers/transformer.cu:9-19 */
int rfk_residual_add(rfk_half* y, const rfk_half* r, long long n, rfk_stream_t stream);
/* y += r (fp32) — replaces rf::residual_add_f32, src/layers/transformer.cu:21-30 */
int rfk_residual_add_f32(float* y, const float* r, long long n, rfk_stream_t stream);
/* y(fp32) += float(r(fp16)) — replaces rf::residual_add_mixed, src/layers/transformer.cu:52-61 */
int rfk_residual_add_mixed(float* y, const rfk_half* r, long long n, rfk_stream_t stream);
/* replaces rf::cast_fp32_to_fp16 / cast_fp16_to_fp32 — src/layers/transformer.cu:32-50 */
int rfk_cast_fp32_to_fp16(const float* in, rfk_half* out, long long n, rfk_stream_t stream);
int rfk_cast_fp16_to_fp32(const rfk_half* in, float* out, long long n, rfk_stream_t stream);
/* out[i] = half(float(out[i]) + float(bc[i % dim])) — replaces k_broadcast_add_s,
 * src/pipeline/render_session.cu:44-47 */
int rfk_broadcast_add(rfk_half* out, const rfk_half* bc, long long n, int dim,
                      rfk_stream_t stream);

/* --------------------------------------------------------------------- RoPE */

/* cos/sin tables [B,1,S,head_dim] fp16 from 9-D triangle positions [B,S,9] fp16 and
 * num_freqs fp32 frequencies; each half of head_dim holds 9*num_freqs angles then zeros.
 * replaces rf::triangle_rope_freqs — src/kernels/rope.h:12, src/kernels/rope.cu:11-57 */
int rfk_triangle_rope_freqs(const rfk_half* pos, const float* learned_freqs,
                            rfk_half* out_cos, rfk_half* out_sin,
                            int batch, int seq_len, int num_freqs, int head_dim,
                            rfk_stream_t stream);

/* In-place rotate-half RoPE on q and k [B,H,S,D] fp16 with tables [B,1,S,D] fp16.
 * replaces rf::apply_rope — src/kernels/rope.h:20, src/kernels/rope.cu:61-105 */
int rfk_apply_rope(rfk_half* q, rfk_half* k, const rfk_half* cos_vals, const rfk_half* sin_vals,
                   int batch, int num_heads, int seq_len, int head_dim, rfk_stream_t stream);
/* replaces rf::apply_rope_one — src/kernels/rope.h:25, src/kernels/rope.cu:108-145 */
int rfk_apply_rope_one(rfk_half* x, const rfk_half* cos_vals, const rfk_half* sin_vals,
                       int batch, int num_heads, int seq_len, int head_dim, rfk_stream_t stream);
/* fp32 data, fp16 tables — replaces rf::apply_rope_f32 / apply_rope_one_f32,
 * src/kernels/rope.h:30-36, src/kernels/rope.cu:148-211 */
int rfk_apply_rope_f32(float* q, float* k, const rfk_half* cos_vals, const rfk_half* sin_vals,
                       int batch, int num_heads, int seq_len, int head_dim, rfk_stream_t stream);
int rfk_apply_rope_one_f32(float* x, const rfk_half* cos_vals, const rfk_half* sin_vals,
                           int batch, int num_heads, int seq_len, int head_dim, rfk_stream_t stream);

/* Out-of-place RoPE: dst = rope(src). Replaces the per-layer pair
 * cudaMemcpyAsync(K_bhsd <- K_cached) + apply_rope_one(K_bhsd) —
 * src/layers/attention.cu:355-361. src_seq_stride/dst_seq_stride are the row
 * counts per head of src and dst (>= seq_len; rows [seq_len, dst_seq_stride) of
 * dst are copied unrotated from src when copy_tail != 0). */
int rfk_rope_one_oop(const rfk_half* src, rfk_half* dst,
                     const rfk_half* cos_vals, const rfk_half* sin_vals,
                     int batch, int num_heads, int seq_len, int head_dim,
                     int src_seq_stride, int dst_seq_stride, int copy_tail,
                     rfk_stream_t stream);

/* The same rotation with explicit batch strides (in elements) for src, dst and the
 * tables, so that one launch serves tensors that are not densely packed: the cached keys
 * of several decoder layers, [layer][K|V][heads][rows][head_dim], are rotated by one
 * shared table (table_batch_stride = 0) with batch = layers and src_batch_stride = two
 * cache slabs. col_scale (may be NULL): [batch][num_heads * head_dim] floats with batch stride
 * col_scale_batch_stride; the rotated value is multiplied by col_scale[b][h * head_dim + d] before its
 * one rounding to fp16 (the query's RMSNorm weight folded into the keys, see rfk_flash_attention_ex;
 * head_dim % 16 == 0 required then). Replaces one cudaMemcpyAsync + apply_rope_one pair per decoder layer —
 * src/layers/attention.cu:355-361. */
int rfk_rope_one_oop_strided(const rfk_half* src, rfk_half* dst,
                             const rfk_half* cos_vals, const rfk_half* sin_vals,
                             int batch, long long src_batch_stride, long long dst_batch_stride,
                             long long table_batch_stride, int num_heads, int seq_len,
                             int head_dim, int src_seq_stride, int dst_seq_stride,
                             const float* col_scale, long long col_scale_batch_stride,
                             rfk_stream_t stream);

/* Fused projection epilogue: for each of the n_parts (1..3) column blocks of a
 * [B*S, row_stride] fp16 GEMM output (block p starts at column p*dim), do
 *   optional RMSNorm over the full dim-wide vector (gamma[p] != NULL),
 *   [B,S,H,D] -> [B,H,S,D] transpose,
 *   optional rotate-half RoPE (use_rope[p] != 0, tables [B,1,S,D]),
 * writing out[p]. One launch instead of deinterleave_qkv + rmsnorm x2 +
 * transpose_bshd_to_bhsd x3 (+ memcpy x3) + apply_rope —
 * src/layers/attention.cu:73-85,184-210 (self), :341-361 (cross Q), :510-530 (swin).
 * Intermediate roundings match the unfused sequence (the normalised value is
 * rounded to fp16 before the rotation). gamma/out/use_rope are HOST arrays.
 * out_seq_stride: rows per head of the outputs (0 = seq_len); rows [seq_len, stride) are
 * left untouched (a padded K/V cache zeroes them once). */
int rfk_qkv_norm_rope_transpose(const rfk_half* x, long long row_stride, int n_parts,
                                const float* const* gamma, rfk_half* const* out,
                                const int* use_rope,
                                const rfk_half* cos_vals, const rfk_half* sin_vals,
                                int batch, int seq_len, int num_heads, int head_dim,
                                float eps, int out_seq_stride, rfk_stream_t stream);

/* [B,S,H,D] -> [B,H,S,D] — replaces transpose_bshd_to_bhsd, src/layers/attention.cu:17-31 */
int rfk_transpose_bshd_to_bhsd(const rfk_half* in, rfk_half* out,
                               int batch, int seq_len, int num_heads, int head_dim,
                               rfk_stream_t stream);
/* [B,H,S,D] -> [B,S,H*D] — replaces transpose_bhsd_to_bsd, src/layers/attention.cu:34-48 */
int rfk_transpose_bhsd_to_bsd(const rfk_half* in, rfk_half* out,
                              int batch, int num_heads, int seq_len, int head_dim,
                              rfk_stream_t stream);

/* ------------------------------------------------------------------ NeRF PE */

/* out[b,s,:] = [x (if include_input), sin(x_d * f_k) (d major, k minor), cos(...)] fp16,
 * f_k = 2^(min_exp + (max_exp-min_exp) * k / max(num_freqs-1,1)). num_freqs <= 32.
 * Unlike the reference wrapper this does not allocate or synchronise.
 * replaces rf::nerf_pe / rf::nerf_pe_f32 — src/kernels/nerf_pe.h:11-20,
 * src/kernels/nerf_pe.cu:9-132 */
int rfk_nerf_pe(const rfk_half* input, rfk_half* output,
                int batch, int seq_len, int in_dim, int num_freqs,
                float min_freq_exp, float max_freq_exp, int include_input,
                rfk_stream_t stream);
int rfk_nerf_pe_f32(const float* input, rfk_half* output,
                    int batch, int seq_len, int in_dim, int num_freqs,
                    float min_freq_exp, float max_freq_exp, int include_input,
                    rfk_stream_t stream);

/* ------------------------------------------------------------------ softmax */

/* In-place fp32 row softmax — replaces rf::softmax_inplace,
 * src/kernels/softmax.h:9, src/kernels/softmax.cu:7-53 */
int rfk_softmax_inplace(float* data, int rows, int cols, rfk_stream_t stream);
/* mask [mask_rows, cols] of bytes (0 = excluded), row r uses mask row r % mask_rows.
 * replaces rf::masked_softmax_inplace — src/kernels/softmax.h:13, softmax.cu:55-106 */
int rfk_masked_softmax_inplace(float* data, const uint8_t* mask, int rows, int cols,
                               int mask_rows, rfk_stream_t stream);
/* scores [BnW*H, ws2, ws2], mask [nW, ws2, ws2]; row (bh,sq) uses mask[(bh/H) % nW][sq].
 * replaces rf::swin_masked_softmax_inplace — src/kernels/softmax.h:21, softmax.cu:108-165 */
int rfk_swin_masked_softmax_inplace(float* data, const uint8_t* mask, int BnW, int num_heads,
                                    int ws2, int nW, rfk_stream_t stream);
/* fp32 scores -> fp16 probabilities, strided rows, columns [cols,out_stride) zero-filled,
 * input columns >= cols never read.
 * replaces rf::softmax_cast_fp16 — src/kernels/softmax.h:27, softmax.cu:168-248 */
int rfk_softmax_cast_fp16(const float* in, rfk_half* out, int rows, int cols,
                          int in_stride, int out_stride, rfk_stream_t stream);
/* replaces rf::softmax_cast_fp16_masked — src/kernels/softmax.h:31, softmax.cu:250-300 */
int rfk_softmax_cast_fp16_masked(const float* in, rfk_half* out, const uint8_t* mask,
                                 int rows, int cols, int in_stride, int out_stride,
                                 int mask_rows, rfk_stream_t stream);
/* softmax(scale * in): lets the caller keep alpha = 1 in the score GEMM. */
int rfk_softmax_cast_fp16_scaled(const float* in, rfk_half* out, int rows, int cols,
                                 int in_stride, int out_stride, float scale,
                                 rfk_stream_t stream);
/* softmax(scale * scores) written as fp16 OVER the score buffer: probability row r occupies
 * the first `stride` halves of fp32 row r (row pitch 2*stride halves), columns
 * [n_valid, stride) are zero. Saves the separate probability buffer the reference allocates
 * per call (cudaMallocAsync of P_half, src/layers/attention.cu:148-149). Rows up to 8192
 * columns (held in registers); longer rows return RFK_EUNSUPPORTED. */
int rfk_softmax_probs_inplace(float* scores, int rows, int n_valid, int stride, float scale,
                              rfk_stream_t stream);
/* The same for swin window scores with the optional shift mask (row pitch 2*ws2 halves). */
int rfk_swin_softmax_probs_inplace(float* scores, const uint8_t* mask, int BnW, int num_heads,
                                   int ws2, int nW, rfk_stream_t stream);
/* Swin window scores fp32 -> fp16 probabilities in one pass (mask may be NULL).
 * replaces swin_masked_softmax_inplace | softmax_inplace followed by fp32_to_fp16 —
 * src/layers/attention.cu:549-555 */
int rfk_swin_softmax_cast_fp16(const float* in, rfk_half* out, const uint8_t* mask,
                               int BnW, int num_heads, int ws2, int nW, rfk_stream_t stream);

/* ---------------------------------------------------------------- attention */

/* O = softmax(scale * Q K^T) V without materialising the scores. Q [B,H,Sq,D], K,V [B,H,Sk,D],
 * fp16, fp32 accumulation; the first n_keys (<= Sk) keys of every head take part. O is written
 * [B,H,Sq,D] or, with o_bshd != 0, [B,Sq,H*D]. D = 64 or 128 (RFK_EUNSUPPORTED otherwise).
 * replaces the contraction behind rf::sdpa — src/layers/attention.cu:89-166 (cuDNN fused
 * attention or GEMM -> softmax_cast_fp16 -> GEMM in the reference) */
int rfk_flash_attention(const rfk_half* Q, const rfk_half* K, const rfk_half* V, rfk_half* O,
                        int B, int H, int Sq, int Sk, int n_keys, int D, int o_bshd, float scale,
                        rfk_stream_t stream);

/* rfk_flash_attention with two optional extensions; tcgen05 kernel only (D = 64: RFK_EUNSUPPORTED otherwise).
 * (1) Queries that come un-normalised out of rfk_gemm_f16_heads (q_row_ss != NULL): q_row_ss [B*Sq][ss_tiles] holds the
 * partial sums of squares of each token's whole projection row (all heads); the kernel multiplies a row's scores by
 * rsqrt(sum / norm_dim + eps), which is what normalising the query first would do up to rounding. The norm's
 * per-element weight has no per-row form: the caller folds it into the keys (col_scale of rfk_rope_one_oop_strided).
 * (2) Key split (workspace != NULL): the kernel's units of work are 256 queries of one head; a grid with fewer units
 * than SMs (a 256 x 256 view has 64) leaves most of the machine idle, so with a workspace - and when the launcher's
 * estimate says it pays - the units' key ranges are cut into one share per SM and merged by the CTA that finishes a
 * unit last (nobody waits). workspace: rfk_flash_attention_workspace_bytes() bytes, 16-byte aligned, its first 1024
 * bytes zero before the first launch (the kernel leaves them zero); launches that may overlap in time need separate
 * workspaces. The result differs from the unsplit kernel's only by rounding (fp32 merge; fp16 probabilities relative to
 * each piece's own maximum) and is bit-reproducible from launch to launch.
 * (3) Shared values (v_shared != 0): V is [H, Sk, D], one set for all B batch elements - views of one scene rendered
 * together have their own queries and (rotated) keys but the same values.
 * replaces rmsnorm(Q) -> transpose -> sdpa — src/layers/attention.cu:341-349,364-366 */
int rfk_flash_attention_ex(const rfk_half* Q, const rfk_half* K, const rfk_half* V, rfk_half* O,
                           const float* q_row_ss, int ss_tiles, int norm_dim, float eps, void* workspace,
                           size_t workspace_bytes, int v_shared, int B, int H, int Sq, int Sk, int n_keys, int D,
                           int o_bshd, float scale, rfk_stream_t stream);
size_t rfk_flash_attention_workspace_bytes(void);
/* The work list rfk_flash_attention_ex would launch for `units` units (256 queries of one head each) of `n_tiles`
 * 64-key tiles on a device with `sms` SMs, given a workspace: units [0, *whole_units) run whole, then *n_pieces pieces
 * in launch order, each six values {unit, first tile, tiles, first slot of its unit, pieces of its unit, own slot}
 * written to pieces[6 i ..] for i < max_pieces. Host only: touches no device. Diagnostic; no reference counterpart. */
int rfk_flash_attention_plan(long long units, int n_tiles, int sms, int* whole_units, int* n_pieces,
                             unsigned short* pieces, int max_pieces);
/* 0: rfk_flash_attention_ex ignores its workspace (every unit whole), to time both schedules side by side; 1 (default):
 * it cuts where that pays. Process-wide. No reference counterpart. */
int rfk_flash_attention_set_split(int on);

/* Which kernel serves rfk_flash_attention at D = 64: 0 automatic (the tcgen05 / tensor-memory
 * kernel; the mma.sync kernel only if the driver cannot encode tensor maps), 1 the mma.sync kernel,
 * 2 the tcgen05 kernel or RFK_EUNSUPPORTED. Process-wide; D = 128 always takes the mma.sync kernel.
 * No reference counterpart (the reference leaves the choice to cuDNN's heuristics,
 * src/layers/attention.cu:100-140). */
int rfk_flash_attention_set_path(int path);

/* Reads (and with clear != 0 resets) the current device's error word of the tcgen05 kernel:
 * 0 none, 1 a bounded wait ran out (the CTA freed its tensor memory and returned; its output rows
 * are undefined), 2 shared memory window not 1024-byte aligned. Synchronises the device.
 * No reference counterpart. */
int rfk_flash_attention_error(int* code, int clear);

/* rfk_window_attention for Q and K that come un-normalised out of rfk_gemm_f16_heads (rows in window order):
 * q_row_ss / k_row_ss [BnW * 64][ss_tiles] partial sums of squares, gamma_q / gamma_k [num_heads * 64] the RMSNorm
 * weights; the kernel forms half((x * rsqrt(sum / norm_dim + eps)) * gamma) - the separate norm kernel's formula and
 * rounding - while it stages the tiles, then proceeds as rfk_window_attention.
 * replaces rmsnorm(Q), rmsnorm(K), the transposes and the window attention core — src/layers/attention.cu:524-566 */
int rfk_window_attention_normed(const rfk_half* Q, const rfk_half* K, const rfk_half* V, rfk_half* O,
                                const uint8_t* mask, const float* q_row_ss, const float* k_row_ss, int ss_tiles,
                                const float* gamma_q, const float* gamma_k, int norm_dim, float eps, int BnW,
                                int num_heads, int window_tokens, int head_dim, int nW, float scale,
                                rfk_stream_t stream);

/* ---------------------------------------------------------------- dense projections
 * C[M,N] = epilogue(A[M,K] W[N,K]^T): row-major fp16 operands with row pitches lda, ldw, ldc
 * (elements), fp32 accumulation on the tcgen05 tensor cores (accumulators in tensor memory,
 * operand tiles by TMA), one rounding to fp16 in the epilogue:
 *   RFK_GEMM_EPI_NONE      C = A W^T, + bias[N] if bias != NULL (the product is rounded to fp16
 *                          before the bias is added, as the unfused GEMM + bias kernel does)
 *   RFK_GEMM_EPI_RESIDUAL  C = A W^T (+ bias) + R, R [M,N] fp16 with pitch ldr; R may be C (in place)
 *   RFK_GEMM_EPI_SWIGLU    C = silu(A W^T) * (A W_up^T), W and W_up both [N,K] with pitch ldw: the
 *                          gate and up projections of a SwiGLU feed-forward and its activation in
 *                          one kernel; no [M, 2N] intermediate exists. bias must be NULL.
 * Needs 16-byte aligned pointers, pitches, N and K multiples of 8 (RFK_EUNSUPPORTED otherwise, and
 * when the path is set to 1 below; callers then use their library GEMM). A kernel that gives up on
 * a bounded wait reports through rfk_gemm_error.
 * replaces rf::linear (cublasGemmEx + add_bias) — src/layers/linear.h:9, src/layers/linear.cu:7-25 —
 * and, with the SwiGLU epilogue, the first two GEMMs + fused_silu_mul of rf::ffn_swiglu —
 * src/layers/transformer.cu:63-76; with the residual epilogue the GEMM + rf::residual_add pairs of
 * src/layers/transformer.cu:176-192. */
enum { RFK_GEMM_EPI_NONE = 0, RFK_GEMM_EPI_RESIDUAL = 1, RFK_GEMM_EPI_SWIGLU = 2 };
int rfk_gemm_f16(const rfk_half* A, long long lda, const rfk_half* W, long long ldw,
                 const rfk_half* W_up, const rfk_half* bias, const rfk_half* R, long long ldr,
                 rfk_half* C, long long ldc, int M, int N, int K, int epilogue,
                 rfk_stream_t stream);
/* Projection whose output feeds an attention: C = A W^T stored head-split and the statistic of the QK-RMSNorm that
 * follows computed on the way, so that no separate norm / head-split kernel runs. N = parts * num_heads * 64 columns
 * (parts = 1: a query projection; 3: packed q | k | v); rows are M = groups * seq_len tokens. Output: part p at
 * out + p * part_stride (elements), each part [groups][num_heads][seq_len][64] fp16. row_ss (may be NULL if
 * ss_parts_mask == 0): [parts][M][num_heads * 64 / 256] floats; entry (p, row, t) = sum of squares of the fp16-rounded
 * outputs of that row in columns [256 t, 256 t + 256) of part p, written (not accumulated, no zeroing needed, bit-
 * reproducible) for the parts whose bit is set in ss_parts_mask; the consumer adds the entries of a row and applies
 * rsqrt(sum / dim + eps) and the norm weight while it loads (rfk_flash_attention_ex, rfk_window_attention_normed).
 * CTA-pair tcgen05 kernel only: RFK_EUNSUPPORTED (nothing launched) unless num_heads % 4 == 0, seq_len % 32 == 0,
 * M % seq_len == 0 and the alignment rules of rfk_gemm_f16 hold; callers then run the projection and
 * rfk_qkv_norm_rope_transpose separately.
 * replaces linear -> (deinterleave_qkv) -> rmsnorm -> transpose_bshd_to_bhsd — src/layers/attention.cu:180-206,336-349,
 * 511-535 — up to the point where the normalised values are formed. */
int rfk_gemm_f16_heads(const rfk_half* A, long long lda, const rfk_half* W, long long ldw, rfk_half* out,
                       long long part_stride, float* row_ss, int ss_parts_mask, int M, int N, int K,
                       int seq_len, int num_heads, rfk_stream_t stream);
/* 0 automatic (the tcgen05 kernel whenever the shape allows: on CTA pairs, tcgen05.mma.cta_group::2,
 * or on single CTAs if the device cannot co-schedule pairs), 1 never (rfk_gemm_f16 returns
 * RFK_EUNSUPPORTED, so the layer functions fall back to their cuBLAS calls: used to time both side
 * by side), 2 as 0, 3 the single-CTA kernel. Process-wide; the environment variable RFK_GEMM_PATH
 * sets the initial value. No reference counterpart. */
int rfk_gemm_set_path(int path);
/* CTA pairs (clusters of two) that the current device runs at once for the pair kernel, as the
 * occupancy query answered at the first launch: 0 before any launch, -1 if pairs cannot be scheduled
 * (the single-CTA kernel then serves every call). Diagnostic. No reference counterpart. */
int rfk_gemm_pair_clusters(void);
/* Reads (and with clear != 0 resets) the current device's error word of the GEMM kernel: 0 none,
 * 1 a bounded wait ran out, 2 shared memory window not 1024-byte aligned. Synchronises the device.
 * No reference counterpart. */
int rfk_gemm_error(int* code, int clear);

/* Swin window attention core in one kernel: per (window, head) O = softmax(scale * Q K^T [masked]) V.
 * Q, K, V [BnW, heads, 64, 64] fp16; O [BnW * 64, heads * 64] fp16 (token-major, what the output
 * projection reads); mask [nW, 64, 64] bytes or NULL, byte 0 = pair masked out (score replaced by
 * -FLT_MAX before the softmax), window index = bw % nW. window_tokens = 64 and head_dim = 64 only
 * (RFK_EUNSUPPORTED otherwise: callers then use the GEMM -> rfk_swin_softmax_probs_inplace -> GEMM path).
 * replaces the batched GEMM -> swin_masked_softmax_inplace | softmax_inplace -> fp32_to_fp16 ->
 * batched GEMM -> transpose_bhsd_to_bsd sequence of rf::swin_self_attention —
 * src/layers/attention.cu:542-566 */
int rfk_window_attention(const rfk_half* Q, const rfk_half* K, const rfk_half* V, rfk_half* O,
                         const uint8_t* mask, int BnW, int num_heads, int window_tokens, int head_dim,
                         int nW, float scale, rfk_stream_t stream);

/* -------------------------------------------------------------- activations */

/* out = half(silu(a) * b), out may alias a — replaces rf::fused_silu_mul,
 * src/kernels/activations.h:8, activations.cu:5-21 */
int rfk_fused_silu_mul(const rfk_half* a, const rfk_half* b, rfk_half* out, long long n,
                       rfk_stream_t stream);
/* replaces rf::fused_silu_mul_f32 — activations.h:12, activations.cu:23-36 */
int rfk_fused_silu_mul_f32(const float* a, const float* b, float* out, long long n,
                           rfk_stream_t stream);
/* SwiGLU on one concatenated GEMM output: gate_up [rows, 2*hidden] (gate | up per row),
 * out [rows, hidden] = half(silu(gate) * up). Serves a single w1||w3 GEMM in place of the
 * two GEMMs + fused_silu_mul of rf::ffn_swiglu, src/layers/transformer.cu:63-79. */
int rfk_swiglu(const rfk_half* gate_up, rfk_half* out, int rows, int hidden,
               rfk_stream_t stream);
/* The same, writing out over the gate half of each row (row pitch 2*hidden): the W2 GEMM
 * then reads it with lda = 2*hidden and no separate activation buffer is needed. */
int rfk_swiglu_inplace(rfk_half* gate_up, int rows, int hidden, rfk_stream_t stream);
/* y = x > 0 ? x : alpha*(exp(x)-1), fp16, in place allowed — replaces rf::elu,
 * activations.h:16, activations.cu:38-50 */
int rfk_elu(const rfk_half* x, rfk_half* y, long long n, float alpha, rfk_stream_t stream);
/* y = 10^x - 1 fp32, in place allowed — replaces rf::pow10_minus1,
 * activations.h:20, activations.cu:52-63 */
int rfk_pow10_minus1(const float* x, float* y, long long n, rfk_stream_t stream);

/* ---- element-wise / layout operators of the DPT head (src/layers/dpt.h, dpt.cu); the convolutions of
 * the head are library calls in the reference and are not part of this library ---- */
/* [N,C,H_in,W_in] -> [N,C,H_out,W_out] fp16, bilinear, align_corners = true, the reference's
 * expression term for term — replaces rf::bilinear_upsample, dpt.h:29-31, dpt.cu:240-286 */
int rfk_bilinear_upsample(const rfk_half* in, rfk_half* out, int N, int C, int H_in, int W_in,
                          int H_out, int W_out, rfk_stream_t stream);
/* x = x * sigmoid(x) in place, fp16 — replaces rf::silu_inplace, dpt.h:34, dpt.cu:289-301 */
int rfk_silu_inplace(rfk_half* x, long long n, rfk_stream_t stream);
/* x[n,c,:] += bias[c] over [N,C,HW] fp16 (one rounding) — replaces add_bias_nchw_kernel,
 * dpt.cu:88-96 (file-local in the reference, launched from conv2d / conv_transpose2d) */
int rfk_add_bias_nchw(rfk_half* x, const rfk_half* bias, int N, int C, long long HW,
                      rfk_stream_t stream);
/* [B,S,D] -> [B,D,S] (= [B,D,pH,pW] with S = pH*pW) — replaces permute_bsd_to_nchw,
 * dpt.cu:303-318 (file-local in the reference, launched from dpt_forward) */
int rfk_permute_bsd_to_nchw(const rfk_half* in, rfk_half* out, int B, int S, int D,
                            rfk_stream_t stream);

/* Channels-last ([N,H,W,C] fp16, C % 8 == 0, 16-byte aligned; RFK_EUNSUPPORTED otherwise) companions of the four
 * operators above: the layout the DPT head runs on (csrc/dpt.cu), where the token maps need no permute, the library's
 * tensor-core convolutions take their operands as they are and a 1x1 convolution is rfk_linear. Values are bit-identical
 * to the NCHW operators applied one after the other (every intermediate is still rounded to fp16).
 * No reference counterpart as functions: they stand for the same lines of src/layers/dpt.cu in another layout. */
/* x[r,c] = act(half(x[r,c] + bias[c])) (+ residual[r,c]) in place over [rows, C]; bias and residual may be NULL,
 * silu != 0 applies x * sigmoid(x): add_bias_nchw (+ silu_inplace) (+ residual_add) in one pass — dpt.cu:88-96,
 * :289-298, :397-409 */
int rfk_bias_act_residual_nhwc(rfk_half* x, const rfk_half* bias, const rfk_half* residual, long long rows, int C,
                               int silu, rfk_stream_t stream);
/* y = x * sigmoid(x), out of place (n % 8 == 0): saves the copy the reference's in-place form needs before a residual
 * unit — dpt.cu:397-400 */
int rfk_silu(const rfk_half* x, rfk_half* y, long long n, rfk_stream_t stream);
/* [N,H_in,W_in,C] -> [N,H_out,W_out,C], bilinear, align_corners = true, the reference's expression term for term —
 * dpt.cu:240-286 */
int rfk_bilinear_upsample_nhwc(const rfk_half* in, rfk_half* out, int N, int H_in, int W_in, int H_out, int W_out, int C,
                               rfk_stream_t stream);
/* Second half of a transposed convolution whose stride equals its kernel size f (the head's x4 and x2 resize layers,
 * dpt.cu:182-236, :372-380): in [N*H*W, f*f*C] is the GEMM of the input pixels with the filter laid out by
 * rfk_permute_filter(mode 1); out [N, H*f, W*f, C] = the scattered pixels + bias[c] (bias may be NULL). */
int rfk_depth_to_space_bias_nhwc(const rfk_half* in, const rfk_half* bias, rfk_half* out, int N, int H, int W, int C, int f,
                                 rfk_stream_t stream);
/* [N, HW, C] -> [N, C, HW], any C (the head's last layer, C = 3) */
int rfk_permute_nhwc_to_nchw(const rfk_half* in, rfk_half* out, int N, long long HW, int C, rfk_stream_t stream);
/* The head's last layer in one launch: 1x1 convolution from C_in channels-last channels (C_in % 8 == 0, <= 2048) to
 * C_out <= 4 planes + bias: in [N*HW, C_in], weight [C_out, C_in], out [N, C_out, HW] (RFK_EUNSUPPORTED otherwise:
 * callers then use rfk_linear + rfk_permute_nhwc_to_nchw). fp32 accumulation, product rounded to fp16 before the bias.
 * replaces conv2d (1x1, cuBLAS) + add_bias_nchw at the end of rf::dpt_forward — dpt.cu:112-126, :456-459 */
int rfk_pointwise_conv_to_planar(const rfk_half* in, const rfk_half* weight, const rfk_half* bias, rfk_half* out, int N,
                                 long long HW, int C_in, int C_out, rfk_stream_t stream);
/* One-off filter layouts for the channels-last head. mode 0: convolution filter [K, C, RS] -> [K, RS, C]; mode 1:
 * transposed-convolution filter [Cin = K, Cout = C, RS = f*f] -> GEMM weight [(p * Cout + co), ci]. */
int rfk_permute_filter(const rfk_half* w, rfk_half* out, int K, int C, int RS, int mode, rfk_stream_t stream);

/* y32 = 10^float(half(elu(x16))) - 1 in one launch — replaces the chain
 * elu -> k_fp16_to_fp32_s -> pow10_minus1, src/pipeline/render_session.cu:249-253 */
int rfk_post_elu_pow10(const rfk_half* x, float* y, long long n, float alpha,
                       rfk_stream_t stream);

/* ------------------------------------------------- per-view ray front end */

/* Pinhole rays: c2w [B,4,4] fp32 row-major, fov [B] radians, rays_o [B,3] fp32,
 * rays_d [B,res,res,3] fp16 unit directions. Bit-identical to the reference kernel.
 * replaces rf::ray_gen — src/kernels/ray_gen.h:11, ray_gen.cu:6-53 */
int rfk_ray_gen(const float* c2w, const float* fov, float* rays_o, rfk_half* rays_d,
                int batch, int img_res, rfk_stream_t stream);
/* Same rays written directly as patch tokens [B, (res/ps)^2, 3*ps*ps]
 * (feature = c*ps*ps + p1*ps + p2). rays_o may be NULL.
 * replaces ray_gen + k_patchify_s — src/pipeline/render_session.cu:48-59,207-212 */
int rfk_ray_gen_patchify(const float* c2w, const float* fov, float* rays_o, rfk_half* ray_pat,
                         int batch, int img_res, int patch_size, rfk_stream_t stream);
/* [H,W,C] -> [pH*pW, C*ps*ps] — replaces k_patchify_s, render_session.cu:48-59 */
int rfk_patchify(const rfk_half* in, rfk_half* out, int H, int W, int C, int ps,
                 rfk_stream_t stream);

/* In place: tri <- R^T (v - t), vn <- R^T n; tri, vn [B,N,3,3] fp16 (vn may be NULL).
 * Bit-identical to the reference kernel.
 * replaces rf::world_to_cam — src/kernels/coord_transform.h:12, coord_transform.cu:7-55 */
int rfk_world_to_cam(const float* c2w, rfk_half* tri, rfk_half* vn, int batch, int n_tris,
                     rfk_stream_t stream);
/* fp32 storage variant of the same transform on [B, n_verts, 3] arrays (normals may be NULL). */
int rfk_world_to_cam_f32(const float* c2w, float* verts, float* normals, int batch, int n_verts,
                         rfk_stream_t stream);
/* Per-view geometry front end in one launch (single camera):
 *   vtri = world_to_cam(tri_world), vvn = world_to_cam_normals(vn_world)  [N,3,3] fp16
 *   vpos[0:nr]    = camera-space scene centre repeated 3x               [nr,9]
 *   vpos[nr:nr+N] = vtri ; vpos[nr+N : seq_pad] = 0
 *   k_cos,k_sin [seq_pad, head_dim] = triangle RoPE tables of vpos
 * replaces 2 D2D copies + world_to_cam + k_center_pos_from_c2w + D2D copy +
 * triangle_rope_freqs — src/pipeline/render_session.cu:73-88,192-203.
 * vvn / vn_world may be NULL. */
int rfk_view_geometry(const float* c2w, const rfk_half* tri_world, const rfk_half* vn_world,
                      const float* world_center, const float* learned_freqs,
                      rfk_half* vtri, rfk_half* vvn, rfk_half* vpos,
                      rfk_half* k_cos, rfk_half* k_sin,
                      int n_tris, int n_register, int seq_pad, int num_freqs, int head_dim,
                      rfk_stream_t stream);

/* ----------------------------------------------------- swin window layout */

/* windows[b*nW + wh*(W/ws) + ww][lh*ws+lw][:] = x[b][(h-shift) mod H][(w-shift) mod W][:],
 * h = wh*ws+lh, w = ww*ws+lw: cyclic_shift_2d(-shift) then window partition, one launch.
 * replaces cyclic_shift_2d(-s) + window_partition — src/layers/attention.cu:377-407,443-472,498-505 */
int rfk_window_gather(const rfk_half* x, rfk_half* windows, int B, int H, int W, int C,
                      int ws, int shift, rfk_stream_t stream);
/* Inverse of rfk_window_gather (window reverse then cyclic shift by +shift).
 * If residual_into != 0, x = half(float(x) + float(value)) instead of x = value.
 * replaces window_reverse + cyclic_shift_2d(+s) (+ residual_add) —
 * src/layers/attention.cu:409-439,569-575; src/layers/transformer.cu:188 */
int rfk_window_scatter(const rfk_half* windows, rfk_half* x, int B, int H, int W, int C,
                       int ws, int shift, int residual_into, rfk_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* RFK_H */
