/*
 * rfk_compat.h — the reference engine's kernel interface (namespace rf, C++ linkage, CUDA
 * `half`, cudaStream_t last with a default) as inline forwards onto the rfk C ABI.
 *
 * Host code written against the reference's src/kernels/{rmsnorm,rope,nerf_pe,softmax,
 * activations,ray_gen,coord_transform}.h and the helper declarations of
 * src/layers/transformer.h:104-116 compiles against this header unchanged and links
 * librfk.so instead of the reference's src/kernels/*.cu.
 *
 * The reference's functions return void and its callers check nothing; build with
 * -DRFK_COMPAT_CHECK to print the status text and exit(1) on failure, the behaviour of the
 * reference's CHECK_CUDA macro (src/core/cuda_utils.h:8-16).
 */
#ifndef RFK_COMPAT_H
#define RFK_COMPAT_H

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "rfk.h"

#ifdef RFK_COMPAT_CHECK
#include <cstdio>
#include <cstdlib>
#define RFK_COMPAT_CALL(expr)                                                          \
    do {                                                                               \
        int rfk_rc_ = (expr);                                                          \
        if (rfk_rc_ != RFK_OK) {                                                       \
            std::fprintf(stderr, "rfk error at %s:%d: %s\n", __FILE__, __LINE__,       \
                         rfk_status_string(rfk_rc_));                                  \
            std::exit(1);                                                              \
        }                                                                              \
    } while (0)
#else
#define RFK_COMPAT_CALL(expr) (void)(expr)
#endif

namespace rf {

constexpr float kEpsFp16 = 0.0009765625f;   /* src/kernels/rmsnorm.h:9  */
constexpr float kEpsFp32 = 1.1920929e-07f;  /* src/kernels/rmsnorm.h:10 */

namespace rfk_detail {
inline rfk_half* h(half* p) { return reinterpret_cast<rfk_half*>(p); }
inline const rfk_half* h(const half* p) { return reinterpret_cast<const rfk_half*>(p); }
inline const uint8_t* m(const bool* p) { return reinterpret_cast<const uint8_t*>(p); }
}  // namespace rfk_detail

/* src/kernels/rmsnorm.h:13-20 */
inline void rmsnorm(const half* x, const float* gamma, half* y, int rows, int dim, float eps = kEpsFp16,
                    cudaStream_t stream = nullptr) {
    RFK_COMPAT_CALL(rfk_rmsnorm(rfk_detail::h(x), gamma, rfk_detail::h(y), rows, dim, eps, stream));
}
inline void rmsnorm_f32(const float* x, const float* gamma, float* y, int rows, int dim, float eps = kEpsFp32,
                        cudaStream_t stream = nullptr) {
    RFK_COMPAT_CALL(rfk_rmsnorm_f32(x, gamma, y, rows, dim, eps, stream));
}

/* src/kernels/rope.h:12-36 */
inline void triangle_rope_freqs(const half* pos, const float* learned_freqs, half* out_cos, half* out_sin, int batch,
                                int seq_len, int num_freqs, int head_dim, cudaStream_t stream = nullptr) {
    RFK_COMPAT_CALL(rfk_triangle_rope_freqs(rfk_detail::h(pos), learned_freqs, rfk_detail::h(out_cos),
                                            rfk_detail::h(out_sin), batch, seq_len, num_freqs, head_dim, stream));
}
inline void apply_rope(half* q, half* k, const half* cos_vals, const half* sin_vals, int batch, int num_heads,
                       int seq_len, int head_dim, cudaStream_t stream = nullptr) {
    RFK_COMPAT_CALL(rfk_apply_rope(rfk_detail::h(q), rfk_detail::h(k), rfk_detail::h(cos_vals),
                                   rfk_detail::h(sin_vals), batch, num_heads, seq_len, head_dim, stream));
}
inline void apply_rope_one(half* x, const half* cos_vals, const half* sin_vals, int batch, int num_heads,
                           int seq_len, int head_dim, cudaStream_t stream = nullptr) {
    RFK_COMPAT_CALL(rfk_apply_rope_one(rfk_detail::h(x), rfk_detail::h(cos_vals), rfk_detail::h(sin_vals), batch,
                                       num_heads, seq_len, head_dim, stream));
}
inline void apply_rope_f32(float* q, float* k, const half* cos_vals, const half* sin_vals, int batch,
                           int num_heads, int seq_len, int head_dim, cudaStream_t stream = nullptr) {
    RFK_COMPAT_CALL(rfk_apply_rope_f32(q, k, rfk_detail::h(cos_vals), rfk_detail::h(sin_vals), batch, num_heads,
                                       seq_len, head_dim, stream));
}
inline void apply_rope_one_f32(float* x, const half* cos_vals, const half* sin_vals, int batch, int num_heads,
                               int seq_len, int head_dim, cudaStream_t stream = nullptr) {
    RFK_COMPAT_CALL(rfk_apply_rope_one_f32(x, rfk_detail::h(cos_vals), rfk_detail::h(sin_vals), batch, num_heads,
                                           seq_len, head_dim, stream));
}

/* src/kernels/nerf_pe.h:11-20 */
inline void nerf_pe(const half* input, half* output, int batch, int seq_len, int in_dim, int num_freqs,
                    float min_freq_exp, float max_freq_exp, bool include_input, cudaStream_t stream = nullptr) {
    RFK_COMPAT_CALL(rfk_nerf_pe(rfk_detail::h(input), rfk_detail::h(output), batch, seq_len, in_dim, num_freqs,
                                min_freq_exp, max_freq_exp, include_input ? 1 : 0, stream));
}
inline void nerf_pe_f32(const float* input, half* output, int batch, int seq_len, int in_dim, int num_freqs,
                        float min_freq_exp, float max_freq_exp, bool include_input, cudaStream_t stream = nullptr) {
    RFK_COMPAT_CALL(rfk_nerf_pe_f32(input, rfk_detail::h(output), batch, seq_len, in_dim, num_freqs, min_freq_exp,
                                    max_freq_exp, include_input ? 1 : 0, stream));
}

/* src/kernels/softmax.h:9-33 */
inline void softmax_inplace(float* data, int rows, int cols, cudaStream_t stream = nullptr) {
    RFK_COMPAT_CALL(rfk_softmax_inplace(data, rows, cols, stream));
}
inline void masked_softmax_inplace(float* data, const bool* mask, int rows, int cols, int mask_rows,
                                   cudaStream_t stream = nullptr) {
    RFK_COMPAT_CALL(rfk_masked_softmax_inplace(data, rfk_detail::m(mask), rows, cols, mask_rows, stream));
}
inline void swin_masked_softmax_inplace(float* data, const bool* mask, int BnW, int num_heads, int ws2, int nW,
                                        cudaStream_t stream = nullptr) {
    RFK_COMPAT_CALL(rfk_swin_masked_softmax_inplace(data, rfk_detail::m(mask), BnW, num_heads, ws2, nW, stream));
}
inline void softmax_cast_fp16(const float* in, half* out, int rows, int cols, int in_stride, int out_stride,
                              cudaStream_t stream = nullptr) {
    RFK_COMPAT_CALL(rfk_softmax_cast_fp16(in, rfk_detail::h(out), rows, cols, in_stride, out_stride, stream));
}
inline void softmax_cast_fp16_masked(const float* in, half* out, const bool* mask, int rows, int cols,
                                     int in_stride, int out_stride, int mask_rows, cudaStream_t stream = nullptr) {
    RFK_COMPAT_CALL(rfk_softmax_cast_fp16_masked(in, rfk_detail::h(out), rfk_detail::m(mask), rows, cols, in_stride,
                                                 out_stride, mask_rows, stream));
}

/* src/kernels/activations.h:8-21 */
inline void fused_silu_mul(const half* a, const half* b, half* out, int n, cudaStream_t stream = nullptr) {
    RFK_COMPAT_CALL(rfk_fused_silu_mul(rfk_detail::h(a), rfk_detail::h(b), rfk_detail::h(out), n, stream));
}
inline void fused_silu_mul_f32(const float* a, const float* b, float* out, int n, cudaStream_t stream = nullptr) {
    RFK_COMPAT_CALL(rfk_fused_silu_mul_f32(a, b, out, n, stream));
}
inline void elu(const half* x, half* y, int n, float alpha = 1e-3f, cudaStream_t stream = nullptr) {
    RFK_COMPAT_CALL(rfk_elu(rfk_detail::h(x), rfk_detail::h(y), n, alpha, stream));
}
inline void pow10_minus1(const float* x, float* y, int n, cudaStream_t stream = nullptr) {
    RFK_COMPAT_CALL(rfk_pow10_minus1(x, y, n, stream));
}

/* src/layers/dpt.h:29-34 (the element-wise operators of the DPT head; its convolutions stay library calls) */
inline void bilinear_upsample(const half* in, half* out, int N, int C, int H_in, int W_in, int H_out, int W_out,
                              cudaStream_t stream = nullptr) {
    RFK_COMPAT_CALL(rfk_bilinear_upsample(rfk_detail::h(in), rfk_detail::h(out), N, C, H_in, W_in, H_out, W_out, stream));
}
inline void silu_inplace(half* x, int n, cudaStream_t stream = nullptr) {
    RFK_COMPAT_CALL(rfk_silu_inplace(rfk_detail::h(x), n, stream));
}

/* src/kernels/ray_gen.h:11 */
inline void ray_gen(const float* c2w, const float* fov, float* rays_o, half* rays_d, int batch, int img_res,
                    cudaStream_t stream = nullptr) {
    RFK_COMPAT_CALL(rfk_ray_gen(c2w, fov, rays_o, rfk_detail::h(rays_d), batch, img_res, stream));
}

/* src/kernels/coord_transform.h:12 */
inline void world_to_cam(const float* c2w, half* tri, half* vn, int batch, int n_tris, cudaStream_t stream = nullptr) {
    RFK_COMPAT_CALL(rfk_world_to_cam(c2w, rfk_detail::h(tri), rfk_detail::h(vn), batch, n_tris, stream));
}

/* src/layers/transformer.h:104-116 */
inline void residual_add(half* y, const half* residual, int n, cudaStream_t stream = nullptr) {
    RFK_COMPAT_CALL(rfk_residual_add(rfk_detail::h(y), rfk_detail::h(residual), n, stream));
}
inline void residual_add_f32(float* y, const float* residual, int n, cudaStream_t stream = nullptr) {
    RFK_COMPAT_CALL(rfk_residual_add_f32(y, residual, n, stream));
}
inline void residual_add_mixed(float* y, const half* residual, int n, cudaStream_t stream = nullptr) {
    RFK_COMPAT_CALL(rfk_residual_add_mixed(y, rfk_detail::h(residual), n, stream));
}
inline void cast_fp32_to_fp16(const float* in, half* out, int n, cudaStream_t stream = nullptr) {
    RFK_COMPAT_CALL(rfk_cast_fp32_to_fp16(in, rfk_detail::h(out), n, stream));
}
inline void cast_fp16_to_fp32(const half* in, float* out, int n, cudaStream_t stream = nullptr) {
    RFK_COMPAT_CALL(rfk_cast_fp16_to_fp32(rfk_detail::h(in), out, n, stream));
}

}  // namespace rf

#endif /* RFK_COMPAT_H */
