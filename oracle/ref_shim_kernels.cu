// Test infrastructure: extern "C" doors onto the reference engine's src/kernels functions
// (C++ linkage, namespace rf), so that a test harness can call the reference's own CUDA
// kernels through ctypes. Compiled together with the reference's unmodified sources by
// oracle/Makefile into oracle/_ref/libref_kernels.so. Not part of the product.
#include "kernels/activations.h"
#include "kernels/coord_transform.h"
#include "kernels/nerf_pe.h"
#include "kernels/ray_gen.h"
#include "kernels/rmsnorm.h"
#include "kernels/rope.h"
#include "kernels/softmax.h"

#define S(s) reinterpret_cast<cudaStream_t>(s)

extern "C" {

void ref_rmsnorm(const half* x, const float* g, half* y, int rows, int dim, float eps, void* s) {
    rf::rmsnorm(x, g, y, rows, dim, eps, S(s));
}
void ref_rmsnorm_f32(const float* x, const float* g, float* y, int rows, int dim, float eps, void* s) {
    rf::rmsnorm_f32(x, g, y, rows, dim, eps, S(s));
}
void ref_triangle_rope_freqs(const half* pos, const float* f, half* c, half* sn, int batch, int seq,
                             int nf, int hd, void* s) {
    rf::triangle_rope_freqs(pos, f, c, sn, batch, seq, nf, hd, S(s));
}
void ref_apply_rope(half* q, half* k, const half* c, const half* sn, int b, int h, int seq, int hd,
                    void* s) {
    rf::apply_rope(q, k, c, sn, b, h, seq, hd, S(s));
}
void ref_apply_rope_one(half* x, const half* c, const half* sn, int b, int h, int seq, int hd, void* s) {
    rf::apply_rope_one(x, c, sn, b, h, seq, hd, S(s));
}
void ref_apply_rope_f32(float* q, float* k, const half* c, const half* sn, int b, int h, int seq,
                        int hd, void* s) {
    rf::apply_rope_f32(q, k, c, sn, b, h, seq, hd, S(s));
}
void ref_apply_rope_one_f32(float* x, const half* c, const half* sn, int b, int h, int seq, int hd,
                            void* s) {
    rf::apply_rope_one_f32(x, c, sn, b, h, seq, hd, S(s));
}
// note: the reference wrappers allocate, copy and free a device table on every call
void ref_nerf_pe(const half* in, half* out, int b, int seq, int in_dim, int nf, float mn, float mx,
                 int inc, void* s) {
    rf::nerf_pe(in, out, b, seq, in_dim, nf, mn, mx, inc != 0, S(s));
}
void ref_nerf_pe_f32(const float* in, half* out, int b, int seq, int in_dim, int nf, float mn,
                     float mx, int inc, void* s) {
    rf::nerf_pe_f32(in, out, b, seq, in_dim, nf, mn, mx, inc != 0, S(s));
}
void ref_softmax_inplace(float* d, int rows, int cols, void* s) { rf::softmax_inplace(d, rows, cols, S(s)); }
void ref_masked_softmax_inplace(float* d, const bool* m, int rows, int cols, int mr, void* s) {
    rf::masked_softmax_inplace(d, m, rows, cols, mr, S(s));
}
void ref_swin_masked_softmax_inplace(float* d, const bool* m, int BnW, int heads, int ws2, int nW,
                                     void* s) {
    rf::swin_masked_softmax_inplace(d, m, BnW, heads, ws2, nW, S(s));
}
void ref_softmax_cast_fp16(const float* in, half* out, int rows, int cols, int is, int os, void* s) {
    rf::softmax_cast_fp16(in, out, rows, cols, is, os, S(s));
}
void ref_softmax_cast_fp16_masked(const float* in, half* out, const bool* m, int rows, int cols,
                                  int is, int os, int mr, void* s) {
    rf::softmax_cast_fp16_masked(in, out, m, rows, cols, is, os, mr, S(s));
}
void ref_fused_silu_mul(const half* a, const half* b, half* o, int n, void* s) {
    rf::fused_silu_mul(a, b, o, n, S(s));
}
void ref_fused_silu_mul_f32(const float* a, const float* b, float* o, int n, void* s) {
    rf::fused_silu_mul_f32(a, b, o, n, S(s));
}
void ref_elu(const half* x, half* y, int n, float alpha, void* s) { rf::elu(x, y, n, alpha, S(s)); }
void ref_pow10_minus1(const float* x, float* y, int n, void* s) { rf::pow10_minus1(x, y, n, S(s)); }
void ref_ray_gen(const float* c2w, const float* fov, float* ro, half* rd, int b, int res, void* s) {
    rf::ray_gen(c2w, fov, ro, rd, b, res, S(s));
}
void ref_world_to_cam(const float* c2w, half* tri, half* vn, int b, int n, void* s) {
    rf::world_to_cam(c2w, tri, vn, b, n, S(s));
}

}  // extern "C"
