// Pinhole ray generation, optionally written directly as 8x8 patch tokens.
//
// Reference semantics (BANANASJIM/renderformer-cuda, src/kernels/ray_gen.cu:25-44):
//   cx = res*0.5 ; fx = cx / tanf(0.5*fov) ; x = (px+0.5-cx)/fx ; y = -(py+0.5-cx)/fx ; z = -1
//   d = R*(x,y,z), sums in the order M0*x + M1*y + M2*z ; d *= rsqrtf(d.d) ; 3 halves per pixel
//   rays_o = c2w[:3,3]
// and src/pipeline/render_session.cu:48-59 for the patch layout
//   token = patch (row-major), feature = c*ps*ps + p1*ps + p2.
//
// The per-pixel arithmetic below is written with the same expression trees as the
// reference so that the compiler contracts the same multiply-adds: the outputs are
// required to be bit-identical. What changes is the memory side: the reference issues
// three 2-byte stores per thread at a 6-byte stride; here a thread computes 8 consecutive
// pixels of a row and emits three 128-bit stores (48 contiguous bytes in pixel order, or
// one 16-byte patch row per channel in token order), and it reuses tanf and the per-column
// divisions across 4 rows.
#include "common.cuh"

namespace rfk {

struct Ray3 { float x, y, z; };

// x, y: camera-plane coordinates (px+0.5-cx)/fx and -(py+0.5-cx)/fx of the pixel
template <typename Mat>
__device__ __forceinline__ Ray3 rotate_normalize(const Mat& M, float x, float y) {
    float z = -1.0f;
    float dx = M[0] * x + M[1] * y + M[2] * z;
    float dy = M[4] * x + M[5] * y + M[6] * z;
    float dz = M[8] * x + M[9] * y + M[10] * z;
    float inv_len = rsqrtf(dx * dx + dy * dy + dz * dz);
    dx *= inv_len; dy *= inv_len; dz *= inv_len;
    return Ray3{dx, dy, dz};
}

__device__ __forceinline__ Ray3 pixel_ray(const float* __restrict__ M, float cx, float fx, int px,
                                          int py) {
    float x = (px + 0.5f - cx) / fx;
    float y = -(py + 0.5f - cx) / fx;
    return rotate_normalize(M, x, y);
}


// A thread owns an 8-pixel-wide, ROWS-tall strip: the 8 x-coordinates (8 IEEE divisions) and
// tanf are computed once and reused for every row. ROWS = 4 keeps the kernel HBM-bound when
// many views are batched; ROWS = 1 gives a single view 4x the threads and the shortest
// critical path. PATCH == 0: rays_d [B,res,res,3]; PATCH == 1: tokens [B,(res/8)^2,192]
// (requires ps == 8).
// COALESCE (PATCH == 0, res a multiple of 256): the 32 lanes of a warp own 256 consecutive pixels of a
// row, 1536 contiguous output bytes; each lane's 48 bytes go through shared memory so that every store
// instruction of the warp writes 512 contiguous bytes instead of 16-byte pieces 48 bytes apart.
template <int PATCH, int ROWS, int COALESCE = 0>
__global__ void __launch_bounds__(256)
ray_gen_vec_kernel(const float* __restrict__ c2w, const float* __restrict__ fov,
                   float* __restrict__ rays_o, __half* __restrict__ out, int batch, int res) {
    __shared__ __align__(16) unsigned char s_stage[COALESCE ? 8 * 1536 : 16];
    const int groups_per_row = res / 8;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long per_image = (long long)groups_per_row * (res / ROWS);
    if (idx >= per_image * batch) return;
    const int b = (int)(idx / per_image);
    const int rem = (int)(idx % per_image);
    const int py0 = (rem / groups_per_row) * ROWS;
    const int px0 = (rem % groups_per_row) * 8;
    float M[11];  // the rotation rows, kept in registers for the whole strip
#pragma unroll
    for (int i = 0; i < 11; ++i) M[i] = __ldg(c2w + b * 16 + i);
    if (rem == 0 && rays_o) {
        rays_o[b * 3 + 0] = M[3];
        rays_o[b * 3 + 1] = M[7];
        rays_o[b * 3 + 2] = __ldg(c2w + b * 16 + 11);
    }
    const float cx = res * 0.5f;
    const float fx = cx / tanf(0.5f * __ldg(fov + b));
    float xs[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) xs[i] = (px0 + i + 0.5f - cx) / fx;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const int py = py0 + r;
        const float y = -(py + 0.5f - cx) / fx;
        __align__(16) __half h[24];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const Ray3 d = rotate_normalize(M, xs[i], y);
            if (PATCH) {  // channel-major: 8 x-values, then 8 y-values, then 8 z-values
                h[i] = __float2half(d.x);
                h[8 + i] = __float2half(d.y);
                h[16 + i] = __float2half(d.z);
            } else {
                h[3 * i] = __float2half(d.x);
                h[3 * i + 1] = __float2half(d.y);
                h[3 * i + 2] = __float2half(d.z);
            }
        }
        const uint4* hv = reinterpret_cast<const uint4*>(h);
        if (PATCH) {
            const int pW = res / 8;
            const long long patch = (long long)b * pW * pW + (py / 8) * pW + px0 / 8;
            __half* o = out + patch * 192 + (py % 8) * 8;
            *reinterpret_cast<uint4*>(o) = hv[0];
            *reinterpret_cast<uint4*>(o + 64) = hv[1];
            *reinterpret_cast<uint4*>(o + 128) = hv[2];
        } else if (COALESCE) {
            const int lane = threadIdx.x & 31;
            unsigned char* stage = s_stage + (threadIdx.x >> 5) * 1536;
            uint4* mine = reinterpret_cast<uint4*>(stage + lane * 48);
            mine[0] = hv[0]; mine[1] = hv[1]; mine[2] = hv[2];
            __syncwarp();
            // first pixel of the warp's 256-pixel run: this lane's px0 minus its 8 * lane
            uint4* o = reinterpret_cast<uint4*>(out + (((long long)b * res + py) * res + (px0 - 8 * lane)) * 3);
            const uint4* sv = reinterpret_cast<const uint4*>(stage);
            __stcs(o + lane, sv[lane]);
            __stcs(o + 32 + lane, sv[32 + lane]);
            __stcs(o + 64 + lane, sv[64 + lane]);
            __syncwarp();
        } else {
            __half* o = out + (((long long)b * res + py) * res + px0) * 3;
            *reinterpret_cast<uint4*>(o) = hv[0];
            *reinterpret_cast<uint4*>(o + 8) = hv[1];
            *reinterpret_cast<uint4*>(o + 16) = hv[2];
        }
    }
}

// any res / patch size / alignment: one pixel per thread
__global__ void __launch_bounds__(256)
ray_gen_generic_kernel(const float* __restrict__ c2w, const float* __restrict__ fov,
                       float* __restrict__ rays_o, __half* __restrict__ out, int batch, int res,
                       int ps) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long per_image = (long long)res * res;
    if (idx >= per_image * batch) return;
    const int b = (int)(idx / per_image);
    const int rem = (int)(idx % per_image);
    const int py = rem / res, px = rem % res;
    const float* M = c2w + b * 16;
    if (rem == 0 && rays_o) {
        rays_o[b * 3 + 0] = M[3];
        rays_o[b * 3 + 1] = M[7];
        rays_o[b * 3 + 2] = M[11];
    }
    const float cx = res * 0.5f;
    const float fx = cx / tanf(0.5f * fov[b]);
    const Ray3 r = pixel_ray(M, cx, fx, px, py);
    if (ps > 0) {
        const int pW = res / ps, pp = ps * ps;
        const long long patch = (long long)b * pW * pW + (py / ps) * pW + px / ps;
        __half* o = out + patch * 3 * pp + (py % ps) * ps + px % ps;
        o[0] = __float2half(r.x);
        o[pp] = __float2half(r.y);
        o[2 * pp] = __float2half(r.z);
    } else {
        __half* o = out + idx * 3;
        o[0] = __float2half(r.x);
        o[1] = __float2half(r.y);
        o[2] = __float2half(r.z);
    }
}

static int launch_ray_gen(const float* c2w, const float* fov, float* rays_o, __half* out,
                          int batch, int res, int ps, cudaStream_t st) {
    if (!c2w || !fov || !out || batch < 0 || res <= 0) return RFK_EINVAL;
    if (ps < 0 || (ps > 0 && res % ps)) return RFK_EINVAL;
    if (batch == 0) return RFK_OK;
    const bool vec = res % 8 == 0 && aligned16(out) && (ps == 0 || ps == 8);
    if (vec) {
        // 4-row strips once the strip threads alone fill every SM (148 x 2048 resident threads)
        const bool strips = res % 4 == 0 && (long long)batch * res * (res / 8) >= 4LL * kNumSMs * 2048;
        const long long n = (long long)batch * (res / (strips ? 4 : 1)) * (res / 8);
        const unsigned grid = ceil_div(n, 256);
        if (ps && strips) ray_gen_vec_kernel<1, 4><<<grid, 256, 0, st>>>(c2w, fov, rays_o, out, batch, res);
        else if (ps) ray_gen_vec_kernel<1, 1><<<grid, 256, 0, st>>>(c2w, fov, rays_o, out, batch, res);
        else if (strips && res % 256 == 0) ray_gen_vec_kernel<0, 4, 1><<<grid, 256, 0, st>>>(c2w, fov, rays_o, out, batch, res);
        else if (strips) ray_gen_vec_kernel<0, 4><<<grid, 256, 0, st>>>(c2w, fov, rays_o, out, batch, res);
        else ray_gen_vec_kernel<0, 1><<<grid, 256, 0, st>>>(c2w, fov, rays_o, out, batch, res);
    } else {
        const long long n = (long long)batch * res * res;
        ray_gen_generic_kernel<<<ceil_div(n, 256), 256, 0, st>>>(c2w, fov, rays_o, out, batch, res,
                                                                 ps);
    }
    return launch_status();
}

}  // namespace rfk

using namespace rfk;

extern "C" int rfk_ray_gen(const float* c2w, const float* fov, float* rays_o, rfk_half* rays_d,
                           int batch, int img_res, rfk_stream_t stream) {
    if (!rays_o) return RFK_EINVAL;
    return launch_ray_gen(c2w, fov, rays_o, (__half*)rays_d, batch, img_res, 0, as_stream(stream));
}

extern "C" int rfk_ray_gen_patchify(const float* c2w, const float* fov, float* rays_o,
                                    rfk_half* ray_pat, int batch, int img_res, int patch_size,
                                    rfk_stream_t stream) {
    if (patch_size <= 0) return RFK_EINVAL;
    return launch_ray_gen(c2w, fov, rays_o, (__half*)ray_pat, batch, img_res, patch_size,
                          as_stream(stream));
}
