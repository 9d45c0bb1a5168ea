// World -> camera transform of triangle vertices / normals, and the fused per-view
// geometry front end (transform + register-token positions + RoPE tables).
//
// Reference semantics (BANANASJIM/renderformer-cuda):
//   src/kernels/coord_transform.cu:16-45   v' = R^T (v - t), n' = R^T n, fp32 math on fp16 data,
//       three-term sums in the order r_0*x + r_1*y + r_2*z, R^T rows (M0,M4,M8),(M1,M5,M9),(M2,M6,M10)
//   src/pipeline/render_session.cu:73-88    register-token position = camera-space scene centre x3
//   src/pipeline/render_session.cu:192-203  copy, transform, position assembly, table generation
//   src/kernels/rope.cu:23-43               table layout
//
// The arithmetic keeps the reference's expression trees (bit-identical results are
// required); the fused entry removes 3 device-to-device copies and 3 launches per view.
#include "common.cuh"

namespace rfk {

struct CamRT {
    float r00, r01, r02, r10, r11, r12, r20, r21, r22, tx, ty, tz;
};

__device__ __forceinline__ CamRT load_cam(const float* __restrict__ M) {
    CamRT c;
    c.r00 = M[0]; c.r10 = M[1]; c.r20 = M[2];
    c.r01 = M[4]; c.r11 = M[5]; c.r21 = M[6];
    c.r02 = M[8]; c.r12 = M[9]; c.r22 = M[10];
    c.tx = M[3]; c.ty = M[7]; c.tz = M[11];
    return c;
}

__device__ __forceinline__ void rot3(const CamRT& c, float vx, float vy, float vz, float& ox,
                                     float& oy, float& oz) {
    ox = c.r00 * vx + c.r01 * vy + c.r02 * vz;
    oy = c.r10 * vx + c.r11 * vy + c.r12 * vz;
    oz = c.r20 * vx + c.r21 * vy + c.r22 * vz;
}

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half(v); }
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }

// one thread per vertex, in place
template <typename T>
__global__ void __launch_bounds__(256)
world_to_cam_kernel(const float* __restrict__ c2w, T* tri, T* vn, int n_verts) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    const int b = blockIdx.y;
    if (idx >= n_verts) return;
    const CamRT c = load_cam(c2w + b * 16);
    const size_t base = ((size_t)b * n_verts + idx) * 3;
    {
        float vx = to_f(tri[base + 0]) - c.tx;
        float vy = to_f(tri[base + 1]) - c.ty;
        float vz = to_f(tri[base + 2]) - c.tz;
        float ox, oy, oz;
        rot3(c, vx, vy, vz, ox, oy, oz);
        tri[base + 0] = from_f<T>(ox);
        tri[base + 1] = from_f<T>(oy);
        tri[base + 2] = from_f<T>(oz);
    }
    if (vn) {
        float ox, oy, oz;
        rot3(c, to_f(vn[base + 0]), to_f(vn[base + 1]), to_f(vn[base + 2]), ox, oy, oz);
        vn[base + 0] = from_f<T>(ox);
        vn[base + 1] = from_f<T>(oy);
        vn[base + 2] = from_f<T>(oz);
    }
}

// fp16, many vertices: a thread owns 8 consecutive vertices of the flat [batch * n_verts] list = 48
// contiguous bytes = three 128-bit accesses per array (the one-vertex kernel above issues 6-byte ones and
// is bound by load latency). A thread whose vertices straddle two batch entries looks the camera up per vertex.
__global__ void __launch_bounds__(256)
world_to_cam_vec8_kernel(const float* __restrict__ c2w, __half* tri, __half* vn, int n_verts, long long n_groups) {
    const long long gidx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (gidx >= n_groups) return;
    const long long v0 = gidx * 8;
    const int b0 = (int)(v0 / n_verts), b1 = (int)((v0 + 7) / n_verts);
    CamRT c = load_cam(c2w + (size_t)b0 * 16);
    auto transform = [&](__half* arr, bool translate) {
        uint4* p = reinterpret_cast<uint4*>(arr + v0 * 3);
        __align__(16) __half h[24];
        uint4* hv = reinterpret_cast<uint4*>(h);
        hv[0] = p[0]; hv[1] = p[1]; hv[2] = p[2];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (b1 != b0) c = load_cam(c2w + (size_t)((v0 + i) / n_verts) * 16);
            float vx = __half2float(h[3 * i]), vy = __half2float(h[3 * i + 1]), vz = __half2float(h[3 * i + 2]);
            if (translate) { vx = vx - c.tx; vy = vy - c.ty; vz = vz - c.tz; }
            float ox, oy, oz;
            rot3(c, vx, vy, vz, ox, oy, oz);
            h[3 * i] = __float2half(ox); h[3 * i + 1] = __float2half(oy); h[3 * i + 2] = __float2half(oz);
        }
        p[0] = hv[0]; p[1] = hv[1]; p[2] = hv[2];
    };
    transform(tri, true);
    if (vn) transform(vn, false);
}

// thread -> (token t in [0, seq_pad), table chunk j in [0, head_dim/16)).
// Every thread rebuilds the token's 9 camera-space coordinates (27 FMAs); the j == 0
// thread also stores the geometry outputs.
__global__ void __launch_bounds__(256)
view_geometry_kernel(const float* __restrict__ c2w, const __half* __restrict__ tri_world,
                     const __half* __restrict__ vn_world, const float* __restrict__ world_center,
                     const float* __restrict__ freqs, __half* __restrict__ vtri,
                     __half* __restrict__ vvn, __half* __restrict__ vpos,
                     __half* __restrict__ k_cos, __half* __restrict__ k_sin, int n_tris, int nr,
                     int seq_pad, int num_freqs, int head_dim) {
    const int cpt = head_dim / 16;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= seq_pad * cpt) return;
    const int t = idx / cpt, j = idx % cpt;
    const CamRT c = load_cam(c2w);
    __half p[9];
    if (t < nr) {
        float ox, oy, oz;
        rot3(c, world_center[0] - c.tx, world_center[1] - c.ty, world_center[2] - c.tz, ox, oy, oz);
        const __half hx = __float2half(ox), hy = __float2half(oy), hz = __float2half(oz);
#pragma unroll
        for (int v = 0; v < 3; ++v) { p[3 * v] = hx; p[3 * v + 1] = hy; p[3 * v + 2] = hz; }
    } else if (t < nr + n_tris) {
        const size_t base = (size_t)(t - nr) * 9;
#pragma unroll
        for (int v = 0; v < 3; ++v) {
            float vx = __half2float(tri_world[base + 3 * v + 0]) - c.tx;
            float vy = __half2float(tri_world[base + 3 * v + 1]) - c.ty;
            float vz = __half2float(tri_world[base + 3 * v + 2]) - c.tz;
            float ox, oy, oz;
            rot3(c, vx, vy, vz, ox, oy, oz);
            p[3 * v] = __float2half(ox);
            p[3 * v + 1] = __float2half(oy);
            p[3 * v + 2] = __float2half(oz);
        }
        if (j == 0) {
#pragma unroll
            for (int i = 0; i < 9; ++i) vtri[base + i] = p[i];
            if (vvn) {
#pragma unroll
                for (int v = 0; v < 3; ++v) {
                    float ox, oy, oz;
                    rot3(c, __half2float(vn_world[base + 3 * v + 0]),
                         __half2float(vn_world[base + 3 * v + 1]),
                         __half2float(vn_world[base + 3 * v + 2]), ox, oy, oz);
                    vvn[base + 3 * v + 0] = __float2half(ox);
                    vvn[base + 3 * v + 1] = __float2half(oy);
                    vvn[base + 3 * v + 2] = __float2half(oz);
                }
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 9; ++i) p[i] = __ushort_as_half(0);
    }
    if (j == 0) {
#pragma unroll
        for (int i = 0; i < 9; ++i) vpos[(size_t)t * 9 + i] = p[i];
    }
    // RoPE table chunk: l = j*8 + i within the first half of head_dim
    const int freq_dim = 9 * num_freqs;
    float cs[8], sn[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int l = j * 8 + i;
        float val = 0.0f;
        if (l < freq_dim) {
            const int coord = l / num_freqs;
            float pc = 0.0f;
#pragma unroll
            for (int q = 0; q < 9; ++q)
                if (q == coord) pc = __half2float(p[q]);  // keeps p[] in registers
            val = pc * __ldg(freqs + l % num_freqs);
        }
        cs[i] = cosf(val);
        sn[i] = sinf(val);
    }
    const size_t o = (size_t)t * head_dim + j * 8;
    const Half8 hc = pack8(cs), hs = pack8(sn);
    st_half8(k_cos + o, hc);
    st_half8(k_cos + o + head_dim / 2, hc);
    st_half8(k_sin + o, hs);
    st_half8(k_sin + o + head_dim / 2, hs);
}

}  // namespace rfk

using namespace rfk;

extern "C" int rfk_world_to_cam(const float* c2w, rfk_half* tri, rfk_half* vn, int batch,
                                int n_tris, rfk_stream_t stream) {
    if (!c2w || !tri || batch < 0 || n_tris < 0) return RFK_EINVAL;
    if (batch == 0 || n_tris == 0) return RFK_OK;
    if (batch > 65535) return RFK_EUNSUPPORTED;
    const int n_verts = n_tris * 3;
    const long long total = (long long)batch * n_verts;
    if (total >= 8 * 256 * (long long)kNumSMs && total % 8 == 0 && aligned16(tri) && (!vn || aligned16(vn))) {
        const long long n_groups = total / 8;
        world_to_cam_vec8_kernel<<<ceil_div(n_groups, 256), 256, 0, as_stream(stream)>>>(c2w, (__half*)tri, (__half*)vn,
                                                                                          n_verts, n_groups);
        return launch_status();
    }
    dim3 grid(ceil_div(n_verts, 256), batch);
    world_to_cam_kernel<__half><<<grid, 256, 0, as_stream(stream)>>>(c2w, (__half*)tri,
                                                                     (__half*)vn, n_verts);
    return launch_status();
}

extern "C" int rfk_world_to_cam_f32(const float* c2w, float* verts, float* normals, int batch,
                                    int n_verts, rfk_stream_t stream) {
    if (!c2w || !verts || batch < 0 || n_verts < 0) return RFK_EINVAL;
    if (batch == 0 || n_verts == 0) return RFK_OK;
    if (batch > 65535) return RFK_EUNSUPPORTED;
    dim3 grid(ceil_div(n_verts, 256), batch);
    world_to_cam_kernel<float><<<grid, 256, 0, as_stream(stream)>>>(c2w, verts, normals, n_verts);
    return launch_status();
}

extern "C" int rfk_view_geometry(const float* c2w, const rfk_half* tri_world,
                                 const rfk_half* vn_world, const float* world_center,
                                 const float* learned_freqs, rfk_half* vtri, rfk_half* vvn,
                                 rfk_half* vpos, rfk_half* k_cos, rfk_half* k_sin, int n_tris,
                                 int n_register, int seq_pad, int num_freqs, int head_dim,
                                 rfk_stream_t stream) {
    if (!c2w || !tri_world || !world_center || !learned_freqs || !vtri || !vpos || !k_cos || !k_sin)
        return RFK_EINVAL;
    if ((vvn != nullptr) != (vn_world != nullptr)) return RFK_EINVAL;
    if (n_tris < 0 || n_register < 0 || num_freqs <= 0 || seq_pad < n_tris + n_register)
        return RFK_EINVAL;
    if (head_dim <= 0 || head_dim % 16 || !aligned16(k_cos) || !aligned16(k_sin))
        return RFK_EUNSUPPORTED;
    if (seq_pad == 0) return RFK_OK;
    const long long n = (long long)seq_pad * (head_dim / 16);
    view_geometry_kernel<<<ceil_div(n, 256), 256, 0, as_stream(stream)>>>(
        c2w, (const __half*)tri_world, (const __half*)vn_world, world_center, learned_freqs,
        (__half*)vtri, (__half*)vvn, (__half*)vpos, (__half*)k_cos, (__half*)k_sin, n_tris,
        n_register, seq_pad, num_freqs, head_dim);
    return launch_status();
}
