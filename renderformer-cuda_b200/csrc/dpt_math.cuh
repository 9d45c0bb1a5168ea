// Arithmetic shared by the element-wise operators of the DPT head in both layouts (dpt_glue.cu: NCHW, the reference's
// operators; dpt_nhwc.cu: channels-last, what the head itself runs on).
#pragma once
#include "common.cuh"

namespace rfk {

// v00*(1-hf)*(1-wf) + v01*(1-hf)*wf + v10*hf*(1-wf) + v11*hf*wf with the roundings written out as nvcc
// contracts the reference's expression: the second term is two rounded products, the first term's last
// product is fused into it, then the third and fourth terms' last products are fused into the running
// sum. Explicit here so that the pattern cannot change with the surrounding code; found by emulating
// the candidate patterns on the CPU against the reference kernel's outputs, and checked bit for bit.
__device__ __forceinline__ float bilerp_ref(float v00, float v01, float v10, float v11, float hf, float wf) {
    const float omh = __fsub_rn(1.0f, hf), omw = __fsub_rn(1.0f, wf);
    float s = __fmul_rn(__fmul_rn(v01, omh), wf);
    s = __fmaf_rn(__fmul_rn(v00, omh), omw, s);
    s = __fmaf_rn(__fmul_rn(v10, hf), omw, s);
    s = __fmaf_rn(__fmul_rn(v11, hf), wf, s);
    return s;
}

__device__ __forceinline__ float silu_sfu(float a) {
    return a * fast_rcp(1.0f + fast_exp2(a * -1.4426950408889634f));
}


}  // namespace rfk
