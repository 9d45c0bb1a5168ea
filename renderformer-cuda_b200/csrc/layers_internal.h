// Internal declarations shared by the layer library sources (not part of the C ABI).
#pragma once
#include <cublas_v2.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "rfk_layers.h"

struct rfk_ctx {
    cublasHandle_t blas = nullptr;
    void* ws = nullptr;      // cuBLAS workspace, set explicitly so capture never allocates
    size_t ws_bytes = 0;
    int device = 0;
};

namespace rfk_layers {
constexpr float kEpsFp16 = 0.0009765625f;   // 2^-10, the reference's kEpsFp16 (src/kernels/rmsnorm.h:9)
constexpr float kEpsFp32 = 1.1920929e-07f;  // 2^-23, the reference's kEpsFp32 (src/kernels/rmsnorm.h:10)
}  // namespace rfk_layers
