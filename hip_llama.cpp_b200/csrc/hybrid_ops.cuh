// Typed loads and stores of the layer-program kernels: matrices and matrix-product inputs are bf16 or fp32.
#pragma once
#include <cuda_bf16.h>

namespace tha {
__device__ __forceinline__ float hyb_load(const float* p) { return *p; }
__device__ __forceinline__ float hyb_load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void hyb_store(float* p, float v) { *p = v; }
__device__ __forceinline__ void hyb_store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
}  // namespace tha
