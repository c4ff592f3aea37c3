// Typed loads and stores of the layer-program kernels (matrices and matrix-product inputs are bf16 or fp32), the scalar
// functions of their gates, and the address of a cache row in the block pool.
#pragma once
#include <cuda_bf16.h>

#include "tha_hybrid.h"

namespace tha {
__device__ __forceinline__ float hyb_load(const float* p) { return *p; }
__device__ __forceinline__ float hyb_load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void hyb_store(float* p, float v) { *p = v; }
__device__ __forceinline__ void hyb_store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float hyb_softcap(float z, float cap) { return cap * tanhf(z / cap); }
__device__ __forceinline__ float hyb_logsigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float hyb_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float hyb_softplus(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

// first float of the cache row of (slot, position t) in cache layer `layer` of a pool
__device__ __forceinline__ size_t hyb_kv_row(const tha_kv_t& kv, int slot, int t, int layer) {
  const int blk = kv.table[(size_t)slot * kv.table_stride + t / kv.block_size];
  return ((size_t)blk * kv.n_cache_layers + layer) * kv.block_size * kv.kv_dim + (size_t)(t % kv.block_size) * kv.kv_dim;
}
}  // namespace tha
