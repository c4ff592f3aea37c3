// Latent attention (tha_latent_t): what surrounds the products and the attention kernel.
//   hyb_latent_prepare_kernel   per row: the query latent's rms norm (dtype-typed, input of the query expansion); the
//                               key/value latent's rms norm and the rotation of the shared key part, written as ONE cache
//                               row [latent | rotated part] of the K pool
//   hyb_latent_split_q_kernel   per row and head: the plain query part as the input of the per-head product with the
//                               transposed key expansion; the rotated part, rotated, behind it in the absorbed query
// The attention itself is tha_hyb_attn with one key/value head whose values are the first kv_rank channels of its keys.
// Norms, rotation and the cache are fp32 in both number formats.
#include <cuda_bf16.h>

#include "common.cuh"
#include "hybrid_ops.cuh"
#include "tha_hybrid.h"

namespace tha {

template <typename T>
__global__ void hyb_latent_prepare_kernel(tha_latent_t a, tha_rows_t rows, tha_kv_t kv, const float* __restrict__ proj, long long ldp,
                                          const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot_dims, T* __restrict__ cq) {
  __shared__ float red[33];
  const int r = blockIdx.x;
  const float* pr = proj + (size_t)r * ldp;
  // query latent
  float ss = 0.f;
  for (int i = threadIdx.x; i < a.q_rank; i += blockDim.x) { const float v = pr[a.o_dq + i]; ss = fmaf(v, v, ss); }
  ss = block_sum(ss, red);
  float inv = 1.0f / sqrtf(ss / (float)a.q_rank + a.eps);
  for (int i = threadIdx.x; i < a.q_rank; i += blockDim.x) hyb_store(cq + (size_t)r * a.q_rank + i, pr[a.o_dq + i] * inv * a.q_norm[i]);
  // key/value latent -> cache row
  const int slot = rows.seq_slot[rows.row_seq[r]], t = rows.pos[r];
  float* krow = kv.k_pool + hyb_kv_row(kv, slot, t, a.cache_layer);
  ss = 0.f;
  for (int i = threadIdx.x; i < a.kv_rank; i += blockDim.x) { const float v = pr[a.o_dkv + i]; ss = fmaf(v, v, ss); }
  ss = block_sum(ss, red);
  inv = 1.0f / sqrtf(ss / (float)a.kv_rank + a.eps);
  for (int i = threadIdx.x; i < a.kv_rank; i += blockDim.x) krow[i] = pr[a.o_dkv + i] * inv * a.kv_norm[i];
  // the shared key part: pairs (2i, 2i+1) below rot_dims rotated, the rest passed through
  const float* kr = pr + a.o_dkv + a.kv_rank;
  const int half = rot_dims / 2;
  for (int i = threadIdx.x; i < (a.rot_dim + 1) / 2; i += blockDim.x) {
    float u = kr[2 * i], v = 2 * i + 1 < a.rot_dim ? kr[2 * i + 1] : 0.f;
    if (i < half) {
      const float c = cos_t[(size_t)r * half + i], s = sin_t[(size_t)r * half + i];
      const float nu = u * c - v * s, nv = v * c + u * s;
      u = nu; v = nv;
    }
    krow[a.kv_rank + 2 * i] = u;
    if (2 * i + 1 < a.rot_dim) krow[a.kv_rank + 2 * i + 1] = v;
  }
}

template <typename T>
__global__ void hyb_latent_split_q_kernel(tha_latent_t a, int n_rows, const float* __restrict__ qfull, const float* __restrict__ cos_t,
                                          const float* __restrict__ sin_t, int rot_dims, T* __restrict__ q_plain, float* __restrict__ q_abs) {
  const int r = blockIdx.x;
  const int per = a.dim + a.rot_dim, DA = a.kv_rank + a.rot_dim, half = rot_dims / 2;
  const float* q = qfull + (size_t)r * a.heads * per;
  for (int i = threadIdx.x; i < a.heads * a.dim; i += blockDim.x) {
    const int h = i / a.dim, d = i - h * a.dim;
    hyb_store(q_plain + (size_t)r * a.heads * a.dim + i, q[h * per + d]);
  }
  const int np = (a.rot_dim + 1) / 2;
  for (int i = threadIdx.x; i < a.heads * np; i += blockDim.x) {
    const int h = i / np, p = i - h * np;
    const float* src = q + h * per + a.dim;
    float u = src[2 * p], v = 2 * p + 1 < a.rot_dim ? src[2 * p + 1] : 0.f;
    if (p < half) {
      const float c = cos_t[(size_t)r * half + p], s = sin_t[(size_t)r * half + p];
      const float nu = u * c - v * s, nv = v * c + u * s;
      u = nu; v = nv;
    }
    float* dst = q_abs + (size_t)r * a.heads * DA + (size_t)h * DA + a.kv_rank;
    dst[2 * p] = u;
    if (2 * p + 1 < a.rot_dim) dst[2 * p + 1] = v;
  }
}

}  // namespace tha

using namespace tha;
typedef __nv_bfloat16 bf16;

extern "C" int tha_hyb_latent_prepare(void* stream, int dtype, const tha_latent_t* a, const tha_rows_t* rows, const tha_kv_t* kv,
                                      const float* proj, long long ldp, const float* cos_t, const float* sin_t, int rot_dims, void* cq) {
  if (rows->n_rows < 1) return THA_STATUS_SUCCESS;
  if (rot_dims > a->rot_dim || (rot_dims & 1) || a->kv_rank + a->rot_dim > kv->kv_dim || a->q_rank < 1 || a->kv_rank < 1 ||
      (rot_dims > 0 && (!cos_t || !sin_t)))
    return THA_STATUS_INVALID_ARG;
  int nt = 64;
  while (nt < a->kv_rank / 2 && nt < 256) nt += 32;
  if (dtype == THA_DT_BF16)
    THA_CUDA_OK(launch(hyb_latent_prepare_kernel<bf16>, dim3(rows->n_rows), dim3(nt), 0, (cudaStream_t)stream, false, *a, *rows, *kv, proj, ldp,
                       cos_t, sin_t, rot_dims, (bf16*)cq));
  else
    THA_CUDA_OK(launch(hyb_latent_prepare_kernel<float>, dim3(rows->n_rows), dim3(nt), 0, (cudaStream_t)stream, false, *a, *rows, *kv, proj, ldp,
                       cos_t, sin_t, rot_dims, (float*)cq));
  return THA_STATUS_SUCCESS;
}

extern "C" int tha_hyb_latent_split_q(void* stream, int dtype, const tha_latent_t* a, int n_rows, const float* qfull, const float* cos_t,
                                      const float* sin_t, int rot_dims, void* q_plain, float* q_abs) {
  if (n_rows < 1) return THA_STATUS_SUCCESS;
  if (rot_dims > a->rot_dim || (rot_dims & 1) || (rot_dims > 0 && (!cos_t || !sin_t))) return THA_STATUS_INVALID_ARG;
  int nt = 64;
  while (nt < a->heads * a->dim / 2 && nt < 256) nt += 32;
  if (dtype == THA_DT_BF16)
    THA_CUDA_OK(launch(hyb_latent_split_q_kernel<bf16>, dim3(n_rows), dim3(nt), 0, (cudaStream_t)stream, false, *a, n_rows, qfull, cos_t, sin_t,
                       rot_dims, (bf16*)q_plain, q_abs));
  else
    THA_CUDA_OK(launch(hyb_latent_split_q_kernel<float>, dim3(n_rows), dim3(nt), 0, (cudaStream_t)stream, false, *a, n_rows, qfull, cos_t, sin_t,
                       rot_dims, (float*)q_plain, q_abs));
  return THA_STATUS_SUCCESS;
}
