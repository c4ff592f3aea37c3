// The mechanisms of the layer-program path (include/tha_hybrid.h), one kernel family each:
//   rmsnorm with an offset weight, the row-gathering / grouped linear map, rotary tables in float64, attention
//   preparation (rotate, unit-rms, cache write), softmax attention over a paged cache limited to the query's block of
//   positions, the matrix-memory scan, the short convolution with its tail, the gated-delta-rule scan, the top-k router
//   with its counting sort, and the clamped gated activation.
// All of them take ragged rows (tha_rows_t): what a row may see depends only on its own sequence, position, block table
// and state slot, never on where it sits in the batch.  Reductions run in a fixed order, so a position's result does
// not depend on how the prompt was cut or on what else is in the step.
#include <cuda_bf16.h>
#include <math.h>

#include "common.cuh"
#include "hybrid_ops.cuh"
#include "tha_hybrid.h"

namespace tha {

// ------------------------------------------------------------------------------------------------------------------
// rmsnorm: one block per row
// ------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void hyb_rmsnorm_kernel(T* __restrict__ out, const float* __restrict__ x, const float* __restrict__ w, float w_offset,
                                   float eps, int width, const int* __restrict__ rows_idx) {
  __shared__ float red[33];
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows_idx ? rows_idx[r] : r) * width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) { const float v = xr[i]; ss = fmaf(v, v, ss); }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x) hyb_store(out + (size_t)r * width + i, xr[i] * inv * (w_offset + (w ? w[i] : 0.f)));
}

// ------------------------------------------------------------------------------------------------------------------
// linear: 64 x 64 output tile per block, 16-deep k slices through shared memory, 4 x 4 per thread, fp32 FMA in
// ascending k: the sum of an output element is the same whatever tile or group it lands in.
// ------------------------------------------------------------------------------------------------------------------
constexpr int LT = 64, LK = 16;

template <typename TA, typename TW>
__global__ void __launch_bounds__(256) hyb_linear_kernel(float* __restrict__ C, long long ldc, const TA* __restrict__ A, long long lda,
                                                         const int* __restrict__ a_rows, const TW* __restrict__ W,
                                                         long long w_group_stride, int M, int N, int K,
                                                         const int* __restrict__ group_off, int n_groups) {
  __shared__ float As[LK][LT + 4];
  __shared__ float Ws[LK][LT + 4];
  // which group and which rows this block covers
  int g = 0, m0 = 0, m_end = M;
  if (group_off) {
    int tile = blockIdx.y, found = 0;
    for (g = 0; g < n_groups; g++) {
      const int lo = group_off[g], hi = group_off[g + 1];
      const int nt = (hi - lo + LT - 1) / LT;
      if (tile < nt) { m0 = lo + tile * LT; m_end = hi; found = 1; break; }
      tile -= nt;
    }
    if (!found) return;
  } else {
    m0 = blockIdx.y * LT;
    if (m0 >= M) return;
  }
  const int n0 = blockIdx.x * LT;
  const TW* Wg = W + (size_t)g * w_group_stride;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;   // tx: columns, ty: rows
  float acc[4][4] = {};
  // loader mapping: thread loads 4 elements of a row of A and of W per slice
  const int lr = threadIdx.x >> 2, lk = (threadIdx.x & 3) * 4;
  const int am = m0 + lr;
  const long long arow = am < m_end ? (long long)(a_rows ? a_rows[am] : am) : -1;
  const int wn = n0 + lr;
  for (int k0 = 0; k0 < K; k0 += LK) {
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const int k = k0 + lk + e;
      As[lk + e][lr] = (arow >= 0 && k < K) ? hyb_load(A + arow * lda + k) : 0.f;
      Ws[lk + e][lr] = (wn < N && k < K) ? hyb_load(Wg + (size_t)wn * K + k) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < LK; k++) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; i++) { a[i] = As[k][ty * 4 + i]; b[i] = Ws[k][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int m = m0 + ty * 4 + i;
    if (m >= m_end) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int n = n0 + tx * 4 + j;
      if (n < N) C[(size_t)m * ldc + n] = acc[i][j];
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------
// rotary tables: float64 angles so that position * frequency keeps its low bits at long contexts
// ------------------------------------------------------------------------------------------------------------------
__global__ void hyb_rotary_kernel(const double* __restrict__ inv_freq, int half, float mag, const int* __restrict__ pos, int n_rows,
                                  float* __restrict__ cos_out, float* __restrict__ sin_out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_rows * half) return;
  const int r = i / half, c = i % half;
  double s, co;
  sincos((double)pos[r] * inv_freq[c], &s, &co);
  cos_out[i] = (float)(co * (double)mag);
  sin_out[i] = (float)(s * (double)mag);
}

// ------------------------------------------------------------------------------------------------------------------
// attention preparation: one block per row, one warp per head (query heads first, then key heads, then value heads)
// ------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ size_t hyb_kv_row(const tha_kv_t& kv, int slot, int t, int layer) {
  const int blk = kv.table[(size_t)slot * kv.table_stride + t / kv.block_size];
  return ((size_t)blk * kv.n_cache_layers + layer) * kv.block_size * kv.kv_dim + (size_t)(t % kv.block_size) * kv.kv_dim;
}

__global__ void hyb_attn_prepare_kernel(tha_attn_t a, tha_rows_t rows, tha_kv_t kv, const float* __restrict__ proj, long long ldp,
                                        const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot_dims,
                                        float* __restrict__ q_out) {
  const int r = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int slot = rows.seq_slot[rows.row_seq[r]], t = rows.pos[r];
  const float* pr = proj + (size_t)r * ldp;
  const int half = rot_dims / 2;
  const size_t krow = hyb_kv_row(kv, slot, t, a.cache_layer);
  for (int h = warp; h < a.heads + 2 * a.kv_heads; h += nwarps) {
    if (h >= a.heads + a.kv_heads) {   // a value head: plain copy
      const int g = h - a.heads - a.kv_heads;
      for (int e = lane; e < a.vdim; e += 32) kv.v_pool[krow + (size_t)g * a.vdim + e] = pr[a.o_v + g * a.vdim + e];
      continue;
    }
    const bool is_q = h < a.heads;
    const float* src = pr + (is_q ? a.o_q + h * a.dim : a.o_k + (h - a.heads) * a.dim);
    float* dst = is_q ? q_out + (size_t)r * a.heads * a.dim + (size_t)h * a.dim : kv.k_pool + krow + (size_t)(h - a.heads) * a.dim;
    // pairs (2i, 2i+1): rotated below `half`, passed through above
    float ss = 0.f;
    const int npairs = (a.dim + 1) / 2;
    for (int i = lane; i < npairs; i += 32) {
      float u = src[2 * i], v = 2 * i + 1 < a.dim ? src[2 * i + 1] : 0.f;
      if (i < half) {
        const float c = cos_t[(size_t)r * half + i], s = sin_t[(size_t)r * half + i];
        const float nu = u * c - v * s, nv = v * c + u * s;
        u = nu; v = nv;
      }
      ss = fmaf(u, u, ss);
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float inv = a.unit_rms ? 1.0f / sqrtf(ss / (float)a.dim + a.eps) : 1.0f;
    for (int i = lane; i < npairs; i += 32) {
      float u = src[2 * i], v = 2 * i + 1 < a.dim ? src[2 * i + 1] : 0.f;
      if (i < half) {
        const float c = cos_t[(size_t)r * half + i], s = sin_t[(size_t)r * half + i];
        const float nu = u * c - v * s, nv = v * c + u * s;
        u = nu; v = nv;
      }
      dst[2 * i] = u * inv;
      if (2 * i + 1 < a.dim) dst[2 * i + 1] = v * inv;
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------
// attention: one block per (row, head).  Scores of the visible keys into shared memory (a warp per key, lanes over the
// head's dimensions), softmax, then the weighted sum of the value rows (threads over value channels x key parts).
// Visible keys: first .. pos with first = the start of pos's block of `chunk` positions (0 when chunk == 0).
// ------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void hyb_attn_kernel(tha_attn_t a, tha_rows_t rows, tha_kv_t kv, const float* __restrict__ q, T* __restrict__ out) {
  extern __shared__ float sm[];
  __shared__ float red[33];
  const int r = blockIdx.x, h = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int slot = rows.seq_slot[rows.row_seq[r]], t = rows.pos[r];
  const int first = a.chunk > 0 ? (t / a.chunk) * a.chunk : 0;
  const int nk = t - first + 1;
  const int g = h / (a.heads / a.kv_heads);
  float* sq = sm;                 // [dim]
  float* sc = sm + a.dim;         // [nk]
  float* part = sc + nk;          // [parts * vdim]
  for (int i = threadIdx.x; i < a.dim; i += blockDim.x) sq[i] = q[(size_t)r * a.heads * a.dim + (size_t)h * a.dim + i];
  __syncthreads();
  float mx = -INFINITY;
  for (int j = warp; j < nk; j += nwarps) {
    const float* kr = kv.k_pool + hyb_kv_row(kv, slot, first + j, a.cache_layer) + (size_t)g * a.dim;
    float s = 0.f;
    for (int i = lane; i < a.dim; i += 32) s = fmaf(sq[i], kr[i], s);
    s = warp_sum(s) * a.scale;
    if (lane == 0) sc[j] = s;
    mx = fmaxf(mx, s);
  }
  mx = block_max(mx, red);
  float sum = 0.f;
  for (int j = threadIdx.x; j < nk; j += blockDim.x) { const float p = expf(sc[j] - mx); sc[j] = p; sum += p; }
  sum = block_sum(sum, red);
  const float inv = 1.0f / sum;
  // weighted values: thread (part, e) sums keys part, part + parts, ...
  const int parts = max(1, (int)blockDim.x / a.vdim);
  for (int idx = threadIdx.x; idx < parts * a.vdim; idx += blockDim.x) {
    const int p = idx / a.vdim, e = idx % a.vdim;
    float acc = 0.f;
    for (int j = p; j < nk; j += parts)
      acc = fmaf(sc[j], kv.v_pool[hyb_kv_row(kv, slot, first + j, a.cache_layer) + (size_t)g * a.vdim + e], acc);
    part[idx] = acc;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < a.vdim; e += blockDim.x) {
    float acc = 0.f;
    for (int p = 0; p < parts; p++) acc += part[p * a.vdim + e];
    hyb_store(out + (size_t)r * a.heads * a.vdim + (size_t)h * a.vdim + e, acc * inv);
  }
}

// ------------------------------------------------------------------------------------------------------------------
// matrix memory: one block per (sequence, head); S [dim, vdim], n [dim] in shared memory, tokens in order.
// ------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float hyb_softcap(float z, float cap) { return cap * tanhf(z / cap); }
__device__ __forceinline__ float hyb_logsigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float hyb_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float hyb_softplus(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

template <typename T>
__global__ void hyb_mem_scan_kernel(tha_mem_t m, tha_rows_t rows, tha_state_store_t st, const float* __restrict__ proj, long long ldp,
                                    T* __restrict__ out) {
  extern __shared__ float sm[];
  __shared__ float red[33];
  const int s = blockIdx.x, h = blockIdx.y;
  const int D = m.dim, E = m.vdim, nt = blockDim.x;
  float* S = sm;              // [D * E]
  float* nv = S + D * E;      // [D]
  float* sq = nv + D;         // [D]
  float* sk = sq + D;         // [D]
  float* sv = sk + D;         // [E]
  const int parts = max(1, nt / E);
  float* part = sv + E;       // [parts * E]
  float* gstate = st.base + (size_t)rows.seq_slot[s] * st.slot_floats + m.state_off + (size_t)h * (D * E + D + 1);
  for (int i = threadIdx.x; i < D * E + D; i += nt) S[i] = gstate[i];   // S then n, adjacent in both places
  float mrun = gstate[D * E + D];
  __syncthreads();
  const float qscale = 1.0f / sqrtf((float)D);
  for (int r = rows.seq_first[s]; r < rows.seq_first[s + 1]; r++) {
    const float* pr = proj + (size_t)r * ldp;
    for (int i = threadIdx.x; i < D; i += nt) { sq[i] = pr[m.o_q + h * D + i] * qscale; sk[i] = pr[m.o_k + h * D + i]; }
    for (int i = threadIdx.x; i < E; i += nt) sv[i] = pr[m.o_v + h * E + i];
    const float ig = hyb_softcap(pr[m.o_i + h] + m.b_i[h], m.gate_cap);
    const float fg = hyb_logsigmoid(hyb_softcap(pr[m.o_f + h] + m.b_f[h], m.gate_cap));
    const float mnew = fmaxf(fg + mrun, ig);
    const float a = expf(fg + mrun - mnew), b = expf(ig - mnew);
    mrun = mnew;
    __syncthreads();
    for (int i = threadIdx.x; i < D * E; i += nt) { const int d = i / E, e = i - d * E; S[i] = fmaf(a, S[i], b * sk[d] * sv[e]); }
    for (int i = threadIdx.x; i < D; i += nt) nv[i] = fmaf(a, nv[i], b * sk[i]);
    __syncthreads();
    for (int idx = threadIdx.x; idx < parts * E; idx += nt) {
      const int p = idx / E, e = idx - p * E;
      float acc = 0.f;
      for (int d = p; d < D; d += parts) acc = fmaf(S[d * E + e], sq[d], acc);
      part[idx] = acc;
    }
    float nq = 0.f;
    for (int i = threadIdx.x; i < D; i += nt) nq = fmaf(nv[i], sq[i], nq);
    nq = block_sum(nq, red);   // also orders `part`
    const float den = fmaxf(fabsf(nq), expf(-mrun)) + 1e-6f;
    float ss = 0.f;
    for (int e = threadIdx.x; e < E; e += nt) {
      float acc = 0.f;
      for (int p = 0; p < parts; p++) acc += part[p * E + e];
      acc /= den;
      sv[e] = acc;            // sv is free again (its last reader was the S update, two barriers back)
      ss = fmaf(acc, acc, ss);
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)E + m.eps);
    for (int e = threadIdx.x; e < E; e += nt)
      hyb_store(out + (size_t)r * m.heads * E + (size_t)h * E + e, sv[e] * inv * m.norm[h * E + e] * hyb_sigmoid(pr[m.o_g + h * E + e]));
    __syncthreads();
  }
  for (int i = threadIdx.x; i < D * E + D; i += nt) gstate[i] = S[i];
  if (threadIdx.x == 0) gstate[D * E + D] = mrun;
}

// ------------------------------------------------------------------------------------------------------------------
// short causal convolution + silu; the slot keeps the last taps-1 inputs of every channel (oldest first)
// ------------------------------------------------------------------------------------------------------------------
__global__ void hyb_conv_silu_kernel(tha_rows_t rows, tha_state_store_t st, long long conv_state_off, const float* __restrict__ proj,
                                     long long ldp, int col0, int channels, int taps, const float* __restrict__ w,
                                     float* __restrict__ out) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x, r = blockIdx.y;
  if (c >= channels) return;
  const int s = rows.row_seq[r], first = rows.seq_first[s];
  const float* tail = st.base + (size_t)rows.seq_slot[s] * st.slot_floats + conv_state_off + (size_t)c * (taps - 1);
  float acc = 0.f;
  for (int j = 0; j < taps; j++) {
    const int rr = r - (taps - 1 - j);
    const float x = rr >= first ? proj[(size_t)rr * ldp + col0 + c] : tail[(taps - 1) - (first - rr)];
    acc = fmaf(w[(size_t)c * taps + j], x, acc);
  }
  out[(size_t)r * channels + c] = acc / (1.0f + expf(-acc));
}
// after the convolution: tail[i] <- the input (taps-1-i) tokens before the end of what the sequence has seen now
__global__ void hyb_conv_tail_kernel(tha_rows_t rows, tha_state_store_t st, long long conv_state_off, const float* __restrict__ proj,
                                     long long ldp, int col0, int channels, int taps) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x, s = blockIdx.y;
  if (c >= channels) return;
  const int first = rows.seq_first[s], n = rows.seq_first[s + 1] - first;
  float* tail = st.base + (size_t)rows.seq_slot[s] * st.slot_floats + conv_state_off + (size_t)c * (taps - 1);
  for (int i = 0; i < taps - 1; i++) {           // ascending: tail[i + n] is read before it is overwritten
    const int back = (taps - 1) - i;             // this entry is the input `back` tokens before the end
    tail[i] = back <= n ? proj[(size_t)(first + n - back) * ldp + col0 + c] : tail[i + n];
  }
}

// ------------------------------------------------------------------------------------------------------------------
// gated delta rule: one block per (sequence, value head); S [dim, vdim] in shared memory.  A thread (part, e) owns the
// rows d = part, part + parts, ... of column e: decay, read S^T k, write k u^T and read S^T q without leaving its column.
// ------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void hyb_delta_scan_kernel(tha_delta_t dl, tha_rows_t rows, tha_state_store_t st, const float* __restrict__ qkv,
                                      const float* __restrict__ proj, long long ldp, const float* __restrict__ dt_raw,
                                      const float* __restrict__ gate_raw, T* __restrict__ out) {
  extern __shared__ float sm[];
  __shared__ float red[33];
  const int s = blockIdx.x, h = blockIdx.y;
  const int D = dl.dim, E = dl.vdim, nt = blockDim.x;
  const int hk = h / (dl.heads / dl.kv_heads);
  const int C = 2 * dl.kv_heads * D + dl.heads * E;
  const int parts = max(1, nt / E);
  float* S = sm;               // [D * E]
  float* sq = S + D * E;       // [D]
  float* sk = sq + D;          // [D]
  float* sg = sk + D;          // [D]
  float* su = sg + D;          // [E]
  float* part = su + E;        // [parts * E]
  float* gstate = st.base + (size_t)rows.seq_slot[s] * st.slot_floats + dl.state_off + (size_t)h * D * E;
  for (int i = threadIdx.x; i < D * E; i += nt) S[i] = gstate[i];
  const float decay_rate = expf(dl.a_log[h]);
  const float qscale = 1.0f / sqrtf((float)D);
  __syncthreads();
  for (int r = rows.seq_first[s]; r < rows.seq_first[s + 1]; r++) {
    const float* x = qkv + (size_t)r * C;
    float qq = 0.f, kk = 0.f;
    for (int i = threadIdx.x; i < D; i += nt) {
      const float a = x[hk * D + i], b = x[dl.kv_heads * D + hk * D + i];
      qq = fmaf(a, a, qq);
      kk = fmaf(b, b, kk);
      sq[i] = a; sk[i] = b;
      sg[i] = expf(-decay_rate * hyb_softplus(dt_raw[(size_t)r * dl.heads * D + h * D + i] + dl.dt_bias[h * D + i]));
    }
    qq = block_sum(qq, red);
    kk = block_sum(kk, red);
    const float qn = qscale / sqrtf(qq + 1e-6f), kn = 1.0f / sqrtf(kk + 1e-6f);
    const float beta = hyb_sigmoid(proj[(size_t)r * ldp + dl.o_b + h]);
    // decay and S^T k
    for (int idx = threadIdx.x; idx < parts * E; idx += nt) {
      const int p = idx / E, e = idx - p * E;
      float acc = 0.f;
      for (int d = p; d < D; d += parts) { const float v = S[d * E + e] * sg[d]; S[d * E + e] = v; acc = fmaf(v, sk[d] * kn, acc); }
      part[idx] = acc;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += nt) {
      float acc = 0.f;
      for (int p = 0; p < parts; p++) acc += part[p * E + e];
      su[e] = beta * (x[2 * dl.kv_heads * D + h * E + e] - acc);
    }
    __syncthreads();
    // write and read-out
    for (int idx = threadIdx.x; idx < parts * E; idx += nt) {
      const int p = idx / E, e = idx - p * E;
      const float u = su[e];
      float acc = 0.f;
      for (int d = p; d < D; d += parts) { const float v = fmaf(sk[d] * kn, u, S[d * E + e]); S[d * E + e] = v; acc = fmaf(v, sq[d] * qn, acc); }
      part[idx] = acc;
    }
    __syncthreads();
    float ss = 0.f;
    for (int e = threadIdx.x; e < E; e += nt) {
      float acc = 0.f;
      for (int p = 0; p < parts; p++) acc += part[p * E + e];
      su[e] = acc;
      ss = fmaf(acc, acc, ss);
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)E + dl.eps);
    for (int e = threadIdx.x; e < E; e += nt)
      hyb_store(out + (size_t)r * dl.heads * E + (size_t)h * E + e,
                su[e] * inv * dl.norm[e] * hyb_sigmoid(gate_raw[(size_t)r * dl.heads * E + h * E + e]));
    __syncthreads();
  }
  for (int i = threadIdx.x; i < D * E; i += nt) gstate[i] = S[i];
}

// ------------------------------------------------------------------------------------------------------------------
// router: a warp per row picks the `top` largest logits (lowest index on ties), softmax over them
// ------------------------------------------------------------------------------------------------------------------
__global__ void hyb_route_kernel(int experts, int top, int o_router, const float* __restrict__ proj, long long ldp, int n_rows,
                                 int* __restrict__ expert_id, float* __restrict__ weight, int* __restrict__ counts) {
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= n_rows) return;
  const float* z = proj + (size_t)r * ldp + o_router;
  float zmax = 0.f, sum = 0.f, mine = 0.f;   // lane j keeps the j-th pick's logit (top <= 32)
  for (int j = 0; j < top; j++) {
    float best = -INFINITY; int bi = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      bool taken = false;
      for (int p = 0; p < j; p++) taken |= expert_id[(size_t)r * top + p] == e;
      const float v = z[e];
      if (!taken && (v > best || (v == best && e < bi))) { best = v; bi = e; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(THA_FULL_MASK, best, o);
      const int oi = __shfl_xor_sync(THA_FULL_MASK, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (lane == 0) { expert_id[(size_t)r * top + j] = bi; atomicAdd(counts + bi, 1); }
    __syncwarp();
    if (j == 0) zmax = best;
    if (lane == j) mine = best;
    sum += expf(best - zmax);
  }
  if (lane < top) weight[(size_t)r * top + lane] = expf(mine - zmax) / sum;
}
// counting sort of the (row, pick) pairs by expert, one block, a warp per expert: within an expert the pairs stay in
// ascending (row, pick) order, so the placement is the same on every run.
__global__ void hyb_route_sort_kernel(int experts, int top, int n_rows, const int* __restrict__ expert_id, const int* __restrict__ counts,
                                      int* __restrict__ group_off, int* __restrict__ sorted_row, int* __restrict__ inv) {
  extern __shared__ int smi[];   // [experts + 1]
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < experts; e++) { smi[e] = acc; group_off[e] = acc; acc += counts[e]; }
    group_off[experts] = acc;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int n = n_rows * top;
  for (int e = warp; e < experts; e += nwarps) {
    int at = smi[e];
    for (int i0 = 0; i0 < n; i0 += 32) {
      const int i = i0 + lane;
      const bool hit = i < n && expert_id[i] == e;
      const unsigned m = __ballot_sync(THA_FULL_MASK, hit);
      if (hit) { const int p = at + __popc(m & ((1u << lane) - 1)); sorted_row[p] = i / top; inv[i] = p; }
      at += __popc(m);
    }
  }
}

template <typename T>
__global__ void hyb_glu_kernel(T* __restrict__ y, const float* __restrict__ gu, long long ldg, int col_g, int col_u, int n, int ff,
                               float limit, float alpha) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)n * ff) return;
  const size_t r = i / ff; const int c = (int)(i - r * ff);
  const float g = fminf(gu[r * ldg + col_g + c], limit);
  const float u = fminf(fmaxf(gu[r * ldg + col_u + c], -limit), limit);
  hyb_store(y + i, g * hyb_sigmoid(alpha * g) * (u + 1.0f));
}

static int pick_threads(int want) {   // a multiple of 32 in 64..256
  int t = 64;
  while (t < want && t < 256) t += 32;
  return t;
}

}  // namespace tha

using namespace tha;
typedef __nv_bfloat16 bf16;

extern "C" int tha_hyb_rmsnorm(void* stream, int dtype, void* out, const float* x, const float* w, float w_offset, float eps,
                               int n_rows, int width, const int* rows_idx) {
  if (n_rows < 1) return THA_STATUS_SUCCESS;
  const int nt = pick_threads(width / 4);
  if (dtype == THA_DT_BF16)
    THA_CUDA_OK(launch(hyb_rmsnorm_kernel<bf16>, dim3(n_rows), dim3(nt), 0, (cudaStream_t)stream, false, (bf16*)out, x, w, w_offset, eps, width, rows_idx));
  else
    THA_CUDA_OK(launch(hyb_rmsnorm_kernel<float>, dim3(n_rows), dim3(nt), 0, (cudaStream_t)stream, false, (float*)out, x, w, w_offset, eps, width, rows_idx));
  return THA_STATUS_SUCCESS;
}

extern "C" int tha_hyb_linear(void* stream, int dtype, float* C, long long ldc, const void* A, long long lda, int a_f32,
                              const int* a_rows, const void* W, long long w_group_stride, int M, int N, int K,
                              const int* group_off, int n_groups) {
  if (M < 1 || N < 1) return THA_STATUS_SUCCESS;
  if (K < 1 || !C || !A || !W) return THA_STATUS_INVALID_ARG;
  const int mt = ceil_div(M, LT) + (group_off ? n_groups : 0);
  const dim3 grid(ceil_div(N, LT), mt), block(256);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == THA_DT_F32)
    THA_CUDA_OK(launch(hyb_linear_kernel<float, float>, grid, block, 0, s, false, C, ldc, (const float*)A, lda, a_rows, (const float*)W,
                       w_group_stride, M, N, K, group_off, n_groups));
  else if (a_f32)
    THA_CUDA_OK(launch(hyb_linear_kernel<float, bf16>, grid, block, 0, s, false, C, ldc, (const float*)A, lda, a_rows, (const bf16*)W,
                       w_group_stride, M, N, K, group_off, n_groups));
  else
    THA_CUDA_OK(launch(hyb_linear_kernel<bf16, bf16>, grid, block, 0, s, false, C, ldc, (const bf16*)A, lda, a_rows, (const bf16*)W,
                       w_group_stride, M, N, K, group_off, n_groups));
  return THA_STATUS_SUCCESS;
}

extern "C" int tha_hyb_rotary_table(void* stream, const tha_rotary_t* rot, const int* pos, int n_rows, float* cos_out, float* sin_out) {
  const int half = rot->dims / 2;
  if (n_rows < 1 || half < 1) return THA_STATUS_SUCCESS;
  THA_CUDA_OK(launch(hyb_rotary_kernel, dim3(ceil_div(n_rows * half, 128)), dim3(128), 0, (cudaStream_t)stream, false, rot->inv_freq, half,
                     rot->mag, pos, n_rows, cos_out, sin_out));
  return THA_STATUS_SUCCESS;
}

extern "C" int tha_hyb_attn_prepare(void* stream, const tha_attn_t* a, const tha_rows_t* rows, const tha_kv_t* kv, const float* proj,
                                    long long ldp, const float* cos_t, const float* sin_t, int rot_dims, float* q_out) {
  if (rows->n_rows < 1) return THA_STATUS_SUCCESS;
  if (a->heads % a->kv_heads || rot_dims > a->dim || (rot_dims & 1) || a->kv_heads * a->dim > kv->kv_dim || a->kv_heads * a->vdim > kv->kv_dim)
    return THA_STATUS_INVALID_ARG;
  const int nt = pick_threads(32 * (a->heads + 2 * a->kv_heads));
  THA_CUDA_OK(launch(hyb_attn_prepare_kernel, dim3(rows->n_rows), dim3(nt), 0, (cudaStream_t)stream, false, *a, *rows, *kv, proj, ldp, cos_t,
                     sin_t, rot_dims, q_out));
  return THA_STATUS_SUCCESS;
}

extern "C" int tha_hyb_attn(void* stream, int dtype, const tha_attn_t* a, const tha_rows_t* rows, const tha_kv_t* kv, const float* q,
                            void* out) {
  if (rows->n_rows < 1) return THA_STATUS_SUCCESS;
  const int nt = 128;
  const int parts = nt / a->vdim > 0 ? nt / a->vdim : 1;
  const int seen = rows->max_pos + 1;   // the most keys a query of this step can see
  const int max_keys = a->chunk > 0 && a->chunk < seen ? a->chunk : seen;
  const size_t smem = sizeof(float) * ((size_t)a->dim + max_keys + (size_t)parts * a->vdim);
  if (smem > 227 * 1024) return THA_STATUS_NOT_SUPPORTED;
  const dim3 grid(rows->n_rows, a->heads);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == THA_DT_BF16) {
    if (smem > 48 * 1024) THA_CUDA_OK(cudaFuncSetAttribute(hyb_attn_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    THA_CUDA_OK(launch(hyb_attn_kernel<bf16>, grid, dim3(nt), smem, s, false, *a, *rows, *kv, q, (bf16*)out));
  } else {
    if (smem > 48 * 1024) THA_CUDA_OK(cudaFuncSetAttribute(hyb_attn_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    THA_CUDA_OK(launch(hyb_attn_kernel<float>, grid, dim3(nt), smem, s, false, *a, *rows, *kv, q, (float*)out));
  }
  return THA_STATUS_SUCCESS;
}

extern "C" int tha_hyb_mem_scan(void* stream, int dtype, const tha_mem_t* m, const tha_rows_t* rows, const tha_state_store_t* st,
                                const float* proj, long long ldp, void* out) {
  if (rows->n_seqs < 1) return THA_STATUS_SUCCESS;
  const int nt = 256;
  const int parts = nt / m->vdim > 0 ? nt / m->vdim : 1;
  const size_t smem = sizeof(float) * ((size_t)m->dim * m->vdim + 3 * (size_t)m->dim + m->vdim + (size_t)parts * m->vdim);
  const dim3 grid(rows->n_seqs, m->heads);
  cudaStream_t s = (cudaStream_t)stream;
  if (smem > 227 * 1024) return THA_STATUS_NOT_SUPPORTED;
  if (dtype == THA_DT_BF16) {
    if (smem > 48 * 1024) THA_CUDA_OK(cudaFuncSetAttribute(hyb_mem_scan_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    THA_CUDA_OK(launch(hyb_mem_scan_kernel<bf16>, grid, dim3(nt), smem, s, false, *m, *rows, *st, proj, ldp, (bf16*)out));
  } else {
    if (smem > 48 * 1024) THA_CUDA_OK(cudaFuncSetAttribute(hyb_mem_scan_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    THA_CUDA_OK(launch(hyb_mem_scan_kernel<float>, grid, dim3(nt), smem, s, false, *m, *rows, *st, proj, ldp, (float*)out));
  }
  return THA_STATUS_SUCCESS;
}

extern "C" int tha_hyb_conv_silu(void* stream, const tha_rows_t* rows, const tha_state_store_t* st, long long conv_state_off,
                                 const float* proj, long long ldp, int col0, int channels, int taps, const float* w, float* out) {
  if (rows->n_rows < 1) return THA_STATUS_SUCCESS;
  if (taps < 1) return THA_STATUS_INVALID_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  THA_CUDA_OK(launch(hyb_conv_silu_kernel, dim3(ceil_div(channels, 128), rows->n_rows), dim3(128), 0, s, false, *rows, *st, conv_state_off,
                     proj, ldp, col0, channels, taps, w, out));
  if (taps > 1)
    THA_CUDA_OK(launch(hyb_conv_tail_kernel, dim3(ceil_div(channels, 128), rows->n_seqs), dim3(128), 0, s, false, *rows, *st, conv_state_off,
                       proj, ldp, col0, channels, taps));
  return THA_STATUS_SUCCESS;
}

extern "C" int tha_hyb_delta_scan(void* stream, int dtype, const tha_delta_t* d, const tha_rows_t* rows, const tha_state_store_t* st,
                                  const float* qkv, const float* proj, long long ldp, const float* dt_raw, const float* gate_raw,
                                  void* out) {
  if (rows->n_seqs < 1) return THA_STATUS_SUCCESS;
  if (d->heads % d->kv_heads) return THA_STATUS_INVALID_ARG;
  const int nt = 256;
  const int parts = nt / d->vdim > 0 ? nt / d->vdim : 1;
  const size_t smem = sizeof(float) * ((size_t)d->dim * d->vdim + 3 * (size_t)d->dim + d->vdim + (size_t)parts * d->vdim);
  if (smem > 227 * 1024) return THA_STATUS_NOT_SUPPORTED;
  const dim3 grid(rows->n_seqs, d->heads);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == THA_DT_BF16) {
    if (smem > 48 * 1024) THA_CUDA_OK(cudaFuncSetAttribute(hyb_delta_scan_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    THA_CUDA_OK(launch(hyb_delta_scan_kernel<bf16>, grid, dim3(nt), smem, s, false, *d, *rows, *st, qkv, proj, ldp, dt_raw, gate_raw, (bf16*)out));
  } else {
    if (smem > 48 * 1024) THA_CUDA_OK(cudaFuncSetAttribute(hyb_delta_scan_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    THA_CUDA_OK(launch(hyb_delta_scan_kernel<float>, grid, dim3(nt), smem, s, false, *d, *rows, *st, qkv, proj, ldp, dt_raw, gate_raw, (float*)out));
  }
  return THA_STATUS_SUCCESS;
}

extern "C" int tha_hyb_moe_route(void* stream, const tha_moe_t* e, const float* proj, long long ldp, int n_rows, int* expert_id,
                                 float* weight, int* group_off, int* sorted_row, int* inv) {
  if (n_rows < 1) return THA_STATUS_SUCCESS;
  if (e->top < 1 || e->top > 32 || e->top > e->experts) return THA_STATUS_INVALID_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  int* counts = group_off + e->experts + 1;   // the second half of group_off is the routers' counters
  THA_CUDA_OK(cudaMemsetAsync(counts, 0, sizeof(int) * e->experts, s));
  THA_CUDA_OK(launch(hyb_route_kernel, dim3(ceil_div(n_rows, 4)), dim3(128), 0, s, false, e->experts, e->top, e->o_router, proj, ldp, n_rows,
                     expert_id, weight, counts));
  const int nt = 32 * (e->experts < 32 ? e->experts : 32);
  THA_CUDA_OK(launch(hyb_route_sort_kernel, dim3(1), dim3(nt), sizeof(int) * (e->experts + 1), s, false, e->experts, e->top, n_rows,
                     (const int*)expert_id, (const int*)counts, group_off, sorted_row, inv));
  return THA_STATUS_SUCCESS;
}

extern "C" int tha_hyb_glu_clamped(void* stream, int dtype, void* y, const float* gu, long long ldg, int col_g, int col_u, int n,
                                   int ff, float limit, float alpha) {
  if (n < 1) return THA_STATUS_SUCCESS;
  const dim3 grid((unsigned)(((size_t)n * ff + 255) / 256));
  if (dtype == THA_DT_BF16)
    THA_CUDA_OK(launch(hyb_glu_kernel<bf16>, grid, dim3(256), 0, (cudaStream_t)stream, false, (bf16*)y, gu, ldg, col_g, col_u, n, ff, limit, alpha));
  else
    THA_CUDA_OK(launch(hyb_glu_kernel<float>, grid, dim3(256), 0, (cudaStream_t)stream, false, (float*)y, gu, ldg, col_g, col_u, n, ff, limit, alpha));
  return THA_STATUS_SUCCESS;
}
