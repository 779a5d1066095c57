// CUDA-core (SIMT) flex-attention kernels: forward, dQ and dK/dV with f32 arithmetic throughout.
//
// They serve the float32 dtype (tcgen05 has no fp32 MMA; the f32 tolerance of 2e-3 on gradients rules
// out tf32) and any head_dim in {32, 64, 128}, and they are the on-GPU cross-check for the tensor-core
// kernels.  One warp owns one row (a query row in fwd/dq, a key row in dkv); the lanes split the
// opposite-side positions 32 at a time for the score dot products and split head_dim for the
// accumulators.  Tile skipping follows the same mask map as the tensor-core kernels.
#include "common.cuh"

namespace flexattn {
namespace {

__device__ __forceinline__ float to_f(float x) { return x; }
__device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ void from_f(float* p, float x) { *p = x; }
__device__ __forceinline__ void from_f(__nv_bfloat16* p, float x) { *p = __float2bfloat16_rn(x); }

// <row in global memory, vector in shared memory>
template <int D>
__device__ __forceinline__ float dot_row(const float* __restrict__ g, const float* __restrict__ s) {
  float acc = 0.f;
#pragma unroll 4
  for (int d = 0; d < D; d += 4) {
    float4 x = *reinterpret_cast<const float4*>(g + d);
    acc = fmaf(x.x, s[d], acc); acc = fmaf(x.y, s[d + 1], acc);
    acc = fmaf(x.z, s[d + 2], acc); acc = fmaf(x.w, s[d + 3], acc);
  }
  return acc;
}
template <int D>
__device__ __forceinline__ float dot_row(const __nv_bfloat16* __restrict__ g, const float* __restrict__ s) {
  float acc = 0.f;
#pragma unroll 4
  for (int d = 0; d < D; d += 8) {
    uint4 raw = *reinterpret_cast<const uint4*>(g + d);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float2 f = __bfloat1622float2(h[u]);
      acc = fmaf(f.x, s[d + 2 * u], acc);
      acc = fmaf(f.y, s[d + 2 * u + 1], acc);
    }
  }
  return acc;
}

__device__ __forceinline__ bool keep_rt(int kind, int i, int j, int window, int stride, int di, int dj) {
  switch (kind) {
    case FLEXATTN_MASK_CAUSAL: return mask_keep<FLEXATTN_MASK_CAUSAL>(i, j, window, stride, di, dj);
    case FLEXATTN_MASK_SLIDING_WINDOW: return mask_keep<FLEXATTN_MASK_SLIDING_WINDOW>(i, j, window, stride, di, dj);
    case FLEXATTN_MASK_SLIDING_WINDOW_CAUSAL:
      return mask_keep<FLEXATTN_MASK_SLIDING_WINDOW_CAUSAL>(i, j, window, stride, di, dj);
    case FLEXATTN_MASK_DOCUMENT: return mask_keep<FLEXATTN_MASK_DOCUMENT>(i, j, window, stride, di, dj);
    case FLEXATTN_MASK_S2: return mask_keep<FLEXATTN_MASK_S2>(i, j, window, stride, di, dj);
    default: return true;
  }
}
__device__ __forceinline__ float score_rt(int kind, float s, int i, int j, float slope, float cap, float inv_cap) {
  switch (kind) {
    case FLEXATTN_SCORE_ALIBI: return score_fwd<FLEXATTN_SCORE_ALIBI>(s, i, j, slope, cap, inv_cap);
    case FLEXATTN_SCORE_SOFTCAP: return score_fwd<FLEXATTN_SCORE_SOFTCAP>(s, i, j, slope, cap, inv_cap);
    default: return s;
  }
}
__device__ __forceinline__ float dsig_rt(int kind, float s, float inv_cap) {
  return kind == FLEXATTN_SCORE_SOFTCAP ? score_dsig<FLEXATTN_SCORE_SOFTCAP>(s, inv_cap) : 1.0f;
}

constexpr int kWarps = 4;

template <typename T, int D>
__global__ void __launch_bounds__(kWarps * 32) simt_fwd_kernel(DevParams P, int score, int mask) {
  __shared__ float s_q[kWarps][D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * kWarps + warp;
  const long long n_rows = (long long)P.batch * P.heads * P.seq_q;
  if (row >= n_rows) return;
  const int i = (int)(row % P.seq_q);
  const int bh = (int)(row / P.seq_q), b = bh / P.heads, h = bh % P.heads;
  const T* q = static_cast<const T*>(P.q) + row * D;
  const T* k = static_cast<const T*>(P.k) + (size_t)bh * P.seq_k * D;
  const T* v = static_cast<const T*>(P.v) + (size_t)bh * P.seq_k * D;
  for (int d = lane; d < D; d += 32) s_q[warp][d] = to_f(q[d]);
  __syncwarp();
  const int4 rm = P.row_map[(size_t)(P.map_rows > 1 ? b : 0) * P.n_qt + i / kTile];
  const int kbeg = rm.x * kTile, kend = min(rm.y * kTile, P.seq_k);
  const int* doc = P.doc_ids ? P.doc_ids + (size_t)b * P.doc_stride : nullptr;
  const int di = doc ? doc[i] : 0;
  const float slope = P.alibi_slopes ? P.alibi_slopes[h] : 0.f;
  const float inv_cap = P.cap != 0.f ? 1.f / P.cap : 0.f;
  float m = kMasked, l = 0.f;
  float acc[D / 32];
#pragma unroll
  for (int t = 0; t < D / 32; ++t) acc[t] = 0.f;
  for (int j0 = kbeg; j0 < kend; j0 += 32) {
    const int j = j0 + lane;
    const bool valid = j < kend;
    float x = kMasked;
    if (valid) {
      float s = dot_row<D>(k + (size_t)j * D, s_q[warp]) * P.sm_scale;
      if (keep_rt(mask, i, j, P.window, P.stride, di, doc ? doc[j] : 0))
        x = score_rt(score, s, i, j, slope, P.cap, inv_cap) + (P.ab ? P.ab[(size_t)row * P.seq_k + j] : 0.f);
    }
    float mx = x;
#pragma unroll
    for (int sft = 16; sft > 0; sft >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, sft));
    const float m_new = fmaxf(m, mx);
    const float alpha = __expf(m - m_new);
    float p = valid ? __expf(x - m_new) : 0.f;
    float ps = p;
#pragma unroll
    for (int sft = 16; sft > 0; sft >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, sft);
    l = l * alpha + ps;
    m = m_new;
#pragma unroll
    for (int t = 0; t < D / 32; ++t) acc[t] *= alpha;
    const int n = min(32, kend - j0);
    for (int jj = 0; jj < n; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const T* vr = v + (size_t)(j0 + jj) * D;
#pragma unroll
      for (int t = 0; t < D / 32; ++t) acc[t] = fmaf(pj, to_f(vr[lane + 32 * t]), acc[t]);
    }
  }
  const float inv_l = l > 0.f ? 1.f / l : 0.f;
  T* o = static_cast<T*>(P.o) + row * D;
#pragma unroll
  for (int t = 0; t < D / 32; ++t) from_f(o + lane + 32 * t, acc[t] * inv_l);
  if (lane == 0) { P.l[row] = l; P.m[row] = m; }
}

template <typename T, int D>
__global__ void __launch_bounds__(kWarps * 32) simt_dq_kernel(DevParams P, int score, int mask) {
  __shared__ float s_q[kWarps][D];
  __shared__ float s_do[kWarps][D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * kWarps + warp;
  const long long n_rows = (long long)P.batch * P.heads * P.seq_q;
  if (row >= n_rows) return;
  const int i = (int)(row % P.seq_q);
  const int bh = (int)(row / P.seq_q), b = bh / P.heads, h = bh % P.heads;
  const T* q = static_cast<const T*>(P.q) + row * D;
  const T* dO = static_cast<const T*>(P.d_o) + row * D;
  const T* k = static_cast<const T*>(P.k) + (size_t)bh * P.seq_k * D;
  const T* v = static_cast<const T*>(P.v) + (size_t)bh * P.seq_k * D;
  for (int d = lane; d < D; d += 32) { s_q[warp][d] = to_f(q[d]); s_do[warp][d] = to_f(dO[d]); }
  __syncwarp();
  const int4 rm = P.row_map[(size_t)(P.map_rows > 1 ? b : 0) * P.n_qt + i / kTile];
  const int kbeg = rm.x * kTile, kend = min(rm.y * kTile, P.seq_k);
  const int* doc = P.doc_ids ? P.doc_ids + (size_t)b * P.doc_stride : nullptr;
  const int di = doc ? doc[i] : 0;
  const float slope = P.alibi_slopes ? P.alibi_slopes[h] : 0.f;
  const float inv_cap = P.cap != 0.f ? 1.f / P.cap : 0.f;
  const float m = P.m[row], l = P.l[row], delta = P.delta[row];
  const float inv_l = l > 0.f ? 1.f / l : 0.f;
  float acc[D / 32];
#pragma unroll
  for (int t = 0; t < D / 32; ++t) acc[t] = 0.f;
  if (P.dab) {  // the bias gradient is dense: zero outside the kv tiles this row visits
    float* dab_row = P.dab + (size_t)row * P.seq_k;
    for (int j = lane; j < kbeg; j += 32) dab_row[j] = 0.f;
    for (int j = kend + lane; j < P.seq_k; j += 32) dab_row[j] = 0.f;
  }
  for (int j0 = kbeg; j0 < kend; j0 += 32) {
    const int j = j0 + lane;
    float ds = 0.f, dt = 0.f;  // dt: gradient of the logit after the score function (what the bias sees)
    if (j < kend && keep_rt(mask, i, j, P.window, P.stride, di, doc ? doc[j] : 0)) {
      const float s = dot_row<D>(k + (size_t)j * D, s_q[warp]) * P.sm_scale;
      const float x = score_rt(score, s, i, j, slope, P.cap, inv_cap) + (P.ab ? P.ab[(size_t)row * P.seq_k + j] : 0.f);
      const float p = __expf(x - m) * inv_l;
      const float dp = dot_row<D>(v + (size_t)j * D, s_do[warp]);
      dt = p * (dp - delta);
      ds = dt * dsig_rt(score, s, inv_cap) * P.sm_scale;
    }
    if (P.dab && j < kend) P.dab[(size_t)row * P.seq_k + j] = dt;
    const int n = min(32, kend - j0);
    for (int jj = 0; jj < n; ++jj) {
      const float dsj = __shfl_sync(0xffffffffu, ds, jj);
      const T* kr = k + (size_t)(j0 + jj) * D;
#pragma unroll
      for (int t = 0; t < D / 32; ++t) acc[t] = fmaf(dsj, to_f(kr[lane + 32 * t]), acc[t]);
    }
  }
  T* dq = static_cast<T*>(P.dq) + row * D;
#pragma unroll
  for (int t = 0; t < D / 32; ++t) from_f(dq + lane + 32 * t, acc[t]);
}

template <typename T, int D>
__global__ void __launch_bounds__(kWarps * 32) simt_dkv_kernel(DevParams P, int score, int mask) {
  __shared__ float s_k[kWarps][D];
  __shared__ float s_v[kWarps][D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * kWarps + warp;
  const long long n_rows = (long long)P.batch * P.heads * P.seq_k;
  if (row >= n_rows) return;
  const int j = (int)(row % P.seq_k);
  const int bh = (int)(row / P.seq_k), b = bh / P.heads, h = bh % P.heads;
  const T* kr = static_cast<const T*>(P.k) + row * D;
  const T* vr = static_cast<const T*>(P.v) + row * D;
  const T* q = static_cast<const T*>(P.q) + (size_t)bh * P.seq_q * D;
  const T* dO = static_cast<const T*>(P.d_o) + (size_t)bh * P.seq_q * D;
  const float* lrow = P.l + (size_t)bh * P.seq_q;
  const float* mrow = P.m + (size_t)bh * P.seq_q;
  const float* drow = P.delta + (size_t)bh * P.seq_q;
  for (int d = lane; d < D; d += 32) { s_k[warp][d] = to_f(kr[d]); s_v[warp][d] = to_f(vr[d]); }
  __syncwarp();
  const int4 cm = P.col_map[(size_t)(P.map_rows > 1 ? b : 0) * P.n_kt + j / kTile];
  const int qbeg = cm.x * kTile, qend = min(cm.y * kTile, P.seq_q);
  const int* doc = P.doc_ids ? P.doc_ids + (size_t)b * P.doc_stride : nullptr;
  const int dj = doc ? doc[j] : 0;
  const float slope = P.alibi_slopes ? P.alibi_slopes[h] : 0.f;
  const float inv_cap = P.cap != 0.f ? 1.f / P.cap : 0.f;
  float acc_k[D / 32], acc_v[D / 32];
#pragma unroll
  for (int t = 0; t < D / 32; ++t) { acc_k[t] = 0.f; acc_v[t] = 0.f; }
  for (int i0 = qbeg; i0 < qend; i0 += 32) {
    const int i = i0 + lane;
    float p = 0.f, ds = 0.f;
    if (i < qend && keep_rt(mask, i, j, P.window, P.stride, doc ? doc[i] : 0, dj)) {
      const float s = dot_row<D>(q + (size_t)i * D, s_k[warp]) * P.sm_scale;
      const float x = score_rt(score, s, i, j, slope, P.cap, inv_cap) +
                      (P.ab ? P.ab[((size_t)bh * P.seq_q + i) * P.seq_k + j] : 0.f);
      const float l = lrow[i];
      p = __expf(x - mrow[i]) * (l > 0.f ? 1.f / l : 0.f);
      const float dp = dot_row<D>(dO + (size_t)i * D, s_v[warp]);
      ds = p * (dp - drow[i]) * dsig_rt(score, s, inv_cap) * P.sm_scale;
    }
    const int n = min(32, qend - i0);
    for (int ii = 0; ii < n; ++ii) {
      const float pi = __shfl_sync(0xffffffffu, p, ii);
      const float dsi = __shfl_sync(0xffffffffu, ds, ii);
      const T* qr = q + (size_t)(i0 + ii) * D;
      const T* dor = dO + (size_t)(i0 + ii) * D;
#pragma unroll
      for (int t = 0; t < D / 32; ++t) {
        acc_v[t] = fmaf(pi, to_f(dor[lane + 32 * t]), acc_v[t]);
        acc_k[t] = fmaf(dsi, to_f(qr[lane + 32 * t]), acc_k[t]);
      }
    }
  }
  T* dk = static_cast<T*>(P.dk) + row * D;
  T* dv = static_cast<T*>(P.dv) + row * D;
#pragma unroll
  for (int t = 0; t < D / 32; ++t) {
    from_f(dk + lane + 32 * t, acc_k[t]);
    from_f(dv + lane + 32 * t, acc_v[t]);
  }
}

#define FLEXATTN_SIMT_DISPATCH(KERNEL)                                                              \
  do {                                                                                              \
    const unsigned blocks = (unsigned)((rows + kWarps - 1) / kWarps);                               \
    if (dtype == FLEXATTN_BF16) {                                                                   \
      if (d.head_dim == 32) KERNEL<__nv_bfloat16, 32><<<blocks, kWarps * 32, 0, st>>>(d, score, mask);        \
      else if (d.head_dim == 64) KERNEL<__nv_bfloat16, 64><<<blocks, kWarps * 32, 0, st>>>(d, score, mask);   \
      else if (d.head_dim == 128) KERNEL<__nv_bfloat16, 128><<<blocks, kWarps * 32, 0, st>>>(d, score, mask); \
      else return cudaErrorInvalidValue;                                                            \
    } else {                                                                                        \
      if (d.head_dim == 32) KERNEL<float, 32><<<blocks, kWarps * 32, 0, st>>>(d, score, mask);      \
      else if (d.head_dim == 64) KERNEL<float, 64><<<blocks, kWarps * 32, 0, st>>>(d, score, mask); \
      else if (d.head_dim == 128) KERNEL<float, 128><<<blocks, kWarps * 32, 0, st>>>(d, score, mask); \
      else return cudaErrorInvalidValue;                                                            \
    }                                                                                               \
    return cudaGetLastError();                                                                      \
  } while (0)

}  // namespace

cudaError_t launch_simt_fwd(cudaStream_t st, const DevParams& d, int dtype, int score, int mask) {
  const long long rows = (long long)d.batch * d.heads * d.seq_q;
  FLEXATTN_SIMT_DISPATCH(simt_fwd_kernel);
}
cudaError_t launch_simt_dq(cudaStream_t st, const DevParams& d, int dtype, int score, int mask) {
  const long long rows = (long long)d.batch * d.heads * d.seq_q;
  FLEXATTN_SIMT_DISPATCH(simt_dq_kernel);
}
cudaError_t launch_simt_dkv(cudaStream_t st, const DevParams& d, int dtype, int score, int mask) {
  const long long rows = (long long)d.batch * d.heads * d.seq_k;
  FLEXATTN_SIMT_DISPATCH(simt_dkv_kernel);
}

}  // namespace flexattn
