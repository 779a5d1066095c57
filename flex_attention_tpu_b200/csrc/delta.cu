// delta = rowsum(o * do): the backward preprocess (reference: host-side `jnp.sum(o * do, -1)`,
// flex_attention_dq_bwd.py:697).  Pure streaming: 2 * rows * D * elt bytes read, rows * 4 written,
// so the bound is HBM bandwidth.  Every thread loads one 16-byte chunk of o and of do (fully
// coalesced), multiplies in f32 and the D*elt/16 threads that share a row reduce with shuffles.
#include "common.cuh"

namespace flexattn {
namespace {

template <typename T>
struct Chunk;
template <>
struct Chunk<__nv_bfloat16> {
  static constexpr int kElems = 8;
  static __device__ __forceinline__ float dot(const uint4& a, const uint4& b) {
    const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 fa = __bfloat1622float2(pa[i]), fb = __bfloat1622float2(pb[i]);
      acc = fmaf(fa.x, fb.x, acc);
      acc = fmaf(fa.y, fb.y, acc);
    }
    return acc;
  }
};
template <>
struct Chunk<float> {
  static constexpr int kElems = 4;
  static __device__ __forceinline__ float dot(const uint4& a, const uint4& b) {
    const float* pa = reinterpret_cast<const float*>(&a);
    const float* pb = reinterpret_cast<const float*>(&b);
    return pa[0] * pb[0] + pa[1] * pb[1] + pa[2] * pb[2] + pa[3] * pb[3];
  }
};

// kTPR = threads per row (power of two <= 32)
template <typename T, int kTPR>
__global__ void __launch_bounds__(256) delta_kernel(const uint4* __restrict__ o, const uint4* __restrict__ d_o,
                                                    float* __restrict__ delta, long long n_chunks) {
  const long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  float acc = 0.f;
  if (c < n_chunks) {
    uint4 a = __ldg(o + c), b = __ldg(d_o + c);
    acc = Chunk<T>::dot(a, b);
  }
#pragma unroll
  for (int s = kTPR / 2; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (c < n_chunks && (threadIdx.x & (kTPR - 1)) == 0) delta[c / kTPR] = acc;
}

template <typename T>
cudaError_t launch_t(cudaStream_t st, const FlexAttnParams& p) {
  const long long rows = (long long)p.batch * p.heads * p.seq_q;
  const int tpr = p.head_dim / Chunk<T>::kElems;
  const long long n_chunks = rows * tpr;
  const unsigned blocks = (unsigned)((n_chunks + 255) / 256);
  const uint4* o = static_cast<const uint4*>(p.o);
  const uint4* d_o = static_cast<const uint4*>(p.d_o);
  switch (tpr) {
    case 4: delta_kernel<T, 4><<<blocks, 256, 0, st>>>(o, d_o, p.delta, n_chunks); break;
    case 8: delta_kernel<T, 8><<<blocks, 256, 0, st>>>(o, d_o, p.delta, n_chunks); break;
    case 16: delta_kernel<T, 16><<<blocks, 256, 0, st>>>(o, d_o, p.delta, n_chunks); break;
    case 32: delta_kernel<T, 32><<<blocks, 256, 0, st>>>(o, d_o, p.delta, n_chunks); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_delta(cudaStream_t st, const FlexAttnParams& p) {
  return p.dtype == FLEXATTN_BF16 ? launch_t<__nv_bfloat16>(st, p) : launch_t<float>(st, p);
}

}  // namespace flexattn
