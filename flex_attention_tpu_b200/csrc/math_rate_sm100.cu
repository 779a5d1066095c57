// Instrumented builds only (FLEXATTN_TRACE): cycles of the element-wise inner loops on register data, to
// separate special-function, conversion and issue costs.
#ifdef FLEXATTN_TRACE
#include "sm100.cuh"

namespace flexattn {
namespace {

template <int V>
__global__ void math_rate_kernel(const float* __restrict__ in, float* __restrict__ outv, long long* out, int reps) {
  __shared__ __align__(16) float s_nl[64];
  __shared__ __align__(16) float s_dl[64];
  if (threadIdx.x < 64) { s_nl[threadIdx.x] = in[threadIdx.x] * 0.01f; s_dl[threadIdx.x] = in[64 + threadIdx.x] * 0.01f; }
  __syncthreads();
  float s[64], dp[64];
#pragma unroll
  for (int c = 0; c < 64; ++c) { s[c] = in[(threadIdx.x * 64 + c) & 4095]; dp[c] = in[(threadIdx.x * 64 + c + 77) & 4095]; }
  uint32_t acc = 0;
  float facc = 0.f;
  const long long t0 = clock64();
#pragma unroll 1
  for (int r = 0; r < reps; ++r) {
    if constexpr (V == 0) {          // 64 independent ex2
#pragma unroll
      for (int c = 0; c < 64; ++c) acc ^= __float_as_uint(ptx::ex2(s[c] + (float)r));
    } else if constexpr (V == 1) {   // 32 cvt.rn.bf16x2 packs of fma results
#pragma unroll
      for (int c = 0; c < 64; c += 2) acc ^= ptx::pack_bf16(fmaf(s[c], 0.127f, (float)r), fmaf(s[c + 1], 0.3f, (float)r));
    } else if constexpr (V == 2 || V == 3) {   // dkv-style half: fma, ex2, sub, mul, truncation packs; V == 2 reads stats from smem
#pragma unroll
      for (int c = 0; c < 64; c += 4) {
        float nl[4], dl[4];
        if constexpr (V == 2) {
          const float4 nl4 = *reinterpret_cast<const float4*>(s_nl + c);
          const float4 dl4 = *reinterpret_cast<const float4*>(s_dl + c);
          nl[0] = nl4.x; nl[1] = nl4.y; nl[2] = nl4.z; nl[3] = nl4.w;
          dl[0] = dl4.x; dl[1] = dl4.y; dl[2] = dl4.z; dl[3] = dl4.w;
        } else {
#pragma unroll
          for (int u = 0; u < 4; ++u) { nl[u] = 0.25f; dl[u] = 0.5f; }
        }
        float pv[4], dv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          pv[u] = ptx::ex2(fmaf(s[c + u], 0.127f, nl[u] + (float)r));
          dv[u] = pv[u] * (dp[c + u] - dl[u]);
        }
        acc ^= ptx::pack_bf16_trunc(pv[0], pv[1]) ^ ptx::pack_bf16_trunc(pv[2], pv[3]) ^ ptx::pack_bf16_trunc(dv[0], dv[1]) ^
               ptx::pack_bf16_trunc(dv[2], dv[3]);
      }
    } else if constexpr (V == 4) {   // 64 fma + 32 truncation packs
#pragma unroll
      for (int c = 0; c < 64; c += 2) acc ^= ptx::pack_bf16_trunc(fmaf(s[c], 0.127f, (float)r), fmaf(s[c + 1], 0.3f, (float)r));
    } else if constexpr (V == 5) {   // 64 (fma + ex2) + 32 truncation packs
#pragma unroll
      for (int c = 0; c < 64; c += 2)
        acc ^= ptx::pack_bf16_trunc(ptx::ex2(fmaf(s[c], 0.127f, (float)r)), ptx::ex2(fmaf(s[c + 1], 0.3f, (float)r)));
    } else {                          // 64 polynomial exp2
#pragma unroll
      for (int c = 0; c < 64; ++c) acc ^= __float_as_uint(fmaf(s[c], s[c], (float)r));
    }
  }
  const long long t1 = clock64();
  outv[blockIdx.x * blockDim.x + threadIdx.x] = facc + __uint_as_float(acc);
  if (threadIdx.x == 0 && blockIdx.x == 0) out[0] = t1 - t0;
}

}  // namespace
}  // namespace flexattn

extern "C" int flexattn_debug_math_rate(int variant, int threads, int reps, const float* in, float* outv,
                                        long long* out_device) {
  using namespace flexattn;
  switch (variant) {
    case 0: math_rate_kernel<0><<<1, threads>>>(in, outv, out_device, reps); break;
    case 1: math_rate_kernel<1><<<1, threads>>>(in, outv, out_device, reps); break;
    case 2: math_rate_kernel<2><<<1, threads>>>(in, outv, out_device, reps); break;
    case 3: math_rate_kernel<3><<<1, threads>>>(in, outv, out_device, reps); break;
    case 4: math_rate_kernel<4><<<1, threads>>>(in, outv, out_device, reps); break;
    case 5: math_rate_kernel<5><<<1, threads>>>(in, outv, out_device, reps); break;
    default: math_rate_kernel<6><<<1, threads>>>(in, outv, out_device, reps); break;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 8;
}
#endif
