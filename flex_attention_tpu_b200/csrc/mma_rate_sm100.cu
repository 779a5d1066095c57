// Instrumented builds only (FLEXATTN_TRACE): measures how many cycles a train of tcgen05.mma instructions
// takes for each operand staging the attention kernels use, to tell tensor-pipe time from operand-fetch time.
#ifdef FLEXATTN_TRACE
#include "sm100.cuh"

namespace flexattn {
namespace {

// variant: 0 = SS, A and B K-major | 1 = TS, B MN-major | 2 = TS, B K-major | 3 = SS, B MN-major
// N = 128 (or n_cols), M = 128, K = 16 per instruction; `reps` trains of 8 instructions.
template <int variant>
__global__ void __launch_bounds__(416) mma_rate_kernel(int reps, int n_cols, long long* out, int bg, float* sink) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = smem + 2 * ptx::kPanelBytes;
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + 6 * ptx::kPanelBytes);
  uint32_t* slot = reinterpret_cast<uint32_t*>(bar + 1);
  const int tid = threadIdx.x, warp = tid >> 5;
  for (int i = tid; i < 6 * (int)ptx::kPanelBytes / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  volatile int* stop = reinterpret_cast<volatile int*>(slot + 1);
  if (tid == 0) *stop = 0;
  if (tid == 0) { ptx::mbar_init(bar, 1); ptx::fence_barrier_init(); }
  if (warp == 0) { ptx::tmem_alloc(slot, 512); ptx::tmem_relinquish(); }
  ptx::fence_proxy_async_smem();
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = *slot;
  if (tid == 0) {
    const uint32_t idesc = ptx::make_idesc(128, n_cols, variant == 1 || variant == 3);
    const ptx::DescBase bA = ptx::base_kmajor(ptx::smem_u32(sA));
    const ptx::DescBase bB = (variant == 1 || variant == 3) ? ptx::base_mnmajor(ptx::smem_u32(sB))
                                                            : ptx::base_kmajor(ptx::smem_u32(sB));
    const long long t0 = clock64();
#pragma unroll 1
    for (int r = 0; r < reps; ++r) {
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint32_t off = (variant == 1 || variant == 3) ? ptx::koff_mnmajor(kk) : ptx::koff_kmajor(kk);
        if (variant == 0 || variant == 3) ptx::mma_ss(tmem, ptx::desc_at(bA, ptx::koff_kmajor(kk)), ptx::desc_at(bB, off), idesc, 1);
        else ptx::mma_ts(tmem, tmem + 256 + kk * 8, ptx::desc_at(bB, off), idesc, 1);
      }
    }
    const long long t1 = clock64();
    ptx::mma_commit(bar);
    const bool ok = ptx::mbar_wait(bar, 0);
    const long long t2 = clock64();
    out[0] = t1 - t0;
    out[1] = t2 - t0;
    out[2] = ok;
    *stop = 1;
  } else if (warp >= 4 && bg != 0) {
    // background load from 8 other warps (two per scheduler) while the MMAs run
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    float acc = (float)tid;
    uint32_t r[32];
    int it = 0;
    while (*stop == 0 && it < 100000) {
      ++it;
      if (bg == 1) {          // ALU + special-function work
#pragma unroll
        for (int c = 0; c < 32; ++c) acc = ptx::ex2(acc * 0.5f - 1.0f) + 0.25f;
      } else if (bg == 2) {   // tensor-memory loads (columns 384..415, not touched by the MMAs)
        ptx::tmem_ld32(lane_base + 384, r);
        ptx::tmem_wait_ld();
        ptx::tmem_ld_acquire(r);
        acc += __uint_as_float(r[it & 31]);
      } else if (bg == 3) {   // shared-memory stores (16-byte, conflict-free)
        *reinterpret_cast<uint4*>(smem + 5 * ptx::kPanelBytes + ((tid - 128) & 255) * 16) = make_uint4(it, it, it, it);
      } else {                // tensor-memory stores
#pragma unroll
        for (int c = 0; c < 32; ++c) r[c] = it;
        ptx::tmem_st32(lane_base + 416, r);
        ptx::tmem_wait_st();
      }
    }
    sink[tid] = acc;
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 0) { ptx::tc_fence_after(); ptx::tmem_dealloc(tmem, 512); }
}

}  // namespace
}  // namespace flexattn

extern "C" int flexattn_debug_mma_rate(int variant, int reps, int n_cols, long long* out_device, int bg, float* sink) {
  const size_t smem = 6 * flexattn::ptx::kPanelBytes + 1024 + 64;
#define FA_RATE(V)                                                                                              \
  case V:                                                                                                       \
    cudaFuncSetAttribute(flexattn::mma_rate_kernel<V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    flexattn::mma_rate_kernel<V><<<1, 384, smem>>>(reps, n_cols, out_device, bg, sink);                                   \
    break;
  switch (variant) {
    FA_RATE(0) FA_RATE(1) FA_RATE(2) FA_RATE(3)
    default: return 2;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 8;
}
#endif
