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
  const bool conv = bg >= 100;  // converged-warp issue: all 32 lanes of warp 0 run the loop, one lane's MMA is predicated on
  if (conv) bg -= 100;
  if (conv && warp == 0) {
    const uint32_t tm = __shfl_sync(0xffffffffu, tmem, 0);
    const uint32_t issue = (tid == 0) ? 1u : 0u;
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
        if (variant == 0 || variant == 3) ptx::mma_ss_if(issue, tm, ptx::desc_at(bA, ptx::koff_kmajor(kk)), ptx::desc_at(bB, off), idesc, 1);
        else ptx::mma_ts_if(issue, tm, tm + 256 + kk * 8, ptx::desc_at(bB, off), idesc, 1);
      }
    }
    const long long t1 = clock64();
    ptx::mma_commit_if(issue, bar);
    bool ok = true;
    if (tid == 0) ok = ptx::mbar_wait(bar, 0);
    __syncwarp();
    const long long t2 = clock64();
    if (tid == 0) {
      out[0] = t1 - t0;
      out[1] = t2 - t0;
      out[2] = ok;
      *stop = 1;
    }
  } else if (!conv && tid == 0) {
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
      if (bg == 5 || bg == 6) {   // instruction-level-parallel FMA (5) or FMA + ex2 (6) work: keeps the schedulers busy
        float a[16];
#pragma unroll
        for (int c = 0; c < 16; ++c) a[c] = acc + (float)c;
#pragma unroll 1
        for (int k = 0; k < 16; ++k) {
#pragma unroll
          for (int c = 0; c < 16; ++c) a[c] = fmaf(a[c], 1.0001f, 0.5f);
          if (bg == 6) {
#pragma unroll
            for (int c = 0; c < 16; ++c) a[c] = ptx::ex2(a[c] * 1e-3f);
          }
        }
#pragma unroll
        for (int c = 0; c < 16; ++c) acc += a[c];
      } else if (bg == 1) {          // ALU + special-function work
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


// Trains of 8 instructions that change accumulator (and operand staging) from train to train, as the attention
// kernels do.  mode 0: one accumulator, SS | 1: four accumulators in rotation, SS | 2: the dK/dV kernel's mix
// (TS MN-major -> acc 384, SS -> acc 0 overwrite, TS MN-major -> acc 256, SS -> acc 128 overwrite; the TS A operand
// aliases the SS accumulator columns) | 3: as 2 but every train accumulates | 4: as 2 with the TS trains reading
// A from columns the SS trains do not write.
__global__ void __launch_bounds__(128) mma_mix_kernel(int reps, int mode, long long* out) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = smem + 2 * ptx::kPanelBytes;
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + 6 * ptx::kPanelBytes);
  uint32_t* slot = reinterpret_cast<uint32_t*>(bar + 1);
  const int tid = threadIdx.x, warp = tid >> 5;
  for (int i = tid; i < 6 * (int)ptx::kPanelBytes / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (tid == 0) { ptx::mbar_init(bar, 1); ptx::fence_barrier_init(); }
  if (warp == 0) { ptx::tmem_alloc(slot, 512); ptx::tmem_relinquish(); }
  ptx::fence_proxy_async_smem();
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = *slot;
  if (tid == 0) {
    const uint32_t idesc_k = ptx::make_idesc(128, 128, false), idesc_mn = ptx::make_idesc(128, 128, true);
    const ptx::DescBase bA = ptx::base_kmajor(ptx::smem_u32(sA));
    const ptx::DescBase bBk = ptx::base_kmajor(ptx::smem_u32(sB)), bBm = ptx::base_mnmajor(ptx::smem_u32(sB));
    const long long t0 = clock64();
#pragma unroll 1
    for (int r = 0; r < reps; ++r) {
      if (mode <= 1) {
        const uint32_t acc = tmem + (mode == 1 ? (uint32_t)(r & 3) * 128 : 0u);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          ptx::mma_ss(acc, ptx::desc_at(bA, ptx::koff_kmajor(kk)), ptx::desc_at(bBk, ptx::koff_kmajor(kk)), idesc_k, 1);
      } else {
        const uint32_t a_s = mode == 4 ? 256u : 0u, a_dp = mode == 4 ? 320u : 128u;
        const uint32_t ow = mode == 3 ? 1u : 0u;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          ptx::mma_ts(tmem + 384, tmem + a_s + 64 * (kk >> 2) + (kk & 3) * 8, ptx::desc_at(bBm, ptx::koff_mnmajor(kk)), idesc_mn, 1);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          ptx::mma_ss(tmem, ptx::desc_at(bA, ptx::koff_kmajor(kk)), ptx::desc_at(bBk, ptx::koff_kmajor(kk)), idesc_k, ow | (kk > 0));
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          ptx::mma_ts(tmem + 256, tmem + a_dp + 64 * (kk >> 2) + (kk & 3) * 8, ptx::desc_at(bBm, ptx::koff_mnmajor(kk)), idesc_mn, 1);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          ptx::mma_ss(tmem + 128, ptx::desc_at(bA, ptx::koff_kmajor(kk)), ptx::desc_at(bBk, ptx::koff_kmajor(kk)), idesc_k, ow | (kk > 0));
      }
    }
    const long long t1 = clock64();
    ptx::mma_commit(bar);
    const bool ok = ptx::mbar_wait(bar, 0);
    const long long t2 = clock64();
    out[0] = t1 - t0;
    out[1] = t2 - t0;
    out[2] = ok;
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

extern "C" int flexattn_debug_mma_mix(int mode, int reps, long long* out_device) {
  const size_t smem = 6 * flexattn::ptx::kPanelBytes + 1024 + 64;
  cudaFuncSetAttribute(flexattn::mma_mix_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  flexattn::mma_mix_kernel<<<1, 128, smem>>>(reps, mode, out_device);
  return cudaGetLastError() == cudaSuccess ? 0 : 8;
}
#endif
