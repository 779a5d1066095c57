// Single-tile tensor-core self checks: the smallest kernels that exercise exactly the operand
// staging the attention kernels rely on (TMA 128-byte swizzle -> tcgen05.mma descriptors, bf16 A
// operand in tensor memory, MN-major B operand).  The test-suite compares them with a host matmul.
#include "sm100.cuh"

namespace flexattn {
namespace {

__global__ void __launch_bounds__(128) selftest_kernel(const __grid_constant__ CUtensorMap tm_a,
                                                       const __grid_constant__ CUtensorMap tm_b,
                                                       const __nv_bfloat16* __restrict__ a_glob,
                                                       float* __restrict__ d_out, int variant, int kdim,
                                                       int32_t* status, int* abort_flag) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;                      // 2 panels x 16 KB
  uint8_t* sB = smem + 2 * ptx::kPanelBytes;
  uint64_t* bar_load = reinterpret_cast<uint64_t*>(smem + 4 * ptx::kPanelBytes);
  uint64_t* bar_mma = bar_load + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_load + 2);
  const int tid = threadIdx.x, warp = tid >> 5;
  constexpr uint32_t kCols = 256;

  if (tid == 0) {
    ptx::mbar_init(bar_load, 1);
    ptx::mbar_init(bar_mma, 1);
    ptx::fence_barrier_init();
  }
  if (warp == 0) {
    ptx::tmem_alloc(tmem_slot, kCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
  const uint32_t tD = 0, tA = 128;  // column offsets
  const int panels = kdim / 64;
  bool ok = true;

  if (tid == 0) {
    // K-major tiles have kdim / 64 panels, the MN-major B tile ([K, 128]) always two
    const int a_panels = variant == 0 ? panels : 0, b_panels = variant == 0 ? panels : 2;
    ptx::mbar_arrive_expect_tx(bar_load, (uint32_t)(a_panels + b_panels) * ptx::kPanelBytes);
    for (int p = 0; p < a_panels; ++p) ptx::tma_load_3d(sA + p * ptx::kPanelBytes, &tm_a, bar_load, p * 64, 0, 0);
    for (int p = 0; p < b_panels; ++p) ptx::tma_load_3d(sB + p * ptx::kPanelBytes, &tm_b, bar_load, p * 64, 0, 0);
  }
  const bool a_tmem = variant == 1;
  const bool b_mn = variant != 0;
  if (a_tmem) {
    // stage A row `tid` into tensor memory as packed bf16 pairs (element k -> column k/2, low half = even k)
    const uint32_t* row = reinterpret_cast<const uint32_t*>(a_glob + (size_t)tid * kdim);
    for (int c0 = 0; c0 < kdim / 2; c0 += 32) {
      uint32_t r[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) r[c] = row[c0 + c];
      ptx::tmem_st32(lane_base + tA + c0, r);
    }
    ptx::tmem_wait_st();
    ptx::tc_fence_before();
  }
  __syncthreads();
  if (tid == 0) {
    ok = ptx::mbar_wait(bar_load, 0);
    if (ok) {
      ptx::tc_fence_after();
      const int ksteps = kdim / 16;
      // exactly the descriptors of the attention kernels: K-major operands step 32 bytes per K step inside a
      // 128-byte-swizzled panel (LBO 16, SBO 1024); MN-major operands step 2048 bytes (LBO = one panel, SBO 1024)
      const uint32_t idesc = ptx::make_idesc(128, 128, b_mn);
      for (int kk = 0; kk < ksteps; ++kk) {
        const uint64_t bdesc = b_mn ? ptx::desc_mnmajor(ptx::smem_u32(sB), kk) : ptx::desc_kmajor(ptx::smem_u32(sB), kk);
        if (a_tmem) ptx::mma_ts(tmem + tD, tmem + tA + kk * 8, bdesc, idesc, kk > 0);
        else ptx::mma_ss(tmem + tD, ptx::desc_kmajor(ptx::smem_u32(sA), kk), bdesc, idesc, kk > 0);
      }
      ptx::mma_commit(bar_mma);
    } else {
      give_up(abort_flag, status, 100, 1);
    }
  }
  __syncwarp();
  if (ptx::mbar_wait(bar_mma, 0)) {
    ptx::tc_fence_after();
#pragma unroll 1
    for (int c0 = 0; c0 < 128; c0 += 32) {
      uint32_t r[32];
      ptx::tmem_ld32(lane_base + tD + c0, r);
      ptx::tmem_wait_ld();
      ptx::tmem_ld_acquire(r);
#pragma unroll
      for (int c = 0; c < 32; ++c) d_out[(size_t)tid * 128 + c0 + c] = __uint_as_float(r[c]);
    }
  } else {
    give_up(abort_flag, status, 100, 2);
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, kCols);
  }
}

// A wait that cannot succeed: nothing ever arrives on the barrier.  It runs out after `limit_ns`, after which the
// thread reports through the same give_up path as the attention kernels (status words + the device's abort word)
// and the kernel returns normally.  Lets the test-suite exercise the time-out handling without a fault or a hang.
__global__ void __launch_bounds__(32) timeout_selftest_kernel(unsigned long long limit_ns, int32_t* status,
                                                              int* abort_flag) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    ptx::mbar_init(&bar, 1);
    ptx::fence_barrier_init();
    const unsigned long long t0 = ptx::globaltimer_ns();
    bool done = false;
    while (!done && ptx::globaltimer_ns() - t0 < limit_ns) {
#pragma unroll 1
      for (int it = 0; it < 64 && !done; ++it) done = ptx::mbar_try_wait(&bar, 0);
    }
    if (!done) give_up(abort_flag, status, 101, 1);
  }
}

}  // namespace
}  // namespace flexattn

using namespace flexattn;

extern "C" int flexattn_selftest_umma(void* stream, int variant, const void* a, const void* b, float* d, int32_t kdim,
                                      int32_t* status) {
  if (a == nullptr || b == nullptr || d == nullptr) return FLEXATTN_ERR_NULL_POINTER;
  if ((variant != 0 && variant != 1) || (kdim != 64 && kdim != 128)) return FLEXATTN_ERR_BAD_SHAPE;
  int* af = abort_flag_ptr();
  if (af == nullptr) return FLEXATTN_ERR_CUDA;
  CUtensorMap tm_a, tm_b;
  int e = make_tile_map(&tm_a, a, 1, 128, kdim);  // [128, K] (only read through TMA by variant 0)
  if (e) return e;
  e = variant == 0 ? make_tile_map(&tm_b, b, 1, 128, kdim) : make_tile_map(&tm_b, b, 1, kdim, 128);
  if (e) return e;
  const size_t smem = 4 * ptx::kPanelBytes + 1024 + 64;
  static SmemAttrOnce attr_once{};
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(selftest_kernel), (int)smem, &attr_once) != FLEXATTN_OK)
    return FLEXATTN_ERR_CUDA;
  selftest_kernel<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(
      tm_a, tm_b, static_cast<const __nv_bfloat16*>(a), d, variant, kdim, status, af);
  return cudaGetLastError() == cudaSuccess ? FLEXATTN_OK : FLEXATTN_ERR_CUDA;
}

extern "C" int flexattn_selftest_timeout(void* stream, int32_t limit_ms, int32_t* status) {
  if (limit_ms < 1 || limit_ms > 1000) return FLEXATTN_ERR_BAD_SHAPE;
  int* af = abort_flag_ptr();
  if (af == nullptr) return FLEXATTN_ERR_CUDA;
  timeout_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(1000000ull * (unsigned long long)limit_ms,
                                                                           status, af);
  return cudaGetLastError() == cudaSuccess ? FLEXATTN_OK : FLEXATTN_ERR_CUDA;
}

extern "C" int flexattn_reset_abort(void* stream) {
  int* af = abort_flag_ptr();
  if (af == nullptr) return FLEXATTN_ERR_CUDA;
  return cudaMemsetAsync(af, 0, sizeof(int), static_cast<cudaStream_t>(stream)) == cudaSuccess ? FLEXATTN_OK
                                                                                               : FLEXATTN_ERR_CUDA;
}
