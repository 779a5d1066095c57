// Thin inline-PTX layer for sm_100a: mbarrier, TMA (cp.async.bulk.tensor, never multicast),
// tcgen05 (tensor memory allocation, MMA, commit, ld/st, fences) and the shared-memory / instruction
// descriptors the MMAs consume.  Every wait is bounded: it gives up after kWaitLimitNs and reports.
#pragma once
#ifndef FLEXATTN_JIT
#include <cuda.h>
#endif

#include "common.cuh"

namespace flexattn {
namespace ptx {

constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s: far beyond any legitimate wait

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}\n"
      : "=r"(pred));
  return pred != 0;
}

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Waits for the phase with the given parity to complete.  false = gave up (time limit).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int it = 0; it < 256; ++it)
      if (mbar_try_wait(bar, parity)) return true;
    if (globaltimer_ns() - t0 > kWaitLimitNs) return false;
  }
}

// Register reallocation between warpgroups (all four warps of a warpgroup execute it): the element-wise warpgroups
// of a kernel take the registers its single-lane TMA / MMA warps do not need.  The two calls must sit at the top of
// the two arms of ONE branch on the warp index, so that the compiler allocates each arm against its own limit.
template <int kRegs>
__device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegs));
}
template <int kRegs>
__device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegs));
}

// One arrival per WARP instead of one per thread: an arrive is a shared-memory atomic, and 32 of them to one
// address serialise.  Every lane has completed its part (its own tcgen05.wait / fence, then the warp barrier,
// which orders memory among the lanes); lane 0's arrive then publishes the whole warp's work.  Barriers used
// this way are initialised with the number of arriving WARPS.
__device__ __forceinline__ void mbar_arrive_warp(uint64_t* bar) {
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}

// The same wait for threads whose wake-up latency does not matter (producers waiting for a free stage): they
// sleep between polls, so that their polling does not take issue slots from the warps that share their scheduler.
__device__ __forceinline__ bool mbar_wait_relaxed(uint64_t* bar, uint32_t parity, unsigned sleep_ns = 100) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int it = 0; it < 256; ++it) {
      __nanosleep(sleep_ns);
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (globaltimer_ns() - t0 > kWaitLimitNs) return false;
  }
}

// 4-byte asynchronous copy global -> shared (no register staging: the issuing thread does not wait for the data)
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gsrc))
               : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// ------------------------------------------------------------------ TMA (no multicast anywhere)
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 3-D tiled load: coordinates (c0 = innermost element, c1 = row, c2 = batch*head slice)
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int c0,
                                            int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1),
      "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* m, const void* smem_src, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// generic-proxy writes to shared memory -> visible to the async proxy (TMA store, tcgen05.mma operands)
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ------------------------------------------------------------------ tensor memory
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {  // whole warp
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp gets lane (32*(warp%4) + t)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
      "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]),
      "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
// tcgen05.ld is asynchronous: its destination registers hold data only after tcgen05.wait::ld.  Passing
// each register through an empty volatile asm AFTER the wait pins every later use behind the wait
// (volatile asm statements keep their program order).
__device__ __forceinline__ void tmem_ld_acquire(uint32_t (&r)[32]) {
#pragma unroll
  for (int c = 0; c < 32; ++c) asm volatile("" : "+r"(r[c]));
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// ------------------------------------------------------------------ descriptors
// Shared-memory matrix descriptor (64 bit): start address >> 4 in [0,14), leading byte offset >> 4 in
// [16,30), stride byte offset >> 4 in [32,46), descriptor version 1 in [46,48), layout type in [61,64)
// (2 = 128-byte swizzle).  Tiles are 1024-byte aligned so the base-offset field stays 0.
constexpr uint64_t kSwizzle128B = 2;
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3fffu);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32;
  d |= (uint64_t)1 << 46;
  d |= kSwizzle128B << 61;
  return d;
}
// Operand tile layouts used by every kernel here (bf16, TMA 128-byte swizzle, 64-element = 128-byte rows,
// one 16 KB "panel" per 64 elements of the contiguous dimension, 128 rows per panel):
//   K-major operand  [rows = M or N][contiguous = K]: 8-row groups 1024 B apart (SBO); one MMA (K=16)
//     reads 32 B of each row; successive K steps advance the start address by 32 B inside a panel and
//     by 16 KB to the next panel.
//   MN-major operand [rows = K][contiguous = M or N]: 64 elements of MN per panel, panels 16 KB apart
//     (LBO); 8-row groups of K 1024 B apart (SBO); successive K steps (16 rows) advance by 2048 B.
constexpr uint32_t kPanelBytes = 16384;
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile_addr, int kstep /*16 elements each*/) {
  return make_smem_desc(tile_addr + (uint32_t)(kstep >> 2) * kPanelBytes + (uint32_t)(kstep & 3) * 32u, 16, 1024);
}
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t tile_addr, int kstep /*16 rows each*/) {
  return make_smem_desc(tile_addr + (uint32_t)kstep * 2048u, kPanelBytes, 1024);
}

// The MMA-issuing thread is a single thread: every integer instruction it spends building a descriptor
// delays the next tcgen05.mma by several cycles, and a 128x128x16 MMA is only 64 cycles of tensor work.
// So descriptors are split into a per-buffer base (built once) and a per-K-step byte offset that is a
// compile-time constant: one 32-bit add per descriptor.
struct DescBase {
  uint32_t lo, hi;
};
__device__ __forceinline__ DescBase desc_base(uint32_t tile_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  DescBase b;
  b.lo = ((tile_addr >> 4) & 0x3fffu) | (((lbo_bytes >> 4) & 0x3fffu) << 16);
  b.hi = ((sbo_bytes >> 4) & 0x3fffu) | (1u << 14) | ((uint32_t)kSwizzle128B << 29);
  return b;
}
__device__ __forceinline__ DescBase base_kmajor(uint32_t tile_addr) { return desc_base(tile_addr, 16, 1024); }
__device__ __forceinline__ DescBase base_mnmajor(uint32_t tile_addr) { return desc_base(tile_addr, kPanelBytes, 1024); }
__device__ __forceinline__ uint64_t desc_at(const DescBase& b, uint32_t byte_off) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(b.lo + (byte_off >> 4)), "r"(b.hi));
  return d;
}
__host__ __device__ constexpr uint32_t koff_kmajor(int kstep) {
  return (uint32_t)(kstep >> 2) * kPanelBytes + (uint32_t)(kstep & 3) * 32u;
}
__host__ __device__ constexpr uint32_t koff_mnmajor(int kstep) { return (uint32_t)kstep * 2048u; }

// Instruction descriptor for kind::f16 with bf16 operands and f32 accumulation:
// [4,6) D format (1 = f32), [7,10) A format (1 = bf16), [10,13) B format (1 = bf16),
// bit 15 A major (0 = K), bit 16 B major (0 = K, 1 = MN), [17,23) N >> 3, [24,29) M >> 4.
// Both operands must have the SAME format: an f16 A operand (format 0) with a bf16 B operand raises an illegal
// instruction on B200, so operands the kernels generate (probabilities, dS) are bf16 like the input tiles.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, bool b_mn_major, bool a_mn_major = false) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// Warp-uniform issue helpers.  The MMA / TMA warps run their control loops with all 32 lanes converged and
// predicate only the asynchronous instruction itself on `issue` (true in one lane): descriptor and address
// arithmetic then stays warp-uniform, which lets the compiler keep it on the uniform datapath instead of
// converting vector registers for every tcgen05.mma (a single diverged lane issues an MMA only every
// 55-75 cycles, less than the 64 cycles of tensor work a 128x128x16 MMA carries).
__device__ __forceinline__ void mma_ss_if(uint32_t issue, uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(issue)
      : "memory");
}
__device__ __forceinline__ void mma_ts_if(uint32_t issue, uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(issue)
      : "memory");
}
__device__ __forceinline__ void mma_commit_if(uint32_t issue, uint64_t* bar) {
  asm volatile(
      "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %1, 0;\n\t"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}\n" ::"r"(smem_u32(bar)),
      "r"(issue)
      : "memory");
}
// all 32 lanes wait; the result is made warp-uniform
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity));
}

// D[tmem] (+)= A[smem] * B[smem]      (issued by ONE thread)
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]      (issued by ONE thread)
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// mbarrier arrives once every MMA issued so far by this thread has completed (implies fence::before).
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// Packed f32x2 arithmetic (sm_100): two IEEE f32 operations per issued instruction.  The element-wise loops
// of the attention kernels are bound by instruction issue (and share their schedulers with the MMA-issuing
// thread), so halving the FMA-pipe instruction count matters more than its raw throughput.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t sub2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
// cvt.rn.bf16x2.f32 runs on the special-function pipe at a quarter of the FP32 rate (measured: 8 cycles per
// warp instruction, the same pipe and cost as ex2), so on the hot path it would double the load of the unit
// that already bounds the softmax.  The hot path therefore packs by TRUNCATION (one byte-permute on the
// integer pipe) of values that were pre-multiplied by (1 + 2^-9): adding between a quarter and half a bf16
// ulp before dropping the low mantissa bits is rounding to nearest up to a bias of about -2^-11.  The
// pre-multiplication is free: probabilities get it by adding kRoundLog2 = log2(1 + 2^-9) to the exp2
// argument, products of such a probability inherit it.  The PACKED value then approximates the original
// number (the factor only compensates the truncation); an f32 sum of the pre-scaled values, such as the
// softmax denominator, still carries the factor kRoundUp and must be divided by it.
constexpr float kRoundLog2 = 0.0028150156f;
constexpr float kRoundUp = 1.001953125f;
constexpr float kRoundInv = 1.0f / kRoundUp;
__device__ __forceinline__ uint32_t pack_bf16_trunc(float lo, float hi) {
  return __byte_perm(__float_as_uint(lo), __float_as_uint(hi), 0x7632);
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Eight consecutive values of a dense bias row (zeros past the first `n`): two 16-byte loads when the row start
// allows it, scalar loads otherwise.  The dense additive bias (the reference's `ab`, flex_attention_kernel.py:262-266)
// is read straight from global memory: with a bias the kernels are bound by those S^2 floats, not by the math.
__device__ __forceinline__ void load_bias8(float (&b)[8], const float* __restrict__ p, int n) {
  if (n >= 8 && (reinterpret_cast<uintptr_t>(p) & 15u) == 0) {
    const float4 lo = __ldg(reinterpret_cast<const float4*>(p)), hi = __ldg(reinterpret_cast<const float4*>(p) + 1);
    b[0] = lo.x; b[1] = lo.y; b[2] = lo.z; b[3] = lo.w;
    b[4] = hi.x; b[5] = hi.y; b[6] = hi.z; b[7] = hi.w;
  } else {
#pragma unroll
    for (int c = 0; c < 8; ++c) b[c] = c < n ? __ldg(p + c) : 0.f;
  }
}
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

}  // namespace ptx

// Per-device abort word (device address): set when any bounded wait gives up, checked by every tensor-core CTA
// on entry so that one failure does not cost a time-out per CTA.  It stays set until flexattn_reset_abort clears
// it; a CTA that leaves on entry because of it reports {TIMEOUT, kernel id, block, kAbortedOnEntry} in the
// caller's status words, so a launch that did no work never looks like a success.  nullptr if the address
// cannot be resolved.
#ifndef FLEXATTN_JIT
int* abort_flag_ptr();
#endif
constexpr int kAbortedOnEntry = 99;

__device__ __forceinline__ void give_up(int* abort_flag, int32_t* status, int kernel_id, int detail) {
  if (abort_flag != nullptr) atomicExch(abort_flag, 1);
  report_timeout(status, kernel_id, detail);
}
// true = the abort word is set: the CTA must return at once (before it allocates tensor memory)
__device__ __forceinline__ bool aborted_on_entry(const int* abort_flag, int32_t* status, int kernel_id) {
  if (*reinterpret_cast<const volatile int*>(abort_flag) == 0) return false;
  if (threadIdx.x == 0) report_timeout(status, kernel_id, kAbortedOnEntry);
  return true;
}

#ifndef FLEXATTN_JIT
// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) applies to the CURRENT device only, so "already done" is kept
// per device (one flag array per kernel instantiation, owned by its launcher).  Returns FLEXATTN_OK or
// FLEXATTN_ERR_CUDA.
constexpr int kMaxDevices = 64;
struct SmemAttrOnce {
  unsigned char done[kMaxDevices];
};
int ensure_dynamic_smem(const void* kernel, int bytes, SmemAttrOnce* once);

// Host side: 3-D tensor map over a [slices, rows, cols] bf16 array, box = {64 cols, 128 rows, 1 slice},
// 128-byte swizzle, out-of-range rows read as zero.
int make_tile_map(CUtensorMap* out, const void* base, int slices, int rows, int cols);
#endif  // !FLEXATTN_JIT

// Kernels live in an unnamed namespace in ahead-of-time builds and in a named one when compiled at run time
// (so that the run-time compiler can be asked for one instantiation by name).
#ifdef FLEXATTN_JIT
#define FLEXATTN_TU_NAMESPACE jit_tu
#else
#define FLEXATTN_TU_NAMESPACE
#endif

}  // namespace flexattn
