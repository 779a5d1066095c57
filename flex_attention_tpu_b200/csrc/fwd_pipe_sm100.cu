// Forward flex attention, software-pipelined variant for long rows (sm_100a).
//
// Same math and interface as fwd_sm100.cu (reference: flex_attention_kernel.py:196-327) but one CTA per SM
// keeps THREE score tiles in flight in tensor memory so that the tensor core and the softmax never wait
// for each other:
//
//   warp 8, lane 0 : MMA issuer.  S[t % 3] = Q K[t]^T runs up to three kv tiles ahead of the softmax;
//                    O += P[n] V[n] is issued as soon as the softmax has written P[n] over S[n % 3].
//   warp 9, lane 0 : TMA producer.  Q once; K and V through two-stage rings, each refilled as soon as the
//                    MMA that read the stage has completed (tcgen05.commit -> mbarrier).
//   warps 0..7     : softmax, two warpgroups.  Threads t and t + 128 share query row t (= TMEM lane t)
//                    and take one 64-column half of every score tile each; partial row maxima are
//                    exchanged through shared memory; P goes back to tensor memory as packed bf16; O is
//                    rescaled in tensor memory only when the running max moved by more than 2^8.
//
// Tensor memory: S0, S1, S2 (3 x 128 columns) + O (D columns) = 512 for D = 128.  Shared memory: Q + 2 K +
// 2 V tiles (160 KB for D = 128).
#include "sm100.cuh"

#ifdef FLEXATTN_TRACE
#define FA_TRACE(slot)                                                          \
  do {                                                                          \
    if (P.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && n < 64)     \
      P.trace[n * 16 + (slot)] = clock64();                                     \
  } while (0)
#define FA_MARK(slot)                                                           \
  do {                                                                          \
    if (P.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0)               \
      P.trace[63 * 16 + (slot)] = clock64();                                    \
  } while (0)
#else
#define FA_TRACE(slot)
#define FA_MARK(slot)
#endif

namespace flexattn {
namespace {

constexpr int kThreads = 320;
constexpr int kMmaWarp = 8, kTmaWarp = 9;
constexpr int kHalf = kTile / 2;
constexpr int kSBufs = 3;
constexpr float kLazyRescale = 8.0f;  // log2 units
constexpr bool kInOrderMma = true;     // rely on issue-order execution of one thread's tcgen05.mma stream

struct PipeSmem {
  uint64_t bar_q, bar_k[2], bar_v[2], bar_kfree[2], bar_s[kSBufs], bar_p[kSBufs], bar_pv[2];
  uint32_t tmem_base;
  float pmax[2][2][kTile];  // [tile parity][column half][row]
  float lsum[2][kTile];     // [column half][row]
  int32_t doc[2][kTile];
};

// x: this thread's 64 raw scores (columns c_base .. c_base+63 of the tile) -> log2-domain logits in place;
// returns their maximum.
template <int SK, int MK, bool kPartial>
__device__ __forceinline__ float score_half(float (&x)[kHalf], int i, int j0, int c_base, int seq_k, int window,
                                            int stride, float c2, float slope2, float capl2, float csc, int di,
                                            const int32_t* s_doc) {
  float mx[4] = {kMasked, kMasked, kMasked, kMasked};
  const float abase = slope2 * (float)(j0 + c_base - i);
#pragma unroll
  for (int c = 0; c < kHalf; ++c) {
    float t;
    if constexpr (SK == FLEXATTN_SCORE_ALIBI) {
      t = fmaf(x[c], c2, fmaf(slope2, (float)c, abase));
    } else if constexpr (SK == FLEXATTN_SCORE_SOFTCAP) {
      t = capl2 * ptx::tanh_approx(x[c] * csc);
    } else {
      t = x[c] * c2;
    }
    if constexpr (kPartial) {
      const int j = j0 + c_base + c;
      const int dj = (MK == FLEXATTN_MASK_DOCUMENT) ? s_doc[c_base + c] : 0;
      const bool keep = (j < seq_k) && mask_keep<MK>(i, j, window, stride, di, dj);
      t = keep ? t : kMasked;
    }
    x[c] = t;
    mx[c & 3] = fmaxf(mx[c & 3], t);
  }
  return fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
}

template <int D, int SK, int MK>
__global__ void __launch_bounds__(kThreads, 1)
    fwd_pipe_sm100_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                          const __grid_constant__ CUtensorMap tm_v, const DevParams P, int* abort_flag) {
  constexpr int kPanels = D / 64;
  constexpr uint32_t kTileBytes = kPanels * ptx::kPanelBytes;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kColO = kSBufs * 128;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sK = smem + kTileBytes;      // two stages
  uint8_t* sV = smem + 3 * kTileBytes;  // two stages
  PipeSmem* sh = reinterpret_cast<PipeSmem*>(smem + 5 * kTileBytes);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) FA_MARK(0);
  const int qt = P.n_qt - 1 - (int)blockIdx.x;  // heavy (late) causal tiles first
  const int bh = blockIdx.y, b = bh / P.heads, h = bh % P.heads;
  const int4 rm = P.row_map[(size_t)(P.map_rows > 1 ? b : 0) * P.n_qt + qt];
  const int N = rm.y - rm.x;

  if (*reinterpret_cast<volatile int*>(abort_flag) != 0) return;
  if (tid == 0) FA_MARK(1);

  if (tid == 0) {
    ptx::mbar_init(&sh->bar_q, 1);
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(&sh->bar_k[s], 1);
      ptx::mbar_init(&sh->bar_v[s], 1);
      ptx::mbar_init(&sh->bar_kfree[s], 1);
      ptx::mbar_init(&sh->bar_pv[s], 1);
    }
    for (int s = 0; s < kSBufs; ++s) {
      ptx::mbar_init(&sh->bar_s[s], 1);
      ptx::mbar_init(&sh->bar_p[s], 256);
    }
    ptx::fence_barrier_init();
  }
  if (warp == kMmaWarp) {
    ptx::tmem_alloc(&sh->tmem_base, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = sh->tmem_base;
  if (tid == 0) FA_MARK(2);

  if (warp == kTmaWarp) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && N > 0) {
      bool ok = true;
      int fail_at = 0;
      ptx::prefetch_tensormap(&tm_q);
      ptx::prefetch_tensormap(&tm_k);
      ptx::prefetch_tensormap(&tm_v);
      auto load_k = [&](int t) {
        uint8_t* dst = sK + (t & 1) * kTileBytes;
        ptx::mbar_arrive_expect_tx(&sh->bar_k[t & 1], kTileBytes);
#pragma unroll
        for (int p = 0; p < kPanels; ++p)
          ptx::tma_load_3d(dst + p * ptx::kPanelBytes, &tm_k, &sh->bar_k[t & 1], p * 64, (rm.x + t) * kTile, bh);
      };
      auto load_v = [&](int t) {
        uint8_t* dst = sV + (t & 1) * kTileBytes;
        ptx::mbar_arrive_expect_tx(&sh->bar_v[t & 1], kTileBytes);
#pragma unroll
        for (int p = 0; p < kPanels; ++p)
          ptx::tma_load_3d(dst + p * ptx::kPanelBytes, &tm_v, &sh->bar_v[t & 1], p * 64, (rm.x + t) * kTile, bh);
      };
      ptx::mbar_arrive_expect_tx(&sh->bar_q, kTileBytes);
#pragma unroll
      for (int p = 0; p < kPanels; ++p)
        ptx::tma_load_3d(sQ + p * ptx::kPanelBytes, &tm_q, &sh->bar_q, p * 64, qt * kTile, bh);
      load_k(0);
      if (N > 1) load_k(1);
      load_v(0);
      if (N > 1) load_v(1);
      FA_MARK(3);
      // K[t] for t = 2..4 replaces K[t-2], read by the Q K^T MMAs the issuer runs ahead of the softmax
      for (int t = 2; t < 5 && t < N && ok; ++t) {
        ok = ptx::mbar_wait(&sh->bar_kfree[t & 1], ((t - 2) >> 1) & 1);
        if (!ok) { fail_at = 20; break; }
        load_k(t);
      }
      for (int n = 0; n < N && ok; ++n) {
        if (n + 2 < N) {  // V[n+2] replaces V[n], read by P V of tile n
          ok = ptx::mbar_wait(&sh->bar_pv[n & 1], (n >> 1) & 1);
          if (!ok) { fail_at = 21; break; }
          load_v(n + 2);
        }
        if (n + 5 < N) {  // K[n+5] replaces K[n+3], read by Q K^T of tile n+3
          ok = ptx::mbar_wait(&sh->bar_kfree[(n + 3) & 1], ((n + 3) >> 1) & 1);
          if (!ok) { fail_at = 22; break; }
          load_k(n + 5);
        }
      }
      if (!ok) give_up(abort_flag, P.status, 4, fail_at);
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && N > 0) {
      bool ok = true;
      int fail_at = 1;
      constexpr uint32_t idesc_qk = ptx::make_idesc(128, 128, false);
      constexpr uint32_t idesc_pv = ptx::make_idesc(128, D, true);
      const ptx::DescBase bQ = ptx::base_kmajor(ptx::smem_u32(sQ));
      const ptx::DescBase bK0 = ptx::base_kmajor(ptx::smem_u32(sK)), bK1 = ptx::base_kmajor(ptx::smem_u32(sK + kTileBytes));
      const ptx::DescBase bV0 = ptx::base_mnmajor(ptx::smem_u32(sV)), bV1 = ptx::base_mnmajor(ptx::smem_u32(sV + kTileBytes));
      auto issue_qk = [&](int t) {
        const ptx::DescBase bk = (t & 1) ? bK1 : bK0;
        const uint32_t dS = tmem + (uint32_t)(t % kSBufs) * 128u;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          ptx::mma_ss(dS, ptx::desc_at(bQ, ptx::koff_kmajor(kk)), ptx::desc_at(bk, ptx::koff_kmajor(kk)), idesc_qk, kk > 0);
        ptx::mma_commit(&sh->bar_s[t % kSBufs]);
        ptx::mma_commit(&sh->bar_kfree[t & 1]);
      };
      ok = ptx::mbar_wait(&sh->bar_q, 0);
      FA_MARK(4);
      for (int t = 0; t < kSBufs && t < N && ok; ++t) {
        ok = ptx::mbar_wait(&sh->bar_k[t & 1], (t >> 1) & 1);
        if (!ok) { fail_at = 2; break; }
        ptx::tc_fence_after();
        if (t == 0) FA_MARK(5);
        issue_qk(t);
      }
      for (int n = 0; n < N && ok; ++n) {
        const int sb = n % kSBufs;
        ok = ptx::mbar_wait(&sh->bar_p[sb], (n / kSBufs) & 1);
        if (!ok) { fail_at = 3; break; }
        FA_TRACE(0);
        ok = ptx::mbar_wait(&sh->bar_v[n & 1], (n >> 1) & 1);
        if (!ok) { fail_at = 4; break; }
        FA_TRACE(1);
        ptx::tc_fence_after();
        const ptx::DescBase bv = (n & 1) ? bV1 : bV0;
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk)
          ptx::mma_ts(tmem + kColO, tmem + (uint32_t)sb * 128u + kk * 8, ptx::desc_at(bv, ptx::koff_mnmajor(kk)), idesc_pv,
                      (n > 0) || (kk > 0));
        ptx::mma_commit(&sh->bar_pv[n & 1]);
        FA_TRACE(2);
        if (n + kSBufs < N) {
          // Q K^T of tile n+3 overwrites the columns P V of tile n reads its A operand from.  MMAs issued by one
          // thread execute in issue order, so no wait for P V to complete is needed between the two.
          if (!kInOrderMma) {
            ok = ptx::mbar_wait(&sh->bar_pv[n & 1], (n >> 1) & 1);
            if (!ok) { fail_at = 5; break; }
          }
          FA_TRACE(3);
          ok = ptx::mbar_wait(&sh->bar_k[(n + kSBufs) & 1], ((n + kSBufs) >> 1) & 1);
          if (!ok) { fail_at = 6; break; }
          FA_TRACE(4);
          ptx::tc_fence_after();
          issue_qk(n + kSBufs);
          FA_TRACE(5);
        }
      }
      if (!ok) give_up(abort_flag, P.status, 4, fail_at);
    }
  } else {
    // ------------------------------------------------------------------ softmax warpgroups
    const int row = tid & 127;
    const int half = tid >> 7;
    const int c_base = half * kHalf;
    const int i = qt * kTile + row;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const float c2 = P.sm_scale * kLog2e;
    const float slope2 = (SK == FLEXATTN_SCORE_ALIBI) ? P.alibi_slopes[h] * kLog2e : 0.f;
    const float capl2 = P.cap * kLog2e;
    const float csc = (SK == FLEXATTN_SCORE_SOFTCAP) ? P.sm_scale / P.cap : 0.f;
    const int32_t* doc = (MK == FLEXATTN_MASK_DOCUMENT) ? P.doc_ids + (size_t)b * P.doc_stride : nullptr;
    const int di = (MK == FLEXATTN_MASK_DOCUMENT && i < P.seq_q) ? doc[i] : 0;
    float m_ref = kMasked, m_true = kMasked, l = 0.f;  // l: sum over this thread's columns only
    bool ok = true;
    int fail_at = 0;

    for (int n = 0; n < N; ++n) {
      const uint32_t par = n & 1;
      const int sb = n % kSBufs;
      const uint32_t colS = (uint32_t)sb * 128u;
      const int kt = rm.x + n, j0 = kt * kTile;
      const bool partial = !(kt >= rm.z && kt < rm.w);
      if (MK == FLEXATTN_MASK_DOCUMENT && partial && half == 0) {
        const int j = j0 + row;
        sh->doc[par][row] = (j < P.seq_k) ? doc[j] : -1;
      }
      // A failed wait never leaves the loop early: every thread keeps executing the same named barriers so
      // that nobody is left waiting on one (the time-out path must not be able to hang either).
      if (ok) {
        ok = __all_sync(0xffffffffu, ptx::mbar_wait(&sh->bar_s[sb], (n / kSBufs) & 1));
        if (!ok) fail_at = 10;
      }
      if (tid == 0) FA_TRACE(8);
      if (tid == 0 && n == 0) FA_MARK(6);
      float x[kHalf];
      if (ok) {
        ptx::tc_fence_after();
        uint32_t xr[2][32];
#pragma unroll
        for (int q2 = 0; q2 < 2; ++q2) ptx::tmem_ld32(lane_base + colS + c_base + q2 * 32, xr[q2]);
        ptx::tmem_wait_ld();
#pragma unroll
        for (int q2 = 0; q2 < 2; ++q2) {
          ptx::tmem_ld_acquire(xr[q2]);
#pragma unroll
          for (int c = 0; c < 32; ++c) x[q2 * 32 + c] = __uint_as_float(xr[q2][c]);
        }
      }
      if (tid == 0) FA_TRACE(9);
      if (MK == FLEXATTN_MASK_DOCUMENT && partial) ptx::named_bar_sync(2, 256);  // kv-tile document ids visible
      // xs: factor still to be applied to x inside the exp2 argument (the plain-score fast path keeps the raw
      // scores and folds sm_scale*log2e into the FMA that also subtracts the running max)
      float tmax = kMasked, xs = 1.0f;
      if (ok) {
        if (partial) {
          tmax = score_half<SK, MK, true>(x, i, j0, c_base, P.seq_k, P.window, P.stride, c2, slope2, capl2, csc, di,
                                          sh->doc[par]);
        } else if constexpr (SK != FLEXATTN_SCORE_NONE) {
          tmax = score_half<SK, MK, false>(x, i, j0, c_base, P.seq_k, P.window, P.stride, c2, slope2, capl2, csc, di,
                                           sh->doc[par]);
        } else {
          float mx[4] = {x[0], x[1], x[2], x[3]};
#pragma unroll
          for (int c = 4; c + 7 < kHalf; c += 8) {
            mx[0] = ptx::max3(mx[0], x[c], x[c + 1]);
            mx[1] = ptx::max3(mx[1], x[c + 2], x[c + 3]);
            mx[2] = ptx::max3(mx[2], x[c + 4], x[c + 5]);
            mx[3] = ptx::max3(mx[3], x[c + 6], x[c + 7]);
          }
          mx[0] = ptx::max3(mx[0], x[kHalf - 4], x[kHalf - 3]);
          mx[1] = ptx::max3(mx[1], x[kHalf - 2], x[kHalf - 1]);
          tmax = ptx::max3(mx[0], mx[1], fmaxf(mx[2], mx[3])) * c2;  // c2 > 0: scaling commutes with max
          xs = c2;
        }
      }
      sh->pmax[par][half][row] = tmax;
      ptx::named_bar_sync(1, 256);  // exchange the partial row maxima of the two halves
      if (tid == 0) FA_TRACE(10);
      if (ok) {
        tmax = fmaxf(tmax, sh->pmax[par][half ^ 1][row]);
        m_true = fmaxf(m_true, tmax);
        const float m_cand = fmaxf(m_ref, tmax);
        if (__any_sync(0xffffffffu, (m_cand - m_ref) > kLazyRescale)) {
          const float alpha = ptx::ex2(m_ref - m_cand);
          l *= alpha;
          m_ref = m_cand;
          if (n > 0) {
            ok = __all_sync(0xffffffffu, ptx::mbar_wait(&sh->bar_pv[(n - 1) & 1], ((n - 1) >> 1) & 1));
            if (!ok) fail_at = 11;
            if (ok) {
              ptx::tc_fence_after();
#pragma unroll 1
              for (int c0 = half * (D / 2); c0 < (half + 1) * (D / 2); c0 += 32) {
                uint32_t r[32];
                ptx::tmem_ld32(lane_base + kColO + c0, r);
                ptx::tmem_wait_ld();
                ptx::tmem_ld_acquire(r);
#pragma unroll
                for (int c = 0; c < 32; ++c) r[c] = __float_as_uint(__uint_as_float(r[c]) * alpha);
                ptx::tmem_st32(lane_base + kColO + c0, r);
              }
              ptx::tmem_wait_st();
            }
          }
        }
      }
      if (tid == 0) FA_TRACE(11);
      if (ok) {
        float ls[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t pk[32];
        const float nm = ptx::kRoundLog2 - m_ref;  // pre-scaled by (1 + 2^-9) for pack_bf16_trunc; compensates the truncation
#pragma unroll
        for (int c = 0; c < kHalf; c += 2) {
          const float p0 = ptx::ex2(fmaf(x[c], xs, nm)), p1 = ptx::ex2(fmaf(x[c + 1], xs, nm));
          ls[(c >> 1) & 3] += p0 + p1;
          pk[c >> 1] = ptx::pack_bf16_trunc(p0, p1);
        }
        ptx::tmem_st32(lane_base + colS + (c_base >> 1), pk);
        l += (ls[0] + ls[1]) + (ls[2] + ls[3]);
        if (tid == 0) FA_TRACE(12);
        ptx::tmem_wait_st();
        ptx::tc_fence_before();
        ptx::mbar_arrive(&sh->bar_p[sb]);
        if (tid == 0) FA_TRACE(13);
      }
    }

    if (tid == 0) FA_MARK(7);
    if (ok && N > 0) {
      ok = __all_sync(0xffffffffu, ptx::mbar_wait(&sh->bar_pv[(N - 1) & 1], ((N - 1) >> 1) & 1));
      if (!ok) fail_at = 12;
    }
    if (tid == 0) FA_MARK(8);
    sh->lsum[half][row] = l;
    ptx::named_bar_sync(1, 256);
    l = sh->lsum[0][row] + sh->lsum[1][row];
    if (ok) {
      const float inv_l = l > 0.f ? ptx::kRoundUp / l : 0.f;  // l sums the pre-scaled probabilities
      const size_t grow = (size_t)bh * P.seq_q + i;
      if (N > 0) ptx::tc_fence_after();
      __nv_bfloat16* orow = static_cast<__nv_bfloat16*>(P.o) + grow * D;
#pragma unroll 1
      for (int c0 = half * (D / 2); c0 < (half + 1) * (D / 2); c0 += 32) {
        uint32_t r[32];
        if (N > 0) {
          ptx::tmem_ld32(lane_base + kColO + c0, r);
          ptx::tmem_wait_ld();
          ptx::tmem_ld_acquire(r);
        } else {
#pragma unroll
          for (int c = 0; c < 32; ++c) r[c] = 0u;
        }
        if (i < P.seq_q) {
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            uint4 v4;
            v4.x = ptx::pack_bf16(__uint_as_float(r[c]) * inv_l, __uint_as_float(r[c + 1]) * inv_l);
            v4.y = ptx::pack_bf16(__uint_as_float(r[c + 2]) * inv_l, __uint_as_float(r[c + 3]) * inv_l);
            v4.z = ptx::pack_bf16(__uint_as_float(r[c + 4]) * inv_l, __uint_as_float(r[c + 5]) * inv_l);
            v4.w = ptx::pack_bf16(__uint_as_float(r[c + 6]) * inv_l, __uint_as_float(r[c + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + c0 + c) = v4;
          }
        }
      }
      if (half == 0 && i < P.seq_q) {
        P.l[grow] = l * ptx::ex2(m_ref - m_true) * ptx::kRoundInv;
        P.m[grow] = m_true * kLn2;
      }
    } else if (lane == 0) {
      give_up(abort_flag, P.status, 4, fail_at);
    }
    if (tid == 0) FA_MARK(9);
  }

  // ------------------------------------------------------------------ teardown
  ptx::tc_fence_before();
  __syncthreads();
  if (tid == 0) FA_MARK(10);
  if (warp == kMmaWarp) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, kTmemCols);
  }
}

template <int D, int SK, int MK>
int launch_one(cudaStream_t st, const DevParams& d, const CUtensorMap& tq, const CUtensorMap& tk,
               const CUtensorMap& tv, int* abort_flag) {
  constexpr size_t need = 5 * (D / 64) * ptx::kPanelBytes + sizeof(PipeSmem) + 1024;
  // 512 TMEM columns per CTA: never let two CTAs share an SM (the second would spin in tcgen05.alloc)
  constexpr size_t smem = need > 120 * 1024 ? need : 120 * 1024;
  auto kern = fwd_pipe_sm100_kernel<D, SK, MK>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return FLEXATTN_ERR_CUDA;
    attr_set = true;
  }
  dim3 grid(d.n_qt, d.batch * d.heads);
  kern<<<grid, kThreads, smem, st>>>(tq, tk, tv, d, abort_flag);
  return cudaGetLastError() == cudaSuccess ? FLEXATTN_OK : FLEXATTN_ERR_CUDA;
}

template <int D, int SK>
int launch_mask(cudaStream_t st, const DevParams& d, int mask, const CUtensorMap& tq, const CUtensorMap& tk,
                const CUtensorMap& tv, int* af) {
  switch (mask) {
    case FLEXATTN_MASK_NONE: return launch_one<D, SK, FLEXATTN_MASK_NONE>(st, d, tq, tk, tv, af);
    case FLEXATTN_MASK_CAUSAL: return launch_one<D, SK, FLEXATTN_MASK_CAUSAL>(st, d, tq, tk, tv, af);
    case FLEXATTN_MASK_SLIDING_WINDOW: return launch_one<D, SK, FLEXATTN_MASK_SLIDING_WINDOW>(st, d, tq, tk, tv, af);
    case FLEXATTN_MASK_SLIDING_WINDOW_CAUSAL:
      return launch_one<D, SK, FLEXATTN_MASK_SLIDING_WINDOW_CAUSAL>(st, d, tq, tk, tv, af);
    case FLEXATTN_MASK_DOCUMENT: return launch_one<D, SK, FLEXATTN_MASK_DOCUMENT>(st, d, tq, tk, tv, af);
    case FLEXATTN_MASK_S2: return launch_one<D, SK, FLEXATTN_MASK_S2>(st, d, tq, tk, tv, af);
    default: return FLEXATTN_ERR_UNSUPPORTED_MOD;
  }
}

template <int D>
int launch_score(cudaStream_t st, const DevParams& d, int score, int mask, const CUtensorMap& tq,
                 const CUtensorMap& tk, const CUtensorMap& tv, int* af) {
  switch (score) {
    case FLEXATTN_SCORE_NONE: return launch_mask<D, FLEXATTN_SCORE_NONE>(st, d, mask, tq, tk, tv, af);
    case FLEXATTN_SCORE_ALIBI: return launch_mask<D, FLEXATTN_SCORE_ALIBI>(st, d, mask, tq, tk, tv, af);
    case FLEXATTN_SCORE_SOFTCAP: return launch_mask<D, FLEXATTN_SCORE_SOFTCAP>(st, d, mask, tq, tk, tv, af);
    default: return FLEXATTN_ERR_UNSUPPORTED_MOD;
  }
}

}  // namespace

int launch_sm100_fwd_pipe(cudaStream_t st, const DevParams& d, int score, int mask) {
  int* af = abort_flag_ptr();
  if (af == nullptr) return FLEXATTN_ERR_CUDA;
  CUtensorMap tq, tk, tv;
  const int slices = d.batch * d.heads;
  int e = make_tile_map(&tq, d.q, slices, d.seq_q, d.head_dim);
  if (e) return e;
  e = make_tile_map(&tk, d.k, slices, d.seq_k, d.head_dim);
  if (e) return e;
  e = make_tile_map(&tv, d.v, slices, d.seq_k, d.head_dim);
  if (e) return e;
  if (d.head_dim == 128) return launch_score<128>(st, d, score, mask, tq, tk, tv, af);
  if (d.head_dim == 64) return launch_score<64>(st, d, score, mask, tq, tk, tv, af);
  return FLEXATTN_ERR_UNSUPPORTED_HEAD_DIM;
}

}  // namespace flexattn
