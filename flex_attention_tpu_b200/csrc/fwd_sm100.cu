// Forward flex attention on the 5th-generation tensor cores (sm_100a).
//
// Replaces the reference's Pallas forward kernel (flex_attention_kernel.py:196-327).  One CTA owns one
// 128-row query tile of one (batch, head) and walks the kv tiles the mask map lists for it:
//
//   warp 4, lane 0  : TMA producer and MMA issuer.  Q once, then per kv tile K and V (each its own
//                     shared-memory buffer and mbarrier); S = Q K^T and O += P V as tcgen05.mma with
//                     f32 accumulators in tensor memory.
//   warps 0..3      : softmax.  Thread t owns query row t (= TMEM lane t): reads its 128 scores with
//                     tcgen05.ld, applies score_mod and, on partial tiles only, the mask functor, keeps
//                     the running max / sum in the log2 domain, writes P as packed bf16 back into the
//                     columns of S (tcgen05.st) so that P V takes its A operand from tensor memory, and
//                     rescales O in tensor memory only when the running max moved by more than 2^8.
//
// Shared memory: Q, K, V tiles (TMA 128-byte swizzle) = 3 * D * 256 B; tensor memory: S/P 128 columns +
// O D columns (256 allocated).  Two CTAs fit on an SM, so one CTA's softmax overlaps the other's MMAs.
#include "sm100.cuh"

#ifdef FLEXATTN_TRACE
#define FA_TRACE(slot)                                                          \
  do {                                                                          \
    if (P.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && n < 64)     \
      P.trace[n * 16 + (slot)] = clock64();                                     \
  } while (0)
#else
#define FA_TRACE(slot)
#endif

namespace flexattn {
namespace {

constexpr int kFwdThreads = 160;
constexpr float kLazyRescale = 8.0f;  // log2 units: rescale O only when the max grew by more than this

struct FwdSmem {
  uint64_t bar_q, bar_k, bar_v, bar_s, bar_p, bar_pv;
  uint32_t tmem_base;
  int32_t doc[2][kTile];
};

template <int SK, int MK, bool kPartial>
__device__ __forceinline__ float score_tile(float (&x)[kTile], int i, int j0, int seq_k, int window, int stride,
                                            float c2, float slope2, float capl2, float csc, int di,
                                            const int32_t* s_doc) {
  float mx[4] = {kMasked, kMasked, kMasked, kMasked};
  const float abase = slope2 * (float)(j0 - i);
#pragma unroll
  for (int c = 0; c < kTile; ++c) {
    float t;
    if constexpr (SK == FLEXATTN_SCORE_ALIBI) {
      t = fmaf(x[c], c2, fmaf(slope2, (float)c, abase));
    } else if constexpr (SK == FLEXATTN_SCORE_SOFTCAP) {
      t = capl2 * ptx::tanh_approx(x[c] * csc);
    } else {
      t = x[c] * c2;
    }
    if constexpr (kPartial) {
      const int j = j0 + c;
      const int dj = (MK == FLEXATTN_MASK_DOCUMENT) ? s_doc[c] : 0;
      const bool keep = (j < seq_k) && mask_keep<MK>(i, j, window, stride, di, dj);
      t = keep ? t : kMasked;
    }
    x[c] = t;
    mx[c & 3] = fmaxf(mx[c & 3], t);
  }
  return fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
}

template <int D, int SK, int MK>
__global__ void __launch_bounds__(kFwdThreads, 2)
    fwd_sm100_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const DevParams P, int* abort_flag) {
  constexpr int kPanels = D / 64;
  constexpr uint32_t kTileBytes = kPanels * ptx::kPanelBytes;
  constexpr uint32_t kTmemCols = 256;
  constexpr uint32_t kColS = 0, kColO = 128;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sK = smem + kTileBytes;
  uint8_t* sV = smem + 2 * kTileBytes;
  FwdSmem* sh = reinterpret_cast<FwdSmem*>(smem + 3 * kTileBytes);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qt = P.n_qt - 1 - (int)blockIdx.x;  // heavy (late) causal tiles first
  const int bh = blockIdx.y, b = bh / P.heads, h = bh % P.heads;
  const int4 rm = P.row_map[(size_t)(P.map_rows > 1 ? b : 0) * P.n_qt + qt];
  const int n_tiles = rm.y - rm.x;

  if (*reinterpret_cast<volatile int*>(abort_flag) != 0) return;  // an earlier wait gave up: do nothing

  if (tid == 0) {
    ptx::mbar_init(&sh->bar_q, 1);
    ptx::mbar_init(&sh->bar_k, 1);
    ptx::mbar_init(&sh->bar_v, 1);
    ptx::mbar_init(&sh->bar_s, 1);
    ptx::mbar_init(&sh->bar_p, 128);
    ptx::mbar_init(&sh->bar_pv, 1);
    ptx::fence_barrier_init();
  }
  if (warp == 4) {
    ptx::tmem_alloc(&sh->tmem_base, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = sh->tmem_base;

  if (warp == 4) {
    // ------------------------------------------------------------------ producer + MMA issuer
    if (lane == 0 && n_tiles > 0) {
      bool ok = true;
      ptx::prefetch_tensormap(&tm_q);
      ptx::prefetch_tensormap(&tm_k);
      ptx::prefetch_tensormap(&tm_v);
      ptx::mbar_arrive_expect_tx(&sh->bar_q, kTileBytes);
      ptx::mbar_arrive_expect_tx(&sh->bar_k, kTileBytes);
      ptx::mbar_arrive_expect_tx(&sh->bar_v, kTileBytes);
#pragma unroll
      for (int p = 0; p < kPanels; ++p) {
        ptx::tma_load_3d(sQ + p * ptx::kPanelBytes, &tm_q, &sh->bar_q, p * 64, qt * kTile, bh);
        ptx::tma_load_3d(sK + p * ptx::kPanelBytes, &tm_k, &sh->bar_k, p * 64, rm.x * kTile, bh);
      }
#pragma unroll
      for (int p = 0; p < kPanels; ++p)
        ptx::tma_load_3d(sV + p * ptx::kPanelBytes, &tm_v, &sh->bar_v, p * 64, rm.x * kTile, bh);
      constexpr uint32_t idesc_qk = ptx::make_idesc(128, 128, false);
      constexpr uint32_t idesc_pv = ptx::make_idesc(128, D, true);
      const ptx::DescBase bQ = ptx::base_kmajor(ptx::smem_u32(sQ)), bK = ptx::base_kmajor(ptx::smem_u32(sK)),
                          bV = ptx::base_mnmajor(ptx::smem_u32(sV));
      ok = ptx::mbar_wait(&sh->bar_q, 0);
      int fail_at = 1;
      for (int n = 0; n < n_tiles && ok; ++n) {
        const uint32_t par = n & 1;
        ok = ptx::mbar_wait(&sh->bar_k, par);
        if (!ok) { fail_at = 2; break; }
        FA_TRACE(0);
        if (n > 0) {
          // P V of the previous tile done: S/P columns and the V buffer are free again
          ok = ptx::mbar_wait(&sh->bar_pv, par ^ 1);
          if (!ok) { fail_at = 3; break; }
          ptx::mbar_arrive_expect_tx(&sh->bar_v, kTileBytes);
#pragma unroll
          for (int p = 0; p < kPanels; ++p)
            ptx::tma_load_3d(sV + p * ptx::kPanelBytes, &tm_v, &sh->bar_v, p * 64, (rm.x + n) * kTile, bh);
        }
        FA_TRACE(1);
        ptx::tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          ptx::mma_ss(tmem + kColS, ptx::desc_at(bQ, ptx::koff_kmajor(kk)), ptx::desc_at(bK, ptx::koff_kmajor(kk)), idesc_qk,
                      kk > 0);
        ptx::mma_commit(&sh->bar_s);
        FA_TRACE(2);
        ok = ptx::mbar_wait(&sh->bar_s, par);  // Q K^T done: the K buffer is free
        if (!ok) { fail_at = 4; break; }
        FA_TRACE(3);
        if (n + 1 < n_tiles) {
          ptx::mbar_arrive_expect_tx(&sh->bar_k, kTileBytes);
#pragma unroll
          for (int p = 0; p < kPanels; ++p)
            ptx::tma_load_3d(sK + p * ptx::kPanelBytes, &tm_k, &sh->bar_k, p * 64, (rm.x + n + 1) * kTile, bh);
        }
        ok = ptx::mbar_wait(&sh->bar_v, par);
        if (!ok) { fail_at = 5; break; }
        FA_TRACE(4);
        ok = ptx::mbar_wait(&sh->bar_p, par);
        if (!ok) { fail_at = 6; break; }
        FA_TRACE(5);
        ptx::tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk)
          ptx::mma_ts(tmem + kColO, tmem + kColS + kk * 8, ptx::desc_at(bV, ptx::koff_mnmajor(kk)), idesc_pv,
                      (n > 0) || (kk > 0));
        ptx::mma_commit(&sh->bar_pv);
        FA_TRACE(6);
      }
      if (!ok) give_up(abort_flag, P.status, 1, fail_at);
    }
  } else {
    // ------------------------------------------------------------------ softmax warps: thread = row
    const int row = tid;                       // TMEM lane
    const int i = qt * kTile + row;            // global query position
    const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
    const float c2 = P.sm_scale * kLog2e;
    const float slope2 = (SK == FLEXATTN_SCORE_ALIBI) ? P.alibi_slopes[h] * kLog2e : 0.f;
    const float capl2 = P.cap * kLog2e;
    const float csc = (SK == FLEXATTN_SCORE_SOFTCAP) ? P.sm_scale / P.cap : 0.f;
    const int32_t* doc = (MK == FLEXATTN_MASK_DOCUMENT) ? P.doc_ids + (size_t)b * P.doc_stride : nullptr;
    const int di = (MK == FLEXATTN_MASK_DOCUMENT && i < P.seq_q) ? doc[i] : 0;
    float m_ref = kMasked, m_true = kMasked, l = 0.f;
    bool ok = true;
    int fail_at = 0;

    for (int n = 0; n < n_tiles; ++n) {
      const uint32_t par = n & 1;
      const int kt = rm.x + n, j0 = kt * kTile;
      const bool partial = !(kt >= rm.z && kt < rm.w);
      if (MK == FLEXATTN_MASK_DOCUMENT && partial) {
        const int j = j0 + row;
        sh->doc[par][row] = (j < P.seq_k) ? doc[j] : -1;
        ptx::named_bar_sync(1, 128);
      }
      // a failed wait never leaves the loop early: every thread keeps executing the same named barriers
      if (ok) {
        ok = __all_sync(0xffffffffu, ptx::mbar_wait(&sh->bar_s, par));
        if (!ok) fail_at = 10;
      }
      if (!ok) continue;
      if (tid == 0) FA_TRACE(8);
      ptx::tc_fence_after();
      float x[kTile];
      {
        uint32_t xr[4][32];
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) ptx::tmem_ld32(lane_base + kColS + q4 * 32, xr[q4]);
        ptx::tmem_wait_ld();
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          ptx::tmem_ld_acquire(xr[q4]);
#pragma unroll
          for (int c = 0; c < 32; ++c) x[q4 * 32 + c] = __uint_as_float(xr[q4][c]);
        }
      }
      if (tid == 0) FA_TRACE(9);
      // xs: factor still to be applied to x inside the exp2 argument (the plain-score fast path keeps the raw
      // scores and folds sm_scale*log2e into the FMA that also subtracts the running max)
      float tmax, xs = 1.0f;
      if (partial) {
        tmax = score_tile<SK, MK, true>(x, i, j0, P.seq_k, P.window, P.stride, c2, slope2, capl2, csc, di, sh->doc[par]);
      } else if constexpr (SK != FLEXATTN_SCORE_NONE) {
        tmax = score_tile<SK, MK, false>(x, i, j0, P.seq_k, P.window, P.stride, c2, slope2, capl2, csc, di, sh->doc[par]);
      } else {
        float mx[4] = {x[0], x[1], x[2], x[3]};
#pragma unroll
        for (int c = 4; c < kTile; c += 8) {
          mx[0] = ptx::max3(mx[0], x[c], x[c + 1]);
          mx[1] = ptx::max3(mx[1], x[c + 2], x[c + 3]);
          if (c + 4 < kTile) {
            mx[2] = ptx::max3(mx[2], x[c + 4], x[c + 5]);
            mx[3] = ptx::max3(mx[3], x[c + 6], x[c + 7]);
          }
        }
        tmax = ptx::max3(mx[0], mx[1], fmaxf(mx[2], mx[3])) * c2;   // c2 > 0: scaling commutes with max
        xs = c2;
      }
      if (tid == 0) FA_TRACE(10);
      m_true = fmaxf(m_true, tmax);
      const float m_cand = fmaxf(m_ref, tmax);
      if (__any_sync(0xffffffffu, (m_cand - m_ref) > kLazyRescale)) {
        const float alpha = ptx::ex2(m_ref - m_cand);
        l *= alpha;
        m_ref = m_cand;
        if (n > 0) {
          ok = __all_sync(0xffffffffu, ptx::mbar_wait(&sh->bar_pv, par ^ 1));
          if (!ok) { fail_at = 11; continue; }
          ptx::tc_fence_after();
#pragma unroll 1
          for (int c0 = 0; c0 < D; c0 += 32) {
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
      if (tid == 0) FA_TRACE(11);
      float ls[4] = {0.f, 0.f, 0.f, 0.f};
      const float nm = ptx::kRoundLog2 - m_ref;
#pragma unroll
      for (int c0 = 0; c0 < kTile; c0 += 64) {
        uint32_t pk[32];
#pragma unroll
        for (int c = 0; c < 64; c += 2) {
          // pre-scaled by (1 + 2^-9) for pack_bf16_trunc; the factor compensates the truncation
          const float p0 = ptx::ex2(fmaf(x[c0 + c], xs, nm)), p1 = ptx::ex2(fmaf(x[c0 + c + 1], xs, nm));
          ls[(c >> 1) & 3] += p0 + p1;
          pk[c >> 1] = ptx::pack_bf16_trunc(p0, p1);
        }
        ptx::tmem_st32(lane_base + kColS + (c0 >> 1), pk);
      }
      l += (ls[0] + ls[1]) + (ls[2] + ls[3]);
      if (tid == 0) FA_TRACE(12);
      ptx::tmem_wait_st();
      ptx::tc_fence_before();
      ptx::mbar_arrive(&sh->bar_p);
      if (tid == 0) FA_TRACE(13);
    }

    if (ok && n_tiles > 0) {
      ok = __all_sync(0xffffffffu, ptx::mbar_wait(&sh->bar_pv, (n_tiles - 1) & 1));
      if (!ok) fail_at = 12;
    }
    if (ok) {
      const float inv_l = l > 0.f ? ptx::kRoundUp / l : 0.f;  // l sums the pre-scaled probabilities
      const size_t grow = (size_t)bh * P.seq_q + i;
      if (n_tiles > 0) ptx::tc_fence_after();
      __nv_bfloat16* orow = static_cast<__nv_bfloat16*>(P.o) + grow * D;
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t r[32];
        if (n_tiles > 0) {
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
      if (i < P.seq_q) {
        P.l[grow] = l * ptx::ex2(m_ref - m_true) * ptx::kRoundInv;
        P.m[grow] = m_true * kLn2;
      }
    } else if (lane == 0) {
      give_up(abort_flag, P.status, 1, fail_at);
    }
  }

  // ------------------------------------------------------------------ teardown
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, kTmemCols);
  }
}

template <int D, int SK, int MK>
int launch_one(cudaStream_t st, const DevParams& d, const CUtensorMap& tq, const CUtensorMap& tk,
               const CUtensorMap& tv, int* abort_flag) {
  // request enough shared memory that at most two CTAs share an SM (2 x 256 TMEM columns = all 512)
  constexpr size_t need = 3 * (D / 64) * ptx::kPanelBytes + sizeof(FwdSmem) + 1024;
  constexpr size_t smem = need > 80 * 1024 ? need : 80 * 1024;
  auto kern = fwd_sm100_kernel<D, SK, MK>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return FLEXATTN_ERR_CUDA;
    attr_set = true;
  }
  dim3 grid(d.n_qt, d.batch * d.heads);
  kern<<<grid, kFwdThreads, smem, st>>>(tq, tk, tv, d, abort_flag);
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

int launch_sm100_fwd(cudaStream_t st, const DevParams& d, int score, int mask) {
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
