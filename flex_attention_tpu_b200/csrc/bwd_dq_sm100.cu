// dQ backward on the 5th-generation tensor cores (sm_100a).
//
// Replaces the reference's Pallas dQ kernel (flex_attention_dq_bwd.py:282-385).  One CTA owns one
// 128-row query tile of one (batch, head): Q and dO stay in shared memory, K/V tiles stream through a
// two-stage ring, and per kv tile
//
//   S  = Q K^T, dP = dO V^T         tcgen05.mma, f32 accumulators in tensor memory (128 + 128 columns)
//   dS = P o (dP - delta) o sigma'  in registers by two warpgroups: threads t and t + 128 own query row t and
//                                   one 64-column half of the tile each; P is rebuilt from (l, m) as
//                                   exp2(x2 - (m log2e + log2 l)); written back as packed bf16 over S
//   dQ += dS K                      tcgen05.mma, A = dS from tensor memory, B = the same K tile read
//                                   MN-major; dQ (D columns) stays in tensor memory across kv tiles
//
// and the epilogue scales by sm_scale and stores bf16.  Masks run only on partial tiles.
#include "sm100.cuh"

namespace flexattn {
namespace {

constexpr int kThreads = 288;   // warps 0-3 and 4-7: element-wise warpgroups; warp 8: TMA + MMA issue
constexpr int kCtrlWarp = 8;

struct DqSmem {
  uint64_t bar_q, bar_kv[2], bar_sdp, bar_ds, bar_dq;
  uint32_t tmem_base;
  int32_t doc[2][kTile];
};

// This thread's 64 columns (keys j_first .. j_first+63) of its query row: raw S and dP in, packed bf16 dS out.
// nlse2 = log2(1 + 2^-9) - (m log2e + log2 l) (pre-scaling for pack_bf16_trunc) and delta belong to the row.  The mask functor is compiled in only for partial
// tiles.
template <int SK, int MK, bool kPartial>
__device__ __forceinline__ void dq_half_math(const uint32_t (&sr)[2][32], const uint32_t (&pr)[2][32],
                                             uint32_t (&pk)[32], float nlse2, float delta,
                                             const int32_t* __restrict__ s_doc, int i, int di, int j_first, int seq_k,
                                             int window, int stride, float c2, float slope2, float abase, float capl2,
                                             float csc) {
  const float bias0 = abase + nlse2;  // ALiBi: slope * (j_first - i), folded with the row's -lse2
#pragma unroll
  for (int c = 0; c < 64; c += 2) {
    float dv[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int cc = c + u;
      const float s = __uint_as_float(sr[cc >> 5][cc & 31]);
      const float dp = __uint_as_float(pr[cc >> 5][cc & 31]);
      float arg, dsig = 1.f;
      if constexpr (SK == FLEXATTN_SCORE_ALIBI) {
        arg = fmaf(s, c2, fmaf(slope2, (float)cc, bias0));
      } else if constexpr (SK == FLEXATTN_SCORE_SOFTCAP) {
        const float th = ptx::tanh_approx(s * csc);
        arg = fmaf(capl2, th, nlse2);
        dsig = fmaf(-th, th, 1.f);
      } else {
        arg = fmaf(s, c2, nlse2);
      }
      float p = ptx::ex2(arg);
      if constexpr (kPartial) {
        const int j = j_first + cc;
        const int dj = (MK == FLEXATTN_MASK_DOCUMENT) ? s_doc[cc] : 0;
        const bool keep = (j < seq_k) && mask_keep<MK>(i, j, window, stride, di, dj);
        p = keep ? p : 0.f;
      }
      float d = p * (dp - delta);
      if constexpr (SK == FLEXATTN_SCORE_SOFTCAP) d *= dsig;
      dv[u] = d;
    }
    pk[c >> 1] = ptx::pack_bf16_trunc(dv[0], dv[1]);
  }
}

template <int D, int SK, int MK>
__global__ void __launch_bounds__(kThreads, 1)
    dq_sm100_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                    const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                    const DevParams P, int* abort_flag) {
  constexpr int kPanels = D / 64;
  constexpr uint32_t kTileBytes = kPanels * ptx::kPanelBytes;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kColS = 0, kColDP = 128, kColDQ = 256;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sDO = smem + kTileBytes;
  uint8_t* sK = smem + 2 * kTileBytes;  // two stages
  uint8_t* sV = smem + 4 * kTileBytes;  // two stages
  DqSmem* sh = reinterpret_cast<DqSmem*>(smem + 6 * kTileBytes);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qt = P.n_qt - 1 - (int)blockIdx.x;
  const int bh = blockIdx.y, b = bh / P.heads, h = bh % P.heads;
  const int4 rm = P.row_map[(size_t)(P.map_rows > 1 ? b : 0) * P.n_qt + qt];
  const int n_tiles = rm.y - rm.x;

  if (*reinterpret_cast<volatile int*>(abort_flag) != 0) return;

  if (tid == 0) {
    ptx::mbar_init(&sh->bar_q, 1);
    ptx::mbar_init(&sh->bar_kv[0], 1);
    ptx::mbar_init(&sh->bar_kv[1], 1);
    ptx::mbar_init(&sh->bar_sdp, 1);
    ptx::mbar_init(&sh->bar_ds, 256);
    ptx::mbar_init(&sh->bar_dq, 1);
    ptx::fence_barrier_init();
  }
  if (warp == kCtrlWarp) {
    ptx::tmem_alloc(&sh->tmem_base, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = sh->tmem_base;

  if (warp == kCtrlWarp) {
    if (lane == 0 && n_tiles > 0) {
      bool ok = true;
      int fail_at = 1;
      ptx::prefetch_tensormap(&tm_q);
      ptx::prefetch_tensormap(&tm_do);
      ptx::prefetch_tensormap(&tm_k);
      ptx::prefetch_tensormap(&tm_v);
      ptx::mbar_arrive_expect_tx(&sh->bar_q, 2 * kTileBytes);
      ptx::mbar_arrive_expect_tx(&sh->bar_kv[0], 2 * kTileBytes);
#pragma unroll
      for (int p = 0; p < kPanels; ++p) {
        ptx::tma_load_3d(sQ + p * ptx::kPanelBytes, &tm_q, &sh->bar_q, p * 64, qt * kTile, bh);
        ptx::tma_load_3d(sDO + p * ptx::kPanelBytes, &tm_do, &sh->bar_q, p * 64, qt * kTile, bh);
        ptx::tma_load_3d(sK + p * ptx::kPanelBytes, &tm_k, &sh->bar_kv[0], p * 64, rm.x * kTile, bh);
        ptx::tma_load_3d(sV + p * ptx::kPanelBytes, &tm_v, &sh->bar_kv[0], p * 64, rm.x * kTile, bh);
      }
      constexpr uint32_t idesc_s = ptx::make_idesc(128, 128, false);
      constexpr uint32_t idesc_dq = ptx::make_idesc(128, D, true);
      const ptx::DescBase bQ = ptx::base_kmajor(ptx::smem_u32(sQ)), bDO = ptx::base_kmajor(ptx::smem_u32(sDO));
      ok = ptx::mbar_wait(&sh->bar_q, 0);
      for (int n = 0; n < n_tiles && ok; ++n) {
        const int st = n & 1;
        const ptx::DescBase bK = ptx::base_kmajor(ptx::smem_u32(sK + st * kTileBytes)),
                            bV = ptx::base_kmajor(ptx::smem_u32(sV + st * kTileBytes)),
                            bKt = ptx::base_mnmajor(ptx::smem_u32(sK + st * kTileBytes));
        if (n > 0) {
          // dQ MMA of the previous tile done: S/dP columns and the other K/V stage are free
          ok = ptx::mbar_wait(&sh->bar_dq, (n - 1) & 1);
          if (!ok) { fail_at = 2; break; }
        }
        if (n + 1 < n_tiles) {
          uint8_t* nK = sK + (st ^ 1) * kTileBytes;
          uint8_t* nV = sV + (st ^ 1) * kTileBytes;
          ptx::mbar_arrive_expect_tx(&sh->bar_kv[st ^ 1], 2 * kTileBytes);
#pragma unroll
          for (int p = 0; p < kPanels; ++p) {
            ptx::tma_load_3d(nK + p * ptx::kPanelBytes, &tm_k, &sh->bar_kv[st ^ 1], p * 64, (rm.x + n + 1) * kTile, bh);
            ptx::tma_load_3d(nV + p * ptx::kPanelBytes, &tm_v, &sh->bar_kv[st ^ 1], p * 64, (rm.x + n + 1) * kTile, bh);
          }
        }
        ok = ptx::mbar_wait(&sh->bar_kv[st], (n >> 1) & 1);
        if (!ok) { fail_at = 3; break; }
        ptx::tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          ptx::mma_ss(tmem + kColS, ptx::desc_at(bQ, ptx::koff_kmajor(kk)), ptx::desc_at(bK, ptx::koff_kmajor(kk)), idesc_s,
                      kk > 0);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          ptx::mma_ss(tmem + kColDP, ptx::desc_at(bDO, ptx::koff_kmajor(kk)), ptx::desc_at(bV, ptx::koff_kmajor(kk)), idesc_s,
                      kk > 0);
        ptx::mma_commit(&sh->bar_sdp);
        ok = ptx::mbar_wait(&sh->bar_ds, n & 1);
        if (!ok) { fail_at = 4; break; }
        ptx::tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk)
          ptx::mma_ts(tmem + kColDQ, tmem + kColS + kk * 8, ptx::desc_at(bKt, ptx::koff_mnmajor(kk)), idesc_dq,
                      (n > 0) || (kk > 0));
        ptx::mma_commit(&sh->bar_dq);
      }
      if (!ok) give_up(abort_flag, P.status, 2, fail_at);
    }
  } else {
    const int row = tid & 127;         // query row inside the tile = TMEM lane
    const int half = tid >> 7;         // which 64-column half of every tile this thread handles
    const int i = qt * kTile + row;
    const bool row_ok = i < P.seq_q;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const float c2 = P.sm_scale * kLog2e;
    const float slope2 = (SK == FLEXATTN_SCORE_ALIBI) ? P.alibi_slopes[h] * kLog2e : 0.f;
    const float capl2 = P.cap * kLog2e;
    const float csc = (SK == FLEXATTN_SCORE_SOFTCAP) ? P.sm_scale / P.cap : 0.f;
    const int32_t* doc = (MK == FLEXATTN_MASK_DOCUMENT) ? P.doc_ids + (size_t)b * P.doc_stride : nullptr;
    const int di = (MK == FLEXATTN_MASK_DOCUMENT && row_ok) ? doc[i] : 0;
    const size_t grow = (size_t)bh * P.seq_q + i;
    float lse2 = 0.f, delta = 0.f;
    if (row_ok) {
      const float l = P.l[grow];
      lse2 = l > 0.f ? fmaf(P.m[grow], kLog2e, log2f(l)) : 1.0e30f;
      delta = P.delta[grow];
    }
    bool ok = true;
    int fail_at = 0;

    for (int n = 0; n < n_tiles; ++n) {
      const int kt = rm.x + n, j0 = kt * kTile;
      const bool partial = !(kt >= rm.z && kt < rm.w);
      if (MK == FLEXATTN_MASK_DOCUMENT && partial) {
        const int j = j0 + row;
        if (half == 0) sh->doc[n & 1][row] = (j < P.seq_k) ? doc[j] : -1;
        ptx::named_bar_sync(1, 256);
      }
      // a failed wait never leaves the loop early: every thread keeps executing the same named barriers
      if (ok) {
        ok = __all_sync(0xffffffffu, ptx::mbar_wait(&sh->bar_sdp, n & 1));
        if (!ok) fail_at = 10;
      }
      if (!ok) continue;
      ptx::tc_fence_after();
      const float abase = slope2 * (float)(j0 - i);
      {
        uint32_t sr[2][32], pr[2][32];
        ptx::tmem_ld32(lane_base + kColS + half * 64, sr[0]);
        ptx::tmem_ld32(lane_base + kColS + half * 64 + 32, sr[1]);
        ptx::tmem_ld32(lane_base + kColDP + half * 64, pr[0]);
        ptx::tmem_ld32(lane_base + kColDP + half * 64 + 32, pr[1]);
        ptx::tmem_wait_ld();
        ptx::tmem_ld_acquire(sr[0]);
        ptx::tmem_ld_acquire(sr[1]);
        ptx::tmem_ld_acquire(pr[0]);
        ptx::tmem_ld_acquire(pr[1]);
        uint32_t pk[32];
        const float abase_h = abase + slope2 * (float)(half * 64);
        if (partial)
          dq_half_math<SK, MK, true>(sr, pr, pk, ptx::kRoundLog2 - lse2, delta, &sh->doc[n & 1][half * 64], i, di, j0 + half * 64,
                                     P.seq_k, P.window, P.stride, c2, slope2, abase_h, capl2, csc);
        else
          dq_half_math<SK, MK, false>(sr, pr, pk, ptx::kRoundLog2 - lse2, delta, &sh->doc[n & 1][half * 64], i, di, j0 + half * 64,
                                      P.seq_k, P.window, P.stride, c2, slope2, abase_h, capl2, csc);
        ptx::tmem_st32(lane_base + kColS + half * 32, pk);
      }
      ptx::tmem_wait_st();
      ptx::tc_fence_before();
      ptx::mbar_arrive(&sh->bar_ds);
    }

    if (ok && n_tiles > 0) {
      ok = __all_sync(0xffffffffu, ptx::mbar_wait(&sh->bar_dq, (n_tiles - 1) & 1));
      if (!ok) fail_at = 12;
    }
    if (ok) {
      if (n_tiles > 0) ptx::tc_fence_after();
      __nv_bfloat16* out = static_cast<__nv_bfloat16*>(P.dq) + grow * D;
      const float sc = P.sm_scale;
#pragma unroll 1
      for (int c0 = half * (D / 2); c0 < (half + 1) * (D / 2); c0 += 32) {
        uint32_t r[32];
        if (n_tiles > 0) {
          ptx::tmem_ld32(lane_base + kColDQ + c0, r);
          ptx::tmem_wait_ld();
          ptx::tmem_ld_acquire(r);
        } else {
#pragma unroll
          for (int c = 0; c < 32; ++c) r[c] = 0u;
        }
        if (row_ok) {
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            uint4 v4;
            v4.x = ptx::pack_bf16(__uint_as_float(r[c]) * sc, __uint_as_float(r[c + 1]) * sc);
            v4.y = ptx::pack_bf16(__uint_as_float(r[c + 2]) * sc, __uint_as_float(r[c + 3]) * sc);
            v4.z = ptx::pack_bf16(__uint_as_float(r[c + 4]) * sc, __uint_as_float(r[c + 5]) * sc);
            v4.w = ptx::pack_bf16(__uint_as_float(r[c + 6]) * sc, __uint_as_float(r[c + 7]) * sc);
            *reinterpret_cast<uint4*>(out + c0 + c) = v4;
          }
        }
      }
    } else if (lane == 0) {
      give_up(abort_flag, P.status, 2, fail_at);
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == kCtrlWarp) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, kTmemCols);
  }
}

template <int D, int SK, int MK>
int launch_one(cudaStream_t st, const DevParams& d, const CUtensorMap& tq, const CUtensorMap& tdo,
               const CUtensorMap& tk, const CUtensorMap& tv, int* abort_flag) {
  constexpr size_t smem = 6 * (D / 64) * ptx::kPanelBytes + sizeof(DqSmem) + 1024;
  // 512 TMEM columns per CTA: never let two CTAs share an SM (the second would spin in tcgen05.alloc)
  constexpr size_t smem_req = smem > 120 * 1024 ? smem : 120 * 1024;
  auto kern = dq_sm100_kernel<D, SK, MK>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_req) != cudaSuccess)
      return FLEXATTN_ERR_CUDA;
    attr_set = true;
  }
  dim3 grid(d.n_qt, d.batch * d.heads);
  kern<<<grid, kThreads, smem_req, st>>>(tq, tdo, tk, tv, d, abort_flag);
  return cudaGetLastError() == cudaSuccess ? FLEXATTN_OK : FLEXATTN_ERR_CUDA;
}

template <int D, int SK>
int launch_mask(cudaStream_t st, const DevParams& d, int mask, const CUtensorMap& tq, const CUtensorMap& tdo,
                const CUtensorMap& tk, const CUtensorMap& tv, int* af) {
  switch (mask) {
    case FLEXATTN_MASK_NONE: return launch_one<D, SK, FLEXATTN_MASK_NONE>(st, d, tq, tdo, tk, tv, af);
    case FLEXATTN_MASK_CAUSAL: return launch_one<D, SK, FLEXATTN_MASK_CAUSAL>(st, d, tq, tdo, tk, tv, af);
    case FLEXATTN_MASK_SLIDING_WINDOW: return launch_one<D, SK, FLEXATTN_MASK_SLIDING_WINDOW>(st, d, tq, tdo, tk, tv, af);
    case FLEXATTN_MASK_SLIDING_WINDOW_CAUSAL:
      return launch_one<D, SK, FLEXATTN_MASK_SLIDING_WINDOW_CAUSAL>(st, d, tq, tdo, tk, tv, af);
    case FLEXATTN_MASK_DOCUMENT: return launch_one<D, SK, FLEXATTN_MASK_DOCUMENT>(st, d, tq, tdo, tk, tv, af);
    case FLEXATTN_MASK_S2: return launch_one<D, SK, FLEXATTN_MASK_S2>(st, d, tq, tdo, tk, tv, af);
    default: return FLEXATTN_ERR_UNSUPPORTED_MOD;
  }
}

template <int D>
int launch_score(cudaStream_t st, const DevParams& d, int score, int mask, const CUtensorMap& tq,
                 const CUtensorMap& tdo, const CUtensorMap& tk, const CUtensorMap& tv, int* af) {
  switch (score) {
    case FLEXATTN_SCORE_NONE: return launch_mask<D, FLEXATTN_SCORE_NONE>(st, d, mask, tq, tdo, tk, tv, af);
    case FLEXATTN_SCORE_ALIBI: return launch_mask<D, FLEXATTN_SCORE_ALIBI>(st, d, mask, tq, tdo, tk, tv, af);
    case FLEXATTN_SCORE_SOFTCAP: return launch_mask<D, FLEXATTN_SCORE_SOFTCAP>(st, d, mask, tq, tdo, tk, tv, af);
    default: return FLEXATTN_ERR_UNSUPPORTED_MOD;
  }
}

}  // namespace

int launch_sm100_dq(cudaStream_t st, const DevParams& d, int score, int mask) {
  int* af = abort_flag_ptr();
  if (af == nullptr) return FLEXATTN_ERR_CUDA;
  CUtensorMap tq, tdo, tk, tv;
  const int slices = d.batch * d.heads;
  int e = make_tile_map(&tq, d.q, slices, d.seq_q, d.head_dim);
  if (e) return e;
  e = make_tile_map(&tdo, d.d_o, slices, d.seq_q, d.head_dim);
  if (e) return e;
  e = make_tile_map(&tk, d.k, slices, d.seq_k, d.head_dim);
  if (e) return e;
  e = make_tile_map(&tv, d.v, slices, d.seq_k, d.head_dim);
  if (e) return e;
  if (d.head_dim == 128) return launch_score<128>(st, d, score, mask, tq, tdo, tk, tv, af);
  if (d.head_dim == 64) return launch_score<64>(st, d, score, mask, tq, tdo, tk, tv, af);
  return FLEXATTN_ERR_UNSUPPORTED_HEAD_DIM;
}

}  // namespace flexattn
