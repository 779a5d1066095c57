// dK / dV backward on the 5th-generation tensor cores (sm_100a).
//
// Replaces the reference's Pallas dK/dV kernel (flex_attention_dkv_kernel.py:177-280 and its mask-aware
// twin flash_attention_dkv_bwd.py:183-308).  One CTA owns one 128-row kv tile of one (batch, head): K and
// V stay in shared memory, Q/dO tiles (and their row statistics) stream through a two-stage ring, and
// per q tile the TRANSPOSED score tile is formed so that the probabilities land in tensor memory in
// the layout the next MMA wants as its A operand:
//
//   S^T  = K Q^T, dP^T = V dO^T      tcgen05.mma, f32 accumulators (128 + 128 TMEM columns)
//   P^T, dS^T                        in registers; thread = key row, columns = query positions, whose statistics
//                                    (m log2e + log2 l, delta) are read from shared memory; written back as
//                                    packed bf16 over S^T / dP^T
//   dV += P^T dO ; dK += dS^T Q      tcgen05.mma, A from tensor memory, B = the dO / Q tile read MN-major
//
// Every tile is processed as two independent half-tile chains (query columns 0..63 and 64..127), each with
// its own warpgroup and barriers: while one chain's warpgroup does its element-wise work the tensor core
// runs the other chain's MMAs, so neither side idles.  dK, dV (D columns each) stay in tensor memory
// across q tiles: 512 columns in total, one CTA per SM.
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

constexpr int kThreads = 320;  // warps 0-3, 4-7: element-wise warpgroups (one per half-tile chain); 8: MMA; 9: TMA
constexpr int kMmaWarp = 8, kTmaWarp = 9;
constexpr bool kInOrderMma = true;  // rely on issue-order execution of one thread's tcgen05.mma stream

struct DkvSmem {
  uint64_t bar_kv, bar_q[2], bar_free[2], bar_sdp[2], bar_pds[2], bar_acc[2], bar_zero;
  uint32_t tmem_base;
  alignas(16) float nlse2[2][kTile];  // -(m log2e + log2 l) of the query rows of the tile in flight
  alignas(16) float delta[2][kTile];
  alignas(16) int32_t doc[2][kTile];
};

// One 64-column half of a transposed tile: this thread's key row against query columns i_first .. i_first+63.
// sr / pr: raw S^T and dP^T values; outputs packed bf16 P^T and dS^T.  Query statistics come from shared memory
// four at a time.  The mask functor is compiled in only for partial tiles.
template <int SK, int MK, bool kPartial>
__device__ __forceinline__ void dkv_half_math(const uint32_t (&sr)[2][32], const uint32_t (&pr)[2][32],
                                              uint32_t (&pk_p)[32], uint32_t (&pk_ds)[32],
                                              const float* __restrict__ s_nlse2, const float* __restrict__ s_delta,
                                              const int32_t* __restrict__ s_doc, int i_first, int j, int dj, int seq_q,
                                              int window, int stride, float c2, float slope2, float abase, float capl2,
                                              float csc) {
#pragma unroll
  for (int c = 0; c < 64; c += 4) {
    const float4 nl4 = *reinterpret_cast<const float4*>(s_nlse2 + c);
    const float4 dl4 = *reinterpret_cast<const float4*>(s_delta + c);
    const float nl[4] = {nl4.x, nl4.y, nl4.z, nl4.w};
    const float dl[4] = {dl4.x, dl4.y, dl4.z, dl4.w};
    float pv[4], dv[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int cc = c + u;
      const float s = __uint_as_float(sr[cc >> 5][cc & 31]);
      const float dp = __uint_as_float(pr[cc >> 5][cc & 31]);
      float arg, dsig = 1.f;  // arg = log2-domain logit minus the row's log-sum-exp
      if constexpr (SK == FLEXATTN_SCORE_ALIBI) {
        arg = fmaf(s, c2, fmaf(-slope2, (float)cc, abase) + nl[u]);
      } else if constexpr (SK == FLEXATTN_SCORE_SOFTCAP) {
        const float th = ptx::tanh_approx(s * csc);
        arg = fmaf(capl2, th, nl[u]);
        dsig = fmaf(-th, th, 1.f);
      } else {
        arg = fmaf(s, c2, nl[u]);
      }
      float p = ptx::ex2(arg);
      if constexpr (kPartial) {
        const int i = i_first + cc;
        const int di = (MK == FLEXATTN_MASK_DOCUMENT) ? s_doc[cc] : 0;
        const bool keep = (i < seq_q) && mask_keep<MK>(i, j, window, stride, di, dj);
        p = keep ? p : 0.f;
      }
      float d = p * (dp - dl[u]);
      if constexpr (SK == FLEXATTN_SCORE_SOFTCAP) d *= dsig;
      pv[u] = p;
      dv[u] = d;
    }
    pk_p[c >> 1] = ptx::pack_bf16_trunc(pv[0], pv[1]);
    pk_p[(c >> 1) + 1] = ptx::pack_bf16_trunc(pv[2], pv[3]);
    pk_ds[c >> 1] = ptx::pack_bf16_trunc(dv[0], dv[1]);
    pk_ds[(c >> 1) + 1] = ptx::pack_bf16_trunc(dv[2], dv[3]);
  }
}

template <int D, int SK, int MK>
__global__ void __launch_bounds__(kThreads, 1)
    dkv_sm100_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                     const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                     const DevParams P, int* abort_flag) {
  constexpr int kPanels = D / 64;
  constexpr uint32_t kTileBytes = kPanels * ptx::kPanelBytes;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kColS = 0, kColDP = 128, kColDK = 256, kColDV = 384;
  constexpr uint32_t kRowsHalfBytes = 64 * 128;  // 64 rows of a K-major panel

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sK = smem;
  uint8_t* sV = smem + kTileBytes;
  uint8_t* sQ = smem + 2 * kTileBytes;   // two stages
  uint8_t* sDO = smem + 4 * kTileBytes;  // two stages
  DkvSmem* sh = reinterpret_cast<DkvSmem*>(smem + 6 * kTileBytes);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kt = blockIdx.x;  // early kv tiles see the most query tiles under a causal mask: run them first
  const int bh = blockIdx.y, b = bh / P.heads, h = bh % P.heads;
  const int4 cm = P.col_map[(size_t)(P.map_rows > 1 ? b : 0) * P.n_kt + kt];
  const int N = cm.y - cm.x;

  if (*reinterpret_cast<volatile int*>(abort_flag) != 0) return;

  if (tid == 0) {
    ptx::mbar_init(&sh->bar_kv, 1);
    ptx::mbar_init(&sh->bar_zero, 256);
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(&sh->bar_q[s], 1);
      ptx::mbar_init(&sh->bar_free[s], 1);
      ptx::mbar_init(&sh->bar_sdp[s], 1);
      ptx::mbar_init(&sh->bar_pds[s], 128);
      ptx::mbar_init(&sh->bar_acc[s], 1);
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

  if (warp == kTmaWarp) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && N > 0) {
      bool ok = true;
      ptx::prefetch_tensormap(&tm_q);
      ptx::prefetch_tensormap(&tm_do);
      ptx::prefetch_tensormap(&tm_k);
      ptx::prefetch_tensormap(&tm_v);
      ptx::mbar_arrive_expect_tx(&sh->bar_kv, 2 * kTileBytes);
#pragma unroll
      for (int p = 0; p < kPanels; ++p) {
        ptx::tma_load_3d(sK + p * ptx::kPanelBytes, &tm_k, &sh->bar_kv, p * 64, kt * kTile, bh);
        ptx::tma_load_3d(sV + p * ptx::kPanelBytes, &tm_v, &sh->bar_kv, p * 64, kt * kTile, bh);
      }
      for (int n = 0; n < N && ok; ++n) {
        const int st = n & 1;
        if (n >= 2) {  // the stage held tile n-2: wait until all of its MMAs have completed
          ok = ptx::mbar_wait(&sh->bar_free[st], ((n - 2) >> 1) & 1);
          if (!ok) break;
        }
        ptx::mbar_arrive_expect_tx(&sh->bar_q[st], 2 * kTileBytes);
#pragma unroll
        for (int p = 0; p < kPanels; ++p) {
          ptx::tma_load_3d(sQ + st * kTileBytes + p * ptx::kPanelBytes, &tm_q, &sh->bar_q[st], p * 64,
                           (cm.x + n) * kTile, bh);
          ptx::tma_load_3d(sDO + st * kTileBytes + p * ptx::kPanelBytes, &tm_do, &sh->bar_q[st], p * 64,
                           (cm.x + n) * kTile, bh);
        }
      }
      if (!ok) give_up(abort_flag, P.status, 3, 20);
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer: two half-tile chains
    // Chain c owns query columns [64c, 64c+64) of every tile: S^T_c / dP^T_c (N = 64) -> warpgroup c ->
    // dV, dK += (P^T_c, dS^T_c) x (dO, Q rows 64c..).  The chains alternate on the tensor core so that one
    // chain's MMAs run while the other chain's warpgroup does its element-wise work.  dK / dV are zeroed by the
    // warpgroups first, so every accumulation MMA adds.  (N = 64 MMAs cost as many cycles as N = 128 ones - the
    // A operand fetch of 128 rows bounds them - so the chains buy overlap at the price of tensor efficiency.)
    if (lane == 0 && N > 0) {
      bool ok = true;
      int fail_at = 1;
      constexpr uint32_t idesc_s = ptx::make_idesc(128, 64, false);
      constexpr uint32_t idesc_acc = ptx::make_idesc(128, D, true);
      const uint32_t aK = ptx::smem_u32(sK), aV = ptx::smem_u32(sV), aQ = ptx::smem_u32(sQ), aDO = ptx::smem_u32(sDO);
      const ptx::DescBase bK = ptx::base_kmajor(aK), bV = ptx::base_kmajor(aV);
      auto issue_sdp = [&](int n, int c) {  // S^T_c = K Q_c^T and dP^T_c = V dO_c^T for tile n
        const uint32_t off = (uint32_t)(n & 1) * kTileBytes + (uint32_t)c * kRowsHalfBytes;
        const ptx::DescBase bQ = ptx::base_kmajor(aQ + off), bDO = ptx::base_kmajor(aDO + off);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          ptx::mma_ss(tmem + kColS + 64 * c, ptx::desc_at(bK, ptx::koff_kmajor(kk)),
                         ptx::desc_at(bQ, ptx::koff_kmajor(kk)), idesc_s, kk > 0);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          ptx::mma_ss(tmem + kColDP + 64 * c, ptx::desc_at(bV, ptx::koff_kmajor(kk)),
                         ptx::desc_at(bDO, ptx::koff_kmajor(kk)), idesc_s, kk > 0);
        ptx::mma_commit(&sh->bar_sdp[c]);
      };
      auto issue_acc = [&](int n, int c) {  // dV += P^T_c dO_c ; dK += dS^T_c Q_c  (four K steps of 16 query rows)
        const uint32_t off = (uint32_t)(n & 1) * kTileBytes + (uint32_t)c * 4 * 2048u;
        const ptx::DescBase bQt = ptx::base_mnmajor(aQ + off), bDOt = ptx::base_mnmajor(aDO + off);
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4)
          ptx::mma_ts(tmem + kColDV, tmem + kColS + 64 * c + k4 * 8, ptx::desc_at(bDOt, ptx::koff_mnmajor(k4)),
                         idesc_acc, 1);
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4)
          ptx::mma_ts(tmem + kColDK, tmem + kColDP + 64 * c + k4 * 8, ptx::desc_at(bQt, ptx::koff_mnmajor(k4)),
                         idesc_acc, 1);
        ptx::mma_commit(&sh->bar_acc[c]);
      };
      ok = ptx::mbar_wait(&sh->bar_kv, 0) && ptx::mbar_wait(&sh->bar_q[0], 0);
      if (ok) {
        ptx::tc_fence_after();
        issue_sdp(0, 0);
        issue_sdp(0, 1);
        ok = ptx::mbar_wait(&sh->bar_zero, 0);  // dK / dV columns zeroed
        if (!ok) fail_at = 7;
      }
      for (int n = 0; n < N && ok; ++n) {
        const uint32_t par = n & 1;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          ok = ptx::mbar_wait(&sh->bar_pds[c], par);
          if (!ok) { fail_at = 2 + c; break; }
          if (c == 0) FA_TRACE(0); else FA_TRACE(3);
          ptx::tc_fence_after();
          issue_acc(n, c);
          if (c == 1) ptx::mma_commit(&sh->bar_free[n & 1]);  // every MMA reading this Q/dO stage is issued
          if (c == 0) FA_TRACE(1); else FA_TRACE(4);
          if (n + 1 < N) {
            if (c == 0) {
              ok = ptx::mbar_wait(&sh->bar_q[(n + 1) & 1], ((n + 1) >> 1) & 1);
              if (!ok) { fail_at = 4; break; }
            }
            // chain c's accumulation MMAs read P^T_c / dS^T_c from the columns the next S^T_c / dP^T_c overwrite.
            // MMAs issued by one thread execute in issue order, so no wait for their completion is needed.
            if (!kInOrderMma) {
              ok = ptx::mbar_wait(&sh->bar_acc[c], par);
              if (!ok) { fail_at = 5 + c; break; }
            }
            ptx::tc_fence_after();
            issue_sdp(n + 1, c);
            if (c == 0) FA_TRACE(2); else FA_TRACE(5);
          }
        }
      }
      if (!ok) give_up(abort_flag, P.status, 3, fail_at);
    }
  } else {
    // ------------------------------------------------------------------ element-wise warpgroups (chain = tid / 128)
    const int row = tid & 127;        // key row inside the tile = TMEM lane
    const int chain = tid >> 7;       // which 64 query columns of every tile this warpgroup handles
    const int j = kt * kTile + row;   // global key position
    const bool row_ok = j < P.seq_k;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t colS = kColS + 64 * chain, colDP = kColDP + 64 * chain;
    const float c2 = P.sm_scale * kLog2e;
    const float slope2 = (SK == FLEXATTN_SCORE_ALIBI) ? P.alibi_slopes[h] * kLog2e : 0.f;
    const float capl2 = P.cap * kLog2e;
    const float csc = (SK == FLEXATTN_SCORE_SOFTCAP) ? P.sm_scale / P.cap : 0.f;
    const int32_t* doc = (MK == FLEXATTN_MASK_DOCUMENT) ? P.doc_ids + (size_t)b * P.doc_stride : nullptr;
    const int dj = (MK == FLEXATTN_MASK_DOCUMENT && row_ok) ? doc[j] : -2;
    const size_t stat_base = (size_t)bh * P.seq_q;
    bool ok = true;
    int fail_at = 0;

    {  // zero the accumulators (warpgroup 0: dK, warpgroup 1: dV): every accumulation MMA adds
      uint32_t z[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) z[c] = 0u;
      const uint32_t col = chain ? kColDV : kColDK;
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) ptx::tmem_st32(lane_base + col + c0, z);
      ptx::tmem_wait_st();
      ptx::tc_fence_before();
      ptx::mbar_arrive(&sh->bar_zero);
    }

    for (int n = 0; n < N; ++n) {
      const int st = n & 1;
      const int qt = cm.x + n, i0 = qt * kTile + 64 * chain;  // first query position of this chain's columns
      const bool partial = !(qt >= cm.z && qt < cm.w);
      if (row < 64) {
        // statistics of this chain's 64 query rows (threads 0..63 of the warpgroup stage one row each)
        const int i = i0 + row;
        float nl = ptx::kRoundLog2, dl = 0.f;
        if (i < P.seq_q) {
          const float l = P.l[stat_base + i];
          // l == 0 (fully masked row): force p to 0; kRoundLog2 pre-scales p for pack_bf16_trunc
          nl = l > 0.f ? ptx::kRoundLog2 - fmaf(P.m[stat_base + i], kLog2e, log2f(l)) : -1.0e30f;
          dl = P.delta[stat_base + i];
        }
        sh->nlse2[st][64 * chain + row] = nl;
        sh->delta[st][64 * chain + row] = dl;
        if (MK == FLEXATTN_MASK_DOCUMENT) sh->doc[st][64 * chain + row] = (i < P.seq_q) ? doc[i] : -1;
      }
      ptx::named_bar_sync(1 + chain, 128);
      if (tid == 0) FA_TRACE(8);
      // a failed wait never leaves the loop early: every thread keeps executing the same named barriers
      if (ok) {
        ok = __all_sync(0xffffffffu, ptx::mbar_wait(&sh->bar_sdp[chain], n & 1));
        if (!ok) fail_at = 10;
      }
      if (!ok) continue;
      if (tid == 0) FA_TRACE(9);
      ptx::tc_fence_after();
      uint32_t sr[2][32], pr[2][32];
      ptx::tmem_ld32(lane_base + colS, sr[0]);
      ptx::tmem_ld32(lane_base + colS + 32, sr[1]);
      ptx::tmem_ld32(lane_base + colDP, pr[0]);
      ptx::tmem_ld32(lane_base + colDP + 32, pr[1]);
      ptx::tmem_wait_ld();
      ptx::tmem_ld_acquire(sr[0]);
      ptx::tmem_ld_acquire(sr[1]);
      ptx::tmem_ld_acquire(pr[0]);
      ptx::tmem_ld_acquire(pr[1]);
      if (tid == 0) FA_TRACE(10);
      uint32_t pk_p[32], pk_ds[32];
      const float abase = slope2 * (float)(j - i0);  // ALiBi bias = slope * (j - i), i = i0 + column
      if (partial)
        dkv_half_math<SK, MK, true>(sr, pr, pk_p, pk_ds, &sh->nlse2[st][64 * chain], &sh->delta[st][64 * chain],
                                    &sh->doc[st][64 * chain], i0, j, dj, P.seq_q, P.window, P.stride, c2, slope2,
                                    abase, capl2, csc);
      else
        dkv_half_math<SK, MK, false>(sr, pr, pk_p, pk_ds, &sh->nlse2[st][64 * chain], &sh->delta[st][64 * chain],
                                     &sh->doc[st][64 * chain], i0, j, dj, P.seq_q, P.window, P.stride, c2, slope2,
                                     abase, capl2, csc);
      ptx::tmem_st32(lane_base + colS, pk_p);
      ptx::tmem_st32(lane_base + colDP, pk_ds);
      if (tid == 0) FA_TRACE(11);
      ptx::tmem_wait_st();
      ptx::tc_fence_before();
      ptx::mbar_arrive(&sh->bar_pds[chain]);
      if (tid == 0) FA_TRACE(12);
    }

    if (ok && N > 0) {
      // both chains' accumulation MMAs of the last tile must have completed
      ok = __all_sync(0xffffffffu, ptx::mbar_wait(&sh->bar_acc[0], (N - 1) & 1) &&
                                       ptx::mbar_wait(&sh->bar_acc[1], (N - 1) & 1));
      if (!ok) fail_at = 12;
    }
    if (ok) {
      if (N > 0) ptx::tc_fence_after();
      const size_t grow = (size_t)bh * P.seq_k + j;
      {
        const int which = chain;  // warpgroup 0 stores dK, warpgroup 1 stores dV
        __nv_bfloat16* out = static_cast<__nv_bfloat16*>(which ? P.dv : P.dk) + grow * D;
        const float sc = which ? 1.f : P.sm_scale;
        const uint32_t col = which ? kColDV : kColDK;
#pragma unroll 1
        for (int c0 = 0; c0 < D; c0 += 32) {
          uint32_t r[32];
          if (N > 0) {
            ptx::tmem_ld32(lane_base + col + c0, r);
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
      }
    } else if (lane == 0) {
      give_up(abort_flag, P.status, 3, fail_at);
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, kTmemCols);
  }
}

template <int D, int SK, int MK>
int launch_one(cudaStream_t st, const DevParams& d, const CUtensorMap& tq, const CUtensorMap& tdo,
               const CUtensorMap& tk, const CUtensorMap& tv, int* abort_flag) {
  constexpr size_t smem = 6 * (D / 64) * ptx::kPanelBytes + sizeof(DkvSmem) + 1024;
  // 512 TMEM columns per CTA: never let two CTAs share an SM (the second would spin in tcgen05.alloc)
  constexpr size_t smem_req = smem > 120 * 1024 ? smem : 120 * 1024;
  auto kern = dkv_sm100_kernel<D, SK, MK>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_req) != cudaSuccess)
      return FLEXATTN_ERR_CUDA;
    attr_set = true;
  }
  dim3 grid(d.n_kt, d.batch * d.heads);
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

int launch_sm100_dkv(cudaStream_t st, const DevParams& d, int score, int mask) {
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
