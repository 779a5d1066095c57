// Forward flex attention, persistent software-pipelined kernel (sm_100a).
//
// Replaces the reference's Pallas forward kernel (flex_attention_kernel.py:196-327): online softmax in the log2
// domain over 128 x 128 score tiles, masks evaluated only on partial tiles.  One CTA per SM stays
// resident and walks a list of work items (q tile, batch*head), heaviest q tiles first, item w going to CTA
// w mod gridDim.x.  Inside a CTA the kv tiles of all its items form ONE stream, numbered T = 0, 1, 2 ...: the
// K/V rings, the three score buffers and every barrier phase are indexed by T, so the loads and the Q K^T MMAs
// of the next item start while the softmax and the epilogue of the current one are still running, and the
// per-item prologue (loads in flight, first scores) and epilogue (normalise, store) cost no tensor-core time.
//
//   warp 8, lane 0 : MMA issuer.  S[T % 3] = Q K[T]^T runs up to three kv tiles ahead of the softmax;
//                    O += P[T] V[T] is issued as soon as the softmax has written P[T] over S[T % 3].
//   warp 9, lane 0 : TMA producer for Q (one buffer: the next item's Q is loaded as soon as the last Q K^T of the
//                    current item has run, three tiles before its softmax ends) and K (two-stage ring).
//   warp 10, lane 0: TMA producer for V (two-stage ring).  Each ring stage is refilled as soon as the MMA that
//                    read it has completed (tcgen05.commit -> mbarrier).
//   warps 0..7     : softmax, two warpgroups.  Threads t and t + 128 share query row t (= TMEM lane t)
//                    and take one 64-column half of every score tile each; partial row maxima are
//                    exchanged through shared memory; P goes back to tensor memory as packed bf16; O is
//                    rescaled in tensor memory only when the running max moved by more than 2^8.  After an
//                    item's last tile they read O out of tensor memory, normalise and store it, and go on
//                    to the next item; the first P V of that item is issued only after they have written
//                    its first P, i.e. after they are done reading the previous O.
//
// Tensor memory: S0, S1, S2 (3 x 128 columns) + O (D columns) = 512 for D = 128.  Shared memory: Q, an output
// staging tile, 2 K and 2 V tiles (192 KB for D = 128).
#include "sched.cuh"
#include "sm100.cuh"

namespace flexattn {
namespace FLEXATTN_TU_NAMESPACE {

constexpr int kThreads = 352;
constexpr int kMmaWarp = 8, kTmaWarp = 9, kTmaWarpV = 10;
constexpr int kHalf = kTile / 2;
constexpr int kSBufs = 3;

// Order in which an item's kv tiles are visited.  The ALiBi bias slope * (k_idx - q_idx) grows with the key
// position, so in ascending order the running row maximum of a steep head rises by more than the lazy-rescale
// threshold at EVERY tile, and each rescale waits for the previous P V and rewrites O.  Visiting the tiles from the
// last one down meets the largest bias first and rescales (almost) never; other score kinds keep ascending order.
template <int SK>
__device__ __forceinline__ int kv_tile_at(int first, int end, int n) {
  return SK == FLEXATTN_SCORE_ALIBI ? end - 1 - n : first + n;
}
constexpr float kLazyRescale = 8.0f;  // log2 units

struct PipeSmem {
  uint64_t bar_q, bar_qfree, bar_k[2], bar_v[2], bar_kfree[2], bar_s[kSBufs], bar_p[kSBufs], bar_pv[kSBufs];
  uint32_t tmem_base;
  int32_t item_tiles[8];  // kv tiles of the CTA's non-empty items (ring; -1 ends the list), producer -> MMA issuer
  float pmax[2][2][kTile];  // [tile parity][column half][row]
  float lsum[2][kTile];     // [column half][row]
  int32_t doc[2][kTile];
};

// x: this thread's 64 raw scores (columns c_base .. c_base+63 of the tile) -> log2-domain logits in place;
// returns their maximum.  kBias: ab_row points at the bias of this row's first column (nullptr for a row past the
// end of the sequence); the bias is added after the score function and before the mask.
// what a user score function sees besides the score and the positions
struct ScoreCtx {
  float sm_scale;
  int b, h;
};

// kInterval: the row's kept keys are the interval [klo, khi) (interval mask kinds; documents over sorted ids): a
// partial tile then tests one bit per element of a bitmap built once per 32 columns.
template <int SK, int MK, bool kPartial, bool kBias = false, bool kInterval = kMaskIsInterval<MK>>
__device__ __forceinline__ float score_half(float (&x)[kHalf], int i, int j0, int c_base, int seq_k, int window,
                                            int stride, float c2, float slope2, float capl2, float csc, int di,
                                            const int32_t* s_doc, const ScoreCtx ctx,
                                            const float* __restrict__ ab_row = nullptr, int klo = 0, int khi = 0) {
  float mx[4] = {kMasked, kMasked, kMasked, kMasked};
  uint32_t keep = 0u;  // kept columns of the current group of 32 (kInterval on partial tiles)
  const float abase = slope2 * (float)(j0 + c_base - i);
  float bias[8];
  if constexpr (SK == FLEXATTN_SCORE_SOFTCAP || SK == FLEXATTN_SCORE_USER) {
    // scalar form: the packed one costs registers here
#pragma unroll
    for (int c = 0; c < kHalf; ++c) {
      float t;
      if constexpr (SK == FLEXATTN_SCORE_USER) t = user_score(x[c] * ctx.sm_scale, ctx.b, ctx.h, i, j0 + c_base + c) * kLog2e;
      else t = capl2 * ptx::tanh_approx(x[c] * csc);
      if constexpr (kBias) {
        if ((c & 7) == 0) {
          if (ab_row != nullptr) ptx::load_bias8(bias, ab_row + c, seq_k - (j0 + c_base + c));
          else
#pragma unroll
            for (int u = 0; u < 8; ++u) bias[u] = 0.f;
        }
        t = fmaf(bias[c & 7], kLog2e, t);
      }
      if constexpr (kPartial && kInterval) {
        if ((c & 31) == 0) keep = range_bits32(klo - (j0 + c_base + c), khi - (j0 + c_base + c));
        t = (keep >> (c & 31)) & 1u ? t : kMasked;
      } else if constexpr (kPartial) {
        const int j = j0 + c_base + c;
        const int dj = (MK == FLEXATTN_MASK_DOCUMENT) ? s_doc[c_base + c] : 0;
        t = ((j < seq_k) && mask_keep<MK>(i, j, window, stride, di, dj)) ? t : kMasked;
      }
      x[c] = t;
      mx[c & 3] = fmaxf(mx[c & 3], t);
    }
    return fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
  } else {
  // the score arithmetic runs two columns per instruction (packed f32x2); masking and the maximum are scalar
  // ALiBi: the bias of columns (c, c + 1) advances by a constant from pair to pair: one packed add instead of
  // rebuilding it from the column numbers
  uint64_t b2 = ptx::pack2(abase, abase + slope2);
  const uint64_t bstep2 = ptx::pack2(2.f * slope2, 2.f * slope2);
#pragma unroll
  for (int c = 0; c < kHalf; c += 2) {
    const uint64_t x2 = ptx::pack2(x[c], x[c + 1]);
    float t0, t1;
    if constexpr (SK == FLEXATTN_SCORE_ALIBI) {
      ptx::unpack2(ptx::fma2(x2, ptx::pack2(c2, c2), b2), t0, t1);
      b2 = ptx::add2(b2, bstep2);
    } else {
      ptx::unpack2(ptx::mul2(x2, ptx::pack2(c2, c2)), t0, t1);
    }
    if constexpr (kBias) {
      if ((c & 7) == 0) {
        if (ab_row != nullptr) ptx::load_bias8(bias, ab_row + c, seq_k - (j0 + c_base + c));
        else
#pragma unroll
          for (int u = 0; u < 8; ++u) bias[u] = 0.f;
      }
      t0 = fmaf(bias[c & 7], kLog2e, t0);
      t1 = fmaf(bias[(c & 7) + 1], kLog2e, t1);
    }
    if constexpr (kPartial && kInterval) {
      if ((c & 31) == 0) keep = range_bits32(klo - (j0 + c_base + c), khi - (j0 + c_base + c));
      t0 = (keep >> (c & 31)) & 1u ? t0 : kMasked;
      t1 = (keep >> ((c & 31) + 1)) & 1u ? t1 : kMasked;
    } else if constexpr (kPartial) {
      const int j = j0 + c_base + c;
      const int d0 = (MK == FLEXATTN_MASK_DOCUMENT) ? s_doc[c_base + c] : 0;
      const int d1 = (MK == FLEXATTN_MASK_DOCUMENT) ? s_doc[c_base + c + 1] : 0;
      t0 = ((j < seq_k) && mask_keep<MK>(i, j, window, stride, di, d0)) ? t0 : kMasked;
      t1 = ((j + 1 < seq_k) && mask_keep<MK>(i, j + 1, window, stride, di, d1)) ? t1 : kMasked;
    }
    x[c] = t0;
    x[c + 1] = t1;
    mx[(c >> 1) & 3] = ptx::max3(mx[(c >> 1) & 3], t0, t1);
  }
  return fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
  }
}

template <int D, int SK, int MK>
__global__ void __launch_bounds__(kThreads, 1)
    fwd_pipe_sm100_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                          const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                          const DevParams P, int* abort_flag) {
  constexpr int kPanels = D / 64;
  constexpr uint32_t kTileBytes = kPanels * ptx::kPanelBytes;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kColO = kSBufs * 128;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                   // the Q tile of the item whose Q K^T MMAs are being issued
  uint8_t* sO = smem + kTileBytes;      // staging of an item's output tile for its bulk store
  uint8_t* sK = smem + 2 * kTileBytes;  // two stages
  uint8_t* sV = smem + 4 * kTileBytes;  // two stages
  PipeSmem* sh = reinterpret_cast<PipeSmem*>(smem + 6 * kTileBytes);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (aborted_on_entry(abort_flag, P.status, 4)) return;

  if (tid == 0) {
    ptx::mbar_init(&sh->bar_q, 1);
    ptx::mbar_init(&sh->bar_qfree, 1);
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(&sh->bar_k[s], 1);
      ptx::mbar_init(&sh->bar_v[s], 1);
      ptx::mbar_init(&sh->bar_kfree[s], 1);
    }
    for (int s = 0; s < kSBufs; ++s) {
      ptx::mbar_init(&sh->bar_pv[s], 1);
      ptx::mbar_init(&sh->bar_s[s], 1);
      ptx::mbar_init(&sh->bar_p[s], 8);  // one arrival per softmax warp
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

  // bar_pv has one barrier per SCORE buffer (three), not per V stage: the softmax warpgroups wait on it only now and
  // then (lazy rescale, item epilogue) and may be up to three tiles ahead of the P V MMAs; a wait by parity is only
  // unambiguous while the waiter is less than two completions ahead of the barrier, and with barrier T % 3 the
  // previous completion, P V of tile T-3, is known to be done once S of tile T has been read.
  // In every role: T = index of a kv tile in this CTA's stream over all its items, qi = index of an item among
  // the CTA's non-empty items.  Ring stage = index & 1, barrier phase = (index >> 1) & 1 (score buffers: % 3, / 3).
  if (warp == kTmaWarp) {
    // ------------------------------------------------------------------ TMA producer: Q and K
    if (lane == 0) {
      bool ok = true;
      int fail_at = 0;
      ptx::prefetch_tensormap(&tm_q);
      ptx::prefetch_tensormap(&tm_k);
      int T = 0, qi = 0;
      for (ItemCursor it(P); ok; it.next(), ++qi) {
        it.skip_empty();
        if (!it.valid()) break;
        const int bh = it.bh(), first = it.rm.x, end = it.rm.y, N = it.tiles();
        if (qi >= 1) {  // the buffer holds the Q tile of the previous item: all of its Q K^T MMAs must have completed
          ok = ptx::mbar_wait(&sh->bar_qfree, (qi - 1) & 1);
          if (!ok) { fail_at = 20; break; }
        }
        sh->item_tiles[qi & 7] = N;  // read by the MMA issuer after it has waited on bar_q (release / acquire)
        ptx::mbar_arrive_expect_tx(&sh->bar_q, kTileBytes);
#pragma unroll
        for (int p = 0; p < kPanels; ++p)
          ptx::tma_load_3d(sQ + p * ptx::kPanelBytes, &tm_q, &sh->bar_q, p * 64, it.qt() * kTile, bh);
        for (int t = 0; t < N; ++t, ++T) {
          if (T >= 2) {  // K[T] replaces K[T-2], read by Q K^T of tile T-2
            ok = ptx::mbar_wait(&sh->bar_kfree[T & 1], ((T - 2) >> 1) & 1);
            if (!ok) { fail_at = 21; break; }
          }
          ptx::mbar_arrive_expect_tx(&sh->bar_k[T & 1], kTileBytes);
#pragma unroll
          for (int p = 0; p < kPanels; ++p)
            ptx::tma_load_3d(sK + (T & 1) * kTileBytes + p * ptx::kPanelBytes, &tm_k, &sh->bar_k[T & 1], p * 64,
                             kv_tile_at<SK>(first, end, t) * kTile, bh);
        }
      }
      if (ok) {
        // End of the list: one more completion of the Q barrier, carrying the terminator.  Like a real item it has to
        // wait for the barrier's previous phase (the Q tile of the previous item) to be over - its bytes landed and consumed -
        // before arriving on it again: an arrive into a phase that still expects bytes would corrupt it.
        if (qi >= 1) ok = ptx::mbar_wait(&sh->bar_qfree, (qi - 1) & 1);
        if (ok) {
          sh->item_tiles[qi & 7] = -1;
          ptx::mbar_arrive(&sh->bar_q);
        } else {
          fail_at = 24;
        }
      }
      if (!ok) give_up(abort_flag, P.status, 4, fail_at);
    }
  } else if (warp == kTmaWarpV) {
    // ------------------------------------------------------------------ TMA producer: V
    if (lane == 0) {
      bool ok = true;
      ptx::prefetch_tensormap(&tm_v);
      int T = 0;
      uint32_t wsb = 0, wph = 0;  // barrier (T-2) % 3 and phase ((T-2) / 3) & 1 of the P V this thread waits for
      for (ItemCursor it(P); ok; it.next()) {
        it.skip_empty();
        if (!it.valid()) break;
        const int bh = it.bh(), first = it.rm.x, end = it.rm.y, N = it.tiles();
        for (int t = 0; t < N; ++t, ++T) {
          if (T >= 2) {  // V[T] replaces V[T-2], read by P V of tile T-2
            ok = ptx::mbar_wait(&sh->bar_pv[wsb], wph);
            if (!ok) break;
            if (++wsb == kSBufs) { wsb = 0; wph ^= 1u; }
          }
          ptx::mbar_arrive_expect_tx(&sh->bar_v[T & 1], kTileBytes);
#pragma unroll
          for (int p = 0; p < kPanels; ++p)
            ptx::tma_load_3d(sV + (T & 1) * kTileBytes + p * ptx::kPanelBytes, &tm_v, &sh->bar_v[T & 1], p * 64,
                             kv_tile_at<SK>(first, end, t) * kTile, bh);
        }
      }
      if (!ok) give_up(abort_flag, P.status, 4, 23);
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer
    // Two positions in the tile stream: `q*` for the next Q K^T (three tiles ahead) and `p*` for the next P V.
    // Q K^T of tile T+3 overwrites the columns P V of tile T reads its A operand from: MMAs issued by one thread
    // execute in issue order, so issuing it after that P V is all the protection needed.  The first P V of an
    // item overwrites O: the softmax warpgroups have read the previous item's O before they write that tile's P.
    if (lane == 0) {
      bool ok = true;
      int fail_at = 1;
      constexpr uint32_t idesc_qk = ptx::make_idesc(128, 128, false);
      constexpr uint32_t idesc_pv = ptx::make_idesc(128, D, true);
      const uint32_t aQ = ptx::smem_u32(sQ);
      const ptx::DescBase bK0 = ptx::base_kmajor(ptx::smem_u32(sK)), bK1 = ptx::base_kmajor(ptx::smem_u32(sK + kTileBytes));
      const ptx::DescBase bV0 = ptx::base_mnmajor(ptx::smem_u32(sV)), bV1 = ptx::base_mnmajor(ptx::smem_u32(sV + kTileBytes));
      // This thread's instruction count per MMA bounds the whole pipeline, so it does no index arithmetic of its own:
      // the number of tiles of each item comes from the producer through item_tiles (valid once bar_q of the item
      // has completed), and score buffer (T % 3) and barrier phase ((T / 3) & 1) are kept as counters.
      int qT = 0, qn = 0, qqi = 0, qN = 0;  // Q K^T position: stream index, tile inside the item, item index, its tiles
      int pT = 0, pn = 0, pqi = 0, pN = 0;  // P V position
      bool q_end = false;
      uint32_t qsb = 0, psb = 0, psph = 0;
      const ptx::DescBase bQ = ptx::base_kmajor(aQ);
      auto issue_qk = [&]() {  // one tile at the Q K^T position, then advance it
        if (qn == 0) {
          ok = ptx::mbar_wait(&sh->bar_q, qqi & 1);
          if (!ok) { fail_at = 2; return; }
          qN = sh->item_tiles[qqi & 7];
          if (qN < 0) { q_end = true; return; }
        }
        ok = ptx::mbar_wait(&sh->bar_k[qT & 1], (qT >> 1) & 1);
        if (!ok) { fail_at = 3; return; }
        ptx::tc_fence_after();
        const ptx::DescBase bk = (qT & 1) ? bK1 : bK0;
        const uint32_t dS = tmem + qsb * 128u;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          ptx::mma_ss(dS, ptx::desc_at(bQ, ptx::koff_kmajor(kk)), ptx::desc_at(bk, ptx::koff_kmajor(kk)), idesc_qk, kk > 0);
        ptx::mma_commit(&sh->bar_s[qsb]);
        ptx::mma_commit(&sh->bar_kfree[qT & 1]);
        ++qT;
        if (++qsb == kSBufs) qsb = 0;
        if (++qn == qN) {
          ptx::mma_commit(&sh->bar_qfree);
          qn = 0;
          ++qqi;
        }
      };
      for (int t = 0; t < kSBufs && ok && !q_end; ++t) issue_qk();
      while (ok && pT < qT) {  // every tile whose Q K^T has been issued gets its P V
        if (pn == 0) pN = sh->item_tiles[pqi & 7];  // written before the Q K^T position passed this item
        ok = ptx::mbar_wait(&sh->bar_p[psb], psph);
        if (!ok) { fail_at = 4; break; }
        ok = ptx::mbar_wait(&sh->bar_v[pT & 1], (pT >> 1) & 1);
        if (!ok) { fail_at = 5; break; }
        ptx::tc_fence_after();
        const ptx::DescBase bv = (pT & 1) ? bV1 : bV0;
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk)
          ptx::mma_ts(tmem + kColO, tmem + psb * 128u + kk * 8, ptx::desc_at(bv, ptx::koff_mnmajor(kk)), idesc_pv,
                      (pn > 0) || (kk > 0));
        ptx::mma_commit(&sh->bar_pv[psb]);
        ++pT;
        if (++psb == kSBufs) { psb = 0; psph ^= 1u; }
        if (++pn == pN) {
          pn = 0;
          ++pqi;
        }
        if (!q_end) issue_qk();
      }
      if (!ok) give_up(abort_flag, P.status, 4, fail_at);
    }
  } else {
    // ------------------------------------------------------------------ softmax warpgroups
    const int row = tid & 127;
    const int half = tid >> 7;
    const int c_base = half * kHalf;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const float c2 = P.sm_scale * kLog2e;
    const float capl2 = P.cap * kLog2e;
    const float csc = (SK == FLEXATTN_SCORE_SOFTCAP) ? P.sm_scale / P.cap : 0.f;
    bool ok = true;
    int fail_at = 0;
    int T = 0;  // stream index of the next kv tile
    bool o_pending = false;  // thread 0: a bulk store out of the staging tile has been issued and not yet waited for
    int sb = 0;          // T % 3: score buffer of that tile
    uint32_t sph = 0;    // (T / 3) & 1: phase of its barriers

    for (ItemCursor it(P); it.valid(); it.next()) {
      const int qt = it.qt(), bh = it.bh(), b = bh / P.heads, h = bh % P.heads;
      const int4 rm = it.rm;
      const int N = rm.y - rm.x;
      const int i = qt * kTile + row;
      const long long n_rows = (long long)P.batch * P.heads * P.seq_q, n_doc = (long long)P.batch * P.doc_stride;
      const float slope2 = (SK == FLEXATTN_SCORE_ALIBI && FLEXATTN_DBG_OK(h, P.heads, 4, 101)) ? P.alibi_slopes[h] * kLog2e : 0.f;
      const int32_t* doc = (MK == FLEXATTN_MASK_DOCUMENT) ? P.doc_ids + (size_t)b * P.doc_stride : nullptr;
      const int di = (MK == FLEXATTN_MASK_DOCUMENT && i < P.seq_q && FLEXATTN_DBG_OK((long long)b * P.doc_stride + i, n_doc, 4, 102))
                         ? doc[i] : 0;
      // the interval [klo, khi) of keys this row keeps, where the mask has one: the interval kinds, and a document
      // mask when the ids of the batch row never decrease (then the mask map holds the start of every row's document)
      constexpr bool kDoc = MK == FLEXATTN_MASK_DOCUMENT;  // (for other kinds the run form below is the default form)
      bool doc_runs = false;
      int klo = 0, khi = P.seq_k;
      if constexpr (kMaskIsInterval<MK>) row_key_interval<MK>(i, P.seq_k, P.window, klo, khi);
      if constexpr (MK == FLEXATTN_MASK_DOCUMENT) {
        doc_runs = FLEXATTN_DBG_OK(b, P.batch, 4, 107) && P.doc_sorted[b] != 0;
        if (doc_runs && i < P.seq_q && FLEXATTN_DBG_OK((long long)b * P.doc_stride + i, n_doc, 4, 108)) {
          klo = P.run_lo[(size_t)b * P.doc_stride + i];
          khi = i + 1 < P.seq_k ? i + 1 : P.seq_k;
        }
      }
      float m_ref = kMasked, m_true = kMasked, l = 0.f;  // l: sum over this thread's columns only
      // dense bias of this query row (nullptr: no bias, or a row past the end of the sequence)
      const float* ab_q = (P.ab != nullptr && i < P.seq_q && FLEXATTN_DBG_OK((long long)bh * P.seq_q + i, n_rows, 4, 103))
                              ? P.ab + ((size_t)bh * P.seq_q + i) * P.seq_k : nullptr;
      const ScoreCtx ctx{P.sm_scale, b, h};

      for (int n = 0; n < N; ++n, ++T) {
        const uint32_t par = T & 1;
        const uint32_t colS = (uint32_t)sb * 128u;
        const int kt = kv_tile_at<SK>(rm.x, rm.y, n), j0 = kt * kTile;
        const bool partial = P.ab != nullptr || !(kt >= rm.z && kt < rm.w);
        if (MK == FLEXATTN_MASK_DOCUMENT && partial && !doc_runs && half == 0) {
          const int j = j0 + row;
          sh->doc[par][row] = (j < P.seq_k && FLEXATTN_DBG_OK((long long)b * P.doc_stride + j, n_doc, 4, 104)) ? doc[j] : -1;
        }
        // A failed wait never leaves the loops early: every thread keeps executing the same named barriers so
        // that nobody is left waiting on one (the time-out path must not be able to hang either).
        if (ok) {
          ok = __all_sync(0xffffffffu, ptx::mbar_wait(&sh->bar_s[sb], sph));
          if (!ok) fail_at = 10;
        }
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
        if (MK == FLEXATTN_MASK_DOCUMENT && partial && !doc_runs) ptx::named_bar_sync(2, 256);  // kv-tile document ids visible
        // xs: factor still to be applied to x inside the exp2 argument (the plain-score fast path keeps the raw
        // scores and folds sm_scale*log2e into the FMA that also subtracts the running max)
        float tmax = kMasked, xs = 1.0f;
        if (ok) {
          if (P.ab != nullptr) {
            // with a bias every tile takes the masked form (the mask functor also clips the ragged last tile):
            // the S^2 floats of the bias bound this path, not the arithmetic
            const float* ab_t = ab_q != nullptr ? ab_q + j0 + c_base : nullptr;
            if constexpr (kDoc) {
              if (doc_runs)
                tmax = score_half<SK, MK, true, true, true>(x, i, j0, c_base, P.seq_k, P.window, P.stride, c2, slope2,
                                                            capl2, csc, di, sh->doc[par], ctx, ab_t, klo, khi);
              else
                tmax = score_half<SK, MK, true, true, false>(x, i, j0, c_base, P.seq_k, P.window, P.stride, c2, slope2,
                                                             capl2, csc, di, sh->doc[par], ctx, ab_t);
            } else {
              tmax = score_half<SK, MK, true, true>(x, i, j0, c_base, P.seq_k, P.window, P.stride, c2, slope2, capl2, csc,
                                                    di, sh->doc[par], ctx, ab_t, klo, khi);
            }
          } else if (partial) {
            if constexpr (kDoc) {
              if (doc_runs)
                tmax = score_half<SK, MK, true, false, true>(x, i, j0, c_base, P.seq_k, P.window, P.stride, c2, slope2,
                                                             capl2, csc, di, sh->doc[par], ctx, nullptr, klo, khi);
              else
                tmax = score_half<SK, MK, true, false, false>(x, i, j0, c_base, P.seq_k, P.window, P.stride, c2, slope2,
                                                              capl2, csc, di, sh->doc[par], ctx);
            } else {
              tmax = score_half<SK, MK, true>(x, i, j0, c_base, P.seq_k, P.window, P.stride, c2, slope2, capl2, csc, di,
                                              sh->doc[par], ctx, nullptr, klo, khi);
            }
          } else if constexpr (SK != FLEXATTN_SCORE_NONE) {
            tmax = score_half<SK, MK, false>(x, i, j0, c_base, P.seq_k, P.window, P.stride, c2, slope2, capl2, csc, di,
                                             sh->doc[par], ctx);
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
        if (ok) {
          tmax = fmaxf(tmax, sh->pmax[par][half ^ 1][row]);
          m_true = fmaxf(m_true, tmax);
          const float m_cand = fmaxf(m_ref, tmax);
          if (__any_sync(0xffffffffu, (m_cand - m_ref) > kLazyRescale)) {
            const float alpha = ptx::ex2(m_ref - m_cand);
            l *= alpha;
            m_ref = m_cand;
            if (n > 0) {  // O holds the sum up to the previous tile of this item: wait for that P V, then rescale
              ok = __all_sync(0xffffffffu, ptx::mbar_wait(&sh->bar_pv[sb == 0 ? kSBufs - 1 : sb - 1], sb == 0 ? sph ^ 1u : sph));
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
        if (ok) {
          uint64_t ls2[2] = {0ull, 0ull};  // packed partial sums (four running sums in two registers pairs)
          uint32_t pk[32];
          const float nm = ptx::kRoundLog2 - m_ref;  // pre-scaled by (1 + 2^-9) for pack_bf16_trunc; compensates the truncation
          const uint64_t xs2 = ptx::pack2(xs, xs), nm2 = ptx::pack2(nm, nm);
#pragma unroll
          for (int c = 0; c < kHalf; c += 2) {
            float a0, a1;
            ptx::unpack2(ptx::fma2(ptx::pack2(x[c], x[c + 1]), xs2, nm2), a0, a1);
            const float p0 = ptx::ex2(a0), p1 = ptx::ex2(a1);
            ls2[(c >> 1) & 1] = ptx::add2(ls2[(c >> 1) & 1], ptx::pack2(p0, p1));
            pk[c >> 1] = ptx::pack_bf16_trunc(p0, p1);
          }
          ptx::tmem_st32(lane_base + colS + (c_base >> 1), pk);
          {
            float s0, s1;
            ptx::unpack2(ptx::add2(ls2[0], ls2[1]), s0, s1);
            l += s0 + s1;
          }
          ptx::tmem_wait_st();
          ptx::tc_fence_before();
          ptx::mbar_arrive_warp(&sh->bar_p[sb]);
        }
        if (++sb == kSBufs) { sb = 0; sph ^= 1u; }
      }

      // ---- item epilogue: O / l of the item, read out of tensor memory BEFORE this warpgroup writes the next
      // item's first P (which is what lets the MMA issuer overwrite O)
      if (ok && N > 0) {
        ok = __all_sync(0xffffffffu, ptx::mbar_wait(&sh->bar_pv[sb == 0 ? kSBufs - 1 : sb - 1], sb == 0 ? sph ^ 1u : sph));
        if (!ok) fail_at = 12;
      }
      if (tid == 0 && o_pending) {  // the previous item's store has read the staging tile (long ago, normally)
        ptx::tma_store_wait_read();
        o_pending = false;
      }
      sh->lsum[half][row] = l;
      ptx::named_bar_sync(1, 256);
      l = sh->lsum[0][row] + sh->lsum[1][row];
      ptx::named_bar_sync(3, 256);  // both halves have read lsum before the next item overwrites it
      const float inv_l = l > 0.f ? ptx::kRoundUp / l : 0.f;  // l sums the pre-scaled probabilities
      const size_t grow = (size_t)bh * P.seq_q + i;
      if (N > 0) {
        // O / l as bf16 into the staging tile in the TMA (128-byte swizzle) layout, then one bulk tensor store per
        // 64-column panel; rows past seq_q are clipped by the tensor map.  (Storing from registers, one 256-byte row
        // per thread, touched 32 different lines per instruction and cost 3400 cycles per item.)
        if (ok) {
          ptx::tc_fence_after();
          uint8_t* stage_row = sO + row * 128;
#pragma unroll 1
          for (int c0 = half * (D / 2); c0 < (half + 1) * (D / 2); c0 += 32) {
            uint32_t r[32];
            ptx::tmem_ld32(lane_base + kColO + c0, r);
            ptx::tmem_wait_ld();
            ptx::tmem_ld_acquire(r);
#pragma unroll
            for (int c = 0; c < 32; c += 8) {
              uint4 v4;
              v4.x = ptx::pack_bf16(__uint_as_float(r[c]) * inv_l, __uint_as_float(r[c + 1]) * inv_l);
              v4.y = ptx::pack_bf16(__uint_as_float(r[c + 2]) * inv_l, __uint_as_float(r[c + 3]) * inv_l);
              v4.z = ptx::pack_bf16(__uint_as_float(r[c + 4]) * inv_l, __uint_as_float(r[c + 5]) * inv_l);
              v4.w = ptx::pack_bf16(__uint_as_float(r[c + 6]) * inv_l, __uint_as_float(r[c + 7]) * inv_l);
              const int col = c0 + c, panel = col >> 6, chunk = (col & 63) >> 3;
              *reinterpret_cast<uint4*>(stage_row + panel * ptx::kPanelBytes + ((chunk ^ (row & 7)) << 4)) = v4;
            }
          }
          ptx::tc_fence_before();
          ptx::fence_proxy_async_smem();  // generic-proxy stores -> visible to the bulk store
        }
        ptx::named_bar_sync(2, 256);
        if (ok && tid == 0) {
#pragma unroll
          for (int p = 0; p < kPanels; ++p) ptx::tma_store_3d(&tm_o, sO + p * ptx::kPanelBytes, p * 64, qt * kTile, bh);
          ptx::tma_store_commit();
          o_pending = true;
        }
      } else if (ok && i < P.seq_q && FLEXATTN_DBG_OK(grow, n_rows, 4, 105)) {  // an item without any kv tile: zeros, written directly
        uint16_t* orow = static_cast<uint16_t*>(P.o) + grow * D;   // bf16 elements
        for (int c0 = half * (D / 2); c0 < (half + 1) * (D / 2); c0 += 8)
          *reinterpret_cast<uint4*>(orow + c0) = make_uint4(0u, 0u, 0u, 0u);
      }
      if (ok && half == 0 && i < P.seq_q && FLEXATTN_DBG_OK(grow, n_rows, 4, 106)) {
        P.l[grow] = l * ptx::ex2(m_ref - m_true) * ptx::kRoundInv;
        P.m[grow] = m_true * kLn2;
      }
    }
    if (tid == 0 && o_pending) ptx::tma_store_wait_read();  // the staging tile must outlive the last store's reads
    if (!ok && lane == 0) give_up(abort_flag, P.status, 4, fail_at);
  }

  // ------------------------------------------------------------------ teardown
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, kTmemCols);
  }
}

#ifndef FLEXATTN_JIT
template <int D, int SK, int MK>
int launch_one(cudaStream_t st, const DevParams& d, const CUtensorMap& tq, const CUtensorMap& tk,
               const CUtensorMap& tv, const CUtensorMap& to, int* abort_flag) {
  constexpr size_t need = 6 * (D / 64) * ptx::kPanelBytes + sizeof(PipeSmem) + 1024;
  // 512 TMEM columns per CTA: never let two CTAs share an SM (the second would spin in tcgen05.alloc)
  constexpr size_t smem = need > 120 * 1024 ? need : 120 * 1024;
  auto kern = fwd_pipe_sm100_kernel<D, SK, MK>;
  static SmemAttrOnce attr_once{};  // per kernel instantiation, per device
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), (int)smem, &attr_once) != FLEXATTN_OK) return FLEXATTN_ERR_CUDA;
  // persistent: one CTA per SM (fewer when there are fewer work items)
  const long long items = (long long)d.n_qt * d.batch * d.heads;
  const int sms = sm_count();
  if (sms <= 0) return FLEXATTN_ERR_CUDA;
  dim3 grid((unsigned)(items < sms ? items : sms));
  kern<<<grid, kThreads, smem, st>>>(tq, tk, tv, to, d, abort_flag);
  return cudaGetLastError() == cudaSuccess ? FLEXATTN_OK : FLEXATTN_ERR_CUDA;
}

template <int D, int SK>
int launch_mask(cudaStream_t st, const DevParams& d, int mask, const CUtensorMap& tq, const CUtensorMap& tk,
                const CUtensorMap& tv, const CUtensorMap& to, int* af) {
  switch (mask) {
    case FLEXATTN_MASK_NONE: return launch_one<D, SK, FLEXATTN_MASK_NONE>(st, d, tq, tk, tv, to, af);
    case FLEXATTN_MASK_CAUSAL: return launch_one<D, SK, FLEXATTN_MASK_CAUSAL>(st, d, tq, tk, tv, to, af);
    case FLEXATTN_MASK_SLIDING_WINDOW: return launch_one<D, SK, FLEXATTN_MASK_SLIDING_WINDOW>(st, d, tq, tk, tv, to, af);
    case FLEXATTN_MASK_SLIDING_WINDOW_CAUSAL:
      return launch_one<D, SK, FLEXATTN_MASK_SLIDING_WINDOW_CAUSAL>(st, d, tq, tk, tv, to, af);
    case FLEXATTN_MASK_DOCUMENT: return launch_one<D, SK, FLEXATTN_MASK_DOCUMENT>(st, d, tq, tk, tv, to, af);
    case FLEXATTN_MASK_S2: return launch_one<D, SK, FLEXATTN_MASK_S2>(st, d, tq, tk, tv, to, af);
    default: return FLEXATTN_ERR_UNSUPPORTED_MOD;
  }
}

template <int D>
int launch_score(cudaStream_t st, const DevParams& d, int score, int mask, const CUtensorMap& tq,
                 const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& to, int* af) {
  switch (score) {
    case FLEXATTN_SCORE_NONE: return launch_mask<D, FLEXATTN_SCORE_NONE>(st, d, mask, tq, tk, tv, to, af);
    case FLEXATTN_SCORE_ALIBI: return launch_mask<D, FLEXATTN_SCORE_ALIBI>(st, d, mask, tq, tk, tv, to, af);
    case FLEXATTN_SCORE_SOFTCAP: return launch_mask<D, FLEXATTN_SCORE_SOFTCAP>(st, d, mask, tq, tk, tv, to, af);
    default: return FLEXATTN_ERR_UNSUPPORTED_MOD;
  }
}

#endif  // !FLEXATTN_JIT

}  // namespace FLEXATTN_TU_NAMESPACE

#ifndef FLEXATTN_JIT
int launch_sm100_fwd_pipe(cudaStream_t st, const DevParams& d, int score, int mask) {
  int* af = abort_flag_ptr();
  if (af == nullptr) return FLEXATTN_ERR_CUDA;
  CUtensorMap tq, tk, tv, to;
  const int slices = d.batch * d.heads;
  int e = make_tile_map(&tq, d.q, slices, d.seq_q, d.head_dim);
  if (e) return e;
  e = make_tile_map(&tk, d.k, slices, d.seq_k, d.head_dim);
  if (e) return e;
  e = make_tile_map(&tv, d.v, slices, d.seq_k, d.head_dim);
  if (e) return e;
  e = make_tile_map(&to, d.o, slices, d.seq_q, d.head_dim);
  if (e) return e;
  if (score == FLEXATTN_SCORE_USER) {
    // a kernel compiled at run time around the registered score function: same parameters, grid and shared memory
    const size_t need = 6 * (size_t)(d.head_dim / 64) * ptx::kPanelBytes + sizeof(PipeSmem) + 1024;
    const long long items = (long long)d.n_qt * d.batch * d.heads;
    const int sms = sm_count();
    if (sms <= 0) return FLEXATTN_ERR_CUDA;
    void* args[] = {&tq, &tk, &tv, &to, const_cast<DevParams*>(&d), &af};
    return jit_launch(0, d.user_score, d.head_dim, mask, (unsigned)(items < sms ? items : sms), 1, kThreads,
                      need > 120 * 1024 ? need : 120 * 1024, st, args);
  }
  if (d.head_dim == 128) return launch_score<128>(st, d, score, mask, tq, tk, tv, to, af);
  if (d.head_dim == 64) return launch_score<64>(st, d, score, mask, tq, tk, tv, to, af);
  return FLEXATTN_ERR_UNSUPPORTED_HEAD_DIM;
}
#endif  // !FLEXATTN_JIT

}  // namespace flexattn
