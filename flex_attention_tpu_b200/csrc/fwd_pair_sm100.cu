// Forward flex attention for long rows, two query tiles per CTA (sm_100a).
//
// Same math and interface as fwd_pipe_sm100.cu (reference: flex_attention_kernel.py:196-327).  A CTA owns two
// adjacent 128-row query tiles of one (batch, head) and runs them as two independent online-softmax streams over the
// SAME K/V tiles, half a period apart: while stream A's warpgroup computes the exponentials of kv tile n, the tensor
// core runs stream B's P V and Q K^T, and the other way round.  In a stream thread t owns query row t (= TMEM lane
// t) and all 128 score columns of it, so a row maximum or sum needs no exchange between threads and there is no
// per-tile barrier between warpgroups; K and V are loaded once for both tiles.
//
//   warps 0..3 / 4..7 : softmax of stream A / B (registers raised to 208 per thread).
//   warp 8, lane 0    : MMA issuer of both streams: O_s += P_s V, then S_s = Q_s K_next^T over the columns P_s
//                       occupied (MMAs of one thread execute in issue order).
//   warp 9, lane 0    : TMA producer: Q_A, Q_B once, K and V through two-stage rings.
//   warps 10, 11      : idle (they complete the warpgroup whose registers are lowered to 88).
//
// Tensor memory: S_A, S_B, O_A, O_B = 4 x 128 columns.  Shared memory: Q_A, Q_B (reused to stage the outputs),
// 2 K, 2 V tiles (192 KB for D = 128).  Not persistent: one CTA per pair of query tiles, heaviest pairs first.
#include "sm100.cuh"

namespace flexattn {
namespace FLEXATTN_TU_NAMESPACE {

constexpr int kThreads = 384;
constexpr int kMmaWarp = 8, kTmaWarp = 9;
constexpr float kLazyRescale = 8.0f;  // log2 units

struct PairSmem {
  uint64_t bar_q[2], bar_k[2], bar_v[2], bar_kfree[2], bar_vfree[2], bar_s[2], bar_p[2], bar_pv[2];
  uint32_t tmem_base;
  int32_t doc[2][kTile];  // per stream: document ids of the kv tile being processed
};

// kv tile visited at step n of the range [first, end): from the last one down under ALiBi (the bias grows with the
// key position, so the running maximum is met first and the lazy rescale almost never fires), ascending otherwise.
template <int SK>
__device__ __forceinline__ int kv_tile_at(int first, int end, int n) {
  return SK == FLEXATTN_SCORE_ALIBI ? end - 1 - n : first + n;
}

// what a user score function sees besides the score and the positions
struct ScoreCtx {
  float sm_scale;
  int b, h;
};

// x: this thread's 128 raw scores of one tile -> log2-domain logits in place; returns their maximum.
// kInterval: the row's kept keys are the interval [klo, khi) (interval mask kinds; documents over sorted ids): a
// partial tile then tests one bit per element of a bitmap built once per 32 columns.
template <int SK, int MK, bool kPartial, bool kInterval = kMaskIsInterval<MK>>
__device__ __forceinline__ float score_row(float (&x)[kTile], int i, int j0, int seq_k, int window, int stride,
                                           float c2, float slope2, float capl2, float csc, int di,
                                           const int32_t* s_doc, const ScoreCtx ctx, int klo = 0, int khi = 0) {
  float mx[4] = {kMasked, kMasked, kMasked, kMasked};
  uint32_t keep = 0u;  // kept columns of the current group of 32 (kInterval on partial tiles)
  if constexpr (SK == FLEXATTN_SCORE_SOFTCAP || SK == FLEXATTN_SCORE_USER) {
#pragma unroll
    for (int c = 0; c < kTile; ++c) {
      float t;
      if constexpr (SK == FLEXATTN_SCORE_USER) t = user_score(x[c] * ctx.sm_scale, ctx.b, ctx.h, i, j0 + c) * kLog2e;
      else t = capl2 * ptx::tanh_approx(x[c] * csc);
      if constexpr (kPartial && kInterval) {
        if ((c & 31) == 0) keep = range_bits32(klo - (j0 + c), khi - (j0 + c));
        t = (keep >> (c & 31)) & 1u ? t : kMasked;
      } else if constexpr (kPartial) {
        const int j = j0 + c;
        const int dj = (MK == FLEXATTN_MASK_DOCUMENT) ? s_doc[c] : 0;
        t = ((j < seq_k) && mask_keep<MK>(i, j, window, stride, di, dj)) ? t : kMasked;
      }
      x[c] = t;
      mx[c & 3] = fmaxf(mx[c & 3], t);
    }
  } else {
    const float abase = slope2 * (float)(j0 - i);
    uint64_t b2 = ptx::pack2(abase, abase + slope2);
    const uint64_t bstep2 = ptx::pack2(2.f * slope2, 2.f * slope2);
#pragma unroll
    for (int c = 0; c < kTile; c += 2) {
      const uint64_t x2 = ptx::pack2(x[c], x[c + 1]);
      float t0, t1;
      if constexpr (SK == FLEXATTN_SCORE_ALIBI) {
        ptx::unpack2(ptx::fma2(x2, ptx::pack2(c2, c2), b2), t0, t1);
        b2 = ptx::add2(b2, bstep2);
      } else {
        ptx::unpack2(ptx::mul2(x2, ptx::pack2(c2, c2)), t0, t1);
      }
      if constexpr (kPartial && kInterval) {  // one bitmap per row and 32 columns instead of per-element tests
        if ((c & 31) == 0) keep = range_bits32(klo - (j0 + c), khi - (j0 + c));
        t0 = (keep >> (c & 31)) & 1u ? t0 : kMasked;
        t1 = (keep >> ((c & 31) + 1)) & 1u ? t1 : kMasked;
      } else if constexpr (kPartial) {
        const int j = j0 + c;
        const int d0 = (MK == FLEXATTN_MASK_DOCUMENT) ? s_doc[c] : 0;
        const int d1 = (MK == FLEXATTN_MASK_DOCUMENT) ? s_doc[c + 1] : 0;
        t0 = ((j < seq_k) && mask_keep<MK>(i, j, window, stride, di, d0)) ? t0 : kMasked;
        t1 = ((j + 1 < seq_k) && mask_keep<MK>(i, j + 1, window, stride, di, d1)) ? t1 : kMasked;
      }
      x[c] = t0;
      x[c + 1] = t1;
      mx[(c >> 1) & 3] = ptx::max3(mx[(c >> 1) & 3], t0, t1);
    }
  }
  return fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
}

template <int D, int SK, int MK>
__global__ void __launch_bounds__(kThreads, 1)
    fwd_pair_sm100_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                          const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                          const DevParams P, int* abort_flag) {
  constexpr int kPanels = D / 64;
  constexpr uint32_t kTileBytes = kPanels * ptx::kPanelBytes;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kColS = 0, kColO = 256;  // stream s: S at kColS + 128 s, O at kColO + 128 s

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                   // Q_A, Q_B; each becomes the output staging tile of its stream
  uint8_t* sK = smem + 2 * kTileBytes;  // two stages
  uint8_t* sV = smem + 4 * kTileBytes;  // two stages
  PairSmem* sh = reinterpret_cast<PairSmem*>(smem + 6 * kTileBytes);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int pair = (int)gridDim.x - 1 - (int)blockIdx.x;  // late query tiles see the most keys under a causal mask: first
  const int bh = blockIdx.y, b = bh / P.heads, h = bh % P.heads;

  // The two streams' kv ranges; the K/V rings walk their union [first, end), a stream takes part in the tiles of its
  // own range.
  const size_t map_row = (size_t)(P.map_rows > 1 ? b : 0) * P.n_qt;
  const int4 rm0 = P.row_map[map_row + 2 * pair];
  const int4 rm1 = 2 * pair + 1 < P.n_qt ? P.row_map[map_row + 2 * pair + 1] : make_int4(0, 0, 0, 0);
  const bool any0 = rm0.y > rm0.x, any1 = rm1.y > rm1.x;
  const int first = any0 && any1 ? min(rm0.x, rm1.x) : (any0 ? rm0.x : rm1.x);
  const int end = any0 && any1 ? max(rm0.y, rm1.y) : (any0 ? rm0.y : rm1.y);
  const int NT = end - first;  // 0 when neither tile has keys
  // (no arrays indexed by the stream: they would live in local memory)

  if (aborted_on_entry(abort_flag, P.status, 5)) return;

  if (tid == 0) {
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(&sh->bar_q[s], 1);
      ptx::mbar_init(&sh->bar_k[s], 1);
      ptx::mbar_init(&sh->bar_v[s], 1);
      ptx::mbar_init(&sh->bar_kfree[s], 1);
      ptx::mbar_init(&sh->bar_vfree[s], 1);
      ptx::mbar_init(&sh->bar_s[s], 1);
      ptx::mbar_init(&sh->bar_p[s], 4);  // one arrival per warp of the stream's warpgroup
      ptx::mbar_init(&sh->bar_pv[s], 1);
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

  if (warp >= 8) {
    ptx::setmaxnreg_dec<88>();
    if (warp == kTmaWarp) {
      // ---------------------------------------------------------------- TMA producer
      if (lane == 0 && NT > 0) {
        bool ok = true;
        ptx::prefetch_tensormap(&tm_q);
        ptx::prefetch_tensormap(&tm_k);
        ptx::prefetch_tensormap(&tm_v);
        auto load_kv = [&](uint8_t* ring, const CUtensorMap* tm, uint64_t* bars, int T) {
          uint8_t* dst = ring + (T & 1) * kTileBytes;
          ptx::mbar_arrive_expect_tx(&bars[T & 1], kTileBytes);
#pragma unroll
          for (int p = 0; p < kPanels; ++p)
            ptx::tma_load_3d(dst + p * ptx::kPanelBytes, tm, &bars[T & 1], p * 64, kv_tile_at<SK>(first, end, T) * kTile, bh);
        };
        // order of first use: Q_A, K(0), Q_B, V(0), K(1), V(1)
        auto load_q = [&](int s) {
          if (s ? any1 : any0) {
            ptx::mbar_arrive_expect_tx(&sh->bar_q[s], kTileBytes);
#pragma unroll
            for (int p = 0; p < kPanels; ++p)
              ptx::tma_load_3d(sQ + s * kTileBytes + p * ptx::kPanelBytes, &tm_q, &sh->bar_q[s], p * 64, (2 * pair + s) * kTile, bh);
          }
        };
        load_q(0);
        load_kv(sK, &tm_k, sh->bar_k, 0);
        load_q(1);
        load_kv(sV, &tm_v, sh->bar_v, 0);
        if (NT > 1) {
          load_kv(sK, &tm_k, sh->bar_k, 1);
          load_kv(sV, &tm_v, sh->bar_v, 1);
        }
        for (int T = 2; T < NT && ok; ++T) {
          const uint32_t par = ((T - 2) >> 1) & 1;
          ok = ptx::mbar_wait_relaxed(&sh->bar_kfree[T & 1], par);  // every Q K^T of tile T-2 has completed
          if (!ok) break;
          load_kv(sK, &tm_k, sh->bar_k, T);
          ok = ptx::mbar_wait_relaxed(&sh->bar_vfree[T & 1], par);  // every P V of tile T-2 has completed
          if (!ok) break;
          load_kv(sV, &tm_v, sh->bar_v, T);
        }
        if (!ok) give_up(abort_flag, P.status, 5, 20);
      }
    } else if (warp == kMmaWarp) {
      // ---------------------------------------------------------------- MMA issuer of both streams.
      // This thread's instruction stream bounds the kernel (about 70 cycles per tcgen05.mma against 64 cycles of
      // tensor work, plus every barrier wait and commit around them), so it waits once per tile for K and V, not
      // once per stream, and commits "P V done" only for a stream's last tile, the only one anybody waits for.
      // (A second issuing thread, one per stream, was measured 13 % slower.)
      if (lane == 0 && NT > 0) {
        bool ok = true;
        int fail_at = 1;
        constexpr uint32_t idesc_qk = ptx::make_idesc(128, 128, false);
        constexpr uint32_t idesc_pv = ptx::make_idesc(128, D, true);
        const ptx::DescBase bQ0 = ptx::base_kmajor(ptx::smem_u32(sQ)), bQ1 = ptx::base_kmajor(ptx::smem_u32(sQ + kTileBytes));
        const ptx::DescBase bK0 = ptx::base_kmajor(ptx::smem_u32(sK)), bK1 = ptx::base_kmajor(ptx::smem_u32(sK + kTileBytes));
        const ptx::DescBase bV0 = ptx::base_mnmajor(ptx::smem_u32(sV)), bV1 = ptx::base_mnmajor(ptx::smem_u32(sV + kTileBytes));
        const int n0 = rm0.y - rm0.x, n1 = rm1.y - rm1.x;
        int done0 = 0, done1 = 0;  // tiles of each stream whose P V has been issued (= tiles whose Q K^T was, minus one)
        auto issue_qk = [&](int s, const ptx::DescBase& bk) {  // S_s = Q_s K^T; K has landed
          const uint32_t dS = tmem + kColS + (uint32_t)s * 128u;
          const ptx::DescBase bq = s ? bQ1 : bQ0;
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk)
            ptx::mma_ss(dS, ptx::desc_at(bq, ptx::koff_kmajor(kk)), ptx::desc_at(bk, ptx::koff_kmajor(kk)), idesc_qk, kk > 0);
          ptx::mma_commit(&sh->bar_s[s]);
        };
        auto issue_pv = [&](int s, const ptx::DescBase& bv) {  // O_s += P_s V; V has landed
          const int done = s ? done1 : done0;
          ok = ptx::mbar_wait(&sh->bar_p[s], done & 1);
          if (!ok) { fail_at = 4; return; }
          ptx::tc_fence_after();
          const uint32_t dS = tmem + kColS + (uint32_t)s * 128u;
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk)
            ptx::mma_ts(tmem + kColO + (uint32_t)s * 128u, dS + kk * 8, ptx::desc_at(bv, ptx::koff_mnmajor(kk)), idesc_pv,
                        (done > 0) || (kk > 0));
          if (done + 1 == (s ? n1 : n0)) ptx::mma_commit(&sh->bar_pv[s]);  // the stream's last tile
          if (s) ++done1; else ++done0;
        };
        auto in0 = [&](int kt) { return kt >= rm0.x && kt < rm0.y; };
        auto in1 = [&](int kt) { return kt >= rm1.x && kt < rm1.y; };
        {  // first scores
          const int kt0 = kv_tile_at<SK>(first, end, 0);
          if (in0(kt0)) ok = ptx::mbar_wait(&sh->bar_q[0], 0);
          if (ok && in1(kt0)) ok = ptx::mbar_wait(&sh->bar_q[1], 0);
          if (ok) ok = ptx::mbar_wait(&sh->bar_k[0], 0);
          if (!ok) fail_at = 2;
          if (ok) {
            ptx::tc_fence_after();
            if (in0(kt0)) issue_qk(0, bK0);
            if (in1(kt0)) issue_qk(1, bK0);
            ptx::mma_commit(&sh->bar_kfree[0]);
          }
        }
        for (int T = 0; T < NT && ok; ++T) {
          const int kt = kv_tile_at<SK>(first, end, T);
          const int kt_next = T + 1 < NT ? kv_tile_at<SK>(first, end, T + 1) : -1;
          const bool a0 = in0(kt), a1 = in1(kt);
          const bool q0 = kt_next >= 0 && in0(kt_next), q1 = kt_next >= 0 && in1(kt_next);
          const ptx::DescBase bv = (T & 1) ? bV1 : bV0, bk = (T & 1) ? bK0 : bK1;  // V(T), K(T+1)
          ok = ptx::mbar_wait(&sh->bar_v[T & 1], (T >> 1) & 1);
          if (!ok) { fail_at = 5; break; }
          if (kt_next >= 0) {
            // K(T+1) was requested a whole tile ago: waiting for it here, once, costs nothing and saves a wait
            // between the two streams
            if (q0 && done0 == 0 && !a0) ok = ptx::mbar_wait(&sh->bar_q[0], 0);  // a stream that starts late
            if (ok && q1 && done1 == 0 && !a1) ok = ptx::mbar_wait(&sh->bar_q[1], 0);
            if (ok) ok = ptx::mbar_wait(&sh->bar_k[(T + 1) & 1], ((T + 1) >> 1) & 1);
            if (!ok) { fail_at = 3; break; }
          }
          if (a0) issue_pv(0, bv);
          if (!ok) break;
          if (q0) issue_qk(0, bk);
          if (a1) issue_pv(1, bv);
          if (!ok) break;
          if (q1) issue_qk(1, bk);
          // both streams' MMAs on V(T) and K(T+1) have been issued: their completion frees the ring stages
          ptx::mma_commit(&sh->bar_vfree[T & 1]);
          if (kt_next >= 0) ptx::mma_commit(&sh->bar_kfree[(T + 1) & 1]);
        }
        if (!ok) give_up(abort_flag, P.status, 5, fail_at);
      }
    }
  } else {
    ptx::setmaxnreg_inc<208>();
    // ------------------------------------------------------------------ softmax: warpgroup s = stream s
    const int row = tid & 127;
    const int s = tid >> 7;
    const int qt = 2 * pair + s;
    const int i = qt * kTile + row;
    const int4 rms = s ? rm1 : rm0;
    const int N = rms.y - rms.x;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t colS = kColS + (uint32_t)s * 128u, colO = kColO + (uint32_t)s * 128u;
    const float c2 = P.sm_scale * kLog2e;
    const long long n_rows = (long long)P.batch * P.heads * P.seq_q, n_doc = (long long)P.batch * P.doc_stride;
    const float slope2 = (SK == FLEXATTN_SCORE_ALIBI && FLEXATTN_DBG_OK(h, P.heads, 5, 501)) ? P.alibi_slopes[h] * kLog2e : 0.f;
    const float capl2 = P.cap * kLog2e;
    const float csc = (SK == FLEXATTN_SCORE_SOFTCAP) ? P.sm_scale / P.cap : 0.f;
    const int32_t* doc = (MK == FLEXATTN_MASK_DOCUMENT) ? P.doc_ids + (size_t)b * P.doc_stride : nullptr;
    const int di = (MK == FLEXATTN_MASK_DOCUMENT && qt < P.n_qt && i < P.seq_q &&
                    FLEXATTN_DBG_OK((long long)b * P.doc_stride + i, n_doc, 5, 502)) ? doc[i] : 0;
    float m_ref = kMasked, m_true = kMasked, l = 0.f;
    const ScoreCtx ctx{P.sm_scale, b, h};
    // the interval [klo, khi) of keys this row keeps, where the mask has one: the interval kinds, and a document mask
    // when the ids of the batch row never decrease (then the mask map holds the start of every row's document)
    constexpr bool kDoc = MK == FLEXATTN_MASK_DOCUMENT;
    bool doc_runs = false;
    int klo = 0, khi = P.seq_k;
    if constexpr (kMaskIsInterval<MK>) row_key_interval<MK>(i, P.seq_k, P.window, klo, khi);
    if constexpr (kDoc) {
      doc_runs = FLEXATTN_DBG_OK(b, P.batch, 5, 506) && P.doc_sorted[b] != 0;
      if (doc_runs && qt < P.n_qt && i < P.seq_q && FLEXATTN_DBG_OK((long long)b * P.doc_stride + i, n_doc, 5, 507)) {
        klo = P.run_lo[(size_t)b * P.doc_stride + i];
        khi = i + 1 < P.seq_k ? i + 1 : P.seq_k;
      }
    }
    bool ok = true;
    int fail_at = 0;

    for (int n = 0; n < N; ++n) {
      const uint32_t par = n & 1;
      const int kt = kv_tile_at<SK>(rms.x, rms.y, n), j0 = kt * kTile;
      const bool partial = !(kt >= rms.z && kt < rms.w);
      if (MK == FLEXATTN_MASK_DOCUMENT && partial && !doc_runs) {
        // one buffer per stream: readers of the previous partial tile are done (first barrier) before the ids of
        // this tile are written; the second barrier publishes them
        ptx::named_bar_sync(1 + s, 128);
        const int j = j0 + row;
        sh->doc[s][row] = (j < P.seq_k && FLEXATTN_DBG_OK((long long)b * P.doc_stride + j, n_doc, 5, 503)) ? doc[j] : -1;
        ptx::named_bar_sync(1 + s, 128);
      }
      // a failed wait never leaves the loop early: every thread keeps executing the same named barriers
      if (ok) {
        ok = __all_sync(0xffffffffu, ptx::mbar_wait(&sh->bar_s[s], par));
        if (!ok) fail_at = 10;
      }
      if (!ok) continue;
      ptx::tc_fence_after();
      float x[kTile];
      {
        uint32_t xr[4][32];
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) ptx::tmem_ld32(lane_base + colS + q4 * 32, xr[q4]);
        ptx::tmem_wait_ld();
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          ptx::tmem_ld_acquire(xr[q4]);
#pragma unroll
          for (int c = 0; c < 32; ++c) x[q4 * 32 + c] = __uint_as_float(xr[q4][c]);
        }
      }
      // xs: factor still to be applied to x inside the exp2 argument (the plain-score fast path keeps the raw
      // scores and folds sm_scale*log2e into the FMA that also subtracts the running max)
      float tmax, xs = 1.0f;
      if (partial) {
        if constexpr (kDoc) {
          if (doc_runs)
            tmax = score_row<SK, MK, true, true>(x, i, j0, P.seq_k, P.window, P.stride, c2, slope2, capl2, csc, di, sh->doc[s],
                                                 ctx, klo, khi);
          else
            tmax = score_row<SK, MK, true, false>(x, i, j0, P.seq_k, P.window, P.stride, c2, slope2, capl2, csc, di,
                                                  sh->doc[s], ctx);
        } else {
          tmax = score_row<SK, MK, true>(x, i, j0, P.seq_k, P.window, P.stride, c2, slope2, capl2, csc, di, sh->doc[s], ctx,
                                         klo, khi);
        }
      } else if constexpr (SK != FLEXATTN_SCORE_NONE) {
        tmax = score_row<SK, MK, false>(x, i, j0, P.seq_k, P.window, P.stride, c2, slope2, capl2, csc, di, sh->doc[s], ctx);
      } else {
        float mx[4] = {x[0], x[1], x[2], x[3]};
#pragma unroll
        for (int c = 4; c + 7 < kTile; c += 8) {
          mx[0] = ptx::max3(mx[0], x[c], x[c + 1]);
          mx[1] = ptx::max3(mx[1], x[c + 2], x[c + 3]);
          mx[2] = ptx::max3(mx[2], x[c + 4], x[c + 5]);
          mx[3] = ptx::max3(mx[3], x[c + 6], x[c + 7]);
        }
        mx[0] = ptx::max3(mx[0], x[kTile - 4], x[kTile - 3]);
        mx[1] = ptx::max3(mx[1], x[kTile - 2], x[kTile - 1]);
        tmax = ptx::max3(mx[0], mx[1], fmaxf(mx[2], mx[3])) * c2;  // c2 > 0: scaling commutes with max
        xs = c2;
      }
      m_true = fmaxf(m_true, tmax);
      const float m_cand = fmaxf(m_ref, tmax);
      if (__any_sync(0xffffffffu, (m_cand - m_ref) > kLazyRescale)) {
        const float alpha = ptx::ex2(m_ref - m_cand);
        l *= alpha;
        m_ref = m_cand;
        if (n > 0) {
          // O_s holds the tiles up to n-1: their P V completed before Q K^T of tile n was issued (same thread,
          // issue order), and S(n) has been read, so it is complete
#pragma unroll 1
          for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t r[32];
            ptx::tmem_ld32(lane_base + colO + c0, r);
            ptx::tmem_wait_ld();
            ptx::tmem_ld_acquire(r);
#pragma unroll
            for (int c = 0; c < 32; ++c) r[c] = __float_as_uint(__uint_as_float(r[c]) * alpha);
            ptx::tmem_st32(lane_base + colO + c0, r);
          }
          ptx::tmem_wait_st();
        }
      }
      {
        uint64_t ls2[2] = {0ull, 0ull};
        const float nm = ptx::kRoundLog2 - m_ref;  // pre-scaled by (1 + 2^-9) for pack_bf16_trunc
        const uint64_t xs2 = ptx::pack2(xs, xs), nm2 = ptx::pack2(nm, nm);
#pragma unroll
        for (int c0 = 0; c0 < kTile; c0 += 64) {
          uint32_t pk[32];
#pragma unroll
          for (int c = 0; c < 64; c += 2) {
            float a0, a1;
            ptx::unpack2(ptx::fma2(ptx::pack2(x[c0 + c], x[c0 + c + 1]), xs2, nm2), a0, a1);
            const float p0 = ptx::ex2(a0), p1 = ptx::ex2(a1);
            ls2[(c >> 1) & 1] = ptx::add2(ls2[(c >> 1) & 1], ptx::pack2(p0, p1));
            pk[c >> 1] = ptx::pack_bf16_trunc(p0, p1);
          }
          ptx::tmem_st32(lane_base + colS + (c0 >> 1), pk);
        }
        float s0, s1;
        ptx::unpack2(ptx::add2(ls2[0], ls2[1]), s0, s1);
        l += s0 + s1;
      }
      ptx::tmem_wait_st();
      ptx::tc_fence_before();
      ptx::mbar_arrive_warp(&sh->bar_p[s]);
    }

    // ---- epilogue of the stream
    if (qt < P.n_qt) {
      if (ok && N > 0) {
        ok = __all_sync(0xffffffffu, ptx::mbar_wait(&sh->bar_pv[s], 0));  // committed once, after the last P V
        if (!ok) fail_at = 12;
      }
      const float inv_l = l > 0.f ? ptx::kRoundUp / l : 0.f;  // l sums the pre-scaled probabilities
      const size_t grow = (size_t)bh * P.seq_q + i;
      if (N > 0) {
        // bf16 O / l into the stream's Q tile (every Q K^T has completed) in the TMA (128-byte swizzle) layout, then
        // one bulk tensor store per 64-column panel; rows past seq_q are clipped by the tensor map
        uint8_t* stage = sQ + s * kTileBytes;
        if (ok) {
          ptx::tc_fence_after();
          uint8_t* stage_row = stage + row * 128;
#pragma unroll 1
          for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t r[32];
            ptx::tmem_ld32(lane_base + colO + c0, r);
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
          ptx::fence_proxy_async_smem();  // generic-proxy stores -> visible to the bulk store
        }
        ptx::named_bar_sync(1 + s, 128);
        if (ok && row == 0) {
#pragma unroll
          for (int p = 0; p < kPanels; ++p) ptx::tma_store_3d(&tm_o, stage + p * ptx::kPanelBytes, p * 64, qt * kTile, bh);
          ptx::tma_store_commit();
          ptx::tma_store_wait_read();  // shared memory must stay intact until the store has read it
        }
      } else if (i < P.seq_q && FLEXATTN_DBG_OK(grow, n_rows, 5, 504)) {  // a query tile without any kv tile: zeros, written directly
        uint16_t* orow = static_cast<uint16_t*>(P.o) + grow * D;  // bf16 elements
        for (int c0 = 0; c0 < D; c0 += 8) *reinterpret_cast<uint4*>(orow + c0) = make_uint4(0u, 0u, 0u, 0u);
      }
      if (ok && i < P.seq_q && FLEXATTN_DBG_OK(grow, n_rows, 5, 505)) {
        P.l[grow] = l * ptx::ex2(m_ref - m_true) * ptx::kRoundInv;
        P.m[grow] = m_true * kLn2;
      }
    }
    if (!ok && lane == 0) give_up(abort_flag, P.status, 5, fail_at);
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
  constexpr size_t need = 6 * (D / 64) * ptx::kPanelBytes + sizeof(PairSmem) + 1024;
  // 512 TMEM columns per CTA: never let two CTAs share an SM (the second would spin in tcgen05.alloc)
  constexpr size_t smem = need > 120 * 1024 ? need : 120 * 1024;
  auto kern = fwd_pair_sm100_kernel<D, SK, MK>;
  static SmemAttrOnce attr_once{};  // per kernel instantiation, per device
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), (int)smem, &attr_once) != FLEXATTN_OK) return FLEXATTN_ERR_CUDA;
  dim3 grid((d.n_qt + 1) / 2, d.batch * d.heads);
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
// No dense bias here; the caller keeps the persistent kernel for that.
int launch_sm100_fwd_pair(cudaStream_t st, const DevParams& d, int score, int mask) {
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
    const size_t need = 6 * (size_t)(d.head_dim / 64) * ptx::kPanelBytes + sizeof(PairSmem) + 1024;
    void* args[] = {&tq, &tk, &tv, &to, const_cast<DevParams*>(&d), &af};
    return jit_launch(3, d.user_score, d.head_dim, mask, (unsigned)((d.n_qt + 1) / 2), (unsigned)(d.batch * d.heads), kThreads,
                      need > 120 * 1024 ? need : 120 * 1024, st, args);
  }
  if (d.head_dim == 128) return launch_score<128>(st, d, score, mask, tq, tk, tv, to, af);
  if (d.head_dim == 64) return launch_score<64>(st, d, score, mask, tq, tk, tv, to, af);
  return FLEXATTN_ERR_UNSUPPORTED_HEAD_DIM;
}
#endif  // !FLEXATTN_JIT

}  // namespace flexattn
