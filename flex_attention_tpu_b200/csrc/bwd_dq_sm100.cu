// dQ backward on the 5th-generation tensor cores (sm_100a), persistent.
//
// Replaces the reference's Pallas dQ kernel (flex_attention_dq_bwd.py:282-385).  One CTA per SM walks a list of
// work items (128-row query tile, batch*head), in the order and dealing of the persistent forward.  Per item Q
// and dO are copied once into tensor memory as A operands; K/V tiles stream through shared memory, and per kv
// tile
//
//   S  = Q K^T, dP = dO V^T         tcgen05.mma, f32 accumulators in tensor memory (128 + 128 columns)
//   dS = P o (dP - delta) o sigma'  in registers by two warpgroups: threads t and t + 128 own query row t and
//                                   64 key columns each; P is rebuilt from (l, m) as
//                                   exp2(x2 - (m log2e + log2 l)); dS is written as bf16 to a shared-memory
//                                   tile in the K-major operand layout
//   dQ += dS K                      tcgen05.mma, A = dS from shared memory, B = the same K tile read MN-major;
//                                   dQ (D columns) stays in tensor memory across kv tiles
//
// Because dS does not go back into the S / dP columns, those are free again as soon as the warpgroups have
// loaded them into registers: the MMAs of tile n+1 run during the element-wise math of tile n.
//
// Shared memory holds ONE ring of three 2-tile stages for everything that is loaded: the ring entries of a
// CTA are, in order, [Q, dO of item 0], [K, V of its tile 0], [K, V of tile 1] ... [Q, dO of item 1] ... so the
// loads of the next item are in flight while the current one is still being computed.  A stage is released by
// the MMA issuer: with tcgen05.commit after the dQ MMA that read a K/V entry, with a plain arrive once every
// warp has copied a Q/dO entry into tensor memory.  The epilogue (dQ * sm_scale as bf16) is staged in the dS
// tile and leaves through TMA bulk stores.  Masks run only on partial tiles.
#include "sched.cuh"
#include "sm100.cuh"


namespace flexattn {
namespace FLEXATTN_TU_NAMESPACE {

constexpr int kThreads = 320;  // warps 0-3, 4-7: element-wise warpgroups (64 key columns each); 8: MMA; 9: TMA
constexpr int kMmaWarp = 8, kTmaWarp = 9;

constexpr int kStages = 3;
constexpr long long kDqL2Budget = 16ll << 20;  // K + V bytes live at a time (sets the head group size of the item list)

struct DqSmem {
  uint64_t bar_full[kStages], bar_free[kStages], bar_qtm, bar_sdp, bar_ld, bar_ds, bar_dq;
  uint32_t tmem_base;
  // descriptors of the CTA's items (ring): written by the producer, which walks the item list, and read by the
  // MMA issuer and the warpgroups (after the Q/dO entry of the item has landed)
  int4 item_a[8];  // {batch*head, q tile, first kv tile, end kv tile}
  int2 item_b[8];  // {first fully kept kv tile, end of the fully kept run}
  alignas(16) int32_t doc[2][kTile];
};

// This thread's 64 columns (keys j_first .. j_first+63) of its query row: raw S and dP in, packed bf16 dS out.
// nlse2 = log2(1 + 2^-9) - (m log2e + log2 l) (pre-scaling for pack_bf16_trunc) and delta belong to the row.  The mask functor is compiled in only for partial
// tiles.
// what a user score function sees besides the score and the positions
struct ScoreCtx {
  float sm_scale;
  int b, h;
};

// kInterval: the row's kept keys are the interval [klo, khi) (interval mask kinds; documents over sorted ids): a
// partial tile then tests one bit per element of a bitmap built once per 32 columns.
template <int SK, int MK, bool kPartial, bool kBias = false, bool kInterval = kMaskIsInterval<MK>>
__device__ __forceinline__ void dq_half_math(const uint32_t (&sr)[2][32], const uint32_t (&pr)[2][32],
                                             uint32_t (&pk)[32], float nlse2, float delta,
                                             const int32_t* __restrict__ s_doc, int i, int di, int j_first, int seq_k,
                                             int window, int stride, float c2, float slope2, float abase, float capl2,
                                             float csc, const ScoreCtx ctx, const float* __restrict__ ab_row = nullptr,
                                             float* __restrict__ dab_row = nullptr, int klo = 0, int khi = 0) {
  const float bias0 = abase + nlse2;  // ALiBi: slope * (j_first - i), folded with the row's -lse2
  uint32_t keep = 0u;  // kept columns of the current group of 32 (kInterval on partial tiles)
  // kBias: ab_row / dab_row point at this row's element of column j_first (nullptr: none, or a row past the end);
  // the bias joins the logit after the score function, and its gradient is p * (dp - delta) before sigma'.
  float bias[8];
  if constexpr (SK == FLEXATTN_SCORE_SOFTCAP || SK == FLEXATTN_SCORE_USER) {
    // scalar form: the packed one costs registers here (tanh, its derivative and the mask live together)
#pragma unroll
    for (int c = 0; c < 64; c += 2) {
      float dv[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int cc = c + u;
        float arg, dsig;  // log2-domain logit minus the row's log-sum-exp; derivative of the score function
        if constexpr (SK == FLEXATTN_SCORE_USER) {
          const float sc = __uint_as_float(sr[cc >> 5][cc & 31]) * ctx.sm_scale;
          arg = fmaf(user_score(sc, ctx.b, ctx.h, i, j_first + cc), kLog2e, nlse2);
          dsig = user_dscore(sc, ctx.b, ctx.h, i, j_first + cc);
        } else {
          const float th = ptx::tanh_approx(__uint_as_float(sr[cc >> 5][cc & 31]) * csc);
          arg = fmaf(capl2, th, nlse2);
          dsig = fmaf(-th, th, 1.f);
        }
        if constexpr (kBias) {
          if ((cc & 7) == 0) {
            if (ab_row != nullptr) ptx::load_bias8(bias, ab_row + cc, seq_k - (j_first + cc));
            else
#pragma unroll
              for (int w = 0; w < 8; ++w) bias[w] = 0.f;
          }
          arg = fmaf(bias[cc & 7], kLog2e, arg);
        }
        float p = ptx::ex2(arg);
        if constexpr (kPartial && kInterval) {
          if ((cc & 31) == 0) keep = range_bits32(klo - (j_first + cc), khi - (j_first + cc));
          p = (keep >> (cc & 31)) & 1u ? p : 0.f;
        } else if constexpr (kPartial) {
          const int j = j_first + cc;
          const int dj = (MK == FLEXATTN_MASK_DOCUMENT) ? s_doc[cc] : 0;
          p = ((j < seq_k) && mask_keep<MK>(i, j, window, stride, di, dj)) ? p : 0.f;
        }
        const float dt = p * (__uint_as_float(pr[cc >> 5][cc & 31]) - delta);
        if constexpr (kBias) {
          // p carries the (1 + 2^-9) pre-scaling meant for the truncating bf16 pack: undo it for the f32 gradient
          if (dab_row != nullptr && j_first + cc < seq_k) dab_row[cc] = dt * ptx::kRoundInv;
        }
        dv[u] = dt * dsig;
      }
      pk[c >> 1] = ptx::pack_bf16_trunc(dv[0], dv[1]);
    }
    return;
  }
  // two columns per instruction (packed f32x2) wherever the arithmetic allows it
  const uint64_t c22 = ptx::pack2(c2, c2), nl2 = ptx::pack2(nlse2, nlse2), dl2 = ptx::pack2(delta, delta);
  // ALiBi: the bias of columns (c, c + 1) advances by a constant from pair to pair (one packed add per pair)
  uint64_t b2 = ptx::pack2(bias0, bias0 + slope2);
  const uint64_t bstep2 = ptx::pack2(2.f * slope2, 2.f * slope2);
#pragma unroll
  for (int c = 0; c < 64; c += 2) {
    const uint64_t s2 = ptx::pack2(__uint_as_float(sr[c >> 5][c & 31]), __uint_as_float(sr[c >> 5][(c & 31) + 1]));
    const uint64_t dp2 = ptx::pack2(__uint_as_float(pr[c >> 5][c & 31]), __uint_as_float(pr[c >> 5][(c & 31) + 1]));
    uint64_t arg2;
    if constexpr (SK == FLEXATTN_SCORE_ALIBI) {
      arg2 = ptx::fma2(s2, c22, b2);
      b2 = ptx::add2(b2, bstep2);
    } else {
      arg2 = ptx::fma2(s2, c22, nl2);
    }
    float a0, a1;
    ptx::unpack2(arg2, a0, a1);
    if constexpr (kBias) {
      if ((c & 7) == 0) {
        if (ab_row != nullptr) ptx::load_bias8(bias, ab_row + c, seq_k - (j_first + c));
        else
#pragma unroll
          for (int w = 0; w < 8; ++w) bias[w] = 0.f;
      }
      a0 = fmaf(bias[c & 7], kLog2e, a0);
      a1 = fmaf(bias[(c & 7) + 1], kLog2e, a1);
    }
    float p0 = ptx::ex2(a0), p1 = ptx::ex2(a1);
    if constexpr (kPartial && kInterval) {  // one bitmap per row and 32 columns instead of per-element tests
      if ((c & 31) == 0) keep = range_bits32(klo - (j_first + c), khi - (j_first + c));
      p0 = (keep >> (c & 31)) & 1u ? p0 : 0.f;
      p1 = (keep >> ((c & 31) + 1)) & 1u ? p1 : 0.f;
    } else if constexpr (kPartial) {
      const int j = j_first + c;
      const int d0 = (MK == FLEXATTN_MASK_DOCUMENT) ? s_doc[c] : 0, d1 = (MK == FLEXATTN_MASK_DOCUMENT) ? s_doc[c + 1] : 0;
      p0 = ((j < seq_k) && mask_keep<MK>(i, j, window, stride, di, d0)) ? p0 : 0.f;
      p1 = ((j + 1 < seq_k) && mask_keep<MK>(i, j + 1, window, stride, di, d1)) ? p1 : 0.f;
    }
    const uint64_t d2 = ptx::mul2(ptx::pack2(p0, p1), ptx::sub2(dp2, dl2));
    float d0f, d1f;
    ptx::unpack2(d2, d0f, d1f);
    if constexpr (kBias) {
      if (dab_row != nullptr) {  // f32 gradient of the bias: undo the pre-scaling meant for the truncating bf16 pack
        if (j_first + c < seq_k) dab_row[c] = d0f * ptx::kRoundInv;
        if (j_first + c + 1 < seq_k) dab_row[c + 1] = d1f * ptx::kRoundInv;
      }
    }
    pk[c >> 1] = ptx::pack_bf16_trunc(d0f, d1f);
  }
}

template <int D, int SK, int MK>
__global__ void __launch_bounds__(kThreads, 1)
    dq_sm100_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                    const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                    const __grid_constant__ CUtensorMap tm_dq, const DevParams P, int* abort_flag) {
  constexpr int kPanels = D / 64;
  constexpr uint32_t kTileBytes = kPanels * ptx::kPanelBytes;
  constexpr uint32_t kStageBytes = 2 * kTileBytes;      // [K, V] or [Q, dO]
  constexpr uint32_t kDsBytes = 2 * ptx::kPanelBytes;   // dS tile: 128 query rows x 128 keys, bf16
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kColS = 0, kColDP = 128, kColDQ = 256;
  constexpr uint32_t kColQ = 384, kColDO = 384 + D / 2;  // Q and dO as packed bf16 A operands (D/2 columns each)

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sRing = smem;
  uint8_t* sDS = smem + kStages * kStageBytes;
  DqSmem* sh = reinterpret_cast<DqSmem*>(smem + kStages * kStageBytes + kDsBytes);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (aborted_on_entry(abort_flag, P.status, 2)) return;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(&sh->bar_full[s], 1);
      ptx::mbar_init(&sh->bar_free[s], 1);
    }
    ptx::mbar_init(&sh->bar_qtm, 8);  // one arrival per warp of the two warpgroups, here and below
    ptx::mbar_init(&sh->bar_sdp, 1);
    ptx::mbar_init(&sh->bar_ld, 8);
    ptx::mbar_init(&sh->bar_ds, 8);
    ptx::mbar_init(&sh->bar_dq, 1);
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

  // In every role: e = index of a ring entry in this CTA's stream (stage e % 3, barrier phase (e / 3) & 1),
  // T = index of a kv tile in the stream (phase T & 1 of the per-tile barriers), r = index of an item.
  if (warp == kTmaWarp) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      bool ok = true;
      ptx::prefetch_tensormap(&tm_q);
      ptx::prefetch_tensormap(&tm_do);
      ptx::prefetch_tensormap(&tm_k);
      ptx::prefetch_tensormap(&tm_v);
      int e = 0, r = 0;
      auto acquire = [&]() -> uint8_t* {  // the stage of entry e, once the entry that used it before is done
        const int st = e % kStages;
        if (e >= kStages) ok = ptx::mbar_wait(&sh->bar_free[st], (uint32_t)((e / kStages - 1) & 1));
        return sRing + st * kStageBytes;
      };
      for (ItemCursor it(P, kDqL2Budget); ok && it.valid(); it.next(), ++r) {
        const int bh = it.bh(), first = it.rm.x, N = it.tiles();
        uint8_t* dst = acquire();
        if (!ok) break;
        sh->item_a[r & 7] = make_int4(bh, it.qt(), it.rm.x, it.rm.y);
        sh->item_b[r & 7] = make_int2(it.rm.z, it.rm.w);
        uint64_t* bar = &sh->bar_full[e % kStages];
        ptx::mbar_arrive_expect_tx(bar, kStageBytes);
#pragma unroll
        for (int p = 0; p < kPanels; ++p) {
          ptx::tma_load_3d(dst + p * ptx::kPanelBytes, &tm_q, bar, p * 64, it.qt() * kTile, bh);
          ptx::tma_load_3d(dst + kTileBytes + p * ptx::kPanelBytes, &tm_do, bar, p * 64, it.qt() * kTile, bh);
        }
        ++e;
        for (int n = 0; n < N && ok; ++n, ++e) {
          dst = acquire();
          if (!ok) break;
          bar = &sh->bar_full[e % kStages];
          ptx::mbar_arrive_expect_tx(bar, kStageBytes);
#pragma unroll
          for (int p = 0; p < kPanels; ++p) {
            ptx::tma_load_3d(dst + p * ptx::kPanelBytes, &tm_k, bar, p * 64, (first + n) * kTile, bh);
            ptx::tma_load_3d(dst + kTileBytes + p * ptx::kPanelBytes, &tm_v, bar, p * 64, (first + n) * kTile, bh);
          }
        }
      }
      if (!ok) give_up(abort_flag, P.status, 2, 20);
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer
    // Q and dO are A operands from tensor memory: an MMA with both operands in shared memory reads 8 KB per 64
    // cycles, the whole shared-memory bandwidth of the SM, and this kernel also streams K, V and dS through
    // shared memory.  S(T+1), dP(T+1) are issued as soon as the warpgroups have READ S(T), dP(T) out of tensor
    // memory, so the tensor core works on the next tile while the warpgroups do the element-wise math of this
    // one; dQ += dS(T) K(T) follows when dS(T) is in place.  This thread does no index arithmetic: it walks the
    // rounds of the item list and takes each item's tile count from the producer.
    if (lane == 0) {
      bool ok = true;
      int fail_at = 1;
      constexpr uint32_t idesc_s = ptx::make_idesc(128, 128, false);
      constexpr uint32_t idesc_dq = ptx::make_idesc(128, D, true);
      const ptx::DescBase bDS = ptx::base_kmajor(ptx::smem_u32(sDS));
      const uint32_t aRing = ptx::smem_u32(sRing);
      const int total = P.n_qt * P.batch * P.heads, G = (int)gridDim.x, c = (int)blockIdx.x;
      // ring position of the next entry: stage e % 3 and fill phase (e / 3) & 1, kept as counters (this thread's
      // instruction count per MMA bounds the kernel)
      uint32_t st = 0, ph = 0;
      int T = 0;
      auto advance = [&]() {
        if (++st == kStages) { st = 0; ph ^= 1u; }
      };
      auto issue_sdp = [&](uint32_t stage) {  // S = Q K^T, dP = dO V^T with the K/V in ring stage `stage`
        const uint32_t st_off = stage * kStageBytes;
        const ptx::DescBase bK = ptx::base_kmajor(aRing + st_off), bV = ptx::base_kmajor(aRing + st_off + kTileBytes);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          ptx::mma_ts(tmem + kColS, tmem + kColQ + kk * 8, ptx::desc_at(bK, ptx::koff_kmajor(kk)), idesc_s, kk > 0);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          ptx::mma_ts(tmem + kColDP, tmem + kColDO + kk * 8, ptx::desc_at(bV, ptx::koff_kmajor(kk)), idesc_s, kk > 0);
        ptx::mma_commit(&sh->bar_sdp);
      };
      auto item_exists = [&](int r) { return r * G + ((r & 1) ? G - 1 - c : c) < total; };
      // Waits until Q, dO of item r are in tensor memory, releases their ring stage and issues the item's first S, dP.
      // Returns the item's number of kv tiles.
      auto start_item = [&](int r) -> int {
        ok = ptx::mbar_wait(&sh->bar_qtm, r & 1);
        if (!ok) { fail_at = 2; return 0; }
        const int4 ia = sh->item_a[r & 7];
        const int n_tiles = ia.w - ia.z;
        ptx::mbar_arrive(&sh->bar_free[st]);  // the Q/dO entry has been copied out of its stage
        advance();
        if (n_tiles > 0) {
          ok = ptx::mbar_wait(&sh->bar_full[st], ph);
          if (!ok) { fail_at = 3; return 0; }
          ptx::tc_fence_after();
          issue_sdp(st);
        }
        return n_tiles;
      };
      int N = item_exists(0) ? start_item(0) : 0;
      for (int r = 0; ok && item_exists(r); ++r) {
        int N_next = 0;
        bool started_next = false;
        for (int n = 0; n < N && ok; ++n, ++T) {
          const uint32_t par = T & 1;
          const uint32_t cur = st;  // stage of this tile's K/V
          advance();
          if (n + 1 < N) {
            ok = ptx::mbar_wait(&sh->bar_ld, par);  // S(T), dP(T) are in registers: their columns are free
            if (!ok) { fail_at = 4; break; }
            ok = ptx::mbar_wait(&sh->bar_full[st], ph);
            if (!ok) { fail_at = 5; break; }
            ptx::tc_fence_after();
            issue_sdp(st);
          } else if (item_exists(r + 1)) {
            // last tile of the item: the warpgroups copy the next item's Q, dO into tensor memory before they read
            // this tile's S, dP, so the next item's first S, dP can run during this tile's element-wise math, the dQ
            // MMA and the epilogue
            ok = ptx::mbar_wait(&sh->bar_ld, par);
            if (!ok) { fail_at = 4; break; }
            N_next = start_item(r + 1);
            started_next = true;
            if (!ok) break;
          }
          ok = ptx::mbar_wait(&sh->bar_ds, par);  // dS(T) written to shared memory
          if (!ok) { fail_at = 6; break; }
          ptx::tc_fence_after();
          const ptx::DescBase bKt = ptx::base_mnmajor(aRing + cur * kStageBytes);
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk)
            ptx::mma_ss(tmem + kColDQ, ptx::desc_at(bDS, ptx::koff_kmajor(kk)), ptx::desc_at(bKt, ptx::koff_mnmajor(kk)),
                        idesc_dq, (n > 0) || (kk > 0));
          ptx::mma_commit(&sh->bar_dq);
          ptx::mma_commit(&sh->bar_free[cur]);  // K/V of this entry have been read
        }
        if (!ok) break;
        if (!started_next && item_exists(r + 1)) N_next = start_item(r + 1);  // (items without kv tiles)
        N = N_next;
      }
      if (!ok) give_up(abort_flag, P.status, 2, fail_at);
    }
  } else {
    // ------------------------------------------------------------------ element-wise warpgroups
    const int row = tid & 127;   // query row inside the tile = TMEM lane
    const int half = tid >> 7;   // which 64 key columns of every tile this thread handles
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const float c2 = P.sm_scale * kLog2e;
    const float capl2 = P.cap * kLog2e;
    const float csc = (SK == FLEXATTN_SCORE_SOFTCAP) ? P.sm_scale / P.cap : 0.f;
    // this thread's 128 bytes of the dS tile: row `row` of panel `half`, 16-byte chunk j at slot j ^ (row & 7)
    uint8_t* ds_row = sDS + half * ptx::kPanelBytes + row * 128;
    bool ok = true;
    int fail_at = 0;
    int e = 0, T = 0;
    const int total = P.n_qt * P.batch * P.heads, G = (int)gridDim.x, cta = (int)blockIdx.x;
    // row statistics of the NEXT item, fetched early when its descriptor is already there
    bool pf_have = false;
    float pf_l = 0.f, pf_m = 0.f, pf_delta = 0.f;
    int pf_di = 0;
    auto row_stats = [&](const int4 ia, float& l, float& m, float& dl, int& di_out) {
      const int i = ia.y * kTile + row;
      l = 0.f; m = 0.f; dl = 0.f; di_out = 0;
      if (i < P.seq_q && FLEXATTN_DBG_OK((long long)ia.x * P.seq_q + i, (long long)P.batch * P.heads * P.seq_q, 2, 201)) {
        const size_t g = (size_t)ia.x * P.seq_q + i;
        l = P.l[g];
        m = P.m[g];
        dl = P.delta[g];
        if (MK == FLEXATTN_MASK_DOCUMENT &&
            FLEXATTN_DBG_OK((long long)(ia.x / P.heads) * P.doc_stride + i, (long long)P.batch * P.doc_stride, 2, 202))
          di_out = (P.doc_ids + (size_t)(ia.x / P.heads) * P.doc_stride)[i];
      }
    };

    // Q and dO rows of an item -> tensor memory as packed bf16 (element d of row r at lane r, column d / 2), from ring
    // entry `entry`.  Thread (row, half) moves the 64 elements of 128-byte panel `half`: chunk j of the row sits at
    // slot j ^ (row & 7).  Every MMA that read the previous Q / dO must have completed: the caller has waited for
    // the S / dP of the previous item's last tile.
    auto copy_q_do = [&](int entry) {
      const uint8_t* sQ = sRing + (entry % kStages) * kStageBytes;
      const uint8_t* sDO = sQ + kTileBytes;
      if constexpr (D == 128) {
#pragma unroll
        for (int which = 0; which < 2; ++which) {
          const uint8_t* src = (which ? sDO : sQ) + half * ptx::kPanelBytes + row * 128;
          uint32_t rr[32];
#pragma unroll
          for (int jc = 0; jc < 8; ++jc) {
            const uint4 v4 = *reinterpret_cast<const uint4*>(src + ((jc ^ (row & 7)) << 4));
            rr[4 * jc] = v4.x; rr[4 * jc + 1] = v4.y; rr[4 * jc + 2] = v4.z; rr[4 * jc + 3] = v4.w;
          }
          ptx::tmem_st32(lane_base + (which ? kColDO : kColQ) + half * 32, rr);
        }
      } else {  // D == 64: one panel per tensor; warpgroup 0 moves Q, warpgroup 1 moves dO
        const uint8_t* src = (half ? sDO : sQ) + row * 128;
        uint32_t rr[32];
#pragma unroll
        for (int jc = 0; jc < 8; ++jc) {
          const uint4 v4 = *reinterpret_cast<const uint4*>(src + ((jc ^ (row & 7)) << 4));
          rr[4 * jc] = v4.x; rr[4 * jc + 1] = v4.y; rr[4 * jc + 2] = v4.z; rr[4 * jc + 3] = v4.w;
        }
        ptx::tmem_st32(lane_base + (half ? kColDO : kColQ), rr);
      }
      ptx::tmem_wait_st();
      ptx::tc_fence_before();
      ptx::mbar_arrive_warp(&sh->bar_qtm);
    };
    bool copied_ahead = false;  // this item's Q, dO were already copied during the previous item's last tile
    const bool has_bias = P.ab != nullptr || P.dab != nullptr;  // dense bias and / or its gradient requested

    for (int r = 0; r * G + ((r & 1) ? G - 1 - cta : cta) < total; ++r) {
      // the Q/dO entry of the item has landed, and with it the item's descriptor
      if (ok && !copied_ahead) {
        ok = __all_sync(0xffffffffu, ptx::mbar_wait(&sh->bar_full[e % kStages], (uint32_t)((e / kStages) & 1)));
        if (!ok) fail_at = 9;
      }
      const int4 ia = sh->item_a[r & 7];
      const int2 ib = sh->item_b[r & 7];
      const int bh = ia.x, qt = ia.y, b = bh / P.heads, h = bh % P.heads;
      const int4 rm = make_int4(ia.z, ia.w, ib.x, ib.y);
      const int N = rm.y - rm.x;
      const int i = qt * kTile + row;
      const bool row_ok = i < P.seq_q;
      const long long n_rows = (long long)P.batch * P.heads * P.seq_q, n_doc = (long long)P.batch * P.doc_stride;
      const float slope2 = (SK == FLEXATTN_SCORE_ALIBI && FLEXATTN_DBG_OK(h, P.heads, 2, 203)) ? P.alibi_slopes[h] * kLog2e : 0.f;
      const int32_t* doc = (MK == FLEXATTN_MASK_DOCUMENT) ? P.doc_ids + (size_t)b * P.doc_stride : nullptr;
      float l_, m_, delta;
      int di;
      if (pf_have) { l_ = pf_l; m_ = pf_m; delta = pf_delta; di = pf_di; }
      else row_stats(ia, l_, m_, delta, di);
      pf_have = false;
      // l == 0 (fully masked row): force p to 0; kRoundLog2 pre-scales p (and so dS) for pack_bf16_trunc
      const float nlse2 = row_ok ? (l_ > 0.f ? ptx::kRoundLog2 - fmaf(m_, kLog2e, log2f(l_)) : -1.0e30f) : ptx::kRoundLog2;

      // the interval [klo, khi) of keys this row keeps, where the mask has one: the interval kinds, and a document
      // mask when the ids of the batch row never decrease (then the mask map holds the start of every row's document)
      constexpr bool kDoc = MK == FLEXATTN_MASK_DOCUMENT;
      bool doc_runs = false;
      int klo = 0, khi = P.seq_k;
      if constexpr (kMaskIsInterval<MK>) row_key_interval<MK>(i, P.seq_k, P.window, klo, khi);
      if constexpr (kDoc) {
        doc_runs = FLEXATTN_DBG_OK(b, P.batch, 2, 207) && P.doc_sorted[b] != 0;
        if (doc_runs && row_ok && FLEXATTN_DBG_OK((long long)b * P.doc_stride + i, n_doc, 2, 208)) {
          klo = P.run_lo[(size_t)b * P.doc_stride + i];
          khi = i + 1 < P.seq_k ? i + 1 : P.seq_k;
        }
      }

      // dense bias / its gradient: this query row's first element (nullptr: none, or a row past the end)
      const ScoreCtx ctx{P.sm_scale, b, h};
      const bool bias_row_ok = row_ok && FLEXATTN_DBG_OK((long long)bh * P.seq_q + i, n_rows, 2, 204);
      const float* ab_q = (P.ab != nullptr && bias_row_ok) ? P.ab + ((size_t)bh * P.seq_q + i) * P.seq_k : nullptr;
      float* dab_q = (P.dab != nullptr && bias_row_ok) ? P.dab + ((size_t)bh * P.seq_q + i) * P.seq_k : nullptr;
      if (P.dab != nullptr) {
        // the bias gradient is dense: the columns of kv tiles this item never visits get their zeros here
        // (warp = row, lanes along the row: coalesced)
        const int kbeg = min(rm.x * kTile, P.seq_k), kend = min(rm.y * kTile, P.seq_k);
        for (int r = warp; r < kTile; r += 8) {
          const int ir = qt * kTile + r;
          if (ir >= P.seq_q || !FLEXATTN_DBG_OK((long long)bh * P.seq_q + ir, n_rows, 2, 205)) break;
          float* zrow = P.dab + ((size_t)bh * P.seq_q + ir) * P.seq_k;
          for (int j = lane; j < kbeg; j += 32) zrow[j] = 0.f;
          for (int j = kend + lane; j < P.seq_k; j += 32) zrow[j] = 0.f;
        }
      }

      if (ok && !copied_ahead) copy_q_do(e);
      copied_ahead = false;
      ++e;
      const bool has_next = (r + 1) * G + (((r + 1) & 1) ? G - 1 - cta : cta) < total;

      for (int n = 0; n < N; ++n, ++T, ++e) {
        const int kt = rm.x + n, j0 = kt * kTile + 64 * half;  // first key position of this thread's columns
        const bool partial = has_bias || !(kt >= rm.z && kt < rm.w);  // with a bias: always the masked form
        if (MK == FLEXATTN_MASK_DOCUMENT && partial && !doc_runs) {
          if (row < 64) {
            const int j = j0 + row;
            sh->doc[T & 1][64 * half + row] =
                (j < P.seq_k && FLEXATTN_DBG_OK((long long)b * P.doc_stride + j, n_doc, 2, 206)) ? doc[j] : -1;
          }
          ptx::named_bar_sync(1 + half, 128);
        }
        // a failed wait never leaves the loops early: every thread keeps executing the same named barriers
        if (ok) {
          ok = __all_sync(0xffffffffu, ptx::mbar_wait(&sh->bar_sdp, T & 1));
          if (!ok) fail_at = 10;
        }
        if (!ok) continue;
        ptx::tc_fence_after();
        if (n == N - 1 && has_next) {
          // Last tile of the item: every MMA that reads this item's Q, dO has completed (S, dP of this tile are
          // ready), so the next item's Q, dO go into tensor memory now.  Its first S, dP then run during this
          // tile's element-wise math, the last dQ MMA and the epilogue.  Entry e + 1 of the ring is that Q/dO pair.
          ok = __all_sync(0xffffffffu, ptx::mbar_wait(&sh->bar_full[(e + 1) % kStages], (uint32_t)(((e + 1) / kStages) & 1)));
          if (!ok) { fail_at = 13; continue; }
          copy_q_do(e + 1);
          copied_ahead = true;
          row_stats(sh->item_a[(r + 1) & 7], pf_l, pf_m, pf_delta, pf_di);  // and its row statistics are fetched early
          pf_have = true;
        }
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
        ptx::tc_fence_before();
        ptx::mbar_arrive_warp(&sh->bar_ld);  // S / dP columns may be overwritten by the next tile's MMAs
        uint32_t pk[32];
        const float abase = slope2 * (float)(j0 - i);
        const int32_t* s_doc = &sh->doc[T & 1][64 * half];
        const float* ab_t = ab_q != nullptr ? ab_q + j0 : nullptr;
        float* dab_t = dab_q != nullptr ? dab_q + j0 : nullptr;
        if (has_bias) {
          if constexpr (kDoc) {
            if (doc_runs)
              dq_half_math<SK, MK, true, true, true>(sr, pr, pk, nlse2, delta, s_doc, i, di, j0, P.seq_k, P.window, P.stride,
                                                     c2, slope2, abase, capl2, csc, ctx, ab_t, dab_t, klo, khi);
            else
              dq_half_math<SK, MK, true, true, false>(sr, pr, pk, nlse2, delta, s_doc, i, di, j0, P.seq_k, P.window, P.stride,
                                                      c2, slope2, abase, capl2, csc, ctx, ab_t, dab_t);
          } else {
            dq_half_math<SK, MK, true, true>(sr, pr, pk, nlse2, delta, s_doc, i, di, j0, P.seq_k, P.window, P.stride, c2,
                                             slope2, abase, capl2, csc, ctx, ab_t, dab_t, klo, khi);
          }
        } else if (partial) {
          if constexpr (kDoc) {
            if (doc_runs)
              dq_half_math<SK, MK, true, false, true>(sr, pr, pk, nlse2, delta, s_doc, i, di, j0, P.seq_k, P.window, P.stride,
                                                      c2, slope2, abase, capl2, csc, ctx, nullptr, nullptr, klo, khi);
            else
              dq_half_math<SK, MK, true, false, false>(sr, pr, pk, nlse2, delta, s_doc, i, di, j0, P.seq_k, P.window,
                                                       P.stride, c2, slope2, abase, capl2, csc, ctx);
          } else {
            dq_half_math<SK, MK, true>(sr, pr, pk, nlse2, delta, s_doc, i, di, j0, P.seq_k, P.window, P.stride, c2, slope2,
                                       abase, capl2, csc, ctx, nullptr, nullptr, klo, khi);
          }
        } else {
          dq_half_math<SK, MK, false>(sr, pr, pk, nlse2, delta, s_doc, i, di, j0, P.seq_k, P.window, P.stride, c2, slope2,
                                      abase, capl2, csc, ctx);
        }
        if (n > 0) {  // the dQ MMA of the previous tile must have read the dS buffer
          ok = __all_sync(0xffffffffu, ptx::mbar_wait(&sh->bar_dq, (T - 1) & 1));
          if (!ok) { fail_at = 11; continue; }
        }
#pragma unroll
        for (int jc = 0; jc < 8; ++jc) {
          const uint4 v4 = make_uint4(pk[4 * jc], pk[4 * jc + 1], pk[4 * jc + 2], pk[4 * jc + 3]);
          *reinterpret_cast<uint4*>(ds_row + ((jc ^ (row & 7)) << 4)) = v4;
        }
        ptx::fence_proxy_async_smem();  // generic-proxy stores -> visible to the MMA's shared-memory reads
        ptx::mbar_arrive_warp(&sh->bar_ds);
      }

      // ---- item epilogue: dQ * sm_scale as bf16 into the dS tile (free: the last dQ MMA has read it) in the TMA
      // (128-byte swizzle) layout, then one bulk tensor store per 64-column panel; rows past seq_q are clipped
      // by the tensor map.
      if (ok && N > 0) {
        ok = __all_sync(0xffffffffu, ptx::mbar_wait(&sh->bar_dq, (T - 1) & 1));
        if (!ok) fail_at = 12;
      }
      if (ok) {
        if (N > 0) ptx::tc_fence_after();
        const float sc = P.sm_scale;
        uint8_t* stage_row = sDS + row * 128;
#pragma unroll 1
        for (int c0 = half * (D / 2); c0 < (half + 1) * (D / 2); c0 += 32) {
          uint32_t rr[32];
          if (N > 0) {
            ptx::tmem_ld32(lane_base + kColDQ + c0, rr);
            ptx::tmem_wait_ld();
            ptx::tmem_ld_acquire(rr);
          } else {
#pragma unroll
            for (int c = 0; c < 32; ++c) rr[c] = 0u;
          }
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            uint4 v4;
            v4.x = ptx::pack_bf16(__uint_as_float(rr[c]) * sc, __uint_as_float(rr[c + 1]) * sc);
            v4.y = ptx::pack_bf16(__uint_as_float(rr[c + 2]) * sc, __uint_as_float(rr[c + 3]) * sc);
            v4.z = ptx::pack_bf16(__uint_as_float(rr[c + 4]) * sc, __uint_as_float(rr[c + 5]) * sc);
            v4.w = ptx::pack_bf16(__uint_as_float(rr[c + 6]) * sc, __uint_as_float(rr[c + 7]) * sc);
            const int col = c0 + c, panel = col >> 6, chunk = (col & 63) >> 3;
            *reinterpret_cast<uint4*>(stage_row + panel * ptx::kPanelBytes + ((chunk ^ (row & 7)) << 4)) = v4;
          }
        }
        if (N > 0) ptx::tc_fence_before();
        ptx::fence_proxy_async_smem();  // generic-proxy stores -> visible to the bulk store
      }
      ptx::named_bar_sync(3, 256);
      if (ok && tid == 0) {
#pragma unroll
        for (int p = 0; p < kPanels; ++p) ptx::tma_store_3d(&tm_dq, sDS + p * ptx::kPanelBytes, p * 64, qt * kTile, bh);
        ptx::tma_store_commit();
        ptx::tma_store_wait_read();  // the dS tile is written again by the next item's first tile
      }
      ptx::named_bar_sync(3, 256);
    }
    if (!ok && lane == 0) give_up(abort_flag, P.status, 2, fail_at);
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, kTmemCols);
  }
}

#ifndef FLEXATTN_JIT
template <int D, int SK, int MK>
int launch_one(cudaStream_t st, const DevParams& d, const CUtensorMap& tq, const CUtensorMap& tdo,
               const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdq, int* abort_flag) {
  constexpr size_t smem = 6 * (D / 64) * ptx::kPanelBytes + 2 * ptx::kPanelBytes + sizeof(DqSmem) + 1024;
  // 512 TMEM columns per CTA: never let two CTAs share an SM (the second would spin in tcgen05.alloc)
  constexpr size_t smem_req = smem > 120 * 1024 ? smem : 120 * 1024;
  auto kern = dq_sm100_kernel<D, SK, MK>;
  static SmemAttrOnce attr_once{};  // per kernel instantiation, per device
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), (int)smem_req, &attr_once) != FLEXATTN_OK) return FLEXATTN_ERR_CUDA;
  // persistent: one CTA per SM (fewer when there are fewer work items)
  const long long items = (long long)d.n_qt * d.batch * d.heads;
  const int sms = sm_count();
  if (sms <= 0) return FLEXATTN_ERR_CUDA;
  dim3 grid((unsigned)(items < sms ? items : sms));
  kern<<<grid, kThreads, smem_req, st>>>(tq, tdo, tk, tv, tdq, d, abort_flag);
  return cudaGetLastError() == cudaSuccess ? FLEXATTN_OK : FLEXATTN_ERR_CUDA;
}

template <int D, int SK>
int launch_mask(cudaStream_t st, const DevParams& d, int mask, const CUtensorMap& tq, const CUtensorMap& tdo,
                const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdq, int* af) {
  switch (mask) {
    case FLEXATTN_MASK_NONE: return launch_one<D, SK, FLEXATTN_MASK_NONE>(st, d, tq, tdo, tk, tv, tdq, af);
    case FLEXATTN_MASK_CAUSAL: return launch_one<D, SK, FLEXATTN_MASK_CAUSAL>(st, d, tq, tdo, tk, tv, tdq, af);
    case FLEXATTN_MASK_SLIDING_WINDOW: return launch_one<D, SK, FLEXATTN_MASK_SLIDING_WINDOW>(st, d, tq, tdo, tk, tv, tdq, af);
    case FLEXATTN_MASK_SLIDING_WINDOW_CAUSAL:
      return launch_one<D, SK, FLEXATTN_MASK_SLIDING_WINDOW_CAUSAL>(st, d, tq, tdo, tk, tv, tdq, af);
    case FLEXATTN_MASK_DOCUMENT: return launch_one<D, SK, FLEXATTN_MASK_DOCUMENT>(st, d, tq, tdo, tk, tv, tdq, af);
    case FLEXATTN_MASK_S2: return launch_one<D, SK, FLEXATTN_MASK_S2>(st, d, tq, tdo, tk, tv, tdq, af);
    default: return FLEXATTN_ERR_UNSUPPORTED_MOD;
  }
}

template <int D>
int launch_score(cudaStream_t st, const DevParams& d, int score, int mask, const CUtensorMap& tq,
                 const CUtensorMap& tdo, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdq, int* af) {
  switch (score) {
    case FLEXATTN_SCORE_NONE: return launch_mask<D, FLEXATTN_SCORE_NONE>(st, d, mask, tq, tdo, tk, tv, tdq, af);
    case FLEXATTN_SCORE_ALIBI: return launch_mask<D, FLEXATTN_SCORE_ALIBI>(st, d, mask, tq, tdo, tk, tv, tdq, af);
    case FLEXATTN_SCORE_SOFTCAP: return launch_mask<D, FLEXATTN_SCORE_SOFTCAP>(st, d, mask, tq, tdo, tk, tv, tdq, af);
    default: return FLEXATTN_ERR_UNSUPPORTED_MOD;
  }
}

#endif  // !FLEXATTN_JIT

}  // namespace FLEXATTN_TU_NAMESPACE

#ifndef FLEXATTN_JIT
int launch_sm100_dq(cudaStream_t st, const DevParams& d, int score, int mask) {
  int* af = abort_flag_ptr();
  if (af == nullptr) return FLEXATTN_ERR_CUDA;
  CUtensorMap tq, tdo, tk, tv, tdq;
  const int slices = d.batch * d.heads;
  int e = make_tile_map(&tq, d.q, slices, d.seq_q, d.head_dim);
  if (e) return e;
  e = make_tile_map(&tdo, d.d_o, slices, d.seq_q, d.head_dim);
  if (e) return e;
  e = make_tile_map(&tk, d.k, slices, d.seq_k, d.head_dim);
  if (e) return e;
  e = make_tile_map(&tv, d.v, slices, d.seq_k, d.head_dim);
  if (e) return e;
  e = make_tile_map(&tdq, d.dq, slices, d.seq_q, d.head_dim);
  if (e) return e;
  if (score == FLEXATTN_SCORE_USER) {
    // a kernel compiled at run time around the registered score function: same parameters, grid and shared memory
    const size_t need = 6 * (size_t)(d.head_dim / 64) * ptx::kPanelBytes + 2 * ptx::kPanelBytes + sizeof(DqSmem) + 1024;
    const long long items = (long long)d.n_qt * d.batch * d.heads;
    const int sms = sm_count();
    if (sms <= 0) return FLEXATTN_ERR_CUDA;
    void* args[] = {&tq, &tdo, &tk, &tv, &tdq, const_cast<DevParams*>(&d), &af};
    return jit_launch(1, d.user_score, d.head_dim, mask, (unsigned)(items < sms ? items : sms), 1, kThreads,
                      need > 120 * 1024 ? need : 120 * 1024, st, args);
  }
  if (d.head_dim == 128) return launch_score<128>(st, d, score, mask, tq, tdo, tk, tv, tdq, af);
  if (d.head_dim == 64) return launch_score<64>(st, d, score, mask, tq, tdo, tk, tv, tdq, af);
  return FLEXATTN_ERR_UNSUPPORTED_HEAD_DIM;
}
#endif  // !FLEXATTN_JIT

}  // namespace flexattn
