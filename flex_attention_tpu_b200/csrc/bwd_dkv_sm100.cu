// dK / dV backward on the 5th-generation tensor cores (sm_100a).
//
// Replaces the reference's Pallas dK/dV kernel (flex_attention_dkv_kernel.py:177-280 and its mask-aware
// twin flash_attention_dkv_bwd.py:183-308).  Persistent: one CTA per SM walks a list of work items (128-row kv
// tile, batch*head), the kv tiles with the most q tiles first (the mask map's column work order), dealt to the
// CTAs in rounds of alternating direction.  Per item K and V stay in shared memory, Q and dO tiles stream through
// two-stage rings, and per q tile the TRANSPOSED score tile is formed so that the probabilities land in tensor
// memory in the layout the next MMA wants as its A operand:
//
//   S^T  = K Q^T, dP^T = V dO^T      tcgen05.mma, f32 accumulators (128 + 128 TMEM columns)
//   P^T, dS^T                        in registers; thread = key row, columns = query positions, whose statistics
//                                    (m log2e + log2 l, delta) are read from shared memory; written back as
//                                    packed bf16 over S^T / dP^T
//   dV += P^T dO ; dK += dS^T Q      tcgen05.mma, A from tensor memory, B = the dO / Q tile read MN-major
//
// The four MMA groups of consecutive tiles are interleaved on the tensor core so that each element-wise phase
// has two other groups to hide behind:
//
//   ... dV(n)  S^T(n+1)  dK(n)  dP^T(n+1)  dV(n+1)  S^T(n+2)  dK(n+1) ...
//
// P^T(n+1) (the exponentials) is computed while dK(n) and dP^T(n+1) run, dS^T(n+1) while dV(n+1) and S^T(n+2)
// run.  S^T(n+1) overwrites the columns dV(n) reads P^T(n) from, and dP^T(n+1) those dK(n) reads dS^T(n) from:
// MMAs issued by one thread execute in issue order, so issuing them in this order is all the protection needed.
// dK, dV (D columns each) stay in tensor memory across the q tiles of an item: 512 columns in total, one CTA per SM.
//
// The q tiles of all of a CTA's items form ONE stream T = 0, 1, 2 ...: the Q / dO rings and the per-tile barriers
// are indexed by T, so the rings keep streaming across item boundaries.  K and V of the next item are loaded as
// soon as the last dP^T of the current item has been issued and completed, i.e. during its last dV / dK MMAs and
// its epilogue; the next item's first S^T and dP^T run during that epilogue too.  The first dV / dK MMA of an
// item overwrites the accumulators instead of adding to them (no zero fill); it is issued only after the
// warpgroups have written that item's first P^T, which they do after reading the previous item's dK, dV out of
// tensor memory.  The epilogue stages dK * sm_scale and dV in the ring stages of the item's last q tile.
#include "sched.cuh"
#include "sm100.cuh"

namespace flexattn {
namespace FLEXATTN_TU_NAMESPACE {

constexpr int kThreads = 384;  // warps 0-3, 4-7: element-wise warpgroups (64 query columns each); 8: MMA; 9: TMA; 10, 11: idle
constexpr int kMmaWarp = 8, kTmaWarp = 9;

constexpr long long kDkvL2Budget = 32ll << 20;  // Q + dO bytes live at a time (sets the head group size of the item list)

struct DkvSmem {
  uint64_t bar_kv, bar_kvfree, bar_q[2], bar_do[2], bar_qfree[2], bar_dofree[2], bar_s, bar_dp, bar_p, bar_ds, bar_acc,
      bar_epi[2];
  uint32_t tmem_base;
  int32_t item_tiles[8];  // q tiles of the CTA's non-empty items (ring; -1 ends the list), producer -> MMA issuer
  alignas(16) float nlse2[2][kTile];  // -(m log2e + log2 l) of the query rows of the tile in flight
  alignas(16) float delta[2][kTile];
  alignas(16) int32_t doc[2][kTile];
};

// Query statistics are read from shared memory 32 columns at a time INTO REGISTERS before they are needed: the
// S^T / dP^T MMAs take both operands from shared memory and saturate its bandwidth, so a shared-memory load
// issued in the middle of the element-wise loop waits a long time.
__device__ __forceinline__ void load_stats32(float (&dst)[32], const float* __restrict__ src) {
#pragma unroll
  for (int c = 0; c < 32; c += 4) {
    const float4 t = *reinterpret_cast<const float4*>(src + c);
    dst[c] = t.x;
    dst[c + 1] = t.y;
    dst[c + 2] = t.z;
    dst[c + 3] = t.w;
  }
}

// First element-wise phase, 32 columns: this thread's key row against query columns i_first .. i_first+31.
// s: raw S^T values in, p * dsigma (the factor dS^T needs) out; pk_p: packed bf16 P^T.  The mask functor is
// compiled in only for partial tiles.
// what a user score function sees besides the score and the positions
struct ScoreCtx {
  float sm_scale;
  int b, h;
};

// kBias: ab_col points at the dense bias element (query i_first, key j) of this thread's key (nullptr: none, or a
// key past the end); consecutive queries are ab_stride floats apart, so a warp (32 consecutive keys) reads 128
// contiguous bytes per query.
template <int SK, int MK, bool kPartial, bool kBias = false>
__device__ __forceinline__ void dkv_p_math32(uint32_t (&s)[32], uint32_t* __restrict__ pk_p, const float (&nl)[32],
                                             const int32_t* __restrict__ s_doc, int i_first, int j, int dj, int seq_q,
                                             int window, int stride, float c2, float slope2, float abase, float capl2,
                                             float csc, const ScoreCtx ctx, const float* __restrict__ ab_col = nullptr,
                                             size_t ab_stride = 0) {
  if constexpr (SK == FLEXATTN_SCORE_SOFTCAP || SK == FLEXATTN_SCORE_USER) {
    // scalar form: the packed one costs registers here (tanh, its derivative and the mask live together)
#pragma unroll
    for (int c = 0; c < 32; c += 2) {
      float pv[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int cc = c + u;
        float arg, dsig;  // log2-domain logit minus the row's log-sum-exp; derivative of the score function
        if constexpr (SK == FLEXATTN_SCORE_USER) {
          const float sc = __uint_as_float(s[cc]) * ctx.sm_scale;
          arg = fmaf(user_score(sc, ctx.b, ctx.h, i_first + cc, j), kLog2e, nl[cc]);
          dsig = user_dscore(sc, ctx.b, ctx.h, i_first + cc, j);
        } else {
          const float th = ptx::tanh_approx(__uint_as_float(s[cc]) * csc);
          arg = fmaf(capl2, th, nl[cc]);
          dsig = fmaf(-th, th, 1.f);
        }
        if constexpr (kBias) {
          if (ab_col != nullptr && i_first + cc < seq_q) arg = fmaf(__ldg(ab_col + (size_t)cc * ab_stride), kLog2e, arg);
        }
        float p = ptx::ex2(arg);
        if constexpr (kPartial) {
          const int i = i_first + cc;
          const int di = (MK == FLEXATTN_MASK_DOCUMENT) ? s_doc[cc] : 0;
          p = ((i < seq_q) && mask_keep<MK>(i, j, window, stride, di, dj)) ? p : 0.f;
        }
        pv[u] = p;
        s[cc] = __float_as_uint(p * dsig);
      }
      pk_p[c >> 1] = ptx::pack_bf16_trunc(pv[0], pv[1]);
    }
    return;
  }
  // two columns per instruction (packed f32x2) wherever the arithmetic allows it
  const uint64_t c22 = ptx::pack2(c2, c2);
#pragma unroll
  for (int c = 0; c < 32; c += 2) {
    const uint64_t sv2 = ptx::pack2(__uint_as_float(s[c]), __uint_as_float(s[c + 1]));
    const uint64_t nl2 = ptx::pack2(nl[c], nl[c + 1]);
    uint64_t arg2;  // arg = log2-domain logit minus the row's log-sum-exp
    if constexpr (SK == FLEXATTN_SCORE_ALIBI) {
      // bias = abase - slope2 * column: the column part is a compile-time pair
      const uint64_t b2 = ptx::fma2(ptx::pack2(-(float)c, -(float)(c + 1)), ptx::pack2(slope2, slope2), ptx::pack2(abase, abase));
      arg2 = ptx::fma2(sv2, c22, ptx::add2(b2, nl2));
    } else {
      arg2 = ptx::fma2(sv2, c22, nl2);
    }
    float a0, a1;
    ptx::unpack2(arg2, a0, a1);
    if constexpr (kBias) {
      if (ab_col != nullptr) {
        if (i_first + c < seq_q) a0 = fmaf(__ldg(ab_col + (size_t)c * ab_stride), kLog2e, a0);
        if (i_first + c + 1 < seq_q) a1 = fmaf(__ldg(ab_col + (size_t)(c + 1) * ab_stride), kLog2e, a1);
      }
    }
    float p0 = ptx::ex2(a0), p1 = ptx::ex2(a1);
    if constexpr (kPartial) {
      const int i = i_first + c;
      const int d0 = (MK == FLEXATTN_MASK_DOCUMENT) ? s_doc[c] : 0, d1 = (MK == FLEXATTN_MASK_DOCUMENT) ? s_doc[c + 1] : 0;
      p0 = ((i < seq_q) && mask_keep<MK>(i, j, window, stride, d0, dj)) ? p0 : 0.f;
      p1 = ((i + 1 < seq_q) && mask_keep<MK>(i + 1, j, window, stride, d1, dj)) ? p1 : 0.f;
    }
    pk_p[c >> 1] = ptx::pack_bf16_trunc(p0, p1);
    s[c] = __float_as_uint(p0);
    s[c + 1] = __float_as_uint(p1);
  }
}

// Second phase, 32 columns: dS^T = (p dsigma) * (dP^T - delta), packed bf16.
__device__ __forceinline__ void dkv_ds_math32(const uint32_t (&pd)[32], const uint32_t (&pr)[32],
                                              uint32_t* __restrict__ pk_ds, const float (&dl)[32]) {
#pragma unroll
  for (int c = 0; c < 32; c += 2) {  // two columns per instruction (packed f32x2)
    float d0, d1;
    const uint64_t pd2 = ptx::pack2(__uint_as_float(pd[c]), __uint_as_float(pd[c + 1]));
    const uint64_t pr2 = ptx::pack2(__uint_as_float(pr[c]), __uint_as_float(pr[c + 1]));
    ptx::unpack2(ptx::mul2(pd2, ptx::sub2(pr2, ptx::pack2(dl[c], dl[c + 1]))), d0, d1);
    pk_ds[c >> 1] = ptx::pack_bf16_trunc(d0, d1);
  }
}

template <int D, int SK, int MK>
__global__ void __launch_bounds__(kThreads, 1)
    dkv_sm100_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                     const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                     const __grid_constant__ CUtensorMap tm_dk, const __grid_constant__ CUtensorMap tm_dv,
                     const DevParams P, int* abort_flag) {
  constexpr int kPanels = D / 64;
  constexpr uint32_t kTileBytes = kPanels * ptx::kPanelBytes;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kColS = 0, kColDP = 128, kColDK = 256, kColDV = 384;
  using Cursor = ItemCursorT<true>;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sK = smem;
  uint8_t* sV = smem + kTileBytes;
  uint8_t* sQ = smem + 2 * kTileBytes;   // two stages
  uint8_t* sDO = smem + 4 * kTileBytes;  // two stages
  DkvSmem* sh = reinterpret_cast<DkvSmem*>(smem + 6 * kTileBytes);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (aborted_on_entry(abort_flag, P.status, 3)) return;

  if (tid == 0) {
    ptx::mbar_init(&sh->bar_kv, 1);
    ptx::mbar_init(&sh->bar_kvfree, 1);
    ptx::mbar_init(&sh->bar_s, 1);
    ptx::mbar_init(&sh->bar_dp, 1);
    ptx::mbar_init(&sh->bar_p, 8);    // one arrival per warp of the two warpgroups
    ptx::mbar_init(&sh->bar_ds, 8);
    ptx::mbar_init(&sh->bar_acc, 1);
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(&sh->bar_epi[s], 2);  // one arrival per warpgroup: its staging tile in ring stage s has been read

      ptx::mbar_init(&sh->bar_q[s], 1);
      ptx::mbar_init(&sh->bar_do[s], 1);
      ptx::mbar_init(&sh->bar_qfree[s], 1);
      ptx::mbar_init(&sh->bar_dofree[s], 1);
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

  // In every role: T = index of a q tile in this CTA's stream over all its items (ring stage T & 1, ring phase
  // (T >> 1) & 1, phase T & 1 of the per-tile barriers), ri = index of an item among the CTA's NON-EMPTY items
  // (phase ri & 1 of the per-item barriers).
  // Registers move from the third warpgroup (MMA issuer, producer, two idle warps that only complete it) to the two
  // element-wise ones: the kernel starts with 168 per thread, the single-thread roles need few, the 64-column math
  // wants more than 168.
  if (warp >= 8) {
  ptx::setmaxnreg_dec<56>();
  if (warp == kTmaWarp) {
    // ------------------------------------------------------------------ TMA producer
    // Q and dO have rings of their own: the Q stage of tile T is free once dK(T) has run, the dO stage once
    // dV(T) has, and each is refilled (tile T+2) as soon as that happens - unless the tile was the last of its
    // item, whose epilogue stages the item's dK / dV in exactly those two stages: then also once the bulk stores
    // have read them.
    if (lane == 0) {
      bool ok = true;
      int fail_at = 20;
      ptx::prefetch_tensormap(&tm_q);
      ptx::prefetch_tensormap(&tm_do);
      ptx::prefetch_tensormap(&tm_k);
      ptx::prefetch_tensormap(&tm_v);
      auto load_tile = [&](uint8_t* dst, const CUtensorMap* tm, uint64_t* bar, int row0, int bh) {
        ptx::mbar_arrive_expect_tx(bar, kTileBytes);
#pragma unroll
        for (int p = 0; p < kPanels; ++p) ptx::tma_load_3d(dst + p * ptx::kPanelBytes, tm, bar, p * 64, row0, bh);
      };
      int T = 0, ri = 0;
      // ring stage s is (also) the staging tile of an item's epilogue: the tile loaded into it last was the item's
      // last.  One barrier per stage: a completion (the stores have read the stage) is always followed by this
      // thread's wait before anything else can be loaded into that stage, so waits and completions alternate.
      bool epi_pending[2] = {false, false};
      uint32_t epi_phase[2] = {0u, 0u};
      for (Cursor it(P, kDkvL2Budget); ok; it.next(), ++ri) {
        it.skip_empty();
        if (!it.valid()) break;
        const int bh = it.bh(), kt = it.qt(), first = it.rm.x, N = it.tiles();
        if (ri >= 1) {  // K, V of the previous item: its last S^T and dP^T must have completed
          ok = ptx::mbar_wait_relaxed(&sh->bar_kvfree, (uint32_t)((ri - 1) & 1));
          if (!ok) { fail_at = 21; break; }
        }
        sh->item_tiles[ri & 7] = N;  // read by the MMA issuer after it has waited on bar_kv (release / acquire)
        ptx::mbar_arrive_expect_tx(&sh->bar_kv, 2 * kTileBytes);
#pragma unroll
        for (int p = 0; p < kPanels; ++p) {
          ptx::tma_load_3d(sK + p * ptx::kPanelBytes, &tm_k, &sh->bar_kv, p * 64, kt * kTile, bh);
          ptx::tma_load_3d(sV + p * ptx::kPanelBytes, &tm_v, &sh->bar_kv, p * 64, kt * kTile, bh);
        }
        for (int n = 0; n < N && ok; ++n, ++T) {
          const int st = T & 1;
          const uint32_t par = ((T - 2) >> 1) & 1;
          if (T >= 2) {
            if (epi_pending[st]) {  // the stage pair also served as the staging tiles of an item's epilogue
              ok = ptx::mbar_wait_relaxed(&sh->bar_epi[st], epi_phase[st]);
              if (!ok) { fail_at = 22; break; }
              epi_phase[st] ^= 1u;
            }
            // dV(T-2) is issued before dK(T-2): the dO stage frees first
            ok = ptx::mbar_wait_relaxed(&sh->bar_dofree[st], par);
            if (!ok) { fail_at = 23; break; }
          }
          // order of first use within a tile: Q (for S^T), then dO (for dP^T); the dO stage frees first, though
          if (T >= 2) {
            load_tile(sDO + st * kTileBytes, &tm_do, &sh->bar_do[st], (first + n) * kTile, bh);
            ok = ptx::mbar_wait_relaxed(&sh->bar_qfree[st], par);
            if (!ok) { fail_at = 24; break; }
            load_tile(sQ + st * kTileBytes, &tm_q, &sh->bar_q[st], (first + n) * kTile, bh);
          } else {
            load_tile(sQ + st * kTileBytes, &tm_q, &sh->bar_q[st], (first + n) * kTile, bh);
            load_tile(sDO + st * kTileBytes, &tm_do, &sh->bar_do[st], (first + n) * kTile, bh);
          }
          epi_pending[st] = (n == N - 1);
        }
      }
      if (ok) {
        // End of the list: one more completion of the K/V barrier, carrying the terminator.  Like a real item it
        // waits for the barrier's previous phase to be over (its bytes landed and consumed) before arriving on it
        // again: an arrive into a phase that still expects bytes would corrupt it.
        if (ri >= 1) ok = ptx::mbar_wait_relaxed(&sh->bar_kvfree, (uint32_t)((ri - 1) & 1));
        if (ok) {
          sh->item_tiles[ri & 7] = -1;
          ptx::mbar_arrive(&sh->bar_kv);
        } else {
          fail_at = 25;
        }
      }
      if (!ok) give_up(abort_flag, P.status, 3, fail_at);
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer
    // It learns each item's tile count from the producer (item_tiles, valid once bar_kv of the item has completed)
    // and does no index arithmetic of its own.
    if (lane == 0) {
      bool ok = true;
      int fail_at = 1;
      constexpr uint32_t idesc_s = ptx::make_idesc(128, 128, false);
      constexpr uint32_t idesc_acc = ptx::make_idesc(128, D, true);
      const uint32_t aQ = ptx::smem_u32(sQ), aDO = ptx::smem_u32(sDO);
      const ptx::DescBase bK = ptx::base_kmajor(ptx::smem_u32(sK)), bV = ptx::base_kmajor(ptx::smem_u32(sV));
      auto issue_s = [&](int t) {  // S^T = K Q^T
        const ptx::DescBase bQ = ptx::base_kmajor(aQ + (uint32_t)(t & 1) * kTileBytes);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          ptx::mma_ss(tmem + kColS, ptx::desc_at(bK, ptx::koff_kmajor(kk)), ptx::desc_at(bQ, ptx::koff_kmajor(kk)),
                      idesc_s, kk > 0);
        ptx::mma_commit(&sh->bar_s);
      };
      auto issue_dp = [&](int t) {  // dP^T = V dO^T
        const ptx::DescBase bDO = ptx::base_kmajor(aDO + (uint32_t)(t & 1) * kTileBytes);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          ptx::mma_ss(tmem + kColDP, ptx::desc_at(bV, ptx::koff_kmajor(kk)), ptx::desc_at(bDO, ptx::koff_kmajor(kk)),
                      idesc_s, kk > 0);
        ptx::mma_commit(&sh->bar_dp);
      };
      // A operand of the accumulation MMAs: packed bf16, 8 columns per K step of 16 query rows; warpgroup w wrote
      // query columns [64w, 64w+64) at column offset 64w of the S^T / dP^T block.  `first`: the item's first q
      // tile, whose MMA overwrites the accumulator instead of adding to it.
      auto issue_dv = [&](int t, bool first) {  // dV (+)= P^T dO
        const ptx::DescBase bDOt = ptx::base_mnmajor(aDO + (uint32_t)(t & 1) * kTileBytes);
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk)
          ptx::mma_ts(tmem + kColDV, tmem + kColS + 64 * (kk >> 2) + (kk & 3) * 8,
                      ptx::desc_at(bDOt, ptx::koff_mnmajor(kk)), idesc_acc, (!first) || (kk > 0));
        ptx::mma_commit(&sh->bar_dofree[t & 1]);
      };
      auto issue_dk = [&](int t, bool first) {  // dK (+)= dS^T Q
        const ptx::DescBase bQt = ptx::base_mnmajor(aQ + (uint32_t)(t & 1) * kTileBytes);
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk)
          ptx::mma_ts(tmem + kColDK, tmem + kColDP + 64 * (kk >> 2) + (kk & 3) * 8,
                      ptx::desc_at(bQt, ptx::koff_mnmajor(kk)), idesc_acc, (!first) || (kk > 0));
        ptx::mma_commit(&sh->bar_qfree[t & 1]);
      };
      int T = 0, ri = 0;  // first tile of the current item in the stream; item index
      // Waits for K, V of item ri, reads its tile count, then issues the item's first S^T and dP^T.  -1: end of list.
      auto start_item = [&]() -> int {
        ok = ptx::mbar_wait(&sh->bar_kv, (uint32_t)(ri & 1));
        if (!ok) { fail_at = 2; return -1; }
        const int n_tiles = sh->item_tiles[ri & 7];
        if (n_tiles < 0) return -1;
        ok = ptx::mbar_wait(&sh->bar_q[T & 1], (uint32_t)((T >> 1) & 1));
        if (!ok) { fail_at = 3; return -1; }
        ptx::tc_fence_after();
        issue_s(T);
        ok = ptx::mbar_wait(&sh->bar_do[T & 1], (uint32_t)((T >> 1) & 1));
        if (!ok) { fail_at = 5; return -1; }
        ptx::tc_fence_after();
        issue_dp(T);
        if (n_tiles == 1) ptx::mma_commit(&sh->bar_kvfree);  // K, V are not read again by this item
        return n_tiles;
      };
      int N = start_item();
      while (ok && N > 0) {
        for (int n = 0; n < N && ok; ++n) {
          const int t = T + n;
          const uint32_t par = t & 1;
          const uint32_t par_next = ((t + 1) >> 1) & 1;
          ok = ptx::mbar_wait(&sh->bar_p, par);  // P^T(t) is in tensor memory
          if (!ok) { fail_at = 6; break; }
          ptx::tc_fence_after();
          issue_dv(t, n == 0);
          if (n + 1 < N) {
            ok = ptx::mbar_wait(&sh->bar_q[(t + 1) & 1], par_next);
            if (!ok) { fail_at = 3; break; }
            ptx::tc_fence_after();
            issue_s(t + 1);
          }
          ok = ptx::mbar_wait(&sh->bar_ds, par);  // dS^T(t) is in tensor memory
          if (!ok) { fail_at = 4; break; }
          ptx::tc_fence_after();
          issue_dk(t, n == 0);
          if (n + 1 < N) {
            ok = ptx::mbar_wait(&sh->bar_do[(t + 1) & 1], par_next);
            if (!ok) { fail_at = 5; break; }
            ptx::tc_fence_after();
            issue_dp(t + 1);
            if (n + 2 == N) ptx::mma_commit(&sh->bar_kvfree);  // the item's last S^T and dP^T have been issued
          }
        }
        if (!ok) break;
        ptx::mma_commit(&sh->bar_acc);  // every MMA of the item
        T += N;
        ++ri;
        N = start_item();
      }
      if (!ok) give_up(abort_flag, P.status, 3, fail_at);
    }
  }
  } else {
    // ------------------------------------------------------------------ element-wise warpgroups
    ptx::setmaxnreg_inc<224>();
    const int row = tid & 127;        // key row inside the tile = TMEM lane
    const int half = tid >> 7;        // which 64 query columns of every tile this warpgroup handles
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t colS = kColS + 64 * half, colDP = kColDP + 64 * half;
    const float c2 = P.sm_scale * kLog2e;
    const float capl2 = P.cap * kLog2e;
    const float csc = (SK == FLEXATTN_SCORE_SOFTCAP) ? P.sm_scale / P.cap : 0.f;
    bool ok = true;
    int fail_at = 0;
    int T = 0, ri = 0;  // stream index of the item's first q tile; index among the non-empty items

    for (Cursor it(P, kDkvL2Budget); it.valid(); it.next()) {
      const int kt = it.qt(), bh = it.bh(), b = bh / P.heads, h = bh % P.heads;
      const int4 cm = it.rm;
      const int N = cm.y - cm.x;
      const int j = kt * kTile + row;   // global key position
      const bool row_ok = j < P.seq_k;
      const float slope2 = (SK == FLEXATTN_SCORE_ALIBI) ? P.alibi_slopes[h] * kLog2e : 0.f;
      const int32_t* doc = (MK == FLEXATTN_MASK_DOCUMENT) ? P.doc_ids + (size_t)b * P.doc_stride : nullptr;
      const int dj = (MK == FLEXATTN_MASK_DOCUMENT && row_ok) ? doc[j] : -2;
      const ScoreCtx ctx{P.sm_scale, b, h};

      // Statistics of the query rows (l, m, delta, document id) are fetched from global memory one tile ahead
      // into registers, so their latency is off the critical path (except for an item's first tile).
      const size_t stat_base = (size_t)bh * P.seq_q;
      // Division of the staging work inside a warpgroup (all of it one tile ahead): threads 0..63 own one query row
      // each for -(m log2e + log2 l) - l and m fetched into registers a tile earlier, one shared-memory store;
      // threads 64..127 own one row each for delta (and the document id), which needs no arithmetic and goes
      // global -> shared with cp.async, costing the thread nothing.  Shared-memory stores are slow while the MMAs
      // saturate shared memory, so no warp issues more than one per tile.  n: tile inside the item; the staging
      // buffer is that of its stream index.
      float pf_l = 0.f, pf_m = 0.f;
      bool pf_ok = false;
      auto fetch_stats = [&](int n) {  // threads 0..63
        const int i = (cm.x + n) * kTile + 64 * half + row;
        pf_ok = i < P.seq_q;
        if (pf_ok) {
          pf_l = P.l[stat_base + i];
          pf_m = P.m[stat_base + i];
        }
      };
      auto stage_stats = [&](int n) {
        const int st = (T + n) & 1;
        if (row < 64) {
          // pre-scaled for pack_bf16_trunc; l == 0 (fully masked row) forces p to 0
          sh->nlse2[st][64 * half + row] =
              pf_ok ? (pf_l > 0.f ? ptx::kRoundLog2 - fmaf(pf_m, kLog2e, log2f(pf_l)) : -1.0e30f) : ptx::kRoundLog2;
        } else {
          const int r = row - 64;
          const int i = (cm.x + n) * kTile + 64 * half + r;
          if (i < P.seq_q) {
            ptx::cp_async4(&sh->delta[st][64 * half + r], &P.delta[stat_base + i]);
            if (MK == FLEXATTN_MASK_DOCUMENT) ptx::cp_async4(&sh->doc[st][64 * half + r], &doc[i]);
          } else {
            sh->delta[st][64 * half + r] = 0.f;
            if (MK == FLEXATTN_MASK_DOCUMENT) sh->doc[st][64 * half + r] = -1;
          }
        }
      };
      if (N > 0) {
        if (row < 64) fetch_stats(0);
        stage_stats(0);
        if (row < 64 && N > 1) fetch_stats(1);
      }

      for (int n = 0; n < N; ++n) {
        const int t = T + n, st = t & 1;
        const int qt = cm.x + n, i0 = qt * kTile + 64 * half;  // first query position of this warpgroup's columns
        const bool partial = P.ab != nullptr || !(qt >= cm.z && qt < cm.w);  // with a dense bias: always the masked form
        // the statistics of this tile were staged during the previous tile (or before the loop)
        // a failed wait never leaves the loop early: every thread keeps executing the same named barriers
        ptx::cp_async_wait_all();  // this thread's asynchronous copies for this tile have landed
        ptx::named_bar_sync(1 + half, 128);
        if (!ok) continue;
        float st0[32], st1[32];
        load_stats32(st0, &sh->nlse2[st][64 * half]);
        ok = __all_sync(0xffffffffu, ptx::mbar_wait(&sh->bar_s, (uint32_t)(t & 1)));
        if (!ok) { fail_at = 10; continue; }
        ptx::tc_fence_after();
        uint32_t sr[2][32];
        ptx::tmem_ld32(lane_base + colS, sr[0]);
        ptx::tmem_ld32(lane_base + colS + 32, sr[1]);
        load_stats32(st1, &sh->nlse2[st][64 * half + 32]);
        ptx::tmem_wait_ld();
        ptx::tmem_ld_acquire(sr[0]);
        ptx::tmem_ld_acquire(sr[1]);
        {
          uint32_t pk_p[32];
          const float abase = slope2 * (float)(j - i0);  // ALiBi bias = slope * (j - i), i = i0 + column
          if (P.ab != nullptr) {
            // element (query i0, key j) of the dense bias; nullptr for a key past the end of the sequence
            const float* ab_col = row_ok ? P.ab + ((size_t)bh * P.seq_q + i0) * P.seq_k + j : nullptr;
            dkv_p_math32<SK, MK, true, true>(sr[0], pk_p, st0, &sh->doc[st][64 * half], i0, j, dj, P.seq_q, P.window,
                                             P.stride, c2, slope2, abase, capl2, csc, ctx, ab_col, (size_t)P.seq_k);
            dkv_p_math32<SK, MK, true, true>(sr[1], pk_p + 16, st1, &sh->doc[st][64 * half + 32], i0 + 32, j, dj, P.seq_q,
                                             P.window, P.stride, c2, slope2, abase - 32.f * slope2, capl2, csc, ctx,
                                             ab_col != nullptr ? ab_col + 32 * (size_t)P.seq_k : nullptr, (size_t)P.seq_k);
          } else if (partial) {
            dkv_p_math32<SK, MK, true>(sr[0], pk_p, st0, &sh->doc[st][64 * half], i0, j, dj, P.seq_q, P.window,
                                       P.stride, c2, slope2, abase, capl2, csc, ctx);
            dkv_p_math32<SK, MK, true>(sr[1], pk_p + 16, st1, &sh->doc[st][64 * half + 32], i0 + 32, j, dj, P.seq_q,
                                       P.window, P.stride, c2, slope2, abase - 32.f * slope2, capl2, csc, ctx);
          } else {
            dkv_p_math32<SK, MK, false>(sr[0], pk_p, st0, &sh->doc[st][64 * half], i0, j, dj, P.seq_q, P.window,
                                        P.stride, c2, slope2, abase, capl2, csc, ctx);
            dkv_p_math32<SK, MK, false>(sr[1], pk_p + 16, st1, &sh->doc[st][64 * half + 32], i0 + 32, j, dj, P.seq_q,
                                        P.window, P.stride, c2, slope2, abase - 32.f * slope2, capl2, csc, ctx);
          }
          ptx::tmem_st32(lane_base + colS, pk_p);  // bf16 P^T over the first half of this warpgroup's S^T columns
          ptx::tmem_wait_st();
          ptx::tc_fence_before();
          ptx::mbar_arrive_warp(&sh->bar_p);
        }
        // While dP^T of this tile is still being computed: stage the statistics of the NEXT tile (its stage was last
        // read two tiles ago) and fetch those of the one after.  Done here, the shared-memory stores - slow while
        // the MMAs saturate shared memory - overlap a wait instead of delaying the first phase.
        if (n + 1 < N) {
          stage_stats(n + 1);
          if (row < 64 && n + 2 < N) fetch_stats(n + 2);
        }
        load_stats32(st0, &sh->delta[st][64 * half]);
        ok = __all_sync(0xffffffffu, ptx::mbar_wait(&sh->bar_dp, (uint32_t)(t & 1)));
        if (!ok) { fail_at = 11; continue; }
        ptx::tc_fence_after();
        {
          uint32_t pr[32], pk_ds[32];
          ptx::tmem_ld32(lane_base + colDP, pr);
          load_stats32(st1, &sh->delta[st][64 * half + 32]);
          ptx::tmem_wait_ld();
          ptx::tmem_ld_acquire(pr);
          dkv_ds_math32(sr[0], pr, pk_ds, st0);
          ptx::tmem_ld32(lane_base + colDP + 32, pr);
          ptx::tmem_wait_ld();
          ptx::tmem_ld_acquire(pr);
          dkv_ds_math32(sr[1], pr, pk_ds + 16, st1);
          ptx::tmem_st32(lane_base + colDP, pk_ds);
          ptx::tmem_wait_st();
          ptx::tc_fence_before();
          ptx::mbar_arrive_warp(&sh->bar_ds);
        }
      }

      // ---- item epilogue.  Warpgroup 0 stores dK * sm_scale, warpgroup 1 dV: bf16 into a shared-memory tile in the
      // TMA (128-byte swizzle) layout, then one bulk tensor store per 64-column panel; rows past seq_k are clipped by
      // the tensor map.  The staging tiles are the Q / dO ring stages of the item's last q tile: free once every MMA
      // of the item has completed, and not refilled by the producer before the stores have read them (bar_epi of that stage).
      if (N > 0) {
        if (ok) {
          ok = __all_sync(0xffffffffu, ptx::mbar_wait(&sh->bar_acc, (uint32_t)(ri & 1)));
          if (!ok) fail_at = 12;
        }
        uint8_t* stage = (half ? sDO : sQ) + (uint32_t)((T + N - 1) & 1) * kTileBytes;
        if (ok) {
          ptx::tc_fence_after();
          const float sc = half ? 1.f : P.sm_scale;
          const uint32_t col0 = half ? kColDV : kColDK;
          uint8_t* stage_row = stage + row * 128;
#pragma unroll 1
          for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t r[32];
            ptx::tmem_ld32(lane_base + col0 + c0, r);
            ptx::tmem_wait_ld();
            ptx::tmem_ld_acquire(r);
#pragma unroll
            for (int c = 0; c < 32; c += 8) {
              uint4 v4;
              v4.x = ptx::pack_bf16(__uint_as_float(r[c]) * sc, __uint_as_float(r[c + 1]) * sc);
              v4.y = ptx::pack_bf16(__uint_as_float(r[c + 2]) * sc, __uint_as_float(r[c + 3]) * sc);
              v4.z = ptx::pack_bf16(__uint_as_float(r[c + 4]) * sc, __uint_as_float(r[c + 5]) * sc);
              v4.w = ptx::pack_bf16(__uint_as_float(r[c + 6]) * sc, __uint_as_float(r[c + 7]) * sc);
              const int col = c0 + c, panel = col >> 6, chunk = (col & 63) >> 3;
              *reinterpret_cast<uint4*>(stage_row + panel * ptx::kPanelBytes + ((chunk ^ (row & 7)) << 4)) = v4;
            }
          }
          ptx::tc_fence_before();         // the accumulators have been read: the next item's first MMAs may overwrite them
          ptx::fence_proxy_async_smem();  // generic-proxy stores -> visible to the bulk store
        }
        ptx::named_bar_sync(1 + half, 128);
        if (ok && row == 0) {
#pragma unroll
          for (int p = 0; p < kPanels; ++p)
            ptx::tma_store_3d(half ? &tm_dv : &tm_dk, stage + p * ptx::kPanelBytes, p * 64, kt * kTile, bh);
          ptx::tma_store_commit();
          ptx::tma_store_wait_read();  // shared memory must stay intact until the store has read it
          ptx::mbar_arrive(&sh->bar_epi[(T + N - 1) & 1]);
        }
        T += N;
        ++ri;
      } else if (ok && row_ok) {
        // a kv tile no query attends to: zero gradients, written directly (warpgroup 0: dK, warpgroup 1: dV)
        uint16_t* out = static_cast<uint16_t*>(half ? P.dv : P.dk) + ((size_t)bh * P.seq_k + j) * D;
        for (int c0 = 0; c0 < D; c0 += 8) *reinterpret_cast<uint4*>(out + c0) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    if (!ok && lane == 0) give_up(abort_flag, P.status, 3, fail_at);
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
               const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdk, const CUtensorMap& tdv,
               int* abort_flag) {
  constexpr size_t smem = 6 * (D / 64) * ptx::kPanelBytes + sizeof(DkvSmem) + 1024;
  // 512 TMEM columns per CTA: never let two CTAs share an SM (the second would spin in tcgen05.alloc)
  constexpr size_t smem_req = smem > 120 * 1024 ? smem : 120 * 1024;
  auto kern = dkv_sm100_kernel<D, SK, MK>;
  static SmemAttrOnce attr_once{};  // per kernel instantiation, per device
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), (int)smem_req, &attr_once) != FLEXATTN_OK) return FLEXATTN_ERR_CUDA;
  // persistent: one CTA per SM (fewer when there are fewer work items)
  const long long items = (long long)d.n_kt * d.batch * d.heads;
  const int sms = sm_count();
  if (sms <= 0) return FLEXATTN_ERR_CUDA;
  dim3 grid((unsigned)(items < sms ? items : sms));
  kern<<<grid, kThreads, smem_req, st>>>(tq, tdo, tk, tv, tdk, tdv, d, abort_flag);
  return cudaGetLastError() == cudaSuccess ? FLEXATTN_OK : FLEXATTN_ERR_CUDA;
}

template <int D, int SK>
int launch_mask(cudaStream_t st, const DevParams& d, int mask, const CUtensorMap& tq, const CUtensorMap& tdo,
                const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdk, const CUtensorMap& tdv, int* af) {
  switch (mask) {
    case FLEXATTN_MASK_NONE: return launch_one<D, SK, FLEXATTN_MASK_NONE>(st, d, tq, tdo, tk, tv, tdk, tdv, af);
    case FLEXATTN_MASK_CAUSAL: return launch_one<D, SK, FLEXATTN_MASK_CAUSAL>(st, d, tq, tdo, tk, tv, tdk, tdv, af);
    case FLEXATTN_MASK_SLIDING_WINDOW: return launch_one<D, SK, FLEXATTN_MASK_SLIDING_WINDOW>(st, d, tq, tdo, tk, tv, tdk, tdv, af);
    case FLEXATTN_MASK_SLIDING_WINDOW_CAUSAL:
      return launch_one<D, SK, FLEXATTN_MASK_SLIDING_WINDOW_CAUSAL>(st, d, tq, tdo, tk, tv, tdk, tdv, af);
    case FLEXATTN_MASK_DOCUMENT: return launch_one<D, SK, FLEXATTN_MASK_DOCUMENT>(st, d, tq, tdo, tk, tv, tdk, tdv, af);
    case FLEXATTN_MASK_S2: return launch_one<D, SK, FLEXATTN_MASK_S2>(st, d, tq, tdo, tk, tv, tdk, tdv, af);
    default: return FLEXATTN_ERR_UNSUPPORTED_MOD;
  }
}

template <int D>
int launch_score(cudaStream_t st, const DevParams& d, int score, int mask, const CUtensorMap& tq,
                 const CUtensorMap& tdo, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdk, const CUtensorMap& tdv, int* af) {
  switch (score) {
    case FLEXATTN_SCORE_NONE: return launch_mask<D, FLEXATTN_SCORE_NONE>(st, d, mask, tq, tdo, tk, tv, tdk, tdv, af);
    case FLEXATTN_SCORE_ALIBI: return launch_mask<D, FLEXATTN_SCORE_ALIBI>(st, d, mask, tq, tdo, tk, tv, tdk, tdv, af);
    case FLEXATTN_SCORE_SOFTCAP: return launch_mask<D, FLEXATTN_SCORE_SOFTCAP>(st, d, mask, tq, tdo, tk, tv, tdk, tdv, af);
    default: return FLEXATTN_ERR_UNSUPPORTED_MOD;
  }
}

#endif  // !FLEXATTN_JIT

}  // namespace FLEXATTN_TU_NAMESPACE

#ifndef FLEXATTN_JIT
int launch_sm100_dkv(cudaStream_t st, const DevParams& d, int score, int mask) {
  int* af = abort_flag_ptr();
  if (af == nullptr) return FLEXATTN_ERR_CUDA;
  CUtensorMap tq, tdo, tk, tv, tdk, tdv;
  const int slices = d.batch * d.heads;
  int e = make_tile_map(&tq, d.q, slices, d.seq_q, d.head_dim);
  if (e) return e;
  e = make_tile_map(&tdo, d.d_o, slices, d.seq_q, d.head_dim);
  if (e) return e;
  e = make_tile_map(&tk, d.k, slices, d.seq_k, d.head_dim);
  if (e) return e;
  e = make_tile_map(&tv, d.v, slices, d.seq_k, d.head_dim);
  if (e) return e;
  e = make_tile_map(&tdk, d.dk, slices, d.seq_k, d.head_dim);
  if (e) return e;
  e = make_tile_map(&tdv, d.dv, slices, d.seq_k, d.head_dim);
  if (e) return e;
  if (score == FLEXATTN_SCORE_USER) {
    // a kernel compiled at run time around the registered score function: same parameters, grid and shared memory
    const size_t need = 6 * (size_t)(d.head_dim / 64) * ptx::kPanelBytes + sizeof(DkvSmem) + 1024;
    const long long items = (long long)d.n_kt * d.batch * d.heads;
    const int sms = sm_count();
    if (sms <= 0) return FLEXATTN_ERR_CUDA;
    void* args[] = {&tq, &tdo, &tk, &tv, &tdk, &tdv, const_cast<DevParams*>(&d), &af};
    return jit_launch(2, d.user_score, d.head_dim, mask, (unsigned)(items < sms ? items : sms), 1, kThreads,
                      need > 120 * 1024 ? need : 120 * 1024, st, args);
  }
  if (d.head_dim == 128) return launch_score<128>(st, d, score, mask, tq, tdo, tk, tv, tdk, tdv, af);
  if (d.head_dim == 64) return launch_score<64>(st, d, score, mask, tq, tdo, tk, tv, tdk, tdv, af);
  return FLEXATTN_ERR_UNSUPPORTED_HEAD_DIM;
}
#endif  // !FLEXATTN_JIT

}  // namespace flexattn
