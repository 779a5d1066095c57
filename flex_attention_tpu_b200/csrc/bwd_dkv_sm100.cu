// dK / dV backward on the 5th-generation tensor cores (sm_100a).
//
// Replaces the reference's Pallas dK/dV kernel (flex_attention_dkv_kernel.py:177-280 and its mask-aware
// twin flash_attention_dkv_bwd.py:183-308).  One CTA owns one 128-row kv tile of one (batch, head): K and
// V stay in shared memory, Q and dO tiles stream through two-stage rings, and per q tile the TRANSPOSED
// score tile is formed so that the probabilities land in tensor memory in the layout the next MMA wants as
// its A operand:
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
// dK, dV (D columns each) stay in tensor memory across q tiles: 512 columns in total, one CTA per SM.
#include "sm100.cuh"

namespace flexattn {
namespace FLEXATTN_TU_NAMESPACE {

constexpr int kThreads = 320;  // warps 0-3, 4-7: element-wise warpgroups (64 query columns each); 8: MMA; 9: TMA
constexpr int kMmaWarp = 8, kTmaWarp = 9;

struct DkvSmem {
  uint64_t bar_kv, bar_q[2], bar_do[2], bar_qfree[2], bar_dofree[2], bar_s, bar_dp, bar_p, bar_ds, bar_acc, bar_zero;
  uint32_t tmem_base;
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
// kInterval: the key row's kept queries are the interval [qlo, qhi) (interval mask kinds; documents over sorted
// ids): a partial tile then tests one bit per element of a bitmap of the 32 columns.
template <int SK, int MK, bool kPartial, bool kBias = false, bool kInterval = kMaskIsInterval<MK>>
__device__ __forceinline__ void dkv_p_math32(uint32_t (&s)[32], uint32_t* __restrict__ pk_p, const float (&nl)[32],
                                             const int32_t* __restrict__ s_doc, int i_first, int j, int dj, int seq_q,
                                             int window, int stride, float c2, float slope2, float abase, float capl2,
                                             float csc, const ScoreCtx ctx, const float* __restrict__ ab_col = nullptr,
                                             size_t ab_stride = 0, int qlo = 0, int qhi = 0) {
  const uint32_t keep = (kPartial && kInterval) ? range_bits32(qlo - i_first, qhi - i_first) : 0u;
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
        if constexpr (kPartial && kInterval) {
          p = (keep >> cc) & 1u ? p : 0.f;
        } else if constexpr (kPartial) {
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
  // ALiBi: bias = abase - slope2 * column advances by a constant from pair to pair (one packed add per pair)
  uint64_t b2 = ptx::pack2(abase, abase - slope2);
  const uint64_t bstep2 = ptx::pack2(-2.f * slope2, -2.f * slope2);
#pragma unroll
  for (int c = 0; c < 32; c += 2) {
    const uint64_t sv2 = ptx::pack2(__uint_as_float(s[c]), __uint_as_float(s[c + 1]));
    const uint64_t nl2 = ptx::pack2(nl[c], nl[c + 1]);
    uint64_t arg2;  // arg = log2-domain logit minus the row's log-sum-exp
    if constexpr (SK == FLEXATTN_SCORE_ALIBI) {
      arg2 = ptx::fma2(sv2, c22, ptx::add2(b2, nl2));
      b2 = ptx::add2(b2, bstep2);
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
    if constexpr (kPartial && kInterval) {  // `keep`: one bitmap of this key row over the 32 query columns
      p0 = (keep >> c) & 1u ? p0 : 0.f;
      p1 = (keep >> (c + 1)) & 1u ? p1 : 0.f;
    } else if constexpr (kPartial) {
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

  if (aborted_on_entry(abort_flag, P.status, 3)) return;

  if (tid == 0) {
    ptx::mbar_init(&sh->bar_kv, 1);
    ptx::mbar_init(&sh->bar_zero, 8);
    ptx::mbar_init(&sh->bar_s, 1);
    ptx::mbar_init(&sh->bar_dp, 1);
    ptx::mbar_init(&sh->bar_p, 8);    // one arrival per warp of the two warpgroups
    ptx::mbar_init(&sh->bar_ds, 8);
    ptx::mbar_init(&sh->bar_acc, 1);
    for (int s = 0; s < 2; ++s) {
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

  if (warp == kTmaWarp) {
    // ------------------------------------------------------------------ TMA producer
    // Q and dO have rings of their own: the Q stage of tile n is free once dK(n) has run, the dO stage once
    // dV(n) has, and each is refilled (tile n+2) as soon as that happens.
    if (lane == 0 && N > 0) {
      bool ok = true;
      ptx::prefetch_tensormap(&tm_q);
      ptx::prefetch_tensormap(&tm_do);
      ptx::prefetch_tensormap(&tm_k);
      ptx::prefetch_tensormap(&tm_v);
      auto load_tile = [&](uint8_t* dst, const CUtensorMap* tm, uint64_t* bar, int row0) {
        ptx::mbar_arrive_expect_tx(bar, kTileBytes);
#pragma unroll
        for (int p = 0; p < kPanels; ++p) ptx::tma_load_3d(dst + p * ptx::kPanelBytes, tm, bar, p * 64, row0, bh);
      };
      // order of first use: K, Q(0), V, dO(0)
      ptx::mbar_arrive_expect_tx(&sh->bar_kv, 2 * kTileBytes);
#pragma unroll
      for (int p = 0; p < kPanels; ++p) ptx::tma_load_3d(sK + p * ptx::kPanelBytes, &tm_k, &sh->bar_kv, p * 64, kt * kTile, bh);
      load_tile(sQ, &tm_q, &sh->bar_q[0], cm.x * kTile);
#pragma unroll
      for (int p = 0; p < kPanels; ++p) ptx::tma_load_3d(sV + p * ptx::kPanelBytes, &tm_v, &sh->bar_kv, p * 64, kt * kTile, bh);
      load_tile(sDO, &tm_do, &sh->bar_do[0], cm.x * kTile);
      if (N > 1) {
        load_tile(sQ + kTileBytes, &tm_q, &sh->bar_q[1], (cm.x + 1) * kTile);
        load_tile(sDO + kTileBytes, &tm_do, &sh->bar_do[1], (cm.x + 1) * kTile);
      }
      for (int n = 2; n < N && ok; ++n) {
        const int st = n & 1;
        const uint32_t par = ((n - 2) >> 1) & 1;
        // dV(n-2) is issued before dK(n-2): the dO stage frees first
        ok = ptx::mbar_wait_relaxed(&sh->bar_dofree[st], par);
        if (!ok) break;
        load_tile(sDO + st * kTileBytes, &tm_do, &sh->bar_do[st], (cm.x + n) * kTile);
        ok = ptx::mbar_wait_relaxed(&sh->bar_qfree[st], par);
        if (!ok) break;
        load_tile(sQ + st * kTileBytes, &tm_q, &sh->bar_q[st], (cm.x + n) * kTile);
      }
      if (!ok) give_up(abort_flag, P.status, 3, 20);
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer
    // dK / dV are zeroed by the warpgroups first, so every accumulation MMA adds.
    if (lane == 0 && N > 0) {
      bool ok = true;
      int fail_at = 1;
      constexpr uint32_t idesc_s = ptx::make_idesc(128, 128, false);
      constexpr uint32_t idesc_acc = ptx::make_idesc(128, D, true);
      const uint32_t aQ = ptx::smem_u32(sQ), aDO = ptx::smem_u32(sDO);
      const ptx::DescBase bK = ptx::base_kmajor(ptx::smem_u32(sK)), bV = ptx::base_kmajor(ptx::smem_u32(sV));
      auto issue_s = [&](int n) {  // S^T = K Q^T
        const ptx::DescBase bQ = ptx::base_kmajor(aQ + (uint32_t)(n & 1) * kTileBytes);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          ptx::mma_ss(tmem + kColS, ptx::desc_at(bK, ptx::koff_kmajor(kk)), ptx::desc_at(bQ, ptx::koff_kmajor(kk)),
                      idesc_s, kk > 0);
        ptx::mma_commit(&sh->bar_s);
      };
      auto issue_dp = [&](int n) {  // dP^T = V dO^T
        const ptx::DescBase bDO = ptx::base_kmajor(aDO + (uint32_t)(n & 1) * kTileBytes);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          ptx::mma_ss(tmem + kColDP, ptx::desc_at(bV, ptx::koff_kmajor(kk)), ptx::desc_at(bDO, ptx::koff_kmajor(kk)),
                      idesc_s, kk > 0);
        ptx::mma_commit(&sh->bar_dp);
      };
      // A operand of the accumulation MMAs: packed bf16, 8 columns per K step of 16 query rows; warpgroup w wrote
      // query columns [64w, 64w+64) at column offset 64w of the S^T / dP^T block
      auto issue_dv = [&](int n) {  // dV += P^T dO
        const ptx::DescBase bDOt = ptx::base_mnmajor(aDO + (uint32_t)(n & 1) * kTileBytes);
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk)
          ptx::mma_ts(tmem + kColDV, tmem + kColS + 64 * (kk >> 2) + (kk & 3) * 8,
                      ptx::desc_at(bDOt, ptx::koff_mnmajor(kk)), idesc_acc, 1);
        ptx::mma_commit(&sh->bar_dofree[n & 1]);
      };
      auto issue_dk = [&](int n) {  // dK += dS^T Q
        const ptx::DescBase bQt = ptx::base_mnmajor(aQ + (uint32_t)(n & 1) * kTileBytes);
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk)
          ptx::mma_ts(tmem + kColDK, tmem + kColDP + 64 * (kk >> 2) + (kk & 3) * 8,
                      ptx::desc_at(bQt, ptx::koff_mnmajor(kk)), idesc_acc, 1);
        ptx::mma_commit(&sh->bar_qfree[n & 1]);
      };
      ok = ptx::mbar_wait(&sh->bar_kv, 0) && ptx::mbar_wait(&sh->bar_q[0], 0);
      if (ok) {
        ptx::tc_fence_after();
        issue_s(0);
        ok = ptx::mbar_wait(&sh->bar_do[0], 0);
      }
      if (ok) {
        ptx::tc_fence_after();
        issue_dp(0);
        ok = ptx::mbar_wait(&sh->bar_zero, 0);  // dK / dV columns zeroed
        if (!ok) fail_at = 7;
      }
      for (int n = 0; n < N && ok; ++n) {
        const uint32_t par = n & 1;
        const uint32_t par_next = ((n + 1) >> 1) & 1;
        ok = ptx::mbar_wait(&sh->bar_p, par);  // P^T(n) is in tensor memory
        if (!ok) { fail_at = 2; break; }
        ptx::tc_fence_after();
        issue_dv(n);
        if (n + 1 < N) {
          ok = ptx::mbar_wait(&sh->bar_q[(n + 1) & 1], par_next);
          if (!ok) { fail_at = 3; break; }
          ptx::tc_fence_after();
          issue_s(n + 1);
        }
        ok = ptx::mbar_wait(&sh->bar_ds, par);  // dS^T(n) is in tensor memory
        if (!ok) { fail_at = 4; break; }
        ptx::tc_fence_after();
        issue_dk(n);
        if (n + 1 < N) {
          ok = ptx::mbar_wait(&sh->bar_do[(n + 1) & 1], par_next);
          if (!ok) { fail_at = 5; break; }
          ptx::tc_fence_after();
          issue_dp(n + 1);
        }
      }
      if (ok) ptx::mma_commit(&sh->bar_acc);
      if (!ok) give_up(abort_flag, P.status, 3, fail_at);
    }
  } else {
    // ------------------------------------------------------------------ element-wise warpgroups
    const int row = tid & 127;        // key row inside the tile = TMEM lane
    const int half = tid >> 7;        // which 64 query columns of every tile this warpgroup handles
    const int j = kt * kTile + row;   // global key position
    const bool row_ok = j < P.seq_k;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t colS = kColS + 64 * half, colDP = kColDP + 64 * half;
    const float c2 = P.sm_scale * kLog2e;
    const long long n_rows = (long long)P.batch * P.heads * P.seq_q, n_doc = (long long)P.batch * P.doc_stride;
    const float slope2 = (SK == FLEXATTN_SCORE_ALIBI && FLEXATTN_DBG_OK(h, P.heads, 3, 301)) ? P.alibi_slopes[h] * kLog2e : 0.f;
    const float capl2 = P.cap * kLog2e;
    const float csc = (SK == FLEXATTN_SCORE_SOFTCAP) ? P.sm_scale / P.cap : 0.f;
    const int32_t* doc = (MK == FLEXATTN_MASK_DOCUMENT) ? P.doc_ids + (size_t)b * P.doc_stride : nullptr;
    const int dj = (MK == FLEXATTN_MASK_DOCUMENT && row_ok && FLEXATTN_DBG_OK((long long)b * P.doc_stride + j, n_doc, 3, 302))
                       ? doc[j] : -2;
    const ScoreCtx ctx{P.sm_scale, b, h};
    // the interval [qlo, qhi) of queries this key row keeps, where the mask has one: the interval kinds, and a
    // document mask when the ids of the batch row never decrease (the mask map then holds the end of every key's
    // document); a key past the end keeps nothing
    constexpr bool kDoc = MK == FLEXATTN_MASK_DOCUMENT;
    bool doc_runs = false;
    int qlo = 0, qhi = 0;
    if constexpr (kMaskIsInterval<MK>) row_query_interval<MK>(j, P.seq_q, P.window, qlo, qhi);
    if constexpr (kDoc) {
      doc_runs = FLEXATTN_DBG_OK(b, P.batch, 3, 307) && P.doc_sorted[b] != 0;
      if (doc_runs && row_ok && FLEXATTN_DBG_OK((long long)b * P.doc_stride + j, n_doc, 3, 308)) {
        const int end = P.run_hi[(size_t)b * P.doc_stride + j];
        qlo = j;
        qhi = end < P.seq_q ? end : P.seq_q;
      }
    }
    bool ok = true;
    int fail_at = 0;

    {  // zero the accumulators (warpgroup 0: dK, warpgroup 1: dV): every accumulation MMA adds
      uint32_t z[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) z[c] = 0u;
      const uint32_t col = half ? kColDV : kColDK;
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) ptx::tmem_st32(lane_base + col + c0, z);
      ptx::tmem_wait_st();
      ptx::tc_fence_before();
      ptx::mbar_arrive_warp(&sh->bar_zero);
    }

    // Statistics of the query rows (l, m, delta, document id) are fetched from global memory one tile ahead
    // into registers, so their latency is off the critical path.
    const size_t stat_base = (size_t)bh * P.seq_q;
    // Division of the staging work inside a warpgroup (all of it one tile ahead): threads 0..63 own one query row
    // each for -(m log2e + log2 l) - l and m fetched into registers a tile earlier, one shared-memory store;
    // threads 64..127 own one row each for delta (and the document id), which needs no arithmetic and goes
    // global -> shared with cp.async, costing the thread nothing.  Shared-memory stores are slow while the MMAs
    // saturate shared memory, so no warp issues more than one per tile.
    float pf_l = 0.f, pf_m = 0.f;
    bool pf_ok = false;
    auto fetch_stats = [&](int n) {  // threads 0..63
      const int i = (cm.x + n) * kTile + 64 * half + row;
      pf_ok = i < P.seq_q && FLEXATTN_DBG_OK((long long)stat_base + i, n_rows, 3, 303);
      if (pf_ok) {
        pf_l = P.l[stat_base + i];
        pf_m = P.m[stat_base + i];
      }
    };
    auto stage_stats = [&](int n) {
      const int st = n & 1;
      if (row < 64) {
        // pre-scaled for pack_bf16_trunc; l == 0 (fully masked row) forces p to 0
        sh->nlse2[st][64 * half + row] =
            pf_ok ? (pf_l > 0.f ? ptx::kRoundLog2 - fmaf(pf_m, kLog2e, __log2f(pf_l)) : -1.0e30f) : ptx::kRoundLog2;
      } else {
        const int r = row - 64;
        const int i = (cm.x + n) * kTile + 64 * half + r;
        if (i < P.seq_q && FLEXATTN_DBG_OK((long long)stat_base + i, n_rows, 3, 304) &&
            (MK != FLEXATTN_MASK_DOCUMENT || FLEXATTN_DBG_OK((long long)b * P.doc_stride + i, n_doc, 3, 305))) {
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
      const int st = n & 1;
      const int qt = cm.x + n, i0 = qt * kTile + 64 * half;  // first query position of this warpgroup's columns
      const bool partial = P.ab != nullptr || !(qt >= cm.z && qt < cm.w);  // with a dense bias: always the masked form
      // the statistics of this tile were staged during the previous tile (or before the loop)
      // a failed wait never leaves the loop early: every thread keeps executing the same named barriers
      ptx::cp_async_wait_all();  // this thread's asynchronous copies for this tile have landed
      ptx::named_bar_sync(1 + half, 128);
      if (!ok) continue;
      float st0[32], st1[32];
      load_stats32(st0, &sh->nlse2[st][64 * half]);
      ok = __all_sync(0xffffffffu, ptx::mbar_wait(&sh->bar_s, n & 1));
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
        const float abase1 = abase - 32.f * slope2;
        const int32_t* d0p = &sh->doc[st][64 * half];
        const int32_t* d1p = d0p + 32;
        if (P.ab != nullptr) {
          // element (query i0, key j) of the dense bias; nullptr for a key past the end of the sequence or when
          // all 64 queries of this warpgroup lie past the end (the upper half of a ragged last tile)
          const float* ab_col = (row_ok && i0 < P.seq_q && FLEXATTN_DBG_OK((long long)bh * P.seq_q + i0, n_rows, 3, 306))
                                    ? P.ab + ((size_t)bh * P.seq_q + i0) * P.seq_k + j : nullptr;
          const float* ab_col1 = ab_col != nullptr ? ab_col + 32 * (size_t)P.seq_k : nullptr;
          if constexpr (kDoc) {
            if (doc_runs) {
              dkv_p_math32<SK, MK, true, true, true>(sr[0], pk_p, st0, d0p, i0, j, dj, P.seq_q, P.window, P.stride, c2, slope2,
                                                     abase, capl2, csc, ctx, ab_col, (size_t)P.seq_k, qlo, qhi);
              dkv_p_math32<SK, MK, true, true, true>(sr[1], pk_p + 16, st1, d1p, i0 + 32, j, dj, P.seq_q, P.window, P.stride, c2,
                                                     slope2, abase1, capl2, csc, ctx, ab_col1, (size_t)P.seq_k, qlo, qhi);
            } else {
              dkv_p_math32<SK, MK, true, true, false>(sr[0], pk_p, st0, d0p, i0, j, dj, P.seq_q, P.window, P.stride, c2, slope2,
                                                      abase, capl2, csc, ctx, ab_col, (size_t)P.seq_k);
              dkv_p_math32<SK, MK, true, true, false>(sr[1], pk_p + 16, st1, d1p, i0 + 32, j, dj, P.seq_q, P.window, P.stride, c2,
                                                      slope2, abase1, capl2, csc, ctx, ab_col1, (size_t)P.seq_k);
            }
          } else {
            dkv_p_math32<SK, MK, true, true>(sr[0], pk_p, st0, d0p, i0, j, dj, P.seq_q, P.window, P.stride, c2, slope2, abase,
                                             capl2, csc, ctx, ab_col, (size_t)P.seq_k, qlo, qhi);
            dkv_p_math32<SK, MK, true, true>(sr[1], pk_p + 16, st1, d1p, i0 + 32, j, dj, P.seq_q, P.window, P.stride, c2, slope2,
                                             abase1, capl2, csc, ctx, ab_col1, (size_t)P.seq_k, qlo, qhi);
          }
        } else if (partial) {
          if constexpr (kDoc) {
            if (doc_runs) {
              dkv_p_math32<SK, MK, true, false, true>(sr[0], pk_p, st0, d0p, i0, j, dj, P.seq_q, P.window, P.stride, c2, slope2,
                                                      abase, capl2, csc, ctx, nullptr, 0, qlo, qhi);
              dkv_p_math32<SK, MK, true, false, true>(sr[1], pk_p + 16, st1, d1p, i0 + 32, j, dj, P.seq_q, P.window, P.stride,
                                                      c2, slope2, abase1, capl2, csc, ctx, nullptr, 0, qlo, qhi);
            } else {
              dkv_p_math32<SK, MK, true, false, false>(sr[0], pk_p, st0, d0p, i0, j, dj, P.seq_q, P.window, P.stride, c2, slope2,
                                                       abase, capl2, csc, ctx);
              dkv_p_math32<SK, MK, true, false, false>(sr[1], pk_p + 16, st1, d1p, i0 + 32, j, dj, P.seq_q, P.window, P.stride,
                                                       c2, slope2, abase1, capl2, csc, ctx);
            }
          } else {
            dkv_p_math32<SK, MK, true>(sr[0], pk_p, st0, d0p, i0, j, dj, P.seq_q, P.window, P.stride, c2, slope2, abase, capl2,
                                       csc, ctx, nullptr, 0, qlo, qhi);
            dkv_p_math32<SK, MK, true>(sr[1], pk_p + 16, st1, d1p, i0 + 32, j, dj, P.seq_q, P.window, P.stride, c2, slope2,
                                       abase1, capl2, csc, ctx, nullptr, 0, qlo, qhi);
          }
        } else {
          dkv_p_math32<SK, MK, false>(sr[0], pk_p, st0, d0p, i0, j, dj, P.seq_q, P.window, P.stride, c2, slope2, abase, capl2,
                                      csc, ctx);
          dkv_p_math32<SK, MK, false>(sr[1], pk_p + 16, st1, d1p, i0 + 32, j, dj, P.seq_q, P.window, P.stride, c2, slope2,
                                      abase1, capl2, csc, ctx);
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
      ok = __all_sync(0xffffffffu, ptx::mbar_wait(&sh->bar_dp, n & 1));
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

    if (ok && N > 0) {
      ok = __all_sync(0xffffffffu, ptx::mbar_wait(&sh->bar_acc, 0));  // every accumulation MMA has completed
      if (!ok) fail_at = 12;
    }
    // Epilogue: warpgroup 0 stores dK * sm_scale, warpgroup 1 dV: bf16 into a shared-memory tile in the TMA
    // (128-byte swizzle) layout, then one bulk tensor store per 64-column panel.  The Q / dO rings are free by now
    // (every MMA has completed); rows past seq_k are clipped by the tensor map.
    uint8_t* stage = half ? sDO : sQ;
    if (ok) {
      if (N > 0) ptx::tc_fence_after();
      const float sc = half ? 1.f : P.sm_scale;
      const uint32_t col0 = half ? kColDV : kColDK;
      uint8_t* stage_row = stage + row * 128;
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t r[32];
        if (N > 0) {
          ptx::tmem_ld32(lane_base + col0 + c0, r);
          ptx::tmem_wait_ld();
          ptx::tmem_ld_acquire(r);
        } else {
#pragma unroll
          for (int c = 0; c < 32; ++c) r[c] = 0u;
        }
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
      ptx::fence_proxy_async_smem();  // generic-proxy stores -> visible to the bulk store
    }
    ptx::named_bar_sync(1 + half, 128);
    if (ok && row == 0) {
#pragma unroll
      for (int p = 0; p < kPanels; ++p)
        ptx::tma_store_3d(half ? &tm_dv : &tm_dk, stage + p * ptx::kPanelBytes, p * 64, kt * kTile, bh);
      ptx::tma_store_commit();
      ptx::tma_store_wait_read();  // shared memory must stay intact until the store has read it
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
  dim3 grid(d.n_kt, d.batch * d.heads);
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
    void* args[] = {&tq, &tdo, &tk, &tv, &tdk, &tdv, const_cast<DevParams*>(&d), &af};
    return jit_launch(2, d.user_score, d.head_dim, mask, (unsigned)d.n_kt, (unsigned)(d.batch * d.heads), kThreads,
                      need > 120 * 1024 ? need : 120 * 1024, st, args);
  }
  if (d.head_dim == 128) return launch_score<128>(st, d, score, mask, tq, tdo, tk, tv, tdk, tdv, af);
  if (d.head_dim == 64) return launch_score<64>(st, d, score, mask, tq, tdo, tk, tv, tdk, tdv, af);
  return FLEXATTN_ERR_UNSUPPORTED_HEAD_DIM;
}
#endif  // !FLEXATTN_JIT

}  // namespace flexattn
