// Internal definitions shared by every translation unit of libflexattn.so.
#pragma once
#ifdef FLEXATTN_JIT
// Run-time compilation (NVRTC) of a tensor-core kernel around a user score function: no host headers exist there,
// so the handful of types the device code needs are spelled out.
typedef signed char int8_t;
typedef unsigned char uint8_t;
typedef unsigned short uint16_t;
typedef int int32_t;
typedef unsigned int uint32_t;
typedef long long int64_t;
typedef unsigned long long uint64_t;
typedef unsigned long long uintptr_t;
struct alignas(64) CUtensorMap_st {
  unsigned long long opaque[16];
};
typedef CUtensorMap_st CUtensorMap;
#else
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#endif

#include "../../include/flexattn.h"

namespace flexattn {

constexpr int kTile = FLEXATTN_TILE;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
// Finite stand-in for -inf (log2 domain in the tensor-core kernels, natural units in the SIMT ones):
// a row whose keys so far are all masked keeps m == kMasked, its garbage weights exp(0) == 1 are
// wiped by alpha == exp(kMasked - m_new) == 0 as soon as a kept key arrives.  The reference kernels use
// -0.7 * FLT_MAX for the same reason (flex_attention_kernel.py:288).
constexpr float kMasked = -1.0e30f;

// ---------------------------------------------------------------------------------------------
// Mask map (lives in the caller's workspace).
// ---------------------------------------------------------------------------------------------
struct MapHeader {
  int32_t magic, mask_kind, window, stride;
  int32_t seq_q, seq_k, n_qt, n_kt;
  int32_t rows;  // batch for document masks, else 1
  int32_t pad[7];
};
constexpr int32_t kMapMagic = 0x464c5841;  // "FLXA"

struct MapLayout {
  int n_qt, n_kt, rows, n_t;
  size_t off_row, off_col, off_doc, off_order, off_order_rm, off_run_lo, off_run_hi, off_sorted, bytes;
};

__host__ __device__ inline MapLayout map_layout(int batch, int seq_q, int seq_k, int mask_kind) {
  MapLayout L;
  L.n_qt = (seq_q + kTile - 1) / kTile;
  L.n_kt = (seq_k + kTile - 1) / kTile;
  L.n_t = L.n_qt > L.n_kt ? L.n_qt : L.n_kt;
  L.rows = (mask_kind == FLEXATTN_MASK_DOCUMENT) ? batch : 1;
  L.off_row = sizeof(MapHeader);
  L.off_col = L.off_row + sizeof(int4) * (size_t)L.rows * L.n_qt;
  L.off_doc = L.off_col + sizeof(int4) * (size_t)L.rows * L.n_kt;
  size_t doc = (mask_kind == FLEXATTN_MASK_DOCUMENT) ? sizeof(int2) * (size_t)batch * L.n_t : 0;
  // q tiles of every map row ordered by their number of kv tiles, largest first (work order of the persistent
  // forward kernel)
  L.off_order = (L.off_doc + doc + 15) & ~(size_t)15;
  // ... and the row-map entries in that order (so that walking the order needs no dependent load)
  L.off_order_rm = (L.off_order + sizeof(int32_t) * (size_t)L.rows * L.n_qt + 15) & ~(size_t)15;
  // document masks: first / one-past-last position of the run of equal ids every position sits in, and one flag per
  // batch row saying that its ids never decrease (then equal ids are contiguous and a row's kept keys are one
  // interval, so the kernels mask partial tiles from these two numbers instead of comparing ids per element)
  const size_t len = (size_t)(seq_q > seq_k ? seq_q : seq_k);
  const size_t runs = (mask_kind == FLEXATTN_MASK_DOCUMENT) ? sizeof(int32_t) * (size_t)batch * len : 0;
  L.off_run_lo = (L.off_order_rm + sizeof(int4) * (size_t)L.rows * L.n_qt + 15) & ~(size_t)15;
  L.off_run_hi = (L.off_run_lo + runs + 15) & ~(size_t)15;
  L.off_sorted = (L.off_run_hi + runs + 15) & ~(size_t)15;
  L.bytes = (L.off_sorted + (runs ? sizeof(int32_t) * (size_t)batch : 0) + 255) & ~(size_t)255;
  return L;
}

// Device-side view of a problem: what the kernels need, already resolved by the host.
struct DevParams {
  const void* q;
  const void* k;
  const void* v;
  void* o;
  const void* d_o;
  void* dq;
  void* dk;
  void* dv;
  float* l;
  float* m;
  float* delta;
  const int32_t* doc_ids;
  const float* alibi_slopes;
  const float* ab;  // optional dense bias [B,H,Sq,Sk] (SIMT backend only)
  float* dab;       // optional bias gradient, written by the SIMT dQ kernel
  const int4* row_map;  // [rows][n_qt]
  const int4* col_map;  // [rows][n_kt]
  const int32_t* order;  // [rows][n_qt]: q tiles by decreasing number of kv tiles
  const int4* order_rm;  // [rows][n_qt]: row_map entry of order[i]
  const int32_t* run_lo;      // document masks: [batch][doc_stride] first position of each position's run of equal ids
  const int32_t* run_hi;      // ... one past its last position
  const int32_t* doc_sorted;  // ... [batch] 1 when the row's ids never decrease (runs are whole documents)
  int32_t* status;
  int batch, heads, seq_q, seq_k, head_dim;
  int n_qt, n_kt, map_rows, doc_stride;
  int window, stride;
  float sm_scale, cap;
  int user_score;  // handle of a run-time compiled score function (host side only)
};

// ---------------------------------------------------------------------------------------------
// Compile-time mask functors.  True = keep.  di/dj are the document ids of positions i/j (only read
// by the document mask).
// ---------------------------------------------------------------------------------------------
template <int MK>
__device__ __forceinline__ bool mask_keep(int i, int j, int window, int stride, int di, int dj) {
  if constexpr (MK == FLEXATTN_MASK_NONE) {
    return true;
  } else if constexpr (MK == FLEXATTN_MASK_CAUSAL) {
    return i >= j;
  } else if constexpr (MK == FLEXATTN_MASK_SLIDING_WINDOW) {
    return (i - j) < window;
  } else if constexpr (MK == FLEXATTN_MASK_SLIDING_WINDOW_CAUSAL) {
    return (unsigned)(i - j) < (unsigned)window;
  } else if constexpr (MK == FLEXATTN_MASK_DOCUMENT) {
    return (i >= j) && (di == dj);
  } else {  // S2
    return ((unsigned)(i - j) < (unsigned)window) || ((i >= j) && (j % stride == 0));
  }
}

// For the mask kinds whose kept keys of a query row (and kept queries of a key row) form ONE interval, a partial tile
// evaluates the mask once per row and 32 columns as a bitmap (range_bits32 of the row's interval, shifted to the
// group's first column) instead of once per element.  S2 masks are not intervals; document masks are when the ids of
// the batch row never decrease.
template <int MK>
constexpr bool kMaskIsInterval = MK == FLEXATTN_MASK_NONE || MK == FLEXATTN_MASK_CAUSAL ||
                                 MK == FLEXATTN_MASK_SLIDING_WINDOW || MK == FLEXATTN_MASK_SLIDING_WINDOW_CAUSAL;
__device__ __forceinline__ uint32_t range_bits32(int lo, int hi) {  // bits [lo, hi) of a word, clipped to [0, 32)
  lo = lo > 0 ? lo : 0;
  hi = hi < 32 ? hi : 32;
  if (hi <= lo) return 0u;
  return (hi == 32 ? 0xffffffffu : ((1u << hi) - 1u)) & ~((1u << lo) - 1u);
}
// Kept keys [klo, khi) of query row i (the sequence end included) for the interval kinds.
template <int MK>
__device__ __forceinline__ void row_key_interval(int i, int seq_k, int window, int& klo, int& khi) {
  const bool lower = MK == FLEXATTN_MASK_SLIDING_WINDOW || MK == FLEXATTN_MASK_SLIDING_WINDOW_CAUSAL;  // j > i - window
  const bool upper = MK == FLEXATTN_MASK_CAUSAL || MK == FLEXATTN_MASK_SLIDING_WINDOW_CAUSAL;           // j <= i
  klo = lower ? i - window + 1 : 0;
  khi = upper ? (i + 1 < seq_k ? i + 1 : seq_k) : seq_k;
}
// Kept queries [qlo, qhi) of key row j.
template <int MK>
__device__ __forceinline__ void row_query_interval(int j, int seq_q, int window, int& qlo, int& qhi) {
  const bool lower = MK == FLEXATTN_MASK_CAUSAL || MK == FLEXATTN_MASK_SLIDING_WINDOW_CAUSAL;           // i >= j
  const bool upper = MK == FLEXATTN_MASK_SLIDING_WINDOW || MK == FLEXATTN_MASK_SLIDING_WINDOW_CAUSAL;  // i < j + window
  qlo = lower ? j : 0;
  qhi = upper ? (j + window < seq_q ? j + window : seq_q) : seq_q;
}
// A document mask over ids that never decrease is an interval as well: query row i keeps the keys [run_lo(i), i],
// key row j the queries [j, run_hi(j)), with run_lo / run_hi from the mask map.

// Compile-time score functors on the scaled score s = sm_scale * <q,k>, natural units.
// score_fwd returns t = score_mod(s) + bias(i, j); score_dsig returns d score_mod / d s.
template <int SK>
__device__ __forceinline__ float score_fwd(float s, int i, int j, float slope, float cap, float inv_cap) {
  if constexpr (SK == FLEXATTN_SCORE_ALIBI) {
    return s - slope * (float)(i - j);
  } else if constexpr (SK == FLEXATTN_SCORE_SOFTCAP) {
    return cap * tanhf(s * inv_cap);
  } else {
    return s;
  }
}
template <int SK>
__device__ __forceinline__ float score_dsig(float s, float inv_cap) {
  if constexpr (SK == FLEXATTN_SCORE_SOFTCAP) {
    float th = tanhf(s * inv_cap);
    return 1.0f - th * th;
  } else {
    return 1.0f;
  }
}

__device__ __forceinline__ void report_status(int32_t* status, int code, int kernel_id, int detail) {
  if (status != nullptr) {
    if (atomicCAS(status, 0, code) == 0) {
      status[1] = kernel_id;
      status[2] = (int)(blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z));
      status[3] = detail;
    }
  }
}
__device__ __forceinline__ void report_timeout(int32_t* status, int kernel_id, int detail) {
  report_status(status, (int)FLEXATTN_ERR_TIMEOUT, kernel_id, detail);
}

// Bounds-checked build (-DFLEXATTN_DEBUG, libflexattn_debug.so): every direct global-memory access of the
// tensor-core kernels (everything that does not go through a TMA tensor map, which clips by itself) is guarded.
// An index outside its array is recorded as {FLEXATTN_ERR_DEBUG_BOUNDS, kernel id, block, site} in the status
// words and the access is skipped, so a wrong index shows up as a status instead of a memory fault.  In the
// ordinary build the check is the constant `true` and disappears.
#ifdef FLEXATTN_DEBUG
constexpr bool kDebugChecks = true;
#else
constexpr bool kDebugChecks = false;
#endif
__device__ __forceinline__ bool dbg_in_bounds(long long idx, long long limit, int32_t* status, int kernel_id, int site) {
  if constexpr (!kDebugChecks) {
    return true;
  } else {
    if (idx >= 0 && idx < limit) return true;
    report_status(status, (int)FLEXATTN_ERR_DEBUG_BOUNDS, kernel_id, site);
    return false;
  }
}
#define FLEXATTN_DBG_OK(idx, limit, kernel_id, site) \
  ::flexattn::dbg_in_bounds((long long)(idx), (long long)(limit), P.status, (kernel_id), (site))

#ifndef FLEXATTN_JIT
// Host-side validation of a forward call, shared by flexattn_fwd and flexattn_fwd_noalloc (api.cu).
int validate_fwd_args(const FlexAttnParams* p, bool* tc);

// ---------------------------------------------------------------------------------------------
// Launchers implemented by the kernel translation units; each returns a cudaError_t.
// ---------------------------------------------------------------------------------------------
cudaError_t launch_mask_map(cudaStream_t st, const FlexAttnParams& p);
cudaError_t launch_delta(cudaStream_t st, const FlexAttnParams& p);
cudaError_t launch_simt_fwd(cudaStream_t st, const DevParams& d, int dtype, int score, int mask);
cudaError_t launch_simt_dq(cudaStream_t st, const DevParams& d, int dtype, int score, int mask);
cudaError_t launch_simt_dkv(cudaStream_t st, const DevParams& d, int dtype, int score, int mask);
// tensor-core (tcgen05) kernels: bf16, D in {64,128}
int launch_sm100_fwd_pipe(cudaStream_t st, const DevParams& d, int score, int mask);  // persistent, three score tiles in flight
int launch_sm100_fwd_pair(cudaStream_t st, const DevParams& d, int score, int mask);  // two query tiles per CTA, one row per thread
int launch_sm100_dq(cudaStream_t st, const DevParams& d, int score, int mask);
int launch_sm100_dkv(cudaStream_t st, const DevParams& d, int score, int mask);

// Launch of a kernel compiled at run time around a user score function (jit.cu).  which: 0 forward, 1 dQ, 2 dK/dV;
// args: the kernel's parameters as for cuLaunchKernel.  Returns a FlexAttnStatus.
int jit_launch(int which, int handle, int head_dim, int mask, unsigned grid_x, unsigned grid_y, unsigned threads,
               size_t smem_bytes, cudaStream_t st, void** args);
#endif  // !FLEXATTN_JIT

}  // namespace flexattn

// user_score(s, b, h, i, j) and user_dscore(...): identity here; a run-time compilation substitutes the user's
// expressions for this header.
#include "user_score.cuh"
