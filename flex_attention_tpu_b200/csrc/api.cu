// The C ABI of libflexattn.so: argument validation, backend choice and dispatch.  No allocation, no
// host synchronisation (except flexattn_read_mask_map, a test/tool helper).  The only state that outlives a
// call is per device: the abort word of the tensor-core kernels (set by a device-side time-out, cleared by
// flexattn_reset_abort) and the caches of device attributes and symbol addresses next to it.
#include <stdlib.h>
#include <string.h>

#include <nvtx3/nvToolsExt.h>

#include "common.cuh"

namespace flexattn {
namespace {


bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// NVTX range around the host side of an entry point (validation, tensor-map encoding, launch): shows up in ncu /
// Nsight timelines and costs nothing when no tool is attached (header-only NVTX resolves to a no-op then).
struct NvtxRange {
  explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
  ~NvtxRange() { nvtxRangePop(); }
  NvtxRange(const NvtxRange&) = delete;
  NvtxRange& operator=(const NvtxRange&) = delete;
};

int validate_common(const FlexAttnParams* p) {
  if (p == nullptr) return FLEXATTN_ERR_NULL_POINTER;
  if (p->batch <= 0 || p->heads <= 0 || p->seq_q <= 0 || p->seq_k <= 0) return FLEXATTN_ERR_BAD_SHAPE;
  if ((long long)p->batch * p->heads > 0x7fffffffLL / 2) return FLEXATTN_ERR_BAD_SHAPE;
  if (p->dtype != FLEXATTN_BF16 && p->dtype != FLEXATTN_F32) return FLEXATTN_ERR_UNSUPPORTED_DTYPE;
  if (p->head_dim != 32 && p->head_dim != 64 && p->head_dim != 128) return FLEXATTN_ERR_UNSUPPORTED_HEAD_DIM;
  if (p->score_kind < FLEXATTN_SCORE_NONE || p->score_kind > FLEXATTN_SCORE_USER) return FLEXATTN_ERR_UNSUPPORTED_MOD;
  if (p->mask_kind < FLEXATTN_MASK_NONE || p->mask_kind > FLEXATTN_MASK_S2) return FLEXATTN_ERR_UNSUPPORTED_MOD;
  if (p->backend < FLEXATTN_BACKEND_AUTO || p->backend > FLEXATTN_BACKEND_TCGEN05) return FLEXATTN_ERR_UNSUPPORTED_BACKEND;
  return FLEXATTN_OK;
}

int validate_mods(const FlexAttnParams* p) {
  const int mk = p->mask_kind;
  if ((mk == FLEXATTN_MASK_SLIDING_WINDOW || mk == FLEXATTN_MASK_SLIDING_WINDOW_CAUSAL || mk == FLEXATTN_MASK_S2) &&
      p->window <= 0)
    return FLEXATTN_ERR_UNSUPPORTED_MOD;
  if (mk == FLEXATTN_MASK_S2 && p->stride <= 0) return FLEXATTN_ERR_UNSUPPORTED_MOD;
  if (mk == FLEXATTN_MASK_DOCUMENT && p->doc_ids == nullptr) return FLEXATTN_ERR_NULL_POINTER;
  if (p->score_kind == FLEXATTN_SCORE_ALIBI && p->alibi_slopes == nullptr) return FLEXATTN_ERR_NULL_POINTER;
  if (p->score_kind == FLEXATTN_SCORE_SOFTCAP && !(p->softcap > 0.f)) return FLEXATTN_ERR_UNSUPPORTED_MOD;
  if (p->score_kind == FLEXATTN_SCORE_USER && p->user_score <= 0) return FLEXATTN_ERR_UNSUPPORTED_MOD;
  return FLEXATTN_OK;
}

int validate_workspace(const FlexAttnParams* p) {
  if (p->workspace == nullptr) return FLEXATTN_ERR_NULL_POINTER;
  if (!aligned16(p->workspace)) return FLEXATTN_ERR_MISALIGNED;
  MapLayout L = map_layout(p->batch, p->seq_q, p->seq_k, p->mask_kind);
  if (p->workspace_bytes < L.bytes) return FLEXATTN_ERR_WORKSPACE_TOO_SMALL;
  return FLEXATTN_OK;
}

// true when the tensor-core kernels serve this problem
bool use_tcgen05(const FlexAttnParams* p, int* err) {
  // the tensor-core kernels take bf16 and D in {64, 128}
  const bool capable = p->dtype == FLEXATTN_BF16 && (p->head_dim == 64 || p->head_dim == 128);
  *err = FLEXATTN_OK;
  // a user score function exists only as a run-time compiled tensor-core kernel
  if (p->score_kind == FLEXATTN_SCORE_USER && (!capable || p->backend == FLEXATTN_BACKEND_SIMT)) {
    *err = FLEXATTN_ERR_UNSUPPORTED_BACKEND;
    return false;
  }
  if (p->backend == FLEXATTN_BACKEND_SIMT) return false;
  if (p->backend == FLEXATTN_BACKEND_TCGEN05 && !capable) *err = FLEXATTN_ERR_UNSUPPORTED_BACKEND;
  return capable;
}

DevParams make_dev(const FlexAttnParams* p) {
  DevParams d{};
  MapLayout L = map_layout(p->batch, p->seq_q, p->seq_k, p->mask_kind);
  char* ws = static_cast<char*>(p->workspace);
  d.q = p->q; d.k = p->k; d.v = p->v; d.o = p->o; d.d_o = p->d_o;
  d.dq = p->dq; d.dk = p->dk; d.dv = p->dv;
  d.l = p->l; d.m = p->m; d.delta = p->delta;
  d.doc_ids = p->mask_kind == FLEXATTN_MASK_DOCUMENT ? p->doc_ids : nullptr;
  d.alibi_slopes = p->score_kind == FLEXATTN_SCORE_ALIBI ? p->alibi_slopes : nullptr;
  d.ab = p->ab;
  d.dab = p->dab;
  d.row_map = reinterpret_cast<const int4*>(ws + L.off_row);
  d.col_map = reinterpret_cast<const int4*>(ws + L.off_col);
  d.order = reinterpret_cast<const int32_t*>(ws + L.off_order);
  d.order_rm = reinterpret_cast<const int4*>(ws + L.off_order_rm);
  if (p->mask_kind == FLEXATTN_MASK_DOCUMENT) {
    d.run_lo = reinterpret_cast<const int32_t*>(ws + L.off_run_lo);
    d.run_hi = reinterpret_cast<const int32_t*>(ws + L.off_run_hi);
    d.doc_sorted = reinterpret_cast<const int32_t*>(ws + L.off_sorted);
  }
  d.status = p->status;
  d.batch = p->batch; d.heads = p->heads; d.seq_q = p->seq_q; d.seq_k = p->seq_k; d.head_dim = p->head_dim;
  d.n_qt = L.n_qt; d.n_kt = L.n_kt; d.map_rows = L.rows;
  d.doc_stride = p->seq_q > p->seq_k ? p->seq_q : p->seq_k;
  d.window = p->window; d.stride = p->stride > 0 ? p->stride : 1;
  d.sm_scale = p->sm_scale; d.cap = p->score_kind == FLEXATTN_SCORE_SOFTCAP ? p->softcap : 0.f;
  d.user_score = p->score_kind == FLEXATTN_SCORE_USER ? p->user_score : 0;
  return d;
}

#define FLEXATTN_REQUIRE(ptr)                                     \
  do {                                                            \
    if ((ptr) == nullptr) return FLEXATTN_ERR_NULL_POINTER;       \
    if (!aligned16(ptr)) return FLEXATTN_ERR_MISALIGNED;          \
  } while (0)

int prologue(const FlexAttnParams* p) {
  int e = validate_common(p);
  if (e) return e;
  e = validate_mods(p);
  if (e) return e;
  return validate_workspace(p);
}

}  // namespace

// Everything flexattn_fwd checks before it launches (shapes, kinds, workspace, pointers, backend).  tc: whether
// the tensor-core kernel serves the call.
int validate_fwd_args(const FlexAttnParams* p, bool* tc) {
  int e = prologue(p);
  if (e) return e;
  FLEXATTN_REQUIRE(p->q); FLEXATTN_REQUIRE(p->k); FLEXATTN_REQUIRE(p->v); FLEXATTN_REQUIRE(p->o);
  FLEXATTN_REQUIRE(p->l); FLEXATTN_REQUIRE(p->m);
  *tc = use_tcgen05(p, &e);
  return e;
}

}  // namespace flexattn

using namespace flexattn;

extern "C" {

int flexattn_abi_version(void) { return FLEXATTN_ABI_VERSION; }

const char* flexattn_status_string(int status) {
  switch (status) {
    case FLEXATTN_OK: return "ok";
    case FLEXATTN_ERR_NULL_POINTER: return "null pointer";
    case FLEXATTN_ERR_BAD_SHAPE: return "bad shape";
    case FLEXATTN_ERR_UNSUPPORTED_DTYPE: return "unsupported dtype";
    case FLEXATTN_ERR_UNSUPPORTED_HEAD_DIM: return "unsupported head_dim (32, 64 or 128)";
    case FLEXATTN_ERR_MISALIGNED: return "pointer not 16-byte aligned";
    case FLEXATTN_ERR_WORKSPACE_TOO_SMALL: return "workspace too small";
    case FLEXATTN_ERR_UNSUPPORTED_MOD: return "unsupported or ill-formed score_mod / mask";
    case FLEXATTN_ERR_CUDA: return "CUDA error at launch";
    case FLEXATTN_ERR_TIMEOUT: return "device-side wait timed out";
    case FLEXATTN_ERR_UNSUPPORTED_BACKEND: return "backend cannot serve this dtype / head_dim";
    case FLEXATTN_ERR_NOALLOC_LIMIT:
      return "mask map larger than the fixed scratch array of the no-allocation entry point (1 MiB)";
    case FLEXATTN_ERR_JIT_UNAVAILABLE: return "run-time compiler (libnvrtc) or driver module loader not available";
    case FLEXATTN_ERR_JIT_COMPILE: return "the user score function did not compile (see flexattn_user_score_log)";
    case FLEXATTN_ERR_DEBUG_BOUNDS: return "bounds-checked build: an out-of-range global-memory access was skipped";
    default: return "unknown status";
  }
}

size_t flexattn_workspace_bytes(const FlexAttnParams* p) {
  if (validate_common(p) != FLEXATTN_OK) return 0;
  return map_layout(p->batch, p->seq_q, p->seq_k, p->mask_kind).bytes;
}

int flexattn_build_mask_map(void* stream, const FlexAttnParams* p) {
  NvtxRange nvtx("flexattn_build_mask_map");
  int e = prologue(p);
  if (e) return e;
  if (p->mask_kind == FLEXATTN_MASK_DOCUMENT && (reinterpret_cast<uintptr_t>(p->doc_ids) & 3u)) return FLEXATTN_ERR_MISALIGNED;
  return launch_mask_map(static_cast<cudaStream_t>(stream), *p) == cudaSuccess ? FLEXATTN_OK : FLEXATTN_ERR_CUDA;
}

namespace {
// kv tiles an average query tile visits, from the mask kind alone (a document mask depends on the data: 0, which
// keeps the persistent kernel).
int mean_kv_tiles(const FlexAttnParams* p) {
  const int n_kt = (p->seq_k + FLEXATTN_TILE - 1) / FLEXATTN_TILE;
  const int in_window = p->window / FLEXATTN_TILE + 1;
  switch (p->mask_kind) {
    case FLEXATTN_MASK_NONE: return n_kt;
    case FLEXATTN_MASK_CAUSAL: return (n_kt + 1) / 2;
    case FLEXATTN_MASK_SLIDING_WINDOW: return n_kt < in_window ? n_kt : (n_kt + in_window) / 2;  // window back, all ahead
    case FLEXATTN_MASK_SLIDING_WINDOW_CAUSAL: return n_kt < in_window ? n_kt : in_window;
    case FLEXATTN_MASK_S2: return (n_kt + 1) / 2;  // strided columns keep every tile below the diagonal alive
    default: return 0;
  }
}
constexpr int kPairMinTiles = 12;  // measured: at 12.5 tiles the two kernels tie, at 16 the pair kernel is 5-12 % faster, at 32 15 %
int forced_fwd_kernel() {  // 0: choose by shape, 1: two-query-tile kernel, 2: persistent kernel
  static const int choice = [] {
    const char* e = getenv("FLEXATTN_FWD_KERNEL");
    if (e == nullptr) return 0;
    if (strcmp(e, "pair") == 0) return 1;
    if (strcmp(e, "pipe") == 0) return 2;
    return 0;
  }();
  return choice;
}
}  // namespace

int flexattn_fwd(void* stream, const FlexAttnParams* p) {
  NvtxRange nvtx("flexattn_fwd");
  bool tc = false;
  const int e = validate_fwd_args(p, &tc);
  if (e) return e;
  DevParams d = make_dev(p);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (tc) {
    // Two tensor-core forward kernels: the persistent one (fwd_pipe_sm100.cu: work items streamed through each CTA,
    // prologue and epilogue hidden, best for short rows) and the two-query-tile one (fwd_pair_sm100.cu: one row per
    // thread, K/V shared by two tiles, best once a query tile sees a few dozen kv tiles).  FLEXATTN_FWD_KERNEL=pair
    // or =pipe in the environment forces one where both can run (read once per process).
    const bool pair_can = p->ab == nullptr;
    const int forced = forced_fwd_kernel();
    if (pair_can && (forced == 1 || (forced == 0 && mean_kv_tiles(p) >= kPairMinTiles)))
      return launch_sm100_fwd_pair(st, d, p->score_kind, p->mask_kind);
    return launch_sm100_fwd_pipe(st, d, p->score_kind, p->mask_kind);
  }
  return launch_simt_fwd(st, d, p->dtype, p->score_kind, p->mask_kind) == cudaSuccess ? FLEXATTN_OK : FLEXATTN_ERR_CUDA;
}

int flexattn_bwd_preprocess(void* stream, const FlexAttnParams* p) {
  NvtxRange nvtx("flexattn_bwd_preprocess");
  int e = validate_common(p);
  if (e) return e;
  FLEXATTN_REQUIRE(p->o); FLEXATTN_REQUIRE(p->d_o); FLEXATTN_REQUIRE(p->delta);
  return launch_delta(static_cast<cudaStream_t>(stream), *p) == cudaSuccess ? FLEXATTN_OK : FLEXATTN_ERR_CUDA;
}

int flexattn_bwd_dq(void* stream, const FlexAttnParams* p) {
  NvtxRange nvtx("flexattn_bwd_dq");
  int e = prologue(p);
  if (e) return e;
  FLEXATTN_REQUIRE(p->q); FLEXATTN_REQUIRE(p->k); FLEXATTN_REQUIRE(p->v); FLEXATTN_REQUIRE(p->d_o);
  FLEXATTN_REQUIRE(p->l); FLEXATTN_REQUIRE(p->m); FLEXATTN_REQUIRE(p->delta); FLEXATTN_REQUIRE(p->dq);
  const bool tc = use_tcgen05(p, &e);
  if (e) return e;
  DevParams d = make_dev(p);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (tc) return launch_sm100_dq(st, d, p->score_kind, p->mask_kind);
  return launch_simt_dq(st, d, p->dtype, p->score_kind, p->mask_kind) == cudaSuccess ? FLEXATTN_OK : FLEXATTN_ERR_CUDA;
}

int flexattn_bwd_dkv(void* stream, const FlexAttnParams* p) {
  NvtxRange nvtx("flexattn_bwd_dkv");
  int e = prologue(p);
  if (e) return e;
  FLEXATTN_REQUIRE(p->q); FLEXATTN_REQUIRE(p->k); FLEXATTN_REQUIRE(p->v); FLEXATTN_REQUIRE(p->d_o);
  FLEXATTN_REQUIRE(p->l); FLEXATTN_REQUIRE(p->m); FLEXATTN_REQUIRE(p->delta);
  FLEXATTN_REQUIRE(p->dk); FLEXATTN_REQUIRE(p->dv);
  const bool tc = use_tcgen05(p, &e);
  if (e) return e;
  DevParams d = make_dev(p);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (tc) return launch_sm100_dkv(st, d, p->score_kind, p->mask_kind);
  return launch_simt_dkv(st, d, p->dtype, p->score_kind, p->mask_kind) == cudaSuccess ? FLEXATTN_OK : FLEXATTN_ERR_CUDA;
}

int flexattn_read_mask_map(void* stream, const FlexAttnParams* p, int which, int b, int index, int32_t out[4]) {
  int e = prologue(p);
  if (e) return e;
  if (out == nullptr) return FLEXATTN_ERR_NULL_POINTER;
  MapLayout L = map_layout(p->batch, p->seq_q, p->seq_k, p->mask_kind);
  const int n = which ? L.n_kt : L.n_qt;
  if (b < 0 || b >= L.rows || index < 0 || index >= n || (which != 0 && which != 1)) return FLEXATTN_ERR_BAD_SHAPE;
  const char* src = static_cast<const char*>(p->workspace) + (which ? L.off_col : L.off_row) +
                    sizeof(int4) * ((size_t)b * n + index);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemcpyAsync(out, src, sizeof(int4), cudaMemcpyDeviceToHost, st) != cudaSuccess) return FLEXATTN_ERR_CUDA;
  return cudaStreamSynchronize(st) == cudaSuccess ? FLEXATTN_OK : FLEXATTN_ERR_CUDA;
}

}  // extern "C"
