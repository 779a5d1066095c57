/*
 * flexattn.h -- C ABI of libflexattn.so: flex attention (score_mod + mask) for NVIDIA B200 (sm_100a).
 *
 * The reference project (james-zhengql/flex_attention_tpu) has no FFI of its own: its API is three
 * Python functions, each wrapping one pl.pallas_call.  Every entry point below names the reference
 * interface it replaces (file:line within that project).  A JAX host would bind these symbols as XLA
 * FFI custom calls; this repository binds them with ctypes.
 *
 * Rules that hold for every entry point unless its comment says otherwise:
 *   - plain pointers and sizes only; no C++ types, no exceptions cross the boundary;
 *   - all tensor pointers are DEVICE pointers to contiguous row-major [B,H,S,D] (q,k,v,o,do,dq,dk,dv)
 *     or [B,H,S] float (l,m,delta) arrays, 16-byte aligned;
 *   - work is enqueued on `stream` (a cudaStream_t passed as void*); the host is never synchronised
 *     and nothing is allocated: outputs and the workspace belong to the caller;
 *   - the return value is a FlexAttnStatus (0 = OK); launch-time CUDA errors are reported as
 *     FLEXATTN_ERR_CUDA, asynchronous device-side time-outs through the optional `status` words;
 *   - device-side time-outs are sticky per device: every wait inside the tensor-core kernels is bounded, and
 *     the first one that gives up sets an abort word on its device.  From then on every tensor-core launch on
 *     that device returns at once, writes {FLEXATTN_ERR_TIMEOUT, kernel id, block, 99} into `status` and
 *     leaves its outputs untouched, until flexattn_reset_abort has run.  The entry points still return
 *     FLEXATTN_OK (they do not synchronise), so a caller that wants to see the failure must pass `status`.
 *
 * Fixed math convention (identical to the reference whenever sm_scale == 1, the only setting its
 * score_fn tests use):
 *     s = sm_scale * <q_i, k_j>;  t = score_mod(s) + bias(i, j);  x = keep(i, j) ? t : -inf
 *     m_i = max_j x;  l_i = sum_j exp(x - m_i);  o_i = sum_j exp(x - m_i) / l_i * v_j
 */
#ifndef FLEXATTN_H_
#define FLEXATTN_H_

#ifndef FLEXATTN_JIT /* run-time compilation of the kernels brings its own fixed-width types */
#include <stddef.h>
#include <stdint.h>
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define FLEXATTN_ABI_VERSION 4
#define FLEXATTN_TILE 128 /* q-tile and kv-tile edge used by the mask map and by every kernel */

typedef enum FlexAttnStatus {
  FLEXATTN_OK = 0,
  FLEXATTN_ERR_NULL_POINTER = 1,
  FLEXATTN_ERR_BAD_SHAPE = 2,
  FLEXATTN_ERR_UNSUPPORTED_DTYPE = 3,
  FLEXATTN_ERR_UNSUPPORTED_HEAD_DIM = 4,
  FLEXATTN_ERR_MISALIGNED = 5,
  FLEXATTN_ERR_WORKSPACE_TOO_SMALL = 6,
  FLEXATTN_ERR_UNSUPPORTED_MOD = 7,
  FLEXATTN_ERR_CUDA = 8,
  FLEXATTN_ERR_TIMEOUT = 9,
  FLEXATTN_ERR_UNSUPPORTED_BACKEND = 10,
  FLEXATTN_ERR_NOALLOC_LIMIT = 11,
  FLEXATTN_ERR_JIT_UNAVAILABLE = 12, /* the run-time compiler (libnvrtc) or the driver's module loader is missing */
  FLEXATTN_ERR_JIT_COMPILE = 13,     /* a user score function did not compile: see flexattn_user_score_log */
  FLEXATTN_ERR_DEBUG_BOUNDS = 14     /* bounds-checked build only: a kernel skipped an out-of-range access (status words) */
} FlexAttnStatus;

typedef enum FlexAttnDType { FLEXATTN_BF16 = 0, FLEXATTN_F32 = 1 } FlexAttnDType;

/* score_mod kinds: reference scores.py:3-11 (ALiBi demo; here real ALiBi with per-head slopes and
 * global distance, bias = -slope_h * (i - j)) and scores.py:13-18 (tanh soft cap). */
typedef enum FlexAttnScoreKind {
  FLEXATTN_SCORE_NONE = 0,
  FLEXATTN_SCORE_ALIBI = 1,
  FLEXATTN_SCORE_SOFTCAP = 2,
  FLEXATTN_SCORE_USER = 3 /* a score function registered with flexattn_user_score_create (params.user_score) */
} FlexAttnScoreKind;

/* mask kinds (keep predicate): reference masks.py:3-6 (none), :15-16 (causal, i >= j),
 * :45-59 (sliding window, i - j < W, NOT causal), window AND causal (0 <= i - j < W,
 * mha_reference.py:59-62 with :80-94), :105-110 (document: same id AND causal),
 * :146-158 (S2: window-causal OR (j % stride == 0 AND causal)). */
typedef enum FlexAttnMaskKind {
  FLEXATTN_MASK_NONE = 0,
  FLEXATTN_MASK_CAUSAL = 1,
  FLEXATTN_MASK_SLIDING_WINDOW = 2,
  FLEXATTN_MASK_SLIDING_WINDOW_CAUSAL = 3,
  FLEXATTN_MASK_DOCUMENT = 4,
  FLEXATTN_MASK_S2 = 5
} FlexAttnMaskKind;

typedef enum FlexAttnBackend {
  FLEXATTN_BACKEND_AUTO = 0,    /* bf16 with D in {64,128}: tcgen05 kernels; otherwise SIMT */
  FLEXATTN_BACKEND_SIMT = 1,    /* fp32-accurate CUDA-core kernels (any dtype, D in {32,64,128}) */
  FLEXATTN_BACKEND_TCGEN05 = 2  /* fail with UNSUPPORTED_BACKEND instead of falling back */
} FlexAttnBackend;

typedef struct FlexAttnParams {
  /* tensors (device) */
  const void* q;     /* [B,H,Sq,D] */
  const void* k;     /* [B,H,Sk,D] */
  const void* v;     /* [B,H,Sk,D] */
  void* o;           /* [B,H,Sq,D]  written by fwd; read by bwd_preprocess */
  const void* d_o;   /* [B,H,Sq,D]  upstream gradient */
  void* dq;          /* [B,H,Sq,D] */
  void* dk;          /* [B,H,Sk,D] */
  void* dv;          /* [B,H,Sk,D] */
  float* l;          /* [B,H,Sq]  sum_j exp(x - m)   (fwd output, bwd input) */
  float* m;          /* [B,H,Sq]  row max of x       (fwd output, bwd input) */
  float* delta;      /* [B,H,Sq]  rowsum(o * do)     (bwd_preprocess output, dq/dkv input) */
  const int32_t* doc_ids;     /* [B, max(Sq,Sk)] document id per position; MASK_DOCUMENT only.  A pair is kept when
                               * the ids are EQUAL (and the key is not ahead of the query); any ids are valid, ids
                               * that never decrease along a batch row (documents laid end to end) run fastest */
  const float* alibi_slopes;  /* [H]; SCORE_ALIBI only */
  /* problem */
  int32_t batch, heads, seq_q, seq_k, head_dim;
  int32_t dtype;              /* FlexAttnDType of q,k,v,o,do,dq,dk,dv */
  float sm_scale;
  int32_t score_kind;         /* FlexAttnScoreKind */
  float softcap;              /* cap of SCORE_SOFTCAP */
  int32_t mask_kind;          /* FlexAttnMaskKind */
  int32_t window;             /* W of the window masks and of S2 */
  int32_t stride;             /* stride of S2 */
  /* caller-owned scratch: holds the mask map written by flexattn_build_mask_map */
  void* workspace;
  size_t workspace_bytes;
  /* optional int32[4] the device can write (device memory, or pinned host memory the device can reach):
   * {code, kernel id, block, detail}; written when a bounded wait inside a kernel gives up, or when the
   * launch found the device's abort word set (code = FLEXATTN_ERR_TIMEOUT; detail 99 = aborted on entry).
   * Only the first report lands: zero it to re-arm.  May be NULL. */
  int32_t* status;
  int32_t backend;            /* FlexAttnBackend */
  int32_t user_score;         /* handle from flexattn_user_score_create; SCORE_USER only, else 0 */
  /* optional dense additive bias, float32 [B,H,Sq,Sk], added to the logits after the score function and before
   * the mask (the reference's `ab`: flex_attention_kernel.py:262-266, flash_attention_dkv_bwd.py:261-266,
   * mha_reference.py:50-51).  NULL = none.  Every backend serves it; the S^2 floats of the bias then bound the
   * kernels (HBM), not the arithmetic. */
  const float* ab;
  /* optional gradient of the bias, float32 [B,H,Sq,Sk], written by flexattn_bwd_dq when not NULL:
   * dab = p * (dp - delta), zero at masked pairs ("dab is just ds", jax_exp.py:1676-1677). */
  float* dab;
} FlexAttnParams;

/* ABI version of the loaded library (== FLEXATTN_ABI_VERSION of the header it was built from). */
int flexattn_abi_version(void);

/* Human-readable name of a FlexAttnStatus.  Never NULL. */
const char* flexattn_status_string(int status);

/* Bytes of workspace the mask map needs for this problem (depends on batch, seq_q, seq_k, mask_kind).
 * Replaces nothing in the reference (its block_mask_fn closures are evaluated inside the grid,
 * flex_attention_kernel.py:97-106,231-236); returns 0 on invalid params. */
size_t flexattn_workspace_bytes(const FlexAttnParams* p);

/* Block-sparse mask-map builder.  Replaces the per-grid-step `block_mask_fn(q_blk, k_blk)` closures of
 * masks.py:20-28,63-81,113-139,161-177 and the "fetch block 0 instead" redirect of
 * flex_attention_kernel.py:97-106: for every q tile (and every kv tile, for the dk/dv kernel) it writes
 * the contiguous range of opposite-side tiles holding at least one kept pair, and the sub-range that
 * is entirely kept (no mask evaluation needed there).  Must run (on the same stream, or ordered before)
 * ahead of fwd / bwd_dq / bwd_dkv for the same mask, shapes and doc_ids. */
int flexattn_build_mask_map(void* stream, const FlexAttnParams* p);

/* Forward.  Replaces `_flex_attention_impl` (flex_attention_kernel.py:66-193) with
 * save_residuals=True: writes o, l, m.  On the tensor-core backend one of two kernels runs, chosen by the mask kind
 * and the shapes (a persistent one for short rows, a two-query-tile one for long rows); the environment variable
 * FLEXATTN_FWD_KERNEL=pipe or =pair, read once per process, forces one where both apply.  Their results agree
 * within the stated tolerance, not bit for bit (the key tiles are summed in the same order but by different
 * threads). */
int flexattn_fwd(void* stream, const FlexAttnParams* p);

/* delta = rowsum(o * do).  Replaces the host-side `jnp.sum(o * do, -1)` every reference call site does
 * before the backward kernels (flex_attention_dq_bwd.py:697,932). */
int flexattn_bwd_preprocess(void* stream, const FlexAttnParams* p);

/* dQ.  Replaces `flex_attention_bwd_dq` (flex_attention_dq_bwd.py:114-267).  Reads q,k,v,do,l,m,delta. */
int flexattn_bwd_dq(void* stream, const FlexAttnParams* p);

/* dK and dV.  Replaces `flash_attention_bwd_dkv` (flex_attention_dkv_kernel.py:23-174 and its
 * mask-aware twin flash_attention_dkv_bwd.py:27-180).  Reads q,k,v,do,l,m,delta. */
int flexattn_bwd_dkv(void* stream, const FlexAttnParams* p);

/* Forward without any caller-provided scratch memory.  It has no counterpart in the reference.
 *
 * For hosts that cannot allocate device memory and were handed only operands and results: code running
 * under a memory planner that assigned every buffer before launch, or inside a process whose allocator
 * owns the whole device.  Same inputs and outputs as flexattn_fwd (q, k, v -> o, l, m; doc_ids /
 * alibi_slopes as the mask / score kinds require); `workspace` and `workspace_bytes` are ignored.  The
 * mask map is built, on `stream`, into a fixed array of flexattn_noalloc_scratch_bytes() = 1 MiB that is
 * part of the library's device image (each GPU that loads the library carries it until the process
 * exits), then the forward kernel runs from it.  The entry point itself never calls an allocating or
 * freeing routine of the CUDA runtime or of any library.  What the driver does on its own when a device
 * first uses the library (loading the module, which is when the array and the kernels' code take their
 * place in device memory) happens during the first call on that device; after that call, device memory
 * does not change across calls.  Arguments are validated before anything is enqueued, so a refused call
 * leaves the array as it was.
 *
 *  - A problem whose mask map needs more than that (flexattn_workspace_bytes(p) > 1 MiB) is refused with
 *    FLEXATTN_ERR_NOALLOC_LIMIT; use flexattn_fwd with your own workspace instead.
 *  - The first call on each device resolves the array's device address (cudaGetSymbolAddress, with that
 *    device current).  Make that first call outside any stream capture.
 *  - All calls on a device share the one array, which always holds the map of the most recent call.  Calls
 *    whose GPU work can overlap (different streams, or threads that do not order their launches) race on
 *    it: serialise them, e.g. by using a single stream. */
int flexattn_fwd_noalloc(void* stream, const FlexAttnParams* p);

/* Size in bytes of the fixed scratch array behind flexattn_fwd_noalloc.  No counterpart in the reference. */
size_t flexattn_noalloc_scratch_bytes(void);

/* Decodes the mask map in `workspace` for tests and tools: copies entry `index` of the row map
 * (which = 0: per q tile) or column map (which = 1: per kv tile) of batch row `b` into out[4] =
 * {first tile, end tile (exclusive), first fully-kept tile, end of fully-kept run}.  Synchronises
 * `stream`.  Replaces nothing in the reference. */
int flexattn_read_mask_map(void* stream, const FlexAttnParams* p, int which, int b, int index,
                           int32_t out[4]);

/* User score functions, compiled into the tensor-core kernels at run time.  Replaces `make_jax_score_fn`
 * (util.py:150-189), which turns a user's Python function into the code the Pallas kernels inline
 * (flex_attention_kernel.py:248-255), and the jax.vjp of that function inside the backward kernels
 * (flex_attention_dq_bwd.py:340-345,373-380).
 *
 * `score_expr` and `dscore_expr` are CUDA C++ float expressions over `s` (float: the scaled score
 * sm_scale * <q_i, k_j>), `b`, `h`, `i`, `j` (int: batch, head, query and key position) and the CUDA math
 * functions: the score function t = f(s, b, h, i, j) and its derivative df/ds.  The call only records them
 * and returns a handle (> 0) in *handle.  A kernel specialised for the function (and for the head dimension
 * and mask kind of the problem) is compiled with NVRTC and loaded the first time a forward / dQ / dK,dV call
 * uses the handle with score_kind = FLEXATTN_SCORE_USER; that first call blocks for the compilation (seconds),
 * lets the driver allocate the module's code, and must not happen during stream capture.  Later calls launch
 * the cached kernel.  bf16 inputs with D in {64, 128} only (the tensor-core kernels).
 * flexattn_user_score_destroy unloads what was compiled for the handle. */
int flexattn_user_score_create(const char* score_expr, const char* dscore_expr, int32_t* handle);
int flexattn_user_score_destroy(int32_t handle);
/* The compiler's log of the most recent failed compilation for `handle` ("" if none).  Valid until the next call
 * that uses the handle.  Never NULL. */
const char* flexattn_user_score_log(int32_t handle);
/* Compiles (without loading or launching: needs no GPU) the kernel `which` (0 forward, 1 dQ, 2 dK/dV, 3 forward for long rows) for the
 * handle, head_dim and mask_kind, exactly as the first launch would.  Returns FLEXATTN_OK, or
 * FLEXATTN_ERR_JIT_COMPILE / FLEXATTN_ERR_JIT_UNAVAILABLE.  A test and warm-up hook. */
int flexattn_user_score_compile(int32_t handle, int which, int32_t head_dim, int32_t mask_kind);

/* Clears the calling device's abort word (stream-ordered memset on `stream`), re-enabling the tensor-core
 * kernels after a device-side time-out.  Replaces nothing in the reference. */
int flexattn_reset_abort(void* stream);

/* Single-tile tensor-core self checks used by the test-suite (not part of the attention path):
 * D[128,128] = A[128,K] * B^T with A,B bf16 in global memory; `variant` selects the operand
 * staging: 0 = A,B K-major from shared memory; 1 = A from tensor memory (bf16 packed), B MN-major
 * from shared memory (then B is [K,128] row-major).  kdim is 64 or 128.  Output f32 [128,128].
 * The shared-memory descriptors are the ones the attention kernels use.  Replaces nothing in the reference. */
int flexattn_selftest_umma(void* stream, int variant, const void* a, const void* b, float* d,
                           int32_t kdim, int32_t* status);

/* Time-out self check used by the test-suite: one warp waits, for `limit_ms` (1..1000) milliseconds, on a
 * barrier nothing arrives on, then reports exactly like an attention kernel whose wait ran out (status =
 * {FLEXATTN_ERR_TIMEOUT, 101, 0, 1}, abort word set) and returns; the context stays usable.  Replaces
 * nothing in the reference. */
int flexattn_selftest_timeout(void* stream, int32_t limit_ms, int32_t* status);

#ifdef __cplusplus
}
#endif
#endif /* FLEXATTN_H_ */
