"""ctypes binding of libflexattn.so (the C ABI declared in include/flexattn.h).

This is the only backend: there is no CPU or PyTorch fallback.  Importing the module without the built
library raises, and every call checks the returned status.
"""
from __future__ import annotations

import ctypes
import os
from collections import OrderedDict

import torch

# FLEXATTN_DEBUG=1 loads the bounds-checked build of the same library (every direct global-memory access of the
# tensor-core kernels guarded; an out-of-range index is reported through the status words as code 14 instead of
# faulting).  Slower; meant for bring-up and for the tests that run without a memory checker.
DEBUG_BUILD = os.environ.get("FLEXATTN_DEBUG", "0") not in ("", "0")
_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)),
                         "libflexattn_debug.so" if DEBUG_BUILD else "libflexattn.so")

DTYPE_BF16, DTYPE_F32 = 0, 1
SCORE_NONE, SCORE_ALIBI, SCORE_SOFTCAP, SCORE_USER = 0, 1, 2, 3
MASK_NONE, MASK_CAUSAL, MASK_SLIDING_WINDOW, MASK_SLIDING_WINDOW_CAUSAL, MASK_DOCUMENT, MASK_S2 = range(6)
BACKEND_AUTO, BACKEND_SIMT, BACKEND_TCGEN05 = 0, 1, 2
TILE = 128
ABI_VERSION = 4   # FLEXATTN_ABI_VERSION of include/flexattn.h this binding was written against

MASK_KIND_IDS = {"none": MASK_NONE, "causal": MASK_CAUSAL, "sliding_window": MASK_SLIDING_WINDOW,
                 "sliding_window_causal": MASK_SLIDING_WINDOW_CAUSAL, "document": MASK_DOCUMENT, "s2": MASK_S2}
SCORE_KIND_IDS = {"none": SCORE_NONE, "alibi": SCORE_ALIBI, "softcap": SCORE_SOFTCAP, "user": SCORE_USER}
BACKEND_IDS = {"auto": BACKEND_AUTO, "simt": BACKEND_SIMT, "tcgen05": BACKEND_TCGEN05}


class FlexAttnParams(ctypes.Structure):
    _fields_ = [
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p), ("o", ctypes.c_void_p),
        ("d_o", ctypes.c_void_p), ("dq", ctypes.c_void_p), ("dk", ctypes.c_void_p), ("dv", ctypes.c_void_p),
        ("l", ctypes.c_void_p), ("m", ctypes.c_void_p), ("delta", ctypes.c_void_p),
        ("doc_ids", ctypes.c_void_p), ("alibi_slopes", ctypes.c_void_p),
        ("batch", ctypes.c_int32), ("heads", ctypes.c_int32), ("seq_q", ctypes.c_int32),
        ("seq_k", ctypes.c_int32), ("head_dim", ctypes.c_int32),
        ("dtype", ctypes.c_int32), ("sm_scale", ctypes.c_float),
        ("score_kind", ctypes.c_int32), ("softcap", ctypes.c_float),
        ("mask_kind", ctypes.c_int32), ("window", ctypes.c_int32), ("stride", ctypes.c_int32),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_size_t),
        ("status", ctypes.c_void_p), ("backend", ctypes.c_int32), ("user_score", ctypes.c_int32),
        ("ab", ctypes.c_void_p), ("dab", ctypes.c_void_p),
    ]


class FlexAttnError(RuntimeError):
    def __init__(self, code, where):
        self.code = code
        super().__init__(f"{where}: {status_string(code)} (status {code})")


def _load():
    if not os.path.exists(_LIB_PATH):
        raise ImportError(
            f"{_LIB_PATH} is missing: build it with `python flex_attention_tpu_b200/build.py` "
            "(there is no fallback implementation)")
    lib = ctypes.CDLL(_LIB_PATH)
    P = ctypes.POINTER(FlexAttnParams)
    lib.flexattn_abi_version.restype = ctypes.c_int
    lib.flexattn_status_string.restype = ctypes.c_char_p
    lib.flexattn_status_string.argtypes = [ctypes.c_int]
    lib.flexattn_workspace_bytes.restype = ctypes.c_size_t
    lib.flexattn_workspace_bytes.argtypes = [P]
    for name in ("flexattn_build_mask_map", "flexattn_fwd", "flexattn_bwd_preprocess", "flexattn_bwd_dq",
                 "flexattn_bwd_dkv"):
        fn = getattr(lib, name)
        fn.restype = ctypes.c_int
        fn.argtypes = [ctypes.c_void_p, P]
    lib.flexattn_fwd_noalloc.restype = ctypes.c_int
    lib.flexattn_fwd_noalloc.argtypes = [ctypes.c_void_p, P]
    lib.flexattn_noalloc_scratch_bytes.restype = ctypes.c_size_t
    lib.flexattn_read_mask_map.restype = ctypes.c_int
    lib.flexattn_read_mask_map.argtypes = [ctypes.c_void_p, P, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                           ctypes.POINTER(ctypes.c_int32)]
    lib.flexattn_selftest_umma.restype = ctypes.c_int
    lib.flexattn_selftest_umma.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                                           ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p]
    lib.flexattn_selftest_timeout.restype = ctypes.c_int
    lib.flexattn_selftest_timeout.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p]
    lib.flexattn_reset_abort.restype = ctypes.c_int
    lib.flexattn_reset_abort.argtypes = [ctypes.c_void_p]
    lib.flexattn_user_score_create.restype = ctypes.c_int
    lib.flexattn_user_score_create.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.POINTER(ctypes.c_int32)]
    lib.flexattn_user_score_destroy.restype = ctypes.c_int
    lib.flexattn_user_score_destroy.argtypes = [ctypes.c_int32]
    lib.flexattn_user_score_log.restype = ctypes.c_char_p
    lib.flexattn_user_score_log.argtypes = [ctypes.c_int32]
    lib.flexattn_user_score_compile.restype = ctypes.c_int
    lib.flexattn_user_score_compile.argtypes = [ctypes.c_int32, ctypes.c_int, ctypes.c_int32, ctypes.c_int32]
    if lib.flexattn_abi_version() != ABI_VERSION:
        raise ImportError("libflexattn.so ABI version mismatch: rebuild the library")
    return lib


lib = _load()


def status_string(code: int) -> str:
    return lib.flexattn_status_string(int(code)).decode()


def check(code: int, where: str):
    if code != 0:
        raise FlexAttnError(code, where)


_USER_SCORES = {}   # (score expression, derivative expression) -> handle of the library


def user_score_handle(score_expr: str, dscore_expr: str) -> int:
    """Registers a pair of CUDA expressions with the library (once per distinct pair) and returns its handle."""
    key = (score_expr, dscore_expr)
    h = _USER_SCORES.get(key)
    if h is None:
        out = ctypes.c_int32(0)
        check(lib.flexattn_user_score_create(score_expr.encode(), dscore_expr.encode(), ctypes.byref(out)),
              "flexattn_user_score_create")
        h = _USER_SCORES[key] = int(out.value)
    return h


def check_user(code: int, where: str, handle: int):
    """`check` that appends the run-time compiler's log when a user score function failed to compile."""
    if code == 13:
        log = lib.flexattn_user_score_log(handle).decode(errors="replace")
        raise FlexAttnError(code, f"{where}\n{log}")
    check(code, where)


def _stream_ptr(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


# ------------------------------------------------------------------------------------------ failure mailbox
# A device-side wait that gives up reports through four status words.  When the caller passes no `status`
# tensor the binding supplies one of its own per device, in pinned host memory the device writes through the
# bus: the host can then look at it at the start of every call WITHOUT synchronising, and raises on the first
# call after the failure became visible.  A time-out is sticky on its device until `reset_abort` has run.
_MAILBOX = {}


def _mailbox(device):
    key = device.index if device.index is not None else torch.cuda.current_device()
    box = _MAILBOX.get(key)
    if box is None:
        box = _MAILBOX[key] = torch.zeros(4, dtype=torch.int32).pin_memory()
    return box


def raise_if_failed(device):
    """Raises FlexAttnError if an earlier launch on `device` reported a device-side time-out into the binding's
    own status words.  Never synchronises."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    box = _MAILBOX.get(key)
    if box is not None and int(box[0]) != 0:
        code, kernel, block, detail = (int(x) for x in box.tolist())
        raise FlexAttnError(code, f"an earlier launch on cuda:{key} (kernel id {kernel}, block {block}, detail {detail}; "
                                  "outputs of launches since then are not valid; call reset_abort() to re-arm)")


def reset_abort(device=None):
    """Clears the device's abort word (stream-ordered on the current stream) and the binding's status words."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    check(lib.flexattn_reset_abort(_stream_ptr(device)), "flexattn_reset_abort")
    torch.cuda.current_stream(device).synchronize()
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key in _MAILBOX:
        _MAILBOX[key].zero_()


# Debug switch for the test-suite: every output tensor the binding allocates is filled with NaN before the
# kernels run, so an element a kernel failed to write cannot pass for a result left over from an earlier call.
POISON_OUTPUTS = os.environ.get("FLEXATTN_POISON_OUTPUTS", "0") not in ("", "0")


class Problem:
    """One attention problem: shapes, score/mask spec and the tensors bound so far.  Owns the mask-map
    workspace (a torch buffer) and rebuilds the map only when the mask inputs change."""

    _map_cache: "OrderedDict[tuple, torch.Tensor]" = OrderedDict()
    _MAP_CACHE_ENTRIES = 16

    def __init__(self, q, k, *, sm_scale, mask_kind=MASK_NONE, window=0, stride=0, doc_ids=None,
                 score_kind=SCORE_NONE, softcap=0.0, alibi_slopes=None, backend=BACKEND_AUTO, status=None, ab=None,
                 user_score=0):
        if not q.is_cuda:
            raise ValueError("flex attention tensors must live on a CUDA device (no CPU path exists)")
        if q.dim() != 4 or k.dim() != 4:
            raise ValueError("expected [batch, heads, seq, head_dim] tensors")
        if q.dtype not in (torch.bfloat16, torch.float32):
            raise NotImplementedError(f"dtype {q.dtype} is not supported (bfloat16 or float32)")
        self.device = q.device
        self.dtype = q.dtype
        B, H, Sq, D = q.shape
        self.shape_q = (B, H, Sq, D)
        self.shape_k = tuple(k.shape)
        p = FlexAttnParams()
        p.batch, p.heads, p.seq_q, p.seq_k, p.head_dim = B, H, Sq, k.shape[2], D
        p.dtype = DTYPE_BF16 if q.dtype == torch.bfloat16 else DTYPE_F32
        p.sm_scale = float(sm_scale)
        p.score_kind, p.softcap = int(score_kind), float(softcap)
        p.mask_kind, p.window, p.stride = int(mask_kind), int(window), int(stride)
        p.backend = int(backend)
        p.user_score = int(user_score)
        self._keep = {}  # tensors whose pointers sit in `p`, by field name
        if mask_kind == MASK_DOCUMENT:
            if doc_ids is None:
                raise ValueError("document mask needs segment/doc ids")
            doc_ids = torch.as_tensor(doc_ids)
            if doc_ids.dim() == 1:
                doc_ids = doc_ids[None].expand(B, -1)
            doc_ids = doc_ids.to(device=self.device, dtype=torch.int32).contiguous()
            if doc_ids.shape != (B, max(Sq, k.shape[2])):
                raise ValueError(f"doc ids must be [batch, {max(Sq, k.shape[2])}], got {tuple(doc_ids.shape)}")
            p.doc_ids = doc_ids.data_ptr()
            self._keep["doc_ids"] = doc_ids
        self.doc_ids = doc_ids if mask_kind == MASK_DOCUMENT else None
        if score_kind == SCORE_ALIBI:
            slopes = self._device_slopes(alibi_slopes, H)
            p.alibi_slopes = slopes.data_ptr()
            self._keep["alibi_slopes"] = slopes
        if status is None:
            raise_if_failed(self.device)
            status = _mailbox(self.device)
        p.status = status.data_ptr()
        self._keep["status"] = status
        self.ab = None
        if ab is not None:
            # dense additive bias [B,H,Sq,Sk], float32
            if not (isinstance(ab, torch.Tensor) and ab.is_cuda):
                raise ValueError("ab must be a CUDA tensor")
            if tuple(ab.shape) != (B, H, Sq, k.shape[2]):
                raise ValueError(f"Attention bias shape mismatch: expected {(B, H, Sq, k.shape[2])}, got {tuple(ab.shape)}")
            self.ab = ab.to(torch.float32).contiguous()
            p.ab = self.ab.data_ptr()
            self._keep["ab"] = self.ab
        self.p = p
        self._bind_workspace()

    _slope_cache: "OrderedDict[tuple, torch.Tensor]" = OrderedDict()

    def _device_slopes(self, alibi_slopes, H):
        """[H] float32 slopes on the device.  Host values are uploaded once and cached: a pageable
        host-to-device copy waits for the stream, which would serialise every call behind the last."""
        if isinstance(alibi_slopes, torch.Tensor) and alibi_slopes.is_cuda:
            slopes = alibi_slopes.to(torch.float32).flatten()
            if slopes.numel() == 1:
                slopes = slopes.expand(H)
            if slopes.numel() != H:
                raise ValueError(f"need one ALiBi slope per head ({H}), got {slopes.numel()}")
            return slopes.contiguous()
        vals = tuple(float(x) for x in torch.as_tensor(alibi_slopes, dtype=torch.float32).flatten().tolist())
        if len(vals) == 1:
            vals = vals * H
        if len(vals) != H:
            raise ValueError(f"need one ALiBi slope per head ({H}), got {len(vals)}")
        key = (self.device.index, vals)
        cache = Problem._slope_cache
        t = cache.get(key)
        if t is None:
            t = torch.tensor(vals, dtype=torch.float32).to(self.device)
            cache[key] = t
            while len(cache) > 16:
                cache.popitem(last=False)
        return t

    # ------------------------------------------------------------------ mask map
    def _bind_workspace(self):
        p = self.p
        nbytes = lib.flexattn_workspace_bytes(ctypes.byref(p))
        if nbytes == 0:
            raise FlexAttnError(2, "flexattn_workspace_bytes")
        doc_key = None
        if self.doc_ids is not None:
            doc_key = (self.doc_ids.data_ptr(), self.doc_ids._version)
        key = (self.device.index, p.mask_kind, p.window, p.stride, p.batch, p.seq_q, p.seq_k, doc_key)
        cache = Problem._map_cache
        hit = cache.get(key)
        ws = None if hit is None else hit[0]
        fresh = ws is None
        if fresh:
            ws = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        else:
            cache.move_to_end(key)
        p.workspace, p.workspace_bytes = ws.data_ptr(), nbytes
        self.workspace = ws
        if fresh:
            check(lib.flexattn_build_mask_map(_stream_ptr(self.device), ctypes.byref(p)), "flexattn_build_mask_map")
            # the entry keeps the doc-id tensor alive, so its (pointer, version) key cannot be recycled
            cache[key] = (ws, self.doc_ids)
            while len(cache) > Problem._MAP_CACHE_ENTRIES:
                cache.popitem(last=False)

    def read_map(self, which: int, b: int, index: int):
        out = (ctypes.c_int32 * 4)()
        check(lib.flexattn_read_mask_map(_stream_ptr(self.device), ctypes.byref(self.p), which, b, index, out),
              "flexattn_read_mask_map")
        return tuple(out)

    # ------------------------------------------------------------------ tensors
    def _bind(self, **tensors):
        for name, t in tensors.items():
            if t is None:
                continue
            if not t.is_cuda or t.device != self.device:
                raise ValueError(f"{name} must be on {self.device}")
            if not t.is_contiguous():
                raise ValueError(f"{name} must be contiguous")
            want = torch.float32 if name in ("l", "m", "delta") else self.dtype
            if t.dtype != want:
                raise ValueError(f"{name} must be {want}, got {t.dtype}")
            setattr(self.p, name, t.data_ptr())
            self._keep[name] = t

    def _new(self, shape, dtype=None):
        if POISON_OUTPUTS:
            return torch.full(shape, float("nan"), dtype=dtype or self.dtype, device=self.device)
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)

    def forward(self, q, k, v):
        B, H, Sq, D = self.shape_q
        o, l, m = self._new(self.shape_q), self._new((B, H, Sq), torch.float32), self._new((B, H, Sq), torch.float32)
        self._bind(q=q, k=k, v=v, o=o, l=l, m=m)
        check_user(lib.flexattn_fwd(_stream_ptr(self.device), ctypes.byref(self.p)), "flexattn_fwd", self.p.user_score)
        return o, l, m

    def preprocess(self, o, do):
        B, H, Sq, _ = self.shape_q
        delta = self._new((B, H, Sq), torch.float32)
        self._bind(o=o, d_o=do, delta=delta)
        check(lib.flexattn_bwd_preprocess(_stream_ptr(self.device), ctypes.byref(self.p)), "flexattn_bwd_preprocess")
        return delta

    def bwd_dq(self, q, k, v, do, l, m, delta, want_dab=False):
        """dq, or (dq, dab) with ``want_dab`` (dab: float32 [B,H,Sq,Sk], the gradient of the dense bias)."""
        dq = self._new(self.shape_q)
        self._bind(q=q, k=k, v=v, d_o=do, l=l, m=m, delta=delta, dq=dq)
        dab = None
        if want_dab:
            if self.ab is None:
                raise ValueError("dab was requested but the problem has no bias `ab`")
            dab = self._new(self.ab.shape, torch.float32)
            self.p.dab = dab.data_ptr()
        try:
            check_user(lib.flexattn_bwd_dq(_stream_ptr(self.device), ctypes.byref(self.p)), "flexattn_bwd_dq", self.p.user_score)
        finally:
            self.p.dab = None
        return (dq, dab) if want_dab else dq

    def bwd_dkv(self, q, k, v, do, l, m, delta):
        dk, dv = self._new(self.shape_k), self._new(self.shape_k)
        self._bind(q=q, k=k, v=v, d_o=do, l=l, m=m, delta=delta, dk=dk, dv=dv)
        check_user(lib.flexattn_bwd_dkv(_stream_ptr(self.device), ctypes.byref(self.p)), "flexattn_bwd_dkv", self.p.user_score)
        return dk, dv

    def backward(self, q, k, v, o, do, l, m, need_dq=True, need_dkv=True, want_dab=False, two_streams=None):
        """delta, then dQ and dK/dV.  The two gradient kernels only share inputs, so dK/dV is launched on a side
        stream: both kernels fill every SM on their own, but the tail of one then overlaps the head of the other.
        Everything is ordered after the current stream's work and the current stream waits for both.
        ``two_streams=False`` launches both on the current stream (the host-buffer pipeline does: there the
        extra stream only adds synchronisation between the copy and compute streams)."""
        delta = self.preprocess(o, do)
        if want_dab:  # the bias gradient comes out of the dQ kernel
            dq, dab = self.bwd_dq(q, k, v, do, l, m, delta, want_dab=True)
            dk, dv = self.bwd_dkv(q, k, v, do, l, m, delta) if need_dkv else (None, None)
            return delta, dq, dk, dv, dab
        if two_streams is None:
            two_streams = TWO_STREAM_BACKWARD
        if not (need_dq and need_dkv and two_streams):
            dq = self.bwd_dq(q, k, v, do, l, m, delta) if need_dq else None
            dk, dv = self.bwd_dkv(q, k, v, do, l, m, delta) if need_dkv else (None, None)
            return delta, dq, dk, dv
        cur = torch.cuda.current_stream(self.device)
        side = _side_stream(self.device)
        dk, dv = self._new(self.shape_k), self._new(self.shape_k)   # allocated on the current stream
        side.wait_stream(cur)
        self._bind(q=q, k=k, v=v, d_o=do, l=l, m=m, delta=delta, dk=dk, dv=dv)
        check_user(lib.flexattn_bwd_dkv(ctypes.c_void_p(side.cuda_stream), ctypes.byref(self.p)), "flexattn_bwd_dkv", self.p.user_score)
        dq = self.bwd_dq(q, k, v, do, l, m, delta)
        cur.wait_stream(side)
        return delta, dq, dk, dv


_SIDE_STREAMS = {}
# dK/dV on a side stream next to dQ (see Problem.backward); False launches the two kernels one after the other
TWO_STREAM_BACKWARD = os.environ.get("FLEXATTN_TWO_STREAM", "1") != "0"


def _side_stream(device):
    """One long-lived side stream per device for `Problem.backward` (created on first use)."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    st = _SIDE_STREAMS.get(key)
    if st is None:
        st = _SIDE_STREAMS[key] = torch.cuda.Stream(device)
    return st


def selftest_umma(variant: int, a: torch.Tensor, b: torch.Tensor, status=None) -> torch.Tensor:
    """Single-tile tensor-core self check (see flexattn_selftest_umma in the header)."""
    kdim = a.shape[1]
    d = torch.empty(128, 128, dtype=torch.float32, device=a.device)
    check(lib.flexattn_selftest_umma(_stream_ptr(a.device), int(variant), _ptr(a), _ptr(b), _ptr(d), int(kdim),
                                     _ptr(status)), "flexattn_selftest_umma")
    return d


def selftest_timeout(limit_ms: int, status=None, device=None):
    """Launches the time-out self check (see flexattn_selftest_timeout in the header): a wait that runs out
    after `limit_ms` and reports like an attention kernel would.  With ``status=None`` the report goes to the
    binding's own status words."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if status is None:
        status = _mailbox(device)
    check(lib.flexattn_selftest_timeout(_stream_ptr(device), int(limit_ms), _ptr(status)), "flexattn_selftest_timeout")
