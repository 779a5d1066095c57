"""JAX binding of the C ABI: the reference's three entry points as `jax.ffi` custom calls.

The reference calls its kernels from jitted JAX code (``pl.pallas_call`` at ``flex_attention_kernel.py:173-187``,
``flex_attention_dq_bwd.py:251-265``, ``flex_attention_dkv_kernel.py:158-172``).  This module is the same call
sites over ``libflexattn_xla.so`` (``csrc/xla_ffi_shim.cc``, handlers registered for platform "CUDA"): arrays
stay JAX arrays, the work is enqueued on XLA's stream, and the functions remain ``jax.jit``-able with the
mask / score factories of this package as static arguments.

It needs JAX with its FFI headers at build time and JAX at run time.  Where JAX is missing, importing this
module still works, ``available()`` is False and every entry point raises ``ImportError``; nothing falls back
to another implementation.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

from . import masks, scores

_PKG = os.path.dirname(os.path.abspath(__file__))
_SHIM = os.path.join(_PKG, "libflexattn_xla.so")
_TARGETS = ("flexattn_fwd_ffi", "flexattn_preprocess_ffi", "flexattn_dq_ffi", "flexattn_dkv_ffi",
            "flexattn_mask_map_ffi")
_MASK_IDS = {"none": 0, "causal": 1, "sliding_window": 2, "sliding_window_causal": 3, "document": 4, "s2": 5}
_SCORE_IDS = {"none": 0, "alibi": 1, "softcap": 2, "user": 3}
_registered = False

try:  # pragma: no cover - JAX is not installed everywhere this package is
    import jax
    import jax.numpy as jnp
except ImportError:  # pragma: no cover
    jax = jnp = None


def available() -> bool:
    return jax is not None and hasattr(jax, "ffi") and os.path.exists(_SHIM)


def register() -> None:
    """Loads libflexattn_xla.so and registers its handlers with XLA (once per process)."""
    global _registered
    if _registered:
        return
    if jax is None:
        raise ImportError("jax is not installed: the jax.ffi binding of flex_attention_tpu_b200 is unavailable")
    if not os.path.exists(_SHIM):
        raise ImportError(f"{_SHIM} is missing: build it with `python flex_attention_tpu_b200/build.py` "
                          "on a machine where jax.ffi.include_dir() exists")
    ctypes.CDLL(os.path.join(_PKG, "libflexattn.so"), mode=ctypes.RTLD_GLOBAL)
    shim = ctypes.CDLL(_SHIM)
    for name in _TARGETS:
        jax.ffi.register_ffi_target(name, jax.ffi.pycapsule(getattr(shim, name)), platform="CUDA")
    _registered = True


def _workspace_bytes(batch, seq_q, seq_k, mask_kind) -> int:
    from . import _binding as B
    p = B.FlexAttnParams()
    p.batch, p.heads, p.seq_q, p.seq_k, p.head_dim, p.mask_kind = batch, 1, seq_q, seq_k, 128, mask_kind
    return int(B.lib.flexattn_workspace_bytes(ctypes.byref(p)))


def _resolve(q, k, segment_ids, causal, mask_fn, block_mask_fn, score_fn):
    """Static attributes and the two optional operands (doc ids, ALiBi slopes) of one call."""
    mspec = masks.spec_of(mask_fn, block_mask_fn)
    sspec = scores.spec_of(score_fn)
    doc = jnp.zeros((0,), jnp.int32)
    if mspec is None:
        kind = "document" if segment_ids is not None else ("causal" if causal else "none")
        mspec = masks.MaskSpec(kind)
    if mspec.kind == "document":
        if segment_ids is None:
            segment_ids = np.broadcast_to(masks.doc_ids_from_lengths(mspec.doc_lengths)[None], (q.shape[0], q.shape[2]))
        doc = jnp.asarray(segment_ids, jnp.int32)
    slopes = jnp.zeros((0,), jnp.float32)
    attrs = dict(score_kind=np.int32(0), softcap=np.float32(0.0), mask_kind=np.int32(_MASK_IDS[mspec.kind]),
                 window=np.int32(mspec.window), stride=np.int32(mspec.stride), backend=np.int32(0), user_score=np.int32(0))
    if sspec is not None:
        attrs["score_kind"] = np.int32(_SCORE_IDS[sspec.kind])
        attrs["softcap"] = np.float32(sspec.cap)
        if sspec.kind == "user":    # traced by util.make_jax_score_fn; registered with the library of this process
            from . import _binding as B
            attrs["user_score"] = np.int32(B.user_score_handle(sspec.expr, sspec.dexpr))
        if sspec.kind == "alibi":
            vals = np.asarray(sspec.slopes, np.float32)
            slopes = jnp.asarray(np.broadcast_to(vals, (q.shape[1],)) if vals.size == 1 else vals)
    ws = jax.ShapeDtypeStruct((_workspace_bytes(q.shape[0], q.shape[2], k.shape[2], int(attrs["mask_kind"])),), jnp.uint8)
    return attrs, doc, slopes, ws


def _flex_attention_impl(q, k, v, ab, segment_ids, save_residuals, causal, sm_scale, block_b, block_q,
                         block_k_major, block_k, debug, block_mask_fn, mask_fn, score_fn):
    """The reference's forward entry point (``flex_attention_kernel.py:66-193``) on JAX arrays."""
    del block_b, block_q, block_k_major, block_k, debug
    if ab is not None:
        raise NotImplementedError("the dense bias `ab` is served through the torch binding only")
    register()
    attrs, doc, slopes, ws = _resolve(q, k, segment_ids, causal, mask_fn, block_mask_fn, score_fn)
    stat = jax.ShapeDtypeStruct(q.shape[:3], jnp.float32)
    o, l, m, _ = jax.ffi.ffi_call("flexattn_fwd_ffi", (jax.ShapeDtypeStruct(q.shape, q.dtype), stat, stat, ws))(
        q, k, v, doc, slopes, sm_scale=np.float32(sm_scale), **attrs)
    return (o, l, m) if save_residuals else o


def bwd_preprocess(o, do):
    """delta = rowsum(o * do), float32 [B, H, Sq] (``flex_attention_dq_bwd.py:697``)."""
    register()
    return jax.ffi.ffi_call("flexattn_preprocess_ffi", jax.ShapeDtypeStruct(o.shape[:3], jnp.float32))(o, do)


def flex_attention_bwd_dq(q, k, v, ab, segment_ids, l, m, o, do, d, *, block_b=None, block_q=None,
                          block_k_major=None, block_k=None, sm_scale=1.0, debug=False, score_fn=None,
                          mask_fn=None, block_mask_fn=None, causal=False):
    """The reference's dQ entry point (``flex_attention_dq_bwd.py:114-267``) on JAX arrays."""
    del block_b, block_q, block_k_major, block_k, debug, ab
    register()
    if d is None:
        d = bwd_preprocess(o, do)
    attrs, doc, slopes, ws = _resolve(q, k, segment_ids, causal, mask_fn, block_mask_fn, score_fn)
    dq, _ = jax.ffi.ffi_call("flexattn_dq_ffi", (jax.ShapeDtypeStruct(q.shape, q.dtype), ws))(
        q, k, v, do, l, m, d, doc, slopes, sm_scale=np.float32(sm_scale), **attrs)
    return dq


def flash_attention_bwd_dkv(k, v, q, ab, segment_ids, l, m, di, do, *, block_b=None, block_q=None,
                            block_q_major=None, block_k_major=None, block_k=None, sm_scale=1.0, causal=False,
                            debug=False, score_fn=None, mask_fn=None, block_mask_fn=None):
    """The reference's dK/dV entry point (``flex_attention_dkv_kernel.py:23-174``) on JAX arrays."""
    del block_b, block_q, block_q_major, block_k_major, block_k, debug, ab
    register()
    attrs, doc, slopes, ws = _resolve(q, k, segment_ids, causal, mask_fn, block_mask_fn, score_fn)
    kv = jax.ShapeDtypeStruct(k.shape, k.dtype)
    dk, dv, _ = jax.ffi.ffi_call("flexattn_dkv_ffi", (kv, kv, ws))(
        q, k, v, do, l, m, di, doc, slopes, sm_scale=np.float32(sm_scale), **attrs)
    return dk, dv
