"""``make_jax_score_fn`` with the reference's name (reference ``util.py:150-189``).

The reference rewrites a user score function's AST into fusable JAX and lets ``jax.vjp`` differentiate it inside
the backward kernels.  Here a score function already made by a factory of ``scores`` passes through unchanged (it
carries the tag that selects a compile-time functor), and any other function is traced into a CUDA expression,
differentiated symbolically and compiled into the tensor-core kernels at run time (``scores.make_user_score_fn``).
A function the tracer cannot follow raises ``NotImplementedError``: nothing is ever evaluated in Python on the
hot path."""
from . import scores


def make_jax_score_fn(fn):
    if getattr(fn, "spec", None) is not None:
        return fn
    try:
        return scores.make_user_score_fn(fn)
    except (TypeError, AttributeError, ValueError) as e:
        raise NotImplementedError(
            f"this score function cannot be traced into the CUDA kernels ({e}); it may use + - * /, constant "
            "integer powers, where() with comparisons and tanh / exp / log / sqrt / abs / sigmoid / minimum / "
            "maximum on the scaled score, batch, head and positions") from e
