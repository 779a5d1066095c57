"""flex_attention_tpu_b200: the flex-attention hot path (forward, delta preprocess, dQ, dK/dV, block-sparse
mask map) as hand-written sm_100a CUDA behind a C ABI, with the reference project's Python entry points
(``_flex_attention_impl``, ``flex_attention_bwd_dq``, ``flash_attention_bwd_dkv`` and the ``masks`` /
``scores`` factories) on top.  Importing the package loads ``libflexattn.so`` and fails if it is missing."""
from . import _binding, masks, scores, util, constants, sharding  # noqa: F401
from .flex_attention_kernel import _flex_attention_impl  # noqa: F401
from .flex_attention_dq_bwd import flex_attention_bwd_dq, bwd_preprocess  # noqa: F401
from .flex_attention_dkv_kernel import flash_attention_bwd_dkv  # noqa: F401
from .flex_attention import flex_attention, flex_attention_bwd  # noqa: F401

__all__ = ["_flex_attention_impl", "flex_attention_bwd_dq", "flash_attention_bwd_dkv", "bwd_preprocess",
           "masks", "scores", "util", "constants"]
