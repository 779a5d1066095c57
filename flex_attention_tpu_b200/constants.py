"""Fixed sizes of the CUDA kernels, for callers that want to pad or tile to them.

The reference's ``constants.py`` exports the smallest Pallas block size under the name ``MIN_BLOCK_SIZE``; the name
is kept.  Here it is the edge of the one tile shape every kernel and the mask map use (``FLEXATTN_TILE`` in
``include/flexattn.h``).  The reference's ``dimension_numbers`` (a ``lax.dot_general`` contraction spec) has no
meaning outside JAX and is not provided.
"""
from ._binding import TILE

MIN_BLOCK_SIZE = TILE                 # q-tile and kv-tile edge: 128
SUPPORTED_HEAD_DIMS_TENSOR_CORE = (64, 128)
SUPPORTED_HEAD_DIMS_SIMT = (32, 64, 128)
