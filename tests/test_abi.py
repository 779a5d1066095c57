"""The C-ABI library: loads, exports every symbol the header declares, validates arguments.  No GPU."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "flexattn.h")


@pytest.fixture(scope="module")
def B():
    from flex_attention_tpu_b200 import _binding
    return _binding


def _declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(flexattn_[a-z_0-9]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(B):
    names = _declared_symbols()
    assert len(names) >= 10
    for n in names:
        assert hasattr(B.lib, n), f"{n} declared in include/flexattn.h but not exported"


def test_struct_layout_matches_header(B):
    # 13 pointers, 5+1 ints, float, int, float, 3 ints, pointer, size_t, pointer, 2 ints, then (ABI 2) ab and dab
    assert ctypes.sizeof(B.FlexAttnParams) == 200
    assert B.FlexAttnParams.workspace.offset == 152 and B.FlexAttnParams.status.offset == 168
    assert B.FlexAttnParams.ab.offset == 184 and B.FlexAttnParams.dab.offset == 192


def test_status_strings(B):
    assert B.status_string(0) == "ok"
    assert "workspace" in B.status_string(6)
    assert B.status_string(12345) == "unknown status"
    assert B.lib.flexattn_abi_version() == 4


def test_workspace_bytes(B):
    p = B.FlexAttnParams()
    assert B.lib.flexattn_workspace_bytes(ctypes.byref(p)) == 0          # invalid shape
    p.batch, p.heads, p.seq_q, p.seq_k, p.head_dim = 2, 4, 1000, 520, 64
    p.mask_kind = B.MASK_CAUSAL
    n = B.lib.flexattn_workspace_bytes(ctypes.byref(p))
    assert n % 256 == 0 and n >= 64 + 16 * (8 + 5)
    p.mask_kind = B.MASK_DOCUMENT
    assert B.lib.flexattn_workspace_bytes(ctypes.byref(p)) > n            # per batch row + doc min/max


def test_argument_validation_needs_no_gpu(B):
    p = B.FlexAttnParams()
    ref = ctypes.byref(p)
    assert B.lib.flexattn_fwd(None, None) == 1                            # null params
    assert B.lib.flexattn_fwd(None, ref) == 2                             # bad shape
    p.batch, p.heads, p.seq_q, p.seq_k, p.head_dim = 1, 1, 128, 128, 48
    assert B.lib.flexattn_fwd(None, ref) == 4                             # head dim
    p.head_dim, p.dtype = 64, 7
    assert B.lib.flexattn_fwd(None, ref) == 3                             # dtype
    p.dtype, p.mask_kind = 0, 9
    assert B.lib.flexattn_fwd(None, ref) == 7                             # mask kind
    p.mask_kind = B.MASK_SLIDING_WINDOW
    assert B.lib.flexattn_fwd(None, ref) == 7                             # window <= 0
    p.mask_kind = B.MASK_DOCUMENT
    assert B.lib.flexattn_fwd(None, ref) == 1                             # doc ids missing
    p.mask_kind = B.MASK_CAUSAL
    assert B.lib.flexattn_fwd(None, ref) == 1                             # workspace missing
    p.workspace, p.workspace_bytes = 0x1000, 16
    assert B.lib.flexattn_fwd(None, ref) == 6                             # workspace too small
    p.workspace_bytes = 1 << 20
    assert B.lib.flexattn_fwd(None, ref) == 1                             # q missing
    p.q = 0x1008
    assert B.lib.flexattn_fwd(None, ref) == 5                             # misaligned
    p.backend = 2
    p.q = p.k = p.v = p.o = p.l = p.m = 0x1000
    p.dtype = 1
    assert B.lib.flexattn_fwd(None, ref) == 10                            # tcgen05 cannot serve f32
    assert B.lib.flexattn_bwd_preprocess(None, ref) == 1                  # do missing


def test_python_layer_rejects_what_the_kernels_cannot_run():
    import numpy as np
    import torch
    import flex_attention_tpu_b200 as fa
    with pytest.raises(NotImplementedError):
        fa.masks.spec_of(lambda a, b: True)
    with pytest.raises(NotImplementedError):
        fa.util.make_jax_score_fn(lambda a, b: (a @ b.T).sum())      # not an element-wise function of the score
    sf = fa.scores.make_softcap_score_fn(30.0)
    assert fa.util.make_jax_score_fn(sf) is sf
    q = torch.zeros(1, 1, 128, 64)
    with pytest.raises(ValueError):                                       # CPU tensors: no CPU path exists
        fa._flex_attention_impl(q, q, q, None, None, True, True, 1.0, 1, 128, 128, 128, False, None, None, None)
    with pytest.raises(ValueError):                                       # the dense bias must be a CUDA tensor too
        fa._flex_attention_impl(q, q, q, np.zeros(1), None, True, True, 1.0, 1, 128, 128, 128, False, None, None,
                                None)
