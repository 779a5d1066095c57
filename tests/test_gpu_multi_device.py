"""One process driving two GPUs, as a JAX host does: per-device state of the library (the raised shared-memory
limit of each kernel, the abort word, the SM count, the no-allocation scratch array) must be set up on every
device, not once per process.  Skipped on a single-GPU box."""
import numpy as np
import pytest
import torch

from helpers import make_qkvdo, oracle_hot_path, run_hot_path, assert_close

pytestmark = pytest.mark.gpu


def test_forward_and_backward_on_two_devices_in_one_process():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import flex_attention_tpu_b200 as fa
    sm = 1.0 / np.sqrt(128)
    want = None
    for dev in (0, 1, 0):
        with torch.cuda.device(dev):
            (q, k, v, do), host = make_qkvdo((1, 2, 384, 128), (1, 2, 384, 128), 7, torch.bfloat16, device=f"cuda:{dev}")
            got = run_hot_path(fa, q, k, v, do, sm_scale=sm, mask_kind="causal", backend="tcgen05")
            if want is None:
                want = oracle_hot_path(*host, sm_scale=sm, mask_kind="causal")
            assert_close(got, want, torch.bfloat16, what=f"cuda:{dev}")
