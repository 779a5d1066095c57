"""Host side of the failure report, without a GPU: the binding keeps four status words per device that the kernels
write when a bounded wait gives up; every entry point looks at them first and raises on the first call after a
failure became visible, naming the kernel, and goes on raising until reset_abort() has cleared them."""
import pytest
import torch

from flex_attention_tpu_b200 import _binding as B


def test_a_reported_timeout_raises_on_the_next_call_and_names_the_kernel(monkeypatch):
    dev = torch.device("cuda", 3)  # never touched: the check reads host memory only
    monkeypatch.setitem(B._MAILBOX, 3, torch.zeros(4, dtype=torch.int32))
    B.raise_if_failed(dev)  # clean words: nothing happens
    B._MAILBOX[3].copy_(torch.tensor([9, 4, 17, 99], dtype=torch.int32))  # TIMEOUT, forward kernel, block 17, aborted on entry
    with pytest.raises(B.FlexAttnError) as e:
        B.raise_if_failed(dev)
    assert e.value.code == 9 and "kernel id 4" in str(e.value) and "block 17" in str(e.value) and "reset_abort" in str(e.value)
    with pytest.raises(B.FlexAttnError):  # sticky until cleared
        B.raise_if_failed(dev)
    B._MAILBOX[3].zero_()
    B.raise_if_failed(dev)


def test_devices_are_kept_apart(monkeypatch):
    monkeypatch.setitem(B._MAILBOX, 0, torch.zeros(4, dtype=torch.int32))
    monkeypatch.setitem(B._MAILBOX, 1, torch.tensor([9, 3, 0, 4], dtype=torch.int32))
    B.raise_if_failed(torch.device("cuda", 0))
    with pytest.raises(B.FlexAttnError):
        B.raise_if_failed(torch.device("cuda", 1))


def test_status_code_9_is_the_timeout():
    assert "time" in B.status_string(9).lower()
