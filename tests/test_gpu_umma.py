"""Single-tile tensor-core self checks through the C ABI: the operand staging every attention kernel
depends on (TMA 128-byte swizzle + tcgen05.mma descriptors; bf16 A operand in tensor memory; MN-major B)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kdim", [64, 128])
@pytest.mark.parametrize("variant", [0, 1])
def test_umma_single_tile(variant, kdim):
    from flex_attention_tpu_b200 import _binding as B
    g = torch.Generator().manual_seed(variant * 10 + kdim)
    a = torch.randn(128, kdim, generator=g).to(torch.bfloat16).cuda()
    if variant == 0:
        b = torch.randn(128, kdim, generator=g).to(torch.bfloat16).cuda()      # [N, K], K contiguous
        want = a.float() @ b.float().T
    else:
        b = torch.randn(kdim, 128, generator=g).to(torch.bfloat16).cuda()      # [K, N], N contiguous
        want = a.float() @ b.float()
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    d = B.selftest_umma(variant, a, b, status=status)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0], f"device-side wait gave up: {status.tolist()}"
    err = (d - want).abs().max().item()
    assert err <= 1e-3 * max(1.0, want.abs().max().item()), f"variant {variant} K={kdim}: max err {err}"
