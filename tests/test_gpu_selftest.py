"""Tensor-core self test on the GPU: the operand paths of the attention kernels (TMA 128-byte swizzle ->
shared-memory descriptors / tensor-memory A operand -> tcgen05.mma -> tcgen05.ld) against torch.matmul."""

import pytest
import torch

from fast_diffusion_attention import _lib

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("n,k", [(128, 128), (64, 64), (128, 64), (256, 128), (64, 128)])
def test_umma_paths(mode, n, k):
    lib = _lib.load()
    torch.manual_seed(mode * 100 + n + k)
    dev = torch.device("cuda", 0)
    a = torch.randn(128, k, device=dev).to(torch.bfloat16)
    a_arg = a.t().contiguous() if mode == 2 else a   # mode 2 takes the left operand transposed: (k, 128)
    if mode == 0:
        b = torch.randn(n, k, device=dev).to(torch.bfloat16)   # C = A @ B^T
        want = a.float() @ b.float().t()
    else:
        b = torch.randn(k, n, device=dev).to(torch.bfloat16)   # C = A @ B
        want = a.float() @ b.float()
    c = torch.full((128, n), float("nan"), device=dev, dtype=torch.float32)
    with torch.cuda.device(dev):
        rc = lib.fda_selftest_umma(mode, a_arg.data_ptr(), b.data_ptr(), c.data_ptr(), n, k,
                                   torch.cuda.current_stream().cuda_stream)
    _lib.check(rc)
    assert _lib.device_status()[0] == 0
    # fp32 accumulation of exact bf16 products: only the summation order differs
    assert torch.allclose(c, want, atol=1e-3, rtol=1e-4), (c - want).abs().max().item()
