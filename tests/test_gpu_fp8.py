"""FP8 (e4m3) forward on the GPU. Method of the reference's own FP8 test (tests/test_diffusion_attn.py:205-247
there): the error against a float32 evaluation of the SAME fp8 inputs must be at most twice the error of a bf16
PyTorch evaluation that also rounds P to e4m3, plus a few ulps; |lse - lse_ref| < 5e-3; the error is unbiased
(|mean err| <= 0.1 * mean |err| + 1e-5). The output is bf16."""

import pytest
import torch

from _util import assert_within_2x
from fast_diffusion_attention import _lib, diffusion_attn_func, diffusion_attn_varlen_func
from oracle import diffusion_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"
E4M3 = torch.float8_e4m3fn


@pytest.mark.parametrize("d", [64, 128, 256])
@pytest.mark.parametrize("heads,heads_k", [(4, 4), (6, 2)])
@pytest.mark.parametrize("use_descale", [False, True])
@pytest.mark.parametrize("varlen", [False, True])
@pytest.mark.parametrize("batch,n,bs", [(2, 300, 4), (1, 517, 32), (2, 64, 1), (1, 400, 160)])
def test_forward_fp8(batch, n, bs, varlen, use_descale, heads, heads_k, d):
    torch.manual_seed(n + d)
    qf, kf, vf = (torch.randn(batch, 2 * n, h, d, device=DEV) for h in (heads, heads_k, heads_k))
    if use_descale:
        descales = [torch.rand(batch, heads_k, device=DEV) + 0.5 for _ in range(3)]
        q8, k8, v8 = ((x / s.repeat_interleave(x.shape[2] // heads_k, dim=1)[:, None, :, None]).to(E4M3)
                      for x, s in zip((qf, kf, vf), descales))
    else:
        descales = [None] * 3
        q8, k8, v8 = (x.to(E4M3) for x in (qf, kf, vf))
    kw = dict(q_descale=descales[0], k_descale=descales[1], v_descale=descales[2])
    if not varlen:
        out, lse = diffusion_attn_func(q8, k8, v8, bs, return_attn_probs=True, **kw)
    else:
        cu = torch.arange(0, batch * 2 * n + 1, 2 * n, device=DEV, dtype=torch.int32)
        flat = [x.reshape(-1, *x.shape[2:]) for x in (q8, k8, v8)]
        out, lse = diffusion_attn_varlen_func(*flat, cu, cu, 2 * n, 2 * n, bs, return_attn_probs=True, **kw)
        out = out.reshape(batch, 2 * n, heads, d)
        lse = lse.reshape(heads, batch, 2 * n).permute(1, 0, 2)
    assert _lib.device_status()[0] == 0
    assert out.dtype == torch.bfloat16
    q16, k16, v16 = (x.to(torch.bfloat16) for x in (q8, k8, v8))  # e4m3 values are exact in bf16
    truth, lse_t = orc.forward(q16, k16, v16, bs, **kw)
    plain, _ = orc.forward(q16, k16, v16, bs, compute_dtype=torch.bfloat16, p_dtype=E4M3, **kw)
    assert_within_2x("out", out, truth, plain)
    assert (lse - lse_t).abs().max().item() < 5e-3
    diff = out.float() - truth.float()
    assert diff.mean().abs().item() <= 0.1 * diff.abs().mean().item() + 1e-5


def test_fp8_backward_is_rejected():
    q8 = torch.randn(1, 64, 2, 64, device=DEV).to(E4M3).requires_grad_()
    out = diffusion_attn_func(q8, q8.detach(), q8.detach(), 4)
    with pytest.raises((AssertionError, RuntimeError)):
        out.float().sum().backward()
