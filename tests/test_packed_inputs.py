"""The packed-projection entry points: one tensor in, one gradient tensor out, the same kernels underneath.

The reference has no such functions (its callers pass views, tests/test_diffusion_attn.py:260-266 there); these tests
therefore compare with this package's own `diffusion_attn_func` / `diffusion_attn_varlen_func` on views of the same
tensor, which the other test files compare with the oracle."""

import pytest
import torch

from fast_diffusion_attention import (
    diffusion_attn_func,
    diffusion_attn_qkvpacked_func,
    diffusion_attn_varlen_func,
    diffusion_attn_varlen_qkvpacked_func,
)
from fast_diffusion_attention.interface import _split_packed
from _util import assert_same_gradients

DEV = "cuda"


# ---------------------------------------------------------------------------------------------- without a GPU
def test_split_views_share_storage():
    qkv = torch.arange(2 * 6 * 3 * 4 * 8, dtype=torch.float32).view(2, 6, 3, 4, 8)
    q, k, v = _split_packed(qkv, None, varlen=False)
    assert q.shape == k.shape == v.shape == (2, 6, 4, 8)
    assert torch.equal(k, qkv[:, :, 1]) and v.data_ptr() == qkv[:, :, 2].data_ptr()
    g = torch.arange(5 * 10 * 8, dtype=torch.float32).view(5, 10, 8)      # (total, 6 + 2 * 2 heads, dim)
    q, k, v = _split_packed(g, 6, varlen=True)
    assert q.shape == (5, 6, 8) and k.shape == v.shape == (5, 2, 8)
    assert torch.equal(v, g[:, 8:10]) and k.data_ptr() == g[:, 6:].data_ptr()
    # (total, 3, heads, dim) has four dimensions like (batch, 2n, heads, dim): the layout decides
    t = torch.zeros(7, 3, 2, 8)
    assert _split_packed(t, None, varlen=True)[0].shape == (7, 2, 8)
    with pytest.raises(ValueError):
        _split_packed(t, None, varlen=False)            # grouped layout without num_heads_q


@pytest.mark.parametrize("shape,heads_q,varlen", [
    ((2, 8, 2, 4, 8), None, False),      # axis of size 2 where 3 belongs
    ((2, 8, 9, 8), 4, False),            # 9 - 4 heads do not split into keys and values
    ((2, 8, 4, 8), 4, False),            # no key / value heads left
    ((2, 8, 3, 4, 8), 5, False),         # num_heads_q disagrees with the head axis
    ((8, 3, 4), None, True),             # too few dimensions
])
def test_split_refuses(shape, heads_q, varlen):
    with pytest.raises(ValueError):
        _split_packed(torch.zeros(shape), heads_q, varlen)


def test_traces_on_meta_tensors():
    qkv = torch.empty(2, 64, 3, 4, 64, dtype=torch.bfloat16, device="meta", requires_grad=True)
    out, lse = diffusion_attn_qkvpacked_func(qkv, 16, return_attn_probs=True)
    assert out.shape == (2, 64, 4, 64) and lse.shape == (2, 4, 64)
    out.sum().backward()
    assert qkv.grad.shape == qkv.shape and qkv.grad.dtype == torch.bfloat16
    g = torch.empty(96, 8 + 2 * 2, 128, dtype=torch.float16, device="meta", requires_grad=True)
    cu = torch.empty(4, dtype=torch.int32, device="meta")
    out = diffusion_attn_varlen_qkvpacked_func(g, cu, 40, 8, num_heads_q=8)
    assert out.shape == (96, 8, 128)
    out.sum().backward()
    assert g.grad.shape == g.shape


# ---------------------------------------------------------------------------------------------- with a GPU
def _randn(*shape, dtype=torch.bfloat16):
    return torch.randn(*shape, device=DEV, dtype=torch.float32).to(dtype).requires_grad_()


def _compare(packed, q, k, v, run_packed, run_views, deterministic):
    out_p, lse_p = run_packed(packed)
    out_v, lse_v = run_views(q, k, v)
    assert torch.equal(out_p, out_v) and torch.equal(lse_p, lse_v)
    g = torch.randn_like(out_p)
    (dpacked,) = torch.autograd.grad(out_p, packed, g)
    dq, dk, dv = torch.autograd.grad(out_v, (q, k, v), g)
    assert dpacked.shape == packed.shape and dpacked.is_contiguous()
    return dpacked, (dq, dk, dv)


@pytest.mark.gpu
@pytest.mark.parametrize("deterministic", [True, False])
@pytest.mark.parametrize("d,dtype", [(128, torch.bfloat16), (64, torch.float16)])
def test_three_way_axis(d, dtype, deterministic):
    torch.manual_seed(3)
    b, n, h, bs = 2, 200, 4, 32
    qkv = _randn(b, 2 * n, 3, h, d, dtype=dtype)
    q, k, v = (qkv.detach()[:, :, i].clone().requires_grad_() for i in range(3))
    dpacked, grads = _compare(
        qkv, q, k, v,
        lambda t: diffusion_attn_qkvpacked_func(t, bs, deterministic=deterministic, return_attn_probs=True),
        lambda a, b_, c: diffusion_attn_func(a, b_, c, bs, deterministic=deterministic, return_attn_probs=True),
        deterministic)
    for i, (name, g) in enumerate(zip(("dq", "dk", "dv"), grads)):
        assert_same_gradients(name, dpacked[:, :, i], g, exact=deterministic or name != "dq")


@pytest.mark.gpu
@pytest.mark.parametrize("heads,heads_k", [(8, 2), (4, 1), (4, 4)])
def test_grouped_head_axis(heads, heads_k):
    torch.manual_seed(4)
    b, n, d, bs = 2, 160, 128, 64
    qkv = _randn(b, 2 * n, heads + 2 * heads_k, d)
    det = qkv.detach()
    q = det[:, :, :heads].clone().requires_grad_()
    k = det[:, :, heads:heads + heads_k].clone().requires_grad_()
    v = det[:, :, heads + heads_k:].clone().requires_grad_()
    dpacked, (dq, dk, dv) = _compare(
        qkv, q, k, v,
        lambda t: diffusion_attn_qkvpacked_func(t, bs, num_heads_q=heads, softcap=20.0, deterministic=True,
                                                return_attn_probs=True),
        lambda a, b_, c: diffusion_attn_func(a, b_, c, bs, softcap=20.0, deterministic=True, return_attn_probs=True),
        True)
    assert torch.equal(dpacked[:, :, :heads], dq)
    assert torch.equal(dpacked[:, :, heads:heads + heads_k], dk)
    assert torch.equal(dpacked[:, :, heads + heads_k:], dv)


@pytest.mark.gpu
@pytest.mark.parametrize("grouped", [False, True])
def test_packed_samples(grouped):
    torch.manual_seed(5)
    lens = [2 * 96, 0, 2 * 37, 2 * 130]
    total, d, bs = sum(lens), 64, 16
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    if grouped:
        heads, heads_k = 6, 3
        qkv = _randn(total, heads + 2 * heads_k, d)
        det = qkv.detach()
        parts = (det[:, :heads], det[:, heads:heads + heads_k], det[:, heads + heads_k:])
        slices = (slice(0, heads), slice(heads, heads + heads_k), slice(heads + heads_k, None))
        num_heads_q = heads
    else:
        qkv = _randn(total, 3, 4, d)
        det = qkv.detach()
        parts = tuple(det[:, i] for i in range(3))
        num_heads_q = None
    q, k, v = (t.clone().requires_grad_() for t in parts)
    dpacked, grads = _compare(
        qkv, q, k, v,
        lambda t: diffusion_attn_varlen_qkvpacked_func(t, cu, max(lens), bs, num_heads_q=num_heads_q,
                                                       deterministic=True, return_attn_probs=True),
        lambda a, b_, c: diffusion_attn_varlen_func(a, b_, c, cu, cu, max(lens), max(lens), bs, deterministic=True,
                                                    return_attn_probs=True),
        True)
    for i, g in enumerate(grads):
        got = dpacked[:, slices[i]] if grouped else dpacked[:, i]
        assert torch.equal(got, g)


@pytest.mark.gpu
def test_compiles_as_one_graph():
    torch.manual_seed(6)
    qkv = torch.randn(1, 2 * 64, 3, 2, 64, device=DEV).to(torch.bfloat16)

    def step(t):
        out = diffusion_attn_qkvpacked_func(t, 16, deterministic=True)
        return out.float().square().sum()

    def run(fn):
        t = qkv.clone().requires_grad_(True)
        fn(t).backward()
        return t.grad

    want = run(step)
    got = run(torch.compile(step, fullgraph=True, backend="aot_eager"))
    assert torch.equal(got, want)
