"""The same inputs many times over: every role of the kernels (TMA warp, MMA issuers, compute and epilogue
warpgroups) hands work to the others through barriers, and a missing dependency would show up as a result that
changes with the timing of a run. Outputs and gradients must be bitwise the same in every repetition, on shapes
that make the CTAs take many items each (item boundaries are where buffers change owners). The one exception is
dq of the default (deterministic=False) backward for head dims up to 128: its fp32 partial sums are added with
global reductions in scheduling order, as in the reference (mainloop_bwd_sm90_tma_gmma_ws.hpp:605-664 there), so
it may differ by one rounding step; with deterministic=True it is bitwise stable too."""

import pytest
import torch

from _util import assert_same_gradients
from fast_diffusion_attention import _lib, diffusion_attn_func, diffusion_attn_varlen_func

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _step(q, k, v, do, bs, cu=None, max_len=None, **kw):
    q, k, v = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    if cu is None:
        out, lse = diffusion_attn_func(q, k, v, bs, return_attn_probs=True, **kw)
    else:
        out, lse = diffusion_attn_varlen_func(q, k, v, cu, cu, max_len, max_len, bs, return_attn_probs=True, **kw)
    out.backward(do)
    return out.detach(), lse.detach(), q.grad, k.grad, v.grad


@pytest.mark.parametrize("deterministic", [False, True])
@pytest.mark.parametrize("heads,heads_k,d,bs,n,batch", [
    (16, 16, 128, 256, 2048, 8),    # the benchmark shape: about 14 / 28 items per CTA
    (8, 2, 128, 96, 1100, 3),       # grouped heads, masked tiles, partial last tile
    (6, 6, 64, 32, 1500, 4),
    (4, 4, 256, 128, 1024, 2),
])
def test_bitwise_stable_over_repetitions(heads, heads_k, d, bs, n, batch, deterministic):
    torch.manual_seed(7)
    q = torch.randn(batch, 2 * n, heads, d, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(batch, 2 * n, heads_k, d, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(batch, 2 * n, heads_k, d, device=DEV, dtype=torch.bfloat16)
    do = torch.randn_like(q)
    first = _step(q, k, v, do, bs, deterministic=deterministic)
    junk = torch.empty(64 << 20, device=DEV, dtype=torch.uint8)
    for rep in range(6):
        if rep % 2:
            junk.random_(0, 255)   # other work in between shifts the timing and the cache state
        again = _step(q, k, v, do, bs, deterministic=deterministic)
        for name, a, b in zip(("out", "lse", "dq", "dk", "dv"), again, first):
            assert_same_gradients(f"{name} (repetition {rep})", a, b, exact=deterministic or d > 128 or name != "dq")
    torch.cuda.synchronize()
    assert _lib.device_status()[0] == 0


@pytest.mark.parametrize("deterministic", [False, True])
def test_bitwise_stable_varlen_with_softcap(deterministic):
    torch.manual_seed(8)
    ns = [700, 64, 1300, 0, 257, 2048, 5, 900]
    cu = torch.tensor([0] + list(torch.tensor([2 * x for x in ns]).cumsum(0)), device=DEV, dtype=torch.int32)
    total = 2 * sum(ns)
    q = torch.randn(total, 8, 128, device=DEV, dtype=torch.float16)
    k = torch.randn(total, 4, 128, device=DEV, dtype=torch.float16)
    v = torch.randn(total, 4, 128, device=DEV, dtype=torch.float16)
    do = torch.randn_like(q)
    first = _step(q, k, v, do, 80, cu=cu, max_len=2 * max(ns), softcap=15.0, deterministic=deterministic)
    for rep in range(4):
        again = _step(q, k, v, do, 80, cu=cu, max_len=2 * max(ns), softcap=15.0, deterministic=deterministic)
        for name, a, b in zip(("out", "lse", "dq", "dk", "dv"), again, first):
            assert_same_gradients(f"{name} (repetition {rep})", a, b, exact=deterministic or name != "dq")
    torch.cuda.synchronize()
    assert _lib.device_status()[0] == 0


def test_sm_margin_changes_the_grid_not_the_result():
    """sm_margin leaves SMs free for other work (flash_api.cpp:168-170, :300-301 of the reference): fewer
    persistent CTAs walk the same items, every output is still produced by one item in one fixed order."""
    torch.manual_seed(9)
    q = torch.randn(2, 2 * 900, 8, 128, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(2, 2 * 900, 4, 128, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(2, 2 * 900, 4, 128, device=DEV, dtype=torch.bfloat16)
    do = torch.randn_like(q)
    base = _step(q, k, v, do, 64)
    for margin in (1, 20, 140, 1000):   # more than there are SMs leaves one CTA
        got = _step(q, k, v, do, 64, sm_margin=margin)
        for name, a, b in zip(("out", "lse", "dq", "dk", "dv"), got, base):
            assert_same_gradients(f"{name} with sm_margin={margin}", a, b, exact=name != "dq")
    base = _step(q, k, v, do, 64, deterministic=True)
    for margin in (20, 1000):
        got = _step(q, k, v, do, 64, sm_margin=margin, deterministic=True)
        for name, a, b in zip(("out", "lse", "dq", "dk", "dv"), got, base):
            assert_same_gradients(f"{name} with sm_margin={margin}, deterministic", a, b, exact=True)
    torch.cuda.synchronize()
    assert _lib.device_status()[0] == 0
