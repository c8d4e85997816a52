"""The benchmark configurations at their full sizes.

The float32 oracle materialises (2n)^2 scores per head, so at these sizes it checks one sample and one key/value
head group; everything else is covered by identities that hold for any correct result whatever the size:

  * rows of the probabilities sum to one: with V = 1 every output element is 1;
  * sum_j dV_j = sum_i dO_i per key/value head (again because the probability rows sum to one);
  * sum_i <q_i, dq_i> = sum_j <k_j, dk_j> per key/value head (the scores depend on q and k through q.k only);
  * the mask: changing the clean tokens of one block changes exactly the outputs the mask lets see that block
    (bitwise nothing else), changing noisy tokens of a block only the noisy outputs of that block;
  * two backward passes over the same inputs give bitwise the same gradients.
"""

import math

import pytest
import torch

from oracle import diffusion_oracle as oracle
from fast_diffusion_attention import diffusion_attn_func, diffusion_attn_varlen_func
from fast_diffusion_attention import _lib

from _util import assert_within_2x

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0) if torch.cuda.is_available() else None


def _randn(shape, seed, dtype=torch.bfloat16):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return torch.randn(shape, generator=g, device=DEV, dtype=torch.float32).to(dtype)


def _grads(q, k, v, do, bs, cu=None, max_n=None, **kw):
    q, k, v = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    if cu is None:
        out, lse = diffusion_attn_func(q, k, v, bs, return_attn_probs=True, **kw)
    else:
        out, lse = diffusion_attn_varlen_func(q, k, v, cu, cu, max_n, max_n, bs, return_attn_probs=True, **kw)
    out.backward(do)
    torch.cuda.synchronize()
    assert _lib.device_status()[0] == 0
    _grads.lse = lse.detach()   # (batch, heads, rows) or (heads, total): checked by _check_slice
    return out.detach(), q.grad, k.grad, v.grad


def _identities(q, k, v, do, out, dq, dk, dv, group, sample_rows=None):
    """The size-independent identities; tensors are (rows, heads, d) per sample (batch folded by the caller)."""
    Hk = k.shape[-2]
    # sum_j dV_j = sum_i dO_i over the query heads of each group
    do_sum = do.float().sum(0).reshape(Hk, group, -1).sum(1)            # (Hk, d)
    dv_sum = dv.float().sum(0)                                          # (Hk, d)
    rows = q.shape[0]
    # dv entries are rounded to 16 bits: a sum of `rows` of them carries about sqrt(rows) * 2^-9 * |dv| of noise
    # (and so does every probability that went into them)
    tol = 6 * math.sqrt(rows) * 2 ** -9 * max(dv.float().abs().mean().item(), do.float().abs().mean().item()) + 1e-3
    assert (do_sum - dv_sum).abs().max().item() <= tol, ((do_sum - dv_sum).abs().max().item(), tol)
    # sum_i <q_i, dq_i> = sum_j <k_j, dk_j>
    lhs = (q.float() * dq.float()).sum((0, 2)).reshape(Hk, group).sum(1)
    rhs = (k.float() * dk.float()).sum((0, 2))
    scale = (q.float() * dq.float()).abs().sum((0, 2)).reshape(Hk, group).sum(1)
    assert ((lhs - rhs).abs() <= 2e-3 * scale + 1e-2).all(), ((lhs - rhs).abs().max().item(), scale.max().item())


def _oracle_slice(q, k, v, do, bs, hk, group, softcap=0.0):
    """float32 truth and the plain same-precision result for one key/value head and its query heads; tensors
    are (1, 2n, heads, d)."""
    hs = slice(hk * group, (hk + 1) * group)
    qs, ks, vs, gs = q[:, :, hs], k[:, :, hk:hk + 1], v[:, :, hk:hk + 1], do[:, :, hs]
    out_t, lse_t = oracle.forward(qs, ks, vs, bs, softcap=softcap)
    out_p, _ = oracle.forward(qs, ks, vs, bs, softcap=softcap, compute_dtype=q.dtype)
    g_t = oracle.backward(qs, ks, vs, gs, bs, softcap=softcap)
    g_p = oracle.backward(qs, ks, vs, gs, bs, softcap=softcap, compute_dtype=q.dtype)
    return hs, out_t, out_p, lse_t, g_t, g_p


def _check_slice(name, q, k, v, do, out, dq, dk, dv, bs, hk, group, softcap=0.0, lse=None):
    """`lse`: the log-sum-exp rows of the same sample, (heads, rows)."""
    hs, out_t, out_p, lse_t, g_t, g_p = _oracle_slice(q, k, v, do, bs, hk, group, softcap)
    assert_within_2x(name + " out", out[:, :, hs], out_t, out_p)
    assert lse is not None
    # natural-log units, float32; the tolerance of the reference's tests (tests/test_diffusion_attn.py:98 there,
    # 2 x the plain error + 1e-4) with the plain error bounded by bf16 rounding of scores of this magnitude
    assert (lse[hs].float() - lse_t[0].float()).abs().max().item() <= 2e-2, name + " lse"
    assert_within_2x(name + " dq", dq[:, :, hs], g_t[0], g_p[0])
    assert_within_2x(name + " dk", dk[:, :, hk:hk + 1], g_t[1], g_p[1])
    assert_within_2x(name + " dv", dv[:, :, hk:hk + 1], g_t[2], g_p[2])


def test_mha_bf16_d128_block256():
    """B=8, n=2048, H=16, d=128, block_size=256 (the configuration the headline number is quoted on)."""
    B, n, H, d, bs = 8, 2048, 16, 128, 256
    q, k, v, do = (_randn((B, 2 * n, H, d), s) for s in (1, 2, 3, 4))
    out, dq, dk, dv = _grads(q, k, v, do, bs)
    for b in (0, B - 1):
        _identities(q[b], k[b], v[b], do[b], out[b], dq[b], dk[b], dv[b], 1)
    _check_slice("C2", q[3:4], k[3:4], v[3:4], do[3:4], out[3:4], dq[3:4], dk[3:4], dv[3:4], bs, 5, 1, lse=_grads.lse[3])
    ones = diffusion_attn_func(q, k, torch.ones_like(v), bs)
    assert (ones.float() - 1).abs().max().item() <= 2 ** -7
    # mask: clean block 3 is seen by noisy blocks 4.. and clean blocks 3..; noisy block 2 only by itself
    k2, v2 = k.clone(), v.clone()
    k2[:, n + 3 * bs:n + 4 * bs] += 1
    v2[:, n + 3 * bs:n + 4 * bs] -= 1
    out2 = diffusion_attn_func(q, k2, v2, bs)
    same = torch.ones(2 * n, dtype=torch.bool, device=DEV)
    same[4 * bs:n] = False
    same[n + 3 * bs:] = False
    assert torch.equal(out2[:, same], out[:, same])
    assert not torch.equal(out2[:, ~same], out[:, ~same])
    k3 = k.clone()
    k3[:, 2 * bs:3 * bs] *= -1
    out3 = diffusion_attn_func(q, k3, v, bs)
    same = torch.ones(2 * n, dtype=torch.bool, device=DEV)
    same[2 * bs:3 * bs] = False
    assert torch.equal(out3[:, same], out[:, same])


def test_gqa_bf16_d128_block1024_deterministic():
    """B=4, n=4096, Hq=32, Hkv=8, d=128, block_size=1024, deterministic backward."""
    B, n, H, Hk, d, bs = 4, 4096, 32, 8, 128, 1024
    q, do = _randn((B, 2 * n, H, d), 11), _randn((B, 2 * n, H, d), 12)
    k, v = _randn((B, 2 * n, Hk, d), 13), _randn((B, 2 * n, Hk, d), 14)
    out, dq, dk, dv = _grads(q, k, v, do, bs, deterministic=True)
    lse_c3 = _grads.lse
    out_b, dq_b, dk_b, dv_b = _grads(q, k, v, do, bs, deterministic=True)
    for a, b in ((out, out_b), (dq, dq_b), (dk, dk_b), (dv, dv_b)):
        assert torch.equal(a, b)
    _identities(q[1], k[1], v[1], do[1], out[1], dq[1], dk[1], dv[1], H // Hk)
    _check_slice("C3", q[2:3], k[2:3], v[2:3], do[2:3], out[2:3], dq[2:3], dk[2:3], dv[2:3], bs, 6, H // Hk,
                 lse=lse_c3[2])


def test_varlen_bf16_d64_block256_softcap():
    """16 packed samples, n a multiple of 256 in [512, 8192], H=32, d=64, block_size=256, softcap=30."""
    H, d, bs, softcap = 32, 64, 256, 30.0
    g = torch.Generator().manual_seed(2024)
    ns = [256 * int(x) for x in torch.randint(2, 33, (16,), generator=g)]
    cu = torch.tensor([0] + list(torch.tensor([2 * x for x in ns]).cumsum(0)), device=DEV, dtype=torch.int32)
    total = 2 * sum(ns)
    q, k, v, do = (_randn((total, H, d), s) for s in (21, 22, 23, 24))
    out, dq, dk, dv = _grads(q, k, v, do, bs, cu=cu, max_n=2 * max(ns), softcap=softcap)
    big = max(range(16), key=lambda i: ns[i])
    small = min(range(16), key=lambda i: ns[i])
    for i in (big, small):
        lo, hi = int(cu[i]), int(cu[i + 1])
        _identities(q[lo:hi], k[lo:hi], v[lo:hi], do[lo:hi], out[lo:hi], dq[lo:hi], dk[lo:hi], dv[lo:hi], 1)
    lo, hi = int(cu[big]), int(cu[big + 1])
    sl = lambda t: t[lo:hi].unsqueeze(0)
    _check_slice("C4", sl(q), sl(k), sl(v), sl(do), sl(out), sl(dq), sl(dk), sl(dv), bs, 17, 1, softcap=softcap,
                 lse=_grads.lse[:, lo:hi])


def test_d256_bf16_and_fp8_forward():
    """B=2, n=8192, H=8, d=256, block_size=256: bf16 forward + backward, and the FP8 forward with per-head
    descales amax / 448."""
    B, n, H, d, bs = 2, 8192, 8, 256, 256
    q, k, v, do = (_randn((B, 2 * n, H, d), s) for s in (31, 32, 33, 34))
    out, dq, dk, dv = _grads(q, k, v, do, bs)
    lse_c5 = _grads.lse
    _identities(q[0], k[0], v[0], do[0], out[0], dq[0], dk[0], dv[0], 1)
    _check_slice("C5", q[1:2], k[1:2], v[1:2], do[1:2], out[1:2], dq[1:2], dk[1:2], dv[1:2], bs, 2, 1, lse=lse_c5[1])

    def quantise(t):
        amax = t.float().abs().amax(dim=(1, 3))                  # (B, heads)
        descale = (amax / 448.0).clamp_min(1e-12)
        t8 = (t.float() / descale[:, None, :, None]).to(torch.float8_e4m3fn)
        return t8, descale.contiguous()

    q8, qd = quantise(q)
    k8, kd = quantise(k)
    v8, vd = quantise(v)
    out8 = diffusion_attn_func(q8, k8, v8, bs, q_descale=qd, k_descale=kd, v_descale=vd)
    torch.cuda.synchronize()
    assert _lib.device_status()[0] == 0
    # against the oracle on the SAME quantised inputs (one head): the only extra rounding is P to e4m3
    h = 5
    s1 = slice(1, 2)
    hs = slice(h, h + 1)
    truth, _ = oracle.forward(q8[s1, :, hs], k8[s1, :, hs], v8[s1, :, hs], bs, q_descale=qd[s1, hs],
                              k_descale=kd[s1, hs], v_descale=vd[s1, hs])
    plain, _ = oracle.forward(q8[s1, :, hs], k8[s1, :, hs], v8[s1, :, hs], bs, q_descale=qd[s1, hs],
                              k_descale=kd[s1, hs], v_descale=vd[s1, hs], p_dtype=torch.float8_e4m3fn)
    assert_within_2x("C5 fp8 out", out8[s1, :, hs], truth, plain)
    # and close to the bf16 result on the unquantised inputs (the reference's own FP8 test: relative error of
    # the whole tensor, tests/test_diffusion_attn.py there)
    rel = (out8.float() - out.float()).norm() / out.float().norm()
    assert rel.item() < 0.1, rel.item()
