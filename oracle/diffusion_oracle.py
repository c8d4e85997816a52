"""CPU oracle for block-diffusion attention (TEST INFRASTRUCTURE ONLY).

This module is the checker for the CUDA kernels: a plain restatement of the reference's algorithm that
materialises the (2n x 2n) visibility mask and evaluates the attention and its gradients with explicit
formulas (no autograd). It is imported only by the tests, by the smoke check and by the CPU-baseline leg
of the benchmark; the library itself never calls it and has no CPU fallback.

Parity is pinned: `tests/golden/*.npz` were produced by importing the reference's
`fast_diffusion_attention/reference.py` (its `attention_ref` + `torch.autograd.grad`), and
`tests/test_oracle.py` checks every function of this module against those vectors.

What follows which part of the reference (paths inside the reference project):
  visibility()            fast_diffusion_attention/reference.py:20-30   (diffusion_mask)
  count_visible_pairs()   fast_diffusion_attention/reference.py:33-43   (num_visible_pairs)
  forward()               fast_diffusion_attention/reference.py:46-100  (attention_ref)
  forward_varlen()        fast_diffusion_attention/reference.py:103-120 (attention_varlen_ref)
  backward()              the gradients autograd derives from attention_ref; the same formulas the kernels
                          use (csrc/fda/mainloop_bwd_sm90_tma_gmma_ws.hpp:815-984: dP = dO V^T,
                          dS = P * (dP - rowsum(dO * O)), softcap factor 1 - tanh^2)
"""

from __future__ import annotations

import math
from typing import Optional, Sequence

import torch


def visibility(n: int, block_size: int, device=None) -> torch.Tensor:
    """(2n, 2n) bool matrix, rows are queries and columns keys of one [noisy | clean] sample.

    The four rules, with blk(x) = x // block_size counted from the start of each half:
    noisy->noisy same block, noisy->clean strictly earlier block, clean->clean same or earlier block,
    clean->noisy never.
    """
    pos = torch.arange(n, device=device)
    blk = pos // block_size
    same = blk[:, None] == blk[None, :]
    earlier = blk[None, :] < blk[:, None]          # key block strictly before query block
    vis = torch.zeros(2 * n, 2 * n, dtype=torch.bool, device=device)
    vis[:n, :n] = same
    vis[:n, n:] = earlier
    vis[n:, n:] = same | earlier
    return vis


def count_visible_pairs(n: int, block_size: int) -> int:
    """Closed-form number of visible (query, key) pairs of one sample with halves of n tokens."""
    full, tail = divmod(n, block_size)
    lengths = [block_size] * full + ([tail] if tail else [])
    seen = 0
    pairs = 0
    for length in lengths:
        # noisy block: itself + clean prefix; clean block: clean prefix + itself
        pairs += length * (length + seen) + length * (seen + length)
        seen += length
    return pairs


def _expand_kv(x: torch.Tensor, groups: int) -> torch.Tensor:
    return x if groups == 1 else x.repeat_interleave(groups, dim=2)


def forward(q, k, v, block_size: int, softmax_scale: Optional[float] = None, softcap: float = 0.0,
            q_descale=None, k_descale=None, v_descale=None, compute_dtype=torch.float32,
            p_dtype: Optional[torch.dtype] = None):
    """Attention of q (B, 2n, H, d) over k / v (B, 2n, Hk, d) under the diffusion mask.

    compute_dtype=float32 is the truth the kernels are compared with. Passing the input dtype instead gives
    the "plain same-precision implementation" whose error sets the tolerance (scale folded into k, as the
    reference's reorder_ops=True does). p_dtype optionally rounds the probabilities once more (FP8 check).
    Returns (out in the input dtype (bf16 for fp8 inputs), lse float32 (B, H, 2n)).
    """
    out_dtype = torch.bfloat16 if q.dtype == torch.float8_e4m3fn else q.dtype
    B, L, H, d = q.shape
    if L % 2:
        raise ValueError("the sequence length must be even")
    Hk = k.shape[2]
    groups = H // Hk
    scale = 1.0 / math.sqrt(d) if softmax_scale is None else softmax_scale
    low = compute_dtype != torch.float32
    if not low:
        q, k, v = q.float(), k.float(), v.float()
    if q_descale is not None:
        q = (q.float() * q_descale.repeat_interleave(groups, dim=1)[:, None, :, None]).to(q.dtype)
    if k_descale is not None:
        k = (k.float() * k_descale[:, None, :, None]).to(k.dtype)
    if v_descale is not None:
        v = (v.float() * v_descale[:, None, :, None]).to(v.dtype)
    if q.dtype == torch.float8_e4m3fn:
        q, k, v = q.to(out_dtype), k.to(out_dtype), v.to(out_dtype)
    k = _expand_kv(k, groups)
    v = _expand_kv(v, groups)
    if low:
        s = torch.einsum("bqhd,bkhd->bhqk", q, k * scale)
    else:
        s = torch.einsum("bqhd,bkhd->bhqk", q * scale, k)
    if softcap > 0:
        s = torch.tanh(s / softcap) * softcap
    vis = visibility(L // 2, block_size, device=q.device)
    s = s.masked_fill(~vis, float("-inf"))
    lse = torch.logsumexp(s.float(), dim=-1)
    p = torch.softmax(s, dim=-1).to(v.dtype)
    if p_dtype is not None:
        p = p.to(p_dtype).to(v.dtype)
    out = torch.einsum("bhqk,bkhd->bqhd", p, v)
    return out.to(out_dtype), lse


def backward(q, k, v, dout, block_size: int, softmax_scale: Optional[float] = None, softcap: float = 0.0,
             compute_dtype=torch.float32):
    """Explicit gradients (dq, dk, dv) of `forward` w.r.t. q, k, v for upstream gradient dout.

    float32: the truth. Low precision: every matrix product takes operands rounded to that dtype, the way a
    straightforward implementation without fused kernels would.
    """
    B, L, H, d = q.shape
    Hk = k.shape[2]
    groups = H // Hk
    scale = 1.0 / math.sqrt(d) if softmax_scale is None else softmax_scale
    cd = compute_dtype
    qf, kf, vf, gf = (t.to(cd) for t in (q, k, v, dout))
    kx = _expand_kv(kf, groups)
    vx = _expand_kv(vf, groups)
    if cd == torch.float32:
        raw = torch.einsum("bqhd,bkhd->bhqk", qf * scale, kx)
    else:
        raw = torch.einsum("bqhd,bkhd->bhqk", qf, kx * scale)
    if softcap > 0:
        t = torch.tanh(raw / softcap)
        s = t * softcap
    else:
        s = raw
    vis = visibility(L // 2, block_size, device=q.device)
    s = s.masked_fill(~vis, float("-inf"))
    p = torch.softmax(s, dim=-1).to(cd)                        # (B, H, q, k)
    o = torch.einsum("bhqk,bkhd->bqhd", p, vx)
    dvx = torch.einsum("bhqk,bqhd->bkhd", p, gf)
    dp = torch.einsum("bqhd,bkhd->bhqk", gf, vx)
    delta = (gf.float() * o.float()).sum(-1).permute(0, 2, 1)  # (B, H, q)
    ds = (p.float() * (dp.float() - delta[..., None]))
    if softcap > 0:
        ds = ds * (1.0 - t.float() * t.float())
    ds = ds.masked_fill(~vis, 0.0).to(cd)
    dq = torch.einsum("bhqk,bkhd->bqhd", ds, kx) * scale
    dkx = torch.einsum("bhqk,bqhd->bkhd", ds, qf) * scale
    if groups > 1:
        dkx = dkx.reshape(B, L, Hk, groups, d).float().sum(3)
        dvx = dvx.reshape(B, L, Hk, groups, d).float().sum(3)
    return dq.to(q.dtype), dkx.to(k.dtype), dvx.to(v.dtype)


def _split(cu_seqlens: Sequence[int]):
    cu = [int(x) for x in cu_seqlens]
    return [(cu[i], cu[i + 1]) for i in range(len(cu) - 1)]


def forward_varlen(q, k, v, cu_seqlens, block_size: int, **kw):
    """Packed samples: q (total, H, d); sample i occupies rows [cu[i], cu[i+1]). lse is (H, total)."""
    outs, lses = [], []
    for b, (s, e) in enumerate(_split(cu_seqlens)):
        kw_b = dict(kw)
        for name in ("q_descale", "k_descale", "v_descale"):
            if kw_b.get(name) is not None:
                kw_b[name] = kw_b[name][b:b + 1]
        if e == s:
            outs.append(q.new_zeros((0,) + tuple(q.shape[1:])).to(
                torch.bfloat16 if q.dtype == torch.float8_e4m3fn else q.dtype))
            lses.append(torch.zeros(q.shape[1], 0, dtype=torch.float32, device=q.device))
            continue
        o, l = forward(q[None, s:e], k[None, s:e], v[None, s:e], block_size, **kw_b)
        outs.append(o[0])
        lses.append(l[0])
    return torch.cat(outs, 0), torch.cat(lses, -1)


def backward_varlen(q, k, v, dout, cu_seqlens, block_size: int, **kw):
    dq, dk, dv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
    for s, e in _split(cu_seqlens):
        if e == s:
            continue
        a, b, c = backward(q[None, s:e], k[None, s:e], v[None, s:e], dout[None, s:e], block_size, **kw)
        dq[s:e], dk[s:e], dv[s:e] = a[0], b[0], c[0]
    return dq, dk, dv


def step_flops(ns: Sequence[int], block_size: int, heads: int, head_dim: int):
    """(forward, backward) FLOPs on visible pairs: 4*pairs*d*H forward, 2.5x that backward
    (benchmarks/benchmark_diffusion.py:175-180 of the reference)."""
    pairs = sum(count_visible_pairs(n, block_size) for n in ns)
    fwd = 4.0 * pairs * head_dim * heads
    return fwd, 2.5 * fwd
