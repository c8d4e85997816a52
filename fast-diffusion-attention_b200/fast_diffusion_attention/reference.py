"""Plain PyTorch statement of block-diffusion attention, the module users of the reference project import as
`fast_diffusion_attention.reference` (diffusion_mask, num_visible_pairs, attention_ref, attention_varlen_ref;
reference.py:20-120 there). It materialises the (2n, 2n) mask and is meant for tests and small problems only.
Differentiable through autograd. Runs on any device; the library itself never calls it.
"""

import math
from typing import Optional

import torch


def _half_blocks(n: int, block_size: int, device=None):
    """Half index (0 noisy, 1 clean) and block index of each of the 2n positions of a sample."""
    pos = torch.arange(2 * n, device=device)
    half = (pos >= n).long()
    return half, (pos - half * n) // block_size


def diffusion_mask(n: int, block_size: int, device=None) -> torch.Tensor:
    """(2n, 2n) bool, True where the query (row) attends to the key (column)."""
    half, blk = _half_blocks(n, block_size, device)
    qh, kh = half[:, None], half[None, :]
    qb, kb = blk[:, None], blk[None, :]
    same_half = qh == kh
    own_block = same_half & (qb == kb)                  # noisy->noisy and the clean diagonal
    clean_prefix = (kh == 1) & (kb < qb)                # earlier clean blocks, seen from both halves
    return own_block | clean_prefix


def num_visible_pairs(n: int, block_size: int) -> int:
    """Exact number of visible (query, key) pairs of one sample, without building the mask."""
    total = 0
    start = 0
    while start < n:
        size = min(block_size, n - start)
        total += size * (2 * size + 2 * start)   # noisy block: size + start keys, clean block: start + size keys
        start += size
    return total


def attention_ref(q, k, v, block_size: int, softmax_scale: Optional[float] = None, softcap: float = 0.0,
                  q_descale=None, k_descale=None, v_descale=None, upcast: bool = True, reorder_ops: bool = False,
                  intermediate_dtype: Optional[torch.dtype] = None):
    """q (batch, 2n, nheads, d), k / v (batch, 2n, nheads_k, d) -> (out like q (bf16 for fp8), lse (batch, nheads, 2n)).

    upcast=True evaluates in float32; upcast=False keeps the input precision (reorder_ops=True then scales k
    instead of q), which measures the error of an unfused same-precision implementation."""
    fp8 = q.dtype not in (torch.float16, torch.bfloat16, torch.float32, torch.float64)
    out_dtype = torch.bfloat16 if fp8 else q.dtype
    _, length, heads, d = q.shape
    assert length % 2 == 0, "the sequence length must be even"
    rep = heads // k.shape[2]
    if upcast:
        q, k, v = q.float(), k.float(), v.float()

    def descaled(x, s, expand):
        if s is None:
            return x
        s = s.repeat_interleave(rep, dim=1) if expand else s
        return (x.float() * s[:, None, :, None]).to(x.dtype)

    q, k, v = descaled(q, q_descale, True), descaled(k, k_descale, False), descaled(v, v_descale, False)
    if q.dtype not in (torch.float16, torch.bfloat16, torch.float32, torch.float64):
        q, k, v = q.to(out_dtype), k.to(out_dtype), v.to(out_dtype)
    if rep > 1:
        k, v = k.repeat_interleave(rep, dim=2), v.repeat_interleave(rep, dim=2)
    scale = 1.0 / math.sqrt(d) if softmax_scale is None else softmax_scale
    if reorder_ops:
        scores = torch.einsum("bqhd,bkhd->bhqk", q, k * scale)
    else:
        scores = torch.einsum("bqhd,bkhd->bhqk", q * scale, k)
    if softcap > 0:
        scores = softcap * torch.tanh(scores / softcap)
    visible = diffusion_mask(length // 2, block_size, device=q.device)
    scores = scores.masked_fill(~visible, float("-inf"))
    lse = torch.logsumexp(scores.float(), dim=-1)
    probs = torch.softmax(scores, dim=-1).to(v.dtype)
    if intermediate_dtype is not None:
        probs = probs.to(intermediate_dtype).to(probs.dtype)
    out = torch.einsum("bhqk,bkhd->bqhd", probs, v)
    return out.to(out_dtype), lse


def attention_varlen_ref(q, k, v, cu_seqlens, block_size: int, **kwargs):
    """Packed samples: q (total, nheads, d); sample i is rows [cu_seqlens[i], cu_seqlens[i+1]). lse: (nheads, total)."""
    bounds = [int(x) for x in cu_seqlens.tolist()]
    outs, lses = [], []
    for lo, hi in zip(bounds[:-1], bounds[1:]):
        if hi == lo:
            continue
        o, l = attention_ref(q[None, lo:hi], k[None, lo:hi], v[None, lo:hi], block_size, **kwargs)
        outs.append(o[0])
        lses.append(l[0])
    return torch.cat(outs, dim=0), torch.cat(lses, dim=-1)
