"""The oracle (oracle/diffusion_oracle.py) and the package's own reference module against the golden vectors
that were produced by the reference project's reference.py (tests/golden/make_golden.py)."""

import numpy as np
import pytest
import torch

from _util import load_golden, make_inputs
from golden.make_golden import DENSE_CASES, MASK_CASES, ROW_STRIDE, VARLEN_CASES
from oracle import diffusion_oracle as orc


def brute_force_visible(n, bs, qi, kj):
    """The four visibility rules, one (query, key) pair at a time, independent of any vectorised code."""
    q_clean, k_clean = qi >= n, kj >= n
    qb = (qi - n if q_clean else qi) // bs
    kb = (kj - n if k_clean else kj) // bs
    if not q_clean and not k_clean:
        return qb == kb
    if not q_clean and k_clean:
        return kb < qb
    if q_clean and k_clean:
        return kb <= qb
    return False


@pytest.mark.parametrize("n,bs", MASK_CASES)
def test_mask_matches_reference_golden(n, bs):
    gold = load_golden("mask_golden.npz")
    want = np.unpackbits(gold[f"mask/{n}/{bs}"])[: 4 * n * n].reshape(2 * n, 2 * n).astype(bool)
    got = orc.visibility(n, bs).numpy()
    assert np.array_equal(got, want)
    assert orc.count_visible_pairs(n, bs) == int(gold[f"pairs/{n}/{bs}"]) == int(want.sum())


@pytest.mark.parametrize("n,bs", [(1, 1), (5, 2), (16, 3), (33, 7), (20, 200)])
def test_mask_matches_brute_force(n, bs):
    got = orc.visibility(n, bs)
    for qi in range(2 * n):
        for kj in range(2 * n):
            assert bool(got[qi, kj]) == brute_force_visible(n, bs, qi, kj)


@pytest.mark.parametrize("name", list(DENSE_CASES))
def test_dense_oracle_matches_golden(name):
    B, n, H, Hk, d, bs, cap, scale, dt = DENSE_CASES[name]
    gold = load_golden("attention_golden.npz")
    dtype = getattr(torch, dt)
    q, k, v, do = make_inputs(int(gold[f"{name}/seed"]), (B, 2 * n, H, d), (B, 2 * n, Hk, d), dtype)
    out, lse = orc.forward(q, k, v, bs, softmax_scale=scale, softcap=cap)
    dq, dk, dv = orc.backward(q, k, v, do, bs, softmax_scale=scale, softcap=cap)
    sub = (lambda t: t[:, ::ROW_STRIDE]) if name == "c1_cpu_config" else (lambda t: t)
    tol = dict(atol=2e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    for key, val in (("out", sub(out)), ("dq", sub(dq)), ("dk", sub(dk)), ("dv", sub(dv))):
        want = torch.from_numpy(gold[f"{name}/{key}"])
        assert torch.allclose(val.float(), want, **tol), (name, key, (val.float() - want).abs().max())
    assert torch.allclose(lse, torch.from_numpy(gold[f"{name}/lse"]), atol=2e-5, rtol=1e-5)
    # the "plain same-precision" arm of the tolerance rule
    out_pt, lse_pt = orc.forward(q, k, v, bs, softmax_scale=scale, softcap=cap, compute_dtype=dtype)
    want = torch.from_numpy(gold[f"{name}/out_pt"])
    assert torch.allclose(sub(out_pt).float(), want, **tol)
    # ... and of the gradients: the oracle's same-precision backward sets the tolerance of dq, dk, dv in the GPU tests,
    # so its error must be the error of the reference's own plain arm (autograd through
    # attention_ref(upcast=False, reorder_ops=True)), not a looser one
    plain = orc.backward(q, k, v, do, bs, softmax_scale=scale, softcap=cap, compute_dtype=dtype)
    for key, val in zip(("dq", "dk", "dv"), plain):
        truth = torch.from_numpy(gold[f"{name}/{key}"])
        e_oracle = sub(val).float() - truth
        e_ref = torch.from_numpy(gold[f"{name}/{key}_pt"]) - truth
        # the root-mean-square errors agree to a percent; the maxima are single elements, a whole number of
        # 16-bit rounding steps each, so they may differ by one step
        rms_oracle, rms_ref = e_oracle.pow(2).mean().sqrt().item(), e_ref.pow(2).mean().sqrt().item()
        assert rms_oracle <= 1.1 * rms_ref + 1e-6, (name, key, rms_oracle, rms_ref)
        assert e_oracle.abs().max().item() <= 1.5 * e_ref.abs().max().item() + 1e-5, (name, key)


@pytest.mark.parametrize("name", list(VARLEN_CASES))
def test_varlen_oracle_matches_golden(name):
    ns, H, Hk, d, bs, cap, dt = VARLEN_CASES[name]
    gold = load_golden("attention_golden.npz")
    total = 2 * sum(ns)
    cu = np.concatenate([[0], np.cumsum([2 * x for x in ns])]).tolist()
    q, k, v, do = make_inputs(int(gold[f"{name}/seed"]), (total, H, d), (total, Hk, d), getattr(torch, dt))
    out, lse = orc.forward_varlen(q, k, v, cu, bs, softcap=cap)
    dq, dk, dv = orc.backward_varlen(q, k, v, do, cu, bs, softcap=cap)
    for key, val in (("out", out), ("dq", dq), ("dk", dk), ("dv", dv), ("lse", lse)):
        want = torch.from_numpy(gold[f"{name}/{key}"])
        assert torch.allclose(val.float(), want, atol=2e-5, rtol=1e-4), (name, key)


def test_package_reference_module_matches_golden():
    """fast_diffusion_attention.reference (the API the reference project exposes for its users' tests)."""
    from fast_diffusion_attention import reference as pref
    gold = load_golden("mask_golden.npz")
    for n, bs in MASK_CASES:
        want = np.unpackbits(gold[f"mask/{n}/{bs}"])[: 4 * n * n].reshape(2 * n, 2 * n).astype(bool)
        assert np.array_equal(pref.diffusion_mask(n, bs).numpy(), want)
        assert pref.num_visible_pairs(n, bs) == int(want.sum())
    att = load_golden("attention_golden.npz")
    name = "odd_n_small_bs"
    B, n, H, Hk, d, bs, cap, scale, dt = DENSE_CASES[name]
    q, k, v, do = make_inputs(int(att[f"{name}/seed"]), (B, 2 * n, H, d), (B, 2 * n, Hk, d), torch.float32)
    q, k, v = (t.requires_grad_() for t in (q, k, v))
    out, lse = pref.attention_ref(q, k, v, bs, softmax_scale=scale, softcap=cap)
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), do)
    for key, val in (("out", out), ("dq", dq), ("dk", dk), ("dv", dv), ("lse", lse)):
        assert torch.allclose(val.float(), torch.from_numpy(att[f"{name}/{key}"]), atol=2e-5, rtol=1e-4)


def test_step_flops_c2():
    fwd, bwd = orc.step_flops([2048] * 8, 256, 16, 128)
    assert abs((fwd + bwd) / 1e9 - 1082.3) < 0.1
