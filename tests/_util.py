"""Shared helpers of the tests: seeded inputs (same generator as tests/golden/make_golden.py), the golden
files, and the tolerance rule of the reference's test-suite (tests/test_diffusion_attn.py:76-104 there)."""

import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = os.path.join(HERE, "golden")


def make_inputs(seed, shape_q, shape_kv, dtype, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(shape_q, generator=g).to(dtype)
    k = torch.randn(shape_kv, generator=g).to(dtype)
    v = torch.randn(shape_kv, generator=g).to(dtype)
    do = torch.randn(shape_q, generator=g).to(dtype)
    return tuple(t.to(device) for t in (q, k, v, do))


def load_golden(name):
    return np.load(os.path.join(GOLDEN, name))


def ulp_atol(ref):
    """A few ulps of the reference values, as the reference's tests compute it."""
    r = ref.float()
    return 2 * (r + 0.3 - 0.3 - r).abs().max().item() + 1e-5


def assert_within_2x(name, got, truth, plain, rtol=2.0, atol=None):
    """max|got - truth| <= 2 * max|plain - truth| + few ulps; `plain` is a same-precision PyTorch result."""
    err = (got.float() - truth.float()).abs().max().item()
    err_plain = (plain.float() - truth.float()).abs().max().item()
    if atol is None:
        atol = ulp_atol(truth)
    assert err <= rtol * err_plain + atol, (
        f"{name}: max error {err:.3e} > {rtol} * {err_plain:.3e} (plain PyTorch) + {atol:.1e}")
    return err, err_plain


def assert_same_gradients(name, got, want, exact):
    """Bitwise equality, or (dq of the single-pass backward, whose fp32 partial sums are added in an order that
    depends on scheduling) equality up to one rounding step of the 16-bit result."""
    if exact:
        assert torch.equal(got, want), f"{name} differs"
        return
    a, b = got.float(), want.float()
    tol = torch.maximum(a.abs(), b.abs()) * 2.0 ** -6 + 1e-6
    bad = (a - b).abs() > tol
    assert not bad.any(), f"{name}: {int(bad.sum())} elements differ by more than one rounding step"
