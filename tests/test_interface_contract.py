"""The Python interface's argument checks (same key words as the reference's check_inputs,
csrc/fda/flash_api.cpp:92-139 there, and the asserts of its interface.py:169-294) and its traceability: the
operators have shape-only implementations, so the functions trace under fake tensors and torch.compile the way
the reference's do (tests/test_diffusion_attn.py there compiles the function once)."""

import pytest
import torch

from fast_diffusion_attention import diffusion_attn_func, diffusion_attn_varlen_func

DEV = torch.device("cuda", 0) if torch.cuda.is_available() else None


# ------------------------------------------------------------------------------------------- without a GPU
def test_host_tensors_have_no_implementation():
    """Like the reference's operators, ours exist for CUDA tensors only: the dispatcher refuses anything else, and
    nothing falls back to a host computation."""
    q = torch.randn(1, 8, 2, 16).bfloat16()
    with pytest.raises((NotImplementedError, RuntimeError), match="CPU"):
        diffusion_attn_func(q, q, q, 4)


def test_varlen_wants_equal_query_and_key_lengths():
    q = torch.randn(8, 2, 16).bfloat16()
    cu = torch.tensor([0, 8], dtype=torch.int32)
    with pytest.raises((AssertionError, RuntimeError), match="cu_seqlens_k must be equal to cu_seqlens_q"):
        diffusion_attn_varlen_func(q, q, q, cu, torch.tensor([0, 4, 8], dtype=torch.int32), 8, 8, 4)
    with pytest.raises((AssertionError, RuntimeError), match="max_seqlen_k must be equal to max_seqlen_q"):
        diffusion_attn_varlen_func(q, q, q, cu, cu, 8, 6, 4)


def test_traces_under_fake_tensors():
    """No kernel runs and no device is needed: only the operators' shape functions."""
    from torch._subclasses.fake_tensor import FakeTensorMode

    with FakeTensorMode():
        q = torch.empty(2, 64, 8, 128, dtype=torch.bfloat16, device="cuda")
        k = torch.empty(2, 64, 2, 128, dtype=torch.bfloat16, device="cuda")
        out, lse = diffusion_attn_func(q, k, k, 16, return_attn_probs=True)
        assert out.shape == q.shape and out.dtype == torch.bfloat16 and out.device.type == "cuda"
        assert lse.shape == (2, 8, 64) and lse.dtype == torch.float32

        total = 96
        cu = torch.empty(4, dtype=torch.int32, device="cuda")
        qv = torch.empty(total, 4, 64, dtype=torch.float16, device="cuda")
        out, lse = diffusion_attn_varlen_func(qv, qv, qv, cu, cu, 40, 40, 8, return_attn_probs=True)
        assert out.shape == qv.shape and lse.shape == (4, total)

        q8 = torch.empty(1, 32, 2, 128, dtype=torch.float8_e4m3fn, device="cuda")
        out = diffusion_attn_func(q8, q8, q8, 16)
        assert out.dtype == torch.bfloat16 and out.shape == q8.shape


def test_shape_functions_cover_the_backward():
    """Forward and backward on meta tensors: the autograd node and both operators' shape functions."""
    q = torch.empty(2, 64, 8, 128, dtype=torch.bfloat16, device="meta", requires_grad=True)
    k = torch.empty(2, 64, 2, 128, dtype=torch.bfloat16, device="meta", requires_grad=True)
    v = torch.empty(2, 64, 2, 128, dtype=torch.bfloat16, device="meta", requires_grad=True)
    out = diffusion_attn_func(q, k, v, 16, softcap=10.0)
    out.sum().backward()
    assert q.grad.shape == q.shape and k.grad.shape == k.shape and v.grad.shape == v.shape
    assert q.grad.dtype == torch.bfloat16


# ---------------------------------------------------------------------------------------------- with a GPU
def _t(*shape, dtype=torch.bfloat16):
    return torch.randn(*shape, device=DEV, dtype=torch.float32).to(dtype)


@pytest.mark.gpu
def test_shape_and_argument_errors():
    q = _t(1, 8, 4, 16)
    cases = [
        (lambda: diffusion_attn_func(_t(1, 7, 4, 16), _t(1, 7, 4, 16), _t(1, 7, 4, 16), 4), "must be even"),
        (lambda: diffusion_attn_func(q, _t(1, 8, 4, 8), _t(1, 8, 4, 8), 4), "k and v must have shape"),
        (lambda: diffusion_attn_func(q, _t(1, 8, 3, 16), _t(1, 8, 3, 16), 4), "must divide number of heads"),
        (lambda: diffusion_attn_func(_t(1, 8, 4, 12), _t(1, 8, 4, 12), _t(1, 8, 4, 12), 4), "multiple of 8"),
        (lambda: diffusion_attn_func(_t(1, 8, 1, 264), _t(1, 8, 1, 264), _t(1, 8, 1, 264), 4), "at most 256"),
        (lambda: diffusion_attn_func(q, q, q, 0), "block_size must be a positive integer"),
        (lambda: diffusion_attn_func(q, q, q, -3), "block_size must be a positive integer"),
        (lambda: diffusion_attn_func(q[0], q[0], q[0], 4), "q must have shape"),
    ]
    f32 = torch.randn(1, 8, 2, 16, device=DEV)
    cases += [
        (lambda: diffusion_attn_func(f32, f32, f32, 4), "only supports fp16, bf16, and fp8_e4m3"),
        (lambda: diffusion_attn_func(q, q.half(), q, 4), "same dtype"),
    ]
    for fn, msg in cases:
        with pytest.raises(RuntimeError, match=msg):
            fn()
    qv = _t(8, 4, 16)
    cu64 = torch.tensor([0, 8], device=DEV)
    cu = cu64.int()
    with pytest.raises(RuntimeError, match="torch.int32"):
        diffusion_attn_varlen_func(qv, qv, qv, cu64, cu64, 8, 8, 4)
    with pytest.raises(RuntimeError, match="contiguous CUDA tensor"):
        diffusion_attn_varlen_func(qv, qv, qv, cu.cpu(), cu.cpu(), 8, 8, 4)
    with pytest.raises(RuntimeError, match=r"\(total, num_heads, head_size\)"):
        diffusion_attn_varlen_func(q, q, q, cu, cu, 8, 8, 4)
    with pytest.raises(RuntimeError, match=r"\(total, num_heads_k, head_size\)"):
        diffusion_attn_varlen_func(qv, _t(6, 4, 16), _t(6, 4, 16), cu, cu, 8, 8, 4)


@pytest.mark.gpu
def test_fp8_has_no_backward():
    q = _t(1, 32, 2, 128).to(torch.float8_e4m3fn)
    out = diffusion_attn_func(q, q, q, 8)
    assert out.dtype == torch.bfloat16 and not out.requires_grad


@pytest.mark.gpu
def test_compiles_as_one_graph_and_matches_eager():
    """torch.compile must see the operators as opaque calls with known output shapes (no graph break)."""
    torch.manual_seed(0)
    q, k, v = _t(2, 256, 4, 64), _t(2, 256, 2, 64), _t(2, 256, 2, 64)

    def step(q, k, v):
        out = diffusion_attn_func(q, k, v, 32, softcap=20.0)
        return out.float().square().sum()

    def run(fn):
        qq, kk, vv = (t.clone().requires_grad_(True) for t in (q, k, v))
        fn(qq, kk, vv).backward()
        return qq.grad, kk.grad, vv.grad

    want = run(step)
    got = run(torch.compile(step, fullgraph=True, backend="aot_eager"))
    from _util import assert_same_gradients
    for name, a, b in zip(("dq", "dk", "dv"), got, want):
        assert_same_gradients(name, a, b, exact=name != "dq")   # dq: global fp32 adds in scheduling order
