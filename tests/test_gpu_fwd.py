"""Forward parity on the GPU, through the public API (which calls the C ABI), against the oracle.

Tolerance (written here as the reference's tests state it, tests/test_diffusion_attn.py:76-104 there):
max|out - truth| <= 2 * max|plain - truth| + a few ulps, truth = float32 oracle on the same low-precision
inputs, plain = the oracle evaluated in the input precision. LSE: <= 2 * err_plain + 1e-4. A second arm uses
torch SDPA with the explicit mask in the same precision as "plain".
"""

import pytest
import torch
import torch.nn.functional as F

from _util import assert_within_2x
from fast_diffusion_attention import _lib, diffusion_attn_func, diffusion_attn_varlen_func
from oracle import diffusion_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"

SHAPES = [(2, 128, 4), (1, 256, 32), (3, 100, 3), (2, 333, 16), (1, 517, 7), (1, 64, 64), (1, 300, 128),
          (2, 191, 200), (1, 1, 1), (2, 5, 2), (1, 1024, 1), (1, 777, 64), (1, 512, 256), (1, 640, 128)]


def check_forward(q, k, v, bs, softcap=0.0, scale=None, cu=None):
    if cu is None:
        out, lse = diffusion_attn_func(q, k, v, bs, softmax_scale=scale, softcap=softcap, return_attn_probs=True)
        truth, lse_t = orc.forward(q, k, v, bs, softmax_scale=scale, softcap=softcap)
        plain, lse_p = orc.forward(q, k, v, bs, softmax_scale=scale, softcap=softcap, compute_dtype=q.dtype)
    else:
        ms = int((cu[1:] - cu[:-1]).max().item())
        out, lse = diffusion_attn_varlen_func(q, k, v, cu, cu, ms, ms, bs, softmax_scale=scale, softcap=softcap,
                                              return_attn_probs=True)
        truth, lse_t = orc.forward_varlen(q, k, v, cu.tolist(), bs, softmax_scale=scale, softcap=softcap)
        plain, lse_p = orc.forward_varlen(q, k, v, cu.tolist(), bs, softmax_scale=scale, softcap=softcap,
                                          compute_dtype=q.dtype)
    assert _lib.device_status()[0] == 0
    assert out.dtype == q.dtype and out.shape == q.shape
    assert not torch.isnan(out.float()).any()
    assert_within_2x("out", out, truth, plain)
    err = (lse - lse_t).abs().max().item()
    err_p = (lse_p - lse_t).abs().max().item()
    assert err <= 2 * err_p + 1e-4, f"lse: {err} > 2 * {err_p} + 1e-4"
    return out, lse


@pytest.mark.parametrize("d", [128, 64])
@pytest.mark.parametrize("heads,heads_k", [(4, 4), (6, 2), (4, 1)])
@pytest.mark.parametrize("batch,n,bs", SHAPES)
def test_forward_bf16(batch, n, bs, heads, heads_k, d):
    torch.manual_seed(n * 1000 + bs)
    q = torch.randn(batch, 2 * n, heads, d, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(batch, 2 * n, heads_k, d, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(batch, 2 * n, heads_k, d, device=DEV, dtype=torch.bfloat16)
    check_forward(q, k, v, bs)


@pytest.mark.parametrize("d", [128, 64])
@pytest.mark.parametrize("batch,n,bs", [(2, 333, 16), (1, 300, 128), (1, 777, 64)])
def test_forward_fp16_softcap(batch, n, bs, d):
    torch.manual_seed(n + bs)
    q, k, v = (torch.randn(batch, 2 * n, h, d, device=DEV, dtype=torch.float16) for h in (4, 2, 2))
    check_forward(q, k, v, bs, softcap=15.0)
    check_forward(q, k, v, bs)


def test_forward_sdpa_rule():
    """max-abs error within 2x the error of torch SDPA run with the same explicit mask in bf16."""
    torch.manual_seed(5)
    B, n, H, d, bs = 2, 384, 4, 128, 48
    q, k, v = (torch.randn(B, 2 * n, H, d, device=DEV, dtype=torch.bfloat16) for _ in range(3))
    out = diffusion_attn_func(q, k, v, bs)
    truth, _ = orc.forward(q, k, v, bs)
    mask = orc.visibility(n, bs, device=DEV)
    sdpa = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                          attn_mask=mask).transpose(1, 2)
    assert_within_2x("out vs sdpa", out, truth, sdpa)


def test_forward_custom_scale_and_strided_views():
    torch.manual_seed(0)
    qkv = torch.randn(1, 400, 3, 2, 128, device=DEV, dtype=torch.bfloat16)
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    for scale in (0.05, 0.3):
        check_forward(q, k, v, 8, scale=scale)


@pytest.mark.parametrize("d", [128, 64])
@pytest.mark.parametrize("bs", [1, 4, 13, 64, 160])
def test_forward_varlen(bs, d):
    torch.manual_seed(bs)
    ns = [17, 300, 1, 128, 513, 64, 2, 255]
    cu = torch.tensor([0] + list(torch.tensor([2 * x for x in ns]).cumsum(0)), device=DEV, dtype=torch.int32)
    total = 2 * sum(ns)
    q = torch.randn(total, 6, d, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(total, 2, d, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(total, 2, d, device=DEV, dtype=torch.bfloat16)
    check_forward(q, k, v, bs, cu=cu)


def test_forward_varlen_zero_length_samples():
    """Samples of length zero between real ones (sentinels around the outputs: tests/test_gpu_parity_extra.py)."""
    torch.manual_seed(3)
    ns = [0, 100, 0, 32]
    cu = torch.tensor([0] + list(torch.tensor([2 * x for x in ns]).cumsum(0)), device=DEV, dtype=torch.int32)
    total = 2 * sum(ns)
    q, k, v = (torch.randn(total, 2, 64, device=DEV, dtype=torch.bfloat16) for _ in range(3))
    check_forward(q, k, v, 8, cu=cu)


def test_forward_matches_golden_fixture():
    """bf16 golden case produced by the reference's reference.py (tests/golden)."""
    from _util import load_golden, make_inputs
    from golden.make_golden import DENSE_CASES
    name = "bf16_gqa"
    B, n, H, Hk, d, bs, cap, scale, dt = DENSE_CASES[name]
    gold = load_golden("attention_golden.npz")
    q, k, v, _ = make_inputs(int(gold[f"{name}/seed"]), (B, 2 * n, H, d), (B, 2 * n, Hk, d), torch.bfloat16, DEV)
    out, lse = diffusion_attn_func(q, k, v, bs, return_attn_probs=True)
    truth = torch.from_numpy(gold[f"{name}/out"]).to(DEV)
    plain = torch.from_numpy(gold[f"{name}/out_pt"]).to(DEV)
    assert_within_2x("out", out, truth, plain)
    assert (lse.cpu() - torch.from_numpy(gold[f"{name}/lse"])).abs().max().item() < 2e-2


@pytest.mark.parametrize("heads,heads_k", [(4, 4), (4, 2)])
@pytest.mark.parametrize("batch,n,bs", [(1, 256, 32), (2, 333, 16), (1, 517, 7), (1, 300, 128), (1, 640, 256), (2, 5, 2)])
def test_forward_head_dim_256(batch, n, bs, heads, heads_k):
    torch.manual_seed(n * 7 + bs)
    q = torch.randn(batch, 2 * n, heads, 256, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(batch, 2 * n, heads_k, 256, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(batch, 2 * n, heads_k, 256, device=DEV, dtype=torch.bfloat16)
    check_forward(q, k, v, bs)


@pytest.mark.parametrize("d", [80, 96, 112, 160, 192, 224])
@pytest.mark.parametrize("bs", [1, 4, 37])
def test_forward_padded_head_dims(bs, d):
    torch.manual_seed(d)
    batch, n, heads, heads_k = 2, 211, 4, 2
    q = torch.randn(batch, 2 * n, heads, d, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(batch, 2 * n, heads_k, d, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(batch, 2 * n, heads_k, d, device=DEV, dtype=torch.bfloat16)
    check_forward(q, k, v, bs)


def _fwd_through_abi(q, k, v, out, lse, bs):
    """fda_fwd called the way a foreign host would: raw pointers and element strides of caller-owned tensors."""
    import ctypes as C
    from fast_diffusion_attention import _lib
    from fast_diffusion_attention.interface import _problem, _tensor_view
    lib = _lib.load()
    B, L = q.shape[0], q.shape[1]
    args = _lib.FdaFwdArgs()
    args.p = _problem(q, k, B, L, B * L, bs, q.shape[-1] ** -0.5, 0.0, 0, False, None)
    args.q, args.k, args.v, args.out = (_tensor_view(t, False) for t in (q, k, v, out))
    args.lse = lse.data_ptr()
    nbytes = lib.fda_fwd_workspace_bytes(C.byref(args.p))
    ws = torch.zeros(max(nbytes, 256), dtype=torch.uint8, device=q.device)
    args.workspace, args.workspace_bytes = ws.data_ptr(), ws.numel()
    rc = lib.fda_fwd(C.byref(args), C.c_void_p(torch.cuda.current_stream(q.device).cuda_stream))
    torch.cuda.synchronize()
    return rc


def test_forward_into_a_strided_output_and_refusal_of_misaligned_ones():
    """out may be a view into a larger buffer as long as base and strides are multiples of 16 bytes; the rest of
    the buffer is left alone. Strides that are not are refused before anything is launched."""
    from fast_diffusion_attention import _lib
    torch.manual_seed(5)
    B, n, H, d, bs = 2, 200, 3, 64, 24
    q, k, v = (torch.randn(B, 2 * n, H, d, device=DEV, dtype=torch.bfloat16) for _ in range(3))
    want = diffusion_attn_func(q, k, v, bs)
    lse = torch.empty(B, H, 2 * n, device=DEV, dtype=torch.float32)
    big = torch.full((B, 2 * n, H, d + 8), float("nan"), device=DEV, dtype=torch.bfloat16)
    assert _fwd_through_abi(q, k, v, big[..., :d], lse, bs) == 0
    assert _lib.device_status()[0] == 0
    assert torch.equal(big[..., :d], want)
    assert torch.isnan(big[..., d:].float()).all()
    odd = torch.empty((B, 2 * n, H, d + 4), device=DEV, dtype=torch.bfloat16)
    assert _fwd_through_abi(q, k, v, odd[..., :d], lse, bs) == 7   # FDA_ERR_STRIDE
