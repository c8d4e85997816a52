"""fda_bwd_noalloc: the backward for hosts that cannot give the library a workspace.

Who needs it: a process that fixed its device-memory plan at start-up and may not call an allocator on its hot
path, or a binding in another language that reaches the GPU only through this C ABI and has no tensor allocator
to ask. The ordinary fda_bwd wants fda_bwd_workspace_bytes() of caller scratch; this variant keeps that scratch in
a fixed array inside the library image and takes only the inputs and outputs.

The test drives both entry points through ctypes on the same inputs, twice in a row with different data (the
built-in array keeps the previous call's contents, which must not leak into the next result). The variant runs
the split form of the backward, so it must equal fda_bwd with deterministic=1 bit for bit, and fda_bwd's default
single-pass form up to one rounding step in dq. The file name sorts last on purpose: if the new entry point breaks, every other test has
already run.
"""

import ctypes as C

import pytest
import torch

from _util import assert_same_gradients
from fast_diffusion_attention import _lib, diffusion_attn_func
from fast_diffusion_attention.interface import _problem, _tensor_view


def _bwd_args(q, k, v, out, lse, dout, grads, block_size, scale, deterministic=False):
    B, L = q.shape[0], q.shape[1]
    args = _lib.FdaBwdArgs()
    args.p = _problem(q, k, B, L, B * L, block_size, scale, 0.0, 0, deterministic, None)
    (args.q, args.k, args.v, args.out, args.dout, args.dq, args.dk, args.dv) = (
        _tensor_view(t, False) for t in (q, k, v, out, dout, *grads))
    args.lse = lse.data_ptr()
    return args


@pytest.mark.gpu
def test_noalloc_backward_matches_workspace_backward_twice():
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    for call, (B, n, H, Hk, d, bs) in enumerate([(2, 300, 4, 2, 128, 48), (1, 517, 6, 2, 64, 7)]):
        torch.manual_seed(100 + call)
        q = torch.randn(B, 2 * n, H, d, device=dev, dtype=torch.bfloat16)
        k = torch.randn(B, 2 * n, Hk, d, device=dev, dtype=torch.bfloat16)
        v = torch.randn(B, 2 * n, Hk, d, device=dev, dtype=torch.bfloat16)
        dout = torch.randn_like(q)
        scale = d ** -0.5
        out, lse = diffusion_attn_func(q, k, v, bs, return_attn_probs=True)

        wants = []
        for deterministic in (True, False):
            want = [torch.empty_like(t) for t in (q, k, v)]
            args = _bwd_args(q, k, v, out, lse, dout, want, bs, scale, deterministic)
            nbytes = lib.fda_bwd_workspace_bytes(C.byref(args.p))
            ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
            args.workspace, args.workspace_bytes = ws.data_ptr(), nbytes
            _lib.check(lib.fda_bwd(C.byref(args), stream))
            wants.append((want, nbytes))

        got = [torch.full_like(t, float("nan")) for t in (q, k, v)]
        args2 = _bwd_args(q, k, v, out, lse, dout, got, bs, scale)  # workspace fields stay NULL / 0 on purpose
        assert wants[0][1] <= _lib.NOALLOC_SCRATCH_BYTES   # its scratch need is the deterministic backward's
        _lib.check(lib.fda_bwd_noalloc(C.byref(args2), stream))
        torch.cuda.synchronize()
        assert _lib.device_status()[0] == 0
        for name, a, b, c in zip(("dq", "dk", "dv"), got, wants[0][0], wants[1][0]):
            assert not torch.isnan(a.float()).any(), name
            # same kernels and the same fixed accumulation order as the deterministic backward: bitwise equal
            assert torch.equal(a, b), f"{name} differs on call {call}"
            # the default backward adds its dq partials in scheduling order: equal up to one rounding step
            assert_same_gradients(f"{name} vs default backward, call {call}", a, c, exact=name != "dq")


def test_noalloc_rejects_problems_beyond_its_scratch():
    """Checked before anything touches the GPU, so this runs everywhere."""
    lib = _lib.load()
    args = _lib.FdaBwdArgs()
    # 16 samples x 32 heads x n=8192: 64 MiB of statistics, four times the built-in array
    args.p = _lib.FdaProblem(_lib.FDA_BF16, 16, 16384, 16 * 16384, 32, 32, 64, 256, 0.125, 0.0, 0, 1, None)
    dummy = C.c_void_p(256)  # never dereferenced: the size check comes first
    for name in ("q", "k", "v", "out", "dout", "dq", "dk", "dv"):
        setattr(args, name, _lib.FdaTensor(dummy, 1, 1, 1))
    args.lse = dummy
    assert lib.fda_bwd_workspace_bytes(C.byref(args.p)) > _lib.NOALLOC_SCRATCH_BYTES
    rc = lib.fda_bwd_noalloc(C.byref(args), None)
    assert rc == _lib.FDA_ERR_SCRATCH_LIMIT
    assert "scratch" in lib.fda_strerror(rc).decode()
