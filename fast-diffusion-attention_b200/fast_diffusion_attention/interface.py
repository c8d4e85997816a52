"""Python interface of block-diffusion attention on B200.

Same public functions, argument order, defaults and return conventions as the reference project's
fast_diffusion_attention/interface.py (diffusion_attn_func :210-253, diffusion_attn_varlen_func :256-299,
the two autograd Functions :148-207 and the two custom operators :40-145). The operators call the C ABI of
libfda_sm100.so through ctypes with raw device pointers, element strides and the current CUDA stream; this
module allocates every output and workspace with torch.empty on q's device, the library allocates nothing.
"""

import ctypes as C
from typing import Optional, Tuple

import torch

from . import _lib

_lib.load()  # fail at import time when the library has not been built: there is no fallback path

_DTYPES = {torch.bfloat16: _lib.FDA_BF16, torch.float16: _lib.FDA_FP16}
if hasattr(torch, "float8_e4m3fn"):
    _DTYPES[torch.float8_e4m3fn] = _lib.FDA_E4M3


def _tile_copy_friendly(x):
    """The kernels move tiles with TMA and rows with 16-byte vector accesses: the base address and every stride
    but the last must be multiples of 16 bytes."""
    size = x.element_size()
    return x.data_ptr() % 16 == 0 and all((st * size) % 16 == 0 for st, n in zip(x.stride()[:-1], x.shape[:-1]) if n > 1)


def maybe_contiguous(x):
    """The reference copies an input only when its last dimension is strided (interface.py:17-18 there, its kernels
    take any other strides). Here a view whose base or strides are not 16-byte multiples (say x[..., 4:68]) is
    copied as well, so that every call the reference accepts is accepted."""
    if x is None:
        return x
    if x.stride(-1) != 1 or (x.dim() >= 3 and not _tile_copy_friendly(x)):
        return x.contiguous()
    return x


def _tensor_view(t: torch.Tensor, varlen: bool) -> _lib.FdaTensor:
    if varlen:
        return _lib.FdaTensor(t.data_ptr(), 0, t.stride(0), t.stride(1))
    return _lib.FdaTensor(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))


def _check_inputs(q, k, v, cu_seqlens, max_seqlen, block_size, backward=False):
    """The checks of the reference's check_inputs (csrc/fda/flash_api.cpp:92-139), same key words."""
    if not backward and q.dtype not in _DTYPES:
        raise RuntimeError("fast-diffusion-attention only supports fp16, bf16, and fp8_e4m3 data type")
    if backward and q.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("fast-diffusion-attention backward only supports fp16 and bf16 data type")
    if k.dtype != q.dtype or v.dtype != q.dtype:
        raise RuntimeError("query, key and value must have the same dtype")
    for t in (q, k, v):
        if not t.is_cuda:
            raise RuntimeError("Input tensor must be on CUDA device")
        if t.stride(-1) != 1:
            raise RuntimeError("Input tensor must have contiguous last dimension")
    if not isinstance(block_size, int) or block_size < 1:
        raise RuntimeError("block_size must be a positive integer")
    heads, head_dim, heads_k = q.shape[-2], q.shape[-1], k.shape[-2]
    if cu_seqlens is None:
        if q.dim() != 4:
            raise RuntimeError("q must have shape (batch_size, seqlen, num_heads, head_size)")
        batch, seqlen = q.shape[0], q.shape[1]
        total = batch * seqlen
        if seqlen % 2 != 0:
            raise RuntimeError("The sequence length must be even: [noisy half | clean half]")
        if tuple(k.shape) != (batch, seqlen, heads_k, head_dim) or tuple(v.shape) != tuple(k.shape):
            raise RuntimeError("k and v must have shape (batch_size, seqlen, num_heads_k, head_size)")
    else:
        if cu_seqlens.dtype != torch.int32:
            raise RuntimeError("cu_seqlens must have dtype torch.int32")
        if not cu_seqlens.is_cuda or not cu_seqlens.is_contiguous():
            raise RuntimeError("cu_seqlens must be a contiguous CUDA tensor")
        if cu_seqlens.dim() != 1 or cu_seqlens.numel() < 1:
            raise RuntimeError("cu_seqlens must be one-dimensional with batch_size + 1 entries")
        if max_seqlen is None:
            raise RuntimeError("max_seqlen must be provided if cu_seqlens is provided")
        if q.dim() != 3:
            raise RuntimeError("q must have shape (total, num_heads, head_size) if cu_seqlens is provided")
        batch, seqlen, total = cu_seqlens.shape[0] - 1, int(max_seqlen), q.shape[0]
        if tuple(k.shape) != (total, heads_k, head_dim) or tuple(v.shape) != tuple(k.shape):
            raise RuntimeError("k and v must have shape (total, num_heads_k, head_size)")
    if head_dim > 256:
        raise RuntimeError("fast-diffusion-attention supports head dimension at most 256")
    if heads % heads_k != 0:
        raise RuntimeError("Number of heads in key/value must divide number of heads in query")
    align = 16 if q.dtype not in (torch.float16, torch.bfloat16) else 8
    if head_dim % align != 0:
        raise RuntimeError(f"head_size should be a multiple of {align}")
    return batch, seqlen, total


def _problem(q, k, batch, seqlen, total, block_size, softmax_scale, softcap, sm_margin, deterministic, cu_seqlens):
    return _lib.FdaProblem(
        _DTYPES[q.dtype], batch, seqlen, total, q.shape[-2], k.shape[-2], q.shape[-1], block_size,
        float(softmax_scale), float(softcap), int(sm_margin), int(bool(deterministic)),
        cu_seqlens.data_ptr() if cu_seqlens is not None else None)


def _padded_half(seqlen: int) -> int:
    """Rows per half in the backward's statistics layout: the half length rounded up to the 128-row tile."""
    return (max(seqlen // 2, 1) + 127) // 128 * 128


def _stream_ptr(device):
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


@torch.library.custom_op("fda::_diffusion_attn_forward", mutates_args=(), device_types="cuda")
def _diffusion_attn_forward(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    block_size: int,
    cu_seqlens: Optional[torch.Tensor] = None,
    max_seqlen: Optional[int] = None,
    q_descale: Optional[torch.Tensor] = None,
    k_descale: Optional[torch.Tensor] = None,
    v_descale: Optional[torch.Tensor] = None,
    softmax_scale: Optional[float] = None,
    softcap: float = 0.0,
    sm_margin: int = 0,
) -> Tuple[torch.Tensor, torch.Tensor]:
    q, k, v = [maybe_contiguous(x) for x in (q, k, v)]
    cu_seqlens = maybe_contiguous(cu_seqlens)
    batch, seqlen, total = _check_inputs(q, k, v, cu_seqlens, max_seqlen, block_size)
    varlen = cu_seqlens is not None
    heads, head_dim = q.shape[-2], q.shape[-1]
    if softmax_scale is None:
        softmax_scale = head_dim ** (-0.5)
    is_fp8 = q.dtype not in (torch.float16, torch.bfloat16)
    if not is_fp8 and any(x is not None for x in (q_descale, k_descale, v_descale)):
        raise RuntimeError("q_descale, k_descale and v_descale are only supported for FP8 inputs")
    out = torch.empty(q.shape, dtype=torch.bfloat16 if is_fp8 else q.dtype, device=q.device)
    if varlen:
        lse = torch.empty((heads, total), dtype=torch.float32, device=q.device)
    else:
        lse = torch.empty((batch, heads, seqlen), dtype=torch.float32, device=q.device)
    if total == 0 or heads == 0:
        out.zero_()
        lse.fill_(float("inf"))
        return out, lse
    lib = _lib.load()
    args = _lib.FdaFwdArgs()
    args.p = _problem(q, k, batch, seqlen, total, block_size, softmax_scale, softcap, sm_margin, False, cu_seqlens)
    args.q, args.k, args.v, args.out = (_tensor_view(t, varlen) for t in (q, k, v, out))
    args.lse = lse.data_ptr()
    keep = []
    for i, (name, ds) in enumerate((("q_descale", q_descale), ("k_descale", k_descale), ("v_descale", v_descale))):
        if ds is not None:
            if tuple(ds.shape) != (batch, k.shape[-2]) or ds.dtype != torch.float32 or not ds.is_cuda:
                raise RuntimeError(f"{name} must be a float32 CUDA tensor of shape (batch_size, num_heads_k)")
            setattr(args, name, ds.data_ptr())
            args.descale_batch_stride[i] = ds.stride(0)
            args.descale_head_stride[i] = ds.stride(1)
            keep.append(ds)
    ws_bytes = lib.fda_fwd_workspace_bytes(C.byref(args.p))
    workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
    args.workspace = workspace.data_ptr()
    args.workspace_bytes = ws_bytes
    with torch.cuda.device(q.device):
        _lib.check(lib.fda_fwd(C.byref(args), _stream_ptr(q.device)))
    return out, lse


@torch.library.register_fake("fda::_diffusion_attn_forward")
def _diffusion_attn_forward_fake(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    block_size: int,
    cu_seqlens: Optional[torch.Tensor] = None,
    max_seqlen: Optional[int] = None,
    q_descale: Optional[torch.Tensor] = None,
    k_descale: Optional[torch.Tensor] = None,
    v_descale: Optional[torch.Tensor] = None,
    softmax_scale: Optional[float] = None,
    softcap: float = 0.0,
    sm_margin: int = 0,
) -> Tuple[torch.Tensor, torch.Tensor]:
    out_dtype = q.dtype if q.dtype in (torch.float16, torch.bfloat16) else torch.bfloat16
    out = torch.empty(q.shape, dtype=out_dtype, device=q.device)
    if cu_seqlens is not None:
        total, heads, _ = q.shape
        lse = torch.empty((heads, total), dtype=torch.float32, device=q.device)
    else:
        batch, seqlen, heads, _ = q.shape
        lse = torch.empty((batch, heads, seqlen), dtype=torch.float32, device=q.device)
    return out, lse


def backward_launch(dout, q, k, v, out, softmax_lse, dq, dk, dv, block_size, cu_seqlens=None, max_seqlen=None,
                    softmax_scale=None, softcap=0.0, deterministic=False, sm_margin=0, workspace=None, stages=7):
    """Validate, size the workspace and enqueue the backward stages selected by `stages` (bit 0 preprocess, bit 1 the
    single-pass kernel or the dK/dV kernel, bit 2 the dQ conversion or the dQ kernel, bit 3 forces the split form;
    7 = the whole backward) on the current stream. A caller that times or profiles single
    stages passes the same `workspace` to every call. Returns the (batch, heads, 2, n_pad) view of rowsum(dO*O)."""
    dout, q, k, v, out = [maybe_contiguous(x) for x in (dout, q, k, v, out)]
    batch, seqlen, total = _check_inputs(q, k, v, cu_seqlens, max_seqlen, block_size, backward=True)
    varlen = cu_seqlens is not None
    heads, head_dim = q.shape[-2], q.shape[-1]
    if out.dtype != q.dtype or dout.dtype != q.dtype:
        raise RuntimeError("query, out and dout must have the same dtype")
    if out.shape != q.shape or dout.shape != q.shape:
        raise RuntimeError("out and dout must have the same shape as q")
    for name, g, ref in (("dq", dq, q), ("dk", dk, k), ("dv", dv, v)):
        if g.dtype != q.dtype or g.shape != ref.shape or g.stride(-1) != 1:
            raise RuntimeError(f"{name} must have the dtype and shape of its input and a contiguous last dimension")
    # the same checks as mha_bwd makes on its arguments (csrc/fda/flash_api.cpp:491, :523-529 of the reference): the
    # kernels index these tensors without looking at them again
    for name, t in (("out", out), ("dout", dout), ("dq", dq), ("dk", dk), ("dv", dv), ("softmax_lse", softmax_lse)):
        if t.device != q.device:
            raise RuntimeError(f"{name} must be on the same device as q")
    if softmax_lse.dtype != torch.float32:
        raise RuntimeError("softmax_lse must have dtype float32")
    want_lse = (heads, total) if varlen else (batch, heads, seqlen)
    if tuple(softmax_lse.shape) != want_lse:
        raise RuntimeError(f"softmax_lse must have shape {want_lse}")
    if not softmax_lse.is_contiguous():
        raise RuntimeError("softmax_lse must be contiguous")
    for name, g in (("dq", dq), ("dk", dk), ("dv", dv)):
        if not _tile_copy_friendly(g):
            raise RuntimeError(f"{name} must have a 16-byte aligned base address and row/head/batch strides")
    if softmax_scale is None:
        softmax_scale = head_dim ** (-0.5)
    n_pad = _padded_half(seqlen)
    if total == 0 or heads == 0:
        dq.zero_(); dk.zero_(); dv.zero_()
        return torch.zeros((batch, heads, 2, n_pad), dtype=torch.float32, device=q.device)
    lib = _lib.load()
    args = _lib.FdaBwdArgs()
    args.p = _problem(q, k, batch, seqlen, total, block_size, softmax_scale, softcap, sm_margin, deterministic,
                      cu_seqlens)
    (args.q, args.k, args.v, args.out, args.dout, args.dq, args.dk, args.dv) = (
        _tensor_view(t, varlen) for t in (q, k, v, out, dout, dq, dk, dv))
    args.lse = softmax_lse.data_ptr()
    ws_bytes = lib.fda_bwd_workspace_bytes(C.byref(args.p))
    if workspace is None:
        workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
    elif workspace.numel() < ws_bytes or workspace.dtype != torch.uint8:
        raise RuntimeError("workspace must be a uint8 CUDA tensor of at least fda_bwd_workspace_bytes bytes")
    args.workspace = workspace.data_ptr()
    args.workspace_bytes = ws_bytes
    with torch.cuda.device(q.device):
        _lib.check(lib.fda_bwd_stages(C.byref(args), int(stages), _stream_ptr(q.device)))
    # the workspace starts with rowsum(dO * O) in the padded (batch, heads, half, n_pad) layout; it plays the
    # part of the reference's softmax_d return value (whose shape there depends on the sm90 tile sizes)
    return workspace[: batch * heads * 2 * n_pad * 4].view(torch.float32).view(batch, heads, 2, n_pad)




@torch.library.custom_op("fda::_diffusion_attn_backward", mutates_args=("dq", "dk", "dv"), device_types="cuda")
def _diffusion_attn_backward(
    dout: torch.Tensor,
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    out: torch.Tensor,
    softmax_lse: torch.Tensor,
    dq: torch.Tensor,
    dk: torch.Tensor,
    dv: torch.Tensor,
    block_size: int,
    cu_seqlens: Optional[torch.Tensor] = None,
    max_seqlen: Optional[int] = None,
    softmax_scale: Optional[float] = None,
    softcap: float = 0.0,
    deterministic: bool = False,
    sm_margin: int = 0,
) -> torch.Tensor:
    return backward_launch(dout, q, k, v, out, softmax_lse, dq, dk, dv, block_size, cu_seqlens, max_seqlen,
                           softmax_scale, softcap, deterministic, sm_margin)


@torch.library.register_fake("fda::_diffusion_attn_backward")
def _diffusion_attn_backward_fake(
    dout: torch.Tensor,
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    out: torch.Tensor,
    softmax_lse: torch.Tensor,
    dq: torch.Tensor,
    dk: torch.Tensor,
    dv: torch.Tensor,
    block_size: int,
    cu_seqlens: Optional[torch.Tensor] = None,
    max_seqlen: Optional[int] = None,
    softmax_scale: Optional[float] = None,
    softcap: float = 0.0,
    deterministic: bool = False,
    sm_margin: int = 0,
) -> torch.Tensor:
    if cu_seqlens is not None:
        batch, seqlen = cu_seqlens.shape[0] - 1, int(max_seqlen)
    else:
        batch, seqlen = q.shape[0], q.shape[1]
    return torch.empty((batch, q.shape[-2], 2, _padded_half(seqlen)), dtype=torch.float32, device=q.device)


class _DiffusionAttention(torch.autograd.Function):
    """One autograd node for both layouts: batched when cu_seqlens is None, packed otherwise. Saves
    q, k, v, out, lse (and cu_seqlens), the same set the reference saves (interface.py:158, :189 there)."""

    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens, max_seqlen, block_size, softmax_scale, descales, softcap,
                deterministic, sm_margin):
        scale = q.shape[-1] ** (-0.5) if softmax_scale is None else softmax_scale
        out, lse = _diffusion_attn_forward(q, k, v, block_size, cu_seqlens, max_seqlen, descales[0], descales[1],
                                           descales[2], scale, softcap, sm_margin)
        saved = (q, k, v, out, lse) + ((cu_seqlens,) if cu_seqlens is not None else ())
        ctx.save_for_backward(*saved)
        ctx.packed = cu_seqlens is not None
        ctx.opts = (block_size, max_seqlen, scale, softcap, deterministic, sm_margin)
        return out, lse

    @staticmethod
    def backward(ctx, dout, *unused):
        q, k, v, out, lse = ctx.saved_tensors[:5]
        cu_seqlens = ctx.saved_tensors[5] if ctx.packed else None
        block_size, max_seqlen, scale, softcap, deterministic, sm_margin = ctx.opts
        assert q.dtype in (torch.float16, torch.bfloat16), "The backward pass only supports fp16 and bf16"
        grads = tuple(torch.empty_like(t) for t in (q, k, v))
        _diffusion_attn_backward(dout, q, k, v, out, lse, *grads, block_size, cu_seqlens, max_seqlen, scale,
                                 softcap, deterministic, sm_margin)
        return grads + (None,) * 8


def _apply(q, k, v, cu_seqlens, max_seqlen, block_size, softmax_scale, descales, softcap, deterministic,
           sm_margin, return_attn_probs):
    out, lse = _DiffusionAttention.apply(q, k, v, cu_seqlens, max_seqlen, block_size, softmax_scale, descales,
                                         softcap, deterministic, sm_margin)
    return (out, lse) if return_attn_probs else out


def diffusion_attn_func(
    q,
    k,
    v,
    block_size,
    softmax_scale=None,
    q_descale=None, k_descale=None, v_descale=None,
    softcap=0.0,
    deterministic=False,
    sm_margin=0,
    return_attn_probs=False,
):
    """Block-diffusion attention on a batch of samples of equal length.

    Every sample is [noisy half (n tokens) | clean half (n tokens)]; each half is cut into blocks of
    `block_size` tokens. A noisy block attends to itself (bidirectionally) and to the clean blocks before it; a
    clean block attends to itself and to the clean blocks before it; clean never attends to noisy.

    Arguments:
        q: (batch_size, 2n, nheads, headdim); k, v: (batch_size, 2n, nheads_k, headdim), nheads_k divides nheads.
        block_size: positive int.
        softmax_scale: scaling of QK^T, default 1 / sqrt(headdim).
        q_descale, k_descale, v_descale: (batch_size, nheads_k) float32, FP8 inputs only.
        softcap: > 0 activates tanh soft-capping.
        deterministic: bitwise-reproducible backward.
        sm_margin: number of SMs to leave free.
        return_attn_probs: also return the log-sum-exp, (batch_size, nheads, 2n) float32.
    Returns out (batch_size, 2n, nheads, headdim) in q's dtype (BF16 for FP8 inputs), or (out, lse).
    """
    return _apply(q, k, v, None, None, block_size, softmax_scale, (q_descale, k_descale, v_descale), softcap,
                  deterministic, sm_margin, return_attn_probs)


def diffusion_attn_varlen_func(
    q,
    k,
    v,
    cu_seqlens_q,
    cu_seqlens_k,
    max_seqlen_q,
    max_seqlen_k,
    block_size,
    softmax_scale=None,
    q_descale=None, k_descale=None, v_descale=None,
    softcap=0.0,
    deterministic=False,
    sm_margin=0,
    return_attn_probs=False,
):
    """Block-diffusion attention on packed samples of variable length.

    Sample i occupies rows [cu_seqlens_q[i], cu_seqlens_q[i + 1]) of q, k and v, laid out as
    [noisy half | clean half] (every length is even); samples never attend to each other.

    Arguments:
        q: (total, nheads, headdim); k, v: (total, nheads_k, headdim).
        cu_seqlens_q: (batch_size + 1,) int32 on the device. cu_seqlens_k must be None or equal to it.
        max_seqlen_q: longest sample (2 max n_i). max_seqlen_k must be None or equal to it.
        Other arguments as in diffusion_attn_func.
    Returns out (total, nheads, headdim), or (out, lse) with lse (nheads, total).
    """
    if cu_seqlens_k is not None and cu_seqlens_k is not cu_seqlens_q:
        assert cu_seqlens_k.shape == cu_seqlens_q.shape, "cu_seqlens_k must be equal to cu_seqlens_q"
    if max_seqlen_k is not None:
        assert max_seqlen_k == max_seqlen_q, "max_seqlen_k must be equal to max_seqlen_q"
    return _apply(q, k, v, cu_seqlens_q, max_seqlen_q, block_size, softmax_scale,
                  (q_descale, k_descale, v_descale), softcap, deterministic, sm_margin, return_attn_probs)


# ---------------------------------------------------------------------------------------------------------------
# Packed projections. The reference takes q, k and v as separate tensors (interface.py:196-250 there); its own test
# feeds it views of one projection output (tests/test_diffusion_attn.py:260-266). These entry points take that one
# tensor, as the callers of an attention layer usually hold it, and hand back ONE gradient tensor of the same layout:
# the kernels read and write the views in place, so neither direction copies or concatenates anything.
# ---------------------------------------------------------------------------------------------------------------
def _split_packed(qkv, num_heads_q, varlen):
    """Views (q, k, v) of a packed projection. Behind the leading axes ((batch, 2n), or (total,) for packed samples)
    it is either (3, heads, dim) or (heads_q + 2 heads_k, dim) with `num_heads_q` = heads_q."""
    lead = 1 if varlen else 2
    if qkv.dim() == lead + 3:
        if qkv.shape[lead] != 3:
            raise ValueError(f"axis {lead} of a packed tensor with {qkv.dim()} dimensions must have size 3")
        if num_heads_q is not None and num_heads_q != qkv.shape[-2]:
            raise ValueError("num_heads_q disagrees with the head axis")
        return qkv.select(lead, 0), qkv.select(lead, 1), qkv.select(lead, 2)
    if qkv.dim() != lead + 2:
        raise ValueError(f"a packed tensor has {lead + 3} or {lead + 2} dimensions here, got {qkv.dim()}")
    if num_heads_q is None:
        raise ValueError("a packed tensor without a separate axis of size 3 needs num_heads_q")
    heads_total = qkv.shape[-2]
    if num_heads_q <= 0 or heads_total <= num_heads_q or (heads_total - num_heads_q) % 2 != 0:
        raise ValueError("the head axis must hold num_heads_q query heads followed by two equal groups of key and "
                         "value heads")
    heads_k = (heads_total - num_heads_q) // 2
    return (qkv.narrow(-2, 0, num_heads_q), qkv.narrow(-2, num_heads_q, heads_k),
            qkv.narrow(-2, num_heads_q + heads_k, heads_k))


@torch.library.custom_op("fda::_diffusion_attn_backward_packed", mutates_args=("dqkv",), device_types="cuda")
def _diffusion_attn_backward_packed(
    dout: torch.Tensor,
    qkv: torch.Tensor,
    out: torch.Tensor,
    softmax_lse: torch.Tensor,
    dqkv: torch.Tensor,
    block_size: int,
    num_heads_q: Optional[int] = None,
    cu_seqlens: Optional[torch.Tensor] = None,
    max_seqlen: Optional[int] = None,
    softmax_scale: Optional[float] = None,
    softcap: float = 0.0,
    deterministic: bool = False,
    sm_margin: int = 0,
) -> None:
    q, k, v = _split_packed(qkv, num_heads_q, cu_seqlens is not None)
    dq, dk, dv = _split_packed(dqkv, num_heads_q, cu_seqlens is not None)
    backward_launch(dout, q, k, v, out, softmax_lse, dq, dk, dv, block_size, cu_seqlens, max_seqlen, softmax_scale,
                    softcap, deterministic, sm_margin)


@torch.library.register_fake("fda::_diffusion_attn_backward_packed")
def _diffusion_attn_backward_packed_fake(dout, qkv, out, softmax_lse, dqkv, block_size, num_heads_q=None,
                                         cu_seqlens=None, max_seqlen=None, softmax_scale=None, softcap=0.0,
                                         deterministic=False, sm_margin=0) -> None:
    return None


class _DiffusionAttentionPacked(torch.autograd.Function):
    """Autograd node of the packed entry points: saves the packed tensor once and returns one packed gradient."""

    @staticmethod
    def forward(ctx, qkv, num_heads_q, cu_seqlens, max_seqlen, block_size, softmax_scale, softcap, deterministic,
                sm_margin):
        q, k, v = _split_packed(qkv, num_heads_q, cu_seqlens is not None)
        scale = q.shape[-1] ** (-0.5) if softmax_scale is None else softmax_scale
        out, lse = _diffusion_attn_forward(q, k, v, block_size, cu_seqlens, max_seqlen, None, None, None, scale,
                                           softcap, sm_margin)
        ctx.save_for_backward(*((qkv, out, lse) + ((cu_seqlens,) if cu_seqlens is not None else ())))
        ctx.packed = cu_seqlens is not None
        ctx.opts = (num_heads_q, block_size, max_seqlen, scale, softcap, deterministic, sm_margin)
        return out, lse

    @staticmethod
    def backward(ctx, dout, *unused):
        qkv, out, lse = ctx.saved_tensors[:3]
        cu_seqlens = ctx.saved_tensors[3] if ctx.packed else None
        num_heads_q, block_size, max_seqlen, scale, softcap, deterministic, sm_margin = ctx.opts
        assert qkv.dtype in (torch.float16, torch.bfloat16), "The backward pass only supports fp16 and bf16"
        dqkv = torch.empty(qkv.shape, dtype=qkv.dtype, device=qkv.device)
        _diffusion_attn_backward_packed(dout, qkv, out, lse, dqkv, block_size, num_heads_q, cu_seqlens, max_seqlen,
                                        scale, softcap, deterministic, sm_margin)
        return (dqkv,) + (None,) * 8


def diffusion_attn_qkvpacked_func(
    qkv,
    block_size,
    num_heads_q=None,
    softmax_scale=None,
    softcap=0.0,
    deterministic=False,
    sm_margin=0,
    return_attn_probs=False,
):
    """diffusion_attn_func on one packed projection.

    Arguments:
        qkv: (batch_size, 2n, 3, nheads, headdim), or, for grouped-query attention,
            (batch_size, 2n, nheads + 2 nheads_k, headdim) with `num_heads_q` = nheads: query heads first, then the
            key heads, then the value heads. FP16 or BF16; the innermost dimension contiguous.
        Other arguments as in diffusion_attn_func.
    Returns out (batch_size, 2n, nheads, headdim), or (out, lse). The gradient of qkv is one tensor of qkv's shape.
    """
    out, lse = _DiffusionAttentionPacked.apply(qkv, num_heads_q, None, None, block_size, softmax_scale, softcap,
                                               deterministic, sm_margin)
    return (out, lse) if return_attn_probs else out


def diffusion_attn_varlen_qkvpacked_func(
    qkv,
    cu_seqlens,
    max_seqlen,
    block_size,
    num_heads_q=None,
    softmax_scale=None,
    softcap=0.0,
    deterministic=False,
    sm_margin=0,
    return_attn_probs=False,
):
    """diffusion_attn_varlen_func on one packed projection: qkv is (total, 3, nheads, headdim) or
    (total, nheads + 2 nheads_k, headdim) with `num_heads_q`; cu_seqlens and max_seqlen as there."""
    out, lse = _DiffusionAttentionPacked.apply(qkv, num_heads_q, cu_seqlens, max_seqlen, block_size, softmax_scale,
                                               softcap, deterministic, sm_margin)
    return (out, lse) if return_attn_probs else out
