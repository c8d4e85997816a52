"""The C ABI loads without a GPU and exports every symbol include/fda.h declares; argument errors map to the
reference's vocabulary (tests/test_diffusion_attn.py:332-348 of the reference grep for the same words)."""

import ctypes as C
import os
import re

import pytest

from fast_diffusion_attention import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "fda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fda_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = declared_functions()
    assert len(names) >= 12
    for name in names:
        assert hasattr(lib, name), name
    assert set(names) == set(_lib.EXPORTS)


def test_version_and_messages():
    lib = _lib.load()
    assert lib.fda_version().decode().count(".") == 2
    assert "even" in lib.fda_strerror(3).decode()
    assert "block_size must be a positive integer" in lib.fda_strerror(4).decode()
    assert "deterministic" in lib.fda_strerror(8).decode()


def _problem(**kw):
    base = dict(dtype=0, batch=1, seqlen=64, total=64, heads=2, heads_k=2, head_dim=64, block_size=4,
                softmax_scale=0.125, softcap=0.0, sm_margin=0, deterministic=0, cu_seqlens=None)
    base.update(kw)
    return _lib.FdaProblem(*[base[f[0]] for f in _lib.FdaProblem._fields_])


@pytest.mark.parametrize("kw,code", [
    (dict(seqlen=63, total=63), 3), (dict(block_size=0), 4), (dict(head_dim=260), 5), (dict(head_dim=60), 5),
    (dict(heads=3), 6), (dict(dtype=7), 2),
])
def test_fwd_argument_errors_without_gpu(kw, code):
    lib = _lib.load()
    args = _lib.FdaFwdArgs()
    args.p = _problem(**kw)
    assert lib.fda_fwd(C.byref(args), None) == code


def test_bwd_rejects_fp8_and_null():
    lib = _lib.load()
    args = _lib.FdaBwdArgs()
    args.p = _problem(dtype=2)
    assert lib.fda_bwd(C.byref(args), None) == 2
    args.p = _problem()
    assert lib.fda_bwd(C.byref(args), None) == 1


def test_workspace_sizes_positive():
    lib = _lib.load()
    p = _problem(batch=8, seqlen=4096, total=8 * 4096, heads=16, heads_k=16, head_dim=128, block_size=256)
    assert lib.fda_fwd_workspace_bytes(C.byref(p)) >= 4
    assert lib.fda_bwd_workspace_bytes(C.byref(p)) >= 4
