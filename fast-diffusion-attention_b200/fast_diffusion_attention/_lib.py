"""ctypes binding of libfda_sm100.so (the C ABI declared in include/fda.h).

The library is built in-tree by build_lib.py / setup.py. There is no fallback: if the shared object is missing
the import fails, exactly as the reference fails without its compiled `_C` module
(fast_diffusion_attention/interface.py:11 there).
"""

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# FDA_LIBRARY names another build of the same library (for instance one compiled with -lineinfo off or with
# ptxas statistics); by default the in-tree build next to this file is loaded.
LIB_PATH = os.environ.get("FDA_LIBRARY") or os.path.join(_HERE, "libfda_sm100.so")

FDA_BF16, FDA_FP16, FDA_E4M3 = 0, 1, 2

FDA_OK = 0
FDA_ERR_DEVICE_WAIT = 14
FDA_ERR_SCRATCH_LIMIT = 15
NOALLOC_SCRATCH_BYTES = 16 << 20


class FdaTensor(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("batch_stride", C.c_int64), ("row_stride", C.c_int64),
                ("head_stride", C.c_int64)]


class FdaProblem(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("batch", C.c_int32), ("seqlen", C.c_int32), ("total", C.c_int32),
                ("heads", C.c_int32), ("heads_k", C.c_int32), ("head_dim", C.c_int32), ("block_size", C.c_int32),
                ("softmax_scale", C.c_float), ("softcap", C.c_float), ("sm_margin", C.c_int32),
                ("deterministic", C.c_int32), ("cu_seqlens", C.c_void_p)]


class FdaFwdArgs(C.Structure):
    _fields_ = [("p", FdaProblem), ("q", FdaTensor), ("k", FdaTensor), ("v", FdaTensor), ("out", FdaTensor),
                ("lse", C.c_void_p), ("q_descale", C.c_void_p), ("k_descale", C.c_void_p),
                ("v_descale", C.c_void_p), ("descale_batch_stride", C.c_int64 * 3),
                ("descale_head_stride", C.c_int64 * 3), ("workspace", C.c_void_p),
                ("workspace_bytes", C.c_size_t)]


class FdaBwdArgs(C.Structure):
    _fields_ = [("p", FdaProblem), ("q", FdaTensor), ("k", FdaTensor), ("v", FdaTensor), ("out", FdaTensor),
                ("dout", FdaTensor), ("dq", FdaTensor), ("dk", FdaTensor), ("dv", FdaTensor),
                ("lse", C.c_void_p), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t)]


EXPORTS = [
    "fda_fwd_workspace_bytes", "fda_bwd_workspace_bytes", "fda_fwd", "fda_bwd", "fda_bwd_stages", "fda_bwd_noalloc", "fda_strerror",
    "fda_last_cuda_error", "fda_device_status", "fda_version", "fda_geom_key_plan", "fda_geom_query_plan",
    "fda_geom_classify", "fda_geom_item_order", "fda_selftest_umma", "fda_selftest_wait",
]

_lib = None


def load():
    """Load the shared library once; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: build it with `python build_lib.py` (or `python setup.py build_ext --inplace`) "
            "in fast-diffusion-attention_b200/. There is no CPU or PyTorch fallback.")
    lib = C.CDLL(LIB_PATH)
    lib.fda_fwd_workspace_bytes.restype = C.c_size_t
    lib.fda_fwd_workspace_bytes.argtypes = [C.POINTER(FdaProblem)]
    lib.fda_bwd_workspace_bytes.restype = C.c_size_t
    lib.fda_bwd_workspace_bytes.argtypes = [C.POINTER(FdaProblem)]
    lib.fda_fwd.restype = C.c_int
    lib.fda_fwd.argtypes = [C.POINTER(FdaFwdArgs), C.c_void_p]
    lib.fda_bwd.restype = C.c_int
    lib.fda_bwd.argtypes = [C.POINTER(FdaBwdArgs), C.c_void_p]
    lib.fda_bwd_stages.restype = C.c_int
    lib.fda_bwd_stages.argtypes = [C.POINTER(FdaBwdArgs), C.c_uint, C.c_void_p]
    lib.fda_bwd_noalloc.restype = C.c_int
    lib.fda_bwd_noalloc.argtypes = [C.POINTER(FdaBwdArgs), C.c_void_p]
    lib.fda_strerror.restype = C.c_char_p
    lib.fda_strerror.argtypes = [C.c_int]
    lib.fda_last_cuda_error.restype = C.c_char_p
    lib.fda_device_status.restype = C.c_int
    lib.fda_device_status.argtypes = [C.POINTER(C.c_int32)]
    lib.fda_version.restype = C.c_char_p
    for name in ("fda_geom_key_plan", "fda_geom_query_plan"):
        fn = getattr(lib, name)
        fn.restype = C.c_int
        fn.argtypes = [C.c_int] * 6 + [C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.c_int]
    lib.fda_geom_classify.restype = C.c_int
    lib.fda_geom_classify.argtypes = [C.c_int] * 10
    lib.fda_geom_item_order.restype = C.c_int
    lib.fda_geom_item_order.argtypes = [C.c_int] * 5 + [C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
    lib.fda_selftest_umma.restype = C.c_int
    lib.fda_selftest_umma.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
    lib.fda_selftest_wait.restype = C.c_int
    lib.fda_selftest_wait.argtypes = [C.c_longlong, C.c_void_p]
    _lib = lib
    return lib


def check(status):
    """Raise RuntimeError with the library's message for a non-zero status."""
    if status != FDA_OK:
        lib = load()
        msg = lib.fda_strerror(status).decode()
        detail = lib.fda_last_cuda_error().decode()
        raise RuntimeError(f"fast-diffusion-attention: {msg}" + (f" [{detail}]" if detail and status == 10 else ""))


def device_status():
    """(code, block, thread, detail) of the first expired device-side wait since the last call; code 0 = none.
    Synchronises the current device."""
    lib = load()
    out = (C.c_int32 * 4)()
    rc = lib.fda_device_status(out)
    if rc not in (FDA_OK, FDA_ERR_DEVICE_WAIT):
        check(rc)
    return tuple(out)
