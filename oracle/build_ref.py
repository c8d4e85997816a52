"""Stage the reference project's own CPU implementation of the path under oracle/_ref/ (TEST INFRASTRUCTURE ONLY).

    python oracle/build_ref.py /path/to/reference

The reference's only code that runs without its sm90 extension is `fast_diffusion_attention/reference.py` (pure
PyTorch; `attention_ref` materialises the mask in float32). Its package `__init__` imports the compiled extension,
so the file is staged by itself and loaded by path. "Building" a Python reference is a copy: the staged file is a
build output like a compiled object (oracle/_ref/ is listed in .gitignore and never committed), used by
`bench.py` as the timed CPU baseline (`cpu_baseline.kind = "reference"`) and by tests that compare the oracle
with it when it is present. Nothing in the library imports it.
"""

import importlib.util
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
STAGED = os.path.join(HERE, "_ref", "reference.py")


def stage(reference_root):
    """Copy reference.py of the checkout at `reference_root`; returns the staged path or None if it is absent."""
    src = os.path.join(reference_root, "fast_diffusion_attention", "reference.py")
    if not os.path.isfile(src):
        return None
    os.makedirs(os.path.dirname(STAGED), exist_ok=True)
    shutil.copyfile(src, STAGED)
    return STAGED


def load():
    """The staged module, or None when it has not been staged on this machine."""
    if not os.path.isfile(STAGED):
        return None
    spec = importlib.util.spec_from_file_location("fda_reference_staged", STAGED)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    out = stage(sys.argv[1]) if len(sys.argv) > 1 else None
    print(out or "reference checkout not found: nothing staged")
