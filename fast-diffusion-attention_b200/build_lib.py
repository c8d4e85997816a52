"""Build libfda_sm100.so in-tree with nvcc, for sm_100a only.

    python build_lib.py            # incremental
    python build_lib.py --force    # rebuild everything

Environment (same names as the reference's setup.py:5-13 where they make sense here):
  FDA_LINEINFO=0        drop -lineinfo (on by default)
  FDA_RESOURCE_USAGE=1  print registers / spills / shared memory per kernel (ptxas -v)
  NVCC_THREADS, MAX_JOBS  parallelism
"""

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "fast_diffusion_attention", "libfda_sm100.so")
SOURCES = ["abi.cu", "fwd_sm100.cu", "bwd_sm100.cu", "bwd_fused_sm100.cu", "selftest_sm100.cu", "varlen_list.cu"]


def _nvcc():
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = os.path.join(cuda_home, "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def _headers():
    out = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    out.append(os.path.join(HERE, "..", "include", "fda.h"))
    return out


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    flags = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC",
             "--expt-relaxed-constexpr", "-Xcudafe", "--diag_suppress=177"]
    if os.environ.get("FDA_LINEINFO", "1") == "1":
        flags.append("-lineinfo")
    if os.environ.get("FDA_RESOURCE_USAGE", "0") == "1":
        flags += ["-Xptxas", "-v"]
    flags += ["--threads", os.environ.get("NVCC_THREADS", "2")]
    headers = _headers()
    jobs = []
    objs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ, src.replace(".cu", ".o"))
        objs.append(o)
        if force or _stale(o, [s] + headers):
            jobs.append([_nvcc(), "-c", s, "-o", o] + flags)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode != 0 or os.environ.get("FDA_RESOURCE_USAGE", "0") == "1":
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed for " + cmd[2])

    with ThreadPoolExecutor(max_workers=int(os.environ.get("MAX_JOBS", "4"))) as ex:
        list(ex.map(run, jobs))
    if force or jobs or _stale(LIB, objs):
        run([_nvcc(), "-shared", "-o", LIB] + objs + ["-cudart", "static"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
