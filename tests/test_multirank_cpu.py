"""Host-side logic of the multi-rank benchmark on CPU ranks (gloo, world size 2): the max-over-ranks reduction
of the step time, the scatter / gather of one problem cut over key/value heads or samples (reassembled results
bitwise equal to the one-rank oracle), and the reference arm printing exactly one line from rank 0."""

import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _torchrun(script_args, port):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(port)] + script_args
    env = dict(os.environ, OMP_NUM_THREADS="2")
    return subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT, env=env)


def test_reduction_scatter_and_gather_with_two_gloo_ranks():
    r = _torchrun([os.path.join(ROOT, "tests", "_gloo_worker.py")], 29631)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "GLOO_WORKER_OK 2" in r.stdout


def test_reference_arm_prints_one_line_from_rank_zero():
    r = _torchrun([os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
                   "--warmup", "0"], 29632)
    assert r.returncode == 0, r.stdout + r.stderr
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference" and rec["n_gpus"] == 2 and rec["cpu_baseline"]["kind"] in ("reference", "port")
    assert rec["e2e"]["h2d_bytes_per_step"] == 0
