"""Benchmark of the block-diffusion attention training step (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (one "step"): forward + backward of `diffusion_attn_func` on the BF16 MHA configuration the headline
metric is quoted on: B=8 samples, n=2048 (2n=4096 rows), 16 heads, head_dim 128, block_size 256; q, k, v, dO ~ N(0,1)
from a seed, cast to bf16 (synthetic stand-in: the reference benchmarks on seeded randn too,
benchmarks/benchmark_diffusion.py there). With N > 1 ranks this ONE problem is cut into N equal slices over
key/value heads (fast_diffusion_attention/sharding.py): rank 0 scatters q, k, v, dO with NCCL, every rank runs the
step on its slice, out, dq, dk, dv are gathered back to rank 0 ("scaling": "strong"; there is no collective inside
the step).

Metric: training-step TFLOPS on visible (query, key) pairs: 3.5 * 4 * pairs * d * H per sample
(forward 4*pairs*d*H, backward 2.5x; benchmarks/benchmark_diffusion.py:175-180 of the reference).

The JSON line carries:
  value        K steps through the public functions (diffusion_attn_func + torch.autograd.grad) with the rank's
               slice resident on the device, CUDA events on the launching stream, max over ranks, whole-job TFLOPS
  with_collectives   the same with the scatter of the inputs and the gather of the results inside the timed region
  replicas     (N > 1) every rank runs the WHOLE problem on its own data: weak scaling, no communication at all
  sustained    a region of at least two seconds of back-to-back steps: TFLOPS of its first 50 steps (burst) and of
               the whole region (sustained), each with the median SM clock, each against the matching measured peak
  e2e          the step with HOST (pinned) buffers: q, k, v, dO copied host->device and out, dq, dk, dv copied
               device->host inside the timed region, every step
  roofline     the kernel with the largest share of the step, timed live with CUDA events between the stage launches
  other_configs   the other benchmark configurations (GQA deterministic, packed varlen with softcap, head dim 256,
               FP8 forward) and small block sizes on the headline shape, through the public functions (N = 1 only)
  cpu_baseline the reference's own CPU implementation (its reference.py, staged under oracle/_ref by
               oracle/build_ref.py; the oracle's port of it if that file is absent) on this box's host cores
`--impl reference` times only that CPU implementation (all host threads) and prints the same line shape.
"""

import argparse
import ctypes
import json
import os
import random
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "fast-diffusion-attention_b200"))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

# dram__bytes_read.sum + dram__bytes_write.sum of one launch on the headline workload, from ncu captures (bytes)
NCU_TRAFFIC_BYTES = {"fwd_kernel": 548.7e6, "bwd_fused_kernel": 1655.3e6, "bwd_dkdv_kernel": 897.0e6,
                     "bwd_dq_kernel": 677.7e6}

WORKLOAD = dict(name="C2 bf16 MHA fwd+bwd", batch=8, n=2048, heads=16, heads_k=16, head_dim=128, block_size=256)
METRIC = "train-step TFLOPS (visible pairs), bf16 d=128"
C1 = dict(batch=2, n=256, heads=4, head_dim=64, block_size=64)   # the reference's own CPU-runnable configuration


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(source="measured", hbm_gbs=d["hbm_gbs"], tflops_burst=d["bf16_tflops"],
                    tflops_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]))
    return dict(source="fallback", hbm_gbs=6650.0, tflops_burst=1590.0, tflops_sustained=1400.0)


class ClockSampler:
    """Samples SM clocks and throttle reasons of ONE physical GPU (read-only NVML queries) while a timed region
    runs. The GPU is found by the UUID of the CUDA device, so CUDA_VISIBLE_DEVICES cannot make it sample a
    neighbour; when that fails nothing is sampled and the summary says so."""

    REASON_BITS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, cuda_index):
        self.mhz, self.reasons, self.max_mhz, self.watts = [], set(), None, []
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._nvml = None
        try:
            import pynvml
            pynvml.nvmlInit()
            uuid = "GPU-" + str(torch.cuda.get_device_properties(cuda_index).uuid)
            try:
                self._handle = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            except TypeError:
                self._handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
            self._nvml = pynvml
        except Exception:
            self._nvml = None

    def _sample(self):
        n = self._nvml
        self.mhz.append(float(n.nvmlDeviceGetClockInfo(self._handle, n.NVML_CLOCK_SM)))
        try:
            self.watts.append(n.nvmlDeviceGetPowerUsage(self._handle) / 1000.0)
        except Exception:
            pass
        try:
            mask = n.nvmlDeviceGetCurrentClocksEventReasons(self._handle)
        except Exception:
            mask = n.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle)
        for name, bit in self.REASON_BITS.items():
            if mask & bit:
                self.reasons.add(name)

    def _run(self):
        while not self._stop.is_set():
            try:
                if self._nvml is not None:
                    self._sample()
            except Exception:
                pass
            self._stop.wait(0.002)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self):
        if not self.mhz:
            return dict(sm_mhz=None, sm_max_mhz=self.max_mhz, reasons=["unsampled"])
        return dict(sm_mhz=statistics.median(self.mhz), sm_max_mhz=self.max_mhz, reasons=sorted(self.reasons),
                    samples=len(self.mhz), power_w_max=max(self.watts) if self.watts else None, source="nvml by uuid")


def max_over_ranks(value, dist_module, world, device):
    """Largest `value` (float) over all ranks; identity when there is one rank."""
    if world <= 1:
        return float(value)
    t = torch.tensor([float(value)], device=device, dtype=torch.float64)
    dist_module.all_reduce(t, op=dist_module.ReduceOp.MAX)
    return float(t.item())


def make_full_inputs(seed=1234, w=WORKLOAD, pin=False):
    """The whole problem on the host: q, k, v, dO of the headline configuration from one seed."""
    gen = torch.Generator().manual_seed(seed)
    out = []
    for h in (w["heads"], w["heads_k"], w["heads_k"], w["heads"]):
        t = torch.randn(w["batch"], 2 * w["n"], h, w["head_dim"], generator=gen).to(torch.bfloat16)
        out.append(t.pin_memory() if pin else t)
    return out


# ---------------------------------------------------------------------------------------------------------------------
# CPU arm: the reference's own reference.py when it has been staged, the oracle's port of it otherwise
# ---------------------------------------------------------------------------------------------------------------------
def use_all_host_threads():
    """The launcher for several ranks pins every process to one OpenMP thread; the CPU arm is meant to use the
    cores this process may run on."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


def make_cpu_step(batch, n, heads, head_dim, block_size, dtype=torch.float32):
    """(run_once, flops, kind, description): forward + gradients of one problem on the CPU in float32, through the
    staged reference (attention_ref + torch.autograd.grad) or, without it, the oracle's explicit formulas."""
    from oracle import build_ref
    from oracle import diffusion_oracle as orc
    ref = build_ref.load()
    g = torch.Generator().manual_seed(0)
    shape = (batch, 2 * n, heads, head_dim)
    q, k, v, do = (torch.randn(shape, generator=g).to(dtype) for _ in range(4))
    fwd, bwd = orc.step_flops([n] * batch, block_size, heads, head_dim)
    if ref is not None:
        def run_once():
            qq, kk, vv = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
            t0 = time.perf_counter()
            out, _ = ref.attention_ref(qq, kk, vv, block_size)
            torch.autograd.grad(out, (qq, kk, vv), do.to(out.dtype))
            return time.perf_counter() - t0
        kind = "reference"
    else:
        def run_once():
            t0 = time.perf_counter()
            orc.forward(q, k, v, block_size)
            orc.backward(q, k, v, do, block_size)
            return time.perf_counter() - t0
        kind = "port"
    how = "attention_ref + torch.autograd.grad of the staged reference.py" if ref is not None else \
        "the oracle's port of reference.py (forward + explicit backward)"
    desc = f"B={batch}, n={n}, H={heads}, d={head_dim}, block_size={block_size}, float32, {how}"
    return run_once, fwd + bwd, kind, desc


def cpu_baseline_run(seconds_budget=12.0):
    """C1 (the reference's own CPU configuration) and a bounded sample of the headline shape."""
    cores = use_all_host_threads()
    out = {}
    for name, cfg in (("c1", dict(batch=C1["batch"], n=C1["n"], heads=C1["heads"], head_dim=C1["head_dim"],
                                  block_size=C1["block_size"])),
                      ("c2_sample", dict(batch=1, n=WORKLOAD["n"], heads=2, head_dim=WORKLOAD["head_dim"],
                                         block_size=WORKLOAD["block_size"]))):
        run_once, flops, kind, desc = make_cpu_step(**cfg)
        run_once()
        run_once()
        times = []
        t_start = time.perf_counter()
        while len(times) < 5 or (time.perf_counter() - t_start < seconds_budget / 2 and len(times) < 50):
            times.append(run_once())
        sec = statistics.median(times)
        out[name] = dict(value=flops / sec / 1e12, unit="TFLOPS", ms_per_step=sec * 1e3, kind=kind,
                         sample=f"{desc}; median of {len(times)} steps")
    head = out["c2_sample"]
    return dict(value=head["value"], unit="TFLOPS", cores=cores, host_cpus=os.cpu_count(), kind=head["kind"],
                sample="bounded sample of the headline workload: " + head["sample"],
                c1=dict(gflops=out["c1"]["value"] * 1e3, ms_per_step=out["c1"]["ms_per_step"], kind=out["c1"]["kind"],
                        sample=out["c1"]["sample"]))


def run_reference_arm(args, rank, world):
    """The reference's CPU implementation of the path on the host cores; each step a bounded sample of the headline
    workload (one sample x two heads of its shape)."""
    if rank != 0:
        return
    cores = use_all_host_threads()
    run_once, flops, kind, desc = make_cpu_step(batch=1, n=WORKLOAD["n"], heads=2, head_dim=WORKLOAD["head_dim"],
                                                block_size=WORKLOAD["block_size"])
    for _ in range(max(args.warmup, 0)):
        run_once()
    times = [run_once() for _ in range(max(args.steps, 1))]
    sec = statistics.mean(times)
    value = flops / sec / 1e12
    line = dict(impl="reference", metric=METRIC, value=value, unit="TFLOPS", n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=sec * 1e3, higher_is_better=True, scaling="strong", vs_baseline=None,
                dtype="f32", data="synthetic",
                config=dict(workload=WORKLOAD["name"] + " (CPU: each step is a bounded sample)", **{
                    k: v for k, v in WORKLOAD.items() if k != "name"}),
                cpu_baseline=dict(value=value, unit="TFLOPS", cores=cores, kind=kind, sample=desc + " per step"),
                e2e=dict(value=value, unit="TFLOPS", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------------------------
def time_steps(step, n_steps, sync):
    """CUDA-event time (ms) of n_steps back-to-back calls of `step` on the current stream."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    e0.record()
    for _ in range(n_steps):
        step()
    e1.record()
    sync()
    return e0.elapsed_time(e1)


def other_config_legs(dev, peaks):
    """The other benchmark configurations through the public functions, a few steps each (one GPU)."""
    from fast_diffusion_attention import _lib, diffusion_attn_func, diffusion_attn_varlen_func
    from fast_diffusion_attention.interface import _problem, backward_launch
    from oracle import diffusion_oracle as orc

    def sync():
        torch.cuda.synchronize(dev)

    def randn(shape, seed, dtype=torch.bfloat16):
        g = torch.Generator(device=dev).manual_seed(seed)
        return torch.randn(shape, generator=g, device=dev, dtype=torch.float32).to(dtype)

    results = {}

    def run_case(name, q, k, v, do, bs, ns, heads, d, cu=None, max_len=None, steps=6, **kw):
        fwd_f, bwd_f = orc.step_flops(ns, bs, heads, d)
        q, k, v = (t.requires_grad_(True) for t in (q, k, v))

        def fwd():
            if cu is None:
                return diffusion_attn_func(q, k, v, bs, return_attn_probs=True, **kw)
            return diffusion_attn_varlen_func(q, k, v, cu, cu, max_len, max_len, bs, return_attn_probs=True, **kw)

        def step():
            out, _ = fwd()
            torch.autograd.grad(out, (q, k, v), do)

        def fwd_only():
            with torch.no_grad():
                fwd()

        # every leg starts as a burst, like the headline: the legs before it leave the clock lower than boost
        sync()
        time.sleep(1.5)
        for _ in range(3):
            step()
        with ClockSampler(dev.index) as clocks:
            ms_fwd = time_steps(fwd_only, steps, sync) / steps
            ms_step = time_steps(step, steps, sync) / steps
        # per-kernel split of the backward: the stages launched one by one with events between them
        with torch.no_grad():
            out, lse = fwd()
        grads = [torch.empty_like(t) for t in (q, k, v)]
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(steps)]
        batch = (cu.numel() - 1) if cu is not None else q.shape[0]
        seqlen = max_len if cu is not None else q.shape[1]
        total_rows = q.shape[0] if cu is not None else q.shape[0] * q.shape[1]
        prob = _problem(q, k, batch, seqlen, total_rows, bs, d ** -0.5, kw.get("softcap", 0.0), 0,
                        kw.get("deterministic", False), cu)
        ws = torch.empty(_lib.load().fda_bwd_workspace_bytes(ctypes.byref(prob)), dtype=torch.uint8, device=dev)
        for i in range(steps + 1):
            for j, stage in enumerate((1, 2, 4)):
                if i > 0:
                    ev[i - 1][j].record()
                backward_launch(do, q.detach(), k.detach(), v.detach(), out, lse, *grads, bs, cu, max_len,
                                softcap=kw.get("softcap", 0.0), deterministic=kw.get("deterministic", False),
                                stages=stage, workspace=ws)
            if i > 0:
                ev[i - 1][3].record()
        sync()
        stage_ms = [statistics.median(ev[i][j].elapsed_time(ev[i][j + 1]) for i in range(steps)) for j in range(3)]
        results[name] = dict(ms_fwd=round(ms_fwd, 4), ms_step=round(ms_step, 4),
                             tflops_fwd=round(fwd_f / ms_fwd / 1e9, 1), tflops_step=round((fwd_f + bwd_f) / ms_step / 1e9, 1),
                             step_gflop=round((fwd_f + bwd_f) / 1e9, 1),
                             bwd_stage_ms=dict(preprocess=round(stage_ms[0], 4), main=round(stage_ms[1], 4),
                                               dq=round(stage_ms[2], 4)),
                             frac_of_burst_peak=round((fwd_f + bwd_f) / ms_step / 1e9 / peaks["tflops_burst"], 3),
                             clocks=clocks.summary())
        return results[name]

    # C3: GQA, deterministic backward
    B, n, H, Hk, d, bs = 4, 4096, 32, 8, 128, 1024
    run_case("c3_gqa_deterministic", randn((B, 2 * n, H, d), 11), randn((B, 2 * n, Hk, d), 13),
             randn((B, 2 * n, Hk, d), 14), randn((B, 2 * n, H, d), 12), bs, [n] * B, H, d, deterministic=True)
    results["c3_gqa_deterministic"]["config"] = dict(batch=B, n=n, heads=H, heads_k=Hk, head_dim=d, block_size=bs)
    r = run_case("c3_gqa_single_pass", randn((B, 2 * n, H, d), 11), randn((B, 2 * n, Hk, d), 13),
                 randn((B, 2 * n, Hk, d), 14), randn((B, 2 * n, H, d), 12), bs, [n] * B, H, d, deterministic=False)
    r["config"] = dict(batch=B, n=n, heads=H, heads_k=Hk, head_dim=d, block_size=bs, note="same shape, deterministic=False")
    torch.cuda.empty_cache()
    # C4: packed varlen, d=64, softcap
    H, d, bs = 32, 64, 256
    rng = random.Random(0)
    ns = [256 * rng.randint(2, 32) for _ in range(16)]
    cu = torch.tensor([0] + list(torch.tensor([2 * x for x in ns]).cumsum(0)), device=dev, dtype=torch.int32)
    total = 2 * sum(ns)
    r = run_case("c4_varlen_softcap", randn((total, H, d), 21), randn((total, H, d), 22), randn((total, H, d), 23),
                 randn((total, H, d), 24), bs, ns, H, d, cu=cu, max_len=2 * max(ns), steps=4, softcap=30.0)
    r["config"] = dict(n_per_sample=ns, total_rows=total, heads=H, head_dim=d, block_size=bs, softcap=30.0)
    torch.cuda.empty_cache()
    # C5: head dim 256, bf16 step and FP8 forward
    B, n, H, d, bs = 2, 8192, 8, 256, 256
    q, k, v, do = (randn((B, 2 * n, H, d), s) for s in (31, 32, 33, 34))
    r = run_case("c5_d256", q, k, v, do, bs, [n] * B, H, d)
    r["config"] = dict(batch=B, n=n, heads=H, head_dim=d, block_size=bs)

    def quantise(t):
        descale = (t.detach().float().abs().amax(dim=(1, 3)) / 448.0).clamp_min(1e-12)
        return (t.detach().float() / descale[:, None, :, None]).to(torch.float8_e4m3fn), descale.contiguous()

    (q8, qd), (k8, kd), (v8, vd) = quantise(q), quantise(k), quantise(v)

    def fwd8():
        diffusion_attn_func(q8, k8, v8, bs, q_descale=qd, k_descale=kd, v_descale=vd)

    sync()
    time.sleep(1.5)
    for _ in range(3):
        fwd8()
    with ClockSampler(dev.index) as clocks:
        ms8 = time_steps(fwd8, 8, sync) / 8
    fwd_f, _ = orc.step_flops([n] * B, bs, H, d)
    fp8 = dict(ms_fwd=round(ms8, 4), tflops_fwd=round(fwd_f / ms8 / 1e9, 1), clocks=clocks.summary(),
               config=dict(batch=B, n=n, heads=H, head_dim=d, block_size=bs, descale="amax / 448 per (sample, head)"))
    try:   # FP8 denominator: a dense e4m3 GEMM of the library everybody uses, measured in the same run
        a = torch.randn(8192, 8192, device=dev).to(torch.float8_e4m3fn)
        b = torch.randn(8192, 8192, device=dev).to(torch.float8_e4m3fn).t()
        one = torch.tensor(1.0, device=dev)

        def mm8():
            torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)

        for _ in range(3):
            mm8()
        best = min(time_steps(mm8, 5, sync) / 5 for _ in range(3))
        fp8["scaled_mm_8192_tflops"] = round(2 * 8192 ** 3 / best / 1e9, 1)
        fp8["frac_of_scaled_mm"] = round(fp8["tflops_fwd"] / fp8["scaled_mm_8192_tflops"], 3)
        del a, b
    except Exception as e:   # pragma: no cover
        fp8["scaled_mm_8192_tflops"] = None
        fp8["scaled_mm_error"] = str(e)[:120]
    results["c5_fp8_forward"] = fp8
    del q, k, v, do, q8, k8, v8
    torch.cuda.empty_cache()
    # small blocks on the headline shape (what block-diffusion language models train with)
    w = WORKLOAD
    B, n, H, d = w["batch"], w["n"], w["heads"], w["head_dim"]
    q, k, v, do = (randn((B, 2 * n, H, d), s) for s in (41, 42, 43, 44))
    small = {}
    for bs in (4, 16, 64, 256):
        r = run_case(f"_bs{bs}", q.detach(), k.detach(), v.detach(), do, bs, [n] * B, H, d, steps=5)
        small[str(bs)] = dict(tflops_fwd=r["tflops_fwd"], tflops_step=r["tflops_step"], ms_step=r["ms_step"],
                              bwd_stage_ms=r["bwd_stage_ms"])
        del results[f"_bs{bs}"]
    results["c2_shape_small_blocks"] = small
    return results


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-cpu-baseline", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-other-configs", action="store_true")
    ap.add_argument("--skip-sustained", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="time the eager step only (for profilers)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch.distributed as dist
    from fast_diffusion_attention import diffusion_attn_func, _lib, sharding
    from fast_diffusion_attention.interface import _diffusion_attn_forward, backward_launch
    from oracle import diffusion_oracle as orc

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    w = WORKLOAD
    B, n, H, Hk, d, bs = w["batch"], w["n"], w["heads"], w["heads_k"], w["head_dim"], w["block_size"]
    kind, _ = sharding.plan(B, H, Hk, world)
    fwd_flops, bwd_flops = orc.step_flops([n] * B, bs, H, d)
    step_flops = fwd_flops + bwd_flops           # of the WHOLE problem
    full_shapes = [(B, 2 * n, h, d) for h in (H, Hk, Hk, H)]
    peaks = measured_peaks()

    # ---- the problem lives on rank 0; every rank gets its slice (NCCL scatter; a plain copy with one rank) -------
    full_host = make_full_inputs(pin=True) if rank == 0 else None
    full_dev = [t.to(dev, non_blocking=True) for t in full_host] if rank == 0 else [None] * 4

    def scatter_inputs():
        if world == 1:
            return [t for t in full_dev]
        return [sharding.scatter(full_dev[i], full_shapes[i], torch.bfloat16, dev, kind) for i in range(4)]

    def gather_results(results):
        if world == 1:
            return results
        return [sharding.gather(t, kind) for t in results]

    q, k, v, do = scatter_inputs()
    q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)

    def step_public():
        """One training step of the hot path through the public function and autograd."""
        out = diffusion_attn_func(q, k, v, bs)
        dq, dk, dv = torch.autograd.grad(out, (q, k, v), do)
        return out, dq, dk, dv

    for _ in range(args.warmup):
        step_public()
    barrier()
    status = _lib.device_status()
    if status[0] != 0:
        raise SystemExit(f"device-side wait expired during warm-up: {status}")

    # ---- value: K steps, CUDA events on the launching (current) stream, max over ranks ------------------------------
    # Eager: the Python calls are made every step. Their host cost (a few hundred microseconds of operator dispatch,
    # autograd bookkeeping and argument marshalling) does not shrink with the slice, so with several ranks the eager
    # step becomes launch-bound; the same calls captured once in a CUDA graph and replayed take the host out of the
    # loop. Both are timed; `value` is the replayed one when the capture works, `eager` is reported beside it.
    eager_ms_total = time_steps(step_public, args.steps, barrier)
    host_enqueue_ms = None
    barrier()
    t_h = time.perf_counter()
    for _ in range(args.steps):
        step_public()
    host_enqueue_ms = (time.perf_counter() - t_h) * 1e3 / args.steps    # time to ENQUEUE a step (no synchronisation)
    barrier()
    eager_ms = max_over_ranks(eager_ms_total, dist, world, dev) / args.steps
    graph, graph_error = None, None
    try:
        if args.no_graph:
            raise RuntimeError("--no-graph")
        if hasattr(torch.autograd.graph, "set_warn_on_accumulate_grad_stream_mismatch"):
            torch.autograd.graph.set_warn_on_accumulate_grad_stream_mismatch(False)
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(3):
                step_public()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            graph_outputs = step_public()
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        ref_outputs = step_public()
        torch.cuda.synchronize()
        for name, a, b in zip(("out", "dq", "dk", "dv"), graph_outputs, ref_outputs):
            # the replay runs the same kernels: everything but dq (fp32 adds in scheduling order) is bitwise equal
            if name != "dq" and not torch.equal(a, b):
                raise RuntimeError(f"graph replay changed {name}")
            if (a.float() - b.float()).abs().max().item() > 0.05 * b.float().abs().max().item() + 1e-3:
                raise RuntimeError(f"graph replay changed {name}")
    except Exception as e:   # pragma: no cover
        graph, graph_error = None, str(e)[:200]
    ok = torch.tensor([1.0 if graph is not None else 0.0], device=dev)
    if world > 1:
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    use_graph = bool(ok.item() > 0)
    with ClockSampler(local_rank) as clocks:
        if use_graph:
            total_ms = time_steps(graph.replay, args.steps, barrier)
        else:
            total_ms = time_steps(step_public, args.steps, barrier)
    ms_per_step = max_over_ranks(total_ms, dist, world, dev) / args.steps
    value = step_flops / (ms_per_step * 1e-3) / 1e12
    eager = dict(value=step_flops / (eager_ms * 1e-3) / 1e12, unit="TFLOPS", ms_per_step=eager_ms,
                 host_enqueue_ms_per_step=host_enqueue_ms, cuda_graph="replayed" if use_graph else
                 f"not used: {graph_error}")

    # ---- the same with scatter and gather inside the timed region (N > 1) ---------------------------------------------
    with_coll = None
    if world > 1:
        def step_with_collectives():
            qq, kk, vv, dd = scatter_inputs()
            qq.requires_grad_(True); kk.requires_grad_(True); vv.requires_grad_(True)
            out = diffusion_attn_func(qq, kk, vv, bs)
            grads = torch.autograd.grad(out, (qq, kk, vv), dd)
            gather_results([out.detach(), *grads])

        for _ in range(2):
            step_with_collectives()
        coll_steps = max(4, min(args.steps, 10))
        coll_ms = max_over_ranks(time_steps(step_with_collectives, coll_steps, barrier), dist, world, dev) / coll_steps
        moved = 2 * sum(B * 2 * n * h * d * 2 for h in (H, Hk, Hk, H)) * (world - 1) / world   # leaves / reaches rank 0
        with_coll = dict(value=step_flops / (coll_ms * 1e-3) / 1e12, unit="TFLOPS", ms_per_step=coll_ms,
                         collective_ms=coll_ms - ms_per_step, bytes_through_rank0=moved,
                         rank0_link_gbs=moved / max(coll_ms - ms_per_step, 1e-6) / 1e6,
                         how="dist.scatter of q, k, v, dO from rank 0 and dist.gather of out, dq, dk, dv to rank 0 (NCCL), "
                             "every step")

    # ---- replicas: every rank steps the whole problem on its own data (weak scaling, no communication) --------------
    replicas = None
    if world > 1:
        gen = torch.Generator().manual_seed(1234 + rank)
        rq, rk, rv, rdo = (torch.randn(s, generator=gen).to(torch.bfloat16).to(dev) for s in full_shapes)
        rq.requires_grad_(True); rk.requires_grad_(True); rv.requires_grad_(True)

        def step_replica():
            out = diffusion_attn_func(rq, rk, rv, bs)
            torch.autograd.grad(out, (rq, rk, rv), rdo)

        for _ in range(3):
            step_replica()
        rep_steps = max(5, min(args.steps, 20))
        rep_ms = max_over_ranks(time_steps(step_replica, rep_steps, barrier), dist, world, dev) / rep_steps
        replicas = dict(value=step_flops * world / (rep_ms * 1e-3) / 1e12, unit="TFLOPS", ms_per_step=rep_ms,
                        scaling="weak", note="one whole problem per rank, independent data")
        del rq, rk, rv, rdo

    # ---- roofline: the stages of a step launched one by one with events between them -----------------------------------
    Hl, Hkl = q.shape[2], k.shape[2]
    Bl = q.shape[0]
    scale = d ** -0.5
    qd, kd, vd = q.detach(), k.detach(), v.detach()
    dq, dk, dv = torch.empty_like(qd), torch.empty_like(kd), torch.empty_like(vd)
    prob = _lib.FdaProblem(0, Bl, 2 * n, Bl * 2 * n, Hl, Hkl, d, bs, scale, 0.0, 0, 0, None)
    ws = torch.empty(_lib.load().fda_bwd_workspace_bytes(ctypes.byref(prob)), dtype=torch.uint8, device=dev)
    stage_steps = max(10, min(args.steps, 20))
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(stage_steps)]

    def step_stages(events):
        events[0].record()
        out, lse = _diffusion_attn_forward(qd, kd, vd, bs, None, None, None, None, None, scale, 0.0, 0)
        for j, stage in enumerate((1, 2, 4)):
            events[1 + j].record()
            backward_launch(do, qd, kd, vd, out, lse, dq, dk, dv, bs, softmax_scale=scale, workspace=ws, stages=stage)
        events[4].record()

    # The denominator is the cuBLAS burst figure (a kernel timed alone, at boost clocks). After a few hundred
    # milliseconds of continuous load the SM clock of these parts settles some 12 % lower with no throttle reason
    # shown, so the stages are timed as a burst too: after a pause, and with the clock sampled beside them.
    barrier()
    time.sleep(1.5)
    for i in range(3):
        step_stages(ev[0])
    barrier()
    with ClockSampler(local_rank) as c_stage:
        for i in range(stage_steps):
            step_stages(ev[i])
        barrier()
    names = ["fwd_kernel", "bwd_preprocess_kernel", "bwd_fused_kernel (+ accumulator zero-fill)", "bwd_dq_convert_kernel"]
    kernel_ms = [statistics.median(ev[i][j].elapsed_time(ev[i][j + 1]) for i in range(stage_steps)) for j in range(4)]
    pairs_flops = fwd_flops / 4.0 / world        # pairs * d * H of this rank's slice
    algorithmic = [4 * pairs_flops, 0.0, 10 * pairs_flops, 0.0]   # forward 2 GEMMs; single-pass backward all 5
    top = max(range(4), key=lambda j: kernel_ms[j])
    achieved = algorithmic[top] / (kernel_ms[top] * 1e-3) / 1e12
    roofline = dict(bound="tensor", kernel=names[top], achieved=achieved, peak=peaks["tflops_burst"], unit="TFLOP/s",
                    frac=achieved / peaks["tflops_burst"],
                    traffic=(NCU_TRAFFIC_BYTES.get(names[top].split(" ")[0]) if world == 1 else None),
                    traffic_note="bytes per launch, dram read + write of one ncu capture of this kernel on this workload "
                                 "(one GPU, whole problem)",
                    peak_source=peaks["source"] + " cuBLAS bf16 burst figure: the stage-by-stage region lasts "
                                                  f"{sum(kernel_ms) * stage_steps:.0f} ms at boost clocks",
                    algorithmic_gflop_per_launch=algorithmic[top] / 1e9,
                    kernel_ms={nm: round(ms, 4) for nm, ms in zip(names, kernel_ms)},
                    clocks=c_stage.summary(),
                    kernel_tflops_algorithmic={nm: (round(f / (ms * 1e-3) / 1e12, 1) if f else None)
                                               for nm, f, ms in zip(names, algorithmic, kernel_ms)})

    # ---- a region of at least two seconds: burst (first 50 steps) against sustained (whole region) -------------------
    sustained = None
    if not args.skip_sustained:
        n_long = max(200, int(2200.0 / ms_per_step))
        e_marks = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        run_step = graph.replay if use_graph else step_public
        with ClockSampler(local_rank) as c_burst:
            barrier()
            e_marks[0].record()
            for _ in range(50):
                run_step()
            e_marks[1].record()
            torch.cuda.synchronize()
        with ClockSampler(local_rank) as c_long:
            for _ in range(n_long - 50):
                run_step()
            e_marks[2].record()
            barrier()
        burst_ms = max_over_ranks(e_marks[0].elapsed_time(e_marks[1]), dist, world, dev) / 50
        long_ms = max_over_ranks(e_marks[0].elapsed_time(e_marks[2]), dist, world, dev) / n_long
        b_tf, s_tf = step_flops / burst_ms / 1e9, step_flops / long_ms / 1e9
        sustained = dict(steps=n_long, region_s=long_ms * n_long / 1e3,
                         burst=dict(tflops=b_tf, per_gpu_frac_of_measured_burst=b_tf / world / peaks["tflops_burst"],
                                    clocks=c_burst.summary()),
                         sustained=dict(tflops=s_tf, per_gpu_frac_of_measured_sustained=s_tf / world / peaks["tflops_sustained"],
                                        clocks=c_long.summary()))

    # ---- end to end with host buffers: the whole problem leaves and reaches pinned host memory on rank 0 ------------------
    e2e = None
    if not args.skip_e2e:
        # Rank 0 copies q, k, v, dO host->device, (N > 1: scatters them,) every rank steps its slice, (the results are
        # gathered,) rank 0 copies out, dq, dk, dv device->host. With one rank the copies of neighbouring steps overlap
        # the kernels: inputs go up on one stream, results come down on another, two buffer sets alternate.
        if world == 1:
            host = full_host
            outs_host = [[torch.empty_like(t).pin_memory() for t in (host[0], host[0], host[1], host[2])] for _ in range(2)]
            dev_in = [[torch.empty_like(t, device=dev) for t in host] for _ in range(2)]
            s_main = torch.cuda.current_stream(dev)
            s_up, s_down = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
            in_ready = [torch.cuda.Event() for _ in range(2)]
            in_free = [torch.cuda.Event() for _ in range(2)]
            out_done = [torch.cuda.Event() for _ in range(2)]
            computed = [torch.cuda.Event() for _ in range(2)]
            count = [0]

            def step_e2e():
                i = count[0]
                count[0] += 1
                slot = i & 1
                with torch.cuda.stream(s_up):
                    if i >= 2:
                        s_up.wait_event(in_free[slot])       # the step that last read these device inputs is done
                    for dst, src in zip(dev_in[slot], host):
                        dst.copy_(src, non_blocking=True)
                    in_ready[slot].record(s_up)
                s_main.wait_event(in_ready[slot])
                qq, kk, vv, dd = dev_in[slot]
                qq.requires_grad_(True); kk.requires_grad_(True); vv.requires_grad_(True)
                out = diffusion_attn_func(qq, kk, vv, bs)
                gq, gk, gv = torch.autograd.grad(out, (qq, kk, vv), dd)
                qq.requires_grad_(False); kk.requires_grad_(False); vv.requires_grad_(False)
                in_free[slot].record(s_main)
                computed[slot].record(s_main)
                results = (out.detach(), gq, gk, gv)
                with torch.cuda.stream(s_down):
                    s_down.wait_event(computed[slot])
                    for dst, src in zip(outs_host[slot], results):
                        src.record_stream(s_down)            # allocated on the main stream, read on this one
                        dst.copy_(src, non_blocking=True)
                    out_done[slot].record(s_down)

            def drain():
                for e in out_done:
                    s_main.wait_event(e)
        else:
            outs_host = [[torch.empty(full_shapes[i], dtype=torch.bfloat16).pin_memory() for i in (0, 0, 1, 2)]] \
                if rank == 0 else [None]

            def step_e2e():
                if rank == 0:
                    for dst, src in zip(full_dev, full_host):
                        dst.copy_(src, non_blocking=True)
                qq, kk, vv, dd = scatter_inputs()
                qq.requires_grad_(True); kk.requires_grad_(True); vv.requires_grad_(True)
                out = diffusion_attn_func(qq, kk, vv, bs)
                grads = torch.autograd.grad(out, (qq, kk, vv), dd)
                got = gather_results([out.detach(), *grads])
                if rank == 0:
                    for dst, src in zip(outs_host[0], got):
                        dst.copy_(src, non_blocking=True)

            def drain():
                pass

        for _ in range(3):
            step_e2e()
        drain()
        e2e_steps = max(4, min(args.steps, 10))

        def run_e2e():
            step_e2e()

        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        if world == 1:
            s_up.wait_event(e0)
        for _ in range(e2e_steps):
            run_e2e()
        drain()
        e1.record()
        barrier()
        e2e_ms = max_over_ranks(e0.elapsed_time(e1), dist, world, dev) / e2e_steps
        e2e = dict(value=step_flops / (e2e_ms * 1e-3) / 1e12, unit="TFLOPS",
                   h2d_bytes_per_step=sum(B * 2 * n * h * d * 2 for h in (H, Hk, Hk, H)),
                   d2h_bytes_per_step=sum(B * 2 * n * h * d * 2 for h in (H, H, Hk, Hk)), ms_per_step=e2e_ms,
                   note="host buffers live on rank 0: the copies cross its PCIe link, the slices its NVLink")

    other = None
    if rank == 0 and world == 1 and not args.skip_other_configs:
        del q, k, v, do, qd, kd, vd, dq, dk, dv, ws
        torch.cuda.empty_cache()
        other = other_config_legs(dev, peaks)

    cpu = None
    if rank == 0 and world == 1 and not args.skip_cpu_baseline:
        cpu = cpu_baseline_run()

    if rank == 0:
        line = dict(metric=METRIC, value=value, unit="TFLOPS", n_gpus=world, steps=args.steps, warmup=args.warmup,
                    ms_per_step=ms_per_step, higher_is_better=True, scaling="strong", vs_baseline=None, dtype="bf16",
                    data="synthetic",
                    config=dict(workload=w["name"], batch=B, n=n, seq_len=2 * n, heads=H, heads_k=Hk, head_dim=d,
                                block_size=bs, global_batch=B,
                                sharding=f"{kind}: {Hk // world if kind == 'heads' else Hk} key/value heads x "
                                         f"{B if kind == 'heads' else B // world} samples per rank",
                                api="diffusion_attn_func + torch.autograd.grad, inputs resident on the device" +
                                    (", captured once in a CUDA graph and replayed" if use_graph else ", eager"),
                                l2=f"a step reads and writes {1.07 / world:.2f} GB of tensors per rank plus a "
                                   f"{0.28 / world:.2f} GB fp32 dQ accumulator: more than the 126 MB L2, no flush used"),
                    per_gpu_tflops=value / world,
                    frac_of_peak=dict(measured_burst=value / world / peaks["tflops_burst"],
                                      measured_sustained=value / world / peaks["tflops_sustained"],
                                      nominal_dense_bf16=value / world / 2250.0,
                                      note="the timed region is short (boost clocks): the burst figure is the matching one"),
                    clocks=clocks.summary(), e2e=e2e, gpu_launches=4 * args.steps,
                    gpu_launches_note="forward, backward preprocess, single-pass backward, dQ convert per step (the two "
                                      "memsets of a step are the runtime's)",
                    eager=eager, roofline=roofline, with_collectives=with_coll, replicas=replicas, sustained=sustained,
                    other_configs=other, cpu_baseline=cpu)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
