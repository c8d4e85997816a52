"""Benchmark of the block-diffusion attention training step (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (one "step"): forward + backward of `diffusion_attn_func` on the BF16 MHA configuration the headline
metric is quoted on: B=8 samples per GPU, n=2048 (2n=4096 rows), 16 heads, head_dim 128, block_size 256,
q, k, v, dO ~ N(0,1) from a seed, cast to bf16 (synthetic stand-in: the reference benchmarks on seeded randn too,
benchmarks/benchmark_diffusion.py there). Every rank owns its own B=8 shard (batch x head units are independent:
no collective in the data path), so scaling is weak; torch.distributed is used only for the barrier and the
max-over-ranks of the device time.

Metric: training-step TFLOPS on visible (query, key) pairs: 3.5 * 4 * pairs * d * H per sample
(forward 4*pairs*d*H, backward 2.5x; benchmarks/benchmark_diffusion.py:175-180 of the reference).

The JSON line carries:
  value      device-resident inputs, CUDA-event time of K steps (max over ranks), aggregate over ranks
  e2e        same step through the public API with HOST (pinned) buffers: q, k, v, dO copied host->device and
             out, dq, dk, dv copied device->host inside the timed region, every step; the copies of neighbouring
             steps overlap the kernels (separate copy streams, two buffer sets)
  roofline   the kernel with the largest share of the step, timed live with CUDA events between the launches
  cpu_baseline   the CPU oracle (oracle/diffusion_oracle.py, a port of the reference's reference.py) on a bounded
             sample of the same workload, on this box's host cores (rank 0, N=1 only)
`--impl reference` times only that CPU implementation (all host threads) and prints the same line shape.
"""

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "fast-diffusion-attention_b200"))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

# dram__bytes_read.sum + dram__bytes_write.sum of one launch on this workload, from the ncu capture summarised in
# profiles/c2_step_kernels_ncu.md (bytes)
NCU_TRAFFIC_BYTES = {"fwd_kernel": 550.7e6, "bwd_dkdv_kernel": 897.0e6, "bwd_dq_kernel": 677.7e6,
                     "bwd_preprocess_kernel": None}

WORKLOAD = dict(name="C2 bf16 MHA fwd+bwd", batch=8, n=2048, heads=16, heads_k=16, head_dim=128, block_size=256)
METRIC = "train-step TFLOPS (visible pairs), bf16 d=128"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(source="measured", hbm_gbs=d["hbm_gbs"], tflops_burst=d["bf16_tflops"],
                    tflops_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]))
    return dict(source="fallback", hbm_gbs=6650.0, tflops_burst=1590.0, tflops_sustained=1400.0)


class ClockSampler:
    """Samples SM clocks and throttle reasons (read-only NVML queries, nvidia-smi as a fallback) while the timed
    region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.mhz, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._nvml = None
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = gpu_index
            if visible:
                ids = [x.strip() for x in visible.split(",") if x.strip()]
                if gpu_index < len(ids) and ids[gpu_index].isdigit():
                    phys = int(ids[gpu_index])
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
            self._nvml = pynvml
        except Exception:
            self._nvml = None

    def _sample_nvml(self):
        n = self._nvml
        self.mhz.append(float(n.nvmlDeviceGetClockInfo(self._handle, n.NVML_CLOCK_SM)))
        try:
            mask = n.nvmlDeviceGetCurrentClocksEventReasons(self._handle)
        except Exception:
            mask = n.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle)
        for name, bit in self.REASON_BITS.items():
            if mask & bit:
                self.reasons.add(name)

    def _sample_smi(self):
        out = subprocess.run(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.QUERY,
                              "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5)
        parts = [x.strip() for x in out.stdout.strip().split(",")]
        if len(parts) >= 6 and parts[0].replace(".", "").isdigit():
            self.mhz.append(float(parts[0]))
            self.max_mhz = float(parts[1]) if parts[1].replace(".", "").isdigit() else self.max_mhz
            for i, name in enumerate(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]):
                if parts[2 + i].lower().startswith("active"):
                    self.reasons.add(name)

    def _run(self):
        while not self._stop.is_set():
            try:
                if self._nvml is not None:
                    self._sample_nvml()
                else:
                    self._sample_smi()
            except Exception:
                pass
            self._stop.wait(0.002 if self._nvml is not None else 0.05)

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
                    samples=len(self.mhz), source="nvml" if self._nvml is not None else "nvidia-smi")


def shard_seed(rank):
    """Every rank owns its own B=8 shard of the global batch: independent samples from its own seed."""
    return 1234 + rank


def max_over_ranks(value, dist_module, world, device):
    """Largest `value` (float) over all ranks; identity when there is one rank."""
    if world <= 1:
        return float(value)
    t = torch.tensor([float(value)], device=device, dtype=torch.float64)
    dist_module.all_reduce(t, op=dist_module.ReduceOp.MAX)
    return float(t.item())


def make_cpu_sample(threads=None):
    """The bounded CPU sample of the workload: ONE sample x 2 heads of the C2 shape (same n, head_dim,
    block_size), float32 forward + explicit backward with the oracle. Returns (run_once, flops, description)."""
    from oracle import diffusion_oracle as orc
    if threads:
        torch.set_num_threads(threads)
    w = WORKLOAD
    heads_sample = 2
    g = torch.Generator().manual_seed(0)
    shape = (1, 2 * w["n"], heads_sample, w["head_dim"])
    q, k, v, do = (torch.randn(shape, generator=g).to(torch.bfloat16) for _ in range(4))
    fwd, bwd = orc.step_flops([w["n"]], w["block_size"], heads_sample, w["head_dim"])

    def run_once():
        t0 = time.perf_counter()
        orc.forward(q, k, v, w["block_size"])
        orc.backward(q, k, v, do, w["block_size"])
        return time.perf_counter() - t0

    desc = (f"1 sample x {heads_sample} heads of the C2 shape (n={w['n']}, d={w['head_dim']}, "
            f"block_size={w['block_size']}), float32 forward + explicit backward")
    return run_once, fwd + bwd, desc


def use_all_host_threads():
    """The launcher for several ranks pins every process to one OpenMP thread; the CPU arm is meant to use the
    cores this process may run on."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


def cpu_reference_run(seconds_budget=20.0):
    use_all_host_threads()
    run_once, flops, desc = make_cpu_sample()
    run_once()  # warm-up (allocator, thread pool)
    times = []
    t_start = time.perf_counter()
    while len(times) < 3 or (time.perf_counter() - t_start < seconds_budget and len(times) < 20):
        times.append(run_once())
    sec = statistics.median(times)
    return dict(value=flops / sec / 1e12, unit="TFLOPS", cores=torch.get_num_threads(), kind="port",
                sample=f"{desc}, median of {len(times)} runs, {sec:.2f} s each")


def run_reference_arm(args, rank, world):
    """The reference's CPU implementation of the path (its reference.py, restated in oracle/) on the host cores."""
    if rank != 0:
        return
    use_all_host_threads()
    run_once, flops, desc = make_cpu_sample()
    for _ in range(max(args.warmup, 0)):
        run_once()
    times = [run_once() for _ in range(max(args.steps, 1))]
    sec = statistics.mean(times)
    value = flops / sec / 1e12
    cores = torch.get_num_threads()
    line = dict(impl="reference", metric=METRIC, value=value, unit="TFLOPS", n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=sec * 1e3, higher_is_better=True, scaling="weak", vs_baseline=None,
                dtype="f32", data="synthetic",
                config=dict(workload=WORKLOAD["name"] + " (CPU: each step is a bounded sample)", **{
                    k: v for k, v in WORKLOAD.items() if k != "name"}),
                cpu_baseline=dict(value=value, unit="TFLOPS", cores=cores, kind="port", sample=desc + " per step"),
                e2e=dict(value=value, unit="TFLOPS", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-cpu-baseline", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch.distributed as dist
    from fast_diffusion_attention import diffusion_attn_func, _lib
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
    gen = torch.Generator().manual_seed(shard_seed(rank))
    host = [torch.randn(B, 2 * n, h, d, generator=gen).to(torch.bfloat16).pin_memory() for h in (H, Hk, Hk, H)]
    q, k, v, do = (t.to(dev) for t in host)
    fwd_flops, bwd_flops = orc.step_flops([n] * B, bs, H, d)
    step_flops = fwd_flops + bwd_flops
    scale = d ** -0.5
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    ws = torch.empty(_lib.load().fda_bwd_workspace_bytes(
        __import__("ctypes").byref(_lib.FdaProblem(0, B, 2 * n, B * 2 * n, H, Hk, d, bs, scale, 0.0, 0, 0, None))),
        dtype=torch.uint8, device=dev)

    def step_device(events=None):
        """One training step of the hot path with device-resident inputs, stage by stage (4 kernels)."""
        if events is not None:
            events[0].record()
        out, lse = _diffusion_attn_forward(q, k, v, bs, None, None, None, None, None, scale, 0.0, 0)
        if events is not None:
            events[1].record()
        backward_launch(do, q, k, v, out, lse, dq, dk, dv, bs, softmax_scale=scale, workspace=ws, stages=1)
        if events is not None:
            events[2].record()
        backward_launch(do, q, k, v, out, lse, dq, dk, dv, bs, softmax_scale=scale, workspace=ws, stages=2)
        if events is not None:
            events[3].record()
        backward_launch(do, q, k, v, out, lse, dq, dk, dv, bs, softmax_scale=scale, workspace=ws, stages=4)
        if events is not None:
            events[4].record()
        return out

    for _ in range(args.warmup):
        step_device()
    barrier()
    status = _lib.device_status()
    if status[0] != 0:
        raise SystemExit(f"device-side wait expired during warm-up: {status}")

    # ---- timed region: K steps, CUDA events on the launching (current) stream --------------------------------------
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(args.steps)]
    e_start, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    with ClockSampler(local_rank) as clocks:
        e_start.record()
        for i in range(args.steps):
            step_device(ev[i])
        e_end.record()
        barrier()
    total_ms = e_start.elapsed_time(e_end)
    ms_per_step = max_over_ranks(total_ms, dist, world, dev) / args.steps
    value = step_flops * world / (ms_per_step * 1e-3) / 1e12

    names = ["fwd_kernel", "bwd_preprocess_kernel", "bwd_dkdv_kernel", "bwd_dq_kernel"]
    kernel_ms = [statistics.mean(ev[i][j].elapsed_time(ev[i][j + 1]) for i in range(args.steps)) for j in range(4)]
    pairs_flops = fwd_flops / 4.0  # pairs * d * H summed over the batch
    algorithmic = [4 * pairs_flops, 0.0, 8 * pairs_flops, 2 * pairs_flops]  # S,dP,dV,dK in dkdv; only dQ is new in dq
    top = max(range(4), key=lambda j: kernel_ms[j])
    peaks = measured_peaks()
    achieved = algorithmic[top] / (kernel_ms[top] * 1e-3) / 1e12
    roofline = dict(bound="tensor", kernel=names[top], achieved=achieved, peak=peaks["tflops_sustained"],
                    unit="TFLOP/s", frac=achieved / peaks["tflops_sustained"], traffic=NCU_TRAFFIC_BYTES.get(names[top]),
                    traffic_unit="bytes per launch (ncu dram read + write, profiles/c2_step_kernels_ncu.md)",
                    peak_source=peaks["source"] + " cuBLAS bf16, sustained (kernel timed inside a long step)",
                    kernel_ms={nm: round(ms, 4) for nm, ms in zip(names, kernel_ms)},
                    kernel_tflops_algorithmic={nm: (round(f / (ms * 1e-3) / 1e12, 1) if f else None)
                                               for nm, f, ms in zip(names, algorithmic, kernel_ms)})

    # ---- end to end through the public API with host buffers ---------------------------------------------------------
    e2e = None
    if not args.skip_e2e:
        # Every step copies its inputs from pinned host memory and its results (out, dq, dk, dv) back to pinned host
        # memory. The copies of neighbouring steps overlap the kernels: inputs go up on one stream, results come
        # down on another, two sets of device and host buffers alternate, events carry the dependencies.
        outs_host = [[torch.empty_like(t).pin_memory() for t in (host[0], host[0], host[1], host[2])] for _ in range(2)]
        dev_in = [[torch.empty_like(t, device=dev) for t in host] for _ in range(2)]
        s_main = torch.cuda.current_stream(dev)
        s_up, s_down = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        in_ready = [torch.cuda.Event() for _ in range(2)]
        in_free = [torch.cuda.Event() for _ in range(2)]
        out_done = [torch.cuda.Event() for _ in range(2)]
        computed = [torch.cuda.Event() for _ in range(2)]
        e2e_count = [0]

        def step_e2e():
            i = e2e_count[0]
            e2e_count[0] += 1
            slot = i & 1
            with torch.cuda.stream(s_up):
                if i >= 2:
                    s_up.wait_event(in_free[slot])       # the step that last read these device inputs is done
                for dst, src in zip(dev_in[slot], host):
                    dst.copy_(src, non_blocking=True)
                in_ready[slot].record(s_up)
            s_main.wait_event(in_ready[slot])
            qd, kd, vd, dod = dev_in[slot]
            qd.requires_grad_(True); kd.requires_grad_(True); vd.requires_grad_(True)
            out = diffusion_attn_func(qd, kd, vd, bs)
            gq, gk, gv = torch.autograd.grad(out, (qd, kd, vd), dod)
            qd.requires_grad_(False); kd.requires_grad_(False); vd.requires_grad_(False)
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

        for _ in range(3):
            step_e2e()
        drain()
        barrier()
        e2e_steps = max(4, min(args.steps, 10))
        e_start.record()
        s_up.wait_event(e_start)
        for _ in range(e2e_steps):
            step_e2e()
        drain()
        e_end.record()
        barrier()
        outs_host = outs_host[0]
        e2e_ms = max_over_ranks(e_start.elapsed_time(e_end), dist, world, dev) / e2e_steps
        e2e = dict(value=step_flops * world / (e2e_ms * 1e-3) / 1e12, unit="TFLOPS",
                   h2d_bytes_per_step=sum(t.numel() * 2 for t in host),
                   d2h_bytes_per_step=sum(t.numel() * 2 for t in outs_host), ms_per_step=e2e_ms)

    cpu = None
    if rank == 0 and world == 1 and not args.skip_cpu_baseline:
        cpu = cpu_reference_run()

    if rank == 0:
        line = dict(metric=METRIC, value=value, unit="TFLOPS", n_gpus=world, steps=args.steps, warmup=args.warmup,
                    ms_per_step=ms_per_step, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16",
                    data="synthetic",
                    config=dict(workload=w["name"], batch_per_gpu=B, n=n, seq_len=2 * n, heads=H, heads_k=Hk,
                                head_dim=d, block_size=bs, global_batch=B * world, sharding="batch over ranks",
                                l2="inputs+outputs per step ~1.1 GB, larger than the 126 MB L2"),
                    per_gpu_tflops=value / world,
                    frac_of_peak=dict(measured_burst=value / world / peaks["tflops_burst"],
                                      measured_sustained=value / world / peaks["tflops_sustained"],
                                      nominal_dense_bf16=value / world / 2250.0),
                    clocks=clocks.summary(), e2e=e2e, gpu_launches=4 * args.steps, roofline=roofline,
                    cpu_baseline=cpu)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
