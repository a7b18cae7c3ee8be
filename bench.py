#!/usr/bin/env python
"""Benchmark of the hot path on B200: BASELINE config 2 (MLP fwd+bwd fp16 + AdamW).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-configs]

One "step" is one forward + backward + AdamW step of the 784 -> 8192 -> 8192 -> 10 MLP on a
256-sample batch, issued as C-ABI launches (torchvulkan_b200.workloads.MLPStep).
`value` is fp16 GEMM TFLOP/s: the step's 109.78 GFLOP of matrix products divided by the whole
step time (elementwise, reductions, loss and optimizer included), summed over ranks (replicas:
the step does not shard, so N > 1 runs N independent replicas, weak scaling).
The timed steps are replays of one captured step (a CUDA graph of the same launches; AdamW is one list
launch whose step count lives in device memory). `e2e` is the same metric with the step's inputs copied
from pinned host memory and the loss read back inside the timed region. `roofline` describes the kernel that takes the largest share of the
step, timed live with CUDA events; `cpu_baseline` is the ATen-CPU fp32 step (the reference's own CPU
path for these ops) on the host cores. `--impl reference` times that CPU path alone.
The same line carries the other BASELINE configs: `sharded_bmm` (bf16 bmm 64x4096^3 with the batches sharded over the
ranks and C completed on every rank, value-checked; at every N, N = 1 included) and, at N = 1, `configs`: fp32 mm
1024^3, the config-2 / 3 / 4 training scripts on the "vulkan" device (eager and torchvulkan.Graph, config 4 in NCHW and
channels-last) beside ATen CPU fp32, and fp32 add/exp/sum/argmax over 2^30 elements as GB/s. `--no-configs` leaves
those out.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SIZES = (784, 8192, 8192, 10)
BATCH = 256
METRIC = "fp16 mm TFLOP/s over the MLP fwd+bwd+AdamW step"
UNIT = "TFLOP/s"
# fp16 loss scaling: the backward pass runs on loss * LOSS_SCALE and AdamW's eps is scaled by the same factor, which in
# exact arithmetic is the unscaled AdamW(eps=1e-8) step (the update m/(sqrt(v)+eps) is homogeneous of degree 0 in the
# gradient scale once eps scales with it). Without it the fp16 second moments of a mean loss over 256 samples underflow
# to zero on any backend and the parameters turn into inf/NaN within a few steps.
LOSS_SCALE = 16384.0
ADAM_EPS = 1e-8 * LOSS_SCALE


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.rows, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except ValueError:
                continue
            for name, val in zip(names, r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_mlp_step_runner(threads: int):
    """ATen CPU fp32 model + AdamW (the reference's CPU fallback path for these ops; fp32 as
    benchmark/benchmark.py:46-48 does for its cpu backend). Returns a closure running one step."""
    import torch

    torch.set_num_threads(threads)
    torch.manual_seed(0)
    layers = []
    for i in range(len(SIZES) - 1):
        layers.append(torch.nn.Linear(SIZES[i], SIZES[i + 1]))
        if i < len(SIZES) - 2:
            layers.append(torch.nn.GELU())
    model = torch.nn.Sequential(*layers)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3, weight_decay=1e-2)
    x = torch.randn(BATCH, SIZES[0])
    y = torch.randint(0, SIZES[-1], (BATCH,))
    loss_fn = torch.nn.CrossEntropyLoss()

    def step():
        opt.zero_grad(set_to_none=True)
        loss = loss_fn(model(x), y)
        loss.backward()
        opt.step()
        return float(loss.detach())

    return step


def gemm_flops():
    f = 0
    for i in range(len(SIZES) - 1):
        f += 2 * 2 * BATCH * SIZES[i] * SIZES[i + 1]
        if i > 0:
            f += 2 * BATCH * SIZES[i] * SIZES[i + 1]
    return f


def time_cpu(steps: int, warmup: int, threads: int):
    step = cpu_mlp_step_runner(threads)
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = time.perf_counter() - t0
    return dt / steps


def run_reference(args, rank: int):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    # The CPU step is 1-2 s on a handful of cores; bound the run to a few minutes.
    spent = time_cpu(1, 1, threads)
    budget = 150.0
    steps = max(1, min(args.steps, int(budget / max(spent, 1e-3))))
    warm = max(0, min(args.warmup, 2))
    sec = time_cpu(steps, warm, threads)
    val = gemm_flops() / sec / 1e12
    sample = f"full config-2 step (batch {BATCH}, {SIZES}), ATen CPU fp32, {steps} of the requested {args.steps} steps timed"
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": steps, "warmup": warm,
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "MLP 784-8192-8192-10 GELU, batch 256, fwd+bwd+AdamW (BASELINE config 2)", "device": "host cores"},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "reference's Vulkan path (GPU or lavapipe) is unavailable on this box; this is its CPU fallback path (ATen CPU kernels)",
    }
    print(json.dumps(line), flush=True)


def summarize_trace(trace):
    """tag -> [launch count, launch count x the MEDIAN launch time in ms]: the median over the repeated steps, so that one
    slow repetition (a launch that waited for the host) does not move the figure."""
    import statistics

    import torch

    torch.cuda.synchronize()
    times = {}
    for tag, a, b in trace:
        times.setdefault(tag, []).append(a.elapsed_time(b))
    return {tag: [len(v), len(v) * statistics.median(v)] for tag, v in times.items()}


# dram__bytes_read.sum + dram__bytes_write.sum per launch from recorded ncu captures of these kernels (bytes, summary
# file). They are NOT measured by this run: the line says where the figure comes from, and a kernel without a capture
# reports null.
NCU_TRAFFIC_BYTES = {"adam_step n67108864": (882.9e6, "profiles/adam_vec_kernel_half_67M_params.md"),
                     "adam_step_multi n73629706": (974.6e6, "profiles/adam_multi_kernel_half_73M_params.md")}


def kernel_algorithmic(tag: str, es: int = 2):
    """(bound, algorithmic bytes or flops per launch) for a launch tag of MLPStep."""
    parts = tag.split()
    if parts[0] == "gemm":
        m, n, k = (int(p[1:]) for p in parts[1:4])
        return "tensor", 2.0 * m * n * k, (m * k + k * n + m * n) * es
    if parts[0] in ("adam_step", "adam_step_multi"):
        n = int(parts[1][1:])
        return "hbm", 7.0 * n * es, 7.0 * n * es           # read p,g,m,v; write p,m,v
    return "hbm", None, None


def run_ours(args, rank: int, world: int, local_rank: int):
    import torch
    import torch.distributed as dist

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from torchvulkan_b200 import capi, cuda_ops
    from torchvulkan_b200.workloads import MLPStep

    capi.lib()  # fail loudly before anything is timed if the CUDA library is missing
    if args.profile_run and args.workload in KERNEL_WORKLOADS:
        profile_kernels(args, dev)
        return
    pk = peaks()
    # one list launch for AdamW over all six parameter tensors, its step count in device memory: the whole step is
    # then a fixed sequence of launches that can be replayed as a CUDA graph
    step = MLPStep(sizes=SIZES, batch=BATCH, dtype=torch.float16, device=dev, seed=0, list_optimizer=True, loss_scale=LOSS_SCALE, eps=ADAM_EPS, fused=True)
    g = torch.Generator().manual_seed(0)
    x_host = torch.randn(BATCH, SIZES[0], generator=g).half().pin_memory()
    y_host = torch.randint(0, SIZES[-1], (BATCH,), generator=g).pin_memory()
    x, y = x_host.to(dev), y_host.to(dev)
    loss_host = torch.empty((), dtype=torch.float16).pin_memory()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        barrier()
        ms = a.elapsed_time(b)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t)
        return ms

    if args.profile_run and args.workload != "c2":
        profile_model_steps(args)
        return
    if args.profile_run:
        # The bare step loop for a profiler: warm-up, then K steps, nothing else.
        for _ in range(args.warmup):
            step.step(x, y)
        for _ in range(args.steps):
            step.step(x, y)
        torch.cuda.synchronize()
        cuda_ops.check_device_status(local_rank)
        print(json.dumps({"profile_run": True, "steps": args.steps, "launches_per_step": step.launches_per_step}), flush=True)
        return

    # ---- device-resident steps -----------------------------------------------------
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    first_loss = None
    for _ in range(max(args.warmup, 3)):
        step.step(x, y)
        if first_loss is None:
            first_loss = float(step.loss)
    cuda_ops.check_device_status(local_rank)
    # nvidia-smi needs a few hundred ms to produce its first samples: keep the same step running
    # (untimed) for about half a second so the clock record is taken under this load.
    t_end = time.perf_counter() + 0.5
    while time.perf_counter() < t_end:
        for _ in range(20):
            step.step(x, y)
        torch.cuda.synchronize()
    # The timed steps are replays of one captured step (the same launches in the same order, issued by the GPU's
    # front end instead of 22 host calls).
    step.capture(x, y)
    for _ in range(3):
        step.replay()
    ms = timed(step.replay, args.steps)
    launches = count_kernels(lambda: step.step(x, y), step.launches_per_step) * args.steps
    ms_per_step = ms / args.steps
    flops = step.gemm_flops()
    value = world * flops / (ms_per_step * 1e-3) / 1e12

    # ---- end to end: host inputs in, loss out, every step ----------------------------
    def e2e_step():
        x.copy_(x_host, non_blocking=True)
        y.copy_(y_host, non_blocking=True)
        step.replay()
        loss_host.copy_(step.loss, non_blocking=False)

    for _ in range(3):
        e2e_step()
    ms_e2e = timed(e2e_step, args.steps) / args.steps
    clocks = sampler.stop() if rank == 0 else None
    final_loss = float(loss_host)
    e2e = {"value": world * flops / (ms_e2e * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms_e2e,
           "h2d_bytes_per_step": x_host.numel() * 2 + y_host.numel() * 8, "d2h_bytes_per_step": 2,
           "api": "C-ABI launches (tvk_* entry points) captured once and replayed as a CUDA graph; inputs from pinned host memory, loss read back"}

    # ---- per-launch timing of the same step (rank 0), for the roofline object ----------
    line = None
    if rank == 0:
        step.trace = []
        reps = 9
        for _ in range(reps):
            step.step(x, y)
        agg = summarize_trace(step.trace)
        step.trace = None
        total = sum(v[1] for v in agg.values())
        kernels = sorted(((t, c, msum) for t, (c, msum) in agg.items()), key=lambda r: -r[2])
        top_tag, top_count, top_ms = kernels[0]
        bound, alg, alg_bytes = kernel_algorithmic(top_tag)
        dur = top_ms / top_count * 1e-3
        if bound == "tensor":
            achieved, peak, unit = alg / dur / 1e12, pk["bf16_tflops"], "TFLOP/s"
        else:
            achieved, peak, unit = (alg / dur / 1e9 if alg else None), pk["hbm_gbs"], "GB/s"
        traffic, traffic_src = NCU_TRAFFIC_BYTES.get(top_tag, (None, None))
        roofline = {"kernel": top_tag, "bound": bound, "achieved": achieved, "peak": peak, "unit": unit,
                    "frac": (achieved / peak if achieved else None), "traffic": traffic,
                    "traffic_source": (traffic_src + " (recorded ncu capture, not this run)") if traffic_src else None,
                    "algorithmic_bytes": alg_bytes, "peak_source": pk["source"], "launch_us": dur * 1e6, "share_of_step": top_ms / total}
        breakdown = [{"kernel": t, "launches_per_step": c // reps, "us_per_launch": msum / c * 1e3, "share": msum / total} for t, c, msum in kernels[:8]]

        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            sec = time_cpu(3, 1, threads)
            cpu = {"value": flops / sec / 1e12, "unit": UNIT, "cores": threads, "kind": "port", "ms_per_step": sec * 1e3,
                   "sample": "3 full config-2 steps (same shapes) after 1 warm-up, ATen CPU fp32 (the reference's CPU fallback path)"}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic",
            "config": {"workload": "MLP 784-8192-8192-10 GELU, batch 256, fwd+bwd+AdamW (BASELINE config 2)",
                       "parallelism": "replicas only" if world > 1 else "single GPU",
                       "l2": "no flush: 0.74 GB of weights, gradients and optimizer state per step exceed the 126 MB L2",
                       "launch": "CUDA-graph replay of the step's launches",
                       "loss_scale": LOSS_SCALE, "adam_eps": ADAM_EPS, "loss_first_step": first_loss, "loss_after_timed_steps": final_loss,
                       "loss_note": "the same batch every step: after the ~1500 steps this run takes, the 73.6 M parameters have memorised its 256 samples"},
            "e2e": e2e, "gpu_launches": launches, "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu, "kernels": breakdown,
        }
    del step
    torch.cuda.empty_cache()
    # the one part of the path that shards: reported with every run (N = 1 is the anchor of the strong-scaling curve)
    sharded = run_sharded_bmm(rank, world, dev, pk)
    if rank == 0:
        line["sharded_bmm"] = sharded
    if world == 1 and not args.no_configs:
        line["configs"] = run_configs(args, dev, pk)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_configs(args, dev, pk):
    """The other single-GPU BASELINE configs: C1 fp32 mm 1024^3 (-> relu -> sum), C5 (ii) fp32 add/exp/sum/argmax over
    2^30 elements, and the training scripts of configs 2, 3 and 4 on the "vulkan" device."""
    import torch
    from torchvulkan_b200 import cuda_ops as ops

    out = {}

    def ev_time(fn, reps, flush=None):
        torch.cuda.synchronize()
        times = []
        for _ in range(reps):
            if flush is not None:
                flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        return statistics.median(times)

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # larger than L2
    torch.manual_seed(0)
    ah, bh = torch.randn(1024, 1024), torch.randn(1024, 1024)
    a, b = ah.to(dev), bh.to(dev)
    for _ in range(3):
        ops.gemm(a, b)
    ms = ev_time(lambda: ops.gemm(a, b), 10, flush)

    def c1_chain():
        return ops.reduce("sum", ops.unary("relu", ops.gemm(a, b)))

    s_dev = float(c1_chain())
    ms_chain = ev_time(c1_chain, 10, flush)
    ref = float((ah.double() @ bh.double()).relu().sum())
    out["c1_fp32_mm_1024"] = {"ms": ms, "tflops": 2 * 1024 ** 3 / ms / 1e9, "ms_mm_relu_sum": ms_chain, "sum": s_dev, "sum_fp64_cpu": ref,
                              "sum_rel_error": abs(s_dev - ref) / abs(ref), "note": "3xTF32, includes the hi/lo split launches; L2 flushed between repetitions"}
    del a, b, flush

    n = 1 << 30
    x = torch.randn(n, device=dev)
    y = torch.randn(n, device=dev)
    z = torch.empty_like(x)
    bw = {}
    for name, fn, nbytes in (("add", lambda: ops.binary("add", x, y, out=z), 12 * n), ("exp", lambda: ops.unary("exp", x, out=z), 8 * n),
                             ("sum", lambda: ops.reduce("sum", x), 4 * n), ("argmax", lambda: ops.argreduce(x), 4 * n)):
        fn()
        ms = ev_time(fn, 5)
        bw[name] = {"ms": ms, "gbs": nbytes / ms / 1e6, "frac_of_hbm_peak": nbytes / ms / 1e6 / pk["hbm_gbs"], "algorithmic_bytes": nbytes}
    bw["peak_gbs"], bw["peak_source"] = pk["hbm_gbs"], pk["source"]
    bw["l2"] = "operands of 4 GiB each: far larger than L2, no flush"
    out["c5_fp32_2p30"] = bw
    del x, y, z
    torch.cuda.empty_cache()
    out.update(run_model_steps(args))
    return out


def run_sharded_bmm(rank, world, dev, pk):
    """BASELINE config 5 (i): bf16 bmm 64 x 4096^3 with the batches sharded over the ranks; every rank ends with the
    full C. Times the local GEMM alone and the three ways of completing C (torchvulkan_b200/sharded.py), each as the
    max over ranks of a CUDA-event interval around `reps` back-to-back steps, and then CHECKS what every mode left in
    this rank's copy of C: for one batch owned by each other rank (and one of its own) the operands are regenerated
    here from the batch's seed, the batch is multiplied locally, and the block that arrived over NVLink must match that
    local product (1e-3 relative Frobenius error; whether it was bit-identical is reported); a 97-row sample of it is
    also held to 1e-2 against an fp32 product by torch. A mode that fails the check fails the run."""
    import torch
    import torch.distributed as dist
    from torchvulkan_b200.sharded import ShardedBmm, shard_range

    lo, hi = shard_range(64, rank, world)
    nb = hi - lo

    def batch_operands(b):
        # operands of global batch b: the same bits on whichever rank generates them
        g = torch.Generator(device=dev).manual_seed(1000 + b)
        a_ = torch.randn(4096, 4096, device=dev, generator=g).bfloat16()
        b_ = torch.randn(4096, 4096, device=dev, generator=g).bfloat16()
        return a_, b_

    A = torch.empty(nb, 4096, 4096, dtype=torch.bfloat16, device=dev)
    B = torch.empty(nb, 4096, 4096, dtype=torch.bfloat16, device=dev)
    for i in range(nb):
        A[i], B[i] = batch_operands(lo + i)
    Cfull = torch.empty(64, 4096, 4096, dtype=torch.bfloat16, device=dev)

    def timed(fn, reps=5):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        a_, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a_.record()
        for _ in range(reps):
            fn()
        b_.record()
        torch.cuda.synchronize()
        ms = a_.elapsed_time(b_) / reps
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t[0])
        return ms

    local = ShardedBmm(Cfull, mode="allgather", compute=None)
    scratch = torch.empty(4096, 4096, dtype=torch.bfloat16, device=dev)
    rows = torch.arange(97, device=dev) * 42 + 7          # 97 rows spread over the 4096

    def verify(run_once):
        """Poisons C, runs one more step and compares the blocks described above. Returns (ok, worst error, bit-equal)."""
        Cfull.fill_(float("nan"))
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        run_once()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        ok, worst, bit_equal = True, 0.0, True
        for q in range(world):
            qlo, qhi = shard_range(64, q, world)
            if qhi <= qlo:
                continue
            b = qlo + (rank + 3 * q) % (qhi - qlo)        # a different batch of rank q on every rank
            a_, b_ = batch_operands(b)
            local._gemm(a_, b_, scratch)
            bit_equal = bit_equal and bool(torch.equal(scratch, Cfull[b]))
            # the whole block against the local product (a line that never arrived is still NaN and fails this)
            whole = float((Cfull[b].float() - scratch.float()).norm() / scratch.float().norm())
            ref = a_[rows].float() @ b_.float()
            err = float((Cfull[b][rows].float() - ref).norm() / ref.norm())
            ok = ok and whole <= 1e-3 and err <= 1e-2
            worst = max([worst] + [e if e == e else float("inf") for e in (err, whole)])
        flag = torch.tensor([0.0 if ok else 1.0, worst, 0.0 if bit_equal else 1.0], device=dev)
        if world > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MAX)
        return bool(flag[0] == 0), float(flag[1]), bool(flag[2] == 0)

    flops = 64 * 2 * 4096 ** 3
    ms_gemm = timed(lambda: local._gemm(A, B, local.mine))
    res = {"n_gpus": world, "batches_per_gpu": nb, "ms_gemm_only": ms_gemm, "tflops_per_gpu_gemm_only": nb * 2 * 4096 ** 3 / ms_gemm / 1e9,
           "frac_of_peak_gemm_only": nb * 2 * 4096 ** 3 / ms_gemm / 1e9 / pk["bf16_tflops_sustained"], "peak": pk["bf16_tflops_sustained"],
           "peak_source": pk["source"] + " (sustained)",
           "check": "per mode: C poisoned with NaN, one more step, then one batch of every rank recomputed locally from its seed: the block in this "
                    "rank's C within 1e-3 relative Frobenius error of it (bit_equal says whether it was identical), and a 97-row sample within 1e-2 "
                    "of an fp32 product"}
    failed = []
    if world == 1:
        ok, worst, biteq = verify(lambda: local._gemm(A, B, local.mine))
        res.update({"ms_per_step": ms_gemm, "tflops_total": flops / ms_gemm / 1e9, "verified": ok, "worst_rel_error": worst, "bit_equal": biteq})
        if not ok:
            failed.append("single")
    else:
        recv = (world - 1) / world * Cfull.numel() * 2
        modes = {}
        for mode in ("allgather", "pipelined", "copy", "push"):
            op = ShardedBmm(Cfull, mode=mode, chunks=4)
            ms = timed(lambda: op.run(A, B))
            ok, worst, biteq = verify(lambda: op.run(A, B))
            op.close()
            modes[mode] = {"ms_per_step": ms, "tflops_total": flops / ms / 1e9, "verified": ok, "worst_rel_error": worst, "bit_equal": biteq,
                           "ingest_gbs": recv / ms / 1e6}
            if not ok:
                failed.append(mode)
        best = min(modes, key=lambda m: modes[m]["ms_per_step"])
        # context for the NVLink bound: the library all-gather of the same bytes with no GEMM at all (what the link delivers
        # when every GPU sends and receives at once, against the one-directional 770 GB/s the bound is computed from)
        ms_ag = None
        if 64 % world == 0:
            mine = Cfull[lo:hi]
            ms_ag = timed(lambda: dist.all_gather_into_tensor(Cfull.view(-1), mine.reshape(-1)))
        # the slower of the tensor-core time of the local GEMM and the NVLink time of the bytes each GPU must receive
        link_ms = recv / 770e9 * 1e3
        target = max(nb * 2 * 4096 ** 3 / (pk["bf16_tflops_sustained"] * 1e12) * 1e3, link_ms)
        res.update({"modes": modes, "best_mode": best, "ms_per_step": modes[best]["ms_per_step"], "tflops_total": modes[best]["tflops_total"],
                    "verified": not failed, "bytes_received_per_gpu": recv, "nvlink_ms_at_770GBs": link_ms, "roofline_target_ms": target,
                    "frac_of_roofline": target / modes[best]["ms_per_step"],
                    "ms_nccl_allgather_only": ms_ag, "nccl_allgather_only_ingest_gbs": (recv / ms_ag / 1e6) if ms_ag else None,
                    "collective": {"allgather": "ncclAllGather after the GEMM", "pipelined": "NCCL send/recv of chunk i under the GEMM of chunk i+1",
                                   "copy": "chunk i copied into every peer's C by the copy engines under the GEMM of chunk i+1, then a 4-byte all-reduce",
                                   "push": "GEMM epilogue stores each tile into every peer's C over NVLink, then a 4-byte all-reduce"}})
    del A, B, Cfull, scratch
    torch.cuda.empty_cache()
    if failed:
        if rank == 0:
            print(json.dumps({"sharded_bmm": res, "error": f"value check failed for {failed}"}), flush=True)
        raise SystemExit(f"sharded bmm: the value check failed for {failed}")
    return res


KERNEL_WORKLOADS = ("k_gemm4096", "k_gemm_mlp", "k_wgrad", "k_add", "k_exp", "k_sum", "k_argmax", "k_softmax", "k_rmsnorm", "k_layernorm",
                    "k_bn", "k_sort", "k_embedding", "k_xent", "k_scaled_mm")


def profile_kernels(args, dev):
    """--profile-run --workload k_*: warm-up + K launches of ONE kernel family at a size a profiler can capture (inputs
    beyond L2, a few GB at most), nothing else. Prints the algorithmic bytes / flops per launch so that a profile summary
    can put the counters next to them."""
    import torch
    from torchvulkan_b200 import cuda_ops as ops

    w = args.workload
    torch.manual_seed(0)
    h = torch.float16
    info = {}
    if w in ("k_gemm4096", "k_gemm_mlp", "k_wgrad"):
        m, n, k, ta, tb = {"k_gemm4096": (4096, 4096, 4096, False, False), "k_gemm_mlp": (256, 8192, 8192, False, True),
                           "k_wgrad": (8192, 8192, 256, True, False)}[w]
        a = torch.randn((k, m) if ta else (m, k), device=dev, dtype=h)
        b = torch.randn((n, k) if tb else (k, n), device=dev, dtype=h)
        A, B = (a.t() if ta else a), (b.t() if tb else b)
        out = torch.empty(m, n, device=dev, dtype=h)
        run = lambda: ops.gemm(A, B, out=out)  # noqa: E731
        info = {"flops": 2.0 * m * n * k, "bytes": 2.0 * (m * k + k * n + m * n), "shape": [m, n, k]}
    elif w == "k_scaled_mm":
        m = n = k = 8192                                              # float8 operands: 64 MiB each, bf16 result 128 MiB
        a = torch.randn(m, k, device=dev).to(torch.float8_e4m3fn)
        b = torch.randn(n, k, device=dev).to(torch.float8_e4m3fn).t()     # k contiguous: read in place by the float8 kernel
        sa, sb = torch.tensor(0.5, device=dev), torch.tensor(2.0, device=dev)
        out = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
        run = lambda: ops.scaled_mm(a, b, sa, sb, out=out)  # noqa: E731
        info = {"flops": 2.0 * m * n * k, "bytes": 1.0 * (m * k + k * n) + 2.0 * m * n, "shape": [m, n, k], "operands": "float8_e4m3fn", "result": "bf16"}
    elif w in ("k_add", "k_exp", "k_sum", "k_argmax"):
        n = 1 << 28          # 1 GiB per fp32 tensor: the code path of the 2^30 config at a quarter of its footprint
        x = torch.randn(n, device=dev)
        if w == "k_add":
            y, z = torch.randn(n, device=dev), torch.empty(n, device=dev)
            run, nbytes = (lambda: ops.binary("add", x, y, out=z)), 12 * n
        elif w == "k_exp":
            z = torch.empty(n, device=dev)
            run, nbytes = (lambda: ops.unary("exp", x, out=z)), 8 * n
        elif w == "k_sum":
            run, nbytes = (lambda: ops.reduce("sum", x)), 4 * n
        else:
            run, nbytes = (lambda: ops.argreduce(x)), 4 * n
        info = {"bytes": float(nbytes), "elements": n}
    elif w == "k_softmax":
        x = torch.randn(8192 * 128, 128, device=dev, dtype=h)         # the config-3 logits shape, 128x the rows (256 MiB: beyond L2)
        g = torch.randn_like(x)
        def run():
            yv = ops.softmax(x, log=True)
            ops.softmax_backward(g, yv, log=True)
        info = {"bytes_fwd": 2.0 * x.numel() * 2, "bytes_bwd": 3.0 * x.numel() * 2, "shape": list(x.shape)}
    elif w in ("k_rmsnorm", "k_layernorm"):
        x = torch.randn(8192 * 32, 512, device=dev, dtype=h)          # config-3 rows x32 (256 MiB: beyond L2)
        wt, g = torch.rand(512, device=dev, dtype=h) + 0.5, torch.randn_like(x)
        if w == "k_rmsnorm":
            def run():
                yv, rstd = ops.rmsnorm_forward(x, wt)
                ops.rmsnorm_backward(g, x, wt, rstd)
        else:
            bs = torch.randn(512, device=dev, dtype=h)
            def run():
                yv, mean, rstd = ops.layernorm_forward(x, wt, bs)
                ops.layernorm_backward(g, x, wt, mean, rstd)
        info = {"bytes_fwd": 2.0 * x.numel() * 2, "bytes_bwd": 3.0 * x.numel() * 2, "shape": list(x.shape)}
    elif w == "k_bn":
        x = torch.randn(256 * 8, 64, 32, 32, device=dev, dtype=h).contiguous(memory_format=torch.channels_last)   # config-4 stage 1, batch x8 (256 MiB: beyond L2)
        wt, bs = torch.rand(64, device=dev, dtype=h) + 0.5, torch.randn(64, device=dev, dtype=h)
        rm, rv = torch.zeros(64, device=dev, dtype=h), torch.ones(64, device=dev, dtype=h)
        g = torch.randn_like(x)
        def run():
            yv, mean, invstd = ops.batchnorm_forward(x, wt, bs, rm, rv)
            ops.batchnorm_backward(g, x, wt, mean, invstd)
        info = {"bytes_fwd": 3.0 * x.numel() * 2, "bytes_bwd": 5.0 * x.numel() * 2, "shape": list(x.shape), "layout": "channels_last"}
    elif w == "k_sort":
        x = torch.randn(4096, 8192, device=dev)
        run = lambda: ops.topk(x, 8192)  # noqa: E731
        info = {"bytes": 4.0 * x.numel() * 4, "shape": list(x.shape)}
    elif w == "k_embedding":
        table = torch.randn(128, 512, device=dev, dtype=h)
        idx = torch.randint(0, 128, (8192 * 32,), device=dev)
        g = torch.randn(8192 * 32, 512, device=dev, dtype=h)
        def run():
            ops.embedding_forward(table, idx)
            ops.embedding_backward(g, idx, 128)
        info = {"bytes_fwd": 2.0 * idx.numel() * 512, "bytes_bwd": 2.0 * idx.numel() * 512, "shape": [idx.numel(), 512]}
    else:   # k_xent
        x = torch.randn(8192 * 128, 128, device=dev, dtype=h)         # config-3 logits, 128x the rows (256 MiB: beyond L2)
        t = torch.randint(0, 128, (x.shape[0],), device=dev)
        one = torch.ones((), device=dev, dtype=h)
        def run():
            loss, total, lse = ops.cross_entropy_forward(x, t)
            ops.cross_entropy_backward(one, x, lse, t, None, "mean", -100, total)
        info = {"bytes_fwd": 1.0 * x.numel() * 2, "bytes_bwd": 2.0 * x.numel() * 2, "shape": list(x.shape)}
    for _ in range(args.warmup):
        run()
    # CUDA events around the K launch groups, on the stream the kernels are launched on (meaningless under a profiler)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)   # cuda_ops launches on torch's current stream
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.steps):
        run()
    e1.record()
    torch.cuda.synchronize()
    ops.check_device_status(dev.index or 0)
    print(json.dumps({"profile_run": True, "workload": w, "launch_groups": args.warmup + args.steps,
                      "event_us_per_group": round(e0.elapsed_time(e1) * 1e3 / max(args.steps, 1), 2), **info}), flush=True)


def profile_model_steps(args):
    """Warm-up + K steps of the config-3 / config-4 training script on the "vulkan" device, nothing else (for a profiler)."""
    import torch
    import torch.nn.functional as F

    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import models

    import torchvulkan

    vk = torch.device("vulkan:0")
    torch.manual_seed(0)
    if args.workload == "c3":
        model = models.Decoder(vocab=128, seq=256, layers=6, width=512, heads=8, kv_heads=2, hidden=1376).half().to(vk)
        ids, tgt = torch.randint(0, 128, (32, 256)).to(vk), torch.randint(0, 128, (32 * 256,)).to(vk)
        opt = torch.optim.AdamW(model.parameters(), lr=1e-3 / 4096.0, fused=True)
        loss_fn = lambda: F.cross_entropy(model(ids).view(-1, 128), tgt) * 4096.0  # noqa: E731
    else:
        model = models.SmallResNet(64).half().to(vk)
        x, y = torch.randn(256, 3, 32, 32).half().to(vk), torch.randint(0, 10, (256,)).to(vk)
        if args.workload == "c4cl":
            model, x = model.to(memory_format=torch.channels_last), x.contiguous(memory_format=torch.channels_last)
        opt = torch.optim.SGD(model.parameters(), lr=0.1 / 1024.0, momentum=0.9)
        loss_fn = lambda: F.cross_entropy(model(x), y) * 1024.0  # noqa: E731
    for _ in range(args.warmup + args.steps):
        opt.zero_grad(set_to_none=True)
        loss_fn().backward()
        opt.step()
    torchvulkan.synchronize()
    print(json.dumps({"profile_run": True, "workload": args.workload, "steps": args.steps}), flush=True)


def run_model_steps(args):
    """BASELINE configs 2, 3 and 4 as a user runs them: a torch script on the "vulkan" device (fwd + bwd + optimizer step),
    timed like the reference's benchmark (warm-up 3, median of 10, zero_grad(set_to_none=True), device synchronize on
    both sides, wall clock), beside the same script in fp32 on ATen CPU (1 warm-up + 2 timed steps)."""
    import torch
    import torch.nn.functional as F

    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import models  # the three example architectures at the BASELINE sizes

    import torchvulkan

    vk = torch.device("vulkan:0")
    out = {}

    def time_script(model, make_loss, opt, sync, reps, warm, read_loss=False):
        times = []
        for i in range(warm + reps):
            sync()
            t0 = time.perf_counter()
            opt.zero_grad(set_to_none=True)
            loss = make_loss(model)
            loss.backward()
            opt.step()
            if read_loss:
                loss.item()               # the device -> host read of the step's result, inside the timed region
            sync()
            if i >= warm:
                times.append(time.perf_counter() - t0)
        return statistics.median(times) * 1e3, float(loss.item())

    torch.manual_seed(0)
    ids, tgt = torch.randint(0, 128, (32, 256)), torch.randint(0, 128, (32 * 256,))
    xr, yr = torch.randn(256, 3, 32, 32), torch.randint(0, 10, (256,))
    xm, ym = torch.randn(BATCH, SIZES[0]), torch.randint(0, SIZES[-1], (BATCH,))
    mlp_loss = lambda m, d, half, t=(xm, ym): F.cross_entropy(m((t[0].half() if half else t[0]).to(d)), t[1].to(d)) * (LOSS_SCALE if half else 1.0)  # noqa: E731
    cfgs = {
        # config 2 as the reference's example script runs it (examples/mlp.py:36-47): inputs moved to the device every step,
        # AdamW(lr=1e-3, weight_decay=1e-2) with torch.optim's default (foreach) implementation, the loss read back
        "c2_mlp_step_default_adamw": (lambda: models.mlp(SIZES), mlp_loss,
                                      lambda ps, half: torch.optim.AdamW(ps, lr=1e-3, weight_decay=1e-2, eps=ADAM_EPS if half else 1e-8), float(gemm_flops())),
        # the same with AdamW(fused=True): one list launch, step count on the device, so the step can also be replayed
        "c2_mlp_step": (lambda: models.mlp(SIZES), mlp_loss,
                        lambda ps, half: torch.optim.AdamW(ps, lr=1e-3, weight_decay=1e-2, eps=ADAM_EPS if half else 1e-8, fused=half), float(gemm_flops())),
        "c3_decoder_step": (lambda: models.Decoder(vocab=128, seq=256, layers=6, width=512, heads=8, kv_heads=2, hidden=1376),
                            lambda m, d, half, t=(ids, tgt): F.cross_entropy(m(t[0].to(d)).view(-1, 128), t[1].to(d)) * (4096.0 if half else 1.0),
                            lambda ps, half: torch.optim.AdamW(ps, lr=1e-3 / (4096.0 if half else 1.0), fused=half), 865e9),
        "c4_resnet_step": (lambda: models.SmallResNet(64),
                           lambda m, d, half, t=(xr, yr): F.cross_entropy(m((t[0].half() if half else t[0]).to(d)), t[1].to(d)) * (1024.0 if half else 1.0),
                           lambda ps, half: torch.optim.SGD(ps, lr=0.1 / (1024.0 if half else 1.0), momentum=0.9), 646e9),
    }
    # the ResNet again with the model and its input in torch.channels_last memory: the layout the convolution and
    # batch-norm kernels read and write in place (same arithmetic, no NCHW <-> NHWC staging copies)
    xr_cl = xr.half().contiguous(memory_format=torch.channels_last)
    cfgs["c4_resnet_step_channels_last"] = (lambda: models.SmallResNet(64).to(memory_format=torch.channels_last),
                                            lambda m, d, half, t=(xr_cl, yr): F.cross_entropy(m((t[0] if half else t[0].float().contiguous()).to(d)), t[1].to(d)) * (1024.0 if half else 1.0),
                                            cfgs["c4_resnet_step"][2], 646e9)
    # and once more with SGD(fused=True): one list launch for the whole optimizer step instead of torch.optim's default
    # three foreach passes (the reference's examples use the default, so that stays the headline variant)
    cfgs["c4_resnet_step_channels_last_fused_sgd"] = (cfgs["c4_resnet_step_channels_last"][0], cfgs["c4_resnet_step_channels_last"][1],
                                                      lambda ps, half: torch.optim.SGD(ps, lr=0.1 / (1024.0 if half else 1.0), momentum=0.9, fused=True), 646e9)
    for name, (make, loss_fn, make_opt, flops) in cfgs.items():
        torch.manual_seed(0)
        model = make().half().to(vk)
        if "channels_last" in name:
            model = model.to(memory_format=torch.channels_last)
        opt = make_opt(model.parameters(), True)
        ms, loss = time_script(model, lambda m: loss_fn(m, vk, True), opt, torchvulkan.synchronize, 10, 3, read_loss=True)
        scale = LOSS_SCALE if name.startswith("c2_") else (4096.0 if name.startswith("c3_") else 1024.0)
        rec = {"ms_per_step": ms, "tflops_algorithmic": flops / ms / 1e9, "loss": loss / scale, "loss_scale": scale, "dtype": "f16",
               "api": "torch script on the vulkan device: host inputs .to(device) and loss.item() every step",
               "protocol": "warm-up 3, median of 10, wall clock with a device synchronize on both sides"}
        # The same step captured once with torchvulkan.Graph and replayed (inputs resident on the device): what the step
        # costs the GPU when the host's per-operator dispatch is out of the way.
        try:
            if name.endswith("default_adamw"):
                raise RuntimeError("not replayable: torch.optim's foreach AdamW keeps its step count on the host")
            host_inputs = loss_fn.__defaults__[0]
            dev_inputs = tuple((t.half() if t.is_floating_point() else t).to(vk) for t in host_inputs)
            if "channels_last" in name:
                dev_inputs = (dev_inputs[0].contiguous(memory_format=torch.channels_last),) + dev_inputs[1:]

            def graph_step():
                opt.zero_grad(set_to_none=True)
                l = loss_fn(model, vk, True, dev_inputs)       # .to(device) of a resident tensor is the tensor itself
                l.backward()
                opt.step()
                return l

            graph_step()                                  # one more eager step, now on the resident inputs
            g = torchvulkan.Graph()
            with g.capture():
                gl = graph_step()
            for _ in range(3):
                g.replay()
            torchvulkan.synchronize()
            t0 = time.perf_counter()
            for _ in range(20):
                g.replay()
            torchvulkan.synchronize()
            gms = (time.perf_counter() - t0) / 20 * 1e3
            rec["graph_replay"] = {"ms_per_step": gms, "tflops_algorithmic": flops / gms / 1e9, "loss": float(gl.item()) / scale,
                                   "protocol": "torchvulkan.Graph: warm-up 3, mean of 20 replays, wall clock with a device synchronize on both sides"}
            g.reset()
        except Exception as e:  # noqa: BLE001
            rec["graph_replay"] = {"unavailable": str(e).splitlines()[0][:200]}
        if "channels_last" in name or name.startswith("c2_"):
            out[name] = rec            # (config 2's CPU leg is the line's cpu_baseline)
            del model
            continue
        if not args.no_cpu_baseline:
            torch.manual_seed(0)
            cpu_model = make()
            torch.set_num_threads(os.cpu_count() or 1)
            cms, closs = time_script(cpu_model, lambda m: loss_fn(m, "cpu", False), make_opt(cpu_model.parameters(), False), lambda: None, 2, 1)
            rec["cpu_fp32_ms_per_step"] = cms
            rec["cpu_cores"] = torch.get_num_threads()
        out[name] = rec
        del model
    return out


def count_kernels(run_step, api_calls):
    """Kernels one step launches, counted from the profiler's record of one eager step (a C-ABI call may launch two or
    three: a split-K product is slices + fold, a repacked operand adds a copy). Falls back to the number of C-ABI calls
    when no kernel activity is recorded."""
    try:
        import torch
        from torch.profiler import ProfilerActivity, profile
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            run_step()
            torch.cuda.synchronize()
        n = sum(1 for e in prof.events() if str(e.device_type).endswith("CUDA") and not e.name.lower().startswith(("memcpy", "memset")))
        if n < api_calls:
            print(f"bench: the profiler recorded {n} kernels for {api_calls} C-ABI calls; counting the calls", file=sys.stderr)
        return n if n >= api_calls else api_calls
    except Exception as e:  # noqa: BLE001
        print(f"bench: kernel count from the profiler unavailable ({type(e).__name__}: {e}); counting C-ABI calls", file=sys.stderr)
        return api_calls


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-configs", action="store_true", help="leave out the `configs` key (BASELINE configs 1, 3, 4, 5(ii) and the vulkan-device scripts)")
    ap.add_argument("--extras", action="store_true", help="accepted for compatibility: the other configs are part of the default line now")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profile-run", action="store_true", help="only warm-up + K device-resident steps (for ncu)")
    ap.add_argument("--workload", default="c2", choices=["c2", "c3", "c4", "c4cl", *KERNEL_WORKLOADS],
                    help="with --profile-run: which BASELINE config's step to run (c4cl: config 4 in channels-last memory), or one "
                         "kernel family alone (k_*)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
