#!/usr/bin/env python
"""Benchmark of the causal linear-attention hot path: causal_dot_product forward+backward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config 2] [--mode fp32|mma]
    python bench.py --impl reference ...      # the reference's CPU kernel on the host cores

One "step" is one forward + backward of ``causal_dot_product`` over the (batch, head)
units one GPU holds.  The default workload is configuration 2 (B8 H8 L4096 D=M=64, fp32,
Q,K = elu(x)+1, V,G ~ N(0,1), seeded synthetic data).  With N > 1 every rank holds its own
B=8 slice of a global batch of 8N (the (batch, head) units are independent, so there is no
data-path collective): weak scaling.  Metric: Mtokens/s, tokens = batch * sequence length.

Printed by rank 0: ONE JSON line.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "causal linear-attn fwd+bwd Mtokens/s"
UNIT = "Mtokens/s"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=2, choices=[1, 2, 3, 4, 5])
    ap.add_argument("--recurrent", action="store_true",
                    help="time the recurrent step (decode) instead of the batch product: "
                         "N256 H16 D=M=128 fp32, one token per sequence and step")
    ap.add_argument("--mode", default="mma", choices=["fp32", "mma", "tf32x3"],
                    help="arithmetic of the kernels: tensor cores (TF32 operands for fp32 tensors, "
                         "bf16 for bf16; <= 2e-2 vs fp64), fp32 CUDA cores (<= 1e-5), or tensor cores "
                         "with split TF32 operands, three products each (<= 1e-5; fp32, D = M = 64)")
    ap.add_argument("--L", type=int, default=None, help="override the sequence length")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-other-mode", action="store_true",
                    help="skip the few eager steps in the other arithmetic mode")
    ap.add_argument("--no-graph", action="store_true", help="time eager calls, not a CUDA graph")
    ap.add_argument("--exchange", choices=["auto", "nccl", "peer"], default="auto",
                    help="the sequence split on several GPUs: how the per-rank states travel (NCCL "
                         "all_gather, or stores into the peers' buffers by this library's own kernels; "
                         "auto = peer memory with the step in a CUDA graph, falling back to eager and "
                         "then to NCCL if that fails; with --config 4 auto means nccl)")
    ap.add_argument("--sp-graph", action="store_true",
                    help="with --exchange peer: capture the sequence-parallel step in a CUDA graph")
    ap.add_argument("--graph-steps", type=int, default=0,
                    help="steps captured per CUDA graph (default: the largest divisor of --steps that keeps "
                         "the graph under about 8 ms, at most 10)")
    ap.add_argument("--no-extra", action="store_true",
                    help="skip the additional records of a default run: on one GPU configs 1, 4 and 5 "
                         "(`configs`), on several GPUs config 4 with the sequence split over the ranks "
                         "(`sequence_parallel`)")
    ap.add_argument("--layers", type=int, default=None, help="config 3: override the layer count")
    ap.add_argument("--batch", type=int, default=None, help="config 3: override the batch size")
    return ap.parse_args()


def workload_name(cfg, shape):
    return "config%d causal_dot_product fwd+bwd N%d H%d L%d D%d M%d %s" % (
        cfg, shape["N"], shape["H"], shape["L"], shape["D"], shape["M"],
        str(shape["dtype"]).replace("torch.", ""))


# ------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi polled every 100 ms in a child process while the timed region runs.  A region of a
    few milliseconds is over before the first sample arrives: `keep_loaded` then repeats the same
    work, untimed, until a few samples have been taken under that load."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.proc, self.lines = None, []
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(index), "--query-gpu=" + self.FIELDS,
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True, bufsize=1)
        except OSError:
            self.proc = None
            return
        import threading
        self.reader = threading.Thread(target=self._read, daemon=True)
        self.reader.start()

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line)

    def samples(self):
        return sum(1 for line in list(self.lines) if len(line.split(",")) >= 7)

    def keep_loaded(self, work, want=3, budget_s=2.0):
        """Run `work()` (the timed region's own launches, untimed now) until `want` samples exist."""
        if self.proc is None:
            return
        t0 = time.time()
        while self.samples() < want and time.time() - t0 < budget_s:
            work()
            torch.cuda.synchronize()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.reader.join(timeout=5)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in list(self.lines):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm),
                "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------
# CPU arm (the reference's own OpenMP kernel, or the C port when it is not built)
# ------------------------------------------------------------------------------------------
def use_all_host_threads():
    """OpenMP threads for the CPU arm: every core this process may run on.  A launcher that
    exports OMP_NUM_THREADS=1 for its ranks (torch.distributed.run does) would otherwise pin the
    reference's OpenMP kernel to one thread."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(n)
    return n


def cpu_arm(Q, K, V, G, budget_s, min_steps=2, max_steps=1000, warmup=1):
    """fwd+bwd of the CPU implementation on the host cores; returns (seconds per step,
    kind, cores, steps timed)."""
    from oracle import causal_oracle as orc
    kind = "reference" if orc.reference_ext() is not None else "port"
    threads = use_all_host_threads()
    Q, K, V, G = (t.float().contiguous() for t in (Q, K, V, G))
    if kind == "reference":
        def step():
            orc.reference_forward(Q, K, V)
            orc.reference_backward(Q, K, V, G)
    else:
        def step():
            orc.c_forward(Q, K, V)
            orc.c_backward(Q, K, V, G)
    for _ in range(warmup):
        step()
    times = []
    t_end = time.perf_counter() + budget_s
    while len(times) < max_steps and (len(times) < min_steps or time.perf_counter() < t_end):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    cores = threads if kind == "reference" else 1
    return statistics.median(times), kind, cores, len(times)


def run_reference(args, shape, inputs, name):
    Q, K, V, G = inputs
    tokens = shape["N"] * shape["L"]
    from oracle import causal_oracle as orc
    kind = "reference" if orc.reference_ext() is not None else "port"
    threads = use_all_host_threads()
    Qf, Kf, Vf, Gf = (t.float().contiguous() for t in (Q, K, V, G))

    def step():
        if kind == "reference":
            orc.reference_forward(Qf, Kf, Vf)
            orc.reference_backward(Qf, Kf, Vf, Gf)
        else:
            orc.c_forward(Qf, Kf, Vf)
            orc.c_backward(Qf, Kf, Vf, Gf)

    for _ in range(max(1, min(args.warmup, 3))):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    cores = threads if kind == "reference" else 1
    value = tokens / dt / 1e6
    sample = "%d steps of the full workload (%s), fp32, all (batch, head) units" % (args.steps, name)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic (seeded)",
        "config": {"workload": name, "device": "host CPU",
                   "parallel_units": shape["N"] * shape["H"]},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind,
                         "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------
# config 3: the 16-layer causal-linear encoder built by TransformerEncoderBuilder
# ------------------------------------------------------------------------------------------
def run_encoder(args):
    """Forward + backward of the encoder (16 layers, 8 heads x 64, FFN 2048, elu+1 feature map,
    random-init weights, dropout 0) on X~U[0,1) of shape (16, 8192, 512), fp32, with a causal
    mask.  Data parallel over ranks (each rank its own batch; no gradient all-reduce is timed:
    the metric is the attention path inside a model, not an optimiser step)."""
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    import fast_transformers_b200 as ftb
    from fast_transformers_b200 import _native, workloads
    from fast_transformers_b200.builders import TransformerEncoderBuilder
    from fast_transformers_b200.masking import LengthMask, TriangularCausalMask
    lib = _native.lib()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    mode = args.mode or ftb.get_mode()
    # In "mma" mode the attention runs TF32 tensor-core MMAs; the Linear layers (torch GEMMs)
    # get the same arithmetic through torch's own switch, otherwise true-fp32 GEMMs dominate.
    torch.backends.cuda.matmul.allow_tf32 = mode == "mma"
    cfg = dict(workloads.ENCODER)
    if args.layers:
        cfg["n_layers"] = args.layers
    io = dict(workloads.ENCODER_INPUT)
    if args.batch:
        io["N"] = args.batch
    if args.L:
        io["L"] = args.L
    torch.manual_seed(3000 + rank)
    model = TransformerEncoderBuilder.from_kwargs(**cfg).get().to(dev)
    gen = workloads.generator(3, rank)
    X = torch.rand(io["N"], io["L"], io["d_model"], generator=gen)
    W = torch.randn(io["N"], io["L"], io["d_model"], generator=gen)
    Xp = X.pin_memory()
    Xd, Wd = X.to(dev), W.to(dev)
    mask = TriangularCausalMask(io["L"], device=dev)
    lengths = LengthMask(torch.full((io["N"],), io["L"], dtype=torch.int64, device=dev), max_len=io["L"])
    tokens = io["N"] * io["L"]

    def step(x):
        model.zero_grad(set_to_none=True)
        with ftb.mode(mode):
            y = model(x, attn_mask=mask, length_mask=lengths)
            loss = (y * Wd).sum()
            loss.backward()
        return loss

    for _ in range(max(args.warmup, 3)):
        step(Xd)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    n0 = lib.ftb_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step(Xd)
    e1.record()
    torch.cuda.synchronize()
    launches = lib.ftb_launch_count() - n0
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = t.item() / args.steps
    clocks = sampler.stop() if sampler else None
    # device time of this library's kernels inside one step (events around every launch)
    lib.ftb_timing_enable(1)
    step(Xd)
    torch.cuda.synchronize()
    kinds = _native.timing_read()
    lib.ftb_timing_enable(0)
    # end to end: the input comes from pinned host memory, the loss goes back to the host
    xd = torch.empty_like(Xd)
    e0.record()
    n_e2e = max(2, min(args.steps, 5))
    for _ in range(n_e2e):
        xd.copy_(Xp, non_blocking=True)
        loss = step(xd)
        loss.item()
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1) / n_e2e
    if rank == 0:
        H, D = cfg["n_heads"], cfg["query_dimensions"]
        attn_bytes = workloads.algorithmic_bytes(D, D, 4) * tokens * H * cfg["n_layers"]
        print(json.dumps({
            "metric": METRIC, "value": world * tokens / (ms_step * 1e-3) / 1e6, "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": {"fp32": "f32", "mma": "tf32", "tf32x3": "tf32x3"}[mode],
            "data": "synthetic (seeded), random-init weights, dropout 0 (builder default 0.1)",
            "config": {"workload": "config3 causal-linear encoder fwd+bwd %d layers H%d d%d FFN%d "
                                   "X(%d,%d,%d) float32" % (cfg["n_layers"], H, D,
                                                            cfg["feed_forward_dimensions"],
                                                            io["N"], io["L"], io["d_model"]),
                       "mode": mode, "global_batch": io["N"] * world, "cuda_graph": False,
                       "linear_layers": "torch GEMMs, allow_tf32=%s" % (mode == "mma"),
                       "l2": "activations per step far exceed the 126 MB L2; no flush"},
            "roofline": {"bound": "hbm", "kernel": "whole model (GEMMs dominate)", "achieved": None,
                         "peak": None, "unit": "GB/s", "frac": None, "traffic": None,
                         "attention_algorithmic_bytes": attn_bytes,
                         "attention_kernels_ms_per_step": {k: v[0] for k, v in kinds.items()},
                         "attention_kernels_share_of_step": sum(v[0] for v in kinds.values()) / ms_step},
            "cpu_baseline": None,
            "e2e": {"value": world * tokens / (e2e_ms * 1e-3) / 1e6, "unit": UNIT,
                    "h2d_bytes_per_step": X.numel() * 4, "d2h_bytes_per_step": 4,
                    "ms_per_step": e2e_ms, "steps": n_e2e},
            "gpu_launches": int(launches), "clocks": clocks}))
    if dist is not None:
        dist.destroy_process_group()
    return 0


# ------------------------------------------------------------------------------------------
# The recurrent step (the same attention as a fixed-state recurrent model, one token per call)
# ------------------------------------------------------------------------------------------
def run_recurrent(args):
    """Decode steps of RecurrentLinearAttention: N sequences advance by one token per step.
    The state (N,H,D,M fp32 = 268 MB here, larger than L2) is read and written once per step,
    which is the algorithmic traffic: 2*D*M*4 bytes per (sequence, head)."""
    N, H, D, M = 256, 16, 128, 128
    unit = "Mtokens/s"
    name = "recurrent linear-attn step N%d H%d D%d M%d float32 (one token per sequence and step)" % (N, H, D, M)
    gq = torch.Generator().manual_seed(6000)
    q, k = (torch.randn(N, H, D, generator=gq) for _ in range(2))
    v = torch.randn(N, H, M, generator=gq)
    if args.impl == "reference":
        from oracle import causal_oracle as orc
        threads = use_all_host_threads()
        state = None
        for _ in range(max(1, min(args.warmup, 2))):
            _, state = orc.recurrent_step(q, k, v, state, dtype=torch.float32)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            _, state = orc.recurrent_step(q, k, v, state, dtype=torch.float32)
        dt = (time.perf_counter() - t0) / args.steps
        value = N / dt / 1e6
        print(json.dumps({
            "impl": "reference", "metric": "recurrent linear-attn step Mtokens/s", "value": value,
            "unit": unit, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic (seeded)", "config": {"workload": name, "device": "host CPU"},
            "cpu_baseline": {"value": value, "unit": unit, "cores": threads, "kind": "port",
                             "sample": "%d steps; the reference module's torch arithmetic restated "
                                       "(oracle.recurrent_step, fp32)" % args.steps},
            "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}))
        return 0
    import fast_transformers_b200 as ftb  # noqa: F401
    from fast_transformers_b200 import _native
    from fast_transformers_b200.recurrent.attention import RecurrentLinearAttention
    lib = _native.lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    torch.set_grad_enabled(False)
    qd, kd, vd = (t.to(dev) for t in (q, k, v))
    att = RecurrentLinearAttention(D)
    _, state = att(qd, kd, vd)
    per_graph = 10
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(per_graph):
            y, state = att(qd, kd, vd, state)
    for _ in range(max(3, args.warmup)):
        graph.replay()
    sampler = ClockSampler(0)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.steps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    sampler.keep_loaded(graph.replay)
    clocks = sampler.stop()
    ms_step = e0.elapsed_time(e1) / (args.steps * per_graph)
    launches = args.steps * per_graph
    alg_bytes = N * H * (2 * D * M + 3 * D + 2 * D + 2 * M) * 4
    peaks = {}
    ppath = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(ppath):
        peaks = json.load(open(ppath))
    peak = peaks.get("hbm_gbs", 6650.0)
    achieved = alg_bytes / (ms_step * 1e-3) / 1e9
    # end to end: the step's inputs from pinned host memory, its output back
    pin = [t.pin_memory() for t in (q, k, v)]
    hout = torch.empty(N, H, M).pin_memory()
    for _ in range(3):
        for d_, h_ in zip((qd, kd, vd), pin):
            d_.copy_(h_, non_blocking=True)
        y, state = att(qd, kd, vd, state)
        hout.copy_(y, non_blocking=True)
    torch.cuda.synchronize()
    e0.record()
    n_e2e = 50
    for _ in range(n_e2e):
        for d_, h_ in zip((qd, kd, vd), pin):
            d_.copy_(h_, non_blocking=True)
        y, state = att(qd, kd, vd, state)
        hout.copy_(y, non_blocking=True)
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1) / n_e2e
    # CPU baseline: the reference module's arithmetic restated, fp32, on the host cores
    from oracle import causal_oracle as orc
    threads = use_all_host_threads()
    cstate = None
    _, cstate = orc.recurrent_step(q, k, v, cstate, dtype=torch.float32)
    t0 = time.perf_counter()
    n_cpu = 5
    for _ in range(n_cpu):
        _, cstate = orc.recurrent_step(q, k, v, cstate, dtype=torch.float32)
    cpu_dt = (time.perf_counter() - t0) / n_cpu
    print(json.dumps({
        "metric": "recurrent linear-attn step Mtokens/s", "value": N / (ms_step * 1e-3) / 1e6, "unit": unit,
        "n_gpus": 1, "steps": args.steps * per_graph, "warmup": max(3, args.warmup) * per_graph,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic (seeded)",
        "config": {"workload": name, "cuda_graph": True,
                   "l2": "the state (%d MB) exceeds the 126 MB L2; no flush" % (N * H * D * M * 4 // 2 ** 20)},
        "roofline": {"bound": "hbm", "kernel": "recurrent_step", "achieved": achieved, "peak": peak,
                     "unit": "GB/s", "frac": achieved / peak, "traffic": None,
                     "algorithmic_bytes_per_launch": alg_bytes, "avg_launch_ms": ms_step},
        "cpu_baseline": {"value": N / cpu_dt / 1e6, "unit": unit, "cores": threads, "kind": "port",
                         "sample": "%d steps; the reference module's torch arithmetic restated "
                                   "(oracle.recurrent_step, fp32)" % n_cpu},
        "e2e": {"value": N / (e2e_ms * 1e-3) / 1e6, "unit": unit,
                "h2d_bytes_per_step": sum(t.numel() * 4 for t in pin), "d2h_bytes_per_step": hout.numel() * 4,
                "ms_per_step": e2e_ms, "steps": n_e2e,
                "api": "RecurrentLinearAttention.forward with the step's q, k, v copied in from pinned "
                       "host memory and its output copied out"},
        "gpu_launches": launches, "clocks": clocks}))
    return 0



# ------------------------------------------------------------------------------------------
# helpers shared by the legs of the GPU arm
# ------------------------------------------------------------------------------------------
def hbm_peak():
    """(GB/s, where the figure comes from)"""
    ppath = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(ppath):
        peaks = json.load(open(ppath))
        if "hbm_gbs" in peaks:
            return float(peaks["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback 6650 GB/s"


def time_steps(step, steps, warmup, dev, dist=None, graph_steps=0):
    """Device time per step of ``step()`` (CUDA events on the current stream, max over ranks):
    ``warmup`` untimed steps, then ``steps`` timed ones; with ``graph_steps`` > 0 that many steps
    are captured into one CUDA graph which is replayed ``steps // graph_steps`` times."""
    for _ in range(max(warmup, 3)):
        step()
    torch.cuda.synchronize()
    graph = None
    if graph_steps:
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            step()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(graph_steps):
                step()
        for _ in range(3):
            graph.replay()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    if graph is not None:
        n = max(1, steps // graph_steps)
        for _ in range(n):
            graph.replay()
        done = n * graph_steps
    else:
        for _ in range(steps):
            step()
        done = steps
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / done], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.barrier()
    return t.item()


def oracle_errors(Q, K, V, G, got, heads, chunk=512):
    """max|x - x64| / max|x64| of (out, gQ, gK, gV) on the (batch 0) heads ``heads`` against the
    fp64 blocked recurrence on the host (every core: a launcher may have set OMP_NUM_THREADS=1)."""
    from oracle import causal_oracle as orc
    use_all_host_threads()
    errs = dict.fromkeys(("out", "gQ", "gK", "gV"), 0.0)
    for i, h in enumerate(heads):
        sub = [t[:1, h:h + 1].float().cpu() for t in (Q, K, V, G)]
        want = (orc.chunked_forward(*sub[:3], chunk=chunk),) + tuple(orc.chunked_backward(*sub, chunk=chunk))
        for name, a, b in zip(errs, got, want):
            errs[name] = max(errs[name], orc.rel_err(a[:1, i:i + 1], b))
    return errs


def product_record(cfg, mode, dev, steps, heads=None, trial=0):
    """One more configuration on this GPU: device-resident fwd+bwd through the autograd Function,
    captured in a CUDA graph; with ``heads`` also the error of those heads against the fp64 oracle."""
    import fast_transformers_b200 as ftb
    from fast_transformers_b200 import workloads
    from fast_transformers_b200.causal_product import causal_dot_product
    shape = workloads.SHAPES[cfg]
    Q, K, V, G = workloads.make_inputs(cfg, trial=trial)
    Qd, Kd, Vd, Gd = (t.to(dev) for t in (Q, K, V, G))
    Qd.requires_grad_(True), Kd.requires_grad_(True), Vd.requires_grad_(True)
    last = {}

    def step():
        Qd.grad = Kd.grad = Vd.grad = None
        with ftb.mode(mode):
            out = causal_dot_product(Qd, Kd, Vd)
            out.backward(Gd)
        last["out"] = out.detach()   # (not `out`: it would keep the autograd graph of the step alive)

    step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    step()
    e1.record()
    torch.cuda.synchronize()
    per_graph = max(1, min(10, int(8.0 / max(e0.elapsed_time(e1), 1e-3))))
    n = max(steps, per_graph) // per_graph * per_graph
    ms = time_steps(step, n, 3, dev, graph_steps=per_graph)
    token_heads = shape["N"] * shape["H"] * shape["L"]
    alg = workloads.algorithmic_bytes(shape["D"], shape["M"], Qd.element_size()) * token_heads
    peak, _ = hbm_peak()
    rec = {"workload": workload_name(cfg, shape), "mode": mode, "ms_per_step": ms,
           "value": shape["N"] * shape["L"] / (ms * 1e-3) / 1e6, "unit": UNIT,
           "steps": n, "steps_per_graph": per_graph, "algorithmic_bytes": alg,
           "achieved_GBps": alg / (ms * 1e-3) / 1e9, "frac_of_hbm_peak": alg / (ms * 1e-3) / 1e9 / peak}
    if heads:
        got = [t[:1, heads].detach() for t in (last["out"], Qd.grad, Kd.grad, Vd.grad)]
        rec["rel_err_vs_fp64"] = oracle_errors(Q, K, V, G, got, heads)
        rec["rel_err_heads"] = list(heads)
        rec["tolerance_vs_fp64"] = 2e-2 if mode == "mma" else 1e-5
    return rec


def sequence_parallel_record(args, dev, dist, rank, world, mode, lib):
    """Config 4 (ONE sequence of 262 144 positions, 16 heads, D = M = 128, bf16) with the sequence
    split over the ranks: every rank holds L / world positions, one exchange of the (N,H,D,M)
    fp32 states per direction.  Reports the time of the split step (max over ranks), the time of
    the SAME whole sequence on rank 0 alone in this process, the efficiency t1 / (world * tN), and
    the error of two heads against the fp64 oracle of the whole sequence."""
    import fast_transformers_b200 as ftb
    from fast_transformers_b200 import workloads
    from fast_transformers_b200.causal_product import causal_dot_product
    from fast_transformers_b200.sequence_parallel import (LocalOps, PeerExchange,
                                                          sequence_parallel_causal_dot_product)
    shape = dict(workloads.SHAPES[4])
    L = shape["L"]
    if L % world:
        return {"skipped": "sequence length %d does not divide over %d ranks" % (L, world)}
    Lr = L // world
    Q, K, V, G = (t.to(dev) for t in workloads.make_inputs(4, trial=rank, scale_L=Lr))
    Q.requires_grad_(True), K.requires_grad_(True), V.requires_grad_(True)
    ops = LocalOps(mode)
    last = {}
    steps = max(args.steps, 10)

    def attempt(use_peer, use_graph):
        """Time the split step one way; returns (exchange, ms per step, steps per graph, error)."""
        exchange = PeerExchange((shape["N"], shape["H"], shape["D"], shape["M"])) if use_peer else None

        def step():
            Q.grad = K.grad = V.grad = None
            with ftb.mode(mode):
                out = sequence_parallel_causal_dot_product(Q, K, V, ops=ops, exchange=exchange)
                out.backward(G)
            last["out"] = out.detach()   # (not `out`: it would keep the autograd graph of the step alive)

        graph_steps, why, tN = 0, None, float("nan")
        try:
            step()
            if exchange is not None:
                exchange.check()
            if use_graph:
                # as many steps per graph as keep it under about 8 ms (longer graphs ran slower per
                # step), the same number on every rank
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                step()
                e1.record()
                torch.cuda.synchronize()
                most = torch.tensor([max(1, min(10, int(8.0 / max(e0.elapsed_time(e1), 1e-3))))], device=dev)
                dist.all_reduce(most, op=dist.ReduceOp.MIN)
                graph_steps = next(d for d in range(int(most.item()), 0, -1) if steps % d == 0)
            tN = time_steps(step, steps, 3, dev, dist, graph_steps=graph_steps)
            if exchange is not None:
                exchange.check()        # a receive that gave up waiting leaves NaN and a status word
            else:
                ftb.check_device_status(dev)
        except Exception as e:          # reported, not hidden
            why = "%s: %s" % (type(e).__name__, e)
        flag = torch.tensor([0 if why is None else 1], device=dev)
        dist.all_reduce(flag)
        if flag.item():
            why = why or "another rank failed"
        return exchange, tN, graph_steps, why

    # --exchange auto (the default): the peer-memory exchange with the step captured in a CUDA graph;
    # should that fail on this machine (a wait that ran out, a refused capture), the same step eager,
    # then over NCCL's all_gather.  Every attempt is listed in the record.
    if args.exchange == "peer":
        plan = [(True, bool(args.sp_graph))]
    elif args.exchange == "nccl":
        plan = [(False, False)]
    else:
        plan = [(True, True), (True, False), (False, False)]
    attempts, exchange, tN, graph_steps = [], None, float("nan"), 0
    for use_peer, use_graph in plan:
        exchange, tN, graph_steps, why = attempt(use_peer, use_graph)
        attempts.append({"exchange": "peer" if use_peer else "nccl", "cuda_graph": use_graph,
                         "ms_per_step": None if why else tN, "error": why})
        if why is None:
            break
        if exchange is not None:
            exchange.close()
        exchange = None
    if attempts[-1]["error"] is not None:
        return {"valid": False, "attempts": attempts}

    # the whole sequence on rank 0: inputs and the split results of two heads
    heads = [0, 11]
    full, got = None, None
    gathered = []
    for t in (Q.detach(), K.detach(), V.detach(), G):
        parts = [torch.empty_like(t) for _ in range(world)] if rank == 0 else None
        dist.gather(t.contiguous(), parts, dst=0)
        gathered.append(torch.cat(parts, dim=2) if rank == 0 else None)
    split = []
    for t in (last["out"].detach(), Q.grad, K.grad, V.grad):
        piece = t[:, heads].contiguous()
        parts = [torch.empty_like(piece) for _ in range(world)] if rank == 0 else None
        dist.gather(piece, parts, dst=0)
        split.append(torch.cat(parts, dim=2) if rank == 0 else None)
    rec = None
    if rank == 0:
        Qf, Kf, Vf, Gf = gathered
        Qf.requires_grad_(True), Kf.requires_grad_(True), Vf.requires_grad_(True)

        def whole():
            Qf.grad = Kf.grad = Vf.grad = None
            with ftb.mode(mode):
                causal_dot_product(Qf, Kf, Vf).backward(Gf)

        t1 = time_steps(whole, 6, 3, dev, graph_steps=2)
        errs = oracle_errors(Qf.detach(), Kf.detach(), Vf.detach(), Gf, split, heads)
        token_heads = shape["N"] * shape["H"] * L
        alg = workloads.algorithmic_bytes(shape["D"], shape["M"], 2) * token_heads
        peak, _ = hbm_peak()
        rec = {"valid": True, "workload": workload_name(4, shape) + ", sequence split over %d ranks" % world,
               "mode": mode, "ms_per_step": tN, "value": shape["N"] * L / (tN * 1e-3) / 1e6, "unit": UNIT,
               "steps": steps, "cuda_graph": bool(graph_steps), "steps_per_graph": graph_steps,
               "positions_per_rank": Lr,
               "exchange": ("stores into the peers' buffers by this library's kernels (PeerExchange)"
                            if exchange is not None else "all_gather of the per-rank states (NCCL)"),
               "attempts": attempts,
               "t1_ms": t1, "t1_how": "the same sequence on rank 0 alone, same process, CUDA graph of 2 steps",
               "efficiency": t1 / (world * tN), "efficiency_formula": "t1_ms / (n_gpus * ms_per_step)",
               "frac_of_hbm_peak_per_gpu": alg / world / (tN * 1e-3) / 1e9 / peak,
               "rel_err_vs_fp64": errs, "rel_err_heads": heads, "tolerance_vs_fp64": 2e-2}
    dist.barrier()
    if exchange is not None:
        exchange.close()
    return rec


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
def main():
    args = parse()
    if args.recurrent:
        return run_recurrent(args)
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))

    from fast_transformers_b200 import workloads
    if args.config == 3:
        if args.impl == "reference":
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable":
                                  "config 3 (whole encoder) is not timed on the CPU; the reference "
                                  "arm covers the causal_dot_product configs"}))
            return 0
        return run_encoder(args)
    shape = dict(workloads.SHAPES[args.config])
    if args.L:
        shape["L"] = args.L
    name = workload_name(args.config, shape)

    if args.impl == "reference":
        if rank != 0:
            return 0
        inputs = workloads.make_inputs(args.config, scale_L=args.L)
        run_reference(args, shape, inputs, name)
        return 0

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200); there is no CPU path")
    import fast_transformers_b200 as ftb
    from fast_transformers_b200 import _native
    from fast_transformers_b200.causal_product import causal_dot_product
    lib = _native.lib()   # raises if the native library is missing

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    mode = args.mode or ftb.get_mode()
    # Config 4 is ONE long sequence: with several ranks it is split over them (strong scaling,
    # one exchange of (N,H,D,M) states per direction); the other configs give every rank its
    # own slice of a global batch (weak scaling, no collective).
    seq_parallel = args.config == 4 and world > 1
    full_L = shape["L"]
    if seq_parallel:
        if full_L % world:
            raise SystemExit("sequence length %d does not divide over %d ranks" % (full_L, world))
        shape["L"] = full_L // world
    # every rank draws its own slice (trial = rank)
    Q, K, V, G = workloads.make_inputs(args.config, trial=rank, scale_L=shape["L"])
    pinned = [t.pin_memory() for t in (Q, K, V, G)]
    Qd, Kd, Vd, Gd = (t.to(dev) for t in (Q, K, V, G))
    Qd.requires_grad_(True), Kd.requires_grad_(True), Vd.requires_grad_(True)
    tokens = shape["N"] * shape["L"]
    token_heads = tokens * shape["H"]
    esize = Qd.element_size()

    if seq_parallel:
        from fast_transformers_b200.sequence_parallel import (LocalOps,
                                                              sequence_parallel_causal_dot_product)
        sp_ops = LocalOps(mode)
        sp_exchange = None
        if args.exchange == "peer":
            from fast_transformers_b200.sequence_parallel import PeerExchange
            sp_exchange = PeerExchange((shape["N"], shape["H"], shape["D"], shape["M"]))

    def step():
        Qd.grad = Kd.grad = Vd.grad = None
        with ftb.mode(mode):
            if seq_parallel:
                out = sequence_parallel_causal_dot_product(Qd, Kd, Vd, ops=sp_ops,
                                                           exchange=sp_exchange)
            else:
                out = causal_dot_product(Qd, Kd, Vd)
            out.backward(Gd)
        return out

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    if seq_parallel and sp_exchange is not None:
        sp_exchange.check()      # raises if a receive gave up waiting for a peer during warm-up
    # One step is a handful of launches of ~50 us each, so the host would set the pace: the
    # step is captured once into a CUDA graph (native launches go to the capturing stream like
    # any other) and replayed.  --no-graph times the eager calls instead.
    graph = None
    per_graph = 1
    launches_per_step = None
    # (the sequence split is captured only on request, and only with the peer-memory exchange:
    # a step with NCCL calls in it did not capture here)
    if not args.no_graph and (not seq_parallel or (args.sp_graph and sp_exchange is not None)):
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            step()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize()
        # the graph holds as many whole steps as divide --steps (at most 10), so that the gap
        # between two graph launches is not paid once per 0.2 ms step
        # (graphs longer than a few milliseconds gained nothing and one of 10 x 3.8 ms ran slower).
        eager_ms = []
        for _ in range(3):
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            step()
            t1.record()
            torch.cuda.synchronize()
            eager_ms.append(t0.elapsed_time(t1))
        most = args.graph_steps or max(1, min(10, int(8.0 / max(min(eager_ms), 1e-3))))
        if dist is not None:      # the same on every rank (ranks that exchange must stay in step)
            m = torch.tensor([most], device=dev)
            dist.all_reduce(m, op=dist.ReduceOp.MIN)
            most = int(m.item())
        per_graph = next(d for d in range(most, 0, -1) if args.steps % d == 0)
        graph = torch.cuda.CUDAGraph()
        n0 = lib.ftb_launch_count()
        with torch.cuda.graph(graph):
            for _ in range(per_graph):
                step()
        launches_per_step = (lib.ftb_launch_count() - n0) // per_graph
        for _ in range(3):
            graph.replay()
        barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    launches0 = lib.ftb_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    if graph is not None:
        for _ in range(args.steps // per_graph):
            graph.replay()
    else:
        for _ in range(args.steps):
            step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    launches = (launches_per_step * args.steps if graph is not None
                else lib.ftb_launch_count() - launches0)
    barrier()
    if sampler and not seq_parallel:
        # (the timed region is a few milliseconds: the same launches go on, untimed, until the
        # clock samples have been taken under their load)
        sampler.keep_loaded((lambda: graph.replay()) if graph is not None else step)
    clocks = sampler.stop() if sampler else None
    # no kernel of the timed region gave up a bounded wait (a timed-out exchange leaves NaN
    # behind and a status word; the number would be meaningless)
    if seq_parallel and sp_exchange is not None:
        sp_exchange.check()
    else:
        ftb.check_device_status(dev)
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = t.item() / args.steps
    global_tokens = tokens * world   # sequence-parallel: the ranks' slices make up one sequence
    value = global_tokens / (ms_step * 1e-3) / 1e6

    # ---- per-kernel device time (instrumented pass, after the timed region) --------------
    lib.ftb_timing_enable(1)
    for _ in range(args.steps):
        if seq_parallel:
            # the split step as it is (every launch is recorded, whichever thread makes it)
            step()
            continue
        # the backward pass runs on an autograd thread; call the native functions directly
        # so every launch is made (and recorded) by this thread
        from fast_transformers_b200.causal_product import (causal_dot_backward_cuda,
                                                           causal_dot_product_cuda)
        o = torch.empty(shape["N"], shape["H"], shape["L"], shape["M"], device=dev, dtype=Qd.dtype)
        gq, gk, gv = torch.empty_like(Qd), torch.empty_like(Kd), torch.empty_like(Vd)
        kept = []
        causal_dot_product_cuda(Qd.data, Kd.data, Vd.data, o, mode, keep_workspace=kept)
        causal_dot_backward_cuda(Qd.data, Kd.data, Vd.data, Gd, gq, gk, gv, mode,
                                 forward_workspace=kept[0] if kept else None)
    torch.cuda.synchronize()
    kinds = _native.timing_read()
    lib.ftb_timing_enable(0)
    peak_gbs, peak_src = hbm_peak()
    total_kernel_ms = sum(v[0] for v in kinds.values()) or 1.0
    top = max(kinds.items(), key=lambda kv: kv[1][0]) if kinds else ("none", (0.0, 0))
    top_name, (top_ms, top_n) = top
    # Algorithmic bytes of one launch: every DISTINCT tensor the grid reads or writes, once
    # (elements per token-head; D-wide: Q, K, grad_Q, grad_K; M-wide: V, grad_out, out, grad_V).
    D, M = shape["D"], shape["M"]
    with_qr = "mma_bwd_qr" in kinds or "mma_bwd" in kinds    # grad_Q has a grid of its own
    per_launch_elems = {
        "simt_scan": (2 * D + 2 * M),               # three operand tensors in, one out (averaged
                                                    # over the four role permutations)
        "mma_fwd": (2 * D + 2 * M),                 # Q, K, V -> out
        "mma_bwd": (2 * D + 2 * M),                 # one gradient scan (grad_Q): three tensors in, one out
        "state_sum": (D + M),
        "mma_state": (D + M),                       # K, V (or Q, grad_out) -> totals
        # grad_Q scan (grad_out, V, K -> grad_Q) with the sweep of (Q, grad_out) beside it
        "mma_bwd_qr": (3 * D + 2 * M),
        # grad_K and grad_V in one grid: Q, K, V, grad_out -> grad_K, grad_V; with grad_Q in the
        # same grid (no sweep needed) one more output
        "mma_bwd_multi": (3 * D + 3 * M) if with_qr else (4 * D + 3 * M),
    }.get(top_name, 0)
    alg_bytes_launch = per_launch_elems * esize * token_heads
    avg_ms = top_ms / top_n if top_n else 0.0
    achieved = alg_bytes_launch / (avg_ms * 1e-3) / 1e9 if avg_ms else 0.0
    step_alg_bytes = workloads.algorithmic_bytes(D, M, esize) * token_heads
    fwd_ms = sum(kinds.get(k, (0.0, 0))[0] for k in ("mma_state", "mma_fwd")) / args.steps
    bwd_ms = sum(kinds.get(k, (0.0, 0))[0] for k in ("mma_bwd", "mma_bwd_qr", "mma_bwd_multi")) / args.steps
    if mode != "mma":
        fwd_ms = bwd_ms = 0.0     # the fp32 kernels are not told apart by direction

    def frac_of(elems, ms_):
        if not ms_:
            return None
        return elems * esize * token_heads / (ms_ * 1e-3) / 1e9 / peak_gbs

    # DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu capture
    # recorded in profiles/dram_bytes_per_launch.json -- reported only while the kernel source is
    # the one that capture was taken from
    traffic, traffic_note = None, "no ncu capture recorded for this kernel and workload"
    tpath = os.path.join(ROOT, "profiles", "dram_bytes_per_launch.json")
    if os.path.exists(tpath) and not args.L:
        import hashlib
        table = json.load(open(tpath))
        src = os.path.join(ROOT, "fast-transformers_b200", "csrc", table.get("source_file", ""))
        sha = hashlib.sha256(open(src, "rb").read()).hexdigest()[:16] if os.path.isfile(src) else None
        entry = table.get("entries", {}).get("config%d/%s/%s" % (args.config, mode, top_name))
        if entry is not None and sha == table.get("source_sha16"):
            traffic, traffic_note = entry["dram_bytes"], entry.get("from")
        elif entry is not None:
            traffic_note = "the recorded capture predates the current kernel source"
    roofline = {
        "bound": "hbm", "kernel": top_name, "achieved": achieved, "peak": peak_gbs,
        "unit": "GB/s", "frac": achieved / peak_gbs if peak_gbs else None,
        "peak_source": peak_src, "traffic": traffic, "traffic_source": traffic_note,
        "algorithmic_bytes_per_launch": alg_bytes_launch,
        "algorithmic_bytes_rule": "every distinct tensor a grid reads or writes, once",
        "avg_launch_ms": avg_ms, "share_of_kernel_time": top_ms / total_kernel_ms,
        "kernels": {k: {"ms_per_step": v[0] / args.steps, "launches_per_step": v[1] / args.steps}
                    for k, v in kinds.items()},
        "forward": {"algorithmic_bytes": (2 * D + 2 * M) * esize * token_heads,
                    "kernel_ms": fwd_ms or None, "frac_of_hbm_peak": frac_of(2 * D + 2 * M, fwd_ms),
                    "how": "sum of the forward's launches, each timed alone by CUDA events"},
        "backward": {"algorithmic_bytes": (4 * D + 3 * M) * esize * token_heads,
                     "kernel_ms": bwd_ms or None, "frac_of_hbm_peak": frac_of(4 * D + 3 * M, bwd_ms),
                     "how": "sum of the backward's launches, each timed alone by CUDA events"},
        "whole_step": {"algorithmic_bytes": step_alg_bytes,
                       "achieved_GBps": step_alg_bytes / (ms_step * 1e-3) / 1e9,
                       "frac_of_hbm_peak": step_alg_bytes / (ms_step * 1e-3) / 1e9 / peak_gbs,
                       "achieved_TFLOPs": workloads.algorithmic_flops(D, M) * token_heads /
                       (ms_step * 1e-3) / 1e12},
    }

    # ---- end to end through the public API with host buffers ------------------------------
    e2e = None
    if not args.no_e2e:
        from fast_transformers_b200.host_io import HostStepPipeline
        host_out = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in (V, Q, K, V)]

        def compute(dq_, dk_, dv_, dg_):
            q, k, v = (d.detach().requires_grad_(True) for d in (dq_, dk_, dv_))
            with ftb.mode(mode):
                if seq_parallel:
                    out = sequence_parallel_causal_dot_product(q, k, v, ops=sp_ops,
                                                               exchange=sp_exchange)
                else:
                    out = causal_dot_product(q, k, v)
                out.backward(dg_)
            return out.detach(), q.grad, k.grad, v.grad

        # every step: its four inputs host -> device, forward + backward, its four results
        # device -> host; the copies of neighbouring steps overlap with the kernels and with each
        # other (PCIe is full duplex): three streams, two sets of device input buffers
        pipe = HostStepPipeline(compute, (Q, K, V, G), device=dev)
        for _ in range(3):
            pipe.run(pinned, host_out)
        pipe.synchronize()
        barrier()
        e0.record()
        n_e2e = max(3, min(args.steps, 10))
        for _ in range(n_e2e):
            pipe.run(pinned, host_out)
        tail = torch.cuda.Event()
        tail.record(pipe.out_stream)
        torch.cuda.current_stream().wait_event(tail)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = t.item() / n_e2e
        nbytes = sum(x.numel() * x.element_size() for x in pinned)
        e2e = {"value": global_tokens / (e2e_ms * 1e-3) / 1e6, "unit": UNIT,
               "h2d_bytes_per_step": nbytes,
               "d2h_bytes_per_step": sum(h.numel() * h.element_size() for h in host_out),
               "ms_per_step": e2e_ms, "steps": n_e2e,
               "api": "fast_transformers_b200.causal_product.causal_dot_product (autograd) with "
                      "pinned host tensors copied in and all four results copied out every step "
                      "(fast_transformers_b200.host_io.HostStepPipeline: copies and kernels of "
                      "neighbouring steps overlap)"}

    # the other arithmetic modes on the same inputs, for reference (a few eager steps each):
    # `other_mode` is the fp32 CUDA-core tier (the tensor-core tier when that one is benchmarked),
    # `other_modes` lists all of them
    other, others = None, []
    if world == 1 and args.config in (1, 2) and Qd.dtype == torch.float32 and not args.no_other_mode:
        mode_saved = mode
        for om in [m for m in ("fp32", "tf32x3", "mma") if m != mode_saved]:
            mode = om
            for _ in range(2):
                step()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(5):
                step()
            e1.record()
            torch.cuda.synchronize()
            oms = e0.elapsed_time(e1) / 5
            others.append({"mode": om, "dtype": {"fp32": "f32", "mma": "tf32", "tf32x3": "tf32x3"}[om],
                           "ms_per_step": oms, "value": tokens / (oms * 1e-3) / 1e6, "unit": UNIT,
                           "cuda_graph": False, "tolerance_vs_fp64": 2e-2 if om == "mma" else 1e-5})
        mode = mode_saved
        other = others[0]

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        sec, kind, cores, nst = cpu_arm(Q, K, V, G, budget_s=12.0)
        cpu_baseline = {"value": tokens / sec / 1e6, "unit": UNIT, "cores": cores, "kind": kind,
                        "sample": "%d timed steps of the full workload (%s) after 1 warm-up, "
                                  "median" % (nst, name), "ms_per_step": sec * 1e3}

    # ---- further records of a default run ------------------------------------------------
    configs_rec, sp_rec = None, None
    if args.config == 2 and not args.no_extra and not args.L and mode == "mma":
        if world == 1:
            # the other single-GPU configurations, device-resident (config 4 with two heads checked
            # against the fp64 oracle at its full length)
            configs_rec = {"config1": product_record(1, mode, dev, 200),
                           "config4": product_record(4, mode, dev, 6, heads=[0, 11]),
                           "config5": product_record(5, mode, dev, 10)}
        else:
            sp_rec = sequence_parallel_record(args, dev, dist, rank, world, mode, lib)

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong" if args.config == 4 else "weak",
            "vs_baseline": None,
            "dtype": {"fp32": "f32", "mma": "tf32" if esize == 4 else "bf16", "tf32x3": "tf32x3"}[mode],
            "data": "synthetic (seeded)",
            "config": {"workload": name, "mode": mode, "io_dtype": str(Qd.dtype).replace("torch.", ""),
                       "global_batch": shape["N"] * (1 if seq_parallel else world), "cuda_graph": graph is not None,
                       "steps_per_graph": per_graph if graph is not None else 0,
                       "sharding": ("sequence split over ranks, %s per direction, L/rank=%d" % (
                           "per-rank states stored into the peers' buffers (own kernels)"
                           if args.exchange == "peer" else "all_gather of per-rank states (NCCL)",
                           shape["L"])) if seq_parallel
                       else "(batch, head) units per rank, no collective",
                       "l2": "inputs+outputs per step (%.0f MB) exceed the 126 MB L2; no flush" %
                             (step_alg_bytes / 1e6)},
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e,
            "gpu_launches": int(launches), "clocks": clocks, "other_mode": other, "other_modes": others or None,
            "tolerance_vs_fp64": 2e-2 if mode == "mma" else 1e-5,
        }
        if configs_rec is not None:
            line["configs"] = configs_rec
        if sp_rec is not None:
            line["sequence_parallel"] = sp_rec
        print(json.dumps(line))
    if seq_parallel and sp_exchange is not None:
        sp_exchange.close()
    if dist is not None:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
