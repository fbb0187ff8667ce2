"""Benchmark of the Mellin-convolution hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--skip train,layers,sweep,latency]

Headline workload (``config.workload``): one 2-D layer, Mellin correlation along
the 41 frequency bins and linear correlation along 800 frames, batch 32 per GPU,
3 -> 64 channels, kernel 8 x 3, stride 1, dilation 1, time padding 1, same-size
output (41 x 800), FP32; inputs ~ N(0, 1), Kaiming-normal weights, zero bias,
upstream gradient ~ N(0, 1); everything synthetic and seeded.

One step = forward, weight(+bias) gradient and input gradient of that layer.
The metric is effective GB/s: the algorithmic bytes of the step (every operand
and result counted once; the upstream gradient once for the whole backward)
divided by the time.  ``value`` is measured with every tensor resident in HBM
(CUDA events on the launching stream around EXACTLY ``--steps`` steps, L2
flushed between steps); the block of K steps is repeated until about two
seconds of device time have passed and the median block is reported, with the
value per sampled SM clock beside it.  ``e2e`` is measured through
``mconv.MCorrLCorr`` with the step's input batch copied from pinned host memory
inside the timed region and the weight and bias gradients copied back.

Further blocks of the same JSON line (each skippable with ``--skip``):
``train_step`` (the ten-layer CNN-CTC training step, utterances/s, data-parallel
with bucketed gradient all-reduce overlapped with backward), ``layers`` (the
wide layers of the three-layer stack against measured TF32 / FP32 peaks),
``sweep`` (the 1-D Mellin and linear operators at batch 64 x 256 channels x
16384 samples, batch-sharded over the ranks), ``latency_us`` (the small 1-D
operator against an empty launch), ``prologue`` (log compression + lift in
front of the first layer as one pass, against the HBM roofline and against the
stock torch operators; single-GPU runs only).

With ``--impl reference`` the headline step is run by the reference's own CPU
kernels (``oracle/_ref``, OpenMP over all host cores; the C restatement when
that library is absent) on the full batch, for the steps asked for.

Multi-GPU (torchrun, one rank per GPU): every rank runs its own batch-32 shard
(weak scaling); the weight and bias gradients land directly in a flat bucket
whose NCCL all-reduce runs while the input gradient is computed.
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
for _p in (ROOT, os.path.join(ROOT, "cnn-mellin_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

WORKLOAD = dict(batch=32, c_in=3, c_out=64, ng=(41, 800), nf=(8, 3), s=(1, 1), d=(1, 1), p=(0, 1), u=(1, 1))
# the other layers of the reference's three-layer stack (kernel 6x3, Mellin dilation 2)
PROFILE_LAYERS = {
    "3to64": {},
    "64to128": dict(c_in=64, c_out=128, nf=(6, 3), d=(2, 1)),
    "128to256": dict(c_in=128, c_out=256, nf=(6, 3), d=(2, 1)),
}
METRIC = "mcorrlcorr_fwd_bwd_effective_bandwidth"
UNIT = "GB/s"


def geometry(batch, w=None):
    w = w or WORKLOAD
    valid = (w["ng"][0] * (w["p"][0] + 1)) // (w["nf"][0] + w["d"][0] - 1) - w["s"][0] + 1
    r = (w["ng"][0] - valid, 1)
    x_shape = (batch, w["c_in"]) + w["ng"]
    w_shape = (w["c_out"], w["c_in"]) + w["nf"]
    y_shape = (batch, w["c_out"]) + w["ng"]
    return x_shape, w_shape, y_shape, r


def numel(shape):
    n = 1
    for v in shape:
        n *= v
    return n


def algorithmic_bytes(batch):
    """Per-kernel and per-step algorithmic bytes (FP32)."""
    xs, ws, ys, _ = geometry(batch)
    x, w, y, b = numel(xs), numel(ws), numel(ys), ws[0]
    fwd = 4 * (x + w + b + y)
    gin = 4 * (y + w + x)
    gwt = 4 * (y + x + w + b)
    step = fwd + 4 * (y + x + w + x + w + b)  # backward reads grad_y once
    return dict(forward=fwd, grad_input=gin, grad_weight=gwt, step=step)


def workload_name():
    return ("config[1]: Mellin(41 bins) x linear(800 frames) 2-D layer fwd+bwd, batch %d/GPU, 3->64 ch, " % WORKLOAD["batch"] +
            "kernel 8x3, s=1, d=1, time pad 1, same-size output, fp32")


def mellin_pairs(nf, ng, nh, s, d, p=0, u=1):
    """(output, tap) pairs of the Mellin axis that read inside the signal: (h + s)(f + d) = (p + 1)(g + u)."""
    import numpy as np

    num = (np.arange(nh, dtype=np.int64)[:, None] + s) * (np.arange(nf, dtype=np.int64)[None, :] + d)
    g = num // (p + 1) - u
    return int(((num % (p + 1) == 0) & (g >= 0) & (g < ng)).sum())


def linear_pairs(nf, ng, nh, s, d, p=0):
    """(output, tap) pairs of the linear axis that read inside the signal: g = s h + d f - p (no up-sampling)."""
    count = 0
    for f in range(nf):
        h_lo = max(0, -((d * f - p) // s))               # ceil((p - d f) / s)
        h_hi = min(nh - 1, (ng - 1 + p - d * f) // s)
        count += max(0, h_hi - h_lo + 1)
    return count


# ---------------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []  # (host time, text)

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def samples(self):
        out = []
        for t, line in list(self.lines):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                out.append((t, float(parts[0]), float(parts[1]), parts[3:7]))
            except ValueError:
                continue
        return out

    def stop(self, windows=None):
        """Summary over the samples taken inside `windows` (list of (t0, t1) host times; None = all samples)."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        clocks, maxes, reasons = [], [], set()
        for t, clk, mx, flags in self.samples():
            if windows is not None and not any(a <= t <= b for a, b in windows):
                continue
            clocks.append(clk)
            maxes.append(mx)
            for name, val in zip(names, flags):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None,
                "sm_max_mhz": max(maxes) if maxes else None, "reasons": sorted(reasons), "samples": len(clocks)}


# ---------------------------------------------------------------------------------
def _use_all_cores():
    """torchrun exports OMP_NUM_THREADS=1 to its workers; the CPU arms are meant to use every host core they may."""
    cores = len(os.sched_getaffinity(0))
    os.environ["OMP_NUM_THREADS"] = str(cores)
    try:  # in case the OpenMP runtime was initialised before the variable was set
        import ctypes

        ctypes.CDLL("libgomp.so.1").omp_set_num_threads(cores)
    except OSError:
        pass
    return cores


def _cpu_step_factory():
    """The headline step (full batch) on the host cores: returns (step function, oracle kind, cores)."""
    import numpy as np

    cores = len(os.sched_getaffinity(0))
    os.environ["OMP_NUM_THREADS"] = str(cores)
    from oracle.oracle import Oracle

    kind = "reference" if Oracle.reference_available() else "port"
    oracle = Oracle(kind)
    _use_all_cores()
    xs, ws, ys, r = geometry(WORKLOAD["batch"])
    w_ = WORKLOAD
    rng = np.random.default_rng(0)
    x = rng.standard_normal(xs).astype(np.float32)
    w = (rng.standard_normal(ws) * (2.0 / (ws[1] * ws[2] * ws[3])) ** 0.5).astype(np.float32)
    b = np.zeros(ws[0], dtype=np.float32)
    go = rng.standard_normal(ys).astype(np.float32)

    def step():
        oracle.mcorrlcorr(x, w, b, w_["s"], w_["d"], w_["p"], w_["u"], r)
        oracle.mcorrlcorr_backward(x, w, go, w_["s"], w_["d"], w_["p"], w_["u"])

    return step, kind, cores


def run_reference(args):
    """The reference's CPU implementation of the same step, same batch, on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    step, kind, cores = _cpu_step_factory()
    budget_s = 150.0  # the whole arm must end within a few minutes whatever K is
    t_begin = time.perf_counter()
    for _ in range(args.warmup):
        step()
        if time.perf_counter() - t_begin > budget_s / 3:
            break
    steps = 0
    t0 = time.perf_counter()
    while steps < args.steps:
        step()
        steps += 1
        if time.perf_counter() - t_begin > budget_s:
            break
    dt = (time.perf_counter() - t0) / steps
    value = algorithmic_bytes(WORKLOAD["batch"])["step"] / dt / 1e9
    sample = "the full %d-utterance batch per step, %d steps%s" % (
        WORKLOAD["batch"], steps, "" if steps == args.steps else " (of %d asked: capped at %.0f s of wall time)" % (args.steps, budget_s))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(), "global_batch": WORKLOAD["batch"]},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def cpu_baseline_leg():
    step, kind, cores = _cpu_step_factory()
    step()
    reps, t0 = 0, time.perf_counter()
    while reps < 3 or (time.perf_counter() - t0 < 12.0 and reps < 40):
        step()
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    return {"value": algorithmic_bytes(WORKLOAD["batch"])["step"] / dt / 1e9, "unit": UNIT, "cores": cores, "kind": kind,
            "ms_per_step": dt * 1e3,
            "sample": "the full %d-utterance batch per step, %d repetitions (about 12 s), OpenMP over all listed cores" % (
                WORKLOAD["batch"], reps)}


# ---------------------------------------------------------------------------------
class Ctx:
    """What every block of the GPU arm needs."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist

        self.torch, self.dist, self.args = torch, dist, args
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise RuntimeError("bench.py needs a CUDA device: the product has no CPU path")
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.flush_buf = torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device=self.dev)  # > 126 MB of L2

    def ev(self):
        return self.torch.cuda.Event(enable_timing=True)

    def flush(self):
        self.flush_buf.zero_()

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
            self.torch.cuda.synchronize()

    def max_over_ranks(self, values):
        t = self.torch.tensor(values, device=self.dev, dtype=self.torch.float64)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t.tolist()]

    def time_ms(self, fn, iters, warm=1, flush=False):
        """Mean device time of fn over iters calls (events on the current stream), max over ranks."""
        for _ in range(warm):
            fn()
        self.barrier()
        total = 0.0
        for _ in range(iters):
            if flush:
                self.flush()
            a, b = self.ev(), self.ev()
            a.record()
            fn()
            b.record()
            self.torch.cuda.synchronize()
            total += a.elapsed_time(b)
        return self.max_over_ranks([total / iters])[0]


def measure_peaks(ctx):
    """Denominators the wide-layer and CUDA-core fractions use, measured here as MEASURED_PEAKS.json measures
    its bf16 entry: a dense TF32 8192^3 product (cuBLAS through torch.matmul: burst = best of 10, sustained =
    back to back for ~1.5 s) and the FMA-bound micro-kernel of this library."""
    import capi

    torch = ctx.torch
    out = {}
    # the FMA kernel first: the sustained TF32 loop below leaves the part power-capped for a while
    sms = torch.cuda.get_device_properties(ctx.dev).multi_processor_count
    buf = torch.empty(sms * 8 * 256, device=ctx.dev)
    capi.fma_rate(buf, sms * 8, 64)
    torch.cuda.synchronize()
    best = None
    for _ in range(5):
        e0, e1 = ctx.ev(), ctx.ev()
        e0.record()
        fmas = capi.fma_rate(buf, sms * 8, 2048)
        e1.record()
        torch.cuda.synchronize()
        rate = 2 * fmas / e0.elapsed_time(e1) / 1e9
        best = rate if best is None else max(best, rate)
    out["fp32_fma_tflops"] = best
    n = 8192
    a = torch.randn(n, n, device=ctx.dev)
    b = torch.randn(n, n, device=ctx.dev)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        c = torch.matmul(a, b)
        torch.cuda.synchronize()
        best = None
        for _ in range(10):
            e0, e1 = ctx.ev(), ctx.ev()
            e0.record()
            c = torch.matmul(a, b)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            best = ms if best is None else min(best, ms)
        out["tf32_tflops"] = 2 * n ** 3 / best / 1e9
        e0, e1 = ctx.ev(), ctx.ev()
        reps = max(10, int(1500.0 / best))
        e0.record()
        for _ in range(reps):
            c = torch.matmul(a, b)
        e1.record()
        torch.cuda.synchronize()
        out["tf32_tflops_sustained"] = 2 * n ** 3 * reps / e0.elapsed_time(e1) / 1e9
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    del a, b, c
    out["how"] = ("tf32: torch.matmul 8192^3 with allow_tf32 (best of 10; back to back for ~1.5 s); "
                  "fp32: FMA-bound micro-kernel, 8 blocks of 256 threads per SM, best of 5")
    return out


# ---------------------------------------------------------------------------------
def bench_headline(ctx, sampler):
    """The config-2 layer: value (resident tensors), per-kernel times, e2e through the public surface."""
    import capi
    import dp
    import mconv

    torch, dist, args = ctx.torch, ctx.dist, ctx.args
    world, rank, dev = ctx.world, ctx.rank, ctx.dev
    w_ = WORKLOAD
    batch = w_["batch"]
    xs, ws, ys, r = geometry(batch)
    s, d, p, u = w_["s"], w_["d"], w_["p"], w_["u"]
    gen = torch.Generator(device="cpu").manual_seed(rank)
    x_host = torch.randn(xs, generator=gen).pin_memory()
    wgen = torch.Generator(device="cpu").manual_seed(12345)  # weights identical on every rank
    w_host = torch.randn(ws, generator=wgen) * (2.0 / (ws[1] * ws[2] * ws[3])) ** 0.5
    go_host = torch.randn(ys, generator=gen)
    x = x_host.to(dev)
    w = w_host.to(dev)
    b = torch.zeros(ws[0], device=dev)
    go = go_host.to(dev)
    del go_host
    y = torch.empty(ys, device=dev)
    gx = torch.empty_like(x)
    # the gradient kernels write straight into the flat bucket that is all-reduced: nothing is packed
    bucket = dp.GradBucket([ws, (ws[0],)], device=dev)
    gw, gb = bucket.views()
    ws_bytes = capi.grad_weight_workspace_bytes(xs, ws, ys, s, d, p, u)
    workspace = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=dev)
    ws_fwd = torch.empty(max(capi.forward_workspace_bytes(xs, ws, ys, s, d, p, u), 256), dtype=torch.uint8, device=dev)
    ws_gin = torch.empty(max(capi.grad_input_workspace_bytes(xs, ws, ys, s, d, p, u), 256), dtype=torch.uint8, device=dev)

    def step(events=None):
        if events:
            events[0].record()
        capi.forward(x, w, b, y, s, d, p, u, workspace=ws_fwd)
        if events:
            events[1].record()
        capi.grad_weight(x, go, gw, gb, s, d, p, u, workspace=workspace)
        if events:
            events[2].record()
        # the reduction of grad_w / grad_b runs on the communication library's stream while grad-input computes
        work = bucket.all_reduce(async_op=True) if world > 1 else None
        capi.grad_input(w, go, gx, s, d, p, u, workspace=ws_gin)
        if events:
            events[3].record()
        if work is not None:
            work.wait()  # orders the compute stream after the reduction
        if events:
            events[4].record()

    for _ in range(args.warmup):
        ctx.flush()
        step()
    ctx.barrier()

    # ---- value: blocks of exactly K steps, repeated until ~2 s of device time ----
    launches0 = capi.launch_count()
    blocks = []  # (host t0, host t1, total ms, per-kernel ms)
    device_ms, n_blocks = 0.0, 0
    max_blocks = 1 if args.kernels_only else 400
    while n_blocks < max_blocks and (n_blocks < 3 or device_ms < 2000.0):
        evs_all = []
        t0 = time.perf_counter()
        for _ in range(args.steps):
            ctx.flush()
            evs = [ctx.ev() for _ in range(5)]
            step(evs)
            evs_all.append(evs)
        ctx.barrier()
        t1 = time.perf_counter()
        per = [0.0, 0.0, 0.0, 0.0]
        total = 0.0
        for evs in evs_all:
            for k in range(4):
                per[k] += evs[k].elapsed_time(evs[k + 1])
            total += evs[0].elapsed_time(evs[4])
        if n_blocks == 0:
            launches = capi.launch_count() - launches0
        # the block's wall time rides in the same reduction: every rank must take the SAME number of blocks (each
        # block ends in collectives), so the decision to go on is made on a value all ranks share
        vals = ctx.max_over_ranks([total / args.steps] + [v / args.steps for v in per] + [(t1 - t0) * 1e3])
        block_ms = vals.pop()
        blocks.append((t0, t1, vals))
        device_ms += block_ms
        n_blocks += 1
    order = sorted(range(len(blocks)), key=lambda i: blocks[i][2][0])
    med = blocks[order[len(order) // 2]][2]
    ms_step, ms_f, ms_w, ms_i, ms_exposed = med
    if args.kernels_only:
        return {"kernels_only": True, "batch": batch, "ms": {"forward": ms_f, "grad_weight": ms_w, "grad_input": ms_i},
                "gpu_launches": launches}

    # value per sampled SM clock: each block takes the median clock of the samples inside its host window
    nbytes = algorithmic_bytes(batch)
    by_clock = {}
    if rank == 0:
        samples = sampler.samples()
        for t0, t1, vals in blocks:
            clk = [c for t, c, _, _ in samples if t0 <= t <= t1]
            if clk:
                by_clock.setdefault(int(statistics.median(clk)), []).append(world * nbytes["step"] / vals[0] / 1e6)
    value_by_clock = [{"sm_mhz": k, "blocks": len(v), "value": statistics.median(v)} for k, v in sorted(by_clock.items())]

    # ---- end to end through the public PyTorch surface, host buffers -------------
    layer = mconv.MCorrLCorr(w_["c_in"], w_["c_out"], w_["nf"], s, d, p, r).to(dev)
    with torch.no_grad():
        layer.weight.copy_(w)
        layer.bias.zero_()
    # Two flat buckets alternate: the gradients of step k accumulate into bucket k % 2 (the layer's .grad tensors
    # are views of it), its all-reduce is launched asynchronously after backward and is waited for -- and the result
    # copied to the host -- only after step k + 1 has been queued, so the reduction never stalls the compute stream.
    e2e_buckets = [bucket, dp.GradBucket([ws, (ws[0],)], device=dev)]
    works = [None, None]
    gw_hosts = [torch.empty(ws, pin_memory=True) for _ in range(2)]
    gb_hosts = [torch.empty(ws[0], pin_memory=True) for _ in range(2)]
    downloaded = [torch.cuda.Event() for _ in range(2)]
    checksum = {"value": 0.0}
    # Double-buffered input: a copy stream uploads the batch of step k + 1 from
    # pinned host memory while step k computes.  Every timed step still owns one
    # upload and one download; the upload before the first timed step is paid by
    # the upload the last timed step issues for a step that never runs.  The host
    # reads the gradients of step k - 2 (pinned buffers, double-buffered too) after
    # it has queued step k, so that the device never waits for the host.
    x_bufs = [torch.empty(xs, device=dev) for _ in range(2)]
    uploaded = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    copy_stream = torch.cuda.Stream(device=dev)
    main_stream = torch.cuda.current_stream()
    counter = {"next_upload": 0, "next_step": 0}
    h2d_events = []

    def upload(timed=False):
        k = counter["next_upload"] % 2
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[k])
            if timed:
                a, b_ = ctx.ev(), ctx.ev()
                a.record(copy_stream)
            x_bufs[k].copy_(x_host, non_blocking=True)
            if timed:
                b_.record(copy_stream)
                h2d_events.append((a, b_))
            uploaded[k].record(copy_stream)
        counter["next_upload"] += 1

    def download(k):
        """Gradients of the step that used bucket k: wait for their reduction, copy them to the host."""
        if works[k] is not None:
            works[k].wait()
            works[k] = None
        gwk, gbk = e2e_buckets[k].views()
        gw_hosts[k].copy_(gwk, non_blocking=True)
        gb_hosts[k].copy_(gbk, non_blocking=True)
        downloaded[k].record(main_stream)

    def e2e_step(timed=False):
        k = counter["next_step"] % 2
        counter["next_step"] += 1
        upload(timed)  # the next step's batch
        main_stream.wait_event(uploaded[k])
        xin = x_bufs[k].detach().requires_grad_(True)
        e2e_buckets[k].flat.zero_()
        layer.weight.grad, layer.bias.grad = e2e_buckets[k].views()  # autograd accumulates into the bucket
        out = layer(xin)
        out.backward(go)
        consumed[k].record(main_stream)
        if world > 1:
            works[k] = e2e_buckets[k].all_reduce(async_op=True)
        download(1 - k)  # the previous step's gradients, reduced while this step ran
        read_back(k)     # the download queued one step ago (long finished): the host never stalls the device

    def read_back(k):
        downloaded[k].synchronize()
        checksum["value"] += float(gw_hosts[k].view(-1)[0]) + float(gb_hosts[k][0])

    for ev_ in consumed + downloaded:
        ev_.record(main_stream)
    upload()
    for _ in range(max(3, args.warmup // 2)):
        e2e_step()
    ctx.barrier()
    e2e_blocks = []
    e2e_device_ms = 0.0
    while len(e2e_blocks) < 3 or (e2e_device_ms < 1000.0 and len(e2e_blocks) < 200):
        e_start, e_end = ctx.ev(), ctx.ev()
        t0 = time.perf_counter()
        e_start.record()
        for _ in range(args.steps):
            e2e_step(timed=True)
        e_end.record()
        download((counter["next_step"] - 1) % 2)  # the last step's gradients
        read_back((counter["next_step"] - 1) % 2)
        ctx.barrier()
        # (as above: the wall time that decides whether to go on is the maximum over the ranks)
        step_ms, wall_ms = ctx.max_over_ranks([e_start.elapsed_time(e_end) / args.steps, (time.perf_counter() - t0) * 1e3])
        e2e_device_ms += wall_ms
        e2e_blocks.append(step_ms)
    ms_e2e = statistics.median(e2e_blocks)
    h2d_ms = ctx.max_over_ranks([statistics.median([a.elapsed_time(b_) for a, b_ in h2d_events])])[0]

    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    else:
        peak, peak_src = 6650.0, "fallback"
    kernels = {
        "forward": {"ms": ms_f, "GBps": nbytes["forward"] / ms_f / 1e6},
        "grad_input": {"ms": ms_i, "GBps": nbytes["grad_input"] / ms_i / 1e6},
        "grad_weight": {"ms": ms_w, "GBps": nbytes["grad_weight"] / ms_w / 1e6},
    }
    for k in kernels.values():
        k["frac_of_hbm_peak"] = k["GBps"] / peak
    dominant = max(kernels, key=lambda k: kernels[k]["ms"])
    achieved = kernels[dominant]["GBps"]
    traffic_path = os.path.join(ROOT, "profiles", "traffic.json")
    traffic = None
    if os.path.isfile(traffic_path):
        try:
            traffic = json.load(open(traffic_path)).get(dominant)
        except ValueError:
            traffic = None
    windows = [(t0, t1) for t0, t1, _ in blocks]
    return {
        "metric": METRIC, "value": world * nbytes["step"] / ms_step / 1e6, "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(), "global_batch": batch * world,
                   "l2": "working set 562 MB per step exceeds the 126 MB L2 and a 192 MB buffer is written between timed steps",
                   "timing": "median of %d timed blocks of %d steps each (about 2 s of device time)" % (n_blocks, args.steps),
                   "parallelism": "dp%d (batch-sharded; grad_w and grad_b are written into one flat bucket whose NCCL "
                                  "all-reduce overlaps grad-input)" % world},
        "roofline": {"bound": "hbm", "kernel": dominant, "achieved": achieved, "peak": peak,
                     "peak_source": peak_src, "unit": "GB/s", "frac": achieved / peak, "traffic": traffic},
        "kernels": kernels,
        "allreduce_exposed_ms": ms_exposed,
        "timed_blocks": n_blocks,
        "value_by_clock": value_by_clock,
        "e2e": {"value": world * nbytes["step"] / ms_e2e / 1e6, "unit": UNIT, "ms_per_step": ms_e2e, "h2d_ms": h2d_ms,
                "h2d_bytes_per_step": 4 * numel(xs), "d2h_bytes_per_step": 4 * (numel(ws) + ws[0]),
                "api": "mconv.MCorrLCorr forward + autograd backward; input batch from pinned host memory "
                       "(double-buffered: the upload of step k+1 runs on a copy stream during step k; h2d_ms is that copy's "
                       "own duration), weight and bias gradients of every step copied to pinned host memory and read by the "
                       "host one step later; upstream gradient resident on the device"},
        "gpu_launches": launches,
        "_windows": windows,
    }


def bench_train_step(ctx):
    """Config 4: the ten-layer CNN-CTC training step, batch 32 per GPU, data-parallel."""
    import ctc_model
    import dp

    torch, world, rank, dev = ctx.torch, ctx.world, ctx.rank, ctx.dev
    per_gpu = 32
    torch.manual_seed(4321)  # identical initial weights on every rank
    model = ctc_model.MellinCTCNet().to(dev)
    reducer = dp.BucketedReducer(model.parameters())
    step = ctc_model.TrainStep(model, lr=1e-4, reducer=reducer)
    n_params = sum(p.numel() for p in model.parameters())

    def make_batch(k):
        # the global batch of 32 * world ragged utterances is dealt so that every rank gets 32 of them and the
        # frame counts are even (each rank computes the same deal from the same seed); features and labels per rank
        lengths = ctc_model.synthetic_lengths(per_gpu * world, seed=1000 + k)
        mine = dp.snake_shards(lengths, world)[rank]
        return ctc_model.synthetic_batch([lengths[i] for i in mine], seed=100000 * (rank + 1) + k, device=dev)

    warm, timed = 3, 20  # about 4 s: long enough for the clocks to settle under the power cap
    distinct = [make_batch(k) for k in range(6)]
    batches = [distinct[k % 6] for k in range(warm + timed)]
    frames = sum(int(b[1].sum()) for b in batches[warm:])
    padded = sum(int(b[0].shape[0] * b[0].shape[3]) for b in batches[warm:])
    losses = []
    for k in range(warm):
        losses.append(step(*batches[k]))
    ctx.barrier()
    sampler = ClockSampler(ctx.local_rank)
    if rank == 0:
        sampler.start()
    e0, e1 = ctx.ev(), ctx.ev()
    t_begin = time.perf_counter()
    e0.record()
    for k in range(warm, warm + timed):
        losses.append(step(*batches[k]))
    e1.record()
    ctx.barrier()
    clocks = sampler.stop([(t_begin, time.perf_counter())]) if rank == 0 else None
    ms = ctx.max_over_ranks([e0.elapsed_time(e1) / timed])[0]
    loss_vals = [float(v) for v in losses]
    import capi

    status = capi.device_status()
    reducer.remove()
    del model, step, batches
    torch.cuda.empty_cache()
    return {
        "workload": "config[3]: 10 Mellin x linear layers 3->128->(x4)128->256->(x4)256, kernel 6x3, same-size, ReLU, dropout 0.05, "
                    "length-masked; FC 10496->1024->1024->62 per frame; log_softmax; CTC(blank=61, zero_infinity); Adam 1e-4; fp32; "
                    "batch 32 per GPU of (3, 41, T), T ~ U{200..800}, labels U{20..80} over 61 phones; synthetic",
        "utts_per_s": per_gpu * world / ms * 1e3, "ms_per_step": ms, "steps": timed, "warmup": warm,
        "global_batch": per_gpu * world, "parameters": n_params, "gradient_bytes_reduced": reducer.reduced_bytes,
        "buckets": len(reducer.buckets),
        "frames_per_step_this_rank": frames / timed, "padded_frames_per_step_this_rank": padded / timed,
        "balance": "global batch dealt longest-first in boustrophedon order: 32 utterances per rank, near-equal frames",
        "loss_first": loss_vals[0], "loss_last": loss_vals[-1], "device_status": status, "clocks": clocks,
    }


def bench_layers(ctx):
    """Wide layers of the three-layer stack (kernel 6x3, Mellin dilation 2, 41 x 800): ms, FP32-equivalent TFLOP/s
    and the fraction of measured TF32 / 3 (the kernels run 3xTF32)."""
    import capi

    torch, dev = ctx.torch, ctx.dev
    out = {}
    for name, batch in (("64to128", 8), ("128to256", 4)):
        cfg = dict(WORKLOAD)
        cfg.update(PROFILE_LAYERS[name])
        xs, ws, ys, r = geometry(batch, cfg)
        s, d, p, u = cfg["s"], cfg["d"], cfg["p"], cfg["u"]
        x = torch.randn(xs, device=dev)
        w = torch.randn(ws, device=dev) * (2.0 / (ws[1] * ws[2] * ws[3])) ** 0.5
        b = torch.zeros(ws[0], device=dev)
        go = torch.randn(ys, device=dev)
        y, gx, gw, gb = torch.empty(ys, device=dev), torch.empty_like(x), torch.empty_like(w), torch.empty_like(b)
        px = mellin_pairs(ws[2], xs[2], ys[2], s[0], d[0])
        py = linear_pairs(ws[3], xs[3], ys[3], s[1], d[1], p[1])
        flop = 2.0 * batch * ws[0] * ws[1] * px * py
        cell = {"batch": batch, "gflop": flop / 1e9}
        for key, fn in (("forward", lambda: capi.forward(x, w, b, y, s, d, p, u)),
                        ("grad_input", lambda: capi.grad_input(w, go, gx, s, d, p, u)),
                        ("grad_weight", lambda: capi.grad_weight(x, go, gw, gb, s, d, p, u))):
            ms = ctx.time_ms(fn, iters=10, warm=2, flush=True)
            tf = flop / ms / 1e9
            cell[key] = {"ms": ms, "tflops_fp32_equiv": tf}
        # the same layer on float16 tensors (float32 accumulation): one TF32 MMA per product instead of three
        xh, wh, bh, goh = x.half(), w.half(), b.half(), go.half()
        yh, gxh, gwh, gbh = torch.empty_like(goh), torch.empty_like(xh), torch.empty_like(wh), torch.empty_like(bh)
        half = {}
        for key, fn in (("forward", lambda: capi.forward_f16(xh, wh, bh, yh, s, d, p, u)),
                        ("grad_input", lambda: capi.grad_input_f16(wh, goh, gxh, s, d, p, u)),
                        ("grad_weight", lambda: capi.grad_weight_f16(xh, goh, gwh, gbh, s, d, p, u))):
            ms = ctx.time_ms(fn, iters=10, warm=2, flush=True)
            half[key] = {"ms": ms, "tflops": flop / ms / 1e9, "speedup_over_f32": cell[key]["ms"] / ms}
        cell["float16"] = half
        out[name] = cell
        del x, w, go, y, gx, gw, xh, wh, goh, yh, gxh, gwh
    out["denominator"] = "measured TF32 dense burst (peaks.tf32_tflops) / 3: every product is three TF32 MMAs"
    return out


def bench_sweep(ctx):
    """Config 5: 1-D Mellin and 1-D linear correlation, batch 64 (sharded over the ranks), 256 -> 256 channels,
    16384 samples, kernel 64, stride and dilation in {1, 2}; forward + grad-input + grad-weight, one all-reduce
    of grad_w (16.8 MB) when sharded."""
    import capi

    torch, dist, world, dev = ctx.torch, ctx.dist, ctx.world, ctx.dev
    total_batch, C, L, K = 64, 256, 16384, 64
    if total_batch % world:
        return {"skipped": "batch 64 does not split over %d ranks" % world}
    N = total_batch // world
    cells = {}
    I = __import__("ctypes").c_int64
    for kind in ("mcorr1d", "lcorr1d"):
        for s in (1, 2):
            for d in (1, 2):
                name = "%s_s%d_d%d" % (kind, s, d)
                if kind == "mcorr1d":
                    nh = L  # same-size output (the variant that keeps every tap of every position)
                    xs, ws_, ys = (N, C, L, 1), (C, C, K, 1), (N, C, nh, 1)
                    S, D, P, U = (s, 1), (d, 1), (0, 0), (1, 1)
                    pairs = mellin_pairs(K, L, nh, s, d)
                else:
                    nh = int(capi.lib().mellin_lcorr_valid_size(I(K), I(L), I(s), I(d), I(0), I(1)))
                    xs, ws_, ys = (N, C, 1, L), (C, C, 1, K), (N, C, 1, nh)
                    S, D, P, U = (1, s), (1, d), (0, 0), (1, 1)
                    pairs = linear_pairs(K, L, nh, s, d)
                flop = 2.0 * total_batch * C * C * pairs
                x = torch.randn(xs, device=dev)
                w = torch.randn(ws_, device=dev)
                b = torch.zeros(C, device=dev)
                go = torch.randn(ys, device=dev)
                y, gx, gw, gb = torch.empty(ys, device=dev), torch.empty_like(x), torch.empty_like(w), torch.empty_like(b)
                cell = {"out_len": nh, "pairs": pairs, "gflop_per_kernel": flop / 1e9, "batch_per_gpu": N}
                try:
                    # a cell the fast kernels do not cover falls to the per-output kernels: seconds per call at this
                    # size.  Time one forward first and skip the cell when it is out of proportion.
                    limit = max(60.0, flop / world / 10e9)  # slower than 10 TFLOP/s: the per-output fallback
                    t_probe = ctx.time_ms(lambda: capi.forward(x, w, b, y, S, D, P, U), iters=1, warm=0)
                    if t_probe > limit:
                        # the first call of a geometry also builds and uploads its index table: judge the second one
                        t_probe = ctx.time_ms(lambda: capi.forward(x, w, b, y, S, D, P, U), iters=1, warm=0)
                    if t_probe > limit:
                        cell["skipped"] = "forward took %.0f ms: not covered by the tensor-core kernels" % t_probe
                    else:
                        def fwd_bwd():
                            capi.forward(x, w, b, y, S, D, P, U)
                            capi.grad_weight(x, go, gw, gb, S, D, P, U)
                            work = dist.all_reduce(gw, async_op=True) if world > 1 else None
                            capi.grad_input(w, go, gx, S, D, P, U)
                            if work is not None:
                                work.wait()
                        for key, fn in (("forward", lambda: capi.forward(x, w, b, y, S, D, P, U)),
                                        ("grad_input", lambda: capi.grad_input(w, go, gx, S, D, P, U)),
                                        ("grad_weight", lambda: capi.grad_weight(x, go, gw, gb, S, D, P, U))):
                            ms = ctx.time_ms(fn, iters=2, warm=1)
                            cell[key] = {"ms": ms, "tflops_fp32_equiv": flop / ms / 1e9}
                        if s == 1 and d == 1:
                            # the reference-shaped operator (accumulates into y, no workspace argument) on the same data
                            if kind == "mcorr1d":
                                op = lambda: capi.op1d("mcorr1d", w[..., 0], x[..., 0], y[..., 0], C, C, N, s, d, 0, 1)
                            else:
                                op = lambda: capi.op2d("mcorrlcorr", w, x, y, C, C, N, S, D, P, U)
                            cell["operator_level_forward_ms"] = ctx.time_ms(op, iters=2, warm=1)
                        ms = ctx.time_ms(fwd_bwd, iters=2, warm=1)
                        cell["fwd_bwd_ms"] = ms
                        cell["tflops_fp32_equiv"] = 3 * flop / ms / 1e9
                except capi.MellinError as e:
                    cell["error"] = str(e)
                cells[name] = cell
                del x, w, go, y, gx, gw
                torch.cuda.empty_cache()
    cells["scaling"] = "strong: batch 64 split over %d rank(s), grad_w summed with one all-reduce" % world
    return cells


def bench_latency(ctx):
    """Config 1: the small 1-D Mellin correlation (batch 8, 4 -> 8 channels, length 256, kernel 16) is
    launch-latency-bound: microseconds per call against an empty-stream event pair and a trivial torch kernel."""
    import capi

    torch, dev = ctx.torch, ctx.dev
    x = torch.randn((8, 4, 256, 1), device=dev)
    w = torch.randn((8, 4, 16, 1), device=dev) / 8.0
    go = torch.randn((8, 8, 16, 1), device=dev)
    y, gx, gw = torch.empty_like(go), torch.empty_like(x), torch.empty_like(w)
    S, D, P, U = (1, 1), (1, 1), (0, 0), (1, 1)
    tiny = torch.zeros(32, device=dev)

    def us(fn, n=200):
        for _ in range(20):
            fn()
        torch.cuda.synchronize()
        a, b = ctx.ev(), ctx.ev()
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n * 1e3

    return {"forward": us(lambda: capi.forward(x, w, None, y, S, D, P, U)),
            "grad_input": us(lambda: capi.grad_input(w, go, gx, S, D, P, U)),
            "grad_weight": us(lambda: capi.grad_weight(x, go, gw, None, S, D, P, U)),
            "trivial_kernel": us(lambda: tiny.add_(1.0)),
            "note": "microseconds per call, 200 back-to-back calls on one stream (host launch cost included); "
                    "config[0] shapes, r = 0 (16 outputs per row)"}


def bench_incumbent():
    """The reference's own CUDA kernels (its stock thread-per-output kernels, unmodified, compiled for sm_100a by
    oracle/build_oracle.py into oracle/_ref/mconv_cuda_profiling) at the headline layer, timed by the reference's
    own harness (CUDA events around back-to-back launches on uninitialised buffers).  Roles as the reference's
    backward assigns them (ext/torch.cpp:261-308): grad-input is its convolution kernel over grad_out with the
    channel roles swapped, grad-weight its correlation kernel with batch and channels transposed."""
    import re

    exe = os.path.join(ROOT, "oracle", "_ref", "mconv_cuda_profiling")
    if not os.path.isfile(exe):
        return {"unavailable": "oracle/_ref/mconv_cuda_profiling was not built (no reference checkout at build time)"}
    w = WORKLOAD
    common = ["-t", "float", "--px", "0", "--py", "1"]
    runs = {
        "forward": ["-k", "MCorrLCorr", "--c-out", str(w["c_out"]), "--c-in", str(w["c_in"]), "--batch", str(w["batch"]),
                    "--nfx", str(w["nf"][0]), "--nfy", str(w["nf"][1]), "--ngx", str(w["ng"][0]), "--ngy", str(w["ng"][1]),
                    "-n", "5", "--burn-in", "2"],
        "grad_input": ["-k", "MConvLConv", "--c-out", str(w["c_in"]), "--c-in", str(w["c_out"]), "--batch", str(w["batch"]),
                       "--nfx", str(w["nf"][0]), "--nfy", str(w["nf"][1]), "--ngx", str(w["ng"][0]), "--ngy", str(w["ng"][1]),
                       "-n", "5", "--burn-in", "2"],
        # "kernel" = grad_out^T (c_out, batch, 41, 800), "input" = x^T (c_in, batch, 41, 800), output (c_in, c_out, 8, 3)
        "grad_weight": ["-k", "MCorrLCorr", "--c-out", str(w["c_out"]), "--c-in", str(w["batch"]), "--batch", str(w["c_in"]),
                        "--nfx", str(w["ng"][0]), "--nfy", str(w["ng"][1]), "--ngx", str(w["ng"][0]), "--ngy", str(w["ng"][1]),
                        "--rx", str(w["nf"][0] - 1), "--ry", "1", "--transpose-f", "--transpose-g", "--transpose-h",
                        "-n", "2", "--burn-in", "1"],
    }
    out = {}
    for name, extra in runs.items():
        try:
            proc = subprocess.run([exe] + extra + common, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                                  timeout=120)
            m = re.search(r"average ([0-9.eE+-]+)ms", proc.stdout)
            out[name] = {"ms": float(m.group(1))} if (m and proc.returncode == 0) else {"error": proc.stdout[-300:]}
        except subprocess.TimeoutExpired:
            out[name] = {"error": "no result within 120 s"}
    out["what"] = "reference's stock CUDA kernels (mconv_cuda.cuh, 32-thread blocks, one thread per output) on this GPU"
    return out


def bench_prologue(ctx):
    """The elementwise layers in front of the first layer (log compression, then the lift along the Mellin axis) as
    ONE pass: device time on a tensor larger than L2 (512 utterances of the headline layer's input, 201 MB) against
    the HBM roofline (8 bytes per element forward, 12 backward), and on the headline batch itself with L2 flushed;
    next to it the reference's formulation (layers.py:8-21,100-101: abs, add, log, arange, pow, mul as stock torch
    kernels, autograd for the backward) on the same GPU.  No collectives: single-GPU runs only."""
    import capi as c
    import layers

    torch, dev = ctx.torch, ctx.dev
    out = {"what": "y = (t+1)^tau log(eps + |x|) along dim 2; fp32; ms per call, CUDA events, L2 flushed between calls"}

    def ms(fn, iters=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(iters):
            ctx.flush()
            a, b = ctx.ev(), ctx.ev()
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            total += a.elapsed_time(b)
        return total / iters

    for name, batch in (("headline_batch", WORKLOAD["batch"]), ("larger_than_l2", 512)):
        shape = (batch, WORKLOAD["c_in"]) + tuple(WORKLOAD["ng"])
        x = torch.randn(shape, device=dev)
        gy = torch.randn(shape, device=dev)
        pair = layers.LogCompressionLift(dim=2).to(dev)
        log_tau, log_eps = pair.lift.log_tau.detach(), pair.log_compression.log_eps.detach()
        y, gx = torch.empty_like(x), torch.empty_like(x)
        g_tau, g_eps = torch.empty_like(log_tau), torch.empty_like(log_eps)
        ws = torch.empty(c.lift_compress_workspace_bytes(), dtype=torch.uint8, device=dev)
        outer, length, inner = batch * shape[1], shape[2], shape[3]
        fwd = ms(lambda: c.lift_compress(x, log_tau, log_eps, True, outer, length, inner, y))
        bwd = ms(lambda: c.lift_compress_backward(x, gy, log_tau, log_eps, True, outer, length, inner, gx, g_tau,
                                                  g_eps, workspace=ws))
        steps = torch.arange(1, length + 1, device=dev, dtype=torch.float32).view(1, 1, length, 1)

        def stock(xin):
            return (xin.abs() + log_eps.exp()).log() * steps ** log_tau.exp()

        xr = x.clone().requires_grad_(True)
        lt, le = log_tau.clone().requires_grad_(True), log_eps.clone().requires_grad_(True)

        def stock_fwd_bwd():
            yy = (xr.abs() + le.exp()).log() * steps ** lt.exp()
            yy.backward(gy)
            xr.grad = None

        stock_f = ms(lambda: stock(x))
        stock_fb = ms(stock_fwd_bwd)
        n = x.numel()
        out[name] = {
            "shape": list(shape), "forward_ms": fwd, "backward_ms": bwd,
            "forward_gbs": 8.0 * n / fwd / 1e6, "backward_gbs": 12.0 * n / bwd / 1e6,
            "stock_torch_forward_ms": stock_f, "stock_torch_forward_backward_ms": stock_fb,
            "launches": {"forward": 1, "backward": 2},
        }
        del x, gy, y, gx, xr
    return out


def run_ours(args):
    t_start = time.time()

    def note(msg):
        # progress on stderr (the JSON line is the only thing on stdout): tells where a multi-rank run stands
        sys.stderr.write("[bench rank %s +%.1fs] %s\n" % (os.environ.get("RANK", "0"), time.time() - t_start, msg))
        sys.stderr.flush()

    note("starting")
    ctx = Ctx(args)
    rank, world = ctx.rank, ctx.world
    if args.prologue_only:
        if world > 1:
            raise SystemExit("--prologue-only is a single-GPU run")
        print(json.dumps({"prologue": bench_prologue(ctx)}), flush=True)
        return
    skip = set(args.skip.split(",")) if args.skip else set()
    sampler = ClockSampler(ctx.local_rank)
    if rank == 0:
        sampler.start()
    note("process group up, headline")
    line = bench_headline(ctx, sampler)
    note("headline done")
    if args.kernels_only:
        if rank == 0:
            sampler.stop()
            print(json.dumps(line), flush=True)
        if world > 1:
            ctx.dist.destroy_process_group()
        return
    windows = line.pop("_windows")
    clocks = sampler.stop(windows) if rank == 0 else None
    line["clocks"] = clocks
    # The peak measurements come LAST: their sustained tensor-core loop leaves the part power-capped for a while,
    # which would tax whatever block ran next.  The blocks record times; fractions are filled in afterwards.
    if "latency" not in skip:
        line["latency_us"] = bench_latency(ctx)
    if "layers" not in skip:
        line["layers"] = bench_layers(ctx)
    note("latency and layers done, sweep")
    if "sweep" not in skip:
        line["sweep"] = bench_sweep(ctx)
    note("sweep done, train step")
    if "train" not in skip:
        line["train_step"] = bench_train_step(ctx)
    if "prologue" not in skip and world == 1:
        try:
            line["prologue"] = bench_prologue(ctx)
        except Exception as e:  # an optional block: the line is printed without it
            line["prologue"] = {"error": "%s: %s" % (type(e).__name__, e)}
    note("train step done, peaks")
    ctx.torch.cuda.synchronize()
    time.sleep(2.0)  # let the clocks recover from the blocks above before the burst figures are taken
    peaks = measure_peaks(ctx)
    line["peaks"] = peaks
    tf32_third = peaks["tf32_tflops"] / 3.0
    for block in ("layers", "sweep"):
        for cell in line.get(block, {}).values():
            if not isinstance(cell, dict):
                continue
            for v in [cell] + [c for c in cell.values() if isinstance(c, dict)]:
                if "tflops_fp32_equiv" in v:
                    v["frac_of_tf32_third"] = v["tflops_fp32_equiv"] / tf32_third
    if rank == 0:
        if world == 1:
            if "incumbent" not in skip:
                ctx.torch.cuda.synchronize()
                line["gpu_incumbent"] = bench_incumbent()
            line["cpu_baseline"] = cpu_baseline_leg()  # timed on rank 0 of the single-GPU run only
        print(json.dumps(line), flush=True)
    note("line printed" if rank == 0 else "done")
    if world > 1:
        ctx.dist.barrier()
        ctx.dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=WORKLOAD["batch"],
                    help="utterances per GPU; values other than 32 are for profiler captures of a smaller case, "
                         "not for bench lines")
    ap.add_argument("--kernels-only", action="store_true",
                    help="one timed block of the headline kernels only (profiler captures)")
    ap.add_argument("--prologue-only", action="store_true",
                    help="only the prologue block (log compression + lift), single GPU (profiler captures)")
    ap.add_argument("--skip", default="", help="comma-separated blocks to leave out: train, layers, sweep, latency, prologue, incumbent")
    ap.add_argument("--engine", default="tensor_cores", choices=["tensor_cores", "cuda_cores"],
                    help="with --kernels-only: cuda_cores switches the tcgen05 kernels off (profiler captures of the "
                         "CUDA-core kernels); bench lines always run the default engine")
    ap.add_argument("--layer", default="3to64", choices=sorted(PROFILE_LAYERS),
                    help="with --kernels-only: time another layer of the reference's stacks (profiler captures of the "
                         "wide-layer kernels); bench lines are always the 3to64 layer")
    args = ap.parse_args()
    WORKLOAD["batch"] = args.batch
    if args.layer != "3to64":
        if not args.kernels_only:
            ap.error("--layer needs --kernels-only")
        WORKLOAD.update(PROFILE_LAYERS[args.layer])
    if args.engine != "tensor_cores":
        if not args.kernels_only:
            ap.error("--engine needs --kernels-only")
        import capi

        capi.set_tensor_cores(False)
    if not args.kernels_only:
        args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
