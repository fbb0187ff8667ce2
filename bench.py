"""Benchmark of the Mellin x linear 2-D layer hot path (forward + backward).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (``config.workload``): one 2-D layer, Mellin correlation along the 41
frequency bins and linear correlation along 800 frames, batch 32 per GPU,
3 -> 64 channels, kernel 8 x 3, stride 1, dilation 1, time padding 1,
same-size output (41 x 800), FP32; inputs ~ N(0, 1), Kaiming-normal weights,
zero bias, upstream gradient ~ N(0, 1); everything synthetic and seeded.

One step = forward, grad-input and grad-weight(+bias) of that layer.  The
metric is effective GB/s: the algorithmic bytes of the step (every operand and
result counted once; the upstream gradient once for the whole backward)
divided by the time.  ``value`` is measured with every tensor resident in
HBM (CUDA events on the launching stream, per step, L2 flushed between
steps); ``e2e`` is measured through ``mconv.MCorrLCorr`` with the step's input
batch copied from pinned host memory inside the timed region and the weight
and bias gradients copied back.

With ``--impl reference`` the same step is run by the reference's own CPU
kernels (``oracle/_ref``, OpenMP over all host cores; the C restatement when
that library is absent) on a bounded sample of the batch.

Multi-GPU (torchrun, one rank per GPU): every rank runs its own batch-32 shard
(weak scaling); the weight and bias gradients are summed with one NCCL
all-reduce inside the step.
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
# the other layers of the reference's three-layer stack (kernel 6x3, Mellin dilation 2), for --kernels-only captures
PROFILE_LAYERS = {
    "3to64": {},
    "64to128": dict(c_in=64, c_out=128, nf=(6, 3), d=(2, 1)),
    "128to256": dict(c_in=128, c_out=256, nf=(6, 3), d=(2, 1)),
}
METRIC = "mcorrlcorr_fwd_bwd_effective_bandwidth"
UNIT = "GB/s"


def geometry(batch):
    w = WORKLOAD
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


# ---------------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

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
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        clocks, maxes, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                clocks.append(float(parts[0]))
                maxes.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
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


def run_reference(args):
    """The reference's CPU implementation of the same step on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np

    # torchrun exports OMP_NUM_THREADS=1 to its workers; this arm is meant to use every host core it may
    cores = len(os.sched_getaffinity(0))
    os.environ["OMP_NUM_THREADS"] = str(cores)
    from oracle.oracle import Oracle

    kind = "reference" if Oracle.reference_available() else "port"
    oracle = Oracle(kind)
    _use_all_cores()
    sample_batch = 2
    xs, ws, ys, r = geometry(sample_batch)
    w_ = WORKLOAD
    rng = np.random.default_rng(0)
    x = rng.standard_normal(xs).astype(np.float32)
    w = (rng.standard_normal(ws) * (2.0 / (ws[1] * ws[2] * ws[3])) ** 0.5).astype(np.float32)
    b = np.zeros(ws[0], dtype=np.float32)
    go = rng.standard_normal(ys).astype(np.float32)

    def step():
        oracle.mcorrlcorr(x, w, b, w_["s"], w_["d"], w_["p"], w_["u"], r)
        oracle.mcorrlcorr_backward(x, w, go, w_["s"], w_["d"], w_["p"], w_["u"])

    for _ in range(max(1, min(args.warmup, 2))):
        step()
    steps = max(1, min(args.steps, 10))
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    value = algorithmic_bytes(sample_batch)["step"] / dt / 1e9
    sample = "batch %d of the %d-utterance batch per step (the step's cost is linear in the batch), %d steps" % (
        sample_batch, WORKLOAD["batch"], steps)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3 * WORKLOAD["batch"] / sample_batch,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(), "sample": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def cpu_baseline_leg():
    import numpy as np
    from oracle.oracle import Oracle

    kind = "reference" if Oracle.reference_available() else "port"
    oracle = Oracle(kind)
    _use_all_cores()
    sample_batch = 2
    xs, ws, ys, r = geometry(sample_batch)
    w_ = WORKLOAD
    rng = np.random.default_rng(0)
    x = rng.standard_normal(xs).astype(np.float32)
    w = (rng.standard_normal(ws) * (2.0 / (ws[1] * ws[2] * ws[3])) ** 0.5).astype(np.float32)
    b = np.zeros(ws[0], dtype=np.float32)
    go = rng.standard_normal(ys).astype(np.float32)

    def step():
        oracle.mcorrlcorr(x, w, b, w_["s"], w_["d"], w_["p"], w_["u"], r)
        oracle.mcorrlcorr_backward(x, w, go, w_["s"], w_["d"], w_["p"], w_["u"])

    step()
    reps, t0 = 0, time.perf_counter()
    while reps < 3 or (time.perf_counter() - t0 < 10.0 and reps < 50):
        step()
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    return {"value": algorithmic_bytes(sample_batch)["step"] / dt / 1e9, "unit": UNIT,
            "cores": len(os.sched_getaffinity(0)) if kind == "reference" else len(os.sched_getaffinity(0)),
            "kind": kind,
            "sample": "batch %d of %d per step, %d repetitions, OpenMP over all listed cores" % (
                sample_batch, WORKLOAD["batch"], reps)}


# ---------------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist

    import capi
    import dp
    import mconv

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

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
    gw = torch.empty_like(w)
    gb = torch.empty_like(b)
    bucket = dp.GradBucket([ws, (ws[0],)], device=dev)
    grads_flat = bucket.flat
    ws_bytes = capi.grad_weight_workspace_bytes(xs, ws, ys, s, d, p, u)
    workspace = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=dev)
    ws_fwd = torch.empty(max(capi.forward_workspace_bytes(xs, ws, ys, s, d, p, u), 256), dtype=torch.uint8, device=dev)
    ws_gin = torch.empty(max(capi.grad_input_workspace_bytes(xs, ws, ys, s, d, p, u), 256), dtype=torch.uint8, device=dev)
    flush = torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device=dev)  # > 126 MB of L2

    def ev():
        return torch.cuda.Event(enable_timing=True)

    def step(events=None):
        if events:
            events[0].record()
        capi.forward(x, w, b, y, s, d, p, u, workspace=ws_fwd)
        if events:
            events[1].record()
        capi.grad_input(w, go, gx, s, d, p, u, workspace=ws_gin)
        if events:
            events[2].record()
        capi.grad_weight(x, go, gw, gb, s, d, p, u, workspace=workspace)
        if events:
            events[3].record()
        if world > 1:
            bucket.pack([gw, gb])
            bucket.all_reduce()
        if events:
            events[4].record()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(args.warmup):
        flush.zero_()
        step()
    barrier()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = capi.launch_count()
    all_events = []
    for _ in range(args.steps):
        flush.zero_()
        evs = [ev() for _ in range(5)]
        step(evs)
        all_events.append(evs)
    barrier()
    launches = capi.launch_count() - launches0
    per = {"forward": 0.0, "grad_input": 0.0, "grad_weight": 0.0, "allreduce": 0.0}
    total_ms = 0.0
    for evs in all_events:
        per["forward"] += evs[0].elapsed_time(evs[1])
        per["grad_input"] += evs[1].elapsed_time(evs[2])
        per["grad_weight"] += evs[2].elapsed_time(evs[3])
        per["allreduce"] += evs[3].elapsed_time(evs[4])
        total_ms += evs[0].elapsed_time(evs[4])

    if args.kernels_only:
        if rank == 0:
            sampler.stop()
            print(json.dumps({"kernels_only": True, "batch": batch, "ms": {k: v / args.steps for k, v in per.items()},
                              "gpu_launches": launches}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- end to end through the public PyTorch surface, host buffers -------------
    layer = mconv.MCorrLCorr(w_["c_in"], w_["c_out"], w_["nf"], s, d, p, r).to(dev)
    with torch.no_grad():
        layer.weight.copy_(w)
        layer.bias.zero_()
    gw_hosts = [torch.empty(ws, pin_memory=True) for _ in range(2)]
    gb_hosts = [torch.empty(ws[0], pin_memory=True) for _ in range(2)]
    downloaded = [torch.cuda.Event() for _ in range(2)]
    checksum = {"value": 0.0}
    # Double-buffered input: a copy stream uploads the batch of step k + 1 from
    # pinned host memory while step k computes.  Every timed step still owns one
    # upload and one download; the upload before the first timed step is paid by
    # the upload the last timed step issues for a step that never runs.  The host
    # reads the gradients of step k - 1 (pinned buffers, double-buffered too) after
    # it has queued step k, so that the device never waits for the host.
    x_bufs = [torch.empty(xs, device=dev) for _ in range(2)]
    uploaded = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    copy_stream = torch.cuda.Stream(device=dev)
    main_stream = torch.cuda.current_stream()
    counter = {"next_upload": 0, "next_step": 0}

    def upload():
        k = counter["next_upload"] % 2
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[k])
            x_bufs[k].copy_(x_host, non_blocking=True)
            uploaded[k].record(copy_stream)
        counter["next_upload"] += 1

    def e2e_step():
        k = counter["next_step"] % 2
        counter["next_step"] += 1
        upload()  # the next step's batch
        main_stream.wait_event(uploaded[k])
        xin = x_bufs[k].detach().requires_grad_(True)
        out = layer(xin)
        layer.weight.grad = None
        layer.bias.grad = None
        out.backward(go)
        consumed[k].record(main_stream)
        if world > 1:
            bucket.pack([layer.weight.grad, layer.bias.grad])
            bucket.all_reduce()
            gw_hosts[k].copy_(grads_flat[: gw.numel()].view(ws), non_blocking=True)
            gb_hosts[k].copy_(grads_flat[gw.numel():], non_blocking=True)
        else:
            gw_hosts[k].copy_(layer.weight.grad, non_blocking=True)
            gb_hosts[k].copy_(layer.bias.grad, non_blocking=True)
        downloaded[k].record(main_stream)
        read_back(1 - k)

    def read_back(k):
        downloaded[k].synchronize()
        checksum["value"] += float(gw_hosts[k].view(-1)[0]) + float(gb_hosts[k][0])

    for ev_ in consumed + downloaded:
        ev_.record(main_stream)
    upload()
    for _ in range(max(3, args.warmup // 2)):
        e2e_step()
    barrier()
    e2e_steps = max(5, args.steps // 4)
    e_start, e_end = ev(), ev()
    e_start.record()
    for _ in range(e2e_steps):
        e2e_step()
    e_end.record()
    read_back((counter["next_step"] - 1) % 2)  # the last step's gradients
    barrier()
    e2e_ms = e_start.elapsed_time(e_end) / e2e_steps
    clocks = sampler.stop() if rank == 0 else None

    times = torch.tensor([total_ms / args.steps, e2e_ms, per["forward"] / args.steps, per["grad_input"] / args.steps,
                          per["grad_weight"] / args.steps, per["allreduce"] / args.steps], device=dev,
                         dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_step, ms_e2e, ms_f, ms_i, ms_w, ms_ar = [float(v) for v in times.tolist()]

    if rank == 0:
        nbytes = algorithmic_bytes(batch)
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
        dominant = max(kernels, key=lambda k: kernels[k]["ms"])
        achieved = kernels[dominant]["GBps"]
        traffic_path = os.path.join(ROOT, "profiles", "traffic.json")
        traffic = None
        if os.path.isfile(traffic_path):
            traffic = json.load(open(traffic_path)).get(dominant)
        line = {
            "metric": METRIC, "value": world * nbytes["step"] / ms_step / 1e6, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name(), "global_batch": batch * world,
                       "l2": "working set 562 MB per step exceeds the 126 MB L2 and a 192 MB buffer is written between timed steps",
                       "parallelism": "dp%d (batch-sharded, NCCL all-reduce of grad_w and grad_b)" % world},
            "roofline": {"bound": "hbm", "kernel": dominant, "achieved": achieved, "peak": peak,
                         "peak_source": peak_src, "unit": "GB/s", "frac": achieved / peak, "traffic": traffic},
            "kernels": kernels,
            "allreduce_ms": ms_ar,
            "e2e": {"value": world * nbytes["step"] / ms_e2e / 1e6, "unit": UNIT, "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": 4 * numel(xs), "d2h_bytes_per_step": 4 * (numel(ws) + ws[0]),
                    "api": "mconv.MCorrLCorr forward + autograd backward; input batch from pinned host memory "
                           "(double-buffered: the upload of step k+1 runs on a copy stream during step k), "
                           "weight and bias gradients of every step copied to pinned host memory and read by the host one step later; upstream gradient resident on the device"},
            "gpu_launches": launches,
            "clocks": clocks,
        }
        if world == 1:
            line["cpu_baseline"] = cpu_baseline_leg()  # timed on rank 0 of the single-GPU run only
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=WORKLOAD["batch"],
                    help="utterances per GPU; values other than 32 are for profiler captures of a smaller case, "
                         "not for bench lines")
    ap.add_argument("--kernels-only", action="store_true",
                    help="skip the end-to-end and CPU-baseline legs (profiler captures)")
    ap.add_argument("--layer", default="3to64", choices=sorted(PROFILE_LAYERS),
                    help="with --kernels-only: time another layer of the reference's stacks (profiler captures of the "
                         "wide-layer kernels); bench lines are always the 3to64 layer")
    args = ap.parse_args()
    WORKLOAD["batch"] = args.batch
    if args.layer != "3to64":
        if not args.kernels_only:
            ap.error("--layer needs --kernels-only")
        WORKLOAD.update(PROFILE_LAYERS[args.layer])
    if not args.kernels_only:
        args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
