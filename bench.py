#!/usr/bin/env python
"""Benchmark of the attention training step (forward + backward) through Boat's C API.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c4] [--impl ours|reference]

One step = boat_attention_forward + boat_attention_backward on one batch of synthetic input
(self-attention: query = key = value), on every rank, plus the all-reduce of the parameter
gradients when N > 1 (data parallel over batch x heads units, weak scaling: every rank holds
the full per-GPU workload).  Prints ONE JSON line on rank 0.

  value   tokens/s over all ranks, inputs resident in HBM, CUDA-event timed, max over ranks
  e2e     the same step called with HOST tensors: uploads and downloads inside the timed region
  roofline  the dominant kernel's algorithmic FLOP/s against the measured BF16 (or TF32) peak
  cpu_baseline  the reference's own CPU code on a bounded sample, extrapolated by FLOP rate

--impl reference times the reference's CPU implementation (oracle/_ref, else the C
restatement) on all host cores with the same metric and config.
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: B (per GPU), S, d_model, heads, causal, arithmetic
    "c2": dict(B=8, S=512, d=512, nh=8, causal=False, mma="tf32"),
    "c3": dict(B=16, S=2048, d=1024, nh=16, causal=True, mma="bf16"),
    "c4": dict(B=4, S=8192, d=2048, nh=16, causal=True, mma="bf16"),
    "target": dict(B=8, S=4096, d=2048, nh=16, causal=True, mma="bf16"),
    # config 5: full pre-LN encoder block step (LN, attention, residual, LN, dense 4d, GELU, dense, residual, MSE)
    "c5": dict(B=32, S=1024, d=1024, nh=16, causal=False, mma="bf16", block=True),
    # one batch entry of c4: same kernels and tile shapes, small enough for ncu --set full
    "c4_small": dict(B=1, S=8192, d=2048, nh=16, causal=True, mma="bf16"),
}
DEFAULT_WORKLOAD = "c4"
SEED = 42


def algorithmic_flops(B, S, d, causal):
    """24*T*d^2 for the four projections (forward + both gradients) + 12*c*B*S^2*d for the
    attention core (c = 1/2 when causal); recomputation inside the backward is not counted."""
    T = B * S
    return 24.0 * T * d * d + 12.0 * (0.5 if causal else 1.0) * B * S * S * d


def block_flops(B, S, d, causal):
    """Attention step plus the MLP: two GEMMs of T x d x 4d forward (16*T*d^2) and their input and
    weight gradients (32*T*d^2).  LayerNorm, GELU and the residual adds are not counted."""
    return algorithmic_flops(B, S, d, causal) + 48.0 * B * S * d * d


def reference_flops(B, S, d):
    """What the reference's CPU code executes: it computes the full S x S product even when
    the mask is causal, so c = 1."""
    return algorithmic_flops(B, S, d, False)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            pk = json.load(f)
        return dict(hbm=pk.get("hbm_gbs", 6650.0), bf16=pk.get("bf16_tflops", 1590.0),
                    bf16_sustained=pk.get("bf16_tflops_sustained", 1400.0), source="measured")
    return dict(hbm=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


def measure_tf32_peak(torch):
    """TF32 tensor-core peak measured the way the BF16 one in MEASURED_PEAKS.json was: torch.matmul
    of two 8192 x 8192 FP32 matrices with TF32 allowed, 2*N^3 FLOP, CUDA events; best of 10 (burst)
    and back to back for about 2 s (sustained).  Returns (burst, sustained) in TFLOP/s."""
    n = 8192
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        a = torch.randn(n, n, device="cuda", dtype=torch.float32)
        b = torch.randn(n, n, device="cuda", dtype=torch.float32)
        c = torch.empty(n, n, device="cuda", dtype=torch.float32)
        for _ in range(3):
            torch.matmul(a, b, out=c)
        torch.cuda.synchronize()
        flop = 2.0 * n ** 3
        best = 0.0
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(10):
            e0.record()
            torch.matmul(a, b, out=c)
            e1.record()
            torch.cuda.synchronize()
            best = max(best, flop / (e0.elapsed_time(e1) * 1e-3) / 1e12)
        iters = max(20, int(2.0 / (flop / (best * 1e12))))
        e0.record()
        for _ in range(iters):
            torch.matmul(a, b, out=c)
        e1.record()
        torch.cuda.synchronize()
        sustained = iters * flop / (e0.elapsed_time(e1) * 1e-3) / 1e12
        return best, sustained
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old


def load_kernel_traffic():
    """DRAM bytes per launch read from ncu captures (dram__bytes_read.sum + dram__bytes_write.sum),
    kept as data next to the ncu summaries: a list of {kernel, S, hs, causal, units, dram_bytes}."""
    path = os.path.join(ROOT, "profiles", "kernel_traffic.json")
    try:
        with open(path) as f:
            return json.load(f)["captures"]
    except (OSError, ValueError, KeyError):
        return []


# ---- clocks ----------------------------------------------------------------------------------------

class ClockSampler:
    """nvidia-smi sampled every `interval_ms`; started before the warm-up (the tool takes a moment
    to start), only the samples between mark() at the start and at the end of the timed
    region are reported."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index, interval_ms=50):
        self.proc = None
        self.lines = []
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", str(interval_ms)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def mark(self):
        """Samples read so far; used to keep only those taken inside the timed region."""
        return len(self.lines)

    def stop(self, first=0, last=None):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        window = self.lines[first:last] if last is not None and last > first else self.lines[first:]
        for line in window or self.lines[-1:]:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
                power.append(float(parts[2]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


# ---- CPU reference timing ------------------------------------------------------------------------------

def cpu_sample_shape(cfg, seconds):
    """A problem with the workload's d_model and head count, one batch, short enough to take
    about `seconds` at the reference's ~1 GFLOP/s per core."""
    d, nh = cfg["d"], cfg["nh"]
    budget = seconds * 0.9e9
    S = int(budget / (24.0 * d * d))
    S = max(nh, min(cfg["S"], S))
    S = max(nh, (S // nh) * nh)
    return 1, S


def cpu_reference_seconds(args):
    """Runs forward + backward once on the sample (in this process); returns seconds."""
    B, S, d, nh, causal, use_ref = args
    from boat_b200 import rng
    from oracle import oracle
    x = rng.normal(SEED, rng.X, (B, S, d))
    w = [rng.normal(SEED, rng.WQ + i, (d, d), 1.0 / np.sqrt(d)) for i in range(4)]
    b = [np.zeros(d, np.float32) for _ in range(4)]
    g = rng.normal(SEED, rng.DOUT, (B, S, d))
    if use_ref:
        layer = oracle.RefLayer(d, nh, causal, w, b)
        t0 = time.perf_counter()
        layer.step(x, x, x, g)
        dt = time.perf_counter() - t0
        layer.free()
    else:
        oracle.port().oracle_set_threads(1)
        t0 = time.perf_counter()
        oracle.port_step(x, x, x, w, b, g, nh, causal)
        dt = time.perf_counter() - t0
    return dt


def cpu_baseline(cfg, seconds, procs):
    """tokens/s of the reference's CPU path for the workload `cfg`, measured on a bounded
    sample by `procs` independent processes and extrapolated by executed FLOPs."""
    from oracle import oracle
    use_ref = oracle.have_ref()
    if not use_ref:
        oracle.port()          # builds the restatement if needed
    Bs, Ss = cpu_sample_shape(cfg, seconds)
    job = (Bs, Ss, cfg["d"], cfg["nh"], cfg["causal"], use_ref)
    if procs == 1:
        times = [cpu_reference_seconds(job)]
    else:
        import multiprocessing as mp
        with mp.get_context("spawn").Pool(procs) as pool:
            times = pool.map(cpu_reference_seconds, [job] * procs)
    dt = max(times)
    rate = procs * reference_flops(Bs, Ss, cfg["d"]) / dt                 # FLOP/s of the box
    full = reference_flops(cfg["B"], cfg["S"], cfg["d"])
    tokens_per_s = cfg["B"] * cfg["S"] / (full / rate)
    return dict(value=tokens_per_s, unit="tokens/s", cores=procs, kind="reference" if use_ref else "port",
                sample=("forward+backward of B=%d S=%d d=%d heads=%d on %d process(es) took %.2f s "
                        "(%.2f GFLOP/s total); scaled to the workload by executed FLOPs "
                        "(the reference computes the full S x S product)" %
                        (Bs, Ss, cfg["d"], cfg["nh"], procs, dt, rate / 1e9)),
                seconds=dt)


def run_reference_arm(args, cfg, rank, world):
    if rank != 0:
        return
    procs = os.cpu_count() or 1
    # each step is one bounded sample; size it so that warm-up + K steps stay within ~2.5 minutes
    per_step = max(1.0, min(15.0, 150.0 / max(1, args.steps + args.warmup)))
    vals = []
    for i in range(args.warmup + args.steps):
        r = cpu_baseline(cfg, per_step, procs)
        if i >= args.warmup:
            vals.append(r)
    value = float(np.mean([v["value"] for v in vals]))
    secs = float(np.mean([v["seconds"] for v in vals]))
    base = dict(vals[-1])
    base["value"] = value
    base.pop("seconds", None)
    line = dict(impl="reference", metric="attention_fwd_bwd_tokens_per_s", value=value, unit="tokens/s", n_gpus=world,
                steps=args.steps, warmup=args.warmup,
                # a step of this arm is one bounded sample (the full workload would take hours on the
                # CPU): ms_per_step is what a step really took; `value` extrapolates it to the workload
                ms_per_step=1e3 * secs, ms_per_workload_step_extrapolated=1e3 * cfg["B"] * cfg["S"] / value,
                higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f32", data="synthetic",
                config=dict(workload_config(args.workload, cfg, world), optimizer=args.optimizer), cpu_baseline=base,
                e2e=dict(value=value, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                sample_seconds_per_step=secs)
    print(json.dumps(line))


def l2_policy(cfg):
    """(flush, text).  A step reads and writes at least 14 activation-sized tensors (X, three projections, the
    attention output, the layer output, dOut, d(ctx), three projection gradients, three input gradients).
    When that stream is several times the 126 MB L2, nothing of one step survives into the next and steps
    are timed back to back; otherwise a 256 MB fill runs between separately timed steps."""
    es = 2 if cfg["mma"] == "bf16" else 4
    stream = 14.0 * cfg["B"] * cfg["S"] * cfg["d"] * es
    if stream > 3 * 126e6:
        return False, "inputs larger than L2: a step streams %.0f MB of activations through the 126 MB L2" % (stream / 1e6)
    return True, "L2 flushed between steps by a 256 MB fill"


def workload_config(name, cfg, world):
    what = "pre-LN encoder block step (LayerNorm, attention, residual, LayerNorm, dense 4d, GELU, dense, residual; MSE)" \
        if cfg.get("block") else "attention fwd+bwd"
    return dict(workload="%s: %s, batch=%d per GPU, seq=%d, d_model=%d, heads=%d (head_dim %d), %s, %s" %
                (name, what, cfg["B"], cfg["S"], cfg["d"], cfg["nh"], cfg["d"] // cfg["nh"],
                 "causal" if cfg["causal"] else "non-causal",
                 "BF16 storage, FP32 accumulate" if cfg["mma"] == "bf16" else "FP32 storage, TF32 MMA"),
                batch_per_gpu=cfg["B"], global_batch=cfg["B"] * world, seq_len=cfg["S"], d_model=cfg["d"],
                heads=cfg["nh"], causal=cfg["causal"], parallelism="dp%d over batch x heads units" % world,
                l2=l2_policy(cfg)[1])


def bind_to_gpu_numa_node(torch, local_rank):
    """Keeps this rank's threads (and so the page-locked host memory they first touch) on the NUMA node its GPU
    hangs off: at N ranks per host the host-tensor path otherwise pushes every rank's copies through one
    socket.  Reads the topology from sysfs; changes nothing on the GPU.  Returns a short description."""
    try:
        prop = torch.cuda.get_device_properties(local_rank)
        bdf = "%04x:%02x:%02x.0" % (prop.pci_domain_id, prop.pci_bus_id, prop.pci_device_id)
        with open("/sys/bus/pci/devices/%s/numa_node" % bdf) as f:
            node = int(f.read().strip())
        if node < 0:
            return "gpu %s reports no NUMA node" % bdf
        with open("/sys/devices/system/node/node%d/cpulist" % node) as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return "NUMA node %d has no CPU this process may use" % node
        os.sched_setaffinity(0, allowed)
        return "gpu %s on NUMA node %d: %d CPUs" % (bdf, node, len(allowed))
    except (OSError, ValueError, AttributeError) as e:
        return "not bound (%s)" % type(e).__name__


# ---- our arm -------------------------------------------------------------------------------------------------

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--optimizer", default="none", choices=["none", "adam"],
                    help="adam: every step ends with boat_optimizer_step over the attention parameters")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-tensor end-to-end measurement")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample")
    ap.add_argument("--clock-interval-ms", type=int, default=50,
                    help="nvidia-smi sampling period; much shorter periods slow down launch-bound workloads")
    args = ap.parse_args()
    cfg = dict(WORKLOADS[args.workload])
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, cfg, rank, world)
        return
    args.warmup = max(args.warmup, 3)
    # Libraries underneath (NCCL prints its version banner on stdout) must not get between the
    # caller and the one JSON line: everything but that line goes to stderr.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)

    import torch
    import boat_b200
    from boat_b200 import capi, rng, shard
    from boat_b200.host import Attention, Tensor, check

    lib = boat_b200.load()
    if lib.boat_cuda_device_count() < 1:
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    affinity = bind_to_gpu_numa_node(torch, local_rank) if world > 1 else "single rank: not bound"
    check(lib.boat_cuda_init(local_rank), "boat_cuda_init")
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        idbuf = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            raw = (C.c_ubyte * 128)()
            check(lib.boat_cuda_comm_unique_id(raw), "comm_unique_id")
            idbuf.copy_(torch.tensor(list(raw), dtype=torch.uint8))
        dist.broadcast(idbuf, 0)
        raw = (C.c_ubyte * 128)(*idbuf.cpu().tolist())
        check(lib.boat_cuda_comm_init(rank, world, raw), "comm_init")

    B, S, d, nh, causal = cfg["B"], cfg["S"], cfg["d"], cfg["nh"], cfg["causal"]
    bf16 = cfg["mma"] == "bf16"
    mma = capi.MMA_BF16 if bf16 else capi.MMA_TF32
    rnd = rng.bf16_round if bf16 else (lambda a: a)
    T = B * S

    # ---- synthetic inputs: X ~ N(0,1) (per-rank slice of the global batch), W ~ N(0, 1/sqrt(d)), dO ~ N(0,1)
    off = shard.element_offset(B * world, S, d, world, rank)
    x_host = rnd(rng.normal(SEED, rng.X, (B, S, d), offset=off))
    g_host = rnd(rng.normal(SEED, rng.DOUT, (B, S, d), offset=off))
    w_host = [rnd(rng.normal(SEED, rng.WQ + i, (d, d), 1.0 / np.sqrt(d))) for i in range(4)]

    is_block = bool(cfg.get("block"))
    block = None
    if is_block:
        from boat_b200.host import EncoderBlock
        std = 0.02
        params = dict(w=[rnd(rng.normal(SEED, rng.WQ + i, (d, d), std)) for i in range(4)],
                      w1=rnd(rng.normal(SEED, 40, (d, 4 * d), std)), w2=rnd(rng.normal(SEED, 41, (4 * d, d), std)))
        block = EncoderBlock(d, nh, causal=causal, device=capi.DEVICE_CUDA, mma=mma, params=params)
        layer = block.attn
    else:
        layer = Attention(d, nh, causal=causal, use_bias=True)
        for i, p in enumerate("qkvo"):
            layer.param("weight_" + p).set(w_host[i])
        layer.to_device(capi.DEVICE_CUDA)
        layer.set_precision(mma)
    if world > 1:
        # The backward itself starts the sum of dWo | dbo (it runs under the attention-core backward).  From
        # four ranks on it also starts the sum of the rest (mode 1), beside the input-gradient GEMMs, which are
        # then launched with one CTA per tile so that the collective's CTAs get SMs while they run: at N=4
        # 7.38-7.41 ms per step against 7.45-7.48 ms, the split problem 1.82 against 1.91 ms.  With two ranks
        # the sum is short and allreduce_grads() starts the rest and joins (mode 2); 0 sums everything at the end.
        overlap_mode = int(os.environ.get("BOAT_GRAD_OVERLAP", "1" if world >= 4 else "2"))
        layer.set_grad_overlap(overlap_mode)
    adam = None
    if args.optimizer == "adam":
        from boat_b200.host import Adam
        adam = Adam(1e-4)
        adam.add_attention(layer)
    x = Tensor.from_numpy(x_host, capi.DEVICE_CUDA, bf16=bf16)
    g = Tensor.from_numpy(g_host, capi.DEVICE_CUDA, bf16=bf16)    # upstream gradient (attention) or MSE target (block)
    flush = None
    if l2_policy(cfg)[0]:
        flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def block_step():
        out, dx = block.step(x, g)
        if world > 1:
            block.allreduce_grads()      # attention bucket, both LayerNorms, both dense layers
        block.zero_dense_grads()
        out.free()
        dx.free()

    def step():
        if is_block:
            block_step()
            if adam:
                adam.step()
            return
        out = layer.forward(x, x, x)
        gq, gk, gv = layer.backward(g)
        if world > 1:
            layer.allreduce_grads()
        if adam:
            adam.step()
        for t in (out, gq, gk, gv):
            t.free()

    def sync_all():
        check(lib.boat_cuda_sync(), "sync")
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    sampler = ClockSampler(local_rank, args.clock_interval_ms) if rank == 0 else None
    for _ in range(args.warmup):
        step()
    sync_all()
    mark0 = sampler.mark() if sampler else 0
    launches0 = lib.boat_cuda_launch_count()
    check(lib.boat_cuda_profile_enable(1), "profile_enable")
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    elapsed_ms = 0.0
    if flush is None:
        start.record()
        for _ in range(args.steps):
            step()
        stop.record()
        sync_all()
        elapsed_ms = start.elapsed_time(stop)
    else:
        for _ in range(args.steps):           # small workload: flush L2 outside the timed intervals
            flush.fill_(1)
            start.record()
            step()
            stop.record()
            torch.cuda.synchronize()
            elapsed_ms += start.elapsed_time(stop)
        sync_all()
    report = C.create_string_buffer(8192)
    check(lib.boat_cuda_profile_report(report, 8192), "profile_report")
    check(lib.boat_cuda_profile_enable(0), "profile_enable")
    launches = lib.boat_cuda_launch_count() - launches0
    clocks = sampler.stop(mark0, sampler.mark()) if sampler else None

    t = torch.tensor([elapsed_ms], dtype=torch.float64, device="cuda")
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t.item()) / args.steps
    tokens_per_s = world * T / (ms_per_step * 1e-3)
    flops = block_flops(B, S, d, causal) if is_block else algorithmic_flops(B, S, d, causal)
    tflops_per_gpu = flops / (ms_per_step * 1e-3) / 1e12

    # ---- data-parallel block: every parameter gradient summed exactly once?  The local gradients of one
    # step (no sums started) are added up over the ranks on the side (float64 checksums through
    # torch.distributed) and compared with what the overlapped, bucketed sums of the library leave.
    block_grad_check = None
    if world > 1 and is_block:
        def grad_checksums():
            check(lib.boat_cuda_sync(), "sync")
            arrays = [layer.param("grad_" + n).numpy() for n in ("weight_q", "weight_k", "weight_v", "weight_o",
                                                                  "bias_q", "bias_k", "bias_v", "bias_o")
                      if layer.param("grad_" + n) is not None]
            for part in (block.ln1, block.ln2, block.fc1, block.fc2):
                arrays += [a for a in part.grads() if a is not None]
            return torch.tensor([[float(a.astype(np.float64).sum()), float(np.abs(a.astype(np.float64)).sum())] for a in arrays],
                                dtype=torch.float64, device="cuda")
        block.zero_dense_grads()
        layer.set_grad_overlap(0)
        out, dx = block.step(x, g)                   # local gradients only
        local = grad_checksums()
        out.free(); dx.free()
        block.zero_dense_grads()
        dist.all_reduce(local, op=dist.ReduceOp.SUM)
        layer.set_grad_overlap(overlap_mode)
        out, dx = block.step(x, g)
        block.allreduce_grads()
        summed = grad_checksums()
        out.free(); dx.free()
        block.zero_dense_grads()
        err = float(((summed[:, 0] - local[:, 0]).abs() / local[:, 1].clamp_min(1e-30)).max().item())
        block_grad_check = dict(tensors=int(summed.shape[0]), rel_err=err, tolerance=1e-3,
                                what="max over the block's gradient tensors of |sum of the summed tensor - sum over ranks of "
                                     "the local tensor's sum| / sum over ranks of the local tensor's absolute sum")
        if not err <= 1e-3:
            raise SystemExit("bench.py: gradient sums of the block differ from the sum of the local gradients: %g" % err)

    # ---- strong scaling: the SAME problem (global batch = the per-GPU batch of the weak run) split over the
    # ranks by (batch, head) units, each rank holding only the token rows of its units ----
    strong = None
    if world > 1 and not is_block and (B * nh) % world == 0 and S % nh == 0:
        u = shard.head_unit_range(B, nh, world, rank)
        r0, r1 = shard.unit_rows(u, S, nh)
        xr = Tensor.from_numpy(rnd(rng.normal(SEED, rng.X, (r1 - r0, d), offset=r0 * d)), capi.DEVICE_CUDA, bf16=bf16)
        gr = Tensor.from_numpy(rnd(rng.normal(SEED, rng.DOUT, (r1 - r0, d), offset=r0 * d)), capi.DEVICE_CUDA, bf16=bf16)

        def strong_step():
            out = layer.forward_units(xr, S)
            gq, gk, gv = layer.backward(gr)
            layer.allreduce_grads()
            for tt in (out, gq, gk, gv):
                tt.free()

        def timed(fn, n):
            for _ in range(3):
                fn()
            sync_all()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(n):
                fn()
            e1.record()
            sync_all()
            tt = torch.tensor([e0.elapsed_time(e1) / n], dtype=torch.float64, device="cuda")
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            return float(tt.item())

        strong_ms = timed(strong_step, args.steps)

        def single_gpu_step():          # the whole problem on one GPU, no exchange: what N=1 does
            out = layer.forward(x, x, x)
            gq, gk, gv = layer.backward(g)
            for tt in (out, gq, gk, gv):
                tt.free()

        def bucket_to_host():
            ptr, n = C.POINTER(C.c_float)(), C.c_size_t()
            check(lib.boat_attention_grad_bucket(layer.h, C.byref(ptr), C.byref(n)), "grad_bucket")
            host = np.empty(n.value, np.float32)
            check(lib.boat_cuda_memcpy_d2h(host.ctypes.data_as(C.c_void_p), C.cast(ptr, C.c_void_p), host.nbytes), "d2h")
            return host

        # numbers, outside the timed regions: the bucket summed over the unit ranges must be the gradient of
        # the whole problem.  Rank 0's own (weak-scaling) batch IS that problem, so it can compute the latter alone.
        strong_step()
        sync_all()
        reduced = bucket_to_host()
        layer.set_grad_overlap(0)
        n1_ms = timed(single_gpu_step, max(3, min(args.steps, 10)))
        whole = bucket_to_host()
        layer.set_grad_overlap(overlap_mode)
        grad_err = float(np.abs(reduced.astype(np.float64) - whole).max() / np.abs(whole).max()) if rank == 0 else None
        strong = dict(workload="the %s problem at GLOBAL batch %d split by (batch, head) units: %d units = %d token rows per GPU" %
                      (args.workload, B, u[1] - u[0], r1 - r0), global_batch=B, units_per_gpu=u[1] - u[0],
                      rows_per_gpu=r1 - r0, ms_per_step=strong_ms, tokens_per_s=T / (strong_ms * 1e-3),
                      n1_ms_per_step=n1_ms, speedup_vs_n1=n1_ms / strong_ms,
                      grad_check=dict(rel_err=grad_err, tolerance=2e-2 if bf16 else 5e-3,
                                      what="max|sum over ranks of the unit-range gradient buckets - single-GPU bucket of "
                                           "the whole problem| / max|single-GPU bucket|, on rank 0"),
                      note="n1_ms_per_step: the whole problem on one GPU without exchange, timed in this run on every rank (max)")

    # ---- roofline of the dominant kernel family ----
    peaks = load_peaks()
    kern = {}
    for line in report.value.decode().splitlines():
        name, n, ms = line.split()
        kern[name] = (int(n), float(ms))
    core_c = 0.5 if causal else 1.0
    # Algorithmic FLOPs per STEP and kernel family.  A GEMM scope may hold several problems (the Q, K, V
    # projections, their weight and their input gradients run as one launch each), so the families are
    # counted per step: attention has four products of 2*T*d*d in each orientation, the encoder block
    # adds two dense products of 8*T*d*d in each.
    gemm_step = 8.0 * T * d * d + (16.0 * T * d * d if is_block else 0.0)
    kflops = {
        "gemm_tc_nn": gemm_step, "gemm_tc_nt": gemm_step, "gemm_tc_tn": gemm_step,
        "gemm_simt": gemm_step,
        "attn_fwd_tc": 4.0 * core_c * B * S * S * d, "attn_fwd_simt": 4.0 * core_c * B * S * S * d,
        "attn_bwd_tc": 8.0 * core_c * B * S * S * d, "attn_bwd_simt": 8.0 * core_c * B * S * S * d,
    }
    kbytes = {"adam_step": 28.0 * (4 * d * d + 4 * d)}     # p, g, m, v read; p, m, v written (FP32)
    roofline = None
    if kern:
        top = max((k for k in kern if k in kflops), key=lambda k: kern[k][1], default=None)
        if top:
            n, ms = kern[top]
            achieved = kflops[top] * args.steps / (ms * 1e-3) / 1e12
            # Denominator: the measured burst figure when the timed region is shorter than a second
            # (clocks have not settled under the power cap yet), the sustained one otherwise; both
            # fractions are on the line.  TF32 has no entry in MEASURED_PEAKS.json: it is measured
            # here, the same way (torch.matmul 8192^3, FP32 storage, TF32 allowed).
            region_s = ms_per_step * args.steps * 1e-3
            if bf16:
                burst, sustained, src = peaks["bf16"], peaks["bf16_sustained"], peaks["source"] + " bf16"
            else:
                burst, sustained = measure_tf32_peak(torch)
                src = "measured live: torch.matmul 8192^3, FP32 storage, TF32 allowed"
            use_burst = region_s < 1.0
            peak = burst if use_burst else sustained
            # DRAM traffic of that kernel from an ncu capture of the same tile shape, scaled by the number
            # of (batch, head) units (every unit of a shape moves the same bytes)
            traffic = None
            for cap in load_kernel_traffic():
                if (cap["kernel"], cap["S"], cap["hs"], bool(cap["causal"])) == (top, S, d // nh, bool(causal)):
                    traffic = cap["dram_bytes"] / cap["units"] * B * nh
            roofline = dict(bound="tensor", kernel=top, achieved=achieved, peak=peak, unit="TFLOP/s",
                            frac=achieved / peak, traffic=traffic,
                            launches=n, avg_ms=ms / n,
                            peak_source=src + (" burst" if use_burst else " sustained") +
                            " (timed region %.2f s)" % region_s,
                            frac_of_burst=achieved / burst, frac_of_sustained=achieved / sustained,
                            peak_burst=burst, peak_sustained=sustained,
                            kernels={k: dict(scopes=v[0], ms=round(v[1], 3), share=round(v[1] / sum(x[1] for x in kern.values()), 4))
                                     for k, v in sorted(kern.items(), key=lambda kv: -kv[1][1])})
            for k, nbytes in kbytes.items():
                if k in kern:
                    gbs = nbytes / (kern[k][1] / kern[k][0] * 1e-3) / 1e9
                    roofline["kernels"][k].update(hbm_gbs=round(gbs, 1), frac_of_hbm_peak=round(gbs / peaks["hbm"], 3))

    # ---- end to end through the public API with host tensors (rank 0 reports) ----
    e2e = None
    if not args.no_e2e and not is_block:
        host_layer = Attention(d, nh, causal=causal, use_bias=True)
        for i, p in enumerate("qkvo"):
            host_layer.param("weight_" + p).set(w_host[i])
        host_layer.set_precision(mma)
        hx = Tensor.from_numpy(x_host, capi.DEVICE_CPU, bf16=bf16)
        hg = Tensor.from_numpy(g_host, capi.DEVICE_CPU, bf16=bf16)

        def host_step():
            out = host_layer.forward(hx, hx, hx)
            gq, gk, gv = host_layer.backward(hg)
            loss_proxy = float(out.host_view().ravel()[0]) if not bf16 else 0.0   # touches the result on the host
            for tt in (out, gq, gk, gv):
                tt.free()
            return loss_proxy

        es = 2 if bf16 else 4
        n_e2e = max(5, min(args.steps, 20))
        for _ in range(2):               # warm-up: page-locked pool growth, copy streams, first-use set-up
            host_step()
        check(lib.boat_cuda_sync(), "sync")
        if dist is not None:
            dist.barrier()
        # Every step is timed on its own (wall clock, synchronised), and the median is reported: on
        # a shared host single steps now and then stall for tens of milliseconds without using CPU
        # time; the mean and the slowest step are given beside it.
        per_step = []
        for _ in range(n_e2e):
            t0 = time.perf_counter()
            host_step()
            check(lib.boat_cuda_sync(), "sync")
            per_step.append(time.perf_counter() - t0)
        per_step.sort()
        dt = per_step[len(per_step) // 2]
        dt_mean, dt_max = sum(per_step) / len(per_step), per_step[-1]
        te = torch.tensor([dt, dt_mean, dt_max], dtype=torch.float64, device="cuda")
        if dist is not None:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        dt, dt_mean, dt_max = (float(v) for v in te.tolist())
        wbytes = (4 * d * d + 4 * d) * 4
        e2e = dict(value=world * T / dt, unit="tokens/s", ms_per_step=dt * 1e3, steps=n_e2e,
                   ms_per_step_mean=dt_mean * 1e3, ms_per_step_max=dt_max * 1e3,
                   h2d_bytes_per_step=2 * T * d * es + 2 * wbytes,        # X, dOut, parameters for fwd and bwd
                   d2h_bytes_per_step=4 * T * d * es + wbytes,            # out, dq, dk, dv, parameter gradients
                   note="host BF16 tensors in and out through boat_attention_forward/backward; wall clock, median step" if bf16
                   else "host FP32 tensors in and out through boat_attention_forward/backward; wall clock, median step")
        host_layer.free()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu and not is_block:
        cpu = cpu_baseline(cfg, 12.0, 1)
        cpu.pop("seconds", None)

    if rank == 0:
        line = dict(metric="encoder_block_step_tokens_per_s" if is_block else "attention_fwd_bwd_tokens_per_s", value=tokens_per_s, unit="tokens/s", n_gpus=world,
                    steps=args.steps, warmup=args.warmup, ms_per_step=ms_per_step, higher_is_better=True,
                    scaling="weak", vs_baseline=None, dtype="bf16" if bf16 else "tf32", data="synthetic",
                    config=dict(workload_config(args.workload, cfg, world), optimizer=args.optimizer),
                    tflops_per_gpu=tflops_per_gpu,
                    frac_of_bf16_peak=(tflops_per_gpu / (peaks["bf16"] if ms_per_step * args.steps < 1e3 else peaks["bf16_sustained"])) if bf16 else None,
                    roofline=roofline, cpu_baseline=cpu, e2e=e2e, gpu_launches=int(launches), clocks=clocks)
        if block_grad_check is not None:
            line["grad_sum_check"] = block_grad_check
        if strong:
            line["strong"] = strong
        line["host_affinity"] = affinity
        sys.stdout.flush()
        os.write(json_fd, (json.dumps(line) + "\n").encode())
    if dist is not None:
        check(lib.boat_cuda_comm_destroy(), "comm_destroy")
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
