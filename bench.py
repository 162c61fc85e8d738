#!/usr/bin/env python
"""Benchmark of the JABAS/IIDP per-iteration gradient path on B200.

    python bench.py --gpus N --steps K --warmup W            # this library (N = 1: plain python;
                                                             # N > 1: launched by torch.distributed.run)
    python bench.py --impl reference --gpus N --steps K --warmup W   # CPU/gloo restatement

A "step" is one pass of the gradient path over one iteration's worth of gradients: K-VSW
aggregation -> (N > 1: cross-GPU reduction) -> fused optimizer update with write-back to the K
replicas, and the two-half cosine statistic.  The default workload is ResNet-50 (25,557,032
fp32 parameters in 5 buckets of at most 25 MiB, two param groups), 4 VSWs per GPU, local batch
64 per VSW, SGD momentum 0.9, statistic every iteration; gradients are synthetic N(0, 1e-3),
weights N(0, 1).

Rank 0 prints ONE JSON line.  ``value`` is samples/sec of the GRADIENT PATH ALONE with the
gradients resident in HBM (``metric_scope``); ``e2e`` is the same metric with every step's K
gradient sets copied from pinned host memory and the cosine read back inside the timed region;
``training_iteration`` is a whole training iteration (forward, backward, path) for context, eager and
(one GPU, or ``--train-graph``) as one CUDA-graph launch.

Timing: the ``--steps`` steps between two barriers are one sample; the sample is repeated until
at least half a second of device time has been measured, and ``ms_per_step`` is the median
sample (``timing`` holds min, max and the count).  Clocks are sampled across all samples.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (model, K, local batch per VSW, optimizer kind)
    "resnet50": ("resnet50", 4, 64, "sgd"),
    "vit_b_16": ("vit_b_16", 8, 32, "adamw"),
    "gnmt8": ("gnmt8", 2, 128, "adam"),
}
# (workload, K, optimizer) of the short extra passes reported under "configs"
EXTRA_CONFIGS = [("vit_b_16", None, None), ("gnmt8", None, None), ("flat27", 4, "sgd"), ("flat29", 8, "adamw")]
NVLINK_PEAK_GBS = 770.0        # measured peer-copy bandwidth per direction on this pool (nominal 900)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="resnet50",
                    help="resnet50 | vit_b_16 | gnmt8 | flat<log2 elements> (e.g. flat27)")
    ap.add_argument("--vsw", type=int, default=None, help="override K (VSWs per GPU)")
    ap.add_argument("--optimizer", default=None, choices=[None, "sgd", "adam", "adamw"])
    ap.add_argument("--similarity-mode", default="fused", choices=["fused", "pair_exchange"])
    ap.add_argument("--collective", default="peer", choices=["peer", "nccl"],
                    help="N > 1: cross-GPU exchange by this library's kernels over NVLink peer memory, or by NCCL")
    ap.add_argument("--peer-form", default="pipeline", choices=["pipeline", "direct"],
                    help="collective=peer: one pipelined kernel (default), or, on two GPUs, an aggregate kernel and "
                         "an update kernel that reads both ranks' sums")
    ap.add_argument("--no-similarity", action="store_true",
                    help="skip the two-half statistic (forced when T is odd, e.g. one GPU with one VSW)")
    ap.add_argument("--no-overlap", action="store_true")
    ap.add_argument("--per-bucket", default="auto", choices=["auto", "yes", "no"],
                    help="yes: walk the DDP buckets as the comm hooks do; no / auto: the whole flat model per launch")
    ap.add_argument("--share-weights", action="store_true",
                    help="the K replicas alias one weight buffer (no write-back to K-1 replicas); not the default")
    ap.add_argument("--staging", default="register", choices=["register", "bulk"],
                    help="how the update kernels fetch their tiles: per-thread 128-bit loads (default) or "
                         "TMA bulk copies into a shared-memory ring (one GPU, or NCCL)")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch every kernel / collective from Python instead of replaying one CUDA graph")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--train-graph", action="store_true",
                    help="on several GPUs too, time the training iteration as one CUDA-graph launch (one GPU: always)")
    ap.add_argument("--no-train-iter", action="store_true",
                    help="skip the supplementary whole-training-iteration measurement (resnet50 workload only)")
    ap.add_argument("--no-configs", action="store_true",
                    help="skip the short passes over the other benchmark configurations")
    ap.add_argument("--no-parity", action="store_true", help="N > 1: skip the check against the CPU/gloo restatement")
    ap.add_argument("--min-timed-ms", type=float, default=500.0,
                    help="repeat the --steps-long sample until this much device time has been measured")
    ap.add_argument("--cpu-steps", type=int, default=None)
    ap.add_argument("--stream-study", action="store_true",
                    help="instead of the benchmark: forward+backward of ResNet-50 for K x LBS images as one model, K "
                         "models serially, K models on K streams (one thread / K threads); prints one JSON line")
    return ap.parse_args()


def make_workload(name, vsw=None, optimizer=None):
    from jabas_b200.layout import build_layout, model_zoo_shapes
    if name.startswith("flat"):
        n = 1 << int(name[4:])
        K, lbs, kind = vsw or 4, 64, optimizer or "sgd"
        layout = build_layout(["flat"], [(n,)], [0], bucket_cap_mb=1 << 30, first_bucket_bytes=1 << 62)
        desc = f"flat fp32 buffer of 2^{name[4:]} elements"
    else:
        model, K, lbs, kind = WORKLOADS[name]
        K, kind = vsw or K, optimizer or kind
        names, shapes, groups = model_zoo_shapes(model)
        layout = build_layout(names, shapes, groups)
        desc = f"{model} parameter layout"
    if kind == "sgd":
        wds = [0.0, 1e-4]
        opt = dict(kind="sgd", groups=[dict(lr=0.1, weight_decay=w) for w in wds], momentum=0.9)
    elif kind == "adamw":
        opt = dict(kind="adamw", groups=[dict(lr=1e-3, weight_decay=w) for w in (0.0, 0.05)],
                   betas=(0.9, 0.999), eps=1e-8)
    else:
        opt = dict(kind="adam", groups=[dict(lr=2e-3, weight_decay=0.0)] * 2, betas=(0.9, 0.999), eps=1e-8)
    return layout, K, lbs, opt, desc


def config_dict(args, layout, K, lbs, opt, desc, world):
    return {
        "workload": args.workload, "layout": desc, "params": layout.num_params,
        "buckets_mib": layout.bucket_sizes_mib(), "vsw_per_gpu": K, "local_batch_per_vsw": lbs,
        "global_batch": world * K * lbs, "optimizer": opt["kind"], "param_groups": len(opt["groups"]),
        "similarity": "every iteration", "similarity_mode": args.similarity_mode if world > 1 else "vsw_parity",
        "overlap": not args.no_overlap,
        "cuda_graph": (not args.no_graph) and args.impl == "ours",
        "replica_weights": "one shared buffer" if getattr(args, "share_weights", False) else "K separate buffers",
        "staging": getattr(args, "staging", "register"),
        "collective": (("peer-memory kernels over NVLink, " + args.peer_form) if args.collective == "peer"
                       else "NCCL allreduce") if world > 1 else "none",
        "launch_granularity": "bucket" if args.per_bucket == "yes" else "whole flat model",
        "parallelism": f"dp{world} x vsw{K}",
        "l2": "inputs larger than L2: %.0f MB of gradients, weights and state per GPU vs 126 MB"
              % (4 * layout.total * (2 * K + 2) / 1e6),
    }


# --------------------------------------------------------------------------------------
# clocks, NUMA
# --------------------------------------------------------------------------------------

class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.path = index, None, None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 8:
                    continue
                try:
                    sm.append(float(f[0])); mx.append(float(f[1]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                      "sw_power_cap"), f[4:8]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            sm.sort()
            out.update(sm_mhz=sm[len(sm) // 2], sm_max_mhz=max(mx), samples=len(sm))
        out["reasons"] = sorted(reasons)
        return out


def bind_to_gpu_numa(local_rank: int):
    """Run this process on the CPUs of the NUMA node its GPU hangs off, so that the pinned host
    buffers of the end-to-end leg are first touched (and therefore placed) there."""
    info = {"numa_node": None, "cpus_bound": None}
    try:
        q = subprocess.run(["nvidia-smi", "-i", str(local_rank), "--query-gpu=pci.bus_id", "--format=csv,noheader"],
                           capture_output=True, text=True, timeout=20).stdout.strip().lower()
        bus = q[-12:] if len(q) >= 12 else q                 # 0000:xx:yy.z
        node = int(open(f"/sys/bus/pci/devices/{bus}/numa_node").read())
        info["numa_node"] = node
        if node >= 0:
            cpus = []
            for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
                a, _, b = part.partition("-")
                cpus.extend(range(int(a), int(b or a) + 1))
            allowed = sorted(set(cpus) & os.sched_getaffinity(0))
            if allowed:
                os.sched_setaffinity(0, allowed)
                info["cpus_bound"] = len(allowed)
    except Exception as e:                                   # best effort: containers often hide sysfs
        info["note"] = f"{type(e).__name__}"
    return info


# --------------------------------------------------------------------------------------
# CPU restatement (cpu_baseline leg and --impl reference)
# --------------------------------------------------------------------------------------

def _cpu_worker(rank, world, port, layout, K, opt, steps, warmup, threads, q, budget_s=60.0):
    import torch
    import torch.distributed as dist
    from oracle.reference_path import ReferencePath
    torch.set_num_threads(max(1, threads))
    # When the parent is a torchrun worker its environment says "the elastic agent hosts the
    # rendezvous store"; these CPU ranks rendezvous among themselves on their own port instead.
    for var in [v for v in os.environ if v.startswith("TORCHELASTIC_")]:
        os.environ.pop(var, None)
    if world > 1:
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    ref = ReferencePath(layout, K, opt, total_num_decoupled_workers=world * K, similarity=True, arith="torch",
                        world=world)
    gen = torch.Generator().manual_seed(7)
    ref.weights[0].normal_(generator=gen)
    for k in range(1, K):
        ref.weights[k].copy_(ref.weights[0])
    for k in range(K):
        g = torch.Generator().manual_seed(1000 * rank + k)
        ref.grads[k].normal_(0.0, 1e-3, generator=g)
    for _ in range(max(1, min(warmup, 3))):
        ref.run_iteration()
    if world > 1:
        dist.barrier()
    # Bounded sample: at most `steps` iterations, and no more than `budget_s` seconds of them.
    stop = torch.zeros(1, dtype=torch.int32)
    done = 0
    t0 = time.perf_counter()
    while done < steps:
        ref.run_iteration()
        done += 1
        stop[0] = 1 if (time.perf_counter() - t0) > budget_s else 0
        if world > 1:
            dist.all_reduce(stop, op=dist.ReduceOp.MAX)
        if int(stop[0]):
            break
    if world > 1:
        dist.barrier()
    dt = (time.perf_counter() - t0) / done * steps          # seconds for `steps` iterations at the sampled rate
    if rank == 0:
        q.put((dt, done))
    if world > 1:
        dist.destroy_process_group()


def run_cpu_path(layout, K, opt, world, steps, warmup, budget_s=60.0):
    """Seconds for `steps` iterations of the CPU/gloo restatement with `world` ranks that
    share this host's cores."""
    import torch.multiprocessing as mp
    cores = os.cpu_count() or 1
    threads = max(1, cores // world)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29650 + (os.getpid() % 200)
    if world == 1:
        import queue
        qq = queue.Queue()
        _cpu_worker(0, 1, port, layout, K, opt, steps, warmup, threads, qq, budget_s)
        dt, done = qq.get()
        return dt, cores, threads, done
    procs = [ctx.Process(target=_cpu_worker, args=(r, world, port, layout, K, opt, steps, warmup, threads, q,
                                                   budget_s)) for r in range(world)]
    for p in procs:
        p.start()
    dt, done = q.get(timeout=1800)
    for p in procs:
        p.join()
    return dt, cores, threads, done


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    layout, K, lbs, opt, desc = make_workload(args.workload, args.vsw, args.optimizer)
    world = args.gpus
    dt, cores, threads, done = run_cpu_path(layout, K, opt, world, args.steps, args.warmup, budget_s=90.0)
    ms = dt / args.steps * 1e3
    value = world * K * lbs / (ms / 1e3)
    cfg = config_dict(args, layout, K, lbs, opt, desc, world)
    cfg["similarity_mode"] = "pair_exchange" if world > 1 else "vsw_parity"
    cfg["collective"] = "gloo allreduce" if world > 1 else "none"
    sample = (f"{done} full iterations of the workload (of {args.steps} asked; at most 90 s are sampled) after "
              f"{max(1, min(args.warmup, 3))} warm-up, {world} gloo rank(s) x {threads} torch threads on {cores} host cores")
    n = layout.num_params
    multi = world > 1
    per = (K + 4) if opt["kind"] == "sgd" else (K + 6)
    unfused = 4 * n * (K + 1) + 4 * n * per + (8 * n if multi else 0)
    line = {
        "impl": "reference", "metric": "samples/sec", "metric_scope": "gradient path only", "value": value,
        "unit": "samples/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": cfg,
        "cpu_baseline": {"value": value, "unit": "samples/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gradient_path_gbs_per_rank": unfused / (ms / 1e3) / 1e9,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------
# this library
# --------------------------------------------------------------------------------------

class Dist:
    """World, rank, device and the parity sub-groups of a run."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus:
            raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={self.world}: launch with torch.distributed.run")
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        self.sub_group = self.pair_group = None
        if self.world > 1:
            import datetime
            if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
                os.environ["NCCL_DEBUG"] = "WARN"       # keep stdout to the one JSON line
            # gloo beside NCCL: the parity check runs the CPU restatement over the same ranks
            dist.init_process_group("cpu:gloo,cuda:nccl", timeout=datetime.timedelta(seconds=300))
            idx = [[r for r in range(self.world) if r % 2 == p] for p in (0, 1)]
            groups = [dist.new_group(ix) for ix in idx]
            self.sub_group = groups[self.rank % 2]
            self.pair_group = dist.new_group([idx[0][0], idx[1][0]])
            self._tok = torch.zeros(1, device=self.dev)
            dist.all_reduce(self._tok)                    # bring the NCCL communicator up now

    def barrier(self):
        if self.world > 1:
            self.dist.all_reduce(self._tok)               # NCCL, on the device
        self.torch.cuda.synchronize()

    def max_over_ranks(self, x: float) -> float:
        if self.world == 1:
            return x
        t = self.torch.tensor([x], dtype=self.torch.float64, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t)

    def all_ok(self, ok: bool) -> bool:
        if self.world == 1:
            return ok
        t = self.torch.tensor([1.0 if ok else 0.0], device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MIN)
        return bool(float(t) > 0.5)


def build_engine(D, args, layout, K, opt, collective, similarity=None):
    from jabas_b200.gradient_path import GradientPath, OptimizerSpec
    spec = OptimizerSpec(kind=opt["kind"], groups=[dict(g) for g in opt["groups"]], momentum=opt.get("momentum", 0.0),
                         betas=opt.get("betas", (0.9, 0.999)), eps=opt.get("eps", 1e-8))
    if similarity is None:
        similarity = not args.no_similarity and (D.world * K) % 2 == 0 and (D.world > 1 or K % 2 == 0)
    return GradientPath(layout, K, D.dev, spec, total_num_decoupled_workers=D.world * K,
                        sub_group=D.sub_group, pair_group=D.pair_group, similarity=similarity,
                        similarity_mode=args.similarity_mode, collective=collective,
                        share_weights=args.share_weights, staging=args.staging, peer_form=args.peer_form)


def seed_engine(D, eng, K, share_weights=False, seed_shift=0):
    torch = D.torch
    gen = torch.Generator(device=D.dev).manual_seed(7 + seed_shift)
    eng.weights[0].normal_(generator=gen)
    if not share_weights:
        for k in range(1, K):
            eng.weights[k].copy_(eng.weights[0])
    for k in range(K):
        g = torch.Generator(device=D.dev).manual_seed(1000 * D.rank + k + seed_shift)
        eng.grads[k].normal_(0.0, 1e-3, generator=g)


def time_engine(D, eng, args, steps, warmup, min_total_ms, use_graph, overlap, per_bucket):
    """Median-of-samples timing of `steps` steps, per-launch time of one replay, and the split
    between kernels from an eager pass with one event pair per kernel."""
    torch = D.torch
    eager_fn = lambda: eng.run_iteration(overlap=overlap, per_bucket=per_bucket)
    if use_graph:
        eng.capture(overlap=overlap, per_bucket=per_bucket, warmup=2)
    step_fn = eng.replay if use_graph else eager_fn
    for _ in range(max(warmup, 3)):
        step_fn()
    D.barrier()
    if getattr(eng, "exchange", None) is not None and not D.all_ok(eng.exchange.status()[0] == 0):
        # a bounded wait already ran out during warm-up: nothing worth timing (the caller falls back)
        return {"ms_per_step": float("nan"), "min": 0.0, "max": 0.0, "samples": 0, "spread": 0.0, "timed_ms_total": 0.0,
                "single_step_ms": float("nan"), "split": {}, "launches_per_step": 0.0, "step_fn": step_fn,
                "eager_fn": eager_fn}
    launches0 = eng.launches
    samples = []
    total_ms, reps = 0.0, 0
    while True:
        D.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step_fn()
        e1.record()
        D.barrier()
        ms = D.max_over_ranks(e0.elapsed_time(e1))
        samples.append(ms / steps)
        total_ms += ms
        reps += 1
        if (total_ms >= min_total_ms and reps >= 3) or reps >= 400:
            break
    launches_per_step = (eng.launches - launches0) / (reps * steps)
    samples.sort()
    med = samples[len(samples) // 2]
    # one event pair per step: the device time of ONE replay / iteration, back to back
    D.barrier()
    n_single = max(10, min(steps, 100))
    pairs = []
    for _ in range(n_single):
        a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); step_fn(); z.record()
        pairs.append((a, z))
    D.barrier()
    single = sorted(a.elapsed_time(z) for a, z in pairs)
    single_ms = D.max_over_ranks(single[len(single) // 2])
    # the split between kernels: eager launches, one event pair each
    eng.profile_events = []
    n_split = max(5, min(steps, 50))
    for _ in range(n_split):
        eager_fn()
    D.barrier()
    events, eng.profile_events = eng.profile_events, None
    per_kernel = {}
    for kind, b, a, z in events:
        d = per_kernel.setdefault(kind, [0.0, 0])
        d[0] += a.elapsed_time(z)
        d[1] += 1
    split = {k: {"launches_per_step": v[1] / n_split, "ms_per_step": v[0] / n_split} for k, v in per_kernel.items()}
    return {"ms_per_step": med, "min": samples[0], "max": samples[-1], "samples": reps,
            "spread": (samples[-1] - samples[0]) / med if med > 0 else 0.0, "timed_ms_total": total_ms,
            "single_step_ms": single_ms, "split": split, "launches_per_step": launches_per_step,
            "step_fn": step_fn, "eager_fn": eager_fn}


def exchange_ok_everywhere(D, eng) -> None:
    """Raise on EVERY rank if a bounded wait of the pipelined exchange ran out on ANY rank, so that
    all ranks leave the measurement together (a one-sided exception would strand the others in
    their next collective)."""
    status = eng.exchange.status()[0] if getattr(eng, "exchange", None) is not None else 0
    if not D.all_ok(status == 0):
        raise RuntimeError(f"pipelined exchange: a bounded wait ran out on some rank (this rank's status {status:#x})")


def hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback"


def traffic_ratio(kernel: str):
    """DRAM bytes / algorithmic bytes of one profiler capture of a kernel (data file shipped with
    the package); None when the kernel has never been captured."""
    try:
        table = json.load(open(os.path.join(ROOT, "jabas_b200", "data", "dram_traffic_ratio.json")))
        return table["kernels"].get(kernel)
    except Exception:
        return None


def roofline_of(eng, T, alg, world, peak, peak_src):
    """Roofline record of the dominant kernel.  One GPU: HBM.  Several GPUs with the pipelined
    exchange: one kernel bounded by the slower of its HBM bytes and its NVLink bytes."""
    split = T["split"]
    dom = max(split, key=lambda k: split[k]["ms_per_step"])
    lps = max(1.0, split[dom]["launches_per_step"])
    whole = len(split) == 1 or (dom == "exchange")
    # a step that is one kernel (plus, with the exchange, the 32-thread statistic kernel): the
    # launch time is the per-step time measured around single replays; otherwise the eager split
    # (the smaller of that and the median back-to-back step time: a step also holds the 288-byte
    # hyper-parameter copy and the graph launch, so either figure is an upper bound on the kernel)
    launch_ms = (min(T["single_step_ms"], T["ms_per_step"]) if whole else split[dom]["ms_per_step"]) / lps
    alg_launch = alg[dom] / lps
    rec = {"kernel": dom, "launches_per_step": lps, "launch_ms": launch_ms,
           "algorithmic_bytes_per_launch": alg_launch, "peak_source": peak_src}
    hbm_gbs = alg_launch / (launch_ms / 1e3) / 1e9
    if dom == "exchange":
        nv = alg["nvlink_in"] / lps
        t_hbm, t_nv = alg_launch / (peak * 1e9), nv / (NVLINK_PEAK_GBS * 1e9)
        nv_gbs = nv / (launch_ms / 1e3) / 1e9
        if t_nv >= t_hbm:
            rec.update(bound="nvlink", achieved=nv_gbs, peak=NVLINK_PEAK_GBS, unit="GB/s", frac=nv_gbs / NVLINK_PEAK_GBS)
        else:
            rec.update(bound="hbm", achieved=hbm_gbs, peak=peak, unit="GB/s", frac=hbm_gbs / peak)
        rec.update(hbm_gbs=hbm_gbs, hbm_frac=hbm_gbs / peak, nvlink_in_gbs=nv_gbs,
                   nvlink_frac_of_measured_770=nv_gbs / NVLINK_PEAK_GBS, nvlink_frac_of_nominal_900=nv_gbs / 900.0,
                   nvlink_in_bytes_per_launch=nv, target_ms=max(t_hbm, t_nv) * 1e3,
                   frac_of_target=max(t_hbm, t_nv) * 1e3 / launch_ms, traffic=None)
    else:
        ratio = traffic_ratio(dom) if world == 1 else None
        rec.update(bound="hbm", achieved=hbm_gbs, peak=peak, unit="GB/s", frac=hbm_gbs / peak,
                   traffic=None if ratio is None else ratio["ratio"] * alg_launch,
                   traffic_source=None if ratio is None else
                   "scaled: DRAM bytes / algorithmic bytes of one earlier profiler capture of this kernel "
                   f"({ratio['captured_on']}) x this launch's algorithmic bytes; not measured in this run")
    return rec


def run_ours(args):
    import torch
    D = Dist(args)
    dist, world, rank, dev = D.dist, D.world, D.rank, D.dev
    numa = bind_to_gpu_numa(D.local_rank)
    layout, K, lbs, opt, desc = make_workload(args.workload, args.vsw, args.optimizer)
    similarity = not args.no_similarity and (world * K) % 2 == 0 and (world > 1 or K % 2 == 0)
    collective, collective_note = args.collective, None
    if world > 1 and args.staging == "bulk" and collective == "peer":
        collective, collective_note = "nccl", "staging=bulk reads through TMA bulk copies: local memory only, NCCL exchange"
    try:
        eng = build_engine(D, args, layout, K, opt, collective)
        ok = True
    except Exception as e:
        if world == 1 or collective != "peer":
            raise
        ok, err = False, f"peer-memory set-up failed ({type(e).__name__}: {e})"[:200]
    if world > 1 and collective == "peer" and not D.all_ok(ok):
        # peer mappings could not be set up on some rank: every rank goes through NCCL instead
        collective, collective_note = "nccl", (err if not ok else "peer-memory set-up failed on another rank")
        eng = build_engine(D, args, layout, K, opt, "nccl")
    seed_engine(D, eng, K, args.share_weights)
    overlap = not args.no_overlap
    per_bucket = None if args.per_bucket == "auto" else (args.per_bucket == "yes")
    use_graph = not args.no_graph

    sampler = ClockSampler(D.local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.2)
    T = time_engine(D, eng, args, args.steps, args.warmup, args.min_timed_ms, use_graph, overlap, per_bucket)
    if world > 1 and eng.exchange is not None:
        status = eng.exchange.status()[0]
        if not D.all_ok(status == 0):
            # a bounded wait of the pipelined exchange ran out on some rank (a rank fell more than the
            # wait limit behind): the measurement is void; every rank redoes it over NCCL and says so
            collective, collective_note = "nccl", f"pipelined exchange gave up (status {status:#x} on rank {rank}); NCCL"
            T.pop("step_fn", None); T.pop("eager_fn", None)
            eng.close()
            del eng
            gc.collect()
            torch.cuda.empty_cache()
            eng = build_engine(D, args, layout, K, opt, "nccl")
            seed_engine(D, eng, K, args.share_weights)
            T = time_engine(D, eng, args, args.steps, args.warmup, args.min_timed_ms, use_graph, overlap, per_bucket)
    clocks = sampler.stop() if rank == 0 else None
    ms_step = T["ms_per_step"]
    step_fn = T["step_fn"]
    cos = float(eng.cos)
    if args.staging == "bulk" and eng.ctx.staging_timeouts() != 0:
        raise RuntimeError("bulk staging: a wait for a copy ran out; the timed steps are incomplete")
    alg = eng.algorithmic_bytes(similarity)
    peak, peak_src = hbm_peak()
    roof = roofline_of(eng, T, alg, world, peak, peak_src)
    launched_bytes = sum(alg[k] for k in T["split"] if k in alg)

    bus = measure_allreduce(D, layout) if world > 1 else None

    # ---- end to end: host gradients in, cosine out ----------------------------------
    e2e = None
    if not args.no_e2e:
        host = [torch.empty(layout.total, dtype=torch.float32, pin_memory=True) for _ in range(K)]
        for k in range(K):
            g = torch.Generator(device=dev).manual_seed(1000 * rank + k)
            host[k].copy_(torch.empty(layout.total, device=dev).normal_(0.0, 1e-3, generator=g))
        cos_host = torch.empty(1, dtype=torch.float32, pin_memory=True)

        def e2e_step():
            for k in range(K):
                eng.grads[k].copy_(host[k], non_blocking=True)
            c = step_fn()
            cos_host.copy_(c if c is not None else eng.cos, non_blocking=True)
            torch.cuda.current_stream().synchronize()      # the caller reads the statistic

        for _ in range(3):
            e2e_step()
        D.barrier()
        n_e2e = max(5, min(args.steps, 30))
        a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n_e2e):
            e2e_step()
        z.record()
        D.barrier()
        ms_e2e = D.max_over_ranks(a.elapsed_time(z) / n_e2e)
        e2e = {"value": world * K * lbs / (ms_e2e / 1e3), "unit": "samples/s",
               "h2d_bytes_per_step": 4 * layout.total * K, "d2h_bytes_per_step": 4,
               "ms_per_step": ms_e2e, "steps": n_e2e, "h2d_gbs_per_gpu": 4 * layout.total * K / (ms_e2e / 1e3) / 1e9,
               "host_placement": numa,
               "api": "GradientPath.run_iteration over the C ABI; gradients from pinned host memory"}
        del host

    # ---- N > 1: one seeded iteration against the CPU/gloo restatement over the same ranks ----
    parity = None
    if world > 1 and not args.no_parity:
        parity = parity_check(D, args, layout, K, opt, collective)

    eng.close()
    del eng, step_fn, T["step_fn"], T["eager_fn"]
    gc.collect()
    torch.cuda.empty_cache()

    configs = None
    if not args.no_configs and args.workload == "resnet50":
        configs = {}
        for name, vsw, okind in EXTRA_CONFIGS:
            configs[f"{name}" + (f"_k{vsw}_{okind}" if vsw else "")] = run_extra_config(D, args, name, vsw, okind, collective)

    train_iter = None
    if args.workload == "resnet50" and not args.no_train_iter:
        train_iter = measure_training_iteration(D, K, lbs, collective, graph=args.train_graph)

    if rank != 0:
        finish(D)
        return

    kern = {k: dict(v, gbs=(alg[k] / (v["ms_per_step"] / 1e3) / 1e9 if k in alg and v["ms_per_step"] > 0 else None))
            for k, v in T["split"].items()}
    line = {
        "metric": "samples/sec", "metric_scope": "gradient path only (forward/backward are not part of the step; "
                                                 "see training_iteration for a whole iteration)",
        "value": world * K * lbs / (ms_step / 1e3), "unit": "samples/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": dict(config_dict(args, layout, K, lbs, opt, desc, world),
                                            similarity="every iteration" if similarity else "off",
                                            **({"collective": "NCCL allreduce", "collective_note": collective_note}
                                               if collective_note else {})),
        "timing": {k: T[k] for k in ("min", "max", "samples", "spread", "timed_ms_total", "single_step_ms")},
        # bytes of the kernels that actually ran in a step / step time
        "gradient_path_gbs_per_gpu": launched_bytes / (ms_step / 1e3) / 1e9,
        # the same time credited with the bytes of the unfused aggregate + update pair (what a
        # two-kernel implementation would move); a comparison figure, never a fraction of peak
        "equivalent_unfused_gbs": alg["total"] / (ms_step / 1e3) / 1e9,
        "roofline": roof, "kernels": kern,
        "gpu_launches": int(round(T["launches_per_step"] * args.steps)), "cosine": cos, "clocks": clocks, "e2e": e2e,
    }
    if parity is not None:
        line["parity"] = parity
    if configs is not None:
        line["configs"] = configs
    if train_iter is not None:
        line["training_iteration"] = train_iter
    if bus is not None:
        line["allreduce"] = bus
    if not args.no_cpu_baseline and world == 1:      # the CPU baseline is reported at N = 1 only
        cpu_steps = args.cpu_steps or 10
        dt, cores, threads, done = run_cpu_path(layout, K, opt, 1, cpu_steps, 2, budget_s=30.0)
        line["cpu_baseline"] = {
            "value": K * lbs / (dt / cpu_steps), "unit": "samples/s", "cores": cores, "kind": "port",
            "ms_per_step": dt / cpu_steps * 1e3,
            "sample": f"{done} iterations of this workload at one rank (K={K}) after 2 warm-up, "
                      f"stock torch CPU ops, {threads} threads"}
    print(json.dumps(line), flush=True)
    finish(D)


def finish(D):
    """Orderly exit of a multi-rank run.  Everything that holds device work or peer mappings
    alive (captured graphs, exchange handles, symmetric-memory buffers) has been released by
    the engines' close(); what is left is a last barrier and the process group.  A watchdog
    thread bounds the teardown: if it has not returned after 60 s the process leaves anyway and
    says so on stderr (the result line is already out)."""
    if D.world == 1:
        return
    gc.collect()
    D.torch.cuda.synchronize()
    D.barrier()
    sys.stdout.flush()

    def _watchdog():
        sys.stderr.write("bench: process-group teardown exceeded 60 s; leaving without it\n")
        sys.stderr.flush()
        os._exit(0)
    timer = threading.Timer(60.0, _watchdog)
    timer.daemon = True
    timer.start()
    D.dist.destroy_process_group()
    timer.cancel()


def parity_check(D, args, layout, K, opt, collective):
    """One seeded iteration of the CUDA path against ``oracle.reference_path`` run by the same
    ranks over gloo (outside every timed region).  Reports the largest relative weight error, the
    cosine difference and whether all ranks hold the same bits."""
    import numpy as np
    torch, dist = D.torch, D.dist
    from oracle.reference_path import ReferencePath
    out = {}
    try:
        eng = build_engine(D, args, layout, K, opt, collective)
        seed_engine(D, eng, K, args.share_weights, seed_shift=31)
        pad = torch.ones(layout.total, dtype=torch.bool, device=D.dev)
        for b, e in layout.buckets:
            pad[b:e] = False
        for t in list(eng.weights) + list(eng.grads):     # padding between buckets is zero and stays zero
            t[pad] = 0.0
        ref = ReferencePath(layout, K, opt, total_num_decoupled_workers=D.world * K, arith="c", world=D.world)
        for k in range(K):
            ref.weights[k].copy_(eng.weights[0].cpu())
            ref.grads[k].copy_(eng.grads[k].cpu())
        cos = float(eng.run_iteration())
        torch.cuda.synchronize()
        exchange_ok_everywhere(D, eng)
        cos_ref = ref.run_iteration()
        w, wr = eng.weights[K - 1].cpu(), ref.weights[0]
        rel = float(((w - wr).abs() / wr.abs().clamp_min(1e-3)).max())
        chk = int(eng.weights[0].view(torch.int32).to(torch.int64).sum())
        sums = [None] * D.world
        dist.all_gather_object(sums, (chk, cos))
        rels = [None] * D.world
        dist.all_gather_object(rels, rel)
        out = {"max_rel_w": max(rels), "cos_abs": abs(cos - cos_ref), "ranks_bit_identical": len(set(sums)) == 1,
               "against": "oracle.reference_path (C arithmetic) over gloo on the same ranks, one iteration",
               "tolerance": {"max_rel_w": 1e-6, "cos_abs": 1e-5}}
        eng.close()
        del eng, ref
        gc.collect()
        torch.cuda.empty_cache()
    except Exception as e:                                  # reported, never fatal to the benchmark line
        out = {"error": f"{type(e).__name__}: {e}"[:300]}
    return out


def run_extra_config(D, args, name, vsw, okind, collective):
    """A short pass of another benchmark configuration, after the headline measurement."""
    torch = D.torch
    try:
        layout, K, lbs, opt, desc = make_workload(name, vsw, okind)
        eng = build_engine(D, args, layout, K, opt, collective)
        seed_engine(D, eng, K, args.share_weights)
        sampler = ClockSampler(D.local_rank)
        if D.rank == 0:
            sampler.start()
        steps = 20 if layout.num_params < (1 << 28) else 8
        T = time_engine(D, eng, args, steps, 3, 150.0, not args.no_graph, True, None)
        clocks = sampler.stop() if D.rank == 0 else None
        exchange_ok_everywhere(D, eng)
        sim = eng.similarity
        alg = eng.algorithmic_bytes(sim)
        peak, peak_src = hbm_peak()
        roof = roofline_of(eng, T, alg, D.world, peak, peak_src)
        out = {"params": layout.num_params, "vsw_per_gpu": K, "optimizer": opt["kind"],
               "ms_per_step": T["ms_per_step"], "min": T["min"], "samples": T["samples"],
               "samples_per_sec": D.world * K * lbs / (T["ms_per_step"] / 1e3),
               "kernel": roof["kernel"], "bound": roof["bound"], "achieved_gbs": roof["achieved"],
               "frac_of_peak": roof["frac"], "peak": roof["peak"], "launch_ms": roof["launch_ms"],
               "cosine": float(eng.cos), "clocks": clocks}
        if roof["kernel"] == "exchange":
            out.update(hbm_gbs=roof["hbm_gbs"], nvlink_in_gbs=roof["nvlink_in_gbs"],
                       nvlink_frac_of_nominal_900=roof["nvlink_frac_of_nominal_900"],
                       frac_of_target=roof["frac_of_target"])
        eng.close()
        del eng, T
        gc.collect()
        torch.cuda.empty_cache()
        if D.world > 1 and name == "flat27":
            out["allreduce"] = measure_allreduce(D, layout)
        return out
    except Exception as e:
        gc.collect()
        torch.cuda.empty_cache()
        return {"error": f"{type(e).__name__}: {e}"[:300]}


def measure_training_iteration(D, K, lbs, collective, iters=8, graph=False):
    """Supplementary: WHOLE training iterations through the trainer mirror — K VSWs' forward and
    backward of torchvision ResNet-50 (stock PyTorch / cuDNN kernels, fp32 with TF32 convolutions) on K
    streams, comm hooks fired per bucket from backward, this library's path overlapping the rest of
    backward — on synthetic N(0,1) images.  Reports samples/sec over all ranks, the EXPOSED time
    of the gradient path (iteration time minus the time of forward + backward alone) and, on one
    GPU, the same iteration as one CUDA-graph launch, at the benchmark's local batch size and at
    the launch-bound local batch size 8 of the reference's CPU-runnable configuration."""
    out = _training_case(D, K, lbs, collective, iters, graph=(D.world == 1 or graph))
    if D.world == 1 and "error" not in out:
        small = _training_case(D, K, 8, collective, iters, graph=True)
        out["local_batch_8"] = {k: small[k] for k in ("ms_per_iteration", "samples_per_sec", "graph", "error")
                                if k in small}
    return out


def _training_case(D, K, lbs, collective, iters, graph):
    torch = D.torch
    ok, err, tr = True, None, None
    try:                                               # local part: no collective may sit in here
        import torchvision
        import jabas_b200
        from jabas_b200.iidp.optim import ShardSGD
        torch.manual_seed(0)
        model = torchvision.models.resnet50().to(D.dev)
        x = torch.randn(K * lbs, 3, 224, 224, device=D.dev)
        y = torch.randint(0, 1000, (K * lbs,), device=D.dev)
    except Exception as e:
        ok, err = False, f"{type(e).__name__}: {e}"[:300]
    if not D.all_ok(ok):                               # every rank takes the same branch
        return {"error": err or "set-up failed on another rank"}
    try:
        cfg = dict(similarity_target=0.1, batch_size_adjust_interval=1, enable_adjust=False)
        tr = jabas_b200.JABASTrainer(D.dev.index, lbs, K, 0, "overlap", cfg)
        tr.prepare_stream_parallel(model, torch.nn.CrossEntropyLoss().to(D.dev), gradient_as_bucket_view=True,
                                   collective=collective if D.world > 1 else "nccl")

        def groups(m):
            named = list(m.named_parameters())
            return [{"params": [p for n, p in named if "bn" in n], "weight_decay": 0},
                    {"params": [p for n, p in named if "bn" not in n], "weight_decay": 1e-4}]
        tr.prepare_weight_sync_method(ShardSGD(groups(tr.main_model), 0.1, momentum=0.9, weight_decay=1e-4), None, groups)
        tr.set_model_train()

        def timed(fn, n):
            D.barrier()
            a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(n):
                fn()
            z.record()
            D.barrier()
            return D.max_over_ranks(a.elapsed_time(z) / n)

        def full():
            tr.compute((x, y)); tr.step()

        def compute_only():                            # no synchronising micro-step: hooks stay silent
            tr.compute((x, y))
            for s in tr.model_streams:
                torch.cuda.current_stream().wait_stream(s)
            tr.local_accum_step = -1
        for _ in range(3):
            full()
        ms = timed(full, iters)
        exchange_ok_everywhere(D, tr.reducer.engine)
        cos = float(tr.cos_placeholder)
        real_accum = tr.accum_step
        tr.accum_step = 1 << 30
        for _ in range(2):
            compute_only()
        ms_fb = timed(compute_only, iters)
        tr.accum_step = real_accum
        tr.reducer.engine.zero_grads()
        out = {"ms_per_iteration": ms, "samples_per_sec": D.world * K * lbs / (ms / 1e3), "iterations": iters,
               "local_batch_size": lbs,
               "forward_backward_alone_ms": ms_fb, "gradient_path_exposed_ms": ms - ms_fb,
               "weight_sync_method": "overlap (per-bucket launches during backward)",
               "collective": ("peer-memory pipelined exchange" if collective == "peer" else "NCCL") if D.world > 1 else "none",
               "model": "torchvision resnet50, fp32 (TF32 convolutions), forward+backward by stock PyTorch kernels",
               "cosine": cos}
        if graph:
            try:                                       # the same iteration as ONE CUDA-graph launch
                launches = tr.reducer.engine.launches
                tr.enable_iteration_graph(warmup=2)
                for _ in range(4):                     # two eager, capture + first replay, one more replay
                    full()
                ms_g = timed(full, iters)
                out["graph"] = {"ms_per_iteration": ms_g, "samples_per_sec": D.world * K * lbs / (ms_g / 1e3),
                                "launches_per_replay": tr._iter_graph["launches"].get(True),
                                "cosine": float(tr.cos_placeholder),
                                "what": "compute() + step() replayed as one CUDA graph: K forward/backward passes on K "
                                        "streams, the hooks' launches, update, statistic, zeroed gradients"}
                assert tr.reducer.engine.launches > launches
            except Exception as e:
                out["graph"] = {"error": f"{type(e).__name__}: {e}"[:300]}
        tr.disable_iteration_graph()
        tr.reducer.engine.close()
        del tr, model, x, y
        gc.collect()
        torch.cuda.empty_cache()
        return out
    except Exception as e:                             # supplementary: never costs the benchmark line
        return {"error": f"{type(e).__name__}: {e}"[:300]}


def measure_allreduce(D, layout):
    """Bus bandwidth of NCCL's world allreduce alone, for comparison: per bucket, and over the
    whole flat gradient in one call.  busBW = bytes * 2(n-1)/n / t."""
    torch, dist, world = D.torch, D.dist, D.world
    fac = 2.0 * (world - 1) / world

    def timed(tensors, iters=10):
        for t in tensors:
            dist.all_reduce(t)
        D.barrier()
        a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            for t in tensors:
                dist.all_reduce(t)
        z.record()
        D.barrier()
        return D.max_over_ranks(a.elapsed_time(z) / iters)

    scratch = torch.zeros(layout.total, device=D.dev)
    buckets = [scratch[b:e] for b, e in layout.buckets]
    ms_b = timed(buckets)
    ms_w = timed([scratch])
    nbytes = 4 * layout.num_params
    out = {"per_bucket_ms": ms_b, "per_bucket_bus_gbs": nbytes * fac / (ms_b / 1e3) / 1e9,
           "whole_model_ms": ms_w, "whole_model_bus_gbs": nbytes * fac / (ms_w / 1e3) / 1e9,
           "bus_peak_gbs": 900.0,
           "frac_per_bucket": nbytes * fac / (ms_b / 1e3) / 1e9 / 900.0,
           "frac_whole_model": nbytes * fac / (ms_w / 1e3) / 1e9 / 900.0}
    del scratch, buckets
    torch.cuda.empty_cache()
    return out


def stream_study(args):
    """Does running the K VSWs on K streams buy anything?  Forward + backward only (stock PyTorch
    kernels), torchvision ResNet-50 fp32/TF32, K x LBS synthetic images, device and wall time."""
    import threading
    import torch
    import torchvision
    K, lbs = args.vsw or 4, 64
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    models = [torchvision.models.resnet50().to(dev).train() for _ in range(K)]
    crit = torch.nn.CrossEntropyLoss()
    x = torch.randn(K * lbs, 3, 224, 224, device=dev)
    y = torch.randint(0, 1000, (K * lbs,), device=dev)
    xs, ys = torch.chunk(x, K), torch.chunk(y, K)
    streams = [torch.cuda.Stream() for _ in range(K)]

    def fb(m, a, b):
        crit(m(a), b).backward()

    def one_model():
        fb(models[0], x, y)

    def serial():
        for k in range(K):
            fb(models[k], xs[k], ys[k])

    def k_streams():
        cur = torch.cuda.current_stream()
        for k in range(K):
            streams[k].wait_stream(cur)
            with torch.cuda.stream(streams[k]):
                fb(models[k], xs[k], ys[k])
        for s in streams:
            cur.wait_stream(s)

    def k_threads():
        cur = torch.cuda.current_stream()

        def run(k):
            torch.cuda.set_device(dev)
            streams[k].wait_stream(cur)
            with torch.cuda.stream(streams[k]):
                fb(models[k], xs[k], ys[k])
        ts = [threading.Thread(target=run, args=(k,)) for k in range(K)]
        for t in ts:
            t.start()
        for t in ts:
            t.join()
        for s in streams:
            cur.wait_stream(s)

    def timed(fn, n=8):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        a.record()
        for _ in range(n):
            fn()
        z.record()
        torch.cuda.synchronize()
        return {"device_ms": a.elapsed_time(z) / n, "wall_ms": (time.perf_counter() - t0) / n * 1e3}
    out = {"study": "vsw stream concurrency", "model": "torchvision resnet50 fp32 (TF32 convolutions)", "vsw": K,
           "local_batch": lbs}
    for name, fn in (("one_model_whole_batch", one_model), ("k_models_one_stream", serial),
                     ("k_models_k_streams_one_thread", k_streams), ("k_models_k_streams_k_threads", k_threads)):
        out[name] = timed(fn)
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    a = parse_args()
    if a.stream_study:
        stream_study(a)
    elif a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
