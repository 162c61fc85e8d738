#!/usr/bin/env python
"""Benchmark of the JABAS/IIDP per-iteration gradient path on B200.

    python bench.py --gpus N --steps K --warmup W            # this library (N = 1: plain python;
                                                             # N > 1: launched by torch.distributed.run)
    python bench.py --impl reference --gpus N --steps K --warmup W   # CPU/gloo restatement

A "step" is one pass of the gradient path over one iteration's worth of gradients:
for every DDP bucket  K-VSW aggregation -> (N > 1: sub-group + world allreduce) ->
fused optimizer update with write-back to the K replicas, and the two-half cosine
statistic.  The default workload is ResNet-50 (25,557,032 fp32 parameters in 5 buckets of
at most 25 MiB, two param groups), 4 VSWs per GPU, local batch 64 per VSW, SGD momentum
0.9, statistic every iteration; gradients are synthetic N(0, 1e-3), weights N(0, 1).

Rank 0 prints ONE JSON line.  ``value`` is samples/sec with the gradients resident in
HBM; ``e2e`` is the same metric with every step's K gradient sets copied from pinned host
memory and the cosine read back to the host inside the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (model, K, local batch per VSW, optimizer kind)
    "resnet50": ("resnet50", 4, 64, "sgd"),
    "vit_b_16": ("vit_b_16", 8, 32, "adamw"),
    "gnmt8": ("gnmt8", 2, 128, "adam"),
}


# dram__bytes_read + dram__bytes_write of one launch divided by the launch's algorithmic bytes,
# from the ncu captures summarised under profiles/ (ResNet-50 layout, K = 4, SGD-momentum); the
# kernels stream every byte once, so the ratio carries over to other sizes.
NCU_TRAFFIC_RATIO = {"fused_step": 1067.4 / 1124.5, "update": 760.1 / 817.8, "aggregate": 457.4 / 511.1}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="resnet50",
                    help="resnet50 | vit_b_16 | gnmt8 | flat<log2 elements> (e.g. flat27)")
    ap.add_argument("--vsw", type=int, default=None, help="override K (VSWs per GPU)")
    ap.add_argument("--optimizer", default=None, choices=[None, "sgd", "adam", "adamw"])
    ap.add_argument("--similarity-mode", default="fused", choices=["fused", "pair_exchange"])
    ap.add_argument("--collective", default="peer", choices=["peer", "nccl"],
                    help="N > 1: cross-GPU exchange by this library's kernels over NVLink peer memory, or by NCCL")
    ap.add_argument("--no-similarity", action="store_true",
                    help="skip the two-half statistic (forced when T is odd, e.g. one GPU with one VSW)")
    ap.add_argument("--no-overlap", action="store_true")
    ap.add_argument("--per-bucket", default="auto", choices=["auto", "yes", "no"],
                    help="yes: walk the DDP buckets as the comm hooks do; no / auto: the whole flat model per launch")
    ap.add_argument("--share-weights", action="store_true",
                    help="the K replicas alias one weight buffer (no write-back to K-1 replicas); not the default")
    ap.add_argument("--staging", default="register", choices=["register", "bulk"],
                    help="how the update kernels fetch their tiles: per-thread 128-bit loads (default) or "
                         "TMA bulk copies into a shared-memory ring")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch every kernel / collective from Python instead of replaying one CUDA graph")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-train-iter", action="store_true",
                    help="skip the supplementary whole-training-iteration measurement (resnet50 workload only)")
    ap.add_argument("--cpu-steps", type=int, default=None)
    return ap.parse_args()


def make_workload(args):
    from jabas_b200.layout import build_layout, model_zoo_shapes
    name = args.workload
    if name.startswith("flat"):
        n = 1 << int(name[4:])
        K, lbs, kind = args.vsw or 4, 64, args.optimizer or "sgd"
        layout = build_layout(["flat"], [(n,)], [0], bucket_cap_mb=1 << 30, first_bucket_bytes=1 << 62)
        desc = f"flat fp32 buffer of 2^{name[4:]} elements"
    else:
        model, K, lbs, kind = WORKLOADS[name]
        K, kind = args.vsw or K, args.optimizer or kind
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
        "collective": ("peer-memory kernels over NVLink" if args.collective == "peer" else "NCCL allreduce")
                      if world > 1 else "none",
        "launch_granularity": "bucket" if args.per_bucket == "yes"
                              else "whole flat model",
        "parallelism": f"dp{world} x vsw{K}",
        "l2": "inputs larger than L2: %.0f MB of gradients, weights and state per GPU vs 126 MB"
              % (4 * layout.total * (2 * K + 2) / 1e6),
    }


# --------------------------------------------------------------------------------------
# clocks
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
    layout, K, lbs, opt, desc = make_workload(args)
    world = args.gpus
    dt, cores, threads, done = run_cpu_path(layout, K, opt, world, args.steps, args.warmup, budget_s=90.0)
    ms = dt / args.steps * 1e3
    value = world * K * lbs / (ms / 1e3)
    cfg = config_dict(args, layout, K, lbs, opt, desc, world)
    cfg["similarity_mode"] = "pair_exchange" if world > 1 else "vsw_parity"
    sample = (f"{done} full iterations of the workload (of {args.steps} asked; at most 90 s are sampled) after "
              f"{max(1, min(args.warmup, 3))} warm-up, {world} gloo rank(s) x {threads} torch threads on {cores} host cores")
    line = {
        "impl": "reference", "metric": "samples/sec", "value": value, "unit": "samples/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": cfg,
        "cpu_baseline": {"value": value, "unit": "samples/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gradient_path_gbs_per_rank": _alg_bytes(layout, K, opt, world)["total"] / (ms / 1e3) / 1e9,
    }
    print(json.dumps(line), flush=True)


def _alg_bytes(layout, K, opt, world):
    n = layout.num_params
    multi = world > 1
    agg = (4 * n * (K + 1) if (K > 1 or multi) else 0) + (4 * n if multi else 0)
    per = (K + 4) if opt["kind"] == "sgd" else (K + 6)
    upd = 4 * n * per + (4 * n if multi else 0)
    return {"aggregate": agg, "update": upd, "total": agg + upd}


# --------------------------------------------------------------------------------------
# this library
# --------------------------------------------------------------------------------------

def run_ours(args):
    import torch
    import torch.distributed as dist
    from jabas_b200.gradient_path import GradientPath, OptimizerSpec

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    sub_group = pair_group = None
    if world > 1:
        import datetime
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"       # keep stdout to the one JSON line
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
        idx = [[r for r in range(world) if r % 2 == p] for p in (0, 1)]
        groups = [dist.new_group(ix) for ix in idx]
        sub_group = groups[rank % 2]
        pair_group = dist.new_group([idx[0][0], idx[1][0]])

    layout, K, lbs, opt, desc = make_workload(args)
    spec = OptimizerSpec(kind=opt["kind"], groups=opt["groups"], momentum=opt.get("momentum", 0.0),
                         betas=opt.get("betas", (0.9, 0.999)), eps=opt.get("eps", 1e-8))
    similarity = not args.no_similarity and (world * K) % 2 == 0 and (world > 1 or K % 2 == 0)
    collective, collective_note = args.collective, None

    def make_engine(coll):
        return GradientPath(layout, K, dev, spec, total_num_decoupled_workers=world * K,
                            sub_group=sub_group, pair_group=pair_group, similarity=similarity,
                            similarity_mode=args.similarity_mode, collective=coll,
                            share_weights=args.share_weights, staging=args.staging)
    try:
        eng = make_engine(collective)
    except Exception as e:
        if world == 1 or collective != "peer":
            raise
        # peer mappings could not be set up on this machine (every rank sees the same failure):
        # the exchange goes through NCCL instead, and the result line says so
        collective, collective_note = "nccl", f"peer-memory set-up failed ({type(e).__name__}: {e})"[:200]
        eng = make_engine("nccl")
    gen = torch.Generator(device=dev).manual_seed(7)
    eng.weights[0].normal_(generator=gen)
    if not args.share_weights:
        for k in range(1, K):
            eng.weights[k].copy_(eng.weights[0])
    for k in range(K):
        g = torch.Generator(device=dev).manual_seed(1000 * rank + k)
        eng.grads[k].normal_(0.0, 1e-3, generator=g)
    overlap = not args.no_overlap
    per_bucket = None if args.per_bucket == "auto" else (args.per_bucket == "yes")
    eager_fn = lambda: eng.run_iteration(overlap=overlap, per_bucket=per_bucket)
    use_graph = not args.no_graph
    step_fn = eng.replay if use_graph else eager_fn

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    # ---- device-resident timing ---------------------------------------------------
    if use_graph:
        eng.capture(overlap=overlap, per_bucket=per_bucket, warmup=2)
    for _ in range(max(args.warmup, 3)):
        step_fn()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    if not use_graph:
        eng.profile_events = []
    launches0 = eng.launches
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step_fn()
    e1.record()
    barrier()
    ms_step = max_over_ranks(e0.elapsed_time(e1) / args.steps)
    launches = eng.launches - launches0
    if use_graph:
        # kernels inside a replayed graph cannot be bracketed by events: time them in a second
        # pass of the same number of steps, launched eagerly, right after the timed region
        eng.profile_events = []
        for _ in range(args.steps):
            eager_fn()
        barrier()
    events, eng.profile_events = eng.profile_events, None
    # a short run (few steps) ends before the 50 ms clock sampler has seen the load: keep the
    # same step running, untimed, until half a second of it has passed (same count on all ranks)
    extra = int(500.0 / max(ms_step, 1e-3)) - args.steps * (2 if use_graph else 1)
    if extra > 0:
        for _ in range(extra):
            step_fn()
        barrier()
    clocks = sampler.stop() if rank == 0 else None
    cos = float(eng.cos)
    if args.staging == "bulk" and eng.ctx.staging_timeouts() != 0:
        raise RuntimeError("bulk staging: a wait for a copy ran out; the timed steps are incomplete")

    per_kernel = {}
    for kind, b, a, z in events:
        d = per_kernel.setdefault(kind, [0.0, 0])
        d[0] += a.elapsed_time(z)
        d[1] += 1
    alg = eng.algorithmic_bytes(similarity)

    # ---- collectives alone (N > 1), outside the timed region ------------------------
    bus = None
    if world > 1:
        bus = measure_allreduce(eng, layout, world, dev)

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
        barrier()
        n_e2e = max(5, min(args.steps, 30))
        a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n_e2e):
            e2e_step()
        z.record()
        barrier()
        ms_e2e = max_over_ranks(a.elapsed_time(z) / n_e2e)
        e2e = {"value": world * K * lbs / (ms_e2e / 1e3), "unit": "samples/s",
               "h2d_bytes_per_step": 4 * layout.total * K, "d2h_bytes_per_step": 4,
               "ms_per_step": ms_e2e, "steps": n_e2e,
               "api": "GradientPath.run_iteration over the C ABI; gradients from pinned host memory"}

    train_iter = None
    if args.workload == "resnet50" and not args.no_train_iter and world == 1:   # one GPU only: a failure
        # on one rank of several must not leave the others waiting in a collective
        try:
            del host
        except NameError:
            pass
        try:
            t = measure_training_iteration(K, lbs, dev, world)
            t["ms_per_iteration"] = max_over_ranks(t["ms_per_iteration"])
            t["samples_per_sec"] = world * K * lbs / (t["ms_per_iteration"] / 1e3)
            train_iter = t
        except Exception as e:                      # supplementary: never costs the benchmark line
            train_iter = {"error": f"{type(e).__name__}: {e}"[:300]}

    if rank != 0:
        _finish(world)
        return

    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    else:
        peak, peak_src = 6650.0, "fallback"
    dom = max(per_kernel, key=lambda k: per_kernel[k][0])
    dom_ms, dom_n = per_kernel[dom]
    achieved = alg[dom] * args.steps / (dom_ms / 1e3) / 1e9
    kern = {k: {"launches": v[1], "ms_per_step": v[0] / args.steps,
                "gbs": alg[k] * args.steps / (v[0] / 1e3) / 1e9} for k, v in per_kernel.items()}
    line = {
        "metric": "samples/sec", "value": world * K * lbs / (ms_step / 1e3), "unit": "samples/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": dict(config_dict(args, layout, K, lbs, opt, desc, world),
                                            similarity="every iteration" if similarity else "off",
                                            **({"collective": "NCCL allreduce", "collective_note": collective_note}
                                               if collective_note else {})),
        "gradient_path_gbs_per_gpu": alg["total"] / (ms_step / 1e3) / 1e9,
        "gradient_path_frac_of_hbm_peak": alg["total"] / (ms_step / 1e3) / 1e9 / peak,
        "roofline": {"bound": "hbm", "kernel": dom, "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_source": peak_src,
                     "traffic": (NCU_TRAFFIC_RATIO[dom] * alg[dom] / max(1, dom_n // args.steps)
                                 if dom in NCU_TRAFFIC_RATIO and world == 1 else None),
                     "algorithmic_bytes_per_launch": alg[dom] / max(1, dom_n // args.steps),
                     "launches_per_step": dom_n // args.steps},
        "kernels": kern, "gpu_launches": launches, "cosine": cos, "clocks": clocks, "e2e": e2e,
    }
    if train_iter is not None:
        line["training_iteration"] = train_iter
    if bus is not None:
        line["allreduce"] = bus
    if world > 1 and eng.collective == "peer":
        kms = sum(v[0] for k, v in per_kernel.items() if k in ("peer_reduce", "update", "fused_step")) / args.steps
        line["exchange"] = {
            "kind": "peer-memory kernels (plain NVLink loads inside the reduce-scatter and update kernels)",
            "form": "direct (2 ranks)" if eng.peer_direct else "reduce-scatter + gathering update",
            "nvlink_in_bytes_per_step": alg["nvlink_in"], "kernels_ms_per_step": kms,
            "nvlink_in_gbs_while_kernels_run": alg["nvlink_in"] / (kms / 1e3) / 1e9,
            "nccl_barriers_per_step": 2, "bus_peak_gbs": 900.0}
    if not args.no_cpu_baseline and world == 1:      # the CPU baseline is reported at N = 1 only
        cpu_steps = args.cpu_steps or 10
        dt, cores, threads, done = run_cpu_path(layout, K, opt, 1, cpu_steps, 2, budget_s=30.0)
        line["cpu_baseline"] = {
            "value": K * lbs / (dt / cpu_steps), "unit": "samples/s", "cores": cores, "kind": "port",
            "ms_per_step": dt / cpu_steps * 1e3,
            "sample": f"{done} iterations of this workload at one rank (K={K}) after 2 warm-up, "
                      f"stock torch CPU ops, {threads} threads"}
    print(json.dumps(line), flush=True)
    _finish(world)


def _finish(world):
    """Leave a multi-rank run: last barrier, then exit without tearing the NCCL communicators
    down one by one (communicator teardown at interpreter exit was seen to block for minutes
    after the result line had been printed; the driver reclaims everything at process exit)."""
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def measure_training_iteration(K, lbs, dev, world, iters=8):
    """Supplementary: a WHOLE training iteration through the trainer mirror — K VSWs' forward and
    backward of torchvision ResNet-50 (stock PyTorch / cuDNN kernels, fp32 with TF32 convolutions) on K
    streams, comm hooks fired from backward, this library's path — on synthetic N(0,1) images.  It puts
    the gradient path's time in proportion; it is not the benchmark's metric."""
    import torch
    import torchvision
    import jabas_b200
    from jabas_b200.iidp.optim import ShardSGD
    cfg = dict(similarity_target=0.1, batch_size_adjust_interval=1, enable_adjust=False)
    tr = jabas_b200.JABASTrainer(dev.index, lbs, K, 0, "overlap", cfg)
    torch.manual_seed(0)
    tr.prepare_stream_parallel(torchvision.models.resnet50().to(dev), torch.nn.CrossEntropyLoss().to(dev),
                               gradient_as_bucket_view=True)

    def groups(m):
        named = list(m.named_parameters())
        return [{"params": [p for n, p in named if "bn" in n], "weight_decay": 0},
                {"params": [p for n, p in named if "bn" not in n], "weight_decay": 1e-4}]
    tr.prepare_weight_sync_method(ShardSGD(groups(tr.main_model), 0.1, momentum=0.9, weight_decay=1e-4), None, groups)
    tr.set_model_train()
    x = torch.randn(K * lbs, 3, 224, 224, device=dev)
    y = torch.randint(0, 1000, (K * lbs,), device=dev)
    for _ in range(3):
        tr.compute((x, y)); tr.step()
    torch.cuda.synchronize()
    a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        tr.compute((x, y)); tr.step()
    z.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(z) / iters
    return {"ms_per_iteration": ms, "samples_per_sec": world * K * lbs / (ms / 1e3), "iterations": iters,
            "model": "torchvision resnet50, fp32 (TF32 convolutions), forward+backward by stock PyTorch kernels",
            "cosine": float(tr.cos_placeholder)}


def measure_allreduce(eng, layout, world, dev):
    """Bus bandwidth of the world allreduce alone: per bucket as the path issues it, and
    over the whole flat gradient in one call.  busBW = bytes * 2(n-1)/n / t."""
    import torch
    import torch.distributed as dist
    fac = 2.0 * (world - 1) / world

    def timed(tensors, iters=10):
        for t in tensors:
            dist.all_reduce(t)
        torch.cuda.synchronize()
        dist.barrier()
        a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            for t in tensors:
                dist.all_reduce(t)
        z.record()
        torch.cuda.synchronize()
        ms = torch.tensor([a.elapsed_time(z) / iters], dtype=torch.float64, device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms)

    scratch = torch.zeros(layout.total, device=dev)
    buckets = [scratch[b:e] for b, e in layout.buckets]
    ms_b = timed(buckets)
    ms_w = timed([scratch])
    nbytes = 4 * layout.num_params
    return {"per_bucket_ms": ms_b, "per_bucket_bus_gbs": nbytes * fac / (ms_b / 1e3) / 1e9,
            "whole_model_ms": ms_w, "whole_model_bus_gbs": nbytes * fac / (ms_w / 1e3) / 1e9,
            "bus_peak_gbs": 900.0,
            "frac_per_bucket": nbytes * fac / (ms_b / 1e3) / 1e9 / 900.0,
            "frac_whole_model": nbytes * fac / (ms_w / 1e3) / 1e9 / 900.0}


if __name__ == "__main__":
    a = parse_args()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
