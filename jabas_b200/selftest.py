"""Self-test and profiling driver of the pipelined cross-GPU exchange on ONE GPU.

    python -m jabas_b200.selftest --ranks 2 --vsw 4 --log2n 24 --iters 3            # run, check the status
    python -m jabas_b200.selftest --ranks 8 --vsw 4 --log2n 24 --iters 10 --time    # + median launch time (JSON)

Kernels that wait on one another may not run as separate launches on one GPU, so all ``--ranks``
ranks of the exchange run as ONE launch here (``jabas_exchange_step_f32(nlocal = nranks)``): the
queue, the per-piece flags, the TMA ring and the arithmetic are the multi-GPU code, only the
"peer" loads are local.  This is the form to put under a profiler (a multi-rank command must
not be), and a quick check that a machine can run the exchange at all.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import ops


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ranks", type=int, default=2)
    ap.add_argument("--vsw", type=int, default=4)
    ap.add_argument("--log2n", type=float, default=24.0, help="log2 of the elements per rank")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--optimizer", default="sgd", choices=["sgd", "adam", "adamw"])
    ap.add_argument("--piece", type=int, default=ops.EXCHANGE_PIECE)
    ap.add_argument("--window", type=int, default=0, help="pieces per pipeline step (0: sized from the grid)")
    ap.add_argument("--time", action="store_true", help="time every launch with CUDA events, print JSON")
    a = ap.parse_args(argv)
    dev = torch.device("cuda", 0)
    ctx = ops.Context(0)
    n, K = a.ranks, a.vsw
    total = int(round(2 ** a.log2n)) // 1024 * 1024
    slots = -(-total // a.piece) + 1
    f32 = dict(dtype=torch.float32, device=dev)
    px = [torch.zeros(total, **f32) for _ in range(n)]
    pg = [torch.zeros(total, **f32) for _ in range(n)]
    fl = [torch.zeros(ops.exchange_flag_words(slots), dtype=torch.int32, device=dev) for _ in range(n)]
    exs = [ops.Exchange(ctx, n, r, [t.data_ptr() for t in px], [t.data_ptr() for t in pg],
                        [t.data_ptr() for t in fl], slots, a.window, a.piece) for r in range(n)]
    adam = a.optimizer != "sgd"
    bufs = [dict(grads=[torch.randn(total, **f32) * 1e-3 for _ in range(K)],
                 weights=[torch.randn(total, **f32) for _ in range(K)], m=torch.zeros(total, **f32),
                 v=torch.zeros(total, **f32) if adam else None,
                 stat=torch.zeros(3, dtype=torch.float64, device=dev)) for _ in range(n)]
    groups = [dict(lr=0.1, weight_decay=1e-4, step=1)]
    kw = dict(kind=a.optimizer, momentum=0.9) if not adam else dict(kind=a.optimizer)
    times = []
    for _ in range(a.iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ops.exchange_step(exs, bufs, total, 0, 0, float(n * K), n * K / 2, groups, **kw)
        e1.record()
        if a.time:
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
    torch.cuda.synchronize()
    bad = [e.status()[0] for e in exs if e.status()[0]]
    for e in exs:
        e.close()
    if bad:
        print(f"a bounded wait ran out: status {bad[0]:#x}")
        return 1
    if a.time:
        times = sorted(times[min(3, len(times) - 1):])
        per = (K + 4) if not adam else (K + 6)
        # bytes through this GPU's HBM for ALL ranks, the "peer" reads included
        nbytes = n * 4 * total * ((K + 1) + 2 + (per - 1) + 1)
        ms = times[len(times) // 2]
        print(json.dumps(dict(ranks=n, vsw=K, elements_per_rank=total, piece=a.piece, window=a.window,
                              optimizer=a.optimizer, ms_per_launch=ms, gbs=nbytes / ms / 1e6)))
    else:
        print("ok")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
