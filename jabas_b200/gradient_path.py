"""The per-iteration gradient path of one GPU, bucket by bucket, over flat HBM buffers.

For every DDP bucket ``b`` (a contiguous element range of the flat buffers) the path is

  1. ``aggregate(b)``  K VSW gradient buckets -> main bucket (÷T)     [one kernel]
                        (+ undivided copy for the parity sub-group, or, on one GPU,
                        the VSW-parity statistic in the same pass)
  2. ``allreduce(b)``  sub-group SUM of the copy, world SUM of the main bucket [NCCL]
  3. ``update(b)``     fused SGD-momentum / Adam / AdamW on the main replica, new weights
                        written to all K replicas, two-half statistic from the sub-group
                        sum in the same pass                                [one kernel]

and once per iteration ``finish_similarity()`` turns the three fp64 sums into the cosine.

This replaces, op for op, the reference's chain
``subgroup_allreduce_hook`` -> ``iidp_allreduce_hook`` -> optimizer step -> weight copy
-> ``_compute_cosine_similarity`` (jabas/ddp_comm_hooks/similarity_allreduce.py:20-45,
jabas/train/trainer.py:470-483).  Two forms of the statistic are provided:

* ``"fused"`` (default): each rank derives the other half as ``o = 2g - e`` from the
  world mean ``g`` and its own sub-group mean ``e``; no model-sized exchange, no extra
  pass.  Rank 0's value is broadcast so that every rank takes the same decision.
* ``"pair_exchange"``: the reference's data flow — materialise ``E = half/(T/2)``,
  ``all_gather`` it between the first rank of each sub-group, reduce on rank 0, broadcast.

All device work is enqueued on the CURRENT CUDA stream; collectives are asynchronous
``torch.distributed`` calls whose completion the current stream waits on (no host sync).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from .layout import FlatLayout


@dataclass
class OptimizerSpec:
    """Hyper-parameters of the fused update.  ``groups`` holds one dict per optimizer
    param group (``lr``, ``weight_decay``); ``lr`` may be changed between iterations, as
    the reference does at jabas/train/trainer.py:693-700."""
    kind: str                                    # "sgd" | "adam" | "adamw"
    groups: List[Dict[str, float]]
    momentum: float = 0.0
    dampening: float = 0.0
    nesterov: bool = False
    betas: Sequence[float] = (0.9, 0.999)
    eps: float = 1e-8

    def __post_init__(self):
        if self.kind not in ("sgd", "adam", "adamw"):
            raise ValueError(f"unsupported optimizer kind {self.kind!r}")


class GradientPath:
    def __init__(self, layout: FlatLayout, num_vsw: int, device, optimizer: Optional[OptimizerSpec] = None, *,
                 total_num_decoupled_workers: int, process_group=None, sub_group=None,
                 pair_group=None, first_subgroup_src_rank: int = 0, second_subgroup_src_rank: int = 1,
                 similarity: bool = True, similarity_mode: str = "fused", backend=None,
                 collective: str = "nccl", share_weights: bool = False, staging: str = "register",
                 peer_form: str = "pipeline", peer_wait_ms: Optional[float] = None,
                 exchange_piece: Optional[int] = None, exchange_window: Optional[int] = None):
        if collective not in ("nccl", "peer"):
            raise ValueError("collective must be 'nccl' or 'peer'")
        if collective == "peer" and staging != "register":
            # a launch that reads another GPU's memory through per-thread loads or the exchange's own
            # TMA ring never goes through the update kernels' bulk-staged form
            raise ValueError("staging='bulk' cannot be combined with collective='peer'")
        if peer_form not in ("pipeline", "direct"):
            raise ValueError("peer_form must be 'pipeline' or 'direct'")
        if backend is None:
            from . import ops as backend          # the CUDA library; raises without a GPU
        self.ops = backend
        self.layout = layout
        self.K = int(num_vsw)
        self.device = torch.device(device)
        self.opt = None
        self.m = self.v = None
        self.T = int(total_num_decoupled_workers)
        self.pg = process_group
        self.sub_group = sub_group
        self.pair_group = pair_group
        self.src0, self.src1 = first_subgroup_src_rank, second_subgroup_src_rank
        self.world = dist.get_world_size(process_group) if (dist.is_available() and dist.is_initialized()) else 1
        self.rank = dist.get_rank(process_group) if self.world > 1 else 0
        self.similarity = bool(similarity)
        if similarity_mode not in ("fused", "pair_exchange"):
            raise ValueError("similarity_mode must be 'fused' or 'pair_exchange'")
        self.similarity_mode = similarity_mode
        if self.similarity:
            # jabas/ddp_comm_hooks/similarity_allreduce.py:13-14
            assert self.T % 2 == 0, f"total_num_decoupled_workers must be even, but {self.T}"
            if self.world > 1:
                assert self.world % 2 == 0          # jabas/train/trainer.py:430
            else:
                assert self.K >= 2 and self.K % 2 == 0, \
                    "on one GPU the two halves are the even and the odd VSWs: K must be even"
        self.ctx = self.ops.Context(self.device)
        if staging != "register":                 # "bulk": TMA bulk copies into shared memory
            self.ctx.set_staging(staging)
        if peer_wait_ms is not None:
            self.ctx.set_wait_limits(peer_ms=peer_wait_ms)
        self.dev_layout = None
        n = layout.total
        f32 = dict(dtype=torch.float32, device=self.device)
        #: K replicas may alias ONE weight buffer: forward/backward only read the weights, and a
        #: bucket is updated only after every VSW has finished with it, so the write-back to the
        #: other K-1 replicas (4(K-1) bytes per element and iteration) has nothing left to do
        self.share_weights = bool(share_weights)
        if self.share_weights:
            w0 = torch.zeros(n, **f32)
            self.weights = [w0] * self.K
        else:
            self.weights = [torch.zeros(n, **f32) for _ in range(self.K)]
        self.grads = [torch.zeros(n, **f32) for _ in range(self.K)]
        self.collective = collective if self.world > 1 else "nccl"
        self.half = torch.zeros(n, **f32) if (self.similarity and self.world > 1
                                              and self.collective == "nccl") else None
        #: how collective="peer" moves the gradients between GPUs:
        #:   "pipeline" (default) ONE persistent kernel per launch draws aggregate / reduce / update
        #:              pieces from an ordered queue; ranks synchronise through epoch flags in peer
        #:              memory (bounded waits), so NVLink and HBM phases overlap chunk by chunk; works
        #:              per bucket (hooks during backward) and over the whole model
        #:   "direct"   two ranks only, whole model at step time: an aggregate kernel, an NCCL barrier,
        #:              and the fused update kernel reads both ranks' sums itself (the remote one over
        #:              NVLink); 10 % faster than the pipeline on a ResNet-50-sized model, slower on
        #:              large ones, and it cannot run per bucket
        self.peer_form = peer_form
        self.peer_direct = peer_form == "direct"
        if self.peer_direct and self.world != 2 and self.collective == "peer":
            raise ValueError("peer_form='direct' needs exactly two ranks")
        self.exchange = None
        self.exchange_piece = exchange_piece          # elements of one work item of the pipelined exchange
        self.exchange_window = exchange_window        # pieces per pipeline step (None: sized from the grid)
        if self.collective == "peer":
            if self.peer_form == "pipeline":
                self._setup_pipeline_exchange()
            else:
                self._setup_peer_exchange()
        self.stat = torch.zeros(3, dtype=torch.float64, device=self.device)
        self.cos = torch.zeros(1, **f32)
        self.steps = 0                               # completed optimizer steps
        self._pending: Dict[int, list] = {}
        self._sim_step = False
        self.half_divided = set()                    # pair_exchange: buckets whose E is materialised
        self.launches = 0                            # kernels of libjabas_b200 enqueued so far
        self.profile_events: Optional[list] = None   # set to [] to time every kernel with CUDA events
        nb = layout.num_buckets
        # gradient-norm clipping: one (sum of squares, coefficient) slot per bucket + one for the model
        self.clip_stat = torch.zeros(nb + 1, 3, dtype=torch.float64, device=self.device)
        self.clip_coef = torch.ones(nb + 1, 2, **f32)
        self._clip_active: Dict[int, bool] = {}
        #: one GPU: hooks may leave a bucket's aggregation to the update, which then runs as ONE
        #: kernel (aggregate + update + write-back + statistic); set by the trainer
        self.defer_local = False
        self._deferred = set()
        self._dyn = None                             # device-resident hyper-parameters (graph mode)
        self._graph = None
        self._graph_stream = None
        if optimizer is not None:
            self.set_optimizer(optimizer)

    def _setup_peer_exchange(self) -> None:
        """The two-rank direct form: one symmetric buffer per rank, mapped into the other rank's
        address space over NVLink (torch symmetric memory does the allocation and the handle
        exchange; the data path is this library's kernels).  ``px`` receives the local sum of
        the K VSW gradients, divided by T."""
        import torch.distributed._symmetric_memory as symm_mem
        n = self.layout.total
        group = self.pg if self.pg is not None else dist.group.WORLD
        self.px = symm_mem.empty(n, dtype=torch.float32, device=self.device)
        self.px.zero_()
        self._px_h = symm_mem.rendezvous(self.px, group)
        self.px_ptrs = [int(p) for p in self._px_h.buffer_ptrs]
        self._tok = torch.zeros(1, dtype=torch.float32, device=self.device)

    def _setup_pipeline_exchange(self) -> None:
        """Buffers of the pipelined exchange, all of them symmetric (allocated and exchanged by
        torch symmetric memory, addressed by this library's kernels): ``px`` takes this rank's
        undivided local sum, ``pgrad`` the shards of the averaged gradient this rank reduces, and
        a block of per-piece epoch flags that the other ranks store into."""
        import torch.distributed._symmetric_memory as symm_mem
        n, world = self.layout.total, self.world
        if world > 8:
            raise ValueError("the pipelined exchange serves up to 8 ranks (one NVSwitch domain)")
        group = self.pg if self.pg is not None else dist.group.WORLD
        import os
        # tuning knobs (environment, for sweeps): elements per work item, pieces per pipeline step
        # (measured: items of 8,192 elements suit models up to ViT-B/16's size — 4 GPUs, ResNet-50
        # layout 0.360 vs 0.374 ms —, items of 16,384 the larger buffers — GNMT on 2 GPUs 2.16 vs 2.25 ms)
        piece = int(self.exchange_piece or os.environ.get("JABAS_EXCHANGE_PIECE", 0)
                    or (self.ops.EXCHANGE_PIECE if n <= 100_000_000 else 2 * self.ops.EXCHANGE_PIECE))
        if self.exchange_window is None and os.environ.get("JABAS_EXCHANGE_SLACK"):
            sms = torch.cuda.get_device_properties(self.device).multi_processor_count
            slack = float(os.environ["JABAS_EXCHANGE_SLACK"])
            self.exchange_window = max(world, int(slack * 2 * sms * world / (2 * world + 1)) // world * world)
        per_bucket = [-(-self._bucket_span(b)[1] // piece) for b in range(self.layout.num_buckets)]
        self._slot_base = [sum(per_bucket[:b]) for b in range(len(per_bucket))]
        max_slots = max(-(-n // piece), sum(per_bucket), 1)
        words = self.ops.exchange_flag_words(max_slots)
        self.px = symm_mem.empty(n, dtype=torch.float32, device=self.device)
        self.pgrad = symm_mem.empty(n, dtype=torch.float32, device=self.device)
        self.xflags = symm_mem.empty(words, dtype=torch.int32, device=self.device)
        self.px.zero_(); self.pgrad.zero_(); self.xflags.zero_()
        self._px_h = symm_mem.rendezvous(self.px, group)
        self._pg_h = symm_mem.rendezvous(self.pgrad, group)
        self._fl_h = symm_mem.rendezvous(self.xflags, group)
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.pg)                   # every rank's flag block is zero before any launch
        self._bucket_grid_limit = int(os.environ.get("JABAS_EXCHANGE_BUCKET_CTAS", 0)) or \
            torch.cuda.get_device_properties(self.device).multi_processor_count
        self._grid_limit_set = 0
        self._exchange_ctas = int(os.environ.get("JABAS_EXCHANGE_CTAS_PER_SM", 0))
        self.exchange = self.ops.Exchange(self.ctx, world, self.rank,
                                          [int(p) for p in self._px_h.buffer_ptrs],
                                          [int(p) for p in self._pg_h.buffer_ptrs],
                                          [int(p) for p in self._fl_h.buffer_ptrs], max_slots, int(self.exchange_window or 0),
                                          piece, int(os.environ.get("JABAS_EXCHANGE_UPDATE_LAG", 0)))
        if self._exchange_ctas != 0:
            self.exchange.set_ctas_per_sm(self._exchange_ctas)

    def _bucket_span(self, b: Optional[int]):
        """(first element, length) of a launch over bucket ``b`` (None: the whole flat buffer); a
        bucket's span runs to the 128-byte boundary its successor starts on (padding is zero)."""
        if b is None:
            return 0, self.layout.total
        begin, end = self.layout.buckets[b]
        nxt = self.layout.buckets[b + 1][0] if b + 1 < self.layout.num_buckets else self.layout.total
        return begin, nxt - begin

    def exchange_launch(self, b: Optional[int] = None) -> None:
        """One launch of the pipelined exchange: aggregation, cross-GPU reduction, update,
        write-back and this rank's share of the statistic for bucket ``b`` (None: the model)."""
        begin, length = self._bucket_span(b)
        if length == 0:
            return
        o = self.opt
        bufs = dict(grads=self.grads, weights=self._replicas(0, self.layout.total), m=self.m, v=self.v,
                    stat=self.stat if self._sim_step else None)
        kw = dict(kind=o.kind, layout=self.dev_layout, dynamic=self._dyn)
        if o.kind == "sgd":
            kw.update(momentum=o.momentum, dampening=o.dampening, nesterov=o.nesterov,
                      first_step=(self.steps == 0))
            groups = o.groups
        else:
            kw.update(beta1=o.betas[0], beta2=o.betas[1], eps=o.eps)
            groups = [dict(gr, step=self.steps + 1) for gr in o.groups]
        # a per-bucket launch runs beside backward: one CTA per SM leaves the rest of each SM to it
        limit = 0 if b is None else self._bucket_grid_limit
        if limit != self._grid_limit_set:
            self.exchange.set_grid_limit(limit)
            self._grid_limit_set = limit
        ev = self._ev_begin()
        self.ops.exchange_step([self.exchange], [bufs], length, begin, 0 if b is None else self._slot_base[b],
                               float(self.T), self.T / 2, groups, **kw)
        self._ev_end("exchange", b, ev)
        self.launches += 1

    def check_exchange(self) -> None:
        """Raise if a bounded wait of the pipelined exchange ever ran out (synchronises the device)."""
        if self.exchange is not None:
            status, _ = self.exchange.status()
            if status:
                phase = {2: "reduce", 3: "update", 4: "statistic"}.get((status >> 24) & 0xf, "?")
                raise RuntimeError(f"pipelined exchange: a wait on another rank ran out in the {phase} phase "
                                   f"(slot {status & 0xffffff}); this iteration's weights are incomplete")

    def _peer_iteration(self) -> Optional[torch.Tensor]:
        """Whole flat model through the peer-memory exchange.  ``peer_form="pipeline"``: one
        launch (plus the 32-thread statistic kernel).  ``"direct"`` (two ranks): aggregate kernel,
        barrier, fused update kernel that reads both ranks' sums, barrier."""
        if self.exchange is not None:
            self.exchange_launch(None)
            return self.finish_similarity()
        sim = self._sim_step
        n = self.layout.total
        ev = self._ev_begin()
        # each rank's sum is divided by T BEFORE the two are added, as everywhere else on the
        # path (the reference's div_(T) before the SUM allreduce): g = fl(S0/T) + fl(S1/T)
        self.ops.vsw_aggregate(self.ctx, self.grads, self.px[:n], float(self.T))
        self._ev_end("aggregate", None, ev)
        dist.all_reduce(self._tok, group=self.pg)                                  # both ranks' sums are in place
        # The update kernel itself reads both ranks' sums (the remote one over NVLink, hidden under
        # its own HBM traffic), adds them as they are (divisor 1), takes the statistic from the two
        # ranks = the two halves (E, O = S_r / (T/2): the divided sums over 1/2, exact) and updates.
        self.fused_local_step(None, sources=self.px_ptrs, divisor=1.0, half_divisor=0.5)
        dist.all_reduce(self._tok, group=self.pg)      # nobody overwrites its sum while the peer still reads it
        self.launches += 1
        if sim:
            self.ops.cosine_finalize(self.ctx, self.stat, self.cos)                # same bits on both ranks
            self.launches += 1
            return self.cos
        return None

    def set_optimizer(self, optimizer: OptimizerSpec) -> None:
        """Bind the fused update: uploads the param-group segment table of the layout and
        allocates the flat momentum / Adam moment buffers (kept if already present)."""
        self.opt = optimizer
        ngroups = 1 + max(g for _, _, g in self.layout.segments)
        if len(optimizer.groups) < ngroups:
            raise ValueError(f"the layout names {ngroups} param groups, the optimizer has {len(optimizer.groups)}")
        if self.dev_layout is not None:
            self.dev_layout.close()
        self.dev_layout = self.ops.Layout(self.ctx, self.layout.segments, self.layout.total) \
            if len(self.layout.segments) > 1 else None
        f32 = dict(dtype=torch.float32, device=self.device)
        n = self.layout.total
        if self.m is None and (optimizer.kind != "sgd" or optimizer.momentum != 0):
            self.m = torch.zeros(n, **f32)
        if self.v is None and optimizer.kind != "sgd":
            self.v = torch.zeros(n, **f32)

    def resize_vsw(self, new_k: int) -> None:
        """Change the number of VSW replicas at run time (jabas/train/trainer.py:485-575)
        without touching the buffers that stay: growing appends flat weight / gradient
        buffers and fills the new weights from the main replica with one kernel; shrinking
        drops the last ones.  Optimizer state, segment table and bucket layout are unchanged."""
        new_k = int(new_k)
        if not 1 <= new_k <= getattr(self.ops, "MAX_VSW", 16):
            raise ValueError("the number of VSWs must be between 1 and 16")
        f32 = dict(dtype=torch.float32, device=self.device)
        if new_k > self.K and self.share_weights:
            self.weights.extend([self.weights[0]] * (new_k - self.K))
            self.grads.extend(torch.zeros(self.layout.total, **f32) for _ in range(new_k - self.K))
        elif new_k > self.K:
            fresh = [torch.empty(self.layout.total, **f32) for _ in range(new_k - self.K)]
            self.ops.replicate(self.ctx, self.weights[0], fresh)
            self.launches += 1
            self.weights.extend(fresh)
            self.grads.extend(torch.zeros(self.layout.total, **f32) for _ in range(new_k - self.K))
        else:
            del self.weights[new_k:]
            del self.grads[new_k:]
        self.K = new_k

    def set_total_workers(self, total_num_decoupled_workers: int) -> None:
        """T changes when VSWs are added or removed at run time
        (jabas/train/trainer.py:543-544, 570-571)."""
        self.T = int(total_num_decoupled_workers)
        if self.similarity:
            assert self.T % 2 == 0

    # -- views ---------------------------------------------------------------------
    def bucket_range(self, b: int):
        return self.layout.buckets[b]

    def _sl(self, t: torch.Tensor, b: Optional[int]) -> torch.Tensor:
        if b is None:                                  # the whole flat buffer, padding included
            return t
        begin, end = self.layout.buckets[b]
        return t[begin:end]

    @property
    def main_grad(self) -> torch.Tensor:
        return self.grads[0]

    def _replicas(self, begin: int, end: int):
        """Weight buffers an update has to write: all K replicas, or the one they share."""
        ws = self.weights[:1] if self.share_weights else self.weights
        return [w[begin:end] for w in ws]

    def _ev_begin(self):
        if self.profile_events is None:
            return None
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        return e

    def _ev_end(self, kind: str, b, e0) -> None:
        if e0 is None:
            return
        e1 = torch.cuda.Event(enable_timing=True)
        e1.record()
        self.profile_events.append((kind, b, e0, e1))

    # -- per iteration ---------------------------------------------------------------
    def begin_iteration(self, similarity_step: Optional[bool] = None) -> None:
        self._sim_step = self.similarity if similarity_step is None else (similarity_step and self.similarity)
        self._pending.clear()
        self._deferred.clear()
        self._clip_active.clear()
        self.half_divided = set()
        if self._sim_step:
            self.stat.zero_()

    def aggregate(self, b: Optional[int], divide: bool = True, similarity: Optional[bool] = None) -> None:
        """Kernel 1: K VSW buckets -> main bucket / T (in place into VSW 0's buffer).
        ``divide=False`` leaves the plain local sum, for a caller-supplied comm hook that
        does its own averaging.  ``similarity`` (default: this iteration's setting) adds
        the undivided copy for the sub-group allreduce or, on one GPU, the statistic."""
        gs = [self._sl(g, b) for g in self.grads]
        out = gs[0]
        kw = {}
        if not divide:
            if self.K > 1:
                self.ops.vsw_aggregate(self.ctx, gs, out, 1.0)
                self.launches += 1
            return
        if similarity is None:
            similarity = self._sim_step
        if similarity:
            if not self._sim_step:                     # first similarity bucket of the iteration
                self._sim_step = True
                self.stat.zero_()
            if self.world > 1:
                kw["half_out"] = self._sl(self.half, b)
            else:
                kw.update(half_divisor=self.T / 2, stat=self.stat)
        ev = self._ev_begin()
        self.ops.vsw_aggregate(self.ctx, gs, out, float(self.T), **kw)
        self._ev_end("aggregate", b, ev)
        self.launches += 1

    def zero_grads(self) -> None:
        """One memset per VSW instead of a per-parameter ``zero_grad`` loop."""
        for g in self.grads:
            g.zero_()

    def allreduce(self, b: Optional[int]) -> None:
        """Sub-group SUM of the undivided copy and world SUM of the (already ÷T) bucket,
        both asynchronous; ``update`` waits for them on the current stream."""
        if self.world == 1:
            return
        works = []
        if self._sim_step and dist.get_world_size(self.sub_group) > 1:     # a one-rank sub-group owns its sum
            works.append(dist.all_reduce(self._sl(self.half, b), group=self.sub_group, async_op=True))
        works.append(dist.all_reduce(self._sl(self.main_grad, b), group=self.pg, async_op=True))
        self._pending[b] = works

    def wait_allreduce(self, b: int) -> None:
        for w in self._pending.pop(b, ()):
            w.wait()                               # stream-level wait, does not block the host

    def update(self, b: Optional[int] = None) -> None:
        """Kernel 2: fused optimizer update + write-back (+ statistic) on bucket ``b``, or
        on the whole flat buffer in one launch when ``b`` is None."""
        if b is None:
            for bb in list(self._pending):
                self.wait_allreduce(bb)
            begin, end = 0, self.layout.total
        else:
            self.wait_allreduce(b)
            begin, end = self.layout.buckets[b]
        if end == begin:
            return
        kw = dict(layout=self.dev_layout, base=begin)
        if self.collective == "peer":
            raise RuntimeError("with collective='peer' the update is part of the exchange")
        fused_stat = self._sim_step and self.world > 1 and self.similarity_mode == "fused"
        if fused_stat:
            kw.update(half=self.half[begin:end], half_divisor=self.T / 2, stat=self.stat)
        elif self._sim_step and self.world > 1:
            for bb in (range(self.layout.num_buckets) if b is None else (b,)):
                if bb not in self.half_divided:                            # E = half / (T/2)
                    self.ops.div_(self.ctx, self._sl(self.half, bb), self.T / 2)
                    self.half_divided.add(bb)
                    self.launches += 1
        nb = self.layout.num_buckets
        if (nb if b is None else b) in self._clip_active:
            kw["grad_scale"] = self.clip_coef[nb if b is None else b]
        elif nb in self._clip_active:
            kw["grad_scale"] = self.clip_coef[nb]
        if self._dyn is not None:
            kw["dynamic"] = self._dyn
        g = self.main_grad[begin:end]
        ws = self._replicas(begin, end)
        o = self.opt
        ev = self._ev_begin()
        if o.kind == "sgd":
            self.ops.sgd_momentum(self.ctx, g, ws, None if self.m is None else self.m[begin:end],
                                  o.groups, momentum=o.momentum, dampening=o.dampening,
                                  nesterov=o.nesterov, first_step=(self.steps == 0), **kw)
        else:
            groups = [dict(gr, step=self.steps + 1) for gr in o.groups]
            self.ops.adam(self.ctx, g, ws, self.m[begin:end], self.v[begin:end], groups,
                          beta1=o.betas[0], beta2=o.betas[1], eps=o.eps,
                          decoupled=(o.kind == "adamw"), **kw)
        self._ev_end("update", b, ev)
        self.launches += 1

    def defer(self, b: int, similarity: bool) -> None:
        """A comm hook hands bucket ``b`` over without aggregating it (see ``defer_local``)."""
        if similarity and not self._sim_step:
            self._sim_step = True
            self.stat.zero_()
        self._deferred.add(b)

    def materialize(self, b: Optional[int] = None) -> None:
        """Run the aggregation of deferred buckets after all (someone needs the averaged
        gradient itself, e.g. norm clipping)."""
        if self.collective == "peer" and self._deferred:
            raise NotImplementedError("norm clipping is not available with the peer-memory exchange")
        for bb in sorted(self._deferred if b is None else ({b} & self._deferred)):
            self._deferred.discard(bb)
            self.aggregate(bb, divide=True, similarity=self._sim_step)

    def step_buckets(self, buckets=None) -> None:
        """Optimizer update of the given buckets (None: the whole model), as one fused
        aggregate+update kernel where the aggregation was deferred."""
        nb = self.layout.num_buckets
        if self.collective == "peer" and self.exchange is not None:
            todo = range(nb) if buckets is None else list(buckets)
            if any(b not in self._deferred for b in todo):
                raise RuntimeError("the pipelined exchange aggregates the VSW gradients itself: the comm hooks "
                                   "must have left the bucket untouched")
            if buckets is None and len(self._deferred) == nb:
                self._deferred.clear()
                self.exchange_launch(None)             # one launch over the whole model
                return
            for b in todo:
                self._deferred.discard(b)
                self.exchange_launch(b)                # per bucket: overlaps the rest of backward
            return
        if self.collective == "peer":
            if buckets is not None or len(self._deferred) != nb:
                raise RuntimeError("this form of the peer-memory exchange runs once over the whole model, after "
                                   "every bucket's hook has deferred to it (weight_sync_method='sequential')")
            self._deferred.clear()
            self._peer_iteration()
            return
        if buckets is None:
            if len(self._deferred) == nb:
                self._deferred.clear()
                self.fused_local_step(None)
                return
            if not self._deferred:
                self.update(None)
                return
            buckets = range(nb)
        for b in buckets:
            if b in self._deferred:
                self._deferred.discard(b)
                self.fused_local_step(b)
            else:
                self.update(b)

    def clip_grad_norm(self, b: Optional[int], max_norm: float) -> torch.Tensor:
        """L2-norm clipping of the averaged gradient of bucket ``b`` (None: the whole model),
        as ``clip_grad_norm_for_overlap`` / ``clip_grad_norm_`` do in the reference
        (examples/gnmt/seq2seq/train/shard_optimizer.py:75-76, seq2seq/train/trainer.py:157-161).
        One reduction kernel over the gradient (after its allreduce) and a 1-thread kernel
        produce the coefficient on the device; the following ``update`` multiplies the
        gradient by it in registers when it is < 1.  Returns the norm (device scalar)."""
        nb = self.layout.num_buckets
        slot = nb if b is None else b
        self.materialize(b)
        if b is None:
            for bb in list(self._pending):
                self.wait_allreduce(bb)
        else:
            self.wait_allreduce(b)
        st = self.clip_stat[slot]
        st.zero_()
        self.ops.sumsq(self.ctx, self._sl(self.main_grad, b), st)
        self.ops.clip_coef(self.ctx, st, float(max_norm), self.clip_coef[slot])
        self.launches += 2
        self._clip_active[slot] = True
        return self.clip_coef[slot][1]

    def can_fuse_local(self) -> bool:
        """One GPU and few enough VSWs: aggregation and update can be one kernel."""
        return self.world == 1 and self.K <= getattr(self.ops, "MAX_FUSED_VSW", 0)

    def fused_local_step(self, b: Optional[int] = None, keep_grad: bool = False, sources=None,
                         divisor: Optional[float] = None, half_divisor: Optional[float] = None) -> None:
        """Single-GPU path in ONE launch over bucket ``b`` (None: the whole flat model):
        sum the K VSW gradients in registers, divide by T, update, write the new weights to
        all K replicas, accumulate the VSW-parity statistic.  The averaged gradient is only
        stored (into VSW 0's buffer) when ``keep_grad`` is set."""
        if b is None:
            begin, end = 0, self.layout.total
        else:
            begin, end = self.layout.buckets[b]
        if end == begin:
            return
        if sources is not None:              # raw device pointers of whole flat buffers (peer mappings)
            assert b is None and not keep_grad
            gs = list(sources)
        else:
            gs = [g[begin:end] for g in self.grads]
        ws = self._replicas(begin, end)
        kw = dict(layout=self.dev_layout, base=begin, grad_out=gs[0] if keep_grad else None)
        divisor = float(self.T) if divisor is None else float(divisor)
        if self._sim_step:
            kw.update(half_divisor=self.T / 2 if half_divisor is None else half_divisor, stat=self.stat)
        if self._dyn is not None:
            kw["dynamic"] = self._dyn
        o = self.opt
        ev = self._ev_begin()
        if o.kind == "sgd":
            self.ops.vsw_sgd_momentum(self.ctx, gs, divisor, ws,
                                      None if self.m is None else self.m[begin:end], o.groups,
                                      momentum=o.momentum, dampening=o.dampening, nesterov=o.nesterov,
                                      first_step=(self.steps == 0), **kw)
        else:
            groups = [dict(gr, step=self.steps + 1) for gr in o.groups]
            self.ops.vsw_adam(self.ctx, gs, divisor, ws, self.m[begin:end], self.v[begin:end], groups,
                              beta1=o.betas[0], beta2=o.betas[1], eps=o.eps,
                              decoupled=(o.kind == "adamw"), **kw)
        self._ev_end("fused_step", b, ev)
        self.launches += 1

    def end_iteration(self) -> None:
        self.steps += 1

    def finish_similarity(self) -> Optional[torch.Tensor]:
        """Cosine of the two half-gradients; identical on every rank (rank 0's value)."""
        if not self._sim_step:
            return None
        if self.exchange is not None:
            # every rank publishes its three sums, adds all ranks' in rank order, finalizes: the
            # cosine has the same bits everywhere and no broadcast is needed
            self.ops.exchange_cosine([self.exchange], [self.stat], [self.cos])
            self.launches += 1
            return self.cos
        if self.collective == "peer":              # finalised inside the exchange, identical on every rank
            return self.cos
        if self.world > 1 and self.similarity_mode == "pair_exchange":
            # jabas/train/trainer.py:470-483
            if self.rank in (self.src0, self.src1):
                n = self.layout.total
                both = [torch.empty(n, dtype=torch.float32, device=self.device) for _ in range(2)]
                dist.all_gather(both, self.half, group=self.pair_group)
                if self.rank == self.src0:
                    self.ops.dot_norms(self.ctx, both[0], both[1], self.stat)
                    self.launches += 1
        if self.rank == self.src0 or self.world == 1:
            self.ops.cosine_finalize(self.ctx, self.stat, self.cos)
            self.launches += 1
        if self.world > 1:
            dist.broadcast(self.cos, self.src0, group=self.pg)
        return self.cos

    # -- whole iteration, buckets in ready order (used by the benchmark and by tests) ---
    def run_iteration(self, similarity_step: Optional[bool] = None, overlap: bool = True,
                      per_bucket: Optional[bool] = None, fuse_local: Optional[bool] = None):
        """One pass of the path.  ``per_bucket=True`` walks the DDP buckets as the comm hooks do
        during backward (update of bucket b overlapping the collectives of bucket b+1); the
        default sends the whole flat model through each kernel and each collective in one
        call, which is faster when there is no backward pass to hide behind."""
        if self._dyn is not None:                      # kernels read the device-resident block
            self.push_hyperparams()
        cos = self._iteration_body(similarity_step, overlap, per_bucket, fuse_local)
        self.end_iteration()
        return cos

    def _iteration_body(self, similarity_step, overlap, per_bucket, fuse_local):
        self.begin_iteration(similarity_step)
        nb = self.layout.num_buckets
        if per_bucket is None:
            per_bucket = False
        if fuse_local is None:
            fuse_local = self.can_fuse_local() and not per_bucket
        if self.collective == "peer":
            return self._peer_iteration()
        if fuse_local:
            self.fused_local_step(None)
        elif not per_bucket:
            self.aggregate(None)
            self.allreduce(None)
            self.update(None)
        elif overlap:
            # software pipeline: bucket b's collectives fly while bucket b-1 is updated
            for b in range(nb):
                self.aggregate(b)
                self.allreduce(b)
                if b > 0:
                    self.update(b - 1)
            self.update(nb - 1)
        else:
            for b in range(nb):
                self.aggregate(b)
                self.allreduce(b)
            self.update(None)
        return self.finish_similarity()

    # -- CUDA-graph mode: the whole iteration (kernels and collectives) is one graph launch ----
    def push_hyperparams(self) -> None:
        """Refresh the device-resident hyper-parameter block with this iteration's values
        (lr and weight decay of every group, first-step flag, Adam step)."""
        o = self.opt
        if o.kind == "sgd":
            self._dyn.push_sgd(o.groups, momentum=o.momentum, dampening=o.dampening, nesterov=o.nesterov,
                               first_step=(self.steps == 0))
        else:
            self._dyn.push_adam([dict(gr, step=self.steps + 1) for gr in o.groups], beta1=o.betas[0],
                                beta2=o.betas[1], eps=o.eps, decoupled=(o.kind == "adamw"))

    def capture(self, similarity_step: Optional[bool] = None, overlap: bool = True,
                per_bucket: Optional[bool] = None, fuse_local: Optional[bool] = None, warmup: int = 2) -> None:
        """Capture one iteration into a CUDA graph.  ``warmup`` real iterations run first on
        the capture stream (they allocate the per-stream reduction workspace and bring up the
        NCCL communicators, neither of which may happen during capture).  Afterwards call
        :meth:`replay` once per iteration; what varies between iterations is read by the
        kernels from a device block that ``replay`` refreshes before the graph launch."""
        if self.profile_events is not None:
            raise RuntimeError("per-kernel event timing cannot be captured: unset profile_events")
        self._dyn = self.ops.DynHp(self.ctx)
        s = torch.cuda.Stream(self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(s):
            for _ in range(max(1, warmup)):
                self.push_hyperparams()
                self._iteration_body(similarity_step, overlap, per_bucket, fuse_local)
                self.end_iteration()
        s.synchronize()
        graph = torch.cuda.CUDAGraph()
        before = self.launches
        with torch.cuda.graph(graph, stream=s):
            self._iteration_body(similarity_step, overlap, per_bucket, fuse_local)
        self._graph, self._graph_stream = graph, s
        self.launches_per_replay = self.launches - before
        self.launches = before
        torch.cuda.current_stream(self.device).wait_stream(s)

    def replay(self) -> Optional[torch.Tensor]:
        """One iteration: a 288-byte hyper-parameter copy, then one graph launch."""
        self.push_hyperparams()
        self._graph.replay()
        self.launches += self.launches_per_replay
        self.end_iteration()
        return self.cos if self._sim_step else None

    # -- bookkeeping for roofline reports ----------------------------------------------
    def algorithmic_bytes(self, similarity_step: bool = True) -> Dict[str, int]:
        """Bytes each stage must move per iteration on this GPU (fp32 = 4 B)."""
        n, K = self.layout.num_params, self.K
        multi = self.world > 1
        Kw = 1 if self.share_weights else K          # weight buffers written by the update
        # K = 1 with nothing to clone: the division by T folds into the update's read of g
        agg = (4 * n * (K + 1) if (K > 1 or multi) else 0) + (4 * n if (similarity_step and multi) else 0)
        per_elem = (Kw + 4) if self.opt.kind == "sgd" else (Kw + 6)
        if self.opt.kind == "sgd" and self.opt.momentum == 0:
            per_elem = Kw + 2
        upd = 4 * n * per_elem + (4 * n if (similarity_step and multi) else 0)
        fused = 4 * n * (K + per_elem - 1)          # the averaged gradient stays in registers
        out = {"aggregate": agg, "update": upd, "total": agg + upd, "fused_step": fused}
        if self.exchange is not None:
            # one kernel; through THIS GPU's HBM: the aggregate pieces read K gradients and write the
            # local sum; the reduce pieces read that sum once (1/n by this rank, the rest by peers) and
            # write this rank's shard; the update pieces read the shard once from HBM (peers' reads of
            # it are served by L2 at best), p, m [, v] and write the replicas and the state
            w = self.world
            out["aggregate"] = 4 * n * (K + 1)
            out["peer_reduce"] = 4 * n + 4 * n // w
            out["update"] = 4 * n * (per_elem - 1) + 4 * n // w
            out["exchange"] = out["aggregate"] + out["peer_reduce"] + out["update"]
            out["nvlink_in"] = 2 * 4 * n * (w - 1) // w
            return out
        if self.collective == "peer":
            # two-rank direct form: an aggregate kernel, then the fused kernel: this GPU's sum is read
            # once by its own update kernel and once by the peer's; the remote sum arrives over
            # NVLink (4n bytes in)
            out["aggregate"] = 4 * n * (K + 1)
            out["fused_step"] = 4 * n * (per_elem + 1)
            out["nvlink_in"] = 4 * n
        return out

    def close(self) -> None:
        """Release in dependency order: captured graph (it holds the kernels and collectives of an
        iteration), exchange handle, symmetric-memory buffers and their handles, layout, context."""
        self._graph = None
        self._graph_stream = None
        if self._dyn is not None:
            self._dyn.close()
            self._dyn = None
        if self.exchange is not None:
            self.exchange.close()
            self.exchange = None
        for name in ("_px_h", "_pg_h", "_fl_h", "px", "pgrad", "xflags"):
            if hasattr(self, name):
                setattr(self, name, None)
        if self.dev_layout is not None:
            self.dev_layout.close()
            self.dev_layout = None
        self.ctx.close()
