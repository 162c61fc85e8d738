"""TEST INFRASTRUCTURE — CPU restatement of the reference's gradient path, op by op.

Only tests, the smoke check and the benchmark's CPU-baseline / reference arm may import
this module; the product never does.

The reference executes this path through stock PyTorch ops and ``torch.distributed``
collectives.  Its own modules cannot be imported here (``import iidp`` fails: the IIDP
submodule is absent), so the sequence is restated on CPU tensors with the gloo backend,
following

  jabas/ddp_comm_hooks/similarity_allreduce.py:20-45   clone -> sub-group SUM -> div_(T/2)
                                                       -> world allreduce averaged over T
  jabas/train/trainer.py:427-483                       parity sub-groups, pair group,
                                                       cat -> all_gather -> cosine_similarity
                                                       on the first rank -> broadcast
  examples/gnmt/seq2seq/train/shard_optimizer.py:30-90 per-parameter optimizer step
  jabas/train/trainer.py:530-534                       per-parameter weight copy to the VSWs

PARITY UNPINNED for the parts whose source is absent (local aggregation order, where
the division by T happens, the optimizer arithmetic of PyTorch v1.8.1): they are fixed
here as  buf = g_0; buf += g_k (k ascending); buf /= T  before the SUM allreduce, and
the v1.8.1 functional forms of SGD / Adam / AdamW.

Two arithmetic back-ends:
  ``arith="torch"``  stock per-tensor torch ops, as the reference would run them on CPU
                     (this is what the CPU baseline times, with all host threads);
  ``arith="c"``      the C oracle (explicit fp32 roundings) — the bit-exact contract
                     the CUDA kernels are tested against.
On one rank the statistic uses the even-index and odd-index VSWs as the two halves (an
extension; the reference asserts an even world size, jabas/train/trainer.py:430).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import numpy as np
import torch
import torch.distributed as dist

from . import gradpath as C


class ReferencePath:
    def __init__(self, layout, num_vsw: int, optimizer: dict, *, total_num_decoupled_workers: int,
                 similarity: bool = True, arith: str = "torch", process_group=None,
                 world: Optional[int] = None):
        self.layout, self.K, self.opt = layout, int(num_vsw), dict(optimizer)
        self.T = int(total_num_decoupled_workers)
        self.similarity = similarity
        self.arith = arith
        if world is None:
            world = dist.get_world_size() if dist.is_initialized() else 1
        self.world = world
        self.rank = dist.get_rank() if self.world > 1 else 0
        self.pg = process_group
        n = layout.total
        self.weights = [torch.zeros(n) for _ in range(self.K)]
        self.grads = [torch.zeros(n) for _ in range(self.K)]
        self.m = torch.zeros(n)
        self.v = torch.zeros(n)
        self.steps = 0
        self.cos: Optional[float] = None
        self.grad_placeholder: List[torch.Tensor] = []     # E_b of this rank's sub-group
        self._other: List[torch.Tensor] = []               # single-rank form: O_b
        if similarity:
            assert self.T % 2 == 0                          # similarity_allreduce.py:13
        if self.world > 1:
            assert self.world % 2 == 0                      # trainer.py:430
            idx = [[], []]
            for i in range(self.world):                     # trainer.py:431-432
                idx[i % 2].append(i)
            self.sub_groups = [dist.new_group(ix) for ix in idx]            # trainer.py:441-442
            self.src0, self.src1 = idx[0][0], idx[1][0]
            self.sub_groups.append(dist.new_group([self.src0, self.src1]))  # trainer.py:445
        # per-parameter views, in optimizer order (parameters() order)
        self._pviews = []
        for s in layout.slots:
            sl = slice(s.offset, s.offset + s.numel)
            self._pviews.append((s, sl))

    # -- hook chain, one bucket -------------------------------------------------------
    def _bucket(self, t: torch.Tensor, b: int) -> torch.Tensor:
        begin, end = self.layout.buckets[b]
        return t[begin:end]

    def reduce_bucket(self, b: int, sim_step: bool) -> None:
        gs = [self._bucket(g, b) for g in self.grads]
        buf = gs[0]
        if sim_step and self.world == 1:
            e = gs[0].clone()
            for k in range(2, self.K, 2):
                e.add_(gs[k])
            o = gs[1].clone()
            for k in range(3, self.K, 2):
                o.add_(gs[k])
            self.grad_placeholder.append(e.div_(self.T / 2))
            self._other.append(o.div_(self.T / 2))
        for k in range(1, self.K):                          # local aggregation, ascending k
            buf.add_(gs[k])
        if sim_step and self.world > 1:
            tensor = buf.detach().clone()                   # similarity_allreduce.py:28
            dist.all_reduce(tensor, group=self.sub_groups[self.rank % 2])   # :30
            self.grad_placeholder.append(tensor.div_(self.T / 2))           # :32
        buf.div_(self.T)                                    # world average over T
        if self.world > 1:
            dist.all_reduce(buf, group=self.pg)             # similarity_allreduce.py:42

    # -- optimizer step + weight copy --------------------------------------------------
    def _groups(self):
        return self.opt["groups"]

    def optimizer_step(self) -> None:
        o = self.opt
        kind = o["kind"]
        step = self.steps + 1
        g_all, p_all = self.grads[0], self.weights[0]
        for s, sl in self._pviews:
            hp = self._groups()[s.group]
            g, p, m, v = g_all[sl], p_all[sl], self.m[sl], self.v[sl]
            if self.arith == "c":
                gn, pn, mn, vn = (x.numpy() for x in (g, p, m, v))
                if kind == "sgd":
                    C.sgd_momentum(gn, pn, mn, lr=hp["lr"], weight_decay=hp.get("weight_decay", 0.0),
                                   momentum=o.get("momentum", 0.0), dampening=o.get("dampening", 0.0),
                                   nesterov=o.get("nesterov", False), first_step=(self.steps == 0))
                else:
                    C.adam(gn, pn, mn, vn, lr=hp["lr"], weight_decay=hp.get("weight_decay", 0.0),
                           beta1=o["betas"][0], beta2=o["betas"][1], eps=o["eps"], step=step,
                           decoupled=(kind == "adamw"))
                continue
            wd = hp.get("weight_decay", 0.0)
            lr = hp["lr"]
            if kind == "sgd":                               # torch/optim/_functional.py v1.8.1 `sgd`
                d_p = g
                mu = o.get("momentum", 0.0)
                if wd != 0:
                    d_p = d_p.add(p, alpha=wd)
                if mu != 0:
                    if self.steps == 0:
                        m.copy_(d_p)
                    else:
                        m.mul_(mu).add_(d_p, alpha=1 - o.get("dampening", 0.0))
                    d_p = d_p.add(m, alpha=mu) if o.get("nesterov", False) else m
                p.add_(d_p, alpha=-lr)
            else:                                           # v1.8.1 `adam` / `adamw`
                b1, b2 = o["betas"]
                grad = g
                if kind == "adamw":
                    p.mul_(1 - lr * wd)
                elif wd != 0:
                    grad = grad.add(p, alpha=wd)
                bc1, bc2 = 1 - b1 ** step, 1 - b2 ** step
                m.mul_(b1).add_(grad, alpha=1 - b1)
                v.mul_(b2).addcmul_(grad, grad, value=1 - b2)
                denom = (v.sqrt() / math.sqrt(bc2)).add_(o["eps"])
                p.addcdiv_(m, denom, value=-(lr / bc1))

    def copy_weights(self) -> None:
        for k in range(1, self.K):                          # trainer.py:530-534 idiom
            for _, sl in self._pviews:
                self.weights[k][sl].copy_(self.weights[0][sl])

    # -- cosine (trainer.py:470-483) ----------------------------------------------------
    def compute_cosine_similarity(self) -> float:
        if self.world == 1:
            e, o = torch.cat(self.grad_placeholder), torch.cat(self._other)
            cos = self._cosine(e, o)
            self._other = []
        else:
            cos_t = torch.zeros(1)
            if self.rank in (self.src0, self.src1):
                gathered = [torch.cat([torch.zeros_like(g) for g in self.grad_placeholder])
                            for _ in range(2)]
                mine = torch.cat(self.grad_placeholder)
                dist.all_gather(gathered, mine, group=self.sub_groups[-1])
                if self.rank == self.src0:
                    cos_t[0] = self._cosine(gathered[0], gathered[1])
            dist.broadcast(cos_t, self.src0)
            cos = float(cos_t)
        self.grad_placeholder = []
        self.cos = cos
        return cos

    def _cosine(self, e: torch.Tensor, o: torch.Tensor) -> float:
        if self.arith == "c":
            return C.cosine_from_stat(C.dot_norms(e.numpy(), o.numpy()))
        return float(torch.nn.functional.cosine_similarity(e, o, dim=0))

    # -- one iteration -------------------------------------------------------------------
    def run_iteration(self, similarity_step: Optional[bool] = None) -> Optional[float]:
        sim = self.similarity if similarity_step is None else (similarity_step and self.similarity)
        for b in range(self.layout.num_buckets):
            self.reduce_bucket(b, sim)
        self.optimizer_step()
        self.copy_weights()
        cos = self.compute_cosine_similarity() if sim else None
        self.steps += 1
        return cos
