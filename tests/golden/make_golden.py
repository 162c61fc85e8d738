"""Generates ``similarity_hook_ws2.npz`` by running the REFERENCE'S OWN code for the part
of the gradient path whose source is present in the reference tree:

  * ``jabas/ddp_comm_hooks/similarity_allreduce.py`` — ``GradientSimilarityState``,
    ``subgroup_allreduce_hook``, ``similimarity_allreduce_hook`` (imported unmodified);
  * ``jabas/train/trainer.py`` — ``JABASTrainer._build_subgroup`` and
    ``JABASTrainer._compute_cosine_similarity`` (imported unmodified, called on a
    stand-in ``self`` that carries only the attributes those two methods read).

The run is two gloo ranks on CPU.  What the reference imports from the absent ``iidp``
package is stubbed in ``sys.modules`` before the import:

  * ``_allreduce_sum_fut(group, tensor)``  = asynchronous SUM allreduce, future -> [tensor];
  * ``IIDPState(process_group, T)``, ``iidp_allreduce_hook(state, bucket)`` = divide the
    bucket by T, SUM-allreduce it over the process group (the averaging convention fixed
    by the oracle, since IIDP's source is not available);
  * every other ``iidp.*`` / ``statsmodels.*`` name resolves to an empty placeholder class,
    only so that ``import jabas`` gets through its unrelated imports.

It needs the reference checkout and therefore only runs where that exists:

    python tests/golden/make_golden.py /path/to/reference

The fixture stores inputs (per rank, per VSW, per bucket) and the reference's outputs
(world-averaged buckets, E placeholders, cosine), all float32.
"""
import importlib.abc
import importlib.machinery
import os
import sys
import types

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
BUCKETS = [1000, 4099, 257]          # elements per bucket (ragged on purpose)
K = 2                                # VSWs per rank
WORLD = 2


class _Placeholder(types.ModuleType):
    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)
        cls = type(name, (object,), {"__init__": lambda self, *a, **k: None})
        setattr(self, name, cls)
        return cls


class _StubFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    PREFIXES = ("iidp", "statsmodels")

    def find_spec(self, fullname, path=None, target=None):
        if fullname.split(".")[0] in self.PREFIXES:
            return importlib.machinery.ModuleSpec(fullname, self, is_package=True)
        return None

    def create_module(self, spec):
        m = _Placeholder(spec.name)
        m.__path__ = []
        return m

    def exec_module(self, module):
        pass


def _install_iidp_stubs():
    sys.meta_path.insert(0, _StubFinder())
    import iidp.ddp_comm_hooks.default_hooks as dh
    import iidp.ddp_comm_hooks.iidp_allreduce as ia
    import iidp.utils.global_vars as gv

    def _allreduce_sum_fut(group, tensor):
        return dist.all_reduce(tensor, group=group, async_op=True).get_future().then(lambda f: [tensor])

    class IIDPState(object):
        def __init__(self, process_group, total_num_decoupled_workers):
            self.process_group = process_group
            self.total_num_decoupled_workers = total_num_decoupled_workers

    def iidp_allreduce_hook(state, bucket):
        t = bucket.get_tensors()[0]
        t.div_(state.total_num_decoupled_workers)
        return _allreduce_sum_fut(state.process_group, t)

    dh._allreduce_sum_fut = _allreduce_sum_fut
    ia.IIDPState, ia.iidp_allreduce_hook = IIDPState, iidp_allreduce_hook
    # names the reference star-imports through jabas/utils/global_vars.py:1; values unused here
    gv.REQUIRED_CONFIG_FILES, gv.REGISTERED_WEIGHT_SYNC_METHODS = [], []
    gv.__all__ = ["REQUIRED_CONFIG_FILES", "REGISTERED_WEIGHT_SYNC_METHODS"]
    if not hasattr(dist, "_GradBucket"):            # the 1.8 name used in a type annotation
        dist._GradBucket = dist.GradBucket


class _Bucket:                                       # dist._GradBucket of PyTorch 1.8, as the hook uses it
    def __init__(self, tensor):
        self._t = tensor

    def get_tensors(self):
        return [self._t]


def _inputs(rank):
    g = torch.Generator().manual_seed(1234 + rank)
    common = [torch.randn(n, generator=g) * 1e-3 for n in BUCKETS]
    return [[(torch.randn(n, generator=g) * 1e-3 + 0.5 * common[b]) for b, n in enumerate(BUCKETS)]
            for _ in range(K)]


def _worker(rank, ref_root, port, q):
    sys.path.insert(0, ref_root)
    _install_iidp_stubs()
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=WORLD)
    from jabas.ddp_comm_hooks import similarity_allreduce as ref_hooks
    from jabas.train.trainer import JABASTrainer

    me = types.SimpleNamespace()
    me.sub_groups_idx = [[], []]
    JABASTrainer._build_subgroup(me)                 # jabas/train/trainer.py:427-432
    me.sub_groups = [dist.new_group(ix) for ix in me.sub_groups_idx]
    me.first_subgroup_src_rank, me.second_subgroup_src_rank = me.sub_groups_idx[0][0], me.sub_groups_idx[1][0]
    me.sub_groups.append(dist.new_group([me.first_subgroup_src_rank, me.second_subgroup_src_rank]))
    me.grad_placeholders = [[], []]
    me.cos_placeholder = torch.rand(1)
    T = WORLD * K
    me.similarity_state = ref_hooks.GradientSimilarityState(
        dist.group.WORLD, T, me.sub_groups[rank % 2], me.grad_placeholders[rank % 2], 1)
    hook = ref_hooks.similimarity_allreduce_hook(ref_hooks.subgroup_allreduce_hook)

    grads = _inputs(rank)
    out = {}
    for b in range(len(BUCKETS)):
        buf = grads[0][b].clone()
        for k in range(1, K):                        # local aggregation, ascending k
            buf.add_(grads[k][b])
        fut = hook(me.similarity_state, _Bucket(buf))
        res = fut.wait()
        out[f"avg_r{rank}_b{b}"] = res[0].numpy().copy()
    for b, e in enumerate(me.similarity_state.grad_placeholder):
        out[f"half_r{rank}_b{b}"] = e.numpy().copy()
    JABASTrainer._compute_cosine_similarity(me)      # jabas/train/trainer.py:470-483
    out[f"cos_r{rank}"] = np.float32(float(me.cos_placeholder))
    for k in range(K):
        for b in range(len(BUCKETS)):
            out[f"grad_r{rank}_k{k}_b{b}"] = grads[k][b].numpy().copy()
    q.put(out)
    dist.barrier()
    dist.destroy_process_group()


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py /path/to/reference-checkout")
    ref_root = sys.argv[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, ref_root, 29871, q)) for r in range(WORLD)]
    for p in procs:
        p.start()
    merged = {}
    for _ in procs:
        merged.update(q.get(timeout=300))
    for p in procs:
        p.join()
    merged["meta_K_world_T"] = np.array([K, WORLD, K * WORLD], np.int64)
    np.savez_compressed(os.path.join(HERE, "similarity_hook_ws2.npz"), **merged)
    print("cos", merged["cos_r0"], merged["cos_r1"], "keys", len(merged))


if __name__ == "__main__":
    main()
