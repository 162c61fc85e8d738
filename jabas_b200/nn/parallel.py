"""``IndependentIdenticalDataParallel`` — the DDP variant the reference expects from its
patched PyTorch (constructor call at jabas/train/trainer.py:515-521; the patch itself is
absent from the reference tree).

K wrappers, one per virtual stream worker (VSW), live in one process and share one
``VSWReducer``.  The reducer owns the flat HBM storage (``GradientPath``): every VSW's
parameters and ``.grad`` tensors are views into it (``gradient_as_bucket_view``), buckets
are assigned DDP-style, and when bucket ``b`` is complete on all K VSWs the comm hook of
VSW 0 is fired once with a lazily aggregating bucket, the hooks of VSWs 1..K-1 with their
own (never communicating) buckets — the hook layout of jabas/train/trainer.py:461-468.
"""
from __future__ import annotations

import contextlib
import threading
from typing import Callable, List, Optional

import torch
import torch.nn as nn

from ..gradient_path import GradientPath
from ..layout import DEFAULT_BUCKET_CAP_MB, FlatLayout, layout_from_module


class VSWGradBucket:
    """What a comm hook receives.  Speaks both bucket protocols: ``get_tensors()`` of
    PyTorch 1.8 (``dist._GradBucket``, used at
    jabas/ddp_comm_hooks/similarity_allreduce.py:21-28) and ``buffer()/index()/is_last()``
    of current PyTorch.  For VSW 0 the local aggregation of the K VSW buckets is lazy so
    that the library's hooks can fuse it with the averaging and the clone."""

    def __init__(self, engine: GradientPath, index: int, is_last: bool, vsw: int, scope=None):
        self.engine, self._index, self._is_last, self.vsw = engine, index, is_last, vsw
        self._summed = self._averaged = False
        self.deferred = False             # the hook left aggregation AND exchange to the optimizer step
        # every kernel of the path runs on ONE stream, whatever stream a future callback
        # happens to be on: the statistic accumulates bucket after bucket
        self._scope = scope if scope is not None else contextlib.nullcontext

    # -- protocol ------------------------------------------------------------------
    def index(self) -> int:
        return self._index

    def is_last(self) -> bool:
        return self._is_last

    def buffer(self, materialize: bool = True) -> torch.Tensor:
        if materialize and self.vsw == 0 and not (self._summed or self._averaged):
            with self._scope():
                self.engine.aggregate(self._index, divide=False)  # plain local sum
            self._summed = True
        begin, end = self.engine.layout.buckets[self._index]
        return self.engine.grads[self.vsw][begin:end]

    def get_tensors(self, materialize: bool = True) -> List[torch.Tensor]:
        return [self.buffer(materialize)]

    def set_buffer(self, tensor: torch.Tensor) -> None:
        buf = self.buffer(materialize=False)
        if tensor.data_ptr() != buf.data_ptr():
            buf.copy_(tensor)

    def gradients(self) -> List[torch.Tensor]:
        lay = self.engine.layout
        flat = self.engine.grads[self.vsw]
        return [flat[lay.slots[i].offset:lay.slots[i].offset + lay.slots[i].numel].view(lay.slots[i].shape)
                for i in lay.bucket_indices[self._index]]

    # -- fused forms used by this library's hooks --------------------------------------
    def ensure_averaged(self, total_num_decoupled_workers) -> None:
        """Main bucket <- (sum of the K VSW buckets) / T, in as few passes as possible."""
        if self._averaged:
            return
        eng = self.engine
        eng.set_total_workers(total_num_decoupled_workers)
        if eng.defer_local and not self._summed:
            with self._scope():
                eng.defer(self._index, similarity=False)
            self._averaged = self.deferred = True
            return
        with self._scope():
            if self._summed:
                eng.ops.div_(eng.ctx, self.buffer(materialize=False), float(total_num_decoupled_workers))
                eng.launches += 1
            else:
                eng.aggregate(self._index, divide=True, similarity=False)
        self._averaged = True

    def aggregate_with_half(self, total_num_decoupled_workers) -> torch.Tensor:
        """One kernel: main bucket <- local sum / T, and the undivided sum for the parity
        sub-group (several GPUs) or the VSW-parity statistic (one GPU).  Returns the tensor
        to SUM-allreduce over the sub-group."""
        eng = self.engine
        eng.set_total_workers(total_num_decoupled_workers)
        if self._summed or self._averaged:
            raise RuntimeError("the bucket was already aggregated by an earlier hook")
        if eng.defer_local:
            with self._scope():
                eng.defer(self._index, similarity=True)
            self._averaged = self.deferred = True
            return eng.stat
        with self._scope():
            eng.aggregate(self._index, divide=True, similarity=True)
        self._averaged = True
        begin, end = eng.layout.buckets[self._index]
        return eng.half[begin:end] if eng.half is not None else eng.stat

    def half_entry(self, tensor: torch.Tensor, subgroup_total):
        """Entry of ``state.grad_placeholder`` for this bucket.  In ``pair_exchange`` mode
        it is the materialised E_b = sum / (T/2), as in the reference; in ``fused`` mode the
        division is folded into the update kernel and the entry is the undivided view."""
        eng = self.engine
        if eng.world > 1 and eng.similarity_mode == "pair_exchange":
            with self._scope():
                eng.ops.div_(eng.ctx, tensor, float(subgroup_total))
            eng.launches += 1
            eng.half_divided.add(self._index)
        return tensor


class VSWReducer:
    """Shared by the K wrappers of one GPU: flat storage, readiness counting, hook firing."""

    def __init__(self, device, num_local_models: int, total_num_models: int,
                 bucket_cap_mb: float = DEFAULT_BUCKET_CAP_MB, similarity: bool = False,
                 similarity_mode: str = "fused", process_group=None, backend=None,
                 first_bucket_bytes: Optional[int] = None, share_weights: bool = False,
                 collective: str = "nccl", staging: str = "register", peer_form: str = "pipeline"):
        self.device = torch.device(device)
        self.staging = staging
        self.peer_form = peer_form
        self.K = int(num_local_models)
        self.T = int(total_num_models)
        self.bucket_cap_mb = bucket_cap_mb
        self.first_bucket_bytes = first_bucket_bytes
        self.share_weights = share_weights
        self.collective = collective
        self.similarity, self.similarity_mode = similarity, similarity_mode
        self.process_group, self.backend = process_group, backend
        self.engine: Optional[GradientPath] = None
        self.layout: Optional[FlatLayout] = None
        self.wrappers: List[Optional["IndependentIdenticalDataParallel"]] = [None] * self.K
        self.path_stream: Optional[torch.cuda.Stream] = None
        self._lock = threading.Lock()
        self._fire_lock = threading.Lock()    # hooks fire one bucket at a time, in bucket order
        self.futures: List[torch.futures.Future] = []
        self.require_sync = True
        self.buffers_flat: List[Optional[torch.Tensor]] = []     # one flat byte buffer of module buffers per VSW
        self.num_module_buffers = 0
        self._reset_counters()

    # -- set-up -------------------------------------------------------------------------
    def attach(self, wrapper: "IndependentIdenticalDataParallel") -> None:
        k = wrapper.model_index
        if self.engine is None:
            extra = {} if self.first_bucket_bytes is None else dict(first_bucket_bytes=self.first_bucket_bytes)
            self.layout = layout_from_module(wrapper.module, None, self.bucket_cap_mb, **extra)
            self.engine = GradientPath(self.layout, self.K, self.device, None,
                                       total_num_decoupled_workers=self.T, process_group=self.process_group,
                                       similarity=self.similarity, similarity_mode=self.similarity_mode,
                                       backend=self.backend, share_weights=self.share_weights,
                                       collective=self.collective, staging=self.staging,
                                       peer_form=self.peer_form)
            if self.device.type == "cuda":
                self.path_stream = torch.cuda.Stream(self.device)
        self.wrappers[k] = wrapper
        params = [p for p in wrapper.module.parameters() if p.requires_grad]
        if len(params) != len(self.layout.slots):
            raise ValueError("every VSW must wrap a copy of the same module")
        wrapper._params = params
        with torch.no_grad():
            for p, slot in zip(params, self.layout.slots):
                if tuple(p.shape) != slot.shape:
                    raise ValueError(f"parameter {slot.name}: shape differs between VSWs")
                w = self.engine.weights[k][slot.offset:slot.offset + slot.numel].view(slot.shape)
                w.copy_(p.data)
                p.data = w
        self.install_grad_views(k)
        self._flatten_buffers(k, wrapper.module)
        for i, p in enumerate(params):
            p.register_post_accumulate_grad_hook(self._make_hook(k, self.layout.slots[i].bucket))

    def _flatten_buffers(self, k: int, module: nn.Module) -> None:
        """Module BUFFERS (BatchNorm running statistics, step counters) of VSW ``k`` become views
        of one flat buffer per dtype and VSW, every buffer on a 16-byte boundary, so that all of
        them are synchronised by one copy kernel (and one broadcast) per dtype instead of one op
        per buffer.  One flat buffer per DTYPE: ``torch.save`` refuses tensors that view one
        storage as different types, and ``state_dict()`` must stay saveable as it is."""
        named = [(n, b) for n, b in module.named_buffers() if b is not None]
        by_dtype = {}
        for name, buf in named:
            by_dtype.setdefault(buf.dtype, []).append(buf)
        flats = []
        for dtype in sorted(by_dtype, key=str):
            bufs = by_dtype[dtype]
            item = bufs[0].element_size()
            align = max(1, 16 // item)
            sizes = [(b.numel() + align - 1) // align * align for b in bufs]
            total = max(align, sum(sizes))
            total = (total * item + 15) // 16 * 16 // item
            flat = torch.zeros(total, dtype=dtype, device=self.device)
            pos = 0
            for buf, size in zip(bufs, sizes):
                view = flat[pos:pos + buf.numel()].view(buf.shape)
                with torch.no_grad():
                    view.copy_(buf)
                # same tensor object, new storage: the buffer keeps a version counter of its own (a
                # view would share the flat buffer's, and BatchNorm's in-place update of one layer's
                # statistics would invalidate the ones another layer saved for backward)
                buf.data = view
                pos += size
            flats.append(flat)
        while len(self.buffers_flat) <= k:
            self.buffers_flat.append(None)
        self.buffers_flat[k] = flats
        self.num_module_buffers = len(named)

    @staticmethod
    def _as_f32(t: torch.Tensor) -> torch.Tensor:
        """A flat buffer of any dtype as float32 words, for the bit-copy kernel."""
        return t.view(torch.uint8).view(torch.float32)

    def sync_buffers(self, group=None) -> None:
        """Module buffers of every VSW on every rank <- rank 0's main replica (VSW 0), the
        ``broadcast_buffers=True`` behaviour of DistributedDataParallel that the reference's
        patched wrapper keeps (it receives ``sync_buffer_barrier`` for exactly this step,
        jabas/train/trainer.py:515-521, 584-588): per dtype one broadcast of the flat buffer
        between ranks and one replicate kernel between the VSWs, on the current stream."""
        sets = [f for f in self.buffers_flat[:self.K] if f]
        if not self.num_module_buffers or not sets:
            return
        import torch.distributed as dist
        multi = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
        eng = self.engine
        for g, main in enumerate(sets[0]):
            if multi:
                dist.broadcast(main, 0, group=group)
            if len(sets) > 1:
                eng.ops.replicate(eng.ctx, self._as_f32(main), [self._as_f32(fs[g]) for fs in sets[1:]])
                eng.launches += 1

    def resize(self, new_k: int, total_num_models: int) -> None:
        """Grow or shrink the set of VSWs.  Wrappers of removed VSWs are dropped here; the
        caller constructs ``IndependentIdenticalDataParallel`` wrappers for the new indices,
        whose ``attach`` finds the flat buffers already in place."""
        self.engine.resize_vsw(new_k)
        if new_k > self.K:
            self.wrappers.extend([None] * (new_k - self.K))
        else:
            del self.wrappers[new_k:]
            del self.buffers_flat[new_k:]
        self.K, self.T = int(new_k), int(total_num_models)
        self.engine.set_total_workers(total_num_models)
        self._reset_counters()

    def install_grad_views(self, k: int) -> None:
        flat = self.engine.grads[k]
        for p, slot in zip(self.wrappers[k]._params, self.layout.slots):
            view = flat[slot.offset:slot.offset + slot.numel].view(slot.shape)
            if p.grad is None or p.grad.data_ptr() != view.data_ptr():
                p.grad = view

    @contextlib.contextmanager
    def stream_scope(self):
        """Run the body on the path stream, ordered after the caller's current stream, and
        make the caller's stream wait for it afterwards."""
        if self.path_stream is None:
            yield
            return
        cur = torch.cuda.current_stream(self.device)
        if cur == self.path_stream:
            yield
            return
        self.path_stream.wait_stream(cur)
        with torch.cuda.stream(self.path_stream):
            yield
        cur.wait_stream(self.path_stream)

    def _reset_counters(self) -> None:
        nb = self.layout.num_buckets if self.layout is not None else 0
        self._param_count = [[0] * nb for _ in range(self.K)]
        self._vsw_done = [0] * nb
        self._events = [[] for _ in range(nb)]
        self._next_bucket = 0

    # -- per iteration -------------------------------------------------------------------
    def prepare_for_backward(self, similarity_step: bool = False) -> None:
        """Called once per synchronising micro-step, before the K backward passes."""
        self._reset_counters()
        self.futures = []
        if self.path_stream is not None:
            self.path_stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.path_stream):
                self.engine.begin_iteration(similarity_step)
        else:
            self.engine.begin_iteration(similarity_step)

    def _make_hook(self, k: int, b: int) -> Callable:
        need = len(self.layout.bucket_indices[b])

        def hook(param):
            if not self.require_sync:
                return
            fire = False
            with self._lock:
                self._param_count[k][b] += 1
                if self._param_count[k][b] == need:
                    if self.device.type == "cuda":
                        ev = torch.cuda.Event()
                        ev.record(torch.cuda.current_stream(self.device))
                        self._events[b].append(ev)
                    self._vsw_done[b] += 1
                    fire = self._vsw_done[b] == self.K
            if fire:
                self._fire_ready_buckets()
        return hook

    def finish_backward(self, k: int, find_unused: bool) -> None:
        """End of VSW ``k``'s backward pass.  Parameters that took no part in the graph never fire
        their hook; their gradient views are the zeros the iteration started with.  With
        ``find_unused_parameters`` their buckets are completed here (a zero contribution, as in
        DistributedDataParallel); without it an incomplete bucket is an error, as there."""
        if not self.require_sync:
            return
        fire = False
        with self._lock:
            for b in range(self.layout.num_buckets):
                need = len(self.layout.bucket_indices[b])
                if self._param_count[k][b] >= need:
                    continue
                if not find_unused:
                    raise RuntimeError(
                        f"VSW {k}: {need - self._param_count[k][b]} parameters of bucket {b} received no gradient in "
                        "this backward pass; pass find_unused_parameters=True if that is intended")
                self._param_count[k][b] = need
                if self.device.type == "cuda":
                    ev = torch.cuda.Event()
                    ev.record(torch.cuda.current_stream(self.device))
                    self._events[b].append(ev)
                self._vsw_done[b] += 1
                fire = fire or self._vsw_done[b] == self.K
        if fire:
            self._fire_ready_buckets()

    def _fire_ready_buckets(self) -> None:
        """Fire comm hooks in bucket order (every rank must issue its collectives in the
        same order), for every bucket that is complete on all K VSWs."""
        with self._fire_lock:                 # K backward passes may run in K threads
            while True:
                with self._lock:
                    b = self._next_bucket
                    if b >= self.layout.num_buckets or self._vsw_done[b] < self.K:
                        return
                    self._next_bucket += 1
                self._fire(b)

    def _fire(self, b: int) -> None:
        last = b == self.layout.num_buckets - 1
        if self.path_stream is not None:
            for ev in self._events[b]:
                self.path_stream.wait_event(ev)
            ctx = torch.cuda.stream(self.path_stream)
        else:
            ctx = contextlib.nullcontext()
        with ctx:
            for k in range(self.K - 1, -1, -1):               # VSW 0 last: it consumes the others
                w = self.wrappers[k]
                bucket = VSWGradBucket(self.engine, b, last, k, self.stream_scope)
                if w._hook is None:
                    if k == 0:
                        raise RuntimeError("no comm hook registered on VSW 0")
                    continue
                fut = w._hook(w._hook_state, bucket)
                if k == 0:
                    self.futures.append(fut)

    def wait(self) -> None:
        """Make the current stream wait for every bucket's hook chain."""
        for fut in self.futures:
            fut.wait()
        self.futures = []
        if self.path_stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.path_stream)


class IndependentIdenticalDataParallel(nn.Module):
    """Constructor arguments follow jabas/train/trainer.py:515-521.  ``reducer`` is the
    object shared by the K wrappers of this GPU (an addition: the patched PyTorch keeps
    that state inside its C++ reducer)."""

    def __init__(self, module: nn.Module, device_ids=None, output_device=None,
                 find_unused_parameters: bool = False, gradient_as_bucket_view: bool = True,
                 model_index: int = 0, num_local_models: int = 1, total_num_models: int = 1,
                 sync_buffer_barrier=None, bucket_cap_mb: float = DEFAULT_BUCKET_CAP_MB,
                 reducer: Optional[VSWReducer] = None, process_group=None):
        super().__init__()
        if not gradient_as_bucket_view:
            raise ValueError("gradient_as_bucket_view must be True")      # jabas/train/trainer.py:82-86
        self.module = module
        self.device_ids, self.output_device = device_ids, output_device
        self.find_unused_parameters = find_unused_parameters
        self.gradient_as_bucket_view = True
        self.model_index, self.num_local_models = int(model_index), int(num_local_models)
        self.total_num_models = int(total_num_models)
        self.sync_buffer_barrier = sync_buffer_barrier
        self._hook = self._hook_state = None
        self._has_rebuilt_buckets = True            # buckets never move after construction
        if reducer is None:
            dev = next(module.parameters()).device
            reducer = VSWReducer(dev, num_local_models, total_num_models, bucket_cap_mb,
                                 process_group=process_group)
        self.reducer = reducer
        reducer.attach(self)

    @property
    def bucket_indices(self):
        return self.reducer.layout.bucket_indices

    def forward(self, *inputs, **kwargs):
        return self.module(*inputs, **kwargs)

    def register_comm_hook(self, state, hook) -> None:
        self._hook_state, self._hook = state, hook

    def reconfigure(self, num_local_models, total_num_models, sync_buffer_barrier=None) -> None:
        """T changed (jabas/train/trainer.py:526-528); a change of K rebuilds the reducer."""
        if int(num_local_models) != self.reducer.K:
            raise ValueError("resize the shared VSWReducer first (VSWReducer.resize), then reconfigure")
        self.num_local_models, self.total_num_models = int(num_local_models), int(total_num_models)
        self.sync_buffer_barrier = sync_buffer_barrier
        self.reducer.T = int(total_num_models)
        self.reducer.engine.set_total_workers(total_num_models)
