"""Flat HBM layout of a model's parameters, gradients and optimizer state.

The reference relies on ``gradient_as_bucket_view=True`` (jabas/train/trainer.py:82-86):
every VSW's ``.grad`` tensors are views into flat per-bucket fp32 buffers, and buckets
are assigned DDP-style, in reverse parameter order with a 1 MiB first bucket and a
``bucket_cap_mb`` cap (the bucket sizes recorded at
examples/resnet50/quickstart/bucket_profile_data/resnet50_bucket_size_profile.json:1).

Here the same assignment is laid out as ONE flat buffer per tensor kind (weights per
replica, gradients per VSW, momentum / Adam moments once), bucket after bucket, each
bucket starting on a 128-byte boundary.  A bucket is then a contiguous element range
``[begin, end)`` of every buffer, the whole model is one contiguous range too, and the
kernels address optimizer param groups through a segment table over that range.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

ALIGN_ELEMS = 32                      # 128 bytes of fp32
DEFAULT_FIRST_BUCKET_BYTES = 1024 * 1024
DEFAULT_BUCKET_CAP_MB = 25


@dataclass
class ParamSlot:
    index: int                        # position in model.parameters() order
    name: str
    shape: Tuple[int, ...]
    numel: int
    group: int                        # optimizer param group
    bucket: int
    offset: int                       # first element in the flat buffers


@dataclass
class FlatLayout:
    slots: List[ParamSlot]            # in parameters() order
    buckets: List[Tuple[int, int]]    # [begin, end) element range per bucket, padding excluded
    bucket_indices: List[List[int]]   # parameter indices per bucket (the DDP `bucket_indices`)
    segments: List[Tuple[int, int, int]]   # (begin, end, group) covering [0, total)
    total: int                        # padded length of every flat buffer
    num_params: int = field(default=0)     # unpadded element count

    @property
    def num_buckets(self) -> int:
        return len(self.buckets)

    def bucket_numel(self, b: int) -> int:
        return self.buckets[b][1] - self.buckets[b][0]

    def set_groups(self, groups: Sequence[int]) -> None:
        """Re-assign the optimizer param group of every parameter (in ``slots`` order) and
        rebuild the segment table; offsets and buckets do not move."""
        for slot, g in zip(self.slots, groups):
            slot.group = int(g)
        runs = sorted((s.offset, s.offset + s.numel, s.group) for s in self.slots if s.numel)
        self.segments = _merge_runs(runs, self.total)

    def bucket_sizes_mib(self) -> List[float]:
        return [round(self.bucket_numel(b) * 4 / 2 ** 20, 2) for b in range(self.num_buckets)]


def assign_buckets(numels: Sequence[int], bucket_cap_mb: float = DEFAULT_BUCKET_CAP_MB,
                   first_bucket_bytes: int = DEFAULT_FIRST_BUCKET_BYTES,
                   elem_size: int = 4) -> List[List[int]]:
    """DDP bucket assignment over parameters taken in REVERSE order: a bucket closes as
    soon as its size reaches the current limit (first ``first_bucket_bytes``, then the
    cap), so a bucket may exceed the cap by its last tensor."""
    limits = [first_bucket_bytes, int(bucket_cap_mb * 1024 * 1024)]
    li, cur, size, out = 0, [], 0, []
    for idx in reversed(range(len(numels))):
        cur.append(idx)
        size += numels[idx] * elem_size
        if size >= limits[li]:
            out.append(cur)
            cur, size = [], 0
            li = min(li + 1, len(limits) - 1)
    if cur:
        out.append(cur)
    return out


def _merge_runs(runs, total: int) -> List[Tuple[int, int, int]]:
    """Merge neighbouring runs of one group; padding joins the run before it."""
    segs: List[List[int]] = []
    for begin, end, g in runs:
        if segs:
            segs[-1][1] = begin
        if segs and segs[-1][2] == g:
            segs[-1][1] = end
        else:
            segs.append([begin if segs else 0, end, g])
    if not segs:
        segs = [[0, total, 0]]
    segs[-1][1] = total
    return [(s[0], s[1], s[2]) for s in segs]


def _align(x: int) -> int:
    return (x + ALIGN_ELEMS - 1) // ALIGN_ELEMS * ALIGN_ELEMS


def build_layout(names: Sequence[str], shapes: Sequence[Sequence[int]], groups: Sequence[int],
                 bucket_cap_mb: float = DEFAULT_BUCKET_CAP_MB,
                 first_bucket_bytes: int = DEFAULT_FIRST_BUCKET_BYTES,
                 bucket_indices: Optional[List[List[int]]] = None) -> FlatLayout:
    numels = []
    for s in shapes:
        n = 1
        for d in s:
            n *= int(d)
        numels.append(n)
    if bucket_indices is None:
        bucket_indices = assign_buckets(numels, bucket_cap_mb, first_bucket_bytes)
    slots: Dict[int, ParamSlot] = {}
    buckets, runs = [], []
    pos = 0
    for b, idxs in enumerate(bucket_indices):
        begin = pos
        for i in idxs:
            slots[i] = ParamSlot(i, names[i], tuple(int(d) for d in shapes[i]), numels[i],
                                 int(groups[i]), b, pos)
            if numels[i]:
                runs.append((pos, pos + numels[i], int(groups[i])))
            pos += numels[i]
        buckets.append((begin, pos))
        pos = _align(pos)
    total = max(pos, ALIGN_ELEMS)
    segments = _merge_runs(runs, total)
    return FlatLayout([slots[i] for i in range(len(names))], buckets, bucket_indices, segments, total,
                      sum(numels))


def layout_from_module(module, param_groups_func: Optional[Callable] = None,
                       bucket_cap_mb: float = DEFAULT_BUCKET_CAP_MB,
                       first_bucket_bytes: int = DEFAULT_FIRST_BUCKET_BYTES) -> FlatLayout:
    """Layout for ``module.parameters()`` (trainable ones).  ``param_groups_func(module)``
    returns the optimizer's list of group dicts, as ``build_param_groups_in_optimizer``
    does at examples/resnet50/main.py:340-349; without it everything is group 0."""
    named = [(n, p) for n, p in module.named_parameters() if p.requires_grad]
    group_of = {}
    if param_groups_func is not None:
        for gi, g in enumerate(param_groups_func(module)):
            for p in g["params"]:
                group_of[id(p)] = gi
    names = [n for n, _ in named]
    shapes = [tuple(p.shape) for _, p in named]
    groups = [group_of.get(id(p), 0) for _, p in named]
    return build_layout(names, shapes, groups, bucket_cap_mb, first_bucket_bytes)


def model_zoo_shapes(model: str):
    """(names, shapes, groups) of the benchmark configurations, built on the meta device
    so that no weights are materialised.  Groups follow the reference recipes: ResNet-50
    puts every parameter whose name contains "bn" in a weight-decay-free group
    (examples/resnet50/main.py:340-349); ViT puts 1-D tensors and biases there
    (examples/vit/main.py:405-423); GNMT uses one group."""
    if model == "gnmt8":
        return _gnmt_shapes(vocab=32000, hidden=1024, layers=8)
    import torch
    with torch.device("meta"):
        if model == "resnet50":
            import torchvision
            net = torchvision.models.resnet50()
            rule = lambda n, p: 0 if "bn" in n else 1
        elif model == "vit_b_16":
            import torchvision
            net = torchvision.models.vit_b_16()
            rule = lambda n, p: 0 if (p.dim() == 1 or n.endswith(".bias")) else 1
        else:
            raise ValueError(f"unknown model {model!r}")
    named = list(net.named_parameters())
    return ([n for n, _ in named], [tuple(p.shape) for _, p in named],
            [rule(n, p) for n, p in named])


def _gnmt_shapes(vocab: int, hidden: int, layers: int):
    """Parameter shapes of a GNMT-v2 seq2seq model in ``named_parameters()`` order, as built
    by examples/gnmt/seq2seq/models/gnmt.py:34 with a shared embedding: a residual LSTM
    encoder (first layer bidirectional, second layer fed with 2*hidden), the shared
    embedding, a decoder whose first LSTM drives a normalised Bahdanau attention, further
    decoder LSTMs fed with [hidden, context], and a biased classifier.  One param group
    (the reference's GNMT optimizer refuses more, shard_optimizer.py:26-29)."""
    names, shapes = [], []

    def lstm(prefix, inp, suffixes=("",)):
        for sfx in suffixes:
            for nm, shp in (("weight_ih_l0", (4 * hidden, inp)), ("weight_hh_l0", (4 * hidden, hidden)),
                            ("bias_ih_l0", (4 * hidden,)), ("bias_hh_l0", (4 * hidden,))):
                names.append(f"{prefix}.{nm}{sfx}")
                shapes.append(shp)

    lstm("encoder.rnn_layers.0", hidden, ("", "_reverse"))
    lstm("encoder.rnn_layers.1", 2 * hidden)
    for i in range(2, layers):
        lstm(f"encoder.rnn_layers.{i}", hidden)
    names.append("encoder.embedder.weight"); shapes.append((vocab, hidden))
    lstm("decoder.att_rnn.rnn", hidden)
    for nm, shp in (("linear_att", (hidden,)), ("normalize_scalar", (1,)), ("normalize_bias", (hidden,)),
                    ("linear_q.weight", (hidden, hidden)), ("linear_k.weight", (hidden, hidden))):
        names.append(f"decoder.att_rnn.attn.{nm}"); shapes.append(shp)
    for i in range(layers - 1):
        lstm(f"decoder.rnn_layers.{i}", 2 * hidden)
    names.append("decoder.classifier.classifier.weight"); shapes.append((vocab, hidden))
    names.append("decoder.classifier.classifier.bias"); shapes.append((vocab,))
    return names, shapes, [0] * len(names)
