"""Flat layout: DDP bucket assignment, 128-byte bucket alignment, segment table."""
import pytest
import torch
import torch.distributed as dist
from hypothesis import given, settings, strategies as st

from jabas_b200.layout import ALIGN_ELEMS, assign_buckets, build_layout, model_zoo_shapes


def test_bucket_assignment_equals_the_stock_reducer():
    torch.manual_seed(0)
    sizes = [1000, 2048 * 1000, 64, 64, 512 * 512 * 9, 7, 3 * 1024 * 1024, 5, 128, 9_000_000, 11]
    params = [torch.empty(n) for n in sizes]
    stock, _ = dist._compute_bucket_assignment_by_size(list(reversed(params)), [1024 * 1024, 25 * 1024 * 1024])
    want = [[len(sizes) - 1 - i for i in b] for b in stock]
    assert assign_buckets(sizes) == want


def test_model_layouts_match_the_recorded_bucket_sizes():
    n, s, g = model_zoo_shapes("resnet50")
    lay = build_layout(n, s, g)
    # examples/resnet50/quickstart/bucket_profile_data/resnet50_bucket_size_profile.json:1
    # records 7.81 / 30.04 / 25.04 / 25.25 / 9.2 MiB for the reference's own model
    assert lay.num_params == 25557032 and lay.bucket_sizes_mib() == [7.82, 30.04, 25.04, 25.32, 9.27]
    n, s, g = model_zoo_shapes("vit_b_16")
    lay = build_layout(n, s, g)
    assert lay.num_params == 86567656 and lay.num_buckets == 14
    n, s, g = model_zoo_shapes("gnmt8")
    lay = build_layout(n, s, g)
    assert lay.num_params == 243967233 and len(n) == 76 and lay.num_buckets == 19
    assert max(lay.bucket_sizes_mib()) == pytest.approx(125.12, abs=0.01)


@settings(max_examples=60, deadline=None)
@given(st.lists(st.tuples(st.integers(0, 5000), st.integers(0, 3)), min_size=1, max_size=40),
       st.sampled_from([0.001, 0.01, 0.05]))
def test_layout_invariants(params, cap_mb):
    numels = [p[0] for p in params]
    groups = [p[1] for p in params]
    lay = build_layout([f"p{i}" for i in range(len(params))], [(n,) for n in numels], groups,
                       bucket_cap_mb=cap_mb, first_bucket_bytes=512)
    assert lay.num_params == sum(numels) and lay.total % ALIGN_ELEMS == 0 and lay.total >= ALIGN_ELEMS
    # every parameter sits inside its bucket, buckets start on 128-byte boundaries and do not overlap
    covered = 0
    for b, (begin, end) in enumerate(lay.buckets):
        assert begin % ALIGN_ELEMS == 0 and begin >= covered and end <= lay.total
        covered = end
        pos = begin
        for i in lay.bucket_indices[b]:
            s = lay.slots[i]
            assert s.bucket == b and s.offset == pos and s.numel == numels[i]
            pos += s.numel
        assert pos == end
    assert sorted(i for b in lay.bucket_indices for i in b) == list(range(len(params)))
    # the segment table covers [0, total) without gaps and names the right group for every element
    pos = 0
    for begin, end, g in lay.segments:
        assert begin == pos and end > begin
        pos = end
    assert pos == lay.total
    for s in lay.slots:
        if s.numel:
            seg = next(x for x in lay.segments if x[0] <= s.offset < x[1])
            assert seg[2] == s.group and seg[1] >= s.offset + s.numel or \
                all(next(x for x in lay.segments if x[0] <= e < x[1])[2] == s.group
                    for e in (s.offset, s.offset + s.numel - 1))
    # regrouping rebuilds only the segments
    lay.set_groups([0] * len(params))
    assert lay.segments == [(0, lay.total, 0)]


def test_engine_refuses_bulk_staging_with_the_peer_exchange():
    """Kernels that read another GPU's memory never take the update kernels' bulk-staged form: the
    combination is refused when the engine is constructed, before any device work."""
    import pytest
    from jabas_b200.gradient_path import GradientPath
    from jabas_b200.layout import build_layout
    layout = build_layout(["w"], [(64,)], [0])
    with pytest.raises(ValueError, match="bulk"):
        GradientPath(layout, 2, "cpu", None, total_num_decoupled_workers=2, collective="peer", staging="bulk",
                     backend=object())
    with pytest.raises(ValueError, match="peer_form"):
        GradientPath(layout, 2, "cpu", None, total_num_decoupled_workers=2, collective="peer", peer_form="ring",
                     backend=object())
