"""Bucket scheduling of the gradient exchange (`flodl_b200/parallel/grad_sync.py`) without a process group: the
reduction itself is replaced by a recorder, the readiness logic is driven by hand."""
import pytest
import torch

from flodl_b200.parallel.flat import FlatParams
from flodl_b200.parallel.grad_sync import GradSync


def make(n_params=6, numel=1000, bucket_params=2):
    params = [torch.zeros(numel, requires_grad=True) for _ in range(n_params)]
    flat = FlatParams(params, shadow=False)
    gs = GradSync(flat, None, bucket_bytes=numel * 4 * bucket_params, overlap=True, backend="nccl", world=2)
    calls = []
    gs._reduce_range = lambda start, end, blocks=None: calls.append((start, end))
    return params, flat, gs, calls


def step(gs, params, order):
    gs.begin_step()
    for i in order:
        gs._on_touch(params[i])
    return gs.finish()


def test_buckets_cover_the_buffer_back_to_front():
    """Bucket 0 holds the LAST parameters of the buffer (their gradients are produced first in backward), the last
    bucket the first ones."""
    params, flat, gs, calls = make()
    assert len(gs.buckets) == 3
    assert [b["start"] for b in gs.buckets] == sorted((b["start"] for b in gs.buckets), reverse=True)
    assert gs.buckets[-1]["start"] == 0 and gs.buckets[0]["end"] == flat.total
    assert [sorted(b["members"]) for b in gs.buckets] == [[4, 5], [2, 3], [0, 1]]


def test_first_step_learns_counts_and_reduces_everything_at_finish():
    params, flat, gs, calls = make()
    step(gs, params, [5, 4, 3, 2, 1, 0])
    assert gs.expected == [1] * 6
    assert calls == [(b["start"], b["end"]) for b in gs.buckets]          # nothing overlapped yet, all in index order


def test_later_steps_launch_in_index_order_whatever_the_arrival_order():
    params, flat, gs, calls = make()
    step(gs, params, [5, 4, 3, 2, 1, 0])
    calls.clear()
    gs.begin_step()
    # bucket 1 (parameters 2, 3) is complete first: it must wait for bucket 0 (parameters 4, 5)
    for i in (3, 2):
        gs._on_touch(params[i])
    assert calls == []
    for i in (5, 4):
        gs._on_touch(params[i])
    assert calls == [(gs.buckets[0]["start"], gs.buckets[0]["end"]), (gs.buckets[1]["start"], gs.buckets[1]["end"])]
    for i in (1, 0):
        gs._on_touch(params[i])
    assert len(calls) == 2                                                 # the last index is always left to finish()
    gs.finish()
    assert calls == [(b["start"], b["end"]) for b in gs.buckets]
    # a rank on which the gradients arrived in another order issues the same sequence
    params2, flat2, gs2, calls2 = make()
    step(gs2, params2, [0, 1, 2, 3, 4, 5])
    calls2.clear()
    step(gs2, params2, [2, 0, 5, 1, 3, 4])
    assert calls2 == calls


def test_a_parameter_touched_twice_per_step_waits_for_its_last_contribution():
    params, flat, gs, calls = make()
    step(gs, params, [5, 5, 4, 3, 2, 1, 0])                                 # tied weight: two contributions
    assert gs.expected[5] == 2
    calls.clear()
    gs.begin_step()
    gs._on_touch(params[5]); gs._on_touch(params[4])
    assert calls == []                                                      # bucket 0 still misses one contribution
    gs._on_touch(params[5])
    assert len(calls) == 1


def test_gradient_after_its_bucket_was_reduced_is_reported_and_overlap_goes_off():
    params, flat, gs, calls = make()
    step(gs, params, [5, 4, 3, 2, 1, 0])
    gs.begin_step()
    for i in (5, 4):
        gs._on_touch(params[i])                                             # bucket 0 reduced
    gs._on_touch(params[5])                                                 # ... and then another gradient for it (a branch taken this step only)
    for i in (3, 2, 1, 0):
        gs._on_touch(params[i])
    with pytest.raises(RuntimeError, match="after its bucket had been reduced"):
        gs.finish()
    assert gs.overlap is False
    # with overlap off every bucket is reduced at finish(), whatever the touch pattern
    calls.clear()
    step(gs, params, [0, 0, 0, 5])
    assert calls == [(b["start"], b["end"]) for b in gs.buckets]


def test_unused_parameter_on_the_learning_step_is_detected_when_it_is_used_later():
    params, flat, gs, calls = make()
    step(gs, params, [5, 3, 2, 1, 0])                                       # parameter 4 unused on step 1 (an untaken switch branch)
    assert gs.expected[4] == 0
    calls.clear()
    gs.begin_step()
    gs._on_touch(params[5])                                                 # bucket 0 looks complete and goes out
    assert len(calls) == 1
    gs._on_touch(params[4])                                                 # the other branch this time
    for i in (3, 2, 1, 0):
        gs._on_touch(params[i])
    with pytest.raises(RuntimeError):
        gs.finish()


def test_world_of_one_is_inert():
    params = [torch.zeros(10, requires_grad=True)]
    gs = GradSync(FlatParams(params, shadow=False), None, world=1)
    gs.begin_step()
    gs._on_touch(params[0])
    assert gs.finish() is None and gs.launch_count == 0


def test_bucket_report_is_empty_without_timed_launches():
    params, flat, gs, calls = make()
    gs.enable_timing()
    step(gs, params, [5, 4, 3, 2, 1, 0])            # CPU: exchanges run in line, nothing is timed
    assert gs.bucket_report() == []
