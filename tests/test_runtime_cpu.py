"""The C++ runtime: RNG, SHA-256, El Che, prefetch worker; datasets, samplers, loaders."""
import gzip
import hashlib
import struct

import pytest
import torch

from flodl_b200 import _ext
from flodl_b200.data import (Batch, DataLoader, DataSet, PrefetchWorker, RandomSampler, SequentialSampler, TensorDataSet,
                             prefetch_depth_from_vram)
from flodl_b200.data.datasets import Cifar10, Mnist, Shakespeare
from flodl_b200.parallel.el_che import ElChe

C = _ext.require()


# ---- Rng / sha ---------------------------------------------------------------------------------------
def test_rng_reproducible_and_ranges():
    a, b, c = C.Rng(7), C.Rng(7), C.Rng(8)
    xs = [a.usize(100) for _ in range(50)]
    assert xs == [b.usize(100) for _ in range(50)] and xs != [c.usize(100) for _ in range(50)]
    assert all(0 <= x < 100 for x in xs)
    fs = [a.f64() for _ in range(1000)]
    assert 0.0 <= min(fs) and max(fs) < 1.0 and 0.4 < sum(fs) / 1000 < 0.6
    ns = [a.normal(1.0, 2.0) for _ in range(4000)]
    m = sum(ns) / len(ns)
    assert abs(m - 1.0) < 0.15
    p = a.permutation(20)
    assert sorted(p) == list(range(20))
    assert sum(a.bernoulli(0.25) for _ in range(4000)) / 4000 == pytest.approx(0.25, abs=0.04)


def test_sha256_matches_hashlib():
    for msg in (b"", b"abc", bytes(range(256)) * 5):
        assert C.sha256_hex(msg) == hashlib.sha256(msg).hexdigest()


# ---- El Che -----------------------------------------------------------------------------------------
def test_el_che_starts_equal_and_follows_speed():
    e = ElChe(2, 10)
    assert e.batch_counts() == [10, 10] and not e.is_calibrated() and e.anchor_wall_ms() == 0.0
    e.report_timing([100.0, 50.0], [10, 10], 1.0)       # rank 1 is twice as fast
    assert e.is_calibrated()
    c = e.batch_counts()
    assert c[0] == e.anchor() and c[1] >= int(1.8 * c[0])
    assert e.anchor_wall_ms() == pytest.approx(e.anchor() * max(e.ms_per_batch()), rel=1e-6)


def test_el_che_anchor_grows_with_overhead_and_respects_max():
    e = ElChe(2, 10).with_overhead_target(0.10).with_max_anchor(40)
    e.report_timing([100.0, 100.0], [10, 10], 50.0)     # sync costs 50 % of compute
    assert e.anchor() > 10
    for _ in range(10):
        e.report_timing([100.0, 100.0], [e.batches(0), e.batches(1)], 500.0)
    assert e.anchor() <= 40


def test_el_che_speed_hint_and_nudge_and_clamp():
    e = ElChe(2, 10).with_speed_ratio(0, 2.0)
    assert e.has_speed_hint() and e.batch_counts()[1] == 2 * e.batch_counts()[0]
    before = e.anchor()
    e.nudge_anchor_down(0.5)
    assert e.anchor() <= before
    cl = e.clamp_total(9)
    assert sum(cl) <= 9 and all(x >= 1 for x in cl)
    assert ElChe(2, 10).with_max_batch_diff(3).max_batch_diff() == 3


# ---- datasets / samplers ------------------------------------------------------------------------------
class Pairs(DataSet):
    def __init__(self, n):
        self.n = n

    def __len__(self):
        return self.n

    def get(self, i):
        return [torch.full((3,), float(i)), torch.tensor(i)]


def test_dataset_adapter_stacks_position_wise():
    dl = DataLoader.from_dataset(Pairs(10)).batch_size(4).shuffle(False).build()
    batches = list(dl.epoch(0))
    assert len(batches) == 2 and list(batches[0][0].shape) == [4, 3] and batches[0][1].tolist() == [0, 1, 2, 3]


def test_batch_indexing():
    b = Batch([torch.zeros(2), torch.ones(2)], ["x", "y"])
    assert torch.equal(b["y"], b[1]) and b.has("x") and not b.has("z") and b.names() == ["x", "y"]
    assert b.get_named("z") is None and len(b) == 2
    with pytest.raises(KeyError):
        b["z"]
    assert Batch([torch.zeros(1)]).names() == ["0"]


def test_samplers():
    r = RandomSampler(50, 3)
    e0, e1 = r.indices(0), r.indices(1)
    assert sorted(e0) == list(range(50)) and e0 != e1 and e0 == RandomSampler(50, 3).indices(0)
    assert RandomSampler(50, 4).indices(0) != e0
    assert SequentialSampler(5).indices(3) == [0, 1, 2, 3, 4]


def test_loader_resident_vs_streaming_see_the_same_samples():
    x = torch.arange(64).float().view(64, 1)
    ds = TensorDataSet(x, torch.arange(64))
    res = DataLoader.from_batch_dataset(ds).batch_size(8).seed(1).build()
    stm = DataLoader.from_batch_dataset(ds).batch_size(8).seed(1).streaming().build()
    assert res.is_resident() and not stm.is_resident()
    a = [b[1].tolist() for b in res.epoch(2)]
    c = [b[1].tolist() for b in stm.epoch(2)]
    assert a == c and len(a) == 8
    assert res.num_batches() == 8 and res.batch_size == 8


def test_loader_drop_last_and_distributed_shards():
    ds = TensorDataSet(torch.arange(50))
    dl = DataLoader.from_batch_dataset(ds).batch_size(8).shuffle(False).drop_last(False).build()
    assert dl.num_batches() == 7 and sum(len(b[0]) for b in dl.epoch(0)) == 50
    seen = []
    for rank in range(2):
        d = DataLoader.from_batch_dataset(ds).batch_size(5).seed(9).build().distributed(rank, 2)
        assert d.is_distributed()
        seen += [i for b in d.epoch(0) for i in b[0].tolist()]
    assert sorted(seen) == list(range(50))


def test_loader_rejects_bad_config():
    ds = TensorDataSet(torch.arange(4))
    with pytest.raises(Exception):
        DataLoader.from_batch_dataset(ds).build()
    with pytest.raises(Exception):
        DataLoader.from_batch_dataset(ds).batch_size(2).names(["a", "b"]).build()


def test_prefetch_worker_python_path_for_generic_datasets():
    class Gen(TensorDataSet.__mro__[1]):
        def __len__(self):
            return 12

        def get_batch(self, idx):
            return [torch.tensor(list(idx))]
    w = PrefetchWorker(Gen(), "cpu", 2)
    assert not w.is_native()
    w.start_epoch(list(range(12)), 4)
    got = []
    while True:
        b = w.next()
        if b is None:
            break
        got += b[0].tolist()
    assert got == list(range(12))


def test_native_prefetch_ring_survives_many_epochs_early_stops_and_a_slow_consumer():
    """The C++ ring (producer thread + bounded queue + two condition variables) under the patterns that would show a
    lost wake-up, a stale batch from a previous epoch, or a join that never returns."""
    import threading, time
    from flodl_b200 import _ext
    if not _ext.available():
        pytest.skip("native extension not built")
    n = 257
    x = torch.arange(n * 3, dtype=torch.float32).view(n, 3)
    y = torch.arange(n)
    for depth in (1, 2, 7):
        w = PrefetchWorker(TensorDataSet(x, y), "cpu", depth)
        assert w.is_native()
        g = torch.Generator().manual_seed(depth)
        for epoch in range(30):
            order = torch.randperm(n, generator=g).tolist()
            drop_last = epoch % 2 == 0
            w.start_epoch(order, 16, drop_last)
            take = None if epoch % 3 else 1 + epoch % 5            # every third epoch is abandoned after a few batches
            seen = []
            while take is None or len(seen) < take * 16:
                if epoch % 7 == 0:
                    time.sleep(0.001)                              # a consumer slower than the producer: the ring fills up
                b = w.next()
                if b is None:
                    break
                assert torch.equal(b[0], x[b[1]])                  # rows of one batch belong together
                seen += b[1].tolist()
            want = order[:n // 16 * 16] if drop_last else order
            assert seen == (want if take is None else want[:take * 16]), (depth, epoch)
            if take is not None:
                w.stop()                                           # producer blocked on a full ring must wake up and leave
        assert w.next() is None                                    # after the last epoch: empty, not blocked
        done = threading.Event()
        w.start_epoch(list(range(n)), 4)
        threading.Thread(target=lambda: (w.stop(), done.set()), daemon=True).start()     # stop from another thread, nothing consumed
        assert done.wait(10), "stop() did not return with a full ring"


def test_prefetch_depth_on_cpu_is_double_buffering():
    assert prefetch_depth_from_vram(1024, 32, "cpu") == 2


# ---- file parsers -------------------------------------------------------------------------------------
def test_mnist_parser():
    n, r, c = 3, 4, 5
    img = struct.pack(">IIII", 2051, n, r, c) + bytes(range(n * r * c))
    lab = struct.pack(">II", 2049, n) + bytes([7, 0, 9])
    m = Mnist.parse(gzip.compress(img), gzip.compress(lab))
    assert list(m.images.shape) == [3, 1, 4, 5] and m.labels.tolist() == [7, 0, 9]
    assert float(m.images[0, 0, 0, 1]) == pytest.approx(1 / 255)
    with pytest.raises(Exception):
        Mnist.parse(struct.pack(">IIII", 1, n, r, c) + bytes(60), lab)
    with pytest.raises(Exception):
        Mnist.parse(img, struct.pack(">II", 2049, 2) + bytes(2))


def test_cifar_parser():
    rec = bytearray(10000 * 3073)
    rec[0] = 3
    rec[1] = 255
    c = Cifar10.parse([bytes(rec)])
    assert list(c.images.shape) == [10000, 3, 32, 32] and int(c.labels[0]) == 3 and float(c.images[0, 0, 0, 0]) == 1.0
    with pytest.raises(Exception):
        Cifar10.parse([bytes(10)])
    rec[0] = 11
    with pytest.raises(Exception):
        Cifar10.parse([bytes(rec)])


def test_shakespeare_parser():
    s = Shakespeare.parse("abcabcabcabc!", 4)
    assert s.vocab_size == 4 and len(s) == 3
    assert s.decode(s.data[0].tolist()) == "abca" and s.decode(s.targets[0].tolist()) == "bcab"
    with pytest.raises(Exception):
        Shakespeare.parse("ab", 4)


def test_eager_dispatch_threshold_is_process_wide_and_cpu_never_native():
    import threading
    import torch
    from flodl_b200.ops import core
    old = core.eager_min_numel()
    try:
        core.set_eager_min_numel(123)
        seen = []
        t = threading.Thread(target=lambda: seen.append(core.eager_min_numel()))
        t.start(); t.join()
        assert seen == [123]                       # autograd's backward thread must see the same value
        assert not core._native_ok(torch.zeros(4))  # CPU tensors never take the native path
    finally:
        core.set_eager_min_numel(old)
