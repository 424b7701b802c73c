"""`.fdl` checkpoints: byte layout, round trip, partial load, shape/hash mismatch, gzip, dtype cast,
migration from version 1, optimizer state streams, model snapshots."""
import gzip
import struct

import pytest
import torch

from flodl_b200 import nn
from flodl_b200.graph import FlowBuilder, snapshot_cpu
from flodl_b200.nn import checkpoint as ck


def _mlp(hidden=8, tag_second="b"):
    torch.manual_seed(0)
    return FlowBuilder.from_(nn.Linear(4, hidden)).tag("a").through(nn.GELU()).through(nn.Linear(hidden, 2)).tag(tag_second).build()


def test_header_layout_and_keys(tmp_path):
    g = _mlp()
    path = str(tmp_path / "m.fdl")
    g.save_checkpoint(path)
    raw = open(path, "rb").read()
    assert raw[:4] == b"FDLC"
    assert struct.unpack("<I", raw[4:8])[0] == 2
    assert raw[8:40].hex() == g.structural_hash()
    assert struct.unpack("<I", raw[40:44])[0] == 4
    name_len = struct.unpack("<I", raw[44:48])[0]
    assert raw[48:48 + name_len] == b"a/weight"
    assert nn.checkpoint_keys(path) == ["a/weight", "a/bias", "b/weight", "b/bias"]
    assert nn.checkpoint_version(path) == 2


def test_roundtrip_restores_values_and_keeps_requires_grad(tmp_path):
    g1, g2 = _mlp(), _mlp()
    with torch.no_grad():
        for p in g1.parameters():
            p.t.add_(1.0)
    path = str(tmp_path / "m.fdl")
    g1.save_checkpoint(path)
    rep = g2.load_checkpoint(path)
    assert sorted(rep.loaded) == sorted(["a/weight", "a/bias", "b/weight", "b/bias"]) and not rep.missing and not rep.skipped
    for p1, p2 in zip(g1.parameters(), g2.parameters()):
        assert torch.equal(p1.t, p2.t) and p2.t.requires_grad


def test_gzip_roundtrip(tmp_path):
    g1, g2 = _mlp(), _mlp()
    with torch.no_grad():
        g1.parameters()[0].t.fill_(3.0)
    path = str(tmp_path / "m.fdl.gz")
    g1.save_checkpoint(path)
    assert open(path, "rb").read()[:2] == b"\x1f\x8b"
    g2.load_checkpoint(path)
    assert float(g2.parameters()[0].t.detach().mean()) == 3.0


def test_hash_mismatch_is_an_error(tmp_path):
    g1, g2 = _mlp(8), _mlp(16)
    path = str(tmp_path / "m.fdl")
    g1.save_checkpoint(path)
    with pytest.raises(Exception) as e:
        g2.load_checkpoint(path)
    assert "hash" in str(e.value).lower() or "architecture" in str(e.value).lower()


def test_partial_load_reports_missing_and_skipped():
    g1 = _mlp()
    g2 = _mlp(tag_second="other")
    blob = nn.save_checkpoint(g1.named_parameters(), g1.named_buffers(), None)
    rep = nn.load_checkpoint(blob, g2.named_parameters(), g2.named_buffers(), None)
    assert sorted(rep.loaded) == ["a/bias", "a/weight"]
    assert sorted(rep.missing) == ["other/bias", "other/weight"]
    assert sorted(rep.skipped) == ["b/bias", "b/weight"]


def test_shape_mismatch_is_an_error():
    g1, g2 = _mlp(8), _mlp(16)
    blob = nn.save_checkpoint(g1.named_parameters(), g1.named_buffers(), None)
    with pytest.raises(Exception) as e:
        nn.load_checkpoint(blob, g2.named_parameters(), g2.named_buffers(), None)
    assert "shape" in str(e.value).lower()


def test_dtype_is_cast_to_the_models():
    g1, g2 = _mlp(), _mlp()
    nn.cast_parameters(g1.parameters(), torch.bfloat16)
    blob = nn.save_checkpoint(g1.named_parameters(), g1.named_buffers(), None)
    nn.load_checkpoint(blob, g2.named_parameters(), g2.named_buffers(), None)
    assert g2.parameters()[0].t.dtype == torch.float32
    torch.testing.assert_close(g2.parameters()[0].t, g1.parameters()[0].t.float())


def test_buffers_travel_with_the_checkpoint(tmp_path):
    def net():
        return FlowBuilder.from_(nn.Conv2d(3, 4, 3)).through(nn.BatchNorm2d(4)).tag("bn").build()
    g1, g2 = net(), net()
    g1.set_training(True)
    g1.forward(torch.randn(4, 3, 8, 8))
    path = str(tmp_path / "bn.fdl")
    g1.save_checkpoint(path)
    g2.load_checkpoint(path)
    b1 = dict(g1.named_buffers())
    b2 = dict(g2.named_buffers())
    assert "bn/running_mean" in b1
    for k in b1:
        assert torch.equal(b1[k].get(), b2[k].get())


def test_migrate_v1_checkpoint():
    g = _mlp()
    blob = nn.save_checkpoint(g.named_parameters(), g.named_buffers(), None)
    # a version-1 file differs by its version word and by positional (legacy) names
    legacy = bytearray(blob)
    legacy[4:8] = struct.pack("<I", 1)
    out, rep = nn.migrate_checkpoint(bytes(legacy), g.named_parameters(), g.named_buffers())
    assert out[:4] == b"FDLC" and struct.unpack("<I", out[4:8])[0] == 2
    assert rep is not None


def test_sidecar_config_path_and_source_config(tmp_path):
    from flodl_b200.graph import sidecar_config_path
    g = _mlp()
    g.set_source_config('{"model_type": "tiny"}')
    path = str(tmp_path / "m.fdl")
    g.save_checkpoint(path)
    side = sidecar_config_path(path)
    assert side.endswith("m.config.json")
    assert open(side).read() == '{"model_type": "tiny"}'


def test_snapshot_cpu_writes_zero_hash(tmp_path):
    g = _mlp()
    snap = snapshot_cpu(g)
    path = str(tmp_path / "snap.fdl")
    snap.save_file(path)
    raw = open(path, "rb").read()
    assert raw[8:40] == bytes(32)
    g2 = _mlp(16)
    # zero hash => no architecture check, but shapes still have to match
    with pytest.raises(Exception):
        g2.load_checkpoint(path)
    g3 = _mlp()
    assert len(g3.load_checkpoint(path).loaded) == 4


def test_optimizer_state_file_roundtrip(tmp_path):
    p = nn.Parameter(torch.ones(4), "p")
    opt = nn.SGD([p], 0.1, 0.9)
    for _ in range(2):
        p.t.grad = torch.ones(4)
        opt.step()
    path = str(tmp_path / "opt.bin.gz")
    opt.save_state_file(path)
    q = nn.Parameter(p.t.detach().clone(), "p")
    opt2 = nn.SGD([q], 0.1, 0.9)
    opt2.load_state_file(path)
    p.t.grad, q.t.grad = torch.ones(4), torch.ones(4)
    opt.step()
    opt2.step()
    torch.testing.assert_close(p.t.detach(), q.t.detach())


def test_corrupt_headers_are_rejected_before_anything_is_allocated():
    """A damaged or hostile file must fail on its header: negative or overflowing dimensions, a byte
    count that does not match the shape, or a record longer than the data that follows."""
    import struct

    from flodl_b200 import _ext
    C = _ext.require()

    def blob(shape, tag, nbytes, payload=b""):
        out = b"FDLC" + struct.pack("<I", 2) + b"\0" * 32 + struct.pack("<I", 1)
        name = b"w"
        out += struct.pack("<I", len(name)) + name + struct.pack("<I", len(shape)) + b"".join(struct.pack("<q", d) for d in shape)
        return out + struct.pack("<BQ", tag, nbytes) + payload

    ok = blob([2, 2], 3, 16, b"\0" * 16)
    assert C.fdl_load_bytes(ok, False)[2][0][1].shape == (2, 2)
    for bad in (blob([-1, 4], 3, 16, b"\0" * 16),                      # negative dimension
                blob([1 << 40, 1 << 40], 3, 16, b"\0" * 16),           # product overflows
                blob([2, 2], 3, 12, b"\0" * 12),                       # byte count != shape
                blob([1 << 20, 1 << 10], 3, 4 << 30, b"\0" * 16)):     # 4 GiB promised, 16 bytes present
        with pytest.raises(RuntimeError):
            C.fdl_load_bytes(bad, False)
    # key listings skip the payloads instead of reading them
    assert [k for k, _ in C.fdl_load_bytes(ok, True)[2]] == ["w"]


def test_reader_survives_random_damage():
    """Property test of the native reader: a valid file with bytes flipped, cut short, or with a stretch overwritten by
    random data either loads (same number of records, sane shapes) or is refused with an ordinary error. It never takes
    the process down and never allocates more than the file could hold."""
    hypothesis = pytest.importorskip("hypothesis")
    from hypothesis import given, settings, strategies as st

    from flodl_b200 import _ext
    C = _ext.require()

    def record(name, shape, tag, payload):
        out = struct.pack("<I", len(name)) + name + struct.pack("<I", len(shape)) + b"".join(struct.pack("<q", d) for d in shape)
        return out + struct.pack("<BQ", tag, len(payload)) + payload
    good = (b"FDLC" + struct.pack("<I", 2) + b"\0" * 32 + struct.pack("<I", 3) + record(b"a.weight", [3, 4], 3, bytes(range(48)))
            + record(b"a.bias", [4], 3, bytes(16)) + record(b"steps", [], 3, bytes(4)))
    assert len(C.fdl_load_bytes(good, False)[2]) == 3

    damage = st.one_of(
        st.tuples(st.just("flip"), st.integers(0, len(good) - 1), st.integers(1, 255)),
        st.tuples(st.just("cut"), st.integers(0, len(good) - 1), st.just(0)),
        st.tuples(st.just("noise"), st.integers(0, len(good) - 1), st.binary(min_size=1, max_size=24)))

    @settings(max_examples=400, deadline=None, derandomize=True, database=None)
    @given(st.lists(damage, min_size=1, max_size=3))
    def run(edits):
        data = bytearray(good)
        for kind, at, arg in edits:
            at = min(at, max(len(data) - 1, 0))
            if not data:
                break
            if kind == "flip":
                data[at] ^= arg
            elif kind == "cut":
                del data[at:]
            else:
                data[at:at + len(arg)] = arg
        for keys_only in (False, True):
            try:
                recs = C.fdl_load_bytes(bytes(data), keys_only)[2]
            except (RuntimeError, ValueError, UnicodeDecodeError, OverflowError):
                continue
            for _, t in recs:
                assert t is None or t.numel() * t.element_size() <= len(data)
    run()
