"""The flodl_b200-vs-PyTorch benchmark suite in its seconds-long smoke mode: every model builds in both
implementations with identical parameter counts, trains without error and reports the harness fields."""
import json

import pytest

from benchmarks import run as bench_run
from benchmarks.harness import BenchConfig, run_benchmark
from benchmarks.models import MODELS, TIER1, TIER2


def test_harness_protocol_counts_epochs_and_discards_first_pass():
    calls = []
    cfg = BenchConfig("x", runs=3, warmup_epochs=2, measured_epochs=4, batches_per_epoch=1, batch_size=1)
    r = run_benchmark(cfg, "flodl", 7, lambda i, warm: calls.append((i, warm)) or 0.5, "cpu")
    assert len(calls) == 3 * (2 + 4) and sum(1 for _, w in calls if w) == 3 * 2
    assert len(r.run_medians_ms) == 2 and r.param_count == 7 and r.final_loss == 0.5 and r.peak_vram_mb is None
    assert json.loads(r.json())["name"] == "x"


def test_registry_has_the_eleven_models():
    assert len(TIER1) == 6 and len(TIER2) == 5 and set(TIER1 + TIER2) == set(MODELS)


@pytest.mark.parametrize("name", ["mlp", "gru_seq", "transformer", "feedback_loop", "gated_routing", "iterative_refine"])
def test_model_runs_in_both_implementations(name):
    a = bench_run.run_model(name, "flodl", "cpu", quick=True)
    b = bench_run.run_model(name, "torch", "cpu", quick=True)
    assert a.param_count == b.param_count > 0
    assert a.median_epoch_ms > 0 and b.median_epoch_ms > 0
    assert a.final_loss == a.final_loss and b.final_loss == b.final_loss      # not NaN


def test_cli_writes_report(tmp_path, capsys):
    out = tmp_path / "r.md"
    assert bench_run.main(["--quick", "--device", "cpu", "--models", "mlp", "--out", str(out)]) == 0
    text = out.read_text()
    assert "| mlp |" in text and "speed-up" in text
    assert bench_run.main(["--models", "nope"]) == 2


# ---- optional clock lock: logic only, against a stand-in for NVML (never the real one) ---------------------------------
class FakeNvml:
    def __init__(self, n=2, base=(1500, None), refuse=()):
        self.n, self.base, self.refuse, self.calls = n, base, set(refuse), []
    def device_count(self): return self.n
    def default_graphics_clock(self, i): return self.base[i]
    def lock(self, i, mhz):
        if i in self.refuse:
            raise PermissionError("insufficient permissions")
        self.calls.append(("lock", i, mhz))
    def reset(self, i): self.calls.append(("reset", i))


def test_clock_lock_locks_resets_and_reports_refusals():
    from benchmarks.clocks import ClockLock, detect_base_clock
    nv, lines = FakeNvml(), []
    assert detect_base_clock(nv, 0) == 1500 and detect_base_clock(nv, 1) is None
    with ClockLock(nv, None, None, lines.append) as lock:
        assert lock.locked == [0] and lock.failed == [1]                  # device 1 reports no base clock: left alone
        assert nv.calls == [("lock", 0, 1500)]
    assert nv.calls[-1] == ("reset", 0) and lock.locked == []
    nv = FakeNvml(base=(1500, 1400), refuse=[1])
    with pytest.raises(RuntimeError):
        with ClockLock(nv, 1800, [0, 1], lines.append) as lock:
            assert lock.locked == [0] and lock.failed == [1] and ("lock", 0, 1800) in nv.calls
            raise RuntimeError("benchmark failed")
    assert ("reset", 0) in nv.calls and ("reset", 1) not in nv.calls      # reset also after an exception; only what was locked
    assert any("could not lock" in ln for ln in lines)


def test_lock_is_off_unless_asked_for_and_warmup_is_a_no_op_without_a_gpu(monkeypatch):
    import benchmarks.clocks as clocks
    from benchmarks import run as bench_run
    made = []
    monkeypatch.setattr(clocks, "NvmlBackend", lambda: made.append(1) or FakeNvml())
    assert bench_run.main(["--models", "mlp", "--impl", "torch", "--device", "cpu", "--quick", "--runs", "1", "--epochs", "1", "--warmup", "0"]) == 0
    assert made == []                                                      # no NVML object without --lock-clocks
    assert clocks.gpu_warmup(5.0, "cpu") == 0 and clocks.gpu_warmup(0.0, "cuda") == 0
