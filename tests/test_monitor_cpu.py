"""Monitor, timeline, dashboard server, CpuWorker, Rng wrapper: host-only tests with a fake NVML."""
import json
import socket
import time

import pytest

from flodl_b200.monitor import (Monitor, ResourceSampler, Timeline, format_bytes, format_eta, format_metric)
from flodl_b200.rng import Rng
from flodl_b200.worker import CpuWorker


class FakeNvml:
    NVML_CLOCK_SM = 1

    def __init__(self, utils):
        self.utils = utils
        self.calls = 0

    def nvmlDeviceGetHandleByIndex(self, i): return i

    def nvmlDeviceGetUtilizationRates(self, h):
        self.calls += 1
        u = self.utils[min(len(self.utils) - 1, self.calls - 1)]
        return type("U", (), {"gpu": u})()

    def nvmlDeviceGetMemoryInfo(self, h): return type("M", (), {"used": 2 << 30, "total": 180 << 30})()
    def nvmlDeviceGetClockInfo(self, h, which): return 1965
    def nvmlDeviceGetPowerUsage(self, h): return 450_000
    def nvmlDeviceGetName(self, h): return b"NVIDIA B200"


def test_format_helpers():
    assert format_eta(0.042) == "42ms" and format_eta(1.0) == "1s" and format_eta(1.5) == "1.5s"
    assert format_eta(90.0) == "1m 30s" and format_eta(3661.0) == "1h 01m" and format_eta(-1) == "—"
    assert format_bytes(512) == "512 B" and format_bytes(1024 * 500) == "500 KB"
    assert format_bytes(1024 * 1024 * 100) == "100 MB" and format_bytes(2_254_857_830) == "2.1 GB"
    assert format_metric(0.0) == "0" and format_metric(0.00012) == "1.20e-04" and format_metric(1.23456) == "1.2346"
    assert format_metric(1234.5678) == "1234.57"


def test_resource_sampler_with_fake_nvml():
    s = ResourceSampler(nvml=FakeNvml([37]), devices=[0]).sample()
    assert s.ram_total_bytes and s.gpus[0].util_percent == 37.0 and s.gpus[0].name == "NVIDIA B200"
    assert s.gpus[0].sm_clock_mhz == 1965 and s.gpus[0].power_w == 450.0 and s.gpu_util_percent == 37.0
    assert "GPU0 37%" in s.summary()


def test_monitor_logs_lines_and_exports(tmp_path, capsys):
    m = Monitor(3, sampler=ResourceSampler(nvml=FakeNvml([50]), devices=[0]))
    line = m.log(0, 1.5, [("loss", 0.5), ("acc", 0.25)])
    assert "epoch 1/3" in line and "loss=0.5000" in line and "[1.5s" in line and "ETA" in line
    m.log(1, 1.0, {"loss": 0.4, "acc": 0.5})
    last = m.log(2, 1.0, {"loss": 0.3, "acc": 0.75})
    assert "ETA" not in last
    html, csvp, logp = (str(tmp_path / n) for n in ("d.html", "m.csv", "m.log"))
    m.set_metadata({"note": "test"})
    m.set_identity("model", "ab" * 32)
    m.save_html(html)
    m.finish()
    m.export_csv(csvp)
    m.write_log(logp)
    page = open(html).read()
    assert "<canvas" in page and '"loss": 0.3' in page and "abababab" in page
    rows = open(csvp).read().strip().splitlines()
    assert rows[0].startswith("epoch,duration_secs,loss,acc") and len(rows) == 4
    assert len(open(logp).read().strip().splitlines()) == 3 and len(m.history()) == 3


def test_dashboard_server_serves_page_and_backfills_events():
    m = Monitor(2, sampler=ResourceSampler(nvml=None, devices=[]))
    port = m.serve(0)
    m.log(0, 0.1, {"loss": 1.0})
    with socket.create_connection(("127.0.0.1", port), timeout=5) as c:
        c.sendall(b"GET / HTTP/1.1\r\nHost: x\r\n\r\n")
        data = b""
        while b"</html>" not in data:
            chunk = c.recv(65536)
            if not chunk:
                break
            data += chunk
    assert b"200 OK" in data and b"EventSource" in data
    with socket.create_connection(("127.0.0.1", port), timeout=5) as c:      # joins late: must still see epoch 0
        c.sendall(b"GET /events HTTP/1.1\r\nHost: x\r\n\r\n")
        c.settimeout(5)
        data = b""
        while data.count(b"event: epoch") < 1:
            data += c.recv(65536)
        m.log(1, 0.1, {"loss": 0.5})
        while data.count(b"event: epoch") < 2:
            data += c.recv(65536)
    assert b"text/event-stream" in data and b"event: init" in data and b'"loss": 0.5' in data
    m.server.shutdown()


def test_timeline_events_summary_idle_gaps_and_exports(tmp_path):
    nv = FakeNvml([90, 90, 2, 1, 0, 3, 95, 95])
    tl = Timeline(1, sampler=ResourceSampler(nvml=nv, devices=[0]))
    sub = tl.subscribe()
    for _ in range(8):
        tl.sample_once()
        time.sleep(0.02)
    tl.event("SyncStart")
    tl.event("SyncEnd", duration_ms=2.5)
    tl.event("AnchorChanged", **{"from": 10, "to": 12})
    tl.event("Throttle", rank=1)
    tl.event("Custom", label="checkpoint")
    assert tl.sample_count() == 8
    gaps = tl.idle_gaps(0, 5.0, 20)
    assert len(gaps) == 1 and gaps[0][1] > gaps[0][0]
    s = tl.summary()
    assert s.sync_count == 1 and s.sync_total_ms == 2.5 and s.anchor_changes == 1 and s.throttle_count == 1
    assert 0 < s.gpu_mean_util[0] < 95 and "1 syncs" in str(s)
    tl.stop()                                  # final broadcast
    msg = sub.get(timeout=2)
    assert len(msg["samples"]) == 8 and msg["events"][1]["kind"] == "SyncEnd"
    j, c, h = (str(tmp_path / n) for n in ("t.json", "t.csv", "t.html"))
    tl.save_json(j)
    tl.save_csv(c)
    tl.save_html(h)
    assert len(json.load(open(j))["events"]) == 5
    assert "SyncEnd" in open(c).read() and "<canvas" in open(h).read()
    samples, events = tl.drain()
    assert len(samples) == 8 and len(events) == 5 and tl.sample_count() == 0


def test_timeline_background_thread():
    tl = Timeline(5, sampler=ResourceSampler(nvml=None, devices=[]))
    tl.start()
    time.sleep(0.1)
    tl.stop()
    assert tl.sample_count() >= 3 and tl.elapsed_ms() >= 100


def test_cpu_worker_runs_jobs_in_order_and_survives_failures():
    out = []
    w = CpuWorker()
    for i in range(5):
        w.submit(lambda i=i: out.append(i))
    w.submit(lambda: 1 / 0)
    w.submit(lambda: out.append(99))
    w.finish()
    assert out == [0, 1, 2, 3, 4, 99] and len(w.errors()) == 1
    with pytest.raises(RuntimeError):
        w.submit(lambda: None)
    w.finish()


def test_rng_wrapper():
    a, b = Rng.seed(5), Rng.seed(5)
    xs = list(range(20))
    ys = list(range(20))
    a.shuffle(xs)
    b.shuffle(ys)
    assert xs == ys and sorted(xs) == list(range(20)) and xs != list(range(20))
    assert 3 <= a.range(3, 9) < 9 and 0.0 <= a.f32() < 1.0 and a.choice([7]) == 7
