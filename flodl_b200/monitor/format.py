"""Human-readable durations, byte counts and metric values (flodl/src/monitor/format.rs)."""
from __future__ import annotations


def format_eta(secs: float) -> str:
    if secs < 0.0:
        return "—"
    if secs < 1.0:
        return f"{int(secs * 1000)}ms"
    if secs < 60.0:
        whole = int(secs)
        frac = int((secs - whole) * 10)
        return f"{whole}.{frac}s" if frac > 0 else f"{whole}s"
    total = int(secs)
    h, m, s = total // 3600, (total % 3600) // 60, total % 60
    return f"{h}h {m:02d}m" if h > 0 else f"{m}m {s:02d}s"


def format_bytes(n: int) -> str:
    b = float(n)
    if b >= 1024 ** 3:
        return f"{b / 1024 ** 3:.1f} GB"
    if b >= 1024 ** 2:
        return f"{b / 1024 ** 2:.0f} MB"
    if b >= 1024:
        return f"{b / 1024:.0f} KB"
    return f"{int(n)} B"


def format_metric(v: float) -> str:
    a = abs(v)
    if a == 0.0:
        return "0"
    if a < 0.001:
        return f"{v:.2e}"
    if a < 100.0:
        return f"{v:.4f}"
    return f"{v:.2f}"
