"""Text renderings of a graph: Graphviz DOT (+ SVG through the external `dot` binary when it is
installed), profile heat-maps, self-contained HTML trend plots, CSV export, training log, tree and
parameter summaries (flodl/src/graph/dot.rs, plot.rs, verbose.rs). Nothing here needs a graphics
stack: DOT and HTML are text; SVG conversion shells out to `dot` and raises if it is absent."""
from __future__ import annotations

import html
import json
import shutil
import subprocess
from typing import Dict, List, Optional, Sequence

from ..tensor import TensorError


def format_duration(seconds: float) -> str:
    if seconds < 1e-3:
        return f"{seconds * 1e6:.0f}µs"
    if seconds < 1.0:
        return f"{seconds * 1e3:.1f}ms"
    if seconds < 60.0:
        return f"{seconds:.1f}s"
    m, s = divmod(int(seconds), 60)
    if m < 60:
        return f"{m}m {s:02d}s"
    h, m = divmod(m, 60)
    return f"{h}h {m:02d}m"


def _heat(frac: float) -> str:
    frac = min(max(frac, 0.0), 1.0)
    r, g = int(255 * frac), int(200 * (1 - frac))
    return f"#{r:02x}{g:02x}40"


class RenderMixin:
    # ---- DOT / SVG ------------------------------------------------------------------------------
    def dot(self) -> str:
        return self._dot(None)

    def dot_with_profile(self) -> str:
        return self._dot(self.last_profile)

    def _dot(self, profile) -> str:
        tags_by_node: Dict[int, List[str]] = {}
        for t, (ni, _) in self.tag_names.items():
            tags_by_node.setdefault(ni, []).append(t)
        dur = {n.id: n.duration for n in profile.nodes} if profile else {}
        peak = max(dur.values(), default=0.0)
        out = ["digraph G {", "  rankdir=TB;", '  node [shape=box, style="rounded,filled", fillcolor="#f0f0f0", fontname="Helvetica"];']
        if self._label:
            out.append(f'  label="{self._label}"; labelloc=t;')
        for ni, node in enumerate(self.nodes):
            label = node.id
            if ni in tags_by_node:
                label += "\\n#" + ",#".join(sorted(tags_by_node[ni]))
            mod = node.module
            if mod is not None:
                n_params = sum(p.numel() for p in mod.parameters())
                if n_params:
                    label += f"\\n{n_params:,} params"
            attrs = [f'label="{label}"']
            if node.id in dur and peak > 0:
                attrs.append(f'fillcolor="{_heat(dur[node.id] / peak)}"')
                attrs[0] = f'label="{label}\\n{format_duration(dur[node.id])}"'
            elif mod is None:
                attrs.append('shape=ellipse, fillcolor="#e8f0ff"')
            out.append(f'  "{node.id}" [{", ".join(attrs)}];')
        for e in self.edges:
            lbl = f' [label="{e.to_port}"]' if e.to_port.startswith("ref_") else ""
            out.append(f'  "{e.from_node}" -> "{e.to_node}"{lbl};')
        for s in self.state:
            reader = next((n.id for n in self.nodes if n.is_state_read and n.id.startswith(f"state_read_{s['name']}_")), None)
            if reader:
                out.append(f'  "{self.nodes[s["writer_ni"]].id}" -> "{reader}" [style=dashed, color="#888888", label="t-1"];')
        out.append("}")
        return "\n".join(out)

    def svg(self) -> bytes:
        return _dot_to_svg(self.dot())

    def svg_with_profile(self) -> bytes:
        return _dot_to_svg(self.dot_with_profile())

    # ---- summaries ------------------------------------------------------------------------------
    def tree_summary(self, indent: int = 0) -> str:
        pad = "  " * indent
        n_params = sum(p.numel() for p in self.parameters())
        lines = [f"{pad}{self._label or 'graph'} [{self.short_hash()}] {len(self.nodes)} nodes, {n_params:,} params"]
        for label, g in sorted(self._child_graphs()):
            lines.append(g.tree_summary(indent + 1))
        return "\n".join(lines)

    def param_summary(self) -> str:
        rows = [(n, p.shape(), p.numel(), p.is_frozen()) for n, p in self.named_parameters()]
        width = max((len(r[0]) for r in rows), default=10)
        lines = [f"{'name':<{width}}  {'shape':<20} {'numel':>12}  frozen"]
        for n, s, k, f in rows:
            lines.append(f"{n:<{width}}  {str(s):<20} {k:>12,}  {'yes' if f else ''}")
        lines.append(f"total: {sum(r[2] for r in rows):,}")
        return "\n".join(lines)

    # ---- trends ---------------------------------------------------------------------------------
    def plot_html(self, path: str, tags: Sequence[str] = ()) -> None:
        """Self-contained HTML (inline SVG polylines, no external assets) of the epoch histories."""
        keys = list(tags) if tags else list(self.metric_order)
        _write_plot(path, {k: self.epoch_history.get(k, []) for k in keys}, self._label or "training")

    def plot_timings_html(self, path: str, tags: Sequence[str] = ()) -> None:
        keys = list(tags) if tags else list(self.timing_history.keys())
        _write_plot(path, {k: self.timing_history.get(k, []) for k in keys}, "node timings (s)")

    def export_trends(self, path: str, tags: Sequence[str] = ()) -> None:
        keys = list(tags) if tags else list(self.metric_order)
        _write_csv(path, {k: self.epoch_history.get(k, []) for k in keys})

    def export_timing_trends(self, path: str, tags: Sequence[str] = ()) -> None:
        keys = list(tags) if tags else list(self.timing_history.keys())
        _write_csv(path, {k: self.timing_history.get(k, []) for k in keys})

    def write_log(self, path: str, total_epochs: int = 0) -> None:
        keys = list(self.metric_order)
        n = max((len(self.epoch_history.get(k, [])) for k in keys), default=0)
        with open(path, "w") as f:
            for e in range(n):
                parts = [f"epoch {e + 1}" + (f"/{total_epochs}" if total_epochs else "")]
                for k in keys:
                    h = self.epoch_history.get(k, [])
                    if e < len(h):
                        parts.append(f"{k}={h[e]:.6g}")
                if e < len(self.flush_times):
                    parts.append(f"t={format_duration(self.flush_times[e])}")
                f.write("  ".join(parts) + "\n")


def _dot_to_svg(dot_text: str) -> bytes:
    exe = shutil.which("dot")
    if exe is None:
        raise TensorError("svg(): the Graphviz `dot` binary is not installed; use dot() for the DOT text")
    res = subprocess.run([exe, "-Tsvg"], input=dot_text.encode(), capture_output=True)
    if res.returncode != 0:
        raise TensorError(f"dot failed: {res.stderr.decode()[:200]}")
    return res.stdout


def _write_csv(path: str, series: Dict[str, List[float]]) -> None:
    keys = list(series)
    n = max((len(v) for v in series.values()), default=0)
    with open(path, "w") as f:
        f.write("epoch," + ",".join(keys) + "\n")
        for e in range(n):
            f.write(str(e + 1) + "," + ",".join(f"{series[k][e]:.8g}" if e < len(series[k]) else "" for k in keys) + "\n")


_COLORS = ["#1f77b4", "#ff7f0e", "#2ca02c", "#d62728", "#9467bd", "#8c564b", "#e377c2", "#7f7f7f"]


def _write_plot(path: str, series: Dict[str, List[float]], title: str) -> None:
    w, h, pad = 860, 360, 40
    body = []
    for i, (k, vals) in enumerate(series.items()):
        if not vals:
            continue
        lo, hi = min(vals), max(vals)
        span = (hi - lo) or 1.0
        n = max(len(vals) - 1, 1)
        pts = " ".join(f"{pad + (w - 2 * pad) * j / n:.1f},{h - pad - (h - 2 * pad) * (v - lo) / span:.1f}" for j, v in enumerate(vals))
        c = _COLORS[i % len(_COLORS)]
        body.append(f'<h3 style="color:{c}">{html.escape(k)} <small>last={vals[-1]:.6g} min={lo:.6g} max={hi:.6g}</small></h3>'
                    f'<svg width="{w}" height="{h}" style="background:#fafafa;border:1px solid #ddd">'
                    f'<polyline fill="none" stroke="{c}" stroke-width="2" points="{pts}"/></svg>')
    doc = (f"<!doctype html><html><head><meta charset='utf-8'><title>{html.escape(title)}</title></head>"
           f"<body style='font-family:sans-serif'><h1>{html.escape(title)}</h1>{''.join(body)}"
           f"<script type='application/json' id='data'>{json.dumps(series)}</script></body></html>")
    with open(path, "w") as f:
        f.write(doc)
