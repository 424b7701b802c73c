"""Turn a directory of run results into the convergence / timing report
(ddp-bench/src/analyze.rs + src/report.rs): per model, every mode's final loss and evaluation metric
next to the solo-0 run, the deltas, total time and speed-up."""
from __future__ import annotations

import glob
import json
import os
from dataclasses import dataclass
from typing import Dict, List, Optional

from .config import ALL_MODES
from .models import all_models


def load_results(directory: str) -> Dict[str, Dict[str, dict]]:
    out: Dict[str, Dict[str, dict]] = {}
    for path in sorted(glob.glob(os.path.join(directory, "*__*.json"))):
        if path.endswith(".timeline.json"):
            continue
        with open(path) as f:
            r = json.loads(f.readline())
        out.setdefault(r["model"], {})[r["mode"]] = r
    return out


def analyze(results: Dict[str, Dict[str, dict]], loss_tolerance: float = 0.15) -> List[dict]:
    """One row per (model, mode): deltas against solo-0 and a verdict. A distributed run "converges" when its
    final loss is within `loss_tolerance` (relative) of the solo run's, or lower."""
    rows = []
    for model, by_mode in results.items():
        base = by_mode.get("solo-0")
        for mode in ALL_MODES:
            r = by_mode.get(mode)
            if r is None:
                continue
            loss = r["epoch_losses"][-1] if r["epoch_losses"] else None
            row = {"model": model, "mode": mode, "world": r["world"], "final_loss": loss, "final_eval": r["final_eval"], "total_ms": r["total_ms"],
                   "error": r.get("error", "")}
            if base is not None and base["epoch_losses"] and loss is not None:
                b = base["epoch_losses"][-1]
                row["loss_delta"] = loss - b
                row["speedup_vs_solo"] = base["total_ms"] / r["total_ms"] if r["total_ms"] > 0 else None
                row["converged"] = (loss <= b * (1.0 + loss_tolerance) + 1e-6) and not row["error"]
                if base["final_eval"] is not None and r["final_eval"] is not None:
                    row["eval_delta"] = r["final_eval"] - base["final_eval"]
            rows.append(row)
    return rows


def render(rows: List[dict]) -> str:
    refs = {m.name: m for m in all_models()}
    lines = ["# DDP validation bench", "", "Synthetic teacher tasks (no dataset downloads); `solo-0` is the convergence reference for each model.", ""]
    for model in dict.fromkeys(r["model"] for r in rows):
        md = refs.get(model)
        lines += [f"## {model}" + (f" - {md.description}" if md else ""), "",
                  "| mode | ranks | final loss | delta vs solo-0 | eval | eval delta | total s | speed-up | verdict |", "|---|---|---|---|---|---|---|---|---|"]
        f = lambda v, spec: "-" if v is None else format(v, spec)
        for r in (x for x in rows if x["model"] == model):
            verdict = "error: " + r["error"] if r["error"] else ("reference" if r["mode"] == "solo-0" else ("ok" if r.get("converged", True) else "DIVERGED"))
            lines.append(f"| {r['mode']} | {r['world']} | {f(r['final_loss'], '.4f')} | {f(r.get('loss_delta'), '+.4f')} | {f(r['final_eval'], '.4f')} | "
                         f"{f(r.get('eval_delta'), '+.4f')} | {r['total_ms'] / 1e3:.2f} | {f(r.get('speedup_vs_solo'), '.2f')} | {verdict} |")
        if md and md.reference:
            pub = f" (published {md.published_eval})" if md.published_eval is not None else ""
            lines += ["", f"Reference task: {md.reference}{pub}; the numbers above are on the synthetic stand-in."]
        lines.append("")
    return "\n".join(lines)


def render_summary(results: Dict[str, Dict[str, dict]], rows: List[dict], timelines=None) -> str:
    """The cross-model sections (ddp-bench/src/report.rs:196-260): best mode per model, loss ratio and speed-up against
    solo-0 as model x mode grids, per-epoch loss trajectories, and what the timelines recorded (synchronisations, El Che
    anchor, GPU utilisation, idle stretches by cause)."""
    timelines = timelines or {}
    models = list(results)
    modes = [m for m in ALL_MODES if any(m in results[x] for x in models)]
    by = {(r["model"], r["mode"]): r for r in rows}
    lines = ["## Best mode per model", "", "| model | best loss | mode | fastest (loss within tolerance of solo-0) | mode |", "|---|---|---|---|---|"]
    for model in models:
        ok = [r for r in rows if r["model"] == model and r["final_loss"] is not None and not r["error"]]
        if not ok:
            lines.append(f"| {model} | - | - | - | - |")
            continue
        best = min(ok, key=lambda r: r["final_loss"])
        fast_pool = [r for r in ok if r.get("converged", True)]
        fast = min(fast_pool, key=lambda r: r["total_ms"]) if fast_pool else None
        lines.append(f"| {model} | {best['final_loss']:.4f} | {best['mode']} | " + (f"{fast['total_ms'] / 1e3:.2f} s | {fast['mode']} |" if fast else "- | - |"))

    def grid(title: str, note: str, cell) -> List[str]:
        out = ["", f"## {title}", "", note, "", "| model | " + " | ".join(modes) + " |", "|---|" + "---|" * len(modes)]
        for model in models:
            out.append(f"| {model} | " + " | ".join(cell(by.get((model, m))) for m in modes) + " |")
        return out

    def ratio(r):
        if r is None or r["final_loss"] is None:
            return "-"
        base = by.get((r["model"], "solo-0"))
        if base is None or not base["final_loss"]:
            return "-"
        return f"{r['final_loss'] / base['final_loss']:.2f}"
    lines += grid("Convergence quality (loss ratio vs solo-0)", "1.00 = the solo run's final loss; below 1 is better.", ratio)
    lines += grid("Speed-up vs solo-0", "Wall time of the solo run divided by the run's.",
                  lambda r: "-" if r is None or r.get("speedup_vs_solo") is None else f"{r['speedup_vs_solo']:.2f}x")
    lines += ["", "## Per-epoch loss trajectory", ""]
    for model in models:
        n = max((len(r["epoch_losses"]) for r in results[model].values()), default=0)
        if n == 0:
            continue
        step = max(1, n // 10)                                  # at most about ten columns
        cols = list(range(0, n, step))
        lines += [f"### {model}" + (f" (every {step}th of {n} epochs)" if step > 1 else ""), "", "| mode | " + " | ".join(f"e{c}" for c in cols) + " |",
                  "|---|" + "---|" * len(cols)]
        for m in modes:
            r = results[model].get(m)
            if r is not None:
                lines.append(f"| {m} | " + " | ".join(f"{r['epoch_losses'][c]:.4f}" if c < len(r["epoch_losses"]) else "-" for c in cols) + " |")
        lines.append("")
    if any(a.sample_count or a.sync_count for a in timelines.values()):
        gpus = sorted({g for a in timelines.values() for g in a.gpu_mean_util})
        lines += ["## Timeline", "", "GPUn = mean compute utilisation in %; idle = total time below 5 % utilisation in stretches of at least 500 ms.", "",
                  "| model | mode | syncs | avg sync ms | sync interval p50 / p95 ms | CPU avgs | avg CPU ms | anchors | throttles | "
                  + " | ".join(f"GPU{g}" for g in gpus) + " | idle s |", "|---|---|---|---|---|---|---|---|---|" + "---|" * len(gpus) + "---|"]
        for (model, mode), a in timelines.items():
            anchors = "-" if not a.anchor_changes else f"{a.anchor_changes[0][0]} -> {a.final_anchor} ({len(a.anchor_changes)} changes)"
            lines.append(f"| {model} | {mode} | {a.sync_count} | {a.avg_sync_ms:.2f} | {a.sync_interval_p50_ms:.0f} / {a.sync_interval_p95_ms:.0f} | {a.cpu_avg_count} | "
                         f"{a.avg_cpu_avg_ms:.2f} | {anchors} | {a.throttle_count} | "
                         + " | ".join(f"{a.gpu_mean_util[g]:.0f}" if g in a.gpu_mean_util else "-" for g in gpus) + f" | {a.idle_ms() / 1e3:.1f} |")
        gaps = [(k, g) for k, a in timelines.items() for g in a.idle_gaps]
        if gaps:
            lines += ["", "## GPU idle analysis", "", "Idle stretches of at least 500 ms, classified by the nearest event.", "",
                      "| model | mode | GPU | start s | duration s | cause |", "|---|---|---|---|---|---|"]
            lines += [f"| {k[0]} | {k[1]} | {g.gpu} | {g.start_ms / 1e3:.1f} | {g.duration_ms / 1e3:.1f} | {g.cause} |" for k, g in gaps]
            lines += ["", "### Idle time by cause", "", "| model | mode | GPU | epoch boundary s | sync s | CPU avg s | unexplained s |", "|---|---|---|---|---|---|---|"]
            for k, a in timelines.items():
                for g in sorted({x.gpu for x in a.idle_gaps}):
                    c = a.idle_by_cause(g)
                    lines.append(f"| {k[0]} | {k[1]} | {g} | {c['epoch boundary'] / 1e3:.1f} | {c['sync'] / 1e3:.1f} | {c['cpu avg'] / 1e3:.1f} | {c['unexplained'] / 1e3:.1f} |")
    missing = [f"{m} / {mode}" for m in models for mode in modes if mode not in results[m]]
    if missing:
        lines += ["", "## Runs not present", ""] + [f"- {x}" for x in missing]
    return "\n".join(lines) + "\n"


def write_report(directory: str, out_path: Optional[str] = None) -> str:
    from .analyze import analyze_dir
    results = load_results(directory)
    rows = analyze(results)
    text = render(rows) + "\n" + render_summary(results, rows, analyze_dir(directory))
    if out_path:
        with open(out_path, "w") as f:
            f.write(text)
    return text


# ---- loss baselines (ddp-bench/src/report.rs:17-150) -----------------------------------------------------------------
@dataclass
class Baseline:
    model: str
    mode: str
    loss: float
    epochs: int = 0
    batches: int = 0
    batch_size: int = 0


def load_baselines(path: str) -> List[Baseline]:
    try:
        data = json.load(open(path))
    except OSError as e:
        raise ValueError(f"cannot read {path}: {e}")
    except ValueError as e:
        raise ValueError(f"invalid JSON in {path}: {e}")
    if not isinstance(data, list):
        raise ValueError(f"{path}: expected a JSON array")
    out = []
    for item in data:
        for key in ("model", "mode", "loss"):
            if key not in item:
                raise ValueError(f"{path}: entry without `{key}`")
        out.append(Baseline(str(item["model"]), str(item["mode"]), float(item["loss"]), int(item.get("epochs", 0)), int(item.get("batches", 0)),
                            int(item.get("batch_size", 0))))
    return out


def save_baselines(path: str, baselines: List[Baseline]) -> None:
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    rows = [f'  {{"model":"{b.model}","mode":"{b.mode}","loss":{b.loss:.6f},"epochs":{b.epochs},"batches":{b.batches},"batch_size":{b.batch_size}}}'
            for b in baselines]
    with open(path, "w") as f:
        f.write("[\n" + ",\n".join(rows) + "\n]\n")


def results_to_baselines(results) -> List[Baseline]:
    """One baseline per finished run: its last epoch's loss with the run's shape."""
    return [Baseline(r.model, r.mode, float(r.epoch_losses[-1]), r.epochs, r.batches_per_epoch, r.batch_size)
            for r in results if r.epoch_losses and not r.error]


def validate_results(results, baselines: List[Baseline], tolerance: float = 0.15):
    """(passed, failed, lines): every run's final loss against the baseline of its model (relative difference, absolute
    when the baseline is ~0); runs without a baseline are reported as skipped."""
    lookup = {b.model: b for b in baselines}
    ok = bad = 0
    lines = []
    for r in results:
        loss = float(r.epoch_losses[-1]) if r.epoch_losses else float("nan")
        b = lookup.get(r.model)
        if b is None:
            lines.append(f"  SKIP  {r.model:<16} {r.mode:<20} loss={loss:.6f} (no baseline)")
            continue
        diff = abs(loss - b.loss) / abs(b.loss) if abs(b.loss) > 1e-10 else abs(loss - b.loss)
        good = diff <= tolerance and not r.error                  # NaN compares false: a diverged run fails
        ok, bad = ok + good, bad + (not good)
        lines.append(f"  {'PASS' if good else 'FAIL'}  {r.model:<16} {r.mode:<20} loss={loss:.6f} (baseline={b.loss:.6f}, diff={diff * 100:.1f}%)")
    return ok, bad, lines
