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


def write_report(directory: str, out_path: Optional[str] = None) -> str:
    text = render(analyze(load_results(directory)))
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
