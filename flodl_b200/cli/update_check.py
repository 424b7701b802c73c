"""A once-a-day look for a newer release, shown as a one-line nudge after the user's command
(flodl-cli/src/update_check.rs). It never delays a command beyond a two-second timeout and every failure is silent.

This package has no release feed of its own: the check is **inert unless a feed is configured** with
`FLODL_B200_UPDATE_URL` (a URL that answers with JSON `{"latest": "X.Y.Z"}` or `{"versions": ["X.Y.Z", ...]}`), so by
default nothing is fetched. The switches are the reference's:

| off when | |
|---|---|
| `FDL_NO_UPDATE_CHECK=1` | this run (wins over everything) |
| `CI=true` | in CI |
| `/.dockerenv` exists | in a container (ephemeral cache, redundant probes) |
| `update_check.enabled = false` in `<config-dir>/flodl/config.json` | persistently |

`<config-dir>` is `$XDG_CONFIG_HOME` or `~/.config`. The file also keeps `last_check` (epoch seconds), `latest_known`
and `first_run_seen` (the first run prints a one-time note that says how to switch the check off)."""
from __future__ import annotations

import json
import os
import re
import time
from typing import Callable, List, Optional, Tuple

DAY_S = 24 * 3600
TIMEOUT_S = 2.0


def config_path() -> str:
    base = os.environ.get("XDG_CONFIG_HOME") or os.path.join(os.path.expanduser("~"), ".config")
    return os.path.join(base, "flodl", "config.json")


def load_config(path: Optional[str] = None) -> dict:
    try:
        data = json.load(open(path or config_path()))
        return data if isinstance(data, dict) else {}
    except (OSError, ValueError):
        return {}


def save_config(cfg: dict, path: Optional[str] = None) -> None:
    p = path or config_path()
    try:
        os.makedirs(os.path.dirname(p), exist_ok=True)
        with open(p, "w") as f:
            json.dump(cfg, f, indent=2)
    except OSError:
        pass                                     # a read-only home must not break the command


def parse_version(v: str) -> Optional[Tuple[int, ...]]:
    """(major, minor, patch) of a stable version; None for pre-releases (`1.2.0-rc1`, `1.2.0b1`) and garbage."""
    m = re.fullmatch(r"v?(\d+)\.(\d+)(?:\.(\d+))?", v.strip())
    return None if m is None else tuple(int(x or 0) for x in m.groups())


def max_stable(versions: List[str]) -> Optional[str]:
    stable = [(parse_version(v), v) for v in versions]
    stable = [(t, v) for t, v in stable if t is not None]
    return max(stable)[1].lstrip("v") if stable else None


def disabled_reason(cfg: dict, env=os.environ, dockerenv: str = "/.dockerenv") -> Optional[str]:
    if env.get("FDL_NO_UPDATE_CHECK", "") not in ("", "0", "false"):
        return "FDL_NO_UPDATE_CHECK"
    if env.get("CI", "").lower() in ("1", "true", "yes"):
        return "CI"
    if os.path.exists(dockerenv):
        return "container"
    if cfg.get("update_check", {}).get("enabled", True) is False:
        return "config"
    if not env.get("FLODL_B200_UPDATE_URL"):
        return "no feed configured"
    return None


def fetch_latest(url: str, timeout_s: float = TIMEOUT_S) -> Optional[str]:
    import urllib.request
    try:
        with urllib.request.urlopen(urllib.request.Request(url, headers={"User-Agent": "flodl_b200"}), timeout=timeout_s) as r:
            data = json.loads(r.read(1 << 20))
    except Exception:  # noqa: BLE001  (offline, slow, not JSON: today's check simply did not happen)
        return None
    if isinstance(data, dict):
        if isinstance(data.get("versions"), list):
            return max_stable([str(v) for v in data["versions"]])
        if data.get("latest") is not None:
            return max_stable([str(data["latest"])])
    return None


def check(current: str, now: Optional[float] = None, path: Optional[str] = None, fetch: Callable[[str], Optional[str]] = fetch_latest,
          env=os.environ, dockerenv: str = "/.dockerenv") -> List[str]:
    """Lines to print after the command (possibly none). Probes at most once a day; between probes the remembered
    answer is used."""
    cfg = load_config(path)
    if disabled_reason(cfg, env, dockerenv) is not None:
        return []
    uc = cfg.setdefault("update_check", {})
    now = time.time() if now is None else now
    lines = []
    if not uc.get("first_run_seen"):
        uc["first_run_seen"] = True
        lines.append("note: fdl looks for a newer release once a day (FDL_NO_UPDATE_CHECK=1, or update_check.enabled=false in "
                     f"{path or config_path()}, switches that off)")
    if now - float(uc.get("last_check", 0)) >= DAY_S:
        latest = fetch(env["FLODL_B200_UPDATE_URL"])
        uc["last_check"] = int(now)
        if latest is not None:
            uc.setdefault("latest_known", {})["flodl_b200"] = latest
    save_config(cfg, path)
    latest = uc.get("latest_known", {}).get("flodl_b200")
    cur, new = parse_version(current), parse_version(latest) if latest else None
    if cur is not None and new is not None and new > cur:
        lines.append(f"flodl_b200 {latest} is available (this is {current}): update the checkout, then `python -m flodl_b200.cli install --check`")
    return lines
