"""`fdl setup`, `fdl libtorch`, `fdl install`, `fdl add`, `fdl skill` (flodl-cli/src/main.rs:111-181).

In the reference these commands exist to get a matching libtorch onto the machine (download or
build it, point `LIBTORCH_PATH` at it), to install the CLI itself, to add the framework to an
existing project and to install the AI-assistant skill. Here libtorch arrives inside the installed
`torch` wheel, so the same verbs answer the questions that remain:

* `setup`     checks interpreter, torch, CUDA toolchain and GPUs against what the native library
              needs (sm_100a, nvcc >= 12.8, torch with CUDA), builds the library, and prints what is
              missing otherwise. `--non-interactive` never prompts (nothing here prompts), `--force`
              rebuilds even if the library is current.
* `libtorch`  `info` prints which libtorch the process would load (version, CUDA, cuDNN, NCCL, arch
              list, library directory); `list` shows every torch installation on `sys.path`;
              `path` prints the directory a C++ build should link against.
* `install`   builds the native library in-tree and verifies it loads (`--check`: verify only;
              `--dev`: also build the bounds-checked debug library).
* `add`       adds a training scaffold (`train.py`, `fdl.yml`) to an existing directory without
              touching files that are already there; `--playground` adds a small script that
              exercises the graph builder.
* `skill`     `install [dir]` writes the assistant guide (a condensed API and porting reference) into
              `<dir>/.fdl/skills/flodl_b200/SKILL.md`; `show` prints it.
"""
from __future__ import annotations

import json
import os
import sys
from dataclasses import dataclass
from typing import List

from .args import FdlArgs, arg


@dataclass
class SetupArgs(FdlArgs):
    """Check the machine and build the native library."""
    non_interactive: bool = arg(False, help="never prompt (accepted for compatibility: nothing prompts)")
    force: bool = arg(False, help="rebuild the native library even if it is up to date")


@dataclass
class InstallArgs(FdlArgs):
    """Build and verify the native library."""
    check: bool = arg(False, help="only verify that the library is built and loads")
    dev: bool = arg(False, help="also build the bounds-checked debug library")


@dataclass
class AddArgs(FdlArgs):
    """Add a training scaffold to an existing directory."""
    target: str = arg(".", positional=True, help="directory to add the files to, or `flodl-hf` (alias `hf`) for the Hugging Face playground")
    playground: bool = arg(False, help="also add playground.py (graph-builder tour)")
    install: bool = arg(False, help="build the native library afterwards")


def _requirements() -> List[dict]:
    """One row per requirement: name, ok, found, needed."""
    import shutil
    import subprocess
    rows = []
    rows.append({"name": "python", "ok": sys.version_info >= (3, 10), "found": sys.version.split()[0], "needed": ">= 3.10"})
    try:
        import torch
        rows.append({"name": "torch", "ok": True, "found": torch.__version__, "needed": "any 2.x with CUDA"})
        rows.append({"name": "torch CUDA build", "ok": torch.version.cuda is not None, "found": str(torch.version.cuda), "needed": ">= 12.8"})
        if torch.cuda.is_available():
            caps = sorted({torch.cuda.get_device_capability(i) for i in range(torch.cuda.device_count())})
            rows.append({"name": "GPU", "ok": any(c[0] == 10 for c in caps), "found": ", ".join(f"sm_{a}{b}" for a, b in caps), "needed": "sm_100 (B200)"})
        else:
            rows.append({"name": "GPU", "ok": None, "found": "none visible", "needed": "sm_100 (B200) to run; not needed to build"})
    except Exception as e:  # noqa: BLE001
        rows.append({"name": "torch", "ok": False, "found": f"import failed: {e}", "needed": "installed"})
    nvcc = shutil.which("nvcc") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    found = "not found"
    ok = False
    try:
        out = subprocess.run([nvcc, "--version"], capture_output=True, text=True, timeout=20).stdout
        line = [l for l in out.splitlines() if "release" in l]
        if line:
            found = line[0].split("release")[-1].strip()
            major, minor = (int(x) for x in found.split(",")[0].split(".")[:2])
            ok = (major, minor) >= (12, 8)
    except Exception:  # noqa: BLE001
        pass
    rows.append({"name": "nvcc", "ok": ok, "found": found, "needed": ">= 12.8 (sm_100a target)"})
    rows.append({"name": "ninja", "ok": shutil.which("ninja") is not None, "found": shutil.which("ninja") or "not found", "needed": "on PATH"})
    rows.append({"name": "g++", "ok": shutil.which("g++") is not None, "found": shutil.which("g++") or "not found", "needed": "C++17"})
    return rows


def setup(argv: List[str]) -> int:
    a = SetupArgs.parse(argv, "fdl setup")
    rows = _requirements()
    for r in rows:
        mark = "ok " if r["ok"] else ("-- " if r["ok"] is None else "NO ")
        print(f"  [{mark}] {r['name']:<18} {r['found']:<34} (needs {r['needed']})")
    blockers = [r["name"] for r in rows if r["ok"] is False]
    if blockers:
        print("setup: cannot build the native library until these are fixed: " + ", ".join(blockers), file=sys.stderr)
        return 1
    from .. import _build
    if a.force or _build.needs_build():
        print("building the native library for sm_100a ...")
        _build.build()
    from .. import _ext
    if not _ext.available():
        print("setup: the library was built but does not load", file=sys.stderr)
        return 1
    print(f"ready: {_build.TARGET}")
    return 0


def libtorch(argv: List[str]) -> int:
    """`libtorch list | info | path | activate | remove | download | build` (see `cli/libtorch.py`)."""
    from . import libtorch as lt
    return lt.main(argv)


def install(argv: List[str]) -> int:
    a = InstallArgs.parse(argv, "fdl install")
    from .. import _build, _ext
    if not a.check:
        _build.build()
        if a.dev:
            import subprocess
            r = subprocess.run([sys.executable, "-c", "from flodl_b200 import _build; print(_build.build())"],
                               env=dict(os.environ, FLODL_B200_BOUNDS_CHECK="1"), capture_output=True, text=True)
            if r.returncode != 0:
                print(r.stderr[-2000:], file=sys.stderr)
                return 1
            print(f"debug library: {r.stdout.strip().splitlines()[-1]}")
    ok = (not _build.needs_build()) and _ext.available()
    print(f"{'ok' if ok else 'NOT READY'}: {_build.TARGET}")
    return 0 if ok else 1


_TRAIN = '''"""Training entry point."""
import torch
from flodl_b200 import nn
from flodl_b200.autograd import Variable
from flodl_b200.graph import FlowBuilder
from flodl_b200.parallel.ddp import Trainer

dev = "cuda" if torch.cuda.is_available() else "cpu"
model = (FlowBuilder.from_(nn.Linear(2, 16, True, dev)).through(nn.GELU()).through(nn.LayerNorm(16, device=dev))
         .also(nn.Linear(16, 16, True, dev)).through(nn.Linear(16, 2, True, dev)).build())
Trainer.setup(model, None, lambda ps: nn.Adam(ps, 1e-2))      # one rank or many: the same three lines below
for step in range(200):
    x = torch.randn(32, 2, device=dev)
    y = torch.stack([x[:, 0].sin(), x[:, 1].cos()], 1)
    loss = nn.mse_loss(model.forward(Variable.wrap(x)), Variable.wrap(y))
    loss.backward()
    model.step()
    if step % 50 == 0:
        print(step, loss.item())
'''

_PLAYGROUND = '''"""A tour of the graph builder: fork / merge / tag / observe."""
import torch
from flodl_b200 import nn
from flodl_b200.autograd import Variable
from flodl_b200.graph import FlowBuilder

g = (FlowBuilder.from_(nn.Linear(8, 16)).tag("stem").through(nn.GELU())
     .also(nn.Linear(16, 16)).tag("residual").through(nn.LayerNorm(16)).through(nn.Linear(16, 4)).build())
print(g.dot())
print(g.forward(Variable.wrap(torch.randn(3, 8))).t.shape)
'''

_MANIFEST = '''description: {name}

commands:
  train:
    description: Train the model
    run: python train.py
  test:
    description: Run the tests
    run: python -m pytest -q
'''


def add(argv: List[str]) -> int:
    a = AddArgs.parse(argv, "fdl add")
    if a.target in ("flodl-hf", "hf"):
        from .scaffold import add_flodl_hf
        try:
            for rel in add_flodl_hf(os.getcwd()):
                print(f"created {rel}")
        except FileExistsError as e:
            print(f"fdl add: {e}", file=sys.stderr)
            return 1
        print("try: python -m flodl_b200.cli flodl-hf classify")
        return 0
    root = os.path.abspath(a.target)
    if not os.path.isdir(root):
        print(f"fdl add: {root} is not a directory", file=sys.stderr)
        return 1
    files = {"train.py": _TRAIN, "fdl.yml": _MANIFEST.format(name=os.path.basename(root) or "project")}
    if a.playground:
        files["playground.py"] = _PLAYGROUND
    for name, text in files.items():
        path = os.path.join(root, name)
        if os.path.exists(path):
            print(f"kept    {path} (already there)")
            continue
        with open(path, "w") as f:
            f.write(text)
        print(f"created {path}")
    return install([]) if a.install else 0


SKILL = '''# flodl_b200: assistant guide

A Blackwell-native (sm_100a) deep-learning framework with floDl's API shape, in Python over PyTorch tensors
with hand-written CUDA kernels for the hot ops and its own NVLink collectives.

## Five things to know
1. `Variable` wraps a `torch.Tensor` (`.t`); modules take and return `Variable`s; method names follow floDl
   (`mul_scalar`, `sum_dim`, `narrow`, ...). `flodl_b200.tensor_ops` holds the rest of the tensor surface.
2. Models are graphs: `FlowBuilder.from_(m).through(m2).also(res).split(...).merge(...).tag("name").build()`.
   Loops: `.loop_body(b).for_n(3)`; routing: `.switch(router, branches)`, `.gate(router, experts)`.
3. Training: `Trainer.setup(model, None, lambda ps: nn.Adam(ps, lr))`, then `loss.backward(); model.step()`.
   The same code runs on 1 or N GPUs (`torchrun --nproc-per-node N`); gradients are exchanged by this
   library's NVLink kernels, overlapped with backward.
4. Fast path: `TrainEngine(model, opt_factory)` + `capture(step_fn, example_inputs)` + `replay(inputs)`:
   the whole step (forward, backward, all-reduce, optimizer) is one CUDA graph; bf16 autocast with
   `nn.AutocastGuard(torch.bfloat16)` puts GEMMs, attention, LayerNorm, cross-entropy on the tcgen05 kernels.
5. Asynchronous / Local SGD: `Trainer.builder(factory, opt_factory, train_fn).dataset(ds).batch_size(b)
   .num_epochs(e).policy(ApplyPolicy.Cadence).backend(AverageBackend.Nccl).run().join()`.

## Porting from floDl (Rust)
| floDl | here |
|---|---|
| `Tensor::randn(&[2,3], opts)?` | `torch.randn(2, 3, device=...)` |
| `Variable::new(t, true)` | `Variable(t, requires_grad=True)` |
| `x.matmul(&w)?.add(&b)?` | `x.matmul(w).add(b)` |
| `Linear::on_device(i, o, dev)?` | `nn.Linear.on_device(i, o, dev)` |
| `FlowBuilder::from(a).through(b).build()?` | `FlowBuilder.from_(a).through(b).build()` |
| `Adam::new(&params, 1e-3)` | `nn.Adam(params, 1e-3)` |
| `clip_grad_norm(&params, 1.0)?` | `nn.clip_grad_norm(params, 1.0)` |
| `Ddp::setup(&model, builder, opt)?` | `Trainer.setup(model, builder, opt)` |
| `save_checkpoint_file(path, ...)` | `nn.save_checkpoint_file(path, ...)` (same `.fdl` v2 format) |
| `AutoModel::from_pretrained(id)` | `hf.AutoModel.from_pretrained(local_dir)` |
Errors are `TensorError` exceptions instead of `Result`.

## Commands
`python -m flodl_b200.cli diagnose | setup | install | bench | api-ref | export-hf`, `python bench.py --gpus N`.
'''


PORT_SKILL = '''# Port a PyTorch training script to flodl_b200

Use when asked to port, convert or migrate PyTorch code to flodl_b200.

## Steps
1. Read the source: find the model (modules, forward), the loss, the optimizer, the data pipeline, the loop.
2. Run `python -m flodl_b200.cli api-ref --json` and match every PyTorch construct to an entry (constructors, builder
   methods); do not guess names.
3. Write the model with `FlowBuilder`: a chain is `.through(m)`, `x + f(x)` is `.also(f)`, parallel branches are
   `.split([...]).merge(MergeOp.Add)`, reused values are `.tag("n")` / `.using("n")`, repeated blocks are
   `.loop_body(b).for_n(k)`. A forward with Python control flow over tensors becomes a custom `nn.Module`.
4. Keep tensors as `torch.Tensor`; wrap model inputs with `Variable.wrap(t)`, read results with `.t`.
5. Training: `Trainer.setup(model, None, lambda ps: nn.AdamW(ps, lr, wd))`, then `loss.backward(); model.step()`. For the
   fast path on a GPU use `TrainEngine(model, optimizer_factory)` + `capture(step_fn, example)` + `replay(batch)` inside
   `nn.AutocastGuard(torch.bfloat16)`.
6. Data: `DataLoader.from_batch_dataset(TensorDataSet(x, y)).batch_size(b).device(dev).build()`; `loader.epoch(e)`.
7. Validate: run a few steps on CPU, compare the first losses with the PyTorch script under the same seed and
   initial weights (`load_state_dict` values copied into `model.named_parameters()`), then run on the GPU.

## Mapping
| PyTorch | flodl_b200 |
|---|---|
| `nn.Sequential(a, b)` | `FlowBuilder.from_(a).through(b).build()` |
| `x + self.block(x)` | `.also(block)` |
| `torch.cat([f(x), g(x)], -1)` | custom module, or `.split([f, g])` + a merge module |
| `nn.Linear(i, o)` / `nn.Conv2d(i, o, k, s, p)` | `nn.Linear(i, o)` / `nn.Conv2d.configure(i, o, k).with_stride(s).with_padding(p).done()` |
| `F.cross_entropy(logits, y)` | `nn.cross_entropy_loss(logits_var, y_var)` (2-D logits, ignore_index -100) |
| `optim.AdamW(ps, lr, weight_decay=wd)` | `nn.AdamW(ps, lr, wd)` |
| `clip_grad_norm_(ps, 1.0)` | `nn.clip_grad_norm(ps, 1.0)` |
| `torch.autocast("cuda", torch.bfloat16)` | `nn.AutocastGuard(torch.bfloat16)` |
| `DistributedDataParallel(m)` | `Trainer.setup(model, None, optimizer_factory)` under `torchrun` |
| `torch.save(m.state_dict(), p)` | `model.save_checkpoint("m.fdl")` |
| `AutoModel.from_pretrained(r)` | `flodl_b200.hf.AutoModel.from_pretrained(r)` |
'''

SKILLS = {"guide": ("The condensed API and porting reference of flodl_b200", None),
          "port": ("Port PyTorch scripts to flodl_b200: read the source, map the patterns, write the project, validate", PORT_SKILL)}
TOOLS = {"claude": "Claude Code (.claude/ directory): .claude/skills/<skill>/SKILL.md",
         "cursor": "Cursor (.cursor/ or .cursorrules): appended to .cursorrules",
         "generic": "no assistant detected: .fdl/skills/<skill>/SKILL.md"}


def detect_tools(root: str) -> List[str]:
    out = []
    if os.path.isdir(os.path.join(root, ".claude")):
        out.append("claude")
    if os.path.isdir(os.path.join(root, ".cursor")) or os.path.isfile(os.path.join(root, ".cursorrules")):
        out.append("cursor")
    return out


def skill_text(name: str) -> str:
    return SKILL if name == "guide" else SKILLS[name][1]


def install_skill(root: str, tool: str, name: str) -> str:
    text = skill_text(name)
    if tool == "cursor":
        path = os.path.join(root, ".cursorrules")
        marker = f"# --- flodl_b200 skill: {name} ---"
        old = open(path).read() if os.path.isfile(path) else ""
        if marker in old:                                   # installed before: replace that block, keep the user's own rules
            head, _, rest = old.partition(marker)
            tail = rest.partition("# --- end flodl_b200 skill ---")[2]
            old = head.rstrip("\n") + ("\n" if head.strip() else "") + tail.lstrip("\n")
        with open(path, "w") as f:
            f.write((old.rstrip("\n") + "\n\n" if old.strip() else "") + f"{marker}\n{text.rstrip()}\n# --- end flodl_b200 skill ---\n")
        return path
    d = os.path.join(root, ".claude", "skills", name) if tool == "claude" else os.path.join(root, ".fdl", "skills", name)
    os.makedirs(d, exist_ok=True)
    path = os.path.join(d, "SKILL.md")
    with open(path, "w") as f:
        f.write(text)
    return path


def skill(argv: List[str]) -> int:
    """`skill list | show [name] | install [--tool claude|cursor|generic] [--skill NAME] [dir]`."""
    sub = argv[0] if argv else "show"
    rest = argv[1:]

    def opt(flag):
        if flag in rest:
            i = rest.index(flag)
            if i + 1 < len(rest):
                v = rest[i + 1]
                del rest[i:i + 2]
                return v
            del rest[i]
        return None
    if sub == "show":
        name = rest[0] if rest else "guide"
        if name not in SKILLS:
            print(f"unknown skill {name!r}; one of: {', '.join(SKILLS)}", file=sys.stderr)
            return 2
        print(skill_text(name))
        return 0
    if sub == "list":
        print("skills:")
        for n, (doc, _t) in SKILLS.items():
            print(f"  {n:<8} {doc}")
        found = detect_tools(os.getcwd())
        print("tools detected here: " + (", ".join(found) if found else "none (install goes to .fdl/skills/)"))
        for t, doc in TOOLS.items():
            print(f"  {t:<8} {doc}")
        return 0
    if sub == "install":
        tool, only = opt("--tool"), opt("--skill")
        root = os.path.abspath(rest[0] if rest else ".")
        if tool is not None and tool not in TOOLS:
            print(f"unknown tool {tool!r}; one of: {', '.join(TOOLS)}", file=sys.stderr)
            return 2
        if only is not None and only not in SKILLS:
            print(f"unknown skill {only!r}; one of: {', '.join(SKILLS)}", file=sys.stderr)
            return 2
        tools = [tool] if tool else (detect_tools(root) or ["generic"])
        for t in tools:
            for n in ([only] if only else list(SKILLS)):
                print(f"installed {install_skill(root, t, n)}")
        return 0
    print("usage: skill [list | show [name] | install [--tool claude|cursor|generic] [--skill NAME] [dir]]", file=sys.stderr)
    return 2
