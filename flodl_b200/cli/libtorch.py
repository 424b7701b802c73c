"""`fdl libtorch`: which libtorch a program links, and side-by-side variants of it
(flodl-cli/src/libtorch/{detect,download,build,manage}.rs).

Python programs use the libtorch inside the installed `torch` wheel; that one is always listed as `wheel/<version>`.
A host written against the C interface (`libflodl_b200_shim.so`, or tch-rs / PyTorch C++) may want another: variants
live under `<root>/libtorch/precompiled/<cpu|cu126|cu128>` (downloaded archives) and `<root>/libtorch/builds/<archs>`
(compiled from source for an exact set of GPU architectures), each with a `.arch` file (`torch=`, `cuda=`, `archs=`,
`source=`), and `<root>/libtorch/.active` names the one in use. `<root>` is the project directory when there is an
`fdl.yml`, else `$FLODL_HOME` (default `~/.flodl`).

    libtorch list [--json] | info [--json] | path | activate <name> | remove <name>
    libtorch download [--cpu | --cuda 12.6|12.8] [--path DIR] [--no-activate] [--dry-run]
    libtorch build [--archs "9.0;10.0"] [--jobs N] [--docker | --native] [--dry-run]
"""
from __future__ import annotations

import json
import os
import shutil
import subprocess
import sys
import zipfile
from typing import Dict, List, Optional

LIBTORCH_VERSION = "2.10.0"
PRECOMPILED = {
    "cpu": {"cuda": None, "archs": "", "bucket": "cpu", "covers": "any machine, no GPU acceleration"},
    "cu126": {"cuda": "12.6", "archs": "5.0 6.0 6.1 7.0 7.5 8.0 8.6 9.0", "bucket": "cu126", "covers": "sm_50 to sm_90 (Maxwell to Ada / Hopper)"},
    "cu128": {"cuda": "12.8", "archs": "7.0 7.5 8.0 8.6 9.0 10.0 12.0", "bucket": "cu128", "covers": "sm_70 to sm_120 (Volta to Blackwell)"},
}


class LibtorchError(Exception):
    pass


# ---- where variants live -------------------------------------------------------------------------------------
def root_dir(start: str = ".") -> str:
    from .manifest import find_manifest
    m = find_manifest(start)
    if m is not None:
        return os.path.dirname(os.path.abspath(m))
    return os.environ.get("FLODL_HOME") or os.path.join(os.path.expanduser("~"), ".flodl")


def _lt(root: str) -> str:
    return os.path.join(root, "libtorch")


def read_arch(variant_dir: str) -> Dict[str, Optional[str]]:
    info: Dict[str, Optional[str]] = {"torch": None, "cuda": None, "archs": None, "source": None}
    try:
        for line in open(os.path.join(variant_dir, ".arch")):
            k, _, v = line.strip().partition("=")
            if k in info:
                info[k] = v
    except OSError:
        pass
    return info


def write_arch(variant_dir: str, torch: str, cuda: Optional[str], archs: str, source: str) -> None:
    with open(os.path.join(variant_dir, ".arch"), "w") as f:
        f.write(f"torch={torch}\ncuda={cuda or 'none'}\narchs={archs}\nsource={source}\n")


def wheel_variant() -> Optional[Dict[str, object]]:
    """The libtorch of the `torch` package this interpreter imports."""
    import importlib.util
    if importlib.util.find_spec("torch") is None:
        return None
    import torch
    archs = " ".join(a.replace("sm_", "")[:-1] + "." + a[-1] for a in torch.cuda.get_arch_list()) if torch.cuda.is_available() else ""
    return {"name": f"wheel/{torch.__version__.split('+')[0]}", "path": os.path.dirname(torch.__file__), "torch": torch.__version__,
            "cuda": torch.version.cuda, "archs": archs, "source": "python wheel"}


def list_variants(root: str) -> List[Dict[str, object]]:
    """Installed variants (a directory counts when it has `lib/`), the wheel's first."""
    out = []
    w = wheel_variant()
    if w is not None:
        out.append(w)
    for sub in ("precompiled", "builds"):
        d = os.path.join(_lt(root), sub)
        if not os.path.isdir(d):
            continue
        for name in sorted(os.listdir(d)):
            vdir = os.path.join(d, name)
            if os.path.isdir(os.path.join(vdir, "lib")):
                out.append({"name": f"{sub}/{name}", "path": vdir, **read_arch(vdir)})
    return out


def read_active(root: str) -> Optional[str]:
    try:
        name = open(os.path.join(_lt(root), ".active")).read().strip()
    except OSError:
        return None
    return name or None


def set_active(root: str, name: str) -> None:
    os.makedirs(_lt(root), exist_ok=True)
    with open(os.path.join(_lt(root), ".active"), "w") as f:
        f.write(name + "\n")


def active_variant(root: str) -> Optional[Dict[str, object]]:
    """The variant `.active` names; without one (or when it is gone) the wheel's libtorch."""
    variants = list_variants(root)
    name = read_active(root)
    for v in variants:
        if v["name"] == name:
            return v
    return variants[0] if variants and str(variants[0]["name"]).startswith("wheel/") else None


def arch_compatible(sm_major: int, sm_minor: int, archs: str) -> bool:
    """Whether a variant compiled for `archs` ("8.0 9.0 10.0") has code for a GPU of that compute capability."""
    toks = archs.replace(";", " ").split()
    return f"{sm_major}.{sm_minor}" in toks or str(sm_major) in toks


def remove_variant(root: str, name: str) -> None:
    if name.startswith("wheel/"):
        raise LibtorchError("the wheel's libtorch belongs to the Python environment; uninstall `torch` with pip instead")
    vdir = os.path.join(_lt(root), name)
    if name.split("/")[0] not in ("precompiled", "builds") or not os.path.isdir(vdir):
        raise LibtorchError(f"no variant `{name}`; installed: {', '.join(str(v['name']) for v in list_variants(root))}")
    shutil.rmtree(vdir)
    if read_active(root) == name:
        os.remove(os.path.join(_lt(root), ".active"))


# ---- download ------------------------------------------------------------------------------------------------
def detect_gpu_archs() -> List[str]:
    """Compute capabilities of the visible GPUs ("10.0"), from torch when CUDA is up, else from nvidia-smi."""
    try:
        import torch
        if torch.cuda.is_available():
            return sorted({"%d.%d" % torch.cuda.get_device_capability(i) for i in range(torch.cuda.device_count())}, key=float)
    except Exception:  # noqa: BLE001
        pass
    try:
        out = subprocess.run(["nvidia-smi", "--query-gpu=compute_cap", "--format=csv,noheader"], capture_output=True, text=True, timeout=10)
        return sorted({ln.strip() for ln in out.stdout.splitlines() if ln.strip()}, key=float) if out.returncode == 0 else []
    except (OSError, subprocess.TimeoutExpired, ValueError):
        return []


def pick_variant(archs: List[str]) -> str:
    """cpu without a GPU; cu128 when every GPU is Volta or newer; cu126 otherwise (it reaches back to sm_50)."""
    if not archs:
        return "cpu"
    return "cu128" if all(float(a) >= 7.0 for a in archs) else "cu126"


def download_url(variant: str, version: str = LIBTORCH_VERSION) -> str:
    spec = PRECOMPILED[variant]
    tag = "cpu" if variant == "cpu" else variant
    return f"https://download.pytorch.org/libtorch/{spec['bucket']}/libtorch-shared-with-deps-{version}%2B{tag}.zip"


def download(root: str, variant: str, dest: Optional[str] = None, activate: bool = True, dry_run: bool = False, out=print) -> str:
    if variant not in PRECOMPILED:
        raise LibtorchError(f"unknown variant `{variant}`; one of {', '.join(PRECOMPILED)}")
    name = f"precompiled/{variant}"
    vdir = dest or os.path.join(_lt(root), name)
    url = download_url(variant)
    out(f"  variant:  {name} ({PRECOMPILED[variant]['covers']})")
    out(f"  from:     {url}")
    out(f"  to:       {vdir}")
    if dry_run:
        out("  dry run: nothing downloaded")
        return vdir
    import urllib.error
    import urllib.request
    os.makedirs(vdir, exist_ok=True)
    tmp = os.path.join(vdir, "libtorch.zip.part")
    try:
        with urllib.request.urlopen(url, timeout=60) as r, open(tmp, "wb") as f:
            shutil.copyfileobj(r, f, 1 << 20)
    except (urllib.error.URLError, OSError) as e:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise LibtorchError(f"download failed: {e}") from e
    install_archive(tmp, vdir)
    os.remove(tmp)
    write_arch(vdir, LIBTORCH_VERSION, PRECOMPILED[variant]["cuda"], PRECOMPILED[variant]["archs"], "precompiled")
    if activate and dest is None:
        set_active(root, name)
    return vdir


def install_archive(zip_path: str, vdir: str) -> None:
    """Unpack a libtorch archive so that `<vdir>/lib`, `<vdir>/include`, ... exist (the archive has one top folder)."""
    with zipfile.ZipFile(zip_path) as z:
        for member in z.namelist():
            parts = member.split("/", 1)
            rel = parts[1] if len(parts) == 2 and parts[0] == "libtorch" else member
            if not rel or rel.endswith("/"):
                continue
            target = os.path.normpath(os.path.join(vdir, rel))
            if not target.startswith(os.path.abspath(vdir) + os.sep) and target != os.path.abspath(vdir):
                raise LibtorchError(f"archive member escapes the install directory: {member}")
            os.makedirs(os.path.dirname(target), exist_ok=True)
            with z.open(member) as src, open(target, "wb") as dst:
                shutil.copyfileobj(src, dst)


# ---- build from source ---------------------------------------------------------------------------------------
def arch_dir_name(archs: str) -> str:
    """"6.1;12.0" -> "sm61-sm120"."""
    return "-".join("sm" + a.replace(".", "") for a in archs.replace(";", " ").split())


def native_tools() -> Dict[str, bool]:
    return {t: shutil.which(t) is not None for t in ("nvcc", "cmake", "python3", "git", "gcc")}


BUILDER_IMAGE = "flodl-libtorch-builder"
BUILDER_DOCKERFILE = """\
FROM nvidia/cuda:12.8.0-cudnn-devel-ubuntu22.04
ARG TORCH_CUDA_ARCH_LIST
ARG MAX_JOBS=6
ARG TORCH_TAG
ENV DEBIAN_FRONTEND=noninteractive
RUN apt-get update && apt-get install -y --no-install-recommends git cmake ninja-build python3 python3-pip python3-dev build-essential \\
    libopenblas-dev && rm -rf /var/lib/apt/lists/*
RUN git clone --recursive --depth 1 --branch ${TORCH_TAG} https://github.com/pytorch/pytorch /src/pytorch
WORKDIR /src/pytorch
RUN python3 -m pip install --no-cache-dir -r requirements.txt
RUN TORCH_CUDA_ARCH_LIST="${TORCH_CUDA_ARCH_LIST}" MAX_JOBS=${MAX_JOBS} USE_CUDA=1 BUILD_TEST=0 USE_DISTRIBUTED=1 USE_NCCL=1 \\
    python3 tools/build_libtorch.py
RUN mkdir -p /opt/libtorch && cp -r torch/lib torch/include torch/share /opt/libtorch/
"""


def build_docker(plan: Dict[str, object], run=subprocess.call, capture=subprocess.check_output) -> None:
    """Build inside a throw-away image (layer caching makes a failed build resumable), then copy `/opt/libtorch` out."""
    import tempfile
    out_dir = str(plan["output"])
    with tempfile.TemporaryDirectory() as tmp:
        df = os.path.join(tmp, "Dockerfile")
        with open(df, "w") as f:
            f.write(BUILDER_DOCKERFILE)
        cmd = ["docker", "build", "--build-arg", f"TORCH_CUDA_ARCH_LIST={plan['archs']}", "--build-arg", f"MAX_JOBS={plan['jobs']}",
               "--build-arg", f"TORCH_TAG=v{LIBTORCH_VERSION}", "-t", BUILDER_IMAGE, "-f", df, tmp]
        if run(cmd) != 0:
            raise LibtorchError("docker build failed (re-running resumes from the cached layers)")
    cid = capture(["docker", "create", BUILDER_IMAGE], text=True).strip()
    try:
        os.makedirs(out_dir, exist_ok=True)
        if run(["docker", "cp", f"{cid}:/opt/libtorch/.", out_dir]) != 0:
            raise LibtorchError("docker cp of /opt/libtorch failed")
    finally:
        run(["docker", "rm", cid])


def build_plan(root: str, archs: Optional[str], jobs: int, backend: Optional[str]) -> Dict[str, object]:
    """What `libtorch build` would do: the architecture list (given or detected), the backend (docker when it is
    there unless `--native`), the output directory and the commands."""
    archs = archs or ";".join(detect_gpu_archs())
    if not archs:
        raise LibtorchError("no GPU detected and no --archs given: nothing to build for (use `libtorch download --cpu`)")
    tools = native_tools()
    has_docker = shutil.which("docker") is not None
    if backend is None:
        backend = "docker" if has_docker else "native"
    if backend == "docker" and not has_docker:
        raise LibtorchError("--docker: docker is not installed (https://docs.docker.com/engine/install/)")
    if backend == "native" and not all(tools.values()):
        raise LibtorchError("--native needs " + ", ".join(t for t, ok in tools.items() if not ok) + "; install them or use --docker")
    out_dir = os.path.join(_lt(root), "builds", arch_dir_name(archs))
    src = os.path.join(_lt(root), ".build-cache", "pytorch")
    env = f'TORCH_CUDA_ARCH_LIST="{archs}" MAX_JOBS={jobs} USE_CUDA=1 BUILD_TEST=0 USE_DISTRIBUTED=1 USE_NCCL=1'
    if backend == "native":
        cmds = [f"test -d {src} || git clone --recursive --depth 1 --branch v{LIBTORCH_VERSION} https://github.com/pytorch/pytorch {src}",
                f"python3 -m pip install -r {src}/requirements.txt",
                f"cd {src} && {env} python3 tools/build_libtorch.py",
                f"mkdir -p {out_dir} && cp -r {src}/torch/lib {src}/torch/include {src}/torch/share {out_dir}/"]
    else:
        cmds = [f"docker build --build-arg TORCH_CUDA_ARCH_LIST=\"{archs}\" --build-arg MAX_JOBS={jobs} --build-arg TORCH_TAG=v{LIBTORCH_VERSION} "
                f"-t {BUILDER_IMAGE} -f <generated Dockerfile> <tmp>",
                f"docker create {BUILDER_IMAGE}",
                f"docker cp <container>:/opt/libtorch/. {out_dir}/",
                "docker rm <container>"]
    return {"archs": archs, "backend": backend, "jobs": jobs, "output": out_dir, "source_cache": src, "commands": cmds}


# ---- the command -----------------------------------------------------------------------------------------------
def _flag_value(argv: List[str], flag: str) -> Optional[str]:
    if flag in argv:
        i = argv.index(flag)
        if i + 1 >= len(argv):
            raise LibtorchError(f"{flag} needs a value")
        return argv[i + 1]
    return None


def main(argv: List[str], out=print) -> int:
    sub = argv[0] if argv else "info"
    rest = argv[1:]
    root = root_dir(os.getcwd())
    try:
        if sub == "path":
            v = active_variant(root)
            if v is None:
                raise LibtorchError("no libtorch found")
            out(os.path.join(str(v["path"]), "lib"))
        elif sub == "list":
            variants, active = list_variants(root), active_variant(root)
            if "--json" in rest:
                out(json.dumps([{**v, "active": active is not None and v["name"] == active["name"]} for v in variants], indent=2))
            elif not variants:
                out("no libtorch installed (pip install torch, or `libtorch download`)")
            else:
                for v in variants:
                    mark = " (active)" if active is not None and v["name"] == active["name"] else ""
                    out(f"  {v['name']}{mark}")
        elif sub == "info":
            v = active_variant(root)
            if v is None:
                raise LibtorchError("no libtorch found (pip install torch, or `libtorch download`)")
            info = dict(v)
            if str(v["name"]).startswith("wheel/"):
                import torch
                info.update(cudnn=torch.backends.cudnn.version() if torch.backends.cudnn.is_available() else None,
                            cxx11_abi=bool(torch._C._GLIBCXX_USE_CXX11_ABI), lib_dir=os.path.join(str(v["path"]), "lib"))
                try:
                    info["nccl"] = ".".join(map(str, torch.cuda.nccl.version()))
                except Exception:  # noqa: BLE001
                    info["nccl"] = None
            if "--json" in rest:
                out(json.dumps(info, indent=2))
            else:
                out(f"Active:   {v['name']}\nVersion:  {v.get('torch')}\nCUDA:     {v.get('cuda')}\nArchs:    {v.get('archs')}\nSource:   {v.get('source')}")
                for k in ("cudnn", "nccl", "cxx11_abi", "lib_dir"):
                    if k in info:
                        out(f"{k + ':':<9} {info[k]}")
        elif sub == "activate":
            names = [str(v["name"]) for v in list_variants(root)]
            if not rest:
                out("variants: " + ", ".join(names))
                return 0
            if rest[0] not in names:
                raise LibtorchError(f"no variant `{rest[0]}`; installed: {', '.join(names)}")
            set_active(root, rest[0])
            out(f"active libtorch: {rest[0]}")
        elif sub == "remove":
            if not rest:
                out("variants: " + ", ".join(str(v["name"]) for v in list_variants(root)))
                return 0
            remove_variant(root, rest[0])
            out(f"removed {rest[0]}")
        elif sub == "download":
            cuda = _flag_value(rest, "--cuda")
            if cuda is not None and cuda not in ("12.6", "12.8"):
                raise LibtorchError("--cuda accepts 12.6 or 12.8 (the published pre-built versions)")
            variant = "cpu" if "--cpu" in rest else {"12.6": "cu126", "12.8": "cu128"}.get(cuda) or pick_variant(detect_gpu_archs())
            download(root, variant, _flag_value(rest, "--path"), "--no-activate" not in rest, "--dry-run" in rest, out)
        elif sub == "build":
            backend = "docker" if "--docker" in rest else "native" if "--native" in rest else None
            plan = build_plan(root, _flag_value(rest, "--archs"), int(_flag_value(rest, "--jobs") or 6), backend)
            out(f"  archs:    {plan['archs']}\n  backend:  {plan['backend']}\n  jobs:     {plan['jobs']}\n  output:   {plan['output']}")
            for c in plan["commands"]:
                out(f"    $ {c}")
            if "--dry-run" in rest:
                out("  dry run: nothing built")
                return 0
            if plan["backend"] == "docker":
                build_docker(plan)
            else:
                for c in plan["commands"]:
                    if subprocess.call(c, shell=True) != 0:
                        raise LibtorchError(f"step failed: {c}")
            write_arch(str(plan["output"]), LIBTORCH_VERSION, None, str(plan["archs"]).replace(";", " "), "compiled")
            set_active(root, "builds/" + arch_dir_name(str(plan["archs"])))
        else:
            print("usage: libtorch [info [--json] | list [--json] | path | activate <name> | remove <name> | download [...] | build [...]]", file=sys.stderr)
            return 2
    except LibtorchError as e:
        print(f"fdl libtorch: {e}", file=sys.stderr)
        return 1
    return 0
