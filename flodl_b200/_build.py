"""In-tree build of the native library (`flodl_b200/_C.so`).

The CUDA kernels (`csrc/kernels`, `csrc/comm`) are plain CUDA with an `extern "C"` surface and do
not include torch headers, so each compiles in seconds; the binding and runtime sources
(`csrc/bindings`, `csrc/runtime`) are C++17 against the libtorch headers that ship inside the
installed `torch` wheel. Everything is linked into ONE shared object that is both a Python
extension module (pybind11) and a C library (the `fb_*` / `flodl_*` symbols of
`csrc/include/flodl_b200.h` can be `dlopen`ed).

This is the counterpart of the reference's `flodl-sys/build.rs` (C++17 unity build linked against
libtorch), with the difference that there is device code to compile:
`nvcc -gencode arch=compute_100a,code=sm_100a`.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
BUILD = ROOT / "build"
TARGET = Path(__file__).resolve().parent / "_C.so"
# The drop-in C library (`csrc/abi`): the `flodl_*` functions of the reference's C interface, no Python in it.
SHIM_TARGET = Path(__file__).resolve().parent / "libflodl_b200_shim.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "--use_fast_math", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


BOUNDS_CHECK = os.environ.get("FLODL_B200_BOUNDS_CHECK", "0") not in ("0", "")
if BOUNDS_CHECK:
    # debug build: device-side index checks that record instead of faulting (see csrc/kernels/common.cuh);
    # it goes to its own file so the regular library stays untouched
    NVCC_FLAGS.append("-DFLODL_BOUNDS_CHECK=1")
    BUILD = ROOT / "build_dbg"
    TARGET = Path(__file__).resolve().parent / "_C_dbg.so"
if os.environ.get("FLODL_B200_TIMELINE", "0") not in ("0", ""):
    NVCC_FLAGS.append("-DFB_TIMELINE=1")      # per-CTA timestamps in the GEMM / convolution kernels (tuning builds only)


def _sources():
    cu = sorted((CSRC / "kernels").glob("*.cu")) + sorted((CSRC / "comm").glob("*.cu"))
    cpp = sorted((CSRC / "runtime").glob("*.cpp")) + sorted((CSRC / "bindings").glob("*.cpp"))
    return cu, cpp


def _abi_sources():
    return sorted((CSRC / "abi").glob("*.cpp"))


def _nccl_flags():
    """(include flag, link flags) for the NCCL that torch itself runs on, else the system one."""
    import torch
    root = Path(torch.__file__).parent.parent / "nvidia" / "nccl"
    if (root / "lib" / "libnccl.so.2").is_file():
        return f"-I{root / 'include'}", f"-L{root / 'lib'} -Wl,-rpath,{root / 'lib'} -l:libnccl.so.2"
    return "", "-lnccl"


def _newest_mtime(paths):
    return max((p.stat().st_mtime for p in paths), default=0.0)


def needs_build() -> bool:
    if not TARGET.exists():
        return True
    cu, cpp = _sources()
    hdrs = list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.hpp"))
    if not BOUNDS_CHECK and (not SHIM_TARGET.exists() or _newest_mtime(cu + _abi_sources() + hdrs) > SHIM_TARGET.stat().st_mtime):
        return True
    return _newest_mtime(cu + cpp + hdrs) > TARGET.stat().st_mtime


def write_ninja() -> Path:
    import torch
    from torch.utils import cpp_extension as ce

    cu, cpp = _sources()
    BUILD.mkdir(exist_ok=True)
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    inc = ce.include_paths() + [sysconfig.get_paths()["include"], f"{cuda_home}/include", str(CSRC / "include")]
    inc_flags = " ".join(f"-I{p}" for p in inc)
    torch_lib = str(Path(torch.__file__).parent / "lib")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cxx_flags = (
        f"-O2 -std=c++17 -fPIC -fvisibility=default {'-DFLODL_BOUNDS_CHECK=1 ' if BOUNDS_CHECK else ''}-DTORCH_EXTENSION_NAME={'_C_dbg' if BOUNDS_CHECK else '_C'} -D_GLIBCXX_USE_CXX11_ABI={abi} "
        f"-DTORCH_API_INCLUDE_EXTENSION_H -Wno-deprecated-declarations -Wno-interference-size {inc_flags}"
    )
    lines = [
        "ninja_required_version = 1.3",
        f"nvcc = {cuda_home}/bin/nvcc",
        "cxx = g++",
        f"nvcc_flags = {' '.join(NVCC_FLAGS)} -I{CSRC / 'include'}",
        f"cxx_flags = {cxx_flags}",
        "rule nvcc",
        "  command = $nvcc $nvcc_flags -MD -MF $out.d -c $in -o $out",
        "  depfile = $out.d",
        "  deps = gcc",
        "  description = NVCC $in",
        "rule cxx",
        "  command = $cxx $cxx_flags -MMD -MF $out.d -c $in -o $out",
        "  depfile = $out.d",
        "  deps = gcc",
        "  description = CXX $in",
        "rule link",
        f"  command = $cxx -shared $in -o $out -L{torch_lib} -L{cuda_home}/lib64 -Wl,-rpath,{torch_lib} "
        "-ltorch -ltorch_cpu -ltorch_cuda -lc10 -lc10_cuda -ltorch_python -lcudart -lz -ldl -lpthread",
        "  description = LINK $out",
    ]
    nccl_inc, nccl_link = _nccl_flags()
    lines += [
        "rule cxx_abi",
        f"  command = $cxx -O2 -std=c++17 -fPIC -fvisibility=hidden -D_GLIBCXX_USE_CXX11_ABI={abi} -Wno-deprecated-declarations "
        f"-Wno-interference-size {' '.join('-I' + p for p in ce.include_paths() + [cuda_home + '/include', str(CSRC / 'include')])} {nccl_inc} "
        "-MMD -MF $out.d -c $in -o $out",
        "  depfile = $out.d",
        "  deps = gcc",
        "  description = CXX $in",
        "rule link_abi",
        f"  command = $cxx -shared $in -o $out -L{torch_lib} -L{cuda_home}/lib64 -Wl,-rpath,{torch_lib} -Wl,--no-undefined "
        f"-ltorch -ltorch_cpu -ltorch_cuda -lc10 -lc10_cuda -lcudart {nccl_link} -ldl -lpthread",
        "  description = LINK $out",
    ]
    objs = []
    for s in cu:
        o = BUILD / (s.stem + ".cu.o")
        lines.append(f"build {o}: nvcc {s}")
        objs.append(str(o))
    for s in cpp:
        o = BUILD / (s.stem + ".cpp.o")
        lines.append(f"build {o}: cxx {s}")
        objs.append(str(o))
    lines.append(f"build {TARGET}: link {' '.join(objs)}")
    defaults = [str(TARGET)]
    if not BOUNDS_CHECK:
        # the drop-in C library shares the kernel objects; the comm kernels stay out (it does its collectives with NCCL)
        abi_objs = [o for o, src in zip(objs, cu) if src.parent.name == "kernels"]
        for s in _abi_sources():
            o = BUILD / (s.stem + ".abi.o")
            lines.append(f"build {o}: cxx_abi {s}")
            abi_objs.append(str(o))
        lines.append(f"build {SHIM_TARGET}: link_abi {' '.join(abi_objs)}")
        defaults.append(str(SHIM_TARGET))
    lines.append(f"default {' '.join(defaults)}")
    path = BUILD / "build.ninja"
    path.write_text("\n".join(lines) + "\n")
    return path


def build(verbose: bool = False) -> Path:
    """Compile every native source for sm_100a and link `_C.so` and `libflodl_b200_shim.so` (incremental)."""
    ninja_file = write_ninja()
    cmd = ["ninja", "-f", str(ninja_file), "-j", str(max(2, os.cpu_count() or 2))]
    if verbose:
        cmd.append("-v")
    res = subprocess.run(cmd, cwd=str(BUILD), capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout[-8000:] + res.stderr[-8000:])
        raise RuntimeError("flodl_b200 native build failed")
    return TARGET


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv))
