"""Builds libctdk.so (the sm_100a kernels + C-ABI) and the command-line tools in-tree with nvcc.

Usage: python -m emberlm_b200.build [--force] [--verbose]
Every .cu / .cpp file under csrc/ is compiled to an object next to this file's build/
directory and linked into emberlm_b200/libctdk.so. Objects are rebuilt only when their
source (or a header) is newer. Each cli/*.cpp becomes an executable of the same name next to the
library (emberlm_b200/ctd_train), linked against it with an $ORIGIN run path.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = HERE / "build"
LIB = HERE / "libctdk.so"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall",
          "-I", str(HERE.parent / "include"), "--expt-relaxed-constexpr"]


def _sources() -> list[Path]:
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp")))


def _headers_mtime() -> float:
    hs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list((HERE.parent / "include").glob("*.h"))
    return max((h.stat().st_mtime for h in hs), default=0.0)


def _compile(src: Path, verbose: bool) -> tuple[Path, str]:
    obj = OBJ / (src.name + ".o")
    cmd = [NVCC, *ARCH, *COMMON, "-Xptxas", "-v", "-c", str(src), "-o", str(obj)]
    if src.suffix == ".cpp":
        cmd.insert(1, "-x")
        cmd.insert(2, "cu")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    return obj, r.stderr if verbose else ""


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    hdr_m = _headers_mtime()
    todo, objs = [], []
    for src in _sources():
        obj = OBJ / (src.name + ".o")
        objs.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_m):
            todo.append(src)
    if todo:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(todo))) as ex:
            for obj, log in ex.map(lambda s: _compile(s, verbose), todo):
                if verbose and log:
                    print(log)
    if todo or not LIB.exists() or any(o.stat().st_mtime > LIB.stat().st_mtime for o in objs):
        cmd = [NVCC, *ARCH, "-shared", "-o", str(LIB), *map(str, objs), "-lcudart"]
        nccl = os.environ.get("CTDK_NCCL_LIB")
        if nccl:
            cmd.append(nccl)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    _build_tools(force)
    return LIB


def _build_tools(force: bool) -> None:
    cli = HERE / "cli"
    hdrs = list(cli.glob("*.hpp")) + list((HERE.parent / "include").glob("*.h"))
    newest_hdr = max((h.stat().st_mtime for h in hdrs), default=0.0)
    for src in sorted(cli.glob("*.cpp")):
        exe = HERE / src.stem
        if not force and exe.exists() and exe.stat().st_mtime >= max(src.stat().st_mtime, newest_hdr, LIB.stat().st_mtime):
            continue
        cmd = [NVCC, "-O2", "-std=c++17", "-Xcompiler", "-Wall", "-o", str(exe), str(src), "-L", str(HERE), "-lctdk",
               "-lcudart", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"building {src.name} failed:\n{r.stdout}\n{r.stderr}")


if __name__ == "__main__":
    lib = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(lib)
