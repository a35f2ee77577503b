"""In-tree build of libflextree.so (host planner + sm_100a kernels + runtime).

`python -m allreduce_over_mpi_b200.build` compiles every source under csrc/ with nvcc for
sm_100a only (`-gencode arch=compute_100a,code=sm_100a -lineinfo`) and links one shared
library next to the package.  nvcc cross-compiles without a GPU.  The CUDA runtime is
linked statically and the driver API is resolved at run time, so the library also loads
on a machine without a driver (the planner, cost model and CPU executors work there).

Counterpart of the reference's three separate builds (allreduce_over_mpi/CMakeLists.txt,
cost_model/CMakeLists.txt, vector_add/Makefile, which targets sm_35..sm_86 only).
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "csrc" / "build"
LIB = PKG / "lib" / "libflextree.so"

NVCC = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fopenmp,-Wall,-Wno-unknown-pragmas",
          "-I", str(CSRC), "--expt-relaxed-constexpr"]


def sources() -> list[Path]:
    out = []
    for sub in ("api", "kernels", "runtime"):
        d = CSRC / sub
        if d.is_dir():
            out += sorted(p for p in d.iterdir() if p.suffix in (".cu", ".cpp"))
    return out


def headers_mtime() -> float:
    m = 0.0
    for p in CSRC.rglob("*"):
        if p.suffix in (".h", ".hpp", ".cuh"):
            m = max(m, p.stat().st_mtime)
    return max(m, Path(__file__).stat().st_mtime)


def compile_one(src: Path, verbose: bool, obj_dir: Path = OBJ, defines: tuple = ()) -> tuple[Path, str]:
    obj = obj_dir / (src.stem + ".o")
    cmd = [NVCC, *ARCH, *COMMON, *defines, "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    return obj, r.stderr


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile what changed and link; returns the path of the shared library."""
    OBJ.mkdir(parents=True, exist_ok=True)
    LIB.parent.mkdir(parents=True, exist_ok=True)
    hm = headers_mtime()
    srcs = sources()
    todo = []
    for s in srcs:
        o = OBJ / (s.stem + ".o")
        if force or not o.exists() or o.stat().st_mtime < max(s.stat().st_mtime, hm):
            todo.append(s)
    logs = []
    if todo:
        with cf.ThreadPoolExecutor(max_workers=min(len(todo), os.cpu_count() or 4)) as ex:
            for obj, log in ex.map(lambda s: compile_one(s, verbose), todo):
                logs.append(log)
    objs = [OBJ / (s.stem + ".o") for s in srcs]
    if todo or not LIB.exists() or any(o.stat().st_mtime > LIB.stat().st_mtime for o in objs):
        cmd = [NVCC, *ARCH, "-shared", "-cudart", "static", "-o", str(LIB), *map(str, objs),
               "-Xcompiler", "-fopenmp", "-lpthread", "-ldl", "-lrt"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    build_tools()
    if verbose:
        print("\n".join(logs))
    return LIB


BOUNDS_LIB = PKG / "lib" / "libflextree_bounds.so"


def build_bounds(force: bool = False) -> Path:
    """The debugging build: the same sources with -DFT_BOUNDS, linked as lib/libflextree_bounds.so.  Its collective
    kernels test every run of heap bytes against the heap size before touching it (csrc/kernels/comm_bounds.h);
    select it with FT_LIB=bounds in the environment of the process that loads the library."""
    obj_dir = PKG / "csrc" / "build_bounds"
    obj_dir.mkdir(parents=True, exist_ok=True)
    hm = headers_mtime()
    srcs = sources()
    todo = [s for s in srcs if force or not (obj_dir / (s.stem + ".o")).exists()
            or (obj_dir / (s.stem + ".o")).stat().st_mtime < max(s.stat().st_mtime, hm)]
    if todo:
        with cf.ThreadPoolExecutor(max_workers=min(len(todo), os.cpu_count() or 4)) as ex:
            list(ex.map(lambda s: compile_one(s, False, obj_dir, ("-DFT_BOUNDS",)), todo))
    objs = [obj_dir / (s.stem + ".o") for s in srcs]
    if todo or not BOUNDS_LIB.exists():
        cmd = [NVCC, *ARCH, "-shared", "-cudart", "static", "-o", str(BOUNDS_LIB), *map(str, objs),
               "-Xcompiler", "-fopenmp", "-lpthread", "-ldl", "-lrt"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return BOUNDS_LIB


def build_tools() -> list[Path]:
    """Native command-line tools next to the library: ft_bench, planner_dump, cost_model_sweep."""
    out = []
    tools = CSRC / "tools"
    hm = headers_mtime()
    for src in sorted(tools.glob("*.cpp")):
        exe = LIB.parent / src.stem
        if exe.exists() and exe.stat().st_mtime >= max(src.stat().st_mtime, hm, LIB.stat().st_mtime):
            out.append(exe)
            continue
        cmd = [NVCC, *ARCH, "-O2", "-std=c++17", "-I", str(CSRC), str(src), "-o", str(exe), "-Xcompiler", "-fopenmp",
               "-L", str(LIB.parent), "-lflextree", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN", "-lpthread"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"tool build failed for {src.name}:\n{r.stdout}\n{r.stderr}")
        out.append(exe)
    return out


def ensure_built() -> Path:
    """Build if the library is missing or older than its sources (needs nvcc)."""
    if LIB.exists():
        newest = max([s.stat().st_mtime for s in sources()] + [headers_mtime()])
        if LIB.stat().st_mtime >= newest:
            return LIB
        if not os.path.exists(NVCC):
            return LIB
    return build()


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(p)
    if "--bounds" in sys.argv:
        print(build_bounds(force="--force" in sys.argv))
