"""Build the UNMODIFIED reference (DictXiong/AllReduce-Over-MPI) for the benchmark's reference arm.

The reference is C++/CUDA with no Python packaging, so ``pip install --target baseline/_ref
<reference checkout>`` cannot work ("neither setup.py nor pyproject.toml found"); its outcome is
recorded in baseline/_ref/INSTALL_LOG.txt.  The checkout is taken from $FT_REFERENCE_SRC.  Instead the
sources are copied verbatim to baseline/_ref/src and compiled as they are:

  * baseline/_ref/ref_nway       nvcc, sm_100a: ref_nway_driver.cu + the reference's
                                 vector_add/reduce_sum_gpu.h (its GPU launcher reduce_sum_gpu<T>)
  * baseline/_ref/ref_mpi_bench  g++: the reference's allreduce_over_mpi/benchmark.cpp + mpi_mod.hpp
                                 against baseline/mpi_shim (shared-memory MPI subset) and
                                 baseline/glog_stub (the image has neither MPI nor glog)
  * baseline/_ref/ref_config1    g++: config1_driver.cpp -DCONFIG1_REFERENCE + the reference's mpi_mod.hpp
                                 over the same shim (seeded uniform data, fp64 check; see config1.py)
  * baseline/_ref/ft_config1     g++: the same driver against this repository's libflextree.so (thread world)
  * baseline/_ref/ft_config1_procs  g++ -DCONFIG1_PROCS: the same driver over the process world (ranks are processes)

Nothing of this repository's library is linked into the three reference binaries.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF = Path(os.environ.get("FT_REFERENCE_SRC", str(Path.home() / "reference")))
OUT = HERE / "_ref"


def run(cmd, log):
    r = subprocess.run(cmd, capture_output=True, text=True)
    log.write(f"$ {' '.join(map(str, cmd))}\nrc={r.returncode}\n{r.stdout[-2000:]}{r.stderr[-2000:]}\n")
    return r.returncode


def main() -> int:
    OUT.mkdir(parents=True, exist_ok=True)
    with open(OUT / "INSTALL_LOG.txt", "w") as log:
        rc = run([sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--find-links", "/opt/wheelhouse",
                  "--target", str(OUT), str(REF)], log)
        log.write(f"pip install of the reference: rc={rc} (expected to fail: not a Python project)\n")
        src = OUT / "src"
        if src.exists():
            shutil.rmtree(src)
        shutil.copytree(REF, src)
        nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
        rc1 = run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++14", "-I", str(HERE / "glog_stub"),
                   "-I", str(src / "vector_add"), str(HERE / "ref_nway_driver.cu"), "-o", str(OUT / "ref_nway")], log)
        # flags of the reference's CMakeLists.txt:5 (minus glog/MPI link libraries, which the stubs replace)
        rc2 = run(["g++", "-std=c++11", "-O2", "-fPIC", "-fopenmp", "-mavx2", "-fpermissive", "-w",
                   "-DGIT_REPO_VERSION=\"reference\"", "-DGIT_REPO_DATE=\"n/a\"", "-DGIT_REPO_HASH=\"n/a\"",
                   "-I", str(HERE / "mpi_shim"), "-I", str(HERE / "glog_stub"), "-I", str(src / "allreduce_over_mpi"),
                   str(src / "allreduce_over_mpi" / "benchmark.cpp"), str(HERE / "mpi_shim" / "mpi_shim.cpp"),
                   "-o", str(OUT / "ref_mpi_bench"), "-lrt", "-lpthread"], log)
        ref_flags = ["g++", "-std=c++11", "-O2", "-fPIC", "-fopenmp", "-mavx2", "-fpermissive", "-w"]
        rc3 = run([*ref_flags, "-DCONFIG1_REFERENCE", "-I", str(HERE / "mpi_shim"), "-I", str(HERE / "glog_stub"),
                   "-I", str(src / "allreduce_over_mpi"), str(HERE / "config1_driver.cpp"), str(HERE / "mpi_shim" / "mpi_shim.cpp"),
                   "-o", str(OUT / "ref_config1"), "-lrt", "-lpthread"], log)
        pkg = HERE.parent / "allreduce_over_mpi_b200"
        rc4 = run(["g++", "-std=c++17", "-O2", "-I", str(pkg / "csrc"), str(HERE / "config1_driver.cpp"), "-L", str(pkg / "lib"),
                   "-lflextree", f"-Wl,-rpath,{pkg / 'lib'}", "-lpthread", "-o", str(OUT / "ft_config1")], log)
        rc5 = run(["g++", "-std=c++17", "-O2", "-DCONFIG1_PROCS", "-I", str(pkg / "csrc"), str(HERE / "config1_driver.cpp"), "-L", str(pkg / "lib"),
                   "-lflextree", f"-Wl,-rpath,{pkg / 'lib'}", "-lpthread", "-o", str(OUT / "ft_config1_procs")], log)
        log.write(f"ref_nway build rc={rc1}; ref_mpi_bench build rc={rc2}; ref_config1 build rc={rc3}; ft_config1 build rc={rc4}; "
                  f"ft_config1_procs build rc={rc5}\n")
    print(open(OUT / "INSTALL_LOG.txt").read()[-1500:])
    return 0 if rc1 == 0 and rc2 == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
