"""In-tree build of the two native libraries.

* ``libtvdcn_b200.so`` -- CUDA kernels + the C ABI (include/tvdcn_b200.h); nvcc only, no torch.
* ``_C.so``            -- PyTorch dispatcher front end (csrc/torch_ops.cpp); g++ against torch headers,
                          linked to the first through an ``$ORIGIN`` rpath.

Both are compiled for sm_100a only and are rebuilt only when a source is newer than the output.
Run ``python -m tvdcn_b200.build`` (add ``--verbose`` for ptxas resource usage).
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = PKG.parent / "include"
OBJ = PKG / "build"
LIB = PKG / "libtvdcn_b200.so"
EXT = PKG / "_C.so"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def _newer(sources, target: Path) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > t for s in sources)


def _run(cmd, **kw):
    res = subprocess.run(cmd, capture_output=True, text=True, **kw)
    if res.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(map(str, cmd)) + "\n" + res.stdout[-4000:] + res.stderr[-8000:])
    return res.stdout + res.stderr


def build_cuda_library(verbose: bool = False, force: bool = False) -> Path:
    cu = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*.h"))
    OBJ.mkdir(exist_ok=True)
    flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if verbose else [])
    if os.environ.get("TVDCN_B200_TUNING"):      # in-kernel cycle counters, never part of a normal build
        flags.append("-DTVDCN_B200_TUNING")
    flags += os.environ.get("TVDCN_B200_NVCC_FLAGS", "").split()   # extra flags for experiments
    jobs = []
    for src in cu:
        obj = OBJ / (src.stem + ".o")
        if force or _newer([src] + headers, obj):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        out = _run(["nvcc", *flags, "-c", str(src), "-o", str(obj)])
        if verbose:
            print(out)

    with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4) or 1) as ex:
        list(ex.map(compile_one, jobs))
    objs = [OBJ / (s.stem + ".o") for s in cu]
    if force or jobs or _newer(objs, LIB):
        _run(["nvcc", "-shared", "-o", str(LIB), *map(str, objs), "-lcudart", "-lcuda"])
    return LIB


def build_torch_extension(force: bool = False) -> Path:
    from torch.utils import cpp_extension as ce

    src = CSRC / "torch_ops.cpp"
    if not (force or _newer([src, INCLUDE / "tvdcn_b200.h", LIB], EXT)):
        return EXT
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cmd = ["g++", "-O2", "-fPIC", "-std=c++17", "-shared", "-D_GLIBCXX_USE_CXX11_ABI=1", "-w",
           str(src), "-o", str(EXT), f"-I{cuda_home}/include"]
    for inc in ce.include_paths():
        cmd += ["-isystem", inc]
    tl = ce.library_paths()[0]
    cmd += [f"-L{PKG}", "-ltvdcn_b200", f"-L{tl}", "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda", "-lc10_cuda",
            "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{tl}", f"-L{cuda_home}/lib64", "-lcudart"]
    _run(cmd)
    return EXT


def build_all(verbose: bool = False, force: bool = False) -> None:
    build_cuda_library(verbose=verbose, force=force)
    build_torch_extension(force=force)


if __name__ == "__main__":
    build_all(verbose="--verbose" in sys.argv, force="--force" in sys.argv)
    print(LIB)
    print(EXT)
