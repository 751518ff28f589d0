#!/usr/bin/env python
"""Build the reference's own CPU implementation of the deformable-convolution path.

TEST INFRASTRUCTURE ONLY.  Nothing under ``oracle/`` is part of the product; only the
tests, the smoke check and the CPU-baseline / reference legs of the benchmark may use it.

The reference (inspiros/tvdcn v1.1.0) keeps its CPU path in a handful of plain C++
translation units:

* ``tvdcn/csrc/ops/deform_conv{1,2,3}d.cpp`` and ``deform_conv_transpose{1,2,3}d.cpp``
  (operator schemas, ``TORCH_LIBRARY_FRAGMENT``),
* ``tvdcn/csrc/ops/cpu/*.cpp`` (host loops + OpenMP kernels, ``TORCH_LIBRARY_IMPL(.., CPU, ..)``),
* ``tvdcn/csrc/ops/utils/tensor_utils.cpp``.

This script compiles exactly those files *where they lie* in the reference checkout with
``g++`` (the reference's own setup.py is not run) and links them into
``oracle/_ref/libtvdcn_ref.so``.  No reference source is copied into this repository.

Two things are changed on the way through the compiler, neither touching arithmetic:

1. The dispatcher namespace is renamed ``tvdcn`` -> ``tvdcn_ref`` so that the reference and
   this repository's own ``tvdcn::*`` operators can be loaded into one process.  Tokens are
   renamed with ``-Dtvdcn=tvdcn_ref``; the ``"tvdcn::..."`` string literals are renamed by
   streaming each translation unit through a one-line substitution into ``g++ -x c++ -``.
2. ``OMP_NUM_THREADS`` (a compile-time constant, 32, in ``cpu/cpu_helpers.h:17-20``) is set to
   ``omp_get_max_threads()`` so the three parallel loops use every host core of whatever box
   the library later runs on.  The scatter loop stays serial, as in the reference
   (``cpu/deform_conv2d_common_kernels.cpp:273``).

The autograd and autocast translation units are left out on purpose: the oracle is driven
through ``torch.ops.tvdcn_ref.deform_convNd`` / ``_deform_convNd_backward`` directly, which is
also what side-steps the reference's optional-tensor autograd failure on recent torch.

With ``--cuda`` (and from ``build_cuda()``) the reference's CUDA backend is built the same way into a second
library, ``oracle/_ref/libtvdcn_ref_cuda.so``: ``tvdcn/csrc/ops/cuda/*.cu`` compiled in place by ``nvcc`` for
sm_100 (no string literal in them names the dispatcher namespace, so ``-Dtvdcn=tvdcn_ref`` is enough) and
``tvdcn/csrc/ops/cuda/*.cpp`` streamed through ``g++`` like the CPU units.  It registers the ``CUDA`` kernels of
the ``tvdcn_ref::*`` operators that the first library declares, and serves as a second checker on the GPU
(full-size parity) and as the timed GPU baseline of the benchmark.

Usage:  python oracle/build_ref.py [--reference /path/to/tvdcn] [--jobs N] [--cuda]
"""
from __future__ import annotations

import argparse
import os
import re
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT_DIR = HERE / "_ref"


def reference_dir() -> Path:
    """Where the reference checkout (the tvdcn project) is looked for: $TVDCN_REFERENCE_DIR, else a directory
    `reference` beside this repository."""
    env = os.environ.get("TVDCN_REFERENCE_DIR")
    return Path(env) if env else Path(__file__).resolve().parent.parent.parent / "reference"


def reference_present() -> bool:
    return (reference_dir() / "tvdcn" / "csrc").is_dir()

LIB_NAME = "libtvdcn_ref.so"
CUDA_LIB_NAME = "libtvdcn_ref_cuda.so"


def _sources(ref: Path) -> list[Path]:
    ops = ref / "tvdcn" / "csrc" / "ops"
    srcs = sorted(ops.glob("deform_conv*.cpp"))
    srcs += sorted((ops / "cpu").glob("*.cpp"))
    srcs += [ops / "utils" / "tensor_utils.cpp"]
    return srcs


def _compile_one(src: Path, obj: Path, flags: list[str]) -> None:
    text = src.read_text()
    # string literals only: "tvdcn::name" -> "tvdcn_ref::name"
    text = re.sub(r'"tvdcn::', '"tvdcn_ref::', text)
    cmd = ["g++", "-x", "c++", "-", "-c", "-o", str(obj), "-iquote", str(src.parent)] + flags
    res = subprocess.run(cmd, input=text.encode(), capture_output=True)
    if res.returncode != 0:
        raise RuntimeError(f"compiling {src} failed:\n{res.stderr.decode()[-4000:]}")


def build(reference: str | os.PathLike | None = None, jobs: int | None = None,
          force: bool = False) -> Path:
    ref = Path(reference) if reference is not None else reference_dir()
    lib = OUT_DIR / LIB_NAME
    srcs = _sources(ref)
    if not srcs or not all(s.exists() for s in srcs):
        raise FileNotFoundError(f"reference sources not found under {ref}")
    if lib.exists() and not force:
        newest = max(s.stat().st_mtime for s in srcs + [Path(__file__)])
        if lib.stat().st_mtime >= newest:
            return lib
    from torch.utils import cpp_extension as ce

    OUT_DIR.mkdir(exist_ok=True)
    obj_dir = OUT_DIR / "obj"
    obj_dir.mkdir(exist_ok=True)
    flags = ["-O2", "-fPIC", "-std=c++17", "-fopenmp", "-DAT_PARALLEL_OPENMP",
             "-Dtvdcn=tvdcn_ref", "-include", "omp.h", "-DOMP_NUM_THREADS=omp_get_max_threads()",
             "-D_GLIBCXX_USE_CXX11_ABI=1", "-w"]
    for inc in ce.include_paths():
        flags += ["-isystem", inc]
    objs = []
    work = []
    for s in srcs:
        # distinct object names: cpu/x_kernel.cpp and ops/x.cpp would otherwise collide
        obj = obj_dir / (s.parent.name + "__" + s.stem + ".o")
        objs.append(obj)
        work.append((s, obj))
    jobs = jobs or os.cpu_count() or 4
    with ThreadPoolExecutor(max_workers=jobs) as ex:
        list(ex.map(lambda a: _compile_one(a[0], a[1], flags), work))
    torch_lib = ce.library_paths()[0]
    cmd = ["g++", "-shared", "-o", str(lib)] + [str(o) for o in objs] + [
        "-fopenmp", f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-lc10",
        f"-Wl,-rpath,{torch_lib}"]
    subprocess.run(cmd, check=True)
    return lib


def build_cuda(reference: str | os.PathLike | None = None, jobs: int | None = None,
               force: bool = False) -> Path:
    """The reference's CUDA kernels and host orchestration -> oracle/_ref/libtvdcn_ref_cuda.so (sm_100)."""
    ref = Path(reference) if reference is not None else reference_dir()
    lib = OUT_DIR / CUDA_LIB_NAME
    cuda_dir = ref / "tvdcn" / "csrc" / "ops" / "cuda"
    cu = sorted(cuda_dir.glob("*.cu"))
    cpp = sorted(cuda_dir.glob("*.cpp")) + [ref / "tvdcn" / "csrc" / "ops" / "utils" / "tensor_utils.cpp"]
    if not cu or not all(s.exists() for s in cu + cpp):
        raise FileNotFoundError(f"reference CUDA sources not found under {ref}")
    if lib.exists() and not force:
        newest = max(s.stat().st_mtime for s in cu + cpp + [Path(__file__)])
        if lib.stat().st_mtime >= newest:
            return lib
    from torch.utils import cpp_extension as ce

    OUT_DIR.mkdir(exist_ok=True)
    obj_dir = OUT_DIR / "obj_cuda"
    obj_dir.mkdir(exist_ok=True)
    cuda_home = Path(ce.CUDA_HOME or "/usr/local/cuda")
    incs = []
    for inc in ce.include_paths("cuda") + [str(cuda_home / "include")]:
        incs += ["-isystem", inc]
    cxx_flags = ["-O2", "-fPIC", "-std=c++17", "-Dtvdcn=tvdcn_ref", "-DWITH_CUDA", "-D_GLIBCXX_USE_CXX11_ABI=1",
                 "-w"] + incs
    nvcc_flags = ["-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-Dtvdcn=tvdcn_ref", "-DWITH_CUDA",
                  "-D_GLIBCXX_USE_CXX11_ABI=1", "-gencode", "arch=compute_100,code=sm_100", "-w",
                  "--expt-relaxed-constexpr", "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__",
                  "-D__CUDA_NO_BFLOAT16_CONVERSIONS__", "-D__CUDA_NO_HALF2_OPERATORS__"] + incs

    def nvcc_one(src: Path, obj: Path) -> None:
        res = subprocess.run([str(cuda_home / "bin" / "nvcc"), "-c", str(src), "-o", str(obj)] + nvcc_flags,
                             capture_output=True)
        if res.returncode != 0:
            raise RuntimeError(f"compiling {src} failed:\n{res.stderr.decode()[-4000:]}")

    objs, work = [], []
    for s_ in cu:
        obj = obj_dir / ("cu__" + s_.stem + ".o")
        objs.append(obj)
        work.append(lambda s_=s_, obj=obj: nvcc_one(s_, obj))
    for s_ in cpp:
        obj = obj_dir / (s_.parent.name + "__" + s_.stem + ".o")
        objs.append(obj)
        work.append(lambda s_=s_, obj=obj: _compile_one(s_, obj, cxx_flags))
    jobs = jobs or os.cpu_count() or 4
    with ThreadPoolExecutor(max_workers=jobs) as ex:
        list(ex.map(lambda f: f(), work))
    torch_lib = ce.library_paths()[0]
    cmd = ["g++", "-shared", "-o", str(lib)] + [str(o) for o in objs] + [
        f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
        f"-L{cuda_home / 'lib64'}", "-lcudart", f"-Wl,-rpath,{torch_lib}"]
    subprocess.run(cmd, check=True)
    return lib


def load_cuda() -> bool:
    """Load the reference's CUDA kernels next to the CPU library; False when either was never built."""
    import torch

    lib = OUT_DIR / CUDA_LIB_NAME
    if not lib.exists() or not load():
        return False
    if not hasattr(load_cuda, "_done"):
        torch.ops.load_library(str(lib))
        load_cuda._done = True
    return True


def load() -> bool:
    """Load the built reference into ``torch.ops.tvdcn_ref``; False when it was never built."""
    import torch

    lib = OUT_DIR / LIB_NAME
    if not lib.exists():
        return False
    if not hasattr(load, "_done"):
        torch.ops.load_library(str(lib))
        load._done = True
    return True


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None, help="reference checkout (default: $TVDCN_REFERENCE_DIR, else ../reference)")
    ap.add_argument("--jobs", type=int, default=None)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--cuda", action="store_true", help="also build the reference's CUDA backend")
    a = ap.parse_args()
    print(build(a.reference, a.jobs, a.force))
    if a.cuda:
        print(build_cuda(a.reference, a.jobs, a.force))
    sys.exit(0)
