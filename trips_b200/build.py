"""In-tree build of libtrips_b200.so (hand-written CUDA for sm_100a, plain C ABI, no torch dependency).

    python -m trips_b200.build [--force] [--verbose]

Flags that matter:
  -gencode arch=compute_100a,code=sm_100a   B200 only, no PTX fallback for other parts
  -fmad=false                               fp32 expressions are not fused, so list construction, alphas and
                                            transmittance cut-offs round exactly like the CPU oracle
  -lineinfo                                 source correlation for ncu
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libtrips_b200.so")
SOURCES = ["forward.cu", "second.cu", "backward.cu", "adam.cu", "rank.cu", "resize.cu", "capi.cu", "noalloc.cu"]
HEADERS = ["common.cuh", "trips_math.h", os.path.join("..", "..", "include", "trips_b200.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo", "-fmad=false",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: libtrips_b200.so cannot be built")


def _sources():
    return [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in _sources()] + [os.path.join(CSRC, h) for h in HEADERS] + [__file__]
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every .cu file to an object and link the shared library next to this file."""
    if not force and not _stale():
        return LIB
    nvcc = _nvcc()
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    objs = []
    procs = []
    for s in _sources():
        obj = os.path.join(objdir, s.replace(".cu", ".o"))
        cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", os.path.join(CSRC, s), "-o", obj]
        procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for s, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(out)
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {s}")
    link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB] + objs + ["-lcudart"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError("link of libtrips_b200.so failed")
    return LIB


SHIM = os.path.join(HERE, "libtrips_b200_torch.so")
SHIM_SRC = os.path.join(CSRC, "torch_shim.cpp")


def build_torch_shim(force: bool = False) -> str:
    """Compile the libtorch host side (csrc/torch_shim.cpp: NeuralRenderInfo, PointRender, BlendPointCloud on top of
    the C ABI) with the host compiler and link it against libtrips_b200.so and libtorch."""
    build()
    deps = [SHIM_SRC, os.path.join(CSRC, "torch_shim.h"), os.path.join(HERE, "..", "include", "trips_b200.h"), __file__]
    if not force and os.path.exists(SHIM) and all(os.path.getmtime(d) <= os.path.getmtime(SHIM) for d in deps):
        return SHIM
    import torch
    from torch.utils import cpp_extension as ce
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else (shutil.which("g++") or "g++")
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           "-I", os.path.join(HERE, "..", "include")]
    for inc in ce.include_paths("cuda"):
        cmd += ["-isystem", inc]
    cmd += [SHIM_SRC, "-o", SHIM, "-L", HERE, "-ltrips_b200", "-Wl,-rpath,$ORIGIN"]
    for lp in ce.library_paths("cuda"):
        cmd += ["-L", lp, f"-Wl,-rpath,{lp}"]
    cmd += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-lcudart"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout[-4000:])
        raise RuntimeError("build of libtrips_b200_torch.so failed")
    return SHIM


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    if "--shim" in sys.argv:
        print(build_torch_shim(force="--force" in sys.argv))
