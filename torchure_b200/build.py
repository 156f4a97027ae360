"""In-tree build of the CUDA extension for sm_100a.

    python -m torchure_b200.build

Kernel sources (``csrc/*.cu``) do not include the PyTorch headers, so they compile in seconds with
``nvcc -gencode arch=compute_100a,code=sm_100a``; only the binding files see torch.  Objects are cached
under ``torchure_b200/_build`` keyed by a hash of the source and headers, and the result is linked to
``torchure_b200/_C.so`` (the path the GPU tests and benchmarks load).
"""

from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
BUILD = PKG / "_build"
TARGET = PKG / "_C.so"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v"]
# fast-math would change softmax/rsqrt numerics in the memory-bound kernels; keep it to the files that opt in
FAST_MATH_FILES: set[str] = set()


def _torch_paths():
    import torch
    from torch.utils.cpp_extension import CUDA_HOME, include_paths, library_paths

    return include_paths("cuda"), library_paths("cuda"), CUDA_HOME or "/usr/local/cuda", torch


def _hash(paths: list[Path], extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()[:16]


def _run(cmd: list[str], verbose: bool) -> str:
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
        raise RuntimeError(f"build step failed: {cmd[0]} {cmd[-1]}")
    return res.stdout + res.stderr


def build_all(verbose: bool = False, force: bool = False) -> Path:
    includes, libdirs, cuda_home, torch = _torch_paths()
    BUILD.mkdir(exist_ok=True)
    headers = sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh"))
    nvcc = os.path.join(cuda_home, "bin", "nvcc")
    jobs = []
    objects = []
    for src in sorted(CSRC.glob("*.cu")):
        flags = [f for f in NVCC_FLAGS if f != "--use_fast_math" or src.name in FAST_MATH_FILES]
        tag = _hash([src] + headers, " ".join(flags))
        obj = BUILD / f"{src.stem}.{tag}.o"
        objects.append(obj)
        if force or not obj.exists():
            jobs.append((src, [nvcc, *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]))
    py_inc = sysconfig.get_paths()["include"]
    cxx_flags = ["-O2", "-std=c++17", "-fPIC", "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
                 f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", "-I", str(CSRC), "-I", py_inc]
    for inc in includes:
        cxx_flags += ["-isystem", inc]
    for src in sorted(CSRC.glob("*.cpp")):
        tag = _hash([src] + headers, " ".join(cxx_flags) + torch.__version__)
        obj = BUILD / f"{src.stem}.{tag}.o"
        objects.append(obj)
        if force or not obj.exists():
            jobs.append((src, ["g++", *cxx_flags, "-c", str(src), "-o", str(obj)]))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            for (src, _), out in zip(jobs, pool.map(lambda j: _run(j[1], verbose), jobs)):
                if verbose:
                    info = [ln for ln in out.splitlines() if "registers" in ln or "spill" in ln]
                    worst = max((int(ln.split("Used ")[1].split(" ")[0]) for ln in info if "Used " in ln), default=0)
                    spills = sum(1 for ln in info if "spill stores" in ln and " 0 bytes spill stores" not in ln)
                    print(f"[build] {src.name}: max {worst} registers, {spills} kernels with spills")
    keep = {o.name for o in objects}
    for old in BUILD.glob("*.o"):
        if old.name not in keep:
            old.unlink()
    if jobs or not TARGET.exists() or force:
        link = ["g++", "-shared", "-o", str(TARGET), *map(str, objects)]
        for d in libdirs:
            link += [f"-L{d}", f"-Wl,-rpath,{d}"]
        link += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
        _run(link, verbose)
        if verbose:
            print(f"[build] linked {TARGET}")
    return TARGET


if __name__ == "__main__":
    build_all(verbose=True, force="--force" in sys.argv)
