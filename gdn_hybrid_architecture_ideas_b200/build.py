"""Builds the in-tree native extension `_native.so` for sm_100a: every `csrc/*.cu` with nvcc
(`-gencode arch=compute_100a,code=sm_100a -lineinfo`), `csrc/binding.cpp` with the host compiler against the torch
headers, linked into one shared object beside this file. Objects are rebuilt when a source or header is newer.

    python -m gdn_hybrid_architecture_ideas_b200.build [--force] [--verbose]
"""

from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
SRC = HERE / "csrc"
OBJ = HERE / "csrc" / "build"
TARGET = HERE / "_native.so"
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def _run(cmd, verbose):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"build step failed: {' '.join(map(str, cmd))}\n{r.stdout}\n{r.stderr}")
    if verbose:
        print(r.stderr)
    return r.stderr


def _stale(out: Path, deps) -> bool:
    return not out.exists() or any(d.stat().st_mtime > out.stat().st_mtime for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    from torch.utils import cpp_extension as ce

    OBJ.mkdir(parents=True, exist_ok=True)
    headers = list(SRC.glob("*.h")) + list(SRC.glob("*.cuh"))
    nvcc = os.path.join(ce.CUDA_HOME or "/usr/local/cuda", "bin", "nvcc")
    cu = sorted(SRC.glob("*.cu"))
    jobs, objs, log = [], [], {}
    for src in cu:
        o = OBJ / (src.stem + ".o")
        objs.append(o)
        if force or _stale(o, [src, *headers]):
            jobs.append((src, [nvcc, *NVCC_FLAGS, "-I", str(SRC), "-c", str(src), "-o", str(o)]))
    inc = [f"-I{p}" for p in ce.include_paths(device_type="cuda")] + [f"-I{sysconfig.get_paths()['include']}", f"-I{SRC}"]
    bobj = OBJ / "binding.o"
    objs.append(bobj)
    if force or _stale(bobj, [SRC / "binding.cpp", *headers]):
        jobs.append((SRC / "binding.cpp", ["g++", "-O2", "-std=c++17", "-fPIC", "-DTORCH_EXTENSION_NAME=_native", "-DTORCH_API_INCLUDE_EXTENSION_H",
                                           "-D_GLIBCXX_USE_CXX11_ABI=1", *inc, "-c", str(SRC / "binding.cpp"), "-o", str(bobj)]))
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        for (src, _), out in zip(jobs, pool.map(lambda j: _run(j[1], verbose), jobs)):
            log[src.name] = out
    if jobs or not TARGET.exists():
        libs = [f"-L{p}" for p in ce.library_paths(device_type="cuda")]
        _run(["g++", "-shared", "-o", str(TARGET), *map(str, objs), *libs, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
              "-ltorch_python", "-lcudart", *[f"-Wl,-rpath,{p}" for p in ce.library_paths(device_type="cuda")]], verbose)
    (OBJ / "ptxas.log").write_text("\n".join(f"== {k}\n{v}" for k, v in log.items()) if log else (OBJ / "ptxas.log").read_text() if (OBJ / "ptxas.log").exists() else "")
    return TARGET


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
