"""In-tree build of the sm_100a extension ``legion_b200/_C.so``.

Kernel sources (``csrc/*.cu``) are compiled by nvcc for ``sm_100a`` only and carry no torch headers,
so they build in seconds; the two binding files are compiled by the host compiler against torch.
Objects are cached under ``legion_b200/csrc/build`` by source hash, so a rebuild only recompiles
what changed.  Run ``python -m legion_b200.build_ext`` (add ``-v`` for ptxas resource usage).
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
BUILD = CSRC / "build"
TARGET = ROOT / "_C.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = Path(cuda_home) / "bin" / "nvcc"
    return str(cand) if cand.exists() else "nvcc"


def _hash(path: Path, extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    h.update(path.read_bytes())
    for hdr in sorted(list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh"))):
        h.update(hdr.read_bytes())
    return h.hexdigest()[:16]


def _run(cmd: list[str]) -> str:
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + p.stdout + p.stderr)
    return p.stdout + p.stderr


def build(verbose: bool = False, force: bool = False) -> Path:
    import torch
    from torch.utils import cpp_extension

    BUILD.mkdir(parents=True, exist_ok=True)
    cu_files = sorted(CSRC.glob("*.cu"))
    cpp_files = sorted(CSRC.glob("*.cpp"))
    inc = [f"-I{p}" for p in cpp_extension.include_paths()] + [f"-I{sysconfig.get_paths()['include']}"]
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    inc.append(f"-I{cuda_home}/include")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cxx_flags = ["-O2", "-std=c++17", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_EXTENSION_NAME=_C",
                 "-DTORCH_API_INCLUDE_EXTENSION_H", "-w"]

    jobs = []
    objs = []
    for src in cu_files:
        flags = NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else [])
        obj = BUILD / f"{src.stem}.{_hash(src, ' '.join(flags))}.o"
        objs.append(obj)
        if force or not obj.exists():
            jobs.append(([_nvcc(), *flags, "-c", str(src), "-o", str(obj)], src))
    for src in cpp_files:
        obj = BUILD / f"{src.stem}.{_hash(src, ' '.join(cxx_flags) + torch.__version__)}.o"
        objs.append(obj)
        if force or not obj.exists():
            jobs.append((["g++", *cxx_flags, *inc, "-c", str(src), "-o", str(obj)], src))

    def work(job):
        cmd, src = job
        out = _run(cmd)
        if verbose and out.strip():
            print(f"--- {src.name}\n{out}")
        return src.name

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for name in ex.map(work, jobs):
                print(f"[build_ext] compiled {name}", file=sys.stderr)
    # drop stale objects
    keep = {o.name for o in objs}
    for o in BUILD.glob("*.o"):
        if o.name not in keep:
            o.unlink()

    newest = max(o.stat().st_mtime for o in objs)
    if force or jobs or not TARGET.exists() or TARGET.stat().st_mtime < newest:
        torch_lib = Path(torch.__file__).parent / "lib"
        link = ["g++", "-shared", "-o", str(TARGET), *map(str, objs), f"-L{torch_lib}", f"-L{cuda_home}/lib64",
                "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart",
                f"-Wl,-rpath,{torch_lib}", f"-Wl,-rpath,{cuda_home}/lib64"]
        _run(link)
        print(f"[build_ext] linked {TARGET}", file=sys.stderr)
    return TARGET


HOST_SRC = ROOT / "csrc_host"
HOST_TARGET = ROOT / "_host.so"


def build_host(force: bool = False) -> Path:
    """The native host runtime ``legion_b200/_host.so`` (block pool, radix cache, step packing): plain C++17 with
    pybind11, no CUDA and no torch, so it also loads in processes that never touch a GPU."""
    import pybind11
    srcs = sorted(HOST_SRC.glob("*.cpp"))
    h = hashlib.sha256()
    for s in srcs:
        h.update(s.read_bytes())
    stamp = HOST_SRC / "build" / f"host.{h.hexdigest()[:16]}.stamp"
    if not force and HOST_TARGET.exists() and stamp.exists():
        return HOST_TARGET
    stamp.parent.mkdir(parents=True, exist_ok=True)
    for old in stamp.parent.glob("host.*.stamp"):
        old.unlink()
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-w",
           f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}",
           *map(str, srcs), "-o", str(HOST_TARGET)]
    _run(cmd)
    stamp.write_text("ok")
    print(f"[build_ext] linked {HOST_TARGET}", file=sys.stderr)
    return HOST_TARGET


if __name__ == "__main__":
    build(verbose="-v" in sys.argv, force="-f" in sys.argv)
    build_host(force="-f" in sys.argv)
