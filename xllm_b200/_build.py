"""In-tree native build for xllm_b200.

Two shared objects are produced next to the Python sources so that they travel
with a snapshot of the tree and are visible in ``/proc/<pid>/maps`` of every
process that uses them:

* ``xllm_b200/lib/libxllm_kernels.so`` — every hand-written sm_100a CUDA kernel
  with a plain C launcher (``extern "C" int xllm_*(..., void* stream)``).  The
  sources contain no torch headers, so each file compiles in seconds.
* ``xllm_b200/_rt*.so`` — the C++ runtime (block manager, prefix cache,
  scheduler, batch builder, tokenizer, safetensors reader, HTTP server, ...)
  exposed through pybind11.

Staleness is decided by a content hash of sources + flags stored beside each
artefact, never by timestamps (a copied tree has fresh timestamps everywhere).

The reference builds through CMake + setup.py (setup.py:1-1070 in the
reference tree); this build is deliberately a ~150-line script because there is
exactly one target architecture.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIBDIR = ROOT / "lib"
OBJDIR = ROOT / "lib" / "obj"

NVCC = os.environ.get("XLLM_NVCC", "/usr/local/cuda/bin/nvcc")
CXX = os.environ.get("CXX", "g++")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
    "-I", str(CSRC),
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-pthread",
             "-I", str(CSRC / "runtime"), "-I", str(CSRC / "frontend"), "-I", str(CSRC / "server"),
             "-Wall", "-Wno-sign-compare", "-I", str(CSRC), "-I", "/usr/local/cuda/include"]

KERNEL_LIB = LIBDIR / "libxllm_kernels.so"


def _rt_path() -> Path:
    return ROOT / ("_rt" + sysconfig.get_config_var("EXT_SUFFIX"))


def _sha(paths, extra: str) -> str:
    # the tree may be copied anywhere: absolute paths must not influence staleness
    h = hashlib.sha256(extra.replace(str(ROOT), "<root>").encode())
    for p in sorted(paths):
        h.update(str(p.relative_to(ROOT)).encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _headers(sub: str):
    return list((CSRC / sub).rglob("*.cuh")) + list((CSRC / sub).rglob("*.h")) \
        + list((CSRC / sub).rglob("*.hpp"))


def _run(cmd, verbose):
    if verbose:
        print("[xllm_b200 build]", " ".join(str(c) for c in cmd), flush=True)
    r = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("build failed: " + " ".join(str(c) for c in cmd[:4]))
    if verbose and (r.stdout or r.stderr):
        print(r.stdout + r.stderr, flush=True)


def kernel_sources():
    return sorted((CSRC / "kernels").glob("*.cu"))


class _BuildLock:
    """Inter-process lock: several ranks importing the package at once must not build concurrently."""

    def __init__(self):
        LIBDIR.mkdir(exist_ok=True)
        self.path = LIBDIR / ".build.lock"

    def __enter__(self):
        import fcntl
        self.f = open(self.path, "w")
        fcntl.flock(self.f, fcntl.LOCK_EX)
        return self

    def __exit__(self, *a):
        import fcntl
        fcntl.flock(self.f, fcntl.LOCK_UN)
        self.f.close()


def _link_atomic(cmd_prefix, out: Path, objs, tail, verbose):
    tmp = out.with_name(out.name + f".tmp{os.getpid()}")
    _run([*cmd_prefix, "-o", tmp, *objs, *tail], verbose)
    os.replace(tmp, out)  # readers never see a half-written library


def build_kernels(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Compile every ``csrc/kernels/*.cu`` for sm_100a and link the C-ABI library."""
    with _BuildLock():
        return _build_kernels(force, verbose, ptxas_info)


def _build_kernels(force, verbose, ptxas_info) -> Path:
    srcs = kernel_sources()
    hdrs = _headers("kernels")
    flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if ptxas_info else [])
    LIBDIR.mkdir(exist_ok=True)
    OBJDIR.mkdir(exist_ok=True)
    hdr_hash = _sha(hdrs, " ".join(flags))
    todo, objs = [], []
    for s in srcs:
        o = OBJDIR / (s.stem + ".o")
        stamp = OBJDIR / (s.stem + ".sha")
        want = _sha([s], hdr_hash)
        objs.append(o)
        if force or not o.exists() or not stamp.exists() or stamp.read_text() != want:
            todo.append((s, o, stamp, want))
    if not shutil.which(NVCC) and todo:
        raise RuntimeError(f"nvcc not found at {NVCC}; cannot build CUDA kernels")

    def one(item):
        s, o, stamp, want = item
        _run([NVCC, *flags, "-c", s, "-o", o], verbose or ptxas_info)
        stamp.write_text(want)

    if todo:
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
            list(ex.map(one, todo))
    link_stamp = LIBDIR / "libxllm_kernels.sha"
    want = _sha(srcs + hdrs, " ".join(flags))
    if todo or force or not KERNEL_LIB.exists() or not link_stamp.exists() \
            or link_stamp.read_text() != want:
        _link_atomic([NVCC, "-shared"], KERNEL_LIB, objs, ["-lcudart"], verbose)
        link_stamp.write_text(want)
    return KERNEL_LIB


def runtime_sources():
    out = []
    for sub in ("runtime", "frontend", "server"):
        out += sorted((CSRC / sub).glob("*.cpp"))
    return out


def build_c_api(force: bool = False, verbose: bool = False) -> Path:
    """Compile ``libxllm_c.so``: the C interface (csrc/c_api/xllm.h) over an embedded interpreter."""
    with _BuildLock():
        src = CSRC / "c_api" / "xllm_c_api.cpp"
        hdr = CSRC / "c_api" / "xllm.h"
        out = LIBDIR / "libxllm_c.so"
        stamp = LIBDIR / "libxllm_c.sha"
        ldlib = sysconfig.get_config_var("LDLIBRARY") or "libpython3.so"
        libname = ldlib[3:].split(".so")[0] if ldlib.startswith("lib") else "python3"
        flags = CXX_FLAGS + ["-I", sysconfig.get_paths()["include"]]
        libs = ["-L", sysconfig.get_config_var("LIBDIR") or "/usr/lib", "-l" + libname, "-pthread", "-ldl"]
        want = _sha([src, hdr], " ".join(map(str, flags + libs)))
        if force or not out.exists() or not stamp.exists() or stamp.read_text() != want:
            LIBDIR.mkdir(parents=True, exist_ok=True)
            OBJDIR.mkdir(parents=True, exist_ok=True)
            obj = OBJDIR / "c_api.o"
            _run([CXX, *flags, "-c", src, "-o", obj], verbose)
            _link_atomic([CXX, "-shared"], out, [obj], libs, verbose)
            stamp.write_text(want)
        return out


def build_runtime(force: bool = False, verbose: bool = False) -> Path:
    """Compile the C++ runtime + pybind11 module ``xllm_b200._rt``."""
    with _BuildLock():
        return _build_runtime(force, verbose)


def _build_runtime(force, verbose) -> Path:
    import pybind11

    srcs = runtime_sources()
    hdrs = _headers("runtime") + _headers("frontend") + _headers("server")
    inc = ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"]]
    flags = CXX_FLAGS + inc
    OBJDIR.mkdir(parents=True, exist_ok=True)
    hdr_hash = _sha(hdrs, " ".join(flags))
    todo, objs = [], []
    for s in srcs:
        o = OBJDIR / ("rt_" + s.parent.name + "_" + s.stem + ".o")
        stamp = OBJDIR / ("rt_" + s.parent.name + "_" + s.stem + ".sha")
        want = _sha([s], hdr_hash)
        objs.append(o)
        if force or not o.exists() or not stamp.exists() or stamp.read_text() != want:
            todo.append((s, o, stamp, want))

    def one(item):
        s, o, stamp, want = item
        _run([CXX, *flags, "-c", s, "-o", o], verbose)
        stamp.write_text(want)

    if todo:
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
            list(ex.map(one, todo))
    out = _rt_path()
    link_stamp = LIBDIR / "_rt.sha"
    want = _sha(srcs + hdrs, " ".join(flags))
    if todo or force or not out.exists() or not link_stamp.exists() \
            or link_stamp.read_text() != want:
        _link_atomic([CXX, "-shared"], out, objs, ["-pthread", "-lrt", "-ldl"], verbose)
        link_stamp.write_text(want)
    return out


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_kernels(force=force, verbose=verbose)
    build_runtime(force=force, verbose=verbose)
    build_c_api(force=force, verbose=verbose)


if __name__ == "__main__":
    import argparse

    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ptxas", action="store_true", help="print registers/spills/smem per kernel")
    ap.add_argument("--only", choices=["kernels", "runtime", "c_api"], default=None)
    a = ap.parse_args()
    if a.only in (None, "kernels"):
        print(build_kernels(force=a.force or a.ptxas, verbose=a.verbose, ptxas_info=a.ptxas))
    if a.only in (None, "runtime"):
        print(build_runtime(force=a.force, verbose=a.verbose))
    if a.only in (None, "c_api"):
        print(build_c_api(force=a.force, verbose=a.verbose))
