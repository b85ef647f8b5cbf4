"""Build recipe for libwholegraph.so (sm_100a only).

Compiles every translation unit under csrc/ with nvcc and links one shared object next to
this file.  Objects are cached under csrc/build/ and rebuilt when a source or header is newer.
Run as a script or call build().
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
OBJ_DIR = os.path.join(CSRC, "build")
LIB_PATH = os.path.join(HERE, "libwholegraph.so")

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC,-Wall",
          "-I", INCLUDE, "-I", CSRC]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; the library has no CPU build")
    return nvcc


def _sources() -> list[str]:
    out = []
    for root, _, files in os.walk(CSRC):
        if os.path.abspath(root).startswith(OBJ_DIR):
            continue
        for f in sorted(files):
            if f.endswith((".cu", ".cpp")):
                out.append(os.path.join(root, f))
    return sorted(out)


def _newest_header() -> float:
    newest = 0.0
    for base in (CSRC, INCLUDE):
        for root, _, files in os.walk(base):
            for f in files:
                if f.endswith((".h", ".hpp", ".cuh")):
                    newest = max(newest, os.path.getmtime(os.path.join(root, f)))
    return newest


def _compile(src: str, obj: str, verbose: bool) -> None:
    cmd = [_nvcc(), *COMMON, *ARCH_FLAGS, "-x", "cu", "-c", src, "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    if verbose and res.stderr:
        sys.stderr.write(res.stderr)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile and link libwholegraph.so; returns its path."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    hdr_time = max(_newest_header(), os.path.getmtime(__file__))
    jobs, objs = [], []
    for src in _sources():
        rel = os.path.relpath(src, CSRC).replace(os.sep, "__")
        obj = os.path.join(OBJ_DIR, rel + ".o")
        objs.append(obj)
        stale = force or not os.path.exists(obj) or \
            os.path.getmtime(obj) < max(os.path.getmtime(src), hdr_time)
        if stale:
            jobs.append((src, obj))
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            for fut in [pool.submit(_compile, s, o, verbose) for s, o in jobs]:
                fut.result()
    if jobs or not os.path.exists(LIB_PATH):
        _link(objs, LIB_PATH + ".tmp", [])
        # Second spelling of the C API: the project this library's interface descends from named
        # its functions wholememory_*, and binaries built against those names still exist.  Every
        # exported wholegraph_* function gets a wholememory_* twin at the same address.
        aliases = [f"--defsym=wholememory_{name[len('wholegraph_'):]}={name}" for name in _exported(LIB_PATH + ".tmp")
                   if name.startswith("wholegraph_") and not name.startswith("wholegraph_b200_")]
        os.unlink(LIB_PATH + ".tmp")
        _link(objs, LIB_PATH, aliases)
    return LIB_PATH


def _link(objs: list[str], out: str, linker_flags: list[str]) -> None:
    cmd = [_nvcc(), "-shared", *ARCH_FLAGS, "-o", out, *objs, "-ldl", "-lpthread", "-lrt"]
    for flag in linker_flags:
        cmd += ["-Xlinker", flag]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")


def _exported(lib: str) -> list[str]:
    """Names of the functions a shared object defines and exports."""
    res = subprocess.run(["nm", "-D", "--defined-only", lib], capture_output=True, text=True, check=True)
    return [parts[2] for parts in (line.split() for line in res.stdout.splitlines())
            if len(parts) == 3 and parts[1] == "T"]


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
