"""In-tree build of the native libraries (nvcc, sm_100a only).

  lib/libscrapgpu_sm100.so        the CUDA compute library (C ABI: include/scrapgpu_sm100.h)
  lib/libscrapgpu_cuda_sm100.so   the ScrapGpuLibrary backend plugin (vtable host layer); it is compiled
                                  against the reference's public headers, so it is (re)built only where a
                                  ScrapGpuLibrary checkout is present (SCRAPGPU_REFERENCE_DIR) and otherwise
                                  used as prebuilt.

Objects go to build/ (ignored by git); a target is rebuilt when any of its inputs is newer.
"""
from __future__ import annotations

import os
import shutil
import subprocess
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
BACKEND = os.path.join(PKG, "backend")
LIBDIR = os.path.join(PKG, "lib")
OBJDIR = os.path.join(ROOT, "build", "obj")
INCLUDE = os.path.join(ROOT, "include")
REFERENCE_DIR = os.environ.get("SCRAPGPU_REFERENCE_DIR", "/root/reference")

SM100_SO = os.path.join(LIBDIR, "libscrapgpu_sm100.so")
PLUGIN_SO = os.path.join(LIBDIR, "libscrapgpu_cuda_sm100.so")

NVCC_FLAGS = ["-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", f"-I{INCLUDE}", f"-I{CSRC}"]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _newer(target: str, inputs) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(i) > t for i in inputs if os.path.exists(i))


def _run(cmd) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)


def build_sm100(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIBDIR, exist_ok=True)
    os.makedirs(OBJDIR, exist_ok=True)
    # several ranks of one job may arrive here at once: one of them builds, the others wait and find the result current
    import fcntl
    with open(os.path.join(OBJDIR, ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            return _build_sm100_locked(force, verbose)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def _build_sm100_locked(force: bool, verbose: bool) -> str:
    srcs = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(INCLUDE, "scrapgpu_sm100.h"))
    nvcc = _nvcc()
    jobs = []
    objs = []
    for s in srcs:
        src = os.path.join(CSRC, s)
        obj = os.path.join(OBJDIR, s[:-3] + ".o")
        objs.append(obj)
        if force or _newer(obj, [src] + headers):
            jobs.append([nvcc] + NVCC_FLAGS + ["-c", src, "-o", obj])
    if jobs:
        if verbose:
            print(f"[build] compiling {len(jobs)} CUDA sources for sm_100a")
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(_run, jobs))
    if force or jobs or _newer(SM100_SO, objs):
        tmp = SM100_SO + ".tmp.%d" % os.getpid()
        _run([nvcc, "-shared", "-o", tmp] + objs)
        os.replace(tmp, SM100_SO)   # readers never see a half-written library
    return SM100_SO


def reference_headers() -> str | None:
    inc = os.path.join(REFERENCE_DIR, "include")
    return inc if os.path.exists(os.path.join(inc, "scrapgpu", "backend.h")) else None


def build_plugin(force: bool = False, verbose: bool = False) -> str | None:
    """The backend plugin; None when it cannot be built here and no prebuilt copy exists."""
    if not os.path.isdir(BACKEND):
        return PLUGIN_SO if os.path.exists(PLUGIN_SO) else None
    srcs = [os.path.join(BACKEND, f) for f in sorted(os.listdir(BACKEND)) if f.endswith(".cpp")]
    inc = reference_headers()
    if inc is None or not srcs:
        return PLUGIN_SO if os.path.exists(PLUGIN_SO) else None
    deps = srcs + [os.path.join(BACKEND, f) for f in os.listdir(BACKEND) if f.endswith(".h")]
    deps += [os.path.join(INCLUDE, "scrapgpu_sm100.h"), SM100_SO]
    deps += [os.path.join(INCLUDE, "scrapgpu", f) for f in os.listdir(os.path.join(INCLUDE, "scrapgpu"))] \
        if os.path.isdir(os.path.join(INCLUDE, "scrapgpu")) else []
    if force or _newer(PLUGIN_SO, deps):
        if verbose:
            print("[build] compiling the cuda_sm100 backend plugin")
        _run(["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall", "-Wextra",
              f"-I{inc}", f"-I{INCLUDE}", f"-I{BACKEND}"] + srcs +
             ["-o", PLUGIN_SO, f"-L{LIBDIR}", "-lscrapgpu_sm100", "-Wl,-rpath,$ORIGIN", "-lpthread"])
    return PLUGIN_SO


def build_all(force: bool = False, verbose: bool = False) -> dict:
    out = {"sm100": build_sm100(force, verbose)}
    out["plugin"] = build_plugin(force, verbose)
    return out


if __name__ == "__main__":
    print(build_all(verbose=True))
