"""Compile the kernel library for sm_100a with nvcc and return the path of the shared object.

The sources are plain CUDA with a C interface (no framework headers), so each file
compiles in seconds and the files compile in parallel.  The library is built in the
source tree (``csrc/_build``) so that a checkout carries it to wherever it runs; if
the tree is read-only the build goes to a per-user folder under the system's
temporary directory.  A hash of the sources and flags names the library, so a stale
build is never loaded.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import List, Optional

CSRC = os.path.dirname(os.path.abspath(__file__))
SOURCES = (
    "hx_elementwise.cu",
    "hx_gemm_simt.cu",
    "hx_gemm_tc.cu",
    "hx_attention.cu",
    "hx_attention_mma.cu",
    "hx_attention_tc.cu",
    "hx_sampling.cu",
)
HEADERS = ("hx_common.cuh", "hx_mma.cuh", "hx_tcgen05.cuh", "hx_no_alloc.h")
NVCC_FLAGS = (
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
    # kernel developers: more flags (for instance -D switches of a kernel under study); they
    # enter the library's name like the sources do
    *os.environ.get("HELIX_NVCC_FLAGS", "").split(),
)


def find_nvcc() -> str:
    candidates = [os.environ.get("HELIX_NVCC"), shutil.which("nvcc"),
                  os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                  "/usr/local/cuda/bin/nvcc"]
    for candidate in candidates:
        if candidate and os.path.isfile(candidate) and os.access(candidate, os.X_OK):
            return candidate
    raise RuntimeError("nvcc was not found (set HELIX_NVCC or CUDA_HOME); the engine has no "
                       "fallback without its CUDA kernels")


def source_hash(extra: str = "") -> str:
    digest = hashlib.sha256()
    for name in (*SOURCES, *HEADERS):
        with open(os.path.join(CSRC, name), "rb") as source:
            digest.update(name.encode())
            digest.update(source.read())
    digest.update(" ".join(NVCC_FLAGS).encode())
    digest.update(extra.encode())
    return digest.hexdigest()[:16]


def _writable_build_dir() -> str:
    preferred = os.path.join(CSRC, "_build")
    try:
        os.makedirs(preferred, exist_ok=True)
        probe = os.path.join(preferred, f".probe{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return preferred
    except OSError:
        fallback = os.path.join(tempfile.gettempdir(), f"helix_runtime_b200_{os.getuid()}")
        os.makedirs(fallback, exist_ok=True)
        return fallback


def library_path(build_dir: Optional[str] = None) -> str:
    return os.path.join(build_dir or _writable_build_dir(), f"libhelix_b200_{source_hash()}.so")


def _run(command: List[str]) -> None:
    result = subprocess.run(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if result.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(command) + "\n" + result.stdout)


def build(verbose: bool = True, force: bool = False) -> str:
    """Build if needed; print a line now and then while compiling."""
    build_dir = _writable_build_dir()
    target = library_path(build_dir)
    if os.path.exists(target) and not force:
        return target
    nvcc = find_nvcc()
    started = time.time()
    stop = threading.Event()

    def say(message: str) -> None:
        if verbose:
            print(f"[helix_runtime_b200] {message}", file=sys.stderr, flush=True)

    def heartbeat() -> None:
        while not stop.wait(10.0):
            say(f"still compiling CUDA kernels for sm_100a ({time.time() - started:.0f} s)")

    say(f"compiling {len(SOURCES)} CUDA files for sm_100a into {build_dir} (first use only)")
    thread = threading.Thread(target=heartbeat, daemon=True)
    thread.start()
    tag = f"{os.getpid()}_{source_hash()}"
    objects = [os.path.join(build_dir, f"{os.path.splitext(name)[0]}_{tag}.o") for name in SOURCES]
    try:
        with ThreadPoolExecutor(max_workers=min(len(SOURCES), os.cpu_count() or 1)) as pool:
            jobs = [pool.submit(_run, [nvcc, *NVCC_FLAGS, "-I", CSRC, "-c",
                                       os.path.join(CSRC, name), "-o", obj])
                    for name, obj in zip(SOURCES, objects)]
            for job in jobs:
                job.result()
        partial = target + f".{os.getpid()}.tmp"
        _run([nvcc, "-shared", "-o", partial, *objects, "-cudart", "static"])
        os.replace(partial, target)
        for name in os.listdir(build_dir):      # libraries of older sources
            if name.startswith("libhelix_b200_") and name.endswith(".so") and \
                    os.path.join(build_dir, name) != target and \
                    not os.environ.get("HELIX_NVCC_FLAGS"):
                try:
                    os.remove(os.path.join(build_dir, name))
                except OSError:
                    pass
    finally:
        stop.set()
        for obj in objects:
            if os.path.exists(obj):
                os.remove(obj)
    say(f"kernel library ready after {time.time() - started:.0f} s: {target}")
    return target


# ------------------------------------------------------------------ host library
#
# Host-only C++ (the native model file reader): compiled with the C++ compiler alone, so that
# everything that needs no GPU also needs no CUDA toolkit.

HOST_DIR = os.path.join(CSRC, "host")
HOST_SOURCES = ("hx_model_file.cpp",)
HOST_HEADERS = ("hx_model_file.h",)
HOST_FLAGS = ("-O2", "-std=c++17", "-fPIC", "-shared", "-pthread", "-fvisibility=default")


def _host_hash() -> str:
    digest = hashlib.sha256()
    for name in (*HOST_SOURCES, *HOST_HEADERS):
        with open(os.path.join(HOST_DIR, name), "rb") as source:
            digest.update(name.encode())
            digest.update(source.read())
    digest.update(" ".join(HOST_FLAGS).encode())
    return digest.hexdigest()[:16]


def find_cxx() -> str:
    for candidate in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"),
                      shutil.which("clang++")):
        if candidate and shutil.which(candidate):
            return shutil.which(candidate)
    raise RuntimeError("no C++ compiler was found (set CXX); the native model file reader "
                       "needs one")


def build_host(force: bool = False) -> str:
    """Build the host library if needed and return its path."""
    build_dir = _writable_build_dir()
    target = os.path.join(build_dir, f"libhelix_host_{_host_hash()}.so")
    if os.path.exists(target) and not force:
        return target
    partial = target + f".{os.getpid()}.tmp"
    _run([find_cxx(), *HOST_FLAGS, "-I", HOST_DIR,
          *(os.path.join(HOST_DIR, name) for name in HOST_SOURCES), "-o", partial])
    os.replace(partial, target)
    for name in os.listdir(build_dir):
        if name.startswith("libhelix_host_") and name.endswith(".so") and \
                os.path.join(build_dir, name) != target:
            try:
                os.remove(os.path.join(build_dir, name))
            except OSError:
                pass
    return target


# ------------------------------------------------------- the engine for C and C++ callers
#
# include/helix_b200/engine.h over an embedded interpreter: compiled against the headers and
# the shared library of the Python that runs this build, under a fixed name so that a C++
# program can link it (-lhelix_b200_engine).

ENGINE_API_SOURCE = os.path.join(HOST_DIR, "hx_engine_api.cpp")
ENGINE_API_HEADER = os.path.join(os.path.dirname(os.path.dirname(CSRC)), "include", "helix_b200",
                                 "engine.h")


def build_engine_api(force: bool = False) -> str:
    """Build ``libhelix_b200_engine.so`` if its sources changed and return its path."""
    import sysconfig
    build_dir = _writable_build_dir()
    target = os.path.join(build_dir, "libhelix_b200_engine.so")
    stamp = target + ".sources"
    digest = hashlib.sha256()
    for path in (ENGINE_API_SOURCE, ENGINE_API_HEADER):
        with open(path, "rb") as source:
            digest.update(source.read())
    digest.update(sys.version.encode())
    wanted = digest.hexdigest()
    if os.path.exists(target) and not force:
        try:
            with open(stamp, "r") as source:
                if source.read().strip() == wanted:
                    return target
        except OSError:
            pass
    include = sysconfig.get_config_var("INCLUDEPY")
    library_dir = sysconfig.get_config_var("LIBDIR")
    version = sysconfig.get_config_var("LDVERSION") or sysconfig.get_python_version()
    if not include or not os.path.exists(os.path.join(include, "Python.h")):
        raise RuntimeError("the C and C++ interface of the engine needs Python's development "
                           f"headers (Python.h not found in {include})")
    partial = target + f".{os.getpid()}.tmp"
    _run([find_cxx(), "-O2", "-std=c++17", "-fPIC", "-shared", "-pthread", f"-I{include}",
          ENGINE_API_SOURCE, "-o", partial, f"-L{library_dir}", f"-lpython{version}", "-ldl",
          f"-Wl,-rpath,{library_dir}"])
    os.replace(partial, target)
    with open(stamp, "w") as output:
        output.write(wanted)
    return target


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
    print(build_host(force="--force" in sys.argv))
    print(build_engine_api(force="--force" in sys.argv))
