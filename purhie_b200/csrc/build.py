"""Compiling the CUDA sources for sm_100a and loading the libraries.

Each *library* is a handful of ``.cu`` files compiled by ``nvcc`` into one shared object next to the
sources (``_build/``), without any Python or torch header, and loaded with ``ctypes``.  A library is
compiled the first time something needs it, so a float32 run compiles the plain kernels only; while it
compiles, a line is printed now and then.  If the package folder cannot be written, a per-user folder
under the temporary directory is used.  A missing compiler or a failed compile raises: there is no
fallback that computes on the host.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import Dict, List, Optional

CSRC = os.path.dirname(os.path.abspath(__file__))

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

# library name -> (sources, extra nvcc flags, extra link flags)
LIBRARIES: Dict[str, dict] = {
    "core": {
        "sources": ["elementwise.cu", "qk_norm_rope.cu", "attention_generic.cu", "gemm_simple.cu", "sampling.cu",
                    "random_fill.cu", "core_lib.cu"],
        "deps": ["../weights/random.h"],
        "flags": [],
        "link": [],
    },
    "flash": {
        "sources": ["attention_flash.cu", "attention_decode_bulk.cu", "attention_prefill_tc5.cu"],
        "deps": ["attention_mma.cuh", "mbarrier.cuh"],
        "flags": [],
        "link": [],
    },
    "gemm100": {
        "sources": ["gemm_tcgen05.cu"],
        "flags": [],
        "link": [],
    },
    # the host library: configuration, weights, parts, cache manager, step function, scheduler, samplers and the C
    # API (api/inference.h); it opens the kernel libraries above by need, from the folder it is loaded from
    "qengine": {
        "sources": ["../host/device.cpp", "../config/config.cpp", "../weights/safetensors.cpp", "../weights/weights.cpp",
                    "../parts/registry.cpp", "../parts/linear.cpp", "../parts/norm.cpp", "../parts/rotary.cpp",
                    "../parts/attention.cpp", "../parts/feed_forward.cpp", "../parts/embedding.cpp", "../parts/block.cpp",
                    "../parts/model.cpp", "../cache/cache.cpp", "../sampling/sampler.cpp", "../engine/engine.cpp",
                    "../engine/scheduler.cpp", "../api/capi.cpp", "../api/capi_generate.cpp", "../api/test_hooks.cpp",
                    "../api/test_hooks_host.cpp", "../api/test_hooks_parts.cpp"],
        "deps": ["../host/common.h", "../host/json.h", "../host/device.h", "../config/config.h", "../weights/safetensors.h",
                 "../weights/weights.h", "../weights/random.h", "../parts/parts.h", "../parts/linear.h", "../parts/model.h",
                 "../cache/cache.h", "../sampling/sampler.h", "../engine/engine.h", "../engine/scheduler.h",
                 "../api/inference.h", "../api/capi_internal.h"],
        "flags": ["-Xcompiler", "-ffp-contract=off"],
        "link": ["-ldl", "-lpthread"],
        "file_name": "libqengine.so",
    },
    # decode attention with its scratch in a fixed device array, for callers that cannot allocate
    "decode_static": {
        "sources": ["attention_decode_static.cu"],
        "deps": ["attention_flash.cu", "attention_decode_static.h", "attention_mma.cuh"],
        "flags": [],
        "link": [],
    },
}

_HEADERS = ["common.cuh"]
_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _log(msg: str) -> None:
    print(f"[purhie_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    cands = []
    for env in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(env):
            cands.append(os.path.join(os.environ[env], "bin", "nvcc"))
    cands.append("/usr/local/cuda/bin/nvcc")
    which = shutil.which("nvcc")
    if which:
        cands.append(which)
    for c in cands:
        if os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise BuildError("nvcc not found (looked in $CUDA_HOME/bin, /usr/local/cuda/bin and PATH); the CUDA kernels "
                     "cannot be compiled and there is no other implementation")


def build_dir() -> str:
    """Where objects and libraries go: ``csrc/_build`` when writable, else a per-user temporary folder."""
    d = os.environ.get("PURHIE_B200_BUILD_DIR") or os.path.join(CSRC, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.unlink(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"purhie_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _digest(paths: List[str], flags: List[str]) -> str:
    h = hashlib.sha256()
    for p in paths:
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:16]


def _run_with_heartbeat(cmds: List[List[str]], what: str) -> None:
    """Run the commands in parallel; print a line every few seconds until all have ended."""
    logs = [tempfile.TemporaryFile(mode="w+") for _ in cmds]
    procs = [subprocess.Popen(c, stdout=log, stderr=subprocess.STDOUT, text=True) for c, log in zip(cmds, logs)]
    start = last = time.time()
    while any(p.poll() is None for p in procs):
        if time.time() - last > 5:
            last = time.time()
            _log(f"still compiling {what} ({int(last - start)} s)")
        time.sleep(0.05)
    for c, p, log in zip(cmds, procs, logs):
        log.seek(0)
        out = log.read()
        log.close()
        if p.returncode != 0:
            raise BuildError(f"command failed ({p.returncode}): {' '.join(c)}\n{out}")


def library_file(name: str) -> str:
    return LIBRARIES[name].get("file_name", f"libpurhie_{name}.so")


def library_path(name: str) -> str:
    return os.path.join(build_dir(), library_file(name))


def build_library(name: str, verbose: bool = True) -> str:
    """Compile library ``name`` if its sources changed since the last build; return the path of the .so."""
    spec = LIBRARIES[name]
    out_dir = build_dir()
    srcs = [os.path.join(CSRC, s) for s in spec["sources"]]
    hdrs = [os.path.join(CSRC, h) for h in _HEADERS + spec.get("deps", [])]
    flags = ARCH_FLAGS + COMMON_FLAGS + spec["flags"]
    so = os.path.join(out_dir, library_file(name))
    stamp = so + ".stamp"
    digest = _digest(srcs + hdrs, flags + spec["link"])
    if os.path.exists(so) and os.path.exists(stamp):
        with open(stamp) as f:
            if f.read().strip() == digest:
                return so
    nvcc = find_nvcc()
    if verbose:
        what = "host library" if name == "qengine" else "kernels for sm_100a"
        _log(f"compiling the '{name}' {what} ({len(srcs)} files) into {out_dir}")
    t0 = time.time()
    objs, cmds = [], []
    for s in srcs:
        o = os.path.join(out_dir, f"{name}_{os.path.basename(s)}.{os.getpid()}.o")
        s = os.path.normpath(s)
        objs.append(o)
        cmds.append([nvcc] + flags + ["-I", CSRC, "-c", s, "-o", o])
    try:
        _run_with_heartbeat(cmds, f"'{name}'")
        tmp_so = f"{so}.{os.getpid()}.tmp"
        _run_with_heartbeat([[nvcc] + ARCH_FLAGS + ["-shared", "-o", tmp_so] + objs + spec["link"]], f"'{name}' (link)")
        os.replace(tmp_so, so)
        with open(stamp + f".{os.getpid()}", "w") as f:
            f.write(digest)
        os.replace(stamp + f".{os.getpid()}", stamp)
    finally:
        for o in objs:
            if os.path.exists(o):
                os.unlink(o)
    if verbose:
        _log(f"'{name}' ready ({time.time() - t0:.0f} s)")
    return so


def load_library(name: str) -> ctypes.CDLL:
    """The loaded library ``name``, compiled first if need be."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            lib = ctypes.CDLL(build_library(name))
            _loaded[name] = lib
        return lib


def build_all(verbose: bool = True) -> List[str]:
    return [build_library(n, verbose) for n in LIBRARIES]


def build_plugin(source: str, out_dir: str, verbose: bool = True) -> str:
    """Compile ``source`` (a .cu or .cpp file of parts that includes ``purhie_b200/parts/parts.h``) for sm_100a into a
    shared object in ``out_dir``, linked against the host library; returns its path.  Open it with
    :func:`purhie_b200.parts.load_plugin`: its ``qe_plugin_init`` registers what it brings."""
    host = build_library("qengine", verbose)
    nvcc = find_nvcc()
    os.makedirs(out_dir, exist_ok=True)
    so = os.path.join(out_dir, "lib" + os.path.splitext(os.path.basename(source))[0] + ".so")
    root = os.path.dirname(os.path.dirname(CSRC))                    # the folder that holds the purhie_b200 package
    lib_dir = os.path.dirname(host)
    cmd = [nvcc] + ARCH_FLAGS + ["-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-shared", "-I", root, "-I", CSRC, source, "-o", so,
                                 "-L", lib_dir, "-lqengine", "-Xlinker", "-rpath", "-Xlinker", lib_dir]
    if verbose:
        _log(f"compiling the plugin {os.path.basename(source)} into {out_dir}")
    _run_with_heartbeat([cmd], os.path.basename(source))
    return so
