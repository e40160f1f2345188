"""Compiling the CUDA sources for sm_100a and loading them.

There are two kinds of library: `core` (norms, embedding, rotary encoding and
cache write, the 32-bit product, the skinny bfloat16 product, sampling) and one
`attention` library per head size, compiled with that size as a constant.  A
library is compiled the first time it is asked for, so a process compiles what
its model needs and nothing else; the file name carries a hash of the sources
and flags, so a stale library is never loaded.  The kernels are plain C entry
points (no Python or torch headers), called through ctypes.

While nvcc runs, a line goes to stderr at the start and every few seconds, so
that a first call in a fresh checkout does not look hung.
"""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor

_HERE = os.path.dirname(os.path.abspath(__file__))

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
# no fast-math: expf, tanhf and sincosf keep their accurate forms
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

CORE_SOURCES = ["elementwise.cu", "gemm_f32.cu", "gemv_bf16.cu", "gemm_tc05.cu", "sampling.cu"]
ATTENTION_SOURCES = ["attention.cu", "attention_prefill_mma.cu", "attention_prefill_tc05.cu", "attention_no_alloc.cu"]
HEADERS = ["common.cuh", "attention_no_alloc.h", "attention_prefill_tiles.cuh"]


class BuildError(RuntimeError):
    """nvcc is missing or a source did not compile."""


def _say(msg: str) -> None:
    print(f"[janis_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("JANIS_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
                 os.path.join(os.environ.get("CUDA_PATH", ""), "bin", "nvcc") if os.environ.get("CUDA_PATH") else None,
                 shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at $JANIS_NVCC, $CUDA_HOME/bin, $PATH, /usr/local/cuda/bin); "
                     "the CUDA kernels of janis_b200 cannot be compiled")


def build_dir() -> str:
    """In the source tree when it can be written, else a per-user folder under the temp dir."""
    env = os.environ.get("JANIS_BUILD_DIR")
    cands = [env] if env else [os.path.join(_HERE, "_build"),
                               os.path.join(tempfile.gettempdir(), f"janis_b200_build_{os.getuid()}")]
    for d in cands:
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".probe.{os.getpid()}")
            with open(probe, "w"):
                pass
            os.unlink(probe)
            return d
        except OSError:
            continue
    raise BuildError(f"no writable build folder among {cands}")


def _digest(sources, defines) -> str:
    h = hashlib.sha256()
    for name in list(sources) + HEADERS:
        with open(os.path.join(_HERE, name), "rb") as f:
            h.update(name.encode())
            h.update(f.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + sorted(defines)).encode())
    return h.hexdigest()[:16]


def _run(cmd, what):
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise BuildError(f"{what} failed (exit {p.returncode}):\n$ {' '.join(cmd)}\n{p.stdout}")
    return p.stdout


def compile_library(name: str, sources, defines=(), verbose_ptxas: bool = False) -> str:
    """Path of lib<name>.<hash>.so, compiled now if it is not there yet."""
    defines = list(defines)
    out_dir = build_dir()
    tag = _digest(sources, defines)
    so = os.path.join(out_dir, f"lib{name}.{tag}.so")
    if os.path.exists(so):
        return so
    lock_path = os.path.join(out_dir, f".{name}.lock")
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if os.path.exists(so):          # another process built it while we waited
                return so
            nvcc = find_nvcc()
            t0 = time.time()
            _say(f"compiling {name} for sm_100a ({', '.join(sources)}) ...")
            done = threading.Event()

            def heartbeat():
                while not done.wait(8.0):
                    _say(f"still compiling {name} ({time.time() - t0:.0f} s)")

            hb = threading.Thread(target=heartbeat, daemon=True)
            hb.start()
            try:
                objs = []

                def one(src):
                    obj = os.path.join(out_dir, f"{name}.{tag}.{os.path.splitext(src)[0]}.o")
                    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, *[f"-D{d}" for d in defines], "-I", _HERE,
                           "-c", os.path.join(_HERE, src), "-o", obj]
                    if verbose_ptxas:
                        cmd[1:1] = ["-Xptxas", "-v"]
                    log = _run(cmd, f"nvcc {src}")
                    if verbose_ptxas and log.strip():
                        _say(log)
                    return obj

                with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
                    objs = list(pool.map(one, sources))
                tmp = f"{so}.tmp.{os.getpid()}"
                # the CUDA runtime is linked statically (nvcc's default): nothing to find at load time
                _run([nvcc, *ARCH_FLAGS, "-shared", "-o", tmp, *objs], f"link {name}")
                os.replace(tmp, so)
                for o in objs:
                    try:
                        os.unlink(o)
                    except OSError:
                        pass
            finally:
                done.set()
            _say(f"compiled {name} in {time.time() - t0:.0f} s -> {so}")
            # libraries of older sources are of no use any more
            for f in os.listdir(out_dir):
                if f.startswith(f"lib{name}.") and f.endswith(".so") and f != os.path.basename(so):
                    try:
                        os.unlink(os.path.join(out_dir, f))
                    except OSError:
                        pass
            return so
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


_loaded: dict[str, ctypes.CDLL] = {}


def _load(name: str, sources, defines=()) -> ctypes.CDLL:
    if name not in _loaded:
        lib = ctypes.CDLL(compile_library(name, sources, defines))
        lib.janis_last_error.restype = ctypes.c_char_p
        _loaded[name] = lib
    return _loaded[name]


def core_library() -> ctypes.CDLL:
    extra = [d for d in os.environ.get("JANIS_CORE_DEFINES", "").split(",") if d]      # tuning experiments
    tag = "_" + "_".join(d.replace("=", "") for d in extra) if extra else ""
    return _load(f"janis_core{tag}", CORE_SOURCES, extra)


def attention_library(head_dim: int) -> ctypes.CDLL:
    if head_dim % 16 or not 16 <= head_dim <= 512:
        raise BuildError(f"attention kernels take head sizes that are multiples of 16 from 16 to 512, "
                         f"found {head_dim}")
    extra = [d for d in os.environ.get("JANIS_ATTN_DEFINES", "").split(",") if d]      # tuning experiments
    tag = "_" + "_".join(d.replace("=", "") for d in extra) if extra else ""
    return _load(f"janis_attn_hd{head_dim}{tag}", ATTENTION_SOURCES, [f"JANIS_HEAD_DIM={head_dim}", *extra])


def build_all(head_dims=(16, 32, 64, 128, 256), verbose_ptxas: bool = False) -> list[str]:
    """Compile the core library and the attention library of each given head size."""
    paths = [compile_library("janis_core", CORE_SOURCES, verbose_ptxas=verbose_ptxas)]
    for hd in head_dims:
        paths.append(compile_library(f"janis_attn_hd{hd}", ATTENTION_SOURCES, [f"JANIS_HEAD_DIM={hd}"],
                                     verbose_ptxas=verbose_ptxas))
    return paths
