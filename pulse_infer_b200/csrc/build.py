"""Compiling the CUDA sources into shared libraries, in-tree, at first use.

Each ``.cu`` file becomes one library with plain C entry points (loaded with ctypes; no Python or
torch headers are involved, so a file compiles in seconds).  Libraries are cached under
``csrc/_build/`` by a hash of their source, the shared header and the flags.  The attention kernel
is specialised per head size, so a model compiles only what it needs; progress lines are printed
while nvcc runs.  If the package folder cannot be written, a per-user folder in the temporary
directory is used instead.
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

CSRC_DIR = os.path.dirname(os.path.abspath(__file__))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-lineinfo", "-std=c++17", "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

# library name -> source file
SOURCES = {
    "elementwise": "elementwise.cu",
    "gemm_f32": "gemm_f32.cu",
    "gemm_small_m": "gemm_small_m.cu",
    "gemm_tcgen05": "gemm_tcgen05.cu",
    "attention_simple": "attention_simple.cu",
    "sampling": "sampling.cu",
}
ATTENTION_MMA_SOURCE = "attention_mma.cu"
ATTENTION_TCGEN05_SOURCE = "attention_tcgen05.cu"
HEADERS = ["common.cuh", "attention_noalloc.h"]

_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for cand in (os.environ.get("PULSE_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (looked at $PULSE_NVCC, PATH and /usr/local/cuda/bin); "
                     "the CUDA kernels cannot be built and there is no fallback")


def build_dir() -> str:
    override = os.environ.get("PULSE_BUILD_DIR")
    candidates = [override] if override else []
    candidates.append(os.path.join(CSRC_DIR, "_build"))
    candidates.append(os.path.join(tempfile.gettempdir(), f"pulse_infer_b200_build_{os.getuid()}"))
    for path in candidates:
        try:
            os.makedirs(path, exist_ok=True)
            probe = os.path.join(path, f".write_probe_{os.getpid()}")
            with open(probe, "w") as fh:
                fh.write("x")
            os.remove(probe)
            return path
        except OSError:
            continue
    raise BuildError(f"no writable build folder among {candidates}")


def _extra_flags() -> list[str]:
    """Extra nvcc flags from $PULSE_NVCC_FLAGS (experiments); they are part of the cache key."""
    return os.environ.get("PULSE_NVCC_FLAGS", "").split()


def _digest(source: str, defines: list[str]) -> str:
    h = hashlib.sha256()
    for name in [source] + HEADERS:
        with open(os.path.join(CSRC_DIR, name), "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(ARCH_FLAGS + BASE_FLAGS + defines + _extra_flags()).encode())
    return h.hexdigest()[:16]


def _compile(source: str, out_path: str, defines: list[str], label: str) -> None:
    nvcc = find_nvcc()
    tmp_out = f"{out_path}.{os.getpid()}.tmp"
    cmd = [nvcc] + ARCH_FLAGS + BASE_FLAGS + defines + _extra_flags() + ["-o", tmp_out, os.path.join(CSRC_DIR, source)]
    print(f"[pulse_infer_b200] compiling {label} for sm_100a ...", file=sys.stderr, flush=True)
    t0 = time.time()
    env = dict(os.environ)
    env.setdefault("TMPDIR", os.path.dirname(out_path))  # nvcc scratch files; HOME may be unusable
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    done = threading.Event()

    def heartbeat():
        while not done.wait(10.0):
            print(f"[pulse_infer_b200]   ... still compiling {label} ({time.time() - t0:.0f} s)",
                  file=sys.stderr, flush=True)
    beat = threading.Thread(target=heartbeat, daemon=True)
    beat.start()
    output, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        if os.path.exists(tmp_out):
            os.remove(tmp_out)
        raise BuildError(f"nvcc failed for {label}:\n{' '.join(cmd)}\n{output}")
    os.replace(tmp_out, out_path)
    print(f"[pulse_infer_b200] compiled {label} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)


def library_path(name: str, head_dim: int | None = None) -> str:
    """Path of the built library, compiling it first if it is missing or stale."""
    if name == "attention_mma":
        if head_dim is None or head_dim % 16 != 0 or not (16 <= head_dim <= 256):
            raise BuildError(f"the tensor-core attention kernel needs a head size that is a multiple of 16 "
                             f"in 16..256, got {head_dim}")
        source, defines, label = ATTENTION_MMA_SOURCE, [f"-DPI_HEAD_DIM={head_dim}"], f"attention (head size {head_dim})"
        stem = f"attention_mma_d{head_dim}"
    elif name == "attention_tcgen05":
        if head_dim not in (64, 128):
            raise BuildError(f"the tcgen05 attention kernel takes head sizes 64 and 128, got {head_dim}")
        source, defines, label = ATTENTION_TCGEN05_SOURCE, [f"-DPI_HEAD_DIM={head_dim}"], f"tcgen05 attention (head size {head_dim})"
        stem = f"attention_tcgen05_d{head_dim}"
    elif name in SOURCES:
        source, defines, label, stem = SOURCES[name], [], name, name
    else:
        raise BuildError(f"unknown kernel library '{name}'")
    out_path = os.path.join(build_dir(), f"libpulse_{stem}-{_digest(source, defines)}.so")
    if not os.path.isfile(out_path):
        with _lock:
            if not os.path.isfile(out_path):
                _compile(source, out_path, defines, label)
    return out_path


def build_all(head_dims=(16, 32, 48, 64, 128)) -> list[str]:
    """Compile every library (attention for the given head sizes); used by the build check."""
    paths = [library_path(name) for name in SOURCES]
    paths += [library_path("attention_mma", d) for d in head_dims]
    paths += [library_path("attention_tcgen05", d) for d in head_dims if d in (64, 128)]
    return paths
