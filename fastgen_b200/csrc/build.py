"""In-tree builder of the CUDA libraries (sm_100a) and their ctypes loader.

Libraries are plain shared objects with an ``extern "C"`` interface; they do
not link against Python or torch, so a build is a few seconds of ``nvcc``.
They are written to ``fastgen_b200/csrc/_build`` (or, when that folder cannot
be written, to ``$FASTGEN_B200_BUILD_DIR`` or a per-user temporary folder) and
rebuilt when a source, a header or a flag changed.  A library is compiled at
the first call that needs it; the attention library is compiled per head size,
so a model compiles only what it needs.

There is no fallback: if a library cannot be built or loaded, the caller gets
a ``RuntimeError`` that says why.
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
from pathlib import Path
from typing import Dict, Iterable, List, Sequence

CSRC = Path(__file__).resolve().parent

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC"]
# more flags for nvcc (say -DNAME=value for an experiment); they are part of a library's stamp
EXTRA_FLAGS = os.environ.get("FASTGEN_B200_NVCC_FLAGS", "").split()

CORE_SOURCES = [
    "errors.cu",
    "embedding.cu",
    "rmsnorm.cu",
    "rope_kv.cu",
    "silu_gate.cu",
    "gemm_f32.cu",
    "gemm_skinny.cu",
    "sampling.cu",
    "tensor_map.cu",
    "selftest.cu",
]

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


def _log(msg: str) -> None:
    print(f"[fastgen_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (
        os.environ.get("FASTGEN_B200_NVCC"),
        shutil.which("nvcc"),
        os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
        "/usr/local/cuda/bin/nvcc",
    ):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise RuntimeError(
        "nvcc was not found (looked at $FASTGEN_B200_NVCC, PATH, $CUDA_HOME/bin and "
        "/usr/local/cuda/bin); the CUDA kernels of fastgen_b200 cannot be built and "
        "there is no fallback path"
    )


def build_dir() -> Path:
    """The folder libraries are built into; the first of these that is writable."""
    candidates = []
    if os.environ.get("FASTGEN_B200_BUILD_DIR"):
        candidates.append(Path(os.environ["FASTGEN_B200_BUILD_DIR"]))
    candidates.append(CSRC / "_build")
    candidates.append(Path(tempfile.gettempdir()) / f"fastgen_b200_build_{os.getuid()}")
    for d in candidates:
        try:
            d.mkdir(parents=True, exist_ok=True)
            probe = d / f".probe_{os.getpid()}"
            probe.write_text("")
            probe.unlink()
            return d
        except OSError:
            continue
    raise RuntimeError(f"no writable build folder among {[str(c) for c in candidates]}")


def _headers() -> List[Path]:
    return sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))


def _digest(sources: Sequence[Path], flags: Sequence[str]) -> str:
    h = hashlib.sha256()
    for p in list(sources) + _headers():
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()


def _run(cmd: List[str], what: str) -> None:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"building {what} failed:\n$ {' '.join(cmd)}\n{proc.stdout}")


def _compile(name: str, sources: Sequence[str], defines: Iterable[str] = ()) -> Path:
    """Build ``lib<name>.so`` from ``sources`` unless an up-to-date one exists."""
    srcs = [CSRC / s for s in sources]
    flags = ARCH_FLAGS + COMMON_FLAGS + EXTRA_FLAGS + [f"-D{d}" for d in defines]
    digest = _digest(srcs, flags)
    # A library shipped beside the sources is used when it matches them, even
    # if this user cannot write there.
    for d in dict.fromkeys([CSRC / "_build", build_dir()]):
        lib, stamp = d / f"lib{name}.so", d / f"lib{name}.stamp"
        if lib.is_file() and stamp.is_file() and stamp.read_text().strip() == digest:
            return lib

    out_dir = build_dir()
    lib, stamp = out_dir / f"lib{name}.so", out_dir / f"lib{name}.stamp"
    nvcc = find_nvcc()
    with open(out_dir / f".{name}.lock", "w") as lock_file:
        fcntl.flock(lock_file, fcntl.LOCK_EX)
        try:
            if lib.is_file() and stamp.is_file() and stamp.read_text().strip() == digest:
                return lib  # another process built it meanwhile
            t0 = time.time()
            _log(f"compiling lib{name}.so for sm_100a ({len(srcs)} files) into {out_dir}")
            obj_dir = out_dir / f"obj_{name}"
            obj_dir.mkdir(exist_ok=True)
            done = []

            def one(src: Path) -> Path:
                obj = obj_dir / (src.stem + ".o")
                _run([nvcc, *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)], src.name)
                done.append(src.name)
                _log(f"  compiled {src.name} ({len(done)}/{len(srcs)}, {time.time() - t0:.0f}s)")
                return obj

            stop = threading.Event()

            def heartbeat() -> None:
                while not stop.wait(10.0):
                    _log(f"  still compiling lib{name}.so ({time.time() - t0:.0f}s)")

            beat = threading.Thread(target=heartbeat, daemon=True)
            beat.start()
            try:
                with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
                    objs = list(pool.map(one, srcs))
                tmp = out_dir / f"lib{name}.so.tmp{os.getpid()}"
                _run([nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp), *map(str, objs)], f"lib{name}.so")
                os.replace(tmp, lib)
                stamp.write_text(digest)
            finally:
                stop.set()
            _log(f"built lib{name}.so in {time.time() - t0:.0f}s")
        finally:
            fcntl.flock(lock_file, fcntl.LOCK_UN)
    return lib


def load(name: str, sources: Sequence[str], defines: Iterable[str] = ()) -> ctypes.CDLL:
    key = name
    with _lock:
        if key in _loaded:
            return _loaded[key]
        path = _compile(name, sources, defines)
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as e:
            raise RuntimeError(f"cannot load {path}: {e}") from None
        _loaded[key] = lib
        return lib


def core_library() -> ctypes.CDLL:
    return load("fg_core", CORE_SOURCES)


def attention_library(head_dim: int) -> ctypes.CDLL:
    if head_dim % 16 != 0 or not 16 <= head_dim <= 256:
        raise ValueError(
            f"head size {head_dim} is not supported: the attention kernels take "
            "multiples of 16 from 16 to 256"
        )
    return load(
        f"fg_attn_hd{head_dim}", ["attention.cu", "errors.cu"], [f"FG_HEAD_DIM={head_dim}"]
    )


def build_all(head_dims: Sequence[int] = (16, 32, 64, 128)) -> None:
    """Compile every library (used by the build check and before shipping)."""
    _compile("fg_core", CORE_SOURCES)
    for hd in head_dims:
        _compile(f"fg_attn_hd{hd}", ["attention.cu", "errors.cu"], [f"FG_HEAD_DIM={hd}"])
