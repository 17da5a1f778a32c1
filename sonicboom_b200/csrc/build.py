"""Builds the kernel library for sm_100a with nvcc and loads it with ctypes.

The library is plain `extern "C"` CUDA (no Python or torch headers), so a full build takes
well under a minute.  It is built at first use into `_build/` beside the sources when that
folder can be written, else into a per-user folder under the system's temporary directory;
a stamp of the sources and flags decides whether a build is current.  There is no other
implementation to fall back to: when the compiler is missing or the build fails, loading
raises with the compiler's output.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

SRC_DIR = Path(__file__).resolve().parent
LIB_NAME = "libsonicboom_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default"]


class BuildError(RuntimeError):
    pass


# Sources that are compiled once per parameter value into libraries of their own, not into the
# core library: {source: macro}.  The attention kernels are specialised by head size.
VARIANT_SOURCES = {"attn_mma.cu": "SB_HD"}
SHARED_SOURCES = ["error.cu"]            # linked into every library
HEAD_DIMS = tuple(range(16, 257, 16))    # head sizes the attention kernels are written for


def sources() -> list[Path]:
    """Sources of the core library."""
    return [p for p in sorted(SRC_DIR.glob("*.cu")) if p.name not in VARIANT_SOURCES]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).is_file():
            return cand
    raise BuildError("nvcc was not found (looked at $NVCC, PATH and /usr/local/cuda/bin); the "
                     "kernel library cannot be built and there is no other implementation")


def _stamp(srcs, defines=()) -> str:
    h = hashlib.sha256()
    for p in list(srcs) + sorted(SRC_DIR.glob("*.cuh")) + sorted(SRC_DIR.glob("*.h")):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + list(defines)).encode())
    return h.hexdigest()


def _build_dir() -> Path:
    in_tree = SRC_DIR / "_build"
    try:
        in_tree.mkdir(exist_ok=True)
        probe = in_tree / f".probe{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return in_tree
    except OSError:
        d = Path(tempfile.gettempdir()) / f"sonicboom_b200-{os.getuid()}"
        d.mkdir(parents=True, exist_ok=True)
        return d


def _say(msg: str) -> None:
    print(f"[sonicboom_b200] {msg}", file=sys.stderr, flush=True)


def _build_lib(lib_name: str, srcs, defines=(), force=False, verbose=True) -> Path:
    out_dir = _build_dir()
    lib, stamp_file = out_dir / lib_name, out_dir / (lib_name + ".stamp")
    stamp = _stamp(srcs, defines)
    if not force and lib.is_file() and stamp_file.is_file() and stamp_file.read_text() == stamp:
        return lib
    nvcc = _nvcc()
    t0 = time.time()
    if verbose:
        _say(f"compiling {lib_name} for sm_100a ({len(srcs)} CUDA files) into {out_dir}")
    tag = lib_name.replace(".so", "")

    def compile_one(src: Path):
        obj = out_dir / f"{tag}.{src.stem}.o"
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, *defines, "-I", str(SRC_DIR), "-c", str(src),
               "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose:
            _say(f"  {src.name}: {'ok' if r.returncode == 0 else 'FAILED'} ({time.time() - t0:.0f}s)")
        return src, obj, r

    objs = []
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
        for src, obj, r in pool.map(compile_one, srcs):
            if r.returncode != 0:
                raise BuildError(f"nvcc failed on {src.name}:\n{r.stdout}\n{r.stderr}")
            objs.append(str(obj))
    tmp_lib = out_dir / (lib_name + f".tmp{os.getpid()}")
    r = subprocess.run([nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp_lib), *objs],
                       capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"linking {lib_name} failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp_lib, lib)
    stamp_file.write_text(stamp)
    if verbose:
        _say(f"built {lib_name} in {time.time() - t0:.0f}s")
    return lib


def build(force: bool = False, verbose: bool = True) -> Path:
    """Compiles the core library (every .cu that is not a variant source)."""
    return _build_lib(LIB_NAME, sources(), (), force, verbose)


def build_attention(head_dim: int, force: bool = False, verbose: bool = True) -> Path:
    """Compiles the tensor-core attention kernels for one head size."""
    if head_dim not in HEAD_DIMS:
        raise BuildError(f"the tensor-core attention kernels take head sizes in steps of 16 up to "
                         f"{HEAD_DIMS[-1]}, not {head_dim}")
    srcs = [SRC_DIR / "attn_mma.cu"] + [SRC_DIR / s for s in SHARED_SOURCES]
    return _build_lib(f"libsonicboom_b200_attn_hd{head_dim}.so", srcs, (f"-DSB_HD={head_dim}",),
                      force, verbose)


def build_all(force: bool = False, verbose: bool = True) -> list[Path]:
    """Everything that can be compiled: the core library and attention for every head size."""
    libs = [build(force, verbose)]
    with ThreadPoolExecutor(max_workers=4) as pool:
        libs += list(pool.map(lambda hd: build_attention(hd, force, verbose), HEAD_DIMS))
    return libs


_LIBS: dict = {}


def _load(path: Path) -> ctypes.CDLL:
    try:
        return ctypes.CDLL(str(path))
    except OSError as e:
        raise BuildError(f"could not load {path}: {e}") from None


def load() -> ctypes.CDLL:
    """The loaded core library; builds it first when needed."""
    if "core" not in _LIBS:
        _LIBS["core"] = _load(build())
    return _LIBS["core"]


def load_attention(head_dim: int) -> ctypes.CDLL:
    """The loaded attention library of one head size; builds it first when needed."""
    key = ("attn", head_dim)
    if key not in _LIBS:
        _LIBS[key] = _load(build_attention(head_dim))
    return _LIBS[key]
