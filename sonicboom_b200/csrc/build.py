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


def sources() -> list[Path]:
    return sorted(SRC_DIR.glob("*.cu"))


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).is_file():
            return cand
    raise BuildError("nvcc was not found (looked at $NVCC, PATH and /usr/local/cuda/bin); the "
                     "kernel library cannot be built and there is no other implementation")


def _stamp() -> str:
    h = hashlib.sha256()
    for p in sources() + sorted(SRC_DIR.glob("*.cuh")) + sorted(SRC_DIR.glob("*.h")):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
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
        d = Path(tempfile.gettempdir()) / f"sonicboom_b200-{os.getuid()}-{_stamp()[:12]}"
        d.mkdir(parents=True, exist_ok=True)
        return d


def _say(msg: str) -> None:
    print(f"[sonicboom_b200] {msg}", file=sys.stderr, flush=True)


def build(force: bool = False, verbose: bool = True) -> Path:
    """Compiles every .cu of this folder and links them; returns the library's path."""
    out_dir = _build_dir()
    lib, stamp_file, stamp = out_dir / LIB_NAME, out_dir / "stamp", _stamp()
    if not force and lib.is_file() and stamp_file.is_file() and stamp_file.read_text() == stamp:
        return lib
    nvcc = _nvcc()
    srcs = sources()
    t0 = time.time()
    if verbose:
        _say(f"compiling {len(srcs)} CUDA files for sm_100a into {out_dir} (first use only)")

    def compile_one(src: Path):
        obj = out_dir / (src.stem + ".o")
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(SRC_DIR), "-c", str(src), "-o", str(obj)]
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
    tmp_lib = out_dir / (LIB_NAME + f".tmp{os.getpid()}")
    r = subprocess.run([nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp_lib), *objs],
                       capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"linking {LIB_NAME} failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp_lib, lib)
    stamp_file.write_text(stamp)
    if verbose:
        _say(f"built {lib.name} in {time.time() - t0:.0f}s")
    return lib


_LIB = None


def load() -> ctypes.CDLL:
    """The loaded library; builds it first when needed."""
    global _LIB
    if _LIB is None:
        path = build()
        try:
            _LIB = ctypes.CDLL(str(path))
        except OSError as e:
            raise BuildError(f"could not load {path}: {e}") from None
    return _LIB
