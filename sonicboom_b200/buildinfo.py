"""What this copy of the library is: version, source revision, compiler, target, and which
kernel libraries have been built.  Counterpart of the reference's `boom_build_info()`
(capi/include/sonicboom/capi.h:165-190), as one line of text and as a dictionary."""
from __future__ import annotations

import re
import subprocess
from pathlib import Path

from .csrc import build as _build

ROOT = Path(__file__).resolve().parent


def _run(cmd, cwd=None) -> str:
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=20, cwd=cwd)
        return r.stdout if r.returncode == 0 else ""
    except (OSError, subprocess.SubprocessError):
        return ""


def git_revision() -> str:
    """The checked-out commit (12 digits, "+" when the tree has changes); "unknown" outside git."""
    rev = _run(["git", "rev-parse", "--short=12", "HEAD"], cwd=ROOT).strip()
    if not rev:
        return "unknown"
    dirty = _run(["git", "status", "--porcelain", "--untracked-files=no"], cwd=ROOT).strip()
    return rev + ("+" if dirty else "")


def nvcc_version() -> str:
    try:
        out = _run([_build._nvcc(), "--version"])
    except _build.BuildError:
        return "not found"
    m = re.search(r"release [\d.]+, V([\d.]+)", out)
    return m.group(1) if m else "unknown"


def built_head_sizes() -> list:
    """Head sizes whose attention library lies built in the build folder."""
    found = []
    for p in _build._build_dir().glob("libsonicboom_b200_attn_hd*.so"):
        m = re.fullmatch(r"libsonicboom_b200_attn_hd(\d+)\.so", p.name)
        if m:
            found.append(int(m.group(1)))
    return sorted(found)


def build_info() -> dict:
    from . import __version__
    return {"version": __version__, "git": git_revision(), "nvcc": nvcc_version(),
            "arch": "sm_100a", "flags": " ".join(_build.NVCC_FLAGS),
            "core_library_built": (_build._build_dir() / _build.LIB_NAME).is_file(),
            "attention_head_sizes_built": built_head_sizes(),
            "attention_head_sizes": [_build.HEAD_DIMS[0], _build.HEAD_DIMS[-1], 16]}


def build_info_line() -> str:
    i = build_info()
    sizes = ",".join(str(h) for h in i["attention_head_sizes_built"]) or "none yet"
    return (f"sonicboom_b200 {i['version']} git {i['git']} nvcc {i['nvcc']} {i['arch']} "
            f"core {'built' if i['core_library_built'] else 'not built yet'} "
            f"attention head sizes built: {sizes}")
