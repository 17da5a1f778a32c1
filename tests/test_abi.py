"""The kernel libraries' public header: it compiles as plain C, and the ctypes table in
sonicboom_b200/abi.py says what the header says."""
import re
import shutil
import subprocess
from pathlib import Path

import pytest

from sonicboom_b200 import abi

CSRC = Path(abi.__file__).resolve().parent / "csrc"


def prototypes() -> dict:
    """name -> (result code, argument codes) of every function the two headers declare."""
    text = (CSRC / "sonicboom_b200.h").read_text() + (CSRC / "no_alloc.h").read_text()
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    text = re.sub(r"//[^\n]*", " ", text)
    text = re.sub(r"^\s*#[^\n]*", " ", text, flags=re.M)
    out = {}
    for m in re.finditer(r"\b(const char\*|size_t|int|void)\s+(sb_\w+)\s*\(([^)]*)\)\s*;", text):
        result = {"const char*": "c", "size_t": "z", "int": "i", "void": "v"}[m.group(1)]
        args = ""
        for a in [a.strip() for a in m.group(3).split(",")]:
            if a in ("void", ""):
                continue
            kind = a.rsplit(None, 1)[0] if not a.endswith("*") else a       # drop the name
            if "*" in a:
                args += "p"
            elif kind == "sb_stream_t":
                args += "s"
            else:
                args += {"int": "i", "float": "f", "size_t": "z", "uint32_t": "u"}[kind]
        out[m.group(2)] = (result, args)
    return out


def test_the_table_says_what_the_header_says():
    declared = prototypes()
    table = {**abi.EVERY_LIBRARY, **abi.CORE, **abi.ATTENTION}
    assert sorted(declared) == sorted(table)
    for name in table:
        assert declared[name] == table[name], name


def test_every_exported_entry_point_is_declared():
    """Each `extern "C"` definition in the sources has its declaration in the header."""
    defined = set()
    for src in list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")):
        defined |= set(re.findall(r'extern "C"[^;{(]*?\b(sb_\w+)\s*\(', src.read_text()))
    assert defined == set(prototypes())


@pytest.mark.skipif(shutil.which("gcc") is None, reason="no C compiler")
def test_the_header_compiles_as_c(tmp_path):
    src = tmp_path / "use.c"
    src.write_text('#include "sonicboom_b200.h"\n'
                   "int use(sb_stream_t s) {\n"
                   "  SbLinearExtras extras = {0};\n"
                   "  SbSampleParams rec = {0};\n"
                   "  float x = 0.0f;\n"
                   "  (void)extras; (void)rec;\n"
                   "  if (sb_abi_version() != 1) return SB_ERR_ARG;\n"
                   "  if (sb_attention_static_scratch_bytes() != SB_STATIC_SCRATCH_BYTES) return SB_ERR_ARG;\n"
                   "  return sb_softcap(&x, 1, 30.0f, s) == SB_OK ? SB_OK : SB_ERR_CUDA;\n"
                   "}\n")
    r = subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-fsyntax-only",
                        "-I", str(CSRC), str(src)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_the_sampler_record_is_the_header_struct():
    import numpy as np
    from sonicboom_b200.sampling.sampler import _RECORD
    fields = re.search(r"typedef struct SbSampleParams \{(.*?)\}", (CSRC / "sonicboom_b200.h").read_text(), re.S).group(1)
    fields = re.sub(r"/\*.*?\*/", "", fields, flags=re.S)
    names = [n.strip() for decl in fields.split(";") if decl.strip()
             for n in decl.strip().split(None, 1)[1].split(",")]
    assert names == list(_RECORD.names)
    assert _RECORD.itemsize == 6 * 4 + 4 + 4 + 8 + 8 and np.dtype(_RECORD).isalignedstruct is False
