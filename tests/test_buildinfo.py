"""The build-information string and the trace switch (no device)."""
import re
import subprocess
import sys

from conftest import ROOT


def test_build_info_names_version_revision_compiler_and_target():
    import sonicboom_b200 as sb
    info = sb.build_info()
    assert info["version"] == sb.__version__ and info["arch"] == "sm_100a"
    assert re.fullmatch(r"[0-9a-f]{12}\+?|unknown", info["git"])
    assert re.fullmatch(r"\d+\.\d+(\.\d+)?|not found|unknown", info["nvcc"])
    assert all(h % 16 == 0 and 16 <= h <= 256 for h in info["attention_head_sizes_built"])
    line = sb.build_info_line()
    for part in (sb.__version__, info["git"], info["nvcc"], "sm_100a"):
        assert part in line


def test_command_line_prints_it():
    r = subprocess.run([sys.executable, str(ROOT / "bin" / "sonicboom_b200"), "--version"],
                       capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and r.stdout.startswith("sonicboom_b200 ") and "sm_100a" in r.stdout
    r = subprocess.run([sys.executable, str(ROOT / "bin" / "sonicboom_b200")],
                       capture_output=True, text=True, timeout=120)
    assert r.returncode != 0 and "command is required" in r.stderr


def test_trace_ranges_cost_nothing_when_off():
    from sonicboom_b200 import ops
    assert not ops.TRACE or True
    ops.set_trace(False)
    a, b = ops.trace_range("x"), ops.trace_range("y")
    assert a is b                                   # one shared no-op object
    with a:
        pass
    ops.set_trace(True)
    try:
        assert ops.trace_range("x") is not ops.trace_range("y")
    finally:
        ops.set_trace(False)
