"""Builds and runs the C++ test program of the host core (CPU)."""

import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
CORE = ROOT / "prefixserve_b200" / "csrc" / "core"


@pytest.mark.skipif(shutil.which("g++") is None, reason="no g++")
def test_core_allocates_nothing_after_construction(tmp_path):
    exe = tmp_path / "test_no_alloc"
    build = subprocess.run(["g++", "-O1", "-std=c++17", "-Wall", "-Wextra", f"-I{CORE}", str(ROOT / "tests" / "cpp" / "test_no_alloc.cpp"),
                            str(CORE / "radix_tree.cpp"), "-o", str(exe)], capture_output=True, text=True)
    assert build.returncode == 0, build.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "ok: no allocation" in run.stdout
