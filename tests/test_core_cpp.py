"""Builds and runs the C++ test programs of the host core (CPU): the no-allocation check, and the behaviour cases
under AddressSanitizer and UndefinedBehaviorSanitizer (PrefixServe offers the same build, CMakeLists.txt:50-54)."""

import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
CORE = ROOT / "prefixserve_b200" / "csrc" / "core"
pytestmark = pytest.mark.skipif(shutil.which("g++") is None, reason="no g++")


def build_and_run(tmp_path, source: str, flags: list[str]) -> str:
    exe = tmp_path / Path(source).stem
    build = subprocess.run(["g++", "-std=c++17", "-Wall", "-Wextra", *flags, f"-I{CORE}", str(ROOT / "tests" / "cpp" / source),
                            str(CORE / "radix_tree.cpp"), "-o", str(exe)], capture_output=True, text=True)
    assert build.returncode == 0, build.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stdout + run.stderr
    return run.stdout


def test_core_allocates_nothing_after_construction(tmp_path):
    assert "ok: no allocation" in build_and_run(tmp_path, "test_no_alloc.cpp", ["-O1"])


def test_core_cases_under_address_and_undefined_behaviour_sanitizers(tmp_path):
    out = build_and_run(tmp_path, "test_core_cases.cpp",
                        ["-O1", "-g", "-fsanitize=address,undefined", "-fno-sanitize-recover=all", "-fno-omit-frame-pointer"])
    assert "ok: host core cases" in out


def test_core_cases_without_sanitizers(tmp_path):
    assert "ok: host core cases" in build_and_run(tmp_path, "test_core_cases.cpp", ["-O2"])
