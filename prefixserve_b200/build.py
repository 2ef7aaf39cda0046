"""Builds the two native libraries in-tree, on first use.

* ``_core``: host C++17 (page pool, prefix tree, slots, page tables), pybind11.
* ``libpsb200_kernels.so``: the CUDA kernels, compiled for sm_100a only and
  called through a C ABI.

Each library is rebuilt when the hash of its sources and flags changes.  The
output goes to ``prefixserve_b200/_build``; if the package folder cannot be
written, to a per-user folder under the system temp dir.  A line is printed to
stderr when a build starts, every few seconds while it runs, and when it ends.
"""

from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC = PACKAGE_DIR / "csrc"
CUDA_ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[prefixserve_b200 build] {msg}", file=sys.stderr, flush=True)


def _writable(folder: Path) -> bool:
    try:
        folder.mkdir(parents=True, exist_ok=True)
        probe = folder / f".probe-{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return True
    except OSError:
        return False


_build_dir: Path | None = None


def build_dir() -> Path:
    global _build_dir
    if _build_dir is None:
        override = os.environ.get("PSB200_BUILD_DIR")
        candidates = [Path(override)] if override else []
        candidates.append(PACKAGE_DIR / "_build")
        candidates.append(Path(tempfile.gettempdir()) / f"prefixserve_b200-build-{os.getuid()}")
        for c in candidates:
            if _writable(c):
                _build_dir = c
                break
        else:
            raise BuildError(f"no writable build folder among {[str(c) for c in candidates]}")
    return _build_dir


def _find(tool: str, env_var: str, extra: list[str]) -> str:
    given = os.environ.get(env_var)
    if given:
        return given
    found = shutil.which(tool)
    if found:
        return found
    for e in extra:
        if Path(e).exists():
            return e
    raise BuildError(f"{tool} was not found (set {env_var})")


def _digest(files: list[Path], flags: list[str]) -> str:
    h = hashlib.sha256()
    for f in sorted(files):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update("\0".join(flags).encode())
    return h.hexdigest()


def _run(cmd: list[str], what: str) -> None:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise BuildError(f"{what} failed ({' '.join(cmd)}):\n{proc.stdout}")


class _Ticker:
    """Prints a line now and then while a build runs."""

    def __init__(self, what: str, every: float = 10.0) -> None:
        self.what, self.every = what, every
        self._stop = threading.Event()
        self._t0 = time.time()
        self._thread = threading.Thread(target=self._loop, daemon=True)

    def _loop(self) -> None:
        while not self._stop.wait(self.every):
            _say(f"{self.what}: still compiling ({time.time() - self._t0:.0f} s)")

    def __enter__(self) -> "_Ticker":
        _say(f"{self.what}: compiling (first use or sources changed)")
        self._thread.start()
        return self

    def __exit__(self, *exc: object) -> None:
        self._stop.set()
        if exc[0] is None:
            _say(f"{self.what}: done in {time.time() - self._t0:.0f} s")


class _Lock:
    def __init__(self, path: Path) -> None:
        self.path = path

    def __enter__(self) -> None:
        self.f = open(self.path, "w")
        fcntl.flock(self.f, fcntl.LOCK_EX)

    def __exit__(self, *exc: object) -> None:
        fcntl.flock(self.f, fcntl.LOCK_UN)
        self.f.close()


def _up_to_date(target: Path, digest: str) -> bool:
    stamp = target.with_suffix(target.suffix + ".stamp")
    return target.exists() and stamp.exists() and stamp.read_text().strip() == digest


def _finish(target: Path, tmp: Path, digest: str) -> None:
    os.replace(tmp, target)
    target.with_suffix(target.suffix + ".stamp").write_text(digest)


# ---------------------------------------------------------------- host core

def core_sources() -> list[Path]:
    return sorted((CSRC / "core").glob("*.cpp")) + sorted((CSRC / "core").glob("*.hpp"))


def ensure_core(force: bool = False) -> Path:
    import pybind11

    out = build_dir() / ("_core" + sysconfig.get_config_var("EXT_SUFFIX"))
    flags = ["-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall", "-Wextra"]
    digest = _digest(core_sources(), flags + [sys.version])
    if not force and _up_to_date(out, digest):
        return out
    with _Lock(build_dir() / ".core.lock"):
        if not force and _up_to_date(out, digest):
            return out
        cxx = _find("g++", "CXX", ["/usr/bin/g++"])
        tmp = out.with_name(out.name + f".tmp{os.getpid()}")
        cmd = [cxx, *flags, f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}", f"-I{CSRC / 'core'}"]
        cmd += [str(p) for p in core_sources() if p.suffix == ".cpp"] + ["-o", str(tmp)]
        with _Ticker("host core (_core)"):
            _run(cmd, "compiling the host core")
        _finish(out, tmp, digest)
    return out


# ------------------------------------------------------------- CUDA kernels

def kernel_sources() -> list[Path]:
    return sorted((CSRC / "kernels").glob("*.cu"))


def kernel_headers() -> list[Path]:
    return sorted((CSRC / "kernels").glob("*.cuh")) + sorted((CSRC / "kernels").glob("*.h"))


def nvcc_flags() -> list[str]:
    return [*CUDA_ARCH_FLAGS, "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
            "-Xcudafe", "--diag_suppress=177"]


def ensure_kernels(force: bool = False) -> Path:
    out = build_dir() / "libpsb200_kernels.so"
    flags = nvcc_flags()
    srcs = kernel_sources()
    digest = _digest(srcs + kernel_headers(), flags)
    if not force and _up_to_date(out, digest):
        return out
    with _Lock(build_dir() / ".kernels.lock"):
        if not force and _up_to_date(out, digest):
            return out
        nvcc = _find("nvcc", "NVCC", ["/usr/local/cuda/bin/nvcc"])
        obj_dir = build_dir() / "obj"
        obj_dir.mkdir(exist_ok=True)
        hdr_digest = _digest(kernel_headers(), flags)

        def compile_one(src: Path) -> Path:
            obj = obj_dir / (src.stem + ".o")
            d = _digest([src], [hdr_digest])
            if not force and _up_to_date(obj, d):
                return obj
            tmp = obj.with_name(obj.name + f".tmp{os.getpid()}")
            _run([nvcc, *flags, f"-I{CSRC / 'kernels'}", "-c", str(src), "-o", str(tmp)], f"compiling {src.name}")
            _finish(obj, tmp, d)
            return obj

        with _Ticker(f"CUDA kernels for sm_100a ({len(srcs)} files)"):
            with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
                objs = list(pool.map(compile_one, srcs))
            tmp = out.with_name(out.name + f".tmp{os.getpid()}")
            _run([nvcc, *CUDA_ARCH_FLAGS, "-shared", "-o", str(tmp), *[str(o) for o in objs]], "linking the kernel library")
        _finish(out, tmp, digest)
    return out


def build_all(force: bool = False) -> dict[str, Path]:
    return {"core": ensure_core(force), "kernels": ensure_kernels(force)}


if __name__ == "__main__":
    for name, path in build_all(force="--force" in sys.argv).items():
        print(f"{name}: {path}")
