"""Builds the two native libraries of the package, in-tree, on first use.

* ``libvcb_kernels.so`` -- the CUDA kernels under ``kernels/``, compiled by nvcc
  for sm_100a only and loaded through ctypes (no torch C++ headers are involved,
  so a cold build takes well under a minute);
* ``_vcb_runtime`` -- the host runtime under ``runtime/`` (cache manager and
  scheduler), a pybind11 module compiled by g++.

Objects land in ``csrc/_build`` when that folder can be written, else in a
per-user folder under the system's temporary directory.  A stamp made of the
sources' contents and the flags decides whether anything is rebuilt.
"""
from __future__ import annotations

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

CSRC = Path(__file__).resolve().parent
KERNEL_DIR = CSRC / "kernels"
RUNTIME_DIR = CSRC / "runtime"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]
# VLLM_CPP_B200_TIMELINE=1 builds the kernels with their timeline marks (see tl_mark in kernels/common.cuh); give such
# a build a folder of its own (VLLM_CPP_B200_BUILD_DIR) so that it does not replace the regular one
if os.environ.get("VLLM_CPP_B200_TIMELINE", "0") == "1":
    NVCC_FLAGS.append("-DVCB_TIMELINE")
# further nvcc flags for experiments (-D switches of single kernels); a build with them wants a folder of its own too
NVCC_FLAGS += os.environ.get("VLLM_CPP_B200_NVCC_EXTRA", "").split()
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall"]

_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[vllm_cpp_b200 build] {msg}", file=sys.stderr, flush=True)


def build_dir() -> Path:
    env = os.environ.get("VLLM_CPP_B200_BUILD_DIR")
    candidates = [Path(env)] if env else []
    candidates += [CSRC / "_build", Path(tempfile.gettempdir()) / f"vllm_cpp_b200_build_{os.getuid()}"]
    for d in candidates:
        try:
            d.mkdir(parents=True, exist_ok=True)
            probe = d / f".w{os.getpid()}"
            probe.write_text("x")
            probe.unlink()
            return d
        except OSError:
            continue
    raise BuildError("no writable folder for build products (tried " + ", ".join(map(str, candidates)) + ")")


def _find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).is_file():
            return cand
    raise BuildError("nvcc not found (set NVCC or put it on PATH); the CUDA kernels cannot be built")


def _digest(files: list[Path], flags: list[str]) -> str:
    h = hashlib.sha256()
    for f in sorted(files):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()


def _run(cmd: list[str], what: str) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"{what} failed:\n$ {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")


def _with_heartbeat(fn, what: str):
    """Runs fn() and prints a line every few seconds while it works."""
    done = threading.Event()
    t0 = time.time()

    def beat():
        while not done.wait(10.0):
            _say(f"still compiling {what} ... {time.time() - t0:.0f} s")

    th = threading.Thread(target=beat, daemon=True)
    th.start()
    try:
        return fn()
    finally:
        done.set()


def kernel_sources() -> list[Path]:
    return sorted(KERNEL_DIR.glob("*.cu"))


def build_kernels(force: bool = False) -> Path:
    """Compiles every ``kernels/*.cu`` for sm_100a and links ``libvcb_kernels.so``."""
    with _lock:
        out_dir = build_dir()
        lib = out_dir / "libvcb_kernels.so"
        stamp = out_dir / "libvcb_kernels.stamp"
        sources = kernel_sources()
        headers = sorted(KERNEL_DIR.glob("*.cuh")) + sorted(KERNEL_DIR.glob("*.h"))
        digest = _digest(sources + headers, NVCC_FLAGS)
        if not force and lib.is_file() and stamp.is_file() and stamp.read_text() == digest:
            return lib
        nvcc = _find_nvcc()
        _say(f"compiling {len(sources)} CUDA sources for sm_100a into {out_dir} (first use)")

        def compile_one(src: Path) -> Path:
            obj = out_dir / (src.stem + ".o")
            _run([nvcc, *NVCC_FLAGS, "-I", str(KERNEL_DIR), "-c", str(src), "-o", str(obj)], f"nvcc {src.name}")
            _say(f"  compiled {src.name}")
            return obj

        def work():
            with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
                objs = list(pool.map(compile_one, sources))
            tmp = out_dir / f"libvcb_kernels.{os.getpid()}.tmp.so"
            _run([nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-lcudart"], "link libvcb_kernels.so")
            os.replace(tmp, lib)

        _with_heartbeat(work, "CUDA kernels")
        stamp.write_text(digest)
        _say("CUDA kernels ready")
        return lib


def runtime_module_path() -> Path:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return build_dir() / f"_vcb_runtime{suffix}"


def build_runtime(force: bool = False) -> Path:
    """Compiles the host runtime (cache manager, scheduler) as a pybind11 module."""
    with _lock:
        out = runtime_module_path()
        stamp = out.parent / "_vcb_runtime.stamp"
        sources = sorted(RUNTIME_DIR.glob("*.cpp"))
        headers = sorted(RUNTIME_DIR.glob("*.h"))
        digest = _digest(sources + headers, CXX_FLAGS)
        if not force and out.is_file() and stamp.is_file() and stamp.read_text() == digest:
            return out
        try:
            import pybind11
        except ImportError as e:  # pragma: no cover
            raise BuildError("pybind11 is needed to build the host runtime") from e
        cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
        if not cxx:
            raise BuildError("no C++ compiler found for the host runtime")
        _say(f"compiling the host runtime into {out.parent} (first use)")
        tmp = out.parent / f"_vcb_runtime.{os.getpid()}.tmp.so"
        cmd = [cxx, *CXX_FLAGS, "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"],
               "-I", str(RUNTIME_DIR), *map(str, sources), "-o", str(tmp)]
        _with_heartbeat(lambda: _run(cmd, "g++ host runtime"), "host runtime")
        os.replace(tmp, out)
        stamp.write_text(digest)
        _say("host runtime ready")
        return out


def build_all(force: bool = False) -> None:
    build_runtime(force)
    build_kernels(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
