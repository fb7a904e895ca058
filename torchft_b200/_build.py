"""In-tree native build for torchft_b200.

Two shared objects are produced next to the Python sources so that they travel
with the source tree:

* ``torchft_b200/_lib/libftb200_kernels.so`` -- every hand-written sm_100a CUDA
  kernel, exported through a plain C ABI (loaded with ``ctypes``).
* ``torchft_b200/_ftcp.<ext-suffix>.so``   -- the C++ control plane (lighthouse,
  manager server/client, quorum math) as a pybind11 module.

The build is a small dependency-free driver around ``nvcc`` / ``g++``: each
translation unit is compiled to an object file in ``build/`` when its content
hash (source + headers + flags) changed, then linked.  ``nvcc`` cross-compiles
for ``sm_100a`` on machines without a GPU.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
import threading
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import List, Sequence

PKG_DIR = Path(__file__).resolve().parent
REPO_DIR = PKG_DIR.parent
CSRC = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "_lib"
BUILD_DIR = REPO_DIR / "build"

KERNEL_LIB = LIB_DIR / "libftb200_kernels.so"
KERNEL_LIB_CHECKED = LIB_DIR / "libftb200_kernels_checked.so"  # -DFT_BOUNDS_CHECK=1 debug build
CONTROL_MOD = PKG_DIR / ("_ftcp" + sysconfig.get_config_var("EXT_SUFFIX"))

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--use_fast_math",
    "-Xcompiler",
    "-fPIC",
    "-Xcompiler",
    "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall", "-pthread"]

_lock = threading.Lock()


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; cannot build torchft_b200 CUDA kernels")
    return cand


def _cuda_home() -> str:
    return str(Path(_nvcc()).resolve().parent.parent)


def _digest(paths: Sequence[Path], flags: Sequence[str]) -> str:
    h = hashlib.sha256()
    for f in flags:
        h.update(f.encode())
    for p in sorted(paths):
        h.update(str(p.name).encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _run(cmd: List[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(
            "build command failed:\n  " + " ".join(cmd) + "\n" + proc.stdout + proc.stderr
        )
    if os.environ.get("FTB200_BUILD_VERBOSE") and (proc.stdout or proc.stderr):
        sys.stderr.write(proc.stdout + proc.stderr)


def _compile_objects(
    sources: Sequence[Path], headers: Sequence[Path], compiler: List[str], flags: List[str], tag: str
) -> List[Path]:
    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    objs: List[Path] = []
    jobs = []
    for src in sources:
        obj = BUILD_DIR / f"{tag}_{src.stem}.o"
        stamp = BUILD_DIR / f"{tag}_{src.stem}.hash"
        want = _digest([src, *headers], flags)
        objs.append(obj)
        if obj.exists() and stamp.exists() and stamp.read_text() == want:
            continue
        jobs.append((src, obj, stamp, want))

    def one(job):
        src, obj, stamp, want = job
        _run([*compiler, *flags, "-c", str(src), "-o", str(obj)])
        stamp.write_text(want)

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(one, jobs))
    return objs


def _needs_link(target: Path, objs: Sequence[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(o.stat().st_mtime > t for o in objs)


def build_kernels(verbose: bool = False, checked: bool = False) -> Path:
    """Compile every ``csrc/kernels/*.cu`` and ``csrc/team/*.cu`` for sm_100a.  ``checked``
    (or ``FTB200_BOUNDS_CHECK=1``) builds the checked-index debug variant next to the normal
    library instead: ``FTB_IN_RANGE`` then records out-of-range indices in a status word that
    ``ftb200_bounds_status_*`` report, and the guarded access is skipped."""
    checked = checked or bool(os.environ.get("FTB200_BOUNDS_CHECK"))
    target = KERNEL_LIB_CHECKED if checked else KERNEL_LIB
    with _lock:
        sources = sorted((CSRC / "kernels").glob("*.cu")) + sorted((CSRC / "team").glob("*.cu"))
        headers = []
        for d in ("kernels", "team"):
            headers += sorted((CSRC / d).glob("*.cuh")) + sorted((CSRC / d).glob("*.h"))
        flags = NVCC_FLAGS + [f"-I{CSRC / 'kernels'}", f"-I{CSRC / 'team'}"]
        if checked:
            flags = flags + ["-DFT_BOUNDS_CHECK=1"]
        if verbose:
            flags = flags + ["-Xptxas", "-v"]
        objs = _compile_objects(sources, headers, [_nvcc()], flags, "kc" if checked else "k")
        LIB_DIR.mkdir(parents=True, exist_ok=True)
        if _needs_link(target, objs):
            _run(
                [
                    _nvcc(),
                    "-shared",
                    "-o",
                    str(target),
                    *map(str, objs),
                    "-gencode",
                    "arch=compute_100a,code=sm_100a",
                    "-cudart",
                    "shared",
                ]
            )
        return target


def build_control() -> Path:
    """Compile the C++ control plane into a pybind11 extension module."""
    import pybind11

    with _lock:
        sources = sorted((CSRC / "control").glob("*.cpp"))
        if not sources:
            raise RuntimeError("no control-plane sources found")
        headers = sorted((CSRC / "control").glob("*.h"))
        flags = CXX_FLAGS + [
            f"-I{pybind11.get_include()}",
            f"-I{sysconfig.get_paths()['include']}",
            f"-I{CSRC / 'control'}",
        ]
        objs = _compile_objects(sources, headers, ["g++"], flags, "c")
        if _needs_link(CONTROL_MOD, objs):
            _run(["g++", "-shared", "-pthread", "-o", str(CONTROL_MOD), *map(str, objs)])
        return CONTROL_MOD


def build_all(verbose: bool = False) -> None:
    build_kernels(verbose=verbose)
    build_kernels(checked=True)  # the checked-index debug variant, used by tests/test_bounds_check_build.py
    build_control()


if __name__ == "__main__":
    build_all(verbose="-v" in sys.argv)
    print("built:", KERNEL_LIB, CONTROL_MOD)
