"""Compiling and loading the CUDA library.

The kernels are plain CUDA with ``extern "C"`` launchers, compiled by ``nvcc`` for sm_100a
into one shared library inside the package (``csrc/_build/``) and loaded with ``ctypes``; no
Python or PyTorch headers are involved, so a cold build takes seconds per file. The library
is rebuilt when a source or a flag changes. If the package folder cannot be written to, the
build goes to a per-user folder under the system's temporary directory. There is no fallback
that computes without the library: loading fails loudly.
"""

from __future__ import annotations

import ctypes
import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC"]
# TINYSERVE_B200_TIMELINE=1 builds a second library (in a folder of its own) whose kernels note
# when they start and when their wait for the kernels before them returns (ops.timeline()).
TIMELINE = os.environ.get("TINYSERVE_B200_TIMELINE", "") not in ("", "0")
if TIMELINE:
    NVCC_FLAGS = NVCC_FLAGS + ["-DTS_TIMELINE"]
LIB_NAME = "libtinyserve_b200.so"

_lock = threading.Lock()
_lib: ctypes.CDLL | None = None


class KernelBuildError(RuntimeError):
    """The CUDA library could not be compiled or loaded."""


def _say(msg: str) -> None:
    print(f"[tinyserve_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for root in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if root and (Path(root) / "bin" / "nvcc").is_file():
            return str(Path(root) / "bin" / "nvcc")
    found = shutil.which("nvcc")
    if found:
        return found
    raise KernelBuildError("nvcc not found (looked in CUDA_HOME, /usr/local/cuda and PATH)")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _fingerprint(files: list[Path]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    for f in sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    return h.hexdigest()


def _writable(d: Path) -> bool:
    try:
        d.mkdir(parents=True, exist_ok=True)
        probe = d / f".probe_{os.getpid()}"
        probe.write_text("x")
        probe.unlink()
        return True
    except OSError:
        return False


def build_dir() -> Path:
    override = os.environ.get("TINYSERVE_B200_BUILD_DIR")
    if override:
        d = Path(override)
        if not _writable(d):
            raise KernelBuildError(f"TINYSERVE_B200_BUILD_DIR={override} is not writable")
        return d
    d = CSRC / ("_build_timeline" if TIMELINE else "_build")
    if _writable(d):
        return d
    d = Path(tempfile.gettempdir()) / f"tinyserve_b200_build_{os.getuid()}{'_timeline' if TIMELINE else ''}"
    if _writable(d):
        return d
    raise KernelBuildError(f"no writable build folder (tried {CSRC / '_build'} and {d})")


def _compile_one(nvcc: str, src: Path, obj: Path, verbose: bool) -> None:
    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise KernelBuildError(f"nvcc failed on {src.name}:\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        _say(f"{src.name}:\n{proc.stderr}")


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``.cu`` of ``csrc/`` for sm_100a and link them; returns the library path."""
    files = sources()
    if not files:
        raise KernelBuildError(f"no CUDA sources in {CSRC}")
    out_dir = build_dir()
    lib = out_dir / LIB_NAME
    stamp = out_dir / "build.json"
    fp = _fingerprint(files)
    if not force and lib.is_file() and stamp.is_file():
        try:
            if json.loads(stamp.read_text()).get("fingerprint") == fp:
                return lib
        except (OSError, ValueError):
            pass
    nvcc = find_nvcc()
    t0 = time.time()
    _say(f"compiling {len(files)} CUDA files for sm_100a into {out_dir} (first call only)")
    objs = [out_dir / (f.stem + ".o") for f in files]
    done = 0

    def one(pair: tuple[Path, Path]) -> None:
        nonlocal done
        _compile_one(nvcc, pair[0], pair[1], verbose)
        done += 1
        _say(f"  compiled {pair[0].name} ({done}/{len(files)}, {time.time() - t0:.0f} s)")

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
        list(pool.map(one, zip(files, objs)))
    tmp = out_dir / f".{LIB_NAME}.{os.getpid()}"
    link = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp), *[str(o) for o in objs]]
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        raise KernelBuildError(f"linking failed:\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp, lib)
    stamp.write_text(json.dumps({"fingerprint": fp, "sources": [f.name for f in files]}))
    _say(f"built {lib.name} in {time.time() - t0:.0f} s")
    return lib


def library() -> ctypes.CDLL:
    """The loaded CUDA library, built first if needed."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            path = build()
            try:
                _lib = ctypes.CDLL(str(path))
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from e
    return _lib
