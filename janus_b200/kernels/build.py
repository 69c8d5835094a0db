"""Compiling the CUDA sources under `csrc/` for sm_100a and loading them.

One shared library per source file (and per set of `-D` definitions, e.g. the
head size an attention kernel is specialised for), built with nvcc on first
use into `csrc/_build/` (or a temporary folder if the package folder cannot be
written) and loaded with ctypes.  A library is rebuilt when its source, a
header or the flags change.  There is no fallback: a kernel that cannot be
built or loaded raises.
"""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import Dict, Iterable, Optional, Tuple

CSRC = Path(__file__).resolve().parent.parent / "csrc"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr",
    "-shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


class KernelBuildError(RuntimeError):
    pass


_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


def _nvcc() -> str:
    for cand in (os.environ.get("JANUS_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 shutil.which("nvcc")):
        if cand and os.path.exists(cand):
            return cand
    raise KernelBuildError("nvcc not found (set CUDA_HOME or JANUS_NVCC); the CUDA kernels cannot be built "
                           "and there is no other code path")


def build_dir() -> Path:
    override = os.environ.get("JANUS_BUILD_DIR")
    if override:
        d = Path(override)
        d.mkdir(parents=True, exist_ok=True)
        return d
    d = CSRC / "_build"
    try:
        d.mkdir(parents=True, exist_ok=True)
        probe = d / f".write_probe_{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return d
    except OSError:
        d = Path(tempfile.gettempdir()) / f"janus_b200_build_{os.getuid()}"
        d.mkdir(parents=True, exist_ok=True)
        return d


def _variant(stem: str, defines: Optional[Dict[str, object]]) -> str:
    if not defines:
        return stem
    return stem + "".join(f"-{k.lower().replace('jb_', '')}{v}" for k, v in sorted(defines.items()))


def _digest(source: Path, defines: Optional[Dict[str, object]]) -> str:
    h = hashlib.sha256()
    h.update(source.read_bytes())
    for header in sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")):
        h.update(header.name.encode())
        h.update(header.read_bytes())
    h.update(repr(NVCC_FLAGS).encode())
    h.update(repr(sorted((defines or {}).items())).encode())
    return h.hexdigest()


def _compile(source: Path, out: Path, defines: Optional[Dict[str, object]], verbose: bool) -> None:
    cmd = [_nvcc(), *NVCC_FLAGS, f"-I{CSRC}"]
    for k, v in sorted((defines or {}).items()):
        cmd.append(f"-D{k}={v}")
    tmp = out.with_suffix(f".tmp{os.getpid()}.so")
    cmd += ["-o", str(tmp), str(source)]
    if os.environ.get("JANUS_PTXAS_VERBOSE"):
        cmd.insert(1, "-Xptxas=-v")
    t0 = time.time()
    print(f"[janus_b200] compiling {out.stem} for sm_100a ...", file=sys.stderr, flush=True)
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def heartbeat():
        while not done.wait(15.0):
            print(f"[janus_b200] still compiling {out.stem} ({time.time() - t0:.0f} s)", file=sys.stderr, flush=True)

    hb = threading.Thread(target=heartbeat, daemon=True)
    hb.start()
    output, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        try:
            tmp.unlink()
        except OSError:
            pass
        raise KernelBuildError(f"nvcc failed for {source.name} (exit {proc.returncode}):\n{output}")
    if os.environ.get("JANUS_PTXAS_VERBOSE") and output:
        print(output, file=sys.stderr)
    os.replace(tmp, out)
    if verbose:
        print(f"[janus_b200] built {out.name} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)


def ensure_built(stem: str, defines: Optional[Dict[str, object]] = None, verbose: bool = True) -> Path:
    """Path of the up-to-date shared library of `csrc/<stem>.cu`."""
    source = CSRC / f"{stem}.cu"
    if not source.exists():
        raise KernelBuildError(f"no such kernel source: {source}")
    name = _variant(stem, defines)
    d = build_dir()
    out = d / f"{name}.so"
    stamp = d / f"{name}.stamp"
    digest = _digest(source, defines)
    if out.exists() and stamp.exists() and stamp.read_text() == digest:
        return out
    lock_path = d / f"{name}.lock"
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if out.exists() and stamp.exists() and stamp.read_text() == digest:
                return out
            _compile(source, out, defines, verbose)
            stamp.write_text(digest)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return out


def library(stem: str, defines: Optional[Dict[str, object]] = None) -> ctypes.CDLL:
    name = _variant(stem, defines)
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = ensure_built(stem, defines)
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from e
            _loaded[name] = lib
        return lib


def build_many(items: Iterable[Tuple[str, Optional[Dict[str, object]]]], jobs: int = 0) -> None:
    """Compile several libraries in parallel (used by the ahead-of-time build)."""
    items = list(items)
    jobs = jobs or min(len(items), max(1, (os.cpu_count() or 2)))
    with ThreadPoolExecutor(max_workers=jobs) as pool:
        for f in [pool.submit(ensure_built, stem, defines) for stem, defines in items]:
            f.result()
