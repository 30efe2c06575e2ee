"""Compile the CUDA sources of this package for sm_100a, one shared library per source.

A library is built the first time an op of it is called and is kept next to the sources
(`_build/<name>-<hash>.so`, the hash covering the source, the shared headers and the
flags), or under the temporary directory when the package folder cannot be written.
Only `nvcc` is needed: the launchers are plain `extern "C"` functions loaded with
ctypes, so no Python or torch header is compiled.  While a compile runs, a line is
printed to stderr at the start, every ten seconds, and at the end.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import Dict, List, Optional

HERE = os.path.dirname(os.path.abspath(__file__))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]

# name -> extra link flags
MODULES: Dict[str, List[str]] = {
    "elementwise": [],
    "gemm_simt": [],
    "gemm_tcgen05": [],
    "qk_norm_rope": [],
    "attention_simple": [],
    "attention_flash": [],
    "attention_tc": [],
    "attention_decode": [],
    "sampling": [],
}

_LOCK = threading.Lock()
_LOADED: Dict[str, ctypes.CDLL] = {}


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[inferloop_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("CUDACXX"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise BuildError("nvcc was not found (looked at $CUDACXX, PATH and /usr/local/cuda/bin); "
                     "the kernels of inferloop_b200 cannot be built")


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))


def source_hash(name: str) -> str:
    h = hashlib.sha256()
    for f in [name + ".cu"] + _headers():
        with open(os.path.join(HERE, f), "rb") as fh:
            h.update(f.encode())
            h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS + MODULES[name]).encode())
    return h.hexdigest()[:16]


def _build_dirs() -> List[str]:
    dirs = [os.path.join(HERE, "_build")]
    uid = os.getuid() if hasattr(os, "getuid") else 0
    dirs.append(os.path.join(tempfile.gettempdir(), f"inferloop_b200-build-{uid}"))
    return dirs


def library_path(name: str) -> Optional[str]:
    """Path of an up-to-date built library, or None."""
    fname = f"{name}-{source_hash(name)}.so"
    for d in _build_dirs():
        p = os.path.join(d, fname)
        if os.path.exists(p):
            return p
    return None


def _writable_dir() -> str:
    for d in _build_dirs():
        try:
            os.makedirs(d, exist_ok=True)
            with tempfile.NamedTemporaryFile(dir=d, prefix=".probe-"):
                pass
            return d
        except OSError:
            continue
    raise BuildError("no writable folder for built kernels: tried " + ", ".join(_build_dirs()))


def compile_module(name: str, verbose: bool = False) -> str:
    if name not in MODULES:
        raise BuildError(f"unknown kernel module {name!r}")
    existing = library_path(name)
    if existing:
        return existing
    nvcc = find_nvcc()
    out_dir = _writable_dir()
    final = os.path.join(out_dir, f"{name}-{source_hash(name)}.so")
    tmp = final + f".tmp{os.getpid()}-{threading.get_ident()}"
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + MODULES[name] + [
        "-I", HERE, "-o", tmp, os.path.join(HERE, name + ".cu")]
    _say(f"compiling {name}.cu for sm_100a ...")
    t0 = time.time()
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    done = threading.Event()

    def ticker() -> None:
        while not done.wait(10.0):
            _say(f"  still compiling {name}.cu ({time.time() - t0:.0f} s)")

    th = threading.Thread(target=ticker, daemon=True)
    th.start()
    out, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise BuildError(f"nvcc failed for {name}.cu:\n{' '.join(cmd)}\n{out}")
    os.replace(tmp, final)
    for old in os.listdir(out_dir):          # libraries of older sources are of no use
        if old.startswith(name + "-") and old.endswith(".so") and old != os.path.basename(final):
            try:
                os.remove(os.path.join(out_dir, old))
            except OSError:
                pass
    _say(f"built {os.path.basename(final)} in {time.time() - t0:.1f} s")
    if verbose and out:
        print(out, file=sys.stderr)
    return final


def load_module(name: str) -> ctypes.CDLL:
    with _LOCK:
        lib = _LOADED.get(name)
        if lib is None:
            path = compile_module(name)
            lib = ctypes.CDLL(path)
            lib.ilb_last_error.restype = ctypes.c_char_p
            _LOADED[name] = lib
        return lib


def build_all(verbose: bool = False) -> List[str]:
    """Compile every module (used by the build check); returns the library paths."""
    from concurrent.futures import ThreadPoolExecutor
    names = list(MODULES)
    with ThreadPoolExecutor(max_workers=min(8, len(names))) as pool:
        return list(pool.map(lambda n: compile_module(n, verbose), names))


if __name__ == "__main__":
    for p in build_all(verbose="-v" in sys.argv):
        print(p)
