"""The C++ host runtime (`ilb_host.cpp`) and its loader.

The library holds what the CPU does for every model load and every step: reading and
checking the safetensors container, the ledger of cache pages and state slots, the
scheduler's planning, and the packing of a step's integer arrays into the staging buffer.  It is compiled with the
C++ compiler the first time it is needed and kept beside the source (`_build/`), or
under the temporary directory when the package folder cannot be written.  There is no
Python stand-in: if it cannot be built, loading fails with the compiler's message.
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
from typing import List, Optional

HERE = os.path.dirname(os.path.abspath(__file__))
SOURCE = "ilb_host.cpp"
CXX_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-Wall"]

# return codes of the library
OK, INVALID, OUT_OF_PAGES, OUT_OF_SLOTS, LEDGER, FORMAT, IO, CAPACITY = 0, -1, -2, -3, -4, -5, -6, -7

_LOCK = threading.Lock()
_LIB: Optional[ctypes.CDLL] = None


class HostBuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[inferloop_b200] {msg}", file=sys.stderr, flush=True)


def find_cxx() -> str:
    for cand in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"), shutil.which("clang++")):
        if cand and (os.path.exists(cand) or shutil.which(cand)):
            return cand
    raise HostBuildError("no C++ compiler was found (looked at $CXX, g++, c++, clang++); "
                         "the host runtime of inferloop_b200 cannot be built")


def source_hash() -> str:
    h = hashlib.sha256()
    with open(os.path.join(HERE, SOURCE), "rb") as fh:
        h.update(fh.read())
    h.update(" ".join(CXX_FLAGS).encode())
    return h.hexdigest()[:16]


def _build_dirs() -> List[str]:
    uid = os.getuid() if hasattr(os, "getuid") else 0
    return [os.path.join(HERE, "_build"), os.path.join(tempfile.gettempdir(), f"inferloop_b200-build-{uid}")]


def library_path() -> Optional[str]:
    fname = f"ilb_host-{source_hash()}.so"
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
    raise HostBuildError("no writable folder for the host library: tried " + ", ".join(_build_dirs()))


def compile_library() -> str:
    existing = library_path()
    if existing:
        return existing
    cxx = find_cxx()
    out_dir = _writable_dir()
    final = os.path.join(out_dir, f"ilb_host-{source_hash()}.so")
    tmp = final + f".tmp{os.getpid()}-{threading.get_ident()}"
    cmd = [cxx] + CXX_FLAGS + ["-o", tmp, os.path.join(HERE, SOURCE)]
    _say(f"compiling {SOURCE} ...")
    t0 = time.time()
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise HostBuildError(f"the C++ compiler failed for {SOURCE}:\n{' '.join(cmd)}\n{proc.stdout}")
    os.replace(tmp, final)
    for old in os.listdir(out_dir):
        if old.startswith("ilb_host-") and old.endswith(".so") and old != os.path.basename(final):
            try:
                os.remove(os.path.join(out_dir, old))
            except OSError:
                pass
    _say(f"built {os.path.basename(final)} in {time.time() - t0:.1f} s")
    return final


def _declare(lib: ctypes.CDLL) -> None:
    c_int, c_ll, c_vp, c_cp = ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_char_p
    ip, llp = ctypes.POINTER(c_int), ctypes.POINTER(c_ll)
    lib.ilb_host_last_error.restype = c_cp
    sig = {
        "ilb_st_open": (c_int, [c_cp, ctypes.POINTER(c_vp)]),
        "ilb_st_count": (c_int, [c_vp]),
        "ilb_st_entry": (c_int, [c_vp, c_int, ctypes.POINTER(c_cp), ctypes.POINTER(c_cp), ip,
                                 ctypes.POINTER(llp), llp, llp]),
        "ilb_st_payload": (c_vp, [c_vp]),
        "ilb_st_data_start": (c_ll, [c_vp]),
        "ilb_st_metadata": (c_cp, [c_vp]),
        "ilb_st_close": (None, [c_vp]),
        "ilb_pool_new": (c_int, [c_int, ctypes.POINTER(c_vp)]),
        "ilb_pool_free": (None, [c_vp]),
        "ilb_pool_take": (c_int, [c_vp, c_ll, c_int, ip]),
        "ilb_pool_give_back": (c_int, [c_vp, c_ll, ip, c_int]),
        "ilb_pool_check": (c_int, [c_vp]),
        "ilb_pool_num_free": (c_int, [c_vp]),
        "ilb_pool_owner_of": (c_ll, [c_vp, c_int]),
        "ilb_pool_counters": (None, [c_vp, llp]),
        "ilb_slots_new": (c_int, [c_int, ctypes.POINTER(c_vp)]),
        "ilb_slots_free": (None, [c_vp]),
        "ilb_slots_take": (c_int, [c_vp, c_ll]),
        "ilb_slots_give_back": (c_int, [c_vp, c_ll]),
        "ilb_slots_slot_of": (c_int, [c_vp, c_ll]),
        "ilb_slots_num_free": (c_int, [c_vp]),
        "ilb_slots_check": (c_int, [c_vp]),
        "ilb_ledger_new": (c_int, [c_int, ip, ip, c_int, c_int, ctypes.POINTER(c_vp)]),
        "ilb_ledger_free": (None, [c_vp]),
        "ilb_ledger_begin": (c_int, [c_vp, c_ll]),
        "ilb_ledger_has": (c_int, [c_vp, c_ll]),
        "ilb_ledger_length": (c_ll, [c_vp, c_ll]),
        "ilb_ledger_slot_of": (c_int, [c_vp, c_ll]),
        "ilb_ledger_pages_needed": (c_int, [c_vp, c_ll, c_ll, ip]),
        "ilb_ledger_ensure": (c_int, [c_vp, c_ll, c_ll]),
        "ilb_ledger_commit": (c_int, [c_vp, c_ll, c_ll]),
        "ilb_ledger_release": (c_int, [c_vp, c_ll]),
        "ilb_ledger_check": (c_int, [c_vp]),
        "ilb_ledger_table_len": (c_int, [c_vp, c_int, c_ll]),
        "ilb_ledger_table": (c_int, [c_vp, c_int, c_ll, ip, c_int]),
        "ilb_ledger_pool": (c_vp, [c_vp, c_int]),
        "ilb_ledger_slots": (c_vp, [c_vp]),
        "ilb_ledger_stats": (None, [c_vp, llp]),
        "ilb_step_check": (c_int, [c_vp, c_int, llp, ip, ip, ip, ip, c_ll, c_ll]),
        "ilb_step_fits": (c_int, [c_vp, c_int, llp, ip]),
        "ilb_sched_new": (c_int, [c_vp, c_ll, c_ll, c_ll, c_ll, ctypes.POINTER(c_vp)]),
        "ilb_sched_free": (None, [c_vp]),
        "ilb_sched_set_limits": (c_int, [c_vp, c_ll, c_ll, c_ll, c_ll]),
        "ilb_sched_set_token_multiple": (c_int, [c_vp, c_ll]),
        "ilb_sched_add": (c_int, [c_vp, c_ll, c_ll, c_ll]),
        "ilb_sched_plan": (c_int, [c_vp, llp, c_int, ip, llp, ip]),
        "ilb_sched_token": (c_int, [c_vp, c_ll, c_int]),
        "ilb_sched_abort": (c_int, [c_vp, c_ll]),
        "ilb_sched_list": (c_int, [c_vp, c_int, llp, c_int]),
        "ilb_sched_stats": (None, [c_vp, llp]),
        "ilb_sched_count_step": (None, [c_vp]),
        "ilb_sched_preemptions_of": (c_int, [c_vp, c_ll]),
        "ilb_step_decode": (c_ll, [c_vp, c_int, llp, ip, c_int, c_int, c_ll, c_ll, c_vp, c_ll, llp]),
        "ilb_step_commit": (c_int, [c_vp, c_int, llp, ip]),
        "ilb_step_build": (c_ll, [c_vp, c_int, llp, ip, ip, ip, ip, c_int, c_int, c_ll, c_ll, c_vp, c_ll, llp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args


def lib() -> ctypes.CDLL:
    """The loaded host library (built on first use)."""
    global _LIB
    with _LOCK:
        if _LIB is None:
            loaded = ctypes.CDLL(compile_library())
            _declare(loaded)
            _LIB = loaded
        return _LIB


def last_error() -> str:
    return lib().ilb_host_last_error().decode("utf-8", "replace")
