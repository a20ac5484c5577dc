"""Compiling and loading the CUDA sources of `csrc/`.

Each `.cu` file becomes one shared library, built for sm_100a by nvcc and loaded
with ctypes; the exported launchers take raw device pointers and a stream, so no
binding layer has to be compiled.  A library is built when it is first needed
(only what the running model uses gets compiled) or all at once by
`build_all()`.  The reference compiles its kernel string with nvrtc at start-up
(src/backend/cuda.rs:462-488); the idea is the same, the unit is a file.

There is no fallback: if nvcc is missing or a source does not compile, the
caller gets a KernelError.
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

from ..errors import KernelError

CSRC_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--shared", "-Xcompiler", "-fPIC",
]
# more flags for experiments (for instance -DRL_TRACE, see csrc/common.cuh); they are part of a
# library's fingerprint, so give such builds a folder of their own with RUSTY_LLAMA_BUILD_DIR
NVCC_FLAGS += os.environ.get("RUSTY_LLAMA_NVCC_EXTRA", "").split()

_lock = threading.Lock()
_dir_lock = threading.Lock()
_loaded: Dict[str, ctypes.CDLL] = {}


def _say(msg: str) -> None:
    print(f"[rusty_llama_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("RUSTY_LLAMA_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelError("nvcc was not found (looked at $RUSTY_LLAMA_NVCC, PATH and /usr/local/cuda/bin): the CUDA kernels cannot be built")


def source_names() -> List[str]:
    return sorted(f[:-3] for f in os.listdir(CSRC_DIR) if f.endswith(".cu"))


_build_dir_cached: Optional[str] = None


def _build_dir() -> str:
    """`csrc/_build` when it can be written, else a per-user folder under the temp dir."""
    global _build_dir_cached
    with _dir_lock:
        if _build_dir_cached is None:
            _build_dir_cached = _find_build_dir()
        return _build_dir_cached


def _find_build_dir() -> str:
    override = os.environ.get("RUSTY_LLAMA_BUILD_DIR")
    cands = [override] if override else []
    cands.append(os.path.join(CSRC_DIR, "_build"))
    cands.append(os.path.join(tempfile.gettempdir(), f"rusty_llama_b200_build_{os.getuid()}"))
    for d in cands:
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".w{os.getpid()}_{threading.get_ident()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return d
        except OSError:
            continue
    raise KernelError(f"no writable folder for built kernels (tried {cands})")


def _fingerprint(name: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for fn in sorted(os.listdir(CSRC_DIR)):
        if fn == name + ".cu" or fn.endswith(".cuh") or fn.endswith(".h"):
            with open(os.path.join(CSRC_DIR, fn), "rb") as f:
                h.update(fn.encode())
                h.update(f.read())
    return h.hexdigest()


def library_path(name: str) -> str:
    return os.path.join(_build_dir(), f"librl_{name}.so")


def build(name: str, verbose: bool = True) -> str:
    """Compile `csrc/<name>.cu` if its library is missing or older than its sources; returns the path."""
    src = os.path.join(CSRC_DIR, name + ".cu")
    if not os.path.isfile(src):
        raise KernelError(f"no CUDA source '{src}'")
    out = library_path(name)
    stamp = out + ".sha256"
    want = _fingerprint(name)
    if os.path.isfile(out) and os.path.isfile(stamp):
        try:
            with open(stamp) as f:
                if f.read().strip() == want:
                    return out
        except OSError:
            pass
    nvcc = find_nvcc()
    tmp = f"{out}.{os.getpid()}.tmp"
    cmd = [nvcc] + NVCC_FLAGS + ["-I", CSRC_DIR, "-o", tmp, src]
    if verbose:
        _say(f"compiling {name}.cu for sm_100a ...")
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    while True:
        try:
            output, _ = proc.communicate(timeout=10)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                _say(f"  still compiling {name}.cu ({time.time() - t0:.0f} s)")
    if proc.returncode != 0:
        try:
            os.remove(tmp)
        except OSError:
            pass
        raise KernelError(f"nvcc failed on {name}.cu (exit {proc.returncode}):\n{output}")
    os.replace(tmp, out)
    with open(stamp, "w") as f:
        f.write(want)
    if verbose:
        _say(f"  built {os.path.basename(out)} in {time.time() - t0:.1f} s")
    return out


def build_all(verbose: bool = True) -> List[str]:
    """Every source, a few at a time in parallel."""
    names = source_names()
    results: Dict[str, object] = {}

    def work(n):
        try:
            results[n] = build(n, verbose)
        except Exception as e:  # reported below, with the name
            results[n] = e

    threads: List[threading.Thread] = []
    width = max(1, min(4, os.cpu_count() or 1))
    for i in range(0, len(names), width):
        batch = [threading.Thread(target=work, args=(n,)) for n in names[i : i + width]]
        for t in batch:
            t.start()
        for t in batch:
            t.join()
        threads += batch
    for n in names:
        if isinstance(results[n], Exception):
            raise results[n]
    return [results[n] for n in names]


def load(name: str) -> ctypes.CDLL:
    """The library of `csrc/<name>.cu`, built first if need be."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = build(name)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelError(f"cannot load '{path}': {e}") from None
            lib.rl_error_text.restype = ctypes.c_char_p
            _loaded[name] = lib
        return lib


def loaded_libraries() -> Dict[str, str]:
    return {n: library_path(n) for n in _loaded}
