"""Builds the CUDA sources of this folder into shared libraries for sm_100a, and the
host-only C++ sources (the cache manager's books) with the host compiler.

Each source file becomes its own library with C linkage, loaded through ``ctypes``; a
library is compiled the first time one of its functions is wanted, so a run compiles
only what its model needs.  The file name of a built library carries a hash of its
source, of the shared header and of the compiler flags: a library that does not match
the sources in the tree is never loaded.  Built libraries live in ``_build/`` beside
the sources when that folder can be written, otherwise in a per-user temporary
folder.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import Dict, Iterable, List, Optional

HERE = os.path.dirname(os.path.abspath(__file__))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17", "--expt-relaxed-constexpr",
    "-shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]

# library name -> source file; headers every library depends on
LIBRARIES: Dict[str, str] = {
    "rowwise": "rowwise.cu",
    "gemm_simt": "gemm_simt.cu",
    "attention_paged": "attention_paged.cu",
    "moe_route": "moe_route.cu",
    "sampling": "sampling.cu",
    "gemm_tc": "gemm_tc.cu",
    "gemm_tc2": "gemm_tc2.cu",
    "attention_decode": "attention_decode.cu",
    "attention_prefill": "attention_prefill.cu",
    "attention_prefill_tc": "attention_prefill_tc.cu",
    "random_fill": "random_fill.cu",
}
HEADERS = ["common.cuh", "tc_common.cuh", "sampling_static.h"]

# host-only libraries (no CUDA): compiled with the host C++ compiler, so that the books of the
# cache manager also load on a machine without nvcc or a GPU
HOST_LIBRARIES: Dict[str, str] = {
    "host_books": "host_books.cpp",
}
LIBRARIES.update(HOST_LIBRARIES)
CXX_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden"]


class BuildError(RuntimeError):
    pass


def _nvcc() -> Optional[str]:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    return None


def _cxx() -> Optional[str]:
    for cand in (os.environ.get("CXX"), "g++", "c++", "clang++"):
        path = shutil.which(cand) if cand else None
        if path:
            return path
    return None


def _digest(name: str) -> str:
    h = hashlib.sha256()
    host = name in HOST_LIBRARIES
    for rel in [LIBRARIES[name]] + ([] if host else HEADERS):
        with open(os.path.join(HERE, rel), "rb") as f:
            h.update(rel.encode())
            h.update(f.read())
    h.update(" ".join(CXX_FLAGS if host else NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _command(name: str, tmp: str) -> List[str]:
    """The compiler call that builds library ``name`` into ``tmp``."""
    src = os.path.join(HERE, LIBRARIES[name])
    if name in HOST_LIBRARIES:
        cxx = _cxx()
        if cxx is None:
            raise BuildError(f"library '{name}' is not built and no C++ compiler (g++, c++, clang++ or $CXX) was found")
        return [cxx] + CXX_FLAGS + ["-o", tmp, src]
    nvcc = _nvcc()
    if nvcc is None:
        raise BuildError(
            f"kernel library '{name}' is not built and nvcc was not found; "
            "this engine has no fallback without its CUDA kernels")
    return [nvcc] + NVCC_FLAGS + ["-I", HERE, "-o", tmp, src]


def _target(name: str) -> str:
    return "the host" if name in HOST_LIBRARIES else "sm_100a"


def _build_dirs() -> List[str]:
    dirs = [os.path.join(HERE, "_build")]
    env = os.environ.get("CAJETA_B200_BUILD_DIR")
    if env:
        dirs.insert(0, env)
    dirs.append(os.path.join(tempfile.gettempdir(), f"cajeta_llm_b200_build_{os.getuid()}"))
    return dirs


def _file_name(name: str) -> str:
    return f"libcj_{name}-{_digest(name)}.so"


def find_built(name: str) -> Optional[str]:
    fn = _file_name(name)
    for d in _build_dirs():
        p = os.path.join(d, fn)
        if os.path.isfile(p):
            return p
    return None


def _writable_dir() -> str:
    last = None
    for d in _build_dirs():
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".probe_{os.getpid()}_{threading.get_ident()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return d
        except OSError as e:
            last = e
    raise BuildError(f"no writable folder for built kernels (tried {_build_dirs()}): {last}")


_lock = threading.Lock()


def _drop_stale(folder: str, name: str, keep: str) -> None:
    """Remove builds of ``name`` from other source versions; a library in use elsewhere stays
    mapped in that process, so this cannot break a running engine."""
    prefix = _file_name(name).rsplit("-", 1)[0] + "-"
    try:
        for f in os.listdir(folder):
            if f.startswith(prefix) and f.endswith(".so") and f != keep:
                os.remove(os.path.join(folder, f))
    except OSError:
        pass


def build(name: str, verbose: bool = True) -> str:
    """Path of the built library ``name``; compiles it when no matching build exists."""
    if name not in LIBRARIES:
        raise BuildError(f"unknown kernel library '{name}'; known: {', '.join(LIBRARIES)}")
    with _lock:
        found = find_built(name)
        if found:
            return found
        out_dir = _writable_dir()
        out = os.path.join(out_dir, _file_name(name))
        tmp = out + f".tmp{os.getpid()}"
        cmd = _command(name, tmp)
        if verbose:
            print(f"[cajeta_llm_b200] compiling {LIBRARIES[name]} for {_target(name)} ...", file=sys.stderr, flush=True)
        t0 = time.time()
        done = threading.Event()

        def tick():
            while not done.wait(10.0):
                print(f"[cajeta_llm_b200]   still compiling {LIBRARIES[name]} ({time.time() - t0:.0f} s)",
                      file=sys.stderr, flush=True)

        ticker = threading.Thread(target=tick, daemon=True)
        if verbose:
            ticker.start()
        try:
            proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                                  env={**os.environ, "TMPDIR": out_dir})
        finally:
            done.set()
        if proc.returncode != 0:
            try:
                os.remove(tmp)
            except OSError:
                pass
            raise BuildError(f"{os.path.basename(cmd[0])} failed for {LIBRARIES[name]}:\n{proc.stdout}")
        os.replace(tmp, out)
        _drop_stale(out_dir, name, os.path.basename(out))
        if verbose:
            print(f"[cajeta_llm_b200] built {os.path.basename(out)} in {time.time() - t0:.1f} s",
                  file=sys.stderr, flush=True)
        return out


def build_all(names: Optional[Iterable[str]] = None, verbose: bool = True) -> Dict[str, str]:
    """Compile every library (in parallel processes of nvcc) and return their paths."""
    names = list(names) if names is not None else list(LIBRARIES)
    missing = [n for n in names if find_built(n) is None]
    results: Dict[str, str] = {}
    if missing:
        # nvcc runs as a subprocess, so threads give real parallelism here; the lock in
        # build() is per call, so compile through a private worker instead
        errors: List[BaseException] = []

        def work(n: str) -> None:
            try:
                _compile_unlocked(n, verbose)
            except BaseException as e:  # noqa: BLE001 - reported below
                errors.append(e)

        threads = [threading.Thread(target=work, args=(n,)) for n in missing]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        if errors:
            raise errors[0]
    for n in names:
        results[n] = build(n, verbose)
    return results


def _compile_unlocked(name: str, verbose: bool) -> None:
    out_dir = _writable_dir()
    out = os.path.join(out_dir, _file_name(name))
    tmp = out + f".tmp{os.getpid()}_{threading.get_ident()}"
    cmd = _command(name, tmp)
    t0 = time.time()
    if verbose:
        print(f"[cajeta_llm_b200] compiling {LIBRARIES[name]} for {_target(name)} ...", file=sys.stderr, flush=True)
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                          env={**os.environ, "TMPDIR": out_dir})
    if proc.returncode != 0:
        try:
            os.remove(tmp)
        except OSError:
            pass
        raise BuildError(f"{os.path.basename(cmd[0])} failed for {LIBRARIES[name]}:\n{proc.stdout}")
    os.replace(tmp, out)
    _drop_stale(out_dir, name, os.path.basename(out))
    if verbose:
        print(f"[cajeta_llm_b200] built {os.path.basename(out)} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)


if __name__ == "__main__":
    for lib, path in build_all().items():
        print(lib, path)
