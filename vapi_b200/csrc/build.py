"""Builds the native sources of this package, one shared library per source: CUDA sources
(``.cu``) for sm_100a with nvcc, host sources (``.cpp``: the host runtime) with the C++ compiler.

Each ``<name>.cu`` / ``<name>.cpp`` becomes ``_build/lib<name>-<hash>.so`` next to it, where the hash covers
the source, the shared headers and the compiler flags, so a stale library is never picked
up.  A library is built the first time something asks for it, which means a program only
compiles what the model it runs needs.  While nvcc runs, a line is printed to stderr now and
then so that a first call does not look hung.

The build needs nothing but ``nvcc``: the libraries export plain C functions that take raw
device pointers, and they are loaded with ``ctypes``.
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
from typing import Dict, List, Optional

CSRC_DIR = os.path.dirname(os.path.abspath(__file__))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC",
                "-Xcompiler", "-fvisibility=hidden"]
#: extra nvcc flags and libraries per source; VAPI_NVCC_FLAGS adds flags to every source
#: (tuning experiments: e.g. -DGV_STAGES_N=6)
EXTRA: Dict[str, List[str]] = {}
_ENV_FLAGS = os.environ.get("VAPI_NVCC_FLAGS", "").split()


class BuildError(RuntimeError):
    pass


HOST_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden"]


def sources() -> List[str]:
    """Names (without extension) of every native source of the package."""
    return sorted(os.path.splitext(f)[0] for f in os.listdir(CSRC_DIR) if f.endswith((".cu", ".cpp")))


def _source(name: str) -> str:
    for ext in (".cu", ".cpp"):
        p = os.path.join(CSRC_DIR, name + ext)
        if os.path.isfile(p):
            return p
    raise BuildError(f"no native source {os.path.join(CSRC_DIR, name)}.cu or .cpp")


def _is_host(name: str) -> bool:
    return _source(name).endswith(".cpp")


def find_cxx() -> str:
    for c in (os.environ.get("VAPI_CXX"), os.environ.get("CXX"), "g++", "c++", "clang++"):
        if not c:
            continue
        path = c if os.path.isabs(c) else shutil.which(c)
        if path and os.access(path, os.X_OK):
            return path
    raise BuildError("no C++ compiler was found (set VAPI_CXX or CXX); the host runtime of vapi_b200 "
                     "cannot be built and there is no fallback")


def find_nvcc() -> str:
    cands = [os.environ.get("VAPI_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"]
    home = os.environ.get("CUDA_HOME") or os.environ.get("CUDA_PATH")
    if home:
        cands.insert(1, os.path.join(home, "bin", "nvcc"))
    for c in cands:
        if c and os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise BuildError("nvcc was not found (set VAPI_NVCC or CUDA_HOME); the CUDA kernels of "
                     "vapi_b200 cannot be built and there is no fallback")


def _headers(name: str) -> List[str]:
    """The package's own headers that ``name``.cu includes, directly or through another."""
    import re
    seen: List[str] = []
    todo = [_source(name)]
    while todo:
        path = todo.pop()
        with open(path, "r", encoding="utf-8") as f:
            for inc in re.findall(r'^\s*#\s*include\s+"([^"]+)"', f.read(), flags=re.M):
                ipath = os.path.join(CSRC_DIR, inc)
                if os.path.isfile(ipath) and ipath not in seen:
                    seen.append(ipath)
                    todo.append(ipath)
    return sorted(seen)


def _digest(name: str) -> str:
    h = hashlib.sha256()
    for path in [_source(name)] + _headers(name):
        with open(path, "rb") as f:
            h.update(f.read())
        h.update(b"\0")
    flags = HOST_FLAGS if _is_host(name) else ARCH_FLAGS + COMMON_FLAGS + _ENV_FLAGS
    h.update(" ".join(flags + EXTRA.get(name, [])).encode())
    return h.hexdigest()[:12]


def _build_dirs() -> List[str]:
    """Where a library may live: in the tree first, else a per-user temporary folder."""
    dirs = []
    env = os.environ.get("VAPI_BUILD_DIR")
    if env:
        dirs.append(env)
    dirs.append(os.path.join(CSRC_DIR, "_build"))
    dirs.append(os.path.join(tempfile.gettempdir(), f"vapi_b200-build-{os.getuid()}"))
    return dirs


def library_path(name: str) -> Optional[str]:
    """Path of an up-to-date built library for ``name`` or None."""
    fname = f"lib{name}-{_digest(name)}.so"
    for d in _build_dirs():
        p = os.path.join(d, fname)
        if os.path.isfile(p):
            return p
    return None


def _writable_dir() -> str:
    last = None
    for d in _build_dirs():
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".probe-{os.getpid()}-{threading.get_ident()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return d
        except OSError as e:  # read-only checkout: try the next place
            last = e
    raise BuildError(f"no writable folder for built kernels (tried {_build_dirs()}): {last}")


def build(name: str, verbose: bool = True) -> str:
    """Build one source if needed and return the library path."""
    src = _source(name)
    base = os.path.basename(src)
    have = library_path(name)
    if have:
        return have
    out_dir = _writable_dir()
    out = os.path.join(out_dir, f"lib{name}-{_digest(name)}.so")
    tmp = out + f".tmp{os.getpid()}"
    if _is_host(name):
        cmd = [find_cxx()] + HOST_FLAGS + ["-I", CSRC_DIR] + EXTRA.get(name, []) + ["-o", tmp, src]
    else:
        cmd = [find_nvcc()] + ARCH_FLAGS + COMMON_FLAGS + ["-I", CSRC_DIR] + EXTRA.get(name, []) + _ENV_FLAGS + ["-o", tmp, src]
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    if verbose:
        print(f"[vapi_b200] compiling {base}" + ("" if _is_host(name) else " for sm_100a") + " ...",
              file=sys.stderr, flush=True)
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env, cwd=out_dir)
    done = threading.Event()

    def ticker() -> None:
        while not done.wait(10.0):
            if verbose:
                print(f"[vapi_b200] still compiling {base} ({time.time() - t0:.0f} s)",
                      file=sys.stderr, flush=True)

    th = threading.Thread(target=ticker, daemon=True)
    th.start()
    try:
        log, _ = proc.communicate()
    finally:
        done.set()
    if proc.returncode != 0:
        try:
            os.remove(tmp)
        except OSError:
            pass
        raise BuildError(f"the compiler failed on {base}:\n{' '.join(cmd)}\n{log.decode(errors='replace')}")
    os.replace(tmp, out)
    for old in ([] if _ENV_FLAGS else os.listdir(out_dir)):          # earlier builds of this source are of no use any more
        if old.startswith(f"lib{name}-") and old.endswith(".so") and os.path.join(out_dir, old) != out:
            try:
                os.remove(os.path.join(out_dir, old))
            except OSError:
                pass
    if verbose:
        print(f"[vapi_b200] built {os.path.basename(out)} in {time.time() - t0:.1f} s",
              file=sys.stderr, flush=True)
    return out


def build_all(verbose: bool = True, jobs: int = 4) -> Dict[str, str]:
    """Build every source (in parallel) and return name -> path."""
    names = sources()
    out: Dict[str, str] = {}
    errs: List[str] = []
    lock = threading.Lock()
    sem = threading.Semaphore(max(1, jobs))

    def one(n: str) -> None:
        with sem:
            try:
                p = build(n, verbose)
                with lock:
                    out[n] = p
            except BuildError as e:
                with lock:
                    errs.append(str(e))

    ths = [threading.Thread(target=one, args=(n,)) for n in names]
    for t in ths:
        t.start()
    for t in ths:
        t.join()
    if errs:
        raise BuildError("\n".join(errs))
    return out


if __name__ == "__main__":
    for k, v in build_all().items():
        print(k, v)
