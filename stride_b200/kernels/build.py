"""Compiles the CUDA sources under `stride_b200/csrc` for sm_100a and loads them.

Each `.cu` file becomes one shared library with a plain C interface, loaded with
ctypes; there is no dependency on torch's headers, so a file compiles in seconds.
A library is built the first time something needs it, into `csrc/_build/` (or, if
the package folder cannot be written, into a per-user folder under the system's
temporary directory). Its file name carries a hash of the source, the shared
header and the flags, so an edited source is never served by a stale binary.

There is no other implementation behind these libraries: if one cannot be built
or loaded, the call raises.
"""
from __future__ import annotations

import ctypes
import fcntl
import functools
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

CSRC = Path(__file__).resolve().parent.parent / "csrc"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

# library name -> source file (relative to csrc/, or absolute for libraries registered from outside the package);
# every name here is built by `build_all()`.
SOURCES = {
    "elementwise": "elementwise.cu",
    "norm": "norm.cu",
    "gemm_f32": "gemm_f32.cu",
    "attention_generic": "attention_generic.cu",
    "sampling": "sampling.cu",
    "gemm_tc": "gemm_tc.cu",
    "attention_tc": "attention_tc.cu",
    "attention_tc5": "attention_tc5.cu",
    "decode_chain": "decode_chain.cu",
    "runtime": "runtime.cpp",        # host code only: the cache manager's books and the scheduler's decisions
}
HOST_FLAGS = ["-O2", "-std=c++17", "-g1", "-shared", "-fPIC", "-fvisibility=hidden"]


def register_kernel_library(name: str, source) -> None:
    """Make `source` (a `.cu` file, or a `.cpp` file of host code, anywhere on disk) known as the kernel library `name`:
    from then on `library(name)` compiles it like the package's own sources (nvcc for sm_100a, the package's `csrc` on
    the include path, so it may use `common.cuh` and `step_ops.h`) and loads it; a part outside the package names it in
    `kernel_libraries()` and in `program.add(name, function, ...)`. Its functions follow the package's convention:
    `extern "C"`, 0 on success, and an `sb_last_error()` (SB_DEFINE_LAST_ERROR) for the reason otherwise."""
    path = Path(source).resolve()
    if not path.is_file():
        raise BuildError(f"kernel library '{name}': no source file at {path}")
    known = SOURCES.get(name)
    if known is not None and _source(name) != path:
        raise BuildError(f"a kernel library named '{name}' is already registered with another source ({_source(name)})")
    SOURCES[name] = str(path)


def _source(name: str) -> Path:
    try:
        p = Path(SOURCES[name])
    except KeyError:
        raise BuildError(f"no kernel library named '{name}' (known: {', '.join(sorted(SOURCES))}); "
                         f"register_kernel_library(name, source) adds one") from None
    return p if p.is_absolute() else CSRC / p

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise BuildError("nvcc not found: the CUDA kernels of stride_b200 cannot be built (set NVCC or put nvcc on PATH)")


def _host_compiler() -> str:
    for cand in (os.environ.get("CXX"), "g++", "c++"):
        found = cand and shutil.which(cand)
        if found:
            return found
    raise BuildError("no C++ compiler found: the host runtime of stride_b200 cannot be built (set CXX)")


@functools.lru_cache(maxsize=1)
def _build_dir() -> Path:
    d = CSRC / "_build"
    try:
        d.mkdir(exist_ok=True)
        probe = d / f".w{os.getpid()}"
        probe.write_bytes(b"")
        probe.unlink()
        return d
    except OSError:
        d = Path(tempfile.gettempdir()) / f"stride_b200-build-{os.getuid()}"
        d.mkdir(parents=True, exist_ok=True)
        return d


def _digest(src: Path) -> str:
    h = hashlib.sha256()
    h.update(src.read_bytes())
    for header in sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(header.read_bytes())
    h.update(" ".join(HOST_FLAGS if src.suffix == ".cpp" else ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()[:12]


def library_path(name: str) -> Path:
    src = _source(name)
    return _build_dir() / f"{name}-{_digest(src)}.so"


def _compile(name: str, out: Path) -> None:
    src = _source(name)
    tmp = out.with_suffix(f".tmp{os.getpid()}.so")
    if src.suffix == ".cpp":
        cmd = [_host_compiler(), *HOST_FLAGS, f"-I{CSRC}", "-o", str(tmp), str(src)]
        print(f"[stride_b200] compiling {src.name} for the host ...", file=sys.stderr, flush=True)
    else:
        cmd = [_nvcc(), *ARCH_FLAGS, *NVCC_FLAGS, f"-I{CSRC}", "-o", str(tmp), str(src)]
        print(f"[stride_b200] compiling {src.name} for sm_100a ...", file=sys.stderr, flush=True)
    t0 = time.time()
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env, cwd=tempfile.gettempdir())
    while True:
        try:
            out_text, _ = proc.communicate(timeout=10)
            break
        except subprocess.TimeoutExpired:
            print(f"[stride_b200]   still compiling {src.name} ({time.time() - t0:.0f} s)", file=sys.stderr, flush=True)
    if proc.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise BuildError(f"{Path(cmd[0]).name} failed on {src}:\n{out_text.decode(errors='replace')}")
    os.replace(tmp, out)
    for stale in out.parent.glob(f"{name}-*.so"):
        if stale != out and ".tmp" not in stale.name:
            stale.unlink(missing_ok=True)
    print(f"[stride_b200] built {out.name} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)


def ensure_built(name: str) -> Path:
    out = library_path(name)
    if out.exists():
        return out
    lock_file = out.parent / f".{name}.lock"
    with open(lock_file, "w") as lf:
        fcntl.flock(lf, fcntl.LOCK_EX)
        try:
            if not out.exists():
                _compile(name, out)
        finally:
            fcntl.flock(lf, fcntl.LOCK_UN)
    return out


def library(name: str) -> ctypes.CDLL:
    """The loaded library `name`, compiled first if its binary is missing or stale."""
    lib = _loaded.get(name)
    if lib is not None:
        return lib
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = ensure_built(name)
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as e:
                raise BuildError(f"cannot load {path}: {e}") from e
            lib.sb_last_error.restype = ctypes.c_char_p
            _loaded[name] = lib
    return lib


def build_all(names=None) -> list[Path]:
    """Compile every library (in parallel); returns their paths."""
    names = list(names or SOURCES)
    _build_dir()
    with ThreadPoolExecutor(max_workers=min(8, len(names))) as pool:
        return list(pool.map(ensure_built, names))
