"""Compiles the CUDA sources of this package for sm_100a and loads them.

Each group of kernels is one ``.cu`` file under ``csrc/`` built by ``nvcc`` into
one shared library with extern "C" launchers, loaded with ``ctypes``.  A library
is compiled at its first use when no up-to-date build exists (the file name
carries a hash of the sources and flags), so a fresh checkout compiles only what
the model that is run needs; while ``nvcc`` works, a line is printed every few
seconds.  Built files go to ``csrc/_build`` inside the package when that is
writable, else to ``$DIB200_BUILD_DIR`` or a per-user folder under the system
temporary directory.

There is no fallback: if a library cannot be built or loaded, the caller gets a
``KernelBuildError``.
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
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"

# library name -> source file (headers every source includes are hashed too)
SOURCES = {
    "elementwise": "elementwise.cu",
    "sampling": "sampling.cu",
    "gemm_fp32": "gemm_fp32.cu",
    "attention_generic": "attention_generic.cu",
    "attention_bf16": "attention_bf16.cu",
    "gemm_bf16": "gemm_bf16.cu",
    "gemm_bf16_large": "gemm_bf16_large.cu",
    "decode_attention_noalloc": "decode_attention_noalloc.cu",
    "attention_prefill_tc": "attention_prefill_tc.cu",
}
HEADERS = ("common.cuh", "attention_merge.cuh")
# further headers a library includes
EXTRA_HEADERS = {
    "attention_bf16": ("attention_bf16_kernels.cuh",),
    "decode_attention_noalloc": ("attention_bf16_kernels.cuh", "decode_attention_noalloc.h"),
    "attention_prefill_tc": ("attention_bf16_kernels.cuh",),
}

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-shared", "-Xcompiler", "-fPIC",
]
# extra flags / link libraries per library
EXTRA_FLAGS = {
    "gemm_bf16": ["-lcuda"],
    "gemm_bf16_large": ["-lcuda"],
}


class KernelBuildError(RuntimeError):
    pass


def register_source(name: str, path, headers=(), flags=()) -> None:
    """Make a CUDA source outside ``csrc/`` buildable and loadable under ``name`` with the
    flags of this package (it may include the package's headers)."""
    SOURCES[name] = str(Path(path).resolve())
    if headers:
        EXTRA_HEADERS[name] = tuple(headers)
    if flags:
        EXTRA_FLAGS[name] = list(flags)


_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()
_dir_lock = threading.Lock()


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise KernelBuildError("nvcc not found (looked at $NVCC, PATH and /usr/local/cuda/bin); "
                           "the CUDA kernels of this package cannot be built")


_build_dir_cache: list = []


def _build_dir() -> Path:
    with _dir_lock:
        if not _build_dir_cache:
            _build_dir_cache.append(_pick_build_dir())
        return _build_dir_cache[0]


def _pick_build_dir() -> Path:
    env = os.environ.get("DIB200_BUILD_DIR")
    cands = [Path(env)] if env else []
    cands.append(CSRC / "_build")
    cands.append(Path(tempfile.gettempdir()) / f"dib200_build_{os.getuid()}")
    for d in cands:
        try:
            d.mkdir(parents=True, exist_ok=True)
            probe = d / f".w{os.getpid()}"
            probe.write_text("")
            probe.unlink()
            return d
        except OSError:
            continue
    raise KernelBuildError(f"no writable build folder among {cands}")


def _digest(name: str) -> str:
    h = hashlib.sha256()
    for f in (SOURCES[name],) + HEADERS + EXTRA_HEADERS.get(name, ()):
        h.update((CSRC / f).read_bytes())
    h.update(" ".join(NVCC_FLAGS + EXTRA_FLAGS.get(name, [])).encode())
    return h.hexdigest()[:16]


def library_path(name: str) -> Path:
    return _build_dir() / f"libdib200_{name}_{_digest(name)}.so"


def _find_built(name: str) -> Path | None:
    """An up-to-date build in any of the candidate folders (a read-only in-tree
    build still counts)."""
    fname = f"libdib200_{name}_{_digest(name)}.so"
    for d in (os.environ.get("DIB200_BUILD_DIR"), CSRC / "_build",
              Path(tempfile.gettempdir()) / f"dib200_build_{os.getuid()}"):
        if d and (Path(d) / fname).exists():
            return Path(d) / fname
    return None


def compile_library(name: str, verbose: bool = True) -> Path:
    """Compile one library if no up-to-date build exists; returns its path."""
    if name not in SOURCES:
        raise KernelBuildError(f"unknown kernel library {name!r}; known: {sorted(SOURCES)}")
    built = _find_built(name)
    if built is not None:
        return built
    out = library_path(name)
    tmp = out.with_suffix(f".tmp{os.getpid()}.so")
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(CSRC), str(CSRC / SOURCES[name]), "-o", str(tmp),
           *EXTRA_FLAGS.get(name, [])]
    t0 = time.time()
    if verbose:
        print(f"[dib200] compiling {Path(SOURCES[name]).name} for sm_100a (first use) ...", file=sys.stderr,
              flush=True)
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def ticker():
        while not done.wait(10.0):
            if verbose:
                print(f"[dib200]   still compiling {SOURCES[name]} ({time.time() - t0:.0f} s)",
                      file=sys.stderr, flush=True)

    th = threading.Thread(target=ticker, daemon=True)
    th.start()
    try:
        log, _ = proc.communicate()
    finally:
        done.set()
    if proc.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise KernelBuildError(f"nvcc failed for {SOURCES[name]}:\n{' '.join(cmd)}\n{log}")
    os.replace(tmp, out)
    for old in out.parent.glob(f"libdib200_{name}_*.so"):
        if old != out and ".tmp" not in old.name:
            old.unlink(missing_ok=True)
    if verbose:
        print(f"[dib200] built {out.name} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return out


def compile_all(names=None, verbose: bool = True) -> dict[str, Path]:
    """Compile several libraries at once (one nvcc process each, in parallel)."""
    names = list(names or [n for n in SOURCES if not Path(SOURCES[n]).is_absolute()])
    names = [n for n in names if (CSRC / SOURCES[n]).exists()]
    out: dict[str, Path] = {}
    errors: list[str] = []

    def work(n):
        try:
            out[n] = compile_library(n, verbose)
        except KernelBuildError as e:  # collect, report all
            errors.append(str(e))

    threads = [threading.Thread(target=work, args=(n,)) for n in names]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        raise KernelBuildError("\n\n".join(errors))
    return out


def load_library(name: str) -> ctypes.CDLL:
    """The loaded library, compiled first if needed."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = compile_library(name)
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from e
            _loaded[name] = lib
        return lib
