"""Build and load the sm_100a kernel libraries.

Each ``.cu`` file here becomes one shared object, compiled with nvcc the first
time something needs it and kept beside the sources under ``_build/`` (or in a
per-user folder under the system's temporary directory when the package folder
cannot be written).  The object's file name carries a hash of its sources and
flags, so an edited source is rebuilt and a stale object is never loaded.
There is no other implementation behind these libraries: if nvcc or a library
is missing the caller gets ``KernelBuildError``.
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
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import Dict, Iterable, List, Optional

HERE = Path(__file__).resolve().parent

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17", "--shared",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]

# library name -> (source file, extra nvcc flags)
LIBRARIES: Dict[str, tuple] = {
    "elementwise": ("elementwise.cu", []),
    "gemm_f32": ("gemm_f32.cu", []),
    "rope_cache": ("rope_cache.cu", []),
    "attention_ref": ("attention_ref.cu", []),
    "sampling": ("sampling.cu", []),
    "attention_decode": ("attention_decode.cu", []),
    "gemm_tcgen05": ("gemm_tcgen05.cu", []),
    "attention_prefill": ("attention_prefill.cu", []),
    "attention_prefill_tc": ("attention_prefill_tc.cu", []),
    "attention_prefill_twin": ("attention_prefill_twin.cu", []),
    "attention_decode_noalloc": ("attention_decode_noalloc.cu", []),
}

_HEADERS = ["common.cuh", "page_map.cuh"]

# The host library (plain C, the system compiler): the safetensors reader and the sampler.
HOST_LIBRARY = "host"
HOST_SOURCE, HOST_HEADERS = "host/lgml_host.c", ["host/lgml_host.h"]
CC_FLAGS = ["-std=c11", "-O2", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall"]
_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class KernelBuildError(RuntimeError):
    """nvcc is missing, a source does not compile, or the library cannot be loaded."""


def find_nvcc() -> str:
    for cand in (os.environ.get("LGML_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelBuildError("nvcc not found (looked at $LGML_NVCC, PATH, $CUDA_HOME/bin and /usr/local/cuda/bin); "
                           "the sm_100a kernels have no other implementation")


def find_cc() -> str:
    for cand in (os.environ.get("LGML_CC"), os.environ.get("CC"), shutil.which("cc"), shutil.which("gcc"), shutil.which("clang")):
        if cand and (os.path.isfile(cand) or shutil.which(cand)):
            return cand
    raise KernelBuildError("no C compiler found (looked at $LGML_CC, $CC, cc, gcc, clang) for the host library")


def _writable(d: Path) -> bool:
    try:
        d.mkdir(parents=True, exist_ok=True)
        probe = d / f".probe-{os.getpid()}-{threading.get_ident()}"
        probe.write_bytes(b"")
        probe.unlink()
        return True
    except OSError:
        return False


_build_dir: Optional[Path] = None


def build_dir() -> Path:
    global _build_dir
    if _build_dir is None:
        _build_dir = _find_build_dir()
    return _build_dir


def _find_build_dir() -> Path:
    env = os.environ.get("LGML_BUILD_DIR")
    if env and _writable(Path(env)):
        return Path(env)
    in_tree = HERE / "_build"
    if _writable(in_tree):
        return in_tree
    fallback = Path(tempfile.gettempdir()) / f"lgml_b200_build_{os.getuid()}"
    if _writable(fallback):
        return fallback
    raise KernelBuildError(f"no writable build folder: tried {in_tree} and {fallback}")


def _digest(name: str) -> str:
    h = hashlib.sha256()
    if name == HOST_LIBRARY:
        files, flags = [HOST_SOURCE] + HOST_HEADERS, CC_FLAGS
    else:
        src, extra = LIBRARIES[name]
        files, flags = [src] + _HEADERS + list(LIBRARY_HEADERS.get(name, [])), NVCC_FLAGS + list(extra)
    for f in files:
        h.update(f.encode())
        h.update((HERE / f).read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:12]


# extra headers a library includes (its hash covers them)
LIBRARY_HEADERS: Dict[str, List[str]] = {
    "attention_decode_noalloc": ["attention_decode.cu", "attention_decode_noalloc.h"],
}


def library_path(name: str) -> Path:
    return build_dir() / f"lgml_{name}.{_digest(name)}.so"


def _say(msg: str) -> None:
    print(f"[lgml_b200] {msg}", file=sys.stderr, flush=True)


def compile_library(name: str, verbose: bool = True) -> Path:
    """Compile one library if its object is not there yet; returns the object's path."""
    if name not in LIBRARIES and name != HOST_LIBRARY:
        raise KernelBuildError(f"unknown kernel library '{name}'")
    out = library_path(name)
    if out.exists():
        return out
    tmp = out.with_suffix(f".tmp{os.getpid()}.so")
    if name == HOST_LIBRARY:
        src = HOST_SOURCE
        cmd = [find_cc()] + CC_FLAGS + ["-I", str(HERE / "host"), str(HERE / src), "-o", str(tmp), "-lm"]
        if verbose:
            _say(f"compiling {src} ...")
    else:
        src, extra = LIBRARIES[name]
        cmd = [find_nvcc()] + NVCC_FLAGS + list(extra) + ["-I", str(HERE), str(HERE / src), "-o", str(tmp)]
        if verbose:
            _say(f"compiling {src} for sm_100a ...")
    t0 = time.time()
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    done = threading.Event()

    def ticker():
        while not done.wait(15.0):
            _say(f"still compiling {src} ({time.time() - t0:.0f} s)")

    th = threading.Thread(target=ticker, daemon=True)
    if verbose:
        th.start()
    log, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        try:
            tmp.unlink()
        except OSError:
            pass
        raise KernelBuildError(f"{cmd[0]} failed on {src} (exit {proc.returncode}):\n{log}")
    for old in out.parent.glob(f"lgml_{name}.*.so"):
        if old != tmp:
            try:
                old.unlink()
            except OSError:
                pass
    os.replace(tmp, out)
    if verbose:
        _say(f"built {out.name} in {time.time() - t0:.1f} s")
    return out


def load(name: str) -> ctypes.CDLL:
    """The loaded library ``name``, compiled first if need be."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = compile_library(name)
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from None
            _loaded[name] = lib
        return lib


def build_all(names: Optional[Iterable[str]] = None, jobs: int = 0, verbose: bool = True) -> List[Path]:
    """Compile every library (in parallel); used by the build check and before a first run."""
    names = list(names or list(LIBRARIES) + [HOST_LIBRARY])
    jobs = jobs or min(len(names), os.cpu_count() or 1)
    with ThreadPoolExecutor(max_workers=jobs) as ex:
        return list(ex.map(lambda n: compile_library(n, verbose), names))


def loaded_libraries() -> List[str]:
    return sorted(_loaded)
