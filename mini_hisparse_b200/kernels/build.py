"""Compile the CUDA sources of ``csrc/`` for sm_100a and load them with ctypes.

Each ``.cu`` file becomes one shared library, built the first time something asks for it:
a float32 model never compiles the tensor-core kernels.  Libraries are named after a hash
of their source, every header of ``csrc/`` and the flags, so a stale build is never loaded.  They
are built in-tree (``csrc/_build``) when that folder can be written, else under the
system's temporary folder; no home directory and no network is needed.
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

CSRC = Path(__file__).resolve().parent.parent / "csrc"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--shared", "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]

# Every module the package has; __graft_entry__.build() compiles all of them.
MODULES = ("elementwise", "gemm_simt", "gemm_tc", "attention_simt", "attention_mma", "attention_tma", "attention_decode",
           "attention_tc", "sampling")


class KernelBuildError(RuntimeError):
    pass


_lock = threading.Lock()
_loaded: dict[str, ctypes.CDLL] = {}


def _say(msg: str) -> None:
    print(f"[mini_hisparse_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise KernelBuildError(
        "nvcc was not found (looked at $NVCC, PATH and /usr/local/cuda/bin): the CUDA kernels of "
        "this engine cannot be built, and there is no fallback path"
    )


def _writable(folder: Path) -> bool:
    try:
        folder.mkdir(parents=True, exist_ok=True)
        probe = folder / f".probe-{os.getpid()}-{threading.get_ident()}"
        probe.write_text("")
        probe.unlink()
        return True
    except OSError:
        return False


def build_dir() -> Path:
    env = os.environ.get("MHB200_BUILD_DIR")
    if env and _writable(Path(env)):
        return Path(env)
    local = CSRC / "_build"
    if _writable(local):
        return local
    fallback = Path(tempfile.gettempdir()) / f"mini_hisparse_b200-build-{os.getuid()}"
    if _writable(fallback):
        return fallback
    raise KernelBuildError(f"no writable build folder: tried {local} and {fallback}")


def _digest(module: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for path in sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + [CSRC / f"{module}.cu"]:
        h.update(path.name.encode())
        h.update(path.read_bytes())
    return h.hexdigest()[:16]


def library_path(module: str) -> Path:
    return build_dir() / f"libmhb_{module}_{_digest(module)}.so"


def compile_module(module: str, verbose: bool = True) -> Path:
    src = CSRC / f"{module}.cu"
    if not src.exists():
        raise KernelBuildError(f"no such kernel module: {src}")
    out = library_path(module)
    if out.exists():
        return out
    nvcc = find_nvcc()
    tmp = out.with_suffix(f".tmp{os.getpid()}.so")
    cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), str(src), "-o", str(tmp)]
    start = time.time()
    if verbose:
        _say(f"compiling {src.name} for sm_100a ...")
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    # a line now and then while nvcc works
    while True:
        try:
            output, _ = proc.communicate(timeout=15)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                _say(f"  still compiling {src.name} ({time.time() - start:.0f} s)")
    if proc.returncode != 0:
        try:
            tmp.unlink()
        except OSError:
            pass
        raise KernelBuildError(f"nvcc failed on {src.name}:\n{output}")
    os.replace(tmp, out)
    for stale in out.parent.glob(f"libmhb_{module}_*.so"):     # older builds of this module
        if stale != out:
            try:
                stale.unlink()
            except OSError:
                pass
    if verbose:
        _say(f"built {out.name} in {time.time() - start:.1f} s")
    return out


def load(module: str) -> ctypes.CDLL:
    """The library of one module, compiled at the first call."""
    with _lock:
        lib = _loaded.get(module)
    if lib is not None:
        return lib
    path = compile_module(module)
    with _lock:
        lib = _loaded.get(module)
        if lib is None:
            lib = ctypes.CDLL(str(path))
            lib.mhb_last_error.restype = ctypes.c_char_p
            _loaded[module] = lib
    return lib


def build_all(modules=MODULES, jobs: int | None = None) -> list[Path]:
    """Compile several modules in parallel (used before a model's first step and by build())."""
    modules = list(modules)
    todo = [m for m in modules if not library_path(m).exists()]
    if todo:
        with ThreadPoolExecutor(max_workers=jobs or min(len(todo), os.cpu_count() or 2)) as pool:
            list(pool.map(compile_module, todo))
    return [library_path(m) for m in modules]
