"""Compile the CUDA sources for sm_100a and load them with ctypes.

Each ``<name>.cu`` in this folder becomes one shared library, built at the first call that
needs it (so a model compiles only what it uses) and kept beside the sources under
``_build/`` (or under ``$SNOWLLM_B200_BUILD_DIR``, or a temporary folder when the checkout
is read-only).  The library name carries a hash of the sources and flags, so an edited
kernel is rebuilt and a stale one is never loaded.  There is no fallback: without nvcc or
without a built library the call fails with an error that says so.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import pathlib
import re
import shutil
import subprocess
import sys
import tempfile
import threading
import time

from ..errors import KernelError

HERE = pathlib.Path(__file__).resolve().parent
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden"]
LIBRARIES = ("elementwise", "rope_cache", "short_conv", "attention", "attention_mma", "attention_tc", "gemm", "gemm_skinny", "gemm_tc", "gemm_tc2", "moe", "sampling")
EXTRA_LINK: dict[str, list[str]] = {}
# more nvcc flags from the environment (-D switches of an experiment); they enter the library's hash
ENV_FLAGS = os.environ.get("SNOWLLM_B200_NVCC_FLAGS", "").split()

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


def _nvcc() -> str:
    for cand in (os.environ.get("SNOWLLM_B200_NVCC"),
                 shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise KernelError("nvcc was not found (PATH, $CUDA_HOME, /usr/local/cuda): the sm_100a kernels "
                      "cannot be built, and this engine has no other code path")


def _build_dir() -> pathlib.Path:
    env = os.environ.get("SNOWLLM_B200_BUILD_DIR")
    for cand in ([pathlib.Path(env)] if env else []) + [HERE / "_build"]:
        try:
            cand.mkdir(parents=True, exist_ok=True)
            probe = cand / f".w{os.getpid()}"
            probe.write_text("")
            probe.unlink()
            return cand
        except OSError:
            continue
    d = pathlib.Path(tempfile.gettempdir()) / f"snowllm_b200_build_{os.getuid()}"
    d.mkdir(parents=True, exist_ok=True)
    return d


def _digest(name: str) -> str:
    h = hashlib.sha256()
    for f in sorted(HERE.glob("*.cuh")) + sorted(HERE.glob("*.h")) + [HERE / f"{name}.cu"]:
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + ENV_FLAGS + EXTRA_LINK.get(name, [])).encode())
    return h.hexdigest()[:16]


def library_path(name: str) -> pathlib.Path:
    return _build_dir() / f"libsnk_{name}_{_digest(name)}.so"


def _compile(name: str, out: pathlib.Path) -> None:
    src = HERE / f"{name}.cu"
    if not src.exists():
        raise KernelError(f"no CUDA source {src}")
    tmp = out.with_suffix(f".tmp{os.getpid()}.so")
    cmd = [_nvcc(), *ARCH_FLAGS, *NVCC_FLAGS, *ENV_FLAGS, "-I", str(HERE), "-o", str(tmp), str(src),
           *EXTRA_LINK.get(name, [])]
    print(f"[snowllm_b200] compiling {src.name} for sm_100a ...", file=sys.stderr, flush=True)
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    while True:
        try:
            log, _ = proc.communicate(timeout=10)
            break
        except subprocess.TimeoutExpired:
            print(f"[snowllm_b200]   still compiling {src.name} ({time.time() - t0:.0f} s)",
                  file=sys.stderr, flush=True)
    if proc.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise KernelError(f"nvcc failed on {src.name}:\n{log}")
    os.replace(tmp, out)            # atomic: a concurrent process sees the old state or the whole file
    stale = re.compile(rf"libsnk_{re.escape(name)}_[0-9a-f]{{16}}\.so")     # this source's older builds only
    for old in out.parent.glob(f"libsnk_{name}_*.so"):
        if old != out and stale.fullmatch(old.name):
            old.unlink(missing_ok=True)
    print(f"[snowllm_b200] built {out.name} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)


def all_libraries() -> tuple:
    """Every CUDA source of this folder."""
    return tuple(sorted(f.stem for f in HERE.glob("*.cu")))


def build(names=LIBRARIES, parallel: bool = True) -> list[pathlib.Path]:
    """Compile the named libraries where no current build exists; returns their paths."""
    todo = [(n, library_path(n)) for n in names]
    missing = [(n, p) for n, p in todo if not p.exists()]
    if parallel and len(missing) > 1:
        errors: list[BaseException] = []

        def work(n, p):
            try:
                _compile(n, p)
            except BaseException as e:  # noqa: BLE001 - reported below
                errors.append(e)
        threads = [threading.Thread(target=work, args=a) for a in missing]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        if errors:
            raise errors[0]
    else:
        for n, p in missing:
            _compile(n, p)
    return [p for _, p in todo]


def is_loaded(name: str) -> bool:
    """Whether this process has loaded the library of ``<name>.cu``."""
    return name in _loaded


def load(name: str) -> ctypes.CDLL:
    """The library of ``<name>.cu``, compiled first if need be."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = library_path(name)
            if not path.exists():
                _compile(name, path)
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as e:
                raise KernelError(f"cannot load {path}: {e}") from e
            _loaded[name] = lib
        return lib
