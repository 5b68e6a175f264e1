"""Compiles the CUDA sources under `wllm_b200/csrc` into shared objects and loads them.

Every kernel family is one `.cu` file with plain C entry points (`extern "C"`,
raw pointers and a stream), compiled by `nvcc` for sm_100a on first use and
loaded with `ctypes`.  A family is compiled only when a model asks for it, so
the first call of a bfloat16 model does not pay for the float32 kernels.  The
object's file name carries a hash of the sources, the headers beside them and
the flags, so an edited kernel is rebuilt and an unchanged one is found again.

Objects go to `wllm_b200/csrc/_build/` inside the checkout; if that folder cannot
be written they go to a per-user folder under the system's temporary directory.
There is no fallback of any other kind: without `nvcc`, or when the compile
fails, `KernelBuildError` is raised with the compiler's output.
"""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


class KernelBuildError(RuntimeError):
    """The CUDA extension could not be built or loaded."""


_loaded: dict[str, ctypes.CDLL] = {}
_plain: dict[str, ctypes.CDLL] = {}          # families built without defines, by name alone
_lock = threading.Lock()


def _nvcc() -> str:
    for cand in (os.environ.get("WLLM_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelBuildError("nvcc not found (looked at $WLLM_NVCC, PATH and /usr/local/cuda/bin): "
                           "the engine's kernels are compiled from source and have no other implementation")


def _build_dir() -> str:
    first = os.path.join(CSRC, "_build")
    for cand in (first, os.path.join(tempfile.gettempdir(), f"wllm_b200_build_{os.getuid()}")):
        try:
            os.makedirs(cand, exist_ok=True)
            fd, probe = tempfile.mkstemp(prefix=".probe", dir=cand)
            os.close(fd)
            os.unlink(probe)
            return cand
        except OSError:
            continue
    raise KernelBuildError(f"no writable folder for compiled kernels (tried {first} and the temporary directory)")


def _deps(source: str) -> list[str]:
    """The source and every file of this folder it includes, directly or not."""
    seen, todo = [], [source]
    while todo:
        path = todo.pop()
        if path in seen or not os.path.isfile(path):
            continue
        seen.append(path)
        with open(path, "r", encoding="utf-8") as f:
            for line in f:
                line = line.strip()
                if line.startswith("#include \""):
                    todo.append(os.path.join(CSRC, line.split('"')[1]))
    return [source] + sorted(p for p in seen if p != source)


def _key(source: str, flags: list[str]) -> str:
    h = hashlib.sha256()
    for path in _deps(source):
        with open(path, "rb") as f:
            h.update(os.path.basename(path).encode() + b"\0" + f.read() + b"\0")
    h.update(" ".join(ARCH_FLAGS + BASE_FLAGS + flags).encode())
    return h.hexdigest()[:16]


def library_path(family: str, defines: dict | None = None) -> tuple[str, list[str], str]:
    source = os.path.join(CSRC, family + ".cu")
    if not os.path.isfile(source):
        raise KernelBuildError(f"no kernel source {source}")
    flags = [f"-D{k}={v}" for k, v in sorted((defines or {}).items())]
    tag = "".join(f"_{k.lower()}{v}" for k, v in sorted((defines or {}).items()))
    name = f"wllm_{family}{tag}-{_key(source, flags)}.so"
    return source, flags, name


def compile_family(family: str, defines: dict | None = None, verbose: bool = True) -> str:
    """Path of the built object of a family, compiling it if it is not there yet."""
    source, flags, name = library_path(family, defines)
    for cand in (os.path.join(CSRC, "_build"), os.path.join(tempfile.gettempdir(), f"wllm_b200_build_{os.getuid()}")):
        if os.path.isfile(os.path.join(cand, name)):
            return os.path.join(cand, name)
    out_dir = _build_dir()
    out = os.path.join(out_dir, name)
    with open(out + ".lock", "w") as lockfile:
        fcntl.flock(lockfile, fcntl.LOCK_EX)   # one compile per object; a second process waits and then finds the file
        try:
            if os.path.isfile(out):
                return out
            tmp = out + f".tmp{os.getpid()}"
            cmd = [_nvcc()] + ARCH_FLAGS + BASE_FLAGS + flags + ["-I", CSRC, "-o", tmp, source, "-lcuda"]
            if verbose:
                print(f"[wllm_b200] compiling {family}{' ' + ' '.join(flags) if flags else ''} for sm_100a ...",
                      file=sys.stderr, flush=True)
            start = time.time()
            proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            done = threading.Event()

            def heartbeat():
                while not done.wait(10.0):
                    if verbose:
                        print(f"[wllm_b200]   still compiling {family} ({time.time() - start:.0f} s)",
                              file=sys.stderr, flush=True)
            t = threading.Thread(target=heartbeat, daemon=True)
            t.start()
            output, _ = proc.communicate()
            done.set()
            if proc.returncode != 0:
                if os.path.exists(tmp):
                    os.unlink(tmp)
                raise KernelBuildError(f"nvcc failed on {source} (exit {proc.returncode}):\n{' '.join(cmd)}\n{output}")
            os.replace(tmp, out)
            prefix = name.rsplit("-", 1)[0] + "-"
            for old in os.listdir(out_dir):      # objects of earlier versions of this family and variant, and their locks
                if old.startswith(prefix) and old.endswith((".so", ".so.lock")) and not old.startswith(name):
                    try:
                        os.unlink(os.path.join(out_dir, old))
                    except OSError:
                        pass
            if verbose:
                print(f"[wllm_b200]   {family} done in {time.time() - start:.1f} s", file=sys.stderr, flush=True)
        finally:
            fcntl.flock(lockfile, fcntl.LOCK_UN)
    return out


def load_family(family: str, defines: dict | None = None) -> ctypes.CDLL:
    """The loaded library of a kernel family (compiled on first use)."""
    if not defines:
        lib = _plain.get(family)          # the common case, asked at every launch: no key to build, no lock
        if lib is not None:
            return lib
    key = family + repr(sorted((defines or {}).items()))
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            path = compile_family(family, defines)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from e
            _loaded[key] = lib
        if not defines:
            _plain[family] = lib
        return lib


def loaded_libraries() -> list[str]:
    return sorted(getattr(lib, "_name", "?") for lib in _loaded.values())
