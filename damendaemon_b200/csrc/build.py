"""Compile the CUDA sources of this folder for sm_100a into shared libraries, on first use.

Two libraries: ``core`` (plain CUDA-core kernels of both engine dtypes: embedding,
LayerNorm, float32 GEMM, cache writes, general attention, sampling) and ``tensor``
(tcgen05/TMA GEMM and tensor-core attention, bfloat16 only). A float32 engine needs
only ``core``; what is compiled at the first call is what the model needs.

The sources have no PyTorch headers, so a build is a few nvcc calls of seconds each.
Objects and libraries go to ``_build/`` beside the sources when that is writable, else
to a per-user folder under the system's temporary directory; a content hash of
sources and flags decides whether a library is still current. Nothing is read from
or written to the home directory. While it compiles it prints a line now and then
to stderr.
"""
from __future__ import annotations

import fcntl
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

HERE = Path(__file__).resolve().parent

LIBRARIES = {
    "core": ["errors.cu", "embed.cu", "layernorm.cu", "gemm_simt.cu", "kv_store.cu", "attention_rows.cu",
             "sampling.cu"],
    "tensor": ["errors.cu", "gemm_tcgen05.cu", "attention_decode.cu", "attention_decode_pages.cu", "attention_prefill.cu", "attention_prefill_tcgen05.cu",
               "wait_probe.cu"],
}
HEADERS = ["common.cuh", "tcgen05.cuh", "no_alloc.h"]
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    candidates = []
    for var in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(var):
            candidates.append(Path(os.environ[var]) / "bin" / "nvcc")
    candidates.append(Path("/usr/local/cuda/bin/nvcc"))
    which = shutil.which("nvcc")
    if which:
        candidates.append(Path(which))
    for c in candidates:
        if c.is_file():
            return str(c)
    raise BuildError("nvcc was not found (looked at CUDA_HOME, /usr/local/cuda and PATH); "
                     "the engine has no CPU or library fallback")


def _sources(name):
    return [HERE / s for s in LIBRARIES[name] if (HERE / s).is_file()]


def _digest(name) -> str:
    h = hashlib.sha256()
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    for p in _sources(name) + [HERE / x for x in HEADERS if (HERE / x).is_file()]:
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()[:16]


def build_dir() -> Path:
    local = HERE / "_build"
    try:
        local.mkdir(exist_ok=True)
        probe = local / f".w{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return local
    except OSError:
        pass
    # A shared temporary directory: the folder's name can be guessed, so it is taken only if it is ours alone
    # (made by this user, closed to group and others); a library found in somebody else's folder is never loaded.
    fallback = Path(tempfile.gettempdir()) / f"damendaemon_b200_build_{os.getuid()}"
    try:
        fallback.mkdir(mode=0o700)
    except FileExistsError:
        pass
    info = fallback.lstat()
    import stat
    if not stat.S_ISDIR(info.st_mode) or info.st_uid != os.getuid() or info.st_mode & 0o022:
        raise BuildError(f"{fallback} exists but is not a folder that only user {os.getuid()} can write; "
                         "remove it, or make the package's csrc/_build folder writable")
    return fallback


def library_path(name) -> Path:
    return build_dir() / f"libdamendaemon_b200_{name}.so"


def _say(text):
    print(f"[damendaemon_b200] {text}", file=sys.stderr, flush=True)


def _run(cmd, what):
    done = threading.Event()

    def ticker():
        start = time.time()
        while not done.wait(10.0):
            _say(f"still compiling {what} ({time.time() - start:.0f} s)")
    t = threading.Thread(target=ticker, daemon=True)
    t.start()
    try:
        proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    finally:
        done.set()
    if proc.returncode:
        raise BuildError(f"{what} failed:\n{' '.join(cmd)}\n{proc.stdout}")
    return proc.stdout


def build_library(name, force=False, verbose=True) -> Path:
    """Return the path of an up-to-date library, compiling it if needed."""
    if name not in LIBRARIES:
        raise BuildError(f"unknown library {name!r}")
    out_dir = build_dir()
    lib, stamp = library_path(name), out_dir / f"{name}.digest"
    digest = _digest(name)
    with (out_dir / f"{name}.lock").open("w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and lib.is_file() and stamp.is_file() and stamp.read_text() == digest:
            return lib
        nvcc = find_nvcc()
        sources = _sources(name)
        if verbose:
            _say(f"compiling the '{name}' kernels for sm_100a ({len(sources)} files) into {out_dir}")
        start = time.time()

        def compile_one(src):
            obj = out_dir / f"{name}_{src.stem}.o"
            _run([nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(HERE), "-c", str(src), "-o", str(obj)], src.name)
            if verbose:
                _say(f"compiled {src.name} ({time.time() - start:.0f} s)")
            return obj
        with ThreadPoolExecutor(max_workers=min(len(sources), os.cpu_count() or 2)) as pool:
            objects = list(pool.map(compile_one, sources))
        tmp = lib.with_suffix(f".{os.getpid()}.tmp")
        _run([nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp), *map(str, objects)], f"linking {lib.name}")
        tmp.replace(lib)
        stamp.write_text(digest)
        if verbose:
            _say(f"built {lib.name} in {time.time() - start:.0f} s")
    return lib


def build_all(force=False):
    return {name: build_library(name, force=force) for name in LIBRARIES}


if __name__ == "__main__":
    for name, path in build_all(force="--force" in sys.argv).items():
        print(name, path)
