"""Compiles the CUDA sources under ``csrc/`` for sm_100a with nvcc and loads them.

Each library is a set of ``.cu`` files plus preprocessor defines (a head size,
for instance), compiled once into ``csrc/_build/<name>-<hash>.so`` and loaded
with ctypes.  The hash covers the sources, the headers beside them, the defines
and the flags, so a stale binary is never loaded, and a binary built on another
machine from the same sources is reused as it is.  What a model needs is compiled
at its first use; a line is printed every few seconds meanwhile.  If neither a
built library nor nvcc can be found the import fails: there is no other path.
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
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]

_loaded: dict = {}
_lock = threading.Lock()


class KernelBuildError(RuntimeError):
    pass


def _nvcc() -> str | None:
    for candidate in (os.environ.get("QIL_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).is_file():
            return candidate
    return None


def build_dir() -> Path:
    """In-tree when the tree is writable, else a per-user folder under the temp dir."""
    override = os.environ.get("QIL_BUILD_DIR")
    candidates = [Path(override)] if override else []
    candidates.append(CSRC / "_build")
    candidates.append(Path(tempfile.gettempdir()) / f"qil_b200_build_{os.getuid()}")
    for folder in candidates:
        try:
            folder.mkdir(parents=True, exist_ok=True)
            probe = folder / f".write_probe_{os.getpid()}"
            probe.write_text("")
            probe.unlink()
            return folder
        except OSError:
            continue
    raise KernelBuildError("no writable folder for compiled kernels")


def _digest(sources, defines, flags, depends=()) -> str:
    h = hashlib.sha256()
    for path in sorted(CSRC.glob("*.cuh")) + [CSRC / s for s in list(sources) + list(depends)]:
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(repr(sorted(defines.items())).encode())
    h.update(repr(flags).encode())
    return h.hexdigest()[:16]


def library_path(name: str, sources, defines=None, depends=()) -> tuple:
    """``depends``: files under csrc/ that the sources include beside the ``.cuh`` headers."""
    defines = dict(defines or {})
    extra = os.environ.get("QIL_NVCC_FLAGS", "").split()
    flags = ARCH_FLAGS + BASE_FLAGS + extra
    tag = _digest(sources, defines, flags, depends)
    return f"{name}-{tag}.so", flags, defines


def _find_built(filename: str) -> Path | None:
    folders = [CSRC / "_build", Path(tempfile.gettempdir()) / f"qil_b200_build_{os.getuid()}"]
    if os.environ.get("QIL_BUILD_DIR"):
        folders.insert(0, Path(os.environ["QIL_BUILD_DIR"]))
    for folder in folders:
        candidate = folder / filename
        if candidate.is_file():
            return candidate
    return None


def _run_with_progress(commands, label):
    """Run the compile commands in parallel; print a line every few seconds."""
    started = time.time()
    procs = [(cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
             for cmd in commands]
    last = started
    while any(p.poll() is None for _, p in procs):
        time.sleep(0.2)
        if time.time() - last >= 5.0:
            last = time.time()
            print(f"[qil-b200] compiling {label} for sm_100a ... {int(last - started)} s", file=sys.stderr, flush=True)
    for cmd, p in procs:
        out = p.stdout.read()
        if p.returncode != 0:
            raise KernelBuildError(f"nvcc failed ({p.returncode}): {' '.join(cmd)}\n{out}")
        if os.environ.get("QIL_BUILD_VERBOSE") and out.strip():
            print(out, file=sys.stderr)


def build(name: str, sources, defines=None, depends=()) -> Path:
    """Return the path of the compiled library, compiling it first if need be."""
    filename, flags, defines = library_path(name, sources, defines, depends)
    found = _find_built(filename)
    if found is not None:
        return found
    nvcc = _nvcc()
    if nvcc is None:
        raise KernelBuildError(
            f"compiled kernels {filename} not found and nvcc is not available to build them")
    folder = build_dir()
    target = folder / filename
    print(f"[qil-b200] compiling {name} ({len(sources)} file(s)) for sm_100a; this happens once",
          file=sys.stderr, flush=True)
    started = time.time()
    work = Path(tempfile.mkdtemp(prefix=f"{name}-", dir=folder))
    try:
        define_flags = [f"-D{k}={v}" for k, v in sorted(defines.items())]
        objects, commands = [], []
        for source in sources:
            obj = work / (Path(source).stem + ".o")
            objects.append(str(obj))
            commands.append([nvcc, *flags, *define_flags, "-I", str(CSRC), "-c", str(CSRC / source), "-o", str(obj)])
        _run_with_progress(commands, name)
        partial = work / filename
        _run_with_progress([[nvcc, *ARCH_FLAGS, "-shared", "-o", str(partial), *objects]], name + " (link)")
        os.replace(partial, target)   # atomic: another process either sees the whole file or none
    finally:
        shutil.rmtree(work, ignore_errors=True)
    print(f"[qil-b200] compiled {name} in {time.time() - started:.0f} s", file=sys.stderr, flush=True)
    return target


def load(name: str, sources, defines=None, depends=()) -> ctypes.CDLL:
    key = (name, tuple(sources), tuple(sorted((defines or {}).items())))
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            path = build(name, sources, defines, depends)
            lib = ctypes.CDLL(str(path))
            lib.qil_last_error.restype = ctypes.c_char_p
            lib._qil_path = str(path)
            _loaded[key] = lib
        return lib
