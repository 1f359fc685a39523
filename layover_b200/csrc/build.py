"""Compile the .cu sources of this folder for sm_100a and load them with ctypes.

Each source becomes one shared library `_build/<name>-<hash>.so` beside the sources (or in
`$LAYOVER_B200_BUILD_DIR`, or in a per-user temporary folder when the source tree cannot be
written). The hash covers the source, the headers of this folder and the compiler flags, so an
outdated library is never loaded. A library is built the first time one of its functions is
wanted; `ensure_built(names)` builds several in parallel and prints a line every few seconds
while nvcc runs. Nothing here needs a home directory, a network or a GPU.

A part that lives outside this package brings its own kernels with `register_source(name,
path)`: the file is compiled with the same flags (and `-I` this folder, so it may include
`common.cuh`), hashed and loaded like the package's own, and the part names the library in its
`kernel_libraries()`.
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

HERE = Path(__file__).resolve().parent

# name -> (source file, relative to this folder or absolute; extra link flags)
SOURCES: dict[str, tuple[str, tuple[str, ...]]] = {
    "elementwise": ("elementwise.cu", ()),
    "gemm_simt": ("gemm_simt.cu", ()),
    "attention_simt": ("attention_simt.cu", ()),
    "sampling": ("sampling.cu", ()),
    "gemm_tcgen05": ("gemm_tcgen05.cu", ()),
    "attention_mma": ("attention_mma.cu", ()),
    "attention_tcgen05": ("attention_tcgen05.cu", ()),
    "decode_attention_static": ("decode_attention_static.cu", ()),
}

# .cu files that a source includes (their text is part of the library's hash)
INCLUDED_SOURCES: dict[str, tuple[str, ...]] = {"decode_attention_static": ("attention_mma.cu",)}

NVCC_FLAGS = (
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
)

_lock = threading.Lock()
_loaded: dict[str, ctypes.CDLL] = {}


class ExtensionError(RuntimeError):
    """The CUDA extension could not be built or loaded. There is no fallback path."""


def register_source(name: str, path: str | Path, link_flags: tuple[str, ...] = (),
                    includes: tuple[str | Path, ...] = ()) -> None:
    """Make the .cu file at `path` (anywhere on disk) loadable as library `name`. `includes` lists
    further files whose text it includes, so that a change to them rebuilds it. Registering the same
    name and path again is a no-op; a package library's name cannot be taken over."""
    path = Path(path).resolve()
    if not path.is_file():
        raise ExtensionError(f"kernel source {path} does not exist")
    known = SOURCES.get(name)
    if known is not None and _source_path(name) != path:
        raise ExtensionError(f"kernel library {name!r} is already registered from {_source_path(name)}")
    SOURCES[name] = (str(path), tuple(link_flags))
    if includes:
        INCLUDED_SOURCES[name] = tuple(str(Path(p).resolve()) for p in includes)


def _source_path(name: str) -> Path:
    return (HERE / SOURCES[name][0]).resolve()      # an absolute entry stays as it is


def available_sources() -> list[str]:
    """The package's own sources (those inside this folder)."""
    return [name for name in SOURCES if _source_path(name).is_file() and _source_path(name).parent == HERE]


def _nvcc() -> str:
    for candidate in (os.environ.get("LAYOVER_B200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).is_file():
            return candidate
    raise ExtensionError("nvcc not found: the CUDA kernels of layover_b200 cannot be compiled")


def _digest(name: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS + SOURCES[name][1]).encode())
    h.update(_source_path(name).read_bytes())
    for included in INCLUDED_SOURCES.get(name, ()):
        h.update((HERE / included).read_bytes())
    for header in sorted(HERE.glob("*.cuh")) + sorted(HERE.glob("*.h")):
        h.update(header.name.encode())
        h.update(header.read_bytes())
    return h.hexdigest()[:16]


def _writable(folder: Path) -> bool:
    try:
        folder.mkdir(parents=True, exist_ok=True)
        probe = folder / f".probe-{os.getpid()}-{threading.get_ident()}"
        probe.write_bytes(b"")
        probe.unlink()
        return True
    except OSError:
        return False


def build_dir() -> Path:
    override = os.environ.get("LAYOVER_B200_BUILD_DIR")
    if override:
        folder = Path(override)
        if not _writable(folder):
            raise ExtensionError(f"LAYOVER_B200_BUILD_DIR={override} cannot be written")
        return folder
    in_tree = HERE / "_build"
    if _writable(in_tree):
        return in_tree
    folder = Path(tempfile.gettempdir()) / f"layover_b200-build-{os.getuid()}"
    if not _writable(folder):
        raise ExtensionError(f"neither {in_tree} nor {folder} can be written")
    return folder


def library_path(name: str) -> Path:
    """Where the library of `name` lies or will lie: an up-to-date in-tree build wins."""
    filename = f"{name}-{_digest(name)}.so"
    in_tree = HERE / "_build" / filename
    if in_tree.is_file():
        return in_tree
    return build_dir() / filename


def is_package_source(name: str) -> bool:
    return _source_path(name).parent == HERE


def _say(message: str) -> None:
    print(f"[layover_b200] {message}", file=sys.stderr, flush=True)


def _compile(name: str) -> Path:
    target = library_path(name)
    if target.is_file():
        return target
    source, link = _source_path(name), SOURCES[name][1]
    partial = target.with_name(f".{target.name}.{os.getpid()}.{threading.get_ident()}.tmp")
    command = [_nvcc(), *NVCC_FLAGS, "-I", str(HERE), "-o", str(partial), str(source), *link]
    source = source.name
    _say(f"compiling {source} for sm_100a (first use) ...")
    began = time.monotonic()
    with tempfile.TemporaryFile() as log:
        process = subprocess.Popen(command, stdout=log, stderr=subprocess.STDOUT, cwd=str(HERE))
        while True:
            try:
                process.wait(timeout=10.0)
                break
            except subprocess.TimeoutExpired:
                _say(f"still compiling {source} ({time.monotonic() - began:.0f} s)")
        log.seek(0)
        output = log.read().decode(errors="replace")
    if process.returncode != 0:
        partial.unlink(missing_ok=True)
        raise ExtensionError(f"nvcc failed on {source} (exit {process.returncode}):\n{output}")
    os.replace(partial, target)
    for stale in target.parent.glob(f"{name}-*.so"):
        if stale != target:
            stale.unlink(missing_ok=True)
    _say(f"compiled {source} in {time.monotonic() - began:.1f} s -> {target}")
    return target


def ensure_built(names) -> None:
    """Compile whichever of `names` has no up-to-date library yet, several at a time."""
    todo = [n for n in dict.fromkeys(names) if n not in _loaded and not library_path(n).is_file()]
    if not todo:
        return
    with ThreadPoolExecutor(max_workers=min(len(todo), os.cpu_count() or 2)) as pool:
        list(pool.map(_compile, todo))


def load(name: str) -> ctypes.CDLL:
    """The shared library of one source, compiled if need be. Raises ExtensionError on failure."""
    lib = _loaded.get(name)
    if lib is not None:
        return lib
    if name not in SOURCES:
        raise ExtensionError(f"unknown kernel library {name!r}")
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = _compile(name)
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as error:
                raise ExtensionError(f"cannot load {path}: {error}") from error
            _loaded[name] = lib
    return lib


def loaded() -> tuple[str, ...]:
    """Names of the libraries this process has loaded so far."""
    return tuple(_loaded)


def build_all() -> list[Path]:
    """Compile every source that exists (the `does it build` check; needs no GPU)."""
    names = available_sources()
    ensure_built(names)
    return [library_path(n) for n in names]
