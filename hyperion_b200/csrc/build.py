"""Compiles the CUDA sources of this folder for sm_100a, and the C++ host runtime of ``host/``, and
loads them with ctypes.

Each ``.cu`` file becomes one shared library, built on first use with ``nvcc`` and kept beside the
package under ``_build/`` (or in a per-user temporary folder when the package folder cannot be
written).  The file name of a library carries a hash of its source, of the shared header and of the
preprocessor definitions it was built with, so an edited source is rebuilt and kernels specialised
for a head size are built once per size.  Only the modules a model asks for are compiled.  There is
no fallback: a missing compiler or a failed build raises.
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
from typing import Iterable, Mapping, Sequence

SOURCE_DIR = Path(__file__).resolve().parent
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

_lock = threading.Lock()
_loaded: dict[str, ctypes.CDLL] = {}


class BuildError(RuntimeError):
    """The native kernels could not be built or loaded."""


def _nvcc() -> str:
    for candidate in (os.environ.get("HYPERION_B200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.isfile(candidate) and os.access(candidate, os.X_OK):
            return candidate
    raise BuildError("nvcc not found (looked at HYPERION_B200_NVCC, PATH and /usr/local/cuda/bin): the CUDA kernels cannot be built")


def _build_dir() -> Path:
    override = os.environ.get("HYPERION_B200_BUILD_DIR")
    candidates = [Path(override)] if override else []
    candidates.append(SOURCE_DIR.parent / "_build")
    candidates.append(Path(tempfile.gettempdir()) / f"hyperion_b200_build_{os.getuid()}")
    for folder in candidates:
        try:
            folder.mkdir(parents=True, exist_ok=True)
            probe = folder / f".probe_{os.getpid()}"
            probe.write_bytes(b"")
            probe.unlink()
            return folder
        except OSError:
            continue
    raise BuildError(f"no writable build folder among {[str(c) for c in candidates]}")


def _key(module: str, defines: Mapping[str, object]) -> str:
    digest = hashlib.sha256()
    includes = sorted(p for p in SOURCE_DIR.iterdir() if p.suffix in (".cuh", ".h") or (p.suffix == ".cu" and f'"{p.name}"' in (SOURCE_DIR / f"{module}.cu").read_text()))
    for path in [SOURCE_DIR / f"{module}.cu", *includes]:
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    digest.update(repr(sorted(defines.items())).encode())
    digest.update(" ".join(ARCH_FLAGS + BASE_FLAGS).encode())
    return digest.hexdigest()[:16]


def _tag(module: str, defines: Mapping[str, object]) -> str:
    suffix = "".join(f"_{k.lower()}{v}" for k, v in sorted(defines.items()))
    return f"{module}{suffix}"


def library_path(module: str, defines: Mapping[str, object] | None = None) -> Path:
    defines = dict(defines or {})
    return _build_dir() / f"hb_{_tag(module, defines)}-{_key(module, defines)}.so"


def _compile(module: str, defines: Mapping[str, object], target: Path, extra: Sequence[str] = ()) -> None:
    source = SOURCE_DIR / f"{module}.cu"
    if not source.is_file():
        raise BuildError(f"no such kernel source: {source}")
    scratch = target.with_suffix(f".tmp{os.getpid()}.so")
    command = [_nvcc(), *ARCH_FLAGS, *BASE_FLAGS, *extra, *[f"-D{k}={v}" for k, v in sorted(defines.items())],
               "-I", str(SOURCE_DIR), "-o", str(scratch), str(source)]
    started = time.time()
    print(f"[hyperion_b200] compiling {_tag(module, defines)} for sm_100a ...", file=sys.stderr, flush=True)
    process = subprocess.Popen(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    while True:
        try:
            output, _ = process.communicate(timeout=15)
            break
        except subprocess.TimeoutExpired:
            print(f"[hyperion_b200] still compiling {_tag(module, defines)} ({time.time() - started:.0f} s)", file=sys.stderr, flush=True)
    if process.returncode != 0:
        if scratch.exists():
            scratch.unlink()
        raise BuildError(f"nvcc failed for {source.name} ({' '.join(command)}):\n{output}")
    os.replace(scratch, target)
    print(f"[hyperion_b200] built {target.name} in {time.time() - started:.1f} s", file=sys.stderr, flush=True)


def load(module: str, defines: Mapping[str, object] | None = None) -> ctypes.CDLL:
    """The library of ``csrc/<module>.cu`` built with ``defines``, compiling it if it is not there."""
    defines = dict(defines or {})
    tag = _tag(module, defines)
    with _lock:
        if tag in _loaded:
            return _loaded[tag]
    target = library_path(module, defines)
    if not target.is_file():
        _compile(module, defines, target)
    try:
        library = ctypes.CDLL(str(target))
    except OSError as error:
        raise BuildError(f"cannot load {target}: {error}") from None
    with _lock:
        _loaded.setdefault(tag, library)
        return _loaded[tag]


def build_many(requests: Iterable[tuple[str, Mapping[str, object]]], workers: int | None = None) -> None:
    """Compile several modules side by side (what a model needs, or everything for a build check)."""
    pending = []
    seen = set()
    for module, defines in requests:
        defines = dict(defines or {})
        tag = _tag(module, defines)
        if tag in seen:
            continue
        seen.add(tag)
        target = library_path(module, defines)
        if not target.is_file():
            pending.append((module, defines, target))
    if not pending:
        return
    with ThreadPoolExecutor(max_workers=workers or min(8, os.cpu_count() or 1)) as pool:
        futures = [pool.submit(_compile, *item) for item in pending]
        for future in futures:
            future.result()


# ---------------------------------------------------------------------- the host runtime (C++, no CUDA)
HOST_DIR = SOURCE_DIR / "host"
HOST_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-Wall"]


def _host_compiler() -> str:
    for candidate in (os.environ.get("HYPERION_B200_CXX"), os.environ.get("CXX"), "g++", "c++", "clang++"):
        found = shutil.which(candidate) if candidate else None
        if found:
            return found
    raise BuildError("no C++ compiler found (looked at HYPERION_B200_CXX, CXX, g++, c++, clang++): the host runtime cannot be built")


def _host_flags() -> list[str]:
    """``HOST_FLAGS`` plus what ``HYPERION_B200_CXXFLAGS`` adds (for instance ``-fsanitize=address,undefined -g`` to run the
    host tests under the sanitizers, with the sanitizer's runtime preloaded into the interpreter)."""
    return HOST_FLAGS + os.environ.get("HYPERION_B200_CXXFLAGS", "").split()


def host_library_path() -> Path:
    digest = hashlib.sha256()
    for path in sorted(HOST_DIR.iterdir()):
        if path.suffix in (".cpp", ".hpp", ".h"):
            digest.update(path.name.encode())
            digest.update(path.read_bytes())
    digest.update(" ".join(_host_flags()).encode())
    return _build_dir() / f"hb_host_runtime-{digest.hexdigest()[:16]}.so"


def load_host() -> ctypes.CDLL:
    """The host runtime (cache index, scheduler, step assembly) of ``csrc/host``, compiled on first use."""
    with _lock:
        if "host_runtime" in _loaded:
            return _loaded["host_runtime"]
    target = host_library_path()
    if not target.is_file():
        scratch = target.with_suffix(f".tmp{os.getpid()}.so")
        sources = sorted(str(p) for p in HOST_DIR.glob("*.cpp"))
        command = [_host_compiler(), *_host_flags(), "-I", str(HOST_DIR), "-o", str(scratch), *sources]
        started = time.time()
        print("[hyperion_b200] compiling the host runtime ...", file=sys.stderr, flush=True)
        done = subprocess.run(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if done.returncode != 0:
            if scratch.exists():
                scratch.unlink()
            raise BuildError(f"the host runtime failed to compile ({' '.join(command)}):\n{done.stdout}")
        os.replace(scratch, target)
        print(f"[hyperion_b200] built {target.name} in {time.time() - started:.1f} s", file=sys.stderr, flush=True)
    try:
        library = ctypes.CDLL(str(target))
    except OSError as error:
        raise BuildError(f"cannot load {target}: {error}") from None
    with _lock:
        _loaded.setdefault("host_runtime", library)
        return _loaded["host_runtime"]


def all_modules() -> list[tuple[str, dict]]:
    """Every module in its default specialisations: what a build check compiles."""
    requests: list[tuple[str, dict]] = []
    for path in sorted(SOURCE_DIR.glob("*.cu")):
        module = path.stem
        text = path.read_text()
        if "HB_HEAD_DIM" in text:
            requests += [(module, {"HB_HEAD_DIM": d}) for d in (64, 128)]
        else:
            requests.append((module, {}))
    return requests
