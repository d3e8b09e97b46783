"""Run-time compilation of small native kernels: ``@jit`` turns C++/CUDA source into a callable.

    @jit(name="scale", sources=["scale.cu"], template_args={"T": "float", "N": 4})
    def scale(lib, x, y): lib.scale_launch(x.data_ptr(), y.data_ptr(), x.numel())

Sources are compiled with ``nvcc`` (``.cu``, for sm_100a) or ``g++`` (``.cpp``) into a shared
library whose ``extern "C"`` symbols are reached through ``ctypes``; template arguments become
``-D`` macros, so one source serves several specialisations. Builds are cached under
``$PHYAI_B200_JIT_CACHE`` (default ``~/.cache/phyai_b200/jit``) keyed by a hash of the sources,
their local ``#include``s, the flags and the macro values; a second call loads the cached library
without touching the compiler. The serving path does not depend on this: its kernels are built
ahead of time by ``phyai_b200.build_ext``. It exists for experiments and for per-shape
specialisations that are not worth carrying in the main extension.

Reference: phyai-kernel/phyai_kernel/jit/*.py (there built on tvm_ffi.cpp.load_inline).
"""

from __future__ import annotations

import ctypes
import functools
import hashlib
import os
import re
import shutil
import subprocess
import threading
from pathlib import Path
from typing import Any, Callable, Mapping, Sequence

NVCC_ARCH = ("-gencode", "arch=compute_100a,code=sm_100a")
_LOCK = threading.Lock()
_LOADED: dict[str, ctypes.CDLL] = {}


def cache_dir() -> Path:
    return Path(os.environ.get("PHYAI_B200_JIT_CACHE", Path.home() / ".cache" / "phyai_b200" / "jit"))


def template_macros(args: Mapping[str, Any] | None) -> list[str]:
    """{"T": "float", "N": 4, "FAST": True} -> ["-DT=float", "-DN=4", "-DFAST=1"] (sorted: stable hashes)."""
    out = []
    for k, v in sorted((args or {}).items()):
        if not re.fullmatch(r"[A-Za-z_]\w*", k):
            raise ValueError(f"template argument name {k!r} is not an identifier")
        if isinstance(v, bool):
            v = int(v)
        out.append(f"-D{k}={v}")
    return out


def _local_includes(src: Path, seen: set[Path]) -> None:
    if src in seen or not src.is_file():
        return
    seen.add(src)
    for m in re.finditer(r'^\s*#\s*include\s*"([^"]+)"', src.read_text(errors="replace"), re.M):
        _local_includes((src.parent / m.group(1)).resolve(), seen)


def build_key(sources: Sequence[Path], flags: Sequence[str]) -> str:
    files: set[Path] = set()
    for s in sources:
        _local_includes(Path(s).resolve(), files)
    h = hashlib.sha256()
    for f in sorted(files):
        h.update(str(f.name).encode())
        h.update(f.read_bytes())
    h.update("\0".join(flags).encode())
    return h.hexdigest()[:20]


def compile_library(name: str, sources: Sequence[str | Path], *, template_args: Mapping[str, Any] | None = None,
                    extra_flags: Sequence[str] = (), include_dirs: Sequence[str | Path] = (), verbose: bool = False) -> Path:
    srcs = [Path(s).resolve() for s in sources]
    for s in srcs:
        if not s.is_file():
            raise FileNotFoundError(s)
    cuda = any(s.suffix == ".cu" for s in srcs)
    flags = [*template_macros(template_args), *extra_flags, *[f"-I{Path(d).resolve()}" for d in include_dirs]]
    key = build_key(srcs, ["cuda" if cuda else "host", *flags])
    out_dir = cache_dir() / f"{name}-{key}"
    lib = out_dir / f"lib{name}.so"
    if lib.is_file():
        return lib
    with _LOCK:
        if lib.is_file():
            return lib
        tmp = out_dir.with_name(out_dir.name + f".tmp{os.getpid()}")
        tmp.mkdir(parents=True, exist_ok=True)
        if cuda:
            cc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
            cmd = [cc, *NVCC_ARCH, "-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC", *flags,
                   *map(str, srcs), "-o", str(tmp / lib.name)]
        else:
            cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", *flags, *map(str, srcs), "-o", str(tmp / lib.name)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode:
            print(" ".join(cmd), r.stdout, r.stderr, sep="\n")
        if r.returncode:
            shutil.rmtree(tmp, ignore_errors=True)
            raise RuntimeError(f"jit build of {name!r} failed:\n{r.stderr[-4000:]}")
        (tmp / "command.txt").write_text(" ".join(cmd))
        try:
            tmp.rename(out_dir)
        except OSError:          # another process won the race
            shutil.rmtree(tmp, ignore_errors=True)
    return lib


def load_library(path: Path) -> ctypes.CDLL:
    key = str(path)
    if key not in _LOADED:
        _LOADED[key] = ctypes.CDLL(key)
    return _LOADED[key]


def jit(*, name: str, sources: Sequence[str | Path], template_args: Mapping[str, Any] | None = None,
        extra_flags: Sequence[str] = (), include_dirs: Sequence[str | Path] = (), signatures: Mapping[str, tuple] | None = None):
    """Decorator: the function's first argument becomes the loaded library (compiled on first call).
    ``signatures`` maps symbol -> (restype, [argtypes]) and is applied once after loading."""
    def deco(fn: Callable) -> Callable:
        state: dict[str, Any] = {}

        def lib() -> ctypes.CDLL:
            if "lib" not in state:
                l = load_library(compile_library(name, sources, template_args=template_args, extra_flags=extra_flags, include_dirs=include_dirs))
                for sym, (res, args) in (signatures or {}).items():
                    f = getattr(l, sym)
                    f.restype, f.argtypes = res, list(args)
                state["lib"] = l
            return state["lib"]

        @functools.wraps(fn)
        def wrapper(*a, **k):
            return fn(lib(), *a, **k)

        wrapper.library = lib
        return wrapper
    return deco


def specializations(base: Mapping[str, Any], **axes: Sequence[Any]) -> list[dict[str, Any]]:
    """Cartesian product of template-argument values: the list of variants to pre-build."""
    out = [dict(base)]
    for k, vals in axes.items():
        out = [{**d, k: v} for d in out for v in vals]
    return out


__all__ = ["jit", "compile_library", "load_library", "template_macros", "build_key", "cache_dir", "specializations", "NVCC_ARCH"]
