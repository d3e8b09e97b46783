"""In-tree build of the native extensions for sm_100a.

``python -m phyai_b200.build_ext`` compiles every ``csrc/*.cu`` with
``nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo`` (cross-compiles without a
GPU), the pybind/torch binding unit with the host compiler, and links them into
``phyai_b200/_C*.so`` next to the Python sources. Objects are cached under
``build/`` keyed by a hash of the source, its headers and the flags, so an
unchanged file is not recompiled.

Variants (objects are cached per flag set, the output replaces the regular ``.so``):

* ``--debug``     ``-DPHYAI_DEBUG=1``: the kernels' index checks are compiled in (a row / column /
  slot index outside its tensor is recorded in the status word as ``kStatusBadArg`` and the access is
  skipped, see ``PB_DEBUG_CHECK`` in ``csrc/ptx.cuh``), device code at ``-O1`` with line info;
* ``--sanitize``  host-only prefix cache with ``-fsanitize=address,undefined``; run the cache tests with
  ``LD_PRELOAD="$(gcc -print-file-name=libasan.so) $(gcc -print-file-name=libstdc++.so)" ASAN_OPTIONS=detect_leaks=0``
  (the C++ runtime has to be loaded with the sanitizer, or its ``__cxa_throw`` hook finds nothing to call at the first
  exception); ``--tsan`` the same with ``-fsanitize=thread`` and ``libtsan.so``.

Building a variant and then the regular flavour again relinks: ``build/_C.linked`` / ``build/_radix.linked`` hold the
link tag of what the output file contains.
"""

from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
BUILD = ROOT.parent / "build"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo"]


def _hash(paths: list[Path], flags: list[str]) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:16]


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError(f"build step failed: {cmd[0]} {cmd[-1]}")


def _torch_paths() -> tuple[list[str], list[str]]:
    import torch  # noqa: F401
    from torch.utils import cpp_extension as ce

    return ce.include_paths(), ce.library_paths()


def ext_suffix() -> str:
    return sysconfig.get_config_var("EXT_SUFFIX") or ".so"


def build_core(verbose: bool = False, debug: bool = False) -> Path:
    """Build ``phyai_b200/_C`` (CUDA kernels + torch bindings)."""
    BUILD.mkdir(exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    inc, libdirs = _torch_paths()
    pyinc = sysconfig.get_paths()["include"]
    import pybind11

    common_inc = [f"-I{CSRC}", f"-I{pyinc}", f"-I{pybind11.get_include()}"]
    cu_flags = ARCH_FLAGS + ["-O3", "-std=c++17", "--use_fast_math", "-Xcompiler", "-fPIC",
                             "--expt-relaxed-constexpr", "-DTORCH_EXTENSION_NAME=_C",
                             "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=1"] + common_inc + [
                                 f"-I{p}" for p in inc]
    if verbose:
        cu_flags += ["-Xptxas", "-v"]
    if debug:
        cu_flags = [f for f in cu_flags if f != "-O3"] + ["-O1", "-DPHYAI_DEBUG=1"]
    cxx_flags = ["-O2", "-std=c++17", "-fPIC", "-DTORCH_EXTENSION_NAME=_C",
                 "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=1",
                 "-I/usr/local/cuda/include"] + common_inc + [f"-I{p}" for p in inc]

    jobs: list[tuple[list[str], Path]] = []
    objs: list[Path] = []
    for src in sorted(CSRC.glob("*.cu")):
        if src.name.startswith("radix") or src.name.startswith("standalone_"):
            continue
        tag = _hash([src] + headers, cu_flags)
        obj = BUILD / f"{src.stem}.{tag}.o"
        objs.append(obj)
        if not obj.exists():
            jobs.append(([NVCC, *cu_flags, "-c", str(src), "-o", str(obj)], obj))
    bsrc = CSRC / "bindings.cpp"
    tag = _hash([bsrc] + headers, cxx_flags)
    bobj = BUILD / f"bindings.{tag}.o"
    objs.append(bobj)
    if not bobj.exists():
        jobs.append((["g++", *cxx_flags, "-c", str(bsrc), "-o", str(bobj)], bobj))

    with ThreadPoolExecutor(max_workers=max(1, min(8, len(jobs) or 1))) as ex:
        list(ex.map(lambda j: _run(j[0]), jobs))

    out = ROOT / f"_C{ext_suffix()}"
    link_tag = _hash(objs, ["link"])
    stamp = BUILD / "_C.linked"           # the link tag of what the output file holds (variants replace one another)
    if not out.exists() or not stamp.exists() or stamp.read_text() != link_tag:
        libs = ["-lc10", "-ltorch", "-ltorch_cpu", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda"]
        cmd = [NVCC, "-shared", *ARCH_FLAGS, "-o", str(out), *map(str, objs),
               *[f"-L{p}" for p in libdirs], *libs,
               *[f"-Xlinker=-rpath={p}" for p in libdirs]]
        _run(cmd)
        stamp.write_text(link_tag)
    return out


def build_radix(verbose: bool = False, sanitize: str | None = None) -> Path | None:
    """Build ``phyai_b200/_radix`` (host-only C++ prefix cache, pybind11). ``sanitize``: ``"address"`` (with
    undefined-behaviour checks) or ``"thread"``."""
    src_dir = CSRC / "radix_cache"
    if not src_dir.exists():
        return None
    BUILD.mkdir(exist_ok=True)
    import pybind11

    srcs = sorted(src_dir.glob("*.cpp"))
    hdrs = sorted(src_dir.glob("*.h"))
    pyinc = sysconfig.get_paths()["include"]
    flags = ["-O2", "-std=c++20", "-fPIC", "-pthread", f"-I{src_dir}", f"-I{pyinc}",
             f"-I{pybind11.get_include()}"]
    san: list[str] = []
    if sanitize == "address":
        san = ["-fsanitize=address,undefined", "-fno-omit-frame-pointer", "-g"]
    elif sanitize == "thread":
        san = ["-fsanitize=thread", "-fno-omit-frame-pointer", "-g"]
    elif sanitize:
        raise ValueError(f"unknown sanitizer {sanitize!r}")
    flags = [f if f != "-O2" else ("-O1" if san else "-O2") for f in flags] + san
    objs, jobs = [], []
    for s in srcs:
        tag = _hash([s] + hdrs, flags)
        o = BUILD / f"radix_{s.stem}.{tag}.o"
        objs.append(o)
        if not o.exists():
            jobs.append(["g++", *flags, "-c", str(s), "-o", str(o)])
    with ThreadPoolExecutor(max_workers=8) as ex:
        list(ex.map(_run, jobs))
    out = ROOT / f"_radix{ext_suffix()}"
    link_tag = _hash(objs, ["link-radix", *san])
    stamp = BUILD / "_radix.linked"       # the link tag of what the output file holds (variants replace one another)
    if not out.exists() or not stamp.exists() or stamp.read_text() != link_tag:
        _run(["g++", "-shared", "-pthread", *san, "-o", str(out), *map(str, objs)])
        stamp.write_text(link_tag)
    return out


def cutlass_include_dirs() -> list[Path]:
    """CUTLASS / CuTe header trees vendored by Python packages of this environment (none: empty list)."""
    import site

    found: list[Path] = []
    for sp in site.getsitepackages():
        for rel in ("flashinfer/data/cutlass", "tilelang/3rdparty/cutlass"):
            inc = Path(sp) / rel / "include"
            if (inc / "cutlass" / "detail" / "sm100_blockscaled_layout.hpp").is_file():
                found = [inc] + ([inc.parent / "tools" / "util" / "include"] if (inc.parent / "tools" / "util" / "include").is_dir() else [])
                return found
    return found


def build_blockscaled(verbose: bool = False) -> Path | None:
    """Build ``phyai_b200/_blockscaled`` (NVFP4 and block-scaled fp8 GEMMs: CUTLASS sm100 collectives instantiated in
    ``csrc/cutlass/``, one translation unit per tile shape, plus this repository's quantisation kernels and bindings in
    ``blockscaled_module.cu``). Skipped, with a note, where no CUTLASS header tree is found."""
    src = CSRC / "cutlass" / "blockscaled_module.cu"
    if not src.is_file():
        return None
    cut = cutlass_include_dirs()
    if not cut:
        sys.stderr.write("build_ext: no CUTLASS headers found, phyai_b200/_blockscaled not built (NVFP4 layers dequantise, block-scaled fp8 keeps the in-tree kernel)\n")
        return None
    BUILD.mkdir(exist_ok=True)
    inc, libdirs = _torch_paths()
    pyinc = sysconfig.get_paths()["include"]
    import pybind11

    flags = ARCH_FLAGS + ["-O3", "-std=c++17", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "--expt-extended-lambda",
                          "-diag-suppress", "20012", "-DTORCH_EXTENSION_NAME=_blockscaled", "-DTORCH_API_INCLUDE_EXTENSION_H",
                          "-D_GLIBCXX_USE_CXX11_ABI=1", f"-I{pyinc}", f"-I{pybind11.get_include()}"] + [f"-I{p}" for p in cut] + [
                              f"-I{p}" for p in inc]
    if verbose:
        flags += ["-Xptxas", "-v"]
    flags += [f"-I{src.parent}"]
    hdrs = sorted(src.parent.glob("*.cuh"))
    objs, jobs = [], []
    for cu in sorted(src.parent.glob("*.cu")):          # one tile shape per translation unit: they compile side by side
        tag = _hash([cu] + hdrs, flags)
        obj = BUILD / f"{cu.stem}.{tag}.o"
        objs.append(obj)
        if not obj.exists():
            jobs.append([NVCC, *flags, "-c", str(cu), "-o", str(obj)])
    with ThreadPoolExecutor(max_workers=max(1, len(jobs))) as ex:
        list(ex.map(_run, jobs))
    out = ROOT / f"_blockscaled{ext_suffix()}"
    stamp = BUILD / f"_blockscaled.{_hash(objs, ['link-blockscaled'])}.stamp"
    if not out.exists() or not stamp.exists():
        libs = ["-lc10", "-ltorch", "-ltorch_cpu", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda"]
        _run([NVCC, "-shared", *ARCH_FLAGS, "-o", str(out), *map(str, objs), *[f"-L{p}" for p in libdirs], *libs,
              *[f"-Xlinker=-rpath={p}" for p in libdirs]])
        stamp.write_text("ok")
    return out


def build_all(verbose: bool = False, debug: bool = False, sanitize: str | None = None) -> list[Path]:
    outs = [build_core(verbose, debug)]
    r = build_radix(verbose, sanitize)
    if r is not None:
        outs.append(r)
    try:
        n = build_blockscaled(verbose)
    except RuntimeError as e:        # optional module (its header tree is not this repository's): say so and go on
        sys.stderr.write(f"build_ext: phyai_b200/_blockscaled not built: {e}\n")
        n = None
    if n is not None:
        outs.append(n)
    return outs


if __name__ == "__main__":
    sanitize = "address" if "--sanitize" in sys.argv else ("thread" if "--tsan" in sys.argv else None)
    if "--radix-only" in sys.argv:      # host-only C++ (no nvcc): what a CPU-only checkout can build
        print("built", build_radix("-v" in sys.argv, sanitize))
    else:
        for p in build_all("-v" in sys.argv, "--debug" in sys.argv, sanitize):
            print("built", p)
