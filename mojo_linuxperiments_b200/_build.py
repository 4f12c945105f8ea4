"""In-tree native build: nvcc for the sm_100a kernel library, g++ for the host runtime.

The shared objects are written next to the Python package (``_lib/``) so that a snapshot of the source tree
carries them to a machine without a compiler cache.  Objects are rebuilt only when a source or header changed
(content hash), files are compiled in parallel, and nothing here needs a GPU: nvcc cross-compiles.
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIBDIR = PKG / "_lib"
OBJDIR = PKG.parent / "build" / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--use_fast_math", "-Xptxas", "-v",
]
# --use_fast_math is dropped for files whose numerics are compared bit-for-bit with an oracle
NO_FAST_MATH = {"act_quant.cu"}
GXX_FLAGS = ["-O2", "-std=c++20", "-fPIC", "-Wall", "-Wextra", "-fno-stack-protector", "-pthread"]

KERNEL_LIB = "libb200_kernels.so"
# Variants of the kernel library: same sources, one extra define each.  "trace": in-kernel %globaltimer stamps
# (csrc/kernels/trace.cuh); "debug": range checks on peer / scratch accesses that record the bad offset in the status
# word and skip the access (csrc/kernels/debug_check.h).  The production library has neither.
KERNEL_VARIANTS = {"": [], "trace": ["-DB200RT_TRACE"], "debug": ["-DB200RT_DEBUG"]}


HOSTRT_LIB = "libb200_hostrt.so"
DEVRT_LIB = "libb200_devrt.so"


def kernel_lib_name(variant: str = "") -> str:
    return KERNEL_LIB if not variant else KERNEL_LIB.replace(".so", f"_{variant}.so")


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def _digest(paths, extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        h.update(str(p.name).encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _run(cmd, log: Path | None = None) -> str:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    out = proc.stdout + proc.stderr
    if log is not None:
        log.write_text(" ".join(map(str, cmd)) + "\n" + out)
    if proc.returncode != 0:
        raise RuntimeError("build step failed:\n" + " ".join(map(str, cmd)) + "\n" + out[-6000:])
    return out


def _stale(stamp: Path, digest: str, product: Path) -> bool:
    if not product.exists() or not stamp.exists():
        return True
    try:
        return json.loads(stamp.read_text()).get("digest") != digest
    except Exception:
        return True


def build_kernels(verbose: bool = False, variant: str = "") -> Path:
    """Compile every .cu under csrc/kernels for sm_100a and link libb200_kernels[_variant].so."""
    srcdir = CSRC / "kernels"
    sources = sorted(srcdir.glob("*.cu"))
    headers = sorted(list(srcdir.glob("*.cuh")) + list(srcdir.glob("*.h")) + list((CSRC / "fabric").glob("*.h")))
    LIBDIR.mkdir(parents=True, exist_ok=True)
    objdir = OBJDIR / variant if variant else OBJDIR
    objdir.mkdir(parents=True, exist_ok=True)
    nvcc = _nvcc()
    vflags = NVCC_FLAGS + KERNEL_VARIANTS[variant]
    hdigest = _digest(headers, " ".join(vflags))

    def compile_one(src: Path) -> Path:
        obj = objdir / (src.stem + ".o")
        stamp = objdir / (src.stem + ".stamp")
        digest = _digest([src], hdigest)
        if _stale(stamp, digest, obj):
            flags = [f for f in vflags if not (f == "--use_fast_math" and src.name in NO_FAST_MATH)]
            out = _run([nvcc, *flags, "-I", str(srcdir), "-I", str(CSRC), "-c", str(src), "-o", str(obj)],
                       objdir / (src.stem + ".log"))
            if verbose:
                print(out, file=sys.stderr)
            stamp.write_text(json.dumps({"digest": digest}))
        return obj

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(sources)))) as ex:
        objs = list(ex.map(compile_one, sources))
    lib = LIBDIR / kernel_lib_name(variant)
    link_digest = _digest(objs, "link")
    stamp = objdir / "kernels.link.stamp"
    if _stale(stamp, link_digest, lib):
        _run([nvcc, "-shared", "-o", str(lib), *map(str, objs), "-cudart", "static"])
        stamp.write_text(json.dumps({"digest": link_digest}))
    return lib


def _build_cpp(name: str, subdir: str, extra_flags=(), libs=()) -> Path:
    srcdir = CSRC / subdir
    sources = sorted(srcdir.glob("*.cpp"))
    headers = sorted(list(srcdir.glob("*.hpp")) + list(srcdir.glob("*.h")) + list((CSRC / "fabric").glob("*.h")))
    LIBDIR.mkdir(parents=True, exist_ok=True)
    OBJDIR.mkdir(parents=True, exist_ok=True)
    lib = LIBDIR / name
    digest = _digest(sources + headers, " ".join(GXX_FLAGS) + " ".join(extra_flags))
    stamp = OBJDIR / (name + ".stamp")
    if _stale(stamp, digest, lib):
        _run(["g++", *GXX_FLAGS, *extra_flags, "-shared", "-I", str(srcdir), "-I", str(CSRC), "-o", str(lib),
              *map(str, sources), *libs])
        stamp.write_text(json.dumps({"digest": digest}))
    return lib


def build_hostrt() -> Path:
    """C++ host runtime: raw syscalls, NUMA topology, CPU masks, NUMA arena, clone3 thread pool, futex gates."""
    return _build_cpp(HOSTRT_LIB, "hostrt")


def build_hostrt_selftest() -> Path:
    """Stand-alone executable that runs the reference's twelve integration scenarios (exit code = failures)."""
    srcdir = CSRC / "hostrt"
    exe = LIBDIR / "hostrt_selftest"
    sources = sorted(srcdir.glob("*.cpp"))
    sources = [s for s in sources if s.name != "capi.cpp"] + [srcdir / "selftest" / "main.cc"]
    headers = sorted(srcdir.glob("*.hpp"))
    digest = _digest(sources + headers, "selftest" + " ".join(GXX_FLAGS))
    stamp = OBJDIR / "hostrt_selftest.stamp"
    LIBDIR.mkdir(parents=True, exist_ok=True)
    OBJDIR.mkdir(parents=True, exist_ok=True)
    if _stale(stamp, digest, exe):
        flags = [f for f in GXX_FLAGS if f != "-fPIC"]
        _run(["g++", *flags, "-I", str(srcdir), "-I", str(CSRC), "-o", str(exe), *map(str, sources)])
        stamp.write_text(json.dumps({"digest": digest}))
    return exe


def build_hostrt_tsan() -> Path:
    """Thread-sanitizer build of the fabric protocols (ranks as std::threads): ``_lib/hostrt_tsan_fabric``."""
    srcdir = CSRC / "hostrt"
    exe = LIBDIR / "hostrt_tsan_fabric"
    sources = [s for s in sorted(srcdir.glob("*.cpp")) if s.name != "capi.cpp"] + [srcdir / "selftest" / "tsan_fabric.cc"]
    headers = sorted(srcdir.glob("*.hpp")) + sorted((CSRC / "fabric").glob("*.h"))
    flags = [f for f in GXX_FLAGS if f != "-fPIC"] + ["-fsanitize=thread", "-g", "-O1", "-DHOSTRT_STD_THREADS"]
    digest = _digest(sources + headers, "tsan" + " ".join(flags))
    stamp = OBJDIR / "hostrt_tsan_fabric.stamp"
    LIBDIR.mkdir(parents=True, exist_ok=True)
    OBJDIR.mkdir(parents=True, exist_ok=True)
    if _stale(stamp, digest, exe):
        _run(["g++", *flags, "-I", str(srcdir), "-I", str(CSRC), "-o", str(exe), *map(str, sources)])
        stamp.write_text(json.dumps({"digest": digest}))
    return exe


def build_devrt() -> Path:
    """C++ device runtime: GPU topology, HBM arena (CUDA virtual memory management), device masks."""
    cuda_inc = Path(_nvcc()).resolve().parent.parent / "include"
    return _build_cpp(DEVRT_LIB, "devrt", extra_flags=("-I", str(cuda_inc)), libs=("-ldl",))


def build_all(verbose: bool = False, variants=("",)) -> dict:
    """Host runtime, device runtime and the kernel library; ``variants`` adds "trace" / "debug" kernel libraries."""
    out = {}
    if any((CSRC / "hostrt").glob("*.cpp")):
        out["hostrt"] = build_hostrt()
        out["hostrt_selftest"] = build_hostrt_selftest()
    if any((CSRC / "devrt").glob("*.cpp")):
        out["devrt"] = build_devrt()
    for v in variants:
        out["kernels" + ("_" + v if v else "")] = build_kernels(verbose, v)
    return out


if __name__ == "__main__":
    want = [""] + [v for v in ("trace", "debug") if ("--" + v) in sys.argv or "--all" in sys.argv]
    if "--tsan" in sys.argv or "--all" in sys.argv:
        print(f"hostrt_tsan_fabric: {build_hostrt_tsan()}")
    for k, v in build_all(verbose="-v" in sys.argv, variants=want).items():
        print(f"{k}: {v}")
