"""In-tree build of the native pieces (no CMake needed: three compiler invocations).

    python fast-kernels_b200/build.py            # library + python module
    python fast-kernels_b200/build.py --oracle   # also the CPU oracle (and the reference .so if present)

Outputs land next to the Python package so that a snapshot of the tree carries them:
    src/fast_kernels/lib/libfk_w4a16.so      C-ABI library (CUDA kernels, sm_100a)
    src/fast_kernels/lib/libfk_page_decode.so  C-ABI library of the paged-KV decode attention
    src/fast_kernels/_native*.so             pybind11 module with the reference's binding names
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

ROOT = Path(__file__).resolve().parent
REPO = ROOT.parent
CSRC = ROOT / "csrc"
PKG = ROOT / "src" / "fast_kernels"
LIB_DIR = PKG / "lib"
VERSION = "0.1.0"

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _run(cmd: list[str]) -> None:
    print("+", " ".join(str(c) for c in cmd), flush=True)
    subprocess.run([str(c) for c in cmd], check=True)


def _newer(target: Path, sources: list[Path]) -> bool:
    if not target.exists():
        return False
    stamp = target.stat().st_mtime
    return all(src.stat().st_mtime <= stamp for src in sources)


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build fast-kernels")
    return found


def build_library(force: bool = False) -> Path:
    """libfk_w4a16.so: every CUDA kernel plus the extern "C" entry points of include/fk_w4a16.h."""
    kernel_dir = CSRC / "kernels" / "decode_quant_linear"
    sources = sorted(kernel_dir.glob("*.cu"))
    deps = sources + sorted(kernel_dir.glob("*.cuh")) + sorted(kernel_dir.glob("*.h")) + [REPO / "include" / "fk_w4a16.h"]
    target = LIB_DIR / "libfk_w4a16.so"
    if not force and _newer(target, deps):
        return target
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    cuda_lib = Path(_nvcc()).resolve().parent.parent / "lib64"
    _run(
        [
            _nvcc(), *NVCC_ARCH, "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
            "--threads", "0",
            "-Xptxas", "-v", f"-DFK_W4A16_VERSION=\"{VERSION}\"",
            "-I", REPO / "include", "-I", kernel_dir,
            "-shared", "-Xcompiler", "-fPIC,-fvisibility=hidden",
            "-Xlinker", f"-rpath,{cuda_lib}",
            "-o", target, *sources, "-lcublasLt",
        ]
    )
    return target


def build_page_decode_library(force: bool = False) -> Path:
    """libfk_page_decode.so: the paged-KV decode attention kernels and the extern "C" entry points
    of include/fk_page_decode.h. One translation unit per (head_dim, page_size), compiled in
    parallel."""
    kernel_dir = CSRC / "kernels" / "clustered_page_decode"
    sources = sorted(kernel_dir.glob("*.cu"))
    deps = (sources + sorted(kernel_dir.glob("*.cuh")) + sorted(kernel_dir.glob("*.h")) + sorted(kernel_dir.glob("*.inc"))
            + [REPO / "include" / "fk_page_decode.h", CSRC / "kernels" / "decode_quant_linear" / "w4a16_common.cuh"])
    target = LIB_DIR / "libfk_page_decode.so"
    if not force and _newer(target, deps):
        return target
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    cuda_lib = Path(_nvcc()).resolve().parent.parent / "lib64"
    _run(
        [
            _nvcc(), *NVCC_ARCH, "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
            "--threads", "0", "-Xptxas", "-v",
            "-I", REPO / "include", "-I", kernel_dir,
            "-shared", "-Xcompiler", "-fPIC,-fvisibility=hidden",
            "-Xlinker", f"-rpath,{cuda_lib}",
            "-o", target, *sources,
        ]
    )
    return target


def build_python_module_without_cuda(out_dir: Path) -> Path:
    """A `_native` module built WITHOUT CUDA into `out_dir`: same names and keyword arguments,
    every op raises RuntimeError("fast-kernels was built without CUDA support"), and
    build_info()["compiled_with_cuda"] is False -- the contract of the reference's CPU-only build
    (csrc/bindings/python_module.cpp:241-287 there). Needs only g++ and pybind11."""
    import pybind11

    out_dir.mkdir(parents=True, exist_ok=True)
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    target = out_dir / f"_native{suffix}"
    cxx = shutil.which("g++") or "g++"
    version = subprocess.run([cxx, "-dumpfullversion"], capture_output=True, text=True).stdout.strip()
    _run(
        [
            cxx, "-O1", "-std=c++20", "-shared", "-fPIC", "-fvisibility=hidden",
            f"-DFK_PROJECT_VERSION=\"{VERSION}\"", "-DFK_COMPILED_WITH_CUDA=0",
            "-DFK_CXX_COMPILER_ID=\"GNU\"", f"-DFK_CXX_COMPILER_VERSION=\"{version}\"",
            "-DFK_CUDA_COMPILER_VERSION=\"\"", "-DFK_CUDA_ARCHITECTURES=\"\"",
            "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"], "-I", CSRC,
            "-o", target,
            CSRC / "bindings" / "python_module.cpp",
            CSRC / "ops" / "decode_quant_linear" / "arc_w4a16_nocuda.cpp",
            CSRC / "ops" / "clustered_page_decode" / "clustered_page_decode_nocuda.cpp",
            CSRC / "ops" / "prefix_union_decode" / "prefix_union_decode.cpp",
        ]
    )
    return target


def build_python_module(force: bool = False) -> Path:
    """fast_kernels._native: the reference's pybind11 surface over the C++ launchers."""
    import pybind11

    sources = [
        CSRC / "bindings" / "python_module.cpp",
        CSRC / "ops" / "decode_quant_linear" / "arc_w4a16.cpp",
        CSRC / "ops" / "clustered_page_decode" / "clustered_page_decode.cpp",
        CSRC / "ops" / "prefix_union_decode" / "prefix_union_decode.cpp",
    ]
    deps = sources + [CSRC / "ops" / "decode_quant_linear" / "arc_w4a16.h", REPO / "include" / "fk_w4a16.h",
                      CSRC / "ops" / "clustered_page_decode" / "clustered_page_decode.h",
                      REPO / "include" / "fk_page_decode.h"]
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    target = PKG / f"_native{suffix}"
    if not force and _newer(target, deps) and _newer(target, [LIB_DIR / "libfk_w4a16.so", LIB_DIR / "libfk_page_decode.so"]):
        return target
    cxx = shutil.which("g++") or "g++"
    version = subprocess.run([cxx, "-dumpfullversion"], capture_output=True, text=True).stdout.strip()
    nvcc_version = "unknown"
    try:
        out = subprocess.run([_nvcc(), "--version"], capture_output=True, text=True).stdout
        nvcc_version = out.split("release")[-1].split(",")[0].strip()
    except Exception:  # pragma: no cover - metadata only
        pass
    cuda_root = Path(_nvcc()).resolve().parent.parent
    _run(
        [
            cxx, "-O2", "-std=c++20", "-shared", "-fPIC", "-fvisibility=hidden",
            f"-DFK_PROJECT_VERSION=\"{VERSION}\"", "-DFK_COMPILED_WITH_CUDA=1",
            "-DFK_CXX_COMPILER_ID=\"GNU\"", f"-DFK_CXX_COMPILER_VERSION=\"{version}\"",
            f"-DFK_CUDA_COMPILER_VERSION=\"{nvcc_version}\"", "-DFK_CUDA_ARCHITECTURES=\"100a\"",
            "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"],
            "-I", CSRC, "-I", REPO / "include", "-I", cuda_root / "include",
            "-o", target, *sources,
            f"-L{LIB_DIR}", "-lfk_w4a16", "-lfk_page_decode", f"-L{cuda_root / 'lib64'}", "-lcudart",
            "-Wl,-rpath,$ORIGIN/lib", f"-Wl,-rpath,{cuda_root / 'lib64'}",
        ]
    )
    return target


def reference_checkout() -> Path | None:
    """Where a checkout of the reference project lies, if anywhere: $FK_REFERENCE_ROOT, else a
    directory named `reference` beside this repository."""
    candidates = []
    if os.environ.get("FK_REFERENCE_ROOT"):
        candidates.append(Path(os.environ["FK_REFERENCE_ROOT"]))
    candidates.append(REPO.parent / "reference")
    for candidate in candidates:
        if (candidate / "csrc" / "kernels" / "decode_quant_linear" / "arc_w4a16.cu").exists():
            return candidate
    return None


def build_oracle(force: bool = False) -> None:
    """The CPU checker (tests and bench baseline only) and, if the reference checkout is there,
    the reference's own kernels as oracle/_ref/libfk_reference.so."""
    oracle_dir = REPO / "oracle"
    args = ["make", "-C", str(oracle_dir), "oracle"]
    if force:
        args.insert(1, "-B")
    _run(args)
    reference = reference_checkout()
    if reference is not None:
        _run(["make", "-C", str(oracle_dir), "ref", "ref_page_decode", f"REF={reference}"])


def build_all(force: bool = False, oracle: bool = False) -> None:
    build_library(force)
    build_page_decode_library(force)
    if (CSRC / "bindings" / "python_module.cpp").exists():
        build_python_module(force)
    if oracle:
        build_oracle(force)


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--force", action="store_true", help="rebuild even if outputs are up to date")
    parser.add_argument("--oracle", action="store_true", help="also build the CPU oracle / reference .so")
    parser.add_argument("--no-cuda", metavar="DIR", default=None,
                        help="build only a CUDA-less _native module into DIR (every op raises)")
    ns = parser.parse_args()
    if ns.no_cuda is not None:
        build_python_module_without_cuda(Path(ns.no_cuda))
        return 0
    build_all(force=ns.force, oracle=ns.oracle)
    return 0


if __name__ == "__main__":
    sys.exit(main())
