"""In-tree build of the native pieces with nvcc / g++ (no cmake, no JIT cache).

Products, all written next to this file so that they are found without installation:

  libaotriton_v2.so            kernels + C-ABI (include/aotriton_b200.h) + C++ operator API
                               (include/aotriton/*.h); the name follows the reference's
                               library (v3src/CMakeLists.txt:383-387)
  pyaotriton.<abi>.so          pybind11 module with the reference's Python surface

`python -m aotriton_b200.build` rebuilds what is out of date.  Set AOTRITON_NAME_SUFFIX
to compile namespace aotriton<suffix> the way the reference's cmake option does.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
OBJ = PKG / "build"
LIB = PKG / "libaotriton_v2.so"

CUDA_SOURCES = ["cabi.cu", "general_kernels.cu", "sm100_fwd.cu", "sm100_bwd.cu"]
CXX_SOURCES = ["api.cc"]
HEADERS = sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list((ROOT / "include").rglob("*.h")))

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; the library has no other implementation to fall back to")


def _suffix_flags() -> list[str]:
    s = os.environ.get("AOTRITON_NAME_SUFFIX", "")
    flags = [f"-DAOTRITON_NAME_SUFFIX={s}"] if s else []
    if os.environ.get("AB200_TRACE"):          # pipeline cycle stamps, see sm100_bwd.cu
        flags.append("-DAB200_TRACE")
        if os.environ.get("AB200_TRACE_TID"):
            flags.append("-DAB200_TRACE_TID=" + os.environ["AB200_TRACE_TID"])
    if os.environ.get("AB200_EXTRA_DEFS"):     # experiments: space-separated -D definitions
        flags += os.environ["AB200_EXTRA_DEFS"].split()
    return flags


def _digest(paths, extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in paths:
        h.update(str(p).encode())
        h.update(Path(p).read_bytes())
    return h.hexdigest()


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("build step failed:\n" + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    if os.environ.get("AB200_BUILD_VERBOSE"):
        sys.stderr.write(proc.stdout + proc.stderr)


def _compile_one(src: Path, verbose_ptxas: bool) -> Path:
    obj = OBJ / (src.name + ".o")
    stamp = OBJ / (src.name + ".stamp")
    common = ["-O3", "-std=c++20", f"-I{ROOT / 'include'}", f"-I{CSRC}", "-Xcompiler", "-fPIC,-fvisibility=hidden"]
    common += _suffix_flags()
    if src.suffix == ".cu":
        cmd = [_nvcc(), *ARCH, "-lineinfo", "--expt-relaxed-constexpr", *common, "-c", str(src), "-o", str(obj)]
        if verbose_ptxas:
            cmd.insert(1, "-Xptxas=-v")
    else:
        cmd = [_nvcc(), "-x", "cu", *ARCH, *common, "-c", str(src), "-o", str(obj)]
    want = _digest([src, *HEADERS], " ".join(cmd))
    if obj.exists() and stamp.exists() and stamp.read_text() == want:
        return obj
    _run(cmd)
    stamp.write_text(want)
    return obj


def build_library(verbose_ptxas: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    srcs = [CSRC / s for s in CUDA_SOURCES + CXX_SOURCES]
    with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 1)) as ex:
        objs = list(ex.map(lambda s: _compile_one(s, verbose_ptxas), srcs))
    link = [_nvcc(), "-shared", *ARCH, "-o", str(LIB), *map(str, objs)]
    stamp = OBJ / "lib.stamp"
    want = _digest(objs, " ".join(link))
    if LIB.exists() and stamp.exists() and stamp.read_text() == want:
        return LIB
    # libcuda is not linked: the TMA descriptor encoder is looked up at run time through
    # cudaGetDriverEntryPoint, so the library also loads on machines without a driver.
    # The CUDA runtime is linked statically (nvcc's default) so that the runtime version always
    # matches the compiler that produced the kernels, whatever else the process has loaded.
    _run(link)
    stamp.write_text(want)
    return LIB


def pymodule_path() -> Path:
    return PKG / ("pyaotriton" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_pymodule() -> Path:
    import pybind11

    OBJ.mkdir(exist_ok=True)
    out = pymodule_path()
    src = CSRC / "pyaotriton.cc"
    cuda_inc = Path(_nvcc()).resolve().parent.parent / "include"
    cmd = ["g++", "-O2", "-std=c++20", "-shared", "-fPIC", "-fvisibility=hidden",
           f"-I{ROOT / 'include'}", f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}",
           f"-I{cuda_inc}", *_suffix_flags(), str(src), "-o", str(out),
           f"-L{PKG}", "-l:libaotriton_v2.so", f"-L{cuda_inc.parent / 'lib64'}", "-lcudart_static",
           "-ldl", "-lrt", "-lpthread", "-Wl,-rpath,$ORIGIN"]
    stamp = OBJ / "pyaotriton.stamp"
    want = _digest([src, *HEADERS, LIB], " ".join(cmd))
    if out.exists() and stamp.exists() and stamp.read_text() == want:
        return out
    _run(cmd)
    stamp.write_text(want)
    return out


def build_all(verbose_ptxas: bool = False) -> None:
    build_library(verbose_ptxas)
    build_pymodule()


if __name__ == "__main__":
    os.environ.setdefault("AB200_BUILD_VERBOSE", "1")
    build_all(verbose_ptxas="-v" in sys.argv)
    print("built", LIB, "and", pymodule_path())
