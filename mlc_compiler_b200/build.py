"""In-tree build of the native pieces.

``libmlcb.so`` (the C-ABI shim, ``csrc/mlcb_shim.cpp``) is compiled next to the
sources so that it travels with the tree; generated kernel modules are compiled
for sm_100a either by NVRTC through the shim (at run time) or by ``nvcc -cubin``
(here: the no-GPU build check, and a fallback when NVRTC is unusable).
"""

from __future__ import annotations

import hashlib
import os
import pathlib
import shutil
import subprocess

PKG = pathlib.Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIB = PKG / "libmlcb.so"
PREBUILT = PKG / "_prebuilt"

ARCH = "sm_100a"
GENCODE = ["-gencode", "arch=compute_100a,code=sm_100a"]
#: flags every generated module is compiled with, whichever compiler runs:
#: no multiply-add contraction and no fast-math, so float results follow the
#: reference's op-by-op rounding
NVCC_FLAGS = ["-std=c++17", "--fmad=false", "-lineinfo"]
NVRTC_FLAGS = ["--std=c++17", "--fmad=false", "--generate-line-info"]


def cuda_home() -> pathlib.Path:
    for env in ("CUDA_HOME", "CUDA_PATH"):
        v = os.environ.get(env)
        if v and (pathlib.Path(v) / "include" / "cuda.h").exists():
            return pathlib.Path(v)
    nvcc = shutil.which("nvcc")
    if nvcc:
        return pathlib.Path(nvcc).resolve().parent.parent
    return pathlib.Path("/usr/local/cuda")


def nvcc_path() -> str | None:
    p = cuda_home() / "bin" / "nvcc"
    return str(p) if p.exists() else shutil.which("nvcc")


def _stale(target: pathlib.Path, sources: list[pathlib.Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(s.stat().st_mtime > t for s in sources)


def build_shim(force: bool = False) -> pathlib.Path:
    """Compile ``libmlcb.so``.  Needs only a C++ compiler and the CUDA headers;
    the driver and NVRTC are opened with dlopen when first used."""
    srcs = [CSRC / "mlcb_shim.cpp", ROOT / "include" / "mlcb.h"]
    extra = sorted(CSRC.glob("*.cu"))
    if not force and not _stale(LIB, srcs + extra):
        return LIB
    inc = cuda_home() / "include"
    tmp = LIB.with_suffix(f".so.{os.getpid()}.tmp")
    if extra:
        # static kernels ride in the same library; nvcc links cudart statically,
        # which itself opens libcuda lazily
        cmd = [nvcc_path(), *GENCODE, "-lineinfo", "-O3", "-std=c++17", "-shared",
               "-Xcompiler", "-fPIC", "-I", str(ROOT / "include"),
               str(CSRC / "mlcb_shim.cpp"), *map(str, extra), "-o", str(tmp), "-ldl"]
    else:
        cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-I", str(inc),
               "-I", str(ROOT / "include"), str(CSRC / "mlcb_shim.cpp"), "-o", str(tmp),
               "-ldl", "-lpthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"building libmlcb.so failed:\n{' '.join(cmd)}\n{r.stderr}")
    tmp.replace(LIB)
    return LIB


def module_key(source: str, arch: str = ARCH) -> str:
    h = hashlib.sha256()
    h.update(source.encode())
    h.update(arch.encode())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def nvcc_cubin(source: str, out: pathlib.Path, verbose: bool = False) -> str:
    """``nvcc -cubin`` for sm_100a; returns the compiler's stderr (``-Xptxas -v``
    resource lines when ``verbose``).  Works without a GPU."""
    nvcc = nvcc_path()
    if nvcc is None:
        raise RuntimeError("nvcc not found")
    out.parent.mkdir(parents=True, exist_ok=True)
    src = out.with_suffix(".cu")
    src.write_text(source)
    tmp = out.with_suffix(f".cubin.{os.getpid()}.tmp")
    cmd = [nvcc, *GENCODE, *NVCC_FLAGS, "-cubin", "-o", str(tmp), str(src)]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{r.stderr[-4000:]}")
    tmp.replace(out)
    return r.stderr


def prebuild(source: str) -> pathlib.Path:
    """Compile ``source`` into the in-tree image cache (content-addressed)."""
    out = PREBUILT / f"mlcb_{module_key(source)}.cubin"
    if not out.exists():
        nvcc_cubin(source, out)
    return out


EXAMPLE = CSRC / "examples" / "bert-base_b8_s128_float16.cu"


def example_source() -> str:
    """The translation unit the executor compiles for BERT-base fp16 at batch 8
    (after producer forwarding): every kernel family in one readable file.  A
    copy is kept under ``csrc/examples`` so that the generated CUDA can be read
    without running anything; ``write_example`` refreshes it and a test keeps it
    honest."""
    from .config import Config
    from .emit import generate_module
    from .frontend import load_schedule
    from .rewrite import prepare

    sched = prepare(load_schedule("bert-base_b8_s128_float16"), Config())
    text = generate_module(sched, Config(), inline_header=False).source
    # the copy lives one directory below the device header
    return text.replace('#include "mlcb_device.cuh"', '#include "../mlcb_device.cuh"')


def write_example() -> pathlib.Path:
    EXAMPLE.parent.mkdir(parents=True, exist_ok=True)
    text = example_source()
    if not EXAMPLE.exists() or EXAMPLE.read_text() != text:
        EXAMPLE.write_text(text)
    return EXAMPLE
