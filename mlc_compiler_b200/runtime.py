"""Compile, load and launch generated CUDA modules through the C ABI.

:class:`CudaRuntime` has the duck type the reference executor expects of its
kernel runtime (``TritonRuntime``, ``mlc/runtime/triton_runtime.py:60-97``):
``Runtime(schedule, cfg, device)``; ``.source``, ``.path``, ``.launch_table``;
``bind(k, buffers) -> (fn, grid, args, consts)`` with the executor later calling
``fn[grid](*args, **consts)`` (``mlc/runtime/executor.py:194-196``); ``launch(k,
buffers)``; both raise ``TypeError`` for extern kernels.  ``buffers[name]`` are
flat 1-D tensors owned by the executor; arguments are ``k.inputs`` then
``k.outputs`` in order.

There is no fallback: if ``libmlcb.so`` is missing or a module does not
compile, construction raises.
"""

from __future__ import annotations

import ctypes
import os
import pathlib

import torch

from . import build as _build
from . import kir
from .emit import generate_module


class BackendError(RuntimeError):
    """The native library is missing, or compiling / loading / launching failed."""


class _LaunchDesc(ctypes.Structure):
    _fields_ = [("kernel", ctypes.c_void_p), ("grid_x", ctypes.c_uint32),
                ("block_x", ctypes.c_uint32), ("smem_bytes", ctypes.c_uint32),
                ("flags", ctypes.c_uint32), ("device_ptrs", ctypes.POINTER(ctypes.c_uint64)),
                ("nptrs", ctypes.c_int32), ("reserved", ctypes.c_int32)]


_lib = None

#: every symbol include/mlcb.h declares, with its ctypes signature
_SIGNATURES = {
    "mlcb_version": (ctypes.c_int, []),
    "mlcb_last_error": (ctypes.c_char_p, []),
    "mlcb_compile": (ctypes.c_int, [ctypes.c_char_p, ctypes.c_char_p,
                                    ctypes.POINTER(ctypes.c_char_p), ctypes.c_int,
                                    ctypes.POINTER(ctypes.c_void_p),
                                    ctypes.POINTER(ctypes.c_size_t), ctypes.c_char_p,
                                    ctypes.c_size_t]),
    "mlcb_free_image": (None, [ctypes.c_void_p]),
    "mlcb_module_load": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int,
                                        ctypes.POINTER(ctypes.c_void_p)]),
    "mlcb_module_unload": (ctypes.c_int, [ctypes.c_void_p]),
    "mlcb_get_kernel": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_char_p,
                                       ctypes.POINTER(ctypes.c_void_p)]),
    "mlcb_kernel_info": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int),
                                        ctypes.POINTER(ctypes.c_int),
                                        ctypes.POINTER(ctypes.c_int)]),
    "mlcb_launch": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint32,
                                   ctypes.c_uint32, ctypes.POINTER(ctypes.c_uint64),
                                   ctypes.c_int, ctypes.c_uint64, ctypes.c_uint32]),
    "mlcb_launch_many": (ctypes.c_int, [ctypes.POINTER(_LaunchDesc), ctypes.c_int,
                                        ctypes.c_uint64, ctypes.POINTER(ctypes.c_int)]),
}


def library_path() -> pathlib.Path:
    return _build.LIB


def load_library(build_if_missing: bool = True):
    """``ctypes`` handle on ``libmlcb.so`` with every signature set."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not path.exists():
        if not build_if_missing:
            raise BackendError(f"{path} is missing: run `python -c 'import __graft_entry__ as g; "
                               "g.build()'` or mlc_compiler_b200.build.build_shim()")
        _build.build_shim()
    lib = ctypes.CDLL(str(path))
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def _check(lib, code: int, what: str) -> None:
    if code != 0:
        msg = lib.mlcb_last_error().decode(errors="replace")
        raise BackendError(f"{what} failed with code {code}: {msg}")


# --------------------------------------------------------------------------
# source -> image, with a content-addressed cache
# --------------------------------------------------------------------------

def cache_dir() -> pathlib.Path:
    """Same convention as the reference (``triton_runtime.py:29-33``)."""
    root = os.environ.get("MLC_CACHE_DIR")
    path = pathlib.Path(root) if root else pathlib.Path.home() / ".cache" / "mlc"
    path.mkdir(parents=True, exist_ok=True)
    return path


def _write_atomic(path: pathlib.Path, data: bytes) -> None:
    tmp = path.with_name(path.name + f".{os.getpid()}.tmp")
    tmp.write_bytes(data)
    tmp.replace(path)


def write_source(source: str) -> pathlib.Path:
    path = cache_dir() / f"mlcb_{_build.module_key(source)}.cu"
    if not path.exists() or path.read_text() != source:
        _write_atomic(path, source.encode())
    return path


def compile_source(source: str, *, use_cache: bool = True) -> bytes:
    """CUDA C++ -> sm_100a cubin.  Order: user cache, in-tree prebuilt images,
    NVRTC through the shim, ``nvcc`` as the last resort.  Raises on failure."""
    key = _build.module_key(source)
    cached = cache_dir() / f"mlcb_{key}.cubin"
    prebuilt = _build.PREBUILT / f"mlcb_{key}.cubin"
    if use_cache:
        for p in (cached, prebuilt):
            if p.exists() and p.stat().st_size > 0:
                return p.read_bytes()
    lib = load_library()
    inc = _build.cuda_home() / "include"
    opts = list(_build.NVRTC_FLAGS) + [f"-I{inc}"]
    arr = (ctypes.c_char_p * len(opts))(*[o.encode() for o in opts])
    image = ctypes.c_void_p()
    size = ctypes.c_size_t()
    log = ctypes.create_string_buffer(1 << 16)
    code = lib.mlcb_compile(source.encode(), _build.ARCH.encode(), arr, len(opts),
                            ctypes.byref(image), ctypes.byref(size), log, len(log))
    if code == 0:
        data = ctypes.string_at(image.value, size.value)
        lib.mlcb_free_image(image)
    else:
        first = lib.mlcb_last_error().decode(errors="replace")
        if _build.nvcc_path() is None:
            raise BackendError(f"NVRTC compile failed (code {code}) and nvcc is absent:\n{first}")
        try:
            _build.nvcc_cubin(source, cached)
        except RuntimeError as e:
            raise BackendError(f"NVRTC compile failed (code {code}): {first}\n"
                               f"nvcc fallback failed too: {e}") from None
        return cached.read_bytes()
    if use_cache:
        _write_atomic(cached, data)
    return data


# --------------------------------------------------------------------------
# loaded module
# --------------------------------------------------------------------------

class LoadedModule:
    """A cubin resident on one device, kernels looked up lazily by symbol."""

    def __init__(self, image: bytes, device_index: int):
        self.lib = load_library()
        self._image = image
        h = ctypes.c_void_p()
        _check(self.lib, self.lib.mlcb_module_load(image, len(image), int(device_index),
                                                   ctypes.byref(h)), "mlcb_module_load")
        self.handle = h
        self._kernels: dict[str, ctypes.c_void_p] = {}

    def kernel(self, symbol: str) -> ctypes.c_void_p:
        k = self._kernels.get(symbol)
        if k is None:
            k = ctypes.c_void_p()
            _check(self.lib, self.lib.mlcb_get_kernel(self.handle, symbol.encode(),
                                                      ctypes.byref(k)), f"mlcb_get_kernel({symbol})")
            self._kernels[symbol] = k
        return k

    def info(self, symbol: str) -> dict:
        regs, smem, mt = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        _check(self.lib, self.lib.mlcb_kernel_info(self.kernel(symbol), ctypes.byref(regs),
                                                   ctypes.byref(smem), ctypes.byref(mt)),
               "mlcb_kernel_info")
        return {"registers": regs.value, "static_smem": smem.value, "max_threads": mt.value}

    def close(self) -> None:
        if self.handle is not None and self.handle.value:
            self.lib.mlcb_module_unload(self.handle)
            self.handle = None

    def __del__(self):  # pragma: no cover - interpreter shutdown order
        try:
            self.close()
        except Exception:
            pass


class BoundLaunch:
    """One resolved launch: ``bound[grid](*tensors, **consts)`` enqueues it on
    torch's current stream.  Pointers are taken once, at bind time, from the
    executor's pointer-stable buffer table; if called with a different tuple of
    tensors they are re-read."""

    __slots__ = ("lib", "kernel", "grid", "block", "smem", "flags", "tensors", "ptrs",
                 "nptrs", "name", "device")

    def __init__(self, lib, kernel, name, grid, block, smem, flags, tensors, device=None):
        self.lib, self.kernel, self.name = lib, kernel, name
        #: the device the module lives on: launches go to *its* current stream
        self.device = device
        self.grid, self.block, self.smem, self.flags = int(grid), int(block), int(smem), int(flags)
        self._set(tuple(tensors))

    def _set(self, tensors) -> None:
        for t in tensors:
            if t.data_ptr() % 32 != 0:
                raise BackendError(f"{self.name}: buffer at {t.data_ptr():#x} is not 32-byte "
                                   "aligned; packed accesses were proven from aligned bases")
        self.tensors = tensors
        self.nptrs = len(tensors)
        self.ptrs = (ctypes.c_uint64 * max(1, self.nptrs))(*[t.data_ptr() for t in tensors])

    def __getitem__(self, grid):
        return self

    def __call__(self, *tensors, **consts) -> None:
        if tensors and tensors is not self.tensors and \
                any(a is not b for a, b in zip(tensors, self.tensors)):
            self._set(tuple(tensors))
        stream = torch.cuda.current_stream(self.device).cuda_stream
        code = self.lib.mlcb_launch(self.kernel, self.grid, self.block, self.smem, self.ptrs,
                                    self.nptrs, stream, self.flags)
        if code != 0:
            _check(self.lib, code, f"launch of {self.name}")

    def desc(self) -> _LaunchDesc:
        return _LaunchDesc(self.kernel.value, self.grid, self.block, self.smem, self.flags,
                           ctypes.cast(self.ptrs, ctypes.POINTER(ctypes.c_uint64)), self.nptrs, 0)


class LaunchRun:
    """Consecutive generated kernels enqueued by one ``mlcb_launch_many`` call."""

    def __init__(self, lib, bound: list[BoundLaunch]):
        self.lib = lib
        self.bound = bound  # keeps pointer arrays alive
        self.device = bound[0].device if bound else None
        self.descs = (_LaunchDesc * len(bound))(*[b.desc() for b in bound])
        self.failed = ctypes.c_int(-1)

    def __call__(self) -> None:
        stream = torch.cuda.current_stream(self.device).cuda_stream
        code = self.lib.mlcb_launch_many(self.descs, len(self.bound), stream,
                                         ctypes.byref(self.failed))
        if code != 0:
            i = self.failed.value
            who = self.bound[i].name if 0 <= i < len(self.bound) else "?"
            _check(self.lib, code, f"launch of {who}")


class CudaRuntime:
    """Drop-in for the reference's ``TritonRuntime``."""

    def __init__(self, schedule, cfg, device) -> None:
        device = torch.device(device)
        if device.type != "cuda":
            raise BackendError(f"the CUDA backend cannot run on {device}; "
                               "use backend='torch' for the reference interpreter")
        self.device = device
        self.cfg = cfg
        self.ir = schedule if isinstance(schedule, kir.Schedule) else kir.from_reference(schedule)
        self.generated = generate_module(self.ir, cfg)
        self.source = self.generated.source
        self.path = write_source(self.source)
        self.launch_table = self.generated.launch_table()
        index = device.index if device.index is not None else torch.cuda.current_device()
        self.device = torch.device("cuda", index)
        torch.cuda.init()
        with torch.cuda.device(index):
            torch.cuda.current_stream()  # makes sure the primary context exists
            self.loaded = LoadedModule(compile_source(self.source), index)
        self.lib = self.loaded.lib
        # "chain" and "auto" are resolved per launch by an executor that knows the stream order;
        # a host that binds kernels one by one gets plain launches
        self.flags = 1 if getattr(cfg, "dependent_launch", False) is True else 0
        self.chain = getattr(cfg, "dependent_launch", False) in ("chain", "auto")

    @staticmethod
    def _is_extern(k) -> bool:
        return type(k).__name__ == "ExternKernel"

    @staticmethod
    def _buffer_names(k) -> list[str]:
        names = []
        for a in list(k.inputs) + list(k.outputs):
            names.append(a.buffer if isinstance(a, kir.Operand) else a.value.buffer.name)
        return names

    def bind(self, k, buffers: dict[str, torch.Tensor], flags: int | None = None):
        if self._is_extern(k):
            raise TypeError("extern kernels do not go through the CUDA runtime")
        spec = self.generated.launch[k.name]
        tensors = tuple(buffers[n] for n in self._buffer_names(k))
        if flags is None:
            flags = self.flags
        fn = BoundLaunch(self.lib, self.loaded.kernel(self.generated.symbol[k.name]), k.name,
                         spec.grid, spec.block, spec.smem, flags, tensors, self.device)
        return fn, spec.grid, tensors, {}

    def launch(self, k, buffers: dict[str, torch.Tensor]) -> None:
        fn, grid, args, consts = self.bind(k, buffers)
        fn[grid](*args, **consts)

    def kernel_info(self, name: str) -> dict:
        return self.loaded.info(self.generated.symbol[name])
