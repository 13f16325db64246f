"""Drop-in installation into the reference, and the ``compile`` entry point.

The reference has no plugin registry: ``CompiledModel.__init__`` imports
``TritonRuntime`` from ``mlc.runtime.triton_runtime`` at every construction
(``mlc/runtime/executor.py:77-80``) after ``select_backend`` (``:28-38``) said
``"triton"``.  :func:`install` replaces those two attributes, so
``mlc.compile(model, example, Config(...))``, ``compiled.schedule``,
``compiled.source()`` and the CLI keep working and run generated CUDA instead.
``mlc.codegen.triton_backend.generate_module`` is re-pointed too, because
``python -m mlc source`` calls it directly (``mlc/__main__.py:116-118``), and the
B200 entry is added to the reference's device table (``mlc/devices.py:107-134``),
which otherwise prices an unknown GPU as an A100.
"""

from __future__ import annotations

import importlib

import torch

from .config import Config
from .emit import generate_module as _generate_module
from .frontend import capture_schedule, reference

_saved: dict = {}


def _select_backend(cfg, device) -> str:
    """``auto`` on a CUDA device is the CUDA backend (reported as ``"triton"``
    so the reference executor takes its generated-kernel branch); ``torch``
    stays the reference interpreter; an explicit ``triton`` is refused; a CUDA
    device never falls back to the interpreter silently."""
    device = torch.device(device)
    if cfg.backend == "torch":
        return "torch"
    if cfg.backend == "triton":
        raise ValueError("the Triton backend has been removed; use backend='auto'")
    if cfg.backend not in ("auto", "cuda"):
        raise ValueError(f"unknown backend {cfg.backend!r}")
    if device.type == "cuda":
        return "triton"
    if cfg.backend == "cuda":
        raise RuntimeError(f"backend='cuda' needs a CUDA device, got {device}")
    return "torch"


def _source_text(schedule, cfg) -> str:
    return _generate_module(schedule, cfg).source


def install(native_executor: bool = False) -> None:
    """Route the reference's generated-kernel path through this backend.

    By default only the kernel runtime is swapped and the reference's own
    executor keeps driving it (same single-stream graph as before).  With
    ``native_executor=True`` ``mlc.compile`` additionally returns this package's
    executor for CUDA devices, which captures the schedule with parallel graph
    branches and folds producers into copies; ``backend="torch"`` and CPU
    devices still get the reference's executor and interpreter."""
    reference()
    from .runtime import CudaRuntime

    ex = importlib.import_module("mlc.runtime.executor")
    tr = importlib.import_module("mlc.runtime.triton_runtime")
    tb = importlib.import_module("mlc.codegen.triton_backend")
    api = importlib.import_module("mlc.api")
    if not _saved:
        _saved.update(select_backend=ex.select_backend, TritonRuntime=tr.TritonRuntime,
                      generate_module=tb.generate_module, CompiledModel=api.CompiledModel)
    ex.select_backend = _select_backend
    tr.TritonRuntime = CudaRuntime
    tb.generate_module = _source_text
    from . import devices

    devices.register_with_reference()      # mlc.devices.profile_for knows the B200 from here on
    api.CompiledModel = _native_factory(_saved["CompiledModel"]) if native_executor \
        else _saved["CompiledModel"]


def uninstall() -> None:
    if not _saved:
        return
    ex = importlib.import_module("mlc.runtime.executor")
    tr = importlib.import_module("mlc.runtime.triton_runtime")
    tb = importlib.import_module("mlc.codegen.triton_backend")
    ex.select_backend = _saved["select_backend"]
    tr.TritonRuntime = _saved["TritonRuntime"]
    tb.generate_module = _saved["generate_module"]
    importlib.import_module("mlc.api").CompiledModel = _saved["CompiledModel"]
    from . import devices

    devices.unregister_from_reference()
    _saved.clear()


def _native_factory(reference_executor):
    """A stand-in for the reference's ``CompiledModel(graph, schedule, cfg, device)``
    constructor (``mlc/api.py:33``) that builds this package's executor."""

    def make(graph, schedule, cfg, device):
        device = torch.device(device)
        if _select_backend(cfg, device) == "torch":
            return reference_executor(graph, schedule, cfg, device)
        return NativeCompiledModel(graph, schedule, cfg, device)

    return make


class NativeCompiledModel:
    """This package's executor behind the reference's ``CompiledModel`` surface:
    ``graph``, ``schedule`` (the reference's own object), ``cfg``, ``device``,
    ``backend``, ``__call__``, ``forward``, ``source()``, ``source_path()``,
    ``profile_kernels()``; outputs are re-assembled with the exporter's pytree
    spec exactly as ``_collect`` does (``mlc/runtime/executor.py:244-261``)."""

    def __init__(self, graph, schedule, cfg, device) -> None:
        from . import kir
        from .executor import CompiledModel

        self.graph, self.schedule, self.cfg = graph, schedule, cfg
        self.device = torch.device(device)
        self.backend = "cuda"
        ours = Config()
        for f in ours.__dataclass_fields__:
            if hasattr(cfg, f):
                setattr(ours, f, getattr(cfg, f))
        params = {v.buffer.name: graph.param_tensors[v.name] for v in graph.params}
        self._impl = CompiledModel(kir.from_reference(schedule), params, ours, self.device)
        self.params = self._impl.params
        self._out_spec = graph.meta.get("out_spec")

    def _shape(self, out):
        if self._out_spec is None:
            return out
        from torch.utils._pytree import tree_unflatten

        flat = list(out) if isinstance(out, tuple) else [out]
        try:
            return tree_unflatten(flat, self._out_spec)
        except Exception:
            return out

    def __call__(self, *inputs):
        return self._shape(self._impl(*inputs))

    def forward(self, *inputs):
        return self._shape(self._impl.forward(*inputs))

    def profile_kernels(self, inputs, iters: int = 20):
        return self._impl.profile_kernels(inputs, iters)

    def source(self) -> str:
        return self._impl.source()

    def source_path(self):
        return self._impl.source_path()

    @property
    def executed_schedule(self):
        return self._impl.executed_schedule

    def __repr__(self) -> str:  # pragma: no cover
        return (f"CompiledModel({self.graph.name}, {len(self.schedule)} kernels, "
                f"backend={self.backend}, device={self.device})")


def compile(model, example_inputs, config: Config | None = None, device=None):
    """Same signature as ``mlc.compile`` (``mlc/api.py:17-33``).  Captures with
    the reference frontend and executes on this package's own executor."""
    from .executor import CompiledModel

    cfg = config or Config()
    if device is None:
        device = next((t.device for t in example_inputs if torch.is_tensor(t)),
                      torch.device("cpu"))
    schedule = capture_schedule(model, example_inputs, cfg)
    return CompiledModel(schedule, model, cfg, device)
