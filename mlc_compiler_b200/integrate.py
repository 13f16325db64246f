"""Drop-in installation into the reference, and the ``compile`` entry point.

The reference has no plugin registry: ``CompiledModel.__init__`` imports
``TritonRuntime`` from ``mlc.runtime.triton_runtime`` at every construction
(``mlc/runtime/executor.py:77-80``) after ``select_backend`` (``:28-38``) said
``"triton"``.  :func:`install` replaces those two attributes, so
``mlc.compile(model, example, Config(...))``, ``compiled.schedule``,
``compiled.source()`` and the CLI keep working and run generated CUDA instead.
``mlc.codegen.triton_backend.generate_module`` is re-pointed too, because
``python -m mlc source`` calls it directly (``mlc/__main__.py:116-118``).
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


def install() -> None:
    """Route the reference's generated-kernel path through this backend."""
    reference()
    from .runtime import CudaRuntime

    ex = importlib.import_module("mlc.runtime.executor")
    tr = importlib.import_module("mlc.runtime.triton_runtime")
    tb = importlib.import_module("mlc.codegen.triton_backend")
    if not _saved:
        _saved.update(select_backend=ex.select_backend, TritonRuntime=tr.TritonRuntime,
                      generate_module=tb.generate_module)
    ex.select_backend = _select_backend
    tr.TritonRuntime = CudaRuntime
    tb.generate_module = _source_text


def uninstall() -> None:
    if not _saved:
        return
    ex = importlib.import_module("mlc.runtime.executor")
    tr = importlib.import_module("mlc.runtime.triton_runtime")
    tb = importlib.import_module("mlc.codegen.triton_backend")
    ex.select_backend = _saved["select_backend"]
    tr.TritonRuntime = _saved["TritonRuntime"]
    tb.generate_module = _saved["generate_module"]
    _saved.clear()


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
