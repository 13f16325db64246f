"""Bridge to the reference frontend.

Capture, fusion, lowering and memory planning are the reference's own
(``mlc/api.py:17-46``: ``capture`` -> ``plan`` -> ``build_schedule`` ->
``plan_memory``); this backend starts at the schedule they produce.  When the
``mlc`` package is importable these helpers run it and convert the result to
this package's IR; on a machine without it, schedules are loaded from their
serialised form instead (:func:`load_schedule`).
"""

from __future__ import annotations

import dataclasses
import importlib
import pathlib

from . import kir
from .config import Config

SCHEDULE_DIR = pathlib.Path(__file__).resolve().parent / "schedules"


class FrontendUnavailable(ImportError):
    pass


def reference():
    """The reference package, or a clear error."""
    try:
        return importlib.import_module("mlc")
    except ImportError as e:
        raise FrontendUnavailable(
            "the mlc frontend (capture, fusion, lowering, memory planning) is not importable; "
            "put the reference checkout on sys.path, or load a serialised schedule with "
            "mlc_compiler_b200.load_schedule()") from e


def reference_config(cfg: Config):
    """This package's ``Config`` as the reference's dataclass (shared fields)."""
    ref_cfg_cls = importlib.import_module("mlc.config").Config
    names = {f.name for f in dataclasses.fields(ref_cfg_cls)}
    kw = {f.name: getattr(cfg, f.name) for f in dataclasses.fields(cfg) if f.name in names}
    if kw.get("backend") == "cuda":
        kw["backend"] = "auto"
    return ref_cfg_cls(**kw)


def capture_schedule(model, example_inputs, cfg: Config | None = None) -> kir.Schedule:
    """Run the reference's frontend and passes on ``model`` and return the
    schedule in this package's IR."""
    reference()
    cfg = cfg or Config()
    capture = importlib.import_module("mlc.ir.capture").capture
    build_pipeline = importlib.import_module("mlc.api").build_pipeline
    graph = capture(model, tuple(example_inputs))
    sched = build_pipeline(graph, reference_config(cfg))
    return kir.from_reference(sched)


def schedule_path(name: str) -> pathlib.Path:
    return SCHEDULE_DIR / f"{name}.json.gz"


def load_schedule(name_or_path) -> kir.Schedule:
    """A shipped schedule by name (``"bert-base_b1_s128_float16"``) or any path."""
    p = pathlib.Path(str(name_or_path))
    if not p.exists():
        p = schedule_path(str(name_or_path))
    if not p.exists():
        have = sorted(q.name[:-8] for q in SCHEDULE_DIR.glob("*.json.gz"))
        raise FileNotFoundError(f"no schedule {name_or_path!r}; shipped: {have}")
    return kir.load(p)
