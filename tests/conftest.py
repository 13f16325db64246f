import os
import pathlib
import sys

import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "oracle"))
os.environ.setdefault("MLC_CACHE_DIR", str(ROOT / ".mlc_cache"))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def tiny_cases():
    return sorted(p.stem for p in (GOLDEN / "tiny").glob("*.pt"))


def load_tiny(stem):
    import torch
    from mlc_compiler_b200 import kir

    d = torch.load(GOLDEN / "tiny" / f"{stem}.pt", weights_only=True)
    d["schedule"] = kir.loads(d["schedule"])
    return d


def tolerance(dtype_name: str) -> float:
    """Parity bar against the torch reference backend: max-abs/rel 1e-4 for
    fp32 (and wider), 1e-2 for fp16/bf16."""
    return 1e-2 if dtype_name in ("float16", "bfloat16") else 1e-4


def assert_close(got, want, dtype_name: str, what: str = ""):
    import torch

    if want.dtype == torch.bool or not want.is_floating_point():
        assert torch.equal(got.cpu(), want.cpu()), f"{what}: integer/bool mismatch"
        return
    tol = tolerance(dtype_name)
    g, w = got.detach().cpu().double(), want.detach().cpu().double()
    assert g.shape == w.shape, f"{what}: shape {tuple(g.shape)} vs {tuple(w.shape)}"
    same_nonfinite = (torch.isnan(g) == torch.isnan(w)).all() and \
        (g[torch.isinf(w)] == w[torch.isinf(w)]).all()
    assert same_nonfinite, f"{what}: non-finite pattern differs"
    fin = torch.isfinite(w)
    err = (g[fin] - w[fin]).abs()
    bound = tol + tol * w[fin].abs()
    assert bool((err <= bound).all()), (
        f"{what}: max abs err {err.max().item():.3e} exceeds {tol:g} abs/rel")


def as_float64(d: dict) -> dict:
    """A float32 fixture with every float32 buffer, operand and tensor made float64
    (index maps are in elements, so nothing else changes).  No golden outputs: the
    caller compares with the oracle."""
    import dataclasses

    import torch
    from mlc_compiler_b200 import kir

    s = d["schedule"]

    def up(dt):
        return "float64" if dt == "float32" else dt

    def operand(a):
        return dataclasses.replace(a, dtype=up(a.dtype))

    kernels = []
    for k in s.kernels:
        if isinstance(k, kir.ExternKernel):
            kernels.append(k)
        else:
            kernels.append(dataclasses.replace(k, inputs=[operand(a) for a in k.inputs],
                                               outputs=[operand(a) for a in k.outputs]))
    buffers = {n: dataclasses.replace(b, dtype=up(b.dtype)) for n, b in s.buffers.items()}
    wide = dataclasses.replace(s, kernels=kernels, buffers=buffers)
    cast = lambda t: t.double() if t.dtype == torch.float32 else t          # noqa: E731
    return {"schedule": wide, "params": {n: cast(t) for n, t in d["params"].items()},
            "inputs": [cast(t) for t in d["inputs"]]}
