"""Generate the golden fixtures by running the reference's own torch backend.

    python tests/golden/make_golden.py --reference /path/to/mlc-compiler

Needs the reference checkout (its ``mlc`` package and its ``tests/models.py``);
the fixtures it writes do not.  Two families:

* ``tiny/<model>__<config>__<dtype>.pt`` -- the reference's ten small test
  modules (``tests/models.py:15-126`` there) under four pass configurations and
  three dtypes, plus LayerNorm / softmax modules at awkward row lengths
  (1, 7, 33, 100, 1000, 1025 columns; 5 and 15 rows), persistent and streamed,
  plus modules that touch every scalar function and every reduction kind in
  fp32 / fp16 / bf16 / fp64 and int64.
  Each file holds the schedule (JSON), the parameters, the seeded
  inputs, the model outputs, and a snapshot of every buffer each kernel wrote,
  all computed by ``mlc.compile(..., Config(backend="torch"))`` on the CPU.
* ``bench/<schedule>.pt`` -- the benchmark-shaped configurations built from
  ``mlc_compiler_b200.models``: strided samples of the reference backend's
  outputs (full tensors would be tens of MB); weights and inputs are regenerated
  from their seeds by whoever checks against them.
"""

from __future__ import annotations

import argparse
import pathlib
import sys

import torch

HERE = pathlib.Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))

TINY_CONFIGS = {
    "default": {},
    "streamed": {"max_persistent_row": 4},
    "elementwise_only": {"reduction_fusion": False},
    "no_fusion": {"elementwise_fusion": False, "recompute": False, "reduction_fusion": False,
                  "memory_planning": False},
}
NARROW_MODELS = ("mlp", "softmax", "layernorm_scale", "attention", "block", "masked",
                 "broadcasting")


def _cast(model, inputs, dtype):
    if dtype == torch.float32:
        return model, inputs
    return model.to(dtype), tuple(a.to(dtype) if a.is_floating_point() else a for a in inputs)


def reference_run(model, inputs, cfg_kw, snapshots=True):
    """Compile with the reference, run on its torch backend, return the schedule
    in this package's IR plus outputs and per-kernel buffer snapshots."""
    import mlc
    from mlc.config import Config
    from mlc_compiler_b200 import kir

    cfg = Config(backend="torch", cuda_graphs=False, **cfg_kw)
    compiled = mlc.compile(model, inputs, cfg, device="cpu")
    out = compiled(*inputs)
    outs = [o.clone() for o in (out if isinstance(out, (tuple, list)) else [out])]
    sched = kir.from_reference(compiled.schedule)
    params = {sched.params[name]: t.clone() for name, t in compiled.params.items()
              if name in sched.params}
    snaps = {}
    if snapshots:
        graph = compiled.graph
        live = compiled._live
        buffers = {n: t.clone() for n, t in compiled.params.items() if n in live}
        for v, t in zip(graph.inputs, inputs):
            buffers[v.buffer.name] = t.contiguous().reshape(-1).clone()
        for b in graph.buffers():
            if b.name in live and b.name not in buffers:
                buffers[b.name] = torch.zeros(b.numel, dtype=b.dtype)
        for k in compiled.schedule.kernels:
            compiled.run_one(k, buffers)
            for v in k.writes():
                snaps[f"{k.name}/{v.buffer.name}"] = buffers[v.buffer.name].clone()
    return sched, params, outs, snaps


def make_tiny(out_dir: pathlib.Path, reference: str) -> None:
    from mlc_compiler_b200 import kir

    sys.path.insert(0, str(pathlib.Path(reference) / "tests"))
    import models as ref_models  # the reference's tests/models.py

    out_dir.mkdir(parents=True, exist_ok=True)
    for dtype in (torch.float32, torch.float16, torch.bfloat16):
        dname = str(dtype).replace("torch.", "")
        for cname, kw in TINY_CONFIGS.items():
            if dtype != torch.float32 and cname not in ("default", "streamed"):
                continue
            for name, model, inputs in ref_models.all_models():
                if dtype != torch.float32 and name not in NARROW_MODELS:
                    continue
                if name == "block_b8" and cname in ("elementwise_only", "no_fusion"):
                    continue  # same kernels as "block", five times the bytes
                model, inputs = _cast(model.eval(), inputs, dtype)
                sched, params, outs, snaps = reference_run(model, inputs, kw)
                path = out_dir / f"{name}__{cname}__{dname}.pt"
                torch.save({"schedule": kir.dumps(sched), "params": params,
                            "inputs": [t.clone() for t in inputs], "outputs": outs,
                            "snapshots": snaps}, path)
                print(f"{path.name}: {len(sched)} kernels {sched.counts()}, "
                      f"{path.stat().st_size / 1024:.1f} KiB", flush=True)


def make_odd(out_dir: pathlib.Path, reference: str) -> None:
    """Row lengths that do not divide any vector width, and row counts that do
    not fill a CTA: the shapes where masking and tail handling can go wrong."""
    from mlc_compiler_b200 import kir

    sys.path.insert(0, str(pathlib.Path(reference) / "tests"))
    import models as ref_models

    out_dir.mkdir(parents=True, exist_ok=True)
    for cols in (1, 7, 33, 100, 1000, 1025):
        for dtype in (torch.float32, torch.float16):
            dname = str(dtype).replace("torch.", "")
            for cname, kw in (("default", {}), ("streamed", {"max_persistent_row": 64})):
                if cname == "streamed" and cols <= 64:
                    continue
                g = torch.Generator().manual_seed(cols)
                cases = [
                    (f"oddln{cols}", ref_models.LayerNormScale(cols),
                     (torch.randn(5, cols, generator=g) * 3.0 + 1.0,)),
                    (f"oddsm{cols}", ref_models.Softmax(),
                     (torch.randn(3, 5, cols, generator=g) * 4.0,
                      torch.randn(1, 1, cols, generator=g))),
                ]
                for name, model, inputs in cases:
                    model, inputs = _cast(model.eval(), inputs, dtype)
                    sched, params, outs, snaps = reference_run(model, inputs, kw)
                    path = out_dir / f"{name}__{cname}__{dname}.pt"
                    torch.save({"schedule": kir.dumps(sched), "params": params,
                                "inputs": [t.clone() for t in inputs], "outputs": outs,
                                "snapshots": snaps}, path)
                    print(f"{path.name}: {sched.counts()}, {path.stat().st_size / 1024:.1f} KiB",
                          flush=True)


class EveryFloatFunction(torch.nn.Module):
    """Touches every float scalar function of the kernel IR at least once."""

    def forward(self, x, y):
        a = torch.exp(x * 0.1) + torch.log(y) + torch.sqrt(y) + torch.rsqrt(y) + torch.reciprocal(y)
        b = torch.sin(x) * torch.cos(x) + torch.tanh(x) + torch.erf(x) + torch.sigmoid(x) + torch.floor(x)
        c = torch.maximum(x, y) - torch.minimum(x, y) + torch.pow(y, x * 0.1) + torch.abs(x) - (-x)
        pick = torch.logical_or(x > y, torch.logical_and(x <= 0.0, torch.logical_not(x == y)))
        d = torch.where(pick, a, b) + (x >= 0.5).to(x.dtype) + (x != y).to(x.dtype) + (x < 0).to(x.dtype)
        e = torch.nn.functional.silu(x) + torch.relu(y) + torch.nn.functional.gelu(x, approximate="tanh")
        return a / c.abs().clamp(min=0.5) + d, e + torch.nn.functional.gelu(y)


class IntegerFunctions(torch.nn.Module):
    def forward(self, i, j):
        k = (i + j) * 3 - i.abs() + torch.maximum(i, j) - torch.minimum(i, j)
        return k, torch.logical_and(i > j, j != 0), -i


class ReductionKinds(torch.nn.Module):
    """sum / max / min / prod, a count of booleans, mean and variance in one graph."""

    def forward(self, x):
        return (x.amin(-1), x.amax(-1), (x > 0).sum(-1), x.mean(-1), x.var(-1),
                x.sum(-1, keepdim=True) * x)


class ProductRows(torch.nn.Module):
    def forward(self, s):
        return (s * 0.25 + 1.0).prod(-1)


def make_functions(out_dir: pathlib.Path) -> None:
    """Coverage of the whole scalar function table and of every reduction kind,
    in every float width, computed by the reference backend."""
    from mlc_compiler_b200 import kir

    out_dir.mkdir(parents=True, exist_ok=True)
    g = torch.Generator().manual_seed(7)
    x = torch.randn(6, 40, generator=g) * 1.5
    y = torch.rand(6, 40, generator=g) * 2.0 + 0.25
    cases = []
    for dtype in (torch.float32, torch.float16, torch.bfloat16, torch.float64):
        cases.append(("fnfloat", EveryFloatFunction(), (x.to(dtype), y.to(dtype)), dtype))
        cases.append(("fnreduce", ReductionKinds(), (x.to(dtype),), dtype))
        cases.append(("fnprod", ProductRows(), (x[:, :5].contiguous().to(dtype),), dtype))
    i = torch.randint(-50, 50, (5, 24), generator=g)
    j = torch.randint(-50, 50, (5, 24), generator=g)
    cases.append(("fnint", IntegerFunctions(), (i, j), torch.int64))
    for name, model, inputs, dtype in cases:
        dname = str(dtype).replace("torch.", "")
        for cname, kw in (("default", {}), ("streamed", {"max_persistent_row": 4})):
            if cname == "streamed" and name not in ("fnreduce", "fnprod"):
                continue
            sched, params, outs, snaps = reference_run(model.eval(), inputs, kw)
            path = out_dir / f"{name}__{cname}__{dname}.pt"
            torch.save({"schedule": kir.dumps(sched), "params": params,
                        "inputs": [t.clone() for t in inputs], "outputs": outs,
                        "snapshots": snaps}, path)
            print(f"{path.name}: {sched.counts()}, {path.stat().st_size / 1024:.1f} KiB", flush=True)


#: (schedule stem, model, batch, dtype, variant, sample stride)
BENCH_CASES = [
    ("encoder-block_b1_s128_float32", "encoder-block", 1, torch.float32, {}, 13),
    ("micro-layernorm_b1_s128_float16", "micro-layernorm", 1, torch.float16, {}, 7),
    ("micro-softmax_b1_s128_float16", "micro-softmax", 1, torch.float16, {}, 11),
    ("micro-gelu_b1_s128_float16", "micro-gelu", 1, torch.float16, {}, 13),
    ("micro-layernorm_b1_s128_bfloat16", "micro-layernorm", 1, torch.bfloat16, {}, 7),
    ("micro-softmax_b1_s128_bfloat16", "micro-softmax", 1, torch.bfloat16, {}, 11),
    ("micro-gelu_b1_s128_bfloat16", "micro-gelu", 1, torch.bfloat16, {}, 13),
    ("bert-base_b1_s128_float16", "bert-base", 1, torch.float16, {}, 1),
    ("bert-base_b1_s128_float32", "bert-base", 1, torch.float32, {}, 1),
    ("gpt2-small_b1_s128_float16", "gpt2-small", 1, torch.float16, {}, 1009),
    ("bert-base_b1_s128_bfloat16", "bert-base", 1, torch.bfloat16, {}, 1),
    ("gpt2-small_b1_s128_bfloat16", "gpt2-small", 1, torch.bfloat16, {}, 1009),
    ("bert-base_b4_s128_float16", "bert-base", 4, torch.float16, {}, 1),
    ("gpt2-small_b4_s128_float16", "gpt2-small", 4, torch.float16, {}, 4001),
    ("gpt2-small-ref_b1_s128_float16", "gpt2-small", 1, torch.float16,
     {"gelu": "erf", "tied_head": False}, 1009),
    ("bert-base-streamed_b1_s128_float16", "bert-base", 1, torch.float16, {}, 1,
     {"max_persistent_row": 64}),
    ("gpt2-small-streamed_b1_s128_float16", "gpt2-small", 1, torch.float16, {}, 1009,
     {"max_persistent_row": 64}),
]


def make_bench(out_dir: pathlib.Path, only: str | None) -> None:
    from mlc_compiler_b200 import models

    out_dir.mkdir(parents=True, exist_ok=True)
    for stem, name, batch, dtype, variant, stride, *rest in BENCH_CASES:
        if only and only not in stem:
            continue
        model, inputs = models.build(name, batch, dtype=dtype, **variant)
        sched, _, outs, _ = reference_run(model, inputs, rest[0] if rest else {}, snapshots=False)
        with torch.no_grad():
            eager = model(*inputs)
        eager = list(eager) if isinstance(eager, (tuple, list)) else [eager]
        path = out_dir / f"{stem}.pt"
        torch.save({"stride": stride, "kernels": len(sched), "counts": sched.counts(),
                    "samples": [o.reshape(-1)[::stride].clone() for o in outs],
                    "eager_samples": [o.reshape(-1)[::stride].clone() for o in eager],
                    "shapes": [tuple(o.shape) for o in outs]}, path)
        err = max(float((a.float() - b.float()).abs().max()) for a, b in zip(outs, eager))
        print(f"{path.name}: {len(sched)} kernels, max |ref backend - eager| = {err:.3e}, "
              f"{path.stat().st_size / 1024:.1f} KiB", flush=True)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--reference", required=True)
    ap.add_argument("--what", choices=("tiny", "odd", "functions", "bench", "all"), default="all")
    ap.add_argument("--only", default=None)
    args = ap.parse_args(argv)
    sys.dont_write_bytecode = True
    sys.path.insert(0, args.reference)
    torch.manual_seed(0)
    if args.what in ("tiny", "all"):
        make_tiny(HERE / "tiny", args.reference)
    if args.what in ("odd", "all"):
        make_odd(HERE / "tiny", args.reference)
    if args.what in ("functions", "all"):
        make_functions(HERE / "tiny")
    if args.what in ("bench", "all"):
        make_bench(HERE / "bench", args.only)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
