"""The CPU oracle against the reference's own outputs (golden fixtures).

Every fixture under tests/golden/tiny was produced by the reference's torch
backend; the oracle has to reproduce each kernel's written buffers and the
model outputs from the same schedule, parameters and inputs.
"""

import pytest
import torch

import kir_oracle as oracle
from conftest import GOLDEN, load_tiny, tiny_cases
from mlc_compiler_b200 import kir, models
from mlc_compiler_b200.frontend import load_schedule


@pytest.mark.parametrize("stem", tiny_cases())
def test_oracle_matches_reference_per_kernel(stem):
    d = load_tiny(stem)
    s = d["schedule"]
    buffers = oracle.allocate(s, d["params"], d["inputs"], fill=0.0)
    for k in s.kernels:
        oracle.run_kernel(k, buffers)
        for b in k.writes():
            want = d["snapshots"][f"{k.name}/{b}"]
            # same operators on the same machine family: equal up to the last bit
            # of libm differences between hosts
            torch.testing.assert_close(buffers[b], want, rtol=1e-6, atol=1e-7,
                                       equal_nan=True, msg=lambda m: f"{stem} {k.name}/{b}: {m}")
            buffers[b] = want.clone()


@pytest.mark.parametrize("stem", tiny_cases())
def test_oracle_matches_reference_end_to_end(stem):
    d = load_tiny(stem)
    out, _ = oracle.run_schedule(d["schedule"], d["params"], d["inputs"])
    outs = list(out) if isinstance(out, tuple) else [out]
    assert len(outs) == len(d["outputs"])
    for got, want in zip(outs, d["outputs"]):
        torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-6, equal_nan=True)


BENCH = sorted(p.stem for p in (GOLDEN / "bench").glob("*.pt"))


@pytest.mark.parametrize("stem", [s for s in BENCH if s.startswith(("micro", "encoder"))])
def test_oracle_matches_reference_on_benchmark_kernels(stem):
    """Benchmark-shaped kernels: weights and inputs regenerated from their seeds,
    outputs compared with strided samples of the reference backend's."""
    g = torch.load(GOLDEN / "bench" / f"{stem}.pt", weights_only=True)
    s = load_schedule(stem)
    m = s.meta
    model, inputs = models.build(m["model"], m["batch"], dtype=kir.torch_dtype(m["dtype"]),
                                 **m.get("variant", {}))
    out, _ = oracle.run_schedule(s, model, inputs)
    outs = list(out) if isinstance(out, tuple) else [out]
    for got, want in zip(outs, g["samples"]):
        torch.testing.assert_close(got.reshape(-1)[::g["stride"]], want, rtol=1e-5, atol=1e-6)


def test_streamed_softmax_with_minus_inf_rows_is_finite():
    """The per-row online recurrence must stay finite on causal fp16 rows whose
    masked entries are -inf (the reference's Triton text does not; its torch
    backend, which the oracle follows, does)."""
    d = load_tiny("softmax__streamed__float16")
    s = d["schedule"]
    x, mask = d["inputs"]
    mask = mask.clone()
    mask[..., 1::2] = float("-inf")
    out, _ = oracle.run_schedule(s, d["params"], [x, mask])
    assert torch.isfinite(out).all()
    want = ((x.float() * 0.125) + mask.float()).softmax(-1)
    torch.testing.assert_close(out.float(), want, rtol=1e-2, atol=1e-2)
