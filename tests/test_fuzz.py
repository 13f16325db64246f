"""Differential fuzzing of the emitter: seeded random kernels, oracle vs CUDA.

The CPU half checks that every random kernel is accepted by the oracle and the
emitter and (in batches) compiles for sm_100a; the GPU half runs them."""

import shutil

import pytest
import torch

import kir_oracle as oracle
from conftest import assert_close
from fuzz_kernels import Gen, special_cases
from mlc_compiler_b200 import Config, kir
from mlc_compiler_b200 import build as B
from mlc_compiler_b200.emit import generate_module

N_POINTWISE, N_REDUCTION = 48, 36


SEEDS = [2024, 7, 99]


def corpus(seed: int = 2024):
    g = Gen(seed)
    kernels, specs, buffers = [], {}, {}
    for i in range(N_POINTWISE):
        k, s, b = g.pointwise(f"p{i}")
        kernels.append(k), specs.update(s), buffers.update(b)
    for i in range(N_REDUCTION):
        k, s, b = g.reduction(f"r{i}", streamed=(i % 3 == 2))
        kernels.append(k), specs.update(s), buffers.update(b)
    sched = kir.Schedule("fuzz", kernels, specs)
    return sched, buffers


@pytest.mark.parametrize("seed", SEEDS)
def test_corpus_is_accepted_by_the_oracle_and_the_emitter(seed):
    sched, buffers = corpus(seed)
    mod = generate_module(sched, Config())
    assert len(mod.launch) == N_POINTWISE + N_REDUCTION
    for k in sched.kernels:
        oracle.run_kernel(k, buffers)
        for a in k.outputs:
            out = buffers[a.buffer]
            if out.is_floating_point():
                assert torch.isfinite(out.float()).all(), (k.name, a.name)   # domains were respected
    # JSON form survives everything the generator can produce
    assert kir.dumps(kir.loads(kir.dumps(sched))) == kir.dumps(sched)


@pytest.mark.skipif(shutil.which("nvcc") is None and B.nvcc_path() is None, reason="nvcc not installed")
def test_corpus_compiles_for_sm_100a(tmp_path):
    sched, _ = corpus()
    log = B.nvcc_cubin(generate_module(sched, Config()).source, tmp_path / "fuzz.cubin", verbose=True)
    assert "error" not in log.lower()


@pytest.mark.gpu
@pytest.mark.parametrize("seed", SEEDS)
def test_corpus_matches_the_oracle_on_the_gpu(seed):
    from mlc_compiler_b200.runtime import CudaRuntime

    dev = torch.device("cuda", 0)
    sched, buffers = corpus(seed)
    rt = CudaRuntime(sched, Config(), dev)
    failures = []
    for k in sched.kernels:
        gpu = {b: buffers[b].to(dev) for b in set(k.reads()) | set(k.writes())}
        for b in k.writes():
            gpu[b].fill_(float("nan")) if gpu[b].is_floating_point() else gpu[b].fill_(1)
        rt.launch(k, gpu)
        oracle.run_kernel(k, buffers)
        torch.cuda.synchronize()
        for a in k.outputs:
            try:
                assert_close(gpu[a.buffer], buffers[a.buffer], a.dtype, f"{k.name}/{a.name}")
            except AssertionError as e:
                failures.append(str(e))
    assert not failures, "\n".join(failures[:10])


def test_special_cases_take_the_intended_code_paths():
    sched, buffers = special_cases()
    mod = generate_module(sched, Config())
    assert "transposing" in mod.kernel_source("tr16") and "transposing" in mod.kernel_source("trbf")
    assert mod.launch["wide"].vector == 16 and "mlcb_load<__half, 16>" in mod.kernel_source("wide")
    assert "double" in mod.kernel_source("fp64")
    for k in sched.kernels:
        oracle.run_kernel(k, buffers)


@pytest.mark.gpu
def test_special_cases_match_the_oracle_on_the_gpu():
    from mlc_compiler_b200.runtime import CudaRuntime

    dev = torch.device("cuda", 0)
    sched, buffers = special_cases()
    rt = CudaRuntime(sched, Config(), dev)
    for k in sched.kernels:
        gpu = {b: buffers[b].to(dev) for b in set(k.reads()) | set(k.writes())}
        for b in k.writes():
            gpu[b].fill_(float("nan")) if gpu[b].is_floating_point() else gpu[b].fill_(1)
        rt.launch(k, gpu)
        oracle.run_kernel(k, buffers)
        torch.cuda.synchronize()
        for a in k.outputs:
            assert_close(gpu[a.buffer], buffers[a.buffer], a.dtype, f"{k.name}/{a.name}")
