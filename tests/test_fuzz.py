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
    sched = kir.Schedule("fuzz", kernels, specs, params={b: b for b in g.params})
    return sched, buffers


@pytest.mark.parametrize("seed", SEEDS)
def test_corpus_is_accepted_by_the_oracle_and_the_emitter(seed):
    sched, buffers = corpus(seed)
    mod = generate_module(sched, Config())
    assert len(mod.launch) == N_POINTWISE + N_REDUCTION
    # the corpus reaches the paths that depend on what a schedule declares: parameters
    # read ahead of the grid-dependency wait (packed and per-row scalar), and element
    # outputs stored before the first reduction
    assert len(sched.params) >= 30
    assert mod.source.count("mlcb_load_raw<") >= 10
    early = [k for k in sched.kernels if isinstance(k, kir.ReductionKernel)
             and sum(a.name not in k.row_outputs for a in k.outputs) == 2]
    assert len(early) >= 3
    for k in early:
        text = mod.kernel_source(k.name)
        assert text.index("out1 + out1_r") < text.index("_reduce<")
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


@pytest.mark.parametrize("seed", SEEDS)
def test_iteration_order_never_matters_for_random_pointwise_kernels(seed):
    """``rewrite.output_major`` renumbers a pointwise kernel's iterations.  Every
    random kernel (strided / broadcast / padded operands) is first scrambled with a
    random digit order, then put back into output order; all three must write the
    same bytes, and the restored one must walk its output in storage order."""
    import random

    from mlc_compiler_b200 import rewrite

    sched, buffers = corpus(seed)
    rng = random.Random(seed)
    scrambled = 0
    for k in sched.kernels:
        if not isinstance(k, kir.PointwiseKernel):
            continue

        def shuffle(n):
            order = list(range(n))
            rng.shuffle(order)
            return order
        mixed = rewrite.output_major(k, order=shuffle)
        back = rewrite.output_major(mixed)
        if mixed is k:
            continue
        scrambled += 1
        assert mixed.numel == back.numel == k.numel
        strides = [t[2] for t in back.outputs[0].index.axes[0].terms]
        assert strides == sorted(strides, reverse=True)
        results = []
        for variant in (k, mixed, back):
            bufs = {n: t.clone() for n, t in buffers.items()
                    if n in set(k.reads()) | set(k.writes())}
            oracle.run_kernel(variant, bufs)
            results.append(bufs)
        # exactly the same (operand offsets..., output offsets...) tuples, in another order
        def visits(v):
            ops = list(v.inputs) + list(v.outputs)
            return sorted(tuple(a.index.offset(idx=i) for a in ops) for i in range(v.numel))
        if k.numel <= 4096:
            assert visits(k) == visits(mixed) == visits(back), k.name
        # and the same values: exact for integers; for floats up to the last bit, because
        # ATen's CPU kernels round exp/tanh/pow differently in their vector body and their
        # scalar tail, and renumbering moves elements between the two
        for out in k.outputs:
            x = results[0][out.buffer]
            for other in results[1:]:
                y = other[out.buffer]
                if not x.is_floating_point():
                    assert torch.equal(x, y), k.name
                    continue
                x64, y64 = x.double(), y.double()
                assert torch.equal(torch.isnan(x64), torch.isnan(y64)), k.name
                torch.testing.assert_close(torch.nan_to_num(y64), torch.nan_to_num(x64),
                                           rtol=2e-6 if x.dtype == torch.float32 else 1e-2, atol=1e-7)
        generate_module(kir.Schedule("one", [mixed, kir.PointwiseKernel(
            back.name + "_b", back.space, back.inputs, back.outputs, back.body, back.out_expr,
            back.ops)], sched.buffers), Config())
    assert scrambled >= 10


@pytest.mark.gpu
def test_scrambled_pointwise_kernels_match_the_oracle_on_the_gpu():
    """The emitter on kernels whose iteration order follows no operand (what a
    layout rewrite can leave behind) and on the same kernels put back in output
    order."""
    import random

    from mlc_compiler_b200 import rewrite
    from mlc_compiler_b200.runtime import CudaRuntime

    dev = torch.device("cuda", 0)
    sched, buffers = corpus(SEEDS[0])
    rng = random.Random(5)
    kernels = []
    for k in sched.kernels:
        if not isinstance(k, kir.PointwiseKernel):
            continue

        def shuffle(n):
            order = list(range(n))
            rng.shuffle(order)
            return order
        mixed = rewrite.output_major(k, order=shuffle)
        if mixed is k:
            continue
        back = rewrite.output_major(mixed)
        kernels.append(kir.PointwiseKernel(k.name + "_m", mixed.space, mixed.inputs, mixed.outputs,
                                           mixed.body, mixed.out_expr, mixed.ops))
        kernels.append(kir.PointwiseKernel(k.name + "_b", back.space, back.inputs, back.outputs,
                                           back.body, back.out_expr, back.ops))
    assert len(kernels) >= 20
    rt = CudaRuntime(kir.Schedule("scrambled", kernels, sched.buffers), Config(), dev)
    failures = []
    for k in kernels:
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
