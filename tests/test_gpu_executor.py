"""Executor contracts on a CUDA device: arena isolation, input checking, output
aliasing, CUDA-graph replay, per-kernel profiling, launches through the C ABI."""

import pytest
import torch

from conftest import assert_close, load_tiny
from mlc_compiler_b200 import Config, kir

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda", 0)


def _model(stem, dev, **cfg):
    from mlc_compiler_b200.executor import CompiledModel

    d = load_tiny(stem)
    return d, CompiledModel(d["schedule"], d["params"], Config(**cfg), dev)


def test_wrong_shape_is_refused_with_the_reference_message(dev):
    from mlc_compiler_b200.executor import ExecutionError

    d, cm = _model("block__default__float32", dev)
    x = d["inputs"][0].to(dev)
    cm(x)
    with pytest.raises(ExecutionError, match="compiled for"):
        cm(x[:, :4])
    with pytest.raises(ExecutionError, match="expected 1 inputs"):
        cm(x, x)


def test_outputs_alias_static_storage_and_inputs_are_copied(dev):
    d, cm = _model("block__default__float32", dev)
    x = d["inputs"][0].to(dev)
    a = cm(x)
    first = a.clone()
    b = cm(x * 2.0)
    assert a.data_ptr() == b.data_ptr()          # same storage, overwritten by the next call
    assert not torch.equal(first, b)
    x2 = x.clone()
    c = cm(x2).clone()
    x2.zero_()                                   # caller's tensor is not aliased by the model
    torch.cuda.synchronize()
    assert_close(cm(x).clone(), first, "float32", "replay after other inputs")
    assert_close(c, first, "float32", "copy of inputs")


def test_kernels_never_write_outside_their_arena_slices(dev):
    """Canaries between planned buffers: pad the arena, fill the padding with a
    pattern, run, and check that only planned byte ranges changed."""
    from mlc_compiler_b200.executor import CompiledModel

    d = load_tiny("block__default__float32")
    s = d["schedule"]
    pad = 256
    shifted = kir.loads(kir.dumps(s))
    order = sorted(shifted.plan.offsets, key=lambda n: shifted.plan.offsets[n])
    # re-pack with a guard band after every buffer, keeping relative order
    live_end = {}
    for n in order:
        shifted.plan.offsets[n] = s.plan.offsets[n] * 2 + pad
        live_end[n] = shifted.plan.offsets[n] + s.buffers[n].nbytes
    shifted.plan.arena_bytes = s.plan.arena_bytes * 2 + 2 * pad + 4096
    cm = CompiledModel(shifted, d["params"],
                       Config(cuda_graphs=False).as_scheduled(), dev)
    assert cm.executed_schedule.plan.offsets == shifted.plan.offsets
    arena = cm._get_arena()
    arena.fill_(0xA5)
    out = cm(d["inputs"][0].to(dev))
    torch.cuda.synchronize()
    assert_close(out, d["outputs"][0], "float32", "padded arena output")
    covered = torch.zeros(arena.numel(), dtype=torch.bool, device=dev)
    for n in order:
        covered[shifted.plan.offsets[n]:live_end[n]] = True
    assert bool((arena[~covered] == 0xA5).all()), "a kernel wrote outside its buffer"


def test_graph_and_plain_execution_agree_bitwise(dev):
    d, plain = _model("block_b8__default__float32", dev, cuda_graphs=False)
    _, graphed = _model("block_b8__default__float32", dev, cuda_graphs=True)
    x = d["inputs"][0].to(dev)
    a = plain(x).clone()
    graphed(x)
    b = graphed(x).clone()
    assert torch.equal(a, b)


def test_unplanned_schedule_runs_the_eager_path(dev):
    d, cm = _model("block__no_fusion__float32", dev)
    assert cm.schedule.plan.mode == "eager"
    out = cm(d["inputs"][0].to(dev))
    assert_close(out, d["outputs"][0], "float32", "no-fusion output")


def test_profile_kernels_reports_every_kernel(dev):
    d, cm = _model("block__default__float32", dev, cuda_graphs=False)
    rows = cm.profile_kernels([t.to(dev) for t in d["inputs"]], iters=3)
    assert [r[0] for r in rows] == [k.name for k in cm.executed_schedule.kernels]
    assert all(r[2] > 0 for r in rows)


def test_source_is_exposed_per_kernel(dev):
    d, cm = _model("block__default__float32", dev)
    assert 'extern "C" __global__' in cm.source()
    name = cm.schedule.generated()[0].name
    assert "__launch_bounds__" in cm.kernel_source(name)
    assert cm.source_path().exists()
    info = cm._module.kernel_info(name)
    assert 0 < info["registers"] <= 255


def test_backend_selection_has_no_silent_fallback(dev):
    from mlc_compiler_b200.executor import CompiledModel, select_backend
    from mlc_compiler_b200.runtime import BackendError

    d = load_tiny("pointwise__default__float32")
    with pytest.raises(ValueError, match="Triton"):
        select_backend(Config(backend="triton"), dev)
    with pytest.raises(BackendError):
        CompiledModel(d["schedule"], d["params"], Config(), "cpu")


def test_dependent_launch_variant_gives_the_same_answer(dev):
    d, cm = _model("block__default__float32", dev, dependent_launch=True)
    x = d["inputs"][0].to(dev)
    cm(x)
    out = cm(x)
    assert_close(out, d["outputs"][0], "float32", "dependent-launch output")


def test_forked_graph_is_bitwise_equal_to_the_serial_chain(dev):
    """Capturing over several streams changes only the edges of the graph."""
    from mlc_compiler_b200 import models
    from mlc_compiler_b200.executor import CompiledModel
    from mlc_compiler_b200.frontend import load_schedule

    s = load_schedule("bert-base_b1_s128_float16")
    model, inputs = models.build("bert-base", 1, dtype=torch.float16)
    di = [t.to(dev) for t in inputs]
    serial = CompiledModel(s, model, Config(graph_streams=1), dev)
    forked = CompiledModel(s, model, Config(graph_streams=4), dev)
    assert forked._streams is not None and forked._streams.forked >= 40
    a = serial(*di).clone()
    forked(*di)
    for _ in range(3):
        b = forked(*di).clone()
        assert torch.equal(a, b)
    assert [k.name for k in forked.schedule.kernels] == [k.name for k in s.kernels]


def test_forked_graph_stays_equal_to_the_serial_chain_under_changing_inputs(dev):
    """Race check for the parallel branches: 40 replays with fresh inputs, each
    compared bitwise with the single-stream graph (batch 8 also exercises the
    forwarded and the transposing kernels)."""
    from mlc_compiler_b200 import models
    from mlc_compiler_b200.executor import CompiledModel
    from mlc_compiler_b200.frontend import load_schedule

    s = load_schedule("bert-base_b8_s128_float16")
    model, inputs = models.build("bert-base", 8, dtype=torch.float16)
    serial = CompiledModel(s, model, Config().as_scheduled(), dev)
    forked = CompiledModel(s, model, Config(graph_streams=4), dev)
    g = torch.Generator().manual_seed(3)
    for _ in range(40):
        ids = torch.randint(0, 30522, (8, 128), generator=g).to(dev)
        mask = (torch.rand(8, 128, generator=g) > 0.2).to(torch.float16).to(dev)
        a = serial(ids, mask).clone()
        b = forked(ids, mask).clone()
        assert torch.equal(a, b)


def test_host_side_failures_are_codes_and_messages_not_faults(dev):
    """Missing symbol, bad device ordinal, misaligned buffer: each is reported by
    the library as an error code with a message; the context stays usable."""
    from mlc_compiler_b200.runtime import BackendError, CudaRuntime, LoadedModule, compile_source

    image = compile_source('extern "C" __global__ void probe(float* p) { p[threadIdx.x] = 1.0f; }')
    with pytest.raises(BackendError, match="mlcb_module_load"):
        LoadedModule(image, 99)
    mod = LoadedModule(image, 0)
    with pytest.raises(BackendError, match="no_such_kernel"):
        mod.kernel("no_such_kernel")
    d = load_tiny("pointwise__default__float32")
    rt = CudaRuntime(d["schedule"], Config(), dev)
    k = d["schedule"].generated()[0]
    bufs = {}
    for b in set(k.reads()) | set(k.writes()):
        n = d["schedule"].buffers[b].numel
        bufs[b] = torch.zeros(n + 1, device=dev)[1:]          # 4-byte, not 16-byte aligned
    with pytest.raises(BackendError, match="aligned"):
        rt.launch(k, bufs)
    # the device is still fine
    x = torch.ones(32, device=dev)
    assert float(x.sum()) == 32.0


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["bert-base", "gpt2-small"])
def test_matmul_writing_the_clone_layout_changes_nothing_but_the_launch_count(name):
    import torch
    from mlc_compiler_b200 import Config, models
    from mlc_compiler_b200.executor import CompiledModel
    from mlc_compiler_b200.frontend import load_schedule

    dev = torch.device("cuda", 0)
    s = load_schedule(models.schedule_name(name, 1, torch.float16))
    model, inputs = models.build(name, 1, dtype=torch.float16)
    di = [t.to(dev) for t in inputs]
    on = CompiledModel(s, model, Config(), dev)
    off = CompiledModel(s, model, Config(write_through_copies=False), dev)
    assert len(off.executed_schedule) - len(on.executed_schedule) == 12
    for _ in range(3):
        a, b = on(*di).float(), off(*di).float()
    torch.cuda.synchronize()
    # same op on the same operands; only the destination's leading dimension differs,
    # which may change cuBLAS's choice of kernel but not what is computed
    assert (a - b).abs().max().item() <= 1e-2 * max(1.0, b.abs().max().item())


@pytest.mark.gpu
@pytest.mark.parametrize("name,batch", [("bert-base", 1), ("gpt2-small", 1), ("bert-base", 8)])
def test_embeddings_gathered_by_the_layernorm_are_bit_identical(name, batch):
    import torch
    from mlc_compiler_b200 import Config, models
    from mlc_compiler_b200.executor import CompiledModel
    from mlc_compiler_b200.frontend import load_schedule

    dev = torch.device("cuda", 0)
    s = load_schedule(models.schedule_name(name, batch, torch.float16))
    model, inputs = models.build(name, batch, dtype=torch.float16)
    on = CompiledModel(s, model, Config(), dev)
    off = CompiledModel(s, model, Config(fold_embeddings=False), dev)
    assert len(off.executed_schedule) - len(on.executed_schedule) == (4 if name == "bert-base" else 2)
    g = torch.Generator().manual_seed(11)
    for _ in range(3):
        ids = torch.randint(0, 30522, inputs[0].shape, generator=g)
        di = [ids.to(dev)] + [t.to(dev) for t in inputs[1:]]
        assert torch.equal(on(*di), off(*di))


@pytest.mark.gpu
def test_auto_dependent_launch_keeps_the_faster_graph_and_the_same_answer():
    import torch
    from mlc_compiler_b200 import Config, models
    from mlc_compiler_b200.executor import CompiledModel
    from mlc_compiler_b200.frontend import load_schedule

    dev = torch.device("cuda", 0)
    s = load_schedule("bert-base_b1_s128_float16")
    model, inputs = models.build("bert-base", 1, dtype=torch.float16)
    di = [t.to(dev) for t in inputs]
    auto = CompiledModel(s, model, Config(), dev)
    assert auto.cfg.dependent_launch == "auto" and auto.dependent_policy is None
    a = auto(*di).clone()
    assert auto.dependent_policy in ("chain", True)
    assert set(auto.policy_timings_ms) == {"chain", "True"}
    # structural, whatever the clock said: the recorded timings and the recorded choice
    # obey the decision rule (library-edge launches are kept only if >= 0.5 % faster)
    t = auto.policy_timings_ms
    assert all(v > 0 for v in t.values())
    assert (auto.dependent_policy is True) == (t["True"] < 0.995 * t["chain"])
    for policy in ("chain", True, False):
        fixed = CompiledModel(s, model, Config(dependent_launch=policy), dev)
        assert torch.equal(fixed(*di), a)
        assert fixed.dependent_policy is None
    assert torch.equal(auto(*di), a)                 # replays of the kept graph


@pytest.mark.gpu
@pytest.mark.parametrize("name,batch", [("bert-base", 8), ("gpt2-small", 4)])
def test_sequence_first_attention_storage_gives_the_same_answer(name, batch):
    import torch
    from mlc_compiler_b200 import Config, models
    from mlc_compiler_b200.executor import CompiledModel
    from mlc_compiler_b200.frontend import load_schedule

    dev = torch.device("cuda", 0)
    s = load_schedule(models.schedule_name(name, batch, torch.float16))
    model, inputs = models.build(name, batch, dtype=torch.float16)
    di = [t.to(dev) for t in inputs]
    on = CompiledModel(s, model, Config(), dev)
    off = CompiledModel(s, model, Config(sequence_first=False), dev)
    assert len(off.executed_schedule) - len(on.executed_schedule) == (12 if name == "bert-base" else 36)
    for _ in range(3):
        a, b = on(*di).float(), off(*di).float()
    torch.cuda.synchronize()
    # same library calls on the same values; rows reach the output projection in
    # another order, which may change cuBLAS's tiling but not what is computed
    assert (a - b).abs().max().item() <= 1e-2 * max(1.0, b.abs().max().item())


@pytest.mark.gpu
@pytest.mark.parametrize("name,batch", [("bert-base", 1), ("bert-base", 8), ("gpt2-small", 4)])
def test_emitter_and_rewrite_options_change_timing_only(name, batch):
    """Where parameters are loaded relative to the grid-dependency wait, where an
    output row is stored, and whether sibling bias adds share a launch are all
    arrangements of the same arithmetic: outputs are bit-identical."""
    import torch
    from mlc_compiler_b200 import Config, models
    from mlc_compiler_b200.executor import CompiledModel
    from mlc_compiler_b200.frontend import load_schedule

    dev = torch.device("cuda", 0)
    s = load_schedule(models.schedule_name(name, batch, torch.float16))
    model, inputs = models.build(name, batch, dtype=torch.float16)
    di = [t.to(dev) for t in inputs]
    base = CompiledModel(s, model, Config(), dev)
    base(*di)
    want = base(*di).clone()
    for kw in ({"hoist_stable_loads": False}, {"hoist_stable_loads": "all"}, {"fuse_siblings": True},
               {"trigger_early": True}, {"reduction_min_ctas": 2}):
        other = CompiledModel(s, model, Config(**kw), dev)
        other(*di)
        assert torch.equal(other(*di), want), kw
    fused = CompiledModel(s, model, Config(fuse_siblings=True), dev)
    if name == "bert-base":
        assert len(fused.executed_schedule) == len(base.executed_schedule) - 24
