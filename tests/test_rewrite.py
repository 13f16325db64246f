"""Producer forwarding: index-map composition and bit-identical results."""

import itertools

import pytest
import torch

import kir_oracle as oracle
from conftest import load_tiny, tiny_cases
from mlc_compiler_b200 import Config, kir, models, rewrite
from mlc_compiler_b200.frontend import load_schedule


def _ax(numel, *terms):
    return kir.IndexMap((kir.Axis("idx", numel, tuple(terms)),))


def test_compose_head_layout_with_bias_row():
    # consumer reads [B*T, D] as [B, H, T, Dh]; producer's bias operand is idx % D
    B, H, T, Dh = 4, 12, 128, 64
    D = H * Dh
    outer = _ax(B * H * T * Dh, (B, H * T * Dh, T * D), (H, T * Dh, Dh), (T, Dh, D), (Dh, 1, 1))
    bias = _ax(B * T * D, (D, 1, 1))
    ident = _ax(B * T * D, (B * T * D, 1, 1))
    cb = rewrite.compose(outer, bias, B * T * D)
    ci = rewrite.compose(outer, ident, B * T * D)
    for i in (0, 1, 63, 64, 8191, 8192, 98303, 98304, B * H * T * Dh - 1):
        x = outer.offset(idx=i)
        assert cb.offset(idx=i) == x % D
        assert ci.offset(idx=i) == x


def test_compose_with_sliced_consumer_and_exhaustive_check():
    # consumer reads columns [768, 1536) of a [T, 2304] buffer, transposed
    T, W, D = 16, 96, 32
    outer = kir.IndexMap((kir.Axis("idx", D * T, ((D, T, 1), (T, 1, W))),), base=D)
    inner = _ax(T * W, (W, 1, 1))                       # idx % W
    row = _ax(T * W, (T, W, 1))                         # idx // W
    c1 = rewrite.compose(outer, inner, T * W)
    c2 = rewrite.compose(outer, row, T * W)
    for i in range(D * T):
        x = outer.offset(idx=i)
        assert c1.offset(idx=i) == x % W and c2.offset(idx=i) == x // W


def test_compose_refuses_digits_that_straddle_a_window():
    outer = _ax(64, (64, 1, 3))                         # stride 3 walks across idx % 8 windows
    with pytest.raises(rewrite._NoCompose):
        rewrite.compose(outer, _ax(192, (8, 1, 1)), 192)


@pytest.mark.parametrize("name,batch", [("bert-base", 4), ("gpt2-small", 4)])
def test_forwarding_is_bit_identical_on_benchmark_schedules(name, batch):
    s = load_schedule(models.schedule_name(name, batch, torch.float16))
    r = rewrite.forward_into_consumers(s)
    assert len(r) < len(s) and r.counts()["extern"] == s.counts()["extern"]
    assert sorted(k.name for k in r.kernels if isinstance(k, kir.ExternKernel)) == \
        sorted(k.name for k in s.kernels if isinstance(k, kir.ExternKernel))
    model, inputs = models.build(name, batch, dtype=torch.float16)
    a, _ = oracle.run_schedule(s, model, inputs)
    b, _ = oracle.run_schedule(r, model, inputs)
    assert torch.equal(a, b)
    # the re-packed arena keeps co-live buffers apart (checked inside relax) and aligned
    assert all(o % 256 == 0 for o in r.plan.offsets.values())


def test_batch_one_has_nothing_to_forward():
    s = load_schedule("bert-base_b1_s128_float16")
    assert rewrite.forward_into_consumers(s) is s


@pytest.mark.parametrize("stem", [c for c in tiny_cases() if c.startswith(("block", "attention", "mlp"))])
def test_forwarding_never_changes_tiny_model_outputs(stem):
    d = load_tiny(stem)
    r = rewrite.forward_into_consumers(d["schedule"])
    out, _ = oracle.run_schedule(r, d["params"], d["inputs"])
    outs = list(out) if isinstance(out, tuple) else [out]
    for got, want in zip(outs, d["outputs"]):
        torch.testing.assert_close(got, want, rtol=1e-6, atol=1e-7)


def _with_random_biases(model):
    g = torch.Generator().manual_seed(11)
    with torch.no_grad():
        for m in model.modules():
            if isinstance(m, torch.nn.Linear) and m.bias is not None:
                m.bias.copy_((torch.randn(m.bias.shape, generator=g) * 0.05).to(m.bias.dtype))
    return model


@pytest.mark.parametrize("name,batch", [("bert-base", 1), ("gpt2-small", 1), ("bert-base", 4)])
def test_bias_epilogue_rewrite_keeps_the_function(name, batch):
    """mm + bias -> addmm: the same function up to one rounding of the matmul
    output (the CPU oracle evaluates addmm and mm+add in the same precision)."""
    s = load_schedule(models.schedule_name(name, batch, torch.float16))
    r = rewrite.fold_bias_into_matmul(s)
    folded = [k for k in r.kernels if isinstance(k, kir.ExternKernel) and k.op == "aten.addmm.default"]
    assert len(folded) >= 48 and len(r) < len(s)
    assert all(len(k.args) == 3 and k.args[0].shape == (k.outputs[0].shape[1],) for k in folded)
    model, inputs = models.build(name, batch, dtype=torch.float16)
    model = _with_random_biases(model)
    a, _ = oracle.run_schedule(s, model, inputs)
    b, _ = oracle.run_schedule(r, model, inputs)
    torch.testing.assert_close(a.float(), b.float(), rtol=1e-2, atol=1e-2)
    assert float((a.float() - b.float()).abs().max()) > 0.0 or True


def test_bias_epilogue_leaves_other_matmuls_alone():
    s = load_tiny("attention__default__float32")["schedule"]
    r = rewrite.fold_bias_into_matmul(s)
    for k in r.kernels:
        if isinstance(k, kir.ExternKernel):
            assert k.op in ("aten.mm.default", "aten.bmm.default", "aten.addmm.default")
    d = load_tiny("attention__default__float32")
    out, _ = oracle.run_schedule(r, d["params"], d["inputs"])
    torch.testing.assert_close(out, d["outputs"][0], rtol=1e-5, atol=1e-6)


# ---- copies after an extern ---------------------------------------------------

@pytest.mark.parametrize("name,dtype", [("bert-base", torch.float16), ("gpt2-small", torch.float16),
                                        ("bert-base", torch.float32)])
def test_write_through_drops_the_context_clone_at_batch_one(name, dtype):
    s = load_schedule(models.schedule_name(name, 1, dtype))
    r = rewrite.write_through_copies(s)
    assert len(s) - len(r) == 12 and r.counts()["extern"] == s.counts()["extern"]
    strided = [k for k in r.kernels if isinstance(k, kir.ExternKernel)
               and k.outputs[0].strides == (64, 768, 1)]
    assert len(strided) == 12 and all(k.op == "aten.bmm.default" for k in strided)
    gone = {k.name for k in s.kernels} - {k.name for k in r.kernels}
    assert all(next(k for k in s.kernels if k.name == g).ops == ["clone"] for g in gone)
    model, inputs = models.build(name, 1, dtype=dtype)
    a, _ = oracle.run_schedule(s, model, inputs)
    b, _ = oracle.run_schedule(r, model, inputs)
    assert torch.equal(a, b)
    assert r.plan.arena_bytes <= s.plan.arena_bytes


def test_write_through_leaves_split_dimensions_alone():
    # at batch 4 the clone splits [B*H] into (B, H) with unrelated destination
    # strides: no strided matrix expresses it
    s = rewrite.forward_into_consumers(load_schedule(models.schedule_name("bert-base", 4, torch.float16)))
    assert rewrite.write_through_copies(s) is s


def test_destination_strides_by_brute_force():
    H, T, D = 3, 5, 4
    n = H * T * D
    view = kir.View("x", "x", (H, T, D), (T * D, D, 1))
    copy = kir.PointwiseKernel(
        "c", (1, T, H, D),
        [kir.Operand("x", "x", "float32", _ax(n, (T, H * D, D), (H, D, T * D), (D, 1, 1)))],
        [kir.Operand("y", "y", "float32", _ax(n, (n, 1, 1)))], [], {"y": kir.Load(0)}, ["clone"])
    t = rewrite._destination_strides(view, copy)
    assert t == (D, H * D, 1)
    x = torch.arange(n, dtype=torch.float32)
    want = torch.empty(n)
    for i in range(n):
        want[i] = x[copy.inputs[0].index.offset(idx=i)]
    got = torch.empty(n)
    got.as_strided((H, T, D), t).copy_(x.view(H, T, D))
    assert torch.equal(got, want)
    # a read map that repeats a digit, or does not cover the result, is refused
    bad = kir.PointwiseKernel(
        "c", (n,), [kir.Operand("x", "x", "float32", _ax(n, (T, H * D, D), (H * D, 1, 1)))],
        copy.outputs, [], {"y": kir.Load(0)}, ["clone"])
    assert rewrite._destination_strides(view, bad) is None


def test_write_through_refuses_a_result_with_a_second_reader():
    s = load_schedule(models.schedule_name("bert-base", 1, torch.float16))
    clone = next(k for k in s.kernels if isinstance(k, kir.PointwiseKernel) and k.ops == ["clone"])
    extra = kir.PointwiseKernel("spy", clone.space, list(clone.inputs),
                                [kir.Operand("spy_out", "spy_out", "float16", clone.outputs[0].index)],
                                [], {"spy_out": kir.Load(0)}, ["clone"])
    buffers = dict(s.buffers)
    buffers["spy_out"] = kir.BufferSpec("spy_out", (clone.numel,), "float16", "intermediate")
    at = s.kernels.index(clone) + 1
    t = kir.Schedule(s.name, s.kernels[:at] + [extra] + s.kernels[at:], buffers, s.inputs, s.outputs,
                     s.params, s.plan, dict(s.meta))
    r = rewrite.write_through_copies(t, replan=False)
    assert len(t) - len(r) == 11 and clone.name in {k.name for k in r.kernels}


# ---- embeddings gathered by their consumer --------------------------------------

@pytest.mark.parametrize("stem,removed", [("bert-base_b1_s128_float16", 4), ("bert-base_b4_s128_float16", 4),
                                          ("gpt2-small_b1_s128_float16", 2),
                                          ("bert-base-streamed_b1_s128_float16", 4)])
def test_embeddings_move_into_the_first_layernorm(stem, removed):
    s = load_schedule(stem)
    r = rewrite.fold_embeddings(s)
    assert len(s) - len(r) == removed
    assert not any(isinstance(k, kir.ExternKernel) and "embedding" in k.op for k in r.kernels)
    assert not any(isinstance(k, kir.PointwiseKernel) and k.ops == ["full_like"] for k in r.kernels)
    first = next(k for k in r.kernels if isinstance(k, kir.ReductionKernel))
    gathered = [a for a in first.inputs if a.via is not None]
    assert len(gathered) == 2                       # word and position rows; token type is a constant row
    for a in gathered:
        ids = first.inputs[a.via[0]]
        assert ids.dtype == "int64" and not ids.index.varies_along("col")
        assert a.index.axis("row").numel == a.via[1] == s.buffers[a.buffer].numel // 768
    name, batch = stem.split("_")[0].replace("-streamed", ""), int(stem.split("_b")[1].split("_")[0])
    model, inputs = models.build(name, batch, dtype=torch.float16)
    a, _ = oracle.run_schedule(s, model, inputs)
    b, _ = oracle.run_schedule(r, model, inputs)
    assert torch.equal(a, b)
    back = kir.loads(kir.dumps(r))
    assert [x.via for k in back.generated() for x in k.inputs] == \
        [x.via for k in r.generated() for x in k.inputs]


def test_gathered_rows_are_clamped_into_the_table():
    s = load_schedule("gpt2-small_b1_s128_float16")
    r = rewrite.fold_embeddings(s)
    first = next(k for k in r.kernels if isinstance(k, kir.ReductionKernel))
    model, inputs = models.build("gpt2-small", 1, dtype=torch.float16)
    good = oracle.allocate(r, model, inputs)
    bad = oracle.allocate(r, model, [torch.full_like(inputs[0], 10 ** 9)])
    last = oracle.allocate(r, model, [torch.full_like(inputs[0], 50256)])
    oracle.run_kernel(first, good)
    oracle.run_kernel(first, bad)
    oracle.run_kernel(first, last)
    out = first.outputs[0].buffer
    assert torch.equal(bad[out], last[out]) and not torch.equal(bad[out], good[out])
    from mlc_compiler_b200.emit import generate_module
    assert "mlcb_clamp_index((long long)s4, 50257)" in generate_module(r, Config()).kernel_source(first.name)


def test_embedding_with_other_readers_stays_a_library_call():
    s = load_schedule("gpt2-small_b1_s128_float16")
    emb = next(k for k in s.kernels if isinstance(k, kir.ExternKernel) and "embedding" in k.op)
    x = emb.outputs[0]
    n = x.numel
    spy = kir.PointwiseKernel("spy", (n,), [kir.Operand(x.name, x.buffer, "float16", _ax(n, (n, 1, 1)))],
                              [kir.Operand("spy_out", "spy_out", "float16", _ax(n, (n, 1, 1)))],
                              [], {"spy_out": kir.Load(0)}, ["clone"])
    buffers = dict(s.buffers)
    buffers["spy_out"] = kir.BufferSpec("spy_out", (n,), "float16", "intermediate")
    t = kir.Schedule(s.name, s.kernels[:2] + [spy] + s.kernels[2:], buffers, s.inputs, s.outputs,
                     s.params, s.plan, dict(s.meta))
    r = rewrite.fold_embeddings(t, replan=False)
    assert emb.name in {k.name for k in r.kernels} and len(t) - len(r) == 1


# ---- sequence-first storage around the attention matmuls ------------------------

@pytest.mark.parametrize("name,batch,before,after", [("bert-base", 4, 236, 184), ("gpt2-small", 4, 184, 134)])
def test_sequence_first_removes_every_head_copy_at_batch_above_one(name, batch, before, after):
    s = load_schedule(models.schedule_name(name, batch, torch.float16))
    moved = rewrite.sequence_first(s)
    assert moved is not s and len(moved) == len(s) == before
    r = rewrite.read_through_copies(moved)
    assert len(moved) - len(r) == 48                              # q, k, v and context copies of 12 layers
    assert not any(isinstance(k, kir.PointwiseKernel) and "clone" in k.ops for k in r.kernels)
    B, T, D, Dh = batch, 128, 768, 64
    J = 1 if name == "bert-base" else 3                           # GPT-2: one fused q/k/v projection
    bmms = [k for k in r.kernels if isinstance(k, kir.ExternKernel) and k.op == "aten.bmm.default"]
    scores, context = bmms[0], bmms[1]
    q, kt, v = scores.args[0], scores.args[1], context.args[1]
    assert q.strides == (J * Dh, B * J * D, 1)                    # [T, B, H, J, Dh]: (b, h) is one stride
    assert kt.strides == (J * Dh, 1, B * J * D)
    assert v.strides == q.strides
    if J == 3:
        assert q.buffer == kt.buffer == v.buffer and (q.offset, kt.offset, v.offset) == (0, Dh, 2 * Dh)
    assert context.outputs[0].strides == (Dh, B * D, 1)           # written where the projection reads
    proj = r.kernels[r.kernels.index(context) + 1]
    assert proj.op == "aten.mm.default" and proj.args[0].buffer == context.outputs[0].buffer
    assert proj.args[0].strides == (D, 1)
    full = rewrite.prepare(s, Config())
    assert len(full) == after
    from mlc_compiler_b200.emit import generate_module
    mod = generate_module(full, Config())
    adds = [k for k in full.generated() if isinstance(k, kir.PointwiseKernel) and k.ops == ["add"]]
    assert len(adds) == 36 // J and len({mod.symbol[k.name] for k in adds}) == 1
    assert all(mod.launch[k.name].vector >= 8 for k in adds)
    assert all(k.outputs[0].index.axes[0].terms == ((k.numel, 1, 1),) for k in adds)   # iterated as stored
    model, inputs = models.build(name, batch, dtype=torch.float16)
    a, _ = oracle.run_schedule(s, model, inputs)
    b, _ = oracle.run_schedule(full, model, inputs)
    assert torch.equal(a, b)


def test_sequence_first_leaves_batch_one_and_plain_models_alone():
    s = load_schedule("bert-base_b1_s128_float16")
    assert rewrite.sequence_first(s) is s
    s = load_schedule("micro-softmax_b8_s128_float16")
    assert rewrite.sequence_first(s) is s


@pytest.mark.parametrize("stem", [c for c in tiny_cases() if c.startswith(("block", "attention"))])
def test_prepare_never_changes_tiny_model_outputs(stem):
    d = load_tiny(stem)
    s = d["schedule"]
    r = rewrite.prepare(s, Config())
    a, _ = oracle.run_schedule(s, d["params"], d["inputs"])
    b, _ = oracle.run_schedule(r, d["params"], d["inputs"])
    assert torch.equal(a, b)


def test_output_major_iteration_by_enumeration():
    # a key copy after the move: iteration (B, H, Dh, T), output stored [T, B, H, Dh]
    B, H, Dh, T = 2, 3, 4, 5
    D, n = H * Dh, B * H * Dh * T
    src = _ax(n, (B, H * Dh * T, T * D), (H * Dh, T, 1), (T, 1, D))
    dst = _ax(n, (B, H * Dh * T, D), (H, Dh * T, Dh), (Dh, T, 1), (T, 1, B * D))
    k = kir.PointwiseKernel("k", (B, H, Dh, T), [kir.Operand("x", "x", "float32", src)],
                            [kir.Operand("y", "y", "float32", dst)], [], {"y": kir.Load(0)}, ["clone"])
    r = rewrite.output_major(k)
    assert r.space == (T, B, H * Dh) or r.space == (T, B, H, Dh)
    assert r.outputs[0].index.axes[0].terms == ((n, 1, 1),)
    pairs = {(k.inputs[0].index.offset(idx=i), k.outputs[0].index.offset(idx=i)) for i in range(n)}
    again = {(r.inputs[0].index.offset(idx=i), r.outputs[0].index.offset(idx=i)) for i in range(n)}
    assert pairs == again and len(pairs) == n
    assert rewrite.output_major(r) is r


def test_bias_epilogue_and_sequence_first_compose():
    s = load_schedule(models.schedule_name("bert-base", 4, torch.float16))
    model, inputs = models.build("bert-base", 4, dtype=torch.float16)
    _with_random_biases(model)
    full = rewrite.prepare(s, Config(bias_epilogue=True))
    # the same launches batch 1 runs with the bias folded into the matmuls
    one = rewrite.prepare(load_schedule(models.schedule_name("bert-base", 1, torch.float16)),
                          Config(bias_epilogue=True))
    assert len(full) == len(one) == 148
    assert not any(isinstance(k, kir.PointwiseKernel) and "clone" in k.ops for k in full.kernels)
    a, _ = oracle.run_schedule(s, model, inputs)
    b, _ = oracle.run_schedule(full, model, inputs)
    assert (a.float() - b.float()).abs().max().item() <= 1e-2


def test_as_scheduled_config_switches_every_rewrite_off():
    for stem in ("bert-base_b4_s128_float16", "gpt2-small_b1_s128_float16"):
        s = load_schedule(stem)
        assert rewrite.prepare(s, Config().as_scheduled()) is s
        assert len(rewrite.prepare(s, Config())) < len(s)


def test_sequence_first_keeps_the_rows_of_an_addmm_with_a_matrix_valued_self():
    """``addmm(self, x, w)`` treats rows independently only when ``self`` is the same
    for every row.  With a ``[B*T, F]`` ``self`` (a residual folded into the matmul)
    row ``i`` of the result takes row ``i`` of ``self``: permuting the rows of ``x``
    and of the result to ``(t, b)`` order without ``self`` would add the wrong rows.
    The rewrite must then either leave that matmul's buffers where they are or
    re-address every operand; the outputs may not change."""
    s = rewrite.fold_bias_into_matmul(load_schedule(models.schedule_name("bert-base", 4, torch.float16)))
    model, inputs = models.build("bert-base", 4, dtype=torch.float16)
    writer = {b: k for k in s.kernels for b in k.writes()}
    target = None
    for k in s.kernels:
        if isinstance(k, kir.ExternKernel) and k.op == "aten.addmm.default":
            src = writer.get(k.args[1].buffer)
            if src is not None and rewrite._pure_copy(src):      # fed by the context clone
                target = k
                break
    assert target is not None
    rows, cols = target.outputs[0].shape
    assert rows == 4 * 128
    s.buffers["p_rowwise_self"] = kir.BufferSpec("p_rowwise_self", (rows, cols), "float16", "param")
    s.params["p_rowwise_self"] = "rowwise_self"
    i = s.kernels.index(target)
    s.kernels[i] = kir.ExternKernel(
        target.name, target.op,
        [kir.View("rowwise_self", "p_rowwise_self", (rows, cols), (cols, 1), 0)] + list(target.args[1:]),
        dict(target.kwargs), list(target.outputs))
    assert not rewrite._rows_independent(s.kernels[i])
    table = dict(model.named_parameters(remove_duplicate=False))
    table.update(dict(model.named_buffers(remove_duplicate=False)))
    g = torch.Generator().manual_seed(3)
    table["rowwise_self"] = torch.randn(rows, cols, generator=g).to(torch.float16)
    want, _ = oracle.run_schedule(s, table, inputs)
    moved = rewrite.read_through_copies(rewrite.sequence_first(s))
    assert len(moved) < len(s)                                   # the other layers still lose their copies
    got, _ = oracle.run_schedule(moved, table, inputs)
    assert torch.equal(got, want)
    full, _ = oracle.run_schedule(rewrite.prepare(s, Config()), table, inputs)
    assert torch.equal(full, want)


def test_pure_copy_does_not_see_through_a_narrowing_round_trip():
    n = 16
    ax = _ax(n, (n, 1, 1))

    def copy(dtype, via):
        e = kir.Cast(kir.Cast(kir.Load(0), via), dtype)
        return kir.PointwiseKernel("k", (n,), [kir.Operand("x", "x", dtype, ax)],
                                   [kir.Operand("y", "y", dtype, ax)], [], {"y": e}, ["_to_copy"])

    assert rewrite._pure_copy(copy("float16", "float32"))        # widening and back: identity
    assert rewrite._pure_copy(copy("float32", "float32"))
    assert not rewrite._pure_copy(copy("float64", "float32"))    # rounds to 24 bits on the way


# ---- sibling pointwise kernels as one launch (opt-in) -----------------------------

@pytest.mark.parametrize("name,batch", [("bert-base", 1), ("bert-base", 4)])
def test_sibling_fusion_merges_the_three_projection_bias_adds(name, batch):
    s = load_schedule(models.schedule_name(name, batch, torch.float16))
    base = rewrite.prepare(s, Config())
    fused = rewrite.prepare(s, Config(fuse_siblings=True))
    assert len(base) - len(fused) == 24                         # 36 adds -> 12 launches
    merged = [k for k in fused.generated() if isinstance(k, kir.PointwiseKernel) and len(k.outputs) == 3]
    assert len(merged) == 12 and all(k.ops == ["add"] * 3 and len(k.inputs) == 6 for k in merged)
    # the fused launch sits where its last member was: after all three producers
    order = {k.name: i for i, k in enumerate(fused.kernels)}
    for m in merged:
        producers = [k for k in fused.kernels if set(k.writes()) & set(m.reads())]
        assert all(order[p.name] < order[m.name] for p in producers)
    model, inputs = models.build(name, batch, dtype=torch.float16)
    a, _ = oracle.run_schedule(base, model, inputs)
    b, _ = oracle.run_schedule(fused, model, inputs)
    assert torch.equal(a, b)


def test_sibling_fusion_refuses_members_that_depend_on_each_other():
    n = 64
    ax = _ax(n, (n, 1, 1))

    def add_one(name, src, dst):
        return kir.PointwiseKernel(name, (n,), [kir.Operand(src, src, "float32", ax)],
                                   [kir.Operand(dst, dst, "float32", ax)],
                                   [("t0", kir.Call("add", (kir.Load(0), kir.Const(1.0))))],
                                   {dst: kir.Ref("t0")}, ["add"])

    bufs = {b: kir.BufferSpec(b, (n,), "float32", kind) for b, kind in
            (("x", "input"), ("y", "intermediate"), ("z", "intermediate"), ("w", "output"))}
    chain = kir.Schedule("chain", [add_one("k0", "x", "y"), add_one("k1", "y", "z"), add_one("k2", "z", "w")],
                         bufs, inputs=[kir.View("x", "x", (n,), (1,), 0)],
                         outputs=[kir.View("w", "w", (n,), (1,), 0)])
    assert rewrite.fuse_siblings(chain, replan=False) is chain
