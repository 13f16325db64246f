"""The CUDA emitter, checked without a GPU: every generated module must compile
for sm_100a, cover every kernel, take one pointer per operand, be deterministic,
and use packed accesses where the index maps allow them."""

import re
import shutil

import pytest

from conftest import load_tiny, tiny_cases
from mlc_compiler_b200 import Config, kir
from mlc_compiler_b200 import build as B
from mlc_compiler_b200.emit import generate_module
from mlc_compiler_b200.emit.indexing import classify
from mlc_compiler_b200.frontend import load_schedule

needs_nvcc = pytest.mark.skipif(shutil.which("nvcc") is None and B.nvcc_path() is None,
                                reason="nvcc not installed")

COMPILE_CASES = [s for s in tiny_cases()
                 if s.endswith(("__default__float32", "__streamed__float32", "__default__float16",
                                "__streamed__bfloat16", "__no_fusion__float32"))
                 and not s.startswith("block_b8")] + [s for s in tiny_cases() if s.startswith("fn")]


def _signature(src: str, symbol: str) -> list[str]:
    m = re.search(rf"{symbol}\((.*?)\) \{{", src, re.S)
    return [p for p in m.group(1).split(",") if p.strip()]


@pytest.mark.parametrize("stem", tiny_cases())
def test_launch_table_covers_every_generated_kernel(stem):
    s = load_tiny(stem)["schedule"]
    mod = generate_module(s, Config())
    gen = [k.name for k in s.generated()]
    assert sorted(mod.launch) == sorted(gen)
    for k in s.generated():
        sym = mod.symbol[k.name]
        assert f'extern "C" __global__' in mod.kernel_source(k.name)
        assert len(_signature(mod.source, sym)) == len(k.inputs) + len(k.outputs)
        spec = mod.launch[k.name]
        assert spec.grid >= 1 and 32 <= spec.block <= 1024


def test_generation_is_deterministic():
    s = load_schedule("bert-base_b1_s128_float16")
    assert generate_module(s, Config()).source == generate_module(s, Config()).source


def test_identical_layers_share_one_function():
    s = load_schedule("bert-base_b1_s128_float16")
    mod = generate_module(s, Config())
    assert len(mod.launch) == 100
    assert len(set(mod.symbol.values())) <= 12


def test_multiply_by_one_never_reaches_the_source():
    s = load_schedule("bert-base_b1_s128_float16")
    src = generate_module(s, Config()).source
    assert "* (0x1.0000000000000p+0f)" not in src


def test_bias_add_is_fully_packed():
    """[128,768] + bias[768] in fp16: one 128-bit load per operand, no tail guard."""
    s = load_schedule("bert-base_b1_s128_float16")
    k = s.kernel("k7")
    text = generate_module(s, Config()).kernel_source("k7")
    # the matmul result is read after the wait, the bias (a parameter) ahead of it
    assert text.count("mlcb_load<__half, 8>") == 1 and text.count("mlcb_load_raw<__half, 8>") == 1
    assert "mlcb_store<__half, 8>" in text
    assert "if (pack >=" not in text
    assert classify(k.inputs[1].index, "idx", 8).width == 8
    plain = generate_module(s, Config(hoist_stable_loads=False)).kernel_source("k7")
    assert plain.count("mlcb_load<__half, 8>") == 2 and "mlcb_load_raw" not in plain


def _before_and_after_the_wait(text: str) -> tuple[str, str]:
    head, _, tail = text.partition("MLCB_GRID_WAIT();")
    assert tail, "kernel has no grid-dependency wait"
    return head, tail


def test_only_parameters_nothing_writes_are_read_ahead_of_the_wait():
    """Under programmatic dependent launch a kernel may run ahead of its
    predecessor up to the wait: weights, biases and masks are loaded there, every
    operand a kernel of the schedule may have produced after it, and no store ever
    precedes it."""
    from mlc_compiler_b200.emit.module import stable_buffers

    for stem, cfg in (("bert-base_b1_s128_float16", Config()),
                      ("gpt2-small_b8_s128_bfloat16", Config()),
                      ("micro-layernorm_b32_s128_float16", Config()),
                      ("micro-softmax_b8_s128_float16", Config()),
                      ("micro-softmax_b32_s128_float16", Config(hoist_stable_loads="all")),
                      ("micro-gelu_b32_s128_float16", Config(hoist_stable_loads="all")),
                      ("bert-base-streamed_b1_s128_float16", Config())):
        s = load_schedule(stem)
        stable = stable_buffers(s)
        assert stable <= set(s.params)
        mod = generate_module(s, cfg)
        hoisted = 0
        for k in s.generated():
            head, tail = _before_and_after_the_wait(mod.kernel_source(k.name))
            assert "mlcb_store" not in head
            for i, a in enumerate(k.inputs):
                early = f"in{i} +" in head
                hoisted += early
                if early:
                    assert a.buffer in stable, (stem, k.name, a.name)
                if a.buffer not in stable:
                    assert f"in{i} +" not in head and f"in{i} +" in tail
        assert hoisted >= 1, stem


def test_launches_of_several_waves_keep_their_loads_behind_the_wait():
    """CTAs of a later wave start after the predecessor has finished: nothing to
    overlap, and words held across the wait would only cost registers."""
    for stem in ("micro-gelu_b32_s128_float16", "micro-softmax_b32_s128_float16"):
        s = load_schedule(stem)
        text = generate_module(s, Config()).kernel_source(s.generated()[0].name)
        head, _ = _before_and_after_the_wait(text)
        assert "mlcb_load" not in head
        assert "mlcb_load_raw" in generate_module(s, Config(hoist_stable_loads="all")).source


def test_hoisting_never_costs_a_row_reduction_its_single_wave():
    """bias + residual + LayerNorm over [4096, 768]: gain and bias (wanted after the
    reductions) cross the wait, the projection bias (needed with the row itself) does
    not, because with it the 1024-CTA launch would no longer fit in one wave."""
    from mlc_compiler_b200 import rewrite

    s = rewrite.prepare(load_schedule("bert-base_b32_s128_float16"), Config())
    k = next(k for k in s.generated() if isinstance(k, kir.ReductionKernel) and len(k.inputs) == 5)
    text = generate_module(s, Config()).kernel_source(k.name)
    head, tail = _before_and_after_the_wait(text)
    assert head.count("mlcb_load_raw<__half, 8>") == 2 and "__launch_bounds__(128, 7)" in text
    one = rewrite.prepare(load_schedule("bert-base_b1_s128_float16"), Config())
    k1 = next(k for k in one.generated() if isinstance(k, kir.ReductionKernel) and len(k.inputs) == 5)
    head1, _ = _before_and_after_the_wait(generate_module(one, Config()).kernel_source(k1.name))
    assert head1.count("mlcb_load_raw<__half, 8>") == 3          # a fraction of a wave: all three


def test_layernorm_weights_cross_the_wait_as_packed_words():
    s = load_schedule("micro-layernorm_b32_s128_float16")
    text = generate_module(s, Config()).source
    head, tail = _before_and_after_the_wait(text[text.index("extern \"C\" __global__"):])
    assert head.count("mlcb_load_raw<__half, 8>") == 2          # gain and bias
    assert tail.count("mlcb_unpack<__half, 8>") == 2
    assert "mlcb_load<__half, 8>(in0" in tail                    # the activations wait


def test_head_merge_copy_keeps_wide_accesses():
    s = load_schedule("bert-base_b1_s128_float16")
    text = generate_module(s, Config()).kernel_source("k15")
    assert "mlcb_load<__half, 8>" in text and "mlcb_load1" not in text


def test_broadcast_and_gather_classification():
    bias = kir.IndexMap((kir.Axis("idx", 98304, ((768, 1, 1),)),))
    assert classify(bias, "idx", 8).mode == "contig"
    per_row = kir.IndexMap((kir.Axis("idx", 98304, ((128, 768, 1),)),))
    a = classify(per_row, "idx", 8)
    assert (a.mode, a.width) == ("bcast", 8)
    transposed = kir.IndexMap((kir.Axis("idx", 8192, ((64, 128, 1), (128, 1, 64))),))
    assert classify(transposed, "idx", 8).width == 1
    odd_base = kir.IndexMap((kir.Axis("idx", 64, ((64, 1, 1),)),), base=4)
    assert classify(odd_base, "idx", 8).width == 4


def test_reductions_accumulate_in_fp32_and_store_narrow():
    s = load_schedule("micro-layernorm_b1_s128_float16")
    text = generate_module(s, Config()).source
    assert "float acc_" in text
    assert "mlcb_store<__half, 8>" in text
    assert "mlcb_load<__half, 8>" in text


def test_out_of_range_index_map_is_refused_at_emit_time():
    s = load_tiny("pointwise__default__float32")["schedule"]
    k = s.generated()[0]
    bad = kir.IndexMap(k.inputs[0].index.axes, base=1)
    k.inputs[0] = kir.Operand(k.inputs[0].name, k.inputs[0].buffer, k.inputs[0].dtype, bad)
    with pytest.raises(ValueError, match="outside a buffer"):
        generate_module(s, Config())


def test_unknown_function_raises_key_error():
    s = load_tiny("pointwise__default__float32")["schedule"]
    k = s.generated()[0]
    k.body.append(("tz", kir.Call("bessel", (kir.Load(0),))))
    with pytest.raises(KeyError):
        generate_module(s, Config())


@needs_nvcc
@pytest.mark.parametrize("stem", COMPILE_CASES)
def test_tiny_modules_compile_for_sm_100a(stem, tmp_path):
    s = load_tiny(stem)["schedule"]
    if not s.generated():
        pytest.skip("no generated kernels")
    src = generate_module(s, Config()).source
    log = B.nvcc_cubin(src, tmp_path / "m.cubin", verbose=True)
    assert "error" not in log.lower()
    assert " bytes spill stores" in log and not re.search(r"[1-9]\d* bytes spill stores", log)


@needs_nvcc
@pytest.mark.parametrize("name", ["bert-base_b1_s128_float16", "gpt2-small_b8_s128_bfloat16",
                                  "micro-gelu_b32_s128_float16", "micro-softmax_b8_s128_float16",
                                  "micro-layernorm_b32_s128_float16",
                                  "bert-base_b32_s128_float16", "gpt2-small_b32_s128_bfloat16",
                                  "bert-base-streamed_b1_s128_float16",
                                  "gpt2-small-streamed_b1_s128_float16"])
def test_benchmark_modules_compile_for_sm_100a(name, tmp_path):
    """As the executor compiles them (rewrites applied); no kernel may spill, the
    ones asked to stay resident for a single wave included."""
    from mlc_compiler_b200 import rewrite

    src = generate_module(rewrite.prepare(load_schedule(name), Config()), Config()).source
    log = B.nvcc_cubin(src, tmp_path / "m.cubin", verbose=True)
    assert not re.search(r"[1-9]\d* bytes spill stores", log)


def test_outputs_are_stored_in_the_first_phase_that_has_their_value():
    """GPT-2's LayerNorm kernels also emit the residual sum they normalise; it is
    stored before the first reduction finishes instead of being carried to the end."""
    from mlc_compiler_b200 import rewrite

    s = rewrite.prepare(load_schedule("gpt2-small_b1_s128_float16"), Config())
    k = next(k for k in s.generated() if isinstance(k, kir.ReductionKernel) and len(k.outputs) == 2)
    text = generate_module(s, Config()).kernel_source(k.name)
    first_reduce = text.index("mlcb_cta_reduce") if "mlcb_cta_reduce" in text else text.index("mlcb_group_reduce")
    assert "out0 + out0_r" in text[:first_reduce] or "out1 + out1_r" in text[:first_reduce]
    assert text.count("mlcb_store<__half, 8>") == 2


def test_row_reductions_ask_for_single_wave_residency_when_the_row_fits():
    from mlc_compiler_b200.emit.reduction import Geometry, resident_ctas

    geo = Geometry(V=8, P=96, G=32, NP=3, block=128, rpb=4, grid=1024, masked=False)
    assert resident_ctas(geo, Config(), 64) == 7           # 1024 CTAs / 148 SMs, 73 registers each
    assert resident_ctas(geo, Config(), 100) == 5          # a fat row keeps its registers
    assert resident_ctas(geo, Config(reduction_min_ctas=3), 64) == 3
    small = Geometry(V=8, P=96, G=128, NP=1, block=128, rpb=1, grid=128, masked=True)
    assert resident_ctas(small, Config(), 40) == 4         # nothing to gain: the floor


@needs_nvcc
def test_dependent_launch_variant_compiles(tmp_path):
    src = generate_module(load_schedule("bert-base_b1_s128_float16"),
                          Config(dependent_launch=True)).source
    assert "#define MLCB_PDL 1" in src
    B.nvcc_cubin(src, tmp_path / "m.cubin")


def test_large_streaming_kernels_use_256_bit_accesses():
    """75 MB bias+GELU+residual: 16 halves per thread, one ld.global.v4.b64 each;
    the 2 MB batch-1 shape keeps 128-bit packs (more threads, lower latency)."""
    big = generate_module(load_schedule("micro-gelu_b32_s128_float16"), Config())
    assert big.launch["k0"].vector == 16 and "mlcb_load<__half, 16>" in big.source
    small = generate_module(load_schedule("micro-gelu_b1_s128_float16"), Config())
    assert small.launch["k0"].vector == 8
    off = generate_module(load_schedule("micro-gelu_b32_s128_float16"), Config(wide_access_bytes=0))
    assert off.launch["k0"].vector == 8


def test_committed_example_translation_unit_is_current():
    """csrc/examples holds the generated CUDA for BERT-base b8 verbatim."""
    assert B.EXAMPLE.exists()
    assert B.EXAMPLE.read_text() == B.example_source(), \
        "regenerate with mlc_compiler_b200.build.write_example()"


@needs_nvcc
def test_example_compiles_against_the_device_header(tmp_path):
    import subprocess

    out = tmp_path / "example.cubin"
    cmd = [B.nvcc_path(), *B.GENCODE, *B.NVCC_FLAGS, "-cubin", "-o", str(out), str(B.EXAMPLE)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]


# ---- counterparts of the reference's checks on generated source -----------------
# (``tests/test_reduction_fusion.py:284-330`` and ``tests/test_dtypes.py:61-69`` read
# the Triton text; these read the CUDA text for the same properties)

def _softmax_kernel(stem):
    from conftest import load_tiny
    s = load_tiny(stem)["schedule"]
    k = next(k for k in s.generated() if isinstance(k, kir.ReductionKernel))
    return generate_module(s, Config()).kernel_source(k.name)


def test_persistent_source_has_no_column_loop_and_streamed_rescales():
    persistent = _softmax_kernel("oddsm100__default__float32")
    assert "c0 +=" not in persistent                      # the row is read once, into registers
    assert "mlcb_op_max" in persistent and "mlcb_op_sum" in persistent
    streamed = _softmax_kernel("oddsm1000__streamed__float32")
    assert streamed.count("c0 += 128") == 2                # max+sum in one pass, then the store pass
    assert "run_l * ((run_m == MLCB_NINF_F) ? 0.0f : expf(run_m - nm))" in streamed
    assert "if (nm != MLCB_NINF_F)" in streamed            # a fully masked chunk cannot produce NaN


def test_dead_lanes_contribute_the_identity_of_the_reduction():
    # 100 columns over 32 lanes x 4: lanes 25..31 hold nothing; the max must see -inf
    # there (not a zero fill) and the sum must see 0
    src = _softmax_kernel("oddsm100__default__float32")
    assert "float acc_r2 = MLCB_NINF_F;" in src and "float acc_r5 = ((float)0);" in src
    body = src[src.index("float acc_r2"):src.index("const float r2")]
    assert "if (c0 < 100) {" in body                       # dead lanes never touch the accumulator
    assert body.index("if (c0 < 100)") < body.index("acc_r2 = mlcb_op_max")


def test_row_statistics_load_as_scalars():
    rows, cols = 6, 32
    rc = kir.IndexMap((kir.Axis("row", rows, ((rows, 1, cols),)), kir.Axis("col", cols, ((cols, 1, 1),))))
    r = kir.IndexMap((kir.Axis("row", rows, ((rows, 1, 1),)), kir.Axis("col", cols, ())))
    k = kir.ReductionKernel(
        "k0", (rows,), (cols,),
        [kir.Operand("x", "x", "float32", rc), kir.Operand("rowbias", "rowbias", "float32", r)],
        [kir.Operand("y", "y", "float32", kir.IndexMap((kir.Axis("row", rows, ((rows, 1, 1),)),)))],
        [kir.Reduce("r0", "max", kir.Load(0)),
         kir.Bind("t1", kir.Call("exp", (kir.Call("sub", (kir.Load(0), kir.Ref("r0"))),))),
         kir.Reduce("r2", "sum", kir.Ref("t1")),
         kir.Bind("t3", kir.Call("mul", (kir.Ref("r2"), kir.Load(1))))],
        {"y": kir.Ref("t3")}, {"y"}, False, ["amax", "sub", "exp", "sum", "mul"])
    from mlc_compiler_b200.emit.reduction import emit_reduction
    src, _ = emit_reduction(k, Config())
    scalar = [l for l in src.splitlines() if "mlcb_load1" in l]
    assert len(scalar) == 1 and "(per row)" in scalar[0] and "c0" not in scalar[0]
    assert "v1[" not in src                                # no register array for the per-row operand
    assert "if (live && lane == 0) mlcb_store1<float>(out0 + (row)" in src


def test_narrow_loads_widen_and_stores_round_back():
    from conftest import load_tiny
    s = load_tiny("layernorm_scale__default__float16")["schedule"]
    src = generate_module(s, Config(), inline_header=False).source     # kernels only, no device library
    loads = [l for l in src.splitlines() if "mlcb_load<" in l]
    assert loads and all("mlcb_load<__half," in l for l in loads)
    arrays = [l for l in src.splitlines() if l.strip().startswith(("float v", "__half v"))]
    assert arrays and all(l.strip().startswith("float v") for l in arrays)   # registers hold fp32
    stores = [l for l in src.splitlines() if "mlcb_store<" in l]
    assert stores and all("mlcb_store<__half," in l for l in stores)


def test_float64_streamed_softmax_keeps_two_float64_passes():
    """The fused online-softmax pass carries its running max and sum in fp32; a
    float64 row must not take it (the reference's torch backend and the
    persistent form both work in float64)."""
    from conftest import as_float64

    narrow = load_tiny("oddsm1025__streamed__float32")["schedule"]
    assert "run_m" in generate_module(narrow, Config()).source
    wide = as_float64(load_tiny("oddsm1025__streamed__float32"))["schedule"]
    src = generate_module(wide, Config()).source
    assert "run_m" not in src and "float acc_" not in src
    assert "double acc_" in src and "exp(" in src
