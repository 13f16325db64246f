"""Drop-in installation into the reference, exercised where the reference can be
imported (the copy ``oracle/ref.py`` installs, else a checkout named by
$MLC_REFERENCE or lying beside this repository); skipped elsewhere.  CPU only:
routing and source generation; ``test_gpu_reference.py`` executes the same
boundary on a GPU."""

import pathlib
import sys

import pytest
import torch

sys.path.insert(0, str(pathlib.Path(__file__).resolve().parent.parent / "oracle"))
import ref as reference_copy  # noqa: E402

REF = reference_copy.path()
pytestmark = pytest.mark.skipif(REF is None, reason="reference not present")


@pytest.fixture()
def installed():
    sys.dont_write_bytecode = True
    sys.path.insert(0, str(REF))
    import mlc_compiler_b200 as mb

    mb.install()
    yield mb
    mb.uninstall()
    sys.path.remove(str(REF))


def test_install_repoints_the_generated_kernel_path(installed):
    import mlc.codegen.triton_backend as tb
    import mlc.runtime.executor as ex
    import mlc.runtime.triton_runtime as tr
    from mlc.config import Config
    from mlc_compiler_b200.runtime import CudaRuntime

    assert tr.TritonRuntime is CudaRuntime
    assert ex.select_backend(Config(), torch.device("cuda")) == "triton"   # generated-kernel branch
    assert ex.select_backend(Config(), torch.device("cpu")) == "torch"
    assert ex.select_backend(Config(backend="torch"), torch.device("cuda")) == "torch"
    with pytest.raises(ValueError, match="Triton"):
        ex.select_backend(Config(backend="triton"), torch.device("cuda"))
    installed.uninstall()
    assert tr.TritonRuntime is not CudaRuntime
    assert "triton" in tb.generate_module.__module__
    installed.install()


def test_reference_source_command_now_emits_cuda(installed):
    import mlc.codegen.triton_backend as tb
    from mlc.api import build_pipeline
    from mlc.config import Config
    from mlc.ir.capture import capture

    class M(torch.nn.Module):
        def forward(self, x, b):
            return torch.nn.functional.layer_norm(x + b, (32,)).softmax(-1)

    g = capture(M(), (torch.randn(6, 32), torch.randn(32)))
    sched = build_pipeline(g, Config())
    src = tb.generate_module(sched, Config())
    assert 'extern "C" __global__' in src and "@triton.jit" not in src
    names = [k.name for k in sched.kernels if type(k).__name__ != "ExternKernel"]
    assert all(f" {n} " in src or f"{n}," in src or f", {n}" in src or f": {n}" in src
               for n in names)


def test_reference_torch_backend_still_runs_after_install(installed):
    import mlc
    from mlc.config import Config

    class M(torch.nn.Module):
        def forward(self, x):
            return torch.tanh(x * 0.5) + 1.0

    x = torch.randn(4, 8)
    out = mlc.compile(M(), (x,), Config(backend="torch", cuda_graphs=False), device="cpu")(x)
    torch.testing.assert_close(out, torch.tanh(x * 0.5) + 1.0)


def test_frontend_bridge_captures_into_this_ir(installed):
    from mlc_compiler_b200 import Config, capture_schedule, kir

    class M(torch.nn.Module):
        def forward(self, x):
            return (x * 2.0).softmax(-1)

    s = capture_schedule(M(), (torch.randn(3, 16),), Config())
    assert isinstance(s, kir.Schedule) and s.counts() == {"reduction": 1}
    assert kir.dumps(kir.loads(kir.dumps(s))) == kir.dumps(s)


def test_native_executor_is_opt_in_and_leaves_the_interpreter_alone(installed):
    import mlc
    import mlc.api as api
    from mlc.config import Config

    reference_cls = api.CompiledModel
    installed.install(native_executor=True)
    assert api.CompiledModel is not reference_cls

    class M(torch.nn.Module):
        def forward(self, x):
            return (x * 2.0).softmax(-1)

    x = torch.randn(3, 16)
    c = mlc.compile(M(), (x,), Config(backend="torch", cuda_graphs=False), device="cpu")
    assert isinstance(c, reference_cls)                 # CPU / torch backend: untouched
    torch.testing.assert_close(c(x), (x * 2.0).softmax(-1))
    installed.install()                                  # default: reference executor again
    assert api.CompiledModel is reference_cls
