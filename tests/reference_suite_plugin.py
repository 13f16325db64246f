"""pytest plugin for running the REFERENCE's own test files on a GPU with this
backend installed (loaded with ``-p reference_suite_plugin`` by
``test_gpu_reference_suite.py`` in a child pytest; never by this repository's
own suite).

The reference's tests build their modules and inputs on the default device and
let ``mlc.compile`` infer the device from the inputs.  Making CUDA the default
device therefore sends every ``mlc.compile`` of the suite down the
generated-kernel path, which ``mlc_compiler_b200.install()`` has re-pointed at
this backend -- under the reference's own executor, or under this package's with
``MLCB_SUITE_MODE=native``.  The plugin counts the runtimes that were really
built on the CUDA device and prints the tally, so that the parent test can tell
a green run from a run that silently stayed on the interpreter.
"""

import os
import pathlib
import sys

import torch

sys.path.insert(0, str(pathlib.Path(__file__).resolve().parent.parent))

COUNT = {"runtimes": 0, "on_cuda": 0, "generated_kernels": 0}


def pytest_configure(config):
    import mlc_compiler_b200 as mb

    if not torch.cuda.is_available():
        raise RuntimeError("the reference suite is only run through this plugin on a CUDA device")
    torch.set_default_device("cuda")
    mb.install(native_executor=os.environ.get("MLCB_SUITE_MODE", "dropin") == "native")


def pytest_sessionstart(session):
    from mlc_compiler_b200 import runtime

    original = runtime.CudaRuntime.__init__

    def counted(self, schedule, cfg, device, *a, **kw):
        original(self, schedule, cfg, device, *a, **kw)
        COUNT["runtimes"] += 1
        COUNT["on_cuda"] += int(torch.device(device).type == "cuda")
        COUNT["generated_kernels"] += len(self.ir.generated())

    runtime.CudaRuntime.__init__ = counted


def pytest_sessionfinish(session, exitstatus):
    print(f"\n[mlcb-suite] runtimes={COUNT['runtimes']} on_cuda={COUNT['on_cuda']} "
          f"generated_kernels={COUNT['generated_kernels']}")
