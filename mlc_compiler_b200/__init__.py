"""B200-native CUDA kernel backend for the mlc inference compiler.

The package replaces one path of the reference: its Triton code generator and
runtime (``mlc/codegen/triton_backend.py``, ``triton_reduction.py``,
``mlc/runtime/triton_runtime.py``) behind the executor.  Fused kernel-IR nodes
are emitted as CUDA C++ for sm_100a, compiled with NVRTC and launched through a
C ABI (``include/mlcb.h``); matmuls stay on cuBLAS exactly as the reference
dispatches them.

Two ways to use it:

* next to the reference: ``mlc_compiler_b200.install()`` re-points the
  reference executor at :class:`CudaRuntime`; ``mlc.compile(...)`` is unchanged;
* without the reference frontend: ``load_schedule(name)`` +
  ``CompiledModel(schedule, params, cfg, device)``.
"""

from . import kir  # noqa: F401
from .config import ELEMENTWISE_ONLY, NO_FUSION, Config  # noqa: F401
from .emit import generate_module  # noqa: F401
from .frontend import FrontendUnavailable, capture_schedule, load_schedule  # noqa: F401


def __getattr__(name):
    # torch.cuda-facing pieces are imported on first use so that emit-only users
    # (source inspection, build checks) do not pay for them
    if name in ("CompiledModel", "ExecutionError", "select_backend"):
        from . import executor
        return getattr(executor, name)
    if name in ("CudaRuntime", "BackendError", "load_library"):
        from . import runtime
        return getattr(runtime, name)
    if name in ("install", "uninstall"):
        from . import integrate
        return getattr(integrate, name)
    if name == "compile":
        from .integrate import compile as _compile
        return _compile
    raise AttributeError(name)
