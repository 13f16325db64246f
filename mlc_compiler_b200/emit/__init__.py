"""CUDA C++ emitter: kernel IR -> sm_100a source."""

from .module import Module, emit_kernel, generate_module  # noqa: F401
from .pointwise import LaunchSpec, emit_pointwise  # noqa: F401
from .reduction import emit_reduction  # noqa: F401
