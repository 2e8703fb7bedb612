"""helium_b200: B200 (sm_100a) kernels for the fused-kernel hot path of caelunshun/helium.

The package is a thin host layer over libhelium_b200.so (C ABI in include/helium_b200.h):
  ir        host mirror of the helium-ir / playground op graph, flattened for the C ABI
  runtime   Context / Plan objects (he_ctx / he_plan)
Importing it requires the built library; there is no fallback path.
"""
from . import configs, ir
from ._lib import LIB_PATH, HeliumError, lib
from .host import Executor, HostGraph
from .runtime import Comm, Context, Plan, permute_output_strides, plan_supported

__all__ = ["ir", "configs", "HostGraph", "Executor", "lib", "LIB_PATH", "HeliumError", "Context", "Plan", "Comm", "permute_output_strides", "plan_supported"]
