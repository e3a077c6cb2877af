"""pcp_b200 — B200-native execution backend for PCP's training hot path.

The product is the C-ABI shared library (include/pcp_b200.h, built from pcp_b200/csrc by
pcp_b200/build.py).  This package holds its ctypes binding (backend.py), the forward-graph
exporter for model shapes the reference does not ship (export.py) and the build script.
"""
from .backend import (BF16, BOOL, F16, F32, F64, I32, I64, Backend, BackendError, DeviceBuffer,  # noqa: F401
                      load_library)
from .export import (NanochatConfig, NanoGPTConfig, QwenConfig, nanochat_forward_mlir, nanogpt_forward_mlir,  # noqa: F401
                     qwen_forward_mlir)
