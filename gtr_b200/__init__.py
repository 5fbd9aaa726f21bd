"""gtr_b200: B200-native (sm_100a) chunkwise gated-linear-attention forward for the GTR backbone.

The package holds the hot path only: CUDA kernels behind a C ABI (csrc/, include/gla_b200.h),
this ctypes/PyTorch front end, and the backbone pieces that call it.
"""
from .ops import (DIRECTIONS, backward_workspace_bytes, check_status, chunk_gla_backward, fused_recurrent_gla, layernorm, chunk_gla, chunk_gla_run, chunk_gla_run_gated, chunk_gla_with_ws, kBT, kK,
                  kV, make_workspace, rmsnorm_gated, stream_probe, swiglu_dwconv, workspace_bytes, workspace_floats)

__all__ = ["DIRECTIONS", "backward_workspace_bytes", "check_status", "chunk_gla_backward", "chunk_gla", "fused_recurrent_gla", "chunk_gla_run", "chunk_gla_run_gated", "chunk_gla_with_ws",
           "kBT", "kK", "kV", "layernorm", "make_workspace", "rmsnorm_gated", "stream_probe", "swiglu_dwconv", "workspace_bytes", "workspace_floats"]
