"""B200-native SSD chunked scan (forward + backward) behind the reference operator interface.

Exports mirror src/kernels/__init__.py of the reference for this path (the scan) and for the two element-wise
operators that feed it (rotation, trapezoidal coefficients).
"""
from .ssd_scan import (FusedSSDScan, LazySSDCache, fused_ssd_scan, resolved_path_name, set_check_status, set_eager_cache, set_save_states,
                       set_kernel_path, ssd_mamba2, ssd_mamba2_gated)
from .host_pipeline import HostPipeline, SequenceStreamer
from .mamba3 import ssd_mamba3
from .elementwise import (FusedRMSNorm, FusedRMSNormModule, FusedRoPE, FusedTrapezoidal, fused_gate_norm, fused_rmsnorm, fused_rope,
                          fused_trapezoidal)
from .workloads import (CONFIGS, SSDConfig, kernel_algorithmic_bytes, make_inputs, make_reference_test_inputs,
                        shrink)

__all__ = ["FusedSSDScan", "LazySSDCache", "fused_ssd_scan", "set_eager_cache", "set_kernel_path", "ssd_mamba2", "ssd_mamba2_gated", "ssd_mamba3", "HostPipeline", "SequenceStreamer",
           "FusedRoPE", "FusedTrapezoidal", "fused_rope", "fused_trapezoidal", "FusedRMSNorm", "FusedRMSNormModule", "fused_rmsnorm",
           "fused_gate_norm",
           "resolved_path_name", "set_check_status", "set_save_states", "kernel_algorithmic_bytes", "CONFIGS", "SSDConfig", "make_inputs", "make_reference_test_inputs", "shrink"]
