"""caffecontroll_b200 — the B200 (sm_100a) convolution hot path of Caffe con Troll behind a C ABI.

The package holds only what that path needs: csrc/ (CUDA kernels + the C ABI of include/cct_b200.h),
capi.py (ctypes binding), bridge.py (mirror of the reference's LogicalCube / Layer / ConvolutionBridge
interface) and parallel.py (ParallelizedBridge's batch partitioning over one process per GPU).
"""
from . import capi  # noqa: F401
from .bridge import Context, ConvolutionBridge, FullyConnectedBridge, Layer, LogicalCube, conv_layer  # noqa: F401

__all__ = ["capi", "Context", "ConvolutionBridge", "FullyConnectedBridge", "Layer", "LogicalCube", "conv_layer"]
