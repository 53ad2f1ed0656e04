"""caffecontroll_b200 — the B200 (sm_100a) convolution hot path of Caffe con Troll, and the layers a CaffeNet iteration
needs around it, behind a C ABI.

The package holds only what that path needs: csrc/ (CUDA kernels + the C ABI of include/cct_b200.h), capi.py (ctypes
binding), bridge.py and layers.py (mirrors of the reference's LogicalCube / Layer / bridge interfaces), parallel.py
(ParallelizedBridge's batch partitioning over one process per GPU, NCCL gradient sums), net.py (prototxt reader, network
builder, model files), nets/ (the CaffeNet description the benchmark runs) and host/ (the C++ mirror and the headers a
maintainer drops into the reference tree).
"""
from . import capi  # noqa: F401
from .bridge import Context, ConvolutionBridge, FullyConnectedBridge, Layer, LogicalCube, conv_layer  # noqa: F401

__all__ = ["capi", "Context", "ConvolutionBridge", "FullyConnectedBridge", "Layer", "LogicalCube", "conv_layer"]
