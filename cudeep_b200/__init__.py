"""cuDeep's dense-contraction path (matmul, Linear forward, Conv2d forward) for NVIDIA B200.

    from cudeep_b200 import Tensor, nn
    y = nn.Linear(4096, 16384)(Tensor.from_numpy(x))

The package is a thin host layer over libcudeep_b200.so (build it with
`python -m cudeep_b200.build`); importing it does not load the library, the first operation does.
"""
from . import nn
from .tensor import (DType, Event, MemoryPool, Stream, Tensor, broadcast_add, conv2d, device_info, gelu, linear,
                     matmul_backward, relu, sigmoid, silu)

__version__ = "0.1.0"

__all__ = ["Tensor", "DType", "Stream", "Event", "MemoryPool", "broadcast_add", "conv2d", "linear", "relu", "gelu",
           "silu", "sigmoid", "device_info", "matmul_backward", "nn"]
