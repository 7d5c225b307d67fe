"""Linear, Conv2d, the activation modules and Sequential: forward of the reference's
python/cuDeep/nn.py:36-189 on this library's kernels.

Same constructor arguments, parameter names ("weight", "bias"), state_dict keys and default
initialisation (randn weights, zero bias, nn.py:104-108,131-137) as the reference.  Differences,
all on the forward path:
  * Linear.forward is one fused kernel (W consumed as stored, bias in the epilogue) instead of
    transpose-copy + matmul + broadcast_add;
  * Sequential.forward folds an activation module that directly follows a Linear or Conv2d into
    that layer's epilogue (the unfused result is the same function applied as a separate pass).
Training (autograd, optimisers) is outside this library's scope.
"""
from __future__ import annotations

from typing import Optional

import numpy as np

from .tensor import DType, Tensor, conv2d, linear


class Parameter(Tensor):
    def __init__(self, data: Tensor):
        super().__init__(data.shape(), data.dtype(), _storage=data._storage, _strides=data.strides())

    def __repr__(self):
        return f"Parameter(shape={self.shape()}, dtype={self.dtype()})"


class Module:
    def __init__(self):
        self._parameters: dict[str, Parameter] = {}
        self._modules: dict[str, "Module"] = {}
        self._training = True

    def forward(self, *args, **kwargs):
        raise NotImplementedError

    def __call__(self, *args, **kwargs):
        return self.forward(*args, **kwargs)

    def register_parameter(self, name: str, tensor):
        if not isinstance(tensor, Parameter):
            tensor = Parameter(tensor)
        self._parameters[name] = tensor

    def register_module(self, name: str, module: "Module"):
        self._modules[name] = module

    def parameters(self) -> list:
        params = list(self._parameters.values())
        for mod in self._modules.values():
            params.extend(mod.parameters())
        return params

    def named_parameters(self):
        for name, p in self._parameters.items():
            yield name, p
        for mod_name, mod in self._modules.items():
            for pname, p in mod.named_parameters():
                yield f"{mod_name}.{pname}", p

    def train(self, mode=True):
        self._training = mode
        for m in self._modules.values():
            m.train(mode)
        return self

    def eval(self):
        return self.train(False)

    @property
    def training(self):
        return self._training

    def state_dict(self) -> dict:
        return {name: p.numpy() for name, p in self.named_parameters()}

    def load_state_dict(self, sd: dict):
        owners = {}
        self._collect_owners("", owners)
        for name, arr in sd.items():
            if name in owners:
                module, key = owners[name]
                module._parameters[key] = Parameter(Tensor.from_numpy(np.ascontiguousarray(arr)))

    def _collect_owners(self, prefix: str, out: dict):
        for key in self._parameters:
            out[prefix + key] = (self, key)
        for mod_name, mod in self._modules.items():
            mod._collect_owners(f"{prefix}{mod_name}.", out)


class Linear(Module):
    """y = x W^T + b  (reference nn.py:97-115)."""

    def __init__(self, in_features, out_features, bias=True, dtype=DType.float32):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.register_parameter("weight", Tensor.randn([out_features, in_features], dtype))
        if bias:
            self.register_parameter("bias", Tensor.zeros([out_features], dtype))

    def forward(self, x, activation=None):
        return linear(x, self._parameters["weight"], self._parameters.get("bias"), activation)


class Conv2d(Module):
    """2-D convolution (reference nn.py:118-142)."""

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, bias=True,
                 dtype=DType.float32):
        super().__init__()
        if isinstance(kernel_size, int):
            kernel_size = (kernel_size, kernel_size)
        if isinstance(stride, int):
            stride = (stride, stride)
        if isinstance(padding, int):
            padding = (padding, padding)
        self.stride = stride
        self.padding = padding
        self.register_parameter(
            "weight", Tensor.randn([out_channels, in_channels, kernel_size[0], kernel_size[1]], dtype))
        if bias:
            self.register_parameter("bias", Tensor.zeros([out_channels], dtype))

    def forward(self, x, activation=None):
        return conv2d(x, self._parameters["weight"], self._parameters.get("bias"), self.stride, self.padding,
                      activation)


class _Activation(Module):
    name: Optional[str] = None

    def forward(self, x):
        return getattr(x, self.name)()


class ReLU(_Activation):
    name = "relu"


class GELU(_Activation):
    name = "gelu"


class SiLU(_Activation):
    name = "silu"


class Sigmoid(_Activation):
    name = "sigmoid"


class Sequential(Module):
    """Runs modules in order (reference nn.py:173-189), fusing Linear/Conv2d + activation pairs."""

    def __init__(self, *modules, fuse=True):
        super().__init__()
        self.fuse = fuse
        for i, m in enumerate(modules):
            self.register_module(str(i), m)

    def forward(self, x):
        mods = list(self._modules.values())
        i = 0
        while i < len(mods):
            m = mods[i]
            nxt = mods[i + 1] if i + 1 < len(mods) else None
            if (self.fuse and isinstance(m, (Linear, Conv2d)) and isinstance(nxt, _Activation)
                    and x.dtype() == DType.float32):
                x = m.forward(x, activation=nxt.name)
                i += 2
            else:
                x = m(x)
                i += 1
        return x

    def __getitem__(self, idx):
        return list(self._modules.values())[idx]

    def __len__(self):
        return len(self._modules)
