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
    """A tensor a Module owns: shares the storage of the tensor it was made from (reference nn.py:20-30)."""

    def __init__(self, data: Tensor):
        super().__init__(data.shape(), data.dtype(), _storage=data._storage, _strides=data.strides())

    def __repr__(self):
        return "Parameter(shape={}, dtype={})".format(self.shape(), self.dtype())


class Module:
    """Container of parameters and sub-modules with the reference's public surface (nn.py:33-90):
    forward / __call__, register_parameter / register_module, parameters / named_parameters,
    train / eval / training, state_dict / load_state_dict.  Parameter names are dotted paths,
    a module's own parameters before those of its children, children in registration order.
    Every query is one depth-first walk (`_owned`)."""

    def __init__(self):
        self._parameters: dict[str, Parameter] = {}
        self._modules: dict[str, "Module"] = {}
        self._training = True

    # -- calling ------------------------------------------------------------------------------
    def forward(self, *args, **kwargs):
        raise NotImplementedError(f"{type(self).__name__} does not define forward()")

    def __call__(self, *args, **kwargs):
        return self.forward(*args, **kwargs)

    # -- registration ---------------------------------------------------------------------------
    def register_parameter(self, name: str, tensor) -> None:
        self._parameters[name] = tensor if isinstance(tensor, Parameter) else Parameter(tensor)

    def register_module(self, name: str, module: "Module") -> None:
        self._modules[name] = module

    # -- traversal ------------------------------------------------------------------------------
    def _owned(self, prefix: str = ""):
        """(dotted name, owning module, key) of every parameter below this module."""
        for key in self._parameters:
            yield prefix + key, self, key
        for child_name, child in self._modules.items():
            yield from child._owned(f"{prefix}{child_name}.")

    def named_parameters(self):
        for name, owner, key in self._owned():
            yield name, owner._parameters[key]

    def parameters(self) -> list:
        return [p for _, p in self.named_parameters()]

    # -- mode -----------------------------------------------------------------------------------
    def train(self, mode=True):
        stack = [self]
        while stack:
            module = stack.pop()
            module._training = mode
            stack.extend(module._modules.values())
        return self

    def eval(self):
        return self.train(False)

    @property
    def training(self):
        return self._training

    # -- state ----------------------------------------------------------------------------------
    def state_dict(self) -> dict:
        return {name: p.numpy() for name, p in self.named_parameters()}

    def load_state_dict(self, sd: dict):
        """Replaces every parameter named in `sd`; names this module does not have are ignored."""
        for name, owner, key in list(self._owned()):
            if name in sd:
                owner._parameters[key] = Parameter(Tensor.from_numpy(np.ascontiguousarray(sd[name])))


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
