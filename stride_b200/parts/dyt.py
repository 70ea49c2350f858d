"""Dynamic Tanh in the place of a norm: ``tanh(alpha * x) * weight + bias`` per element, with a learned scalar
``alpha``; no mean and no variance is computed (Zhu et al., "Transformers without Normalization"). Tensors:
``<prefix>`` (the weight), ``<prefix>.b``, ``<prefix>.alpha``. The residual sum before it, with the architecture's
multiplier, is part of the same kernel."""

from __future__ import annotations

from ..csrc import ops
from .base import Norm, TensorDecl, register_part


class DynamicTanh(Norm):
    takes_scale = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.width = int(spec.width)
        names = dict(spec.params)
        self._weight_name = spec.prefix + names.get("weight", "")
        self._bias_name = spec.prefix + names.get("bias", ".b")
        self._alpha_name = spec.prefix + names.get("alpha", ".alpha")
        self.weight = self.bias = self._alpha_tensor = None
        self.alpha = 0.0

    def declare(self):
        return {self._weight_name: TensorDecl((self.width,), "vector"), self._bias_name: TensorDecl((self.width,), "vector"),
                self._alpha_name: TensorDecl((), "vector")}

    def bind(self, weights):
        self.weight, self.bias = weights[self._weight_name], weights[self._bias_name]
        self._alpha_tensor = weights[self._alpha_name]
        self.alpha = float(self._alpha_tensor) if self._alpha_tensor.device.type != "meta" else 0.0

    def named_tensors(self):
        return {self._weight_name: self.weight, self._bias_name: self.bias, self._alpha_name: self._alpha_tensor}

    def apply(self, residual, pending, out, rows=None, scale: float = 1.0):
        ops.add_dyt(residual, pending, scale, self.weight, self.bias, self.alpha, out, rows=rows)


register_part("norm", "dyt", DynamicTanh)
