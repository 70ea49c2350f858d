"""RMSNorm: ``x * rsqrt(mean(x^2) + eps) * weight`` in float32, the weight
multiplying after the normalisation (python/stride_worker/layers.py:24-35).

Spec params: ``tensor`` names the weight (default: the prefix + ``weight``); ``weight_offset`` c makes the factor
``c + w`` for checkpoints that keep w = factor - c (the sum is formed once, in float32, when the weight is bound)."""

from __future__ import annotations

from ..csrc import ops
from .base import Norm, TensorDecl, register_part


class RMSNorm(Norm):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.eps = float(spec.eps)
        self.width = int(spec.width)
        self.weight = None
        p = dict(spec.params)
        self._name = p.get("tensor", spec.prefix + "weight")
        self.offset = float(p.get("weight_offset", 0.0))
        self.stored = None

    def declare(self):
        return {self._name: TensorDecl((self.width,), "vector")}

    def bind(self, weights):
        self.stored = weights[self._name]
        self.weight = self.stored + self.offset if self.offset else self.stored

    def named_tensors(self):
        return {self._name: self.stored}

    def fold_inputs(self):
        return self.weight, self.eps

    def apply(self, residual, pending, out, rows=None):
        ops.add_rmsnorm(residual, pending, self.weight, out, self.eps, rows=rows)      # sum, write-back and norm in one kernel


register_part("norm", "rmsnorm", RMSNorm)
