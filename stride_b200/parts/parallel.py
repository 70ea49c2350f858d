"""Several mixers side by side: all read the same normed input, and the layer's mixer output is the weighted sum of
theirs, ``sum_i scale_i * mixer_i(h)``.

Spec params: ``branches``, a tuple of ``(MixerSpec, scale)``; each branch is built from the part registry by its own
kind and finds its tensors under its own prefix. The branches share the run's cache slot: at most one of them may keep
pages and at most one a state of fixed size (an attention beside a recurrence, say), so the cache manager sees one
mixer. The sum is formed in float32 and handed on in the compute type.
"""

from __future__ import annotations

import torch

from ..csrc import ops
from .base import Mixer, build_part, register_part


class ParallelMixer(Mixer):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        branches = dict(spec.params).get("branches", ())
        if not branches:
            raise ValueError("a parallel mixer needs at least one branch")
        self.branches = [(build_part("mixer", s, runtime), float(scale)) for s, scale in branches]
        if sum(m.cache_request() is not None for m, _ in self.branches) > 1 or sum(m.state_request() is not None for m, _ in self.branches) > 1:
            raise ValueError("at most one branch of a parallel mixer may keep pages, and at most one a state")
        self.hidden = int(spec.hidden)
        self.graph_safe = all(getattr(m, "graph_safe", True) for m, _ in self.branches)

    def declare(self):
        d = {}
        for m, _ in self.branches:
            d.update(m.declare())
        return d

    def bind(self, weights):
        for m, _ in self.branches:
            m.bind(weights)

    def named_tensors(self):
        d = {}
        for m, _ in self.branches:
            d.update(m.named_tensors())
        return d

    def cache_request(self):
        return next((r for r in (m.cache_request() for m, _ in self.branches) if r is not None), None)

    def state_request(self):
        return next((r for r in (m.state_request() for m, _ in self.branches) if r is not None), None)

    def forward(self, x, ctx, cache):
        tokens = x.shape[0]
        total = self.rt.buffer("parallel_sum", tokens, self.hidden, torch.float32)
        total.zero_()
        for mixer, scale in self.branches:
            # branch by branch: the branches' outputs may share a buffer
            ops.add_scaled(total, mixer.forward(x, ctx, cache), scale)
        if self.rt.dtype == torch.float32:
            return total
        result = self.rt.buffer("parallel_out", tokens, self.hidden)
        ops.cast_rows(total, result)
        return result


register_part("mixer", "parallel", ParallelMixer)
