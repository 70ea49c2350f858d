"""Several mixers side by side: all read the same normed input, and the layer's mixer output is the weighted sum of
theirs, ``sum_i scale_i * mixer_i(h)``.

Spec params: ``branches``, a tuple of ``(MixerSpec, scale)``; each branch is built from the part registry by its own
kind and finds its tensors under its own prefix. The branches share the run's cache slot: at most one of them may keep
pages and at most one a state of fixed size (an attention beside a recurrence, say), so the cache manager sees one
mixer. The sum is formed in float32, in one kernel, and handed on in the compute type.
"""

from __future__ import annotations

import torch

from ..csrc import ops
from .base import Mixer, Projection, build_part, register_part


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
        outs = []
        for i, (mixer, _scale) in enumerate(self.branches):
            # every branch's output in a buffer of this part's own: the branches' own output buffers may be one and the same
            out = self.rt.buffer(f"parallel_branch{i}", tokens, self.hidden)
            if mixer.lazy_output:
                p = mixer.forward(x, ctx, cache, lazy_output=True)
                if isinstance(p, Projection):
                    ops.linear(p.x, p.weight, out)
                else:
                    out.copy_(p)
            else:
                out.copy_(mixer.forward(x, ctx, cache))
            outs.append(out)
        total = outs[0]
        if len(outs) == 1:
            ops.weighted_sum(total, outs[0], self.branches[0][1], outs[0], 0.0)
        for i in range(1, len(outs)):
            ops.weighted_sum(total, total, self.branches[0][1] if i == 1 else 1.0, outs[i], self.branches[i][1])
        return total


register_part("mixer", "parallel", ParallelMixer)
