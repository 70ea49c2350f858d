"""Routed feed-forward (a mixture of experts) with an optional shared expert.

Router logits ``z = W_r h + b`` in float32; a token uses the ``top`` experts with the largest logits, weighted with
the softmax over those logits only; an expert is ``W_down act(W_up h)`` without biases, ``act`` the square of relu;
a shared expert of the same form runs for every token and is added.

On the device: the router's product leaves float32 logits, a kernel chooses, a one-CTA plan lays the (token, choice) pairs out expert by expert, two
grouped products run all experts' rows in one launch each (the first gathers its rows through the plan and applies
the activation, the second leaves float32 rows), and one kernel sums a token's rows with its weights and the
shared expert's output. Nothing returns to the host, so a step can be captured in a graph.

Spec: ``hidden``, ``intermediate`` (an expert's width), ``activation`` (``relu_squared``), params ``experts``, ``top``,
``shared`` (the shared expert's width, 0 for none), ``router_bias``. Tensors under the prefix: ``router``, ``router.b``,
``e<k>.up``, ``e<k>.down``, ``shared.up``, ``shared.down``.
"""

from __future__ import annotations

import torch

from ..csrc import ops
from .base import FeedForward, TensorDecl, register_part


class RoutedExperts(FeedForward):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = dict(spec.params)
        self.hidden, self.ff = int(spec.hidden), int(spec.intermediate)
        self.experts, self.top, self.shared_ff = int(p["experts"]), int(p["top"]), int(p.get("shared", 0))
        self.router_bias = bool(p.get("router_bias", False))
        if spec.activation != "relu_squared":
            raise ValueError(f"activation {spec.activation!r} is not supported by the routed experts (relu_squared is)")
        if not 1 <= self.top <= min(self.experts, 32) or self.experts > 256:
            raise ValueError(f"top {self.top} of {self.experts} experts is not supported (up to 32 of up to 256 are)")
        self.w_router = self.bias = self.w_up = self.w_down = self.shared_up = self.shared_down = None

    def _n(self, short):
        return self.spec.prefix + short

    def declare(self):
        d = {self._n("router"): TensorDecl((self.experts, self.hidden))}
        if self.router_bias:
            d[self._n("router.b")] = TensorDecl((self.experts,), "vector")
        for e in range(self.experts):
            d[self._n(f"e{e}.up")] = TensorDecl((self.ff, self.hidden))
            d[self._n(f"e{e}.down")] = TensorDecl((self.hidden, self.ff))
        if self.shared_ff:
            d[self._n("shared.up")] = TensorDecl((self.shared_ff, self.hidden))
            d[self._n("shared.down")] = TensorDecl((self.hidden, self.shared_ff))
        return d

    def bind(self, weights):
        self.w_router = weights[self._n("router")]
        self.bias = weights[self._n("router.b")] if self.router_bias else None
        self.w_up = torch.stack([weights[self._n(f"e{e}.up")] for e in range(self.experts)]).contiguous()
        self.w_down = torch.stack([weights[self._n(f"e{e}.down")] for e in range(self.experts)]).contiguous()
        if self.shared_ff:
            self.shared_up, self.shared_down = weights[self._n("shared.up")], weights[self._n("shared.down")]

    def named_tensors(self):
        out = {self._n("router"): self.w_router}
        if self.router_bias:
            out[self._n("router.b")] = self.bias
        for e in range(self.experts):
            out[self._n(f"e{e}.up")], out[self._n(f"e{e}.down")] = self.w_up[e], self.w_down[e]
        if self.shared_ff:
            out[self._n("shared.up")], out[self._n("shared.down")] = self.shared_up, self.shared_down
        return out

    def forward(self, x, ctx):
        tokens, top = x.shape[0], self.top
        pairs = tokens * top
        i32 = torch.int32
        ids = self.rt.buffer("moe_ids", tokens, top, i32)
        weights = self.rt.buffer("moe_weights", tokens, top, torch.float32)
        logits = self.rt.buffer("moe_logits", tokens, self.experts, torch.float32)
        ops.linear(x, self.w_router, logits)            # float32 sums of exact products, float32 logits
        ops.moe_select(logits, self.bias, ctx.seq_of_token[:tokens], ids, weights)
        row_of = self.rt.buffer("moe_row_of", tokens, top, i32)
        perm = self.rt.buffer("moe_perm", tokens, top, i32).view(-1)
        rank = self.rt.buffer("moe_rank", tokens, top, i32).view(-1)
        offsets = self.rt.scratch(f"moe_offsets_{self.experts}", self.experts + 1, i32)
        ops.moe_plan(ids, self.experts, offsets, perm, row_of, rank)
        hidden_rows = self.rt.buffer("moe_hidden", tokens, top * self.ff).view(pairs, self.ff)
        ops.grouped_gemm(x, perm, self.w_up, offsets, hidden_rows, pairs, act=1)
        y = self.rt.buffer("moe_y", tokens, top * self.hidden, torch.float32).view(pairs, self.hidden)
        ops.grouped_gemm(hidden_rows, None, self.w_down, offsets, y, pairs, act=0)
        shared = None
        if self.shared_ff:
            mid = self.rt.buffer("moe_shared_mid", tokens, self.shared_ff)
            ops.linear(x, self.shared_up, mid)
            ops.relu_squared(mid)
            shared = self.rt.buffer("moe_shared_out", tokens, self.hidden)
            ops.linear(mid, self.shared_down, shared)
        out = self.rt.buffer("ffn_out", tokens, self.hidden)
        ops.moe_combine(y, row_of, weights, shared, out)
        return out


register_part("feed_forward", "routed_experts", RoutedExperts)
