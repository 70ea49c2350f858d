"""A per-layer token input: every layer adds to the stream a slice of a second embedding of the token, gated by
the stream itself.

    e = table[token, offset : offset + dim]
    g = gelu_tanh(W_gate x) * e
    y = W_proj g
    x <- x + scale * y / sqrt(mean(y^2) + eps) * norm_weight

Tensors: the table under ``spec.table_name`` (one copy on the device for all layers), ``<prefix>gate`` [dim, hidden],
``<prefix>proj`` [hidden, dim], ``<prefix>norm`` [hidden]. The two products run as matrix products (on the stream rounded
to the compute type; the 32-bit path reads the float32 stream itself), the rest in two small kernels; the normalisation
and the sum into the stream are float32."""

from __future__ import annotations

import torch

from ..csrc import ops
from .base import StreamInput, TensorDecl, register_part


class TokenSideInput(StreamInput):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        s = spec
        if s.dim <= 0 or s.offset < 0 or s.offset + s.dim > s.table_width:
            raise ValueError(f"a slice of {s.dim} at {s.offset} does not fit a table row of {s.table_width}")
        self.table = self.gate = self.proj = self.norm = None

    def _names(self):
        p = self.spec.prefix
        return p + "gate", p + "proj", p + "norm"

    def declare(self):
        s = self.spec
        gate, proj, norm = self._names()
        return {s.table_name: TensorDecl((s.vocab, s.table_width)), gate: TensorDecl((s.dim, s.hidden)),
                proj: TensorDecl((s.hidden, s.dim)), norm: TensorDecl((s.hidden,), "vector")}

    def bind(self, weights):
        gate, proj, norm = self._names()
        name = self.spec.table_name
        self.table = self.rt.shared(("token_side_table", name), lambda: weights[name])
        self.gate, self.proj, self.norm = weights[gate], weights[proj], weights[norm]

    def named_tensors(self):
        gate, proj, norm = self._names()
        return {self.spec.table_name: self.table, gate: self.gate, proj: self.proj, norm: self.norm}

    def forward(self, stream, ctx, scale: float) -> None:
        x = stream.materialize()
        tokens, s = x.shape[0], self.spec
        ids, seq = ctx.token_ids[:tokens], ctx.seq_of_token[:tokens]
        if self.rt.dtype == torch.float32:
            rounded = x
        else:
            rounded = self.rt.buffer("side_x", tokens, s.hidden)
            ops.cast_rows(x, rounded)
        pre = self.rt.buffer("side_pre", tokens, s.dim)
        ops.linear(rounded, self.gate, pre)
        gated = self.rt.buffer("side_gated", tokens, s.dim)
        ops.side_gate(pre, ids, seq, self.table, s.offset, gated)
        y = self.rt.buffer("side_y", tokens, s.hidden)
        ops.linear(gated, self.proj, y)
        ops.side_norm_add(x, y, seq, self.norm, s.eps, scale)


register_part("stream_input", "token_side", TokenSideInput)
