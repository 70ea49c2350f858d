"""Recurrent block with a real-gated linear recurrent unit (the recurrent layer of Griffin).

Two branches of ``width`` channels from the layer's input h: ``y = gelu_tanh(W_y h + b_y)`` and
``u = conv(W_x h + b_x)``, a causal convolution per channel over the last ``taps`` inputs. In each of ``blocks``
equal parts of the channels, ``r = sigmoid(W_a u + b_a)`` and ``i = sigmoid(W_i u + b_i)`` with square matrices;
``a = exp(-decay_scale * r * softplus(lam))`` and ``S_t = a S_(t-1) + sqrt(1 - a^2) * i * u`` from S = 0; the output is
``W_o (S * y)``. Everything after the two projections is float32.

Per request the mixer keeps, in one state slot of shape [taps, width] float32, the last taps-1 inputs of the
convolution (oldest first) and S (last row). The framework hands the slot out and clears it when a request starts;
the kernels read the step from its device arrays, so a decode step can be replayed from a graph. In bfloat16 a
portion of 256 tokens or more runs the recurrence in pieces of 64 tokens (the map of a piece, S -> P S + B, first; then
the states at the pieces' starts; then every piece from its start), parallel over the pieces; the 32-bit path and short
steps keep the one chain in token order.

Spec params: ``width``, ``blocks``, ``taps``, ``decay_scale``. Tensors under the prefix: ``y``, ``y.b``, ``x``, ``x.b``,
``conv`` [width, taps] (the last column weighs the current token), ``conv.b``, ``ra`` / ``ri`` [blocks, out, in],
``ra.b`` / ``ri.b`` [blocks, out], ``lam``, ``o``.
"""

from __future__ import annotations

import torch

from ..csrc import ops
from .base import Mixer, Projection, StateRequest, TensorDecl, register_part


class RecurrentGatedUnit(Mixer):
    lazy_output = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = dict(spec.params)
        self.hidden = int(spec.hidden)
        self.width, self.blocks, self.taps = int(p["width"]), int(p["blocks"]), int(p["taps"])
        self.decay = float(p.get("decay_scale", 8.0))
        if self.width <= 0 or self.blocks <= 0 or self.width % self.blocks:
            raise ValueError(f"{self.width} channels do not split into {self.blocks} equal blocks")
        if not 1 <= self.taps <= 16:
            raise ValueError(f"a convolution of {self.taps} taps is not supported (1 to 16 are)")
        self.bw = self.width // self.blocks
        self.w_in = self.w_o = None

    def _n(self, short):
        return self.spec.prefix + short

    def declare(self):
        w, h, b, bw = self.width, self.hidden, self.blocks, self.bw
        return {self._n("y"): TensorDecl((w, h)), self._n("y.b"): TensorDecl((w,), "vector"),
                self._n("x"): TensorDecl((w, h)), self._n("x.b"): TensorDecl((w,), "vector"),
                self._n("conv"): TensorDecl((w, self.taps)), self._n("conv.b"): TensorDecl((w,), "vector"),
                self._n("ra"): TensorDecl((b, bw, bw)), self._n("ra.b"): TensorDecl((b, bw), "vector"),
                self._n("ri"): TensorDecl((b, bw, bw)), self._n("ri.b"): TensorDecl((b, bw), "vector"),
                self._n("lam"): TensorDecl((w,), "vector"), self._n("o"): TensorDecl((h, w))}

    def bind(self, weights):
        g = lambda short: weights[self._n(short)]
        self.w_in = torch.cat([g("y"), g("x")], dim=0).contiguous()           # one product for both branches: [y | x]
        self.bias_y, self.bias_x = g("y.b"), g("x.b")
        self.conv_w, self.conv_b = g("conv"), g("conv.b")
        self.wa_t = g("ra").transpose(1, 2).contiguous()                        # [blocks, in, out]
        self.wi_t = g("ri").transpose(1, 2).contiguous()
        self.ba, self.bi = g("ra.b").reshape(-1).contiguous(), g("ri.b").reshape(-1).contiguous()
        self.lam, self.w_o = g("lam"), g("o")

    def named_tensors(self):
        w = self.width
        return {self._n("y"): self.w_in[:w], self._n("x"): self.w_in[w:], self._n("y.b"): self.bias_y, self._n("x.b"): self.bias_x,
                self._n("conv"): self.conv_w, self._n("conv.b"): self.conv_b, self._n("ra"): self.wa_t.transpose(1, 2),
                self._n("ri"): self.wi_t.transpose(1, 2), self._n("ra.b"): self.ba.view(self.blocks, self.bw),
                self._n("ri.b"): self.bi.view(self.blocks, self.bw), self._n("lam"): self.lam, self._n("o"): self.w_o}

    def state_request(self):
        return StateRequest((self.taps, self.width), torch.float32)

    def forward(self, x, ctx, cache, lazy_output: bool = False):
        tokens, w = x.shape[0], self.width
        xy = self.rt.buffer("rglru_xy", tokens, 2 * w)
        ops.linear(x, self.w_in, xy)
        u = self.rt.buffer("rglru_u", tokens, w, torch.float32)
        ops.rglru_conv(xy, w, self.bias_x, self.conv_w, self.conv_b, cache.state, ctx.seq_of_token[:tokens], ctx.q_start, ctx.state_slot, u)
        a = self.rt.buffer("rglru_a", tokens, w, torch.float32)
        gx = self.rt.buffer("rglru_gx", tokens, w, torch.float32)
        ops.rglru_gates(u, self.wa_t, self.wi_t, self.ba, self.bi, self.lam, self.decay, a, gx, self.blocks)
        mixed = self.rt.buffer("rglru_out", tokens, w)
        seqs = ctx.q_len.shape[0]
        if x.dtype == torch.bfloat16 and ctx.max_q_len >= ops.SCAN_PIECES_MIN_TOKENS:
            # a long portion: the recurrence in pieces of 64 tokens, parallel over the pieces
            piece = self.rt.scratch("rglru_pieces", (tokens // 64 + seqs + 1) * 2 * w)
            ops.rglru_scan_pieces(a, gx, xy, w, 0, self.bias_x, self.bias_y, cache.state, ctx.q_start, ctx.q_len, ctx.state_slot, mixed,
                                  piece, seqs, ctx.max_q_len, self.taps)
        else:
            ops.rglru_scan(a, gx, xy, w, 0, self.bias_x, self.bias_y, cache.state, ctx.q_start, ctx.q_len, ctx.state_slot, mixed,
                           seqs, self.taps)
        if lazy_output:
            return Projection(mixed, self.w_o)
        out = self.rt.buffer("mixer_out", tokens, self.hidden)
        ops.linear(mixed, self.w_o, out)
        return out


register_part("mixer", "rglru", RecurrentGatedUnit)
