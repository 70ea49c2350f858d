"""Mixers whose memory is a matrix per head, updated once a token (``csrc/kernels/linear_recurrence.cu``).

``gated_delta`` — the gated delta rule. From the layer's input h: q and k ([kv_heads, dim]) and v ([heads, vdim]) pass a
causal convolution per channel over the last ``taps`` tokens and SiLU; q and k become unit vectors per head (q also
times dim^-1/2); ``beta = sigmoid(W_b h)`` per head; a decay per head and key channel
``g = exp(-exp(A_log) softplus(W_a2 W_a1 h + dt_bias))``. Per head, with S [dim, vdim] from zero:
``S = diag(g) S; u = beta (v - S^T k); S = S + k u^T; o = S^T q``. Each head's o is normed to unit root mean square,
times a weight [vdim] shared by the heads, times ``sigmoid(W_g2 W_g1 h)``, then projected out. Head a of v reads q/k head
``a // (heads / kv_heads)``. Everything after the projections and the convolution is float32.

``wkv`` — a decayed memory read with a bonus for the current token. With h' the previous token's input, each of r, k,
v, g, w reads its own mix ``h + (h' - h) mu``; r, k, v are projections of theirs ([heads, dim]), the gate is
``silu(W_g mix_g)``, the decay ``w = exp(-exp(W_w2 tanh(W_w1 mix_w) + w0))`` per head and key channel. Per head:
``o = (S + diag(u) k v^T)^T r``, then ``S = diag(w) S + k v^T``. Each head's o is normed to unit root mean square, the
heads side by side are multiplied by a weight and the gate, then projected out.

State per request, one float32 row handed out by the cache manager and cleared when a request starts: S for every head,
then the convolution's last ``taps - 1`` inputs (``gated_delta``) or the previous token's input (``wkv``). The kernels
read the step from its device arrays, so single-token steps replay from a graph.

Sizes that config.json does not name are read off the checkpoint by the configuration class and handed over as params:
the low ranks ``decay_rank`` and ``gate_rank``.

Spec: ``num_heads``, ``num_kv_heads`` (gated_delta), ``head_dim``; params ``value_dim``, ``taps``, ``norm_eps``,
``unit_eps``, ``decay_rank``, ``gate_rank``. Tensors under the prefix — gated_delta: ``q, k, v, b, a1, a2, g1, g2, o``,
``q.conv, k.conv, v.conv`` [channels, taps] (the last column weighs the current token), ``A_log, dt_bias, norm``; wkv:
``mu.r, mu.k, mu.v, mu.g, mu.w, r, k, v, g, w1, w2, w0, u, norm, o``.
"""

from __future__ import annotations

import torch

from ..csrc import ops
from .base import Mixer, Projection, StateRequest, TensorDecl, register_part


def _pad8(n: int) -> int:
    return -(-n // 8) * 8


class GatedDeltaMixer(Mixer):
    lazy_output = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = dict(spec.params)
        self.hidden, self.H, self.G, self.D = int(spec.hidden), int(spec.num_heads), int(spec.num_kv_heads), int(spec.head_dim)
        self.DV, self.taps = int(p["value_dim"]), int(p["taps"])
        self.norm_eps, self.unit_eps = float(p.get("norm_eps", 0.0)), float(p.get("unit_eps", 1e-6))
        self.ra, self.rg = int(p.get("decay_rank", 0)), int(p.get("gate_rank", 0))
        if min(self.H, self.G, self.D, self.DV) <= 0 or self.H % self.G:
            raise ValueError(f"{self.H} heads do not group into {self.G} q/k heads")
        if self.ra <= 0 or self.rg <= 0:
            raise ValueError("the gated delta rule needs decay_rank and gate_rank (read off the checkpoint, or given in the configuration)")
        if self.D > 256 or self.DV > 256 or not 1 <= self.taps <= 16:
            raise ValueError(f"sizes not supported by the recurrence kernels: dim {self.D} (up to 256), vdim {self.DV} (up to 256), "
                             f"{self.taps} taps (1 to 16)")
        self.GD, self.HD, self.HV = self.G * self.D, self.H * self.D, self.H * self.DV
        self.C = 2 * self.GD + self.HV                       # channels that pass the convolution
        self.c_in = _pad8(self.C + self.H)                   # columns of the first product: q, k, v, beta
        self.r_pad = _pad8(self.ra + self.rg)
        self.s_floats = self.H * self.D * self.DV
        self.w_in = self.w_low = self.w_two = self.w_o = None

    def _n(self, short):
        return self.spec.prefix + short

    def declare(self):
        h = self.hidden
        return {self._n("q"): TensorDecl((self.GD, h)), self._n("k"): TensorDecl((self.GD, h)), self._n("v"): TensorDecl((self.HV, h)),
                self._n("q.conv"): TensorDecl((self.GD, self.taps), "vector"), self._n("k.conv"): TensorDecl((self.GD, self.taps), "vector"),
                self._n("v.conv"): TensorDecl((self.HV, self.taps), "vector"), self._n("b"): TensorDecl((self.H, h)),
                self._n("A_log"): TensorDecl((self.H,), "vector"), self._n("norm"): TensorDecl((self.DV,), "vector"),
                self._n("a1"): TensorDecl((self.ra, h)), self._n("a2"): TensorDecl((self.HD, self.ra)),
                self._n("dt_bias"): TensorDecl((self.HD,), "vector"), self._n("g1"): TensorDecl((self.rg, h)),
                self._n("g2"): TensorDecl((self.HV, self.rg)), self._n("o"): TensorDecl((h, self.HV))}

    def bind(self, weights):
        g = lambda short: weights[self._n(short)]
        q = g("q")
        w = torch.zeros((self.c_in, self.hidden), dtype=q.dtype, device=q.device)
        w[:self.GD], w[self.GD:2 * self.GD], w[2 * self.GD:self.C], w[self.C:self.C + self.H] = q, g("k"), g("v"), g("b")
        self.w_in = w
        low = torch.zeros((self.r_pad, self.hidden), dtype=q.dtype, device=q.device)
        low[:self.ra], low[self.ra:self.ra + self.rg] = g("a1"), g("g1")
        self.w_low = low
        # the second halves of the two low-rank products as one: rows [0, HD) read the decay's rank, rows [HD, HD + HV)
        # the gate's; the zeros add nothing
        two = torch.zeros((self.HD + self.HV, self.r_pad), dtype=q.dtype, device=q.device)
        two[:self.HD, :self.ra], two[self.HD:, self.ra:self.ra + self.rg] = g("a2"), g("g2")
        self.w_two = two
        self.conv_w = torch.cat([g("q.conv"), g("k.conv"), g("v.conv")], dim=0).contiguous()
        self.a_log, self.dt_bias, self.norm_w, self.w_o = g("A_log"), g("dt_bias"), g("norm"), g("o")

    def named_tensors(self):
        GD, C, ra, rg, HD = self.GD, self.C, self.ra, self.rg, self.HD
        return {self._n("q"): self.w_in[:GD], self._n("k"): self.w_in[GD:2 * GD], self._n("v"): self.w_in[2 * GD:C],
                self._n("b"): self.w_in[C:C + self.H], self._n("a1"): self.w_low[:ra], self._n("g1"): self.w_low[ra:ra + rg],
                self._n("a2"): self.w_two[:HD, :ra], self._n("g2"): self.w_two[HD:, ra:ra + rg], self._n("q.conv"): self.conv_w[:GD],
                self._n("k.conv"): self.conv_w[GD:2 * GD], self._n("v.conv"): self.conv_w[2 * GD:], self._n("A_log"): self.a_log,
                self._n("dt_bias"): self.dt_bias, self._n("norm"): self.norm_w, self._n("o"): self.w_o}

    def state_request(self):
        return StateRequest((self.s_floats + (self.taps - 1) * self.C,), torch.float32)

    def forward(self, x, ctx, cache, lazy_output: bool = False):
        tokens, f32 = x.shape[0], torch.float32
        state = cache.state
        proj = self.rt.buffer("delta_proj", tokens, self.c_in)
        ops.linear(x, self.w_in, proj)
        low = self.rt.buffer("delta_low", tokens, self.r_pad)
        ops.linear(x, self.w_low, low)
        two = self.rt.buffer("delta_two", tokens, self.HD + self.HV, f32)
        ops.linear(low, self.w_two, two)
        qk = self.rt.buffer("delta_qk", tokens, 2 * self.GD, f32)
        v = self.rt.buffer("delta_v", tokens, self.HV, f32)
        beta = self.rt.buffer("delta_beta", tokens, self.H, f32)
        decay = self.rt.buffer("delta_decay", tokens, self.HD, f32)
        seqs = ctx.q_len.shape[0]
        ops.delta_prepare(proj, self.conv_w, two, self.a_log, self.dt_bias, state, self.s_floats, ctx.seq_of_token[:tokens], ctx.q_start,
                          ctx.state_slot, qk, v, beta, decay, self.G, self.H, self.D, self.DV, self.taps, self.unit_eps)
        o = self.rt.buffer("delta_o", tokens, self.HV, f32)
        scratch = None
        if x.dtype == torch.bfloat16 and 0 < ops.DELTA_PIECES_MIN_TOKENS <= ctx.max_q_len:
            # a long portion in pieces, parallel over the pieces (off by default: slower than the chain at the sizes measured)
            seqs = ctx.num_seqs
            scratch = self.rt.scratch("delta_pieces", ops.delta_scan_scratch_floats(seqs, ctx.max_q_len, self.H, self.D, self.DV))
        ops.delta_scan(qk, v, beta, decay, o, state, self.s_floats, proj, ctx.q_start, ctx.q_len, ctx.state_slot, seqs, self.G, self.H,
                       self.D, self.DV, self.taps, ctx.max_q_len, scratch)
        mixed = self.rt.buffer("delta_mixed", tokens, self.HV)
        ops.head_norm_gate(o, self.norm_w, False, two, "sigmoid", mixed, self.H, self.DV, self.norm_eps, gate_off=self.HD)
        if lazy_output:
            return Projection(mixed, self.w_o)
        out = self.rt.buffer("mixer_out", tokens, self.hidden)
        ops.linear(mixed, self.w_o, out)
        return out


class BonusMemoryMixer(Mixer):
    lazy_output = True
    MIXES = "rkvgw"

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = dict(spec.params)
        self.hidden, self.H, self.D = int(spec.hidden), int(spec.num_heads), int(spec.head_dim)
        self.norm_eps = float(p.get("norm_eps", 0.0))
        self.rw = int(p.get("decay_rank", 0))
        if self.H <= 0 or self.D <= 0:
            raise ValueError("the mixer needs positive heads and dim")
        if self.rw <= 0:
            raise ValueError("the mixer needs decay_rank (read off the checkpoint, or given in the configuration)")
        if self.D > 256:
            raise ValueError(f"dim {self.D} is not supported by the recurrence kernels (up to 256 is)")
        self.HD = self.H * self.D
        self.r_pad = _pad8(self.rw)
        self.s_floats = self.H * self.D * self.D

    def _n(self, short):
        return self.spec.prefix + short

    def declare(self):
        h, HD = self.hidden, self.HD
        d = {self._n("mu." + s): TensorDecl((h,), "vector") for s in self.MIXES}
        d.update({self._n(s): TensorDecl((HD, h)) for s in "rkvg"})
        d.update({self._n("w1"): TensorDecl((self.rw, h)), self._n("w2"): TensorDecl((HD, self.rw)), self._n("w0"): TensorDecl((HD,), "vector"),
                  self._n("u"): TensorDecl((self.H, self.D), "vector"), self._n("norm"): TensorDecl((HD,), "vector"),
                  self._n("o"): TensorDecl((h, HD))})
        return d

    def bind(self, weights):
        g = lambda short: weights[self._n(short)]
        self.mu = torch.stack([g("mu." + s) for s in self.MIXES]).contiguous()
        self.w_r, self.w_k, self.w_v, self.w_g = g("r"), g("k"), g("v"), g("g")
        w1 = torch.zeros((self.r_pad, self.hidden), dtype=self.w_r.dtype, device=self.w_r.device)
        w1[:self.rw] = g("w1")
        w2 = torch.zeros((self.HD, self.r_pad), dtype=self.w_r.dtype, device=self.w_r.device)
        w2[:, :self.rw] = g("w2")
        self.w_1, self.w_2 = w1, w2
        self.w0, self.bonus, self.norm_w, self.w_o = g("w0"), g("u").reshape(-1).contiguous(), g("norm"), g("o")

    def named_tensors(self):
        out = {self._n("mu." + s): self.mu[i] for i, s in enumerate(self.MIXES)}
        out.update({self._n("r"): self.w_r, self._n("k"): self.w_k, self._n("v"): self.w_v, self._n("g"): self.w_g,
                    self._n("w1"): self.w_1[:self.rw], self._n("w2"): self.w_2[:, :self.rw], self._n("w0"): self.w0,
                    self._n("u"): self.bonus.view(self.H, self.D), self._n("norm"): self.norm_w, self._n("o"): self.w_o})
        return out

    def state_request(self):
        return StateRequest((self.s_floats + self.hidden,), torch.float32)

    def forward(self, x, ctx, cache, lazy_output: bool = False):
        tokens, f32 = x.shape[0], torch.float32
        state = cache.state
        mixes = self.rt.buffer("wkv_mixes", tokens, len(self.MIXES) * self.hidden).view(len(self.MIXES), tokens, self.hidden)
        ops.shift_mix(x, self.mu, state, self.s_floats, ctx.seq_of_token[:tokens], ctx.q_start, ctx.q_len, ctx.state_slot, mixes)
        r = self.rt.buffer("wkv_r", tokens, self.HD)
        k = self.rt.buffer("wkv_k", tokens, self.HD)
        v = self.rt.buffer("wkv_v", tokens, self.HD)
        gate = self.rt.buffer("wkv_g", tokens, self.HD)
        for out, w, i in ((r, self.w_r, 0), (k, self.w_k, 1), (v, self.w_v, 2), (gate, self.w_g, 3)):
            ops.linear(mixes[i], w, out)
        low = self.rt.buffer("wkv_low", tokens, self.r_pad)
        ops.linear(mixes[4], self.w_1, low)
        ops.tanh_(low)
        wlog = self.rt.buffer("wkv_wlog", tokens, self.HD, f32)
        ops.linear(low, self.w_2, wlog)
        o = self.rt.buffer("wkv_o", tokens, self.HD, f32)
        seqs, scratch = ctx.q_len.shape[0], None
        if x.dtype == torch.bfloat16 and ctx.max_q_len >= ops.SCAN_PIECES_MIN_TOKENS:
            # a long portion: the recurrence in pieces, parallel over the pieces (the 32-bit path keeps the one chain, whose
            # sums do not depend on the cutting)
            seqs = ctx.num_seqs
            scratch = self.rt.scratch("wkv_pieces", ops.bonus_scan_scratch_floats(seqs, ctx.max_q_len, self.H, self.D))
        ops.bonus_scan(r, k, v, wlog, self.w0, self.bonus, o, state, ctx.q_start, ctx.q_len, ctx.state_slot, seqs, self.H, self.D,
                       ctx.max_q_len, scratch)
        mixed = self.rt.buffer("wkv_mixed", tokens, self.HD)
        ops.head_norm_gate(o, self.norm_w, True, gate, "silu", mixed, self.H, self.D, self.norm_eps)
        if lazy_output:
            return Projection(mixed, self.w_o)
        out = self.rt.buffer("mixer_out", tokens, self.hidden)
        ops.linear(mixed, self.w_o, out)
        return out


register_part("mixer", "gated_delta", GatedDeltaMixer)
register_part("mixer", "wkv", BonusMemoryMixer)
