"""Rotary position encoding with optional llama3 frequency rescaling.

The table is built once per distinct spec, in float32, as the reference builds it
(python/stride_worker/layers.py:38-82): inv_freq = theta^(-2j/hd); with llama3
scaling, wavelengths above original/low are divided by ``factor``, those between
original/high and original/low are interpolated, the rest stay; angle =
position * inv_freq. Only the half table [max_positions, hd/2] is kept, since the
reference's full table repeats it. The rotation itself and the write of keys and
values into pages are one kernel (``rope_kv_write``); angles, products and sums
are float32 in both modes.

Other forms of the same rotation, chosen by spec params and all served by the same tables and kernels:

* ``rotated`` r < head_dim: only the first r entries of a head turn. The table then holds cos 1 and sin 0 for the
  pairs that pass unchanged.
* ``pairing`` ``neighbours``: entry 2i turns with entry 2i+1 (the kernels pair entry i with entry i + head_dim/2).
  A score does not change when queries and keys are permuted alike inside a head, so the part offers
  ``head_permutation()``: the order in which a mixer lays out the rows of its query and key projections at load so that
  the kernels' pairing is the wanted one. Position n of the new order holds the old entry ``perm[n]``.
* scaling ``yarn`` (Peng et al., "YaRN: Efficient Context Window Extension of Large Language Models"): pair i's
  frequency f_i goes over from kept to ``f_i / factor`` along a ramp between the pair whose wave makes
  ``high_freq_factor`` turns over the original length and the one that makes ``low_freq_factor`` turns, and cos and sin
  are multiplied by ``0.1 ln(factor) + 1``.
"""

from __future__ import annotations

import math

import torch

from ..csrc import ops
from .base import PositionEncoding, register_part


def rope_inverse_frequencies(head_dim: int, theta: float, scaling) -> torch.Tensor:
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    if scaling is not None and scaling.rope_type == "llama3":
        original = scaling.original_max_position_embeddings
        wavelength = 2 * math.pi / inv_freq
        low_wavelength = original / scaling.low_freq_factor
        high_wavelength = original / scaling.high_freq_factor
        scaled = inv_freq / scaling.factor
        smooth = ((original / wavelength - scaling.low_freq_factor) /
                  (scaling.high_freq_factor - scaling.low_freq_factor)).clamp(0.0, 1.0)
        blended = (1 - smooth) * scaled + smooth * inv_freq
        inv_freq = torch.where(wavelength > low_wavelength, scaled, inv_freq)
        inv_freq = torch.where((wavelength <= low_wavelength) & (wavelength >= high_wavelength), blended, inv_freq)
    return inv_freq


def yarn_frequencies(dims: int, theta: float, scaling):
    """float64 frequencies [dims / 2] and the factor on cos and sin."""
    i = torch.arange(0, dims // 2, dtype=torch.float64)
    f = float(theta) ** (-2.0 * i / max(dims, 1))

    def pair_of(turns: float) -> float:      # the (fractional) pair whose wave makes `turns` turns over the original length
        return dims * math.log(scaling.original_max_position_embeddings / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

    lo = max(math.floor(pair_of(scaling.high_freq_factor)), 0)
    hi = min(math.ceil(pair_of(scaling.low_freq_factor)), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / scaling.factor * ramp + f * (1.0 - ramp), 0.1 * math.log(scaling.factor) + 1.0


class RotaryEncoding(PositionEncoding):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if spec.head_dim % 2:
            raise ValueError(f"rotary encoding needs an even head_dim, got {spec.head_dim}")
        p = dict(spec.params)
        self.rotated = int(p.get("rotated", spec.head_dim))
        self.pairing = p.get("pairing", "halves")
        if self.rotated % 2 or not 0 <= self.rotated <= spec.head_dim or self.pairing not in ("halves", "neighbours"):
            raise ValueError(f"cannot turn {self.rotated} of {spec.head_dim} entries with the pairing {self.pairing!r}")
        self.general = self.rotated != spec.head_dim or self.pairing != "halves" or (spec.scaling is not None and spec.scaling.rope_type == "yarn")
        self.max_positions = int(spec.max_positions)
        self._tables = None

    def head_permutation(self):
        """None when the kernels' pairing (i with i + head_dim/2, every entry turned) is the wanted one. Otherwise the
        order of a head's entries under which it is: turned pair i at (i, i + head_dim/2), the entries that pass
        unchanged behind the turned ones in both halves."""
        hd, r = self.spec.head_dim, self.rotated
        if not self.general or (self.pairing == "halves" and r == hd):
            return None
        half = hd // 2
        if self.pairing == "neighbours":
            first, second = list(range(0, r, 2)), list(range(1, r, 2))
        else:
            first, second = list(range(0, r // 2)), list(range(r // 2, r))
        rest = list(range(r, hd))
        fill = half - r // 2
        return first + rest[:fill] + second + rest[fill:]

    def _build_general(self):
        """Tables in the kernels' layout [max_positions, head_dim / 2] for a partial rotation, YaRN or both: angles in
        float64, rounded once; pairs that pass unchanged get cos 1 and sin 0."""
        hd, r, sc = self.spec.head_dim, self.rotated, self.spec.scaling
        if sc is not None and sc.rope_type == "yarn":
            f, magnitude = yarn_frequencies(r, self.spec.theta, sc)
        elif sc is not None:
            raise ValueError(f"rope scaling {sc.rope_type!r} is not available for a partial or neighbour-paired rotation")
        else:
            f, magnitude = float(self.spec.theta) ** (-torch.arange(0, r, 2, dtype=torch.float64) / max(r, 1)), 1.0
        angles = torch.outer(torch.arange(self.max_positions, dtype=torch.float64), f)
        cos = torch.ones((self.max_positions, hd // 2), dtype=torch.float32)
        sin = torch.zeros((self.max_positions, hd // 2), dtype=torch.float32)
        cos[:, :r // 2] = (angles.cos() * magnitude).float()
        sin[:, :r // 2] = (angles.sin() * magnitude).float()
        return cos.to(self.rt.device), sin.to(self.rt.device)

    def _build(self):
        if self.general:
            return self._build_general()
        if dict(self.spec.params).get("angles") == "float64":
            # angle = position * theta^(-2i/dims) formed in float64 and rounded once, to float32 tables: at position
            # p a float32 product would be off by up to p * 2^-24 radians
            exponent = torch.arange(0, self.spec.head_dim, 2, dtype=torch.float64) / max(self.spec.head_dim, 1)
            angles = torch.outer(torch.arange(self.max_positions, dtype=torch.float64), float(self.spec.theta) ** -exponent)
            return angles.cos().float().to(self.rt.device), angles.sin().float().to(self.rt.device)
        inv_freq = rope_inverse_frequencies(self.spec.head_dim, self.spec.theta, self.spec.scaling)
        angles = torch.outer(torch.arange(self.max_positions, dtype=torch.float32), inv_freq)
        return angles.cos().to(self.rt.device), angles.sin().to(self.rt.device)

    def tables(self):
        """(cos, sin), each float32 [max_positions, head_dim / 2]; one pair per distinct spec."""
        if self._tables is None:
            self._tables = self.rt.shared(("rope", self.spec), self._build)
        return self._tables

    def rotation_tables(self):
        cos, sin = self.tables()
        return cos, sin, True

    def encode_and_store(self, qkv, bias, ctx, cache, num_heads, num_kv_heads, head_dim):
        cos, sin = self.tables()
        ops.rope_kv_write(qkv, bias, ctx.positions[:qkv.shape[0]],
                          ctx.slot_mapping[cache.group][:qkv.shape[0]] if cache.writes else None,
                          cos, sin, cache.k_pages, cache.v_pages, num_heads, num_kv_heads, head_dim,
                          cache.page_size, rotate=True)


class NoPositionEncoding(PositionEncoding):
    """Keys and queries stay as they are; keys and values are still stored."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.max_positions = int(spec.max_positions) if spec.max_positions else 1
        self._dummy = runtime.shared(("rope-dummy",), lambda: torch.zeros(8, dtype=torch.float32, device=runtime.device))

    def rotation_tables(self):
        return self._dummy, self._dummy, False

    def encode_and_store(self, qkv, bias, ctx, cache, num_heads, num_kv_heads, head_dim):
        ops.rope_kv_write(qkv, bias, ctx.positions[:qkv.shape[0]],
                          ctx.slot_mapping[cache.group][:qkv.shape[0]] if cache.writes else None,
                          self._dummy, self._dummy, cache.k_pages, cache.v_pages, num_heads, num_kv_heads, head_dim,
                          cache.page_size, rotate=False)


register_part("position", "rope", RotaryEncoding)
register_part("position", "none", NoPositionEncoding)
