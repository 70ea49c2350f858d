"""Typed configuration of the Nidilix decoder.

config.json gives ``vocab``, ``width``, ``residual_mult``, ``norm.eps``, ``token_side.dim`` and a list ``layers``;
each entry names its mixer (``type``: ``rglru`` or ``latent_attention``), the mixer's sizes (``mixer``) and its
feed-forward (``mlp``: a routed mixture with an optional shared expert, or null). Nothing else is read, and no size
stands in code. The architecture is laid out from the package's parts:

* norms are Dynamic Tanh (``dyt``), tensors ``<name>``, ``<name>.b``, ``<name>.alpha``;
* ``latent_attention`` keeps one latent vector and one rotated key part per token in pages; a layer whose mixer
  gives ``kv_from: j`` runs on layer j's cache slot without writing it;
* ``rglru`` keeps its recurrent state and the last inputs of its convolution in a state slot;
* the feed-forward is ``routed_experts``;
* after the feed-forward a ``token_side`` input adds a gated slice of a second embedding;
* every sum into the stream is scaled by ``residual_mult``.

The design names no longest sequence; ``max_positions`` only sizes the rotation table and is grown on demand
(``with_max_positions``).
"""

from __future__ import annotations

import copy
import json
from dataclasses import dataclass, field

from .registry import ConfigError, register_architecture
from .specs import (FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec, ScheduleEntry,
                    StreamInputSpec)

MIXERS = ("rglru", "latent_attention")
DEFAULT_MAX_POSITIONS = 32768


def _int(d: dict, key: str, where: str, minimum: int = 1) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v < minimum:
        raise ConfigError(f"{where}: `{key}` must be an integer >= {minimum}, got {v!r}")
    return v


def _num(d: dict, key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"{where}: `{key}` must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class NidilixConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    side_dim: int                           # 0: no per-layer token input
    layers_json: str                        # the ``layers`` list as canonical JSON (keeps the record hashable)
    max_position_embeddings: int = DEFAULT_MAX_POSITIONS
    extra: dict = field(default_factory=dict, compare=False)

    @property
    def layers(self) -> list:
        return json.loads(self.layers_json)

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: dict) -> "NidilixConfig":
        for key in ("vocab", "width", "layers", "norm", "residual_mult"):
            if key not in d:
                raise ConfigError(f"config.json is missing `{key}`")
        if not isinstance(d["norm"], dict):
            raise ConfigError("`norm` must be an object with `eps`")
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError("`layers` must be a list with at least one layer")
        side = d.get("token_side")
        if side is not None and not isinstance(side, dict):
            raise ConfigError("`token_side` must be an object with `dim`, or absent")
        cfg = cls(vocab=_int(d, "vocab", "config.json"), width=_int(d, "width", "config.json"),
                  norm_eps=_num(d["norm"], "eps", "norm"), residual_mult=_num(d, "residual_mult", "config.json"),
                  side_dim=_int(side, "dim", "token_side") if side else 0,
                  layers_json=json.dumps(d["layers"], sort_keys=True),
                  max_position_embeddings=int(d.get("max_positions", DEFAULT_MAX_POSITIONS)),
                  extra={k: v for k, v in d.items() if k not in ("architecture", "architectures", "vocab", "width", "layers", "norm",
                                                                  "residual_mult", "token_side", "max_positions")})
        cfg.validate()
        return cfg

    def validate(self) -> None:
        layers = self.layers
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or layer.get("type") not in MIXERS:
                raise ConfigError(f"{where}: `type` must be one of {MIXERS}, got {layer.get('type') if isinstance(layer, dict) else layer!r}")
            m = layer.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"{where}: `mixer` must be an object")
            if layer["type"] == "rglru":
                width, blocks = _int(m, "width", where), _int(m, "blocks", where)
                _int(m, "conv", where)
                if width % blocks:
                    raise ConfigError(f"{where}: width {width} does not split into {blocks} equal blocks")
            else:
                for key in ("heads", "dim", "vdim", "kv_rank"):
                    _int(m, key, where)
                rot_dim = _int(m, "rot_dim", where, minimum=0)
                _num(m, "scale", where)
                rot = m.get("rot")
                if not isinstance(rot, dict):
                    raise ConfigError(f"{where}: `rot` must be an object with `base` and `dims`")
                dims = _int(rot, "dims", where + ".rot", minimum=0)
                if dims % 2 or dims > rot_dim or not _num(rot, "base", where + ".rot") > 0:
                    raise ConfigError(f"{where}: rot.dims must be even and at most rot_dim, rot.base positive")
                source = m.get("kv_from")
                if source is not None:
                    if isinstance(source, bool) or not isinstance(source, int) or not 0 <= source < i:
                        raise ConfigError(f"{where}: kv_from must name an earlier layer, got {source!r}")
                    other = layers[source]
                    om = other.get("mixer", {})
                    if other.get("type") != "latent_attention" or om.get("kv_from") is not None:
                        raise ConfigError(f"{where}: kv_from {source} must name a latent_attention layer with a cache of its own")
                    if (om.get("kv_rank"), om.get("rot_dim"), om.get("rot")) != (m["kv_rank"], m["rot_dim"], m["rot"]):
                        raise ConfigError(f"{where}: kv_rank, rot_dim and rot must equal those of layer {source}")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind", "moe") != "moe":
                raise ConfigError(f"{where}: `mlp` must be a routed mixture (kind 'moe') or null")
            router = mlp.get("router")
            if not isinstance(router, dict) or not isinstance(mlp.get("expert"), dict):
                raise ConfigError(f"{where}: mlp needs `router` and `expert`")
            experts, top = _int(router, "experts", where + ".mlp.router"), _int(router, "top", where + ".mlp.router")
            if top > experts:
                raise ConfigError(f"{where}: top {top} exceeds the {experts} experts")
            _int(mlp["expert"], "ff", where + ".mlp.expert")
            if mlp.get("shared") is not None:
                _int(mlp["shared"], "ff", where + ".mlp.shared")
        if not self.norm_eps >= 0:
            raise ConfigError("norm.eps must not be negative")

    def to_dict(self) -> dict:
        d = {"architecture": "Nidilix", "layers": self.layers, "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult,
             "vocab": self.vocab, "width": self.width}
        if self.side_dim:
            d["token_side"] = {"dim": self.side_dim}
        if self.max_position_embeddings != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_position_embeddings
        d.update(copy.deepcopy(self.extra))
        return d

    def with_max_positions(self, count: int) -> "NidilixConfig":
        import dataclasses
        return dataclasses.replace(self, max_position_embeddings=int(count))

    # ------------------------------------------------------------------- layout
    def _norm(self, name: str) -> NormSpec:
        return NormSpec(kind="dyt", width=self.width, eps=self.norm_eps, prefix=name)

    def to_model_spec(self) -> ModelSpec:
        layers, schedule = [], []
        count = len(self.layers)
        for i, layer in enumerate(self.layers):
            m, p = layer["mixer"], f"l{i}."
            cache = i
            if layer["type"] == "rglru":
                mixer = MixerSpec(kind="rglru", hidden=self.width, prefix=p + "mix.",
                                  params=(("width", m["width"]), ("blocks", m["blocks"]), ("taps", m["conv"]),
                                          ("decay_scale", 8.0)))
            else:
                position = PositionSpec(kind="rope", head_dim=m["rot"]["dims"], theta=float(m["rot"]["base"]),
                                        max_positions=self.max_position_embeddings, params=(("angles", "float64"),))
                source = m.get("kv_from")
                if source is not None:
                    cache = source
                mixer = MixerSpec(kind="latent_attention", hidden=self.width, num_heads=m["heads"], head_dim=m["dim"],
                                  scale=float(m["scale"]), position=position, prefix=p + "mix.",
                                  params=(("rot_dim", m["rot_dim"]), ("value_dim", m["vdim"]), ("kv_rank", m["kv_rank"]),
                                          ("latent_eps", self.norm_eps), ("own_latent", source is None), ("output_gate", True)))
            mlp = layer.get("mlp")
            ffn = None
            if mlp is not None:
                shared = mlp.get("shared")
                ffn = FeedForwardSpec(kind="routed_experts", hidden=self.width, intermediate=mlp["expert"]["ff"],
                                      activation="relu_squared", prefix=p + "mlp.",
                                      params=(("experts", mlp["router"]["experts"]), ("top", mlp["router"]["top"]),
                                              ("shared", shared["ff"] if shared else 0), ("router_bias", True)))
            after = ()
            if self.side_dim:
                after = (StreamInputSpec(kind="token_side", hidden=self.width, vocab=self.vocab, dim=self.side_dim,
                                         offset=i * self.side_dim, table_width=count * self.side_dim, table_name="side.embed",
                                         eps=self.norm_eps, prefix=p + "side."),)
            layers.append(LayerSpec(kind="pre_norm", mixer=mixer, feed_forward=ffn, mixer_norm=self._norm(p + "norm1"),
                                    ffn_norm=self._norm(p + "norm2") if ffn is not None else None,
                                    residual_mult=self.residual_mult, after=after))
            schedule.append(ScheduleEntry(layer=i, cache=cache, writes_cache=cache == i))
        return ModelSpec(architecture="Nidilix", hidden=self.width, vocab=self.vocab, layers=tuple(layers),
                         schedule=tuple(schedule), final_norm=self._norm("final.norm"), embed_name="embed", head_name="head",
                         max_positions=self.max_position_embeddings, extra=self)


register_architecture("Nidilix", NidilixConfig)
