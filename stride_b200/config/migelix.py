"""Typed configuration of the Migelix decoder.

config.json gives ``vocab``, ``width``, ``norm.eps``, optionally ``logit_softcap``, and a list ``layers``; each entry
names its mixer (``type``: ``parallel``, ``wkv`` or ``attention``), the mixer's sizes and constants (``mixer``), its
feed-forward (``mlp``: a dense gated one, or null) and optionally ``weights_of: j``, which makes the entry a second
run of layer j's tensors with a cache and state of its own. Nothing else is read, and no size stands in code. The
architecture is laid out from the package's parts:

* norms are ``rmsnorm`` whose factor is one plus the stored weight (``weight_offset`` 1);
* ``attention`` is the paged attention part with the values taken from the keys before their rotation, a window, and per
  layer a cap on the scores, a gate on the output, biases or a sink in the softmax; its rotation turns neighbouring
  pairs of the first ``rot.dims`` entries of a head, with optional YaRN rescaling of the frequencies;
* ``parallel`` runs two mixers on the same input and adds their outputs with a weight each: such an attention beside a
  ``gated_delta`` recurrence;
* ``wkv`` is a decaying outer-product memory read with a bonus for the current token, fed by token-shifted inputs;
* the feed-forward is ``swiglu`` with the tanh form of GELU;
* the head shares the embedding table and caps its logits.

Two sizes appear in no key of the design's config.json: the inner widths of the low-rank products of the recurrent
mixers. They are read off the checkpoint's shapes (``complete_from_checkpoint``) and kept as ``decay_rank`` /
``gate_rank`` in the mixer's entry, where a configuration made by hand (a random model) gives them directly.

The design names no longest sequence; ``max_positions`` only sizes the rotation tables and is grown on demand
(``with_max_positions``).
"""

from __future__ import annotations

import copy
import json
from dataclasses import dataclass, field

from .registry import ConfigError, register_architecture
from .specs import (FeedForwardSpec, HeadSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec, RopeScaling,
                    ScheduleEntry)

MIXERS = ("parallel", "wkv", "attention")
DEFAULT_MAX_POSITIONS = 32768
_KNOWN = ("architecture", "architectures", "vocab", "width", "layers", "norm", "logit_softcap", "max_positions")


def _int(d: dict, key: str, where: str, minimum: int = 1) -> int:
    v = d.get(key) if isinstance(d, dict) else None
    if isinstance(v, bool) or not isinstance(v, int) or v < minimum:
        raise ConfigError(f"{where}: `{key}` must be an integer >= {minimum}, got {v!r}")
    return v


def _num(d: dict, key: str, where: str) -> float:
    v = d.get(key) if isinstance(d, dict) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"{where}: `{key}` must be a number, got {v!r}")
    return float(v)


def _check_attention(m: dict, where: str) -> None:
    heads, kv = _int(m, "heads", where), _int(m, "kv_heads", where)
    dim, vdim = _int(m, "dim", where), _int(m, "vdim", where)
    if heads % kv:
        raise ConfigError(f"{where}: {heads} heads do not group into {kv} kv_heads")
    if vdim != dim:
        raise ConfigError(f"{where}: the values are the keys, so vdim {vdim} must equal dim {dim}")
    _num(m, "scale", where)
    if m.get("softcap") is not None and not _num(m, "softcap", where) > 0:
        raise ConfigError(f"{where}: softcap must be positive")
    if m.get("mask") is not None:
        _int(m["mask"], "size", where + ".mask")
    rot = m.get("rot")
    if not isinstance(rot, dict):
        raise ConfigError(f"{where}: `rot` must be an object with `base` and `dims`")
    dims = _int(rot, "dims", where + ".rot", minimum=0)
    if dims % 2 or dims > dim or not _num(rot, "base", where + ".rot") > 0:
        raise ConfigError(f"{where}: rot.dims must be even and at most dim, rot.base positive")
    sc = rot.get("scaling")
    if sc is not None:
        for key in ("factor", "original", "fast", "slow"):
            if not _num(sc, key, where + ".rot.scaling") > 0:
                raise ConfigError(f"{where}.rot.scaling: `{key}` must be positive")


def _check_delta(m: dict, where: str) -> None:
    heads, kv = _int(m, "heads", where), _int(m, "kv_heads", where)
    if heads % kv:
        raise ConfigError(f"{where}: {heads} heads do not group into {kv} kv_heads")
    for key in ("dim", "vdim", "conv"):
        _int(m, key, where)
    for key in ("decay_rank", "gate_rank"):
        if key in m:
            _int(m, key, where)


@dataclass(frozen=True)
class MigelixConfig:
    vocab: int
    width: int
    norm_eps: float
    logit_softcap: float                    # 0: the logits are not capped
    layers_json: str                        # the ``layers`` list as canonical JSON (keeps the record hashable)
    max_position_embeddings: int = DEFAULT_MAX_POSITIONS
    extra: dict = field(default_factory=dict, compare=False)

    @property
    def layers(self) -> list:
        return json.loads(self.layers_json)

    # ------------------------------------------------------------------ reading
    @staticmethod
    def complete_from_checkpoint(d: dict, tensor_names: set, tensor_shapes: dict | None = None) -> dict:
        """Fills in the low ranks from the shapes of ``a1`` / ``g1`` / ``w1`` where the entry does not give them."""
        if not tensor_shapes or not isinstance(d.get("layers"), list):
            return d
        d = copy.deepcopy(d)
        layers = d["layers"]

        def rank(name):
            shape = tensor_shapes.get(name)
            return int(shape[0]) if shape else None

        for i, layer in enumerate(layers):
            if not isinstance(layer, dict) or not isinstance(layer.get("mixer"), dict):
                continue
            source = layer.get("weights_of")
            p = f"l{source if isinstance(source, int) and not isinstance(source, bool) else i}.mix."
            m = layer["mixer"]
            if layer.get("type") == "parallel" and isinstance(m.get("right"), dict):
                for key, tensor in (("decay_rank", "right.a1"), ("gate_rank", "right.g1")):
                    if key not in m["right"] and rank(p + tensor):
                        m["right"][key] = rank(p + tensor)
            elif layer.get("type") == "wkv" and "decay_rank" not in m and rank(p + "w1"):
                m["decay_rank"] = rank(p + "w1")
        return d

    @classmethod
    def from_dict(cls, d: dict) -> "MigelixConfig":
        for key in ("vocab", "width", "layers", "norm"):
            if key not in d:
                raise ConfigError(f"config.json is missing `{key}`")
        if not isinstance(d["norm"], dict):
            raise ConfigError("`norm` must be an object with `eps`")
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError("`layers` must be a list with at least one layer")
        cap = d.get("logit_softcap")
        cfg = cls(vocab=_int(d, "vocab", "config.json"), width=_int(d, "width", "config.json"),
                  norm_eps=_num(d["norm"], "eps", "norm"), logit_softcap=_num(d, "logit_softcap", "config.json") if cap is not None else 0.0,
                  layers_json=json.dumps(d["layers"], sort_keys=True),
                  max_position_embeddings=int(d.get("max_positions", DEFAULT_MAX_POSITIONS)),
                  extra={k: v for k, v in d.items() if k not in _KNOWN})
        cfg.validate()
        return cfg

    def validate(self) -> None:
        layers = self.layers
        if not self.norm_eps >= 0 or self.logit_softcap < 0:
            raise ConfigError("norm.eps and logit_softcap must not be negative")
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or layer.get("type") not in MIXERS:
                raise ConfigError(f"{where}: `type` must be one of {MIXERS}, got {layer.get('type') if isinstance(layer, dict) else layer!r}")
            m = layer.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"{where}: `mixer` must be an object")
            if layer["type"] == "parallel":
                if not isinstance(m.get("left"), dict) or not isinstance(m.get("right"), dict):
                    raise ConfigError(f"{where}: a parallel mixer needs `left` and `right`")
                _check_attention(m["left"], where + ".left")
                _check_delta(m["right"], where + ".right")
                _num(m, "left_scale", where), _num(m, "right_scale", where)
            elif layer["type"] == "wkv":
                _int(m, "heads", where), _int(m, "dim", where)
                if "decay_rank" in m:
                    _int(m, "decay_rank", where)
            else:
                _check_attention(m, where)
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"{where}: `mlp` must be a dense feed-forward (kind 'dense') or null")
                _int(mlp, "ff", where + ".mlp")
            source = layer.get("weights_of")
            if source is not None:
                if isinstance(source, bool) or not isinstance(source, int) or not 0 <= source < len(layers) or source == i:
                    raise ConfigError(f"{where}: weights_of must name another layer, got {source!r}")
                other = layers[source]
                if not isinstance(other, dict) or other.get("weights_of") is not None:
                    raise ConfigError(f"{where}: weights_of {source} must name a layer with tensors of its own")
                if any(other.get(k) != layer.get(k) for k in ("type", "mixer", "mlp")):
                    raise ConfigError(f"{where}: type, mixer and mlp must equal those of layer {source}")

    def to_dict(self) -> dict:
        d = {"architecture": "Migelix", "layers": self.layers, "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.logit_softcap:
            d["logit_softcap"] = self.logit_softcap
        if self.max_position_embeddings != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_position_embeddings
        d.update(copy.deepcopy(self.extra))
        return d

    def with_max_positions(self, count: int) -> "MigelixConfig":
        import dataclasses
        return dataclasses.replace(self, max_position_embeddings=int(count))

    # ------------------------------------------------------------------- layout
    def _norm(self, name: str) -> NormSpec:
        return NormSpec(kind="rmsnorm", width=self.width, eps=self.norm_eps, prefix=name,
                        params=(("tensor", name), ("weight_offset", 1.0)))

    def _attention(self, m: dict, prefix: str, *, bias: bool, sinks: bool, gate: bool) -> MixerSpec:
        rot = m["rot"]
        sc = rot.get("scaling")
        scaling = None
        if sc:
            # YaRN: `fast` and `slow` are the numbers of turns over the original length between which the
            # frequencies go over from kept to divided by `factor`
            scaling = RopeScaling(rope_type="yarn", factor=float(sc["factor"]), low_freq_factor=float(sc["slow"]),
                                  high_freq_factor=float(sc["fast"]), original_max_position_embeddings=int(sc["original"]))
        position = PositionSpec(kind="rope", head_dim=m["dim"], theta=float(rot["base"]), max_positions=self.max_position_embeddings,
                                scaling=scaling, params=(("angles", "float64"), ("pairing", "neighbours"), ("rotated", int(rot["dims"]))))
        params = [("values", "keys"), ("names", "short")]
        if m.get("softcap"):
            params.append(("softcap", float(m["softcap"])))
        if sinks:
            params.append(("sinks", True))
        if gate:
            params.append(("output_gate", True))
        return MixerSpec(kind="attention", hidden=self.width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"],
                         scale=float(m["scale"]), window=int(m["mask"]["size"]) if m.get("mask") else None, bias=bias,
                         position=position, prefix=prefix, params=tuple(params))

    def _mixer(self, layer: dict, prefix: str) -> MixerSpec:
        m = layer["mixer"]
        if layer["type"] == "attention":
            return self._attention(m, prefix, bias=False, sinks=False, gate=True)
        if layer["type"] == "wkv":
            return MixerSpec(kind="wkv", hidden=self.width, num_heads=m["heads"], head_dim=m["dim"], prefix=prefix,
                             params=(("norm_eps", self.norm_eps), ("decay_rank", int(m.get("decay_rank", 0)))))
        left = self._attention(m["left"], prefix + "left.", bias=True, sinks=True, gate=False)
        r = m["right"]
        right = MixerSpec(kind="gated_delta", hidden=self.width, num_heads=r["heads"], num_kv_heads=r["kv_heads"], head_dim=r["dim"],
                          prefix=prefix + "right.", params=(("value_dim", r["vdim"]), ("taps", r["conv"]), ("norm_eps", self.norm_eps),
                                                            ("unit_eps", 1e-6),
                                                            ("decay_rank", int(r.get("decay_rank", 0))), ("gate_rank", int(r.get("gate_rank", 0)))))
        return MixerSpec(kind="parallel", hidden=self.width, prefix=prefix,
                         params=(("branches", ((left, float(m["left_scale"])), (right, float(m["right_scale"])))),))

    def to_model_spec(self) -> ModelSpec:
        layers, index_of, schedule = [], {}, []
        for i, layer in enumerate(self.layers):
            if layer.get("weights_of") is not None:
                continue
            p = f"l{i}."
            mlp = layer.get("mlp")
            ffn = None
            if mlp is not None:
                ffn = FeedForwardSpec(kind="swiglu", hidden=self.width, intermediate=mlp["ff"], activation="gelu_tanh", prefix=p + "mlp.",
                                      params=(("names", "short"),))
            index_of[i] = len(layers)
            layers.append(LayerSpec(kind="pre_norm", mixer=self._mixer(layer, p + "mix."), feed_forward=ffn, mixer_norm=self._norm(p + "norm1"),
                                    ffn_norm=self._norm(p + "norm2") if ffn is not None else None))
        for i, layer in enumerate(self.layers):
            source = layer.get("weights_of")
            schedule.append(ScheduleEntry(layer=index_of[i if source is None else source], cache=i))
        head = HeadSpec("linear", self.vocab, self.width, None, params=(("softcap", self.logit_softcap),) if self.logit_softcap else ())
        return ModelSpec(architecture="Migelix", hidden=self.width, vocab=self.vocab, layers=tuple(layers), schedule=tuple(schedule),
                         final_norm=self._norm("final.norm"), embed_name="embed", head_name=None,
                         max_positions=self.max_position_embeddings, extra=self, head=head)


register_architecture("Migelix", MigelixConfig)
