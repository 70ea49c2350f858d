"""Small Nidilix configurations and seeded weights for the tests. Nothing here imports the product package."""

from __future__ import annotations

import math

import torch


def attention(heads, dim, rot_dim, rot_dims, vdim, rank, base=10000.0, kv_from=None, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "rot": {"base": base, "dims": rot_dims},
         "scale": scale if scale is not None else 1.0 / math.sqrt(dim + rot_dim)}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def recurrent(width, blocks, taps):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": taps}}


def moe(experts, top, ff, shared=None):
    d = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        d["shared"] = {"ff": shared}
    return d


def config(width, vocab, layers, mult=0.5, eps=1e-6, side=None):
    """``layers``: list of (mixer entry, mlp or None)."""
    d = {"architecture": "Nidilix", "width": width, "vocab": vocab, "residual_mult": mult, "norm": {"eps": eps},
         "layers": [dict(m, mlp=mlp) for m, mlp in layers]}
    if side:
        d["token_side"] = {"dim": side}
    return d


# Sizes unlike one another: odd head counts, rotated entries fewer than the rotated part, one block, one tap, a
# router that takes every expert, no shared expert, no feed-forward, no token input, a borrowed cache in the middle.
CASE_A = config(96, 211, [
    (recurrent(120, 3, 4), moe(5, 2, 40, shared=24)),
    (attention(3, 16, 8, 8, 24, 40, base=50000.0), moe(5, 2, 40, shared=24)),
    (recurrent(120, 3, 4), None),
    (attention(3, 16, 8, 8, 24, 40, base=50000.0, kv_from=1), moe(5, 2, 40, shared=24)),
], mult=0.5, eps=1e-6, side=12)

CASE_B = config(80, 157, [
    (attention(5, 8, 12, 6, 8, 24, base=300.0), moe(3, 3, 56)),            # every expert chosen; 6 of 12 entries rotated
    (attention(2, 24, 4, 4, 40, 56, base=1e6), None),                       # a second cache of another shape
    (recurrent(80, 1, 1), moe(7, 1, 16, shared=48)),                        # one block, one tap, top 1
    (attention(5, 8, 12, 6, 8, 24, base=300.0, kv_from=0), moe(3, 1, 56)),
    (recurrent(64, 8, 7), moe(4, 2, 32)),
], mult=1.0, eps=1e-5, side=None)

CASE_C = config(64, 97, [
    (attention(1, 32, 16, 16, 16, 32), moe(2, 1, 24, shared=8)),            # a single head
    (recurrent(96, 2, 2), moe(2, 1, 24, shared=8)),
], mult=0.25, eps=1e-4, side=4)

# Latent widths in multiples of 16 (the sizes the tensor-core attention kernel takes in bfloat16), with head counts that
# do not fill its tiles of 16 rows evenly.
CASE_D = config(128, 263, [
    (attention(6, 48, 16, 16, 24, 80, base=100000.0), moe(8, 2, 48, shared=32)),
    (recurrent(160, 5, 3), moe(8, 2, 48, shared=32)),
    (attention(6, 48, 16, 16, 24, 80, base=100000.0, kv_from=0), None),
    (attention(20, 16, 32, 32, 16, 128, base=10000.0), moe(8, 2, 48)),
], mult=0.6, eps=2e-6, side=24)

# Sizes that are multiples of 2 only: rows of 16-bit numbers that start off a 16-byte boundary, so every vector path has
# to step aside.
CASE_E = config(100, 103, [
    (recurrent(60, 3, 2), moe(3, 2, 36, shared=18)),
    (attention(3, 10, 6, 4, 14, 20, base=4000.0), moe(3, 2, 36, shared=18)),
    (attention(3, 10, 6, 4, 14, 20, base=4000.0), None),                    # a second cache of the same shape: one group, two slots
    (attention(3, 10, 6, 4, 14, 20, base=4000.0, kv_from=1), moe(3, 2, 36)),
], mult=0.8, eps=1e-6, side=6)

CASES = {"A": CASE_A, "B": CASE_B, "C": CASE_C, "D": CASE_D, "E": CASE_E}


def seeded_state(cfg: dict, seed: int, sharp: float = 1.0, router_gain: float = 4.0) -> dict:
    """float32 weights by checkpoint name. Matrices N(0, 1/in); ``sharp`` multiplies the query projections so that the
    softmax settles on few keys, wherever they lie; ``router_gain`` spreads the router's logits."""
    g = torch.Generator().manual_seed(seed)
    width, vocab = cfg["width"], cfg["vocab"]

    def mat(rows, cols, gain=1.0):
        return torch.randn(rows, cols, generator=g) * (gain / math.sqrt(cols))

    def vec(n, mean=0.0, std=0.3):
        return mean + std * torch.randn(n, generator=g)

    s = {"embed": torch.randn(vocab, width, generator=g), "head": mat(vocab, width)}

    def norm(name):
        s[name], s[name + ".b"] = vec(width, 1.0, 0.2), vec(width, 0.0, 0.1)
        s[name + ".alpha"] = torch.tensor(0.6 + 0.6 * float(torch.rand((), generator=g)))

    side = cfg.get("token_side")
    if side:
        s["side.embed"] = torch.randn(vocab, side["dim"] * len(cfg["layers"]), generator=g)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        norm(p + "norm1")
        if layer["type"] == "rglru":
            w, b, taps = m["width"], m["blocks"], m["conv"]
            s[p + "mix.y"], s[p + "mix.y.b"] = mat(w, width), vec(w)
            s[p + "mix.x"], s[p + "mix.x.b"] = mat(w, width), vec(w)
            s[p + "mix.conv"], s[p + "mix.conv.b"] = torch.randn(w, taps, generator=g) * 0.5, vec(w)
            s[p + "mix.ra"], s[p + "mix.ra.b"] = torch.randn(b, w // b, w // b, generator=g) / math.sqrt(w // b), vec(w).view(b, w // b)
            s[p + "mix.ri"], s[p + "mix.ri.b"] = torch.randn(b, w // b, w // b, generator=g) / math.sqrt(w // b), vec(w).view(b, w // b)
            s[p + "mix.lam"], s[p + "mix.o"] = vec(w, -1.0, 1.5), mat(width, w)
        else:
            h, d, r, v, k = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            s[p + "mix.q"] = mat(h * (d + r), width, sharp)
            if m.get("kv_from") is None:
                s[p + "mix.dkv"], s[p + "mix.dkv.norm"] = mat(k + r, width), vec(k, 1.0, 0.2)
            s[p + "mix.uk"], s[p + "mix.uv"] = mat(h * d, k), mat(h * v, k)
            s[p + "mix.g"], s[p + "mix.o"] = mat(h, width, 2.0), mat(width, h * v)
        mlp = layer.get("mlp")
        if mlp:
            norm(p + "norm2")
            e, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            s[p + "mlp.router"], s[p + "mlp.router.b"] = mat(e, width, router_gain), vec(e, 0.0, 1.0)
            for j in range(e):
                s[p + f"mlp.e{j}.up"], s[p + f"mlp.e{j}.down"] = mat(ff, width), mat(width, ff)
            if mlp.get("shared"):
                s[p + "mlp.shared.up"], s[p + "mlp.shared.down"] = mat(mlp["shared"]["ff"], width), mat(width, mlp["shared"]["ff"])
        if side:
            s[p + "side.gate"], s[p + "side.proj"] = mat(side["dim"], width), mat(width, side["dim"])
            s[p + "side.norm"] = vec(width, 1.0, 0.2)
    norm("final.norm")
    return s
