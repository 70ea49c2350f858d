"""Small Migelix configurations and seeded weights for the tests. Nothing here imports the product package."""

from __future__ import annotations

import copy
import math

import torch


def rot(dims, base=10000.0, yarn=None):
    r = {"base": base, "dims": dims}
    if yarn:
        factor, original, fast, slow = yarn
        r["scaling"] = {"factor": factor, "original": original, "fast": fast, "slow": slow}
    return r


def attn_sizes(heads, kv, dim, rotation, window=None, scale=None, softcap=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "rot": rotation, "scale": scale if scale is not None else dim ** -0.5}
    if window:
        m["mask"] = {"size": window}
    if softcap:
        m["softcap"] = softcap
    return m


def attention(*a, **k):
    return {"type": "attention", "mixer": attn_sizes(*a, **k)}


def delta_sizes(heads, kv, dim, vdim, conv, decay_rank=None, gate_rank=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}
    if decay_rank:
        m["decay_rank"] = decay_rank
    if gate_rank:
        m["gate_rank"] = gate_rank
    return m


def parallel(left, right, left_scale=1.0, right_scale=1.0):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}}


def wkv(heads, dim, decay_rank=None):
    m = {"heads": heads, "dim": dim}
    if decay_rank:
        m["decay_rank"] = decay_rank
    return {"type": "wkv", "mixer": m}


def config(width, vocab, layers, eps=1e-6, logit_softcap=None):
    """``layers``: list of (mixer entry, ff or None) or of an int j, which repeats layer j with its weights."""
    out = []
    for entry in layers:
        if isinstance(entry, int):
            out.append(dict(copy.deepcopy(out[entry]), weights_of=entry))
        else:
            m, ff = entry
            out.append(dict(m, mlp={"kind": "dense", "ff": ff} if ff else None))
    d = {"architecture": "Migelix", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": out}
    if logit_softcap:
        d["logit_softcap"] = logit_softcap
    return d


# Sizes unlike one another. A: a key head shared by three query heads, half the entries rotated, YaRN whose ramp lies
# inside the prompts' lengths, a recurrence whose heads share q/k heads in pairs and whose values are wider than its keys,
# a layer without feed-forward, layers that run twice.
CASE_A = config(96, 211, [
    (parallel(attn_sizes(3, 1, 32, rot(16, 10000.0, yarn=(8.0, 64, 16.0, 2.0)), window=21, scale=0.2), delta_sizes(4, 2, 24, 40, 3), 0.6, 1.3), 72),
    (wkv(3, 20), None),
    (attention(4, 4, 16, rot(16, 500.0), window=9, scale=0.3, softcap=5.0), 40),
    0, 2,
], eps=1e-6, logit_softcap=6.0)

# B: no window, no cap on scores or logits, a single wide memory head, no rotation at all, one tap, one q/k head.
CASE_B = config(80, 157, [
    (attention(2, 1, 48, rot(8, 300.0)), 56),
    (wkv(1, 64), 24),
    (parallel(attn_sizes(2, 2, 16, rot(0, 100.0), window=5), delta_sizes(2, 1, 8, 16, 1), 1.0, 0.5), None),
    1,
], eps=1e-5)

# C: head sizes of 64 and 128 with pages of 16: the sizes the tensor-core attention kernels take in bfloat16.
CASE_C = config(128, 263, [
    (parallel(attn_sizes(4, 2, 64, rot(32, 20000.0, yarn=(2.0, 128, 8.0, 1.0)), window=70), delta_sizes(2, 2, 64, 64, 4), 0.9, 0.7), 96),
    (attention(6, 2, 128, rot(64, 1e5), window=33, softcap=30.0), 64),
    (wkv(2, 64), 96),
    0,
], eps=2e-6, logit_softcap=20.0)

# D: sizes that are multiples of 2 only, so rows of 16-bit numbers start off a 16-byte boundary and every vector path has
# to step aside; ranks given in the configuration.
CASE_D = config(100, 103, [
    (wkv(3, 10, decay_rank=7), 36),
    (parallel(attn_sizes(3, 3, 20, rot(10, 4000.0), window=12), delta_sizes(3, 3, 12, 20, 2, decay_rank=4, gate_rank=6), 1.1, 0.8), 36),
    (attention(2, 1, 24, rot(24, 9000.0), window=30, softcap=12.0), None),
], eps=1e-6, logit_softcap=9.0)

CASES = {"A": CASE_A, "B": CASE_B, "C": CASE_C, "D": CASE_D}


def seeded_state(cfg: dict, seed: int, sharp: float = 1.0, decay_rank: int = 6, gate_rank: int = 10, shift_rank: int = 5) -> dict:
    """float32 weights by checkpoint name. Matrices N(0, 1/in); ``sharp`` multiplies the query projections of the
    attention mixers so that a softmax settles on few keys, wherever they lie."""
    g = torch.Generator().manual_seed(seed)
    width, vocab = cfg["width"], cfg["vocab"]

    def mat(rows, cols, gain=1.0):
        return torch.randn(rows, cols, generator=g) * (gain / math.sqrt(cols))

    def vec(n, mean=0.0, std=0.3):
        return mean + std * torch.randn(n, generator=g)

    # the table is the head too: rows of norm about 2.5, so that logits stay within a few units
    s = {"embed": torch.randn(vocab, width, generator=g) * (2.5 / math.sqrt(width)), "final.norm": vec(width, 0.0, 0.2)}

    def attn(p, m, biased, sinks, gated):
        h, kv, d = m["heads"], m["kv_heads"], m["dim"]
        s[p + "q"], s[p + "k"], s[p + "o"] = mat(h * d, width, sharp), mat(kv * d, width), mat(width, h * d)
        if biased:
            s[p + "q.b"], s[p + "k.b"] = vec(h * d), vec(kv * d)
        if sinks:
            s[p + "sink"] = vec(h, 0.5, 1.0)
        if gated:
            s[p + "g"] = mat(h * d, width, 2.0)

    for i, layer in enumerate(cfg["layers"]):
        if layer.get("weights_of") is not None:
            continue
        p, m = f"l{i}.", layer["mixer"]
        s[p + "norm1"] = vec(width, 0.0, 0.2)
        if layer["type"] == "attention":
            attn(p + "mix.", m, False, False, True)
        elif layer["type"] == "wkv":
            h, d = m["heads"], m["dim"]
            r = m.get("decay_rank", shift_rank)
            for name in "rkvgw":
                s[p + "mix.mu." + name] = torch.rand(width, generator=g)
            for name in "rkvg":
                s[p + "mix." + name] = mat(h * d, width)
            s[p + "mix.w1"], s[p + "mix.w2"] = mat(r, width), mat(h * d, r, 1.5)
            s[p + "mix.w0"], s[p + "mix.u"] = vec(h * d, -1.5, 1.0), vec(h * d, 0.3, 0.5).view(h, d)
            s[p + "mix.norm"], s[p + "mix.o"] = vec(h * d, 1.0, 0.2), mat(width, h * d)
        else:
            attn(p + "mix.left.", m["left"], True, True, False)
            r, q = m["right"], p + "mix.right."
            h, kv, d, dv, taps = r["heads"], r["kv_heads"], r["dim"], r["vdim"], r["conv"]
            ra, rg = r.get("decay_rank", decay_rank), r.get("gate_rank", gate_rank)
            s[q + "q"], s[q + "k"], s[q + "v"] = mat(kv * d, width), mat(kv * d, width), mat(h * dv, width)
            for name, rows in (("q", kv * d), ("k", kv * d), ("v", h * dv)):
                s[q + name + ".conv"] = torch.randn(rows, taps, generator=g) * 0.6
            s[q + "b"], s[q + "A_log"], s[q + "norm"] = mat(h, width, 2.0), vec(h, -0.5, 0.8), vec(dv, 1.0, 0.2)
            s[q + "a1"], s[q + "a2"], s[q + "dt_bias"] = mat(ra, width), mat(h * d, ra, 1.5), vec(h * d, -1.0, 1.0)
            s[q + "g1"], s[q + "g2"], s[q + "o"] = mat(rg, width), mat(h * dv, rg, 1.5), mat(width, h * dv)
        if layer.get("mlp"):
            ff = layer["mlp"]["ff"]
            s[p + "norm2"] = vec(width, 0.0, 0.2)
            s[p + "mlp.gate"], s[p + "mlp.up"], s[p + "mlp.down"] = mat(ff, width), mat(ff, width), mat(width, ff)
    return s
