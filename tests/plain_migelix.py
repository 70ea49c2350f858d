"""The Migelix decoder written out plainly in float64, one function per mechanism, token by token where a recurrence is
involved. Slow on purpose; shares no code with the package. Weights are a dict name -> float64 tensor, the
configuration is the config.json dictionary.

Notation: h is a layer's normed input [T, width]; every function returns [T, ...] for the T tokens of one sequence
that starts at position 0.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x, w, eps):
    """RMS norm with the factor 1 + w."""
    return unit_rms(x, eps) * (1.0 + w)


# ------------------------------------------------------------------------------------------------- rotation
def rotary_frequencies(rot: dict):
    """Per pair i: the frequency and the factor on cos and sin."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def where(turns):           # the (fractional) dimension whose wave makes `turns` turns over the original length
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(where(float(sc["fast"]))), 0)
    hi = min(math.ceil(where(float(sc["slow"]))), dims - 1)
    ramp = torch.tensor([min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(dims // 2)], dtype=F64)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x, positions, rot: dict):
    """x [T, heads, dim]: entries 2i and 2i+1 of the first rot.dims are turned by position * f_i; the rest pass."""
    f, mag = rotary_frequencies(rot)
    dims = int(rot["dims"])
    a = positions.to(F64)[:, None] * f[None, :]                    # [T, dims/2]
    c, s = (a.cos() * mag)[:, None, :], (a.sin() * mag)[:, None, :]
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ------------------------------------------------------------------------------------------------ attention
def windowed_attention(q, k, v, scale, window, softcap=None, sink=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; token i reads j with 0 <= i - j < window. ``softcap`` c turns a
    score s into c tanh(s / c); ``sink`` [H] adds exp(sink_h) to the softmax's denominator."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            j0 = max(0, i - window + 1) if window else 0
            s = (k[j0:i + 1, g] @ q[i, h]) * scale
            if softcap:
                s = softcap * torch.tanh(s / softcap)
            m = s.max() if sink is None else torch.maximum(s.max(), sink[h])
            e = torch.exp(s - m)
            den = e.sum() + (torch.exp(sink[h] - m) if sink is not None else 0.0)
            out[i, h] = (e / den) @ v[j0:i + 1, g]
    return out


def keys_as_values_attention(h, w, p, m, biased, gated, sinks):
    """The attention mixer whose values are its keys before the rotation. ``p``: tensor prefix, ``m``: its sizes."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q, k = h @ w[p + "q"].T, h @ w[p + "k"].T
    if biased:
        q, k = q + w[p + "q.b"], k + w[p + "k.b"]
    q, k = q.view(T, H, d), k.view(T, G, d)
    pos = torch.arange(T)
    o = windowed_attention(rotate_pairs(q, pos, m["rot"]), rotate_pairs(k, pos, m["rot"]), k, float(m["scale"]),
                           int(m["mask"]["size"]) if m.get("mask") else 0, m.get("softcap"), w[p + "sink"] if sinks else None)
    o = o.reshape(T, -1)
    if gated:
        o = o * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


# ---------------------------------------------------------------------------------------- gated delta rule
def causal_conv_silu(x, taps_w):
    """x [T, C], taps_w [C, taps]: the last column weighs the current token; zeros before the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=F64), x])
    y = sum(padded[j:j + T] * taps_w[:, j] for j in range(taps))
    return y * torch.sigmoid(y)


def gated_delta(h, w, p, m, eps):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = causal_conv_silu(h @ w[p + "q"].T, w[p + "q.conv"]).view(T, G, d)
    k = causal_conv_silu(h @ w[p + "k"].T, w[p + "k.conv"]).view(T, G, d)
    v = causal_conv_silu(h @ w[p + "v"].T, w[p + "v.conv"]).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                               # [T, H]
    dt = torch.nn.functional.softplus((h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]).view(T, H, d)
    decay = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * dt)                   # [T, H, d]
    gate = torch.sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=F64)
    for a in range(H):
        g = a // (H // G)
        S = torch.zeros(d, dv, dtype=F64)
        for t in range(T):
            S = decay[t, a][:, None] * S
            u = beta[t, a] * (v[t, a] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, a] = S.T @ q[t, g]
    out = unit_rms(out, eps) * w[p + "norm"] * gate
    return out.reshape(T, H * dv) @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps):
    left = keys_as_values_attention(h, w, p + "left.", m["left"], biased=True, gated=False, sinks=True)
    right = gated_delta(h, w, p + "right.", m["right"], eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


# ------------------------------------------------------------------------------------------------------ wkv
def wkv_mixer(h, w, p, m, eps):
    T, width = h.shape
    H, d = m["heads"], m["dim"]
    prev = torch.cat([torch.zeros(1, width, dtype=F64), h[:-1]])
    mix = {s: h + (prev - h) * w[p + "mu." + s] for s in "rkvgw"}
    r, k, v = ((mix[s] @ w[p + s].T).view(T, H, d) for s in "rkv")
    gate = mix["g"] @ w[p + "g"].T
    gate = gate * torch.sigmoid(gate)
    decay = torch.exp(-torch.exp(torch.tanh(mix["w"] @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"])).view(T, H, d)
    bonus = w[p + "u"]                                                                   # [H, d]
    out = torch.zeros(T, H, d, dtype=F64)
    for a in range(H):
        S = torch.zeros(d, d, dtype=F64)
        for t in range(T):
            kv = torch.outer(k[t, a], v[t, a])
            out[t, a] = (S + bonus[a][:, None] * kv).T @ r[t, a]
            S = decay[t, a][:, None] * S + kv
    out = unit_rms(out, eps).reshape(T, H * d) * w[p + "norm"] * gate
    return out @ w[p + "o"].T


# ------------------------------------------------------------------------------------------- the whole model
def dense_feed_forward(h, w, p):
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def forward(config: dict, weights: dict, tokens, capture=None):
    """Logits [T, vocab] for one sequence from position 0. ``capture``: a list that receives the stream after every layer."""
    w = {k: v.to(F64) for k, v in weights.items() if v.is_floating_point()}
    eps = float(config["norm"]["eps"])
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(config["layers"]):
        src = layer.get("weights_of", i)
        p, m = f"l{src}.", layer["mixer"]
        h = offset_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "parallel":
            x = x + parallel_mixer(h, w, p + "mix.", m, eps)
        elif layer["type"] == "wkv":
            x = x + wkv_mixer(h, w, p + "mix.", m, eps)
        elif layer["type"] == "attention":
            x = x + keys_as_values_attention(h, w, p + "mix.", m, biased=False, gated=True, sinks=False)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            x = x + dense_feed_forward(offset_norm(x, w[p + "norm2"], eps), w, p + "mlp.")
        if capture is not None:
            capture.append(x.clone())
    logits = offset_norm(x, w["final.norm"], eps) @ w["embed"].T
    cap = config.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits
