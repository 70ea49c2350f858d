"""A plain, slow statement of the Nidilix decoder in float64, one function per mechanism.

It is the oracle of the tests: it takes a configuration dictionary (the keys of config.json) and a dictionary of
tensors by checkpoint name, runs a whole sequence at once with loops where the formulas have them, and shares no
code with the package. Linear weights are [out, in] and applied as ``x @ W.T``.

Mechanisms
----------
dynamic_tanh       y = tanh(alpha x) w + b
rms_unit           x / sqrt(mean(x^2) + eps)
rotate_pairs       pair (2i, 2i+1) of the first ``dims`` entries turns by position * base^(-2i/dims)
latent_attention   queries per head [plain | rotated]; one latent vector and one rotated key part per token; keys
                   and values are products of the latent; causal softmax; a sigmoid gate per head on the output
rglru              gelu branch times a gated linear recurrence over a short causal convolution
routed_experts     top-k of the router's logits, softmax over the chosen, relu^2 experts, plus a shared expert
token_side_input   a per-layer slice of a second embedding, gated by the stream, projected, normed to unit RMS
"""

import math

import torch

F64 = torch.float64


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def dynamic_tanh(x, w, prefix):
    return torch.tanh(w[prefix + ".alpha"] * x) * w[prefix] + w[prefix + ".b"]


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rotate_pairs(x, positions, base, dims):
    """x [tokens, ..., n]; entries 2i and 2i+1 (i < dims/2) are one pair."""
    out = x.clone()
    for i in range(dims // 2):
        angle = positions.to(F64) * (float(base) ** (-2.0 * i / dims))
        cos, sin = torch.cos(angle), torch.sin(angle)
        while cos.dim() < x.dim() - 1:
            cos, sin = cos.unsqueeze(-1), sin.unsqueeze(-1)
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * cos - v * sin
        out[..., 2 * i + 1] = v * cos + u * sin
    return out


def latent_of(h, w, p, m, eps, positions):
    """What a latent-attention layer keeps per token: (latent [tokens, rank], rotated key part [tokens, rot])."""
    rank, rot = m["kv_rank"], m["rot_dim"]
    d = h @ w[p + "dkv"].T
    latent = rms_unit(d[:, :rank], eps) * w[p + "dkv.norm"]
    shared = rotate_pairs(d[:, rank:rank + rot], positions, m["rot"]["base"], m["rot"]["dims"])
    return latent, shared


def latent_attention(h, w, p, m, eps, positions, kept):
    """``kept``: (latent, rotated key part) of this layer or of the layer it borrows them from."""
    heads, dim, rot, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    n = h.shape[0]
    latent, shared = kept
    q = (h @ w[p + "q"].T).view(n, heads, dim + rot)
    q_plain = q[..., :dim]
    q_rot = rotate_pairs(q[..., dim:], positions, m["rot"]["base"], m["rot"]["dims"])
    keys = (latent @ w[p + "uk"].T).view(n, heads, dim)
    values = (latent @ w[p + "uv"].T).view(n, heads, vdim)
    gate = torch.sigmoid(h @ w[p + "g"].T)                      # [n, heads]
    out = torch.zeros(n, heads, vdim, dtype=F64)
    for i in range(n):
        for a in range(heads):
            s = (keys[: i + 1, a] @ q_plain[i, a] + shared[: i + 1] @ q_rot[i, a]) * m["scale"]
            prob = torch.softmax(s, 0)
            out[i, a] = (prob.unsqueeze(1) * values[: i + 1, a]).sum(0) * gate[i, a]
    return out.reshape(n, heads * vdim) @ w[p + "o"].T


def rglru(h, w, p, m):
    width, blocks, taps = m["width"], m["blocks"], m["conv"]
    n = h.shape[0]
    y = gelu_tanh(h @ w[p + "y"].T + w[p + "y.b"])
    x = h @ w[p + "x"].T + w[p + "x.b"]
    padded = torch.cat([torch.zeros(taps - 1, width, dtype=F64), x])
    u = torch.zeros(n, width, dtype=F64)
    for t in range(n):
        for j in range(taps):           # the last column weighs the current token
            u[t] += w[p + "conv"][:, j] * padded[t + j]
        u[t] += w[p + "conv.b"]
    bw = width // blocks
    r = torch.zeros(n, width, dtype=F64)
    i_gate = torch.zeros(n, width, dtype=F64)
    for b in range(blocks):
        ub = u[:, b * bw:(b + 1) * bw]
        r[:, b * bw:(b + 1) * bw] = torch.sigmoid(ub @ w[p + "ra"][b].T + w[p + "ra.b"][b])
        i_gate[:, b * bw:(b + 1) * bw] = torch.sigmoid(ub @ w[p + "ri"][b].T + w[p + "ri.b"][b])
    log_a = -8.0 * r * torch.nn.functional.softplus(w[p + "lam"])
    a = torch.exp(log_a)
    state = torch.zeros(width, dtype=F64)
    out = torch.zeros(n, width, dtype=F64)
    for t in range(n):
        state = a[t] * state + torch.sqrt(1.0 - a[t] ** 2) * i_gate[t] * u[t]
        out[t] = state * y[t]
    return out @ w[p + "o"].T


def relu_squared_expert(h, w, p):
    return (torch.relu(h @ w[p + "up"].T) ** 2) @ w[p + "down"].T


def routed_experts(h, w, p, mlp):
    experts, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = h @ w[p + "router"].T + w[p + "router.b"]
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        order = sorted(range(experts), key=lambda e: (-float(z[t, e]), e))[:top]
        weights = torch.softmax(z[t, order], 0)
        for k, e in enumerate(order):
            out[t] += weights[k] * relu_squared_expert(h[t:t + 1], w, f"{p}e{e}.")[0]
    if mlp.get("shared"):
        out = out + relu_squared_expert(h, w, p + "shared.")
    return out


def token_side_input(x, tokens, layer, w, side_dim, eps):
    e = w["side.embed"][tokens][:, layer * side_dim:(layer + 1) * side_dim]
    g = gelu_tanh(x @ w[f"l{layer}.side.gate"].T) * e
    y = g @ w[f"l{layer}.side.proj"].T
    return rms_unit(y, eps) * w[f"l{layer}.side.norm"]


def forward(config, weights, tokens, want_layers=False):
    """float64 logits [tokens, vocab] (and the stream after every layer)."""
    w = {k: v.to(F64) if v.is_floating_point() else v for k, v in weights.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(len(tokens))
    eps, mult = config["norm"]["eps"], config["residual_mult"]
    side = config.get("token_side")
    x = w["embed"][tokens]
    kept, after = {}, []
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        h = dynamic_tanh(x, w, f"l{i}.norm1")
        if layer["type"] == "latent_attention":
            source = m.get("kv_from")
            if source is None:
                kept[i] = latent_of(h, w, p, m, eps, positions)
                source = i
            x = x + mult * latent_attention(h, w, p, m, eps, positions, kept[source])
        elif layer["type"] == "rglru":
            x = x + mult * rglru(h, w, p, m)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp"):
            x = x + mult * routed_experts(dynamic_tanh(x, w, f"l{i}.norm2"), w, f"l{i}.mlp.", layer["mlp"])
        if side:
            x = x + mult * token_side_input(x, tokens, i, w, side["dim"], eps)
        after.append(x)
    logits = dynamic_tanh(x, w, "final.norm") @ w["head"].T
    return (logits, after) if want_layers else logits
