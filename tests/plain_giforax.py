"""A plain, slow Giforax forward pass for the tests: whole sequences, no cache, one function per mechanism.

Giforax is a decoder-only design whose layers put a layer norm (weight and bias) before and after each sublayer, whose
mixers are an attention with sigmoid weights inside chunks of the sequence or a minimal GRU, whose feed-forward is a
set of routed experts (each a clamped gated unit fed with the router weight times the token) plus a shared expert,
and in which every layer ends with a weighted sum over the results of all layers so far.  This file shares no code
with ``torchinferno_b200``: it reads config.json and model.safetensors itself and computes on the CPU in float64,
token by token where the design is a recurrence, so that its own rounding does not count against the engine.

Notation: T tokens, W the model width, x the residual stream [T, W].
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

GLU_ALPHA = 1.702


def read_model_folder(folder, dtype=torch.float64):
    from safetensors import safe_open
    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    weights = {}
    with safe_open(str(folder / "model.safetensors"), framework="pt", device="cpu") as handle:
        for name in handle.keys():
            t = handle.get_tensor(name)
            weights[name] = t.to(dtype) if t.is_floating_point() else t
    return config, weights


# ------------------------------------------------------------- small pieces
def layer_norm(x, w, name, eps):
    """(x - mean) / sqrt(mean((x - mean)^2) + eps) * weight + bias; the bias is the tensor ``name`` + '.b'."""
    mean = x.mean(dim=-1, keepdim=True)
    var = (x - mean).pow(2).mean(dim=-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * w[name] + w[name + ".b"]


def unit_rms(x, eps):
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def rotate_half(x, positions, base, dims):
    """Rotary on the first ``dims`` elements of the last axis of x [T, heads, d]: element i pairs with i + dims / 2,
    angle = position * base^(-2i / dims); the rest pass unchanged."""
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = torch.tensor(float(base), dtype=torch.float64) ** (-2 * i / dims)
    angle = positions.to(torch.float64)[:, None] * freq[None, :]
    cos, sin = angle.cos()[:, None, :], angle.sin()[:, None, :]
    lo, hi = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = lo * cos - hi * sin
    out[..., half:dims] = hi * cos + lo * sin
    return out


def visible(positions, size):
    """[T, T] bool: key j is seen by query i iff j <= i and both lie in the same run of ``size`` positions."""
    i, j = positions[:, None], positions[None, :]
    return (j <= i) & (torch.div(i, size, rounding_mode="floor") == torch.div(j, size, rounding_mode="floor"))


# ------------------------------------------------------------------- mixers
def attention_keys_values(h, w, prefix, m, eps, positions):
    """What an attention layer with projections of its own caches: keys after rotation and unit norm, values as projected."""
    T = h.shape[0]
    k = (h @ w[prefix + "k"].T).view(T, m["kv_heads"], m["dim"])
    k = unit_rms(rotate_half(k, positions, m["rot"]["base"], m["rot"]["dims"]), eps)
    v = (h @ w[prefix + "v"].T).view(T, m["kv_heads"], m["vdim"])
    return k, v


def attention_mixer(h, w, prefix, m, eps, positions, keys, values):
    """h: [T, W] normed input; keys / values: [T, kv_heads, dim / vdim] (this layer's own or another layer's)."""
    T, H, G = h.shape[0], m["heads"], m["kv_heads"]
    q = (h @ w[prefix + "q"].T).view(T, H, m["dim"])
    q = unit_rms(rotate_half(q, positions, m["rot"]["base"], m["rot"]["dims"]), eps)
    gate = torch.sigmoid(h @ w[prefix + "g"].T)                         # [T, H]
    seen = visible(positions, m["mask"]["size"])
    out = torch.zeros(T, H, m["vdim"], dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        score = (q[:, head] @ keys[:, g].T) * m["scale"] + w[prefix + "pb"][head]
        weight = torch.sigmoid(score) * seen                           # not normalised over the keys
        out[:, head] = (weight @ values[:, g]) * gate[:, head:head + 1]
    return out.reshape(T, H * m["vdim"]) @ w[prefix + "o"].T


def min_gru_mixer(h, w, prefix, m, state=None):
    """Token by token: S <- (1 - z) S + z c.  Returns (output [T, W], final state)."""
    z = torch.sigmoid(h @ w[prefix + "z"].T + w[prefix + "z.b"])
    u = h @ w[prefix + "x"].T + w[prefix + "x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    gate = h @ w[prefix + "g"].T
    S = torch.zeros(m["width"], dtype=h.dtype) if state is None else state.clone()
    rows = []
    for t in range(h.shape[0]):
        S = (1 - z[t]) * S + z[t] * cand[t]
        rows.append(S * (gate[t] * torch.sigmoid(gate[t])))
    return torch.stack(rows) @ w[prefix + "o"].T, S


# ------------------------------------------------------------- feed-forward
def gated_unit(x, w, prefix, limit):
    g = torch.clamp(x @ w[prefix + "gate"].T, max=limit)
    u = torch.clamp(x @ w[prefix + "up"].T, -limit, limit)
    return (g * torch.sigmoid(GLU_ALPHA * g) * (u + 1)) @ w[prefix + "down"].T


def routed_feed_forward(h, w, prefix, mlp, gaps=None):
    """Sigmoid scores, the ``top`` largest (lowest index among equals), weights = the scores as they are, each chosen
    expert fed with weight * h; plus the shared expert.  ``gaps[t]`` collects, per token, how far the last chosen score
    lies above the best one left out, as a share of itself."""
    T = h.shape[0]
    experts, top = mlp["router"]["experts"], mlp["router"]["top"]
    scores = torch.sigmoid(h @ w[prefix + "router"].T)
    out = torch.zeros_like(h)
    for t in range(T):
        order = sorted(range(experts), key=lambda e: (-float(scores[t, e]), e))
        if gaps is not None and top < experts:
            last, nxt = float(scores[t, order[top - 1]]), float(scores[t, order[top]])
            gaps[t].append((last - nxt) / max(abs(last), 1e-30))
        for e in order[:top]:
            out[t] += gated_unit(scores[t, e] * h[t:t + 1], w, f"{prefix}e{e}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        out = out + gated_unit(h, w, prefix + "shared.", mlp["shared"]["limit"])
    return out


# ----------------------------------------------------------------- the model
def forward(config, w, tokens, return_layers=False, gaps=None):
    """Logits [T, vocab] for one sequence from position 0 (and, asked for, the stream after every layer)."""
    eps = config["norm"]["eps"]
    positions = torch.arange(len(tokens))
    x = w["embed"][torch.tensor(tokens)] * config["embedding"]["scale"]
    results = [x]                   # X_0, then every layer's result before its average
    cached = {}
    streams = []
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = layer_norm(x, w, p + "norm1", eps)
        if layer["type"] == "mingru":
            y, _ = min_gru_mixer(h, w, p + "mix.", m)
        else:
            if m.get("kv_from") is None:
                cached[i] = attention_keys_values(h, w, p + "mix.", m, eps, positions)
            keys, values = cached[i if m.get("kv_from") is None else m["kv_from"]]
            y = attention_mixer(h, w, p + "mix.", m, eps, positions, keys, values)
        x = x + layer_norm(y, w, p + "norm1b", eps)
        if layer["mlp"] is not None:
            h = layer_norm(x, w, p + "norm2", eps)
            x = x + layer_norm(routed_feed_forward(h, w, p + "mlp.", layer["mlp"], gaps), w, p + "norm2b", eps)
        results.append(x)
        x = sum(w[p + "dwa"][j] * results[j] for j in range(i + 2))
        streams.append(x)
    logits = layer_norm(x, w, "final.norm", eps) @ w["head"].T
    return (logits, torch.stack(streams)) if return_layers else logits
