"""A plain, slow Zipedra forward pass for the tests: whole sequences, no cache, one function per mechanism.

Zipedra is a decoder-only design whose layers run norm -> (mixer + feed-forward side by side) -> a small
per-layer token input, whose mixers are either a decayed linear attention ('lightning') or an attention over
a low-rank latent ('latent_attention'), whose feed-forwards are dense or routed, and in which a range of
layers may run several times in a row ('loop').  This file shares no code with ``torchinferno_b200``: it reads
config.json and model.safetensors itself and computes on the CPU in float64, token by token where the design
is a recurrence, so that its own rounding does not count against the engine.

Notation: T tokens, W the model width, x the residual stream [T, W], h = norm(x).
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch


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
def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    return unit_rms(x, eps) * weight


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate_pairs(x, positions, base, dims):
    """Rotary on the first ``dims`` elements of the last axis of x [T, ..., d]; element 2i pairs with 2i + 1,
    angle = position * base^(-2i / dims); the rest pass unchanged."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    freq = torch.tensor(float(base), dtype=torch.float64) ** (-2 * i / dims)
    angle = positions.to(torch.float64)[:, None] * freq[None, :]                # [T, dims / 2]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    cos, sin = angle.cos().reshape(shape), angle.sin().reshape(shape)
    even, odd = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = even * cos - odd * sin
    out[..., 1:dims:2] = odd * cos + even * sin
    return out


# ------------------------------------------------------------------- mixers
def lightning_mixer(h, w, p, m, eps):
    """Decayed linear attention.  Per head: S_t = decay * S_(t-1) + k_t v_t^T, o_t = S_t^T q_t with q, k, v
    passed through silu; all heads' outputs normed together, gated by sigmoid(W_g h), projected by W_o."""
    T, H, D, V = h.shape[0], m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).view(T, H, D)
    k = silu(h @ w[p + "k"].T).view(T, H, D)
    v = silu(h @ w[p + "v"].T).view(T, H, V)
    decay = torch.tensor([float(d) for d in m["decay"]], dtype=h.dtype)
    state = torch.zeros(H, D, V, dtype=h.dtype)
    out = torch.empty(T, H, V, dtype=h.dtype)
    for t in range(T):
        state = decay[:, None, None] * state + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", state, q[t])
    y = rms_norm(out.reshape(T, H * V), w[p + "norm"], eps) * torch.sigmoid(h @ w[p + "g"].T)
    return y @ w[p + "o"].T


def latent_attention_mixer(h, w, p, m, eps, positions):
    """Attention whose keys and values are made from one low-rank latent per token.  The key of head j is
    [W_uk_j c ; r] with r a rotated part shared by all heads, its value W_uv_j c; causal softmax; the heads'
    outputs are gated by sigmoid(W_g h) and projected by W_o."""
    T, H, D, R, V, C = h.shape[0], m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    base, dims = m["rot"]["base"], m["rot"]["dims"]
    q = (h @ w[p + "q"].T).view(T, H, D + R)
    q_plain, q_rot = q[..., :D], rotate_pairs(q[..., D:].contiguous(), positions, base, dims)
    dkv = h @ w[p + "dkv"].T
    latent = rms_norm(dkv[:, :C], w[p + "dkv.norm"], eps)
    k_rot = rotate_pairs(dkv[:, C:].contiguous(), positions, base, dims)          # [T, R], one for all heads
    k_plain = (latent @ w[p + "uk"].T).view(T, H, D)
    value = (latent @ w[p + "uv"].T).view(T, H, V)
    scores = (torch.einsum("thd,shd->hts", q_plain, k_plain) + torch.einsum("thr,sr->hts", q_rot, k_rot)) * m["scale"]
    hidden = positions[None, :] > positions[:, None]                              # key s later than query t
    scores = scores.masked_fill(hidden[None], float("-inf"))
    out = torch.einsum("hts,shv->thv", torch.softmax(scores, dim=-1), value).reshape(T, H * V)
    return (out * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


# ------------------------------------------------------------ feed-forwards
def dense_feed_forward(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def squared_relu_expert(h, up, down):
    return torch.relu(h @ up.T).pow(2) @ down.T


def routed_feed_forward(h, w, p, mlp, gaps=None):
    """softmax over all experts, the ``top`` largest chosen (lowest index first among equals), their scores
    divided by their sum (+ 1e-20) as weights; plus a shared expert gated by one sigmoid per token.
    ``gaps`` (a list per token) collects how far the last chosen score lies above the first one left out, as a
    share of itself."""
    experts, top = mlp["router"]["experts"], mlp["router"]["top"]
    scores = torch.softmax(h @ w[p + "router"].T, dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        ranked = sorted(range(experts), key=lambda e: (-float(scores[t, e]), e))
        order = ranked[:top]
        if gaps is not None and top < experts:
            gaps[t].append(float(1 - scores[t, ranked[top]] / scores[t, ranked[top - 1]]))
        total = sum(scores[t, e] for e in order) + 1e-20
        for e in order:
            out[t] += (scores[t, e] / total) * squared_relu_expert(h[t], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"])
    if mlp.get("shared"):
        gate = torch.sigmoid(h @ w[p + "shared.sg"].T)                           # [T, 1]
        out = out + gate * squared_relu_expert(h, w[p + "shared.up"], w[p + "shared.down"])
    return out


# --------------------------------------------------------------- the model
def token_side(x, tokens, w, layer, dim, eps):
    """The per-layer token input: a slice of a second embedding, gated by gelu(W x), projected, unit-normed."""
    p = f"l{layer}.side."
    e = w["side.embed"][tokens][:, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ w[p + "gate"].T) * e) @ w[p + "proj"].T
    return x + rms_norm(y, w[p + "norm"], eps)


def layer_runs(config):
    """[(layer, pass number or None, first of its pass)] in the order the layers run."""
    n, loop = len(config["layers"]), config.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, None, False) for i in range(start)]
    for t in range(times):
        runs += [(i, t, i == start) for i in range(start, stop)]
    return runs + [(i, None, False) for i in range(stop, n)]


def forward(config, w, tokens, return_layers=False, gaps=None):
    """Logits [T, vocab] of one whole sequence (and, on request, the residual stream after every layer run).
    ``gaps``: a list of one list per token, filled with the routers' margins at that token."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(len(tokens))
    eps = config["norm"]["eps"]
    x0 = w["embed"][tokens]
    x, after = x0, []
    for layer, t, first in layer_runs(config):
        if first:
            x = torch.cat([x, x0], dim=-1) @ w["loop.in"].T + w["loop.step"][t]
        spec, p = config["layers"][layer], f"l{layer}."
        h = rms_norm(x, w[p + "norm1"], eps)
        if spec["type"] == "lightning":
            delta = lightning_mixer(h, w, p + "mix.", spec["mixer"], eps)
        elif spec["type"] == "latent_attention":
            delta = latent_attention_mixer(h, w, p + "mix.", spec["mixer"], eps, positions)
        else:
            raise ValueError(spec["type"])
        mlp = spec.get("mlp")
        if mlp is not None:
            delta = delta + (dense_feed_forward(h, w, p + "mlp.") if mlp["kind"] == "dense"
                             else routed_feed_forward(h, w, p + "mlp.", mlp, gaps))
        x = x + delta
        if config.get("token_side"):
            x = token_side(x, tokens, w, layer, config["token_side"]["dim"], eps)
        after.append(x)
    logits = (rms_norm(x, w["final.norm"], eps) @ w["head"].T) * config["logit_scale"]
    return (logits, torch.stack(after)) if return_layers else logits
