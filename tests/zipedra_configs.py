"""Small Zipedra configurations for the tests: sizes that differ from one another in every place, values that
happen to be 1 or equal to one another, every kind of layer, with and without a loop and a token side input."""
from __future__ import annotations


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, base=10000.0, rot_dims=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
            "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}


def lightning(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def moe(experts, top, ff, shared=None):
    out = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


# a loop from the first layer on, three passes; rotary on part of the rotated width; a layer without feed-forward
ZA = {
    "architecture": "Zipedra", "vocab": 97, "width": 64, "logit_scale": 0.7, "norm": {"eps": 1e-5},
    "token_side": {"dim": 10}, "loop": {"start": 0, "stop": 2, "times": 3},
    "layers": [
        {"type": "lightning", "mixer": lightning(3, 16, 24, [1.0, 0.9, 0.5]), "mlp": moe(5, 2, 24, shared=40)},
        {"type": "latent_attention", "mixer": latent(2, 16, 8, 24, 40, 0.2, rot_dims=4), "mlp": {"kind": "dense", "ff": 72}},
        {"type": "latent_attention", "mixer": latent(3, 8, 4, 8, 24, 0.3, base=500.0), "mlp": None},
    ],
}
# no loop, no token side input; one head; every expert chosen (top = experts); a routed layer without shared expert;
# a latent rank that is no multiple of 32 and an odd vocabulary
ZB = {
    "architecture": "Zipedra", "vocab": 131, "width": 48, "logit_scale": 1.0, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "latent_attention", "mixer": latent(1, 24, 6, 20, 36, 0.25, base=200000.0), "mlp": moe(3, 3, 20)},
        {"type": "lightning", "mixer": lightning(1, 40, 8, [0.97]), "mlp": {"kind": "dense", "ff": 56}},
        {"type": "latent_attention", "mixer": latent(4, 12, 2, 12, 16, 0.4), "mlp": moe(6, 1, 16, shared=24)},
    ],
}
# only state, no keys at all: every mixer is a linear attention; the loop covers the last two layers, one pass
ZC = {
    "architecture": "Zipedra", "vocab": 60, "width": 40, "logit_scale": 2.0, "norm": {"eps": 1e-6},
    "token_side": {"dim": 4}, "loop": {"start": 1, "stop": 3, "times": 1},
    "layers": [
        {"type": "lightning", "mixer": lightning(2, 8, 8, [0.8, 0.999]), "mlp": {"kind": "dense", "ff": 48}},
        {"type": "lightning", "mixer": lightning(4, 4, 12, [0.3, 0.6, 0.9, 1.0]), "mlp": moe(4, 2, 12, shared=12)},
        {"type": "lightning", "mixer": lightning(1, 16, 16, [0.95]), "mlp": None},
    ],
}
CONFIGS = {"ZA": (ZA, 11), "ZB": (ZB, 12), "ZC": (ZC, 13)}
