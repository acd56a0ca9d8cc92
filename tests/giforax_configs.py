"""Small Giforax configurations for the tests: sizes that differ from one another in every place, values that happen
to be 1 or equal to one another, both kinds of layer in several orders, layers that read another layer's keys."""
from __future__ import annotations


def attention(heads, kv_heads, dim, vdim, size, scale, rot_dims, base=10000.0, kv_from=None):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": size}, "scale": scale,
           "rot": {"base": base, "dims": rot_dims}}
    if kv_from is not None:
        out["kv_from"] = kv_from
    return out


def moe(experts, top, ff, limit, shared=None, shared_limit=None):
    out = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
    if shared:
        out["shared"] = {"ff": shared, "limit": limit if shared_limit is None else shared_limit}
    return out


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


# grouped heads, values wider than keys, rotary on part of a head, chunks of 24 (not a multiple of the pages used),
# two experts of three chosen, a layer that reads the keys of the first, a recurrence between two attentions
GA = {
    "architecture": "Giforax", "vocab": 101, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
    "layers": [
        layer("attention", attention(4, 2, 16, 24, 24, 0.2, 8), moe(3, 2, 24, 1.5, shared=40, shared_limit=2.5)),
        layer("mingru", {"width": 72}, moe(5, 1, 16, 2.0)),
        layer("attention", attention(4, 2, 16, 24, 40, 0.3, 16, base=500.0, kv_from=0), None),
        layer("attention", attention(2, 2, 8, 8, 7, 0.25, 4), moe(4, 4, 12, 0.75, shared=16)),
    ],
}
# one head, sizes that are no multiple of 8, an odd vocabulary, a recurrence first, every layer after the second reads
# the second's keys (with a mask of its own), chunks of one page, top 1, no shared expert anywhere
GB = {
    "architecture": "Giforax", "vocab": 131, "width": 44, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
    "layers": [
        layer("mingru", {"width": 20}, None),
        layer("attention", attention(1, 1, 12, 20, 16, 0.5, 12, base=200000.0), moe(6, 1, 20, 3.0)),
        layer("attention", attention(1, 1, 12, 20, 5, 0.4, 2, kv_from=1), moe(2, 1, 8, 1.0)),
        layer("attention", attention(1, 1, 12, 20, 64, 0.1, 6, kv_from=1), None),
    ],
}
# only state, no keys at all
GC = {
    "architecture": "Giforax", "vocab": 60, "width": 40, "norm": {"eps": 1e-6}, "embedding": {"scale": 0.5},
    "layers": [
        layer("mingru", {"width": 40}, moe(2, 2, 12, 2.0, shared=12)),
        layer("mingru", {"width": 136}, None),
    ],
}
# six query heads on one key head, keys wider than values, a head of 40 (no multiple of 16), chunks longer than any prompt
# of the tests beside chunks of 2
GD = {
    "architecture": "Giforax", "vocab": 97, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 10.0},
    "layers": [
        layer("attention", attention(6, 1, 40, 16, 1000, 0.15, 40), moe(8, 3, 32, 2.0, shared=64)),
        layer("attention", attention(3, 3, 32, 32, 2, 0.2, 32, base=100.0), moe(8, 8, 8, 2.0)),
        layer("attention", attention(6, 1, 40, 16, 33, 0.15, 20, kv_from=0), None),
    ],
}
# nothing is a multiple of 4: width 50, heads of 6 and 10, a recurrence of 7 channels, experts of 9, a vocabulary of 53
GE = {
    "architecture": "Giforax", "vocab": 53, "width": 50, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
    "layers": [
        layer("attention", attention(3, 3, 6, 10, 9, 0.4, 2), moe(3, 2, 9, 1.0, shared=5)),
        layer("mingru", {"width": 7}, moe(2, 1, 3, 2.0)),
        layer("attention", attention(6, 3, 6, 10, 21, 0.4, 2, kv_from=0), None),
    ],
}
CONFIGS = {"GA": (GA, 21), "GB": (GB, 22), "GC": (GC, 23), "GD": (GD, 24), "GE": (GE, 25)}
