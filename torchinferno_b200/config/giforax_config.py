"""Typed configuration of the Giforax design, read from a checkpoint's ``config.json``.

The file names the design under ``architecture``, gives the global sizes (``vocab``, ``width``), the norms' ``eps``,
the embedding's multiplier (``embedding.scale``) and a list ``layers`` whose entries each name a mixer ``type`` with
its sizes (``mixer``) and a feed-forward (``mlp``, or null).  An attention mixer may name an earlier layer whose keys
and values it reads (``kv_from``).  No size or constant has a default: a missing key is an error that names it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

from torchinferno_b200.config.model_config import ConfigError

MIXERS = ("attention", "mingru")
# The design names no limit.  Positions are exact in the 32-bit floats the rotary angles are made from up to 2^24; the
# limit given here is what block tables and default pools are sized by when the user names none.
MAX_POSITIONS = 1 << 20


def _need(data: Mapping[str, Any], key: str, where: str) -> Any:
    if not isinstance(data, Mapping) or key not in data:
        raise ConfigError(f"config.json: {where} lacks {key!r}")
    return data[key]


def _positive(data: Mapping[str, Any], key: str, where: str) -> int:
    value = _need(data, key, where)
    if not isinstance(value, int) or isinstance(value, bool) or value < 1:
        raise ConfigError(f"config.json: {where}.{key} must be a positive integer, got {value!r}")
    return value


def _positive_float(data: Mapping[str, Any], key: str, where: str) -> float:
    value = _need(data, key, where)
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not float(value) > 0:
        raise ConfigError(f"config.json: {where}.{key} must be a positive number, got {value!r}")
    return float(value)


@dataclass(frozen=True)
class GiforaxLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Mapping[str, Any] | None

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], index: int) -> "GiforaxLayer":
        where = f"layers[{index}]"
        kind = _need(data, "type", where)
        if kind not in MIXERS:
            raise ConfigError(f"config.json: {where}.type={kind!r}; known mixers: {list(MIXERS)}")
        mixer = _need(data, "mixer", where)
        at = where + ".mixer"
        if kind == "mingru":
            _positive(mixer, "width", at)
        else:
            heads, kv_heads = _positive(mixer, "heads", at), _positive(mixer, "kv_heads", at)
            if heads % kv_heads:
                raise ConfigError(f"config.json: {at}.heads must be a multiple of kv_heads")
            dim = _positive(mixer, "dim", at)
            _positive(mixer, "vdim", at)
            _positive_float(mixer, "scale", at)
            _positive(_need(mixer, "mask", at), "size", at + ".mask")
            rot = _need(mixer, "rot", at)
            _positive_float(rot, "base", at + ".rot")
            dims = _positive(rot, "dims", at + ".rot")
            if dims % 2 or dims > dim:
                raise ConfigError(f"config.json: {at}.rot.dims must be even and at most dim")
            source = mixer.get("kv_from")
            if source is not None and (not isinstance(source, int) or isinstance(source, bool) or not 0 <= source < index):
                raise ConfigError(f"config.json: {at}.kv_from must name an earlier layer, got {source!r}")
        mlp = data.get("mlp")
        if mlp is not None:
            at = where + ".mlp"
            form = _need(mlp, "kind", at)
            if form != "moe":
                raise ConfigError(f"config.json: {at}.kind={form!r}; known: ['moe']")
            router = _need(mlp, "router", at)
            experts, top = _positive(router, "experts", at + ".router"), _positive(router, "top", at + ".router")
            if top > experts:
                raise ConfigError(f"config.json: {at}.router.top exceeds the number of experts")
            for part in ("expert", "shared"):
                if part == "shared" and mlp.get("shared") is None:
                    continue
                _positive(_need(mlp, part, at), "ff", f"{at}.{part}")
                _positive_float(mlp[part], "limit", f"{at}.{part}")
        return cls(kind, dict(mixer), None if mlp is None else dict(mlp))


@dataclass(frozen=True)
class GiforaxConfig:
    vocab: int
    width: int
    layers: tuple[GiforaxLayer, ...]
    eps: float
    embedding_scale: float
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "GiforaxConfig":
        where = "the model"
        layers = _need(data, "layers", where)
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: layers must be a list with at least one entry")
        typed = tuple(GiforaxLayer.from_dict(entry, i) for i, entry in enumerate(layers))
        for i, layer in enumerate(typed):
            source = layer.mixer.get("kv_from") if layer.type == "attention" else None
            if source is None:
                continue
            other = typed[source]
            if other.type != "attention" or other.mixer.get("kv_from") is not None:
                raise ConfigError(f"config.json: layers[{i}].mixer.kv_from={source}: that layer has no keys and values of its own")
            for key in ("kv_heads", "dim", "vdim"):
                if other.mixer[key] != layer.mixer[key]:
                    raise ConfigError(f"config.json: layers[{i}] reads the keys of layers[{source}], whose {key} differs")
        return cls(vocab=_positive(data, "vocab", where), width=_positive(data, "width", where), layers=typed,
                   eps=_positive_float(_need(data, "norm", where), "eps", "norm"),
                   embedding_scale=float(_need(_need(data, "embedding", where), "scale", "embedding")), raw=dict(data))

    def to_dict(self) -> dict[str, Any]:
        return dict(self.raw)
