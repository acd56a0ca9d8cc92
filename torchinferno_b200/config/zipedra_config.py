"""Typed configuration of the Zipedra design, read from a checkpoint's ``config.json``.

The file names the design under ``architecture``, gives the global sizes (``vocab``, ``width``), the norm's
``eps``, the output ``logit_scale``, and a list ``layers`` whose entries each name a mixer ``type`` with its sizes
(``mixer``) and a feed-forward (``mlp``, or null).  ``loop`` (optional) makes layers start .. stop-1 run ``times``
times; ``token_side`` (optional) gives the width of the per-layer token input.  No size has a default: a
missing key is an error that names it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

from torchinferno_b200.config.model_config import ConfigError

MIXERS = ("lightning", "latent_attention")
FEED_FORWARDS = ("dense", "moe")
# The design names no limit.  Positions are exact in the 32-bit floats the rotary angles are made from up to 2^24; the
# limit given here is what block tables and default pools are sized by when the user names none
# (EngineConfig.max_model_len).
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


@dataclass(frozen=True)
class ZipedraLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Mapping[str, Any] | None

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], index: int) -> "ZipedraLayer":
        where = f"layers[{index}]"
        kind = _need(data, "type", where)
        if kind not in MIXERS:
            raise ConfigError(f"config.json: {where}.type={kind!r}; known mixers: {list(MIXERS)}")
        mixer = _need(data, "mixer", where)
        at = where + ".mixer"
        if kind == "lightning":
            heads = _positive(mixer, "heads", at)
            _positive(mixer, "dim", at), _positive(mixer, "vdim", at)
            decay = _need(mixer, "decay", at)
            if not isinstance(decay, (list, tuple)) or len(decay) != heads or not all(0.0 < float(d) <= 1.0 for d in decay):
                raise ConfigError(f"config.json: {at}.decay must hold one constant in (0, 1] per head")
        else:
            for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank"):
                _positive(mixer, key, at)
            float(_need(mixer, "scale", at))
            rot = _need(mixer, "rot", at)
            if not float(_need(rot, "base", at + ".rot")) > 0:
                raise ConfigError(f"config.json: {at}.rot.base must be positive")
            dims = _positive(rot, "dims", at + ".rot")
            if dims % 2 or dims > mixer["rot_dim"]:
                raise ConfigError(f"config.json: {at}.rot.dims must be even and at most rot_dim")
        mlp = data.get("mlp")
        if mlp is not None:
            at = where + ".mlp"
            form = _need(mlp, "kind", at)
            if form not in FEED_FORWARDS:
                raise ConfigError(f"config.json: {at}.kind={form!r}; known: {list(FEED_FORWARDS)}")
            if form == "dense":
                _positive(mlp, "ff", at)
            else:
                router = _need(mlp, "router", at)
                experts, top = _positive(router, "experts", at + ".router"), _positive(router, "top", at + ".router")
                if top > experts:
                    raise ConfigError(f"config.json: {at}.router.top exceeds the number of experts")
                _positive(_need(mlp, "expert", at), "ff", at + ".expert")
                if mlp.get("shared") is not None:
                    _positive(mlp["shared"], "ff", at + ".shared")
        return cls(kind, dict(mixer), None if mlp is None else dict(mlp))


@dataclass(frozen=True)
class ZipedraConfig:
    vocab: int
    width: int
    layers: tuple[ZipedraLayer, ...]
    eps: float
    logit_scale: float
    loop: tuple[int, int, int] | None          # (start, stop, times)
    token_side_dim: int | None
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "ZipedraConfig":
        where = "the model"
        layers = _need(data, "layers", where)
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: layers must be a list with at least one entry")
        typed = tuple(ZipedraLayer.from_dict(entry, i) for i, entry in enumerate(layers))
        eps = float(_need(_need(data, "norm", where), "eps", "norm"))
        if not eps > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        loop = None
        if data.get("loop") is not None:
            block = data["loop"]
            start, stop, times = int(_need(block, "start", "loop")), int(_need(block, "stop", "loop")), _positive(block, "times", "loop")
            if not 0 <= start < stop <= len(typed):
                raise ConfigError(f"config.json: loop.start .. loop.stop = {start} .. {stop} is no range of the {len(typed)} layers")
            loop = (start, stop, times)
        side = None if data.get("token_side") is None else _positive(data["token_side"], "dim", "token_side")
        return cls(vocab=_positive(data, "vocab", where), width=_positive(data, "width", where), layers=typed, eps=eps,
                   logit_scale=float(data.get("logit_scale", 1.0)), loop=loop, token_side_dim=side, raw=dict(data))

    def to_dict(self) -> dict[str, Any]:
        return dict(self.raw)
