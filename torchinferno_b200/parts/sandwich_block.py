"""A block with a norm before and after each sublayer, optionally ending in an average over depth:

    x <- x + norm_b(mixer(norm_a(x)));   x <- x + norm_d(feed_forward(norm_c(x)))      (the second line may be absent)
    X_new = x;   x <- sum over j <= this layer of  w[j] * X_j                           (``depth_average``)

where X_0 is the embedding output and X_(i+1) the result of layer i before its average.  The average needs every
earlier result: the model keeps them (``ModelSpec.history_depth`` slices of the residual's size, handed over as
``ResidualStream.history``); layer i works in slice i + 1 and leaves the stream in slice i + 2.  The weights w
(``depth_average`` of them: i + 2 for layer i) are the block's own tensor.

The norms are layer norms with weight and bias.  What follows a sublayer runs as one launch: the norm of its output,
the sum into the 32-bit residual and either the norm that opens the next sublayer or the depth average
(csrc/layernorm.cu).
"""
from __future__ import annotations

from typing import Mapping

import torch

from torchinferno_b200.kernels import ops
from torchinferno_b200.parts.base import (Block, LayerContext, Part, PartSpec, ResidualStream, WeightSpec, build_part,
                                          register_part)
from torchinferno_b200.parts.norm import LayerNorm


def _spec(value: PartSpec | Mapping | None) -> PartSpec | None:
    return value if value is None or isinstance(value, PartSpec) else PartSpec(**value)


class SandwichBlock(Block):
    def __init__(self, *, mixer: PartSpec, mixer_norm: PartSpec, mixer_out_norm: PartSpec, feed_forward: PartSpec | None = None,
                 feed_forward_norm: PartSpec | None = None, feed_forward_out_norm: PartSpec | None = None,
                 depth_average: int | None = None, depth_name: str = "dwa", dtype: torch.dtype, device: torch.device) -> None:
        super().__init__(dtype=dtype, device=device)
        self.specs = {"mixer": _spec(mixer), "mixer_norm": _spec(mixer_norm), "mixer_out_norm": _spec(mixer_out_norm),
                      "feed_forward": _spec(feed_forward), "feed_forward_norm": _spec(feed_forward_norm),
                      "feed_forward_out_norm": _spec(feed_forward_out_norm)}
        if feed_forward is not None and (feed_forward_norm is None or feed_forward_out_norm is None):
            raise ValueError("a feed-forward needs its two norms")
        self.mixer = build_part("mixer", self.specs["mixer"], dtype=dtype, device=device)
        self.feed_forward = None if feed_forward is None else \
            build_part("feed_forward", self.specs["feed_forward"], dtype=dtype, device=device)
        self.norms: dict[str, LayerNorm] = {}
        for key in ("mixer_norm", "mixer_out_norm", "feed_forward_norm", "feed_forward_out_norm"):
            if self.specs[key] is None or (self.feed_forward is None and key.startswith("feed_forward")):
                continue
            norm = build_part("norm", self.specs[key], dtype=dtype, device=device)
            if not isinstance(norm, LayerNorm):
                raise ValueError(f"{key}: this block fuses layer norms with the sums around them; got {type(norm).__name__}")
            self.norms[key] = norm
        if len({norm.eps for norm in self.norms.values()}) != 1:
            raise ValueError("the norms of one block share their eps")
        self.eps = self.norms["mixer_norm"].eps
        if depth_average is not None and depth_average < 2:
            raise ValueError("a depth average reads at least the embedding output and this layer's result")
        self.depth_average, self.depth_name = depth_average, depth_name
        self.depth_weight: torch.Tensor | None = None

    # (the block owns the weights of its depth average itself)
    def weight_specs(self) -> list[WeightSpec]:
        if self.depth_average is None:
            return []
        return [WeightSpec(self.depth_name, (self.depth_average,), std=0.5, role="vector")]

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        if self.depth_average is not None:
            self.depth_weight = weights[self.depth_name].to(torch.float32).contiguous()

    def named_parts(self) -> list[tuple[str, Part]]:
        parts: list[tuple[str, Part]] = [(self.specs[key].prefix, norm) for key, norm in self.norms.items()]
        parts.append((self.specs["mixer"].prefix, self.mixer))
        if self.feed_forward is not None:
            parts.append((self.specs["feed_forward"].prefix, self.feed_forward))
        parts.append(("", self))
        return parts

    def forward(self, stream: ResidualStream, ctx: LayerContext) -> None:
        residual = stream.settle()
        stream.activation_copy = None
        n, width = residual.shape
        norms, eps = self.norms, self.eps
        history = coef = None
        count = 0
        if self.depth_average is not None:
            history, coef, count = stream.history, self.depth_weight, self.depth_average
            if history is None or count >= history.shape[0] or history[count - 1].data_ptr() != residual.data_ptr():
                raise RuntimeError("the depth average needs the model's history of layer outputs, with the stream in its slice "
                                   f"{count - 1} (ModelSpec.history_depth)")

        def pair(key):
            return norms[key].weight, norms[key].bias

        rows = stream.normed(norms["mixer_norm"])
        mixed = self.mixer.forward(rows, ctx)
        if self.feed_forward is None:
            ops.layernorm_tail(residual, eps, y=mixed, y_norm=pair("mixer_out_norm"), history=history, coef=coef, count=count)
        else:
            rows = torch.empty((n, width), dtype=stream.dtype, device=residual.device)
            ops.layernorm_tail(residual, eps, y=mixed, y_norm=pair("mixer_out_norm"), out=rows, out_norm=pair("feed_forward_norm"))
            fed = self.feed_forward.forward(rows, ctx)
            ops.layernorm_tail(residual, eps, y=fed, y_norm=pair("feed_forward_out_norm"), history=history, coef=coef, count=count)
        if history is not None:
            stream.residual = history[count]


register_part("block", "sandwich", SandwichBlock)
