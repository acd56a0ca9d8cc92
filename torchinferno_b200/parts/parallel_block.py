"""A block whose mixer and feed-forward read the same normed rows:
    h = norm(x);  x <- x + (mixer(h) + feed_forward(h))
(the feed-forward may be absent), optionally followed by a stage on the residual (a per-layer token input).
Both outputs are summed into the 32-bit residual by one kernel, which also leaves the new rows in the activation
type for the stage that follows.
"""
from __future__ import annotations

from typing import Mapping

import torch

from torchinferno_b200.kernels import ops
from torchinferno_b200.parts.base import Block, LayerContext, Part, PartSpec, ResidualStream, build_part, register_part


def _spec(value: PartSpec | Mapping | None) -> PartSpec | None:
    return value if value is None or isinstance(value, PartSpec) else PartSpec(**value)


class ParallelBlock(Block):
    def __init__(self, *, mixer: PartSpec, norm: PartSpec, feed_forward: PartSpec | None = None,
                 after: PartSpec | None = None, dtype: torch.dtype, device: torch.device) -> None:
        super().__init__(dtype=dtype, device=device)
        self.specs = {"norm": _spec(norm), "mixer": _spec(mixer), "feed_forward": _spec(feed_forward), "after": _spec(after)}
        self.norm = build_part("norm", self.specs["norm"], dtype=dtype, device=device)
        self.mixer = build_part("mixer", self.specs["mixer"], dtype=dtype, device=device)
        self.feed_forward = None if feed_forward is None else \
            build_part("feed_forward", self.specs["feed_forward"], dtype=dtype, device=device)
        self.after = None if after is None else build_part("stream_stage", self.specs["after"], dtype=dtype, device=device)

    def named_parts(self) -> list[tuple[str, Part]]:
        parts = [(self.specs["norm"].prefix, self.norm), (self.specs["mixer"].prefix, self.mixer)]
        if self.feed_forward is not None:
            parts.append((self.specs["feed_forward"].prefix, self.feed_forward))
        if self.after is not None:
            parts.append((self.specs["after"].prefix, self.after))
        return parts

    def forward(self, stream: ResidualStream, ctx: LayerContext) -> None:
        rows = stream.normed(self.norm)
        mixed = self.mixer.forward(rows, ctx)
        fed = None if self.feed_forward is None else self.feed_forward.forward(rows, ctx)
        copy = None
        if self.after is not None and stream.dtype != torch.float32:
            copy = torch.empty(stream.residual.shape, dtype=stream.dtype, device=stream.residual.device)
        ops.add_pair(stream.residual, mixed, fed, copy)
        stream.activation_copy = copy
        if self.after is not None:
            self.after.forward(stream, ctx)


register_part("block", "parallel", ParallelBlock)
