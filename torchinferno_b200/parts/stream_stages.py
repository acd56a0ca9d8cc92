"""Stages that work on the residual stream outside the mixer / feed-forward pair.

``token_side``  a small per-layer input that depends on the token itself: e = a slice of a second embedding
                table (one table for the whole model, shared by the layers, each reading its own columns),
                g = gelu_tanh(W_gate x) * e, y = W_proj g, x <- x + y / rms(y) * w.  It runs inside a block, after
                the sublayers' sum (parts/parallel_block.py), and reads the residual itself, not a normed copy.
``loop_input``  before a pass over a range of layers that runs several times: x <- W_in [x ; x0] + step[t], with
                x0 the embedding output and t the number of the pass (the schedule's stage-call argument).
Sums into the residual and the unit norm are fp32.
"""
from __future__ import annotations

from typing import Mapping

import torch

from torchinferno_b200.kernels import ops
from torchinferno_b200.kernels.gemm import LinearWeight, linear
from torchinferno_b200.parts.base import LayerContext, ResidualStream, StreamStage, WeightSpec, register_part


def _activation_rows(stream: ResidualStream) -> torch.Tensor:
    """The settled residual in the activation type (the copy its last writer left, or a cast)."""
    residual = stream.settle()
    if stream.dtype == torch.float32:
        return residual
    if stream.activation_copy is not None:
        return stream.activation_copy
    return ops.cast(residual, torch.empty(residual.shape, dtype=stream.dtype, device=residual.device))


class TokenSideInput(StreamStage):
    def __init__(self, *, width: int, dim: int, index: int, vocab_size: int, table_width: int, eps: float,
                 table_name: str = "side.embed", gate_name: str = "gate", proj_name: str = "proj", norm_name: str = "norm",
                 dtype: torch.dtype, device: torch.device) -> None:
        super().__init__(dtype=dtype, device=device)
        if (index + 1) * dim > table_width:
            raise ValueError("the table has no columns for this index")
        self.width, self.dim, self.index, self.vocab_size, self.table_width, self.eps = width, dim, index, vocab_size, table_width, float(eps)
        self.names = (table_name, gate_name, proj_name, norm_name)

    def weight_specs(self) -> list[WeightSpec]:
        _, gate, proj, norm = self.names
        return [WeightSpec(gate, (self.dim, self.width), std=0.2), WeightSpec(proj, (self.width, self.dim), std=0.2),
                WeightSpec(norm, (self.width,), init="ones", role="vector")]

    def shared_weight_specs(self) -> list[WeightSpec]:
        return [WeightSpec(self.names[0], (self.vocab_size, self.table_width), std=1.0)]

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        table, gate, proj, norm = self.names
        self.table = weights[table]
        self.gate_weight = LinearWeight(weights[gate], few_rows_tcgen05=False)
        self.proj_weight = LinearWeight(weights[proj], few_rows_tcgen05=False)
        self.norm_weight = weights[norm].to(torch.float32).contiguous()

    def forward(self, stream: ResidualStream, ctx: LayerContext) -> None:
        rows = _activation_rows(stream)
        stream.activation_copy = None
        gated = torch.empty((rows.shape[0], self.dim), dtype=rows.dtype, device=rows.device)
        ops.gelu_gate_table(linear(rows, self.gate_weight), ctx.batch.token_ids, self.table, self.index * self.dim, gated)
        y = linear(gated, self.proj_weight, out_dtype=torch.float32)
        ops.unit_norm_add(stream.residual, y, self.norm_weight, self.eps)


class LoopInput(StreamStage):
    capturable = True

    def __init__(self, *, width: int, passes: int, in_name: str = "in", step_name: str = "step",
                 dtype: torch.dtype, device: torch.device) -> None:
        super().__init__(dtype=dtype, device=device)
        self.width, self.passes, self.names = width, passes, (in_name, step_name)

    def weight_specs(self) -> list[WeightSpec]:
        return [WeightSpec(self.names[0], (self.width, 2 * self.width), std=(2 * self.width) ** -0.5),
                WeightSpec(self.names[1], (self.passes, self.width), std=0.5, role="vector")]

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        self.in_weight = LinearWeight(weights[self.names[0]], few_rows_tcgen05=None)
        self.step = weights[self.names[1]].to(torch.float32).contiguous()

    def forward(self, stream: ResidualStream, ctx: LayerContext) -> None:
        if stream.origin is None:
            raise RuntimeError("loop_input needs the embedding output (ModelSpec.keeps_embedding_output)")
        if not 0 <= ctx.call_arg < self.passes:
            raise RuntimeError(f"pass {ctx.call_arg} of {self.passes}")
        residual = stream.settle()
        stream.activation_copy = None
        pair = torch.empty((residual.shape[0], 2 * self.width), dtype=stream.dtype, device=residual.device)
        ops.pair_rows(residual, stream.origin, pair)
        linear(pair, self.in_weight, out_dtype=torch.float32, out=residual)
        ops.add_vector(residual, self.step[ctx.call_arg])


register_part("stream_stage", "token_side", TokenSideInput)
register_part("stream_stage", "loop_input", LoopInput)
