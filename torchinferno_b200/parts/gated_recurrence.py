"""An element-wise gated recurrence whose gates read only the current token (the minimal GRU form).

z = sigmoid(W_z x + b_z) and u = W_x x + b_x, both ``width`` wide; the candidate is u + 1/2 where u >= 0 and
sigmoid(u) where u < 0; element by element S_t = (1 - z) S_(t-1) + z * candidate; the output is W_o (S_t * silu(W_g x)).
S starts at zero for a new request, lives in 32-bit in the cache manager's state slots and is carried from step to
step; the mixer keeps no keys.  The three input projections are one product; the scan (csrc/gated_recurrence.cu)
takes the step's whole ragged batch and reads it through its device arrays only.
"""
from __future__ import annotations

from typing import Mapping

import torch

from torchinferno_b200.kernels import ops
from torchinferno_b200.kernels.gemm import LinearWeight, linear
from torchinferno_b200.parts.base import LayerContext, Mixer, StateSpec, WeightSpec, register_part


class MinimalGRU(Mixer):
    capturable = True       # (state is read and written by the kernel through the slots array)

    def __init__(self, *, hidden_size: int, width: int, output_gate: bool = True, z_name: str = "z", x_name: str = "x",
                 g_name: str = "g", o_name: str = "o", bias_suffix: str = ".b", dtype: torch.dtype, device: torch.device) -> None:
        super().__init__(dtype=dtype, device=device)
        self.hidden_size, self.width, self.output_gate = hidden_size, width, bool(output_gate)
        self.names = {"z": z_name, "x": x_name, "g": g_name, "o": o_name, "zb": z_name + bias_suffix, "xb": x_name + bias_suffix}
        self.in_weight: LinearWeight | None = None
        self.o_weight: LinearWeight | None = None

    def weight_specs(self) -> list[WeightSpec]:
        n, w, c = self.names, self.hidden_size, self.width
        std = w ** -0.5
        specs = [WeightSpec(n["z"], (c, w), std=std), WeightSpec(n["zb"], (c,), std=0.5, role="vector"),
                 WeightSpec(n["x"], (c, w), std=std), WeightSpec(n["xb"], (c,), std=0.5, role="vector")]
        if self.output_gate:
            specs.append(WeightSpec(n["g"], (c, w), std=std))
        specs.append(WeightSpec(n["o"], (w, c), std=c ** -0.5))
        return specs

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        rows = [weights[n["z"]], weights[n["x"]]] + ([weights[n["g"]]] if self.output_gate else [])
        total = sum(r.shape[0] for r in rows)
        if total % 8:
            rows.append(torch.zeros((8 - total % 8, self.hidden_size), dtype=rows[0].dtype, device=rows[0].device))
        self.in_weight = LinearWeight(torch.cat(rows, dim=0), few_rows_tcgen05=None)
        self.o_weight = LinearWeight(weights[n["o"]], few_rows_tcgen05=None)
        self.bias_z = weights[n["zb"]].to(torch.float32).contiguous()
        self.bias_u = weights[n["xb"]].to(torch.float32).contiguous()

    def state_spec(self) -> StateSpec:
        return StateSpec((self.width,), torch.float32)

    def forward(self, x: torch.Tensor, ctx: LayerContext) -> torch.Tensor:
        if ctx.state is None:
            raise RuntimeError("the recurrence needs a state tensor")
        batch, c = ctx.batch, self.width
        proj = linear(x, self.in_weight)
        rows = torch.empty((x.shape[0], c), dtype=x.dtype, device=x.device)
        ops.gated_recurrence(proj, 0, c, 2 * c if self.output_gate else -1, self.bias_z, self.bias_u, ctx.state, batch.q_start,
                             batch.slots, rows, batch.n_entries, batch.max_q_len)
        return linear(rows, self.o_weight)


register_part("mixer", "min_gru", MinimalGRU)
