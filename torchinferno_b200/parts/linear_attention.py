"""Linear attention with a fixed decay per head, over state kept per request.

Per head, with q, k of ``key_dim`` and v of ``value_dim`` elements (after an optional activation):
    S_t = decay * S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t
The heads' outputs, side by side, are optionally RMS-normed together (plain weight) and multiplied by
sigmoid(W_g x), then projected by W_o.  S lives in 32-bit in the cache manager's state slots (zero for a new
request) and is carried from step to step; it does not grow with the context, and the mixer keeps no keys.
The four input projections run as one product; the kernel (csrc/linear_attention.cu) takes the step's whole
ragged batch, prompt portions and single tokens alike, and reads the batch through its device arrays only.
"""
from __future__ import annotations

from typing import Mapping, Sequence

import torch

from torchinferno_b200.kernels import ops
from torchinferno_b200.kernels.gemm import LinearWeight, linear
from torchinferno_b200.parts.base import LayerContext, Mixer, StateSpec, WeightSpec, register_part


class DecayLinearAttention(Mixer):
    capturable = True       # (state is read and written by the kernel through the slots array)

    def __init__(self, *, hidden_size: int, heads: int, key_dim: int, value_dim: int, decay: Sequence[float],
                 activation: str = "silu", output_norm: bool = True, eps: float = 1e-6, gate: bool = True,
                 q_name: str = "q", k_name: str = "k", v_name: str = "v", g_name: str = "g", o_name: str = "o",
                 norm_name: str = "norm", dtype: torch.dtype, device: torch.device) -> None:
        super().__init__(dtype=dtype, device=device)
        if len(decay) != heads:
            raise ValueError(f"{len(decay)} decay constants for {heads} heads")
        if activation not in ("silu", "none"):
            raise ValueError(f"unknown activation {activation!r}")
        self.hidden_size, self.heads, self.key_dim, self.value_dim = hidden_size, heads, key_dim, value_dim
        self.decay = [float(d) for d in decay]
        self.activation, self.output_norm, self.eps, self.gate = activation, bool(output_norm), float(eps), bool(gate)
        self.names = {"q": q_name, "k": k_name, "v": v_name, "g": g_name, "o": o_name, "norm": norm_name}
        self.in_weight: LinearWeight | None = None
        self.o_weight: LinearWeight | None = None
        self.norm_weight: torch.Tensor | None = None
        self.powers: torch.Tensor | None = None

    def weight_specs(self) -> list[WeightSpec]:
        n, qk, vv = self.names, self.heads * self.key_dim, self.heads * self.value_dim
        std = self.hidden_size ** -0.5          # (random weights: rows of about unit size from normed input)
        specs = [WeightSpec(n["q"], (qk, self.hidden_size), std=std), WeightSpec(n["k"], (qk, self.hidden_size), std=std),
                 WeightSpec(n["v"], (vv, self.hidden_size), std=std)]
        if self.gate:
            specs.append(WeightSpec(n["g"], (vv, self.hidden_size), std=std))
        specs.append(WeightSpec(n["o"], (self.hidden_size, vv), std=vv ** -0.5))
        if self.output_norm:
            specs.append(WeightSpec(n["norm"], (vv,), init="ones", role="vector"))
        return specs

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        rows = [weights[n["q"]], weights[n["k"]], weights[n["v"]]] + ([weights[n["g"]]] if self.gate else [])
        self.in_weight = LinearWeight(torch.cat(rows, dim=0), few_rows_tcgen05=None)
        self.o_weight = LinearWeight(weights[n["o"]], few_rows_tcgen05=None)
        self.norm_weight = weights[n["norm"]].to(torch.float32).contiguous() if self.output_norm else None
        device = weights[n["q"]].device
        chunk = ops.linear_attention_chunk(self.key_dim, self.value_dim) if device.type == "cuda" else 1
        if chunk < 1:
            raise ValueError(f"heads of {self.key_dim} x {self.value_dim} do not fit the linear attention kernel")
        # decay^m for m = 0 .. chunk, made in double precision
        table = torch.tensor(self.decay, dtype=torch.float64)[:, None] ** torch.arange(chunk + 1, dtype=torch.float64)[None, :]
        self.powers = table.to(torch.float32).contiguous().to(device)

    def state_spec(self) -> StateSpec:
        return StateSpec((self.heads, self.key_dim, self.value_dim), torch.float32)

    def forward(self, x: torch.Tensor, ctx: LayerContext) -> torch.Tensor:
        if ctx.state is None:
            raise RuntimeError("linear attention needs a state tensor")
        batch, n = ctx.batch, x.shape[0]
        qk, vv = self.heads * self.key_dim, self.heads * self.value_dim
        proj = linear(x, self.in_weight)
        q, k, v = proj[:, :qk], proj[:, qk:2 * qk], proj[:, 2 * qk:2 * qk + vv]
        mixed = torch.empty((n, vv), dtype=torch.float32, device=x.device)
        ops.linear_attention(q, k, v, mixed, ctx.state, self.powers, batch.q_start, batch.slots, batch.n_entries, self.heads,
                             self.key_dim, self.value_dim, silu=self.activation == "silu")
        if self.gate:
            rows = torch.empty((n, vv), dtype=x.dtype, device=x.device)
            ops.sigmoid_gate(mixed, proj[:, 2 * qk + vv:], rows, self.norm_weight, self.eps)
        elif self.output_norm:
            rows = ops.rmsnorm(mixed, self.norm_weight, self.eps, torch.empty_like(mixed))
            rows = rows if x.dtype == torch.float32 else ops.cast(rows, torch.empty((n, vv), dtype=x.dtype, device=x.device))
        else:
            rows = mixed if x.dtype == torch.float32 else ops.cast(mixed, torch.empty((n, vv), dtype=x.dtype, device=x.device))
        return linear(rows, self.o_weight)


register_part("mixer", "decay_linear_attention", DecayLinearAttention)
