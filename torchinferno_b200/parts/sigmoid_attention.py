"""Attention with sigmoid weights, a per-head bias and a per-head output gate, over the paged cache.

q = W_q x, k = W_k x, v = W_v x (no biases); q and k get the position encoding (``position``: a rotary part, possibly on
part of a head) and are then, with ``qk_norm_eps``, divided by their root mean square over the head (no weight);
score = q . k * scale; a key j is visible to a query i when j <= i and, with ``chunk``, both lie in the same run of
``chunk`` positions counted from the start of the sequence (and, with ``window``, i - j < window); the weight of a
visible key is sigmoid(score + bias[h]) and nothing is normalised over the keys; head h's output is multiplied by
sigmoid(W_g x)_h; then the output projection.  Keys may be wider or narrower than values.  Query head h reads
key/value head h // (heads / kv_heads).

``own_kv=False``: the layer has no key and value projections; it reads what another layer call stored in the cache
it is given (``ctx.kv.writes`` False), keys as they were cached there, after rotation and norm.

All input projections are one product; the kernels are in csrc/sigmoid_attention.cu.
"""
from __future__ import annotations

from typing import Mapping

import torch

from torchinferno_b200.kernels import ops
from torchinferno_b200.kernels.gemm import LinearWeight, linear
from torchinferno_b200.parts.base import (CacheSpec, LayerContext, Mixer, PartSpec, WeightSpec, build_part,
                                          register_part)


class SigmoidAttention(Mixer):
    capturable = True

    def __init__(self, *, hidden_size: int, heads: int, kv_heads: int, dim: int, value_dim: int, scale: float,
                 position: PartSpec | Mapping, qk_norm_eps: float | None = None, chunk: int | None = None,
                 window: int | None = None, head_bias: bool = True, head_gate: bool = True, own_kv: bool = True,
                 q_name: str = "q", k_name: str = "k", v_name: str = "v", o_name: str = "o", bias_name: str = "pb",
                 gate_name: str = "g", dtype: torch.dtype, device: torch.device) -> None:
        super().__init__(dtype=dtype, device=device)
        if heads % kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        if (chunk is not None and chunk < 1) or (window is not None and window < 1):
            raise ValueError("chunk and window are positive when given")
        self.hidden_size, self.heads, self.kv_heads, self.dim, self.value_dim = hidden_size, heads, kv_heads, dim, value_dim
        self.scale, self.qk_norm_eps, self.chunk, self.window = float(scale), qk_norm_eps, chunk, window
        self.head_bias, self.head_gate, self.own_kv = bool(head_bias), bool(head_gate), bool(own_kv)
        self.names = {"q": q_name, "k": k_name, "v": v_name, "o": o_name, "pb": bias_name, "g": gate_name}
        if not isinstance(position, PartSpec):
            position = PartSpec(**position)
        self.position = build_part("position", position, dtype=dtype, device=device)
        self.in_weight: LinearWeight | None = None
        self.o_weight: LinearWeight | None = None
        self.bias: torch.Tensor | None = None
        qw, kw, vw = heads * dim, kv_heads * dim, kv_heads * value_dim
        self.k_off = qw if own_kv else -1
        self.v_off = qw + kw if own_kv else -1
        self.g_off = qw + (kw + vw if own_kv else 0)

    def weight_specs(self) -> list[WeightSpec]:
        n, w = self.names, self.hidden_size
        std = w ** -0.5                     # (random weights: rows of about unit size from normed input)
        specs = [WeightSpec(n["q"], (self.heads * self.dim, w), std=std)]
        if self.own_kv:
            specs += [WeightSpec(n["k"], (self.kv_heads * self.dim, w), std=std),
                      WeightSpec(n["v"], (self.kv_heads * self.value_dim, w), std=std)]
        if self.head_bias:
            specs.append(WeightSpec(n["pb"], (self.heads,), std=1.0, role="vector"))
        if self.head_gate:
            specs.append(WeightSpec(n["g"], (self.heads, w), std=std))
        specs.append(WeightSpec(n["o"], (w, self.heads * self.value_dim), std=(self.heads * self.value_dim) ** -0.5))
        return specs

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        rows = [weights[n["q"]]] + ([weights[n["k"]], weights[n["v"]]] if self.own_kv else []) \
            + ([weights[n["g"]]] if self.head_gate else [])
        total = sum(r.shape[0] for r in rows)
        if total % 8:       # (rows of the product's output then start on 16-byte boundaries in bfloat16)
            rows.append(torch.zeros((8 - total % 8, self.hidden_size), dtype=rows[0].dtype, device=rows[0].device))
        self.in_weight = LinearWeight(torch.cat(rows, dim=0), few_rows_tcgen05=None)
        self.o_weight = LinearWeight(weights[n["o"]], few_rows_tcgen05=None)
        self.bias = weights[n["pb"]].to(torch.float32).contiguous() if self.head_bias else None

    def cache_spec(self) -> CacheSpec:
        # (no window of the cache's own: pages are kept while the request lives)
        return CacheSpec(self.kv_heads, self.dim, None, None if self.value_dim == self.dim else self.value_dim)

    def forward(self, x: torch.Tensor, ctx: LayerContext) -> torch.Tensor:
        kv, batch = ctx.kv, ctx.batch
        if kv is None or kv.keys is None or kv.values is None:
            raise RuntimeError("this attention needs a cache binding with keys and values")
        if kv.writes != self.own_kv:
            raise RuntimeError("a layer with key and value projections writes its cache layer; one without reads another's")
        n, h, g = x.shape[0], self.heads, self.kv_heads
        proj = linear(x, self.in_weight)
        q = torch.empty((n, h * self.dim), dtype=x.dtype, device=x.device)
        inv_freq, rot_dim, interleaved = self.position.rotary_table()
        ops.qk_norm_append(proj, 0, self.k_off, self.v_off, q, kv.keys if self.own_kv else None,
                           kv.values if self.own_kv else None, batch.positions, batch.token_slot, kv.block_table, inv_freq,
                           h, g, self.dim, self.value_dim, rot_dim=rot_dim, interleaved=interleaved,
                           eps=-1.0 if self.qk_norm_eps is None else self.qk_norm_eps, error_word=ctx.error_word)
        out = torch.empty((n, h * self.value_dim), dtype=x.dtype, device=x.device)
        ops.sigmoid_attention(q, kv.keys, kv.values, out, batch.q_start, batch.kv_start, batch.slots, kv.block_table,
                              batch.n_entries, batch.max_q_len, h, g, scale=self.scale, chunk=self.chunk or 0,
                              window=self.window or 0, head_bias=self.bias,
                              gate=proj[:, self.g_off:self.g_off + h] if self.head_gate else None, error_word=ctx.error_word,
                              max_kv_len=batch.max_kv_len)
        return linear(out, self.o_weight)


register_part("mixer", "sigmoid_attention", SigmoidAttention)
