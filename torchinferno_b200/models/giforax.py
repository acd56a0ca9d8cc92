"""Giforax as a description made of parts.

The embedding output is multiplied by a constant.  Every layer is a block with a layer norm (weight and bias) before
and after each sublayer, x <- x + norm1b(mixer(norm1(x))), x <- x + norm2b(ff(norm2(x))), and ends in a weighted sum
over the results of all layers so far (and the embedding output), which is what the next layer reads.  The mixer is
an attention with sigmoid weights inside chunks of the sequence, or a minimal GRU over per-request state; an
attention layer may read the keys and values another layer cached (``kv_from``) instead of projecting its own.  The
feed-forward is a set of routed experts, each a clamped gated unit, whose router weight multiplies the expert's
input, plus a shared expert; or it is absent.  The model's norm is a layer norm too.  Tensor names: ``embed``,
``head``, ``final.norm`` (+ ``.b``), and per layer ``l<i>.norm1`` / ``norm1b`` / ``norm2`` / ``norm2b`` (+ ``.b``),
``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.dwa``.
"""
from __future__ import annotations

from torchinferno_b200.config.giforax_config import MAX_POSITIONS, GiforaxConfig, GiforaxLayer
from torchinferno_b200.config.registry import ArchitectureEntry, register_architecture
from torchinferno_b200.models.spec import BlockSpec, LayerCall, ModelSpec
from torchinferno_b200.parts.base import PartSpec

GLU_ALPHA = 1.702       # g * sigmoid(1.702 g): the design fixes it


def _mixer(layer: GiforaxLayer, config: GiforaxConfig) -> PartSpec:
    m = layer.mixer
    if layer.type == "mingru":
        return PartSpec("min_gru", {"hidden_size": config.width, "width": m["width"]}, prefix="mix.")
    position = PartSpec("rotary", {"head_dim": m["dim"], "theta": float(m["rot"]["base"]), "rot_dim": m["rot"]["dims"]})
    return PartSpec("sigmoid_attention", {
        "hidden_size": config.width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "value_dim": m["vdim"],
        "scale": float(m["scale"]), "position": position, "qk_norm_eps": config.eps, "chunk": m["mask"]["size"],
        "head_bias": True, "head_gate": True, "own_kv": m.get("kv_from") is None}, prefix="mix.")


def _feed_forward(layer: GiforaxLayer, config: GiforaxConfig) -> PartSpec | None:
    mlp = layer.mlp
    if mlp is None:
        return None
    shared = mlp.get("shared")
    return PartSpec("routed_experts", {
        "hidden_size": config.width, "experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
        "expert_size": mlp["expert"]["ff"], "activation": "glu_clamp", "limit": float(mlp["expert"]["limit"]),
        "alpha": GLU_ALPHA, "scores": "sigmoid", "normalize": False, "weight_on_input": True,
        "shared_size": 0 if shared is None else shared["ff"], "shared_limit": None if shared is None else float(shared["limit"]),
        "shared_gate": False}, prefix="mlp.")


def build_giforax(config: GiforaxConfig) -> ModelSpec:
    def norm(name: str) -> PartSpec:
        return PartSpec("layernorm", {"width": config.width, "eps": config.eps, "weight_name": name})

    blocks, schedule = [], []
    cache_of: dict[int, int] = {}       # layer with keys of its own -> its cache layer
    for i, layer in enumerate(config.layers):
        feed_forward = _feed_forward(layer, config)
        block = PartSpec("sandwich", {
            "mixer": _mixer(layer, config), "mixer_norm": norm("norm1"), "mixer_out_norm": norm("norm1b"),
            "feed_forward": feed_forward, "feed_forward_norm": None if feed_forward is None else norm("norm2"),
            "feed_forward_out_norm": None if feed_forward is None else norm("norm2b"),
            "depth_average": i + 2, "depth_name": "dwa"})
        blocks.append(BlockSpec(block, f"l{i}."))
        if layer.type != "attention":
            schedule.append(LayerCall(i, None))
        elif layer.mixer.get("kv_from") is None:
            cache_of[i] = len(cache_of)
            schedule.append(LayerCall(i, cache_of[i]))
        else:
            schedule.append(LayerCall(i, cache_of[layer.mixer["kv_from"]], writes_cache=False))
    return ModelSpec(
        architecture="Giforax", hidden_size=config.width, vocab_size=config.vocab, max_positions=MAX_POSITIONS,
        embedding_name="embed", layers=tuple(blocks), schedule=tuple(schedule),
        final_norm=PartSpec("layernorm", {"width": config.width, "eps": config.eps, "weight_name": "norm"}, prefix="final."),
        head_name="head", tie_head_to_embedding=False, config=config.to_dict(),
        embedding_scale=config.embedding_scale, history_depth=len(config.layers) + 2)


GIFORAX = register_architecture(ArchitectureEntry(
    name="Giforax", model_types=("giforax",), config_class=GiforaxConfig, build=build_giforax))
