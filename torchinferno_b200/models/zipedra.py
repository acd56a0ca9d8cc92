"""Zipedra as a description made of parts.

Every layer is a parallel block (one RMS norm; mixer and feed-forward read its output and are summed into the
residual) followed by the per-layer token input.  The mixer is a decayed linear attention ('lightning') or an
attention over a low-rank latent ('latent_attention'); the feed-forward is dense SwiGLU, routed experts with a
gated shared expert, or absent.  A range of layers may run several times with the same weights: each pass
begins with the stage that mixes the embedding output back in, and every run of a layer has a cache layer or
state of its own.  Tensor names: ``embed``, ``head``, ``final.norm``, ``side.embed``, ``loop.in``, ``loop.step``,
and per layer ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.side.*``.
"""
from __future__ import annotations

from torchinferno_b200.config.registry import ArchitectureEntry, register_architecture
from torchinferno_b200.config.zipedra_config import MAX_POSITIONS, ZipedraConfig, ZipedraLayer
from torchinferno_b200.models.spec import BlockSpec, LayerCall, ModelSpec, StageCall
from torchinferno_b200.parts.base import PartSpec


def _mixer(layer: ZipedraLayer, config: ZipedraConfig) -> tuple[PartSpec, bool]:
    """The mixer's description, and whether it keeps keys in the paged cache."""
    m = layer.mixer
    if layer.type == "lightning":
        return PartSpec("decay_linear_attention", {
            "hidden_size": config.width, "heads": m["heads"], "key_dim": m["dim"], "value_dim": m["vdim"],
            "decay": tuple(float(d) for d in m["decay"]), "activation": "silu", "output_norm": True, "eps": config.eps,
            "gate": True}, prefix="mix."), False
    return PartSpec("latent_attention", {
        "hidden_size": config.width, "heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "value_dim": m["vdim"],
        "kv_rank": m["kv_rank"], "scale": float(m["scale"]), "rot_base": float(m["rot"]["base"]), "rot_dims": m["rot"]["dims"],
        "eps": config.eps, "gate": True}, prefix="mix."), True


def _feed_forward(layer: ZipedraLayer, config: ZipedraConfig) -> PartSpec | None:
    mlp = layer.mlp
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return PartSpec("swiglu", {"hidden_size": config.width, "intermediate_size": mlp["ff"], "gate_name": "gate",
                                   "up_name": "up", "down_name": "down"}, prefix="mlp.")
    shared = mlp.get("shared")
    return PartSpec("routed_experts", {
        "hidden_size": config.width, "experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
        "expert_size": mlp["expert"]["ff"], "activation": "relu2", "scores": "softmax", "normalize": True, "norm_eps": 1e-20,
        "shared_size": 0 if shared is None else shared["ff"], "shared_gate": shared is not None}, prefix="mlp.")


def build_zipedra(config: ZipedraConfig) -> ModelSpec:
    n = len(config.layers)
    blocks, keeps_keys = [], []
    for i, layer in enumerate(config.layers):
        mixer, cached = _mixer(layer, config)
        keeps_keys.append(cached)
        after = None
        if config.token_side_dim is not None:
            after = PartSpec("token_side", {"width": config.width, "dim": config.token_side_dim, "index": i,
                                            "vocab_size": config.vocab, "table_width": n * config.token_side_dim,
                                            "eps": config.eps, "table_name": "side.embed"}, prefix="side.")
        block = PartSpec("parallel", {
            "mixer": mixer, "feed_forward": _feed_forward(layer, config), "after": after,
            "norm": PartSpec("rmsnorm", {"width": config.width, "eps": config.eps, "weight_name": "norm1"})})
        blocks.append(BlockSpec(block, f"l{i}."))
    schedule: list[LayerCall | StageCall] = []
    caches = 0

    def run(layer: int) -> None:
        nonlocal caches
        if keeps_keys[layer]:
            schedule.append(LayerCall(layer, caches))
            caches += 1
        else:
            schedule.append(LayerCall(layer, None))

    stages: tuple[PartSpec, ...] = ()
    if config.loop is None:
        for i in range(n):
            run(i)
    else:
        start, stop, times = config.loop
        stages = (PartSpec("loop_input", {"width": config.width, "passes": times}, prefix="loop."),)
        for i in range(start):
            run(i)
        for t in range(times):
            schedule.append(StageCall(0, t))
            for i in range(start, stop):
                run(i)
        for i in range(stop, n):
            run(i)
    return ModelSpec(
        architecture="Zipedra", hidden_size=config.width, vocab_size=config.vocab, max_positions=MAX_POSITIONS,
        embedding_name="embed", layers=tuple(blocks), schedule=tuple(schedule),
        final_norm=PartSpec("rmsnorm", {"width": config.width, "eps": config.eps, "weight_name": "norm"}, prefix="final."),
        head_name="head", tie_head_to_embedding=False, config=config.to_dict(), stages=stages,
        logit_scale=config.logit_scale, keeps_embedding_output=config.loop is not None)


ZIPEDRA = register_architecture(ArchitectureEntry(
    name="Zipedra", model_types=("zipedra",), config_class=ZipedraConfig, build=build_zipedra))
