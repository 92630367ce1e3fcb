"""The Fororax design as a ``ModelSpec`` (``config/fororax_config.py`` describes the design and its keys).

Tensor names: ``embed``, ``pos`` (a learned vector per position), ``final.norm``, ``head``; for layer i ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.mix.*`` (the mixer's: ``q k v o`` with ``.b`` biases, ``q.norm k.norm``, ``r1 r2``, ``sink``,
``talk``, ``g``) and ``l<i>.mlp.*`` (``router``, ``correction``, ``e<j>.{gate,up,down}``, ``shared.{gate,up,down,sg}``).
Every mechanism is a registered part with its constants as parameters: ``postnorm_residual`` (block),
``rmsnorm_after_sum`` (the layers' norms, with alpha), ``rmsnorm`` (the final norm), ``normed_attention`` (both mixers,
by switches), ``clamped_moe``; the embedding's constant, the position table and the cap on the logits are fields of
the ``ModelSpec``.
"""
from __future__ import annotations

from ..config.fororax_config import FororaxConfig
from ..config.model_config import LayerSpec, ModelSpec, PartSpec
from ..config.registry import register_architecture


def _mixer_spec(kind: str, mixer: dict, eps: float) -> PartSpec:
    second = kind == "attention_2"
    return PartSpec("normed_attention", {
        "heads": int(mixer["heads"]), "kv_heads": int(mixer["kv_heads"]), "dim": int(mixer["dim"]),
        "vdim": int(mixer["vdim"]), "scale": float(mixer["scale"]), "eps": eps, "bias": second,
        "distance_penalty": not second, "sink": second, "head_mixing": second, "gate": second,
        "own_cache": mixer.get("kv_from") is None})


def _feed_forward_spec(mlp: dict, correction: bool) -> PartSpec:
    router, expert, shared = mlp["router"], mlp["expert"], mlp.get("shared")
    return PartSpec("clamped_moe", {
        "experts": int(router["experts"]), "identity": int(router.get("identity", 0)), "top": int(router["top"]),
        "ff": int(expert["ff"]), "limit": float(expert["limit"]), "correction": correction,
        "shared": {"ff": int(shared["ff"]), "limit": float(shared["limit"])} if shared else None})


def build_fororax_spec(config: FororaxConfig) -> ModelSpec:
    def layer_norm() -> PartSpec:
        return PartSpec("rmsnorm_after_sum", {"eps": config.norm_eps, "residual_mult": config.postln_alpha, "weight_name": ""})

    layers = []
    for index, entry in enumerate(config.layers):
        mlp = entry.get("mlp")
        # the norms' tensors are named without a suffix: the part's prefix is the whole name
        block = PartSpec("postnorm_residual", {"tensor_prefixes": {
            "mixer_norm": "norm1", "mixer": "mix.", "feed_forward_norm": "norm2", "feed_forward": "mlp."}})
        source = entry["mixer"].get("kv_from")
        layers.append(LayerSpec(
            prefix=f"l{index}.", block=block, mixer=_mixer_spec(entry["type"], entry["mixer"], config.norm_eps),
            feed_forward=None if mlp is None else _feed_forward_spec(mlp, config.router_correction),
            mixer_norm=layer_norm(), feed_forward_norm=None if mlp is None else layer_norm(),
            cache_from=None if source is None else int(source)))
    return ModelSpec(
        architecture="Fororax", vocab_size=config.vocab, hidden_size=config.width, layers=tuple(layers),
        order=tuple(range(len(layers))), final_norm=PartSpec("rmsnorm", {"eps": config.norm_eps, "weight_name": ""}),
        embedding_name="embed", final_norm_prefix="final.norm", lm_head_name="head", tie_word_embeddings=False,
        max_position_embeddings=config.max_positions, embedding_scale=config.embedding_scale,
        position_table_name="pos", logit_softcap=config.logit_softcap)


register_architecture("Fororax", FororaxConfig, build_fororax_spec, model_types=("fororax",))
