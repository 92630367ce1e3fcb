"""The Givelix design as a ``ModelSpec`` (``config/givelix_config.py`` describes the design and its keys).

Tensor names: ``embed`` (also the head), ``final.norm``; for layer i ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``
(the mixer's), ``l<i>.mlp.{gate,up,down}``, ``l<i>.ls1``, ``l<i>.ls2`` (layer scales) and ``l<i>.hc<q>.{in,out,mix}``
(hyper-connection tables of branch q).  Every mechanism is a registered part with its constants as parameters:
``residual_streams`` (block), ``rmsnorm`` with ``offset`` 1, ``decayed_linear_attention``, ``latent_attention``,
``gated_mlp`` with the tanh form of GELU.
"""
from __future__ import annotations

from ..config.givelix_config import GivelixConfig
from ..config.model_config import LayerSpec, ModelSpec, PartSpec
from ..config.registry import register_architecture


def _mixer_spec(kind: str, mixer: dict, eps: float) -> PartSpec:
    if kind == "lightning":
        return PartSpec("decayed_linear_attention", {
            "heads": int(mixer["heads"]), "dim": int(mixer["dim"]), "vdim": int(mixer["vdim"]),
            "decay": [float(value) for value in mixer["decay"]], "eps": eps, "activation": "silu"})
    second = kind == "latent_attention_2"
    return PartSpec("latent_attention", {
        "heads": int(mixer["heads"]), "dim": int(mixer["dim"]), "rot_dim": int(mixer["rot_dim"]),
        "vdim": int(mixer["vdim"]), "kv_rank": int(mixer["kv_rank"]),
        "q_rank": 0 if second else int(mixer["q_rank"]), "scale": float(mixer["scale"]), "rot": dict(mixer["rot"]),
        "eps": eps, "sink": second, "gate": second, "own_cache": mixer.get("kv_from") is None})


def build_givelix_spec(config: GivelixConfig) -> ModelSpec:
    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"eps": config.norm_eps, "offset": 1.0, "weight_name": name})

    layers = []
    for index, entry in enumerate(config.layers):
        mlp = entry.get("mlp")
        block = PartSpec("residual_streams", {
            "streams": config.streams, "residual_mult": config.residual_mult, "layer_scale": config.layer_scale,
            "hyper": config.hyper_connections, "feed_forward": mlp is not None,
            # the norms' tensors are named without a suffix: the part's prefix is the whole name
            "tensor_prefixes": {"mixer_norm": "norm1", "mixer": "mix.", "feed_forward_norm": "norm2", "feed_forward": "mlp."}})
        feed_forward = None if mlp is None else PartSpec("gated_mlp", {
            "intermediate_size": int(mlp["ff"]), "activation": "gelu_tanh",
            "tensor_names": {"gate": "gate", "up": "up", "down": "down"}})
        source = entry["mixer"].get("kv_from")
        layers.append(LayerSpec(prefix=f"l{index}.", block=block, mixer=_mixer_spec(entry["type"], entry["mixer"], config.norm_eps),
                                feed_forward=feed_forward, mixer_norm=norm(""),
                                feed_forward_norm=None if mlp is None else norm(""),
                                cache_from=None if source is None else int(source)))
    return ModelSpec(
        architecture="Givelix", vocab_size=config.vocab, hidden_size=config.width, layers=tuple(layers),
        order=tuple(range(len(layers))), final_norm=norm(""), embedding_name="embed", final_norm_prefix="final.norm",
        lm_head_name="lm_head", tie_word_embeddings=True, max_position_embeddings=config.max_position_embeddings,
        residual_streams=config.streams, logit_scale=config.logit_scale)


register_architecture("Givelix", GivelixConfig, build_givelix_spec, model_types=("givelix",))
