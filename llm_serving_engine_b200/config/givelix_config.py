"""Typed ``config.json`` of the Givelix design.

Givelix is a decoder whose layers are listed one by one in the configuration: each entry names its token mixer
(``lightning``: linear attention with a decay per head; ``latent_attention``: attention over a cached latent with
queries through a latent of their own, optionally reading an earlier layer's cache; ``latent_attention_2``:
attention over a cached latent with scaled rotary frequencies, a sink per head and a gate per head) with its
sizes, and its feed-forward or none.  The residual is kept in ``streams`` copies (hyper-connections), every branch
output is scaled by a learned vector and by ``residual_mult``, the norms' weights are stored as offsets from one,
and the logits of the tied head are multiplied by ``logit_scale``.

Keys: ``architecture`` ("Givelix"), ``vocab``, ``width``, ``layers`` (a list of ``{"type", "mixer", "mlp"}``),
``norm.eps``, ``residual_mult``, ``streams``, ``logit_scale``; ``max_position_embeddings`` is this engine's own
optional key (the design itself sets no limit).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .model_config import ConfigError

MIXER_TYPES = ("lightning", "latent_attention", "latent_attention_2")
_MIXER_KEYS = {
    "lightning": ("heads", "dim", "vdim", "decay"),
    "latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale", "rot"),
    "latent_attention_2": ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot"),
}


@dataclass(frozen=True)
class GivelixConfig:
    vocab: int
    width: int
    layers: tuple
    norm_eps: float
    residual_mult: float = 1.0
    streams: int = 1
    logit_scale: float = 1.0
    hyper_connections: bool = False     # the layers have tables that read, mix and write the copies of the residual
    layer_scale: bool = True            # the layers have a learned vector on every branch output
    max_position_embeddings: int = 131_072

    def __post_init__(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or not self.layers:
            raise ConfigError("vocab, width and the number of layers must be positive")
        if not 1 <= self.streams <= 8:
            raise ConfigError(f"streams must lie in 1 .. 8, got {self.streams}")
        if self.streams > 1 and not self.hyper_connections:
            raise ConfigError("several residual streams need the layers' hyper-connection tables")
        if not self.norm_eps > 0:
            raise ConfigError("norm.eps must be positive")
        for index, layer in enumerate(self.layers):
            kind = layer.get("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"layer {index}: unknown type {kind!r}; known: {list(MIXER_TYPES)}")
            mixer = layer.get("mixer") or {}
            missing = [key for key in _MIXER_KEYS[kind] if key not in mixer]
            if missing:
                raise ConfigError(f"layer {index} ({kind}): mixer lacks {missing}")
            if kind == "lightning":
                if len(mixer["decay"]) != int(mixer["heads"]):
                    raise ConfigError(f"layer {index}: {len(mixer['decay'])} decays for {mixer['heads']} heads")
            else:
                rot = mixer["rot"]
                if "base" not in rot or "dims" not in rot:
                    raise ConfigError(f"layer {index}: rot needs base and dims")
                if int(rot["dims"]) > int(mixer["rot_dim"]) or int(rot["dims"]) % 2:
                    raise ConfigError(f"layer {index}: rot.dims must be even and at most rot_dim")
                scaling = rot.get("scaling")
                if scaling and any(key not in scaling for key in ("factor", "original", "fast", "slow")):
                    raise ConfigError(f"layer {index}: rot.scaling needs factor, original, fast and slow")
            source = mixer.get("kv_from")
            if source is not None:
                if kind != "latent_attention":
                    raise ConfigError(f"layer {index}: only latent_attention layers read another layer's cache")
                if not 0 <= int(source) < index or self.layers[int(source)].get("type") not in MIXER_TYPES[1:]:
                    raise ConfigError(f"layer {index}: kv_from must name an earlier latent attention layer")
                other = self.layers[int(source)]["mixer"]
                if other.get("kv_from") is not None or any(int(other[key]) != int(mixer[key]) for key in ("kv_rank", "rot_dim")):
                    raise ConfigError(f"layer {index}: layer {source} must own a cache with the same kv_rank and rot_dim")
            mlp = layer.get("mlp")
            if mlp is not None and (mlp.get("kind", "dense") != "dense" or int(mlp.get("ff", 0)) <= 0):
                raise ConfigError(f"layer {index}: the feed-forward must be dense with a positive ff")

    @classmethod
    def from_dict(cls, values: dict[str, Any], tensor_names=None) -> "GivelixConfig":
        """``tensor_names``: the names in the checkpoint, when there is one: whether the layers have layer scales and
        hyper-connection tables is then read off the tensors (the configuration has no key for either)."""
        missing = [key for key in ("vocab", "width", "layers", "norm") if key not in values]
        if missing:
            raise ConfigError(f"config.json lacks required keys: {missing}")
        if "eps" not in values["norm"]:
            raise ConfigError("config.json lacks norm.eps")
        if tensor_names is not None:
            hyper, scaled = "l0.hc1.in" in tensor_names, "l0.ls1" in tensor_names
        else:
            hyper = bool(values.get("hyper_connections", "streams" in values))
            scaled = bool(values.get("layer_scale", True))
        return cls(vocab=int(values["vocab"]), width=int(values["width"]), layers=tuple(values["layers"]),
                   norm_eps=float(values["norm"]["eps"]), residual_mult=float(values.get("residual_mult", 1.0)),
                   streams=int(values.get("streams", 1)), logit_scale=float(values.get("logit_scale", 1.0)),
                   hyper_connections=hyper, layer_scale=scaled,
                   max_position_embeddings=int(values.get("max_position_embeddings", 131_072)))
