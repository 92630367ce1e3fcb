"""Typed ``config.json`` of the Fororax design.

Fororax is a decoder that normalises after the residual sum (x <- norm(alpha x + sublayer(x))), takes positions from a
learned table, and lists its layers one by one: each entry names its token mixer (``attention``: grouped-query
attention with normed heads and a learned distance penalty on the scores, optionally reading an earlier layer's keys
and values; ``attention_2``: the same heads with biases, a sink in the softmax, mixing of the heads' weights and an
output gate) with its sizes, and its feed-forward, a mixture of experts, or none.

Keys: ``architecture`` ("Fororax"), ``vocab``, ``width``, ``max_positions``, ``embedding.scale``, ``postln_alpha``,
``norm.eps``, ``logit_softcap``, ``layers`` (a list of ``{"type", "mixer", "mlp"}``; mixer: ``heads``, ``kv_heads``,
``dim``, ``vdim``, ``scale``, ``kv_from``; mlp: ``kind`` "moe", ``router {experts, identity, top}``, ``expert {ff,
limit}``, ``shared {ff, limit}`` or none).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .model_config import ConfigError

MIXER_TYPES = ("attention", "attention_2")
_MIXER_KEYS = ("heads", "kv_heads", "dim", "vdim", "scale")


@dataclass(frozen=True)
class FororaxConfig:
    vocab: int
    width: int
    max_positions: int
    layers: tuple
    norm_eps: float
    embedding_scale: float = 1.0
    postln_alpha: float = 1.0
    logit_softcap: float = 0.0
    router_correction: bool = True     # the routers have a correction vector (read off the tensors when there are some)

    def __post_init__(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or self.max_positions <= 0 or not self.layers:
            raise ConfigError("vocab, width, max_positions and the number of layers must be positive")
        if not self.norm_eps > 0:
            raise ConfigError("norm.eps must be positive")
        if self.logit_softcap < 0:
            raise ConfigError("logit_softcap must not be negative")
        for index, layer in enumerate(self.layers):
            kind = layer.get("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"layer {index}: unknown type {kind!r}; known: {list(MIXER_TYPES)}")
            mixer = layer.get("mixer") or {}
            missing = [key for key in _MIXER_KEYS if key not in mixer]
            if missing:
                raise ConfigError(f"layer {index} ({kind}): mixer lacks {missing}")
            if int(mixer["heads"]) % int(mixer["kv_heads"]):
                raise ConfigError(f"layer {index}: heads must be a multiple of kv_heads")
            source = mixer.get("kv_from")
            if source is not None:
                if kind != "attention":
                    raise ConfigError(f"layer {index}: only attention layers read another layer's keys and values")
                if not 0 <= int(source) < index:
                    raise ConfigError(f"layer {index}: kv_from must name an earlier layer")
                other = self.layers[int(source)]["mixer"]
                if other.get("kv_from") is not None or any(int(other[key]) != int(mixer[key]) for key in ("kv_heads", "dim", "vdim")):
                    raise ConfigError(f"layer {index}: layer {source} must own keys and values of the same head count and sizes")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind", "moe") != "moe":
                    raise ConfigError(f"layer {index}: the feed-forward must be a mixture of experts")
                router = mlp.get("router") or {}
                missing = [key for key in ("experts", "top") if key not in router]
                if missing or "expert" not in mlp:
                    raise ConfigError(f"layer {index}: the mixture lacks router.{missing} or its expert's sizes")
                if int(router["top"]) > int(router["experts"]) + int(router.get("identity", 0)) or int(router["top"]) <= 0:
                    raise ConfigError(f"layer {index}: router.top must lie in 1 .. experts + identity")

    @classmethod
    def from_dict(cls, values: dict[str, Any], tensor_names=None) -> "FororaxConfig":
        missing = [key for key in ("vocab", "width", "layers", "norm", "max_positions") if key not in values]
        if missing:
            raise ConfigError(f"config.json lacks required keys: {missing}")
        if "eps" not in values["norm"]:
            raise ConfigError("config.json lacks norm.eps")
        correction = bool(values.get("router_correction", True))
        if tensor_names is not None:
            routed = [index for index, layer in enumerate(values["layers"]) if layer.get("mlp") is not None]
            if routed:
                correction = f"l{routed[0]}.mlp.correction" in tensor_names
        return cls(vocab=int(values["vocab"]), width=int(values["width"]), max_positions=int(values["max_positions"]),
                   layers=tuple(values["layers"]), norm_eps=float(values["norm"]["eps"]),
                   embedding_scale=float((values.get("embedding") or {}).get("scale", 1.0)),
                   postln_alpha=float(values.get("postln_alpha", 1.0)),
                   logit_softcap=float(values.get("logit_softcap") or 0.0), router_correction=correction)
