"""Plain, slow, whole-sequence implementation of the Fororax decoder.

The oracle of the Fororax tests: no cache, no batching, no kernels, one function per mechanism, float64 torch ops on
the CPU.  It shares no code with the engine package: it reads ``config.json`` and the safetensors file by itself and
takes every size and constant from the configuration dictionary.

Notation: T tokens, W the model width, H query heads, G key/value heads, x [T, W].  Linear weights are kept
[out, in] and applied as x @ W^T.

The design
* embeds a token as table[token] * embedding.scale + positions[p] (a learned vector per position);
* normalises AFTER the sum: x <- norm(alpha x + sublayer(x)), the sublayer reading x itself;
* has two token mixers, both grouped-query attention with an RMS norm on every head's query and key and no
  rotation: ``attention`` takes a distance penalty r1_h ln(1 + r2_h (i - j)) off the scores and may read the keys
  and values of an earlier layer; ``attention_2`` has biases, a learned sink in the softmax's denominator, mixes
  the heads' softmax weights with a learned H x H table and gates its output elementwise;
* feeds forward through a mixture of experts with identity experts, a correction on the choice scores only, weights
  that are not renormalised, and a gated shared expert;
* caps the logits with a tanh.
"""
from __future__ import annotations

import json
import struct
from pathlib import Path

import torch


# --------------------------------------------------------------------------- small parts
def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return rms(x, eps) * weight


def embed(tokens: list[int], table: torch.Tensor, positions: torch.Tensor, scale: float, first: int = 0) -> torch.Tensor:
    ids = torch.tensor(tokens, dtype=torch.long)
    return table[ids] * scale + positions[first:first + len(tokens)]


def head_norm(x: torch.Tensor, heads: int, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """[T, heads * d] -> [T, heads, d], every head normed with the one weight [d]."""
    return norm(x.view(x.shape[0], heads, -1), weight, eps)


# --------------------------------------------------------------------------- attention
def causal_scores(q: torch.Tensor, k: torch.Tensor, scale: float) -> torch.Tensor:
    """q [T, H, d], k [T, G, d] -> scores [H, T, T] (row i, column j), -inf where j > i."""
    heads, groups = q.shape[1], k.shape[1]
    k = k.repeat_interleave(heads // groups, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * scale
    count = q.shape[0]
    hidden = torch.ones(count, count, dtype=torch.bool).triu(1)
    return scores.masked_fill(hidden, float("-inf"))


def distance_penalty(count: int, r1: torch.Tensor, r2: torch.Tensor) -> torch.Tensor:
    """[H, T, T]: r1_h ln(1 + r2_h (i - j)) for j <= i (zero elsewhere: those places are masked anyway)."""
    index = torch.arange(count, dtype=r1.dtype)
    distance = (index[:, None] - index[None, :]).clamp_min(0)
    return r1[:, None, None] * torch.log1p(r2[:, None, None] * distance[None])


def softmax_with_sink(scores: torch.Tensor, sink: torch.Tensor | None) -> torch.Tensor:
    """Softmax over the last axis; with ``sink`` [H] the denominator also holds exp(sink_h)."""
    if sink is None:
        return torch.softmax(scores, dim=-1)
    top = torch.maximum(scores.max(dim=-1, keepdim=True).values, sink[:, None, None])
    weights = torch.exp(scores - top)
    return weights / (weights.sum(-1, keepdim=True) + torch.exp(sink[:, None, None] - top))


def mix_heads(weights: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """weights [H, T, T], table [H, H]: new_h = sum_g table[h, g] old_g."""
    return torch.einsum("hg,gij->hij", table, weights)


def apply_weights(weights: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """weights [H, T, T], v [T, G, dv] -> [T, H * dv]; head h reads the values of its own group."""
    heads, groups = weights.shape[0], v.shape[1]
    v = v.repeat_interleave(heads // groups, dim=1)
    return torch.einsum("hij,jhd->ihd", weights, v).reshape(v.shape[0], -1)


def keys_and_values(x, w, prefix, mixer, eps, biased):
    groups = int(mixer["kv_heads"])
    k = x @ w[prefix + "k"].t()
    v = x @ w[prefix + "v"].t()
    if biased:
        k = k + w[prefix + "k.b"]
        v = v + w[prefix + "v.b"]
    return head_norm(k, groups, w[prefix + "k.norm"], eps), v.view(x.shape[0], groups, -1)


def attention(x, w, prefix, mixer, eps, shared=None):
    """The mixer ``attention``.  ``shared``: (keys, values) of the layer named by ``kv_from``.  Returns (y, (k, v))."""
    heads = int(mixer["heads"])
    q = head_norm(x @ w[prefix + "q"].t(), heads, w[prefix + "q.norm"], eps)
    k, v = shared if shared is not None else keys_and_values(x, w, prefix, mixer, eps, False)
    scores = causal_scores(q, k, float(mixer["scale"])) - distance_penalty(x.shape[0], w[prefix + "r1"], w[prefix + "r2"])
    y = apply_weights(torch.softmax(scores, dim=-1), v)
    return y @ w[prefix + "o"].t(), (k, v)


def attention_2(x, w, prefix, mixer, eps):
    """The mixer ``attention_2``.  Returns (y, (k, v))."""
    heads = int(mixer["heads"])
    q = head_norm(x @ w[prefix + "q"].t() + w[prefix + "q.b"], heads, w[prefix + "q.norm"], eps)
    k, v = keys_and_values(x, w, prefix, mixer, eps, True)
    weights = softmax_with_sink(causal_scores(q, k, float(mixer["scale"])), w[prefix + "sink"])
    y = apply_weights(mix_heads(weights, w[prefix + "talk"]), v)
    y = y * torch.sigmoid(x @ w[prefix + "g"].t())
    return y @ w[prefix + "o"].t() + w[prefix + "o.b"], (k, v)


# --------------------------------------------------------------------------- feed-forward
def expert(x, gate, up, down, limit: float) -> torch.Tensor:
    g = (x @ gate.t()).clamp(max=limit)
    u = (x @ up.t()).clamp(-limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.t()


def route(x, router, correction, top: int):
    """(scores [T, E], chosen [T, top]): softmax over all experts; the correction moves the choice only."""
    scores = torch.softmax(x @ router.t(), dim=-1)
    chosen = torch.topk(scores + correction, top, dim=-1).indices
    return scores, chosen


def mixture(x, w, prefix, mlp) -> torch.Tensor:
    experts, identity, top = (int(mlp["router"].get(key, 0)) for key in ("experts", "identity", "top"))
    scores, chosen = route(x, w[prefix + "router"], w[prefix + "correction"], top)
    limit = float(mlp["expert"]["limit"])
    y = torch.zeros_like(x)
    for row in range(x.shape[0]):
        for index in chosen[row].tolist():
            weight = scores[row, index]
            if index >= experts:          # one of the `identity` last outputs of the router: the input itself
                y[row] += weight * x[row]
            else:
                name = f"{prefix}e{index}."
                y[row] += weight * expert(x[row:row + 1], w[name + "gate"], w[name + "up"], w[name + "down"], limit)[0]
    assert scores.shape[1] == experts + identity
    shared = mlp.get("shared")
    if shared:
        name = prefix + "shared."
        out = expert(x, w[name + "gate"], w[name + "up"], w[name + "down"], float(shared["limit"]))
        y = y + out * torch.sigmoid(x @ w[name + "sg"].t())
    return y


# --------------------------------------------------------------------------- the model
def forward_layers(cfg: dict, w: dict, tokens: list[int]) -> list[torch.Tensor]:
    """The residual after the embedding and after every layer: a list of [T, W]."""
    eps, alpha = float(cfg["norm"]["eps"]), float(cfg["postln_alpha"])
    x = embed(tokens, w["embed"], w["pos"], float(cfg["embedding"]["scale"]))
    seen = [x]
    kept = {}
    for index, layer in enumerate(cfg["layers"]):
        prefix = f"l{index}."
        mixer = layer["mixer"]
        if layer["type"] == "attention":
            source = mixer.get("kv_from")
            y, kept[index] = attention(x, w, prefix + "mix.", mixer, eps, None if source is None else kept[int(source)])
        elif layer["type"] == "attention_2":
            y, kept[index] = attention_2(x, w, prefix + "mix.", mixer, eps)
        else:
            raise ValueError(f"unknown layer type {layer['type']!r}")
        x = norm(alpha * x + y, w[prefix + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = norm(alpha * x + mixture(x, w, prefix + "mlp.", layer["mlp"]), w[prefix + "norm2"], eps)
        seen.append(x)
    return seen


def logits_of(cfg: dict, w: dict, x: torch.Tensor) -> torch.Tensor:
    cap = float(cfg["logit_softcap"])
    z = norm(x, w["final.norm"], float(cfg["norm"]["eps"])) @ w["head"].t()
    return cap * torch.tanh(z / cap)


def forward_full(cfg: dict, w: dict, tokens: list[int]) -> torch.Tensor:
    """Logits [T, vocab] of the whole sequence."""
    return logits_of(cfg, w, forward_layers(cfg, w, tokens)[-1])


# --------------------------------------------------------------------------- files
_STORED = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32, "F64": torch.float64}


def read_safetensors(path) -> dict[str, torch.Tensor]:
    """The file format read directly: an 8-byte little-endian length, that many bytes of JSON (name -> dtype, shape,
    data_offsets), then the data."""
    raw = Path(path).read_bytes()
    (length,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + length])
    data = raw[8 + length:]
    out = {}
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        lo, hi = entry["data_offsets"]
        tensor = torch.frombuffer(bytearray(data[lo:hi]), dtype=_STORED[entry["dtype"]])
        out[name] = tensor.reshape(entry["shape"])
    return out


def load_folder(folder, round_to=None):
    """(config dictionary, weights in float64).  ``round_to`` (e.g. torch.bfloat16): matrices are rounded to it first,
    as an engine that holds them so would see them."""
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    weights = {}
    for name, tensor in read_safetensors(folder / "model.safetensors").items():
        if tensor.is_floating_point():
            if round_to is not None and tensor.dim() >= 2:
                tensor = tensor.to(round_to)
            tensor = tensor.to(torch.float64)
        weights[name] = tensor
    return cfg, weights


# --------------------------------------------------------------------------- random models for the tests
def tensor_shapes(cfg: dict) -> dict[str, tuple]:
    """Every tensor of a model of this configuration, by name."""
    width = int(cfg["width"])
    shapes = {"embed": (int(cfg["vocab"]), width), "pos": (int(cfg["max_positions"]), width), "final.norm": (width,),
              "head": (int(cfg["vocab"]), width)}
    for index, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{index}."
        heads, groups, dim, vdim = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
        second = layer["type"] == "attention_2"
        shapes[p + "norm1"] = (width,)
        shapes[p + "mix.q"] = (heads * dim, width)
        shapes[p + "mix.q.norm"] = (dim,)
        shapes[p + "mix.o"] = (width, heads * vdim)
        if m.get("kv_from") is None:
            shapes[p + "mix.k"] = (groups * dim, width)
            shapes[p + "mix.v"] = (groups * vdim, width)
            shapes[p + "mix.k.norm"] = (dim,)
        if second:
            for name in ("q", "k", "v", "o"):
                shapes[p + f"mix.{name}.b"] = (shapes[p + f"mix.{name}"][0],)
            shapes[p + "mix.sink"] = (heads,)
            shapes[p + "mix.talk"] = (heads, heads)
            shapes[p + "mix.g"] = (heads * vdim, width)
        else:
            shapes[p + "mix.r1"] = (heads,)
            shapes[p + "mix.r2"] = (heads,)
        mlp = layer.get("mlp")
        if mlp is not None:
            shapes[p + "norm2"] = (width,)
            outputs = int(mlp["router"]["experts"]) + int(mlp["router"].get("identity", 0))
            shapes[p + "mlp.router"] = (outputs, width)
            shapes[p + "mlp.correction"] = (outputs,)
            sized = [(f"e{j}.", int(mlp["expert"]["ff"])) for j in range(int(mlp["router"]["experts"]))]
            if mlp.get("shared"):
                sized.append(("shared.", int(mlp["shared"]["ff"])))
                shapes[p + "mlp.shared.sg"] = (1, width)
            for name, ff in sized:
                shapes[p + "mlp." + name + "gate"] = (ff, width)
                shapes[p + "mlp." + name + "up"] = (ff, width)
                shapes[p + "mlp." + name + "down"] = (width, ff)
    return shapes


def random_weights(cfg: dict, seed: int) -> dict[str, torch.Tensor]:
    """Random float32 weights with large gains, so that every mechanism moves the logits: peaked routers, clamps that
    act, sinks and penalties of the size of the scores, a head table far from the identity."""
    generator = torch.Generator().manual_seed(seed)

    def normal(shape, std):
        return torch.randn(shape, generator=generator) * std

    def uniform(shape, lo, hi):
        return lo + (hi - lo) * torch.rand(shape, generator=generator)

    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if name == "embed":
            tensor = normal(shape, 1.0)
        elif name == "pos":
            tensor = normal(shape, 0.5)
        elif last in ("norm", "norm1", "norm2"):
            tensor = uniform(shape, 0.6, 1.4)
        elif last == "b":
            tensor = normal(shape, 0.3)
        elif last == "r1":
            tensor = uniform(shape, 0.2, 1.5)
        elif last == "r2":
            tensor = uniform(shape, 0.05, 1.0)
        elif last == "sink":
            tensor = normal(shape, 1.5)
        elif last == "talk":
            tensor = 0.7 * torch.eye(shape[0]) + normal(shape, 0.3)
        elif last == "correction":
            tensor = normal(shape, 0.1)
        elif last == "router":
            tensor = normal(shape, 4.0 / shape[1] ** 0.5)
        elif name == "head":
            tensor = normal(shape, 3.0 / shape[1] ** 0.5)
        elif last in ("gate", "up"):
            tensor = normal(shape, 1.5 / shape[1] ** 0.5)
        else:
            tensor = normal(shape, 1.0 / shape[1] ** 0.5)
        out[name] = tensor.to(torch.bfloat16).to(torch.float32).contiguous()   # values that bfloat16 holds exactly
    return out


def write_model(folder, cfg: dict, seed: int) -> dict[str, torch.Tensor]:
    """config.json and model.safetensors (float32) of a random model; returns the weights."""
    from safetensors.torch import save_file

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    weights = random_weights(cfg, seed)
    (folder / "config.json").write_text(json.dumps(cfg, indent=1))
    save_file(weights, str(folder / "model.safetensors"))
    return weights
