"""Plain, slow, whole-sequence implementation of the Givelix decoder.

The oracle of the Givelix tests: no cache, no batching, no kernels, one function
per mechanism, float64 (or float32) torch ops on the CPU.  It shares no code
with the engine package: it reads ``config.json`` and the safetensors file by
itself and takes every size and constant from the configuration dictionary.

Notation: T tokens, W the model width, H heads, x [T, W] the input of a
sublayer.  Linear weights are kept [out, in] and applied as x @ W^T.

The design
* keeps ``streams`` copies of the residual (hyper-connections): a sublayer
  reads a weighted sum of the copies, and its output is written back into every
  copy while the copies are mixed with a small square matrix;
* scales every sublayer output by a per-channel vector (layer scale) and by one
  constant of the model (``residual_mult``);
* norms are RMS norms whose stored weight is an offset from one;
* has three kinds of token mixers: a linear attention with a per-head decay
  ("lightning"), and two attentions over a low-rank latent of keys and values
  ("latent_attention", whose queries go through a latent too and which may
  read the latent of an earlier layer, and "latent_attention_2" with scaled
  rotary frequencies, a per-head sink in the softmax and a per-head output gate);
* a layer may have no feed-forward; where it has one it is gated with the tanh
  form of GELU;
* the logits are the tied embedding times the normed sum of the copies, times
  ``logit_scale``.
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch


# --------------------------------------------------------------------------- small parts
def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def offset_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """The layer norms and the final norm: the weight is stored around zero."""
    return rms(x, eps) * (1.0 + weight)


def plain_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """The norms inside the mixers: an ordinary weight."""
    return rms(x, eps) * weight


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z.pow(3))))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def feed_forward(x: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return (gelu_tanh(x @ gate.t()) * (x @ up.t())) @ down.t()


# --------------------------------------------------------------------------- rotary
def rotary_frequencies(rot: dict, dtype=torch.float64) -> tuple[torch.Tensor, float]:
    """Frequency of every pair and the factor on cos and sin.  Without ``scaling``: f_i = base^(-2i/dims),
    factor 1.  With it (factor s, original length n, fast and slow turn counts): pairs that turn more than
    ``fast`` times over n positions keep their frequency, pairs that turn fewer than ``slow`` times get f_i / s,
    a linear ramp over the pair index in between; cos and sin are multiplied by 0.1 ln(s) + 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    index = torch.arange(dims // 2, dtype=dtype)
    freq = base ** (-2.0 * index / dims)
    scaling = rot.get("scaling")
    if not scaling:
        return freq, 1.0
    s, n = float(scaling["factor"]), float(scaling["original"])

    def pair_that_turns(times: float) -> float:
        return dims * math.log(n / (2.0 * math.pi * times)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_that_turns(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_that_turns(float(scaling["slow"]))), dims - 1)
    ramp = ((index - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return freq / s * ramp + freq * (1.0 - ramp), 0.1 * math.log(s) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """Rotate the first rot.dims values of the last axis of x [T, ..., D]: the pair (2i, 2i+1) by position * f_i."""
    dims = int(rot["dims"])
    freq, factor = rotary_frequencies(rot, x.dtype)
    angle = positions.to(x.dtype)[:, None] * freq[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    cos, sin = (angle.cos() * factor).view(shape), (angle.sin() * factor).view(shape)
    out = x.clone()
    even, odd = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = even * cos - odd * sin
    out[..., 1:dims:2] = odd * cos + even * sin
    return out


# --------------------------------------------------------------------------- mixers
def lightning_mixer(x: torch.Tensor, m: dict, w: dict, eps: float) -> torch.Tensor:
    """Linear attention with a decay per head, token by token:
    S_t = decay_h S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t, S_(-1) = 0."""
    tokens = x.shape[0]
    heads, dim, vdim = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(x @ w["q"].t()).view(tokens, heads, dim)
    k = silu(x @ w["k"].t()).view(tokens, heads, dim)
    v = silu(x @ w["v"].t()).view(tokens, heads, vdim)
    out = torch.zeros(tokens, heads, vdim, dtype=x.dtype)
    for h in range(heads):
        decay = float(m["decay"][h])
        state = torch.zeros(dim, vdim, dtype=x.dtype)
        for t in range(tokens):
            state = decay * state + torch.outer(k[t, h], v[t, h])
            out[t, h] = state.t() @ q[t, h]
    merged = plain_norm(out.reshape(tokens, heads * vdim), w["norm"], eps)
    return (merged * torch.sigmoid(x @ w["g"].t())) @ w["o"].t()


def latent_keys_values(x: torch.Tensor, positions: torch.Tensor, m: dict, w: dict, eps: float):
    """What a latent attention layer keeps of every token: the normed latent c [T, kv_rank] and the rotated
    key part that all heads share [T, rot_dim]."""
    rank = int(m["kv_rank"])
    down = x @ w["dkv"].t()
    latent = plain_norm(down[:, :rank], w["dkv.norm"], eps)
    shared = rotate(down[:, rank:], positions, m["rot"])
    return latent, shared


def latent_attention(q: torch.Tensor, latent: torch.Tensor, shared: torch.Tensor, m: dict, w: dict,
                     sink: torch.Tensor | None) -> torch.Tensor:
    """Causal softmax attention; q [T, H, dim + rot_dim] already rotated.  Returns [T, H, vdim]."""
    tokens = q.shape[0]
    heads, dim, vdim = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    keys = (latent @ w["uk"].t()).view(tokens, heads, dim)
    values = (latent @ w["uv"].t()).view(tokens, heads, vdim)
    scores = torch.einsum("ihd,jhd->hij", q[..., :dim], keys) + torch.einsum("ihd,jd->hij", q[..., dim:], shared)
    scores = scores * float(m["scale"])
    visible = torch.tril(torch.ones(tokens, tokens, dtype=torch.bool))
    scores = scores.masked_fill(~visible, -math.inf)
    top = scores.max(-1, keepdim=True).values
    if sink is not None:
        top = torch.maximum(top, sink.view(heads, 1, 1).to(scores.dtype))
    weights = torch.exp(scores - top)
    total = weights.sum(-1, keepdim=True)
    if sink is not None:
        total = total + torch.exp(sink.view(heads, 1, 1).to(scores.dtype) - top)   # no key, no value, counted once
    return torch.einsum("hij,jhd->ihd", weights / total, values)


def latent_mixer(x, positions, m, w, eps, borrowed=None):
    """Kind ``latent_attention``: queries through a normed latent; keys and values from the layer's own latent or,
    with ``kv_from``, from the latent and shared key part that the named layer made (``borrowed``)."""
    tokens = x.shape[0]
    heads, dim, rot_dim = int(m["heads"]), int(m["dim"]), int(m["rot_dim"])
    q = (plain_norm(x @ w["dq"].t(), w["dq.norm"], eps) @ w["uq"].t()).view(tokens, heads, dim + rot_dim)
    q = torch.cat([q[..., :dim], rotate(q[..., dim:], positions, m["rot"])], dim=-1)
    latent, shared = borrowed if borrowed is not None else latent_keys_values(x, positions, m, w, eps)
    attended = latent_attention(q, latent, shared, m, w, None)
    return attended.reshape(tokens, -1) @ w["o"].t(), (latent, shared)


def latent_mixer_2(x, positions, m, w, eps):
    """Kind ``latent_attention_2``: direct queries, scaled rotary frequencies, a sink per head, a gate per head."""
    tokens = x.shape[0]
    heads, dim, rot_dim = int(m["heads"]), int(m["dim"]), int(m["rot_dim"])
    q = (x @ w["q"].t()).view(tokens, heads, dim + rot_dim)
    q = torch.cat([q[..., :dim], rotate(q[..., dim:], positions, m["rot"])], dim=-1)
    latent, shared = latent_keys_values(x, positions, m, w, eps)
    attended = latent_attention(q, latent, shared, m, w, w["sink"].to(x.dtype))
    attended = attended * torch.sigmoid(x @ w["g"].t())[:, :, None]
    return attended.reshape(tokens, -1) @ w["o"].t(), (latent, shared)


# --------------------------------------------------------------------------- the model
def sub(weights: dict, prefix: str) -> dict:
    return {name[len(prefix):]: tensor for name, tensor in weights.items() if name.startswith(prefix)}


def forward_full(config: dict, weights: dict, tokens: list[int], dtype=torch.float64, layer_outputs: list | None = None):
    """Logits [T, vocab] of a whole sequence.  ``layer_outputs``: a list that receives the sum of the residual
    copies after every layer."""
    weights = {name: (t.to(dtype) if t.is_floating_point() else t) for name, t in weights.items()}
    eps = float(config["norm"]["eps"])
    mult = float(config.get("residual_mult", 1.0))
    streams = int(config.get("streams", 1))
    ids = torch.tensor(tokens, dtype=torch.long)
    positions = torch.arange(len(tokens))
    copies = weights["embed"][ids].unsqueeze(0).repeat(streams, 1, 1)   # [streams, T, W]
    kept: dict[int, tuple] = {}

    def sublayer(copies, layer: str, number: int, run):
        hyper = f"{layer}.hc{number}.in" in weights
        read = torch.einsum("s,stw->tw", weights[f"{layer}.hc{number}.in"], copies) if hyper else copies[0]
        y = run(offset_norm(read, weights[f"{layer}.norm{number}"], eps))
        if f"{layer}.ls{number}" in weights:
            y = y * weights[f"{layer}.ls{number}"]
        if hyper:
            mixed = torch.einsum("sr,stw->rtw", weights[f"{layer}.hc{number}.mix"], copies)
            return mixed + mult * weights[f"{layer}.hc{number}.out"][:, None, None] * y[None]
        return copies + mult * y[None]

    for index, entry in enumerate(config["layers"]):
        layer = f"l{index}"
        m, kind = entry["mixer"], entry["type"]
        w = sub(weights, layer + ".mix.")

        def mixer(x):
            if kind == "lightning":
                return lightning_mixer(x, m, w, eps)
            if kind == "latent_attention":
                borrowed = kept[int(m["kv_from"])] if m.get("kv_from") is not None else None
                y, kept[index] = latent_mixer(x, positions, m, w, eps, borrowed)
                return y
            if kind == "latent_attention_2":
                y, kept[index] = latent_mixer_2(x, positions, m, w, eps)
                return y
            raise ValueError(kind)

        copies = sublayer(copies, layer, 1, mixer)
        if entry.get("mlp") is not None:
            f = sub(weights, layer + ".mlp.")
            copies = sublayer(copies, layer, 2, lambda x: feed_forward(x, f["gate"], f["up"], f["down"]))
        if layer_outputs is not None:
            layer_outputs.append(copies.sum(0) if streams > 1 else copies[0])
    total = copies.sum(0) if streams > 1 else copies[0]
    x = offset_norm(total, weights["final.norm"], eps)
    return (x @ weights["embed"].t()) * float(config.get("logit_scale", 1.0))


def load_folder(folder, round_to=None):
    """(config dictionary, weights by name as float32) of a model folder; ``round_to=torch.bfloat16`` rounds the
    matrices first, as an engine that holds them in bfloat16 does."""
    from safetensors import safe_open

    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    weights = {}
    with safe_open(str(folder / "model.safetensors"), framework="pt", device="cpu") as source:
        for name in source.keys():
            tensor = source.get_tensor(name)
            if tensor.is_floating_point():
                if round_to is not None and tensor.dim() >= 2:
                    tensor = tensor.to(round_to)
                tensor = tensor.to(torch.float32)
            weights[name] = tensor
    return config, weights


# --------------------------------------------------------------------------- making a model for a test
def tensor_shapes(config: dict, layer_scale: bool = True) -> dict[str, tuple]:
    """Name -> shape of every tensor of a model of this configuration (hyper-connection tables when the
    configuration has ``streams``)."""
    width, streams = int(config["width"]), config.get("streams")
    out = {"embed": (int(config["vocab"]), width), "final.norm": (width,)}
    for index, entry in enumerate(config["layers"]):
        layer, m = f"l{index}", entry["mixer"]
        branches = (1, 2) if entry.get("mlp") is not None else (1,)
        for number in branches:
            out[f"{layer}.norm{number}"] = (width,)
            if layer_scale:
                out[f"{layer}.ls{number}"] = (width,)
            if streams is not None:
                out[f"{layer}.hc{number}.in"] = (int(streams),)
                out[f"{layer}.hc{number}.out"] = (int(streams),)
                out[f"{layer}.hc{number}.mix"] = (int(streams), int(streams))
        heads = int(m["heads"])
        if entry["type"] == "lightning":
            dim, vdim = int(m["dim"]), int(m["vdim"])
            out.update({f"{layer}.mix.q": (heads * dim, width), f"{layer}.mix.k": (heads * dim, width),
                        f"{layer}.mix.v": (heads * vdim, width), f"{layer}.mix.g": (heads * vdim, width),
                        f"{layer}.mix.o": (width, heads * vdim), f"{layer}.mix.norm": (heads * vdim,)})
        else:
            dim, rot, vdim, rank = int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
            if entry["type"] == "latent_attention":
                out.update({f"{layer}.mix.dq": (int(m["q_rank"]), width), f"{layer}.mix.dq.norm": (int(m["q_rank"]),),
                            f"{layer}.mix.uq": (heads * (dim + rot), int(m["q_rank"]))})
            else:
                out.update({f"{layer}.mix.q": (heads * (dim + rot), width), f"{layer}.mix.sink": (heads,),
                            f"{layer}.mix.g": (heads, width)})
            if m.get("kv_from") is None:
                out.update({f"{layer}.mix.dkv": (rank + rot, width), f"{layer}.mix.dkv.norm": (rank,)})
            out.update({f"{layer}.mix.uk": (heads * dim, rank), f"{layer}.mix.uv": (heads * vdim, rank),
                        f"{layer}.mix.o": (width, heads * vdim)})
        if entry.get("mlp") is not None:
            ff = int(entry["mlp"]["ff"])
            out.update({f"{layer}.mlp.gate": (ff, width), f"{layer}.mlp.up": (ff, width), f"{layer}.mlp.down": (width, ff)})
    return out


def random_weights(config: dict, seed: int, layer_scale: bool = True) -> dict[str, torch.Tensor]:
    """Weights of a size that makes every mechanism matter: matrices with unit-size outputs, norm offsets and
    layer scales well away from their neutral values, sinks comparable with the scores, mixing tables dense.
    Matrices are rounded to bfloat16 values (kept in float32) so that a bfloat16 engine holds the same numbers."""
    generator = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config, layer_scale).items():
        last = name.split(".", 1)[-1]
        if len(shape) == 2 and ".hc" not in name:
            tensor = torch.randn(shape, generator=generator) * (1.2 / math.sqrt(shape[1]))
            tensor = tensor.to(torch.bfloat16).to(torch.float32)
        elif last.endswith("mix") and ".hc" in name:
            tensor = torch.eye(shape[0]) * 0.7 + torch.rand(shape, generator=generator) * 0.4 - 0.1
        elif last.endswith(".in"):
            tensor = torch.rand(shape, generator=generator) * 0.6 + 0.2
        elif last.endswith(".out"):
            tensor = torch.rand(shape, generator=generator) * 1.0 + 0.5
        elif last.startswith("ls"):
            tensor = torch.rand(shape, generator=generator) * 1.0 + 0.5
        elif last == "mix.sink":
            tensor = torch.randn(shape, generator=generator) * 1.5
        elif last in ("mix.norm", "mix.dq.norm", "mix.dkv.norm"):
            tensor = 1.0 + torch.rand(shape, generator=generator) * 0.6 - 0.3
        else:   # the offset norms: weights around zero
            tensor = torch.rand(shape, generator=generator) * 0.6 - 0.3
        out[name] = tensor.contiguous()
    return out


def write_model(folder, config: dict, seed: int, layer_scale: bool = True) -> dict[str, torch.Tensor]:
    """config.json and model.safetensors (float32) of a random model; returns the weights."""
    from safetensors.torch import save_file

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    weights = random_weights(config, seed, layer_scale)
    (folder / "config.json").write_text(json.dumps(config, indent=1))
    save_file(weights, str(folder / "model.safetensors"))
    return weights
