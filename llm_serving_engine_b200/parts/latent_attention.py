"""Attention whose keys and values are made from a cached low-rank latent."""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from ..weights.tensor_spec import TensorSpec
from .base import Mixer, PagedLatent, register_mixer
from .linear import linear_partials

PER_HEAD_LIBRARY_ROWS = 32    # above this many bfloat16 rows the per-head products are the library's batched product

_DEFAULT_NAMES = {"q_down": "dq", "q_down_norm": "dq.norm", "q_up": "uq", "q": "q", "kv_down": "dkv",
                  "kv_down_norm": "dkv.norm", "k_up": "uk", "v_up": "uv", "sink": "sink", "gate": "g", "out": "o"}


def rotary_frequencies(rot: dict) -> tuple[torch.Tensor, float]:
    """Frequencies (float64 [dims / 2]) and the factor on cos and sin of a rotary description ``{base, dims,
    scaling}``.  Without ``scaling``: f_i = base^(-2i / dims), factor 1.  With ``scaling`` = {factor s, original n,
    fast, slow} (the scheme known as YaRN): with pair(t) = dims ln(n / (2 pi t)) / (2 ln base) the index of the pair
    that makes t turns over n positions, lo = max(floor(pair(fast)), 0), hi = min(ceil(pair(slow)), dims - 1) and
    ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), the frequency is f_i / s * ramp_i + f_i (1 - ramp_i):
    fast pairs keep theirs, slow pairs are stretched by s; cos and sin are multiplied by 0.1 ln(s) + 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    index = torch.arange(dims // 2, dtype=torch.float64)
    freq = base ** (-2.0 * index / dims)
    scaling = rot.get("scaling")
    if not scaling:
        return freq, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair(float(scaling["slow"]))), dims - 1)
    ramp = ((index - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return freq / factor * ramp + freq * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    """params: ``heads``, ``dim`` (unrotated query/key size of a head), ``rot_dim`` (rotated size), ``vdim``,
    ``kv_rank`` (the latent), ``q_rank`` (0: queries are projected directly; else they go through a normed latent of
    this size), ``scale`` (on the scores), ``rot`` ({base, dims, scaling}: see :func:`rotary_frequencies`; the first
    ``dims`` of the ``rot_dim`` values are rotated in interleaved pairs), ``eps`` (of the latent norms), ``sink`` (a
    learned number per head in the softmax's denominator), ``gate`` (head h's output times sigmoid(W_g x)_h),
    ``own_cache`` (false: the layer reads the latent rows of another layer, ``LayerSpec.cache_from``, and has no
    down-projection of its own), ``tensor_names``.

    c = norm(W_dkv x)[:kv_rank] and the rotated last rot_dim values of W_dkv x (shared by the heads) are the cached
    row of a token; head h's key is [W_uk,h c | shared part], its value W_uv,h c.  The per-head maps are folded
    around the attention: q' = W_uk,h^T q_unrotated before it, W_uv,h after it, so that the attention runs over the
    cached rows themselves (``csrc/attention_latent.cu``)."""

    graph_safe = True

    def __init__(self, params, weights, ctx) -> None:
        super().__init__(params, weights, ctx)
        p = params
        self.heads, self.dim, self.rot_dim = int(p["heads"]), int(p["dim"]), int(p["rot_dim"])
        self.vdim, self.rank, self.q_rank = int(p["vdim"]), int(p["kv_rank"]), int(p.get("q_rank") or 0)
        self.scale, self.eps = float(p["scale"]), float(p["eps"])
        self.window = int(p.get("window", 0))
        self.own_cache = bool(p.get("own_cache", True))
        self.rot_dims = int(p["rot"]["dims"])
        if self.rot_dims > self.rot_dim or self.rot_dims % 2:
            raise ops.KernelError(f"latent attention: {self.rot_dims} rotated values of {self.rot_dim}")
        freq, self.rot_factor = rotary_frequencies(p["rot"])
        self.freq = freq.to(ctx.device)
        names = {**_DEFAULT_NAMES, **p.get("tensor_names", {})}
        stacked, self.q_off, self.kv_off, self.g_off = [], 0, -1, -1
        width = 0
        if self.q_rank:
            stacked.append(weights[names["q_down"]])
            self.q_norm = weights[names["q_down_norm"]].to(torch.float32).contiguous()
            self.q_up = weights[names["q_up"]].contiguous()
            width += self.q_rank
        else:
            stacked.append(weights[names["q"]])
            width += self.heads * (self.dim + self.rot_dim)
        self.kv_norm = None
        if self.own_cache:
            stacked.append(weights[names["kv_down"]])
            self.kv_norm = weights[names["kv_down_norm"]].to(torch.float32).contiguous()
            self.kv_off = width
            width += self.rank + self.rot_dim
        if p.get("gate", False):
            stacked.append(weights[names["gate"]])
            self.g_off = width
            width += self.heads
        self.in_weight = torch.cat(stacked, dim=0).contiguous()
        self.k_up = weights[names["k_up"]].contiguous().view(self.heads, self.dim, self.rank)
        self.v_up = weights[names["v_up"]].contiguous().view(self.heads, self.vdim, self.rank).transpose(1, 2)
        self.sink = weights[names["sink"]].to(torch.float32).contiguous() if p.get("sink", False) else None
        self.out_weight = weights[names["out"]].contiguous()

    @classmethod
    def expected_tensors(cls, params, hidden_size):
        p = params
        heads, dim, rot, vdim, rank = int(p["heads"]), int(p["dim"]), int(p["rot_dim"]), int(p["vdim"]), int(p["kv_rank"])
        q_rank = int(p.get("q_rank") or 0)
        names = {**_DEFAULT_NAMES, **p.get("tensor_names", {})}
        out = {}
        if q_rank:
            out[names["q_down"]] = TensorSpec((q_rank, hidden_size))
            out[names["q_down_norm"]] = TensorSpec((q_rank,), "norm")
            out[names["q_up"]] = TensorSpec((heads * (dim + rot), q_rank))
        else:
            out[names["q"]] = TensorSpec((heads * (dim + rot), hidden_size))
        if p.get("own_cache", True):
            out[names["kv_down"]] = TensorSpec((rank + rot, hidden_size))
            out[names["kv_down_norm"]] = TensorSpec((rank,), "norm")
        out[names["k_up"]] = TensorSpec((heads * dim, rank))
        out[names["v_up"]] = TensorSpec((heads * vdim, rank))
        if p.get("sink", False):
            out[names["sink"]] = TensorSpec((heads,), "bias")
        if p.get("gate", False):
            out[names["gate"]] = TensorSpec((heads, hidden_size))
        out[names["out"]] = TensorSpec((hidden_size, heads * vdim))
        return out

    @classmethod
    def cache_requirement(cls, params, hidden_size):
        return PagedLatent(int(params["kv_rank"]) + int(params["rot_dim"]), int(params.get("window", 0)))

    @staticmethod
    def _per_head(a, weight, out, gate) -> None:
        """out[t, h] = gate[t, h] * a[t, h] @ weight[h]: many bfloat16 rows go to the library's batched product (the
        tensor cores), few rows and float32 to the engine's own kernel (true float32, one summation order)."""
        if a.dtype == torch.bfloat16 and a.shape[0] > PER_HEAD_LIBRARY_ROWS:
            product = torch.bmm(a.transpose(0, 1), weight)            # [heads, T, N], float32 accumulation
            if gate is None:
                out.copy_(product.transpose(0, 1))
            else:
                torch.mul(product.transpose(0, 1), gate.unsqueeze(-1), out=out)
        else:
            ops.head_gemm(a, weight, out, gate)

    def forward(self, x, step, cache):
        tokens, heads = x.shape[0], self.heads
        proj = linear_partials(x, self.in_weight)
        q_latent = torch.empty((tokens, self.q_rank), dtype=x.dtype, device=x.device) if self.q_rank else None
        gate = torch.empty((tokens, heads), dtype=torch.float32, device=x.device) if self.g_off >= 0 else None
        if self.q_rank or self.own_cache or gate is not None:
            ops.latent_prepare(proj, step.positions, cache.slot_mapping, self.eps,
                               q_off=self.q_off, q_rank=self.q_rank, q_norm=self.q_norm if self.q_rank else None,
                               q_latent=q_latent, kv_off=self.kv_off, rank=self.rank, kv_norm=self.kv_norm,
                               rot=self.rot_dim, rot_dims=self.rot_dims, freq=self.freq, rot_factor=self.rot_factor,
                               cache=cache.keys, g_off=self.g_off, heads=heads, gate=gate)
        queries = linear_partials(q_latent, self.q_up) if self.q_rank else proj
        wide = self.rank + self.rot_dim
        q_plain = torch.empty((tokens, heads, self.dim), dtype=x.dtype, device=x.device)
        q_wide = torch.empty((tokens, heads, wide), dtype=x.dtype, device=x.device)
        ops.latent_query(queries, 0, heads, self.dim, self.rot_dim, self.rot_dims, self.freq, self.rot_factor,
                         step.positions, step.segment_of_token, q_plain, q_wide, self.rank)
        self._per_head(q_plain, self.k_up, q_wide[:, :, :self.rank], None)
        attended = torch.empty((tokens, heads, self.rank), dtype=x.dtype, device=x.device)
        ops.latent_attention(q_wide, cache.keys, attended, cache.block_tables, step.segment_of_token, step.positions,
                             self.scale, self.sink, self.window, segment_start=step.segment_start,
                             segment_first_position=step.segment_first_position)
        values = torch.empty((tokens, heads, self.vdim), dtype=x.dtype, device=x.device)
        self._per_head(attended, self.v_up, values, gate)
        return linear_partials(values.view(tokens, heads * self.vdim), self.out_weight)
