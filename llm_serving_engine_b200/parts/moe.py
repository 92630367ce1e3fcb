"""Mixture-of-experts feed-forward: a softmax router over experts and identity experts, clamped gated experts, and a
gated shared expert."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.tensor_spec import TensorSpec
from .base import FeedForward, register_feed_forward
from .linear import linear, linear_partials, SKINNY_MAX_ROWS

_DEFAULT_NAMES = {"router": "router", "correction": "correction", "expert": "e{index}.", "shared": "shared.",
                  "gate": "gate", "up": "up", "down": "down", "shared_gate": "sg"}


@register_feed_forward("clamped_moe")
class ClampedMoE(FeedForward):
    """params: ``experts``, ``identity`` (the router's last ``identity`` outputs stand for experts whose output is the
    input itself), ``top``, ``ff`` and ``limit`` of an expert, ``correction`` (a learned vector added to the scores for
    the choice only; default true), ``shared`` ({"ff", "limit"} or None: an expert that every token uses, times
    sigmoid(w_sg . x)), ``tensor_names``.

    Expert: g = min(W_gate x, limit), u = clamp(W_up x, -limit, limit), y = W_down (g sigmoid(1.702 g) (u + 1)).
    Router: s = softmax(W_router x) over all outputs, in float32; the ``top`` outputs with the largest s + correction
    are chosen; the weights are their s, not renormalised.

    All experts run side by side as two products: [all gates | all ups] of every expert and the shared one stacked into
    one matrix, the activation kernel multiplying each expert's columns by the token's weight for it (zero where it
    was not chosen), and the down matrices side by side, so that the second product is the weighted sum over the
    experts.  Which kernels run does not depend on the routing (the step can be replayed from a CUDA graph); the price
    is that every expert's product is taken for every token."""

    graph_safe = True

    def __init__(self, params, weights, ctx) -> None:
        super().__init__(params, weights, ctx)
        p = params
        self.experts, self.identity, self.top = int(p["experts"]), int(p.get("identity", 0)), int(p["top"])
        self.ff, self.limit = int(p["ff"]), float(p["limit"])
        shared = p.get("shared")
        self.shared_ff = int(shared["ff"]) if shared else 0
        self.shared_limit = float(shared["limit"]) if shared else 0.0
        names = {**_DEFAULT_NAMES, **p.get("tensor_names", {})}
        prefixes = [names["expert"].format(index=index) for index in range(self.experts)]
        if shared:
            prefixes.append(names["shared"])
        gates = [weights[prefix + names["gate"]] for prefix in prefixes]
        ups = [weights[prefix + names["up"]] for prefix in prefixes]
        self.inter = self.experts * self.ff + self.shared_ff
        self.gate_up_weight = torch.cat(gates + ups, dim=0).contiguous() if prefixes else None
        self.down_weight = torch.cat([weights[prefix + names["down"]] for prefix in prefixes], dim=1).contiguous() if prefixes else None
        self.router = weights[names["router"]].contiguous()
        self.correction = weights[names["correction"]].float().contiguous() if p.get("correction", True) else None
        self.shared_gate_w = weights[names["shared"] + names["shared_gate"]].reshape(-1).contiguous() if shared else None

    @classmethod
    def expected_tensors(cls, params, hidden_size):
        p = params
        experts, identity, ff = int(p["experts"]), int(p.get("identity", 0)), int(p["ff"])
        names = {**_DEFAULT_NAMES, **p.get("tensor_names", {})}
        out = {names["router"]: TensorSpec((experts + identity, hidden_size))}
        if p.get("correction", True):
            out[names["correction"]] = TensorSpec((experts + identity,), "bias")
        sized = [(names["expert"].format(index=index), ff) for index in range(experts)]
        if p.get("shared"):
            sized.append((names["shared"], int(p["shared"]["ff"])))
            out[names["shared"] + names["shared_gate"]] = TensorSpec((1, hidden_size))
        for prefix, width in sized:
            out[prefix + names["gate"]] = TensorSpec((width, hidden_size))
            out[prefix + names["up"]] = TensorSpec((width, hidden_size))
            out[prefix + names["down"]] = TensorSpec((hidden_size, width))
        return out

    def forward(self, x):
        tokens = x.shape[0]
        expert_weights, identity_weight, shared_gate = ops.moe_route(x, self.router, self.correction, self.shared_gate_w,
                                                                     self.identity, self.top)
        if self.inter:
            gate_up = linear_partials(x, self.gate_up_weight)
            act = torch.empty((tokens, self.inter), dtype=x.dtype, device=x.device)
            ops.moe_gated_act(gate_up, expert_weights, shared_gate, act, self.experts, self.ff, self.shared_ff,
                              self.limit, self.shared_limit)
            if x.dtype == torch.bfloat16 and tokens > SKINNY_MAX_ROWS:
                y = linear(act, self.down_weight, out_dtype=torch.float32)   # the identity experts' share is added in float32
            else:
                y = linear_partials(act, self.down_weight)
        else:
            y = torch.zeros((tokens, x.shape[1]), dtype=torch.float32, device=x.device)
        if self.identity:
            ops.add_scaled_rows(y[0] if y.dim() == 3 else y, identity_weight, x)
        return y
