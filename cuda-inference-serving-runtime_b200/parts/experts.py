"""Routed experts: many small feed-forward layers of which each token uses a few.

    scores    s = sigmoid(W_router h): float sums (one of the engine's matrix products), float sigmoid; or
              s = softmax(W_router h) over all router outputs (`scores` "softmax")
    bias      a per-output choice bias (`names["choice_bias"]`), added to s for the choice only; the weights use s
    groups    the experts form `groups` equal groups of neighbours; a group's score is the sum of its two best members;
              only members of the `keep` best groups can be chosen (groups 0: every expert can)
    choice    the `top` best open experts, each weighted by s * route_scale; with `renormalize` the chosen scores are
              divided by their sum (+ 1e-20) before the scale
    expert    W_down act(W_up h), no biases; act(z) = max(z, 0)^2 ("relu_squared") or the exact gelu z Phi(z) ("gelu");
              or gated ("gated_clamp"):
              g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit), W_down (g sigmoid(1.702 g) (u + 1))
    identity  the last `identity` router outputs have no matrices: such an expert's output is h itself
    shared    an expert of the same form (its own width and limit) that every token uses, times sigmoid(w_sg . h)
    output    the weighted sum of the chosen experts' outputs (+ the shared expert's)

The experts' matrices are stacked at load ([experts, ff, hidden] and [experts, hidden, ff]) so one launch serves
whichever experts a step's tokens chose.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..ops import kernels
from .base import FEED_FORWARDS, FeedForward, TensorNeed, register
from .linear import linear, linear_add

ACTIVATIONS = ("relu_squared", "gelu", "gated_clamp")
DEFAULT_NAMES = {"router": "router.weight", "up": "experts.{}.up.weight", "down": "experts.{}.down.weight",
                 "gate": "experts.{}.gate.weight", "choice_bias": "correction", "shared_gate": "shared.gate", "shared_up": "shared.up",
                 "shared_down": "shared.down", "shared_scale": "shared.sg"}


@register(FEED_FORWARDS, "routed_experts")
class RoutedExperts(FeedForward):
    """params: hidden_size, expert_size, experts, top, groups, keep, route_scale, activation, names (local tensor names:
    router, and up / down (/ gate) with {} for the expert's number); scores ("sigmoid" or "softmax"), choice_bias (bool),
    identity (router outputs beyond `experts` without matrices), limit (of the gated activation), shared (None, or
    {"size", "limit"}: the shared expert), renormalize (bool: the chosen scores are divided by their sum)."""

    applies_output_scale = True      # forward(h, ctx, out_scale): a per-channel layer scale is the epilogue of the last kernel

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.hidden = int(spec["hidden_size"])
        self.ff = int(spec["expert_size"])
        self.experts = int(spec["experts"])
        self.top = int(spec["top"])
        self.groups = int(spec.get("groups") or 0)
        self.keep = int(spec.get("keep") or 0)
        self.route_scale = float(spec.get("route_scale", 1.0))
        self.activation = spec.get("activation", "relu_squared")
        self.names = {**DEFAULT_NAMES, **dict(spec.get("names") or {})}
        self.scores = spec.get("scores", "sigmoid")
        self.has_choice_bias = bool(spec.get("choice_bias", False))
        self.identity = int(spec.get("identity") or 0)
        self.renormalize = bool(spec.get("renormalize", False))
        self.gated = self.activation == "gated_clamp"
        self.limit = float(spec["limit"]) if self.gated else None
        shared = spec.get("shared")
        self.shared_size = int(shared["size"]) if shared else 0
        self.shared_limit = float(shared["limit"]) if shared else None
        if self.scores not in ("sigmoid", "softmax"):
            raise ValueError(f"router scores {self.scores!r} are not implemented; known: sigmoid, softmax")
        if self.identity and self.groups:
            raise ValueError("identity experts and expert groups are not combined")
        if self.activation not in ACTIVATIONS:
            raise ValueError(f"expert activation {self.activation!r} is not implemented; known: {', '.join(ACTIVATIONS)}")
        if not 0 < self.top <= self.experts + self.identity:
            raise ValueError("top must lie between 1 and the number of router outputs")
        if self.groups and (self.experts % self.groups or not 0 < self.keep <= self.groups
                            or self.keep * (self.experts // self.groups) < self.top):
            raise ValueError("groups must divide the experts, and the kept groups must hold at least top experts")
        self.router = self.up = self.down = self.choice_bias = None
        self.shared_in = self.shared_down = None

    def tensor_needs(self) -> Dict[str, TensorNeed]:
        # seeded random routers are drawn wide enough that a token's scores differ clearly
        outputs = self.experts + self.identity
        needs = {self.names["router"]: TensorNeed((outputs, self.hidden), init_std=4.0 / self.hidden ** 0.5)}
        if self.has_choice_bias:
            needs[self.names["choice_bias"]] = TensorNeed((outputs,), role="vector", init_mean=0.0, init_std=0.02)
        for e in range(self.experts):
            if self.gated:
                needs[self.names["gate"].format(e)] = TensorNeed((self.ff, self.hidden))
            needs[self.names["up"].format(e)] = TensorNeed((self.ff, self.hidden))
            needs[self.names["down"].format(e)] = TensorNeed((self.hidden, self.ff))
        if self.shared_size:
            needs[self.names["shared_gate"]] = TensorNeed((self.shared_size, self.hidden))
            needs[self.names["shared_up"]] = TensorNeed((self.shared_size, self.hidden))
            needs[self.names["shared_down"]] = TensorNeed((self.hidden, self.shared_size))
            needs[self.names["shared_scale"]] = TensorNeed((1, self.hidden))
        return needs

    def load(self, tensors):
        n = self.names
        self.router = tensors[n["router"]].contiguous()
        if self.has_choice_bias:
            self.choice_bias = tensors[n["choice_bias"]].float().contiguous()
        if self.gated:      # an expert's gate rows on top of its up rows: one product (or one pass over h) serves both
            self.up = torch.stack([torch.cat((tensors[n["gate"].format(e)], tensors[n["up"].format(e)]), dim=0)
                                   for e in range(self.experts)]).contiguous()
        else:
            self.up = torch.stack([tensors[n["up"].format(e)] for e in range(self.experts)]).contiguous()
        self.down = torch.stack([tensors[n["down"].format(e)] for e in range(self.experts)]).contiguous()
        if self.shared_size:
            # gate rows, up rows, then the row whose product with h is the logit of the shared expert's per-token factor
            self.shared_in = torch.cat((tensors[n["shared_gate"]], tensors[n["shared_up"]], tensors[n["shared_scale"]]), dim=0).contiguous()
            from .feedforward import pad_columns
            self.shared_down = pad_columns(tensors[n["shared_down"]], 8)

    def kernel_jobs(self):
        return (kernels.moe_jobs() + kernels.gemm_jobs(self.dtype) + (kernels.skinny_jobs() if self.dtype == torch.bfloat16 else [])
                + (kernels.ffn_rows_jobs() if self.gated or self.shared_size else [])
                + ([("elementwise.cu", {}, ())] if self.shared_size else []))

    def route(self, h: torch.Tensor):
        """(chosen experts int32 [tokens, top], best first; their weights float [tokens, top])."""
        tokens = h.shape[0]
        chosen = torch.empty((tokens, self.top), dtype=torch.int32, device=h.device)
        weight = torch.empty((tokens, self.top), dtype=torch.float32, device=h.device)
        logits = linear(h, self.router)          # float sums, by the engine's products for this many tokens
        kernels.moe_select(logits, self.top, self.groups, self.keep, self.route_scale, chosen, weight, scores=self.scores,
                           choice_bias=self.choice_bias, renormalize=self.renormalize)
        return chosen, weight

    def shared_expert(self, h: torch.Tensor, into: torch.Tensor) -> torch.Tensor:
        """into += sigmoid(w_sg . h) * W_down act(W_gate h, W_up h): the factor is applied to the activations (the product
        after it is linear), in float, before their one rounding; the add is the last product's epilogue."""
        sums = linear(h, self.shared_in)                   # float [tokens, gate | up | factor logit]
        act = torch.empty((h.shape[0], self.shared_down.shape[1]), dtype=self.dtype, device=h.device)
        kernels.gated_clamp(sums, self.shared_size, self.shared_limit, act, scale_col=2 * self.shared_size)
        return linear_add(act, self.shared_down, into)

    def forward(self, h, ctx, out_scale=None):
        tokens = h.shape[0]
        chosen, weight = self.route(h)
        out = torch.empty((tokens, self.hidden), dtype=torch.float32, device=h.device)
        if self.shared_size and out_scale is not None:
            raise NotImplementedError("a shared expert under a per-channel output scale is not built")
        if kernels.moe_grouped_ok(h, self.up, self.top, gated=self.gated):
            kernels.moe_grouped(h, self.up, self.down, chosen, weight, out, out_scale, gate_limit=self.limit,
                                activation=self.activation)                                         # many tokens: sorted by expert, tcgen05
        else:
            act = torch.empty((tokens * self.top, self.ff), dtype=self.dtype, device=h.device)
            kernels.moe_rows(h, self.up, self.down, chosen, weight, act, out, out_scale, gate_limit=self.limit,
                             activation=self.activation)
        if self.shared_size:
            self.shared_expert(h, out)
        return out
