"""Lightning attention: linear attention with one fixed decay per head and a matrix state per head instead of a cache of keys.

    q = silu(W_q h), k = silu(W_k h)  [heads x key_dim],   v = silu(W_v h)  [heads x value_dim]
    per head:  S <- decay_h S + k v^T;   o = S^T q          (S [key_dim, value_dim]; no other scale)
    out = W_o [ o / sqrt(mean(o^2) + eps) * w_norm * sigmoid(W_g h) ]      the mean over all heads of the token at once

A request's state is S of every head, float, one row of a state tensor of the cache manager (`CacheUse("state", ...)`),
zero when the request starts and carried from step to step.  One product serves every projection that reads h
(q | k | v | gate, float sums); the activations, the decay, the state and its recurrence, the norm and the gate are float
arithmetic in the row kernels (csrc/lightning.cu).  Single tokens and short portions walk a request's tokens in order;
portions of CHUNKED_FROM tokens and more run the chunked form of the same recurrence, which differs by rounding only.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..config.spec import CacheUse
from ..ops import kernels
from .base import MIXERS, Mixer, TensorNeed, register
from .feedforward import pad_columns
from .linear import as_tensor, linear, linear_to_stream

CHUNKED_FROM = kernels.LIGHTNING_CHUNK
LIGHTNING_PLAN_KEY = ("lightning_chunks", CHUNKED_FROM)
DEFAULT_NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "norm": "norm", "o": "o"}


def long_and_short(q_len) -> tuple:
    """How many of a step's requests bring at least CHUNKED_FROM tokens, and how many fewer."""
    n_long = sum(1 for n in q_len if n >= CHUNKED_FROM)
    return n_long, len(q_len) - n_long


@register(MIXERS, "lightning")
class LightningAttention(Mixer):
    """params: hidden_size, num_heads, key_dim, value_dim, decay (one number in (0, 1] per head), eps (of the output norm),
    names (local tensor names of q, k, v, gate, norm, o)."""

    # forward reads the step through device tensors only.  A captured step's warm-up run outside the graph would advance
    # the state once too often: the graph code keeps the state tensors and puts them back after it (engine/graph.py).
    graph_safe = True
    accepts_pending_norm = True      # for its last product, which may add its result to the residual stream in place

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.hidden = int(spec["hidden_size"])
        self.heads = int(spec["num_heads"])
        self.key_dim, self.value_dim = int(spec["key_dim"]), int(spec["value_dim"])
        self.decay_values = [float(d) for d in spec["decay"]]
        self.eps = float(spec["eps"])
        self.names = {**DEFAULT_NAMES, **dict(spec.get("names") or {})}
        if len(self.decay_values) != self.heads or not all(0.0 < d <= 1.0 for d in self.decay_values):
            raise ValueError("lightning attention needs one decay in (0, 1] per head")
        if self.key_dim > kernels.LIGHTNING_MAX_KEY_DIM:
            raise ValueError(f"key heads of {self.key_dim} are not supported: the recurrence holds up to {kernels.LIGHTNING_MAX_KEY_DIM} rows per column")
        self.nqk, self.nv = self.heads * self.key_dim, self.heads * self.value_dim
        self.w_in = self.norm = self.o = self.decay = None

    def tensor_needs(self) -> Dict[str, TensorNeed]:
        n = self.names
        return {n["q"]: TensorNeed((self.nqk, self.hidden)), n["k"]: TensorNeed((self.nqk, self.hidden)),
                n["v"]: TensorNeed((self.nv, self.hidden)), n["gate"]: TensorNeed((self.nv, self.hidden)),
                n["norm"]: TensorNeed((self.nv,), role="vector"), n["o"]: TensorNeed((self.hidden, self.nv))}

    def load(self, tensors):
        n = self.names
        stacked = torch.cat([tensors[n[key]] for key in ("q", "k", "v", "gate")], dim=0)      # one product for everything that reads h
        extra = -stacked.shape[0] % 16
        if extra:
            stacked = torch.cat((stacked, torch.zeros((extra, self.hidden), dtype=stacked.dtype, device=stacked.device)), dim=0)
        self.w_in = stacked.contiguous()
        self.norm = tensors[n["norm"]].float().contiguous()
        self.o = pad_columns(tensors[n["o"]], 8)
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=stacked.device)     # float, as everything of the recurrence

    def kernel_jobs(self):
        return (kernels.lightning_jobs() + kernels.gemm_jobs(self.dtype)
                + (kernels.skinny_jobs() if self.dtype == torch.bfloat16 else []))

    def cache_use(self) -> CacheUse:
        return CacheUse("state", state_shape=(self.heads * self.key_dim * self.value_dim,), state_dtype="float32")

    # ---------------------------------------------------------------- the launch plan of a step
    def plan_key(self):
        return LIGHTNING_PLAN_KEY

    def step_plan(self, host):
        from ..engine.batch import StepPlan
        n_long, n_short = long_and_short(host.q_len)
        return StepPlan(arrays={}, info={"n_long": n_long, "n_short": n_short})

    def forward(self, h, ctx, cache):
        tokens = ctx.n_tokens
        proj = linear(as_tensor(h), self.w_in)                      # float [tokens, q | k | v | gate | padding]
        o = torch.empty((tokens, self.nv), dtype=torch.float32, device=ctx.device)
        plan = ctx.plan_for(self)
        kernels.lightning_recurrence(proj, 0, self.nqk, 2 * self.nqk, self.decay, cache.state, ctx.req_slot, ctx.q_start, ctx.q_len,
                                     ctx.n_requests, o, self.heads, self.key_dim, self.value_dim,
                                     least=CHUNKED_FROM if plan.info["n_long"] else 0, n_long=plan.info["n_long"],
                                     n_short=plan.info["n_short"])
        width = self.o.shape[1]
        make = torch.zeros if width != self.nv else torch.empty
        gated = make((tokens, width), dtype=self.dtype, device=ctx.device)
        kernels.lightning_output(o, proj, 2 * self.nqk + self.nv, self.norm, self.eps, gated)
        return linear_to_stream(gated, self.o, h)
