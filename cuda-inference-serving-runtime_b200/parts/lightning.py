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
from .linear import linear_normed, linear_to_stream

CHUNKED_FROM = kernels.LIGHTNING_CHUNK
LIGHTNING_PLAN_KEY = ("lightning_chunks", CHUNKED_FROM)
DEFAULT_NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "norm": "norm", "o": "o"}


def chunk_plan(q_len) -> tuple:
    """Which chunks the chunked recurrence runs for a step whose requests bring `q_len` tokens: per chunk its request and
    its first token inside the portion, per request the index of its first chunk; and how many requests stay with the
    token-by-token kernel.  Depends on the portion lengths alone, so steps of one shape share it."""
    chunk_req, chunk_t0, req_chunk0, short = [], [], [], 0
    for r, n in enumerate(q_len):
        req_chunk0.append(len(chunk_req))
        if n < CHUNKED_FROM:
            short += 1
            continue
        for t0 in range(0, n, kernels.LIGHTNING_CHUNK):
            chunk_req.append(r)
            chunk_t0.append(t0)
    return chunk_req, chunk_t0, req_chunk0, short


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
        import numpy as np

        from ..engine.batch import StepPlan
        chunk_req, chunk_t0, req_chunk0, short = chunk_plan(host.q_len)
        as_i32 = lambda values: np.asarray(values, dtype=np.int32)
        return StepPlan(arrays={"chunk_req": as_i32(chunk_req), "chunk_t0": as_i32(chunk_t0), "req_chunk0": as_i32(req_chunk0)},
                        info={"n_chunks": len(chunk_req), "n_short": short})

    def forward(self, h, ctx, cache):
        tokens = ctx.n_tokens
        proj = linear_normed(h, self.w_in, tokens)                  # float [tokens, q | k | v | gate | padding]
        o = torch.empty((tokens, self.nv), dtype=torch.float32, device=ctx.device)
        plan = ctx.plan_for(self)
        chunks = (plan["chunk_req"], plan["chunk_t0"], plan["req_chunk0"], plan.info["n_chunks"]) if plan.info["n_chunks"] else None
        kernels.lightning_recurrence(proj, 0, self.nqk, 2 * self.nqk, self.decay, cache.state, ctx.req_slot, ctx.q_start, ctx.q_len,
                                     ctx.n_requests, o, self.heads, self.key_dim, self.value_dim,
                                     least=CHUNKED_FROM if chunks else 0, n_short=plan.info["n_short"], chunks=chunks)
        width = self.o.shape[1]
        make = torch.zeros if width != self.nv else torch.empty
        gated = make((tokens, width), dtype=self.dtype, device=ctx.device)
        kernels.lightning_output(o, proj, 2 * self.nqk + self.nv, self.norm, self.eps, gated)
        return linear_to_stream(gated, self.o, h)
