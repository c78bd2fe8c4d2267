"""Differential attention: every head runs two softmax attention maps over the same values and keeps their difference.

    q = conv(W_q h) [heads x (map 1 | map 2) x key_dim],  k = conv(W_k h) [kv_heads x (map 1 | map 2) x key_dim],
    v = conv(W_v h) [kv_heads x value_dim];  conv: a short causal convolution over time per channel (taps weights, no
    bias, zeros before the sequence), right after the projection
    a_m = softmax_j(q_m . k_m * scale) v  over the keys j <= i with i - j < window or j < keep_first   (m = 1, 2)
    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff            (one number for the layer)
    o = a_1 - lambda a_2;   o <- o / sqrt(mean(o^2) + eps) * (1 - diff)  per head;   o <- o * sigmoid(W_g h)
    out = W_o [heads of o]

`conv` 0: no convolution (and no kept inputs); `gate` False: no output gate; `position`: a rotary encoding that turns the
leading coordinates of each map of each head of q and k (keys are cached turned), or none.  `shared_kv`: the layer has no
key and value tensors and reads the pages of an earlier run entry (the run list's `cache_of`), with its own queries, mask
and everything else.

How it runs on the engine's paged attention kernels: the two maps are two query heads each (2 * heads query heads over
kv_heads key heads of one width D = max(2 key_dim, value_dim) rounded up to 16).  A key row of the cache is
[k_1 | k_2 | 0], the query row of map m has its key_dim numbers where k_m lies and zeros elsewhere, so the score is
exactly q_m . k_m, and a value row is stored once per key head.  Portions and single tokens take the same path.  What a
request keeps besides its pages: the last taps - 1 projected values of its convolved channels (`side_state`).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.spec import CacheUse
from ..ops import kernels
from .attention import ATTENTION_PLAN_KEY, attention_step_plan, paged_attention
from .base import MIXERS, POSITIONS, Mixer, TensorNeed, build_part, register
from .linear import linear_normed, linear_to_stream

DEFAULT_NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "o": "o", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv",
                 "lq1": "lq1", "lk1": "lk1", "lq2": "lq2", "lk2": "lk2"}
HEAD_STEP, HEAD_MAX = 16, 256      # the attention kernels are built per head width: multiples of 16 up to 256


@register(MIXERS, "diff_attention")
class DiffAttention(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, key_dim, value_dim, scale, diff, eps, conv (taps; 1: one weight per
    channel, 0: no convolution and no tensors for it), gate (bool, default True), position (PartSpec of a rotary encoding
    over the leading coordinates of each map, default none; only without a convolution), window (None or int), keep_first
    (int), shared_kv (bool: no key/value tensors, the pages of another run entry), in_place (bool, default False: the
    mixer takes its input as a pending norm and its output projection may add its result to the residual stream in
    place, where the arrangement allows that), names."""

    graph_safe = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.hidden = int(spec["hidden_size"])
        self.hq, self.hkv = int(spec["num_heads"]), int(spec["num_kv_heads"])
        self.key_dim, self.value_dim = int(spec["key_dim"]), int(spec["value_dim"])
        self.scale = float(spec["scale"])
        self.diff = float(spec["diff"])
        self.eps = float(spec["eps"])
        self.taps = int(spec.get("conv", 1))
        self.gate = bool(spec.get("gate", True))
        self.accepts_pending_norm = bool(spec.get("in_place", False))
        self.position = build_part(POSITIONS, spec["position"], dtype, "position encoding") if spec.get("position") is not None else None
        self.window = spec.get("window")
        self.keep_first = int(spec.get("keep_first") or 0)
        self.shared_kv = bool(spec.get("shared_kv", False))
        self.names = {**DEFAULT_NAMES, **dict(spec.get("names") or {})}
        if self.hq % self.hkv:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if self.taps < 0:
            raise ValueError("conv must not be negative (0: no convolution)")
        if self.position is not None and (self.taps or getattr(self.position, "dim", 0) > self.key_dim):
            raise ValueError("a position encoding turns at most key_dim coordinates of a map, and only where there is no convolution")
        self.width = -(-max(2 * self.key_dim, self.value_dim) // HEAD_STEP) * HEAD_STEP
        if self.width > HEAD_MAX:
            raise ValueError(f"two maps of {self.key_dim} or values of {self.value_dim} do not fit the attention kernels' rows of {HEAD_MAX}")
        self.nq, self.nk, self.nv = self.hq * 2 * self.key_dim, self.hkv * 2 * self.key_dim, self.hkv * self.value_dim
        self.channels = self.nq + (0 if self.shared_kv else self.nk + self.nv)       # convolved columns of the stacked projection
        self.w_in = self.o = self.conv_w = None
        self.lam = 0.0

    # ---------------------------------------------------------------- tensors
    def tensor_needs(self) -> Dict[str, TensorNeed]:
        n, taps = self.names, self.taps
        needs = {n["q"]: TensorNeed((self.nq, self.hidden))}
        if taps:
            needs[n["q_conv"]] = TensorNeed((self.nq, taps), role="vector", init_mean=1.0 / taps, init_std=0.3 / taps)
        if not self.shared_kv:
            needs[n["k"]] = TensorNeed((self.nk, self.hidden))
            needs[n["v"]] = TensorNeed((self.nv, self.hidden))
            if taps:
                needs[n["k_conv"]] = TensorNeed((self.nk, taps), role="vector", init_mean=1.0 / taps, init_std=0.3 / taps)
                needs[n["v_conv"]] = TensorNeed((self.nv, taps), role="vector", init_mean=1.0 / taps, init_std=0.3 / taps)
        for name in ("lq1", "lk1", "lq2", "lk2"):
            needs[n[name]] = TensorNeed((self.key_dim,), role="vector", init_mean=0.0, init_std=0.1)
        if self.gate:
            needs[n["gate"]] = TensorNeed((self.hq * self.value_dim, self.hidden))
        needs[n["o"]] = TensorNeed((self.hidden, self.hq * self.value_dim))
        return needs

    def load(self, tensors):
        n = self.names
        which = ("q",) if self.shared_kv else ("q", "k", "v")
        self.w_in = torch.cat([tensors[n[w]] for w in which] + ([tensors[n["gate"]]] if self.gate else []), dim=0).contiguous()     # convolved columns first
        if self.taps:
            # tap by tap [taps, channels]: neighbouring channels are neighbours in memory, as the row kernel's lanes read them
            self.conv_w = torch.cat([tensors[n[w + "_conv"]].float() for w in which], dim=0).t().contiguous()
        self.o = tensors[n["o"]].contiguous()
        l = {name: tensors[n[name]].float() for name in ("lq1", "lk1", "lq2", "lk2")}
        # one number for the layer, in float: exp(lq1 . lk1) - exp(lq2 . lk2) + diff
        self.lam = float((torch.exp((l["lq1"] * l["lk1"]).sum()) - torch.exp((l["lq2"] * l["lk2"]).sum())
                          + torch.tensor(self.diff, dtype=torch.float32, device=l["lq1"].device)).item())

    def kernel_jobs(self):
        return ([kernels.attention_jobs(self.width, self.dtype)] + kernels.diff_jobs() + (self.position.kernel_jobs() if self.position else [])
                + kernels.attention_tcgen05_jobs(self.width, self.dtype) + kernels.gemm_jobs(self.dtype)
                + (kernels.skinny_jobs() if self.dtype == torch.bfloat16 else []))

    def cache_use(self) -> CacheUse:
        return CacheUse("pages", kv_heads=self.hkv, head_dim=self.width, window=self.window,
                        keep_first=self.keep_first if self.window is not None else 0)

    def side_state(self) -> Optional[CacheUse]:
        """The request's last taps - 1 inputs of the convolution: the entry's own, also where it reads another's pages."""
        if not self.taps:
            return None
        return CacheUse("state", state_shape=(max(self.taps - 1, 1), self.channels), state_dtype="float32")

    # ---------------------------------------------------------------- the step
    def plan_key(self):
        return ATTENTION_PLAN_KEY

    def step_plan(self, host):
        return attention_step_plan(host)

    def begin_step(self, ctx) -> None:
        if self.position is not None:
            self.position.rotation(ctx)          # the rotation tables of the step, shared by every layer with the same encoding

    def forward(self, h, ctx, cache):
        if cache.write == self.shared_kv:
            raise ValueError("diff_attention: a layer with key and value tensors writes its own pages, one without reads another entry's")
        if self.taps and cache.state is None:
            raise ValueError("diff_attention needs its side state (the convolution's kept inputs) from the cache manager")
        tokens = ctx.n_tokens
        proj = linear_normed(h, self.w_in, tokens)                  # float [tokens, q (| k | v) (| gate)]
        q = torch.empty((tokens, 2 * self.hq, self.width), dtype=self.dtype, device=ctx.device)
        if not self.taps:
            rot = self.position.rotation(ctx) if self.position is not None else None
            kernels.diff_rope_rows(proj, self.nq, self.nq + self.nk, cos=rot.cos if rot else None, sin=rot.sin if rot else None,
                                   rot_half=rot.rot_half if rot else 0, interleaved=rot.interleaved if rot else False,
                                   token_req=ctx.token_req, req_slot=ctx.req_slot, positions=ctx.positions, q_out=q,
                                   k_cache=cache.k if cache.write else None, v_cache=cache.v if cache.write else None,
                                   block_table=cache.block_table, page_size=cache.page_size, hq=self.hq, hkv=self.hkv,
                                   key_dim=self.key_dim, value_dim=self.value_dim)
            return self.attend(q, proj, ctx, cache, h)
        kernels.diff_rows(proj, self.conv_w, self.taps, cache.state, token_req=ctx.token_req, req_slot=ctx.req_slot, q_start=ctx.q_start,
                          positions=ctx.positions, q_out=q, k_cache=cache.k if cache.write else None,
                          v_cache=cache.v if cache.write else None, block_table=cache.block_table, page_size=cache.page_size,
                          hq=self.hq, hkv=self.hkv, key_dim=self.key_dim, value_dim=self.value_dim)
        kernels.conv_keep(proj, cache.state, ctx.req_slot, ctx.q_start, ctx.q_len, ctx.n_requests, self.taps, self.channels)
        return self.attend(q, proj, ctx, cache, h)

    def attend(self, q, proj, ctx, cache, h):
        """The two maps of every head over the pages, their combination, the head norm, the gate and the output projection."""
        tokens = ctx.n_tokens
        mixed = paged_attention(ctx.plan_for(self), q, cache.k, cache.v, cache, ctx, 2 * self.hq, self.hkv, self.scale, self.window,
                                keep_first=self.keep_first if self.window is not None else 0)
        gated = torch.empty((tokens, self.hq * self.value_dim), dtype=self.dtype, device=ctx.device)
        kernels.diff_combine(mixed, proj if self.gate else None, self.channels, gated, self.hq, self.value_dim, self.lam, self.eps,
                             1.0 - self.diff)
        return linear_to_stream(gated, self.o, h)
