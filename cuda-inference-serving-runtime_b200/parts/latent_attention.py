"""Latent attention: keys and values of all heads are derived from one small latent per token, and only that
latent and one rotated key part shared by the heads are cached.

Per token, with input h (the normed stream):

    queries      q = W_q h, or through a latent: q = W_qup unit(W_qdown h) * w_qnorm
                 each head's q is [plain part (plain_dim) | rotated part (rot_dim)]
    latent       [c_raw | k_raw] = W_kvdown h;  c = unit(c_raw) * w_kvnorm (kv_rank wide);  k_rot = rotate(k_raw)
    per head     key_h = [W_kup_h c | k_rot],  value_h = W_vup_h c
    scores       (q_h . key_h) * scale over the keys j <= i (with `window`: i - j < window), softmax (with `sink`: one more
                 term exp(sink_h) per head in the denominator, with no key and no value), out_h = sum of weights * value_h
    output       W_out (concatenated heads [* sigmoid(W_gate h)])

`shared_kv`: the layer has no down projection of its own and reads the cache rows of an earlier run entry (the run list's
`cache_of`) as they are stored, with its own up projections, queries, window and sink.

unit(v) = v / sqrt(mean(v^2) + eps).  The cache row of a token is [c | k_rot | 0 pad]: one plane, one "head".  Since
q_h,plain . (W_kup_h c) = (W_kup_h^T q_h,plain) . c, each query is carried into the latent's basis once
([W_kup_h^T q_h,plain | rotated part], one product per head), attention then runs over the cache rows as they are
stored with every query head sharing the one row per key (the paged attention kernels, keys = values = the rows), and
W_vup_h is applied to the weighted sum of latents afterwards (again one product per head).  Prompt portions and
single tokens take the same path, so a position's result does not depend on how its prompt was cut.

Unit norms, rotation, scores, softmax and the gate's sigmoid are float arithmetic; in bfloat16 serving the operands of
the matrix products and the cache rows are rounded to bfloat16 once.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..config.spec import CacheUse
from ..ops import kernels
from .attention import ATTENTION_PLAN_KEY, attention_step_plan, paged_attention
from .base import MIXERS, POSITIONS, Mixer, TensorNeed, build_part, register
from .linear import as_tensor, linear, linear_to_stream, norm_fusable

ROW_STEP = 16          # cache rows are padded to a multiple of this (the attention kernels' head sizes)
DEFAULT_NAMES = {"sink": "sink", "q": "q_proj.weight", "q_down": "q_down.weight", "q_norm": "q_norm.weight", "q_up": "q_up.weight",
                 "kv_down": "kv_down.weight", "kv_norm": "kv_norm.weight", "k_up": "k_up.weight", "v_up": "v_up.weight",
                 "gate": "gate.weight", "out": "o_proj.weight"}


@register(MIXERS, "latent_attention")
class LatentAttention(Mixer):
    """params: hidden_size, num_heads, plain_dim, rot_dim, value_dim, kv_rank, q_rank (0: queries straight from the
    input), gate (bool: sigmoid output gate), position (PartSpec of a rotary encoding over rot_dim), scale, eps,
    window (None or int: the keys a query keeps in sight), sink (bool: a learned softmax sink per head), shared_kv (bool:
    no down projection, the cache rows of another run entry), names (local tensor names of q, q_down, q_norm, q_up,
    kv_down, kv_norm, k_up, v_up, gate, out, sink)."""

    graph_safe = True
    accepts_pending_norm = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.hidden = int(spec["hidden_size"])
        self.heads = int(spec["num_heads"])
        self.plain = int(spec["plain_dim"])
        self.rot = int(spec["rot_dim"])
        self.vdim = int(spec["value_dim"])
        self.kv_rank = int(spec["kv_rank"])
        self.q_rank = int(spec.get("q_rank") or 0)
        self.gate = bool(spec.get("gate", False))
        self.scale = float(spec["scale"])
        self.eps = float(spec["eps"])
        self.window = spec.get("window")
        self.has_sink = bool(spec.get("sink", False))
        self.shared_kv = bool(spec.get("shared_kv", False))
        self.sink = None
        self.names = {**DEFAULT_NAMES, **dict(spec.get("names") or {})}
        self.position = build_part(POSITIONS, spec["position"], dtype, "position encoding")
        if self.rot % 2 or getattr(self.position, "dim", self.rot) != self.rot:
            raise ValueError("the rotated part must be even and as wide as the position encoding turns")
        self.row = -(-(self.kv_rank + self.rot) // ROW_STEP) * ROW_STEP
        if self.row > 256:
            raise ValueError(f"kv_rank + rot_dim = {self.kv_rank + self.rot} is not supported: cache rows are at most 256 wide")
        self.head_w = self.plain + self.rot

    # ---------------------------------------------------------------- tensors
    def tensor_needs(self) -> Dict[str, TensorNeed]:
        n, H = self.names, self.heads
        needs = {n["k_up"]: TensorNeed((H * self.plain, self.kv_rank)),
                 n["v_up"]: TensorNeed((H * self.vdim, self.kv_rank)),
                 n["out"]: TensorNeed((self.hidden, H * self.vdim))}
        if not self.shared_kv:
            needs[n["kv_down"]] = TensorNeed((self.kv_rank + self.rot, self.hidden))
            needs[n["kv_norm"]] = TensorNeed((self.kv_rank,), role="vector")
        if self.has_sink:
            needs[n["sink"]] = TensorNeed((H,), role="vector", init_mean=0.0, init_std=1.0)
        if self.q_rank:
            needs[n["q_down"]] = TensorNeed((self.q_rank, self.hidden))
            needs[n["q_norm"]] = TensorNeed((self.q_rank,), role="vector")
            needs[n["q_up"]] = TensorNeed((H * self.head_w, self.q_rank))
        else:
            needs[n["q"]] = TensorNeed((H * self.head_w, self.hidden))
        if self.gate:
            needs[n["gate"]] = TensorNeed((H * self.vdim, self.hidden))
        return needs

    def load(self, tensors):
        n, H = self.names, self.heads
        # one product serves every projection that reads the layer's input: [queries or their latent | kv latent + key part | gate]
        first = tensors[n["q_down"]] if self.q_rank else tensors[n["q"]]
        stacked = [first] + ([] if self.shared_kv else [tensors[n["kv_down"]]]) + ([tensors[n["gate"]]] if self.gate else [])
        self.w_in = torch.cat(stacked, dim=0).contiguous()
        self.c_col = first.shape[0]
        self.gate_col = self.c_col + (0 if self.shared_kv else self.kv_rank + self.rot)
        self.q_up = tensors[n["q_up"]].contiguous() if self.q_rank else None
        self.q_norm = tensors[n["q_norm"]].float().contiguous() if self.q_rank else None
        self.kv_norm = None if self.shared_kv else tensors[n["kv_norm"]].float().contiguous()
        self.sink = tensors[n["sink"]].float().contiguous() if self.has_sink else None      # a score: float whatever the storage type
        self.k_up = tensors[n["k_up"]].contiguous().view(H, self.plain, self.kv_rank)     # per head [plain_dim (k), kv_rank (n)]
        self.v_up = tensors[n["v_up"]].contiguous().view(H, self.vdim, self.kv_rank)      # per head [value_dim (n), kv_rank (k)]
        self.o = tensors[n["out"]].contiguous()

    def kernel_jobs(self):
        return ([("elementwise.cu", {}, ()), kernels.attention_jobs(self.row, self.dtype)] + kernels.latent_jobs()
                + kernels.attention_tcgen05_jobs(self.row, self.dtype) + kernels.gemm_jobs(self.dtype) + self.position.kernel_jobs()
                + (kernels.skinny_jobs() if self.dtype == torch.bfloat16 else []))

    def cache_use(self) -> CacheUse:
        return CacheUse("pages", kv_heads=1, head_dim=self.row, window=self.window, planes=1)

    # ---------------------------------------------------------------- the step
    def plan_key(self):
        return ATTENTION_PLAN_KEY

    def step_plan(self, host):
        return attention_step_plan(host)

    def begin_step(self, ctx) -> None:
        self.position.rotation(ctx)

    def forward(self, h, ctx, cache):
        if cache.write == self.shared_kv:
            raise ValueError("latent_attention: a layer with a down projection writes its own cache rows, one without reads another entry's")
        tokens, H, device = ctx.n_tokens, self.heads, ctx.device
        rot = self.position.rotation(ctx)
        table = dict(cos=rot.cos, sin=rot.sin, rot_half=rot.rot_half, interleaved=rot.interleaved)
        if norm_fusable(h, tokens, self.w_in):
            # few tokens: the residual add and the norm are the prologue of the stacked input product
            proj = torch.empty((tokens, self.w_in.shape[0]), dtype=torch.float32, device=device)
            x_out = h.new_stream_buffer()
            kernels.skinny_gemm(self.w_in, tokens, x=h.x, delta=h.delta, norm_w=h.weight, eps=h.eps, x_out=x_out,
                                epilogue=kernels.EPI_PLAIN, out=proj)
            h.done(x_out)
        else:
            proj = linear(as_tensor(h), self.w_in)                             # float [tokens, stacked rows]
        cq = torch.empty((tokens, self.q_rank), dtype=self.dtype, device=device) if self.q_rank else None
        if self.q_rank or cache.write:
            kernels.latent_rows(proj, 0, self.q_rank, self.q_norm, cq, self.c_col, self.kv_rank, self.kv_norm, self.eps,
                                cache=cache.k if cache.write else None, token_req=ctx.token_req, positions=ctx.positions,
                                req_slot=ctx.req_slot, block_table=cache.block_table, page_size=cache.page_size, **table)
        q = linear(cq, self.q_up) if self.q_rank else proj                     # heads of [plain | rotated part] from column 0
        q_rows = torch.empty((tokens, H, self.row), dtype=self.dtype, device=device)
        few = tokens <= kernels.LATENT_ROW_KERNEL_MAX_TOKENS
        if few:      # a decode step: rotation and the product with W_kup_h in one row kernel
            kernels.latent_absorb(q, 0, H, self.plain, k_up=self.k_up, q_rows=q_rows, kv_rank=self.kv_rank, **table)
        else:
            q_plain = torch.empty((tokens, H, self.plain), dtype=self.dtype, device=device)
            kernels.latent_query(q, 0, H, self.plain, plain_out=q_plain, q_rows=q_rows, kv_rank=self.kv_rank, **table)
            kernels.gemm_heads(q_plain, self.k_up, q_rows, w_is_nk=False)      # q_rows[:, h, :kv_rank] = W_kup_h^T q_plain_h
        mixed = paged_attention(ctx.plan_for(self), q_rows, cache.k, cache.k, cache, ctx, H, 1, self.scale, self.window, sink=self.sink)
        if few:      # W_vup_h (weighted sum of latents), gate and rounding in one row kernel
            values = kernels.latent_values(mixed, self.v_up, proj if self.gate else None, self.gate_col,
                                           torch.empty((tokens, H * self.vdim), dtype=self.dtype, device=device))
            return linear_to_stream(values, self.o, h)
        values = torch.empty((tokens, H, self.vdim), dtype=torch.float32, device=device)
        kernels.gemm_heads(mixed, self.v_up, values, w_is_nk=True)             # W_vup_h (weighted sum of latents)
        values = values.view(tokens, H * self.vdim)
        if self.gate or self.dtype != torch.float32:
            values = kernels.latent_gate(values, proj if self.gate else None, self.gate_col,
                                         torch.empty((tokens, H * self.vdim), dtype=self.dtype, device=device))
        return linear_to_stream(values, self.o, h)
