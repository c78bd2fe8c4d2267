"""SwiGLU feed-forward: down(silu(gate(h)) * up(h)).

Parity: runtime/model.py:116-119, kernels/execution.cu:7-10.  gate_proj and up_proj
are stacked into one [2I, H] matrix at load so one product serves both.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..ops import kernels
from .base import FEED_FORWARDS, FeedForward, TensorNeed, register
from .linear import as_tensor, linear, linear_to_stream, norm_fusable


@register(FEED_FORWARDS, "swiglu")
class SwiGLU(FeedForward):
    """params: hidden_size, intermediate_size; names (local tensor names of gate, up, down)."""

    accepts_pending_norm = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        self.names = dict({"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}, **dict(spec.get("names") or {}))
        self.gate_up = None
        self.down = None

    def tensor_needs(self) -> Dict[str, TensorNeed]:
        return {self.names["gate"]: TensorNeed((self.inter, self.hidden)),
                self.names["up"]: TensorNeed((self.inter, self.hidden)),
                self.names["down"]: TensorNeed((self.hidden, self.inter))}

    def load(self, tensors):
        self.gate_up = torch.cat((tensors[self.names["gate"]], tensors[self.names["up"]]), dim=0).contiguous()
        self.down = tensors[self.names["down"]].contiguous()

    def kernel_jobs(self):
        return ([("elementwise.cu", {}, ())] + kernels.gemm_jobs(self.dtype)
                + (kernels.skinny_jobs() if self.dtype == torch.bfloat16 else []))

    def forward(self, h, ctx):
        h0 = h
        tokens = h.x.shape[0] if not isinstance(h, torch.Tensor) else h.shape[0]
        device = h.x.device if not isinstance(h, torch.Tensor) else h.device
        act = torch.empty((tokens, self.inter), dtype=self.dtype, device=device)
        if kernels.skinny_ok(tokens, self.gate_up):
            # few tokens: (norm,) gate and up products and the activation in one launch
            if norm_fusable(h, tokens, self.gate_up):
                x_out = h.new_stream_buffer()
                kernels.skinny_gemm(self.gate_up, tokens, x=h.x, delta=h.delta, norm_w=h.weight, eps=h.eps, x_out=x_out,
                                    epilogue=kernels.EPI_SWIGLU, out=act)
                h.done(x_out)
            else:
                kernels.skinny_gemm(self.gate_up, tokens, act=as_tensor(h), epilogue=kernels.EPI_SWIGLU, out=act)
        else:
            hn = as_tensor(h)
            if kernels.tcgen05_ok(hn, self.gate_up):
                kernels.gemm_tcgen05_swiglu(hn, self.gate_up, act)      # many tokens: SwiGLU is the product's epilogue
            else:
                kernels.swiglu(linear(hn, self.gate_up), act)
        return linear_to_stream(act, self.down, h0)


def pad_columns(w: torch.Tensor, multiple: int) -> torch.Tensor:
    """w [N, K] with zero columns appended until K is a multiple (the products take K in whole 16-byte groups)."""
    extra = -w.shape[1] % multiple
    return w.contiguous() if not extra else torch.nn.functional.pad(w, (0, extra)).contiguous()


@register(FEED_FORWARDS, "dense_mlp")
class DenseMLP(FeedForward):
    """down(act(up(h))) without a gate and without biases.  params: hidden_size, intermediate_size, activation
    ("relu_squared": max(z, 0)^2, "gelu_tanh", "silu"); names (up, down).  The activation is taken in float on the
    product's float sums and rounded once to the operand type of the second product."""

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        self.activation = spec.get("activation", "relu_squared")
        if self.activation not in kernels.ACTIVATIONS:
            raise ValueError(f"unknown activation {self.activation!r}")
        self.names = dict({"up": "up", "down": "down"}, **dict(spec.get("names", {})))
        self.up = None
        self.down = None
        self._groups = {}

    def tensor_needs(self) -> Dict[str, TensorNeed]:
        return {self.names["up"]: TensorNeed((self.inter, self.hidden)),
                self.names["down"]: TensorNeed((self.hidden, self.inter))}

    def load(self, tensors):
        self.up = tensors[self.names["up"]].contiguous()
        self.down = pad_columns(tensors[self.names["down"]], 8)

    def kernel_jobs(self):
        return ([("elementwise.cu", {}, ())] + kernels.gemm_jobs(self.dtype)
                + (kernels.skinny_jobs() if self.dtype == torch.bfloat16 else []))

    def _single_group(self, tiles: int, device) -> torch.Tensor:
        """Tile -> weight block list of the grouped tensor-core product, for one block: all zeros."""
        groups = self._groups.get(tiles)
        if groups is None:
            groups = self._groups[tiles] = torch.zeros(tiles, dtype=torch.int32, device=device)
        return groups

    def forward(self, h, ctx):
        h = as_tensor(h)
        tokens = h.shape[0]
        if (self.activation == "relu_squared" and self.down.shape[1] == self.inter and kernels.tcgen05_ok(h, self.up)):
            # many tokens: the squared relu is the epilogue of the first product (the grouped tcgen05 product with one
            # group, which takes whole 128-row tiles: the last tile is filled up with zero rows)
            rows = -(-tokens // kernels.MOE_TILE) * kernels.MOE_TILE
            if rows != tokens:
                padded = torch.zeros((rows, self.hidden), dtype=self.dtype, device=h.device)
                padded[:tokens].copy_(h)
                h = padded
            act = torch.empty((rows, self.inter), dtype=self.dtype, device=h.device)
            kernels.gemm_tcgen05_grouped(h, self.up.view(1, self.inter, self.hidden), act, self._single_group(rows // kernels.MOE_TILE, h.device),
                                         rows_in_use=tokens)
            return linear(act[:tokens], self.down)
        act = torch.empty((tokens, self.down.shape[1]), dtype=self.dtype, device=h.device)
        kernels.activation(linear(h, self.up), act, self.activation)
        return linear(act, self.down)


@register(FEED_FORWARDS, "polynorm_mlp")
class PolyNormMLP(FeedForward):
    """down(act(up(h))) without biases, act = a N(z) + b N(z^2) + c N(z^3) + e with powers taken element by element and
    N(u) = u / sqrt(mean(u^2) + eps) over a token's ff values; (a, b, c, e) is a tensor of the layer.  params: hidden_size,
    intermediate_size, eps; names (up, down, act).  The activation needs the whole row, so it is a row kernel between
    the two products (float on the first product's float sums, rounded once)."""

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        self.eps = float(spec["eps"])
        self.names = dict({"up": "up", "down": "down", "act": "act"}, **dict(spec.get("names", {})))
        self.up = self.down = self.coef = None

    def tensor_needs(self) -> Dict[str, TensorNeed]:
        return {self.names["up"]: TensorNeed((self.inter, self.hidden)),
                self.names["down"]: TensorNeed((self.hidden, self.inter)),
                self.names["act"]: TensorNeed((4,), role="vector", init_mean=0.4, init_std=0.2)}

    def load(self, tensors):
        self.up = tensors[self.names["up"]].contiguous()
        self.down = pad_columns(tensors[self.names["down"]], 8)
        self.coef = tensors[self.names["act"]].float().contiguous()

    def kernel_jobs(self):
        return (kernels.ffn_rows_jobs() + kernels.gemm_jobs(self.dtype)
                + (kernels.skinny_jobs() if self.dtype == torch.bfloat16 else []))

    def forward(self, h, ctx):
        h = as_tensor(h)
        act = torch.empty((h.shape[0], self.down.shape[1]), dtype=self.dtype, device=h.device)
        kernels.polynorm(linear(h, self.up), self.coef, self.eps, act)
        return linear(act, self.down)
