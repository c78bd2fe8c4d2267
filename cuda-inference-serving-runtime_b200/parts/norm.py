"""RMSNorm and layer norm, fused with the residual add that precedes them.

Parity: runtime/reference.py:5-6, kernels/ops.cu:3-19, kernels/execution.cu:12-24
(y = x * rsqrt(mean(x^2) + eps) * w; no bias, no 1+w offset).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..ops import kernels
from .base import NORMS, Norm, TensorNeed, register


@register(NORMS, "rms_norm")
class RMSNorm(Norm):
    """params: size (width), eps; weight_name (the tensor's name below the part's prefix, default "weight")."""

    fusable_into_product = True     # y = x * rsqrt(mean(x^2) + eps) * w is what the products' norm prologue computes
    kind = "rms"                    # what the kernels that take a norm as their last step call this form

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.weight_name = spec.get("weight_name", "weight")
        self.weight: Optional[torch.Tensor] = None

    def tensor_needs(self) -> Dict[str, TensorNeed]:
        return {self.weight_name: TensorNeed((self.size,), role="vector")}

    def load(self, tensors):
        self.weight = tensors[self.weight_name]

    def kernel_jobs(self):
        return [("elementwise.cu", {}, ())]

    def forward(self, x, delta, out_dtype, rows=None, write_back=True, delta_scale=None):
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.size), dtype=out_dtype, device=x.device)
        return kernels.add_rmsnorm(x, delta, self.weight, self.eps, out, rows=rows, write_back=write_back,
                                   delta_scale=delta_scale)


@register(NORMS, "rms_norm_scalar")
class ScalarRMSNorm(RMSNorm):
    """x / sqrt(mean(x^2) + eps) * g with ONE weight g for all channels (a tensor without dimensions).  params: size,
    eps; weight_name.  The weight is spread over the channels at load, so every kernel that takes RMSNorm (the norm
    kernel, the products' norm prologues, the kernels that end in a norm) takes this one as it is."""

    def tensor_needs(self) -> Dict[str, TensorNeed]:
        return {self.weight_name: TensorNeed((), role="vector")}

    def load(self, tensors):
        self.weight = tensors[self.weight_name].float().reshape(1).expand(self.size).contiguous()


@register(NORMS, "rms_norm_offset")
class OffsetRMSNorm(RMSNorm):
    """x / sqrt(mean(x^2) + eps) * (1 + w): the tensor holds the factor's offset from one.  params: size, eps; weight_name.  1 + w is
    formed once at load, in float (it has no exact bfloat16 form), so every kernel that takes RMSNorm takes this one as
    it is: their weights may be float whatever the storage type."""

    def load(self, tensors):
        self.weight = (1.0 + tensors[self.weight_name].float()).contiguous()


@register(NORMS, "layer_norm")
class LayerNorm(Norm):
    """(x - mean) / sqrt(var + eps) * w over the channels, var the mean squared deviation, no bias.
    params: size (width), eps; weight_name.  The statistics are float whatever the storage type."""

    kind = "layer"       # what the kernels that take a norm as their last step call this form

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.weight_name = spec.get("weight_name", "weight")
        self.weight: Optional[torch.Tensor] = None

    def tensor_needs(self) -> Dict[str, TensorNeed]:
        return {self.weight_name: TensorNeed((self.size,), role="vector")}

    def load(self, tensors):
        self.weight = tensors[self.weight_name]

    def kernel_jobs(self):
        return kernels.hyper_jobs()

    def forward(self, x, delta, out_dtype, rows=None, write_back=True, delta_scale=None):
        if delta_scale is not None:
            raise NotImplementedError("layer_norm: a per-channel scale of the pending output is not built")
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.size), dtype=out_dtype, device=x.device)
        # one stream: x += delta, then the norm (the general kernel with the identity as its mixing)
        one = x.view(x.shape[0], 1, self.size)
        return kernels.hyper_mix_norm(one, one, 1, y=delta, norm_w=self.weight, eps=self.eps, norm_kind=self.kind, h=out,
                                      rows=rows, store=write_back and delta is not None)
