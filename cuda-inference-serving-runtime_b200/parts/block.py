"""How a layer's parts are arranged around the residual stream.

"pre_norm" (runtime/model.py:109-119): x += mixer(norm1(x)); x += feed_forward(norm2(x)).
The add of one sub-block's output is fused into the next norm, so a layer leaves
its feed-forward output pending in the stream instead of adding it itself.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..config.spec import LayerSpec
from .base import ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, STREAMS, Part, PendingNorm, TensorNeed, build_part, register


@register(STREAMS, "single")
class ResidualStream:
    """The float residual stream x [tokens, hidden] and an output not added to it yet."""

    def __init__(self, x: torch.Tensor, spec=None):
        self.x = x
        self.pending: Optional[torch.Tensor] = None
        self.pending_scale: Optional[torch.Tensor] = None    # per-channel factor the pending output is added with

    def take_pending(self) -> Optional[torch.Tensor]:
        """The pending output; whoever takes it adds it (times `pending_scale`, read before this call) to x."""
        pending, self.pending = self.pending, None
        self.pending_scale = None
        return pending

    def finish(self, norm, dtype: torch.dtype, rows: torch.Tensor) -> torch.Tensor:
        """The model's last step: norm(x + pending) at the wanted rows."""
        scale = self.pending_scale
        extra = {} if scale is None else {"delta_scale": scale}
        return norm.forward(self.x, self.take_pending(), dtype, rows=rows, write_back=False, **extra)

    def total(self) -> torch.Tensor:
        """x with the pending output added, as a new tensor; the stream object stays as it was."""
        x = self.x.clone()
        if self.pending is not None:
            from ..ops import kernels
            kernels.stream_add(x, self.pending, self.pending_scale, None)
        return x


@register(ARRANGEMENTS, "pre_norm")
class PreNormBlock:
    slots = ("mixer_norm", "mixer", "feed_forward_norm", "feed_forward")

    def __init__(self, spec: LayerSpec, dtype: torch.dtype):
        self.spec = spec
        self.dtype = dtype
        self.mixer_norm = build_part(NORMS, spec.mixer_norm, dtype, "norm")
        self.mixer = build_part(MIXERS, spec.mixer, dtype, "mixer")
        self.feed_forward_norm = build_part(NORMS, spec.feed_forward_norm, dtype, "norm")
        self.feed_forward = build_part(FEED_FORWARDS, spec.feed_forward, dtype, "feed-forward")

    def parts(self):
        return {slot: getattr(self, slot) for slot in self.slots}

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        h = PendingNorm(stream, self.mixer_norm, self.dtype)
        mixed = self.mixer.forward(h if self.mixer.accepts_pending_norm else h.materialize(), ctx, cache)
        stream.pending = mixed
        h = PendingNorm(stream, self.feed_forward_norm, self.dtype)
        stream.pending = self.feed_forward.forward(h if self.feed_forward.accepts_pending_norm else h.materialize(), ctx)


class ChannelScale(Part):
    """One factor per channel (a layer scale).  params: size; weight_name; value (optional: one constant for all channels,
    a multiplier of the residual branch that the configuration gives; the part then has no tensor)."""

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.size = int(spec["size"])
        self.weight_name = spec.get("weight_name", "")
        self.value = spec.get("value")
        self.weight = None

    def tensor_needs(self):
        return {} if self.value is not None else {self.weight_name: TensorNeed((self.size,), role="vector")}

    def load(self, tensors):
        if self.value is not None:
            from ..engine.model import require_cuda
            self.weight = torch.full((self.size,), float(self.value), dtype=torch.float32, device=require_cuda())
            return
        self.weight = tensors[self.weight_name].float().contiguous()    # applied to a float output on its way into the float stream


@register(ARRANGEMENTS, "pre_norm_scaled")
class PreNormScaledBlock:
    """x += s1 * mixer(norm1(x)); x += s2 * feed_forward(norm2(x)), with s1, s2 one factor per channel; the feed-forward
    half may be absent.  The scaled add of each output is made by the norm kernel that follows it; a feed-forward that
    says `applies_output_scale` multiplies by s2 in its own last kernel instead, and its output is then pending like any
    other (so the next layer's first product may take the add and the norm into its prologue).  Where a scale is one
    constant for all channels (`ChannelScale` with a `value`), the sub-block is told the constant and may add its
    output, multiplied, to the stream in the epilogue of its last product (`parts/linear.py: linear_to_stream`)."""

    def __init__(self, spec: LayerSpec, dtype: torch.dtype):
        self.spec = spec
        self.dtype = dtype
        self.mixer_norm = build_part(NORMS, spec.mixer_norm, dtype, "norm")
        self.mixer = build_part(MIXERS, spec.mixer, dtype, "mixer")
        self.mixer_scale = ChannelScale(spec.extras["mixer_scale"], dtype)
        self.feed_forward = self.feed_forward_norm = self.feed_forward_scale = None
        if spec.feed_forward is not None:
            self.feed_forward_norm = build_part(NORMS, spec.feed_forward_norm, dtype, "norm")
            self.feed_forward = build_part(FEED_FORWARDS, spec.feed_forward, dtype, "feed-forward")
            self.feed_forward_scale = ChannelScale(spec.extras["feed_forward_scale"], dtype)

    def parts(self):
        slots = ("mixer_norm", "mixer", "mixer_scale", "feed_forward_norm", "feed_forward", "feed_forward_scale")
        return {slot: getattr(self, slot) for slot in slots if getattr(self, slot) is not None}

    @staticmethod
    def _run(part, h, scale, *args):
        """A factor per channel is applied on the output's way into the stream, so no part adds it there itself; one
        constant for all channels (`scale.value`) can be the factor of a product's in-place add, and the part is told so."""
        if scale.value is None:
            h.in_place_ok = False
        else:
            h.out_mult = float(scale.value)
        return part.forward(h if part.accepts_pending_norm else h.materialize(), *args)

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        mixed = self._run(self.mixer, PendingNorm(stream, self.mixer_norm, self.dtype), self.mixer_scale, ctx, cache)
        if mixed is not None:          # None: the mixer added its output, multiplied, to the stream itself
            stream.pending, stream.pending_scale = mixed, self.mixer_scale.weight
        if self.feed_forward is not None:
            h = PendingNorm(stream, self.feed_forward_norm, self.dtype)
            if getattr(self.feed_forward, "applies_output_scale", False):
                stream.pending = self._run(self.feed_forward, h, self.feed_forward_scale, ctx, self.feed_forward_scale.weight)
            else:
                out = self._run(self.feed_forward, h, self.feed_forward_scale, ctx)
                if out is not None:
                    stream.pending, stream.pending_scale = out, self.feed_forward_scale.weight
