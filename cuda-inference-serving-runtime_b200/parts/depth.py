"""Depth-weighted average of the residual stream: what a layer hands to the next one is a weighted sum of the embedding
and of every layer's result so far.

    X_0 = the embedding;   layer i: y = x + mixer(norm1(x)); y = y + feed_forward(norm2(y));   X_(i+1) = y
    x <- sum_(j <= i + 1) w_i[j] * X_j          (w_i: i + 2 numbers of layer i; the last x is what the model's norm reads)

The results of a step's tokens are kept for the step only (`DepthStream.hist`, float [entries + 1, tokens, hidden]); a
layer's end, the weighted sum and the next layer's first norm are one kernel (`kernels.depth_mix_norm`): the layer's last
output stays pending in the stream object, with the layer's weights, until the next layer (or the final norm) asks for
its input.  Inside a layer the stream behaves like the plain residual stream, so the norm kernels, the products' norm
prologues and the in-place adds of the products' epilogues serve it as they serve `pre_norm`.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.spec import LayerSpec
from ..ops import kernels
from .base import ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, STREAMS, Part, PendingNorm, TensorNeed, build_part, register


class DepthWeights(Part):
    """The weights of one layer's average: `count` numbers, the last one the layer's own result's.  params: count;
    weight_name."""

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.count = int(spec["count"])
        self.weight_name = spec.get("weight_name", "")
        self.weight = None

    def tensor_needs(self) -> Dict[str, TensorNeed]:
        # seeded random weights: a sum that stays near the latest result
        return {self.weight_name: TensorNeed((self.count,), role="vector", init_mean=1.0 / self.count, init_std=0.3 / self.count)}

    def load(self, tensors):
        self.weight = tensors[self.weight_name].float().contiguous()      # applied to float results


@register(STREAMS, "depth_average")
class DepthStream:
    """x [tokens, hidden] (float) as a layer sees it, an output not added to it yet, the results so far, and the weights
    of an average that has not been formed yet.  params of the spec: entries (how many layers run)."""

    def __init__(self, embedded: torch.Tensor, spec):
        entries = int(spec["entries"])
        tokens, hidden = embedded.shape
        self.hist = torch.empty((entries + 1, tokens, hidden), dtype=torch.float32, device=embedded.device)
        self.hist[0].copy_(embedded)           # X_0; `embedded` itself becomes the first layer's stream and is written to
        self.x = embedded
        self.filled = 1                        # results held so far
        self.pending: Optional[torch.Tensor] = None
        self.pending_scale = None              # the plain stream's interface (`PendingNorm`): never set here
        self.average: Optional[torch.Tensor] = None

    def take_pending(self) -> Optional[torch.Tensor]:
        pending, self.pending = self.pending, None
        return pending

    def close_layer(self, weights: torch.Tensor) -> None:
        """The layer is over: its result is x + pending, and what follows reads the average with these weights."""
        if self.average is not None:
            raise RuntimeError("a layer closed while the average before it was still waiting")
        if weights.numel() != self.filled + 1:
            raise ValueError(f"the average after {self.filled} layers needs {self.filled + 1} weights, not {weights.numel()}")
        self.average = weights

    def open_layer(self, norm, dtype: torch.dtype):
        """The normed input of the next layer's first sub-block: a `PendingNorm` where no average waits (the first layer),
        else the tensor the seam kernel made."""
        if self.average is None:
            return PendingNorm(self, norm, dtype)
        h = torch.empty(self.x.shape, dtype=dtype, device=self.x.device)
        kernels.depth_mix_norm(self.hist, self.x, self.take_pending(), self.average, self.filled, norm_w=norm.weight, eps=norm.eps, h=h)
        self.filled += 1
        self.average = None
        return h

    def finish(self, norm, dtype: torch.dtype, rows: torch.Tensor) -> torch.Tensor:
        """The model's last step: the norm of the last average at the wanted rows."""
        if self.average is None:
            return norm.forward(self.x, self.take_pending(), dtype, rows=rows, write_back=False)
        h = torch.empty((rows.numel(), self.x.shape[1]), dtype=dtype, device=self.x.device)
        return kernels.depth_mix_norm(self.hist, self.x, self.pending, self.average, self.filled, norm_w=norm.weight, eps=norm.eps,
                                      h=h, rows=rows)

    def total(self) -> torch.Tensor:
        """What the next layer would read, as a new tensor; the stream object stays as it was."""
        if self.average is None:
            x = self.x.clone()
            if self.pending is not None:
                kernels.stream_add(x, self.pending)
            return x
        out = torch.empty_like(self.x)
        kernels.depth_mix_norm(self.hist, self.x, self.pending, self.average, self.filled, mixed_out=out, store=False)
        return out


@register(ARRANGEMENTS, "pre_norm_depth")
class PreNormDepthBlock:
    """x += mixer(norm1(x)); x += feed_forward(norm2(x)) (the feed-forward half may be absent), then the depth-weighted
    average with the layer's weights (`extras["depth"]`), formed by the next reader of the stream."""

    def __init__(self, spec: LayerSpec, dtype: torch.dtype):
        self.spec = spec
        self.dtype = dtype
        self.mixer_norm = build_part(NORMS, spec.mixer_norm, dtype, "norm")
        self.mixer = build_part(MIXERS, spec.mixer, dtype, "mixer")
        self.depth = DepthWeights(spec.extras["depth"], dtype)
        self.feed_forward = self.feed_forward_norm = None
        if spec.feed_forward is not None:
            self.feed_forward_norm = build_part(NORMS, spec.feed_forward_norm, dtype, "norm")
            self.feed_forward = build_part(FEED_FORWARDS, spec.feed_forward, dtype, "feed-forward")
        if not getattr(self.mixer_norm, "fusable_into_product", False):
            raise ValueError("the depth-average arrangement takes norms of RMSNorm's form (its seam kernel ends in one)")

    def parts(self):
        slots = ("mixer_norm", "mixer", "feed_forward_norm", "feed_forward", "depth")
        return {slot: getattr(self, slot) for slot in slots if getattr(self, slot) is not None}

    def kernel_jobs(self):
        return kernels.depth_jobs()

    @staticmethod
    def _input(part, h):
        if isinstance(h, PendingNorm) and not part.accepts_pending_norm:
            return h.materialize()
        return h

    def forward(self, stream: DepthStream, ctx, cache) -> None:
        h = stream.open_layer(self.mixer_norm, self.dtype)
        stream.pending = self.mixer.forward(self._input(self.mixer, h), ctx, cache)
        if self.feed_forward is not None:
            h = PendingNorm(stream, self.feed_forward_norm, self.dtype)
            stream.pending = self.feed_forward.forward(self._input(self.feed_forward, h), ctx)
        stream.close_layer(self.depth.weight)
