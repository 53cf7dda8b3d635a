"""Block arrangements: how norms, mixer and feed-forward sit around the residual stream."""

from __future__ import annotations

from typing import Optional

import torch

from yalis_b200.ops.linear import linear, linear_partial
from .base import Block, NormedSum, Projected, ResidualStream, register_part, stack_rows


class PreNormResidualBlock(Block):
    """x += mixer(norm_1(x)); x += feed_forward(norm_2(x))
    (the non-parallel branch of yalis/external/model.py:414-438).
    Each addition is parked in the stream and performed by the next norm.  A layer may leave out the position part
    (a mixer that sees to positions itself) and the feed-forward with its norm.

    With ``norm_1_post`` / ``norm_2_post`` a sub-layer's result is normed before it is added:
    x += norm_1_post(mixer(norm_1(x))); x += norm_2_post(feed_forward(norm_2(x))).  A norm of the plain
    root-mean-square kind rides along with the result (``NormedSum``) and is applied, in float32, by the pass
    that adds it; any other kind norms the result on its own first."""

    slots = {"position": "position", "norm_1": "norm", "mixer": "mixer", "norm_1_post": "norm", "norm_2": "norm",
             "feed_forward": "feed_forward", "norm_2_post": "norm"}
    optional = ("position", "norm_2", "feed_forward", "norm_1_post", "norm_2_post")

    def __init__(self, spec, parts):
        super().__init__(spec, parts)
        if ("norm_2" in self.parts) != ("feed_forward" in self.parts):
            raise ValueError("a pre-norm block has a feed-forward and its norm, or neither")
        if "norm_2_post" in self.parts and "feed_forward" not in self.parts:
            raise ValueError("a norm behind the feed-forward needs a feed-forward")

    @staticmethod
    def _normed(result, norm):
        """A sub-layer's result with the norm that follows it."""
        if norm is None:
            return result
        if not isinstance(result, NormedSum):
            result = NormedSum(result)
        if result.norm is not None:
            raise ValueError("the result already carries a norm")
        params = norm.rms_parameters()
        if params is not None:
            return NormedSum(result.y, result.bias, params)
        y = result.y if result.y.dim() == 2 else result.y.sum(dim=0)
        if result.bias is not None:
            y = y.float() + result.bias
        return norm.normalize(y.to(result.y.dtype if result.y.dim() == 2 else torch.float32).contiguous())

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        h = self.norm_1.forward(stream)
        stream.add(self._normed(self.mixer.forward(h, ctx, cache), self.parts.get("norm_1_post")))
        if "feed_forward" in self.parts:
            h = self.norm_2.forward(stream)
            stream.add(self._normed(self.feed_forward.forward(h, ctx), self.parts.get("norm_2_post")))


class ParallelResidualBlock(Block):
    """h = norm_1(x);  x += mixer(h) + feed_forward(h): one norm, both sub-layers read its output (the parallel
    branch of yalis/external/model.py:414-438).  A layer may have no feed-forward.

    When mixer and feed-forward are both of the form W_out core(W_in h) (``Projected``), their input matrices are
    stacked and their output matrices laid side by side when the weights are loaded, so a layer runs two products:
    z = h [W_in_mixer; W_in_ff]^T, and after the cores have written their results next to each other,
    [y_mixer, y_ff] [W_out_mixer, W_out_ff]^T, which is the sum of both sub-layers."""

    slots = {"norm_1": "norm", "mixer": "mixer", "feed_forward": "feed_forward"}
    optional = ("feed_forward",)

    def __init__(self, spec, parts):
        super().__init__(spec, parts)
        self.ff = self.parts.get("feed_forward")
        self.w_in: Optional[torch.Tensor] = None
        self.w_out: Optional[torch.Tensor] = None
        self.spans = []

    def _fuse(self) -> bool:
        """Stack the matrices of mixer and feed-forward once (the parts have their weights by the first step)."""
        if self.w_in is not None:
            return True
        shared = [p for p in (self.mixer, self.ff) if p is not None]
        if len(shared) < 2 or not all(isinstance(p, Projected) for p in shared):
            return False
        if any(p.in_weight().dtype != shared[0].in_weight().dtype or p.out_weight().dtype != shared[0].out_weight().dtype
               for p in shared):
            return False
        self.w_in, self.spans = stack_rows([p.in_weight() for p in shared])
        self.w_out = torch.cat([p.out_weight() for p in shared], dim=1).contiguous()
        for p in shared:
            p.release_projections()
        return True

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        h = self.norm_1.forward(stream)
        if self._fuse():
            z = linear(h, self.w_in)
            km = self.mixer.hidden_width
            y = torch.empty((h.shape[0], km + self.ff.hidden_width), dtype=h.dtype, device=h.device)
            (a, b), (c, d) = self.spans
            self.mixer.mix(z[:, a:b], ctx, cache, y[:, :km])
            self.ff.mix(z[:, c:d], ctx, None, y[:, km:])
            stream.add(linear_partial(y, self.w_out))
            return
        stream.add(self.mixer.forward(h, ctx, cache))
        if self.ff is not None:
            stream.add(self.ff.forward(h, ctx))


register_part("block", "pre_norm_residual", PreNormResidualBlock)
register_part("block", "parallel_residual", ParallelResidualBlock)
