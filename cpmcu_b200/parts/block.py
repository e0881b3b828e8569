"""Arrangements of a layer's parts around the residual stream."""
from __future__ import annotations

from .base import BLOCKS, Block, ResidualStream


@BLOCKS.register("pre_norm_residual")
class PreNormResidualBlock(Block):
    """x += s * mixer(norm1(x)); x += s * feed_forward(norm2(x)), with one residual scale s.

    The reference scales each part's output by ``scale_depth / sqrt(layers)`` and adds
    it inside the next norm kernel (src/model/layer.cuh:47-67, src/model/norm.cuh:53-99).
    The scale is a parameter of the block; the block does not know where it comes from.
    """

    recordable_prompt = True

    def __init__(self, ops, mixer, feed_forward, mixer_norm, feed_forward_norm, names,
                 residual_scale: float = 1.0):
        super().__init__(ops, mixer, feed_forward, mixer_norm, feed_forward_norm, names)
        self.residual_scale = float(residual_scale)

    def forward(self, ctx, stream: ResidualStream, lane, writes_cache: bool) -> None:
        y = stream.normed(self.mixer_norm)
        a = self.mixer.forward(ctx, y, lane, writes_cache)
        stream.add(a, self.residual_scale)
        if self.feed_forward is None:
            return                                   # a layer of a mixer alone
        y2 = stream.normed(self.feed_forward_norm)
        f = self.feed_forward.forward(ctx, y2)
        stream.add(f, self.residual_scale)
