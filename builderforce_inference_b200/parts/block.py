"""Pre-norm residual block: ``x += mixer(norm1(x)); x += ffn(norm2(x))``
(crates/bfi-models/src/qwen3.rs:217-250).  The residual stream stays float32 in every run
dtype; the two adds happen inside the mixer's and the feed-forward's last matrix product."""
from __future__ import annotations

from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, PartSpec


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    graph_safe = True

    def __init__(self, norm1: PartSpec, mixer: PartSpec, norm2: PartSpec, ffn: PartSpec):
        self.norm1 = NORMS.build(norm1)
        self._mixer = MIXERS.build(mixer)
        self.norm2 = NORMS.build(norm2)
        self.ffn = FEED_FORWARDS.build(ffn)

    def children(self):
        return {"norm1": self.norm1, "mixer": self._mixer, "norm2": self.norm2, "ffn": self.ffn}

    def mixer(self):
        return self._mixer

    def forward(self, ctx, residual, run) -> None:
        h = self.norm1.forward(ctx, residual)
        self._mixer.forward(ctx, h, residual, run)
        h = self.norm2.forward(ctx, residual)
        self.ffn.forward(ctx, h, residual)
