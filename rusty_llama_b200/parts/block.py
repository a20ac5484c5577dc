"""Arrangements of a layer's parts."""

from __future__ import annotations

from .base import BLOCKS, Block, ResidualStream


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    """x += mixer(norm_m(x)); x += feed_forward(norm_f(x)) (src/model.rs:1244-1357).

    Each sum is left pending on the stream and performed by the next norm's
    kernel, the following layer's or the model's final one."""

    def forward(self, stream: ResidualStream, step, cache, shared_cache: bool = False) -> None:
        xn = self.norms["mixer"].forward(stream)
        stream.add(self.mixer.forward(xn, step, cache, shared_cache))
        xn = self.norms["feed_forward"].forward(stream)
        stream.add(self.feed_forward.forward(xn, step))
