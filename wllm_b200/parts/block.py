"""Arrangements of norms, mixer and feed-forward around the residual stream.

'pre_norm' (Gemma 1, src/wllm/models/gemma.py:83-93):
    x = x + mixer(norm_in(x));  x = x + feed_forward(norm_post(x))
A branch's output is left pending on the residual and folded in by the next norm
(the next block's, or the model's final one).

spec options: norm_in, mixer, norm_post, feed_forward (specs).
"""
from __future__ import annotations

from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, CacheRef, Residual


@BLOCKS.register("pre_norm")
class PreNormBlock:
    graph_safe = True
    def __init__(self, spec, hidden_size: int, model_dtype):
        kw = dict(hidden_size=hidden_size, model_dtype=model_dtype)
        self.norm_in = NORMS.build(spec.norm_in, **kw)
        self.mixer = MIXERS.build(spec.mixer, **kw)
        self.norm_post = NORMS.build(spec.norm_post, **kw)
        self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, **kw)

    def parts(self):
        return [self.norm_in, self.mixer, self.norm_post, self.feed_forward]

    def cache_need(self):
        return self.mixer.cache_need()

    def __call__(self, residual: Residual, ctx, cache: CacheRef) -> None:
        residual.pending = self.mixer(self.norm_in(residual, ctx), ctx, cache)
        residual.pending = self.feed_forward(self.norm_post(residual, ctx), ctx)
