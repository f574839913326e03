"""Block arrangements.  ``pre_norm``: h += mixer(norm(h)); h += feed_forward(norm(h)),
the residual stream kept and summed in float32 (crates/runner/src/prefill_engine.rs:1116-1222)."""
from __future__ import annotations

from ..csrc.kernel_sets import NormedInput
from .registry import register_block


@register_block("pre_norm")
class PreNormBlock:
    """Interface of a block: ``forward(ctx, residual, cache_id, writes_cache)`` updates the
    float32 residual stream ``[T, hidden]`` in place."""

    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm, position):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm
        self.position = position

    @staticmethod
    def _give(x, part):
        """Parts that set ``takes_lazy_input`` get the norm unapplied (a NormedInput) so that
        their kernels may fold it in; all others get the normed activations."""
        return x if getattr(part, "takes_lazy_input", False) else x.tensor()

    def forward(self, ctx, residual, cache_id, writes_cache):
        x = NormedInput(ctx, residual, self.mixer_norm)
        ctx.stage = "mixer"           # names the running part for stage timings; nothing depends on it
        self.mixer.forward(ctx, self._give(x, self.mixer), residual, cache_id, writes_cache, self.position)
        x2 = NormedInput(ctx, residual, self.feed_forward_norm)
        ctx.stage = "feed_forward"
        self.feed_forward.forward(ctx, self._give(x2, self.feed_forward), residual)
