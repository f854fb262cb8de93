"""Arrangements of a layer's parts around the residual stream.

``prenorm``: ``x += mixer(norm1(x)); x += feed_forward(norm2(x))`` — the reference's decoder layer
(csrc/model/causal_lm.cpp:138-188).  Each sub-layer's output stays pending until the next norm, which
adds it to the 32-bit residual and normalises in one pass (the reference fuses only the first add,
csrc/ops/residual_rms_norm_fused.cu:58-109); the last pending delta of the last layer is folded by
the model's final norm.  Spec: ``PartSpec("prenorm", norm_names=(first, second), after=None)``.  A layer whose
feed-forward is of kind ``none`` has the mixer's sub-layer only.  ``after``: the spec of a part from the ``TAILS``
registry that runs on the stream once both sub-layers are done (a per-layer input from the token's id, say), with
``index`` set to the layer's place among the model's layers.
"""
from __future__ import annotations

from typing import Callable, List

from .base import Block, FeedForward, LazyNorm, Mixer, Norm, Part, ResidualStream
from .context import StepContext
from .registry import BLOCKS, TAILS
from .spec import PartSpec


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    def __init__(self, spec: PartSpec, *, mixer: Mixer, feed_forward: FeedForward,
                 make_norm: Callable[[str], Norm], prefix: str) -> None:
        super().__init__(spec, mixer=mixer, feed_forward=feed_forward, make_norm=make_norm, prefix=prefix)
        first, second = spec.get("norm_names", ("input_layernorm", "post_attention_layernorm"))
        self.mixer_norm = make_norm(f"{prefix}.{first}")
        self.has_feed_forward = not getattr(feed_forward, "absent", False)
        self.feed_forward_norm = make_norm(f"{prefix}.{second}") if self.has_feed_forward else None
        after = spec.get("after")
        self.tail = None
        if after is not None:
            self.tail = TAILS.get(after.kind)(after, hidden_size=mixer.hidden_size, prefix=f"{prefix}.{after.get('name', 'side')}",
                                              dtype=mixer.dtype)

    def parts(self) -> List[Part]:
        out: List[Part] = [self.mixer_norm, self.mixer]
        if self.has_feed_forward:
            out += [self.feed_forward_norm, self.feed_forward]
        if self.tail is not None:
            out += self.tail.parts()
        return out

    def forward(self, stream: ResidualStream, ctx: StepContext, run: int) -> None:
        h = self._normed(stream, self.mixer_norm, self.mixer)
        stream.pending = self.mixer.forward(h, ctx, run)
        if self.has_feed_forward:
            h = self._normed(stream, self.feed_forward_norm, self.feed_forward)
            stream.pending = self.feed_forward.forward(h, ctx)
        if self.tail is not None:
            self.tail.forward(stream, ctx)

    @staticmethod
    def _normed(stream: ResidualStream, norm: Norm, consumer: Part):
        """The normed rows for ``consumer``: computed now, or handed over uncomputed when the consumer can
        fold the norm into its first projection."""
        if getattr(consumer, "accepts_lazy_norm", False):
            return LazyNorm(stream, norm)
        return norm.add_norm(stream)


@BLOCKS.register("sandwich")
class SandwichBlock(Block):
    """``x += post1(mixer(pre1(x))); x += post2(feed_forward(pre2(x)))``: every sub-layer has a norm on its input and
    another on its output.  Spec: ``PartSpec("sandwich", norm_names=(pre1, post1, pre2, post2))``.  A layer whose
    feed-forward is of kind ``none`` has the first two norms only.

    A sub-layer's output stays pending together with its output norm (``stream.pending_norm``); the next input norm —
    this layer's or the next layer's — applies that norm, adds, stores the residual and norms again in one kernel."""

    def __init__(self, spec: PartSpec, *, mixer: Mixer, feed_forward: FeedForward,
                 make_norm: Callable[[str], Norm], prefix: str) -> None:
        super().__init__(spec, mixer=mixer, feed_forward=feed_forward, make_norm=make_norm, prefix=prefix)
        pre1, post1, pre2, post2 = spec.get("norm_names", ("norm1", "norm1b", "norm2", "norm2b"))
        self.mixer_norm = make_norm(f"{prefix}.{pre1}")
        self.mixer_out_norm = make_norm(f"{prefix}.{post1}")
        self.has_feed_forward = not getattr(feed_forward, "absent", False)
        self.feed_forward_norm = make_norm(f"{prefix}.{pre2}") if self.has_feed_forward else None
        self.feed_forward_out_norm = make_norm(f"{prefix}.{post2}") if self.has_feed_forward else None

    def parts(self) -> List[Part]:
        out: List[Part] = [self.mixer_norm, self.mixer, self.mixer_out_norm]
        if self.has_feed_forward:
            out += [self.feed_forward_norm, self.feed_forward, self.feed_forward_out_norm]
        return out

    def forward(self, stream: ResidualStream, ctx: StepContext, run: int) -> None:
        h = self.mixer_norm.add_norm(stream)
        stream.pending = self.mixer.forward(h, ctx, run)
        stream.pending_norm = self.mixer_out_norm
        if self.has_feed_forward:
            h = self.feed_forward_norm.add_norm(stream)
            stream.pending = self.feed_forward.forward(h, ctx)
            stream.pending_norm = self.feed_forward_out_norm
