"""The pre-norm arrangement of a decoder layer.

x = norm_in(h + pending); a = mixer(x); x = norm_post(h + a); f = feed_forward(x); the layer returns
(h, f) and the next norm (the next layer's, or the final one) adds f, which is how the reference
fuses the second residual add with the following norm
(helios/crates/helios-hal/src/backends/hopper_sm90/session.rs:710,774,795-799).  Norm names:
``input`` and ``post_mixer``.
"""
from __future__ import annotations

from .base import Arrangement, register_arrangement


class PreNormBlock(Arrangement):
    def forward(self, h, delta, step, cache, own_cache):
        x = self.norms["input"].forward(h, delta)
        a = self.mixer.forward(x, step, cache, own_cache)
        x = self.norms["post_mixer"].forward(h, a)
        return h, self.feed_forward.forward(x, step)


register_arrangement("prenorm", PreNormBlock)


class OutputNormBlock(Arrangement):
    """The norm stands on each sublayer's output and the sublayers read the stream itself:
    h <- h + norm_mixer(mixer(h)); h <- h + norm_ff(feed_forward(h)), the second line only when the layer has a
    feed-forward.  Norm names: ``mixer_out`` and ``feed_forward_out``.  The stream stays float; in bfloat16 the
    sublayers read a rounded copy of it, which the kernel that adds a sublayer's normalised output writes beside
    the sum (``step.scratch`` hands it from layer to layer), so only a model's first layer makes one itself."""

    COPY = "stream_in_activation_type"

    def forward(self, h, delta, step, cache, own_cache):
        from .. import ops

        norm = self.norms["mixer_out"]
        if delta is not None:  # a block before this one left an addition pending
            if hasattr(delta, "apply"):
                delta.apply(h)
            else:
                h += (delta.tensor() if hasattr(delta, "tensor") else delta).to(h.dtype)
            step.scratch.pop(self.COPY, None)
        if norm.dtype == h.dtype:
            x = h
        else:
            x = step.scratch.get(self.COPY)
            if x is None:
                x = ops.stream_copy(h)
        x = norm.add_normed(h, self.mixer.forward(x, step, cache, own_cache))
        if self.feed_forward is not None:
            x = self.norms["feed_forward_out"].add_normed(h, self.feed_forward.forward(x, step))
        step.scratch[self.COPY] = x
        return h, None


register_arrangement("output_norm", OutputNormBlock)


class SandwichNormBlock(Arrangement):
    """Every sublayer is normalised on both sides: h <- h + norm_b(mixer(norm_a(h))); h <- h + norm_d(feed_forward(norm_c(h))),
    the second line only when the layer has a feed-forward.  Norm names: ``input``, ``mixer_out``, ``post_mixer``,
    ``feed_forward_out``.  What a sublayer returns travels on as a :class:`NormedDelta`; the next norm that reads the stream
    (this layer's, the next layer's or the model's last) normalises it, adds it and normalises the sum in one launch."""

    def forward(self, h, delta, step, cache, own_cache):
        from .norm import NormedDelta

        x = self.norms["input"].forward(h, delta)
        pending = NormedDelta(self.mixer.forward(x, step, cache, own_cache), self.norms["mixer_out"])
        if self.feed_forward is not None:
            x = self.norms["post_mixer"].forward(h, pending)
            pending = NormedDelta(self.feed_forward.forward(x, step), self.norms["feed_forward_out"])
        return h, pending


register_arrangement("sandwich_norm", SandwichNormBlock)


class SideBySideBlock(Arrangement):
    """Mixer and feed-forward read the same normalised rows and their results are added to the stream together:
    x = norm(h);  h <- h + (mixer(x) + feed_forward(x)).  One norm per layer (name ``input``).  What the two return travels
    on as a :class:`SumOfTwo`; the next norm that reads the stream adds it in its own launch.  A layer without a
    feed-forward adds the mixer's result alone."""

    def forward(self, h, delta, step, cache, own_cache):
        from .norm import SumOfTwo

        x = self.norms["input"].forward(h, delta)
        mixed = self.mixer.forward(x, step, cache, own_cache)
        fed = self.feed_forward.forward(x, step) if self.feed_forward is not None else None
        return h, SumOfTwo(mixed, fed)


register_arrangement("side_by_side", SideBySideBlock)
