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
