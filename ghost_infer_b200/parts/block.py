"""Arrangements of a layer's parts around the residual stream."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Block
from .registry import register


@register("block", "prenorm_residual")
class PreNormResidual(Block):
    """x += mixer(norm(x)); x += ffn(norm(x)), the residual stream x kept in 32-bit
    (src/model.rs:996-1147; the reference's stream is f32 too, src/model.rs:704-705)."""

    def forward(self, x, step, memory) -> None:
        # The last product of the mixer and of the feed-forward adds into x; in a decode step it may leave
        # partial sums pending for the norm that reads x next (a norm that cannot add them has them settled first).
        if x.is_cuda and not getattr(self.mixer_norm, "settles_pending", False):
            ops.settle(x)
        h = self.mixer_norm.forward(x)
        with ops.defer_into(x):
            self.mixer.forward(h, x, step, memory)
        if self.ffn is None:          # a layer without a feed-forward: the mixer alone
            return
        if x.is_cuda and not getattr(self.ffn_norm, "settles_pending", False):
            ops.settle(x)
        h = self.ffn_norm.forward(x)
        with ops.defer_into(x):
            self.ffn.forward(h, x, step)


@register("block", "residual_postnorm")
class ResidualPostNorm(Block):
    """x += s1 * norm(mixer(x)); x += s2 * norm(ffn(x)): the sublayers read the stream itself (in the activation type)
    and the norm sits on what they give back; s1 and s2 are learned per-channel scales (`extra["mixer_scale"]`,
    `extra["ffn_scale"]`, each optional).  Then every `extra` part named "after..." runs in order as a feed-forward
    on the stream (it adds to it by itself).  Norms, scales and sums are 32-bit."""

    def forward(self, x, step, memory) -> None:
        if x.is_cuda:
            ops.settle(x)             # nothing here defers into the stream; what a layer before left is added first
        dt = self.mixer_norm.rt.dtype
        low = dt != torch.float32     # the 32-bit path reads the stream itself
        subs = [(self.mixer_norm, self.extra.get("mixer_scale"), lambda h, y: self.mixer.forward(h, y, step, memory))]
        if self.ffn is not None:
            subs.append((self.ffn_norm, self.extra.get("ffn_scale"), lambda h, y: self.ffn.forward(h, y, step)))
        after = [part for name, part in self.extra.items() if name.startswith("after")]
        # one matrix of 32-bit rows that every sublayer adds into, and one copy of the stream in the activation type: the
        # pass that joins a sublayer's output to the stream zeroes the first and renews the second for the next reader
        y = torch.empty(x.shape, dtype=torch.float32, device=x.device)
        h = ops.cast_rows(x, dt, zero=y)
        for i, (norm, scale, run) in enumerate(subs):
            run(h, y)
            more, reader = i + 1 < len(subs), i + 1 < len(subs) or bool(after)
            norm.add_normed(x, y, scale.weight if scale is not None else None, cast_out=h if (low and reader) else None, zero_y=more)
        for i, part in enumerate(after):
            part.forward(h, x, step)
            if low and i + 1 < len(after):
                h = ops.cast_rows(x, dt)
