"""How a mixer, a feed-forward and their norms are wired into one layer.

"pre_norm" carries (h, residual) and defers each residual add into the next norm: the first
block takes residual = h; afterwards every norm first does residual = h + residual in the model
dtype (turingserve/model/qwen2.py:42-57).
"""

from __future__ import annotations

import torch

from turingserve_b200 import kernels
from turingserve_b200.parts.base import BuildContext, build, register


class PreNormBlock:
    def __init__(self, spec, ctx: BuildContext) -> None:
        self.mixer_norm = build("norm", spec.mixer_norm, ctx)
        self.mixer = build("mixer", spec.mixer, ctx)
        self.ffn_norm = build("norm", spec.ffn_norm, ctx)
        self.feed_forward = build("feed_forward", spec.feed_forward, ctx)

    def parts(self) -> dict[str, object]:
        """Sub-parts by the role names used in ``LayerTensorNames``."""
        return {"mixer_norm": self.mixer_norm, "mixer": self.mixer,
                "ffn_norm": self.ffn_norm, "feed_forward": self.feed_forward}

    def forward(self, h, residual, step, cache, state, inject=None):
        """``inject``: a tensor added to the stream before this layer (a model that re-injects its input)."""
        if inject is not None:
            h = kernels.ops().materialize(h) + inject
        if residual is None:
            residual = h
            x = self.mixer_norm.forward(h)
        else:
            x = self.mixer_norm.forward(h, residual)
        a = self.mixer.forward(x, step, cache, state)
        x = self.ffn_norm.forward(a, residual)
        h = self.feed_forward.forward(x)
        return h, residual


def _build_block(spec, ctx: BuildContext):
    return PreNormBlock(spec, ctx)


class StreamBlock:
    """Pre-norm wiring over a residual stream in 32-bit: x += mixer(norm(x)); x += ff(norm(x)), where
    x is a float32 tensor whatever the engine's type and the branch outputs are in the engine's type.
    Each add is deferred into the norm that follows (``StreamRMSNorm``): the block carries
    (pending branch output, stream).  The feed-forward role may be missing (a layer that is only a mixer)."""

    def __init__(self, spec, ctx: BuildContext) -> None:
        self.mixer_norm = build("norm", spec.mixer_norm, ctx)
        self.mixer = build("mixer", spec.mixer, ctx)
        self.has_ff = "feed_forward" in spec.roles
        self.ffn_norm = build("norm", spec.ffn_norm, ctx) if self.has_ff else None
        self.feed_forward = build("feed_forward", spec.feed_forward, ctx) if self.has_ff else None

    def parts(self) -> dict[str, object]:
        p = {"mixer_norm": self.mixer_norm, "mixer": self.mixer}
        if self.has_ff:
            p.update(ffn_norm=self.ffn_norm, feed_forward=self.feed_forward)
        return p

    def forward(self, h, residual, step, cache, state, inject=None):
        first = residual is None
        if first:
            residual = torch.empty(h.shape, dtype=torch.float32, device=h.device)
        x = self.mixer_norm.forward(h, residual, extra=inject, first=first)
        h = self.mixer.forward(x, step, cache, state)
        if self.has_ff:
            x = self.ffn_norm.forward(h, residual)
            h = self.feed_forward.forward(x)
        return h, residual


register("block", "pre_norm", _build_block)
register("block", "pre_norm_stream", lambda spec, ctx: StreamBlock(spec, ctx))
