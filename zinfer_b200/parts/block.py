"""The pre-norm arrangement: h1 = h + mixer(norm(h)); h2 = h1 + ffn(norm(h1))
(src/model/layers/rmsnorm_gqa_swiglu_block.zig:86-88,161-163).

The residual stream ``h`` is 32-bit.  An update that has not yet been added is
carried as ``pending`` into the next norm, where the add is fused with the norm;
the block therefore returns its feed-forward's output instead of adding it.

Options: ``residual_scale`` m multiplies both updates (h + m * mixer(..), h1 + m * ffn(..));
``feed_forward`` None leaves the second half out; ``verbatim_names`` takes the four name
parameters as complete prefixes (``norm1`` for a tensor called just that) instead of
appending a dot."""
from __future__ import annotations

from .. import ops
from .base import Block, make_part, prefixed, take


class PreNormBlock(Block):
    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.mixer = make_part(params["mixer"], ctx)
        self.mixer_norm = make_part(params["mixer_norm"], ctx)
        has_ffn = params.get("feed_forward") is not None
        self.feed_forward = make_part(params["feed_forward"], ctx) if has_ffn else None
        self.ffn_norm = make_part(params["ffn_norm"], ctx) if has_ffn else None
        self.residual_scale = float(params.get("residual_scale", 1.0))
        dot = "" if params.get("verbatim_names") else "."
        self._names = {
            "mixer": params.get("mixer_name", "mixer") + dot,
            "feed_forward": params.get("ffn_name", "feed_forward") + dot,
            "mixer_norm": params.get("mixer_norm_name", "mixer_norm") + dot,
            "ffn_norm": params.get("ffn_norm_name", "ffn_norm") + dot,
        }

    def _parts(self):
        return [(self._names[k], getattr(self, k)) for k in ("mixer_norm", "mixer", "ffn_norm", "feed_forward")
                if getattr(self, k) is not None]

    def tensor_specs(self):
        out = {}
        for prefix, part in self._parts():
            out.update(prefixed(prefix, part.tensor_specs()))
        return out

    def bind(self, tensors):
        for prefix, part in self._parts():
            part.bind(take(tensors, prefix))

    def _update(self, delta):
        return delta if self.residual_scale == 1.0 else ops.Scaled(delta, self.residual_scale)

    def forward(self, h, pending, step, cache, bias=None):
        x = self.mixer_norm.forward(h, pending) if bias is None else self.mixer_norm.forward(h, pending, bias=bias)
        a = self._update(self.mixer.forward(x, step, cache))
        if self.feed_forward is None:
            return a
        x = self.ffn_norm.forward(h, a)
        return self._update(self.feed_forward.forward(x))
