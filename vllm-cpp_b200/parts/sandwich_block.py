"""An arrangement with a norm on both sides of every sublayer and a learned scale per channel on what is added:

    x += l1 * n1b(mixer(n1(x)))              n(v) = w * v / sqrt(mean(v^2) + eps), each norm with a gain of its own
    x += l2 * n2b(feed_forward(n2(x)))       l1, l2: one number per channel ("layer scale"; left out: none)

A layer may have no feed-forward.  Norms, scales and the additions are 32-bit on the 32-bit residual stream.

What a sublayer returns is not added here at once: the block hands it on as a :class:`PendingPostNorm`, and whichever
norm reads the stream next does the norm on the result, the scale, the addition and its own norm in one kernel (the
norm in front of the feed-forward, the first norm of the next layer, or the model's last norm on the wanted rows).
"""
from __future__ import annotations

from .. import ops
from ..weights.loader import TensorSpec
from .base import Block


class PendingPostNorm:
    """A sublayer's result (32-bit sums or k-slice partial sums, plus an output bias) that is still to be normed,
    scaled and added to the residual stream."""

    def __init__(self, delta, bias, gain, layer_scale, eps, ctx):
        self.delta, self.bias, self.gain, self.layer_scale, self.eps, self.ctx = delta, bias, gain, layer_scale, eps, ctx

    def add_then_norm(self, resid, next_gain, next_eps, out, rows=None):
        ctx = self.ctx
        ops.postnorm_add_norm(resid, self.delta, self.gain, self.eps, ctx.q_start, ctx.q_len, ctx.E, y_bias=self.bias,
                              layer_scale=self.layer_scale, next_weight=next_gain, next_eps=next_eps, out=out, rows=rows)

    def add(self, resid):
        """The addition alone (whoever reads the stream next has no norm of this kind in front of it)."""
        ctx = self.ctx
        ops.postnorm_add_norm(resid, self.delta, self.gain, self.eps, ctx.q_start, ctx.q_len, ctx.E, y_bias=self.bias,
                              layer_scale=self.layer_scale)


class SandwichNormBlock(Block):
    """parts: ``norm1``, ``mixer``, ``norm1b`` and, unless the layer has none, ``norm2``, ``feed_forward``, ``norm2b``.
    params: ``hidden_size``; ``layer_scale`` (default False): tensors ``<prefix>ls1`` and ``<prefix>ls2`` [hidden]
    (names changeable through ``scale_tensors``).  A sublayer with an output bias offers it as ``output_bias``."""

    def __init__(self, params, prefix, build, parts):
        super().__init__(params, prefix, build, parts)
        self.hidden = int(params["hidden_size"])
        self.has_scale = bool(params.get("layer_scale", False))
        self.scale_names = tuple(params.get("scale_tensors", ("ls1", "ls2")))
        self.has_ff = "feed_forward" in parts
        for role in ("norm1", "norm1b") + (("norm2", "norm2b") if self.has_ff else ()):
            if role not in parts:
                raise ValueError(f"this arrangement needs a '{role}' part")
        self.scale = [None, None]

    def tensor_specs(self):
        specs = super().tensor_specs()
        if self.has_scale:
            specs += [TensorSpec(self.prefix + n, (self.hidden,), "vector") for n in self.scale_names[:2 if self.has_ff else 1]]
        return specs

    def bind(self, store):
        super().bind(store)
        if self.has_scale:
            for i, n in enumerate(self.scale_names[:2 if self.has_ff else 1]):
                self.scale[i] = store.vector(self.prefix + n).float().contiguous()

    def _pending(self, i, delta, part, ctx):
        post = self.parts["norm1b" if i == 0 else "norm2b"]
        return PendingPostNorm(delta, getattr(part, "output_bias", None), post.gain32(), self.scale[i], post.eps, ctx)

    def forward(self, resid, pending, ctx, cache, writes=True):
        mark = getattr(ctx, "mark", lambda label: None)
        y = self.parts["norm1"].forward(resid, pending)
        mixer = self.parts["mixer"]
        pending = self._pending(0, mixer.forward(y, ctx, cache, writes), mixer, ctx)
        mark("mixer")
        if self.has_ff:
            y = self.parts["norm2"].forward(resid, pending)
            ff = self.parts["feed_forward"]
            pending = self._pending(1, ff.forward(y, ctx), ff, ctx)
            mark("feed_forward")
        return pending
