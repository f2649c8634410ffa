"""An arrangement with the norm on the sublayer's result and a gate on what it adds:

    x += n1(g1(x) * mixer(x + conv(x)))          g(x) = sigmoid(W x + b), elementwise
    x += n2(g2(x) * feed_forward(x))             n(v) = w * v / sqrt(mean(v^2) + eps)

The sublayers read the residual stream itself (no norm in front of them).  What the mixer reads passes a causal
convolution over time first, per channel: conv(x)_t = sum_j c[:, j] x_(t - taps + 1 + j), zero before a request's first
token; the taps - 1 rows before a portion are part of the request's state, kept here (a fixed-size state beside
whatever the mixer keeps).  The gate reads the stream as it is, before that convolution.  A layer may have no
feed-forward.  Gates, norms and the addition are 32-bit; the products read the stream in the compute dtype.

The block does its additions itself (each is fused with the gate and the norm), so it hands nothing pending on.
"""
from __future__ import annotations

import torch

from .. import ops, workspace
from ..weights.loader import TensorSpec
from .base import Block, CacheSpec
from .linear import matmul_tn


class GatedPostNormBlock(Block):
    """parts: ``norm1``, ``mixer`` and, unless the layer has none, ``norm2`` and ``feed_forward``.
    params: ``hidden_size``; ``conv_taps`` (0: no convolution on the mixer's input); ``gated`` (default True).
    Tensors under the layer's prefix: ``canon1`` [hidden, taps], ``rg1`` [hidden, hidden], ``rg1.b`` [hidden], and
    ``rg2``, ``rg2.b`` with a feed-forward."""

    def __init__(self, params, prefix, build, parts):
        super().__init__(params, prefix, build, parts)
        self.hidden = int(params["hidden_size"])
        self.taps = int(params.get("conv_taps") or 0)
        self.gated = bool(params.get("gated", True))
        self.has_ff = "feed_forward" in parts
        if self.has_ff != ("norm2" in parts):
            raise ValueError("a feed-forward and its norm come together")
        self.conv_w = None
        self.gate_w = [None, None]
        self.gate_b = [None, None]
        self.norm_w = [None, None]
        self.gate_in_ff = False

    # ---- weights ----
    def tensor_specs(self):
        p, H = self.prefix, self.hidden
        specs = super().tensor_specs()
        if self.taps:
            specs.append(TensorSpec(p + "canon1", (H, self.taps), "bias"))
        if self.gated:
            for n in ("rg1", "rg2")[:2 if self.has_ff else 1]:
                specs += [TensorSpec(p + n, (H, H)), TensorSpec(p + n + ".b", (H,), "bias")]
        return specs

    def bind(self, store):
        super().bind(store)
        p = self.prefix
        if self.taps:
            self.conv_w = store.vector(p + "canon1").float().contiguous()
        for i, (n, norm) in enumerate((("rg1", "norm1"), ("rg2", "norm2"))[:2 if self.has_ff else 1]):
            if self.gated:
                self.gate_w[i] = store.matrix(p + n)
                self.gate_b[i] = store.vector(p + n + ".b").float().contiguous()
            self.norm_w[i] = self.parts[norm].weight.float().contiguous()
        # the feed-forward's gate reads what the feed-forward reads: one product for both where the part offers it
        self.gate_in_ff = self.gated and self.has_ff and hasattr(self.parts["feed_forward"], "attach_side_rows")
        if self.gate_in_ff:
            self.parts["feed_forward"].attach_side_rows(self.gate_w[1])
            self.gate_w[1] = None

    # ---- per-request state ----
    def _own_spec(self):
        return CacheSpec("state", shape=(self.taps - 1, self.hidden), dtype="float32") if self.taps > 1 else None

    def cache_spec(self):
        mine, theirs = self._own_spec(), self.mixer.cache_spec()
        theirs = () if theirs is None else (theirs if isinstance(theirs, tuple) else (theirs,))
        out = (() if mine is None else (mine,)) + theirs
        return out or None

    def _split(self, cache):
        """(this block's state view or None, what the mixer is handed)."""
        if cache is None:
            return None, None
        views = cache if isinstance(cache, tuple) else (cache,)
        mine = None
        if self.taps > 1:
            mine, views = views[0], views[1:]
        theirs = self.mixer.cache_spec()
        return mine, (views if isinstance(theirs, tuple) else (views[0] if views else None))

    # ---- one step ----
    def _sublayer_add(self, i, resid, delta, h, ctx, out_cast=None, gate=None):
        if gate is None and self.gated:
            gate = matmul_tn(h, self.gate_w[i], ctx.status, out_dtype=torch.float32, allow_partials=True)
        norm = self.parts["norm1" if i == 0 else "norm2"]
        ops.gated_norm_add(resid, delta, gate, self.gate_b[i], self.norm_w[i], norm.eps, ctx.q_start, ctx.q_len, ctx.E,
                           out_cast=out_cast)

    def forward(self, resid, pending, ctx, cache, writes=True):
        mark = getattr(ctx, "mark", lambda label: None)
        if hasattr(pending, "add"):
            pending.add(resid)
        elif pending is not None:
            # a layer of another arrangement came before and left its last addition to this one
            resid.add_((pending.sum(0) if pending.dim() == 3 else pending).float())
        T, H = resid.shape
        dt, dev = self.build.compute_dtype, resid.device
        own, mixer_cache = self._split(cache)
        state = own.state if own is not None else None
        # what the gate reads (the stream in the compute dtype) and what the mixer reads (the same plus its convolution)
        h = resid if dt == torch.float32 else workspace.empty((T, H), dt, dev)
        if self.taps:
            hc = workspace.empty((T, H), dt, dev)
            ops.causal_conv(resid, self.conv_w, state, ctx.q_start, ctx.q_len, ctx.slots, ctx.E, out_conv=hc,
                            out_copy=None if h is resid else h, add_input=True)
            if self.taps > 1 and any(n > 1 for n in ctx.host_q_len):
                # (entries of one token were brought up to date by the convolution itself)
                ops.conv_state_update(resid, state, ctx.q_start, ctx.q_len, ctx.slots, ctx.E)
        else:
            if h is not resid:
                ops.causal_conv(resid, None, None, ctx.q_start, ctx.q_len, ctx.slots, ctx.E, out_copy=h)
            hc = h
        d = self.mixer.forward(hc, ctx, mixer_cache, writes)
        x2 = None
        if self.has_ff and dt != torch.float32:
            x2 = workspace.empty((T, H), dt, dev)
        self._sublayer_add(0, resid, d, h, ctx, out_cast=x2)
        mark("mixer")
        if self.has_ff:
            h2 = resid if x2 is None else x2
            ff = self.parts["feed_forward"]
            d2 = ff.forward(h2, ctx)
            self._sublayer_add(1, resid, d2, h2, ctx, gate=ff.side if self.gate_in_ff else None)
            mark("feed_forward")
        return None
