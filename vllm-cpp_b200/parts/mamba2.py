"""A selective state-space mixer with a scalar decay per head (the Mamba-2 form):

    [z | x B C | dt] = W_in y                 z, x: heads * P lanes; B, C: groups * N lanes each; dt: one per head
    x B C  <-  silu(conv(x B C) + b)          a short causal convolution per channel, zero before the first token
    dt     <-  softplus(dt + dt_bias)
    S_t = exp(-exp(A_log_h) dt_t) S_(t-1) + dt_t B_t x_t^T ,   y_t = S_t^T C_t + D_h x_t      per head, S is [N, P]
    out = W_o (w * n_g(y * silu(z)))          n_g: the row in ``norm_groups`` equal parts, each by its own root mean square

Head h reads B and C of group h // (heads / groups).  Per request the part keeps the state S of every head (32-bit,
zero before the first token) and the convolution's last taps - 1 inputs, both in slots.  The projection's sums, dt,
softplus, the decay, the state and the gated norm are 32-bit; x, B and C leave the convolution in the compute dtype.
Long portions are cut into chunks whose local states are computed side by side and then chained (ops.ssm_scan).
"""
from __future__ import annotations

import torch

from .. import ops, workspace
from ..weights.loader import TensorSpec
from .base import CacheSpec, Mixer
from .linear import matmul_tn

CHUNK_TOKENS = 64         # tokens of a chunk of the recurrence
LONG_CHUNK_TOKENS = 256   # the same for steps of more than LONG_STEP_TOKENS tokens (fewer chunk states to keep)
LONG_STEP_TOKENS = 8192


class Mamba2Mixer(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``head_dim`` (P), ``state_size`` (N), ``groups``, ``conv_taps``,
    ``norm_groups``, ``eps``.  Tensors under the prefix: ``in`` [2 heads P + 2 groups N + heads, H], ``conv``
    [heads P + 2 groups N, taps], ``conv.b``, ``dt_bias``, ``A_log``, ``D`` [heads], ``norm`` [heads P], ``o`` [H, heads P]."""

    def __init__(self, params, prefix, build):
        super().__init__(params, prefix, build)
        p = params
        self.hidden = int(p["hidden_size"])
        self.heads, self.P, self.N = int(p["num_heads"]), int(p["head_dim"]), int(p["state_size"])
        self.groups, self.taps = int(p.get("groups", 1)), int(p["conv_taps"])
        self.norm_groups, self.eps = int(p.get("norm_groups", 1)), float(p.get("eps", 1e-5))
        if self.heads % self.groups:
            raise ValueError(f"{self.heads} heads are not a multiple of {self.groups} groups")
        self.inner = self.heads * self.P
        if self.inner % self.norm_groups:
            raise ValueError(f"{self.inner} lanes cannot be normed in {self.norm_groups} equal parts")
        self.conv_channels = self.inner + 2 * self.groups * self.N
        self.in_rows = 2 * self.inner + 2 * self.groups * self.N + self.heads
        self.w_in = self.w_o = self.conv_w = self.conv_b = self.dt_bias = self.rate = self.skip = self.norm_w = None

    def cache_spec(self):
        state = CacheSpec("state", shape=(self.heads, self.P, self.N), dtype="float32")
        if self.taps > 1:
            return (state, CacheSpec("state", shape=(self.taps - 1, self.conv_channels), dtype="float32"))
        return state

    def tensor_specs(self):
        p, H = self.prefix, self.hidden
        return [TensorSpec(p + "in", (self.in_rows, H)), TensorSpec(p + "conv", (self.conv_channels, self.taps), "bias"),
                TensorSpec(p + "conv.b", (self.conv_channels,), "bias"), TensorSpec(p + "dt_bias", (self.heads,), "bias"),
                TensorSpec(p + "A_log", (self.heads,), "bias"), TensorSpec(p + "D", (self.heads,), "vector"),
                TensorSpec(p + "norm", (self.inner,), "vector"), TensorSpec(p + "o", (H, self.inner))]

    def bind(self, store):
        p = self.prefix
        f32 = lambda name: store.vector(p + name).float().contiguous()
        self.w_in, self.w_o = store.matrix(p + "in"), store.matrix(p + "o")
        self.conv_w, self.conv_b = f32("conv"), f32("conv.b")
        self.dt_bias, self.skip, self.norm_w = f32("dt_bias"), f32("D"), f32("norm")
        self.rate = torch.exp(f32("A_log")).contiguous()      # the decay's rate, 32-bit

    def forward(self, x, ctx, cache, writes=True):
        if not writes:
            raise ValueError("a state-space mixer keeps a state of its own: it cannot read one another run left")
        state, conv_state = (cache[0].state, cache[1].state) if isinstance(cache, tuple) else (cache.state, None)
        T, dev = x.shape[0], x.device
        inner, cc = self.inner, self.conv_channels
        u = matmul_tn(x, self.w_in, ctx.status, out_dtype=torch.float32, allow_partials=True, after_small_kernel=True)
        xbc_in = u[..., inner:inner + cc]
        xbc = workspace.empty((T, cc), x.dtype, dev)
        ops.causal_conv(xbc_in, self.conv_w, conv_state, ctx.q_start, ctx.q_len, ctx.slots, ctx.E, out_conv=xbc,
                        out_bias=self.conv_b, act="silu")
        if self.taps > 1 and any(n > 1 for n in ctx.host_q_len):
            # (entries of one token were brought up to date by the convolution itself)
            ops.conv_state_update(xbc_in, conv_state, ctx.q_start, ctx.q_len, ctx.slots, ctx.E)
        chunk = LONG_CHUNK_TOKENS if T > LONG_STEP_TOKENS else CHUNK_TOKENS
        n_chunks = sum(-(-n // chunk) for n in ctx.host_q_len)
        scratch = decay = None
        if any(n > chunk for n in ctx.host_q_len):
            scratch = workspace.empty((n_chunks, self.heads, self.P, self.N), torch.float32, dev)
            decay = workspace.empty((n_chunks, self.heads), torch.float32, dev)
        y = workspace.empty((T, inner), torch.float32, dev)
        ops.ssm_scan(u, inner + cc, xbc, self.dt_bias, self.rate, self.skip, state, ctx.q_start, ctx.q_len, ctx.slots, ctx.E,
                     self.heads, self.P, self.N, self.groups, y, chunk=chunk, n_chunks=n_chunks, scratch=scratch,
                     chunk_decay=decay)
        g = workspace.empty((T, inner), x.dtype, dev)
        ops.gated_group_norm(y, u, self.norm_w, self.eps, ctx.q_start, ctx.q_len, ctx.E, self.norm_groups, g)
        return matmul_tn(g, self.w_o, ctx.status, out_dtype=torch.float32, allow_partials=True, after_small_kernel=True)
