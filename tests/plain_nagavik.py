"""Plain, slow Nagavik decoder used as the oracle of the test-suite.

Whole sequences, no cache, no batching, one function per mechanism, float64.  It shares no code with the package
under test: it reads config.json as a plain dictionary and the weights with the test-suite's own safetensors reader,
and states every formula itself.

Notation: t, i, j are token positions of one sequence (from 0), c a channel, h a head, n a state lane, p a value
lane, W the model width.
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch

from plain_qwen3 import read_safetensors

F64 = torch.float64


def read_model(model_dir):
    model_dir = Path(model_dir)
    return json.loads((model_dir / "config.json").read_text()), read_safetensors(model_dir / "model.safetensors")


# -------------------------------------------------------------------------- mechanisms, one function each


def embed(tokens, table, pos_table, scale, first_position=0):
    """x_t = scale * E[token_t] + P[t]."""
    ids = torch.as_tensor(tokens, dtype=torch.long)
    where = torch.arange(first_position, first_position + len(tokens))
    return table[ids] * scale + pos_table[where]


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x, gain, eps):
    return unit_rms(x, eps) * gain


def silu(z):
    return z / (1.0 + torch.exp(-z))


def softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + torch.clamp(z, min=0.0)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def head_slope(h, heads):
    """2^(-8 (h + 1) / heads)."""
    return 2.0 ** (-8.0 * (h + 1) / heads)


def capped(s, cap):
    """cap * tanh(s / cap)."""
    return cap * torch.tanh(s / cap)


def sink_softmax(s):
    """p_j = exp(s_j) / (1 + sum_j exp(s_j)): a silent extra key of score 0 takes its share."""
    m = max(float(s.max()), 0.0)
    e = torch.exp(s - m)
    return e / (math.exp(-m) + e.sum())


def attend_head(q, k, v, scale, cap, slope):
    """One head: the last len(q) positions of a sequence of len(k) query all keys up to their own.  Capped scaled
    scores less slope * distance, softmax with the silent sink.  q [n, d], k [L, d], v [L, dv] -> [n, dv]."""
    n, L = q.shape[0], k.shape[0]
    out = torch.zeros(n, v.shape[1], dtype=F64)
    for r in range(n):
        i = L - n + r
        s = (k[:i + 1] @ q[r]) * scale
        if cap:
            s = capped(s, cap)
        s = s - slope * (i - torch.arange(i + 1)).to(F64)
        out[r] = sink_softmax(s) @ v[:i + 1]
    return out


def attention(x, w, pre, m, eps):
    """Grouped-query attention on full-projection-normed queries and keys, capped scores less a slope times the
    distance, causal, softmax with a silent sink.  x [T, W]."""
    T = x.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm(x @ w[pre + "q"].T, w[pre + "q.norm"], eps).reshape(T, H, d)
    k = rms_norm(x @ w[pre + "k"].T, w[pre + "k.norm"], eps).reshape(T, G, d)
    v = (x @ w[pre + "v"].T).reshape(T, G, dv)
    out = torch.zeros(T, H, dv, dtype=F64)
    for h in range(H):
        g = h // (H // G)
        out[:, h] = attend_head(q[:, h], k[:, g], v[:, g], m["scale"], m.get("softcap"), head_slope(h, H))
    return out.reshape(T, H * dv) @ w[pre + "o"].T


def causal_conv(u, taps_weight, bias):
    """y_t = b + sum_j w[:, j] u_(t - taps + 1 + j) per channel; u is zero before the sequence.  u [T, C], w [C, taps]."""
    T, C = u.shape
    taps = taps_weight.shape[1]
    full = torch.cat([torch.zeros(taps - 1, C, dtype=F64), u])
    y = torch.zeros(T, C, dtype=F64)
    for t in range(T):
        y[t] = bias
        for j in range(taps):
            y[t] += taps_weight[:, j] * full[t + j]
    return y


def ssm_scan(xs, B, C, dt, a, D, start=None):
    """Per head h (group g = h // (heads / groups)), from S = 0 (or ``start`` [heads, N, P]):
    S <- exp(-a_h dt_t) S + dt_t B_t x_t^T,  y_t = S^T C_t + D_h x_t.
    xs [T, heads, P], B and C [T, groups, N], dt [T, heads], a and D [heads].  Returns y and the last states."""
    T, Hn, P = xs.shape
    Gn, N = B.shape[1], B.shape[2]
    y = torch.zeros(T, Hn, P, dtype=F64)
    last = torch.zeros(Hn, N, P, dtype=F64)
    for h in range(Hn):
        g = h // (Hn // Gn)
        S = torch.zeros(N, P, dtype=F64) if start is None else start[h].clone()
        for t in range(T):
            S = math.exp(-float(a[h]) * float(dt[t, h])) * S + float(dt[t, h]) * torch.outer(B[t, g], xs[t, h])
            y[t, h] = S.T @ C[t, g] + D[h] * xs[t, h]
        last[h] = S
    return y, last


def grouped_rms_norm(y, gain, parts, eps):
    """The row cut into ``parts`` equal pieces, each divided by its own root mean square; then the gain."""
    T, C = y.shape
    return (unit_rms(y.reshape(T, parts, C // parts), eps)).reshape(T, C) * gain


def mamba2(x, w, pre, m, eps):
    T = x.shape[0]
    Hn, P, N, Gn = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = Hn * P
    u = x @ w[pre + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * Gn * N], u[:, 2 * inner + 2 * Gn * N:]
    xbc = silu(causal_conv(xbc, w[pre + "conv"], w[pre + "conv.b"]))
    xs = xbc[:, :inner].reshape(T, Hn, P)
    B = xbc[:, inner:inner + Gn * N].reshape(T, Gn, N)
    C = xbc[:, inner + Gn * N:].reshape(T, Gn, N)
    dt = softplus(dt + w[pre + "dt_bias"])
    y = ssm_scan(xs, B, C, dt, torch.exp(w[pre + "A_log"]), w[pre + "D"])[0].reshape(T, inner)
    y = grouped_rms_norm(y * silu(z), w[pre + "norm"], m["norm_groups"], eps)
    return y @ w[pre + "o"].T


def dense_ff(x, w, pre):
    g = x @ w[pre + "gate"].T + w[pre + "gate.b"]
    u = x @ w[pre + "up"].T + w[pre + "up.b"]
    return (gelu_tanh(g) * u) @ w[pre + "down"].T + w[pre + "down.b"]


def expert(x, w, pre):
    """down(relu(up x)^2), no biases."""
    return torch.clamp(x @ w[pre + "up"].T, min=0.0) ** 2 @ w[pre + "down"].T


def routed(x, router):
    """For each token the chosen experts and their weights: the sigmoid of the router's logit, as it is."""
    return torch.sigmoid(x @ router.T)


def moe_ff(x, w, pre, mlp):
    T = x.shape[0]
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    s = routed(x, w[pre + "router"])
    out = torch.zeros(T, w[pre + "e0.down"].shape[0], dtype=F64)
    for t in range(T):
        for e in torch.topk(s[t], top).indices.tolist():
            out[t] += expert((s[t, e] * x[t])[None], w, f"{pre}e{e}.")[0]
    if mlp.get("shared") is not None:
        out = out + expert(x, w, pre + "shared.")
    return out


MIXERS = {"attention": attention, "mamba2": mamba2}

# -------------------------------------------------------------------------- the model


def forward(cfg, weights, tokens, keep_layers=False):
    """Logits [T, vocab] of one whole sequence (and, with keep_layers, the stream after every layer)."""
    w = {k: v.to(F64) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = embed(tokens, w["embed"], w["pos"], (cfg.get("embedding") or {}).get("scale", 1.0))
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        d = MIXERS[layer["type"]](rms_norm(x, w[p + "norm1"], eps), w, p + "mix.", layer["mixer"], eps)
        x = x + rms_norm(d, w[p + "norm1b"], eps) * w[p + "ls1"]
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rms_norm(x, w[p + "norm2"], eps)
            d = dense_ff(h, w, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(h, w, p + "mlp.", mlp)
            x = x + rms_norm(d, w[p + "norm2b"], eps) * w[p + "ls2"]
        after.append(x.clone())
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    if cfg.get("logit_softcap"):
        logits = capped(logits, cfg["logit_softcap"])
    return (logits, after) if keep_layers else logits


def greedy(cfg, weights, prompt, n_new):
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(forward(cfg, weights, tokens)[-1].argmax()))
    return tokens[len(prompt):]
