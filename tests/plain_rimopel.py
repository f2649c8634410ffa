"""Plain, slow Rimopel decoder used as the oracle of the test-suite.

Whole sequences, no cache, no batching, one function per mechanism, float64.  It shares no code with the package
under test: it reads config.json as a plain dictionary and the weights with the test-suite's own safetensors reader,
and states every formula itself.

Notation: t, i, j are token positions of one sequence (from 0), c a channel, h a query head, W the model width.
"""
from __future__ import annotations

import functools
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


def sinusoid(positions, width, base=10000.0):
    """s[p, 2i] = sin(p * base^(-2i/width)), s[p, 2i+1] = cos(p * base^(-2i/width))."""
    p = torch.as_tensor(positions, dtype=F64)[:, None]
    out = torch.zeros(len(positions), width, dtype=F64)
    for c in range(width):
        ang = p[:, 0] * base ** (-2.0 * (c // 2) / width)
        out[:, c] = torch.cos(ang) if c % 2 else torch.sin(ang)
    return out


def embed(tokens, table, first_position=0):
    """x_t = E[token_t] + s(t)."""
    T = len(tokens)
    return table[torch.as_tensor(tokens, dtype=torch.long)] + sinusoid(range(first_position, first_position + T), table.shape[1])


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x, gain, eps):
    return unit_rms(x, eps) * gain


def causal_conv(u, taps_weight, before=None):
    """y_t = sum_j w[:, j] u_(t - taps + 1 + j) per channel; u is zero before the sequence (or ``before``: the rows
    that precede u, oldest first).  u [T, C], w [C, taps]."""
    T, C = u.shape
    taps = taps_weight.shape[1]
    pad = torch.zeros(taps - 1, C, dtype=F64)
    if before is not None and taps > 1:
        b = before[-(taps - 1):]
        pad[taps - 1 - b.shape[0]:] = b
    full = torch.cat([pad, u])
    y = torch.zeros(T, C, dtype=F64)
    for t in range(T):
        for j in range(taps):
            y[t] += taps_weight[:, j] * full[t + j]
    return y


def gate(h, weight, bias):
    """sigmoid(W h + b), one number per channel."""
    return torch.sigmoid(h @ weight.T + bias)


def visible(i, j, window, keep_first):
    """Whether the query at i sees the key at j."""
    if j > i:
        return False
    if window is None:
        return True
    return i - j < window or j < keep_first


def distance_penalty(i, j, a, b):
    """What is taken off the score of key j (a number or a tensor of positions) for the query at i."""
    return a * torch.log(1.0 + b * (i - torch.as_tensor(j, dtype=F64)))


@functools.lru_cache(maxsize=None)
def visible_keys(i, window, keep_first):
    return tuple(j for j in range(i + 1) if visible(i, j, window, keep_first))


def attend_head(q, k, v, scale, a, b, window, keep_first, first_position=0):
    """One query head over its key/value head.  q [Tq, d], k [Tk, d], v [Tk, dv]; the queries are the last Tq
    positions of the Tk keys (which start at position 0)."""
    Tq, Tk = q.shape[0], k.shape[0]
    out = torch.zeros(Tq, v.shape[1], dtype=F64)
    for n in range(Tq):
        i = Tk - Tq + n
        js = torch.tensor(visible_keys(i, window, keep_first), dtype=torch.long)
        s = scale * (k[js] @ q[n]) - distance_penalty(i, js, a, b)
        out[n] = torch.softmax(s, dim=0) @ v[js]
    return out


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def attention_mixer(h, w, p, m, eps):
    """The 'attention' mixer on its input h [T, W]; ``p`` the tensor-name prefix, ``m`` the mixer's config."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    proj = {}
    for n in ("q", "k", "v"):
        u = h @ w[p + n].T + w[p + n + ".b"]
        if m.get("conv"):
            u = causal_conv(u, w[p + n + ".conv"])
        proj[n] = u
    q = unit_rms(proj["q"].view(T, H, d), eps)
    k = unit_rms(proj["k"].view(T, G, d), eps)
    v = proj["v"].view(T, G, dv)
    mask = m.get("mask")
    window, keep = (mask["size"], mask.get("keep_first", 0)) if mask else (None, 0)
    heads = []
    for hh in range(H):
        g = hh // (H // G)
        heads.append(attend_head(q[:, hh], k[:, g], v[:, g], m["scale"], float(w[p + "r1"][hh]), float(w[p + "r2"][hh]), window, keep))
    return torch.cat(heads, dim=1) @ w[p + "o"].T


def dense_mlp(h, w, p):
    return gelu_erf(h @ w[p + "up"].T) @ w[p + "down"].T


def layer(x, cfg, w, i):
    """x += n1(g1(x) * mixer(x + conv(x))); x += n2(g2(x) * mlp(x))."""
    L, p, eps = cfg["layers"][i], f"l{i}.", cfg["norm"]["eps"]
    if L["type"] != "attention":
        raise ValueError(L["type"])
    h = x
    hc = h + causal_conv(h, w[p + "canon1"]) if cfg.get("canon") else h
    y = attention_mixer(hc, w, p + "mix.", L["mixer"], eps)
    x = x + rms_norm(y * gate(h, w[p + "rg1"], w[p + "rg1.b"]), w[p + "norm1"], eps)
    if L.get("mlp"):
        h = x
        x = x + rms_norm(dense_mlp(h, w, p + "mlp.") * gate(h, w[p + "rg2"], w[p + "rg2.b"]), w[p + "norm2"], eps)
    return x


def forward(cfg, w, tokens):
    """Logits [T, vocab] of a whole sequence."""
    x = embed(tokens, w["embed"])
    for i in range(len(cfg["layers"])):
        x = layer(x, cfg, w, i)
    return rms_norm(x, w["final.norm"], cfg["norm"]["eps"]) @ w["head"].T


def greedy(cfg, w, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]
