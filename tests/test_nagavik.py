"""Nagavik in the engine against the plain implementation (tests/plain_nagavik.py): each mechanism's kernel alone, then
whole models through bin/trace_run (whole prompts, decoding, portions down to two tokens, mixed batches with pages and
slots used again) and greedy generation through the engine's entry point, on small configurations of its own."""
import json
import math

import numpy as np
import pytest
import torch

import plain_nagavik as P
import replay_util as R
from conftest import random_tokens

gpu = pytest.mark.gpu
F64 = torch.float64


def configs():
    from vllm_cpp_b200.config.nagavik import NagavikAttention as A, NagavikConfig, NagavikLayer as L, NagavikMamba2 as M, NagavikMlp as F
    return {
        # no experts anywhere (bfloat16 can be judged row by row): a recurrence in two groups with four taps, an attention
        # layer without a feed-forward whose values are wider than its keys, a recurrence of odd sizes with one group and
        # two taps; capped logits, a scaled embedding; pages of 4
        "A": (NagavikConfig(vocab=150, width=48, max_positions=512, norm_eps=1e-5, embedding_scale=3.0, logit_softcap=8.0, layers=(
            L("mamba2", M(heads=4, vdim=8, state=16, groups=2, conv=4, norm_groups=2), F("dense", ff=40)),
            L("attention", A(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.3, softcap=20.0)),
            L("mamba2", M(heads=3, vdim=5, state=7, groups=1, conv=2, norm_groups=1), F("dense", ff=24)))), 4),
        # experts: two of five without a shared one, all three of three beside a shared one of another size; scores that
        # are not capped; keys and values of 64 lanes; a recurrence with 128 state lanes and 64 value lanes; logits not
        # capped, embedding not scaled; pages of 16
        "B": (NagavikConfig(vocab=260, width=64, max_positions=512, norm_eps=1e-6, layers=(
            L("attention", A(heads=6, kv_heads=6, dim=8, vdim=8, scale=0.5), F("moe", ff=24, experts=5, top=2)),
            L("mamba2", M(heads=2, vdim=64, state=128, groups=2, conv=3, norm_groups=4), F("moe", ff=16, experts=3, top=3, shared_ff=40)),
            L("attention", A(heads=2, kv_heads=1, dim=64, vdim=64, scale=0.125, softcap=5.0), F("dense", ff=72)))), 16),
        # a width that is no multiple of 4 (rows the tensor-core product cannot address), a convolution of one tap (no
        # state of its own), as many groups as heads, one expert of seven with a shared one, twenty query heads on one
        # KV head with values of 12 lanes; pages of 8
        "C": (NagavikConfig(vocab=97, width=50, max_positions=384, norm_eps=1e-4, embedding_scale=0.5, logit_softcap=30.0, layers=(
            L("mamba2", M(heads=5, vdim=6, state=33, groups=5, conv=1, norm_groups=5), F("moe", ff=9, experts=7, top=1, shared_ff=11)),
            L("attention", A(heads=20, kv_heads=1, dim=12, vdim=12, scale=0.2, softcap=2.0), F("moe", ff=10, experts=2, top=1, shared_ff=6)),
            L("mamba2", M(heads=2, vdim=10, state=20, groups=1, conv=8, norm_groups=2)))), 8),
    }


LENGTHS = {"A": [40, 75, 150, 33, 90, 64, 17, 2], "B": [1, 7, 33, 64, 170, 97, 130, 3], "C": [50, 3, 77, 140, 9, 31]}
REL_TOL = {"float32": 2e-5, "bfloat16": 3e-2}


@pytest.fixture(scope="module")
def nagavik_dirs(tmp_path_factory):
    """Random weights, then two things made by hand.  The recurrences' decay rates are spread from fast to very slow, so
    that a lost state or a token far back shows in the logits.  And the routers are made decisive: random routers have
    close calls between two experts every hundred tokens or so, which 16-bit activations decide differently from the
    64-bit plain implementation, and a token sent to another expert moves every later row.  So each token's embedding
    gets a large entry in one of the first lanes and one of half the size in another (by its id), and the routers read
    those lanes: which experts a token takes is then settled by a wide margin, in every number format."""
    from vllm_cpp_b200 import write_random_model
    from vllm_cpp_b200.weights.safetensors_io import read_safetensors, write_safetensors
    out = {}
    for i, (name, (cfg, _)) in enumerate(configs().items()):
        d = tmp_path_factory.mktemp(f"nagavik_{name}")
        write_random_model(cfg, 21 + i, d, dtype="bfloat16")
        tensors = {k: v.clone() for k, v in read_safetensors(d / "model.safetensors").items()}
        lanes = max([l.mlp.experts for l in cfg.layers if l.mlp is not None and l.mlp.kind == "moe"] + [0])
        if lanes:
            emb = tensors["embed"].float()
            emb[:, :lanes] = 0
            for t in range(cfg.vocab):
                first = t % lanes
                second = (first + 1 + (t // lanes) % (lanes - 1)) % lanes
                emb[t, first] = 30.0 / cfg.embedding_scale
                emb[t, second] = 15.0 / cfg.embedding_scale
            tensors["embed"] = emb.to(torch.bfloat16)
        for k in tensors:
            if k.endswith("mix.A_log"):
                tensors[k] = torch.linspace(-6.0, 0.5, tensors[k].numel()).to(torch.bfloat16)
            elif k.endswith("mlp.router"):
                E, W = tensors[k].shape
                r = torch.zeros(E, W)
                for lane in range(lanes):
                    r[lane % E, lane] = 1.0
                tensors[k] = r.to(torch.bfloat16)
        write_safetensors(d / "model.safetensors", tensors, {"format": "pt"})
        out[name] = d
    return out


class Oracle:
    def __init__(self, dirs):
        self.models = {n: P.read_model(d) for n, d in dirs.items()}
        self.cache = {}

    def __call__(self, name, tokens):
        key = (name, tuple(tokens))
        if key not in self.cache:
            self.cache[key] = P.forward(*self.models[name], list(tokens)).numpy()
        return self.cache[key]


@pytest.fixture(scope="module")
def oracle(nagavik_dirs):
    return Oracle(nagavik_dirs)


def requests_of(name):
    vocab = configs()[name][0].vocab
    return {f"r{i}": random_tokens(vocab, n, 5 * i + len(name)) for i, n in enumerate(LENGTHS[name])}


# -------------------------------------------------------------------------- without a GPU


def test_config_reads_every_size_and_constant():
    from vllm_cpp_b200 import ConfigError
    from vllm_cpp_b200.config.nagavik import NagavikConfig
    d = {"architecture": "Nagavik", "vocab": 50, "width": 24, "max_positions": 77, "norm": {"eps": 3e-4}, "embedding": {"scale": 2.5},
         "logit_softcap": 11.0,
         "layers": [{"type": "attention", "mlp": None,
                     "mixer": {"heads": 6, "kv_heads": 3, "dim": 10, "vdim": 14, "scale": 0.5, "softcap": 7.0}},
                    {"type": "mamba2", "mlp": {"kind": "dense", "ff": 31},
                     "mixer": {"heads": 4, "vdim": 6, "state": 9, "groups": 2, "conv": 3, "norm_groups": 4}},
                    {"type": "attention", "mixer": {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 1.0},
                     "mlp": {"kind": "moe", "router": {"experts": 9, "top": 2}, "expert": {"ff": 5}, "shared": {"ff": 13}}},
                    {"type": "attention", "mixer": {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 1.0},
                     "mlp": {"kind": "moe", "router": {"experts": 2, "top": 1}, "expert": {"ff": 3}, "shared": None}}]}
    cfg = NagavikConfig.from_dict(d)
    assert (cfg.vocab, cfg.width, cfg.max_positions, cfg.norm_eps, cfg.embedding_scale, cfg.logit_softcap) == (50, 24, 77, 3e-4, 2.5, 11.0)
    a, b, c, e = cfg.layers
    assert (a.mixer.heads, a.mixer.kv_heads, a.mixer.dim, a.mixer.vdim, a.mixer.scale, a.mixer.softcap, a.mlp) == (6, 3, 10, 14, 0.5, 7.0, None)
    assert (b.mixer.heads, b.mixer.vdim, b.mixer.state, b.mixer.groups, b.mixer.conv, b.mixer.norm_groups) == (4, 6, 9, 2, 3, 4)
    assert (b.mlp.kind, b.mlp.ff) == ("dense", 31)
    assert (c.mixer.softcap, c.mlp.kind, c.mlp.experts, c.mlp.top, c.mlp.ff, c.mlp.shared_ff) == (0.0, "moe", 9, 2, 5, 13)
    assert e.mlp.shared_ff == 0
    assert NagavikConfig.from_dict(cfg.to_dict()) == cfg
    # what is left out is off: no caps, a scale of one
    bare = NagavikConfig.from_dict({k: v for k, v in d.items() if k not in ("logit_softcap", "embedding")})
    assert bare.logit_softcap == 0.0 and bare.embedding_scale == 1.0
    layer = d["layers"]
    for bad in ({"layers": []}, {"layers": [dict(layer[0], type="other")]},
                {"layers": [dict(layer[0], mixer=dict(layer[0]["mixer"], kv_heads=4))]},
                {"layers": [dict(layer[1], mixer=dict(layer[1]["mixer"], groups=3))]},
                {"layers": [dict(layer[1], mixer=dict(layer[1]["mixer"], norm_groups=5))]},
                {"layers": [dict(layer[2], mlp=dict(layer[2]["mlp"], router={"experts": 2, "top": 3}))]},
                {"layers": [dict(layer[1], mlp={"kind": "routed", "ff": 3})]}, {"max_positions": None}):
        with pytest.raises(ConfigError):
            NagavikConfig.from_dict(dict(d, **bad))


def test_model_folder_is_recognised_and_names_its_tensors(tmp_path):
    from vllm_cpp_b200.models import expected_tensors, load_config
    cfg, _ = configs()["A"]
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
    assert load_config(tmp_path) == cfg
    s = {t.name: tuple(t.shape) for t in expected_tensors(cfg)}
    assert s["embed"] == (150, 48) and s["pos"] == (512, 48) and s["head"] == (150, 48) and s["final.norm"] == (48,)
    assert s["l0.mix.in"] == (2 * 32 + 2 * 2 * 16 + 4, 48) and s["l0.mix.conv"] == (32 + 64, 4) and s["l0.mix.conv.b"] == (96,)
    assert s["l0.mix.dt_bias"] == s["l0.mix.A_log"] == s["l0.mix.D"] == (4,) and s["l0.mix.norm"] == (32,) and s["l0.mix.o"] == (48, 32)
    assert s["l0.mlp.gate"] == (40, 48) and s["l0.mlp.up.b"] == (40,) and s["l0.mlp.down.b"] == (48,)
    assert s["l1.mix.q"] == (64, 48) and s["l1.mix.k"] == (32, 48) and s["l1.mix.v"] == (48, 48) and s["l1.mix.o"] == (48, 96)
    assert s["l1.mix.q.norm"] == (64,) and s["l1.mix.k.norm"] == (32,)
    for n in ("norm1", "norm1b", "ls1"):
        assert s[f"l1.{n}"] == (48,)
    assert not any(k.startswith(("l1.mlp", "l1.norm2", "l1.ls2")) for k in s)      # a layer without a feed-forward
    b, _ = configs()["B"]
    s = {t.name: tuple(t.shape) for t in expected_tensors(b)}
    assert s["l0.mlp.router"] == (5, 64) and s["l0.mlp.e4.up"] == (24, 64) and s["l0.mlp.e4.down"] == (64, 24)
    assert "l0.mlp.shared.up" not in s and s["l1.mlp.shared.up"] == (40, 64) and s["l1.mlp.shared.down"] == (64, 40)
    assert "l0.mlp.e5.up" not in s


def test_what_a_layer_keeps_per_request():
    import vllm_cpp_b200.models as models
    cfg, _ = configs()["A"]
    model = models.build_model(cfg, torch.float32, "cpu")
    specs = model.cache_specs()
    state, conv = specs[(0, 0)], specs[(0, 1)]
    assert (state.kind, state.shape, state.dtype) == ("state", (4, 8, 16), "float32")
    assert (conv.kind, conv.shape) == ("state", (3, 96))
    kv = specs[1]
    assert (kv.kind, kv.num_kv_heads, kv.head_dim, kv.v_head_dim, kv.window) == ("kv", 2, 16, 24, 0)
    c, _ = configs()["C"]
    specs = models.build_model(c, torch.float32, "cpu").cache_specs()
    assert specs[0].shape == (5, 6, 33)       # one tap: the convolution keeps nothing


def test_oracle_mechanisms_by_hand():
    # the sink takes its share: two keys of score 0 get a third each
    p = P.sink_softmax(torch.zeros(2, dtype=F64))
    assert torch.allclose(p, torch.full((2,), 1 / 3, dtype=F64))
    assert float(P.sink_softmax(torch.tensor([-800.0], dtype=F64))) == 0.0 and abs(float(P.sink_softmax(torch.tensor([800.0], dtype=F64))) - 1) < 1e-12
    assert P.head_slope(0, 8) == 0.5 and P.head_slope(7, 8) == 2.0 ** -8 and P.head_slope(0, 1) == 2.0 ** -8
    assert abs(float(P.capped(torch.tensor(1e9, dtype=F64), 50.0)) - 50.0) < 1e-9
    # one head, two tokens: the far key pays the slope once
    q = torch.tensor([[1.0, 0.0], [1.0, 0.0]], dtype=F64)
    k = torch.tensor([[2.0, 0.0], [0.0, 0.0]], dtype=F64)
    v = torch.tensor([[1.0], [10.0]], dtype=F64)
    out = P.attend_head(q, k, v, 0.5, None, 0.25)
    e0, e1 = math.exp(1.0 - 0.25), math.exp(0.0)
    assert abs(float(out[0, 0]) - math.e / (1 + math.e)) < 1e-12
    assert abs(float(out[1, 0]) - (e0 + 10 * e1) / (1 + e0 + e1)) < 1e-12
    # the recurrence by hand: one head, one state lane, one value lane
    y, last = P.ssm_scan(torch.tensor([[[2.0]], [[3.0]]], dtype=F64), torch.tensor([[[1.0]], [[0.5]]], dtype=F64),
                         torch.tensor([[[1.0]], [[4.0]]], dtype=F64), torch.tensor([[0.5], [2.0]], dtype=F64),
                         torch.tensor([0.1], dtype=F64), torch.tensor([10.0], dtype=F64))
    s0 = 0.5 * 1.0 * 2.0
    s1 = math.exp(-0.1 * 2.0) * s0 + 2.0 * 0.5 * 3.0
    assert abs(float(y[0, 0, 0]) - (s0 * 1.0 + 20.0)) < 1e-12 and abs(float(y[1, 0, 0]) - (s1 * 4.0 + 30.0)) < 1e-12
    assert abs(float(last[0, 0, 0]) - s1) < 1e-12
    # the gate comes before the grouped norm; each part has its own root mean square
    g = P.grouped_rms_norm(torch.tensor([[3.0, 4.0, 0.0, 10.0]], dtype=F64), torch.ones(4, dtype=F64), 2, 0.0)
    assert torch.allclose(g, torch.tensor([[3.0, 4.0, 0.0, 10.0]], dtype=F64) / torch.tensor([[12.5 ** 0.5] * 2 + [50 ** 0.5] * 2], dtype=F64))
    # an expert reads w * x: with the square of ReLU that is w^2 times what it returns for x
    w = {"up": torch.tensor([[1.0, -1.0]], dtype=F64), "down": torch.tensor([[2.0], [1.0]], dtype=F64)}
    x = torch.tensor([[3.0, 1.0]], dtype=F64)
    assert torch.allclose(P.expert(0.5 * x, w, ""), 0.25 * P.expert(x, w, ""))
    assert torch.allclose(P.expert(x, w, ""), torch.tensor([[8.0, 4.0]], dtype=F64)) and float(P.expert(-x, w, "").abs().sum()) == 0.0


# -------------------------------------------------------------------------- each kernel alone


def dev():
    return torch.device("cuda:0")


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=dev())


def entries_of(lengths):
    """(q_start, q_len) device arrays of a step whose entries have these token counts, rows in entry order."""
    starts = np.concatenate([[0], np.cumsum(lengths)])[:-1]
    return i32(starts.tolist()), i32(list(lengths))


def partial_sums(x, S, g):
    """x [T, C] (64-bit) as S 32-bit partial sums that add up to it (to 32-bit rounding)."""
    if S == 1:
        return x.float().to(dev())
    parts = torch.randn(S - 1, *x.shape, generator=g, dtype=F64)
    return torch.cat([parts, (x - parts.sum(0))[None]]).float().to(dev())


@gpu
@pytest.mark.parametrize("width", [6, 64, 257])
def test_scaled_embedding_with_learned_positions(width):
    from vllm_cpp_b200 import ops
    g = torch.Generator().manual_seed(width)
    table, pos = torch.randn(11, width, generator=g, dtype=F64), torch.randn(40, width, generator=g, dtype=F64)
    ids, where = [3, 0, 10, 3, 7], [0, 1, 39, 17, 2]
    out = torch.empty(5, width, device=dev())
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    ops.embed_scaled_pos(table.float().to(dev()), i32(ids), i32(where), pos.float().to(dev()), 2.5, out, status)
    want = torch.stack([P.embed([t], table, pos, 2.5, first_position=p)[0] for t, p in zip(ids, where)])
    torch.testing.assert_close(out.double().cpu(), want, atol=1e-5, rtol=1e-6)
    assert status.item() == 0
    ops.embed_scaled_pos(table.float().to(dev()), i32([1]), i32([40]), pos.float().to(dev()), 1.0, out[:1], status)
    assert status.item() == 8      # a position beyond the table is reported, not read
    status.zero_()


@gpu
@pytest.mark.parametrize("H,S,bias,scale,out_dtype", [(7, 1, False, False, None), (192, 3, True, True, torch.bfloat16),
                                                      (1500, 1, True, False, torch.float32), (13000, 2, False, True, torch.float32)])
def test_postnorm_scale_add_and_next_norm(H, S, bias, scale, out_dtype):
    """x += l * w_b * n(y + b), then w_n * n(x): rows outside the entries untouched; with a row list the stream is left alone."""
    from vllm_cpp_b200 import ops
    g = torch.Generator().manual_seed(H)
    T = 9
    x, y = torch.randn(T, H, generator=g, dtype=F64), torch.randn(T, H, generator=g, dtype=F64) * 3
    wb, wn, ls = (1 + 0.1 * torch.randn(H, generator=g, dtype=F64) for _ in range(3))
    b = torch.randn(H, generator=g, dtype=F64) if bias else None
    eps_b, eps_n = 1e-3, 1e-5
    f = lambda t: None if t is None else t.float().to(dev())
    d = P.rms_norm(y + (b if bias else 0), wb, eps_b) * (ls if scale else 1)
    want_x = x + d
    want_out = P.rms_norm(want_x, wn, eps_n)
    qs, ql = i32([0, 2, 2]), i32([2, 0, 5])       # rows 0..6 belong to entries (one of them empty), 7 and 8 are padding
    resid = f(x)
    out = torch.full((T, H), 7.0, device=dev(), dtype=out_dtype) if out_dtype else None
    ops.postnorm_add_norm(resid, partial_sums(y, S, g), f(wb), eps_b, qs, ql, 3, y_bias=f(b), layer_scale=f(ls) if scale else None,
                          next_weight=f(wn) if out_dtype else None, next_eps=eps_n, out=out)
    torch.testing.assert_close(resid.double().cpu()[:7], want_x[:7], atol=2e-5, rtol=2e-5)
    assert torch.equal(resid.cpu()[7:], x.float()[7:])
    if out_dtype:
        tol = dict(atol=2e-5, rtol=2e-5) if out_dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
        torch.testing.assert_close(out.double().cpu()[:7], want_out[:7], **tol)
        assert bool((out[7:] == 7.0).all())
        # the wanted rows only: the stream stays, the output is compact
        resid2 = f(x)
        rows = i32([5, 0])
        out2 = torch.empty(2, H, device=dev(), dtype=out_dtype)
        ops.postnorm_add_norm(resid2, partial_sums(y, S, g), f(wb), eps_b, qs, ql, 3, y_bias=f(b), layer_scale=f(ls) if scale else None,
                              next_weight=f(wn), next_eps=eps_n, out=out2, rows=rows)
        assert torch.equal(resid2.cpu(), x.float())
        torch.testing.assert_close(out2.double().cpu(), want_out[[5, 0]], **tol)


def flat_pages(num_pages, nkv, ps, d, dv, dtype):
    return torch.full((num_pages, nkv * ps * (d + dv)), float("nan"), device=dev(), dtype=dtype)


def page_key(pages, page, kvh, off, nkv, ps, d, dv):
    base = (kvh * ps + off) * d
    return pages[page, base:base + d]


def page_value(pages, page, kvh, off, nkv, ps, d, dv):
    base = nkv * ps * d + (kvh * ps + off) * dv
    return pages[page, base:base + dv]


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,d,dv,S", [(4, 2, 16, 24, 1), (3, 3, 20, 12, 2), (2, 1, 64, 64, 3), (20, 1, 12, 12, 1), (2, 2, 256, 8, 1)])
def test_whole_projection_norm_and_store(dtype, nh, nkv, d, dv, S):
    """One root mean square over all query lanes of a token (not one per head), one over all key lanes, gains per lane;
    keys and values land in the tokens' slots, in both page layouts; padding rows store nothing."""
    from vllm_cpp_b200 import ops
    g = torch.Generator().manual_seed(nh * d)
    T, ps, num_pages = 7, 4, 5
    C = nh * d + nkv * (d + dv)
    u = torch.randn(T, C, generator=g, dtype=F64) * torch.linspace(0.2, 3.0, C, dtype=F64)     # heads of unequal size
    qw, kw = 1 + 0.2 * torch.randn(nh * d, generator=g, dtype=F64), 1 + 0.2 * torch.randn(nkv * d, generator=g, dtype=F64)
    eps = 1e-4
    same = d == dv
    pages = torch.full((num_pages, 2, nkv, ps, d), float("nan"), device=dev(), dtype=dtype) if same else flat_pages(num_pages, nkv, ps, d, dv, dtype)
    slot_map = [9, 10, 11, 0, 17, -1, 3]         # row 5 belongs to no entry
    qs, ql = i32([0, 3, 6]), i32([3, 2, 1])
    q_out = torch.full((T, nh * d), float("nan"), device=dev(), dtype=dtype)
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    ops.qkv_wholenorm_store(partial_sums(u, S, g), qw.float().to(dev()), kw.float().to(dev()), eps, qs, ql, i32(slot_map), 3,
                            q_out, pages, nh, nkv, d, dv, status)
    assert status.item() == 0
    tol = dict(atol=3e-5, rtol=3e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    want_q = P.rms_norm(u[:, :nh * d], qw, eps)
    want_k = P.rms_norm(u[:, nh * d:nh * d + nkv * d], kw, eps)
    host = pages.cpu().double()
    for t in (0, 1, 2, 3, 4, 6):
        torch.testing.assert_close(q_out[t].double().cpu(), want_q[t], **tol)
        page, off = slot_map[t] // ps, slot_map[t] % ps
        for h in range(nkv):
            if same:
                key, val = host[page, 0, h, off], host[page, 1, h, off]
            else:
                key, val = page_key(host, page, h, off, nkv, ps, d, dv), page_value(host, page, h, off, nkv, ps, d, dv)
            torch.testing.assert_close(key, want_k[t, h * d:(h + 1) * d], **tol)
            torch.testing.assert_close(val, u[t, nh * d + nkv * d + h * dv:nh * d + nkv * d + (h + 1) * dv], **tol)
    assert bool(torch.isnan(q_out[5]).all())
    written = (~torch.isnan(host)).sum().item()
    assert written == 6 * nkv * (d + dv)


@gpu
@pytest.mark.parametrize("kind", ["gelu_tanh", "silu", "relu2"])
def test_gated_activation_and_capped_logits(kind):
    from vllm_cpp_b200 import ops
    g = torch.Generator().manual_seed(3)
    T, I = 5, 37
    x = torch.randn(T, 2 * I, generator=g, dtype=F64) * 2
    b = torch.randn(2 * I, generator=g, dtype=F64)
    act = {"gelu_tanh": P.gelu_tanh, "silu": P.silu, "relu2": lambda z: torch.clamp(z, min=0) ** 2}[kind]
    want = act(x[:, :I] + b[:I]) * (x[:, I:] + b[I:])
    out = torch.empty(T, I, device=dev())
    ops.gated_act(partial_sums(x, 3, g), out, kind, b.float().to(dev()))
    torch.testing.assert_close(out.double().cpu(), want, atol=2e-5, rtol=2e-5)
    ops.bias_act(partial_sums(x, 2, g), (o2 := torch.empty(T, 2 * I, device=dev())), kind)
    torch.testing.assert_close(o2.double().cpu(), act(x), atol=2e-5, rtol=2e-5)
    z = (x * 30).float().to(dev())
    ops.softcap(z, 15.0)
    torch.testing.assert_close(z.double().cpu(), P.capped(x * 30, 15.0), atol=2e-5, rtol=2e-5)


def conv_in_steps(C, taps, steps, dtype, S):
    """Runs causal_conv with an output bias and SiLU step by step for two requests in slots 2 and 0; returns what the
    kernel wrote per request and the plain convolution of the whole sequences."""
    from vllm_cpp_b200 import ops
    g = torch.Generator().manual_seed(C * 31 + taps)
    total = [sum(s[0] for s in steps), sum(s[1] for s in steps)]
    seqs = [torch.randn(n, C, generator=g, dtype=F64) for n in total]
    w, b = torch.randn(C, taps, generator=g, dtype=F64), torch.randn(C, generator=g, dtype=F64)
    state = torch.zeros(3, max(taps - 1, 1), C, device=dev())
    state[1] = float("nan")
    got = [[], []]
    at = [0, 0]
    for n0, n1 in steps:
        lens = [n0, n1]
        rows = torch.cat([seqs[r][at[r]:at[r] + lens[r]] for r in range(2)] + [torch.full((2, C), float("nan"), dtype=F64)])
        T = rows.shape[0]
        qs, ql = entries_of(lens)
        out = torch.full((T, C), 5.0, device=dev(), dtype=dtype)
        x = partial_sums(rows, S, g)
        ops.causal_conv(x, w.float().to(dev()), state if taps > 1 else None, qs, ql, i32([2, 0]), 2, out_conv=out,
                        out_bias=b.float().to(dev()), act="silu")
        if taps > 1 and any(n > 1 for n in lens):
            ops.conv_state_update(x, state, qs, ql, i32([2, 0]), 2)
        o = out.double().cpu()
        assert bool((o[n0 + n1:] == 5.0).all())
        got[0].append(o[:n0]); got[1].append(o[n0:n0 + n1])
        at = [at[0] + n0, at[1] + n1]
    want = [P.silu(P.causal_conv(s, w, b)) for s in seqs]
    return [torch.cat(x) for x in got], want


@gpu
@pytest.mark.parametrize("taps", [1, 2, 4, 8])
@pytest.mark.parametrize("C,S,dtype", [(5, 1, torch.float32), (96, 2, torch.bfloat16), (300, 3, torch.float32)])
def test_convolution_with_bias_and_silu_in_portions_equals_the_whole(taps, C, S, dtype):
    steps = [(3, 1), (1, 1), (2, 7), (1, 2), (9, 1), (1, 0), (2, 2)]
    got, want = conv_in_steps(C, taps, steps, dtype, S)
    tol = dict(atol=3e-5, rtol=3e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=2e-2)
    for a, b in zip(got, want):
        torch.testing.assert_close(a, b, **tol)


@gpu
@pytest.mark.parametrize("taps,C,S,dtype", [(4, 96, 1, torch.bfloat16), (1, 8, 2, torch.float32), (8, 300, 1, torch.float32), (3, 20, 3, torch.float32)])
def test_convolution_of_long_steps(taps, C, S, dtype):
    """Steps of more than 512 rows (the kernel that walks runs of rows with the taps' inputs in registers): entries that
    start and end inside a run, a run that begins in the middle of an entry, single tokens between long portions."""
    steps = [(530, 1), (1, 1), (300, 411), (2, 2), (1, 700), (17, 1)]
    got, want = conv_in_steps(C, taps, steps, dtype, S)
    tol = dict(atol=3e-5, rtol=3e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=2e-2)
    for a, b in zip(got, want):
        torch.testing.assert_close(a, b, **tol)


def run_attention(dtype, nh, nkv, d, dv, ps, shapes, cap, slope_exponent=8.0, sink=True, craft=None, scale=0.3, kernels=("plain",)):
    """shapes: [(tokens cached before the step, query tokens of the step)]; compares the attention kernels (decoded tokens
    with sliced key ranges, prompt portions in query tiles) with the plain attention of one head at a time."""
    from vllm_cpp_b200 import ops
    from vllm_cpp_b200.parts import attention as A
    g = torch.Generator().manual_seed(5)
    slopes = torch.tensor([2.0 ** (-slope_exponent * (h + 1) / nh) for h in range(nh)], dtype=F64)
    num_pages = sum(-(-(s + n) // ps) for s, n in shapes) + 3
    perm = torch.randperm(num_pages, generator=g).tolist()
    same = d == dv
    pages = (torch.full((num_pages, 2, nkv, ps, d), float("nan"), device=dev(), dtype=dtype) if same else flat_pages(num_pages, nkv, ps, d, dv, dtype))
    host = pages.cpu()
    seqs, qs, tables = [], [], []
    for start, n in shapes:
        k = torch.randn(start + n, nkv, d, generator=g, dtype=F64)
        v = torch.randn(start + n, nkv, dv, generator=g, dtype=F64)
        q = torch.randn(n, nh, d, generator=g, dtype=F64)
        if craft:
            craft(q, k, v, start, n)
        k, v, q = k.to(dtype).double(), v.to(dtype).double(), q.to(dtype).double()
        tab = [perm.pop() for _ in range(-(-(start + n) // ps))]
        for p in range(start + n):
            for h in range(nkv):
                if same:
                    host[tab[p // ps], 0, h, p % ps], host[tab[p // ps], 1, h, p % ps] = k[p, h].to(dtype), v[p, h].to(dtype)
                else:
                    page_key(host, tab[p // ps], h, p % ps, nkv, ps, d, dv)[:] = k[p, h].to(dtype)
                    page_value(host, tab[p // ps], h, p % ps, nkv, ps, d, dv)[:] = v[p, h].to(dtype)
        seqs.append((k, v)); qs.append(q); tables.append(tab)
    pages.copy_(host)

    class Ctx:
        pass
    ctx = Ctx()
    ctx.device = dev()
    ctx.host_q_len = [n for _, n in shapes]
    ctx.host_ctx_len = [s + n for s, n in shapes]
    ctx.host_q_start = [int(x) for x in np.cumsum([0] + ctx.host_q_len[:-1])]
    E, T = len(shapes), sum(ctx.host_q_len)
    bt = torch.full((E, max(len(t) for t in tables)), -1, dtype=torch.int32)
    for i, t in enumerate(tables):
        bt[i, :len(t)] = torch.tensor(t)
    q_flat = torch.cat(qs).to(dtype).to(dev()).view(T, nh * d)
    args = (pages, bt.to(dev()), i32(ctx.host_q_start), i32(ctx.host_q_len), i32(ctx.host_ctx_len))
    opts = dict(scale=scale, softcap=cap or 0.0, slope=slopes.float().to(dev()), sink=sink)
    wants = [[P.attend_head(q[:, h], k[:, h // (nh // nkv)], v[:, h // (nh // nkv)], scale, cap, float(slopes[h]) if slope_exponent else 0.0)
              for h in range(nh)] for q, (k, v) in zip(qs, seqs)]
    plans = {}
    for kernel in kernels:
        mma = kernel != "plain"
        DEC, SPAN = (A.MMA_DECODE_ROWS, A.MMA_SPAN_ROWS) if mma else (A.DECODE_ROWS, A.SPAN_ROWS)
        plan = plans[kernel] = A.AttentionPlan(ctx, nh, nkv, DEC, SPAN, d if kernel == "mma_cluster" else None)
        out = torch.full((T, nh * dv), float("nan"), device=dev(), dtype=dtype)
        status = torch.zeros(1, dtype=torch.int32, device=dev())
        if mma:
            run = lambda *x, **k: ops.attn_mma(*x, allow_tma=kernel != "mma_no_tma", **k, **opts)
        else:
            run = lambda *x, **k: ops.attn_window_bias(*x, hd_v=dv, **opts)
        if plan.n_dec:
            S = plan.nslices
            cluster = plan.cluster if kernel == "mma_cluster" else 0
            po = torch.empty(plan.n_dec * nh * S, dv, device=dev()) if S > 1 and not cluster else None
            pm = torch.empty(plan.n_dec * nh * S, 2, device=dev()) if S > 1 and not cluster else None
            run(q_flat, out, *args, plan.dec_items, plan.n_dec * S, DEC, po, pm, nh, nkv, d, 0, status,
                slice_counters=plan.slice_counters if S > 1 else None, dec_rows=plan.dec_rows, cluster=cluster)
            if S > 1 and not mma:
                ops.attn_merge(po, pm, plan.dec_rows, out, plan.n_dec, nh, dv, S)
        if plan.n_span_items and kernel == "tc":
            ops.attn_tc(q_flat, out, *args, plan.span_items, plan.n_span_items, nh, nkv, d, 0, status, **opts)
        elif plan.n_span_items:
            run(q_flat, out, *args, plan.span_items, plan.n_span_items, SPAN, None, None, nh, nkv, d, 0, status)
        torch.cuda.synchronize()
        assert status.item() == 0
        got = out.double().cpu().view(T, nh, dv)
        tol = dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
        t = 0
        for (start, n), want in zip(shapes, wants):
            for h in range(nh):
                torch.testing.assert_close(got[t:t + n, h], want[h], **tol, msg=lambda m: f"{kernel}, entry at {start}+{n}, head {h}: {m}")
            t += n
    return plans


def attention_kernels(dtype, d, dv, ps):
    """The kernels that take these sizes with the design's options: the plain one, and in bfloat16 with keys and values of
    64 or 128 lanes the tensor-core ones."""
    from vllm_cpp_b200 import ops
    from vllm_cpp_b200.parts.window_attention import EXTRAS_ON_TENSOR_CORES
    kernels = ["plain"]
    if EXTRAS_ON_TENSOR_CORES and d == dv and ops.attn_mma_supported(dtype, d):
        kernels += ["mma", "mma_no_tma", "mma_cluster"]
        if ops.attn_tc_supported(dtype, d, ps):
            kernels.append("tc")
    return tuple(kernels)


MIXED_SHAPES = [(0, 1), (0, 37), (300, 1), (5, 2), (63, 1), (64, 1), (17, 130), (1500, 1), (128, 64), (0, 2)]


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,d,dv,ps,cap", [(4, 2, 16, 24, 4, 20.0), (3, 3, 20, 12, 8, None), (8, 2, 64, 64, 16, 4.0), (2, 1, 128, 128, 32, 50.0),
                                                (40, 1, 8, 256, 5, 1.5), (1, 1, 64, 64, 8, None)])
def test_capped_sloped_sink_attention_mixed_batch(dtype, nh, nkv, d, dv, ps, cap):
    """First tokens of a sequence, single tokens behind short and long contexts (sliced key ranges that are merged, the
    sink counted once), portions that start inside a page and span many tiles; one head (slope 2^-8) to forty."""
    # (forty heads on the plain implementation: the shorter contexts are enough to see every one of them)
    shapes = MIXED_SHAPES if nh <= 8 else [s for s in MIXED_SHAPES if s[0] + s[1] <= 200] + [(1100, 1)]
    plans = run_attention(dtype, nh, nkv, d, dv, ps, shapes, cap, kernels=attention_kernels(dtype, d, dv, ps))
    assert plans["plain"].nslices > 1


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("which", ["far_key", "all_low", "capped_high", "first_token"])
@pytest.mark.parametrize("d,dv,ps", [(24, 40, 8), (64, 64, 16), (128, 128, 32)])
def test_one_mechanism_decides_the_row(dtype, which, d, dv, ps):
    """Inputs made so that one mechanism shows: a key 900 tokens back that outweighs its slope; scores so low that
    the sink takes nearly all the weight (without it the row would be an average of values); a score far above the
    cap, which must not swamp the others; the first token of a sequence, which shares its weight with the sink only."""
    def craft(q, k, v, start, n):
        L = start + n
        if which == "far_key" and L > 950:
            j = L - 1 - 900
            k[j] = 0
            k[j, :, 0] = 8.0
            q[:, :, 0] = 8.0            # score 0.3 * 64 = 19.2 at key j, for every query row
            v[j] = 3.0
        elif which == "all_low":
            k[:, :, :] = -k.abs()
            q[:, :, :] = q.abs() * 3    # every score far below zero
        elif which == "capped_high":
            k[L // 2] = 0
            k[L // 2, :, 1] = 30.0
            q[:, :, 1] = 30.0           # 0.3 * 900 = 270, capped to 6
            v[L // 2] = -2.0
    cap = 6.0 if which != "far_key" else 25.0
    shapes = [(1000, 1), (960, 48), (0, 1), (0, 3), (40, 1)]
    # the last head's slope is 2^-8: the far key keeps 19.2 - 3.5; the first head's is steep and loses it
    run_attention(dtype, 4, 2, d, dv, ps, shapes, cap, craft=craft, kernels=attention_kernels(dtype, d, dv, ps))


def run_recurrence(heads, Pv, N, groups, steps, dtype, S, rates, n_slots=3):
    """The recurrence step by step for two requests in slots 2 and 0 (slot 1 holds NaN); returns y per request, the
    final states, and the plain recurrence over the whole sequences."""
    from vllm_cpp_b200 import ops
    g = torch.Generator().manual_seed(heads * 100 + N)
    inner, gn = heads * Pv, groups * N
    total = [sum(s[0] for s in steps), sum(s[1] for s in steps)]
    seqs = []
    for n in total:
        xbc = (torch.randn(n, inner + 2 * gn, generator=g, dtype=F64)).to(dtype).double()
        dt_raw = torch.randn(n, heads, generator=g, dtype=F64)
        seqs.append((xbc, dt_raw))
    dt_bias = torch.randn(heads, generator=g, dtype=F64) * 0.5
    skip = torch.randn(heads, generator=g, dtype=F64)
    rate = torch.as_tensor(rates, dtype=F64)
    state = torch.zeros(n_slots, heads, Pv, N, device=dev())
    state[1] = float("nan")
    got, at = [[], []], [0, 0]
    pad_cols = 3                                       # dt sits behind other columns of a wider projection
    for n0, n1 in steps:
        lens = [n0, n1]
        T = n0 + n1 + 2
        xbc = torch.cat([seqs[r][0][at[r]:at[r] + lens[r]] for r in range(2)] + [torch.full((2, inner + 2 * gn), float("nan"), dtype=F64)])
        dt_raw = torch.cat([seqs[r][1][at[r]:at[r] + lens[r]] for r in range(2)] + [torch.full((2, heads), float("nan"), dtype=F64)])
        u = partial_sums(torch.cat([torch.zeros(T, pad_cols, dtype=F64), dt_raw], dim=1), S, g)
        qs, ql = entries_of(lens)
        y = torch.full((T, inner), 9.0, device=dev())
        chunk = 32
        n_chunks = sum(-(-n // chunk) for n in lens)
        multi = any(n > chunk for n in lens)
        scratch = torch.full((n_chunks, heads, Pv, N), float("nan"), device=dev()) if multi else None
        decay = torch.full((n_chunks, heads), float("nan"), device=dev()) if multi else None
        ops.ssm_scan(u, pad_cols, xbc.to(dtype).to(dev()), dt_bias.float().to(dev()), rate.float().to(dev()), skip.float().to(dev()),
                     state, qs, ql, i32([2, 0]), 2, heads, Pv, N, groups, y, chunk=chunk, n_chunks=n_chunks, scratch=scratch,
                     chunk_decay=decay)
        o = y.double().cpu()
        assert bool((o[n0 + n1:] == 9.0).all())
        got[0].append(o[:n0]); got[1].append(o[n0:n0 + n1])
        at = [at[0] + n0, at[1] + n1]
    want = []
    for xbc, dt_raw in seqs:
        n = xbc.shape[0]
        y, last = P.ssm_scan(xbc[:, :inner].reshape(n, heads, Pv), xbc[:, inner:inner + gn].reshape(n, groups, N),
                             xbc[:, inner + gn:].reshape(n, groups, N), P.softplus(dt_raw + dt_bias), rate, skip)
        want.append((y.reshape(n, inner), last))
    assert bool(torch.isnan(state[1]).all())
    return [torch.cat(x) for x in got], state.double().cpu(), want


@gpu
@pytest.mark.parametrize("dtype,S", [(torch.float32, 1), (torch.bfloat16, 3)])
@pytest.mark.parametrize("heads,Pv,N,groups", [(4, 8, 16, 2), (3, 5, 7, 1), (2, 64, 128, 2), (5, 6, 33, 5), (1, 20, 200, 1), (2, 40, 56, 1), (1, 300, 4, 1), (1, 8, 300, 1)])
def test_recurrence_in_portions_equals_the_whole(dtype, S, heads, Pv, N, groups):
    """Portions of one token, of two, of a chunk and one more, of several chunks, beside a request of other lengths; decay
    rates from 0.002 (the first tokens still count after hundreds) to 3 (the state is gone in two); the state in its slot
    between the steps.  Shapes: state lanes that are no multiple of four, one state lane run per thread and four, more
    value lanes than a block takes, 300 state lanes (more shared memory than a block has by default)."""
    steps = [(3, 1), (1, 1), (2, 33), (1, 2), (70, 1), (32, 64), (1, 97), (2, 2), (129, 1)]
    rates = torch.logspace(math.log10(0.002), math.log10(3.0), heads).tolist()
    got, state, want = run_recurrence(heads, Pv, N, groups, steps, dtype, S, rates)
    for r, slot in ((0, 2), (1, 0)):
        y, last = want[r]
        scale = float(y.abs().max())
        assert float((got[r] - y).abs().max()) < 3e-5 * scale, (r, float((got[r] - y).abs().max()), scale)
        torch.testing.assert_close(state[slot], last.transpose(1, 2), atol=3e-5 * float(last.abs().max()), rtol=1e-4)


@gpu
@pytest.mark.parametrize("C,parts,S,dtype", [(32, 2, 1, torch.float32), (30, 5, 2, torch.bfloat16), (4096, 4, 1, torch.float32), (21, 1, 3, torch.float32)])
def test_gate_then_norm_in_parts(C, parts, S, dtype):
    from vllm_cpp_b200 import ops
    g = torch.Generator().manual_seed(C)
    T = 6
    y, z = torch.randn(T, C, generator=g, dtype=F64) * torch.linspace(0.1, 5, C, dtype=F64), torch.randn(T, C + 9, generator=g, dtype=F64)
    w = 1 + 0.2 * torch.randn(C, generator=g, dtype=F64)
    qs, ql = i32([0, 4]), i32([4, 1])           # row 5 is padding
    out = torch.full((T, C), 3.0, device=dev(), dtype=dtype)
    ops.gated_group_norm(y.float().to(dev()), partial_sums(z, S, g), w.float().to(dev()), 1e-5, qs, ql, 2, parts, out)
    want = P.grouped_rms_norm(y * P.silu(z[:, :C]), w, parts, 1e-5)
    tol = dict(atol=3e-5, rtol=3e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(out.double().cpu()[:5], want[:5], **tol)
    assert bool((out[5] == 3.0).all())


@gpu
@pytest.mark.parametrize("tile_rows", [16, 32, 64, 128, 256])
@pytest.mark.parametrize("T,H,E,top,ff,sff,on_input", [(1, 16, 4, 1, 8, 0, True), (37, 48, 5, 2, 24, 12, True), (300, 64, 3, 3, 16, 40, True),
                                                       (64, 56, 70, 4, 200, 0, False), (9, 192, 10, 1, 72, 72, True), (700, 128, 6, 2, 136, 0, True)])
def test_routed_experts_on_tensor_cores(tile_rows, T, H, E, top, ff, sff, on_input):
    """The same through the gathered rows and the grouped tcgen05 product, at every tile size: experts of fewer rows than
    a block of 128 features (the next expert's rows in the same weight tile must not leak), of more, of no multiple."""
    check_routed_experts(torch.bfloat16, T, H, E, top, ff, sff, on_input, tile_rows)


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,E,top,ff,sff,on_input", [(1, 16, 4, 1, 8, 0, True), (37, 48, 5, 2, 24, 12, True), (150, 64, 3, 3, 16, 40, True),
                                                       (64, 50, 70, 4, 9, 0, False), (9, 32, 11, 1, 88, 88, True)])
def test_routed_experts(dtype, T, H, E, top, ff, sff, on_input):
    check_routed_experts(dtype, T, H, E, top, ff, sff, on_input, None)


def check_routed_experts(dtype, T, H, E, top, ff, sff, on_input, tile_rows):
    """Router, sorting into tiles, the experts' two products and the sum per token against the plain feed-forward; experts
    that no token chose, more experts than tokens, every expert chosen by every token; rows of padding route nowhere."""
    from vllm_cpp_b200 import ops
    g = torch.Generator().manual_seed(T + E)
    x = torch.randn(T + 2, H, generator=g, dtype=F64).to(dtype).double()
    router = torch.randn(E, H, generator=g, dtype=F64)
    w = {"router": router}
    for e in range(E):
        w[f"e{e}.up"] = (torch.randn(ff, H, generator=g, dtype=F64) / H ** 0.5).to(dtype).double()
        w[f"e{e}.down"] = (torch.randn(H, ff, generator=g, dtype=F64) / ff ** 0.5).to(dtype).double()
    logits = x @ router.T
    qs, ql = entries_of([T // 2, 0, T - T // 2])          # the last two rows belong to no entry
    sel_e = torch.full((T + 2, top), -7, dtype=torch.int32, device=dev())
    sel_w = torch.full((T + 2, top), float("nan"), device=dev())
    ops.moe_route(partial_sums(logits, 2, g), qs, ql, 3, top, sel_e, sel_w)
    order = torch.topk(logits[:T], top, dim=1)
    assert torch.equal(sel_e.cpu()[:T].long(), order.indices) and bool((sel_e[T:] == -1).all())
    torch.testing.assert_close(sel_w.double().cpu()[:T], torch.sigmoid(order.values), atol=1e-5, rtol=1e-5)
    BM = tile_rows or ops.moe_tile_rows()
    tiles = ops.moe_tiles_cap((T + 2) * top, E, BM)
    pos_of = torch.empty((T + 2) * top, dtype=torch.int32, device=dev())
    src_of = torch.empty(tiles * BM, dtype=torch.int32, device=dev())
    tile_expert = torch.empty(tiles, dtype=torch.int32, device=dev())
    ops.moe_group(sel_e, E, tiles, pos_of, src_of, tile_expert, BM)
    po, so, te, se = pos_of.cpu().tolist(), src_of.cpu().tolist(), tile_expert.cpu().tolist(), sel_e.cpu().view(-1).tolist()
    for a, pos in enumerate(po):
        if se[a] < 0:
            assert pos == -1
        else:
            assert so[pos] == a and te[pos // BM] == se[a]      # every pair sits in a tile of its expert
    assert sum(1 for s in so if s >= 0) == T * top and sorted(e for e in te if e >= 0) == [e for e in te if e >= 0]
    xd = x.to(dtype).to(dev())
    w_up = torch.stack([w[f"e{e}.up"] for e in range(E)]).to(dtype).to(dev())
    w_down = torch.stack([w[f"e{e}.down"] for e in range(E)]).to(dtype).to(dev())
    h1 = torch.full((tiles * BM, ff), float("nan"), device=dev(), dtype=dtype)
    y = torch.full((tiles * BM, H), float("nan"), device=dev())
    if tile_rows:
        # the tensor-core products: the rows gathered and weighted in sorted order first
        assert ops.gemm_grouped_ok(xd, w_up) and ops.gemm_grouped_ok(xd, w_down)
        xs = torch.full((tiles * BM, H), float("nan"), device=dev(), dtype=dtype)
        status = torch.zeros(1, dtype=torch.int32, device=dev())
        ops.moe_gather(xd, src_of, sel_w if on_input else None, top, xs)
        ops.gemm_bf16_grouped(w_up, xs, tile_expert, BM, h1, status, act="relu2")
        ops.gemm_bf16_grouped(w_down, h1, tile_expert, BM, y, status)
        assert status.item() == 0
    else:
        ops.moe_gemm(xd, w_up, tile_expert, h1, src_of=src_of, sel_w=sel_w if on_input else None, top=top, act="relu2")
        ops.moe_gemm(h1, w_down, tile_expert, y)
    shared = torch.randn(T + 2, H, generator=g, dtype=F64) if sff else None
    out = torch.full((T + 2, H), 4.0, device=dev())
    ops.moe_combine(y, pos_of, top, qs, ql, 3, out, shared=None if shared is None else partial_sums(shared, 2, g),
                    sel_w=None if on_input else sel_w)
    want = torch.zeros(T, H, dtype=F64)
    for t in range(T):
        for e, z in zip(order.indices[t].tolist(), order.values[t].tolist()):
            s = 1 / (1 + math.exp(-z))
            want[t] += P.expert((s * x[t])[None], w, f"e{e}.")[0] if on_input else s * P.expert(x[t][None], w, f"e{e}.")[0]
    if sff:
        want += shared[:T]
    tol = dict(atol=3e-5, rtol=3e-5) if dtype == torch.float32 else dict(atol=4e-2, rtol=3e-2)
    torch.testing.assert_close(out.double().cpu()[:T], want, **tol)
    assert bool((out[T:] == 4.0).all())


# -------------------------------------------------------------------------- whole models through the trace replay


def compare(name, dtype, trace, out_dir, requests, oracle):
    vocab = configs()[name][0].vocab
    worst = 0.0
    for step, want in enumerate(trace.wanted):
        got = R.read_step(out_dir, step, vocab)
        if not want:
            assert got is None
            continue
        assert got is not None and got.shape == (len(want), vocab), f"step {step}: {None if got is None else got.shape}"
        ref = np.stack([oracle(name, requests[rid])[pos] for rid, pos in want])
        err = np.abs(got - ref).max(axis=1) / np.abs(ref).max()
        bad = np.nonzero(~(err <= REL_TOL[dtype]))[0]
        assert len(bad) == 0, (f"{name} {dtype}: step {step}, first wrong row {want[bad[0]]} (request, position): "
                               f"relative error {err[bad[0]]:.3e} > {REL_TOL[dtype]}")
        worst = max(worst, err.max())
    return worst


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "portions_last", "mixed", "mixed_last"])
def test_replay(name, dtype, mode, nagavik_dirs, oracle, tmp_path):
    """Whole prompts; the last 32 tokens one by one; portions of changing size down to two tokens; up to four live
    requests with pages and slots used again -- the last two also as serving asks (logits of an entry's last token
    only: captured steps), all over a NaN-filled cache."""
    requests = requests_of(name)
    trace = {"whole": R.whole, "tail": R.tail_one_by_one, "portions": R.portions, "portions_last": R.portions_last,
             "mixed": R.mixed, "mixed_last": R.mixed_last}[mode](requests)
    out = R.run_trace(nagavik_dirs[name], dtype, trace, tmp_path / "out", configs()[name][1], extra_args=["--poison"])
    worst = compare(name, dtype, trace, out, requests, oracle)
    print(f"{name} {dtype} {mode}: worst relative error {worst:.3e}, pool {trace.max_tokens} tokens, {len(trace.steps)} steps")


@gpu
def test_replay_modes_agree_with_each_other(nagavik_dirs, tmp_path):
    """Cutting and batching change the logits by rounding only."""
    for name in ("A", "B"):
        requests = requests_of(name)
        vocab = configs()[name][0].vocab
        rows = {}
        for mode, build in (("whole", R.whole), ("mixed", R.mixed), ("portions", R.portions)):
            trace = build(requests)
            out = R.run_trace(nagavik_dirs[name], "float32", trace, tmp_path / (name + mode), configs()[name][1])
            for step, want in enumerate(trace.wanted):
                got = R.read_step(out, step, vocab)
                for i, key in enumerate(want):
                    rows.setdefault(key, {})[mode] = got[i]
        worst = max(np.abs(v["whole"] - v[m]).max() / np.abs(v["whole"]).max() for v in rows.values() for m in ("mixed", "portions"))
        assert worst < 2e-5, (name, worst)


@gpu
def test_long_decoding(nagavik_dirs, oracle, tmp_path):
    """A short prompt, then 250 tokens one by one: the states carried through 250 steps, the keys of 260 positions."""
    for name in ("A", "B"):
        toks = random_tokens(configs()[name][0].vocab, 260, 99)
        trace = R.tail_one_by_one({"long": toks}, tail=250)
        out = R.run_trace(nagavik_dirs[name], "float32", trace, tmp_path / name, configs()[name][1], extra_args=["--poison"])
        compare(name, "float32", trace, out, {"long": toks}, oracle)


# -------------------------------------------------------------------------- generation through the engine's entry point


@gpu
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_scheduler(name, nagavik_dirs):
    """Several prompts at once through LLM.generate (scheduler, portions under a small token budget, captured decoding
    steps, device-side sampling at temperature 0) against the plain implementation's greedy continuation."""
    from vllm_cpp_b200 import LLM
    cfg, w = P.read_model(nagavik_dirs[name])
    vocab, page = configs()[name][0].vocab, configs()[name][1]
    prompts = [random_tokens(vocab, n, 3 + n) for n in (5, 41, 18, 70, 2)]
    llm = LLM(str(nagavik_dirs[name]), dtype="float32", page_size=page, max_tokens=page * 64, max_num_seqs=3, max_step_tokens=32,
              max_model_len=256)
    got = llm.generate(prompts, max_new_tokens=24, temperature=0.0, top_p=1.0, repeat_penalty=1.0, ignore_eos=True)
    for prompt, g in zip(prompts, got):
        want = P.greedy(cfg, w, prompt, 24)
        # a near tie between two logits may fall the other way in 32-bit: compare up to the first such place
        for i, (a, b) in enumerate(zip(g, want)):
            if a != b:
                logits = P.forward(cfg, w, prompt + want[:i])[-1]
                assert abs(float(logits[a] - logits[b])) < 1e-4, (i, a, b)
                break
        assert len(g) == 24
