"""Rimopel in the engine against the plain implementation (tests/plain_rimopel.py): each mechanism's kernel alone, then
whole models through bin/trace_run (whole prompts, decoding, portions down to two tokens, mixed batches with pages and
slots used again) and greedy generation through the engine's entry point, on small configurations of its own."""
import json
import math

import numpy as np
import pytest
import torch

import plain_rimopel as P
import replay_util as R
from conftest import random_tokens


def mixer(heads, kv, dim, vdim, scale, conv=0, window=0, keep=0):
    from vllm_cpp_b200.config.rimopel import RimopelMixer
    return RimopelMixer(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale, conv=conv, window=window, keep_first=keep)


def configs():
    from vllm_cpp_b200.config.rimopel import RimopelConfig, RimopelLayer
    L = RimopelLayer
    return {
        # values of another size than keys, taps 4 and 2, a window shorter than a prompt portion, more kept keys than
        # the window is wide, a layer without feed-forward, a convolution of one tap; pages of 4
        "P": (RimopelConfig(vocab=200, width=64, norm_eps=1e-5, canon_taps=2, layers=(
            L("attention", mixer(4, 2, 16, 24, 0.3, conv=4, window=12, keep=3), "dense", 96),
            L("attention", mixer(2, 2, 32, 16, 0.2, conv=1, window=40, keep=0)),
            L("attention", mixer(6, 1, 8, 8, 3.0, conv=2, window=5, keep=7), "dense", 40))), 4),
        # no input convolution, no short convolution, no mask, head sizes that are no multiple of 8, an inner size of
        # the output projection that is no multiple of 8; pages of 8
        "Q": (RimopelConfig(vocab=300, width=96, norm_eps=1e-6, layers=(
            L("attention", mixer(3, 3, 20, 12, 0.25), "dense", 100),
            L("attention", mixer(2, 1, 64, 64, 0.125, conv=3, window=33, keep=1), "dense", 72))), 8),
        # head size 64 with values of 32, windows that end inside a page, one query head per KV head; pages of 16
        "S": (RimopelConfig(vocab=260, width=128, norm_eps=1e-5, canon_taps=4, layers=(
            L("attention", mixer(4, 2, 64, 32, 0.15, conv=2, window=48, keep=2), "dense", 192),
            L("attention", mixer(2, 2, 32, 64, 0.2, conv=3, window=70, keep=17)))), 16),
        # a width that is no multiple of 4 (rows the tensor-core product cannot address), five taps, eight taps on the
        # mixer's input, as many KV heads as query heads; pages of 4
        "U": (RimopelConfig(vocab=97, width=50, norm_eps=1e-4, canon_taps=8, layers=(
            L("attention", mixer(5, 5, 6, 10, 0.4, conv=5, window=9, keep=2), "dense", 33),
            L("attention", mixer(1, 1, 36, 4, 0.1, conv=2, window=30, keep=30), "dense", 7))), 4),
        # an inner size below one k-block of the products, forty query heads on one KV head (more than a block of the
        # plain attention kernel holds), a window of one key; pages of 8
        "V": (RimopelConfig(vocab=128, width=40, norm_eps=1e-5, canon_taps=3, layers=(
            L("attention", mixer(40, 1, 12, 12, 0.3, conv=3, window=1, keep=1), "dense", 24),
            L("attention", mixer(8, 2, 16, 8, 0.25, conv=3, window=21, keep=4)))), 8),
    }


LENGTHS = {"P": [40, 75, 128, 33, 90, 64, 17, 2], "Q": [1, 7, 33, 64, 150, 97, 130, 3], "S": [200, 65, 256, 3, 129, 64, 48, 100],
           "U": [50, 3, 77, 120, 9, 31], "V": [90, 2, 41, 70, 1, 33]}
REL_TOL = {"float32": 2e-5, "bfloat16": 3e-2}


@pytest.fixture(scope="module")
def rimopel_dirs(tmp_path_factory):
    from vllm_cpp_b200 import write_random_model
    out = {}
    for i, (name, (cfg, _)) in enumerate(configs().items()):
        d = tmp_path_factory.mktemp(f"rimopel_{name}")
        write_random_model(cfg, 11 + i, d, dtype="bfloat16")
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
def oracle(rimopel_dirs):
    return Oracle(rimopel_dirs)


def requests_of(name):
    vocab = configs()[name][0].vocab
    return {f"r{i}": random_tokens(vocab, n, 7 * i + len(name)) for i, n in enumerate(LENGTHS[name])}


# -------------------------------------------------------------------------- without a GPU


def test_config_reads_every_size_and_constant():
    from vllm_cpp_b200 import ConfigError
    from vllm_cpp_b200.config.rimopel import RimopelConfig
    from vllm_cpp_b200.models import load_config
    d = {"architecture": "Rimopel", "vocab": 50, "width": 24, "norm": {"eps": 3e-4}, "canon": {"taps": 5},
         "layers": [{"type": "attention", "mlp": None,
                     "mixer": {"heads": 6, "kv_heads": 3, "dim": 10, "vdim": 14, "scale": 0.5, "conv": 2,
                               "mask": {"size": 9, "keep_first": 4}}},
                    {"type": "attention", "mlp": {"kind": "dense", "ff": 31},
                     "mixer": {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 1.0}}]}
    cfg = RimopelConfig.from_dict(d)
    assert (cfg.vocab, cfg.width, cfg.norm_eps, cfg.canon_taps) == (50, 24, 3e-4, 5)
    a, b = cfg.layers
    assert (a.mixer.heads, a.mixer.kv_heads, a.mixer.dim, a.mixer.vdim, a.mixer.scale, a.mixer.conv) == (6, 3, 10, 14, 0.5, 2)
    assert (a.mixer.window, a.mixer.keep_first, a.mlp_kind) == (9, 4, None)
    assert (b.mixer.window, b.mixer.keep_first, b.mixer.conv, b.mlp_kind, b.ff) == (0, 0, 0, "dense", 31)
    assert RimopelConfig.from_dict(cfg.to_dict()) == cfg
    for bad in ({"layers": []}, {"layers": [dict(d["layers"][0], type="other")]},
                {"layers": [dict(d["layers"][0], mixer=dict(d["layers"][0]["mixer"], kv_heads=4))]},
                {"layers": [dict(d["layers"][1], mlp={"kind": "routed", "ff": 3})]}):
        with pytest.raises(ConfigError):
            RimopelConfig.from_dict(dict(d, **bad))


def test_model_folder_is_recognised_and_names_its_tensors(tmp_path):
    from vllm_cpp_b200.models import expected_tensors, load_config
    cfg, _ = configs()["P"]
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
    assert load_config(tmp_path) == cfg
    specs = {s.name: tuple(s.shape) for s in expected_tensors(cfg)}
    assert specs["embed"] == (200, 64) and specs["head"] == (200, 64) and specs["final.norm"] == (64,)
    assert specs["l0.mix.q"] == (64, 64) and specs["l0.mix.k"] == (32, 64) and specs["l0.mix.v"] == (48, 64)
    assert specs["l0.mix.v.conv"] == (48, 4) and specs["l0.mix.o"] == (64, 96) and specs["l0.mix.r2"] == (4,)
    assert specs["l0.canon1"] == (64, 2) and specs["l0.rg2.b"] == (64,) and specs["l0.mlp.up"] == (96, 64)
    assert "l1.mlp.up" not in specs and "l1.rg2" not in specs and "l1.norm2" not in specs and "l1.rg1" in specs
    assert specs["l1.mix.q.conv"] == (64, 1)
    q, _ = configs()["Q"]
    names = {s.name for s in expected_tensors(q)}
    assert "l0.canon1" not in names and "l0.mix.q.conv" not in names and "l1.mix.q.conv" in names


def test_what_a_layer_keeps_per_request():
    import vllm_cpp_b200.models as M
    from vllm_cpp_b200.cache.device_cache import CacheLayout
    cfg, _ = configs()["P"]
    model = M.build_model(cfg, torch.float32, "cpu")
    specs = model.cache_specs()
    # layer 0: the block's state (one row of the stream), pages with kept first keys, the projection's last three rows
    assert specs[(0, 0)].kind == "state" and specs[(0, 0)].shape == (1, 64)
    assert (specs[(0, 1)].window, specs[(0, 1)].keep_first, specs[(0, 1)].head_dim, specs[(0, 1)].v_head_dim) == (12, 3, 16, 24)
    assert specs[(0, 2)].shape == (3, 64 + 32 + 48)
    # layer 1: a convolution of one tap keeps nothing
    assert set(k for k in specs if k[0] == 1) == {(1, 0), (1, 1)} and specs[(1, 1)].v_head_dim == 16
    layout = CacheLayout(specs)
    assert len(layout.paged) == 3 and all(g.paged for g in layout.groups[:3])


def test_pages_of_kept_first_keys_are_never_given_back():
    from vllm_cpp_b200.runtime import runtime
    rt = runtime()
    m = rt.CacheManager([rt.GroupSpec(4, 64, 10, 6), rt.GroupSpec(4, 64, 10)], 2)
    assert m.open(1) == 0 and m.reserve(1, 100)
    m.commit(1, 100)
    kept, plain = m.block_table(1, 0), m.block_table(1, 1)
    first_needed = 100 - 10 + 1
    for b in range(25):
        dead = (b + 1) * 4 <= first_needed
        assert (plain[b] < 0) == dead
        assert (kept[b] < 0) == (dead and b >= 2)      # positions 0..5 lie in pages 0 and 1
    assert m.peak_pages(0, 1000, 16) == m.peak_pages(1, 1000, 16) + 2
    m.check_invariants()
    m.close(1)
    assert m.free_pages(0) == 64 and m.free_pages(1) == 64


def test_oracle_mechanisms_by_hand():
    assert [P.visible(10, j, 4, 2) for j in (0, 1, 2, 6, 7, 10, 11)] == [True, True, False, False, True, True, False]
    assert P.visible(3, 0, None, 0) and P.visible_keys(9, 3, 2) == (0, 1, 7, 8, 9)
    assert abs(float(P.distance_penalty(5, 5, 2.0, 0.3))) == 0.0
    assert abs(float(P.distance_penalty(9, 4, 2.0, 0.3)) - 2.0 * math.log(2.5)) < 1e-12
    u = torch.arange(10, dtype=torch.float64).view(5, 2)
    w = torch.tensor([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]], dtype=torch.float64)
    y = P.causal_conv(u, w)
    assert y[:, 1].tolist() == u[:, 1].tolist() and y[:, 0].tolist() == [0.0, 200.0, 420.0, 642.0, 864.0]
    assert torch.equal(P.causal_conv(u[3:], w, before=u[:3]), y[3:])
    s = P.sinusoid([0, 3], 6)
    assert s[0].tolist() == [0, 1, 0, 1, 0, 1] and abs(float(s[1, 2]) - math.sin(3 * 10000 ** (-2 / 6))) < 1e-12


# -------------------------------------------------------------------------- kernels, one mechanism each

gpu = pytest.mark.gpu


def dev():
    return torch.device("cuda:0")


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=dev())


@gpu
@pytest.mark.parametrize("width", [6, 64, 257])
def test_sinusoid_is_added_to_the_embedding(width):
    from vllm_cpp_b200 import ops
    table = torch.randn(11, width, dtype=torch.float64)
    ids, pos = [3, 0, 10, 3, 7], [0, 1, 2, 500, 70001]
    out = torch.empty(5, width, device=dev())
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    inv = torch.tensor([10000.0 ** (-2.0 * i / width) for i in range((width + 1) // 2)], dtype=torch.float64).float().to(dev())
    ops.embed_sinusoid(table.float().to(dev()), i32(ids), i32(pos), inv, out, status)
    want = table[ids] + P.sinusoid(pos, width)
    # a 32-bit angle of 70,001 is exact to 0.004: the low frequencies carry that
    torch.testing.assert_close(out.double().cpu()[:4], want[:4], atol=5e-5, rtol=0)
    torch.testing.assert_close(out.double().cpu()[4], want[4], atol=8e-3, rtol=0)
    assert status.item() == 0


def conv_in_steps(C, taps, steps, dtype, add_input, bias, S):
    """Runs sequences through causal_conv + conv_state_update in the given steps ([(slot, n tokens), ...] each) and
    returns per slot what came out, with the inputs."""
    from vllm_cpp_b200 import ops
    g = torch.Generator().manual_seed(C * 31 + taps)
    w = torch.randn(C, taps, generator=g, dtype=torch.float64)
    b = torch.randn(C, generator=g, dtype=torch.float64) if bias else None
    state = torch.full((5, max(taps - 1, 1), C), float("nan"), device=dev())[:, :taps - 1]
    seen = {}
    got = {}
    for entries in steps:
        T = sum(n for _, n in entries)
        parts = torch.randn(S, T + 2, C, generator=g, dtype=torch.float64)      # two padding rows at the end
        x = parts.sum(0)[:T] + (b if bias else 0)
        q_start = list(np.cumsum([0] + [n for _, n in entries[:-1]]))
        q_len = [n for _, n in entries]
        slots = [s for s, _ in entries]
        fresh = [s for s, _ in entries if s not in seen]
        for s in fresh:
            state[s] = 0.0                      # what the engine does for a request that starts
        xin = parts.float().to(dev())
        out = torch.full((T + 2, C), 7.0, device=dev(), dtype=dtype)
        copy = torch.full((T + 2, C), 7.0, device=dev(), dtype=dtype)
        # an entry without tokens (a captured step's empty slot) sits in the middle
        qs, ql, sl = q_start[:1] + [q_start[1] if len(q_start) > 1 else T] + q_start[1:], q_len[:1] + [0] + q_len[1:], slots[:1] + [4] + slots[1:]
        args = (i32(qs), i32(ql), i32(sl), len(qs))
        ops.causal_conv(xin if S > 1 else xin[0], w.float().to(dev()), state if taps > 1 else None, *args, out_conv=out,
                        out_copy=copy, bias=None if b is None else b.float().to(dev()), add_input=add_input)
        if taps > 1:
            ops.conv_state_update(xin if S > 1 else xin[0], state, *args, bias=None if b is None else b.float().to(dev()))
        torch.cuda.synchronize()
        assert (out[T:] == 7.0).all() and (copy[T:] == 7.0).all()          # rows of no entry are left alone
        for (s, n), t0 in zip(entries, q_start):
            seen.setdefault(s, []).append(x[t0:t0 + n])
            got.setdefault(s, []).append(out[t0:t0 + n].double().cpu())
            torch.testing.assert_close(copy[t0:t0 + n].double().cpu(), x[t0:t0 + n].to(dtype).double(), atol=1e-6, rtol=1e-6)
    return w, {s: torch.cat(v) for s, v in seen.items()}, {s: torch.cat(v) for s, v in got.items()}


@gpu
@pytest.mark.parametrize("taps", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("C,S,add_input,bias", [(5, 1, True, False), (300, 3, False, True)])
def test_causal_conv_in_portions_equals_the_whole(taps, C, S, add_input, bias):
    """Portions of one, two and more tokens, shorter and longer than the state, several requests in a step."""
    steps = [[(0, 5), (1, 1)], [(1, 1), (0, 2)], [(0, 1), (2, 9), (1, 1)], [(1, 2)], [(0, 1), (1, 1), (2, 1)], [(2, 2), (0, 7)], [(1, 30)]]
    w, seen, got = conv_in_steps(C, taps, steps, torch.float32, add_input, bias, S)
    for s in seen:
        want = P.causal_conv(seen[s], w) + (seen[s] if add_input else 0)
        torch.testing.assert_close(got[s], want, atol=2e-5, rtol=1e-5)


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
@pytest.mark.parametrize("nh,nkv,d,dv,taps,S", [(4, 2, 16, 24, 3, 1), (3, 3, 20, 12, 0, 2), (2, 1, 64, 64, 2, 3), (2, 2, 256, 8, 4, 1)])
def test_projection_convolution_unit_norm_and_store(dtype, nh, nkv, d, dv, taps, S):
    from vllm_cpp_b200 import ops
    g = torch.Generator().manual_seed(nh * 100 + d)
    C, ps, eps = nh * d + nkv * (d + dv), 4, 1e-5
    entries = [(2, 6), (0, 1), (3, 2)]            # (slot, tokens): a portion, a single token, a portion of two
    T = sum(n for _, n in entries)
    parts = torch.randn(S, T, C, generator=g, dtype=torch.float64)
    bias = torch.randn(C, generator=g, dtype=torch.float64)
    w = torch.randn(C, max(taps, 1), generator=g, dtype=torch.float64)
    before = {s: torch.randn(max(taps - 1, 0), C, generator=g, dtype=torch.float64).float().double() for s, _ in entries}
    state = torch.zeros(4, max(taps - 1, 1), C, device=dev())[:, :max(taps - 1, 0)]
    for s, b in before.items():
        state[s] = b.float().to(dev())
    same = d == dv
    pages = (torch.full((9, 2, nkv, ps, d), float("nan"), device=dev(), dtype=dtype) if same else flat_pages(9, nkv, ps, d, dv, dtype))
    slot_map = torch.randperm(9 * ps, generator=g)[:T].tolist()
    q_out = torch.empty(T, nh * d, device=dev(), dtype=dtype)
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    q_start = list(np.cumsum([0] + [n for _, n in entries[:-1]]))
    xin = parts.float().to(dev())
    args = (i32(q_start), i32([n for _, n in entries]), i32([s for s, _ in entries]))
    ops.qkv_conv_norm_store(xin if S > 1 else xin[0], bias.float().to(dev()), w.float().to(dev()) if taps else None,
                            state if taps > 1 else None, *args, i32(slot_map), len(entries), q_out, pages, nh, nkv, d, dv, eps, status)
    if taps > 1:
        ops.conv_state_update(xin if S > 1 else xin[0], state, *args, len(entries), bias=bias.float().to(dev()))
    torch.cuda.synchronize()
    assert status.item() == 0
    tol = dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    u = parts.float().double().sum(0) + bias.float().double()
    for (s, n), t0 in zip(entries, q_start):
        y = P.causal_conv(u[t0:t0 + n], w.float().double(), before=before[s]) if taps else u[t0:t0 + n]
        q = P.unit_rms(y[:, :nh * d].reshape(n, nh, d), eps).reshape(n, nh * d)
        k = P.unit_rms(y[:, nh * d:(nh + nkv) * d].reshape(n, nkv, d), eps)
        v = y[:, (nh + nkv) * d:].reshape(n, nkv, dv)
        torch.testing.assert_close(q_out[t0:t0 + n].double().cpu(), q, **tol)
        for i in range(n):
            page, off = divmod(slot_map[t0 + i], ps)
            for h in range(nkv):
                gk = pages[page, 0, h, off] if same else page_key(pages, page, h, off, nkv, ps, d, dv)
                gv = pages[page, 1, h, off] if same else page_value(pages, page, h, off, nkv, ps, d, dv)
                torch.testing.assert_close(gk.double().cpu(), k[i, h], **tol)
                torch.testing.assert_close(gv.double().cpu(), v[i, h], **tol)
        if taps > 1:
            rows = torch.cat([before[s], u[t0:t0 + n]])[-(taps - 1):]
            torch.testing.assert_close(state[s].double().cpu(), rows, atol=1e-5, rtol=1e-5)
    assert int(torch.isfinite(pages.float()).sum()) == T * nkv * (d + dv)       # nothing else was written


@gpu
@pytest.mark.parametrize("H,Sy,Sg,cast", [(7, 1, 1, None), (192, 3, 2, torch.bfloat16), (1500, 1, 4, torch.float32), (13000, 2, 0, None)])
def test_gate_norm_and_add(H, Sy, Sg, cast):
    from vllm_cpp_b200 import ops
    g = torch.Generator().manual_seed(H)
    T, eps = 6, 1e-5
    resid = torch.randn(T + 1, H, generator=g, dtype=torch.float64).float()
    y = torch.randn(Sy, T + 1, H, generator=g, dtype=torch.float64).float()
    wide = torch.randn(max(Sg, 1), T + 1, H + 24, generator=g, dtype=torch.float64).float()      # the gate's sums: columns 24.. of a wider product
    gb, w = torch.randn(H, generator=g).float(), torch.randn(H, generator=g).float()
    r_dev = resid.to(dev())
    out_cast = torch.full((T + 1, H), 3.0, device=dev(), dtype=cast) if cast else None
    gate = wide.to(dev())[:, :, 24:] if Sg else None
    # the last row belongs to no entry
    ops.gated_norm_add(r_dev, y.to(dev()) if Sy > 1 else y.to(dev())[0], gate if Sg != 1 else gate[0], gb.to(dev()), w.to(dev()),
                       eps, i32([0, 2, 2]), i32([2, 0, 4]), 3, out_cast=out_cast)
    v = y.double().sum(0)
    if Sg:
        v = v * torch.sigmoid(wide.double().sum(0)[:, 24:] + gb.double())
    want = resid.double() + P.rms_norm(v, w.double(), eps)
    torch.testing.assert_close(r_dev.double().cpu()[:T], want[:T], atol=2e-5, rtol=2e-5)
    assert torch.equal(r_dev.cpu()[T], resid[T])
    if cast:
        torch.testing.assert_close(out_cast[:T].double().cpu(), want[:T].to(cast).double(), atol=1e-2 if cast == torch.bfloat16 else 2e-5, rtol=1e-2)
        assert (out_cast[T] == 3.0).all()


@gpu
@pytest.mark.parametrize("kind", ["gelu_erf", "gelu_tanh", "silu"])
def test_activation_of_partial_sums(kind):
    from vllm_cpp_b200 import ops
    x = torch.randn(3, 5, 77, dtype=torch.float64).float() * 3
    out = torch.empty(5, 77, device=dev())
    ops.bias_act(x.to(dev()), out, kind)
    z = x.double().sum(0)
    want = {"gelu_erf": P.gelu_erf(z), "silu": z * torch.sigmoid(z),
            "gelu_tanh": 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))}[kind]
    torch.testing.assert_close(out.double().cpu(), want, atol=2e-6, rtol=2e-6)


def run_window_attention(dtype, nh, nkv, d, dv, ps, window, keep, shapes, craft=None, penalty=True, scale=0.3):
    """Runs the plain kernel, and the tensor-core kernel too (with TMA tile loads, with cp.async loads, and with a
    token's key slices merged within a cluster) where it takes the type and the head sizes."""
    from vllm_cpp_b200 import ops
    plan = _run_window_attention(dtype, nh, nkv, d, dv, ps, window, keep, shapes, craft, penalty, scale, "plain")
    if d == dv and ops.attn_mma_supported(dtype, d):
        for kernel in ("mma", "mma_no_tma", "mma_cluster"):
            plan = _run_window_attention(dtype, nh, nkv, d, dv, ps, window, keep, shapes, craft, penalty, scale, kernel)
        if ops.attn_tc_supported(dtype, d, ps):
            plan = _run_window_attention(dtype, nh, nkv, d, dv, ps, window, keep, shapes, craft, penalty, scale, "tc")   # tcgen05 for the prompt portions
    return plan


def _run_window_attention(dtype, nh, nkv, d, dv, ps, window, keep, shapes, craft, penalty, scale, kernel):
    """shapes: [(tokens cached before the step, query tokens of the step)]; compares the kernel (decoded tokens with
    sliced key ranges, prompt portions in query tiles) with the plain attention of one head at a time."""
    from vllm_cpp_b200 import ops
    from vllm_cpp_b200.parts import attention as A
    mma = kernel != "plain"
    DEC, SPAN = (A.MMA_DECODE_ROWS, A.MMA_SPAN_ROWS) if mma else (A.DECODE_ROWS, A.SPAN_ROWS)
    g = torch.Generator().manual_seed(5)
    a = (0.05 + torch.rand(nh, generator=g, dtype=torch.float64) * 2).float() if penalty else None
    b = (0.05 + torch.rand(nh, generator=g, dtype=torch.float64) * 0.3).float() if penalty else None
    num_pages = sum(-(-(s + n) // ps) for s, n in shapes) + 3
    perm = torch.randperm(num_pages, generator=g).tolist()
    same = d == dv
    pages = (torch.full((num_pages, 2, nkv, ps, d), float("nan"), device=dev(), dtype=dtype) if same else flat_pages(num_pages, nkv, ps, d, dv, dtype))
    host = pages.cpu()
    seqs, qs, tables = [], [], []
    for start, n in shapes:
        k = P.unit_rms(torch.randn(start + n, nkv, d, generator=g, dtype=torch.float64), 1e-6)
        v = torch.randn(start + n, nkv, dv, generator=g, dtype=torch.float64)
        q = P.unit_rms(torch.randn(n, nh, d, generator=g, dtype=torch.float64), 1e-6)
        if craft:
            craft(q, k, v, start, n)
        k, v, q = k.to(dtype).double(), v.to(dtype).double(), q.to(dtype).double()
        tab = [perm.pop() for _ in range(-(-(start + n) // ps))]
        first_needed = max(0, start - window + 1) if window else 0
        for p in range(start + n):
            if window and (p // ps + 1) * ps <= first_needed and p // ps >= -(-keep // ps):
                continue                       # a page the window has passed: given back, left unwritten
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
    plan = A.AttentionPlan(ctx, nh, nkv, DEC, SPAN, d if kernel == "mma_cluster" else None, max_keys=(window + keep) if window else 0)
    E, T = len(shapes), sum(ctx.host_q_len)
    bt = torch.full((E, max(len(t) for t in tables)), -1, dtype=torch.int32)
    for i, t in enumerate(tables):
        bt[i, :len(t)] = torch.tensor(t)
    out = torch.full((T, nh * dv), float("nan"), device=dev(), dtype=dtype)
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    q_flat = torch.cat(qs).to(dtype).to(dev()).view(T, nh * d)
    args = (pages, bt.to(dev()), i32(ctx.host_q_start), i32(ctx.host_q_len), i32(ctx.host_ctx_len))
    opts = dict(scale=scale, keep_first=keep, dist_a=None if a is None else a.to(dev()), dist_b=None if b is None else b.to(dev()))
    if mma:
        run = lambda *x, **k: ops.attn_mma(*x, allow_tma=kernel != "mma_no_tma", **k, **opts)
    else:
        run = lambda *x, **k: ops.attn_window_bias(*x, hd_v=dv, **opts)
    if plan.n_dec:
        S = plan.nslices
        cluster = plan.cluster if kernel == "mma_cluster" else 0
        po = torch.empty(plan.n_dec * nh * S, dv, device=dev()) if S > 1 and not cluster else None
        pm = torch.empty(plan.n_dec * nh * S, 2, device=dev()) if S > 1 and not cluster else None
        run(q_flat, out, *args, plan.dec_items, plan.n_dec * S, DEC, po, pm, nh, nkv, d, window, status,
            slice_counters=plan.slice_counters if S > 1 else None, dec_rows=plan.dec_rows, cluster=cluster)
        if S > 1 and not mma:
            ops.attn_merge(po, pm, plan.dec_rows, out, plan.n_dec, nh, dv, S)
    if plan.n_span_items and kernel == "tc":
        ops.attn_tc(q_flat, out, *args, plan.span_items, plan.n_span_items, nh, nkv, d, window, status, **opts)
    elif plan.n_span_items:
        run(q_flat, out, *args, plan.span_items, plan.n_span_items, SPAN, None, None, nh, nkv, d, window, status)
    torch.cuda.synchronize()
    assert status.item() == 0
    got = out.double().cpu().view(T, nh, dv)
    tol = dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    t = 0
    for (start, n), q, (k, v) in zip(shapes, qs, seqs):
        for h in range(nh):
            kv = h // (nh // nkv)
            want = P.attend_head(q[:, h], k[:, kv], v[:, kv], scale, float(a[h]) if penalty else 0.0, float(b[h]) if penalty else 0.0,
                                 window or None, keep)
            torch.testing.assert_close(got[t:t + n, h], want, **tol)
        t += n
    return plan


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,d,dv,ps", [(4, 2, 16, 24, 4), (3, 3, 20, 12, 8), (8, 2, 64, 64, 16), (2, 1, 128, 32, 16), (40, 1, 8, 256, 5),
                                            (4, 1, 128, 128, 8), (6, 3, 64, 64, 5), (8, 2, 128, 128, 64), (4, 4, 64, 64, 32)])
def test_window_attention_mixed_batch(dtype, nh, nkv, d, dv, ps):
    """Decoded tokens beside prompt portions: at the very start, before the window is full, far beyond it."""
    shapes = [(0, 1), (0, 7), (3, 1), (11, 1), (30, 2), (64, 33), (300, 1), (250, 70), (1, 2)]
    run_window_attention(dtype, nh, nkv, d, dv, ps, 37, 5, shapes)
    run_window_attention(dtype, nh, nkv, d, dv, ps, 0, 0, shapes[:6])                 # no window: every key
    run_window_attention(dtype, nh, nkv, d, dv, ps, 16, 0, shapes, penalty=False)     # a bare window


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("which", ["kept_last", "first_not_kept", "window_first", "before_window", "position_0"])
@pytest.mark.parametrize("d,dv,ps", [(24, 40, 8), (64, 64, 16), (128, 128, 32)])
def test_one_key_stands_out_at_every_edge(dtype, which, d, dv, ps):
    """A key whose score dominates: the last kept first key and the window's first key must count, the first key that is
    not kept and the key just before the window must not, for a decoded token and inside a prompt portion."""
    W, keep = 37, 5
    for start, n in ((299, 1), (280, 20), (1000, 1)):
        last = start + n - 1
        j = {"kept_last": keep - 1, "first_not_kept": keep, "window_first": last - W + 1, "before_window": last - W, "position_0": 0}[which]

        def craft(q, k, v, s, m):
            k[j] = q[-1, 0] * 1.0          # cosine 1 with the last query's first head
            v[j] = 50.0
        run_window_attention(dtype, 2, 2, d, dv, ps, W, keep, [(start, n)], craft, scale=40.0 / d)


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_many_kept_first_keys_and_long_windows(dtype):
    """More kept first keys than one key tile holds, before a window of several tiles; a window of two keys."""
    shapes = [(2000, 1), (1500, 140), (100, 1), (60, 30), (0, 300)]
    run_window_attention(dtype, 4, 2, 64, 64, 16, 300, 150, shapes)
    run_window_attention(dtype, 4, 4, 128, 128, 16, 2, 1, shapes[1:4])
    run_window_attention(dtype, 2, 1, 64, 64, 8, 1, 70, shapes[2:4])


@gpu
def test_long_contexts_are_sliced_only_as_far_as_the_window_reaches():
    plan = run_window_attention(torch.float32, 8, 2, 64, 64, 16, 0, 0, [(3000, 1), (1025, 1)])
    assert plan.nslices > 1
    plan = run_window_attention(torch.float32, 8, 2, 64, 64, 16, 700, 9, [(3000, 1), (1025, 1)])
    assert 1 < plan.nslices <= 5
    plan = run_window_attention(torch.float32, 8, 2, 64, 64, 16, 100, 9, [(3000, 1), (1025, 1)])
    assert plan.nslices == 1


# -------------------------------------------------------------------------- whole models through the trace runner


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
@pytest.mark.parametrize("name", ["P", "Q", "S"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "portions_last", "mixed", "mixed_last"])
def test_replay(name, dtype, mode, rimopel_dirs, oracle, tmp_path):
    """Whole prompts; the last 32 tokens one by one (the windows pass over decoded tokens); portions of changing size
    down to two tokens; up to four live requests with pages and slots used again -- the last two also as serving asks
    (logits of an entry's last token only: captured steps), all over a NaN-filled cache."""
    requests = requests_of(name)
    trace = {"whole": R.whole, "tail": R.tail_one_by_one, "portions": R.portions, "portions_last": R.portions_last,
             "mixed": R.mixed, "mixed_last": R.mixed_last}[mode](requests)
    out = R.run_trace(rimopel_dirs[name], dtype, trace, tmp_path / "out", configs()[name][1], extra_args=["--poison"])
    worst = compare(name, dtype, trace, out, requests, oracle)
    print(f"{name} {dtype} {mode}: worst relative error {worst:.3e}, pool {trace.max_tokens} tokens, {len(trace.steps)} steps")


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["U", "V"])
@pytest.mark.parametrize("mode", ["tail", "mixed", "mixed_last"])
def test_replay_of_awkward_sizes(name, dtype, mode, rimopel_dirs, oracle, tmp_path):
    requests = requests_of(name)
    trace = {"tail": R.tail_one_by_one, "mixed": R.mixed, "mixed_last": R.mixed_last}[mode](requests)
    out = R.run_trace(rimopel_dirs[name], dtype, trace, tmp_path / "out", configs()[name][1], extra_args=["--poison"])
    compare(name, dtype, trace, out, requests, oracle)


@gpu
def test_replay_modes_agree_with_each_other(rimopel_dirs, tmp_path):
    """Cutting and batching change the logits by rounding only."""
    name = "P"
    requests = requests_of(name)
    vocab = configs()[name][0].vocab
    rows = {}
    for mode, build in (("whole", R.whole), ("mixed", R.mixed), ("portions", R.portions)):
        trace = build(requests)
        out = R.run_trace(rimopel_dirs[name], "float32", trace, tmp_path / mode, configs()[name][1])
        for step, want in enumerate(trace.wanted):
            got = R.read_step(out, step, vocab)
            for i, key in enumerate(want):
                rows.setdefault(key, {})[mode] = got[i]
    worst = max(np.abs(v["whole"] - v[m]).max() / np.abs(v["whole"]).max() for v in rows.values() for m in ("mixed", "portions"))
    assert worst < 1e-5, worst


@gpu
def test_long_decoding_far_past_every_window(rimopel_dirs, oracle, tmp_path):
    """A short prompt, then 250 tokens one by one: windows, kept first keys and given-back pages in steady state."""
    name = "P"
    toks = random_tokens(configs()[name][0].vocab, 260, 99)
    trace = R.tail_one_by_one({"long": toks}, tail=250)
    out = R.run_trace(rimopel_dirs[name], "float32", trace, tmp_path / "out", configs()[name][1], extra_args=["--poison"])
    compare(name, "float32", trace, out, {"long": toks}, oracle)


# -------------------------------------------------------------------------- generation through the engine's entry point


@gpu
@pytest.mark.parametrize("name", ["P", "S"])
def test_greedy_generation_through_the_scheduler(name, rimopel_dirs):
    """Several prompts at once through LLM.generate (scheduler, portions under a small token budget, captured decoding
    steps, device-side sampling at temperature 0) against the plain implementation's greedy continuation."""
    from vllm_cpp_b200 import LLM
    cfg, w = P.read_model(rimopel_dirs[name])
    vocab, page = configs()[name][0].vocab, configs()[name][1]
    prompts = [random_tokens(vocab, n, 3 + n) for n in (5, 41, 18, 70, 2)]
    llm = LLM(str(rimopel_dirs[name]), dtype="float32", page_size=page, max_tokens=page * 64, max_num_seqs=3, max_step_tokens=32,
              max_model_len=512)
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
