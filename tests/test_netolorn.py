"""Netolorn (squashing norms on both sides of every sublayer; grouped-query attention with a partial rotation, unit-RMS queries
and keys, a sliding window that keeps the first tokens and a sink; latent attention without positions over a window; dense and
routed clamped feed-forwards; a per-layer token input; looped layer ranges entered through a projection of stream and embedding)
through the framework's own entry points (Context, TextModelBase, Sessions, Master) against the plain restatement in
oracle/netolorn_plain.py, on small configurations made here with random weights.

What a schedule must not change: the logits at a position are the same whether the prompt went in whole, token by token or in
portions, whatever ran before in the same cache slot, and whatever other request is interleaved.  fp32 (D = float) is the sharp
comparison: the GPU and the plain code differ by summation order only.  The error of a position is the root mean square over
the vocabulary of the difference (mean removed) over the spread of the expected logits.  Where random weights would hide a
fault (a key at a window's edge, a kept first token, the sink, a far key) the test first shows that the plain model with that
fault differs by many tolerances, then that the framework agrees with the right one.
"""
import copy
import json

import numpy as np
import pytest
import torch

from cake_b200.config import Config
from cake_b200.synth import make_netolorn_checkpoint
from oracle import netolorn_plain as P

TOL = {"f32": 2e-4, "bf16": 1e-1, "f16": 2e-2}   # bf16 at widths of a few dozen: every projection is rounded to 8 bits
YARN = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}


def dense(ff=24):
    return {"kind": "dense", "ff": ff}


def moe(experts=5, top=2, ff=12, limit=1.0, shared=16, shared_limit=2.0):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit},
            "shared": {"ff": shared, "limit": shared_limit} if shared else None}


def attn(heads=4, kv_heads=2, dim=12, vdim=10, size=7, keep=2, scale=0.4, rot=8, base=100.0, scaling=YARN, mlp="dense"):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
         "mask": {"size": size, "keep_first": keep} if size else None,
         "rot": ({"dims": rot, "base": base, "scaling": dict(scaling)} if scaling else {"dims": rot, "base": base}) if rot else None}
    return {"type": "attention", "mixer": m, "mlp": dense() if mlp == "dense" else mlp}


def latent(heads=3, dim=8, vdim=6, q_rank=10, kv_rank=14, size=9, scale=0.5, mlp="moe"):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale, "mask": {"size": size} if size else None}
    return {"type": "latent_attention", "mixer": m, "mlp": moe() if mlp == "moe" else mlp}


def make_config(layers, loop=None, width=40, vocab=53, eps=1e-5, side=5) -> Config:
    d = {"architecture": "Netolorn", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": layers}
    if side:
        d["token_side"] = {"dim": side}
    if loop:
        d["loop"] = loop
    return Config.from_hf(json.loads(json.dumps(d)))


def full_config(**kw) -> Config:
    """Every mechanism, unequal sizes, a loop over the middle layers, one layer without a feed-forward."""
    layers = [attn(), latent(), attn(heads=6, kv_heads=6, dim=8, vdim=8, size=12, keep=0, rot=4, scaling=None, mlp=moe(experts=3, top=1, shared=0)),
              latent(heads=2, dim=16, vdim=12, q_rank=6, kv_rank=20, size=0, mlp=None)]
    return make_config(layers, loop={"start": 1, "stop": 3, "times": 2}, **kw)


def tokens(n, vocab, seed=0):
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


def errors(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    assert np.isfinite(got).all()
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    return np.sqrt((d * d).mean(-1)) / max(float(want.std()), 1e-3)


def close(got, want, dtype, what="", bar=None):
    e = errors(got, want)
    if dtype == "f32":
        assert e.max() < TOL[dtype], f"{what}: worst {e.max():.3g} at position {int(e.argmax())}"
    else:   # a router's close call may flip under 16-bit rounding
        bar = bar or TOL[dtype]
        assert np.quantile(e, 0.95) < bar and e.max() < 6 * bar, f"{what}: 95 % within {np.quantile(e, 0.95):.3g}, worst {e.max():.3g} (bar {bar:.3g})"


def plain(cfg, sd, toks, streams=None, d=None):
    wt = {k: v.float() for k, v in sd.items()}
    return P.forward(toks, wt, d or cfg.to_hf(), torch.float32, streams).numpy()


def plain_with_rounded_products(cfg, sd, toks, to=torch.bfloat16):
    """The plain model with the input and the result of every matrix product rounded to 16 bits: how far that rounding alone
    moves the logits of a configuration (a router's close call, a sharp softmax), which is the bar a 16-bit run is held to."""
    exact = P.lin
    P.lin = lambda W, x, b=None: exact(W, x.to(to).float(), b).to(to).float()
    try:
        return plain(cfg, sd, toks)
    finally:
        P.lin = exact


class Runner:
    """The framework side: a model on the GPU and its Sessions."""

    def __init__(self, cfg, sd, dtype, max_seq=None):
        from cake_b200.model import Context, Sessions, TextModelBase
        self.ctx = Context(cfg, sd, dtype, device=0, max_seq=max_seq or cfg.max_seq_len)
        self.model = TextModelBase.load(self.ctx)
        self.ses = Sessions(self.model, max_seq or cfg.max_seq_len)

    def run(self, rid, toks, cuts=None, end=True):
        """Feed ``toks`` as request ``rid`` in portions of the sizes ``cuts`` (cycled; None = whole) -> logits of every position."""
        out, p, i = [], 0, 0
        while p < len(toks):
            n = len(toks) - p if not cuts else min(cuts[i % len(cuts)], len(toks) - p)
            lg = self.ses.step(rid, toks[p:p + n], want=list(range(n)))
            self.ctx.sync()
            out.append(lg.cpu().numpy())
            p, i = p + n, i + 1
        if end:
            self.ses.end(rid)
        return np.concatenate(out, 0)

    def close(self):
        self.ctx.close()


# ---------------------------------------------------------------------------------------------- no GPU needed
def test_config_round_trip_and_run_order():
    cfg = full_config()
    d = cfg.to_hf()
    assert d["architecture"] == "Netolorn" and len(d["layers"]) == 4 and d["layers"][3]["mlp"] is None and d["token_side"] == {"dim": 5}
    back = Config.from_hf(json.loads(json.dumps(d)))
    assert back.layers == cfg.layers and back.loop == cfg.loop
    assert back.layer_list and back.block_kind == "netolorn" and back.loop_mode == "project" and back.final_norm_kind == 1
    assert [i for i, _ in cfg.run_plan()] == [0, 1, 2, 1, 2, 3] == [i for i, _ in P.run_order(d)]
    assert [t for _, t in cfg.run_plan()] == [None, 0, None, 1, None, None]     # the first pass is entered through the projection too
    a, b = back.layers[0], back.layers[1]
    assert a.type == "sink_attention" and (a.window, a.keep_first, a.qk_unit, a.norm_kind, a.side_dim, a.side_col) == (7, 2, True, 1, 5, 0)
    assert a.rot.dims == 8 and a.rot.factor == 4.0 and a.dense_ff == 24 and a.dense_act == 0
    assert b.type == "latent_window" and (b.q_rank, b.kv_rank, b.window, b.side_col) == (10, 14, 9, 5)
    assert b.moe.logit_bias and b.moe.act == 2 and (b.moe.limit, b.moe.shared_limit, b.moe.shared_ff) == (1.0, 2.0, 16)
    assert back.layers[2].rot.factor == 0.0 and back.layers[2].moe.shared_ff == 0 and back.layers[3].window == 0
    for path, value in ((("layers", 0, "type"), "retention"), (("layers", 0, "mixer", "kv_heads"), 3), (("loop", "stop"), 9),
                        (("layers", 0, "mixer", "rot", "dims"), 14), (("layers", 1, "mlp", "kind"), "other")):
        bad = json.loads(json.dumps(d))
        node = bad
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(ValueError):
            Config.from_hf(bad)
    plainer = Config.from_hf({"architecture": "Netolorn", "width": 8, "vocab": 9, "norm": {"eps": 1e-6},
                              "layers": [{"type": "attention", "mixer": {"heads": 2, "dim": 4, "vdim": 4, "scale": 0.5}, "mlp": None}]})
    sp = plainer.layers[0]
    assert (sp.n_kv, sp.window, sp.keep_first, sp.rot.dims, sp.side_dim) == (2, 0, 0, 0, 0) and plainer.loop is None and not plainer.token_side_dim


def test_checkpoint_names_and_shapes():
    from cake_b200.loader import netolorn_block_tensors
    cfg = full_config()
    sd = make_netolorn_checkpoint(cfg, "bf16", seed=1)
    assert sd["loop.in"].shape == (40, 80) and sd["side.embed"].shape == (53, 20) and sd["final.norm.alpha"].shape == ()
    t0, t1 = netolorn_block_tensors(sd, cfg, 0), netolorn_block_tensors(sd, cfg, 1)
    assert t0["q"].shape == (48, 40) and t0["k_b"].shape == (24,) and t0["v"].shape == (20, 40) and t0["sink"].shape == (4,) and t0["g"].shape == (40, 40)
    assert t1["dq"].shape == (10, 40) and t1["uq"].shape == (24, 10) and t1["uk"].shape == (24, 14) and t1["uv"].shape == (18, 14) and t1["g"].shape == (3, 40)
    assert len(t1["e_gate"]) == 5 and t1["correction"].shape == (5,) and t1["s_sg"].shape == (1, 40) and t1["side_proj"].shape == (40, 5)
    assert cfg.layers[1].norm_alpha == [float(sd[f"l1.{n}.alpha"].float()) for n in ("norm1", "norm1b", "norm2", "norm2b")]
    assert "norm2" not in netolorn_block_tensors(sd, cfg, 3)
    bad = dict(sd)
    bad["l0.mix.sink"] = sd["l0.mix.sink"][:3]
    with pytest.raises(ValueError):
        netolorn_block_tensors(bad, cfg, 0)
    del bad["l1.mix.dq.norm"]
    with pytest.raises(KeyError):
        netolorn_block_tensors(bad, cfg, 1)


def test_plain_window_and_kept_tokens():
    v = P.visible(9, 3, 2)
    assert v[8].tolist() == [True, True, False, False, False, False, True, True, True]
    assert v[2].tolist() == [True, True, True] + [False] * 6 and v[3].tolist() == [True, True, True, True] + [False] * 5
    assert P.visible(5, 0, 0).tolist() == torch.tril(torch.ones(5, 5, dtype=torch.bool)).tolist()


def test_plain_rotation_tables():
    rot = {"dims": 8, "base": 100.0}
    c, s = P.rotary_tables(rot, [0, 3], torch.float64)
    f = [100.0 ** (-2 * i / 8) for i in range(4)]
    assert torch.allclose(c[1], torch.cos(3 * torch.tensor(f, dtype=torch.float64))) and torch.allclose(s[0], torch.zeros(4, dtype=torch.float64))
    c2, s2 = P.rotary_tables(dict(rot, scaling=YARN), [0, 3], torch.float64)
    amp = 0.1 * np.log(4.0) + 1.0
    assert abs(float(c2[0, 0]) - amp) < 1e-12                                   # both tables carry the amplitude
    assert abs(float(s2[1, 0]) - amp * np.sin(3 * f[0])) < 1e-12                # the fastest pair keeps its frequency
    assert abs(float(s2[1, 3]) - amp * np.sin(3 * f[3] / 4.0)) < 1e-12          # the slowest is divided by the factor
    x = torch.randn(2, 1, 12, dtype=torch.float64)
    y = P.rotate(x, c, s)
    assert torch.allclose(y[..., 8:], x[..., 8:]) and torch.allclose(y[0], x[0])
    assert torch.allclose((y[1, 0, :8] ** 2).sum(), (x[1, 0, :8] ** 2).sum())


def test_plain_sink_takes_weight_and_router_weights_sum_to_one():
    cfg = make_config([attn(size=0, keep=0)], side=0)
    sd = {k: v.float() for k, v in make_netolorn_checkpoint(cfg, "f32", seed=3).items()}
    h = torch.randn(6, 40)
    m = cfg.to_hf()["layers"][0]["mixer"]
    lo, hi = dict(sd), dict(sd)
    lo["l0.mix.sink"] = torch.full((4,), -40.0)
    hi["l0.mix.sink"] = torch.full((4,), 40.0)
    a, b = P.sink_attention(h, lo, "l0.mix.", m, 1e-5), P.sink_attention(h, hi, "l0.mix.", m, 1e-5)
    assert a.abs().max() > 1e-3 and b.abs().max() < 1e-12 * a.abs().max() + 1e-9   # a huge sink takes all the weight, and it has no value
    mlp = moe(experts=4, top=4, shared=0)
    c2 = make_config([latent(mlp=mlp)], side=0)
    s2 = {k: v.float() for k, v in make_netolorn_checkpoint(c2, "f32", seed=4).items()}
    one = P.routed_ff(h, s2, "l0.mlp.", mlp)
    want = sum(torch.softmax(P.lin(s2["l0.mlp.router"], h, s2["l0.mlp.router.b"]), -1)[:, e:e + 1] * P.clamped_expert(h, s2, f"l0.mlp.e{e}.", 1.0) for e in range(4))
    assert torch.allclose(one, want, atol=1e-5)


# ---------------------------------------------------------------------------------------------- GPU
MECHANISMS = {
    "attention_plain": [attn(size=0, keep=0, rot=0, mlp=None)],
    "attention_window": [attn(size=5, keep=0, rot=0, mlp=None)],
    "attention_window_kept": [attn(size=5, keep=3, rot=0, mlp=None)],
    "attention_kept_beyond_window": [attn(size=3, keep=9, rot=0, mlp=None)],
    "attention_window_one": [attn(size=1, keep=1, mlp=None)],
    "attention_full_rotation": [attn(dim=12, rot=12, scaling=None, mlp=None)],
    "attention_blend": [attn(dim=16, rot=16, base=50.0, scaling={"factor": 8.0, "original": 32, "fast": 4.0, "slow": 0.5}, mlp=None)],
    "attention_every_head_its_keys": [attn(heads=3, kv_heads=3, mlp=None)],
    "attention_one_key_head": [attn(heads=5, kv_heads=1, dim=20, vdim=36, rot=6, mlp=None)],
    "attention_wide_heads": [attn(heads=2, kv_heads=1, dim=72, vdim=136, rot=40, mlp=None)],
    "latent_plain": [latent(size=0, mlp=None)],
    "latent_window": [latent(size=4, mlp=None)],
    "latent_one_head": [latent(heads=1, dim=24, vdim=20, q_rank=5, kv_rank=40, mlp=None)],
    "latent_wide": [latent(heads=2, dim=16, vdim=8, q_rank=48, kv_rank=200, size=11, mlp=None)],
    "dense": [attn(size=0, keep=0, rot=0, mlp=dense(56))],
    "experts": [latent(mlp=moe())],
    "experts_top_one_no_shared": [latent(mlp=moe(experts=4, top=1, shared=0))],
    "experts_all_chosen": [latent(mlp=moe(experts=3, top=3, limit=0.3, shared_limit=0.2))],
    "experts_one_expert": [latent(mlp=moe(experts=1, top=1, ff=20))],
    "experts_many": [attn(mlp=moe(experts=40, top=5, ff=8, shared=8))],
}
LOOPS = {"loop_from_the_start": {"start": 0, "stop": 2, "times": 3}, "loop_of_one_pass": {"start": 1, "stop": 2, "times": 1},
         "loop_over_the_tail": {"start": 1, "stop": 3, "times": 2}}


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(MECHANISMS) + sorted(LOOPS) + ["no_token_input", "token_input_of_one"])
def test_each_mechanism_alone(name):
    if name in MECHANISMS:
        cfg = make_config(MECHANISMS[name], side=0)
    elif name in LOOPS:
        cfg = make_config([attn(), latent(), attn(kv_heads=4, size=0, keep=0)], loop=LOOPS[name], side=3)
    else:
        cfg = make_config([attn(), latent()], side=0 if name == "no_token_input" else 1)
    sd = make_netolorn_checkpoint(cfg, "f32", seed=sum(map(ord, name)) % 1000)
    toks = tokens(37, cfg.vocab_size, seed=3)
    want = plain(cfg, sd, toks)
    r = Runner(cfg, sd, "f32")
    try:
        close(r.run("a", toks), want, "f32", "whole")
        close(r.run("b", toks, cuts=[1]), want, "f32", "token by token")
        close(r.run("c", toks, cuts=[2, 5, 3]), want, "f32", "portions")
    finally:
        r.close()


@pytest.mark.gpu
def test_residual_after_every_layer_run():
    from cake_b200.capi import check, lib, ptr
    import ctypes
    cfg = full_config()
    sd = make_netolorn_checkpoint(cfg, "f32", seed=5)
    toks = tokens(29, cfg.vocab_size, seed=4)
    streams = []
    plain(cfg, sd, toks, streams)
    r = Runner(cfg, sd, "f32")
    try:
        ctx, model = r.ctx, r.model
        for lo, hi in ((0, 17), (17, 29)):     # two portions: the second reads cache rows of the first in every run
            ids = np.ascontiguousarray([toks[lo:hi]], dtype=np.uint32)
            x0 = ctx.empty(1, hi - lo, cfg.hidden_size, dtype=torch.float32)
            check(lib().cake_b200_embed(ctx.h, ids.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32)), 1, hi - lo, ptr(x0)))
            with torch.cuda.stream(ctx.torch_stream):
                x = x0.clone()
            for j, blk in enumerate(model.blocks):
                if j in model.injections:
                    check(lib().cake_b200_stream_project(ctx.h, ptr(x), ptr(x0), ptr(model.loop_in), hi - lo))
                x = blk.forward_batch(x, [(blk.layer_name(), lo, j)], ctx, blocks=[blk])
                ctx.sync()
                want = streams[j][lo:hi].numpy()
                assert np.abs(x[0].cpu().numpy() - want).max() < 2e-4 * max(1.0, np.abs(want).max()), f"run {j}, tokens {lo}..{hi}"
        assert len(model.blocks) == len(streams) == 6
    finally:
        r.close()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
def test_schedules_agree_with_the_plain_model(dtype):
    cfg = full_config()
    sd = make_netolorn_checkpoint(cfg, dtype, seed=11)
    toks = tokens(83, cfg.vocab_size, seed=5)
    want = plain(cfg, sd, toks)
    r = Runner(cfg, sd, dtype)
    try:
        whole = r.run("w", toks)
        close(whole, want, dtype, "whole")
        for cuts in ([1], [2], [2, 3, 5], [17], [64, 1], [1, 40, 2]):
            got = r.run("c", toks, cuts=cuts)
            close(got, want, dtype, f"portions {cuts}")
            if dtype == "f32":
                assert errors(got, whole).max() < TOL["f32"], f"portions {cuts} against whole"
        close(r.run("one", toks[:1]), want[:1], dtype, "a sequence of one token")
        close(r.run("few", toks[:3], cuts=[1]), want[:3], dtype, "the first tokens")
    finally:
        r.close()


@pytest.mark.gpu
def test_interleaved_requests_and_reused_slots():
    cfg = full_config()
    sd = make_netolorn_checkpoint(cfg, "f32", seed=21)
    a, b, c = tokens(50, cfg.vocab_size, seed=6), tokens(31, cfg.vocab_size, seed=7), tokens(64, cfg.vocab_size, seed=8)
    wa, wb, wc = plain(cfg, sd, a), plain(cfg, sd, b), plain(cfg, sd, c)
    r = Runner(cfg, sd, "f32")
    try:
        ga, gb, pa, pb = [], [], 0, 0
        for na, nb in ((7, 3), (1, 1), (20, 9), (2, 18), (20, 0)):      # two unequal requests, step by step in turns
            if na:
                ga.append(r.ses.step("a", a[pa:pa + na], want=list(range(na))).cpu().numpy())
                pa += na
            if nb:
                gb.append(r.ses.step("b", b[pb:pb + nb], want=list(range(nb))).cpu().numpy())
                pb += nb
        r.ses.end("a")
        r.ses.end("b")
        close(np.concatenate(ga), wa, "f32", "request a beside b")
        close(np.concatenate(gb), wb, "f32", "request b beside a")
        assert len(r.ses.free) == 2
        close(r.run("c", c, cuts=[9, 1]), wc, "f32", "a longer request in a used slot")    # rows and windows of the old request lie beyond
        close(r.run("d", b, cuts=[4]), wb, "f32", "a shorter request in a used slot")
        close(r.run("e", a), wa, "f32", "whole in a used slot")
        assert len(r.ses.free) == 2 and not r.ses.live
    finally:
        r.close()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_batch_rows_against_each_alone(dtype):
    from cake_b200.model import Cache
    cfg = full_config()
    sd = make_netolorn_checkpoint(cfg, dtype, seed=31)
    rows = [tokens(40, cfg.vocab_size, seed=20 + i) for i in range(3)]
    want = [plain(cfg, sd, t) for t in rows]
    r = Runner(cfg, sd, dtype)
    try:
        r.ctx.cache = Cache(r.ctx, 3, 64)
        got, p = [], 0
        for n in (23, 1, 1, 15):
            lg = r.model.forward(np.array([t[p:p + n] for t in rows], dtype=np.uint32), p, want=list(range(3 * n)))
            r.ctx.sync()
            got.append(lg.cpu().numpy().reshape(3, n, -1))
            p += n
        got = np.concatenate(got, 1)
        for i in range(3):
            close(got[i], want[i], dtype, f"batch row {i}")
    finally:
        r.close()


def sharp(layer, scale):
    layer = copy.deepcopy(layer)
    layer["mixer"]["scale"] = scale
    return layer


def faulty(cfg, edit):
    d = cfg.to_hf()
    edit(d)
    return d


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["attention", "latent"])
def test_window_edges_kept_tokens_and_the_sink(kind):
    """Sharp scores, so that single keys carry a row.  A window one token longer or shorter, one kept token more or fewer, or no
    sink changes the plain model's logits by many tolerances; the framework agrees with the right one in a whole prompt, in
    portions cut at and around the window's size, and token by token (decoding past the window)."""
    if kind == "attention":
        layers = [sharp(attn(size=11, keep=3, scale=3.0, mlp=None), 3.0), sharp(attn(heads=2, kv_heads=1, size=6, keep=1, scale=2.5, rot=4), 2.5)]
    else:
        layers = [sharp(latent(size=11, mlp=None), 4.0), sharp(latent(heads=2, size=6, mlp=dense()), 4.0)]
    cfg = make_config(layers, side=0)
    sd = make_netolorn_checkpoint(cfg, "f32", seed=41)
    if kind == "latent":
        for i in (0, 1):
            sd[f"l{i}.mix.uk"] = sd[f"l{i}.mix.uk"] * 2.0
    toks = tokens(90, cfg.vocab_size, seed=9)
    want = plain(cfg, sd, toks)

    def window(dl, which):
        def edit(d):
            d["layers"][0]["mixer"]["mask"][which] += dl
        return edit
    faults = {"window + 1": window(1, "size"), "window - 1": window(-1, "size")}
    if kind == "attention":
        faults.update({"kept + 1": window(1, "keep_first"), "kept - 1": window(-1, "keep_first")})
    for what, edit in faults.items():
        e = errors(plain(cfg, sd, toks, d=faulty(cfg, edit)), want)
        assert e.max() > 50 * TOL["f32"], f"{what} would not show: {e.max():.3g}"
    if kind == "attention":
        nosink = dict(sd)
        nosink["l0.mix.sink"] = torch.full_like(sd["l0.mix.sink"], -60.0)
        assert errors(plain(cfg, nosink, toks), want).max() > 50 * TOL["f32"]
    r = Runner(cfg, sd, "f32")
    try:
        close(r.run("w", toks), want, "f32", "whole")
        for cuts in ([11], [10], [12], [6, 5], [1], [3, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1], [40, 2]):
            close(r.run("c", toks, cuts=cuts), want, "f32", f"portions {cuts}")
    finally:
        r.close()
    rb = Runner(cfg, {k: v.to(torch.bfloat16) for k, v in sd.items()}, "bf16")
    try:
        wb = plain(cfg, {k: v.to(torch.bfloat16) for k, v in sd.items()}, toks)
        close(rb.run("w", toks), wb, "bf16", "whole, bf16")
        close(rb.run("c", toks, cuts=[30, 1]), wb, "bf16", "decoded, bf16")
    finally:
        rb.close()


@pytest.mark.gpu
def test_key_size_128_portions_on_the_tensor_core_attention():
    """Key and value size 128 in 16-bit D: portions of 64 rows and more take the tensor-core attention (kept first keys ahead of the
    window's tiles, the sink in the denominator, a gate per element; the latent kind with keys and values expanded for the rows a
    step sees), shorter ones the other kernels.  Flat scores in f16, where rounding is small: a window or a kept range that is one
    off, or a missing sink, moves the plain model's logits by several bars at most positions."""
    layers = [sharp(attn(heads=4, kv_heads=2, dim=128, vdim=128, size=70, keep=5, rot=64, mlp=None), 0.2),
              sharp(latent(heads=2, dim=128, vdim=128, q_rank=64, kv_rank=64, size=90, mlp=None), 0.05),
              sharp(attn(heads=2, kv_heads=2, dim=128, vdim=128, size=0, keep=0, rot=32, scaling=None, mlp=dense(128)), 0.2),
              sharp(latent(heads=2, dim=128, vdim=128, q_rank=64, kv_rank=128, size=0, mlp=None), 0.05)]
    cfg = make_config(layers, width=128, vocab=96, side=0)
    sd = make_netolorn_checkpoint(cfg, "f16", seed=47)
    toks = tokens(400, cfg.vocab_size, seed=13)
    want = plain(cfg, sd, toks)
    bar = max(4 * float(np.quantile(errors(plain_with_rounded_products(cfg, sd, toks, torch.float16), want), 0.95)), 4e-3)

    def mask(layer, which, dl):
        def edit(d):
            d["layers"][layer]["mixer"]["mask"][which] += dl
        return edit
    faults = {"window + 1": mask(0, "size", 1), "window - 1": mask(0, "size", -1), "kept + 1": mask(0, "keep_first", 1), "kept - 1": mask(0, "keep_first", -1),
              "latent window + 1": mask(1, "size", 1), "latent window - 1": mask(1, "size", -1)}
    for what, edit in faults.items():
        e = errors(plain(cfg, sd, toks, d=faulty(cfg, edit))[200:], want[200:])
        assert np.quantile(e, 0.5) > 2 * bar, f"{what} would not show: {np.quantile(e, 0.5):.3g} against {bar:.3g}"
    nosink = dict(sd)
    nosink["l0.mix.sink"] = torch.full_like(sd["l0.mix.sink"], -60.0)
    assert np.quantile(errors(plain(cfg, nosink, toks), want), 0.5) > 2 * bar
    r = Runner(cfg, sd, "f16")
    try:
        whole = r.run("w", toks)
        close(whole, want, "f16", "whole", bar)
        for cuts in ([200, 130, 70], [64, 65, 128, 143], [37], [150, 1, 1, 1, 100, 2, 145]):
            got = r.run("c", toks, cuts=cuts)
            close(got, want, "f16", f"portions {cuts}", bar)
            close(got, whole, "f16", f"portions {cuts} against whole", bar)
        # two unequal batch rows in one call, in two portions (the second starts inside every window)
        from cake_b200.model import Cache
        rows = [toks[:300], tokens(300, cfg.vocab_size, seed=14)]
        wants = [want[:300], plain(cfg, sd, rows[1])]
        r.ctx.cache = Cache(r.ctx, 2, 320)
        got, at = [], 0
        for n in (200, 100):
            lg = r.model.forward(np.array([t[at:at + n] for t in rows], dtype=np.uint32), at, want=list(range(2 * n)))
            r.ctx.sync()
            got.append(lg.cpu().numpy().reshape(2, n, -1))
            at += n
        got = np.concatenate(got, 1)
        for i in range(2):
            close(got[i], wants[i], "f16", f"batch row {i}", bar)
    finally:
        r.close()


@pytest.mark.gpu
def test_far_keys_in_prompt_portions_and_decoding():
    """Attention without a window over 330 positions with sharp scores: hiding the keys beyond 100 positions changes the plain
    model's logits, so far keys matter; long rows take the split-key kernels when a step has few rows."""
    layers = [sharp(attn(heads=4, kv_heads=2, size=0, keep=0, mlp=None), 3.0), sharp(latent(size=0, mlp=None), 4.0),
              sharp(attn(heads=2, kv_heads=2, size=300, keep=4, mlp=None), 3.0)]
    cfg = make_config(layers, side=2)
    sd = make_netolorn_checkpoint(cfg, "f32", seed=43)
    sd["l1.mix.uk"] = sd["l1.mix.uk"] * 2.0
    toks = tokens(330, cfg.vocab_size, seed=10)
    want = plain(cfg, sd, toks)
    P.KEYS_VISIBLE = 100
    try:
        near = plain(cfg, sd, toks)
    finally:
        P.KEYS_VISIBLE = None
    assert errors(near[150:], want[150:]).max() > 50 * TOL["f32"]
    r = Runner(cfg, sd, "f32")
    try:
        close(r.run("w", toks), want, "f32", "whole")
        close(r.run("c", toks, cuts=[129, 127, 2, 1]), want, "f32", "portions")
        close(r.run("d", toks, cuts=[270] + [1] * 60), want, "f32", "decoded over 270 cached keys")
    finally:
        r.close()
    rb = Runner(cfg, {k: v.to(torch.bfloat16) for k, v in sd.items()}, "bf16")
    try:
        wb = plain(cfg, {k: v.to(torch.bfloat16) for k, v in sd.items()}, toks)
        close(rb.run("d", toks, cuts=[270] + [1] * 60), wb, "bf16", "decoded, bf16")
    finally:
        rb.close()


@pytest.mark.gpu
def test_long_decoding_past_every_window():
    cfg = full_config()
    sd = make_netolorn_checkpoint(cfg, "f32", seed=45)
    toks = tokens(230, cfg.vocab_size, seed=11)
    want = plain(cfg, sd, toks)
    r = Runner(cfg, sd, "f32")
    try:
        close(r.run("d", toks, cuts=[10] + [1] * 220), want, "f32", "a short prompt then long decoding")
    finally:
        r.close()


@pytest.mark.gpu
def test_other_sizes_and_tensor_core_shapes():
    """Sizes whose projections, experts and attention take the tensor-core kernels (multiples of 128 / 64 / 16) next to ones
    that do not; long portions and decoding; against the plain model and whole against portions."""
    layers = [attn(heads=4, kv_heads=2, dim=64, vdim=64, size=96, keep=5, scale=0.3, rot=32, base=1000.0, mlp=dense(128)),
              latent(heads=4, dim=32, vdim=32, q_rank=64, kv_rank=128, size=70, scale=0.3, mlp=moe(experts=6, top=2, ff=64, shared=64)),
              attn(heads=2, kv_heads=1, dim=128, vdim=128, size=0, keep=0, scale=0.2, rot=64, scaling=None, mlp=moe(experts=4, top=2, ff=128, shared=0)),
              attn(heads=3, kv_heads=3, dim=24, vdim=40, size=33, keep=2, rot=6, mlp=None)]
    cfg = make_config(layers, width=128, vocab=256, side=16, loop={"start": 0, "stop": 2, "times": 2})
    for dtype in ("bf16", "f32"):
        sd = make_netolorn_checkpoint(cfg, dtype, seed=51)
        toks = tokens(300, cfg.vocab_size, seed=12)
        want = plain(cfg, sd, toks)
        # 16 bits: twice what rounding the products alone does to this configuration (its routed layers flip experts)
        bar = 2 * float(np.quantile(errors(plain_with_rounded_products(cfg, sd, toks), want), 0.95)) if dtype == "bf16" else None
        r = Runner(cfg, sd, dtype)
        try:
            whole = r.run("w", toks)
            close(whole, want, dtype, "whole", bar)
            close(r.run("c", toks, cuts=[133, 2, 1, 150, 1]), want, dtype, "portions", bar)
            close(r.run("d", toks, cuts=[260] + [1] * 40), want, dtype, "decoded", bar)
            if dtype == "bf16":   # the schedules agree with each other far more closely than with the exact model
                close(r.run("c", toks, cuts=[133, 2, 1, 150, 1]), whole, dtype, "portions against whole", bar / 2)
        finally:
            r.close()


@pytest.mark.gpu
def test_greedy_generation_through_master():
    from cake_b200.model import Context, Master, TextModelBase
    cfg = full_config()
    sd = make_netolorn_checkpoint(cfg, "f32", seed=61)
    prompt = tokens(9, cfg.vocab_size, seed=12)
    ctx = Context(cfg, sd, "f32", device=0, max_seq=64)
    try:
        out = Master(TextModelBase.load(ctx)).generate_text(prompt, 12)["tokens"]
    finally:
        ctx.close()
    seq = list(prompt)
    for tok in out:   # every generated token is the plain model's greedy choice, or within a hair of it
        lg = plain(cfg, sd, seq)[-1]
        assert lg[tok] >= lg.max() - 1e-2 * np.abs(lg).max(), (len(seq), tok, int(lg.argmax()))   # the sampler reads 16-bit logits
        seq.append(tok)
    assert len(out) == 12


@pytest.mark.gpu
def test_checkpoint_on_disk_through_the_trace_replayer_and_the_generate_command(tmp_path):
    """config.json + model.safetensors on disk -> `bin/trace_run` (steps on standard input, logits as files) and
    `python -m cake_b200.run` (token ids out): the model class follows the config in both."""
    import os
    import subprocess
    import sys
    from cake_b200.loader import open_model, save_checkpoint
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = full_config()
    sd = make_netolorn_checkpoint(cfg, "bf16", seed=81)
    model_dir, out_dir = str(tmp_path / "model"), str(tmp_path / "out")
    save_checkpoint(model_dir, cfg, sd)
    back, vb = open_model(model_dir)
    assert back.loop == cfg.loop and set(vb.keys()) == set(sd.keys()) and back.block_kind == "netolorn"
    toks = tokens(21, cfg.vocab_size, seed=14)
    want = plain(cfg, sd, toks)
    steps = [{"step": 0, "entries": [{"id": "r", "tokens": toks[:9], "want": [0, 8]}], "end": []},
             {"step": 1, "entries": [{"id": "r", "tokens": toks[9:11], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "r", "tokens": toks[11:], "want": [9]}], "end": ["r"]},
             {"step": 3, "entries": [{"id": "s", "tokens": toks[:4], "want": [3]}], "end": ["s"]}]
    for dtype in ("float32", "bfloat16"):
        res = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype, "--out", out_dir, "--max-tokens", "40"],
                             input="".join(json.dumps(x) + "\n" for x in steps), capture_output=True, text=True, timeout=900)
        assert res.returncode == 0, res.stderr[-2000:]
        assert [ln for ln in res.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
        assert not os.path.exists(os.path.join(out_dir, "1.f32"))
        got = {i: np.fromfile(os.path.join(out_dir, f"{i}.f32"), dtype="<f4").reshape(-1, cfg.vocab_size) for i in (0, 2, 3)}
        short = "f32" if dtype == "float32" else "bf16"
        close(np.concatenate([got[0], got[2], got[3]]), want[[0, 8, 20, 3]], short, f"trace replay in {dtype}")
    res = subprocess.run([sys.executable, "-m", "cake_b200.run", model_dir, "--prompt-ids", ",".join(map(str, toks[:6])), "-n", "5", "--dtype", "f32"],
                         capture_output=True, text=True, timeout=900, cwd=root)
    assert res.returncode == 0, res.stderr[-2000:]
    out = [int(t) for t in res.stdout.split("tokens:")[1].splitlines()[0].split()]
    assert len(out) == 5 and all(0 <= t < cfg.vocab_size for t in out)
