"""Nuvarax (gated delta rule layers; layers with softmax attention whose heads are mixed, beside a matrix memory; norms on both
sides of every sublayer; a convolution in front of every mixer; pair and position embeddings; looped layer ranges) through the
framework's own entry points (Context, TextModelBase, Sessions, Master) against the plain restatement in
oracle/nuvarax_plain.py, on small configurations made here with random weights.

What a schedule must not change: the logits at a position are the same whether the prompt went in whole, token by token or in
portions, whatever ran before in the same cache slot, and whatever other request is interleaved.  fp32 (D = float) is the sharp
comparison: the GPU and the plain code differ by summation order only.  The error of a position is the root mean square over
the vocabulary of the difference (mean removed) over the spread of the expected logits.
"""
import json

import numpy as np
import pytest
import torch

from cake_b200.config import Config
from cake_b200.synth import make_nuvarax_checkpoint
from oracle import nuvarax_plain as P

TOL = {"f32": 2e-4, "bf16": 1e-1, "f16": 2e-2}   # bf16 at widths of a few dozen: every projection is rounded to 8 bits


def delta(heads=4, kv_heads=2, dim=12, vdim=10, conv=3, ff=24, limit=0.8):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": {"kind": "dense", "ff": ff, "limit": limit} if ff else None}


def pair(heads=6, kv_heads=2, dim=8, vdim=6, scale=0.3, bias_max=20, rows=10, mheads=3, mdim=8, mvdim=12, cap=9.0, ff=24, limit=1.5):
    return {"type": "parallel", "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "bias_max": bias_max},
                                          "right": {"heads": mheads, "dim": mdim, "vdim": mvdim, "gate_cap": cap}},
            "mlp": {"kind": "dense", "ff": ff, "limit": limit} if ff else None, "_rows": rows}


def make_config(layers, loop=None, width=40, vocab=53, eps=1e-5, scale=2.0, taps=3, positions=512, bigram=(11, 5, 3)) -> Config:
    rows = [L.get("_rows") for L in layers]
    d = {"architecture": "Nuvarax", "width": width, "vocab": vocab, "norm": {"eps": eps}, "max_positions": positions,
         "canon": {"taps": taps} if taps else None,
         "embedding": {"scale": scale, "bigram": {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]} if bigram else None},
         "layers": [{k: v for k, v in L.items() if k != "_rows"} for L in layers]}
    if loop:
        d["loop"] = loop
    cfg = Config.from_hf(json.loads(json.dumps(d)))
    for sp, r in zip(cfg.layers, rows):
        if r:
            sp.bias_rows = r      # the table's rows are a tensor shape, not a config entry
    return cfg


def full_config(**kw) -> Config:
    """Every mechanism, unequal sizes, a loop over the middle layers, one layer without a feed-forward."""
    layers = [pair(), delta(), pair(heads=4, kv_heads=4, dim=12, vdim=8, scale=0.2, bias_max=33, rows=7, mheads=2, mdim=16, mvdim=8, cap=5.0, ff=0),
              delta(heads=2, kv_heads=2, dim=8, vdim=16, conv=2, ff=16, limit=1.0)]
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


def close(got, want, dtype, what=""):
    e = errors(got, want)
    if dtype == "f32":
        assert e.max() < TOL[dtype], f"{what}: worst {e.max():.3g} at position {int(e.argmax())}"
    else:
        assert np.quantile(e, 0.95) < TOL[dtype] and e.max() < 4 * TOL[dtype], f"{what}: 95 % within {np.quantile(e, 0.95):.3g}, worst {e.max():.3g}"


def plain(cfg, sd, toks, streams=None):
    wt = {k: v.float() for k, v in sd.items()}
    return P.forward(toks, wt, cfg.to_hf(), torch.float32, streams).numpy()


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
    assert d["architecture"] == "Nuvarax" and len(d["layers"]) == 4 and d["layers"][2]["mlp"] is None
    back = Config.from_hf(json.loads(json.dumps(d)))
    for sp in cfg.layers:
        sp.bias_rows = 0
    assert back.layers == cfg.layers and back.loop == cfg.loop and back.embed_scale == cfg.embed_scale
    assert back.layer_list and back.tie_word_embeddings and not back.loop_injects and back.final_norm_offset == 1.0
    assert back.pair_embedding == {"buckets": 11, "mul_prev": 5, "mul_cur": 3} and back.learned_positions == 512
    assert [i for i, _ in cfg.run_plan()] == [0, 1, 2, 1, 2, 3] == P.run_order(d)
    assert back.layers[0].type == "talking_attention" and back.layers[0].side.type == "matrix_memory" and back.layers[1].type == "delta"
    assert back.layers[1].dense_act == 2 and back.layers[1].dense_limit == 0.8 and back.layers[1].canon_taps == 3 and back.layers[1].norm_offset == 1.0
    bad = json.loads(json.dumps(d))
    bad["layers"][0]["type"] = "attention"
    with pytest.raises(ValueError):
        Config.from_hf(bad)
    bad = json.loads(json.dumps(d))
    bad["layers"][1]["mixer"]["kv_heads"] = 3
    with pytest.raises(ValueError):
        Config.from_hf(bad)
    bad = json.loads(json.dumps(d))
    bad["loop"]["stop"] = 9
    with pytest.raises(ValueError):
        Config.from_hf(bad)


def test_checkpoint_names_and_shapes():
    from cake_b200.loader import nuvarax_block_tensors
    cfg = full_config()
    sd = make_nuvarax_checkpoint(cfg, "bf16", seed=1)
    assert sd["bigram"].shape == (12, cfg.hidden_size) and sd["pos"].shape == (512, cfg.hidden_size) and "head" not in sd
    for i, sp in enumerate(cfg.layers):
        sp.bias_rows = 0
        main, side = nuvarax_block_tensors(sd, cfg, i)
        assert main["o"].shape == (cfg.hidden_size, sp.inner) and main["canon"].shape == (cfg.hidden_size, 3)
        assert (side is None) == (sp.type == "delta") and ("ff_gate" in main) == bool(sp.dense_ff)
        if side is not None:
            assert sp.bias_rows == main["rel"].shape[0] and side["i_proj"].shape == (sp.side.heads, cfg.hidden_size)
    assert [sp.bias_rows for sp in cfg.layers] == [10, 0, 7, 0]
    broken = dict(sd)
    broken["l1.mix.q.conv"] = sd["l1.mix.q.conv"][:, :-1]
    with pytest.raises(ValueError):
        nuvarax_block_tensors(broken, cfg, 1)
    # a config that leaves the taps to the tensors' shapes
    d = cfg.to_hf()
    d["canon"] = None
    del d["layers"][1]["mixer"]["conv"]
    bare = Config.from_hf(json.loads(json.dumps(d)))
    assert bare.layers[1].conv == 0 and bare.layers[1].canon_taps == 0
    main, _ = nuvarax_block_tensors(sd, bare, 1)
    assert bare.layers[1].conv == 3 and bare.layers[1].canon_taps == 3 and main["canon"].shape == (cfg.hidden_size, 3)


def test_plain_distance_buckets():
    b = [P.distance_bucket(n, 10, 20.0) for n in range(40)]
    assert b[:5] == [0, 1, 2, 3, 4] and b[5] == 5 and b == sorted(b) and b[15] == 8 and b[16] == 9 and b[39] == 9
    assert [P.distance_bucket(n, 7, 33.0) for n in (0, 2, 3, 32, 33, 500)] == [0, 2, 3, 6, 6, 6]


def test_plain_delta_rule_stores_and_replaces():
    """With beta = 1 and no decay the memory returns exactly the last value written under a key."""
    torch.manual_seed(0)
    k = torch.nn.functional.normalize(torch.randn(6), dim=0)
    S = torch.zeros(6, 4)
    for v in (torch.randn(4), torch.randn(4)):
        S = S + k[:, None] * (v - S.t() @ k)[None, :]
        assert torch.allclose(S.t() @ k, v, atol=1e-6)


def test_plain_matrix_memory_equals_its_unstabilised_form():
    """The running maximum only rescales numerator and denominator: for mild gates the read-out equals the direct sums."""
    torch.manual_seed(1)
    W, S, m = 10, 7, {"heads": 2, "dim": 4, "vdim": 3, "gate_cap": 6.0}
    wt = {"r.q": torch.randn(8, W) * 0.3, "r.k": torch.randn(8, W) * 0.3, "r.v": torch.randn(6, W) * 0.3, "r.g": torch.randn(6, W) * 0.3,
          "r.o": torch.eye(W)[:, :6].contiguous(), "r.norm": torch.ones(6), "r.i": torch.randn(2, W) * 0.3, "r.i.b": torch.randn(2) * 0.3 - 8.0,
          "r.f": torch.randn(2, W) * 0.3, "r.f.b": torch.ones(2)}
    h = torch.randn(S, W, dtype=torch.float64)
    got = P.matrix_memory(h, wt, "r.", m, 1e-6)
    q, k, v = (P.lin(wt["r." + n], h).view(S, 2, -1) for n in "qkv")
    li = 6.0 * torch.tanh(P.lin(wt["r.i"], h, wt["r.i.b"]) / 6.0)
    lf = torch.nn.functional.logsigmoid(6.0 * torch.tanh(P.lin(wt["r.f"], h, wt["r.f.b"]) / 6.0))
    out = torch.zeros(S, 2, 3, dtype=torch.float64)
    for t in range(S):
        for hd in range(2):
            w = torch.stack([torch.exp(li[j, hd] + lf[j + 1: t + 1, hd].sum()) for j in range(t + 1)])
            num = torch.einsum("j,jd,jv->dv", w, k[: t + 1, hd], v[: t + 1, hd]).t() @ (q[t, hd] * 0.5)
            den = (w[:, None] * k[: t + 1, hd]).sum(0) @ (q[t, hd] * 0.5)
            mx = max(0.0, max(float(li[j, hd] + lf[j + 1: t + 1, hd].sum()) for j in range(t + 1)), float(lf[: t + 1, hd].sum()))
            out[t, hd] = num / (max(abs(float(den)), float(np.exp(-mx)) * float(np.exp(mx))) + 1e-6 * float(np.exp(mx)))
    want = P.lin(wt["r.o"], P.rms_unit(out, 1e-6).reshape(S, 6) * torch.sigmoid(P.lin(wt["r.g"], h)))
    assert torch.allclose(got, want, atol=1e-9)


# ---------------------------------------------------------------------------------------------- on the GPU
MECHANISMS = {
    "delta": lambda: make_config([delta()]),
    "delta_one_key_head_one_tap": lambda: make_config([delta(heads=3, kv_heads=1, dim=8, vdim=8, conv=1, ff=0)]),
    "delta_key_size_24_five_taps": lambda: make_config([delta(heads=2, kv_heads=2, dim=24, vdim=40, conv=5)]),
    "delta_key_size_48": lambda: make_config([delta(heads=2, kv_heads=1, dim=48, vdim=32, conv=2)]),
    "delta_key_size_80": lambda: make_config([delta(heads=1, kv_heads=1, dim=80, vdim=72, conv=4)]),
    "delta_key_size_128": lambda: make_config([delta(heads=2, kv_heads=2, dim=128, vdim=64, conv=4)], width=64),
    "delta_key_size_160": lambda: make_config([delta(heads=1, kv_heads=1, dim=160, vdim=24, conv=3)]),
    "delta_key_size_272_in_shared_memory": lambda: make_config([delta(heads=2, kv_heads=1, dim=272, vdim=40, conv=2, ff=0)]),
    "pair_memory_key_size_288": lambda: make_config([pair(mheads=1, mdim=288, mvdim=32, ff=0)]),
    "canon_nine_taps": lambda: make_config([delta(ff=0), pair(ff=0)], taps=9),
    "pair": lambda: make_config([pair()]),
    "pair_every_head_its_own_keys": lambda: make_config([pair(heads=3, kv_heads=3, dim=12, vdim=12, rows=7, bias_max=33)]),
    "pair_ten_heads_one_key_head": lambda: make_config([pair(heads=10, kv_heads=1, dim=16, vdim=8, rows=16, bias_max=100, scale=0.6)]),
    "pair_wide_values": lambda: make_config([pair(heads=10, kv_heads=2, dim=12, vdim=420, rows=4, bias_max=9, ff=0)]),
    "pair_memory_in_registers_32": lambda: make_config([pair(mheads=2, mdim=32, mvdim=32)]),
    "pair_memory_in_registers_64": lambda: make_config([pair(mheads=1, mdim=64, mvdim=64, cap=15.0)]),
    "pair_memory_odd_sizes": lambda: make_config([pair(mheads=3, mdim=20, mvdim=28, cap=2.0)]),
    "pair_sharp_scores": lambda: make_config([pair(scale=3.0)]),
    "no_feed_forward_no_canon": lambda: make_config([delta(ff=0), pair(ff=0)], taps=0),
    "canon_one_tap": lambda: make_config([pair(), delta()], taps=1),
    "canon_five_taps": lambda: make_config([delta(), pair()], taps=5),
    "no_pair_embedding_no_scale": lambda: make_config([pair(), delta()], bigram=None, scale=1.0),
    "pair_embedding_large_multipliers": lambda: make_config([delta()], bigram=(50021, 2000003, 1999993), vocab=300),
    "loop_from_layer0": lambda: make_config([pair(), delta()], loop={"start": 0, "stop": 2, "times": 3}),
    "loop_once_tail_only": lambda: make_config([delta(), pair()], loop={"start": 1, "stop": 2, "times": 1}),
    "loop_in_the_middle": lambda: make_config([delta(), pair(), delta(ff=0)], loop={"start": 1, "stop": 2, "times": 4}),
}


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(MECHANISMS))
def test_each_mechanism_alone(name):
    cfg = MECHANISMS[name]()
    sd = make_nuvarax_checkpoint(cfg, "f32", seed=11)
    toks = tokens(45, cfg.vocab_size, seed=3)
    want = plain(cfg, sd, toks)
    r = Runner(cfg, sd, "f32")
    try:
        close(r.run("a", toks), want, "f32", name)
        close(r.run("b", toks, cuts=[1]), want, "f32", name + " token by token")
        close(r.run("c", toks, cuts=[7, 2, 3]), want, "f32", name + " portions")
    finally:
        r.close()


@pytest.mark.gpu
def test_residual_after_every_layer_run():
    """Block by block with the framework's own calls: the stream after every run of the plan."""
    import ctypes
    from cake_b200.capi import c_uint32, check, lib, ptr
    cfg = full_config()
    sd = make_nuvarax_checkpoint(cfg, "f32", seed=5)
    toks = tokens(19, cfg.vocab_size, seed=8)
    streams = []
    plain(cfg, sd, toks, streams)
    r = Runner(cfg, sd, "f32")
    try:
        ctx, model = r.ctx, r.model
        assert len(model.blocks) == 6 and not model.injections and model.blocks[1] is model.blocks[3]
        for pos, n in ((0, 8), (8, 11)):   # two portions: the second starts from the state the first left
            ids = np.ascontiguousarray([toks[pos:pos + n]], dtype=np.uint32)
            x = ctx.empty(1, n, cfg.hidden_size, dtype=torch.float32)
            check(lib().cake_b200_embed_at(ctx.h, ctx.cache.h, ids.ctypes.data_as(ctypes.POINTER(c_uint32)), 1, n, pos, ptr(x)))
            for j, blk in enumerate(model.blocks):
                x = blk.forward_batch(x, [(blk.layer_name(), pos, j)], ctx, blocks=[blk])
                ctx.sync()
                want = streams[j][pos:pos + n].numpy()
                assert np.abs(x[0].cpu().numpy() - want).max() < 2e-4 * max(1.0, np.abs(want).max()), f"run {j} ({blk.layer_name()}) at {pos}"
    finally:
        r.close()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
def test_schedules_agree_with_the_plain_model(dtype):
    """Whole, token by token and portions down to two tokens, first tokens included, on the model with everything."""
    cfg = full_config()
    sd = make_nuvarax_checkpoint(cfg, dtype, seed=21)
    toks = tokens(83, cfg.vocab_size, seed=4)
    want = plain(cfg, sd, toks)
    r = Runner(cfg, sd, dtype)
    try:
        whole = r.run("w", toks)
        close(whole, want, dtype, "whole")
        for cuts in ([1], [2], [2, 3, 5], [17], [64, 1], [1, 40, 2]):
            got = r.run("c", toks, cuts=cuts)
            close(got, want, dtype, f"portions {cuts}")
            if dtype == "f32":
                close(got, whole, dtype, f"portions {cuts} against whole")
        close(r.run("f", toks[:3], cuts=[1]), want[:3], dtype, "the first tokens")
        close(r.run("g", toks[:1]), want[:1], dtype, "a one-token sequence")
    finally:
        r.close()


@pytest.mark.gpu
def test_interleaved_requests_and_reused_slots():
    """Two unequal requests whose steps alternate give what each gives alone; a slot that a longer request left behind is
    reused by a shorter one and by a longer one (state, histories, the previous token and cache rows of the previous owner
    must not leak)."""
    cfg = full_config()
    sd = make_nuvarax_checkpoint(cfg, "f32", seed=31)
    a, b, c = tokens(37, cfg.vocab_size, 1), tokens(12, cfg.vocab_size, 2), tokens(50, cfg.vocab_size, 3)
    wa, wb, wc = plain(cfg, sd, a), plain(cfg, sd, b), plain(cfg, sd, c)
    r = Runner(cfg, sd, "f32")
    try:
        ga, gb, pa, pb = [], [], 0, 0
        while pa < len(a) or pb < len(b):
            if pa < len(a):
                n = min(5, len(a) - pa)
                lg = r.ses.step("a", a[pa:pa + n], want=list(range(n)))
                r.ctx.sync()
                ga.append(lg.cpu().numpy())
                pa += n
            if pb < len(b):
                n = min(2, len(b) - pb)
                lg = r.ses.step("b", b[pb:pb + n], want=list(range(n)))
                r.ctx.sync()
                gb.append(lg.cpu().numpy())
                pb += n
        close(np.concatenate(ga), wa, "f32", "interleaved a")
        close(np.concatenate(gb), wb, "f32", "interleaved b")
        r.ses.end("a")
        r.ses.end("b")
        n_caches = len(r.ses.free)
        close(r.run("b2", b, cuts=[3]), wb, "f32", "shorter request in a used slot")
        close(r.run("c", c, cuts=[9, 1]), wc, "f32", "longer request in a used slot")
        close(r.run("a2", a), wa, "f32", "whole prompt in a used slot")
        assert len(r.ses.free) == n_caches   # slots were reused, none added
    finally:
        r.close()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_batch_rows_against_each_alone(dtype):
    """Three equal-length rows in one call (a prompt portion, a second portion, then single tokens) give what each row gives
    alone: cache rows, recurrent state, histories and previous tokens are per batch row."""
    from cake_b200.model import Cache
    cfg = full_config()
    sd = make_nuvarax_checkpoint(cfg, dtype, seed=91)
    rows = [tokens(40, cfg.vocab_size, seed=20 + i) for i in range(3)]
    want = np.stack([plain(cfg, sd, r) for r in rows])
    r = Runner(cfg, sd, dtype)
    try:
        ctx, model = r.ctx, r.model
        ctx.cache = Cache(ctx, 3, cfg.max_seq_len)
        got, pos = [[] for _ in rows], 0
        for n in (23, 9, 1, 1, 6):
            ids = np.array([row[pos:pos + n] for row in rows], dtype=np.uint32)
            lg = model.forward(ids, pos, want=list(range(3 * n)))
            ctx.sync()
            lg = lg.cpu().numpy().reshape(3, n, -1)
            for b in range(3):
                got[b].append(lg[b])
            pos += n
        for b in range(3):
            close(np.concatenate(got[b]), want[b], dtype, f"batch row {b}")
    finally:
        r.close()


@pytest.mark.gpu
def test_far_keys_and_distance_buckets_in_prompt_portions_and_decoding():
    """Sharp attention (one key dominates each row, most of them far back) with a strong distance bias whose logarithmic buckets
    end well inside the sequence, over a few hundred positions: whole, in portions, and with the tail decoded token by token
    (single-token steps over that many keys split them over several CTAs).  That far keys matter is checked on the plain
    model itself: with keys further back than 100 hidden, its last rows come out differently."""
    cfg = make_config([pair(heads=4, kv_heads=2, dim=16, vdim=8, scale=2.5, rows=12, bias_max=150), pair(heads=3, kv_heads=1, dim=8, vdim=16, scale=1.5, rows=21, bias_max=40)])
    sd = make_nuvarax_checkpoint(cfg, "f32", seed=41)
    for i in (0, 1):
        sd[f"l{i}.mix.left.rel"] = sd[f"l{i}.mix.left.rel"] * 3.0
    toks = tokens(330, cfg.vocab_size, seed=6)
    want = plain(cfg, sd, toks)
    P.KEYS_VISIBLE = 100
    try:
        near = plain(cfg, sd, toks)
    finally:
        P.KEYS_VISIBLE = None
    assert errors(near[-20:], want[-20:]).max() > 50 * TOL["f32"]
    for dtype in ("f32", "bf16"):
        r = Runner(cfg, {k: v.to(torch.bfloat16) if dtype == "bf16" else v for k, v in sd.items()}, dtype)
        ref = want if dtype == "f32" else plain(cfg, {k: v.to(torch.bfloat16) for k, v in sd.items()}, toks)
        try:
            close(r.run("w", toks), ref, dtype, "whole")
            close(r.run("d", toks, cuts=[128] * 2 + [1] * 74), ref, dtype, "prompt portions then decoding")
            close(r.run("p", toks, cuts=[63, 2, 31]), ref, dtype, "odd portions")
        finally:
            r.close()


@pytest.mark.gpu
def test_long_decoding_through_recurrent_state():
    """Delta-rule and matrix-memory layers decoded token by token far past anything a portion covered; the forget gates are
    pushed towards one so that the memory keeps what the prompt wrote."""
    cfg = make_config([delta(heads=2, kv_heads=1), pair(mheads=2, mdim=8, mvdim=8), delta(heads=1, kv_heads=1, dim=8, vdim=8, conv=2)])
    sd = make_nuvarax_checkpoint(cfg, "f32", seed=43)
    sd["l1.mix.right.f.b"] = sd["l1.mix.right.f.b"] + 4.0
    sd["l0.mix.dt_bias"] = sd["l0.mix.dt_bias"] - 4.0
    toks = tokens(260, cfg.vocab_size, seed=7)
    want = plain(cfg, sd, toks)
    r = Runner(cfg, sd, "f32")
    try:
        close(r.run("d", toks, cuts=[40] + [1] * 220), want, "f32", "a short prompt then long decoding")
    finally:
        r.close()


@pytest.mark.gpu
def test_other_sizes_bf16_and_tensor_core_shapes():
    """Sizes whose projections take the tensor-core GEMM (multiples of 128 / 64) next to ones that do not."""
    layers = [pair(heads=4, kv_heads=2, dim=32, vdim=32, scale=0.15, rows=24, bias_max=64, mheads=2, mdim=32, mvdim=64, ff=64, limit=2.0),
              delta(heads=2, kv_heads=1, dim=64, vdim=64, conv=4, ff=128, limit=0.5),
              pair(heads=2, kv_heads=1, dim=24, vdim=40, rows=5, bias_max=7, mheads=1, mdim=16, mvdim=48, ff=0)]
    cfg = make_config(layers, width=128, vocab=256, taps=2)
    for dtype in ("bf16", "f32"):
        sd = make_nuvarax_checkpoint(cfg, dtype, seed=51)
        toks = tokens(70, cfg.vocab_size, seed=9)
        want = plain(cfg, sd, toks)
        r = Runner(cfg, sd, dtype)
        try:
            close(r.run("w", toks), want, dtype, "whole")
            close(r.run("c", toks, cuts=[33, 2, 1]), want, dtype, "portions")
        finally:
            r.close()


@pytest.mark.gpu
def test_long_portions_on_the_tensor_cores():
    """Sizes at which long portions in bf16 take the matrix-product form of the attention (several blocks of rows per key head,
    with and without keys from earlier portions), against the plain model and against the same positions through the per-row
    kernels; two batch rows through the same path."""
    layers = [pair(heads=8, kv_heads=2, dim=64, vdim=128, scale=0.35, rows=14, bias_max=200, mheads=2, mdim=32, mvdim=64, ff=64, limit=3.0),
              delta(heads=2, kv_heads=2, dim=32, vdim=64, conv=4, ff=0),
              pair(heads=4, kv_heads=4, dim=128, vdim=128, scale=0.2, rows=6, bias_max=50, mheads=1, mdim=64, mvdim=32, ff=64, limit=1.0)]
    cfg = make_config(layers, width=128, vocab=96, positions=1024)
    sd = make_nuvarax_checkpoint(cfg, "bf16", seed=71)
    toks = tokens(700, cfg.vocab_size, seed=13)
    want = plain(cfg, sd, toks)
    r = Runner(cfg, sd, "bf16")
    try:
        whole = r.run("w", toks)
        close(whole, want, "bf16", "whole")
        close(r.run("c", toks, cuts=[300, 390, 2, 1]), want, "bf16", "portions")
        small = r.run("s", toks, cuts=[100])       # every portion below the matrix-product threshold
        close(small, want, "bf16", "short portions")
        assert np.quantile(errors(whole, small), 0.95) < TOL["bf16"]
        from cake_b200.model import Cache
        a, b = toks[:340], toks[340:680]
        wa, wb = plain(cfg, sd, a), plain(cfg, sd, b)
        r.ctx.cache = Cache(r.ctx, 2, cfg.max_seq_len)
        g1 = r.model.forward(np.array([a[:200], b[:200]], dtype=np.uint32), 0, want=list(range(400)))
        g2 = r.model.forward(np.array([a[200:], b[200:]], dtype=np.uint32), 200, want=list(range(280)))
        r.ctx.sync()
        g1, g2 = g1.cpu().numpy().reshape(2, 200, -1), g2.cpu().numpy().reshape(2, 140, -1)
        close(np.concatenate([g1[0], g2[0]]), wa, "bf16", "batch row 0")
        close(np.concatenate([g1[1], g2[1]]), wb, "bf16", "batch row 1")
    finally:
        r.close()


@pytest.mark.gpu
def test_many_heads_on_the_tensor_cores():
    """More heads than the register form of the softmax-and-mix kernel holds: the shared-memory form, against the plain model."""
    cfg = make_config([pair(heads=36, kv_heads=4, dim=64, vdim=128, scale=0.3, rows=9, bias_max=60, mheads=1, mdim=16, mvdim=32, ff=0)], width=128, vocab=64)
    sd = make_nuvarax_checkpoint(cfg, "bf16", seed=77)
    toks = tokens(150, cfg.vocab_size, seed=15)
    want = plain(cfg, sd, toks)
    r = Runner(cfg, sd, "bf16")
    try:
        close(r.run("w", toks), want, "bf16", "whole")
        close(r.run("c", toks, cuts=[40, 110]), want, "bf16", "portions")
    finally:
        r.close()


@pytest.mark.gpu
def test_greedy_generation_through_master():
    from cake_b200.model import Context, Master, TextModelBase
    cfg = full_config()
    sd = make_nuvarax_checkpoint(cfg, "f32", seed=61)
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
    cfg = full_config(positions=64)
    sd = make_nuvarax_checkpoint(cfg, "bf16", seed=81)
    model_dir, out_dir = str(tmp_path / "model"), str(tmp_path / "out")
    save_checkpoint(model_dir, cfg, sd)
    back, vb = open_model(model_dir)
    assert back.loop == cfg.loop and set(vb.keys()) == set(sd.keys()) and back.block_kind == "nuvarax"
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
