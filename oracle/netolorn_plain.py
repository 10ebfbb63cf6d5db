"""Plain, slow restatement of the Netolorn design in torch on the CPU: one function per mechanism, whole sequences only
(no cache, no portions, which is the point: the framework's scheduled runs are compared with it).
Test infrastructure: nothing under cake_b200/ imports it and it imports nothing from there.

Notation: x [S, W] residual stream, h a normed copy.  The model is a plain dict ``cfg`` (the parsed config.json) and a
dict ``wt`` name -> tensor.  ``dt`` is the torch dtype the arithmetic runs in (float32, or float64 for a sharper bar)."""
import math

import torch


def lin(W, x, b=None):
    y = x @ W.to(x.dtype).t()
    return y if b is None else y + b.to(x.dtype)


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def tanh_norm(x, wt, name):
    """The design's norm: no statistics of x, an element-wise squashing with one learned slope, then gain and offset."""
    return torch.tanh(wt[name + ".alpha"].to(x.dtype) * x) * wt[name].to(x.dtype) + wt[name + ".b"].to(x.dtype)


def rotary_tables(rot, positions, dt):
    """cos / sin [S, dims / 2] of a rotation over the first ``dims`` entries of a head, pairs (i, i + dims / 2), with the
    frequency blend between fast and slow pairs and the amplitude correction when ``scaling`` is given."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    f = [base ** (-2.0 * i / dims) for i in range(half)]
    amp = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])
        pair_of = lambda turns: dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo, hi = max(math.floor(pair_of(float(sc["fast"]))), 0), min(math.ceil(pair_of(float(sc["slow"]))), dims - 1)
        for i in range(half):
            ramp = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
            f[i] = f[i] / factor * ramp + f[i] * (1.0 - ramp)
        amp = 0.1 * math.log(factor) + 1.0
    ang = torch.tensor(positions, dtype=torch.float64)[:, None] * torch.tensor(f, dtype=torch.float64)[None, :]
    return (torch.cos(ang) * amp).to(dt), (torch.sin(ang) * amp).to(dt)


def rotate(x, cos, sin):
    """x [S, heads, dim]: the first 2 * cos.shape[1] entries of every head are rotated, the rest pass."""
    half = cos.shape[1]
    u, v, rest = x[..., :half], x[..., half: 2 * half], x[..., 2 * half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([u * c - v * s, v * c + u * s, rest], -1)


KEYS_VISIBLE = None   # tests only: an int hides keys further back than that, to show that far keys matter in a test's model


def visible(S, size, keep_first):
    """[S, S] bool: row i sees key j when j <= i and (i - j < size or j < keep_first); size 0 = no window."""
    i, j = torch.arange(S)[:, None], torch.arange(S)[None, :]
    vis = j <= i
    if size:
        vis = vis & ((i - j < size) | (j < keep_first))
    if KEYS_VISIBLE is not None:
        vis = vis & (i - j <= KEYS_VISIBLE)
    return vis


def sink_attention(h, wt, p, m, eps):
    """Grouped-query softmax attention: projection biases, a rotation of part of every head, unit-RMS queries and keys,
    a sliding window that keeps the sequence's first tokens, a learned sink in the softmax's denominator, and a sigmoid
    gate on the concatenated heads."""
    S = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m.get("kv_heads") or m["heads"]), int(m["dim"]), int(m["vdim"])
    q = lin(wt[p + "q"], h, wt[p + "q.b"]).view(S, H, D)
    k = lin(wt[p + "k"], h, wt[p + "k.b"]).view(S, G, D)
    v = lin(wt[p + "v"], h, wt[p + "v.b"]).view(S, G, V)
    rot = m.get("rot")
    if rot and int(rot.get("dims") or 0) > 0:
        cos, sin = rotary_tables(rot, list(range(S)), h.dtype)
        q, k = rotate(q, cos, sin), rotate(k, cos, sin)
    q, k = rms_unit(q, eps), rms_unit(k, eps)
    kk, vv = k.repeat_interleave(H // G, 1), v.repeat_interleave(H // G, 1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * float(m["scale"])
    mask = m.get("mask") or {}
    vis = visible(S, int(mask.get("size") or 0), int(mask.get("keep_first") or 0))
    s = s.masked_fill(~vis[None], float("-inf"))
    sink = wt[p + "sink"].to(h.dtype)                       # [H]: a logit without key or value
    top = torch.maximum(s.max(-1).values, sink[:, None])    # [H, S]
    e = torch.exp(s - top[..., None])
    w = e / (e.sum(-1) + torch.exp(sink[:, None] - top))[..., None]
    o = torch.einsum("hij,jhv->ihv", w, vv).reshape(S, H * V)
    o = o * torch.sigmoid(lin(wt[p + "g"], h))
    return lin(wt[p + "o"], o)


def latent_attention(h, wt, p, m, eps):
    """Softmax attention without positions whose queries pass a normed low-rank latent and whose keys and values are
    expanded per head from one normed low-rank latent per token; a sliding window; one sigmoid gate per head."""
    S = h.shape[0]
    H, D, V = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    cq = rms_unit(lin(wt[p + "dq"], h), eps) * wt[p + "dq.norm"].to(h.dtype)
    q = lin(wt[p + "uq"], cq).view(S, H, D)
    c = rms_unit(lin(wt[p + "dkv"], h), eps) * wt[p + "dkv.norm"].to(h.dtype)
    k = lin(wt[p + "uk"], c).view(S, H, D)
    v = lin(wt[p + "uv"], c).view(S, H, V)
    s = torch.einsum("ihd,jhd->hij", q, k) * float(m["scale"])
    mask = m.get("mask") or {}
    vis = visible(S, int(mask.get("size") or 0), 0)
    w = torch.softmax(s.masked_fill(~vis[None], float("-inf")), -1)
    o = torch.einsum("hij,jhv->ihv", w, v) * torch.sigmoid(lin(wt[p + "g"], h))[:, :, None]
    return lin(wt[p + "o"], o.reshape(S, H * V))


def dense_ff(h, wt, p):
    g = lin(wt[p + "gate"], h)
    return lin(wt[p + "down"], g * torch.sigmoid(g) * lin(wt[p + "up"], h))


def clamped_expert(h, wt, p, limit):
    g = torch.clamp(lin(wt[p + "gate"], h), max=limit)
    u = torch.clamp(lin(wt[p + "up"], h), -limit, limit)
    return lin(wt[p + "down"], g * torch.sigmoid(1.702 * g) * (u + 1.0))


def routed_ff(h, wt, p, mlp):
    """The ``top`` experts with the largest router logits, weighted by the softmax over the chosen logits alone, plus a
    shared expert behind one sigmoid gate per token."""
    r = mlp["router"]
    E, top = int(r["experts"]), int(r["top"])
    z = lin(wt[p + "router"], h, wt[p + "router.b"])
    val, idx = torch.topk(z, top, dim=-1)
    wgt = torch.softmax(val, -1)
    limit = float(mlp["expert"]["limit"])
    y = torch.zeros_like(h)
    for e in range(E):
        rows, slot = (idx == e).nonzero(as_tuple=True)
        if len(rows):
            y[rows] = y[rows] + wgt[rows, slot][:, None] * clamped_expert(h[rows], wt, f"{p}e{e}.", limit)
    sh = mlp.get("shared")
    if sh:
        y = y + torch.sigmoid(lin(wt[p + "shared.sg"], h)) * clamped_expert(h, wt, p + "shared.", float(sh["limit"]))
    return y


def token_side(x, tokens, wt, p, i, dim, eps):
    """The per-layer token input: a slice of a second embedding table, gated by the stream, projected back and RMS-normed."""
    e = wt["side.embed"].to(x.dtype)[torch.as_tensor(tokens, dtype=torch.long)][:, i * dim: (i + 1) * dim]
    y = lin(wt[p + "side.proj"], gelu_tanh(lin(wt[p + "side.gate"], x)) * e)
    return x + rms_unit(y, eps) * wt[p + "side.norm"].to(x.dtype)


def layer(x, tokens, wt, cfg, i):
    L, p, eps = cfg["layers"][i], f"l{i}.", float(cfg["norm"]["eps"])
    mixer = sink_attention if L["type"] == "attention" else latent_attention
    x = x + tanh_norm(mixer(tanh_norm(x, wt, p + "norm1"), wt, p + "mix.", L["mixer"], eps), wt, p + "norm1b")
    mlp = L.get("mlp")
    if mlp is not None:
        h = tanh_norm(x, wt, p + "norm2")
        y = dense_ff(h, wt, p + "mlp.") if mlp["kind"] == "dense" else routed_ff(h, wt, p + "mlp.", mlp)
        x = x + tanh_norm(y, wt, p + "norm2b")
    side = cfg.get("token_side")
    if side:
        x = token_side(x, tokens, wt, p, i, int(side["dim"]), eps)
    return x


def run_order(cfg):
    """[(layer, starts a pass)] in execution order."""
    n, lp = len(cfg["layers"]), cfg.get("loop")
    if not lp:
        return [(i, False) for i in range(n)]
    a, b, t = int(lp["start"]), int(lp["stop"]), int(lp["times"])
    return [(i, False) for i in range(a)] + [(i, i == a) for _ in range(t) for i in range(a, b)] + [(i, False) for i in range(b, n)]


def forward(tokens, wt, cfg, dt=torch.float32, trace=None):
    """Logits [S, vocab]; ``trace`` (a list) receives the stream after every layer run."""
    x0 = wt["embed"].to(dt)[torch.as_tensor(tokens, dtype=torch.long)]
    x = x0
    for i, first in run_order(cfg):
        if first:
            x = lin(wt["loop.in"], torch.cat([x, x0], -1))
        x = layer(x, tokens, wt, cfg, i)
        if trace is not None:
            trace.append(x.clone())
    return lin(wt["head"], tanh_norm(x, wt, "final.norm"))
