"""Plain, slow restatement of the Nuvarax design in torch on the CPU: one function per mechanism, whole sequences only
(no cache, no carried state, no portions, which is the point: the framework's scheduled runs are compared with it).
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


def norm1p(x, w, eps):
    """RMS norm whose gain is stored as an offset from one."""
    return rms_unit(x, eps) * (1.0 + w.to(x.dtype))


def silu(z):
    return z * torch.sigmoid(z)


def causal_conv(x, w):
    """x [S, C], w [C, taps]: y_t = sum_j w[:, j] x_(t - taps + 1 + j), zeros before the start (the last tap is the current token)."""
    S, taps = x.shape[0], w.shape[1]
    xp = torch.cat([x.new_zeros(taps - 1, x.shape[1]), x], 0)
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + xp[j: j + S] * w[:, j].to(x.dtype)
    return y


def embed(tokens, wt, cfg, dt):
    """Scaled token embedding + a hashed (previous, current) pair embedding + a learned position vector."""
    e = cfg["embedding"]
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x = wt["embed"].to(dt)[ids] * float(e["scale"])
    bg = e.get("bigram")
    if bg:
        nb = int(bg["buckets"])
        prev = torch.cat([ids[:1], ids[:-1]])
        rows = (prev * int(bg["mul_prev"]) + ids * int(bg["mul_cur"])) % nb
        rows[0] = nb          # the first token of a sequence has no predecessor: the table's last row
        x = x + wt["bigram"].to(dt)[rows]
    return x + wt["pos"].to(dt)[: len(tokens)] if "pos" in wt else x


def distance_bucket(n, rows, dmax):
    """Exact buckets below rows / 2, logarithmic ones from there up to dmax, the last bucket beyond."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(dmax / half) * (rows - half))))


KEYS_VISIBLE = None   # tests only: an int hides keys further back than that, to show that far keys matter in a test's model


def mixed_attention(h, wt, p, m):
    """Grouped-query softmax attention with projection biases, a bucketed distance bias per head, the heads' weights mixed
    by a matrix after the softmax, and a sigmoid gate on the concatenated heads."""
    S = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = lin(wt[p + "q"], h, wt[p + "q.b"]).view(S, H, D)
    k = lin(wt[p + "k"], h, wt[p + "k.b"]).view(S, G, D)
    v = lin(wt[p + "v"], h, wt[p + "v.b"]).view(S, G, V)
    rel = wt[p + "rel"].to(h.dtype)
    B = rel.shape[0]
    idx = torch.tensor([[distance_bucket(i - j, B, float(m["bias_max"])) if j <= i else 0 for j in range(S)] for i in range(S)])
    kk, vv = k.repeat_interleave(H // G, 1), v.repeat_interleave(H // G, 1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * float(m["scale"]) + rel[idx].permute(2, 0, 1)
    vis = torch.arange(S)[:, None] >= torch.arange(S)[None, :]
    if KEYS_VISIBLE is not None:
        vis = vis & (torch.arange(S)[:, None] - torch.arange(S)[None, :] < KEYS_VISIBLE)
    pr = torch.softmax(s.masked_fill(~vis[None], float("-inf")), -1)
    pr = torch.einsum("hg,gij->hij", wt[p + "talk"].to(h.dtype), pr)
    o = torch.einsum("hij,jhv->ihv", pr, vv).reshape(S, H * V)
    o = o * torch.sigmoid(lin(wt[p + "g"], h))
    return lin(wt[p + "o"], o, wt[p + "o.b"])


def matrix_memory(h, wt, p, m, eps):
    """A matrix memory per head with exponential input and forget gates, kept in range by a running maximum of their logs."""
    S = h.shape[0]
    H, D, V, cap = int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["gate_cap"])
    q = lin(wt[p + "q"], h).view(S, H, D) * D ** -0.5
    k = lin(wt[p + "k"], h).view(S, H, D)
    v = lin(wt[p + "v"], h).view(S, H, V)
    li = cap * torch.tanh(lin(wt[p + "i"], h, wt[p + "i.b"]) / cap)
    lf = torch.nn.functional.logsigmoid(cap * torch.tanh(lin(wt[p + "f"], h, wt[p + "f.b"]) / cap))
    St, n, mx = h.new_zeros(H, D, V), h.new_zeros(H, D), h.new_zeros(H)
    out = []
    for t in range(S):
        mn = torch.maximum(lf[t] + mx, li[t])
        a, b = torch.exp(lf[t] + mx - mn), torch.exp(li[t] - mn)
        St = a[:, None, None] * St + b[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = a[:, None] * n + b[:, None] * k[t]
        mx = mn
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        out.append(torch.einsum("hdv,hd->hv", St, q[t]) / den[:, None])
    o = rms_unit(torch.stack(out), eps).reshape(S, H * V) * wt[p + "norm"].to(h.dtype)
    return lin(wt[p + "o"], o * torch.sigmoid(lin(wt[p + "g"], h)))


def parallel_mixer(h, wt, p, m, eps):
    """Two mixers read the same input; each output is RMS-normed over the width with a plain gain, and they are averaged."""
    a = mixed_attention(h, wt, p + "left.", m["left"])
    b = matrix_memory(h, wt, p + "right.", m["right"], eps)
    return 0.5 * (rms_unit(a, eps) * wt[p + "left.out"].to(h.dtype) + rms_unit(b, eps) * wt[p + "right.out"].to(h.dtype))


def delta_mixer(h, wt, p, m, eps):
    """Gated delta rule: the memory first decays, then the value stored under the key is moved towards the new one, then it is read."""
    S = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])

    def branch(name):
        return silu(causal_conv(lin(wt[p + name], h), wt[p + name + ".conv"]))

    def unit(z):
        return z / torch.sqrt((z * z).sum(-1, keepdim=True) + 1e-6)

    q = unit(branch("q").view(S, G, D)) * D ** -0.5
    k = unit(branch("k").view(S, G, D))
    v = branch("v").view(S, H, V)
    q, k = q.repeat_interleave(H // G, 1), k.repeat_interleave(H // G, 1)
    beta = torch.sigmoid(lin(wt[p + "b"], h))
    g = torch.exp(-torch.exp(wt[p + "A_log"].to(h.dtype)) * torch.nn.functional.softplus(lin(wt[p + "a"], h) + wt[p + "dt_bias"].to(h.dtype)))
    St = h.new_zeros(H, D, V)
    out = []
    for t in range(S):
        St = g[t][:, None, None] * St
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", St, k[t]))
        St = St + k[t][:, :, None] * u[:, None, :]
        out.append(torch.einsum("hdv,hd->hv", St, q[t]))
    o = rms_unit(torch.stack(out), eps) * wt[p + "norm"].to(h.dtype)
    o = o.reshape(S, H * V) * silu(lin(wt[p + "g"], h))
    return lin(wt[p + "o"], o)


def feed_forward(h, wt, p, mlp):
    """Clamped gated feed-forward: the gate is capped from above, the linear branch from both sides and shifted by one."""
    lim = float(mlp["limit"])
    g = lin(wt[p + "gate"], h).clamp(max=lim)
    u = lin(wt[p + "up"], h).clamp(-lim, lim)
    return lin(wt[p + "down"], g * torch.sigmoid(1.702 * g) * (u + 1.0))


def run_order(cfg):
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return list(range(n))
    a, b, times = int(lp["start"]), int(lp["stop"]), int(lp["times"])
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(tokens, wt, cfg, dt=torch.float32, streams=None):
    """Logits [S, vocab] of a whole sequence; ``streams`` (a list) receives the residual stream after every layer run."""
    eps = float(cfg["norm"]["eps"])
    x = embed(tokens, wt, cfg, dt)
    for i in run_order(cfg):
        L, p = cfg["layers"][i], f"l{i}."
        h = norm1p(x, wt[p + "norm1"], eps)
        if (cfg.get("canon") or {}).get("taps"):
            h = h + causal_conv(h, wt[p + "canon1"])
        if L["type"] == "delta":
            y = delta_mixer(h, wt, p + "mix.", L["mixer"], eps)
        elif L["type"] == "parallel":
            y = parallel_mixer(h, wt, p + "mix.", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = x + norm1p(y, wt[p + "norm1b"], eps)
        if L.get("mlp") is not None:
            y = feed_forward(norm1p(x, wt[p + "norm2"], eps), wt, p + "mlp.", L["mlp"])
            x = x + norm1p(y, wt[p + "norm2b"], eps)
        if streams is not None:
            streams.append(x.clone())
    return lin(wt["embed"], norm1p(x, wt["final.norm"], eps))
