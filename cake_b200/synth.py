"""Synthetic HF-layout checkpoints (there are no real weights offline).

Tensor names and shapes are the ones the reference loads:
  transformer.rs:89-90   {layer}.input_layernorm.weight / post_attention_layernorm.weight  (H)
  attention.rs:96-129    {layer}.self_attn.{q,k,v,o}_proj.weight [out,in] (+ .bias, q_norm/k_norm.weight)
  mlp.rs:43-49           {layer}.mlp.{gate,up,down}_proj.weight
  text_model.rs:159-193  {prefix}.embed_tokens.weight, {prefix}.norm.weight, lm_head.weight
"""
from __future__ import annotations

import torch

from .config import Config

TORCH_DTYPES = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}


def layer_tensor_shapes(cfg: Config) -> dict:
    H, I = cfg.hidden_size, cfg.intermediate_size
    s = {
        "input_layernorm.weight": (H,),
        "post_attention_layernorm.weight": (H,),
        "self_attn.q_proj.weight": (cfg.size_q, H),
        "self_attn.k_proj.weight": (cfg.size_kv, H),
        "self_attn.v_proj.weight": (cfg.size_kv, H),
        "self_attn.o_proj.weight": (H, cfg.size_q),
        "mlp.gate_proj.weight": (I, H),
        "mlp.up_proj.weight": (I, H),
        "mlp.down_proj.weight": (H, I),
    }
    if cfg.use_qkv_bias:
        s["self_attn.q_proj.bias"] = (cfg.size_q,)
        s["self_attn.k_proj.bias"] = (cfg.size_kv,)
        s["self_attn.v_proj.bias"] = (cfg.size_kv,)
    if cfg.use_qk_norm:  # attention.rs:121-122: over head_dim, or over the whole projection (OLMo2)
        pre = getattr(cfg, "pre_reshape_qk_norm", False)
        s["self_attn.q_norm.weight"] = (cfg.size_q if pre else cfg.hd,)
        s["self_attn.k_norm.weight"] = (cfg.size_kv if pre else cfg.hd,)
    kind = getattr(cfg, "block_kind", "llama")
    if kind in ("olmo2", "exaone4_hf"):     # olmo2/block.rs:49-52: two post-norms, no input norms
        del s["input_layernorm.weight"]
        s["post_feedforward_layernorm.weight"] = (H,)
    elif kind == "gemma3":  # gemma3/block.rs:84-91: four norms
        s["pre_feedforward_layernorm.weight"] = (H,)
        s["post_feedforward_layernorm.weight"] = (H,)
    return s


def residual_deltas(sd: dict) -> dict:
    """Checkpoints of ``residual_rms_norm`` models (Gemma3) store norm weights as deltas around 0 (forward weight = 1 + w,
    config.rs:155-173): turn a synthetic checkpoint whose norm vectors sit around 1 into that convention."""
    return {k: ((v.float() - 1.0).to(v.dtype) if (k.endswith("norm.weight") or k.endswith("layernorm.weight")) else v)
            for k, v in sd.items()}


def _fill(shape, name: str, gen: torch.Generator, device, dtype, std: float):
    t = torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * std
    if name.endswith("norm.weight") or name.endswith("layernorm.weight"):
        t = t + 1.0
    return t.to(dtype)


def make_layer(cfg: Config, i: int, dtype: str = "bf16", seed: int = 1234, device="cpu", std: float = 0.02) -> dict:
    """Weights of one block, keyed by full HF name.  Deterministic per (seed, layer, device type).  With
    ``cfg.fused_qkv_proj`` / ``cfg.fused_gate_up_proj`` (Phi-3/4 checkpoints) the same values are stored as
    ``self_attn.qkv_proj.weight = cat(q, k, v)`` / ``mlp.gate_up_proj.weight = cat(gate, up)``."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed * 1000003 + i)
    out = {}
    for short, shape in layer_tensor_shapes(cfg).items():
        out[short] = _fill(shape, short, gen, device, TORCH_DTYPES[dtype], std)
    if cfg.fused_qkv_proj:
        out["self_attn.qkv_proj.weight"] = torch.cat([out.pop(f"self_attn.{p}_proj.weight") for p in "qkv"], 0)
    if cfg.fused_gate_up_proj:
        out["mlp.gate_up_proj.weight"] = torch.cat([out.pop("mlp.gate_proj.weight"), out.pop("mlp.up_proj.weight")], 0)
    return {f"{cfg.layer_name(i)}.{short}": t for short, t in out.items()}


def make_head(cfg: Config, dtype: str = "bf16", seed: int = 1234, device="cpu", std: float = 0.02,
              peaked: bool = False) -> dict:
    """embed / final norm / lm_head.  ``peaked``: lm_head rows are scaled copies of the embedding rows,
    which gives large top-1/top-2 logit margins (used for greedy token-id parity)."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed * 1000003 + 999983)
    td = TORCH_DTYPES[dtype]
    p = cfg.model_prefix
    out = {
        f"{p}.embed_tokens.weight": _fill((cfg.vocab_size, cfg.hidden_size), "embed", gen, device, td, std),
        f"{p}.norm.weight": _fill((cfg.hidden_size,), "norm.weight", gen, device, td, std),
    }
    if not cfg.tie_word_embeddings:
        if peaked:
            out["lm_head.weight"] = (out[f"{p}.embed_tokens.weight"].float() * 4.0).to(td)
        else:
            out["lm_head.weight"] = _fill((cfg.vocab_size, cfg.hidden_size), "lm_head", gen, device, td, std)
    return out


def make_checkpoint(cfg: Config, dtype: str = "bf16", seed: int = 1234, device="cpu", std: float = 0.02,
                    peaked: bool = False) -> dict:
    sd = make_head(cfg, dtype, seed, device, std, peaked)
    for i in range(cfg.num_hidden_layers):
        sd.update(make_layer(cfg, i, dtype, seed, device, std))
    return sd


class LazyCheckpoint(dict):
    """var_builder that materialises ONE block at a time on ``device`` — a 15 GB (8B) or 141 GB (70B) synthetic
    checkpoint never exists whole; ``Forwarder::load`` pulls a layer's tensors, the previous layer is dropped.
    Head tensors (embed / norm / lm_head) are created on first use and kept until ``drop_head()``.
    ``host_copy=True`` also keeps a CPU copy of everything handed out in ``self.host`` (what a checker needs to see
    the same weights).  Values are those of ``make_layer`` / ``make_head`` for (seed, device type)."""

    def __init__(self, cfg: Config, dtype: str = "bf16", seed: int = 1234, device="cuda", std: float = 0.02,
                 host_copy: bool = False, peaked: bool = False):
        super().__init__()
        self.cfg, self.dtype, self.seed, self.device, self.std, self.peaked = cfg, dtype, seed, device, std, peaked
        self.host = {} if host_copy else None

    def _ensure(self, k: str):
        if k in self:
            return
        if ".layers." in k:
            i = int(k.split(".layers.")[1].split(".")[0])
            self.drop_layers()
            new = make_layer(self.cfg, i, self.dtype, self.seed, self.device, self.std)
        elif k.startswith(self.cfg.model_prefix + ".") or k == "lm_head.weight":
            new = make_head(self.cfg, self.dtype, self.seed, self.device, self.std, self.peaked)
        else:
            return
        self.update(new)
        if self.host is not None:
            for kk, t in new.items():
                self.host[kk] = t.cpu()

    def get(self, k, d=None):
        self._ensure(k)
        return dict.get(self, k, d)

    def __getitem__(self, k):
        self._ensure(k)
        return dict.__getitem__(self, k)

    def drop_layers(self):
        for kk in [kk for kk in self if ".layers." in kk]:
            del self[kk]

    def drop_head(self):
        for kk in [kk for kk in self if ".layers." not in kk]:
            del self[kk]


def make_listed_checkpoint(cfg: Config, dtype: str = "bf16", seed: int = 1234, device="cpu", std: float = 0.05) -> dict:
    """Random weights of a layer-list (Nigenex) model under the names its checkpoints use: ``embed``, ``head``,
    ``final.norm`` (one number) and per layer ``l<i>.norm1`` (one number), ``l<i>.shift`` [width] in (0, 1),
    ``l<i>.mix.{q,k,o,g}``, ``l<i>.mix.{r1,r2}`` [heads] > 0 and, when the layer has a feed-forward, ``l<i>.mlp.{gate,up,down}``."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed * 1000003 + 424243)
    td, H = TORCH_DTYPES[dtype], cfg.hidden_size

    def rn(*shape, s=std):
        return (torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * s).to(td)

    def ru(*shape, lo=0.0, hi=1.0):
        return (torch.rand(shape, generator=gen, device=device, dtype=torch.float32) * (hi - lo) + lo).to(td)

    sd = {"embed": rn(cfg.vocab_size, H, s=1.0), "head": rn(cfg.vocab_size, H, s=4.0 * std), "final.norm": ru(lo=0.8, hi=1.2).reshape(())}
    for i, sp in enumerate(cfg.layers):
        p, sq, skv = cfg.layer_name(i), sp.heads * sp.head_dim, sp.kv_heads * sp.head_dim
        sd[f"{p}.norm1"] = ru(lo=0.8, hi=1.2).reshape(())
        sd[f"{p}.shift"] = ru(H)
        sd[f"{p}.mix.q"], sd[f"{p}.mix.k"] = rn(sq, H), rn(skv, H)
        sd[f"{p}.mix.r1"], sd[f"{p}.mix.r2"] = ru(sp.heads, lo=0.1, hi=1.0), ru(sp.heads, lo=0.05, hi=2.0)
        sd[f"{p}.mix.g"], sd[f"{p}.mix.o"] = rn(sp.heads, H), rn(H, sq)
        if sp.ff:
            sd[f"{p}.mlp.gate"], sd[f"{p}.mlp.up"], sd[f"{p}.mlp.down"] = rn(sp.ff, H), rn(sp.ff, H), rn(H, sp.ff)
    return sd


def make_mixer_checkpoint(cfg: Config, dtype: str = "bf16", seed: int = 1234, device="cpu", std: float = 0.05, router_std: float = 0.5) -> dict:
    """Random weights of a mixer-list (Setodra) model under the names its checkpoints use: ``embed``, ``head``, ``final.norm``
    [width], ``loop.step`` [times, width] when the config loops, and per layer ``l<i>.norm1``, ``l<i>.mix.*`` (latent attention:
    q, dkv, dkv.norm, uk, uv, o; retention: q, k, v, g, o; state space: in, conv, conv.b, dt_bias, A_log, D, norm, o) and, with a
    feed-forward, ``l<i>.norm2``, ``l<i>.mlp.{router, correction, e<j>.{gate,up,down}, shared.{gate,up,down,sg}}``."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed * 1000003 + 77377)
    td, H = TORCH_DTYPES[dtype], cfg.hidden_size

    def rn(*shape, s=std):
        return (torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * s).to(td)

    def ru(*shape, lo=0.0, hi=1.0):
        return (torch.rand(shape, generator=gen, device=device, dtype=torch.float32) * (hi - lo) + lo).to(td)

    sd = {"embed": rn(cfg.vocab_size, H, s=1.0), "head": rn(cfg.vocab_size, H, s=4.0 * std), "final.norm": ru(H, lo=0.8, hi=1.2)}
    if cfg.loop:
        sd["loop.step"] = rn(int(cfg.loop["times"]), H, s=0.5)
    for i, sp in enumerate(cfg.layers):
        p = cfg.layer_name(i)
        sd[f"{p}.norm1"] = ru(H, lo=0.8, hi=1.2)
        sd[f"{p}.mix.o"] = rn(H, sp.inner)
        if sp.type == "latent_attention":
            sd[f"{p}.mix.q"] = rn(sp.heads * (sp.dim + sp.rot_dim), H, s=4 * std)
            sd[f"{p}.mix.dkv"] = rn(sp.kv_rank + sp.rot_dim, H, s=4 * std)
            sd[f"{p}.mix.dkv.norm"] = ru(sp.kv_rank, lo=0.8, hi=1.2)
            sd[f"{p}.mix.uk"], sd[f"{p}.mix.uv"] = rn(sp.heads * sp.dim, sp.kv_rank, s=4 * std), rn(sp.inner, sp.kv_rank, s=2 * std)
        elif sp.type == "retention":
            sd[f"{p}.mix.q"], sd[f"{p}.mix.k"] = rn(sp.heads * sp.dim, H, s=2 * std), rn(sp.heads * sp.dim, H, s=2 * std)
            sd[f"{p}.mix.v"], sd[f"{p}.mix.g"] = rn(sp.inner, H, s=2 * std), rn(sp.inner, H, s=2 * std)
        else:
            ch = sp.inner + 2 * sp.groups * sp.state
            sd[f"{p}.mix.in"] = rn(2 * sp.inner + 2 * sp.groups * sp.state + sp.heads, H, s=2 * std)
            sd[f"{p}.mix.conv"], sd[f"{p}.mix.conv.b"] = rn(ch, sp.conv, s=0.4), rn(ch, s=0.1)
            sd[f"{p}.mix.dt_bias"], sd[f"{p}.mix.A_log"] = ru(sp.heads, lo=-3.0, hi=0.5), ru(sp.heads, lo=-1.5, hi=1.0)
            sd[f"{p}.mix.D"], sd[f"{p}.mix.norm"] = ru(sp.heads, lo=0.5, hi=1.5), ru(sp.inner, lo=0.8, hi=1.2)
        mo = sp.moe
        if mo is not None:
            et = mo.experts + mo.identity
            sd[f"{p}.norm2"] = ru(H, lo=0.8, hi=1.2)
            sd[f"{p}.mlp.router"], sd[f"{p}.mlp.correction"] = rn(et, H, s=router_std), rn(et, s=0.05)
            for j in range(mo.experts):
                sd[f"{p}.mlp.e{j}.gate"], sd[f"{p}.mlp.e{j}.up"], sd[f"{p}.mlp.e{j}.down"] = rn(mo.ff, H, s=2 * std), rn(mo.ff, H, s=2 * std), rn(H, mo.ff, s=2 * std)
            if mo.shared_ff:
                sd[f"{p}.mlp.shared.gate"], sd[f"{p}.mlp.shared.up"] = rn(mo.shared_ff, H, s=2 * std), rn(mo.shared_ff, H, s=2 * std)
                sd[f"{p}.mlp.shared.down"], sd[f"{p}.mlp.shared.sg"] = rn(H, mo.shared_ff, s=2 * std), rn(1, H, s=4 * std)
    return sd


def make_nuvarax_checkpoint(cfg: Config, dtype: str = "bf16", seed: int = 1234, device="cpu", std: float = 0.05) -> dict:
    """Random weights of a Nuvarax model under the names its checkpoints use: ``embed`` (also the output projection), ``bigram``
    [buckets + 1, width], ``pos`` [positions, width], ``final.norm`` and per layer ``l<i>.{norm1, norm1b, norm2, norm2b}`` (gains
    stored as offsets from one), ``l<i>.canon1`` [width, taps], ``l<i>.mlp.{gate, up, down}`` and the mixer under ``l<i>.mix.``:
    a delta layer has ``q, k, v`` (each with ``.conv``), ``b``, ``a``, ``A_log``, ``dt_bias``, ``norm`` [vdim], ``g``, ``o``; a parallel
    layer ``left.{q, k, v, o}`` (each with ``.b``), ``left.{rel, talk, g, out}`` and ``right.{q, k, v, g, o, norm, out}``,
    ``right.{i, f}`` (each with ``.b``).  ``rel`` has ``bias_rows`` rows (32 when the spec leaves it 0)."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed * 1000003 + 909091)
    td, H = TORCH_DTYPES[dtype], cfg.hidden_size

    def rn(*shape, s=std):
        return (torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * s).to(td)

    def ru(*shape, lo=0.0, hi=1.0):
        return (torch.rand(shape, generator=gen, device=device, dtype=torch.float32) * (hi - lo) + lo).to(td)

    sd = {"embed": rn(cfg.vocab_size, H, s=0.3), "final.norm": rn(H, s=0.1)}
    if cfg.pair_embedding:
        sd["bigram"] = rn(cfg.pair_embedding["buckets"] + 1, H, s=0.5)
    if cfg.learned_positions:
        sd["pos"] = rn(cfg.learned_positions, H, s=0.5)
    for i, sp in enumerate(cfg.layers):
        p = cfg.layer_name(i)
        sd[f"{p}.norm1"] = rn(H, s=0.1)
        if sp.post_norms:
            sd[f"{p}.norm1b"] = rn(H, s=0.1)
        if sp.canon_taps >= 1:
            sd[f"{p}.canon1"] = rn(H, sp.canon_taps, s=0.3)
        if sp.dense_ff:
            sd[f"{p}.norm2"] = rn(H, s=0.1)
            if sp.post_norms:
                sd[f"{p}.norm2b"] = rn(H, s=0.1)
            sd[f"{p}.mlp.gate"], sd[f"{p}.mlp.up"], sd[f"{p}.mlp.down"] = rn(sp.dense_ff, H, s=4 * std), rn(sp.dense_ff, H, s=4 * std), rn(H, sp.dense_ff)
        if sp.type == "delta":
            qk, m = sp.n_kv * sp.dim, f"{p}.mix"
            sd[f"{m}.q"], sd[f"{m}.k"], sd[f"{m}.v"] = rn(qk, H, s=2 * std), rn(qk, H, s=2 * std), rn(sp.inner, H, s=2 * std)
            sd[f"{m}.q.conv"], sd[f"{m}.k.conv"], sd[f"{m}.v.conv"] = rn(qk, sp.conv, s=0.4), rn(qk, sp.conv, s=0.4), rn(sp.inner, sp.conv, s=0.4)
            sd[f"{m}.b"], sd[f"{m}.a"] = rn(sp.heads, H, s=2 * std), rn(sp.heads, H, s=2 * std)
            sd[f"{m}.A_log"], sd[f"{m}.dt_bias"] = ru(sp.heads, lo=-2.5, hi=0.5), ru(sp.heads, lo=-3.0, hi=0.5)
            sd[f"{m}.norm"], sd[f"{m}.g"], sd[f"{m}.o"] = ru(sp.vdim, lo=0.8, hi=1.2), rn(sp.inner, H, s=2 * std), rn(H, sp.inner)
        else:
            a, r, rows = f"{p}.mix.left", sp.side, sp.bias_rows or 32
            sq, skv, svv = sp.heads * sp.dim, sp.n_kv * sp.dim, sp.n_kv * sp.vdim
            sd[f"{a}.q"], sd[f"{a}.k"], sd[f"{a}.v"] = rn(sq, H, s=4 * std), rn(skv, H, s=4 * std), rn(svv, H, s=2 * std)
            sd[f"{a}.q.b"], sd[f"{a}.k.b"], sd[f"{a}.v.b"], sd[f"{a}.o.b"] = rn(sq, s=0.2), rn(skv, s=0.2), rn(svv, s=0.2), rn(H, s=0.2)
            sd[f"{a}.rel"] = rn(rows, sp.heads, s=0.7)
            sd[f"{a}.talk"] = (torch.eye(sp.heads, device=device) * 0.7 + torch.randn((sp.heads, sp.heads), generator=gen, device=device) * 0.25).to(td)
            sd[f"{a}.g"], sd[f"{a}.o"], sd[f"{a}.out"] = rn(sp.inner, H, s=2 * std), rn(H, sp.inner), ru(H, lo=0.8, hi=1.2)
            b, rq = f"{p}.mix.right", r.heads * r.dim
            sd[f"{b}.q"], sd[f"{b}.k"], sd[f"{b}.v"], sd[f"{b}.g"] = rn(rq, H, s=2 * std), rn(rq, H, s=2 * std), rn(r.inner, H, s=2 * std), rn(r.inner, H, s=2 * std)
            sd[f"{b}.o"], sd[f"{b}.norm"], sd[f"{b}.out"] = rn(H, r.inner), ru(r.inner, lo=0.8, hi=1.2), ru(H, lo=0.8, hi=1.2)
            sd[f"{b}.i"], sd[f"{b}.f"] = rn(r.heads, H, s=4 * std), rn(r.heads, H, s=4 * std)
            sd[f"{b}.i.b"], sd[f"{b}.f.b"] = rn(r.heads, s=0.5), ru(r.heads, lo=1.0, hi=4.0)
    return sd


def make_netolorn_checkpoint(cfg: Config, dtype: str = "bf16", seed: int = 1234, device="cpu", std: float = 0.05, router_std: float = 0.5) -> dict:
    """Random weights of a Netolorn model under the names its checkpoints use: ``embed``, ``head``, ``final.norm`` (+ ``.b``,
    ``.alpha``), ``side.embed`` [vocab, layers * dim] with a token input, ``loop.in`` [width, 2 width] when the config loops, and per
    layer ``l<i>.{norm1, norm1b, norm2, norm2b}`` (each with ``.b`` and ``.alpha``), ``l<i>.side.{gate, proj, norm}`` and the mixer under
    ``l<i>.mix.``: attention ``q, k, v`` (each with ``.b``), ``sink``, ``g``, ``o``; latent attention ``dq``, ``dq.norm``, ``uq``, ``dkv``,
    ``dkv.norm``, ``uk``, ``uv``, ``g``, ``o``; the feed-forward under ``l<i>.mlp.``: ``gate, up, down`` or ``router`` (+ ``.b``),
    ``e<j>.{gate, up, down}``, ``shared.{gate, up, down, sg}``."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed * 1000003 + 515151)
    td, H = TORCH_DTYPES[dtype], cfg.hidden_size

    def rn(*shape, s=std):
        return (torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * s).to(td)

    def ru(*shape, lo=0.0, hi=1.0):
        return (torch.rand(shape, generator=gen, device=device, dtype=torch.float32) * (hi - lo) + lo).to(td)

    def norm(name, sd):
        sd[name], sd[name + ".b"], sd[name + ".alpha"] = ru(H, lo=0.8, hi=1.2), rn(H, s=0.1), ru(lo=0.5, hi=1.5).reshape(())

    sd = {"embed": rn(cfg.vocab_size, H, s=1.0), "head": rn(cfg.vocab_size, H, s=4.0 * std)}
    norm("final.norm", sd)
    if cfg.token_side_dim:
        sd["side.embed"] = rn(cfg.vocab_size, cfg.token_side_dim * len(cfg.layers), s=1.0)
    if cfg.loop:
        sd["loop.in"] = (torch.cat([torch.eye(H), torch.zeros(H, H)], 1).to(device) * 0.8 + torch.randn((H, 2 * H), generator=gen, device=device) * (0.5 / H ** 0.5)).to(td)
    for i, sp in enumerate(cfg.layers):
        p, m = cfg.layer_name(i), cfg.layer_name(i) + ".mix"
        norm(f"{p}.norm1", sd)
        norm(f"{p}.norm1b", sd)
        sd[f"{m}.o"] = rn(H, sp.inner, s=4 * std)
        if sp.type == "sink_attention":
            sq, skv, svv = sp.heads * sp.dim, sp.n_kv * sp.dim, sp.n_kv * sp.vdim
            sd[f"{m}.q"], sd[f"{m}.k"], sd[f"{m}.v"] = rn(sq, H, s=4 * std), rn(skv, H, s=4 * std), rn(svv, H, s=4 * std)
            sd[f"{m}.q.b"], sd[f"{m}.k.b"], sd[f"{m}.v.b"] = rn(sq, s=0.2), rn(skv, s=0.2), rn(svv, s=0.2)
            sd[f"{m}.sink"], sd[f"{m}.g"] = rn(sp.heads, s=1.0), rn(sp.inner, H, s=2 * std)
        else:
            sd[f"{m}.dq"], sd[f"{m}.dq.norm"], sd[f"{m}.uq"] = rn(sp.q_rank, H, s=4 * std), ru(sp.q_rank, lo=0.8, hi=1.2), rn(sp.heads * sp.dim, sp.q_rank, s=sp.q_rank ** -0.5)
            sd[f"{m}.dkv"], sd[f"{m}.dkv.norm"] = rn(sp.kv_rank, H, s=4 * std), ru(sp.kv_rank, lo=0.8, hi=1.2)
            sd[f"{m}.uk"], sd[f"{m}.uv"] = rn(sp.heads * sp.dim, sp.kv_rank, s=sp.kv_rank ** -0.5), rn(sp.inner, sp.kv_rank, s=sp.kv_rank ** -0.5)
            sd[f"{m}.g"] = rn(sp.heads, H, s=2 * std)
        mo = sp.moe
        if sp.dense_ff or mo is not None:
            norm(f"{p}.norm2", sd)
            norm(f"{p}.norm2b", sd)
        if sp.dense_ff:
            sd[f"{p}.mlp.gate"], sd[f"{p}.mlp.up"], sd[f"{p}.mlp.down"] = rn(sp.dense_ff, H, s=4 * std), rn(sp.dense_ff, H, s=4 * std), rn(H, sp.dense_ff, s=4 * std)
        elif mo is not None:
            sd[f"{p}.mlp.router"], sd[f"{p}.mlp.router.b"] = rn(mo.experts, H, s=router_std), rn(mo.experts, s=0.5)
            for j in range(mo.experts):
                sd[f"{p}.mlp.e{j}.gate"], sd[f"{p}.mlp.e{j}.up"], sd[f"{p}.mlp.e{j}.down"] = rn(mo.ff, H, s=8 * std), rn(mo.ff, H, s=8 * std), rn(H, mo.ff, s=4 * std)
            if mo.shared_ff:
                sd[f"{p}.mlp.shared.gate"], sd[f"{p}.mlp.shared.up"] = rn(mo.shared_ff, H, s=8 * std), rn(mo.shared_ff, H, s=8 * std)
                sd[f"{p}.mlp.shared.down"], sd[f"{p}.mlp.shared.sg"] = rn(H, mo.shared_ff, s=4 * std), rn(1, H, s=4 * std)
        if sp.side_dim:
            sd[f"{p}.side.gate"], sd[f"{p}.side.proj"], sd[f"{p}.side.norm"] = rn(sp.side_dim, H, s=4 * std), rn(H, sp.side_dim, s=0.3), ru(H, lo=0.2, hi=0.6)
    return sd
