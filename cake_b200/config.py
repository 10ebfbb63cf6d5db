"""Model configuration for the block-forward path.

Mirrors the reference's generalized ``Config`` (cake-core/src/models/common/config.rs:87-150) for the
fields the dense Llama-family block path reads, and the HF ``config.json`` mappings of the architectures
whose blocks are exactly that path: ``LlamaConfig::into_config`` (models/llama3/config.rs:62-98),
``Qwen3Config`` (qwen3/config.rs:55-93), ``Qwen2Config`` (qwen2/config.rs:69-105, q/k/v bias),
``MistralConfig`` (mistral/config.rs:56-93, without an active sliding window), ``Falcon3Config``
(falcon3/config.rs:53-90) and ``Phi4Config`` (phi4/config.rs:63-100: pre-fused qkv / gate_up tensors, partial
rotary).  Field names follow the reference.
"""
from __future__ import annotations

import ctypes
import json
from dataclasses import dataclass, field, asdict
from typing import Optional

import numpy as np

DTYPES = {"bf16": 0, "f16": 1, "f32": 2}


@dataclass
class RopeScaling:
    """config.rs RopeScaling (llama3 type only; cache.rs:49-80)."""
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 0
    rope_type: Optional[str] = None


@dataclass
class LayerSpec:
    """One entry of a layer-list config (``cake_b200_layer_spec`` in include/cake_b200.h): a parallel block whose mixer is
    grouped-query attention with a score soft cap, a distance bias, a sliding window, keys used as values and a per-head
    output gate, next to an optional gated feed-forward.  Every size and constant is per layer."""
    heads: int
    kv_heads: int
    head_dim: int
    window: int = 0          # row i attends to the keys j with i - window < j <= i; 0 = all j <= i
    scale: float = 1.0
    softcap: float = 0.0     # 0 = none
    ff: int = 0              # 0 = the layer has no feed-forward
    act: int = 1             # 0 silu, 1 tanh-gelu


@dataclass
class RotarySpec:
    """``cake_b200_rotary_spec``: rotation of the first ``dims`` entries of a head, pair (i, i + dims/2); ``factor`` > 0 blends
    the frequencies towards f / factor between the pairs that complete ``fast`` and ``slow`` turns over ``original`` positions."""
    dims: int = 0
    base: float = 10000.0
    factor: float = 0.0
    fast: float = 0.0
    slow: float = 0.0
    original: int = 0

    @staticmethod
    def from_dict(d: Optional[dict]) -> "RotarySpec":
        if not d:
            return RotarySpec()
        sc = d.get("scaling") or {}
        return RotarySpec(dims=int(d["dims"]), base=float(d["base"]), factor=float(sc.get("factor") or 0.0), fast=float(sc.get("fast") or 0.0),
                          slow=float(sc.get("slow") or 0.0), original=int(sc.get("original") or 0))

    def to_dict(self) -> Optional[dict]:
        if not self.dims:
            return None
        d = {"dims": self.dims, "base": self.base}
        if self.factor:
            d["scaling"] = {"factor": self.factor, "fast": self.fast, "slow": self.slow, "original": self.original}
        return d


@dataclass
class MoeSpec:
    """``cake_b200_moe_spec``: ``experts`` gated feed-forwards of width ``ff`` plus ``identity`` pass-through experts, ``top`` per
    token, weights scaled by ``scale``; ``shared_ff`` > 0: one more expert of that width for every token, behind a sigmoid gate."""
    experts: int = 0
    identity: int = 0
    top: int = 1
    scale: float = 1.0
    ff: int = 0
    shared_ff: int = 0
    act: int = 0             # 0 silu, 1 tanh-gelu, 2 clamped (min(g, limit) sigmoid(1.702 g) (clamp(u) + 1))
    limit: float = 0.0
    shared_limit: float = 0.0
    logit_bias: bool = False  # the router's correction is a bias of the logits; choice by logit, softmax over the chosen alone


MIXER_KINDS = {"latent_attention": 1, "retention": 2, "mamba2": 3, "delta": 4, "talking_attention": 5, "matrix_memory": 6,
               "sink_attention": 7, "latent_window": 8}


@dataclass
class MixerSpec:
    """One entry of a mixer-list config (``cake_b200_mixer_spec`` in include/cake_b200.h): a sequential pre-norm block whose
    mixer is latent attention, retention or a state-space layer, with an optional routed feed-forward."""
    type: str
    heads: int
    vdim: int
    dim: int = 0
    rot_dim: int = 0
    kv_rank: int = 0
    scale: float = 1.0
    rot: RotarySpec = field(default_factory=RotarySpec)
    decay: list = field(default_factory=list)
    state: int = 0
    groups: int = 1
    conv: int = 1
    norm_groups: int = 1
    moe: Optional[MoeSpec] = None
    # delta (gated delta rule), talking_attention (softmax attention with a bucketed distance bias whose heads' weights are mixed
    # after the softmax) and matrix_memory (a matrix memory with exponential gates), and the block structure switches they come
    # with: gains stored as offsets, post norms, a convolution in front of the mixer, a side mixer, a dense feed-forward
    kv_heads: int = 0        # delta, talking_attention (0 = heads)
    bias_rows: int = 0       # talking_attention: rows of the distance-bias table (read from the tensor's shape at load)
    bias_max: float = 0.0
    gate_cap: float = 0.0    # matrix_memory
    norm_offset: float = 0.0
    post_norms: bool = False
    canon_taps: int = 0
    dense_ff: int = 0
    dense_act: int = 0       # 0 silu, 1 tanh-gelu, 2 clamped (min(g, limit) sigmoid(1.702 g) (clamp(u) + 1))
    dense_limit: float = 0.0
    side: Optional["MixerSpec"] = None   # a second mixer beside this one, reading the same input
    # sink_attention (grouped-query attention with a rotation of part of every head, unit-RMS q and k, a sliding window that keeps
    # the first tokens and a sink) and latent_window (latent attention without positions, queries through a latent of their own,
    # a sliding window, one gate per head), and the switches they come with: the squashing norm and the per-layer token input
    window: int = 0          # 0 = every earlier key
    keep_first: int = 0
    qk_unit: bool = False
    q_rank: int = 0
    norm_kind: int = 0       # 0 RMS, 1 tanh(alpha x) * w + b
    norm_alpha: list = field(default_factory=lambda: [0.0, 0.0, 0.0, 0.0])   # norm1, norm1b, norm2, norm2b (read from the checkpoint)
    side_dim: int = 0
    side_col: int = 0

    @property
    def inner(self) -> int:
        return self.heads * self.vdim

    @property
    def n_kv(self) -> int:
        return self.kv_heads or self.heads


@dataclass
class Config:
    hidden_size: int
    intermediate_size: int
    vocab_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_scaling: Optional[RopeScaling] = None
    tie_word_embeddings: bool = False
    max_seq_len: int = 4096
    use_qkv_bias: bool = False
    model_prefix: str = "model"
    head_dim: Optional[int] = None
    partial_rotary_factor: float = 1.0
    use_qk_norm: bool = False
    eos_token_id: list = field(default_factory=list)
    sliding_window: Optional[int] = None
    fused_qkv_proj: bool = False      # Phi-3/4: one 'qkv_proj' tensor = cat(q, k, v) (attention.rs:90-94)
    fused_gate_up_proj: bool = False  # Phi-3/4: one 'gate_up_proj' tensor = cat(gate, up) (mlp.rs:38-40)
    use_gelu_mlp: bool = False        # config.rs:133: gelu_tanh(gate) * up (mlp.rs:25-26)
    embed_scale: Optional[float] = None   # config.rs:136: embeddings scaled before the blocks (text_model.rs:274-276)
    residual_rms_norm: bool = False   # config.rs:113: norm weights stored as deltas; (1 + w) in f32 at LOAD time (config.rs:155-173)
    pre_reshape_qk_norm: bool = False  # config.rs:116 (OLMo2): QK-norm over the whole q / k projection, before the head reshape
    global_layers: list = field(default_factory=list)  # config.rs:126-130: per-layer schedule, True = global (full context)
    block_kind: str = "llama"         # which block.rs the layers are: "llama" (transformer.rs), "olmo2", "gemma3", "exaone4";
                                      # "nigenex": a layer-list model (``layers`` below), not a reference block
    layers: list = field(default_factory=list)  # layer-list models: one LayerSpec per layer (sizes differ between layers)
    logit_softcap: float = 0.0        # logits <- cap * tanh(logits / cap) after the head (0 = none)
    loop: Optional[dict] = None       # mixer-list models: {"start", "stop", "times"}: layers start..stop-1 run `times` times in a row
    loop_injects: bool = True         # the stream receives a per-pass vector (and the embedding output again) in front of every pass
    pair_embedding: Optional[dict] = None  # {"buckets", "mul_prev", "mul_cur"}: a hashed (previous, current) token embedding is added
    learned_positions: int = 0        # > 0: a learned vector per position is added to the embedding (rows of the table)
    final_norm_offset: float = 0.0    # the final norm's gain is stored as an offset from this number
    loop_mode: str = "step"           # in front of every pass: "step" (x += [x0] + vector), "none", "project" (x <- W [x; x0])
    token_side_dim: int = 0           # > 0: a per-layer token input of that width (table `side.embed` [vocab, layers * dim])
    final_norm_kind: int = 0          # 1: the final norm is the squashing norm

    def layer_variant(self, i: int, max_seq: Optional[int] = None) -> dict:
        """Norm placement and attention mode of layer ``i``, as the reference's per-architecture block.rs sets them up:
          llama   (common/transformer.rs:103-135)  pre-norms, the config's window, RoPE
          olmo2   (olmo2/block.rs:62-90)           NO pre-norms, post-attention / post-feedforward norms, RoPE
          gemma3  (gemma3/block.rs:60-135)         all four norms; global layers: full context + RoPE, local: window, NO RoPE
          exaone4 (exaone4/block.rs:50-110)        pre-norms; global layers: full context, NO RoPE, local: window + RoPE
        ``window``: -1 = the config's, 0 = none, > 0 = this layer's (passed as 0 when it can never bite)."""
        def win(w):
            return int(w) if (w and w < (max_seq or self.max_seq_len)) else 0
        is_global = bool(self.global_layers[i]) if i < len(self.global_layers) else False
        if self.block_kind == "olmo2":
            return dict(pre_norms=False, post_norms=True, window=-1, no_rope=False)
        if self.block_kind == "gemma3":
            return dict(pre_norms=True, post_norms=True, window=0 if is_global else win(self.sliding_window), no_rope=not is_global)
        if self.block_kind == "exaone4":
            return dict(pre_norms=True, post_norms=False, window=0 if is_global else win(self.sliding_window), no_rope=is_global)
        if self.block_kind == "exaone4_hf":
            # NOT a reference block: the structure HF transformers gives EXAONE 4.0 (post-norms like OLMo2 + the hybrid
            # schedule).  Test-only: it pins the oracle's per-layer NoPE / window handling to an independent implementation
            # (tests/golden/hf_exaone4_hf_tiny.npz); the reference's own EXAONE4 block is pre-norm (exaone4/block.rs:96-110).
            return dict(pre_norms=False, post_norms=True, window=0 if is_global else win(self.sliding_window), no_rope=is_global)
        return dict(pre_norms=True, post_norms=False, window=-1, no_rope=False)

    @property
    def standard_blocks(self) -> bool:
        return self.block_kind == "llama"

    @property
    def layer_list(self) -> bool:
        """The checkpoint's config lists its layers one by one; such models keep an fp32 residual stream."""
        return self.block_kind in ("nigenex", "setodra", "nuvarax", "netolorn")

    @property
    def scalar_final_norm(self) -> bool:
        return self.block_kind == "nigenex"

    def run_plan(self) -> list:
        """[(layer index, pass number or None)] in execution order.  Without a loop every layer runs once.  With one, the
        layers start..stop-1 run ``times`` times with the same weights; the first layer of pass t carries t: the stream
        receives the embedding output again (t > 0) and the pass's step vector right before it.  Every run owns a cache slot."""
        n = len(self.layers) if self.layers else self.num_hidden_layers
        if not self.loop:
            return [(i, None) for i in range(n)]
        a, b, times = int(self.loop["start"]), int(self.loop["stop"]), int(self.loop["times"])
        runs = [(i, None) for i in range(a)]
        for t in range(times):
            runs += [(i, t if i == a else None) for i in range(a, b)]
        return runs + [(i, None) for i in range(b, n)]

    def head_tensor_names(self):
        """(embedding, final norm, lm_head or None when tied) as the checkpoint names them (text_model.rs:159-193)."""
        if self.layer_list:
            return "embed", "final.norm", None if self.tie_word_embeddings else "head"
        p = self.model_prefix
        return f"{p}.embed_tokens.weight", f"{p}.norm.weight", None if self.tie_word_embeddings else "lm_head.weight"

    @property
    def hd(self) -> int:
        # attention.rs:85
        return self.head_dim if self.head_dim else self.hidden_size // self.num_attention_heads

    @property
    def size_q(self) -> int:
        return self.hd * self.num_attention_heads

    @property
    def size_kv(self) -> int:
        return self.hd * self.num_key_value_heads

    def layer_name(self, i: int) -> str:
        # text_model.rs:205  "{prefix}.layers.{i}"
        if self.layer_list:
            return f"l{i}"
        return f"{self.model_prefix}.layers.{i}"

    # ---- HF config.json mappings -------------------------------------------------------------
    # arch -> (default rope_theta, default max_position_embeddings, fixed flags): the serde defaults and the
    # constants each ``into_config`` hard-wires.  Strings the reference does not know fall back to Llama
    # (cake/mod.rs:81-109); architectures it knows but whose block is not this path are refused here.
    _ARCHS = {
        "LlamaForCausalLM": (500000.0, 4096, dict()),
        "Qwen2ForCausalLM": (1000000.0, 32768, dict(use_qkv_bias=True)),
        "Qwen3ForCausalLM": (1000000.0, 40960, dict(use_qk_norm=True, _head_dim=True)),
        "MistralForCausalLM": (1000000.0, 131072, dict(_head_dim=True, _sliding_window=True)),
        "FalconForCausalLM": (500000.0, 131072, dict(_head_dim=True)),
        "Phi3ForCausalLM": (1000000.0, 131072, dict(_head_dim=True, _partial=True, _fused=True)),
        "Phi4ForCausalLM": (1000000.0, 131072, dict(_head_dim=True, _partial=True, _fused=True)),
    }
    _OTHER_BLOCKS = ("Qwen3_5ForConditionalGeneration", "Qwen3MoeForCausalLM", "Qwen3_5MoeForConditionalGeneration",
                     "LuxTTSForTextToSpeech")
    _SIBLING_BLOCKS = {"Gemma3ForCausalLM": "gemma3", "OLMo2ForCausalLM": "olmo2", "Olmo2ForCausalLM": "olmo2",
                       "ExaoneForCausalLM": "exaone4"}  # cake/mod.rs:99-105

    @staticmethod
    def detect_arch(d: dict) -> str:
        """config.rs:175-190 detect_text_model_arch: the first *string* entry of ``architectures``, else ""."""
        archs = d.get("architectures")
        if isinstance(archs, list):
            for a in archs:
                if isinstance(a, str):
                    return a
        return ""

    @staticmethod
    def _from_nigenex(d: dict, max_seq: int = 4096) -> "Config":
        """Nigenex ``config.json``: ``width``, ``vocab``, ``norm.eps``, ``logit_softcap`` and ``layers``, a list whose
        entries give ``type`` (the mixer; only ``attention`` exists), the mixer's sizes and constants (``mixer``: heads,
        kv_heads, dim, vdim, scale, softcap, mask.size) and the feed-forward (``mlp``: kind ``dense`` with ``ff``, or null).
        Nothing is assumed equal between layers."""
        specs = []
        for i, L in enumerate(d["layers"]):
            if L.get("type") != "attention":
                raise ValueError(f"layer {i}: mixer type {L.get('type')!r} is not part of this design")
            m = L["mixer"]
            if int(m.get("vdim", m["dim"])) != int(m["dim"]):
                raise ValueError(f"layer {i}: the keys double as values, so vdim {m['vdim']} must equal dim {m['dim']}")
            mlp = L.get("mlp")
            if mlp is not None and mlp.get("kind") != "dense":
                raise ValueError(f"layer {i}: feed-forward kind {mlp.get('kind')!r} is not part of this design")
            mask = m.get("mask") or {}
            specs.append(LayerSpec(heads=int(m["heads"]), kv_heads=int(m["kv_heads"]), head_dim=int(m["dim"]),
                                   window=int(mask.get("size") or 0), scale=float(m["scale"]), softcap=float(m.get("softcap") or 0.0),
                                   ff=int(mlp["ff"]) if mlp is not None else 0, act=1))
        if not specs:
            raise ValueError("config lists no layers")
        return Config(hidden_size=int(d["width"]), intermediate_size=max(s.ff for s in specs), vocab_size=int(d["vocab"]),
                      num_hidden_layers=len(specs), num_attention_heads=specs[0].heads, num_key_value_heads=specs[0].kv_heads,
                      rms_norm_eps=float(d["norm"]["eps"]), head_dim=specs[0].head_dim, max_seq_len=int(max_seq),
                      block_kind="nigenex", layers=specs, logit_softcap=float(d.get("logit_softcap") or 0.0), model_prefix="")

    @staticmethod
    def _from_setodra(d: dict, max_seq: int = 4096) -> "Config":
        """Setodra ``config.json``: ``width``, ``vocab``, ``norm.eps``, ``embedding.scale``, an optional ``loop`` and ``layers``,
        whose entries give ``type`` (latent_attention | retention | mamba2), the mixer's sizes (``mixer``) and the routed
        feed-forward (``mlp``: kind ``moe`` with ``router``, ``expert.ff`` and an optional ``shared.ff``, or null)."""
        specs = []
        for i, L in enumerate(d["layers"]):
            kind, m = L.get("type"), L["mixer"]
            if kind not in MIXER_KINDS:
                raise ValueError(f"layer {i}: mixer type {kind!r} is not part of this design")
            sp = MixerSpec(type=kind, heads=int(m["heads"]), vdim=int(m["vdim"]), rot=RotarySpec.from_dict(m.get("rot")))
            if kind == "latent_attention":
                sp.dim, sp.rot_dim, sp.kv_rank, sp.scale = int(m["dim"]), int(m["rot_dim"]), int(m["kv_rank"]), float(m["scale"])
            elif kind == "retention":
                sp.dim, sp.decay = int(m["dim"]), [float(x) for x in m["decay"]]
                if len(sp.decay) != sp.heads:
                    raise ValueError(f"layer {i}: {len(sp.decay)} decays for {sp.heads} heads")
            else:
                sp.state, sp.groups, sp.conv, sp.norm_groups = int(m["state"]), int(m["groups"]), int(m["conv"]), int(m["norm_groups"])
            mlp = L.get("mlp")
            if mlp is not None:
                if mlp.get("kind") != "moe":
                    raise ValueError(f"layer {i}: feed-forward kind {mlp.get('kind')!r} is not part of this design")
                r, sh = mlp["router"], mlp.get("shared")
                sp.moe = MoeSpec(experts=int(r["experts"]), identity=int(r.get("identity") or 0), top=int(r["top"]), scale=float(r.get("scale", 1.0)),
                                 ff=int((mlp.get("expert") or {}).get("ff") or 0), shared_ff=int(sh["ff"]) if sh else 0, act=0)
            specs.append(sp)
        if not specs:
            raise ValueError("config lists no layers")
        loop = d.get("loop") or None
        if loop and not (0 <= int(loop["start"]) < int(loop["stop"]) <= len(specs) and int(loop["times"]) >= 1):
            raise ValueError(f"bad loop {loop}")
        cfg = Config(hidden_size=int(d["width"]), intermediate_size=0, vocab_size=int(d["vocab"]), num_hidden_layers=len(specs),
                     num_attention_heads=specs[0].heads, num_key_value_heads=specs[0].heads, rms_norm_eps=float(d["norm"]["eps"]),
                     head_dim=specs[0].vdim, max_seq_len=int(max_seq), block_kind="setodra", layers=specs, model_prefix="",
                     embed_scale=float((d.get("embedding") or {}).get("scale") or 0.0) or None, loop=loop)
        return cfg

    @staticmethod
    def _from_nuvarax(d: dict) -> "Config":
        """Nuvarax ``config.json``: ``width``, ``vocab``, ``norm.eps``, ``max_positions``, ``embedding.{scale, bigram.{buckets,
        mul_prev, mul_cur}}``, ``canon.taps``, an optional ``loop`` and ``layers``, whose entries give ``type`` (``delta``: a gated
        delta rule mixer; ``parallel``: attention with mixed heads (``mixer.left``) beside a matrix memory (``mixer.right``)), the
        mixer's sizes and the dense feed-forward (``mlp``: kind ``dense`` with ``ff`` and ``limit``, or null).  Every norm's gain
        is stored as an offset from one; the output projection is the embedding table."""
        taps = int((d.get("canon") or {}).get("taps") or 0)
        specs = []
        for i, L in enumerate(d["layers"]):
            kind, m = L.get("type"), L["mixer"]
            if kind == "delta":
                sp = MixerSpec(type="delta", heads=int(m["heads"]), kv_heads=int(m.get("kv_heads") or m["heads"]), dim=int(m["dim"]),
                               vdim=int(m["vdim"]), conv=int(m.get("conv") or 0))   # 0: the taps are the convolution tensors' second size
            elif kind == "parallel":
                a, b = m["left"], m["right"]
                sp = MixerSpec(type="talking_attention", heads=int(a["heads"]), kv_heads=int(a.get("kv_heads") or a["heads"]), dim=int(a["dim"]),
                               vdim=int(a["vdim"]), scale=float(a["scale"]), bias_max=float(a.get("bias_max") or 0.0),
                               side=MixerSpec(type="matrix_memory", heads=int(b["heads"]), dim=int(b["dim"]), vdim=int(b["vdim"]),
                                              gate_cap=float(b["gate_cap"])))
            else:
                raise ValueError(f"layer {i}: mixer type {kind!r} is not part of this design")
            if sp.heads % sp.n_kv:
                raise ValueError(f"layer {i}: {sp.heads} heads over {sp.n_kv} key heads")
            mlp = L.get("mlp")
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise ValueError(f"layer {i}: feed-forward kind {mlp.get('kind')!r} is not part of this design")
                sp.dense_ff, sp.dense_act, sp.dense_limit = int(mlp["ff"]), 2, float(mlp["limit"])
            sp.norm_offset, sp.post_norms, sp.canon_taps = 1.0, True, taps
            specs.append(sp)
        if not specs:
            raise ValueError("config lists no layers")
        loop = d.get("loop") or None
        if loop and not (0 <= int(loop["start"]) < int(loop["stop"]) <= len(specs) and int(loop["times"]) >= 1):
            raise ValueError(f"bad loop {loop}")
        emb = d.get("embedding") or {}
        bg = emb.get("bigram") or None
        npos = int(d.get("max_positions") or 0)
        return Config(hidden_size=int(d["width"]), intermediate_size=0, vocab_size=int(d["vocab"]), num_hidden_layers=len(specs),
                      num_attention_heads=specs[0].heads, num_key_value_heads=specs[0].n_kv, rms_norm_eps=float(d["norm"]["eps"]),
                      head_dim=specs[0].vdim, max_seq_len=npos or 4096, block_kind="nuvarax", layers=specs, model_prefix="",
                      embed_scale=float(emb.get("scale") or 0.0) or None, loop=loop, loop_injects=False, tie_word_embeddings=True,
                      pair_embedding={k: int(bg[k]) for k in ("buckets", "mul_prev", "mul_cur")} if bg else None,
                      learned_positions=npos, final_norm_offset=1.0)

    @staticmethod
    def _from_netolorn(d: dict, max_seq: int = 4096) -> "Config":
        """Netolorn ``config.json``: ``width``, ``vocab``, ``norm.eps``, an optional ``token_side.dim``, an optional ``loop`` and
        ``layers``, whose entries give ``type`` (``attention``: grouped-query attention with ``rot`` (dims, base, scaling), ``mask``
        (size, keep_first), ``scale``; ``latent_attention``: ``q_rank``, ``kv_rank``, ``mask.size``, ``scale``), the mixer's sizes
        and the feed-forward (``mlp``: kind ``dense`` with ``ff``; kind ``moe`` with ``router`` (experts, top), ``expert`` (ff, limit)
        and an optional ``shared`` (ff, limit); or null).  Every norm is tanh(alpha x) * w + b."""
        side = int((d.get("token_side") or {}).get("dim") or 0)
        specs = []
        for i, L in enumerate(d["layers"]):
            kind, m = L.get("type"), L["mixer"]
            mask = m.get("mask") or {}
            if kind == "attention":
                sp = MixerSpec(type="sink_attention", heads=int(m["heads"]), kv_heads=int(m.get("kv_heads") or m["heads"]), dim=int(m["dim"]),
                               vdim=int(m.get("vdim") or m["dim"]), scale=float(m["scale"]), rot=RotarySpec.from_dict(m.get("rot")), qk_unit=True,
                               window=int(mask.get("size") or 0), keep_first=int(mask.get("keep_first") or 0))
                if sp.rot.dims % 2 or sp.rot.dims > sp.dim:
                    raise ValueError(f"layer {i}: rot.dims {sp.rot.dims} must be even and at most dim {sp.dim}")
            elif kind == "latent_attention":
                sp = MixerSpec(type="latent_window", heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m.get("vdim") or m["dim"]), scale=float(m["scale"]),
                               q_rank=int(m["q_rank"]), kv_rank=int(m["kv_rank"]), window=int(mask.get("size") or 0))
            else:
                raise ValueError(f"layer {i}: mixer type {kind!r} is not part of this design")
            if sp.heads % sp.n_kv:
                raise ValueError(f"layer {i}: {sp.heads} heads over {sp.n_kv} key heads")
            mlp = L.get("mlp")
            if mlp is not None:
                if mlp.get("kind") == "dense":
                    sp.dense_ff, sp.dense_act = int(mlp["ff"]), 0
                elif mlp.get("kind") == "moe":
                    r, ex, sh = mlp["router"], mlp.get("expert") or {}, mlp.get("shared")
                    sp.moe = MoeSpec(experts=int(r["experts"]), top=int(r["top"]), ff=int(ex["ff"]), limit=float(ex["limit"]), act=2, logit_bias=True,
                                     shared_ff=int(sh["ff"]) if sh else 0, shared_limit=float(sh["limit"]) if sh else 0.0)
                else:
                    raise ValueError(f"layer {i}: feed-forward kind {mlp.get('kind')!r} is not part of this design")
            sp.norm_kind, sp.post_norms, sp.side_dim, sp.side_col = 1, True, side, i * side
            specs.append(sp)
        if not specs:
            raise ValueError("config lists no layers")
        loop = d.get("loop") or None
        if loop and not (0 <= int(loop["start"]) < int(loop["stop"]) <= len(specs) and int(loop["times"]) >= 1):
            raise ValueError(f"bad loop {loop}")
        return Config(hidden_size=int(d["width"]), intermediate_size=0, vocab_size=int(d["vocab"]), num_hidden_layers=len(specs),
                      num_attention_heads=specs[0].heads, num_key_value_heads=specs[0].n_kv, rms_norm_eps=float(d["norm"]["eps"]),
                      head_dim=specs[0].vdim, max_seq_len=int(max_seq), block_kind="netolorn", layers=specs, model_prefix="", loop=loop,
                      loop_mode="project", token_side_dim=side, final_norm_kind=1)

    def to_netolorn(self) -> dict:
        """The ``config.json`` of a Netolorn Config (inverse of ``_from_netolorn``)."""
        layers = []
        for s in self.layers:
            if s.type == "sink_attention":
                mask = {"size": s.window, "keep_first": s.keep_first} if s.window else None
                kind, m = "attention", {"heads": s.heads, "kv_heads": s.n_kv, "dim": s.dim, "vdim": s.vdim, "scale": s.scale, "rot": s.rot.to_dict(), "mask": mask}
            else:
                kind, m = "latent_attention", {"heads": s.heads, "dim": s.dim, "vdim": s.vdim, "scale": s.scale, "q_rank": s.q_rank, "kv_rank": s.kv_rank,
                                               "mask": {"size": s.window} if s.window else None}
            mo = s.moe
            if mo is not None:
                mlp = {"kind": "moe", "router": {"experts": mo.experts, "top": mo.top}, "expert": {"ff": mo.ff, "limit": mo.limit},
                       "shared": {"ff": mo.shared_ff, "limit": mo.shared_limit} if mo.shared_ff else None}
            else:
                mlp = {"kind": "dense", "ff": s.dense_ff} if s.dense_ff else None
            layers.append({"type": kind, "mixer": m, "mlp": mlp})
        d = {"architecture": "Netolorn", "width": self.hidden_size, "vocab": self.vocab_size, "norm": {"eps": self.rms_norm_eps}, "layers": layers}
        if self.token_side_dim:
            d["token_side"] = {"dim": self.token_side_dim}
        if self.loop:
            d["loop"] = dict(self.loop)
        return d

    def to_nuvarax(self) -> dict:
        """The ``config.json`` of a Nuvarax Config (inverse of ``_from_nuvarax``)."""
        layers = []
        for s in self.layers:
            if s.type == "delta":
                kind, m = "delta", {"heads": s.heads, "kv_heads": s.n_kv, "dim": s.dim, "vdim": s.vdim, "conv": s.conv}
            else:
                r = s.side
                kind, m = "parallel", {"left": {"heads": s.heads, "kv_heads": s.n_kv, "dim": s.dim, "vdim": s.vdim, "scale": s.scale, "bias_max": s.bias_max},
                                       "right": {"heads": r.heads, "dim": r.dim, "vdim": r.vdim, "gate_cap": r.gate_cap}}
            layers.append({"type": kind, "mixer": m, "mlp": {"kind": "dense", "ff": s.dense_ff, "limit": s.dense_limit} if s.dense_ff else None})
        d = {"architecture": "Nuvarax", "width": self.hidden_size, "vocab": self.vocab_size, "norm": {"eps": self.rms_norm_eps},
             "max_positions": self.learned_positions, "canon": {"taps": self.layers[0].canon_taps},
             "embedding": {"scale": self.embed_scale if self.embed_scale else 1.0, "bigram": dict(self.pair_embedding) if self.pair_embedding else None},
             "layers": layers}
        if self.loop:
            d["loop"] = dict(self.loop)
        return d

    def to_setodra(self) -> dict:
        """The ``config.json`` of a mixer-list Config (inverse of ``_from_setodra``)."""
        layers = []
        for s in self.layers:
            if s.type == "latent_attention":
                m = {"heads": s.heads, "dim": s.dim, "rot_dim": s.rot_dim, "vdim": s.vdim, "kv_rank": s.kv_rank, "scale": s.scale, "rot": s.rot.to_dict()}
            elif s.type == "retention":
                m = {"heads": s.heads, "dim": s.dim, "vdim": s.vdim, "decay": list(s.decay), "rot": s.rot.to_dict()}
            else:
                m = {"heads": s.heads, "vdim": s.vdim, "state": s.state, "groups": s.groups, "conv": s.conv, "norm_groups": s.norm_groups}
            mo = s.moe
            mlp = None if mo is None else {"kind": "moe", "router": {"experts": mo.experts, "identity": mo.identity, "top": mo.top, "scale": mo.scale},
                                           "expert": {"ff": mo.ff}, "shared": {"ff": mo.shared_ff} if mo.shared_ff else None}
            layers.append({"type": s.type, "mixer": m, "mlp": mlp})
        d = {"architecture": "Setodra", "width": self.hidden_size, "vocab": self.vocab_size, "norm": {"eps": self.rms_norm_eps},
             "embedding": {"scale": self.embed_scale if self.embed_scale else 1.0}, "layers": layers}
        if self.loop:
            d["loop"] = dict(self.loop)
        return d

    def to_nigenex(self) -> dict:
        """The ``config.json`` of a layer-list Config (inverse of ``_from_nigenex``)."""
        return {"architecture": "Nigenex", "width": self.hidden_size, "vocab": self.vocab_size, "norm": {"eps": self.rms_norm_eps},
                "logit_softcap": self.logit_softcap,
                "layers": [{"type": "attention",
                            "mixer": {"heads": s.heads, "kv_heads": s.kv_heads, "dim": s.head_dim, "vdim": s.head_dim, "scale": s.scale,
                                      "softcap": s.softcap, "mask": {"size": s.window}},
                            "mlp": {"kind": "dense", "ff": s.ff} if s.ff else None} for s in self.layers]}

    @staticmethod
    def from_hf(d: dict) -> "Config":
        if d.get("architecture") == "Nigenex":  # a single string, not HF's ``architectures`` list
            return Config._from_nigenex(d)
        if d.get("architecture") == "Setodra":
            return Config._from_setodra(d)
        if d.get("architecture") == "Nuvarax":
            return Config._from_nuvarax(d)
        if d.get("architecture") == "Netolorn":
            return Config._from_netolorn(d)
        arch = Config.detect_arch(d)
        if arch in Config._OTHER_BLOCKS:
            raise ValueError(f"architecture {arch!r} is outside the block-forward path built here")
        if arch in Config._SIBLING_BLOCKS:
            return Config._from_hf_sibling(d, Config._SIBLING_BLOCKS[arch])
        rope_default, max_default, flags = Config._ARCHS.get(arch, Config._ARCHS["LlamaForCausalLM"])
        rs = d.get("rope_scaling")
        rope = None
        if rs:
            rope = RopeScaling(
                # serde defaults of the reference's RopeScaling: every missing number is 0.0 (config.rs)
                factor=float(rs.get("factor", 0.0)),
                low_freq_factor=float(rs.get("low_freq_factor", 0.0)),
                high_freq_factor=float(rs.get("high_freq_factor", 0.0)),
                original_max_position_embeddings=int(rs.get("original_max_position_embeddings", 0)),
                rope_type=rs.get("rope_type"),
            )
        eos = d.get("eos_token_id")
        eos = [] if eos is None else (list(eos) if isinstance(eos, (list, tuple)) else [eos])
        return Config(
            hidden_size=d["hidden_size"],
            intermediate_size=d["intermediate_size"],
            vocab_size=d["vocab_size"],
            num_hidden_layers=d["num_hidden_layers"],
            num_attention_heads=d["num_attention_heads"],
            num_key_value_heads=d.get("num_key_value_heads") or d["num_attention_heads"],
            rms_norm_eps=d["rms_norm_eps"],
            rope_theta=float(d.get("rope_theta") or rope_default),
            rope_scaling=rope,
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            max_seq_len=int(d.get("max_position_embeddings") or max_default),
            eos_token_id=eos,
            use_qkv_bias=bool(flags.get("use_qkv_bias", False)),
            use_qk_norm=bool(flags.get("use_qk_norm", False)),
            head_dim=d.get("head_dim") if flags.get("_head_dim") else None,
            sliding_window=d.get("sliding_window") if flags.get("_sliding_window") else None,
            partial_rotary_factor=float(d.get("partial_rotary_factor") or 1.0) if flags.get("_partial") else 1.0,
            fused_qkv_proj=bool(flags.get("_fused")), fused_gate_up_proj=bool(flags.get("_fused")),
        )

    @staticmethod
    def _from_hf_sibling(d: dict, kind: str) -> "Config":
        """models/{gemma3,olmo2,exaone4}/config.rs ``into_config``: the serde defaults and the flags each hard-wires."""
        n = int(d["num_hidden_layers"])
        rs = d.get("rope_scaling")
        rope = RopeScaling(factor=float(rs.get("factor", 0.0)), low_freq_factor=float(rs.get("low_freq_factor", 0.0)),
                           high_freq_factor=float(rs.get("high_freq_factor", 0.0)),
                           original_max_position_embeddings=int(rs.get("original_max_position_embeddings", 0)),
                           rope_type=rs.get("rope_type")) if rs else None
        eos = d.get("eos_token_id")
        eos = [] if eos is None else (list(eos) if isinstance(eos, (list, tuple)) else [eos])
        base = dict(hidden_size=d["hidden_size"], intermediate_size=d["intermediate_size"], vocab_size=d["vocab_size"],
                    num_hidden_layers=n, num_attention_heads=d["num_attention_heads"],
                    num_key_value_heads=d.get("num_key_value_heads") or d["num_attention_heads"],
                    rms_norm_eps=d["rms_norm_eps"], rope_scaling=rope, eos_token_id=eos, head_dim=d.get("head_dim"),
                    use_qk_norm=True, block_kind=kind)
        if kind == "olmo2":    # olmo2/config.rs:52-90
            return Config(**base, rope_theta=float(d.get("rope_theta") or 500000.0),
                          tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
                          max_seq_len=int(d.get("max_position_embeddings") or 4096), pre_reshape_qk_norm=True)
        if kind == "exaone4":  # exaone4/config.rs:62-110: every `global_layer_period`-th layer is global
            period = int(d.get("global_layer_period") or 4)
            return Config(**base, rope_theta=float(d.get("rope_theta") or 500000.0),
                          tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
                          max_seq_len=int(d.get("max_position_embeddings") or 131072),
                          sliding_window=int(d.get("sliding_window") or 4096),
                          global_layers=[(i + 1) % period == 0 for i in range(n)])
        # gemma3/config.rs:76-125: explicit schedule (true = global) or every `sliding_window_pattern`-th layer
        sched = d.get("sliding_window_attention_schedule") or []
        pattern = int(d.get("sliding_window_pattern") or 6)
        gl = [bool(sched[i]) if i < len(sched) else False for i in range(n)] if sched else [(i + 1) % pattern == 0 for i in range(n)]
        return Config(**base, rope_theta=float(d.get("rope_theta") or 10000.0), tie_word_embeddings=True,
                      max_seq_len=int(d.get("max_position_embeddings") or 131072),
                      sliding_window=int(d.get("sliding_window") or 1024), global_layers=gl, residual_rms_norm=True,
                      use_gelu_mlp=True, embed_scale=float(np.sqrt(np.float32(d["hidden_size"]))))

    @staticmethod
    def from_path(path: str) -> "Config":
        with open(path) as f:
            return Config.from_hf(json.load(f))

    def to_hf(self, arch: str = "LlamaForCausalLM") -> dict:
        if self.block_kind == "nigenex":
            return self.to_nigenex()
        if self.block_kind == "setodra":
            return self.to_setodra()
        if self.block_kind == "nuvarax":
            return self.to_nuvarax()
        if self.block_kind == "netolorn":
            return self.to_netolorn()
        d = dict(
            architectures=[arch], hidden_size=self.hidden_size, intermediate_size=self.intermediate_size,
            vocab_size=self.vocab_size, num_hidden_layers=self.num_hidden_layers,
            num_attention_heads=self.num_attention_heads, num_key_value_heads=self.num_key_value_heads,
            rms_norm_eps=self.rms_norm_eps, rope_theta=self.rope_theta,
            tie_word_embeddings=self.tie_word_embeddings, max_position_embeddings=self.max_seq_len,
        )
        if self.head_dim:
            d["head_dim"] = self.head_dim
        if self.sliding_window:
            d["sliding_window"] = self.sliding_window
        if self.partial_rotary_factor != 1.0:
            d["partial_rotary_factor"] = self.partial_rotary_factor
        if self.rope_scaling:
            d["rope_scaling"] = asdict(self.rope_scaling)
        # the keys the sibling architectures' config.rs read (models/{gemma3,exaone4}/config.rs)
        if self.block_kind == "gemma3":
            d["sliding_window_attention_schedule"] = [bool(g) for g in self.global_layers]
        elif self.block_kind == "exaone4":
            hits = [i + 1 for i, g in enumerate(self.global_layers) if g]
            period = hits[0] if hits else self.num_hidden_layers + 1
            if [(i + 1) % period == 0 for i in range(self.num_hidden_layers)] != [bool(g) for g in self.global_layers]:
                raise ValueError("EXAONE4 can only express an every-n-th global-layer schedule (global_layer_period)")
            d["global_layer_period"] = period
        return d

    def is_eos(self, tok: int) -> bool:
        # config.rs:6-19 EosTokenId::is_eos
        return tok in self.eos_token_id


class CConfig(ctypes.Structure):
    """``cake_b200_config`` from include/cake_b200.h (and the oracle's ora_config prefix)."""
    _fields_ = [
        ("hidden", ctypes.c_int), ("inter", ctypes.c_int), ("n_heads", ctypes.c_int),
        ("n_kv_heads", ctypes.c_int), ("head_dim", ctypes.c_int), ("n_layers", ctypes.c_int),
        ("vocab", ctypes.c_int), ("max_seq", ctypes.c_int),
        ("rms_eps", ctypes.c_float), ("rope_theta", ctypes.c_float), ("partial_rotary", ctypes.c_float),
        ("qkv_bias", ctypes.c_int), ("qk_norm", ctypes.c_int), ("tie_embeddings", ctypes.c_int),
        ("rope_llama3", ctypes.c_int),
        ("rope_factor", ctypes.c_float), ("rope_low", ctypes.c_float), ("rope_high", ctypes.c_float),
        ("rope_orig_max", ctypes.c_int),
        ("dtype", ctypes.c_int),
        ("sliding_window", ctypes.c_int), ("use_gelu_mlp", ctypes.c_int), ("embed_scale", ctypes.c_float),
        ("pre_reshape_qk_norm", ctypes.c_int),
        ("layer_list", ctypes.c_int), ("logit_softcap", ctypes.c_float), ("scalar_final_norm", ctypes.c_int),
    ]

    @staticmethod
    def from_config(c: Config, dtype: str = "bf16", max_seq: Optional[int] = None) -> "CConfig":
        rs = c.rope_scaling
        llama3 = bool(rs and rs.rope_type == "llama3" and rs.original_max_position_embeddings > 0)
        # cache.rs:173-205 limit = min(window, max_seq_len); a window that never bites is passed as 0
        win = int(c.sliding_window) if (c.sliding_window and c.sliding_window < (max_seq or c.max_seq_len)) else 0
        return CConfig(
            c.hidden_size, c.intermediate_size, c.num_attention_heads, c.num_key_value_heads, c.hd,
            len(c.run_plan()) if c.layer_list else c.num_hidden_layers, c.vocab_size, max_seq or c.max_seq_len,
            c.rms_norm_eps, c.rope_theta, c.partial_rotary_factor,
            int(c.use_qkv_bias), int(c.use_qk_norm), int(c.tie_word_embeddings),
            int(llama3),
            rs.factor if llama3 else 1.0, rs.low_freq_factor if llama3 else 1.0,
            rs.high_freq_factor if llama3 else 4.0, rs.original_max_position_embeddings if llama3 else 0,
            DTYPES[dtype],
            win, int(c.use_gelu_mlp), float(c.embed_scale or 0.0), int(c.pre_reshape_qk_norm),
            int(c.layer_list), float(c.logit_softcap), int(c.scalar_final_norm),
        )


# Named shapes used by tests / bench.
def llama3_8b(max_seq: int = 8192) -> Config:
    return Config(4096, 14336, 128256, 32, 32, 8, rms_norm_eps=1e-5, rope_theta=500000.0, max_seq_len=max_seq,
                  eos_token_id=[128001, 128009])


def llama3_70b(max_seq: int = 8192) -> Config:
    return Config(8192, 28672, 128256, 80, 64, 8, rms_norm_eps=1e-5, rope_theta=500000.0, max_seq_len=max_seq,
                  eos_token_id=[128001, 128009])


def qwen3_0_6b(max_seq: int = 4096) -> Config:
    return Config(1024, 3072, 151936, 28, 16, 8, rms_norm_eps=1e-6, rope_theta=1000000.0, max_seq_len=max_seq,
                  head_dim=128, use_qk_norm=True, tie_word_embeddings=True, eos_token_id=[151645])


def reference_test_config(**kw) -> Config:
    """tests/unit_tests/helpers.rs:8-44 ``test_config()``."""
    base = dict(hidden_size=64, intermediate_size=128, vocab_size=256, num_hidden_layers=4,
                num_attention_heads=4, num_key_value_heads=2, rms_norm_eps=1e-6, rope_theta=10000.0,
                max_seq_len=64)
    base.update(kw)
    return Config(**base)
