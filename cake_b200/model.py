"""Host-side mirror of the reference's interface for the block-forward path, over the C ABI.

Same names, argument meaning and error behaviour as the reference so that tests read like its own:

  Forwarder            cake-core/src/cake/mod.rs:510-556   (load / forward / forward_mut / forward_batch /
                                                            goodbye / layer_name / ident)
  B200Transformer      models/common/transformer.rs:14-150 (`type Shardable`, the local block)
  Cache                models/common/cache.rs:9-254        (clear / as_new; K,V live on the GPU)
  Context              cake/mod.rs:41-65                   (config, dtype, device, var_builder, cache, topology)
  TextModelBase        models/common/text_model.rs:133-530 (forward / prepare_prompt / next_token / reset / goodbye)
  Master               cake/sharding/master.rs:14-191      (generate_text and its tok/s definition)

torch is used for device memory and (in parallel.py) torch.distributed rendezvous only.  There is no
PyTorch or CPU fallback: every forward goes through libcake_b200.so.
"""
from __future__ import annotations

import ctypes
import time
import weakref
from abc import ABC, abstractmethod
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import capi
from .capi import byref, c_uint32, c_void_p, check, int_array, lib, ptr, ptr_array
from .config import CConfig, Config
from .synth import TORCH_DTYPES


class Cache:
    """KV cache of one session (cache.rs:9).  RoPE tables live in the ctx (computed once per model)."""

    def __init__(self, ctx: "Context", batch: int = 1, max_seq: Optional[int] = None):
        self.ctx, self.batch = ctx, batch
        self.max_seq = max_seq or ctx.max_seq
        self.h = c_void_p()
        self._lib = lib()  # a handle is only ever given back to the library that made it
        check(self._lib.cake_b200_cache_create(ctx.h, batch, self.max_seq, byref(self.h)))
        ctx._children.append(weakref.ref(self))

    def close(self):
        if self.h:
            self._lib.cake_b200_cache_free(self.h)
            self.h = None

    def clear(self) -> None:  # cache.rs:247-253
        check(lib().cake_b200_cache_clear(self.h))

    def as_new(self) -> "Cache":  # cache.rs:241-245
        return Cache(self.ctx, self.batch, self.max_seq)

    def with_kv_cache(self) -> bool:
        return True

    def len(self, block_idx: int) -> int:
        return lib().cake_b200_cache_len(self.h, block_idx)

    def kv(self, block_idx: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """(K, V) copies of shape (batch, n_kv, len, hd) on the host, dtype D (a layer whose values are its keys returns
        the same tensor twice: it keeps no V cache)."""
        c = self.ctx.config
        n = self.len(block_idx)
        out = []
        if c.layer_list:
            sp = c.layers[block_idx]
            t = torch.empty((self.batch, sp.kv_heads, n, sp.head_dim), dtype=TORCH_DTYPES[self.ctx.dtype])
            check(lib().cake_b200_cache_read(self.h, block_idx, 0, ptr(t), t.numel() * t.element_size()))
            return t, t
        for which in (0, 1):
            t = torch.empty((self.batch, c.num_key_value_heads, n, c.hd), dtype=TORCH_DTYPES[self.ctx.dtype])
            check(lib().cake_b200_cache_read(self.h, block_idx, which, ptr(t), t.numel() * t.element_size()))
            out.append(t)
        return out[0], out[1]

    def fill_synthetic(self, block_idx: Sequence[int], length: int, seed: int = 7) -> None:
        check(lib().cake_b200_cache_fill_synthetic(self.h, int_array(list(block_idx)), len(block_idx), length, seed))

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Context:
    """cake/mod.rs:41-65: shared state handed to Forwarder::load / forward."""

    def __init__(self, config: Config, var_builder: Dict[str, torch.Tensor], dtype: str = "bf16", device: int = 0,
                 max_seq: Optional[int] = None, topology: Optional[dict] = None):
        if not torch.cuda.is_available():
            raise RuntimeError("cake_b200 needs a CUDA device (B200, sm_100a); there is no CPU fallback")
        self.config, self.var_builder, self.dtype, self.device = config, var_builder, dtype, device
        self.max_seq = max_seq or config.max_seq_len
        self.topology = topology or {}
        self.ccfg = CConfig.from_config(config, dtype, self.max_seq)
        self.h = c_void_p()
        self._children = []  # weakrefs to caches / blocks: freed before the ctx (they point into it)
        torch.cuda.set_device(device)
        check(lib().cake_b200_ctx_create(device, byref(self.ccfg), byref(self.h)))
        self.cache: Optional[Cache] = Cache(self)
        self.torch_dtype = TORCH_DTYPES[dtype]
        # layer-list models keep the residual stream in fp32 and hand their samplers 16-bit logits (bf16 when D is fp32)
        self.stream_dtype = torch.float32 if config.layer_list else self.torch_dtype
        self.logits_dtype = torch.bfloat16 if dtype == "f32" else self.torch_dtype
        # torch sees the library's stream as an ExternalStream: tensors handed to the C ABI are allocated
        # on it, so the caching allocator orders their reuse after the kernels that touch them.
        self.torch_stream = torch.cuda.ExternalStream(self.stream_ptr, device=device)

    def sync(self) -> None:
        check(lib().cake_b200_sync(self.h))

    @property
    def stream_ptr(self) -> int:
        return lib().cake_b200_stream(self.h)

    def launch_count(self) -> int:
        n = ctypes.c_uint64()
        check(lib().cake_b200_launch_count(self.h, byref(n)))
        return n.value

    def empty(self, *shape, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        with torch.cuda.stream(self.torch_stream):
            return torch.empty(shape, dtype=dtype or self.torch_dtype, device=f"cuda:{self.device}")

    def to_device(self, t: torch.Tensor) -> torch.Tensor:
        """Host tensor (values in D) -> device tensor on the library's stream."""
        with torch.cuda.stream(self.torch_stream):
            return t.to(self.torch_dtype).to(f"cuda:{self.device}", non_blocking=False)

    def close(self):
        if self.h:
            self.sync()
            for ref in self._children:
                obj = ref()
                if obj is not None:
                    obj.close()
            self._children = []
            self.cache = None
            lib().cake_b200_ctx_destroy(self.h)
            self.h = None


class Forwarder(ABC):
    """cake/mod.rs:510-556."""

    @classmethod
    @abstractmethod
    def load(cls, name: str, ctx: Context) -> "Forwarder": ...

    @abstractmethod
    def forward(self, x: torch.Tensor, index_pos: int, block_idx: int, ctx: Context) -> torch.Tensor: ...

    def forward_mut(self, x, index_pos, block_idx, ctx):
        return self.forward(x, index_pos, block_idx, ctx)

    def forward_batch(self, x, batch: List[Tuple[str, int, int]], ctx):
        raise NotImplementedError  # mod.rs:538-543 unimplemented!() by default

    def goodbye(self) -> None:
        return None

    @abstractmethod
    def layer_name(self) -> str: ...

    def ident(self) -> str:
        return "local"


def _layer_index(name: str) -> int:
    return int(name.rsplit(".", 1)[1])


class B200Transformer(Forwarder):
    """The local transformer block (`type Shardable = Transformer`, llama.rs:52 / qwen3/model.rs:24),
    backed by a cake_b200_block handle."""

    def __init__(self, name: str, handle: c_void_p, ctx: Context):
        self.name, self.h = name, handle
        self._lib = lib()
        ctx._children.append(weakref.ref(self))

    def close(self):
        if self.h:
            self._lib.cake_b200_block_free(self.h)
            self.h = None

    @classmethod
    def load(cls, name: str, ctx: Context) -> "B200Transformer":
        from .loader import BLOCK_TENSORS, block_tensors
        views = block_tensors(ctx.var_builder, ctx.config, name)
        keep = []
        for short in BLOCK_TENSORS:  # the argument order of cake_b200_block_load
            t = views[short]
            if t is not None:
                if t.dtype != ctx.torch_dtype:
                    t = t.to(ctx.torch_dtype)
                t = t.contiguous()   # row views of a fused tensor are contiguous already
            keep.append(t)
        h = c_void_p()
        check(lib().cake_b200_block_load(ctx.h, _layer_index(name), *[ptr(t) for t in keep], byref(h)))
        blk = cls(name, h, ctx)
        # the sibling block structures (models/{olmo2,gemma3,exaone4}/block.rs): post-norms and the per-layer attention mode
        var = ctx.config.layer_variant(_layer_index(name), getattr(ctx, "max_seq", None))
        if var["post_norms"] or var["window"] >= 0 or var["no_rope"]:
            from .capi import CBlockVariant
            extra = []
            for k in ("post_attn_norm", "post_ffn_norm"):
                t = views.get(k)
                if t is not None:
                    t = t.to(ctx.torch_dtype).contiguous()
                extra.append(t)
            cv = CBlockVariant(var["window"], 0 if var["no_rope"] else 1, ptr(extra[0]), ptr(extra[1]))
            check(lib().cake_b200_block_set_variant(h, byref(cv)))
        return blk

    def forward(self, x, index_pos, block_idx, ctx):
        return self.forward_batch(x, [(self.name, index_pos, block_idx)], ctx, blocks=[self])

    def forward_batch(self, x, batch, ctx, blocks: Optional[List["B200Transformer"]] = None):
        """x: (b, s, H) device tensor in D.  `batch` = [(layer_name, index_pos, block_idx)] for
        consecutive local layers (text_model.rs:298-321); all entries share index_pos."""
        blocks = blocks or [self]
        assert len(blocks) == len(batch)
        b, s, _ = x.shape
        with torch.cuda.stream(ctx.torch_stream):
            x = x.contiguous()
            y = torch.empty_like(x)
        cache = ctx.cache
        if cache is None:
            raise RuntimeError("No cache specified")  # transformer.rs:120 expect()
        check(lib().cake_b200_forward_batch(ctx.h, ptr_array([blk.h for blk in blocks]),
                                            int_array([bi for _, _, bi in batch]), len(blocks), cache.h,
                                            ptr(x), ptr(y), b, s, batch[0][1]))
        return y

    def forward_host(self, x_host: np.ndarray, index_pos: int, block_idx: int, ctx: Context) -> np.ndarray:
        """Forwarder::forward with HOST buffers (uint16 bit patterns of D), copies inside the call."""
        b, s, H = x_host.shape
        y = np.empty_like(x_host)
        check(lib().cake_b200_forward_batch_host(ctx.h, ptr_array([self.h]), int_array([block_idx]), 1, ctx.cache.h,
                                                 ptr(x_host), ptr(y), b, s, index_pos))
        return y

    def layer_name(self) -> str:
        return self.name

    def __str__(self):
        return f"{self.name} (local)"  # transformer.rs:72-76

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class ListedBlock(B200Transformer):
    """A layer of a layer-list model (``Config.layers``; ``cake_b200_block_load_spec``): same Forwarder surface and the same
    ``cake_b200_forward_batch`` call as the Llama-family block, with an fp32 activation."""

    @classmethod
    def load(cls, name: str, ctx: Context) -> "ListedBlock":
        from .capi import CLayerSpec, CLayerTensors
        from .loader import LISTED_TENSORS, listed_block_tensors
        cfg = ctx.config
        index = [cfg.layer_name(i) for i in range(cfg.num_hidden_layers)].index(name)
        sp = cfg.layers[index]
        views = listed_block_tensors(ctx.var_builder, cfg, index)
        keep = {}
        for fld, _ in LISTED_TENSORS:
            t = views[fld]
            keep[fld] = None if t is None else t.to(ctx.torch_dtype).contiguous()
        spec = CLayerSpec(sp.heads, sp.kv_heads, sp.head_dim, sp.window, sp.scale, sp.softcap, 1, sp.ff, sp.act, 1)
        tens = CLayerTensors(*[ptr(keep[fld]) for fld, _ in LISTED_TENSORS])
        h = c_void_p()
        check(lib().cake_b200_block_load_spec(ctx.h, index, byref(spec), byref(tens), byref(h)))
        return cls(name, h, ctx)


class MixerBlock(B200Transformer):
    """A layer of a mixer-list model (``Config.layers`` of MixerSpec; ``cake_b200_block_load_mixer``): same Forwarder surface
    and the same ``cake_b200_forward_batch`` call, fp32 activation.  A layer inside a looped range is loaded once and run
    under one block_idx (cache slot) per pass."""

    @classmethod
    def load(cls, name: str, ctx: Context) -> "MixerBlock":
        from .loader import mixer_block_tensors
        cfg = ctx.config
        index = [cfg.layer_name(i) for i in range(len(cfg.layers))].index(name)
        sp = cfg.layers[index]
        views = mixer_block_tensors(ctx.var_builder, cfg, index)
        keep = []
        spec, tens = _mixer_struct(sp, views, ctx, keep)
        h = c_void_p()
        check(lib().cake_b200_block_load_mixer(ctx.h, index, byref(spec), byref(tens), byref(h)))
        return cls(name, h, ctx)


def _mixer_struct(sp, views, ctx, keep):
    """(CMixerSpec, CMixerTensors) of one MixerSpec and its tensors (by field name; missing = NULL); device / host copies
    that must outlive the load call are appended to ``keep``."""
    from .capi import CMixerSpec, CMixerTensors, CMoeSpec, CRotarySpec, MIXER_TENSOR_FIELDS, MIXER_TENSOR_FIELDS_2
    from .config import MIXER_KINDS
    args = {}
    for fld in MIXER_TENSOR_FIELDS + MIXER_TENSOR_FIELDS_2:
        t = views.get(fld)
        if isinstance(t, list):
            ts = [x.to(ctx.torch_dtype).contiguous() for x in t]
            keep.append(ts)
            arr = ptr_array([ptr(x) for x in ts]) if ts else None
            keep.append(arr)
            args[fld] = arr
        elif fld.startswith("e_"):
            args[fld] = None
        else:
            t = None if t is None else t.to(ctx.torch_dtype).contiguous()
            keep.append(t)
            args[fld] = ptr(t)
    r, mo = sp.rot, sp.moe
    decay = (ctypes.c_float * max(1, len(sp.decay)))(*sp.decay)
    keep.append(decay)
    spec = CMixerSpec(MIXER_KINDS[sp.type], sp.heads, sp.dim, sp.vdim, sp.rot_dim, sp.kv_rank, sp.scale,
                      CRotarySpec(r.dims, r.base, r.factor, r.fast, r.slow, r.original),
                      decay if sp.decay else None, sp.state, sp.groups, sp.conv, sp.norm_groups,
                      CMoeSpec(mo.experts, mo.identity, mo.top, mo.scale, mo.ff, mo.shared_ff, mo.act, mo.limit, mo.shared_limit, int(mo.logit_bias))
                      if mo else CMoeSpec(),
                      sp.kv_heads, sp.bias_rows, sp.bias_max, sp.gate_cap, sp.norm_offset, sp.canon_taps, sp.dense_ff, sp.dense_act,
                      sp.dense_limit, None, sp.window, sp.keep_first, int(sp.qk_unit), sp.q_rank, sp.norm_kind, (ctypes.c_float * 4)(*sp.norm_alpha),
                      sp.side_dim, sp.side_col)
    return spec, CMixerTensors(**args)


class SandwichBlock(MixerBlock):
    """A layer of a Nuvarax model: a mixer-list block (``cake_b200_block_load_mixer``) with the structure switches set — gains
    stored as offsets from one, a norm behind every sublayer, a convolution in front of the mixer, a dense clamped
    feed-forward — whose mixer is a gated delta rule or attention with mixed heads beside a matrix memory."""

    @classmethod
    def load(cls, name: str, ctx: Context) -> "SandwichBlock":
        from .loader import nuvarax_block_tensors
        cfg = ctx.config
        index = [cfg.layer_name(i) for i in range(len(cfg.layers))].index(name)
        sp = cfg.layers[index]
        main, side = nuvarax_block_tensors(ctx.var_builder, cfg, index)
        keep = []
        spec, tens = _mixer_struct(sp, main, ctx, keep)
        if side is not None:
            sspec, stens = _mixer_struct(sp.side, side, ctx, keep)
            keep += [sspec, stens]
            spec.side, tens.side = ctypes.pointer(sspec), ctypes.pointer(stens)
        h = c_void_p()
        check(lib().cake_b200_block_load_mixer(ctx.h, index, byref(spec), byref(tens), byref(h)))
        return cls(name, h, ctx)


class SquashBlock(MixerBlock):
    """A layer of a Netolorn model: a mixer-list block (``cake_b200_block_load_mixer``) with the squashing norm on both sides of
    every sublayer, a per-layer token input behind the feed-forward, a dense or routed (clamped, logit-biased) feed-forward, and
    sink attention or windowed latent attention as its mixer."""

    @classmethod
    def load(cls, name: str, ctx: Context) -> "SquashBlock":
        from .loader import netolorn_block_tensors
        cfg = ctx.config
        index = [cfg.layer_name(i) for i in range(len(cfg.layers))].index(name)
        sp = cfg.layers[index]
        views = netolorn_block_tensors(ctx.var_builder, cfg, index)   # also fills sp.norm_alpha
        keep = []
        spec, tens = _mixer_struct(sp, views, ctx, keep)
        h = c_void_p()
        check(lib().cake_b200_block_load_mixer(ctx.h, index, byref(spec), byref(tens), byref(h)))
        return cls(name, h, ctx)


# Config.block_kind -> the Forwarder that loads and runs its layers
BLOCK_CLASSES = {"nigenex": ListedBlock, "setodra": MixerBlock, "nuvarax": SandwichBlock, "netolorn": SquashBlock}


@dataclass
class Token:
    id: int
    text: Optional[str]
    is_end_of_stream: bool


class TextModelBase:
    """text_model.rs:133-530 for token-id prompts (tokenizer / chat template stay in the caller)."""

    def __init__(self, ctx: Context, blocks: List[Forwarder], repeat_penalty: float = 1.0, repeat_last_n: int = 128,
                 temperature: float = 0.0, top_k: Optional[int] = None, top_p: Optional[float] = None, seed: int = 299792458):
        """temperature / top_k / top_p / seed: the reference's Args that create_logits_processor reads
        (text_model.rs:102-118): temperature <= 0 -> ArgMax, else GumbelSoftmax | TopK | TopP | TopKThenTopP."""
        self.ctx, self.blocks = ctx, blocks
        self.sampling = sampling_from_args(temperature, top_k, top_p, seed)
        self.tokens: List[int] = []
        self.index_pos = 0
        self.generated = 0
        self.prompt_len = 0
        self.repeat_penalty, self.repeat_last_n = repeat_penalty, repeat_last_n
        self._graph_ready = False

    @classmethod
    def load(cls, ctx: Context, block_cls=None, make_remote: Optional[Callable] = None, **kw):
        """text_model.rs:150-264: embed, lm_head (tied -> embed), ln_f, then one block per layer —
        local ones via Forwarder::load, layers the topology assigns elsewhere via `make_remote`.  The block class follows
        the config (``BLOCK_CLASSES``) unless one is given."""
        cfg, vb = ctx.config, ctx.var_builder
        block_cls = block_cls or BLOCK_CLASSES.get(cfg.block_kind, B200Transformer)
        def get(tname: str, shape):
            t = vb[tname]
            if shape == () and t.numel() == 1:
                t = t.reshape(())      # a one-number gain may be stored as [] or [1]
            if tuple(t.shape) != tuple(shape):
                raise ValueError(f"shape mismatch for {tname}, expected: {list(shape)}, got: {list(t.shape)}")
            return t.to(ctx.torch_dtype).contiguous()

        n_emb, n_norm, n_head = cfg.head_tensor_names()
        emb = get(n_emb, (cfg.vocab_size, cfg.hidden_size))
        from .loader import rms_norm_weight
        lnf = rms_norm_weight(get(n_norm, () if cfg.scalar_final_norm else (cfg.hidden_size,)), cfg)   # text_model.rs:186-192
        head = None if n_head is None else get(n_head, (cfg.vocab_size, cfg.hidden_size))
        check(lib().cake_b200_head_load(ctx.h, ptr(emb), ptr(lnf), ptr(head)))
        tables = cfg.pair_embedding or cfg.learned_positions or cfg.final_norm_offset or cfg.token_side_dim or cfg.final_norm_kind
        if tables:   # embeddings that depend on a token's place in its sequence; the final norm's gain offset or squashing form; the token inputs
            from .capi import CEmbedTables
            pe = cfg.pair_embedding
            big = get("bigram", (pe["buckets"] + 1, cfg.hidden_size)) if pe else None
            pos = vb["pos"].to(ctx.torch_dtype).contiguous() if cfg.learned_positions else None
            if pos is not None and (pos.dim() != 2 or pos.shape[1] != cfg.hidden_size):
                raise ValueError(f"shape mismatch for pos, expected: [positions, {cfg.hidden_size}], got: {list(pos.shape)}")
            side_cols = cfg.token_side_dim * len(cfg.layers)
            side = get("side.embed", (cfg.vocab_size, side_cols)) if cfg.token_side_dim else None
            fb = get(n_norm + ".b", (cfg.hidden_size,)) if cfg.final_norm_kind else None
            fa = float(get(n_norm + ".alpha", ()).to(torch.float32)) if cfg.final_norm_kind else 0.0
            et = CEmbedTables(ptr(big), pe["buckets"] + 1 if pe else 0, pe["mul_prev"] if pe else 0, pe["mul_cur"] if pe else 0,
                              ptr(pos), int(pos.shape[0]) if pos is not None else 0, float(cfg.final_norm_offset),
                              ptr(side), side_cols, int(cfg.final_norm_kind), fa, ptr(fb))
            check(lib().cake_b200_head_load_tables(ctx.h, byref(et)))
        blocks: List[Forwarder] = []
        loaded: Dict[int, Forwarder] = {}   # a layer of a looped range appears once per pass and is loaded once
        plan = cfg.run_plan() if cfg.layer_list else [(i, None) for i in range(cfg.num_hidden_layers)]
        for i, _ in plan:
            if i in loaded:
                blocks.append(loaded[i])
                continue
            name = cfg.layer_name(i)
            owner = _topology_owner(ctx.topology, name)
            if owner is None:
                blocks.append(block_cls.load(name, ctx))
            else:
                if make_remote is None:
                    raise RuntimeError(f"layer {name} is assigned to worker {owner!r} but no transport was given")
                blocks.append(make_remote(owner, name, ctx))
            loaded[i] = blocks[-1]
        model = cls(ctx, blocks, **kw)
        # run index -> pass number, for the runs in front of which the stream receives the pass's additions
        model.injections = {j: t for j, (_, t) in enumerate(plan) if t is not None} if cfg.loop_injects else {}
        model.embed_at = bool(cfg.pair_embedding or cfg.learned_positions)
        model.loop_in = None
        if model.injections and cfg.loop_mode == "project":   # x <- W [x; x0] in front of every pass
            model.loop_in = get("loop.in", (cfg.hidden_size, 2 * cfg.hidden_size))
        elif model.injections:
            steps = get("loop.step", (int(cfg.loop["times"]), cfg.hidden_size))
            model.loop_steps = [steps[t].contiguous() for t in range(steps.shape[0])]
        return model

    # -- forward (text_model.rs:266-368) ---------------------------------------------------------
    def forward(self, ids, idx: int, want: Optional[Sequence[int]] = None) -> torch.Tensor:
        """ids: (batch, seq) token ids at absolute position idx -> logits (batch, vocab) device tensor in D.
        ``want`` (layer-list models): rows b * seq + t whose logits are asked for instead of the last position's ->
        (len(want), vocab) in fp32; an empty list runs the step for its cache and state only and returns None."""
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        b, s = ids.shape
        ctx = self.ctx
        x = ctx.empty(b, s, ctx.config.hidden_size, dtype=ctx.stream_dtype)
        if getattr(self, "embed_at", False):   # the cache supplies the previous token of every row and checks the position
            check(lib().cake_b200_embed_at(ctx.h, ctx.cache.h, ids.ctypes.data_as(ctypes.POINTER(c_uint32)), b, s, idx, ptr(x)))
        else:
            check(lib().cake_b200_embed(ctx.h, ids.ctypes.data_as(ctypes.POINTER(c_uint32)), b, s, ptr(x)))
        n, i = len(self.blocks), 0
        inject = getattr(self, "injections", None) or {}
        x0 = x if inject else None
        if inject:
            with torch.cuda.stream(ctx.torch_stream):
                x = x0.clone()
        while i < n:
            if i in inject:  # a pass of a looped range starts: x += (embedding output, from the second pass on) + step vector
                t = inject[i]
                if getattr(self, "loop_in", None) is not None:
                    check(lib().cake_b200_stream_project(ctx.h, ptr(x), ptr(x0), ptr(self.loop_in), b * s))
                else:
                    check(lib().cake_b200_stream_inject(ctx.h, ptr(x), ptr(x0) if t > 0 else None, ptr(self.loop_steps[t]), t, b * s))
            ident = self.blocks[i].ident()
            j = i
            group = []
            while j < n and self.blocks[j].ident() == ident and (j == i or j not in inject):  # contiguous run on the same node (:298-321)
                group.append((self.blocks[j].layer_name(), idx, j))
                j += 1
            if ident == "local":
                x = self.blocks[i].forward_batch(x, group, ctx, blocks=self.blocks[i:j])
            else:
                x = self.blocks[i].forward_batch(x, group, ctx)
            i = j
        if want is not None:
            if not len(want):
                return None
            rows = int_array([int(w) for w in want])
            logits = ctx.empty(len(want), ctx.config.vocab_size, dtype=torch.float32)
            check(lib().cake_b200_logits_rows(ctx.h, ptr(x), b * s, rows, len(want), ptr(logits)))
            return logits
        logits = ctx.empty(b, ctx.config.vocab_size, dtype=ctx.logits_dtype)
        check(lib().cake_b200_logits(ctx.h, ptr(x), b, s, ptr(logits), None))
        return logits

    # -- generation state (text_model.rs:371-530) ------------------------------------------------
    def prepare_prompt(self, token_ids: Sequence[int]) -> None:
        self.tokens = list(token_ids)
        self.ctx.cache.clear()
        self.index_pos = 0
        self.prompt_len = len(self.tokens)
        self._graph_ready = False

    def next_token(self, index: int) -> Token:
        if index > 0:
            ctx_tokens, ctx_index = self.tokens[-1:], self.index_pos
        else:
            ctx_tokens, ctx_index = self.tokens, 0
        logits = self.forward([ctx_tokens], ctx_index)[0]
        self.index_pos += len(ctx_tokens)
        out = c_uint32()
        if self.repeat_penalty == 1.0:
            pen = []
        else:  # text_model.rs:435-452: only generated tokens, last repeat_last_n of them
            gen = self.tokens[self.prompt_len:]
            pen = gen[max(0, len(gen) - self.repeat_last_n):]
        arr = (c_uint32 * max(1, len(pen)))(*pen)
        if self.sampling.kind == 0:
            check(lib().cake_b200_repeat_penalty_argmax(self.ctx.h, ptr(logits), self.repeat_penalty, arr, len(pen), byref(out)))
        else:  # the sampled token is drawn on the device: only 4 bytes come back (never the 256 KB of logits)
            check(lib().cake_b200_sample(self.ctx.h, ptr(logits), byref(self.sampling), self.repeat_penalty, arr, len(pen),
                                         self.generated, None, byref(out)))
        self.last_logits = logits
        tok = int(out.value)
        self.generated += 1
        self.tokens.append(tok)
        return Token(tok, None, self.ctx.config.is_eos(tok))

    def reset(self) -> None:
        self.tokens.clear()
        self.ctx.cache.clear()
        self.index_pos = self.generated = self.prompt_len = 0
        self._graph_ready = False

    def goodbye(self) -> None:
        for b in self.blocks:
            b.goodbye()

    # -- the graph-captured greedy decode loop (all layers local) ----------------------------------
    def local_handles(self):
        assert all(b.ident() == "local" for b in self.blocks)
        return ptr_array([b.h for b in self.blocks]), int_array(list(range(len(self.blocks))))

    def decode_build(self, rank: int = 0, world: int = 1, blocks: Optional[List[B200Transformer]] = None,
                     block_idx: Optional[List[int]] = None) -> None:
        if rank == 0 and (self.sampling.kind != 0 or getattr(self, "_sampling_set", False)):
            check(lib().cake_b200_decode_set_sampling(self.ctx.h, byref(self.sampling)))
            self._sampling_set = True
        if blocks is None:
            hs, idx = self.local_handles()
            n = len(self.blocks)
        else:
            hs, idx, n = ptr_array([b.h for b in blocks]), int_array(block_idx), len(blocks)
        check(lib().cake_b200_decode_build(self.ctx.h, hs, idx, n, self.ctx.cache.h, rank, world))
        self._graph_ready = True

    def decode_greedy(self, first_token: int, n_steps: int, sync: bool = True) -> List[int]:
        """n_steps greedy tokens fed back on the device (no host work between steps)."""
        L = lib()
        check(L.cake_b200_decode_begin(self.ctx.h, first_token, self.index_pos))
        check(L.cake_b200_decode_run(self.ctx.h, n_steps))
        self.index_pos += n_steps
        if not sync:
            return []
        out = (c_uint32 * n_steps)()
        check(L.cake_b200_decode_tokens(self.ctx.h, out, n_steps))
        toks = [int(t) for t in out]
        self.tokens.extend(toks)
        self.generated += n_steps
        return toks


class Sessions:
    """Requests that run one after the other or interleaved over ONE model: every live request id owns a Cache (its K rows
    and, for layer-list models, its token-shift state); a finished request gives its cache back and the next request reuses
    it after ``clear()`` (worker.rs:60-75 gives every connection its own cache the same way).  A step feeds the request's
    next tokens at the position its cache has reached."""

    def __init__(self, model: TextModelBase, max_seq: Optional[int] = None):
        self.model, self.max_seq = model, max_seq
        self.live: Dict[str, Cache] = {}
        self.free: List[Cache] = []

    def cache_of(self, rid: str) -> Cache:
        c = self.live.get(rid)
        if c is None:
            c = self.free.pop() if self.free else Cache(self.model.ctx, 1, self.max_seq)
            c.clear()
            self.live[rid] = c
        return c

    def step(self, rid: str, tokens: Sequence[int], want: Optional[Sequence[int]] = None) -> Optional[torch.Tensor]:
        cache = self.cache_of(rid)
        ctx = self.model.ctx
        prev, ctx.cache = ctx.cache, cache
        try:
            return self.model.forward([list(tokens)], cache.len(0), want=want)
        finally:
            ctx.cache = prev

    def end(self, rid: str) -> None:
        c = self.live.pop(rid, None)
        if c is not None:
            self.free.append(c)


def sampling_from_args(temperature: float, top_k: Optional[int], top_p: Optional[float], seed: int) -> "capi.CSampling":
    """text_model.rs:102-118 create_logits_processor."""
    if temperature is None or temperature <= 0.0:
        kind = 0
    elif top_k is None and top_p is None:
        kind = 5
    elif top_p is None:
        kind = 2
    elif top_k is None:
        kind = 3
    else:
        kind = 4
    return capi.CSampling(kind, int(top_k or 0), float(temperature or 0.0), float(top_p or 0.0), int(seed))


def _topology_owner(topology: dict, layer_name: str) -> Optional[str]:
    """topology.rs:44-56 Node::is_text_model_layer_owner over expanded layer lists."""
    for worker, node in (topology or {}).items():
        if layer_name in node.get("layers", []):
            return worker
    return None


class Master:
    """sharding/master.rs:14-191 for token-id prompts."""

    def __init__(self, model: TextModelBase):
        self.model = model

    def generate_text(self, prompt_ids: Sequence[int], sample_len: int,
                      stream: Optional[Callable[[Token], None]] = None) -> dict:
        """master.rs:109-168.  tok/s = (generated - 1) / time since the first token (:131-134,160-166)."""
        m = self.model
        m.prepare_prompt(prompt_ids)
        start = time.perf_counter()
        out: List[int] = []
        for index in range(sample_len):
            if index == 1:
                start = time.perf_counter()  # master.rs:132-134: timer restarts after the first token
            tok = m.next_token(index)
            if tok.is_end_of_stream:
                break
            out.append(tok.id)
            if stream:
                stream(tok)
        dt = time.perf_counter() - start
        n = m.generated
        return {"tokens": out, "generated": n, "tok_s": (n - 1) / dt if n > 1 and dt > 0 else 0.0}

    def goodbye(self):
        self.model.goodbye()
