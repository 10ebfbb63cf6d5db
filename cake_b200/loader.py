"""Weight loading: HF safetensors checkpoints -> host tensors that alias the mmapped shards.

Mirrors the reference's loading path for the block-forward scope:

  utils/mod.rs:160-206     model.safetensors | model.safetensors.index.json -> shard list
  utils/mod.rs:250-267     load_var_builder_from_index            (every shard)
  utils/mod.rs:272-329     load_var_builder_for_local_layers      (master: skip shards that hold only worker layers)
  utils/mod.rs:334-384     load_var_builder_for_specific_layers   (worker: only shards that hold its layers)
  utils/mod.rs:209-247     prefetch_safetensors                   (here: madvise(WILLNEED) on the mapping)
  cake/mod.rs:335-357      weight-prefix auto-detection from the index ("….layers.0.")

The safetensors container is parsed here (8-byte little-endian header length, JSON header, raw little-endian
tensor bytes) rather than through a library so that the tensors handed to ``cake_b200_block_load`` are *views of
the mapping*: the H2D copy into the fused qkv / gate_up layouts reads the page cache directly and nothing is staged
twice.  A ``VarBuilder`` is a read-only mapping ``name -> torch.Tensor`` (what ``Context.var_builder`` expects).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from collections.abc import Mapping
from typing import Dict, Iterable, Iterator, List, Optional, Sequence, Tuple

import torch

from .config import Config

INDEX_NAME = "model.safetensors.index.json"
SINGLE_NAME = "model.safetensors"
MAX_HEADER = 100 * 1024 * 1024  # the format's own limit

_DTYPES = {
    "BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F64": torch.float64,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool, "F8_E4M3": torch.float8_e4m3fn, "F8_E5M2": torch.float8_e5m2,
}


class CheckpointError(RuntimeError):
    """Malformed or incomplete checkpoint (the reference bails with an anyhow error naming the file)."""


class SafetensorsFile:
    """One mmapped ``.safetensors`` shard."""

    def __init__(self, path: str):
        self.path = path
        try:
            size = os.path.getsize(path)
            f = open(path, "rb")
        except OSError as e:
            raise CheckpointError(f"can't open {path}: {e}") from e
        with f:
            head = f.read(8)
            if len(head) != 8:
                raise CheckpointError(f"{path}: shorter than a safetensors header")
            (n,) = struct.unpack("<Q", head)
            if n > MAX_HEADER or 8 + n > size:
                raise CheckpointError(f"{path}: header length {n} does not fit the file ({size} bytes)")
            try:
                header = json.loads(f.read(n))
            except (UnicodeDecodeError, json.JSONDecodeError) as e:
                raise CheckpointError(f"{path}: header is not JSON: {e}") from e
            if not isinstance(header, dict):
                raise CheckpointError(f"{path}: header is not a JSON object")
            # private copy-on-write mapping: never written, but a writable buffer lets torch alias it silently
            self._mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_COPY) if size else None
        self.metadata = header.pop("__metadata__", None)
        self._base = 8 + n
        self._entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        data_len = size - self._base
        for name, e in header.items():
            try:
                dt, shape, (b, en) = _DTYPES[e["dtype"]], tuple(int(d) for d in e["shape"]), e["data_offsets"]
            except (KeyError, TypeError, ValueError) as err:
                raise CheckpointError(f"{path}: bad entry for tensor {name!r}: {err!r}") from err
            numel = 1
            for d in shape:
                numel *= d
            if not (0 <= b <= en <= data_len) or en - b != numel * dt.itemsize:
                raise CheckpointError(f"{path}: tensor {name!r} has offsets [{b},{en}) for shape {shape}")
            self._entries[name] = (dt, shape, b, numel)

    def names(self) -> Iterable[str]:
        return self._entries.keys()

    def __contains__(self, name: str) -> bool:
        return name in self._entries

    def nbytes(self, name: str) -> int:
        dt, _, _, numel = self._entries[name]
        return numel * dt.itemsize

    def get(self, name: str) -> torch.Tensor:
        dt, shape, b, numel = self._entries[name]
        if numel == 0:
            return torch.empty(shape, dtype=dt)
        off = self._base + b
        if off % dt.itemsize:  # header not padded to the element size: alias is impossible, copy once
            raw = bytearray(self._mm[off:off + numel * dt.itemsize])
            return torch.frombuffer(raw, dtype=dt, count=numel).view(shape)
        return torch.frombuffer(self._mm, dtype=dt, count=numel, offset=off).view(shape)

    def prefetch(self) -> None:
        """Ask the kernel to read the shard ahead (the reference reads every shard once into a scratch Vec)."""
        if self._mm is not None and hasattr(self._mm, "madvise"):
            self._mm.madvise(mmap.MADV_WILLNEED)


def _read_weight_map(index_path: str) -> Dict[str, str]:
    try:
        with open(index_path) as f:
            j = json.load(f)
    except OSError as e:
        raise CheckpointError(f"can't open {index_path}: {e}") from e
    except json.JSONDecodeError as e:
        raise CheckpointError(f"can't parse {index_path}: {e}") from e
    wm = j.get("weight_map") if isinstance(j, dict) else None
    if wm is None:
        raise CheckpointError(f"no weight map in {index_path}")
    if not isinstance(wm, dict):
        raise CheckpointError(f"weight map in {index_path} is not a map")
    return {k: v for k, v in wm.items() if isinstance(v, str)}


def _under(name: str, prefixes: Iterable[str]) -> bool:
    return any(name.startswith(p + ".") for p in prefixes)


class VarBuilder(Mapping):
    """Read-only ``name -> tensor`` view over a set of shards (candle's mmapped VarBuilder, as the path uses it)."""

    def __init__(self, files: Sequence[SafetensorsFile], prefetch: bool = True):
        self.files = list(files)
        self._where: Dict[str, SafetensorsFile] = {}
        for f in self.files:
            for n in f.names():
                self._where[n] = f
            if prefetch:
                f.prefetch()

    # -- the three reference entry points --------------------------------------------------------
    @classmethod
    def from_index(cls, index_path: str, **kw) -> "VarBuilder":
        """utils/mod.rs:250-267: every shard of the index, or ``model.safetensors`` next to it when there is none."""
        parent = os.path.dirname(index_path) or "."
        if os.path.exists(index_path):
            shards = sorted(set(_read_weight_map(index_path).values()))
        else:
            shards = [SINGLE_NAME]
        return cls([SafetensorsFile(os.path.join(parent, s)) for s in shards], **kw)

    @classmethod
    def for_local_layers(cls, index_path: str, worker_layers: Iterable[str], **kw) -> "VarBuilder":
        """utils/mod.rs:272-329 (master): keep a shard iff it holds at least one tensor that is NOT under a worker layer."""
        worker_layers = set(worker_layers)
        if not os.path.exists(index_path) or not worker_layers:
            return cls.from_index(index_path, **kw)
        parent = os.path.dirname(index_path) or "."
        need = sorted({shard for name, shard in _read_weight_map(index_path).items() if not _under(name, worker_layers)})
        return cls([SafetensorsFile(os.path.join(parent, s)) for s in need], **kw)

    @classmethod
    def for_specific_layers(cls, index_path: str, layer_prefixes: Iterable[str], **kw) -> "VarBuilder":
        """utils/mod.rs:334-384 (worker): keep a shard iff it holds a tensor under one of ``layer_prefixes``."""
        layer_prefixes = list(layer_prefixes)
        if not os.path.exists(index_path) or not layer_prefixes:
            return cls.from_index(index_path, **kw)
        parent = os.path.dirname(index_path) or "."
        need = sorted({shard for name, shard in _read_weight_map(index_path).items() if _under(name, layer_prefixes)})
        return cls([SafetensorsFile(os.path.join(parent, s)) for s in need], **kw)

    # -- Mapping ---------------------------------------------------------------------------------
    def __getitem__(self, name: str) -> torch.Tensor:
        f = self._where.get(name)
        if f is None:
            raise KeyError(f"cannot find tensor {name}")  # candle's VarBuilder error text
        return f.get(name)

    def __iter__(self) -> Iterator[str]:
        return iter(self._where)

    def __len__(self) -> int:
        return len(self._where)

    def __contains__(self, name) -> bool:
        return name in self._where

    def shard_paths(self) -> List[str]:
        return [f.path for f in self.files]

    def nbytes(self) -> int:
        return sum(f.nbytes(n) for n, f in self._where.items())


BLOCK_TENSORS = ("self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight", "self_attn.o_proj.weight",
                 "mlp.gate_proj.weight", "mlp.up_proj.weight", "mlp.down_proj.weight", "input_layernorm.weight",
                 "post_attention_layernorm.weight", "self_attn.q_proj.bias", "self_attn.k_proj.bias", "self_attn.v_proj.bias",
                 "self_attn.q_norm.weight", "self_attn.k_norm.weight")


# the two extra RmsNorm vectors of the sandwich-norm blocks (olmo2/block.rs:49-52, gemma3/block.rs:84-91), by logical role
EXTRA_TENSORS = ("post_attn_norm", "post_ffn_norm")


def rms_norm_weight(t: torch.Tensor, cfg: Config) -> torch.Tensor:
    """config.rs:155-173 load_rms_norm_weight: with ``residual_rms_norm`` the checkpoint stores deltas and the forward
    weight is (1 + w), added in f32 and cast back to the model dtype AT LOAD TIME — the kernels never see the flag."""
    if not cfg.residual_rms_norm:
        return t
    return (t.to(torch.float32) + 1.0).to(t.dtype)


def block_tensors(vb, cfg: Config, name: str) -> Dict[str, Optional[torch.Tensor]]:
    """The tensors `Transformer::load` reads for layer ``name`` (transformer.rs:79-101, attention.rs:76-149,
    mlp.rs:34-59), by the short names of BLOCK_TENSORS, each checked against the shape the layer declares (candle's
    ``vb.get(shape, name)``).  Pre-fused checkpoints (Phi-3/4: ``cfg.fused_qkv_proj`` / ``cfg.fused_gate_up_proj``,
    attention.rs:90-94, mlp.rs:38-40) are split into row views of the fused tensor — q, k, v and gate, up are
    contiguous row ranges of it, so no copy is made.  Biases / QK-norm weights are None unless the config uses them."""
    H, I, sq, skv, hd = cfg.hidden_size, cfg.intermediate_size, cfg.size_q, cfg.size_kv, cfg.hd

    def get(short: str, shape) -> torch.Tensor:
        t = vb.get(f"{name}.{short}")
        if t is None:
            raise KeyError(f"tensor {name}.{short} not found")  # candle VarBuilder error
        if tuple(t.shape) != tuple(shape):
            raise ValueError(f"shape mismatch for {name}.{short}, expected: {list(shape)}, got: {list(t.shape)}")
        return t

    out: Dict[str, Optional[torch.Tensor]] = {k: None for k in BLOCK_TENSORS}
    if cfg.fused_qkv_proj:
        w = get("self_attn.qkv_proj.weight", (sq + 2 * skv, H))
        out["self_attn.q_proj.weight"], out["self_attn.k_proj.weight"], out["self_attn.v_proj.weight"] = \
            w[:sq], w[sq:sq + skv], w[sq + skv:]
    else:
        out["self_attn.q_proj.weight"] = get("self_attn.q_proj.weight", (sq, H))
        out["self_attn.k_proj.weight"] = get("self_attn.k_proj.weight", (skv, H))
        out["self_attn.v_proj.weight"] = get("self_attn.v_proj.weight", (skv, H))
    out["self_attn.o_proj.weight"] = get("self_attn.o_proj.weight", (H, sq))
    if cfg.fused_gate_up_proj:
        w = get("mlp.gate_up_proj.weight", (2 * I, H))
        out["mlp.gate_proj.weight"], out["mlp.up_proj.weight"] = w[:I], w[I:]
    else:
        out["mlp.gate_proj.weight"] = get("mlp.gate_proj.weight", (I, H))
        out["mlp.up_proj.weight"] = get("mlp.up_proj.weight", (I, H))
    out["mlp.down_proj.weight"] = get("mlp.down_proj.weight", (H, I))
    # Norm vectors by ROLE.  out["input_layernorm.weight"] is the pre-attention norm and out["post_attention_layernorm.weight"]
    # the pre-MLP norm (the Llama naming, transformer.rs:84-90); the sibling blocks name theirs differently:
    #   gemma3 (block.rs:84-91): input_layernorm | post_attention_layernorm = POST-attention | pre_feedforward_layernorm = pre-MLP
    #                            | post_feedforward_layernorm
    #   olmo2  (block.rs:49-52): no pre-norms; post_attention_layernorm and post_feedforward_layernorm are post-norms
    kind = getattr(cfg, "block_kind", "llama")
    out.update({k: None for k in EXTRA_TENSORS})
    norm = lambda short: rms_norm_weight(get(short, (H,)), cfg)
    if kind in ("olmo2", "exaone4_hf"):
        out["post_attn_norm"], out["post_ffn_norm"] = norm("post_attention_layernorm.weight"), norm("post_feedforward_layernorm.weight")
    elif kind == "gemma3":
        out["input_layernorm.weight"] = norm("input_layernorm.weight")
        out["post_attn_norm"] = norm("post_attention_layernorm.weight")
        out["post_attention_layernorm.weight"] = norm("pre_feedforward_layernorm.weight")
        out["post_ffn_norm"] = norm("post_feedforward_layernorm.weight")
    else:
        out["input_layernorm.weight"] = norm("input_layernorm.weight")
        out["post_attention_layernorm.weight"] = norm("post_attention_layernorm.weight")
    if cfg.use_qkv_bias:  # attention.rs:96-107 (never together with a fused qkv_proj)
        out["self_attn.q_proj.bias"] = get("self_attn.q_proj.bias", (sq,))
        out["self_attn.k_proj.bias"] = get("self_attn.k_proj.bias", (skv,))
        out["self_attn.v_proj.bias"] = get("self_attn.v_proj.bias", (skv,))
    if cfg.use_qk_norm:   # attention.rs:120-129
        pre = getattr(cfg, "pre_reshape_qk_norm", False)  # attention.rs:121-122: norm dim = size_q / size_kv (OLMo2) or head_dim
        out["self_attn.q_norm.weight"] = rms_norm_weight(get("self_attn.q_norm.weight", (sq if pre else hd,)), cfg)
        out["self_attn.k_norm.weight"] = rms_norm_weight(get("self_attn.k_norm.weight", (skv if pre else hd,)), cfg)
    return out


# argument order of ``cake_b200_layer_tensors`` (include/cake_b200.h) -> tensor name under the layer of a Nigenex checkpoint
LISTED_TENSORS = (("norm", "norm1"), ("shift", "shift"), ("q", "mix.q"), ("k", "mix.k"), ("v", None), ("o", "mix.o"),
                  ("r1", "mix.r1"), ("r2", "mix.r2"), ("gate", "mix.g"), ("ff_gate", "mlp.gate"), ("ff_up", "mlp.up"),
                  ("ff_down", "mlp.down"))


def listed_block_tensors(vb, cfg: Config, index: int) -> Dict[str, Optional[torch.Tensor]]:
    """The tensors of layer ``index`` of a layer-list (Nigenex) checkpoint by the field names of ``cake_b200_layer_tensors``,
    each checked against the shape its LayerSpec declares.  Linear weights are [out, in]; the norm gain is a single number."""
    sp, H, name = cfg.layers[index], cfg.hidden_size, cfg.layer_name(index)
    sq, skv = sp.heads * sp.head_dim, sp.kv_heads * sp.head_dim
    shapes = {"norm": (), "shift": (H,), "q": (sq, H), "k": (skv, H), "o": (H, sq), "r1": (sp.heads,), "r2": (sp.heads,),
              "gate": (sp.heads, H), "ff_gate": (sp.ff, H), "ff_up": (sp.ff, H), "ff_down": (H, sp.ff)}
    out: Dict[str, Optional[torch.Tensor]] = {}
    for fld, short in LISTED_TENSORS:
        if short is None or (fld.startswith("ff_") and not sp.ff):
            out[fld] = None
            continue
        t = vb.get(f"{name}.{short}")
        if t is None:
            raise KeyError(f"tensor {name}.{short} not found")
        if fld == "norm" and t.numel() == 1:
            t = t.reshape(())          # a one-number gain may be stored as [] or [1]
        if tuple(t.shape) != tuple(shapes[fld]):
            raise ValueError(f"shape mismatch for {name}.{short}, expected: {list(shapes[fld])}, got: {list(t.shape)}")
        out[fld] = t
    return out


def mixer_block_tensors(vb, cfg: Config, index: int) -> Dict[str, object]:
    """The tensors of layer ``index`` of a mixer-list (Setodra) checkpoint by the field names of ``cake_b200_mixer_tensors``
    (``e_gate`` / ``e_up`` / ``e_down``: lists, one tensor per expert), each checked against the shape its MixerSpec declares.
    Names under ``l<i>.``: ``norm1``, ``norm2``, ``mix.*`` (the mixer) and ``mlp.*`` (``e<j>.{gate,up,down}``, ``router``,
    ``correction``, ``shared.{gate,up,down,sg}``)."""
    sp, H, name = cfg.layers[index], cfg.hidden_size, cfg.layer_name(index)

    def get(short, shape):
        t = vb.get(f"{name}.{short}")
        if t is None:
            raise KeyError(f"tensor {name}.{short} not found")
        if tuple(t.shape) != tuple(shape):
            raise ValueError(f"shape mismatch for {name}.{short}, expected: {list(shape)}, got: {list(t.shape)}")
        return t

    out: Dict[str, object] = {"norm1": get("norm1", (H,)), "o": get("mix.o", (H, sp.inner))}
    if sp.type == "latent_attention":
        out.update(q=get("mix.q", (sp.heads * (sp.dim + sp.rot_dim), H)), dkv=get("mix.dkv", (sp.kv_rank + sp.rot_dim, H)),
                   dkv_norm=get("mix.dkv.norm", (sp.kv_rank,)), uk=get("mix.uk", (sp.heads * sp.dim, sp.kv_rank)),
                   uv=get("mix.uv", (sp.inner, sp.kv_rank)))
    elif sp.type == "retention":
        out.update(q=get("mix.q", (sp.heads * sp.dim, H)), k=get("mix.k", (sp.heads * sp.dim, H)), v=get("mix.v", (sp.inner, H)),
                   g=get("mix.g", (sp.inner, H)))
    else:
        ch = sp.inner + 2 * sp.groups * sp.state
        out.update({"in": get("mix.in", (2 * sp.inner + 2 * sp.groups * sp.state + sp.heads, H)), "conv": get("mix.conv", (ch, sp.conv)),
                    "conv_b": get("mix.conv.b", (ch,)), "dt_bias": get("mix.dt_bias", (sp.heads,)), "a_log": get("mix.A_log", (sp.heads,)),
                    "d": get("mix.D", (sp.heads,)), "norm": get("mix.norm", (sp.inner,))})
    mo = sp.moe
    if mo is not None:
        et = mo.experts + mo.identity
        out.update(norm2=get("norm2", (H,)), router=get("mlp.router", (et, H)), correction=get("mlp.correction", (et,)),
                   e_gate=[get(f"mlp.e{j}.gate", (mo.ff, H)) for j in range(mo.experts)],
                   e_up=[get(f"mlp.e{j}.up", (mo.ff, H)) for j in range(mo.experts)],
                   e_down=[get(f"mlp.e{j}.down", (H, mo.ff)) for j in range(mo.experts)])
        if mo.shared_ff:
            out.update(s_gate=get("mlp.shared.gate", (mo.shared_ff, H)), s_up=get("mlp.shared.up", (mo.shared_ff, H)),
                       s_down=get("mlp.shared.down", (H, mo.shared_ff)), s_sg=get("mlp.shared.sg", (1, H)))
    return out


def nuvarax_block_tensors(vb, cfg: Config, index: int):
    """The tensors of layer ``index`` of a Nuvarax checkpoint by the field names of ``cake_b200_mixer_tensors``: (main, side or
    None), each checked against the shape its MixerSpec declares.  Names under ``l<i>.``: ``norm1``, ``norm1b``, ``norm2``,
    ``norm2b``, ``canon1``, ``mlp.{gate,up,down}`` and ``mix.*``: a delta layer has ``q, k, v`` (+ ``.conv``), ``b``, ``a``, ``A_log``,
    ``dt_bias``, ``norm``, ``g``, ``o``; a parallel layer ``left.{q,k,v,o}`` (+ ``.b``), ``left.{rel,talk,g,out}`` and
    ``right.{q,k,v,g,o,norm,out}``, ``right.{i,f}`` (+ ``.b``).  The rows of ``rel`` set the spec's ``bias_rows``."""
    sp, H, name = cfg.layers[index], cfg.hidden_size, cfg.layer_name(index)

    def get(short, shape):
        t = vb.get(f"{name}.{short}")
        if t is None:
            raise KeyError(f"tensor {name}.{short} not found")
        if tuple(t.shape) != tuple(shape):
            raise ValueError(f"shape mismatch for {name}.{short}, expected: {list(shape)}, got: {list(t.shape)}")
        return t

    def taps_of(short):   # a size the config may leave to the tensor's shape
        t = vb.get(f"{name}.{short}")
        return int(t.shape[1]) if t is not None and t.dim() == 2 else 0

    if not sp.canon_taps:
        sp.canon_taps = taps_of("canon1")
    if sp.type == "delta" and not sp.conv:
        sp.conv = taps_of("mix.q.conv") or 1
    main = {"norm1": get("norm1", (H,))}
    if sp.post_norms:
        main["post1"] = get("norm1b", (H,))
    if sp.canon_taps >= 1:
        main["canon"] = get("canon1", (H, sp.canon_taps))
    if sp.dense_ff:
        main.update(norm2=get("norm2", (H,)), ff_gate=get("mlp.gate", (sp.dense_ff, H)), ff_up=get("mlp.up", (sp.dense_ff, H)),
                    ff_down=get("mlp.down", (H, sp.dense_ff)))
        if sp.post_norms:
            main["post2"] = get("norm2b", (H,))
    side = None
    if sp.type == "delta":
        qk = sp.n_kv * sp.dim
        main.update(q=get("mix.q", (qk, H)), k=get("mix.k", (qk, H)), v=get("mix.v", (sp.inner, H)), g=get("mix.g", (sp.inner, H)),
                    o=get("mix.o", (H, sp.inner)), q_conv=get("mix.q.conv", (qk, sp.conv)), k_conv=get("mix.k.conv", (qk, sp.conv)),
                    v_conv=get("mix.v.conv", (sp.inner, sp.conv)), beta=get("mix.b", (sp.heads, H)), a_proj=get("mix.a", (sp.heads, H)),
                    a_log=get("mix.A_log", (sp.heads,)), dt_bias=get("mix.dt_bias", (sp.heads,)), norm=get("mix.norm", (sp.vdim,)))
    else:
        r = sp.side
        sq, skv, svv = sp.heads * sp.dim, sp.n_kv * sp.dim, sp.n_kv * sp.vdim
        rel = vb.get(f"{name}.mix.left.rel")
        if rel is None or rel.dim() != 2 or rel.shape[1] != sp.heads:
            raise ValueError(f"{name}.mix.left.rel must be [rows, {sp.heads}]")
        sp.bias_rows = int(rel.shape[0])
        main.update(q=get("mix.left.q", (sq, H)), q_b=get("mix.left.q.b", (sq,)), k=get("mix.left.k", (skv, H)), k_b=get("mix.left.k.b", (skv,)),
                    v=get("mix.left.v", (svv, H)), v_b=get("mix.left.v.b", (svv,)), rel=rel, talk=get("mix.left.talk", (sp.heads, sp.heads)),
                    g=get("mix.left.g", (sp.inner, H)), o=get("mix.left.o", (H, sp.inner)), o_b=get("mix.left.o.b", (H,)),
                    branch_norm=get("mix.left.out", (H,)))
        rq = r.heads * r.dim
        side = dict(q=get("mix.right.q", (rq, H)), k=get("mix.right.k", (rq, H)), v=get("mix.right.v", (r.inner, H)), g=get("mix.right.g", (r.inner, H)),
                    o=get("mix.right.o", (H, r.inner)), norm=get("mix.right.norm", (r.inner,)), i_proj=get("mix.right.i", (r.heads, H)),
                    i_b=get("mix.right.i.b", (r.heads,)), f_proj=get("mix.right.f", (r.heads, H)), f_b=get("mix.right.f.b", (r.heads,)),
                    branch_norm=get("mix.right.out", (H,)))
    return main, side


def netolorn_block_tensors(vb, cfg: Config, index: int) -> Dict[str, object]:
    """The tensors of layer ``index`` of a Netolorn checkpoint by the field names of ``cake_b200_mixer_tensors``, each checked
    against the shape its MixerSpec declares.  Names under ``l<i>.``: ``norm1``, ``norm1b``, ``norm2``, ``norm2b`` (each with ``.b``
    [width] and ``.alpha``, one number, which lands in the spec's ``norm_alpha``), ``side.{gate,proj,norm}`` and ``mix.*``: an
    attention layer has ``q, k, v`` (+ ``.b``), ``sink``, ``g``, ``o``; a latent layer ``dq``, ``dq.norm``, ``uq``, ``dkv``, ``dkv.norm``,
    ``uk``, ``uv``, ``g`` [heads, width], ``o``; ``mlp.{gate,up,down}`` (dense) or ``mlp.{router, router.b, e<j>.*, shared.*}``."""
    sp, H, name = cfg.layers[index], cfg.hidden_size, cfg.layer_name(index)

    def get(short, shape):
        t = vb.get(f"{name}.{short}")
        if t is None:
            raise KeyError(f"tensor {name}.{short} not found")
        if shape == () and t.numel() == 1:
            t = t.reshape(())          # a single number may be stored as [] or [1]
        if tuple(t.shape) != tuple(shape):
            raise ValueError(f"shape mismatch for {name}.{short}, expected: {list(shape)}, got: {list(t.shape)}")
        return t

    has_ff = bool(sp.dense_ff or sp.moe is not None)
    out: Dict[str, object] = {}
    for k, (fld, fld_b, short) in enumerate((("norm1", "norm1_b", "norm1"), ("post1", "post1_b", "norm1b"), ("norm2", "norm2_b", "norm2"),
                                             ("post2", "post2_b", "norm2b"))):
        if k >= 2 and not has_ff:
            continue
        out[fld], out[fld_b] = get(short, (H,)), get(short + ".b", (H,))
        sp.norm_alpha[k] = float(get(short + ".alpha", ()).to(torch.float32))
    out["o"] = get("mix.o", (H, sp.inner))
    if sp.type == "sink_attention":
        sq, skv, svv = sp.heads * sp.dim, sp.n_kv * sp.dim, sp.n_kv * sp.vdim
        out.update(q=get("mix.q", (sq, H)), q_b=get("mix.q.b", (sq,)), k=get("mix.k", (skv, H)), k_b=get("mix.k.b", (skv,)),
                   v=get("mix.v", (svv, H)), v_b=get("mix.v.b", (svv,)), sink=get("mix.sink", (sp.heads,)), g=get("mix.g", (sp.inner, H)))
    else:
        out.update(dq=get("mix.dq", (sp.q_rank, H)), dq_norm=get("mix.dq.norm", (sp.q_rank,)), uq=get("mix.uq", (sp.heads * sp.dim, sp.q_rank)),
                   dkv=get("mix.dkv", (sp.kv_rank, H)), dkv_norm=get("mix.dkv.norm", (sp.kv_rank,)), uk=get("mix.uk", (sp.heads * sp.dim, sp.kv_rank)),
                   uv=get("mix.uv", (sp.inner, sp.kv_rank)), g=get("mix.g", (sp.heads, H)))
    mo = sp.moe
    if sp.dense_ff:
        out.update(ff_gate=get("mlp.gate", (sp.dense_ff, H)), ff_up=get("mlp.up", (sp.dense_ff, H)), ff_down=get("mlp.down", (H, sp.dense_ff)))
    elif mo is not None:
        out.update(router=get("mlp.router", (mo.experts, H)), correction=get("mlp.router.b", (mo.experts,)),
                   e_gate=[get(f"mlp.e{j}.gate", (mo.ff, H)) for j in range(mo.experts)],
                   e_up=[get(f"mlp.e{j}.up", (mo.ff, H)) for j in range(mo.experts)],
                   e_down=[get(f"mlp.e{j}.down", (H, mo.ff)) for j in range(mo.experts)])
        if mo.shared_ff:
            out.update(s_gate=get("mlp.shared.gate", (mo.shared_ff, H)), s_up=get("mlp.shared.up", (mo.shared_ff, H)),
                       s_down=get("mlp.shared.down", (H, mo.shared_ff)), s_sg=get("mlp.shared.sg", (1, H)))
    if sp.side_dim:
        out.update(side_gate=get("side.gate", (sp.side_dim, H)), side_proj=get("side.proj", (H, sp.side_dim)), side_norm=get("side.norm", (H,)))
    return out


def detect_model_prefix(index_path: str, configured: str) -> str:
    """cake/mod.rs:335-357: the text before the first ``.layers.0.`` key of the index wins over the configured prefix."""
    if not os.path.exists(index_path):
        return configured
    try:
        wm = _read_weight_map(index_path)
    except CheckpointError:
        return configured  # the reference ignores an unreadable index at this point
    for key in wm:
        pos = key.find(".layers.0.")
        if pos >= 0:
            return key[:pos]
    return configured


def worker_layer_names(topology: Optional[dict]) -> List[str]:
    """Topology::all_worker_layers (topology.rs:174-185) for an already-expanded topology
    ``{worker: {"layers": [...]}}`` (see parallel.parse_topology)."""
    out: List[str] = []
    for node in (topology or {}).values():
        out.extend(node.get("layers", []))
    return out


def open_model(path: str, topology: Optional[dict] = None, worker: Optional[str] = None,
               prefetch: bool = True) -> Tuple[Config, VarBuilder]:
    """Context::from_args' model part (cake/mod.rs:280-392): ``config.json`` -> Config (prefix auto-detected),
    then the VarBuilder variant the node's role calls for:

    * master (``worker is None``): everything except shards that hold only worker layers;
    * worker ``worker``: only the shards that hold its layers.
    """
    cfg_path = os.path.join(path, "config.json")
    if not os.path.exists(cfg_path):
        raise CheckpointError(f"can't open {cfg_path}")
    cfg = Config.from_path(cfg_path)
    index = os.path.join(path, INDEX_NAME)
    cfg.model_prefix = detect_model_prefix(index, cfg.model_prefix)
    if worker is None:
        vb = VarBuilder.for_local_layers(index, worker_layer_names(topology), prefetch=prefetch)
    else:
        if not topology or worker not in topology:
            raise CheckpointError(f"worker {worker!r} is not in the topology")
        vb = VarBuilder.for_specific_layers(index, topology[worker].get("layers", []), prefetch=prefetch)
    return cfg, vb


def save_checkpoint(path: str, cfg: Config, tensors: Dict[str, torch.Tensor], arch: str = "LlamaForCausalLM",
                    shard_bytes: Optional[int] = None) -> List[str]:
    """Write an HF-layout checkpoint (config.json + model.safetensors, or shards + index when ``shard_bytes`` is
    given).  Test / benchmark utility (the synthetic checkpoints of SURVEY.md §8d); tensors are written in name
    order, a new shard starts when the current one would exceed ``shard_bytes``."""
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg.to_hf(arch), f)  # a layer-list Config writes its own format whatever ``arch`` says
    rev = {v: k for k, v in _DTYPES.items()}
    groups: List[List[str]] = [[]]
    used = 0
    for name in sorted(tensors):
        nb = tensors[name].numel() * tensors[name].element_size()
        if shard_bytes and groups[-1] and used + nb > shard_bytes:
            groups.append([])
            used = 0
        groups[-1].append(name)
        used += nb
    files = [SINGLE_NAME] if len(groups) == 1 and not shard_bytes else \
        [f"model-{i + 1:05d}-of-{len(groups):05d}.safetensors" for i in range(len(groups))]
    weight_map = {}
    for fname, names in zip(files, groups):
        header, off = {}, 0
        for n in names:
            t = tensors[n]
            nb = t.numel() * t.element_size()
            header[n] = {"dtype": rev[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nb]}
            off += nb
            weight_map[n] = fname
        blob = json.dumps(header, separators=(",", ":")).encode()
        blob += b" " * (-len(blob) % 8)  # keep tensor data 8-byte aligned, as the safetensors writers do
        with open(os.path.join(path, fname), "wb") as f:
            f.write(struct.pack("<Q", len(blob)))
            f.write(blob)
            for n in names:
                t = tensors[n].detach().cpu().contiguous()
                f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b"")  # reshape: a 0-dim tensor has no byte view
    if files != [SINGLE_NAME]:
        with open(os.path.join(path, INDEX_NAME), "w") as f:
            json.dump({"metadata": {"total_size": sum(t.numel() * t.element_size() for t in tensors.values())},
                       "weight_map": weight_map}, f)
    return files
