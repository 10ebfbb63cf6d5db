"""ctypes binding of include/cake_b200.h (libcake_b200.so).

There is no CPU fallback: importing this module without the built library, or calling into it
without a B200, raises.  The oracle under oracle/ is test infrastructure and is never imported here.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, byref, c_char_p, c_float, c_int, c_size_t, c_uint32, c_uint64, c_void_p

from .config import CConfig

_HERE = os.path.dirname(os.path.abspath(__file__))
# CAKE_B200_LIB: profiling / A-B builds of the same library (bench_tools/); the product library is the in-tree default
SO_PATH = os.environ.get("CAKE_B200_LIB") or os.path.join(_HERE, "libcake_b200.so")

# every symbol include/cake_b200.h declares: (name, restype, argtypes)
_VP, _I = c_void_p, c_int
SYMBOLS = [
    ("cake_b200_last_error", c_char_p, []),
    ("cake_b200_version", c_char_p, []),
    ("cake_b200_ctx_create", _I, [_I, POINTER(CConfig), POINTER(_VP)]),
    ("cake_b200_ctx_destroy", None, [_VP]),
    ("cake_b200_sync", _I, [_VP]),
    ("cake_b200_stream", _VP, [_VP]),
    ("cake_b200_launch_count", _I, [_VP, POINTER(c_uint64)]),
    ("cake_b200_dev_alloc", _I, [_VP, c_size_t, POINTER(_VP)]),
    ("cake_b200_dev_free", _I, [_VP, _VP]),
    ("cake_b200_block_load", _I, [_VP, _I] + [_VP] * 14 + [POINTER(_VP)]),
    ("cake_b200_block_free", None, [_VP]),
    ("cake_b200_block_layer", _I, [_VP]),
    ("cake_b200_cache_create", _I, [_VP, _I, _I, POINTER(_VP)]),
    ("cake_b200_cache_clear", _I, [_VP]),
    ("cake_b200_cache_free", None, [_VP]),
    ("cake_b200_cache_len", _I, [_VP, _I]),
    ("cake_b200_cache_read", _I, [_VP, _I, _I, _VP, c_size_t]),
    ("cake_b200_cache_fill_synthetic", _I, [_VP, POINTER(_I), _I, _I, c_uint32]),
    ("cake_b200_forward_batch", _I, [_VP, POINTER(_VP), POINTER(_I), _I, _VP, _VP, _VP, _I, _I, _I]),
    ("cake_b200_forward_batch_host", _I, [_VP, POINTER(_VP), POINTER(_I), _I, _VP, _VP, _VP, _I, _I, _I]),
    ("cake_b200_head_load", _I, [_VP, _VP, _VP, _VP]),
    ("cake_b200_embed", _I, [_VP, POINTER(c_uint32), _I, _I, _VP]),
    ("cake_b200_logits", _I, [_VP, _VP, _I, _I, _VP, POINTER(c_uint32)]),
    ("cake_b200_repeat_penalty_argmax", _I, [_VP, _VP, c_float, POINTER(c_uint32), _I, POINTER(c_uint32)]),
    ("cake_b200_comm_unique_id", _I, [_VP]),
    ("cake_b200_comm_init", _I, [_VP, _VP, _I, _I]),
    ("cake_b200_send", _I, [_VP, _VP, c_size_t, _I]),
    ("cake_b200_recv", _I, [_VP, _VP, c_size_t, _I]),
    ("cake_b200_ring_export", _I, [_VP, _VP]),
    ("cake_b200_ring_import", _I, [_VP, _VP]),
    ("cake_b200_decode_build", _I, [_VP, POINTER(_VP), POINTER(_I), _I, _VP, _I, _I]),
    ("cake_b200_decode_begin", _I, [_VP, c_uint32, _I]),
    ("cake_b200_decode_run", _I, [_VP, _I]),
    ("cake_b200_decode_tokens", _I, [_VP, POINTER(c_uint32), _I]),
    ("cake_b200_decode_step_host", _I, [_VP, c_uint32, POINTER(c_uint32)]),
    ("cake_b200_decode_logits", _I, [_VP, _VP, c_size_t]),
    ("cake_b200_bench_kernel", _I, [_VP, POINTER(_VP), POINTER(_I), _I, _VP, _I, _I, POINTER(c_float)]),
    ("cake_b200_decode_trace", _I, [_VP, POINTER(c_uint64), _I]),
]


class CSampling(ctypes.Structure):
    """``cake_b200_sampling`` (include/cake_b200.h)."""
    _fields_ = [("kind", c_int), ("top_k", c_int), ("temperature", c_float), ("top_p", c_float), ("seed", c_uint64)]


SYMBOLS += [
    ("cake_b200_sample", _I, [_VP, _VP, POINTER(CSampling), c_float, POINTER(c_uint32), _I, c_uint64, POINTER(c_float), POINTER(c_uint32)]),
    ("cake_b200_decode_set_sampling", _I, [_VP, POINTER(CSampling)]),
    ("cake_b200_load_stats", _I, [_VP, POINTER(ctypes.c_double), POINTER(ctypes.c_double)]),
]


class CBlockVariant(ctypes.Structure):
    """``cake_b200_block_variant`` (include/cake_b200.h)."""
    _fields_ = [("sliding_window", c_int), ("use_rope", c_int), ("post_attention_norm", _VP), ("post_feedforward_norm", _VP)]


SYMBOLS += [("cake_b200_block_set_variant", _I, [_VP, POINTER(CBlockVariant)])]


class CLayerSpec(ctypes.Structure):
    """``cake_b200_layer_spec`` (include/cake_b200.h)."""
    _fields_ = [("heads", c_int), ("kv_heads", c_int), ("head_dim", c_int), ("window", c_int), ("scale", c_float),
                ("softcap", c_float), ("values_are_keys", c_int), ("ff", c_int), ("act", c_int), ("scalar_norm", c_int)]


class CLayerTensors(ctypes.Structure):
    """``cake_b200_layer_tensors`` (include/cake_b200.h)."""
    _fields_ = [(n, _VP) for n in ("norm", "shift", "q", "k", "v", "o", "r1", "r2", "gate", "ff_gate", "ff_up", "ff_down")]


SYMBOLS += [
    ("cake_b200_block_load_spec", _I, [_VP, _I, POINTER(CLayerSpec), POINTER(CLayerTensors), POINTER(_VP)]),
    ("cake_b200_logits_rows", _I, [_VP, _VP, _I, POINTER(_I), _I, _VP]),
]


class CRotarySpec(ctypes.Structure):
    """``cake_b200_rotary_spec`` (include/cake_b200.h)."""
    _fields_ = [("dims", c_int), ("base", ctypes.c_double), ("yarn_factor", ctypes.c_double), ("yarn_fast", ctypes.c_double),
                ("yarn_slow", ctypes.c_double), ("yarn_original", c_int)]


class CMoeSpec(ctypes.Structure):
    """``cake_b200_moe_spec`` (include/cake_b200.h)."""
    _fields_ = [("experts", c_int), ("identity", c_int), ("top", c_int), ("scale", c_float), ("ff", c_int), ("shared_ff", c_int), ("act", c_int),
                ("limit", c_float), ("shared_limit", c_float), ("logit_bias", c_int)]


class CMixerSpec(ctypes.Structure):
    """``cake_b200_mixer_spec`` (include/cake_b200.h); ``side`` points to the spec of a second mixer beside this one."""


CMixerSpec._fields_ = [("kind", c_int), ("heads", c_int), ("dim", c_int), ("vdim", c_int), ("rot_dim", c_int), ("kv_rank", c_int), ("scale", c_float),
                       ("rot", CRotarySpec), ("decay", POINTER(c_float)), ("state", c_int), ("groups", c_int), ("conv", c_int), ("norm_groups", c_int),
                       ("moe", CMoeSpec),
                       ("kv_heads", c_int), ("bias_rows", c_int), ("bias_max", c_float), ("gate_cap", c_float), ("norm_offset", c_float),
                       ("canon_taps", c_int), ("dense_ff", c_int), ("dense_act", c_int), ("dense_limit", c_float), ("side", POINTER(CMixerSpec)),
                       ("window", c_int), ("keep_first", c_int), ("qk_unit", c_int), ("q_rank", c_int), ("norm_kind", c_int), ("norm_alpha", c_float * 4),
                       ("side_dim", c_int), ("side_col", c_int)]


MIXER_TENSOR_FIELDS = ("norm1", "norm2", "q", "k", "v", "g", "o", "dkv", "dkv_norm", "uk", "uv", "in", "conv", "conv_b", "dt_bias", "a_log", "d",
                       "norm", "router", "correction", "e_gate", "e_up", "e_down", "s_gate", "s_up", "s_down", "s_sg",
                       "post1", "post2", "canon", "q_conv", "k_conv", "v_conv", "beta", "a_proj", "q_b", "k_b", "v_b", "o_b", "rel", "talk",
                       "i_proj", "i_b", "f_proj", "f_b", "ff_gate", "ff_up", "ff_down", "branch_norm")


class CMixerTensors(ctypes.Structure):
    """``cake_b200_mixer_tensors`` (include/cake_b200.h); e_gate / e_up / e_down are arrays of ``experts`` pointers, ``side`` the
    tensors of a second mixer beside this one."""


# fields behind `side` in the C struct (the newer mechanisms)
MIXER_TENSOR_FIELDS_2 = ("sink", "dq", "dq_norm", "uq", "norm1_b", "post1_b", "norm2_b", "post2_b", "side_gate", "side_proj", "side_norm")
CMixerTensors._fields_ = [(n, POINTER(_VP) if n.startswith("e_") else _VP) for n in MIXER_TENSOR_FIELDS] + [("side", POINTER(CMixerTensors))] + \
                         [(n, _VP) for n in MIXER_TENSOR_FIELDS_2]


class CEmbedTables(ctypes.Structure):
    """``cake_b200_embed_tables`` (include/cake_b200.h)."""
    _fields_ = [("bigram", _VP), ("bigram_rows", c_int), ("mul_prev", c_int), ("mul_cur", c_int), ("pos", _VP), ("pos_rows", c_int),
                ("final_norm_offset", c_float), ("side", _VP), ("side_cols", c_int), ("final_norm_kind", c_int), ("final_alpha", c_float),
                ("final_bias", _VP)]


SYMBOLS += [
    ("cake_b200_block_load_mixer", _I, [_VP, _I, POINTER(CMixerSpec), POINTER(CMixerTensors), POINTER(_VP)]),
    ("cake_b200_stream_inject", _I, [_VP, _VP, _VP, _VP, _I, _I]),
    ("cake_b200_stream_project", _I, [_VP, _VP, _VP, _VP, _I]),
    ("cake_b200_head_load_tables", _I, [_VP, POINTER(CEmbedTables)]),
    ("cake_b200_embed_at", _I, [_VP, _VP, POINTER(c_uint32), _I, _I, _I, _VP]),
]


class CakeB200Error(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"cake_b200 error {code}: {msg}")
        self.code = code


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(SO_PATH):
            raise ImportError(
                f"{SO_PATH} is missing: build it with `python -m cake_b200.build` "
                "(libcake_b200 has no CPU or PyTorch fallback)")
        L = ctypes.CDLL(SO_PATH, mode=ctypes.RTLD_GLOBAL)
        for name, res, args in SYMBOLS:
            if os.environ.get("CAKE_B200_LIB") and not hasattr(L, name):
                continue  # A/B against an older build of the library (bench_tools/ab.sh); the product library must export everything
            fn = getattr(L, name)  # AttributeError if the library does not export a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        raise CakeB200Error(rc, lib().cake_b200_last_error().decode(errors="replace"))


def ptr(t) -> int:
    """Raw address of a torch tensor / numpy array / int / None."""
    if t is None:
        return 0
    if isinstance(t, int):
        return t
    if hasattr(t, "data_ptr"):
        return t.data_ptr()
    return t.ctypes.data


def ptr_array(handles):
    return (c_void_p * len(handles))(*handles)


def int_array(vals):
    return (c_int * len(vals))(*vals)


__all__ = ["lib", "check", "ptr", "ptr_array", "int_array", "CakeB200Error", "SYMBOLS", "SO_PATH", "byref",
           "c_uint32", "c_uint64", "c_void_p", "c_int"]
