"""ctypes binding of libeos_b200.so (the C ABI declared in include/eos_b200.h).

The library is loaded from this directory; nothing here falls back to a CPU implementation:
without the built library, or without a compute-capability 10.x device, calls raise.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("EOS_B200_LIBRARY") or os.path.join(_HERE, "libeos_b200.so")

OK, ERROR, DEVICE_STATUS = 0, 1, 2


class EosB200Error(RuntimeError):
    """A C-ABI call returned 1."""


class EosB200DeviceStatusError(EosB200Error):
    """A C-ABI call returned 2: a kernel flagged bad input (for example an out-of-range token id)."""


class Stats(C.Structure):
    _fields_ = [("kernel_launches", C.c_int32), ("reserved", C.c_int32), ("uploaded_bytes", C.c_int64),
                ("downloaded_bytes", C.c_int64), ("valid_tokens", C.c_int64), ("device_ms", C.c_float),
                ("reserved2", C.c_float)]


class TokenPoolDesc(C.Structure):
    _fields_ = [("vocab", C.c_int32), ("dim", C.c_int32), ("hidden", C.c_int32), ("encoder_repeats", C.c_int32),
                ("attention_residual", C.c_int32), ("attention_layer_norm", C.c_int32), ("ffn_residual", C.c_int32),
                ("ffn_layer_norm", C.c_int32), ("token_embedding", C.c_void_p), ("attention_query", C.c_void_p),
                ("attention_key", C.c_void_p), ("attention_value", C.c_void_p), ("attention_output", C.c_void_p),
                ("hidden_projection", C.c_void_p), ("projection", C.c_void_p)]


class EncoderTimes(C.Structure):
    _fields_ = [("steps", C.c_int32), ("gemm_launches", C.c_int32), ("attention_launches", C.c_int32),
                ("layernorm_launches", C.c_int32), ("other_launches", C.c_int32), ("gemm_ms", C.c_float),
                ("attention_ms", C.c_float), ("layernorm_ms", C.c_float), ("embed_ms", C.c_float),
                ("pool_ms", C.c_float), ("layout_ms", C.c_float), ("gemm_kind_ms", C.c_float * 4)]


class DeviceInfo(C.Structure):
    _fields_ = [("device", C.c_int32), ("cc_major", C.c_int32), ("cc_minor", C.c_int32), ("sm_count", C.c_int32),
                ("total_memory_bytes", C.c_int64), ("name", C.c_char * 128)]


class Matrix(C.Structure):
    _fields_ = [("rows", C.c_int32), ("cols", C.c_int32), ("q8_codes", C.c_void_p), ("q8_scales", C.c_void_p),
                ("n_scales", C.c_int32), ("reserved", C.c_int32), ("dense", C.c_void_p)]


class EncoderLayer(C.Structure):
    _fields_ = [("query", Matrix), ("query_bias", C.c_void_p), ("key", Matrix), ("key_bias", C.c_void_p),
                ("value", Matrix), ("value_bias", C.c_void_p), ("attn_out", Matrix), ("attn_out_bias", C.c_void_p),
                ("attn_ln_gamma", C.c_void_p), ("attn_ln_beta", C.c_void_p), ("inter", Matrix),
                ("inter_bias", C.c_void_p), ("out", Matrix), ("out_bias", C.c_void_p), ("out_ln_gamma", C.c_void_p),
                ("out_ln_beta", C.c_void_p)]


class EncoderDesc(C.Structure):
    _fields_ = [("layers", C.c_int32), ("hidden", C.c_int32), ("heads", C.c_int32), ("intermediate", C.c_int32),
                ("vocab", C.c_int32), ("max_positions", C.c_int32), ("type_vocab", C.c_int32),
                ("activation", C.c_int32), ("pooling", C.c_int32), ("weight_mode", C.c_int32),
                ("attention_window", C.c_int32), ("head_out", C.c_int32), ("epsilon", C.c_double),
                ("token_embeddings", C.c_void_p), ("position_embeddings", C.c_void_p),
                ("type_embeddings", C.c_void_p), ("embedding_ln_gamma", C.c_void_p),
                ("embedding_ln_beta", C.c_void_p), ("layer", C.POINTER(EncoderLayer)), ("head_weights", C.c_void_p)]


class CompactLayer(C.Structure):
    _fields_ = [("attn_q", Matrix), ("attn_k", Matrix), ("attn_v", Matrix), ("attn_o", Matrix), ("ffn_up", Matrix),
                ("ffn_down", Matrix)]


class CompactEncoderDesc(C.Structure):
    _fields_ = [("layers", C.c_int32), ("hidden", C.c_int32), ("heads", C.c_int32), ("intermediate", C.c_int32),
                ("vocab", C.c_int32), ("role_vocab", C.c_int32), ("output_dim", C.c_int32), ("weight_mode", C.c_int32),
                ("token_embedding", C.c_void_p), ("role_embedding", C.c_void_p), ("layer", C.POINTER(CompactLayer)),
                ("output_projection", Matrix)]


# name -> (restype, argtypes); every symbol include/eos_b200.h declares
_P = C.c_void_p
_ERR = C.POINTER(C.c_char_p)
SYMBOLS = {
    "eos_b200_runtime_create": (C.c_int, [C.c_int, C.POINTER(_P), _ERR]),
    "eos_b200_runtime_destroy": (None, [_P]),
    "eos_b200_runtime_info": (C.c_int, [_P, C.POINTER(DeviceInfo), _ERR]),
    "eos_b200_selftest_bounded_wait": (C.c_int, [_P, C.c_int64, _ERR]),
    "eos_b200_free_cstring": (None, [_P]),
    "eos_b200_version": (C.c_char_p, []),
    "eos_b200_encoder_bind": (C.c_int, [_P, C.POINTER(EncoderDesc), C.POINTER(_P), _ERR]),
    "eos_b200_compact_encoder_bind": (C.c_int, [_P, C.POINTER(CompactEncoderDesc), C.POINTER(_P), _ERR]),
    "eos_b200_encoder_destroy": (None, [_P]),
    "eos_b200_encoder_reserve": (C.c_int, [_P, C.c_int, C.c_int, _ERR]),
    "eos_b200_encoder_run": (C.c_int, [_P, _P, _P, _P, C.c_int, C.c_int, _P, C.POINTER(Stats), _ERR]),
    "eos_b200_encoder_submit": (C.c_int, [_P, _P, _P, _P, C.c_int, C.c_int, _P, _ERR]),
    "eos_b200_encoder_wait": (C.c_int, [_P, C.POINTER(Stats), _ERR]),
    "eos_b200_encoder_run_device": (C.c_int, [_P, _P, _P, _P, C.c_int, C.c_int, _P, _P, C.POINTER(Stats), _ERR]),
    "eos_b200_encoder_set_token_head": (C.c_int, [_P, _P, C.c_int, _ERR]),
    "eos_b200_encoder_token_vectors_device": (C.c_int, [_P, _P, _P, _P, C.c_int, C.c_int, _P, _P, _P, C.POINTER(Stats),
                                                        _ERR]),
    "eos_b200_encoder_sync": (C.c_int, [_P, _P, _ERR]),
    "eos_b200_encoder_profile_begin": (C.c_int, [_P, C.c_int, _ERR]),
    "eos_b200_encoder_profile_end": (C.c_int, [_P, _P, C.POINTER(EncoderTimes), _ERR]),
    "eos_b200_corpus_profile_begin": (C.c_int, [_P, C.c_int, _ERR]),
    "eos_b200_corpus_profile_end": (C.c_int, [_P, _P, C.POINTER(C.c_float), C.POINTER(C.c_int), _ERR]),
    "eos_b200_linear": (C.c_int, [_P, _P, C.c_int64, C.POINTER(Matrix), _P, C.c_int, _P, C.c_int, _P,
                                  C.POINTER(Stats), _ERR]),
    "eos_b200_embed_pooled_bind": (C.c_int, [_P, _P, C.c_int, C.c_int, _P, C.c_int, C.POINTER(_P), _ERR]),
    "eos_b200_embed_pooled_destroy": (None, [_P]),
    "eos_b200_embed_pooled_run": (C.c_int, [_P, _P, _P, C.c_int, C.c_int, C.c_int, _P, C.POINTER(Stats), _ERR]),
    "eos_b200_quantizer_create": (C.c_int, [_P, C.c_int, C.c_int, _P, _P, _P, _P, _P, C.POINTER(_P), _ERR]),
    "eos_b200_quantizer_destroy": (None, [_P]),
    "eos_b200_quantize": (C.c_int, [_P, _P, C.c_int64, _P, _P, C.POINTER(Stats), _ERR]),
    "eos_b200_quantize_device": (C.c_int, [_P, _P, C.c_int64, _P, _P, _P, _ERR]),
    "eos_b200_corpus_bind": (C.c_int, [_P, _P, _P, C.c_int64, C.c_int64, C.c_int, C.POINTER(_P), _ERR]),
    "eos_b200_corpus_bind_device": (C.c_int, [_P, _P, _P, C.c_int64, C.c_int64, C.POINTER(_P), _ERR]),
    "eos_b200_corpus_destroy": (None, [_P]),
    "eos_b200_corpus_vector_bytes": (C.c_int64, [_P]),
    "eos_b200_score_topk": (C.c_int, [_P, _P, C.c_int, C.c_int, C.c_int, _P, _P, C.POINTER(Stats), _ERR]),
    "eos_b200_score_topk_device": (C.c_int, [_P, _P, C.c_int, C.c_int, C.c_int, _P, _P, _P, _P, C.POINTER(Stats),
                                             _ERR]),
    "eos_b200_score_seed_device": (C.c_int, [_P, _P, C.c_int, C.c_int, _P, _P, _ERR]),
    "eos_b200_score_topk_seeded_device": (C.c_int, [_P, _P, C.c_int, C.c_int, _P, _P, _P, _P, _P, C.POINTER(Stats),
                                                    _ERR]),
    "eos_b200_corpus_sync": (C.c_int, [_P, _P, _ERR]),
    "eos_b200_score_topk_noalloc": (C.c_int, [_P, _P, C.c_int, C.c_int, C.c_int, _P, _P, _P, _ERR]),
    "eos_b200_topk_merge_device": (C.c_int, [_P, _P, C.c_int, C.c_int, C.c_int, _P, _P, _P, _ERR]),
    "eos_b200_comm_unique_id": (C.c_int, [_P, _ERR]),
    "eos_b200_comm_init": (C.c_int, [_P, C.c_int, C.c_int, _P, C.POINTER(_P), _ERR]),
    "eos_b200_comm_destroy": (None, [_P]),
    "eos_b200_score_topk_sharded": (C.c_int, [_P, _P, _P, C.c_int, C.c_int, C.c_int, _P, _P, _P, C.POINTER(Stats),
                                              _ERR]),
    "eos_b200_maxsim_topk_device": (C.c_int, [_P, _P, C.c_int, C.c_int, C.c_int, C.c_int, _P, _P, _P, _P,
                                              C.POINTER(Stats), _ERR]),
    "eos_b200_comm_merge_keys": (C.c_int, [_P, _P, C.c_int, C.c_int, _P, _P, _P, _ERR]),
    "eos_b200_score_all": (C.c_int, [_P, _P, C.c_int, _P, _ERR]),
    "eos_b200_parent_topk": (C.c_int, [_P, _P, C.c_int, _P, C.c_int, C.c_int, C.c_int, C.c_double, C.c_int, _P, _P,
                                       C.POINTER(Stats), _ERR]),
    "eos_b200_dense_bind": (C.c_int, [_P, _P, C.c_int64, C.c_int, C.c_int, C.POINTER(_P), _ERR]),
    "eos_b200_dense_destroy": (None, [_P]),
    "eos_b200_dense_score_topk": (C.c_int, [_P, _P, C.c_int, C.c_int, C.c_int, _P, _P, C.POINTER(Stats), _ERR]),
    "eos_b200_dense_rerank": (C.c_int, [_P, _P, C.c_int, _P, C.c_int, C.c_int, _P, _P, C.POINTER(Stats), _ERR]),
    "eos_b200_ip_corpus_bind": (C.c_int, [_P, C.c_int, C.c_int, _P, _P, _P, _P, _P, _P, _P, _P, C.c_int64, C.c_int64, C.c_int,
                                          C.POINTER(C.c_void_p), _ERR]),
    "eos_b200_ip_corpus_destroy": (None, [_P]),
    "eos_b200_ip_corpus_vector_bytes": (C.c_int64, [C.c_int, C.c_int]),
    "eos_b200_norm_encode_log8": (None, [_P, C.c_int64, _P]),
    "eos_b200_norm_decode_log8": (None, [_P, C.c_int64, _P]),
    "eos_b200_embed_pooled_set_matmul_scale": (C.c_int, [_P, C.c_float, _ERR]),
    "eos_b200_ip_score_topk": (C.c_int, [_P, _P, _P, C.c_float, C.c_int, C.c_int, _P, _P, C.POINTER(Stats), _ERR]),
    "eos_b200_token_pool_bind": (C.c_int, [_P, C.POINTER(TokenPoolDesc), C.POINTER(C.c_void_p), _ERR]),
    "eos_b200_token_pool_destroy": (None, [_P]),
    "eos_b200_token_pool_encode": (C.c_int, [_P, _P, _P, C.c_int, C.c_int, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int,
                                             C.c_int, C.c_int, _P, _P, _P, C.c_int, C.POINTER(C.c_int), C.POINTER(Stats),
                                             _ERR]),
    "eos_b200_sparse_attention": (C.c_int, [_P, _P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                            C.c_int, _P, C.POINTER(Stats), _ERR]),
    "eos_b200_turbo_sparse_attention": (C.c_int, [_P, _P, _P, _P, _P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                                  C.c_int, _P, C.POINTER(Stats), _ERR]),
    "eos_b200_synth_gaussian_device": (C.c_int, [_P, C.c_uint64, C.c_int64, C.c_int64, C.c_int, C.c_int, _P, _P,
                                                 _ERR]),
}

_lib = None


def lib() -> C.CDLL:
    """Loads libeos_b200.so (raises if it has not been built: there is no other code path)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise EosB200Error(f"{LIB_PATH} is missing: build it with `python -m eos_b200.build` "
                               "(there is no CPU or PyTorch fallback)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(rc: int, err: C.c_char_p) -> None:
    if rc == OK:
        return
    msg = err.value.decode("utf-8", "replace") if err.value else "unknown error"
    if err.value:
        # the message is malloc'd by the library and owned by the caller
        lib().eos_b200_free_cstring(C.cast(err, C.c_void_p))
    if rc == DEVICE_STATUS:
        raise EosB200DeviceStatusError(msg)
    raise EosB200Error(msg)


def call(name: str, *args) -> None:
    """Calls an int-returning entry point with a trailing char** err and raises on failure."""
    err = C.c_char_p()
    rc = getattr(lib(), name)(*args, C.byref(err))
    check(rc, err)
