"""ctypes front end to the CPU oracle (oracle/eos_oracle.c).

TEST INFRASTRUCTURE ONLY.  Importable from tests/, __graft_entry__.smoke() and the
cpu-baseline / reference legs of bench.py; the shipped package never imports it.
Each wrapper takes and returns numpy arrays; see the C file for the Eos source lines every
function follows.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from typing import Optional, Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libeos_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile libeos_oracle.so next to its source (gcc via oracle/Makefile)."""
    src = os.path.join(_HERE, "eos_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "libeos_oracle.so"])
    return _LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.eos_oracle_f16_bits_to_f32.restype = C.c_float
        _lib.eos_oracle_f16_bits_to_f32.argtypes = [C.c_uint16]
        _lib.eos_oracle_f32_to_f16_bits.restype = C.c_uint16
        _lib.eos_oracle_f32_to_f16_bits.argtypes = [C.c_float]
        _lib.eos_oracle_exact_gelu.restype = C.c_float
        _lib.eos_oracle_exact_gelu.argtypes = [C.c_float]
        _lib.eos_oracle_tanh_gelu.restype = C.c_float
        _lib.eos_oracle_tanh_gelu.argtypes = [C.c_float]
        _lib.eos_oracle_tq_code_bytes.restype = C.c_int64
        _lib.eos_oracle_dot.restype = C.c_float
    return _lib


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.int32)


def _p(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def default_workers() -> int:
    return os.cpu_count() or 1


# ----------------------------------------------------------------------------- quant grid
def quantize_symmetric(data, group: int = 0, bits: int = 8, scale_round_f16: bool = False):
    """Returns (int8 codes shaped like data, float32 scales[n/group])."""
    d = _f32(data)
    n = d.size
    g = n if group <= 0 else group
    codes = np.empty(d.shape, dtype=np.int8)
    scales = np.empty((n + g - 1) // g, dtype=np.float32)
    lib().eos_oracle_quantize_symmetric(_p(d), C.c_int64(n), C.c_int64(g), C.c_int(bits),
                                        C.c_int(1 if scale_round_f16 else 0), _p(codes), _p(scales))
    return codes, scales


def dequantize(codes, scales, group: int = 0):
    c = np.ascontiguousarray(codes, dtype=np.int8)
    s = _f32(scales)
    out = np.empty(c.shape, dtype=np.float32)
    lib().eos_oracle_dequantize(_p(c), C.c_int64(c.size), C.c_int64(group if group > 0 else c.size), _p(s), _p(out))
    return out


def f32_to_f16_bits(x: float) -> int:
    return int(lib().eos_oracle_f32_to_f16_bits(C.c_float(x)))


def f16_bits_to_f32(b: int) -> float:
    return float(lib().eos_oracle_f16_bits_to_f32(C.c_uint16(b)))


# ----------------------------------------------------------------------- pipeline tensor ops
def gather(table, indices):
    t = _f32(table)
    idx = _i32(indices)
    out = np.empty(idx.shape + (t.shape[1],), dtype=np.float32)
    rc = lib().eos_oracle_gather(_p(t), C.c_int(t.shape[0]), C.c_int(t.shape[1]), _p(idx), C.c_int64(idx.size), _p(out))
    if rc:
        raise IndexError("gather index out of range")
    return out


def matmul(lhs, rhs, scale: float = 1.0):
    a = _f32(lhs)
    b = _f32(rhs)
    k = a.shape[-1]
    rows = a.size // k
    out = np.empty(a.shape[:-1] + (b.shape[1],), dtype=np.float32)
    lib().eos_oracle_matmul(_p(a), C.c_int64(rows), C.c_int(k), _p(b), C.c_int(b.shape[1]), C.c_float(scale), _p(out))
    return out


def normalize_rows(x):
    a = _f32(x)
    cols = a.shape[-1]
    out = np.empty_like(a)
    lib().eos_oracle_normalize_rows(_p(a), C.c_int64(a.size // cols), C.c_int(cols), _p(out))
    return out


def mean_pool_masked(x, mask):
    a = _f32(x)
    m = _i32(mask)
    b, t, c = a.shape
    out = np.empty((b, c), dtype=np.float32)
    lib().eos_oracle_mean_pool_masked(_p(a), _p(m), C.c_int(b), C.c_int(t), C.c_int(c), _p(out))
    return out


def embed_pooled(table, projection, tokens, mask, pool_then_l2: bool = False, matmul_scale: float = 1.0):
    t = _f32(table)
    pr = _f32(projection)
    tok = _i32(tokens)
    m = _i32(mask)
    b, tl = tok.shape
    out = np.empty((b, pr.shape[1]), dtype=np.float32)
    rc = lib().eos_oracle_embed_pooled(_p(t), C.c_int(t.shape[0]), C.c_int(t.shape[1]), _p(pr), C.c_int(pr.shape[1]),
                                       _p(tok), _p(m), C.c_int(b), C.c_int(tl), C.c_int(1 if pool_then_l2 else 0),
                                       C.c_float(matmul_scale), _p(out))
    if rc:
        raise IndexError("gather index out of range")
    return out


# ------------------------------------------------------------------------------ BERT family
def bert_embeddings(tok, pos, typ, gamma, beta, input_ids, position_ids, type_ids, eps=1e-12):
    tok, pos, typ, gamma, beta = map(_f32, (tok, pos, typ, gamma, beta))
    ids, pids, tids = map(_i32, (input_ids, position_ids, type_ids))
    dim = tok.shape[1]
    out = np.empty(ids.shape + (dim,), dtype=np.float32)
    rc = lib().eos_oracle_bert_embeddings(_p(tok), C.c_int(tok.shape[0]), _p(pos), C.c_int(pos.shape[0]), _p(typ),
                                          C.c_int(typ.shape[0]), _p(gamma), _p(beta), _p(ids), _p(pids), _p(tids),
                                          C.c_int64(ids.size), C.c_int(dim), C.c_double(eps), _p(out))
    if rc:
        raise IndexError(["", "input_ids", "position_ids", "token_type_ids"][rc] + " value out of range")
    return out


def dense_hf(x, weight, bias, workers: int = 1):
    a = _f32(x)
    w = _f32(weight)
    b = _f32(bias)
    rows = a.size // a.shape[-1]
    out = np.empty(a.shape[:-1] + (w.shape[0],), dtype=np.float32)
    lib().eos_oracle_dense_hf(_p(a), C.c_int64(rows), C.c_int(a.shape[-1]), _p(w), _p(b), C.c_int(w.shape[0]), _p(out),
                              C.c_int(workers))
    return out


def bert_attention(q, k, v, mask, heads: int, workers: int = 1):
    q, k, v = map(_f32, (q, k, v))
    m = _i32(mask)
    b, t, h = q.shape
    out = np.empty_like(q)
    lib().eos_oracle_bert_attention(_p(q), _p(k), _p(v), _p(m), C.c_int(b), C.c_int(t), C.c_int(h), C.c_int(heads),
                                    _p(out), C.c_int(workers))
    return out


def layernorm_affine(x, gamma, beta, eps=1e-12):
    a = _f32(x)
    g = _f32(gamma)
    bt = _f32(beta)
    out = np.empty_like(a)
    lib().eos_oracle_layernorm_affine(_p(a), C.c_int64(a.size // a.shape[-1]), C.c_int(a.shape[-1]), _p(g), _p(bt),
                                      C.c_double(eps), _p(out))
    return out


def exact_gelu(x):
    a = _f32(x)
    f = lib().eos_oracle_exact_gelu
    return np.array([f(C.c_float(v)) for v in a.ravel()], dtype=np.float32).reshape(a.shape)


def _ptr_array(arrays: Sequence[np.ndarray]):
    arr = (C.c_void_p * len(arrays))()
    for i, a in enumerate(arrays):
        arr[i] = a.ctypes.data
    return arr


def bert_layer(hidden_states, mask, weights16: Sequence[np.ndarray], heads: int, eps=1e-12, workers: int = 1):
    hs = _f32(hidden_states).copy()
    m = _i32(mask)
    ws = [_f32(w) for w in weights16]
    assert len(ws) == 16
    b, t, h = hs.shape
    inter = ws[10].shape[0]
    lib().eos_oracle_bert_layer(_p(hs), _p(m), C.c_int(b), C.c_int(t), C.c_int(h), C.c_int(inter), C.c_int(heads),
                                _ptr_array(ws), C.c_double(eps), C.c_int(workers))
    return hs


def bert_embedder(input_ids, mask, type_ids, tok, pos, typ, emb_gamma, emb_beta, layer_weights: Sequence[np.ndarray],
                  heads: int, eps=1e-12, pooling: str = "masked_mean", head_w=None, workers: int = 1,
                  window: int = 0):
    """layer_weights: 16 float32 tensors per layer, dequantised, dense weights in HF [out,in]."""
    ids, m, tids = map(_i32, (input_ids, mask, type_ids))
    tok, pos, typ, eg, eb = map(_f32, (tok, pos, typ, emb_gamma, emb_beta))
    ws = [_f32(w) for w in layer_weights]
    layers = len(ws) // 16
    assert layers * 16 == len(ws)
    b, t = ids.shape
    hidden = tok.shape[1]
    inter = ws[10].shape[0]
    hw = None if head_w is None else _f32(head_w)
    out_dim = hidden if hw is None else hw.shape[1]
    out = np.empty((b, out_dim), dtype=np.float32)
    rc = lib().eos_oracle_bert_embedder(_p(ids), _p(m), _p(tids), C.c_int(b), C.c_int(t), _p(tok), C.c_int(tok.shape[0]),
                                        _p(pos), C.c_int(pos.shape[0]), _p(typ), C.c_int(typ.shape[0]), _p(eg), _p(eb),
                                        _ptr_array(ws), C.c_int(layers), C.c_int(hidden), C.c_int(inter),
                                        C.c_int(heads), C.c_double(eps), C.c_int(1 if pooling == "cls" else 0),
                                        _p(hw), C.c_int(out_dim), C.c_int(window), _p(out), C.c_int(workers))
    if rc:
        raise IndexError(["", "input_ids", "position_ids", "token_type_ids"][rc] + " value out of range")
    return out


def bert_token_vectors(input_ids, mask, type_ids, tok, pos, typ, emb_gamma, emb_beta, layer_weights: Sequence[np.ndarray],
                       heads: int, token_w, eps=1e-12, workers: int = 1, window: int = 0):
    """[B, T, token_dim] per-token vectors: final hidden rows times token_w [hidden, token_dim], L2-normalised;
    masked tokens give zero rows."""
    ids, m, tids = map(_i32, (input_ids, mask, type_ids))
    tok, pos, typ, eg, eb = map(_f32, (tok, pos, typ, emb_gamma, emb_beta))
    ws = [_f32(w) for w in layer_weights]
    layers = len(ws) // 16
    b, t = ids.shape
    hidden = tok.shape[1]
    inter = ws[10].shape[0]
    tw = _f32(token_w)
    out = np.empty((b, t, tw.shape[1]), dtype=np.float32)
    rc = lib().eos_oracle_bert_token_vectors(_p(ids), _p(m), _p(tids), C.c_int(b), C.c_int(t), _p(tok), C.c_int(tok.shape[0]),
                                             _p(pos), C.c_int(pos.shape[0]), _p(typ), C.c_int(typ.shape[0]), _p(eg), _p(eb),
                                             _ptr_array(ws), C.c_int(layers), C.c_int(hidden), C.c_int(inter),
                                             C.c_int(heads), C.c_double(eps), _p(tw), C.c_int(tw.shape[1]),
                                             C.c_int(window), _p(out), C.c_int(workers))
    if rc:
        raise IndexError(["", "input_ids", "position_ids", "token_type_ids"][rc] + " value out of range")
    return out


def sparse_attention_budget(top_k: int, key_len: int) -> int:
    return int(lib().eos_oracle_sparse_attention_budget(C.c_int(top_k), C.c_int(key_len)))


def sparse_attention_route(key_len: int, block_size: int, top_blocks: int):
    bs, tb = C.c_int(), C.c_int()
    lib().eos_oracle_sparse_attention_route(C.c_int(key_len), C.c_int(block_size), C.c_int(top_blocks), C.byref(bs),
                                            C.byref(tb))
    return bs.value, tb.value


def sparse_attention(query, key, value, top_k: int = 0, route_block_size: int = 0, route_top_blocks: int = 0):
    """sparseAttentionTensor (runtime/backend/attention_ops.go:218-276) for rank-2 or rank-3 q / k / v."""
    q, k, v = map(_f32, (query, key, value))
    squeeze = q.ndim == 2
    if squeeze:
        q, k, v = q[None], k[None], v[None]
    b, ql, dim = q.shape
    kl, vdim = k.shape[1], v.shape[2]
    out = np.zeros((b, ql, vdim), dtype=np.float32)
    lib().eos_oracle_sparse_attention(_p(q), _p(k), _p(v), C.c_int(b), C.c_int(ql), C.c_int(kl), C.c_int(dim),
                                      C.c_int(vdim), C.c_int(top_k), C.c_int(route_block_size), C.c_int(route_top_blocks),
                                      _p(out))
    return out[0] if squeeze else out


# --------------------------------------------------------------------------------- TurboQuant
def tq_code_bytes(dim: int, bits: int) -> int:
    return int(lib().eos_oracle_tq_code_bytes(C.c_int(dim), C.c_int(bits)))


def tq_rotate(x, perm, signs1, signs2, prescale: float = 1.0):
    a = _f32(x)
    out = np.empty_like(a)
    lib().eos_oracle_tq_rotate(_p(a), C.c_int(a.size), _p(_i32(perm)), _p(_f32(signs1)), _p(_f32(signs2)),
                               C.c_float(prescale), _p(out))
    return out


def tq_encode(x, bits, perm, signs1, signs2, boundaries):
    a = _f32(x)
    n, dim = a.shape
    cb = tq_code_bytes(dim, bits)
    codes = np.empty((n, cb), dtype=np.uint8)
    norms = np.empty(n, dtype=np.float32)
    lib().eos_oracle_tq_encode(_p(a), C.c_int64(n), C.c_int(dim), C.c_int(bits), _p(_i32(perm)), _p(_f32(signs1)),
                               _p(_f32(signs2)), _p(_f32(boundaries)), _p(codes), _p(norms))
    return codes, norms


def tq_decode(codes, norms, dim, bits, perm, signs1, signs2, centroids):
    c = np.ascontiguousarray(codes, dtype=np.uint8)
    nr = _f32(norms)
    out = np.empty((c.shape[0], dim), dtype=np.float32)
    lib().eos_oracle_tq_decode(_p(c), _p(nr), C.c_int64(c.shape[0]), C.c_int(dim), C.c_int(bits), _p(_i32(perm)),
                               _p(_f32(signs1)), _p(_f32(signs2)), _p(_f32(centroids)), _p(out))
    return out


def tq_norm_code(norms):
    """f32 norms -> the reference's 8-bit log-scale norm codes (native_linux.go:1879-1893)."""
    a = _f32(norms).reshape(-1)
    out = np.empty(a.size, dtype=np.uint8)
    lib().eos_oracle_tq_norm_code(_p(a), C.c_int64(a.size), _p(out))
    return out


def tq_norm_value(codes):
    """8-bit norm codes -> f32 norms (native_linux.go:1895-1904)."""
    c = np.ascontiguousarray(codes, dtype=np.uint8).reshape(-1)
    out = np.empty(c.size, dtype=np.float32)
    lib().eos_oracle_tq_norm_value(_p(c), C.c_int64(c.size), _p(out))
    return out


def tq_prepare_query(q, perm, signs1, signs2):
    a = _f32(q)
    out = np.empty_like(a)
    lib().eos_oracle_tq_prepare_query(_p(a), C.c_int(a.size), _p(_i32(perm)), _p(_f32(signs1)), _p(_f32(signs2)),
                                      _p(out))
    return out


def tq_score(codes, norms, dim, bits, centroids, prepared):
    c = np.ascontiguousarray(codes, dtype=np.uint8)
    nr = _f32(norms)
    out = np.empty(c.shape[0], dtype=np.float32)
    lib().eos_oracle_tq_score(_p(c), _p(nr), C.c_int64(c.shape[0]), C.c_int(dim), C.c_int(bits), _p(_f32(centroids)),
                              _p(_f32(prepared)), _p(out))
    return out


def tq_ip_score(mse_idx, signs, resnorms, norms, centroids, prepared, sketch, qjl_scale: float):
    """Score of IP-quantised rows (MSE stage + QJL sign stage); the module is absent: parity unpinned."""
    idx = np.ascontiguousarray(mse_idx, dtype=np.uint8)
    sg = np.ascontiguousarray(signs, dtype=np.uint8)
    n, dim = idx.shape
    out = np.empty(n, dtype=np.float32)
    lib().eos_oracle_tq_ip_score(_p(idx), _p(sg), _p(_f32(resnorms)), _p(_f32(norms)), C.c_int64(n), C.c_int(dim),
                                 _p(_f32(centroids)), _p(_f32(prepared)), _p(_f32(sketch)), C.c_float(qjl_scale), _p(out))
    return out


def topk(scores, k: int, id_base: int = 0):
    s = _f32(scores)
    kk = s.size if (k <= 0 or k > s.size) else k
    ids = np.empty(kk, dtype=np.int64)
    out = np.empty(kk, dtype=np.float32)
    r = lib().eos_oracle_topk(_p(s), C.c_int64(s.size), C.c_int64(id_base), C.c_int(k), _p(ids), _p(out))
    return ids[:r], out[:r]


def tq_score_topk(codes, norms, dim, bits, centroids, prepared, k, id_base: int = 0):
    return topk(tq_score(codes, norms, dim, bits, centroids, prepared), k, id_base)


def topk_merge(ids, scores, k: int):
    i = np.ascontiguousarray(ids, dtype=np.int64).ravel()
    s = _f32(scores).ravel()
    kk = s.size if (k <= 0 or k > s.size) else k
    oi = np.empty(kk, dtype=np.int64)
    os_ = np.empty(kk, dtype=np.float32)
    lib().eos_oracle_topk_merge(_p(i), _p(s), C.c_int64(s.size), C.c_int(k), _p(oi), _p(os_))
    return oi, os_


def parent_topk(child_scores, parent_of_child, parents: int, k: int, top_n: int = 1, penalty: float = 0.0):
    s = _f32(child_scores)
    p = _i32(parent_of_child)
    oi = np.empty(parents, dtype=np.int64)
    os_ = np.empty(parents, dtype=np.float32)
    r = lib().eos_oracle_parent_topk(_p(s), _p(p), C.c_int64(s.size), C.c_int(parents), C.c_int(top_n),
                                     C.c_double(penalty), C.c_int(k), _p(oi), _p(os_))
    return oi[:r], os_[:r]


def dot_rows(query, docs):
    q = _f32(query).ravel()
    d = _f32(docs)
    out = np.empty(d.shape[0], dtype=np.float32)
    lib().eos_oracle_dot_rows(_p(q), _p(d), C.c_int64(d.shape[0]), C.c_int(d.shape[1]), _p(out))
    return out


def cosine_rows(query, docs):
    q = _f32(query).ravel()
    d = _f32(docs)
    out = np.empty(d.shape[0], dtype=np.float32)
    lib().eos_oracle_cosine_rows(_p(q), _p(d), C.c_int64(d.shape[0]), C.c_int(d.shape[1]), _p(out))
    return out


def rerank(query, docs, candidates, k: int):
    """topDenseRerankScores (runtime/retrieval_turboquant.go:1610-1635): dot product of the query with every
    candidate that has a vector, best k by score descending then id ascending."""
    cand = [int(c) for c in np.asarray(candidates).ravel() if 0 <= int(c) < len(docs)]
    if not cand:
        return np.empty(0, np.int64), np.empty(0, np.float32)
    scores = dot_rows(query, _f32(docs)[cand])
    return topk_merge(np.asarray(cand, np.int64), scores, k)


def rope_rows(x):
    a = _f32(x)
    cols = a.shape[-1]
    rows = a.size // cols
    seq_rows = a.shape[1] if a.ndim == 3 else rows
    out = np.empty_like(a)
    lib().eos_oracle_rope_rows(_p(a), C.c_int64(rows), C.c_int(seq_rows), C.c_int(cols), _p(out))
    return out


def layernorm_rows(x):
    a = _f32(x)
    cols = a.shape[-1]
    out = np.empty_like(a)
    lib().eos_oracle_layernorm_rows(_p(a), C.c_int64(a.size // cols), C.c_int(cols), _p(out))
    return out


def gelu_tanh(x):
    a = _f32(x)
    out = np.empty_like(a)
    lib().eos_oracle_gelu_tanh_rows(_p(a), C.c_int64(a.size), _p(out))
    return out


def compact_encoder(tokens, mask, role_ids, token_embedding, role_embedding, layers, heads: int,
                    output_projection=None, workers: int = 1):
    """The native compact encoder graph, step by step as models/default_embedding.go:461-505 emits it:
    gather + gather -> add -> rope -> per layer { q, k, v = hidden @ W ([in, out], no bias); multi-head attention
    over the unmasked keys; @ Wo; layernorm(attended + hidden); tanh-GELU FFN; layernorm(projected + attn_hidden) }
    -> per-token normalize -> optional output projection -> masked mean pool.  `layers` holds
    (wq, wk, wv, wo, w_up, w_down) per layer as dequantised fp32 [in, out] matrices."""
    tokens = _i32(tokens)
    mask = _i32(mask)
    hidden = rope_rows(gather(token_embedding, tokens) + gather(role_embedding, _i32(role_ids)))
    for wq, wk, wv, wo, w_up, w_down in layers:
        q, k, v = matmul(hidden, wq), matmul(hidden, wk), matmul(hidden, wv)
        mixed = bert_attention(q, k, v, mask, heads, workers)
        attn_hidden = layernorm_rows(matmul(mixed, wo) + hidden)
        activated = gelu_tanh(matmul(attn_hidden, w_up))
        hidden = layernorm_rows(matmul(activated, w_down) + attn_hidden)
    normalized = normalize_rows(hidden)
    if output_projection is not None:
        normalized = matmul(normalized, output_projection)
    return mean_pool_masked(normalized, mask)


# ------------------------------------------------------------------------------ token-pool encoder
def token_pool_rows(weights: dict, tokens, mode: int = 0, key_spec=None, value_spec=None, top_k: int = 0,
                    route_block_size: int = 0, route_top_blocks: int = 0):
    """embedTextFullEncoderRows (runtime/sparse_token_pool_vector_export.go:1301-1335).  weights: token_embedding,
    attention_query / key / value / output, hidden_projection, projection (fp32), encoder_repeats and the four
    manifest flags; key_spec / value_spec: objects with bits, perm, signs1, signs2, centroids, boundaries."""
    te = _f32(weights["token_embedding"])
    w = [_f32(weights[n]) for n in ("attention_query", "attention_key", "attention_value", "attention_output",
                                    "hidden_projection", "projection")]
    tok = _i32(tokens).reshape(-1)
    dim, hidden = te.shape[1], w[4].shape[1]
    flags = _i32([int(bool(weights.get(n, False))) for n in ("attention_residual", "attention_layer_norm",
                                                                "ffn_residual", "ffn_layer_norm")])
    out = np.empty((tok.size, dim), dtype=np.float32)

    def spec_args(sp):
        if sp is None:
            return [C.c_int(0), None, None, None, None, None], []
        keep = [_i32(sp.perm), _f32(sp.signs1), _f32(sp.signs2), _f32(sp.centroids), _f32(sp.boundaries)]
        return [C.c_int(sp.bits)] + [_p(a) for a in keep], keep

    ka, kkeep = spec_args(key_spec)
    va, vkeep = spec_args(value_spec)
    lib().eos_oracle_token_pool_rows(_p(te), C.c_int(te.shape[0]), C.c_int(dim), C.c_int(hidden), *[_p(a) for a in w],
                                     C.c_int(int(weights["encoder_repeats"])), _p(flags), _p(tok), C.c_int(tok.size),
                                     C.c_int(mode), *ka, *va, C.c_int(top_k), C.c_int(route_block_size),
                                     C.c_int(route_top_blocks), _p(out))
    del kkeep, vkeep
    return out


def token_spans(token_count: int, span_tokens: int, overlap: int, min_tokens: int):
    cap = max(1, token_count)
    starts, ends = np.zeros(cap, np.int32), np.zeros(cap, np.int32)
    n = lib().eos_oracle_token_spans(C.c_int(token_count), C.c_int(span_tokens), C.c_int(overlap), C.c_int(min_tokens),
                                     _p(starts), _p(ends), C.c_int(cap))
    return [(int(starts[i]), int(ends[i])) for i in range(n)]


def token_span_pool(rows, mask, start: int, end: int, fallback_all: bool = False):
    """(vector, active rows): poolSparseTokenRowsRange / maskedMeanPoolNormalized."""
    r = _f32(rows)
    m = _i32(mask).reshape(-1)
    out = np.empty(r.shape[1], dtype=np.float32)
    active = lib().eos_oracle_token_span_pool(_p(r), _p(m), C.c_int(start), C.c_int(end), C.c_int(r.shape[1]),
                                              C.c_int(1 if fallback_all else 0), _p(out))
    return out, int(active)
