"""Host-side mirror of the reference's token-pool encoder and its token-span child vectors
(sparseTokenPoolEncoder, runtime/sparse_token_pool_vector_export.go:1290-1335, 802-890) over the C ABI."""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Tuple

import numpy as np

from . import _lib
from ._lib import Stats, TokenPoolDesc
from .encoder import Runtime, _f32, _i32, _ptr

ATTENTION_DENSE, ATTENTION_TURBO_SPARSE = 0, 1


def token_spans(token_count: int, span_tokens: int, overlap: int = 0, min_tokens: int = 1) -> List[Tuple[int, int]]:
    """sparseTokenPoolTokenSpans (:1561-1595): [start, end) spans of span_tokens tokens stepping by span_tokens - overlap."""
    if token_count <= 0 or span_tokens <= 0:
        return []
    if min_tokens <= 0:
        min_tokens = 1
    if token_count <= span_tokens:
        return [] if token_count < min_tokens else [(0, token_count)]
    step = span_tokens - overlap
    if step <= 0:
        return []
    spans = []
    for start in range(0, token_count, step):
        end = min(start + span_tokens, token_count)
        if end - start < min_tokens:
            break
        spans.append((start, end))
        if end >= token_count:
            break
    return spans


def span_child_ids(record_id: str, count: int) -> List[str]:
    """Child ids of a record's span vectors, as the cache writer names them (:862-866)."""
    return [f"{record_id}#token-span-{i:04d}" for i in range(count)]


class TokenPoolEncoder:
    """The fp32 single-head encoder whose normalised token rows are pooled over spans into child vectors.

    weights: token_embedding [V, D], attention_query / attention_key / attention_value / attention_output [D, D],
    hidden_projection [D, H], projection [H, D] in the reference's [in, out] layout; encoder_repeats applications of
    the one layer; the manifest's four switches."""

    def __init__(self, rt: Runtime, token_embedding, attention_query, attention_key, attention_value, attention_output,
                 hidden_projection, projection, encoder_repeats: int = 1, attention_residual: bool = False,
                 attention_layer_norm: bool = False, ffn_residual: bool = False, ffn_layer_norm: bool = False):
        self.rt = rt
        arrs = [_f32(a) for a in (token_embedding, attention_query, attention_key, attention_value, attention_output,
                                  hidden_projection, projection)]
        te, wq, wk, wv, wo, w1, w2 = arrs
        dim, hidden = te.shape[1], w1.shape[1]
        for name, a, shape in (("attention_query", wq, (dim, dim)), ("attention_key", wk, (dim, dim)),
                               ("attention_value", wv, (dim, dim)), ("attention_output", wo, (dim, dim)),
                               ("hidden_projection", w1, (dim, hidden)), ("projection", w2, (hidden, dim))):
            if a.shape != shape:
                raise ValueError(f"{name} has shape {a.shape}, want {shape}")
        self.dim, self.hidden = dim, hidden
        desc = TokenPoolDesc(te.shape[0], dim, hidden, int(encoder_repeats), int(attention_residual),
                             int(attention_layer_norm), int(ffn_residual), int(ffn_layer_norm), *[_ptr(a) for a in arrs])
        self.handle = C.c_void_p()
        _lib.call("eos_b200_token_pool_bind", rt.handle, C.byref(desc), C.byref(self.handle))
        self.last_stats = Stats()

    def _encode(self, tokens, mask, mode, key_quantizer, value_quantizer, top_k, route_block_size, route_top_blocks,
                span, want_rows, want_pooled):
        tok = _i32(tokens).reshape(-1)
        if tok.size == 0:
            raise ValueError("token_pool expects a non-empty token sequence")
        m = None if mask is None else _i32(mask).reshape(-1)
        if m is not None and m.size != tok.size:
            raise ValueError("mask length does not match the tokens")
        rows = np.empty((tok.size, self.dim), np.float32) if want_rows else None
        pooled = np.empty(self.dim, np.float32) if want_pooled else None
        children, n_children, max_children = None, C.c_int(0), 0
        span_tokens = overlap = min_tokens = 0
        if span is not None:
            span_tokens, overlap, min_tokens = span
            max_children = max(1, len(token_spans(tok.size, span_tokens, overlap, min_tokens)))
            children = np.empty((max_children, self.dim), np.float32)
        _lib.call("eos_b200_token_pool_encode", self.handle, _ptr(tok), _ptr(m), tok.size, int(mode),
                  None if key_quantizer is None else key_quantizer.handle,
                  None if value_quantizer is None else value_quantizer.handle, int(top_k), int(route_block_size),
                  int(route_top_blocks), int(span_tokens), int(overlap), int(min_tokens), _ptr(rows), _ptr(pooled),
                  _ptr(children), max_children, C.byref(n_children), C.byref(self.last_stats))
        return rows, pooled, None if children is None else children[: n_children.value]

    def token_rows(self, tokens, attention_mode: int = ATTENTION_DENSE, key_quantizer=None, value_quantizer=None,
                   top_k: int = 0, route_block_size: int = 0, route_top_blocks: int = 0) -> np.ndarray:
        """embedTextFullEncoderRows: one L2-normalised row per token."""
        return self._encode(tokens, None, attention_mode, key_quantizer, value_quantizer, top_k, route_block_size,
                            route_top_blocks, None, True, False)[0]

    def embed(self, tokens, mask, **kw) -> np.ndarray:
        """embedTextFullEncoder: the masked mean of the rows, normalised."""
        return self._encode(tokens, mask, kw.pop("attention_mode", ATTENTION_DENSE), kw.pop("key_quantizer", None),
                            kw.pop("value_quantizer", None), kw.pop("top_k", 0), kw.pop("route_block_size", 0),
                            kw.pop("route_top_blocks", 0), None, False, True)[1]

    def span_child_vectors(self, tokens, mask, span_tokens: int, span_overlap: int = 0, span_min_tokens: int = 1,
                           attention_mode: int = ATTENTION_DENSE, key_quantizer=None, value_quantizer=None, top_k: int = 0,
                           route_block_size: int = 0, route_top_blocks: int = 0) -> np.ndarray:
        """One unit vector per token span (the rows of `child-doc-vectors.jsonl` for one document)."""
        return self._encode(tokens, mask, attention_mode, key_quantizer, value_quantizer, top_k, route_block_size,
                            route_top_blocks, (span_tokens, span_overlap, span_min_tokens), False, False)[2]

    def close(self) -> None:
        if self.handle:
            _lib.lib().eos_b200_token_pool_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
