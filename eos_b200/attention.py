"""Host-side mirror of the reference's sparse attention operators over the C ABI.

sparse_attention        <- SparseAttentionReference        runtime/backend/attention_ops.go:218-281
turbo_sparse_attention  <- TurboSparseAttentionReference   :283-311
plan_sparse_attention   <- PlanSparseAttention             :78-141 (the auditable budget of one query row)
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import Optional

import numpy as np

from . import _lib
from ._lib import Stats
from .encoder import Runtime, _f32, _ptr


@dataclass
class SparseAttentionPlan:
    query_len: int
    key_len: int
    top_k: int
    routing: str
    selected_key_count: int
    candidate_key_budget: int
    dense_score_count_per_query: int
    estimated_score_count_per_query: int
    candidate_key_fraction: float
    score_count_fraction: float
    route_block_size: int = 0
    route_top_blocks: int = 0
    route_block_count: int = 0
    subquadratic_score_plan: bool = False


def plan_sparse_attention(query_len: int, key_len: int, top_k: int = 0, route_block_size: int = 0,
                          route_top_blocks: int = 0) -> SparseAttentionPlan:
    """The routing knobs normalised as the kernels use them, and the score budget of one query row."""
    if key_len > 0:
        if top_k <= 0:
            top_k = int(math.ceil(math.sqrt(key_len)))
        top_k = max(1, min(top_k, key_len))
    plan = SparseAttentionPlan(query_len, key_len, top_k, "exact", top_k, key_len, key_len, key_len, 1.0, 1.0)
    if key_len <= 0:
        plan.candidate_key_budget = plan.dense_score_count_per_query = plan.estimated_score_count_per_query = 0
        plan.candidate_key_fraction = plan.score_count_fraction = 0.0
        return plan
    if route_block_size <= 0 or route_top_blocks <= 0:
        return plan
    bs = min(route_block_size, key_len)
    blocks = (key_len + bs - 1) // bs
    tb = min(route_top_blocks, blocks)
    budget = min(tb * bs, key_len)
    est = blocks + budget
    plan.routing = "block_anchor"
    plan.route_block_size, plan.route_top_blocks, plan.route_block_count = bs, tb, blocks
    plan.selected_key_count = min(top_k, budget)
    plan.candidate_key_budget = budget
    plan.estimated_score_count_per_query = est
    plan.candidate_key_fraction = budget / key_len
    plan.score_count_fraction = est / key_len
    plan.subquadratic_score_plan = est < key_len
    return plan


def sparse_attention(rt: Runtime, query, key, value, top_k: int = 0, route_block_size: int = 0,
                     route_top_blocks: int = 0, stats: Optional[Stats] = None) -> np.ndarray:
    """Rank-2 ([T, D]) or rank-3 ([B, T, D]) query / key / value, fp32; returns the attended values."""
    q, k, v = _f32(query), _f32(key), _f32(value)
    if not (q.ndim == k.ndim == v.ndim and q.ndim in (2, 3)):
        raise ValueError("sparse_attention expects rank-2 or rank-3 query/key/value tensors")
    squeeze = q.ndim == 2
    if squeeze:
        q, k, v = q[None], k[None], v[None]
    if q.shape[0] != k.shape[0] or q.shape[0] != v.shape[0]:
        raise ValueError(f"sparse_attention batch mismatch: query {q.shape[0]} key {k.shape[0]} value {v.shape[0]}")
    if q.shape[2] != k.shape[2]:
        raise ValueError(f"sparse_attention query dim {q.shape[2]} does not match key dim {k.shape[2]}")
    if k.shape[1] != v.shape[1]:
        raise ValueError(f"sparse_attention key length {k.shape[1]} does not match value length {v.shape[1]}")
    out = np.empty((q.shape[0], q.shape[1], v.shape[2]), dtype=np.float32)
    st = stats if stats is not None else Stats()
    _lib.call("eos_b200_sparse_attention", rt.handle, _ptr(q), _ptr(k), _ptr(v), q.shape[0], q.shape[1], k.shape[1],
              q.shape[2], v.shape[2], int(top_k), int(route_block_size), int(route_top_blocks), _ptr(out), C.byref(st))
    return out[0] if squeeze else out


def turbo_sparse_attention(key_quantizer, value_quantizer, query, key_codes, key_norm_codes, value_codes,
                           value_norm_codes, top_k: int = 0, route_block_size: int = 0, route_top_blocks: int = 0,
                           stats: Optional[Stats] = None) -> np.ndarray:
    """Keys / values as TurboQuant codes ([B, T, D] uint8, one code per byte) and 8-bit log norm codes ([B, T])."""
    q = _f32(query)
    squeeze = q.ndim == 2
    if squeeze:
        q = q[None]
    kc = np.ascontiguousarray(key_codes, dtype=np.uint8).reshape(q.shape[0], -1, key_quantizer.spec.dim)
    vc = np.ascontiguousarray(value_codes, dtype=np.uint8).reshape(q.shape[0], -1, value_quantizer.spec.dim)
    kn = np.ascontiguousarray(key_norm_codes, dtype=np.uint8).reshape(q.shape[0], -1)
    vn = np.ascontiguousarray(value_norm_codes, dtype=np.uint8).reshape(q.shape[0], -1)
    if q.shape[2] != key_quantizer.spec.dim:
        raise ValueError("turbo_sparse_attention query dim does not match the key quantizer")
    if not (kc.shape[1] == vc.shape[1] == kn.shape[1] == vn.shape[1]):
        raise ValueError("turbo_sparse_attention key / value lengths disagree")
    out = np.empty((q.shape[0], q.shape[1], value_quantizer.spec.dim), dtype=np.float32)
    st = stats if stats is not None else Stats()
    _lib.call("eos_b200_turbo_sparse_attention", key_quantizer.handle, value_quantizer.handle, _ptr(q), _ptr(kc), _ptr(kn),
              _ptr(vc), _ptr(vn), q.shape[0], q.shape[1], kc.shape[1], int(top_k), int(route_block_size),
              int(route_top_blocks), _ptr(out), C.byref(st))
    return out[0] if squeeze else out
