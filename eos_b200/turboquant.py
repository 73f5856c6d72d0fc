"""Host-side mirror of the reference's TurboQuant retrieval interfaces over the C ABI.

Quantizer.quantize      <- `for doc: q.Quantize(doc)`        runtime/retrieval_turboquant.go:700-711
Corpus.score_topk       <- PrepareQuery + topTurboQuantRetrievalScoresWithStats  :1324-1325, 1853-1887
Corpus.parent_topk      <- topTurboQuantMultiVectorParentScores  runtime/retrieval_multivector_turboquant.go:746-810
RotationSpec            <- the fields of turboquant Spec() (runtime/backends/cuda/native_linux.go:9532-9545)

The arithmetic of the reference's quantiser lives in the un-vendored module m31labs.dev/turboquant; the
seeded permutation / sign generator and the Lloyd-Max tables below are this library's own (a Go host that owns
the real module passes its own Spec instead).
"""
from __future__ import annotations

import ctypes as C
import math
import weakref
from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np

from . import _lib
from ._lib import Stats
from .encoder import Runtime, _f32, _i32, _ptr

DEFAULT_SEED = 0x4D756C7469566563  # runtime/retrieval_multivector_turboquant.go:18


@dataclass
class RotationSpec:
    dim: int
    bits: int
    perm: np.ndarray        # int32 [dim]
    signs1: np.ndarray      # float32 [dim], +-1
    signs2: np.ndarray      # float32 [dim], +-1
    centroids: np.ndarray   # float32 [2^bits], ascending, symmetric
    boundaries: np.ndarray  # float32 [2^bits - 1]

    @property
    def code_bytes(self) -> int:
        return (self.dim * self.bits + 7) // 8

    @property
    def vector_bytes(self) -> int:
        """Packed bytes per vector incl. the f32 norm (runtime/turboquant_bytes.go:22-25 accounting)."""
        return self.code_bytes + 4


def _phi(x: float) -> float:
    return math.exp(-0.5 * x * x) / math.sqrt(2.0 * math.pi)


def _cdf(x: float) -> float:
    return 0.5 * (1.0 + math.erf(x / math.sqrt(2.0)))


def lloyd_max_gaussian(levels: int, sigma: float, iters: int = 500) -> Tuple[np.ndarray, np.ndarray]:
    """Lloyd-Max scalar quantiser for N(0, sigma^2): (centroids[levels], boundaries[levels-1]) as float32.

    Fixed-point iteration of centroid = E[x | cell], boundary = midpoint, in float64 on the unit normal; the
    result is made exactly symmetric (c[L-1-i] = -c[i]) before rounding to float32.
    """
    c = np.array([(i + 0.5) / levels * 6.0 - 3.0 for i in range(levels)], dtype=np.float64)
    for _ in range(iters):
        b = (c[:-1] + c[1:]) / 2.0
        edges = [-math.inf] + list(b) + [math.inf]
        new = np.empty_like(c)
        for i in range(levels):
            lo, hi = edges[i], edges[i + 1]
            p = _cdf(hi) - _cdf(lo)
            new[i] = (_phi(lo) - _phi(hi)) / p if p > 0 else c[i]
        if np.max(np.abs(new - c)) < 1e-14:
            c = new
            break
        c = new
    c = (c - c[::-1]) / 2.0
    cf = (c * sigma).astype(np.float32)
    cf[: levels // 2] = -cf[::-1][: levels // 2]
    bf = ((cf[:-1].astype(np.float64) + cf[1:].astype(np.float64)) / 2.0).astype(np.float32)
    return cf, bf


def make_rotation_spec(dim: int, bits: int, seed: int = DEFAULT_SEED) -> RotationSpec:
    """Seeded random-sign Hadamard rotation + Lloyd-Max codebook for N(0, 1/dim)."""
    rng = np.random.default_rng(seed)
    perm = rng.permutation(dim).astype(np.int32)
    signs1 = rng.choice(np.array([-1.0, 1.0], dtype=np.float32), size=dim).astype(np.float32)
    signs2 = rng.choice(np.array([-1.0, 1.0], dtype=np.float32), size=dim).astype(np.float32)
    cent, bound = lloyd_max_gaussian(1 << bits, 1.0 / math.sqrt(dim))
    return RotationSpec(dim, bits, perm, signs1, signs2, cent, bound)


class Quantizer:
    def __init__(self, rt: Runtime, spec: RotationSpec):
        self.rt, self.spec = rt, spec
        self._keep = [_i32(spec.perm), _f32(spec.signs1), _f32(spec.signs2), _f32(spec.centroids), _f32(spec.boundaries)]
        if self._keep[0].size != spec.dim or self._keep[3].size != (1 << spec.bits) or \
                self._keep[4].size != (1 << spec.bits) - 1:
            raise ValueError("rotation spec arrays do not match dim / bits")
        self.handle = C.c_void_p()
        _lib.call("eos_b200_quantizer_create", rt.handle, spec.dim, spec.bits, *[_ptr(a) for a in self._keep],
                  C.byref(self.handle))
        rt._adopt(self)
        self._children = weakref.WeakSet()
        self.last_stats = Stats()

    def quantize(self, x) -> Tuple[np.ndarray, np.ndarray]:
        """[n, dim] fp32 -> (codes uint8 [n, dim*bits/8], norms fp32 [n])."""
        a = _f32(x)
        if a.ndim != 2 or a.shape[1] != self.spec.dim or a.shape[0] == 0:
            raise ValueError(f"quantize expects a non-empty [n, {self.spec.dim}] array, got {a.shape}")
        codes = np.empty((a.shape[0], self.spec.code_bytes), dtype=np.uint8)
        norms = np.empty(a.shape[0], dtype=np.float32)
        _lib.call("eos_b200_quantize", self.handle, _ptr(a), a.shape[0], _ptr(codes), _ptr(norms),
                  C.byref(self.last_stats))
        return codes, norms

    def quantize_device(self, d_x: int, n: int, d_codes: int, d_norms: int, stream: Optional[int] = None) -> None:
        _lib.call("eos_b200_quantize_device", self.handle, d_x, int(n), d_codes, d_norms, stream)

    def close(self) -> None:
        if self.handle:
            for child in list(self._children):
                child.close()
            _lib.lib().eos_b200_quantizer_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Corpus:
    """Packed vectors resident on one GPU (one shard); row i has document id id_base + i."""

    def __init__(self, quantizer: Quantizer, codes=None, norms=None, id_base: int = 0, allow_zero_norm: bool = False,
                 device_ptrs: Optional[Tuple[int, int, int]] = None):
        self.qz = quantizer
        self.handle = C.c_void_p()
        self.id_base = int(id_base)
        if device_ptrs is not None:
            d_codes, d_norms, n = device_ptrs
            self.n = int(n)
            _lib.call("eos_b200_corpus_bind_device", quantizer.handle, d_codes, d_norms, int(n), int(id_base),
                      C.byref(self.handle))
            quantizer._children.add(self)
        else:
            c = np.ascontiguousarray(codes, dtype=np.uint8)
            nr = _f32(norms).reshape(-1)
            if c.ndim != 2 or c.shape[1] != quantizer.spec.code_bytes or c.shape[0] != nr.size:
                raise ValueError("corpus codes / norms do not match the quantizer")
            self.n = c.shape[0]
            _lib.call("eos_b200_corpus_bind", quantizer.handle, _ptr(c), _ptr(nr), c.shape[0], int(id_base),
                      1 if allow_zero_norm else 0, C.byref(self.handle))
            quantizer._children.add(self)
        self.last_stats = Stats()

    def score_topk(self, queries, k: int, queries_per_pass: int = 0) -> Tuple[np.ndarray, np.ndarray]:
        """Exact top-k per query: (ids int64 [Q,k], scores fp32 [Q,k]); score desc, then id asc.
        queries_per_pass: 0 = automatic (streaming scan up to 8 queries, tensor-core batch kernels above),
        or 8 / 16 / 32 (streaming scan), 128 / 256 (batch kernels)."""
        q = _f32(queries)
        if q.ndim != 2 or q.shape[1] != self.qz.spec.dim or q.shape[0] == 0:
            raise ValueError(f"score_topk expects non-empty [Q, {self.qz.spec.dim}] queries, got {q.shape}")
        ids = np.empty((q.shape[0], k), dtype=np.int64)
        scores = np.empty((q.shape[0], k), dtype=np.float32)
        _lib.call("eos_b200_score_topk", self.handle, _ptr(q), q.shape[0], int(k), int(queries_per_pass), _ptr(ids),
                  _ptr(scores), C.byref(self.last_stats))
        return ids, scores

    def score_topk_device(self, d_queries: int, q_count: int, k: int, queries_per_pass: int, d_ids: Optional[int],
                          d_scores: Optional[int], d_keys: Optional[int] = None, stream: Optional[int] = None) -> int:
        st = Stats()
        _lib.call("eos_b200_score_topk_device", self.handle, d_queries, int(q_count), int(k), int(queries_per_pass),
                  d_ids, d_scores, d_keys, stream, C.byref(st))
        return st.kernel_launches

    def score_seed_device(self, d_queries: int, q_count: int, k: int, d_tau_out: int,
                          stream: Optional[int] = None) -> None:
        """Pruning thresholds (uint64 keys, [q_count]) of these queries from a sample of this shard.  With a corpus
        sharded over several GPUs each rank seeds a slice of the batch and the slices are all-gathered: a threshold
        from any shard is a lower bound of the k-th best score of the whole corpus."""
        _lib.call("eos_b200_score_seed_device", self.handle, d_queries, int(q_count), int(k), d_tau_out, stream)

    def score_topk_seeded_device(self, d_queries: int, q_count: int, k: int, d_tau: int, d_ids: Optional[int],
                                 d_scores: Optional[int], d_keys: Optional[int] = None,
                                 stream: Optional[int] = None) -> int:
        """Batch scoring with caller-supplied thresholds ([q_count] uint64 keys, 0 = none): this shard's part of the
        top-k of the whole sharded corpus (empty slots: id -1 / key 0)."""
        st = Stats()
        _lib.call("eos_b200_score_topk_seeded_device", self.handle, d_queries, int(q_count), int(k), d_tau, d_ids,
                  d_scores, d_keys, stream, C.byref(st))
        return st.kernel_launches

    def score_topk_sharded(self, comm, d_queries: int, q_count: int, k: int, queries_per_pass: int, d_ids: int,
                           d_scores: int, stream: Optional[int] = None) -> int:
        """Collective over the ranks of `comm` (eos_b200.dist.Comm): this rank's shard is scored and every rank
        receives the exact top-k of the whole corpus; thresholds and key lists travel by NCCL all-gathers issued
        inside the library.  Returns the kernel launches of this rank."""
        st = Stats()
        _lib.call("eos_b200_score_topk_sharded", self.handle, comm.handle, d_queries, int(q_count), int(k),
                  int(queries_per_pass), d_ids, d_scores, stream, C.byref(st))
        return st.kernel_launches

    def maxsim_topk_device(self, d_queries: int, q_vectors: int, query_group: int, children_per_parent: int, k: int,
                           d_ids: Optional[int], d_scores: Optional[int], d_keys: Optional[int] = None,
                           stream: Optional[int] = None) -> int:
        """Late interaction over fixed-size parents (rows = child vectors, children_per_parent consecutive rows per
        parent): per query (query_group consecutive query vectors) the sum of the best child scores, exact top-k
        over parents.  Results [q_vectors / query_group, k]."""
        st = Stats()
        _lib.call("eos_b200_maxsim_topk_device", self.handle, d_queries, int(q_vectors), int(query_group),
                  int(children_per_parent), int(k), d_ids, d_scores, d_keys, stream, C.byref(st))
        return st.kernel_launches

    def score_topk_noalloc(self, d_queries: int, q_count: int, k: int, queries_per_pass: int, d_ids: int,
                           d_scores: int, stream: Optional[int] = None) -> None:
        """score_topk_device for callers that may not allocate device memory while serving (a fixed memory
        arena, allocation locked after start-up, or a latency path where cudaMalloc would stall the device).
        The scratch is a fixed array inside the library: at most 32 queries per call, dim <= 1024; calls on one
        device share it, so keep them ordered on one stream.  Make the first call before any stream capture."""
        _lib.call("eos_b200_score_topk_noalloc", self.handle, d_queries, int(q_count), int(k), int(queries_per_pass),
                  d_ids, d_scores, stream)

    def sync(self, stream: Optional[int] = None) -> None:
        """Waits for the stream of the *_device / _noalloc calls; raises EosB200DeviceStatusError if one of their
        kernels gave up on a bounded wait (the results are then incomplete)."""
        _lib.call("eos_b200_corpus_sync", self.handle, stream)

    def profile_begin(self, max_launches: int) -> None:
        _lib.call("eos_b200_corpus_profile_begin", self.handle, int(max_launches))

    def profile_end(self, stream: Optional[int] = None) -> Tuple[float, int]:
        """(total milliseconds, launches) of the scan kernel since profile_begin."""
        ms, n = C.c_float(), C.c_int()
        _lib.call("eos_b200_corpus_profile_end", self.handle, stream, C.byref(ms), C.byref(n))
        return float(ms.value), int(n.value)

    def score_all(self, queries) -> np.ndarray:
        q = _f32(queries)
        out = np.empty((q.shape[0], self.n), dtype=np.float32)
        _lib.call("eos_b200_score_all", self.handle, _ptr(q), q.shape[0], _ptr(out))
        return out

    def parent_topk(self, parent_of_child, parents: int, queries, k: int, query_group: int = 1, top_n: int = 1,
                    penalty: float = 0.0) -> Tuple[np.ndarray, np.ndarray]:
        p = _i32(parent_of_child).reshape(-1)
        if p.size != self.n:
            raise ValueError("parent_of_child must have one entry per corpus row")
        q = _f32(queries)
        groups = q.shape[0] // max(1, query_group)
        ids = np.empty((groups, k), dtype=np.int64)
        scores = np.empty((groups, k), dtype=np.float32)
        _lib.call("eos_b200_parent_topk", self.handle, _ptr(p), int(parents), _ptr(q), q.shape[0], int(query_group),
                  int(top_n), float(penalty), int(k), _ptr(ids), _ptr(scores), C.byref(self.last_stats))
        return ids, scores

    @property
    def vector_bytes(self) -> int:
        return int(_lib.lib().eos_b200_corpus_vector_bytes(self.handle))

    def close(self) -> None:
        if self.handle:
            _lib.lib().eos_b200_corpus_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


METRIC_DOT, METRIC_COSINE = 0, 1


def norm_encode_log8(norms) -> np.ndarray:
    """fp32 norms -> the 8-bit log-scale side-car of the reference's device encode (native_linux.go:1879-1893)."""
    a = _f32(norms).reshape(-1)
    out = np.empty(a.size, dtype=np.uint8)
    _lib.lib().eos_b200_norm_encode_log8(_ptr(a), a.size, _ptr(out))
    return out


def norm_decode_log8(codes) -> np.ndarray:
    """8-bit log-scale norm codes -> fp32 norms (native_linux.go:1895-1904)."""
    c = np.ascontiguousarray(codes, dtype=np.uint8).reshape(-1)
    out = np.empty(c.size, dtype=np.float32)
    _lib.lib().eos_b200_norm_decode_log8(_ptr(c), c.size, _ptr(out))
    return out


class IpCorpus:
    """Rows quantised by the inner-product quantiser -- turboquant.IPQuantized{MSE, Signs, ResNorm, Norm}
    (runtime/turboquant_quantized_vector.go:43-49) -- resident on one GPU.  The fields come from a host that holds the
    quantiser module; the score is Norm * (<R q, centroids[MSE]> + ResNorm * qjl_scale * <sketch_q, +-1 signs>)."""

    def __init__(self, rt: Runtime, dim: int, perm, signs1, signs2, mse_centroids, mse_indices, signs, resnorms, norms,
                 id_base: int = 0, allow_zero_norm: bool = False):
        self.rt, self.dim = rt, int(dim)
        cent = _f32(mse_centroids).reshape(-1)
        idx = np.ascontiguousarray(mse_indices, dtype=np.uint8)
        sg = np.ascontiguousarray(signs, dtype=np.uint8)
        rn, nr = _f32(resnorms).reshape(-1), _f32(norms).reshape(-1)
        if idx.ndim != 2 or idx.shape[1] != dim or sg.shape != (idx.shape[0], (dim + 7) // 8) or \
                rn.size != idx.shape[0] or nr.size != idx.shape[0]:
            raise ValueError("ip corpus fields do not match dim / row count")
        pm, s1, s2 = _i32(perm), _f32(signs1), _f32(signs2)   # named, so that they outlive the call
        if pm.size != dim or s1.size != dim or s2.size != dim:
            raise ValueError("rotation arrays do not match dim")
        self.n = idx.shape[0]
        self.handle = C.c_void_p()
        _lib.call("eos_b200_ip_corpus_bind", rt.handle, int(dim), int(cent.size), _ptr(pm), _ptr(s1), _ptr(s2), _ptr(cent),
                  _ptr(idx), _ptr(sg), _ptr(rn), _ptr(nr), self.n, int(id_base), 1 if allow_zero_norm else 0,
                  C.byref(self.handle))
        self.last_stats = Stats()

    @staticmethod
    def vector_bytes(dim: int, bit_width: int) -> int:
        """turboquantVectorBytes (runtime/turboquant_bytes.go:22-25)."""
        return int(_lib.lib().eos_b200_ip_corpus_vector_bytes(int(dim), int(bit_width)))

    def score_topk(self, queries, query_sketch, qjl_scale: float, k: int) -> Tuple[np.ndarray, np.ndarray]:
        q, sk = _f32(queries), _f32(query_sketch)
        if q.ndim != 2 or q.shape[1] != self.dim or q.shape[0] == 0 or sk.shape != q.shape:
            raise ValueError(f"ip score_topk expects non-empty [Q, {self.dim}] queries and sketches")
        ids = np.empty((q.shape[0], k), dtype=np.int64)
        scores = np.empty((q.shape[0], k), dtype=np.float32)
        _lib.call("eos_b200_ip_score_topk", self.handle, _ptr(q), _ptr(sk), float(qjl_scale), q.shape[0], int(k),
                  _ptr(ids), _ptr(scores), C.byref(self.last_stats))
        return ids, scores

    def close(self) -> None:
        if self.handle:
            _lib.lib().eos_b200_ip_corpus_destroy(self.handle)
            self.handle = C.c_void_p()


class DenseIndex:
    """Uncompressed document vectors on one GPU: the dense scoring operators (dotRows / cosineRows + topKTensor,
    runtime/backend/tensor_ops.go:1967-2057, 2124-2193) and the rerank stage after a TurboQuant top-k
    (topDenseRerankScores / topFP16RerankScores, runtime/retrieval_turboquant.go:1610-1662).  store_f16 keeps the
    vectors rounded to f16 (the reference's fp16 sidecar)."""

    def __init__(self, runtime, vectors, store_f16: bool = False):
        v = _f32(vectors)
        if v.ndim != 2 or v.shape[0] == 0 or v.shape[1] == 0:
            raise ValueError(f"DenseIndex expects non-empty [n, dim] vectors, got {v.shape}")
        self.rt = runtime
        self.n, self.dim = v.shape
        self.handle = C.c_void_p()
        _lib.call("eos_b200_dense_bind", runtime.handle, _ptr(v), self.n, self.dim, 1 if store_f16 else 0,
                  C.byref(self.handle))
        runtime._adopt(self)
        self.last_stats = Stats()

    def score_topk(self, queries, k: int, metric: int = METRIC_DOT) -> Tuple[np.ndarray, np.ndarray]:
        """Every query against every row: (row ids int64 [Q,k], scores fp32 [Q,k]); score desc, then row asc."""
        q = _f32(queries)
        if q.ndim != 2 or q.shape[1] != self.dim or q.shape[0] == 0:
            raise ValueError(f"score_topk expects non-empty [Q, {self.dim}] queries, got {q.shape}")
        ids = np.empty((q.shape[0], k), dtype=np.int64)
        scores = np.empty((q.shape[0], k), dtype=np.float32)
        _lib.call("eos_b200_dense_score_topk", self.handle, _ptr(q), q.shape[0], int(metric), int(k), _ptr(ids),
                  _ptr(scores), C.byref(self.last_stats))
        return ids, scores

    def rerank(self, queries, candidates, k: int) -> Tuple[np.ndarray, np.ndarray]:
        """Exact dot products of each query with its own candidate rows ([Q, C] row indices, negative = no vector),
        best k by score desc / row asc; unused result slots hold id -1."""
        q = _f32(queries)
        c = np.ascontiguousarray(candidates, dtype=np.int64)
        if q.ndim != 2 or q.shape[1] != self.dim or c.ndim != 2 or c.shape[0] != q.shape[0] or c.shape[1] == 0:
            raise ValueError("rerank expects [Q, dim] queries and [Q, C] candidates")
        kk = c.shape[1] if (k <= 0 or k > c.shape[1]) else int(k)
        ids = np.empty((q.shape[0], kk), dtype=np.int64)
        scores = np.empty((q.shape[0], kk), dtype=np.float32)
        _lib.call("eos_b200_dense_rerank", self.handle, _ptr(q), q.shape[0], _ptr(c), c.shape[1], kk, _ptr(ids),
                  _ptr(scores), C.byref(self.last_stats))
        return ids, scores

    def close(self) -> None:
        if self.handle:
            _lib.lib().eos_b200_dense_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass



def topk_merge_device(rt: Runtime, d_keys: int, shards: int, q_count: int, k: int, d_ids: int, d_scores: int,
                      stream: Optional[int] = None) -> None:
    """Global top-k from all-gathered per-shard key lists [shards, Q, k] (device pointers)."""
    _lib.call("eos_b200_topk_merge_device", rt.handle, d_keys, int(shards), int(q_count), int(k), d_ids, d_scores,
              stream)


def synth_gaussian_device(rt: Runtime, seed: int, row_offset: int, n: int, dim: int, normalize: bool, d_out: int,
                          stream: Optional[int] = None) -> None:
    _lib.call("eos_b200_synth_gaussian_device", rt.handle, C.c_uint64(seed), int(row_offset), int(n), int(dim),
              1 if normalize else 0, d_out, stream)
