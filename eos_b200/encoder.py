"""Host-side mirror of the reference's encoder interfaces over the C ABI.

BertEmbedder   <- StepBERTEmbedder / BERTEmbedderReferenceWithPooling
                  (runtime/backend/bert_embedder_ops.go:101-197): same tensor order
                  (16 tensors per layer, runtime/pretrained_bert_importer.go:936-951), same attributes
                  (num_attention_heads, epsilon, pooling), same error behaviour (out-of-range ids are
                  an error, all-masked sequences give zero vectors).
EmbedPooledPipeline <- the compiled pipeline examples/embed_masked_pooled.eos.
linear         <- one dense projection with denseHF semantics
                  (runtime/backend/bert_encoder_layer_ops.go:452-462).
"""
from __future__ import annotations

import ctypes as C
import weakref
from dataclasses import dataclass
from typing import Optional, Sequence, Union

import numpy as np

from . import _lib
from ._lib import EncoderDesc, EncoderLayer, Matrix, Stats

ACT_GELU_ERF, ACT_GELU_TANH = 0, 1
WEIGHTS_Q8_SMEM_DEQUANT, WEIGHTS_F16_RESIDENT = 0, 1
EPILOGUE_NONE, EPILOGUE_GELU_ERF, EPILOGUE_RESIDUAL, EPILOGUE_GELU_TANH = 0, 1, 2, 3


@dataclass
class Q8Weight:
    """int8 codes [out, in] + fp32 scales (1 = per tensor, out = per output channel); value = code * scale."""
    codes: np.ndarray
    scales: np.ndarray

    def dequantized(self) -> np.ndarray:
        s = np.asarray(self.scales, np.float32).reshape(-1)
        c = np.asarray(self.codes, np.int8).astype(np.float32)
        return c * (s[0] if s.size == 1 else s[:, None])


@dataclass
class Q8WeightInOut:
    """int8 codes in Eos's matmul layout [in, out] + fp32 scales (1 = per tensor, out = per output channel)."""
    codes: np.ndarray
    scales: np.ndarray

    def dequantized(self) -> np.ndarray:
        s = np.asarray(self.scales, np.float32).reshape(-1)
        c = np.asarray(self.codes, np.int8).astype(np.float32)
        return c * (s[0] if s.size == 1 else s[None, :])


Weight = Union[np.ndarray, Q8Weight, Q8WeightInOut]


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.int32)


def _ptr(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data


class Runtime:
    """One device + stream (newDeviceRuntime, runtime/backends/cuda/native_linux.go:3127)."""

    def __init__(self, device: int = 0):
        self.handle = C.c_void_p()
        _lib.call("eos_b200_runtime_create", int(device), C.byref(self.handle))
        self.device = int(device)
        self._children = weakref.WeakSet()  # handles bound to this runtime; they must be destroyed first

    def _adopt(self, child) -> None:
        self._children.add(child)

    def info(self) -> dict:
        out = _lib.DeviceInfo()
        _lib.call("eos_b200_runtime_info", self.handle, C.byref(out))
        return {"device": out.device, "cc": (out.cc_major, out.cc_minor), "sm_count": out.sm_count,
                "total_memory_bytes": out.total_memory_bytes, "name": out.name.decode()}

    def selftest_bounded_wait(self, limit_cycles: int = 1_000_000) -> None:
        """Runs the bounded-wait self-test: raises EosB200DeviceStatusError when the wait ran out as designed."""
        _lib.call("eos_b200_selftest_bounded_wait", self.handle, int(limit_cycles))

    def close(self) -> None:
        if self.handle:
            for child in list(self._children):
                child.close()
            _lib.lib().eos_b200_runtime_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _matrix(w: Weight, keep: list) -> Matrix:
    m = Matrix()
    if isinstance(w, (Q8Weight, Q8WeightInOut)):
        codes = np.ascontiguousarray(w.codes, dtype=np.int8)
        scales = _f32(w.scales).reshape(-1)
        keep += [codes, scales]
        m.rows, m.cols = codes.shape
        m.q8_codes, m.q8_scales, m.n_scales = codes.ctypes.data, scales.ctypes.data, scales.size
    else:
        dense = _f32(w)
        keep.append(dense)
        m.rows, m.cols = dense.shape
        m.dense = dense.ctypes.data
    return m


class BertEmbedder:
    """q8 / dense BERT-family encoder bound to a device: embeddings -> layers -> pooling -> L2 (-> head -> L2)."""

    def __init__(self, rt: Runtime, token_embeddings, position_embeddings, token_type_embeddings,
                 embedding_ln_weight, embedding_ln_bias, layer_weights: Sequence[Weight], num_attention_heads: int,
                 epsilon: float = 1e-12, pooling: str = "masked_mean", hidden_act: str = "gelu",
                 head_weights=None, weight_mode: int = WEIGHTS_F16_RESIDENT, attention_window: int = 0):
        # weight_mode: WEIGHTS_F16_RESIDENT expands the 8-bit codes to f16 once at bind (the code values are
        # exact in f16, the per-channel scale stays in the fp32 epilogue); WEIGHTS_Q8_SMEM_DEQUANT keeps the
        # codes 8-bit in HBM and expands them in shared memory inside the projection kernel.  Both feed the
        # same values to the same tensor-core instruction, so their results are bit-identical; the resident
        # form is faster when the batch makes the projections compute-bound, the 8-bit form halves weight
        # bytes when they are not.
        if pooling not in ("masked_mean", "cls"):
            raise ValueError(f"bert_embedder unsupported pooling {pooling!r}; supported values are masked_mean and cls")
        if hidden_act not in ("gelu", "gelu_tanh"):
            raise ValueError(f"bert_encoder_layer unsupported hidden_act {hidden_act!r}")
        if len(layer_weights) == 0 or len(layer_weights) % 16 != 0:
            raise ValueError(f"bert_embedder expects 16 tensors per encoder layer, got {len(layer_weights)}")
        self.rt = rt
        keep: list = []
        tok, pos, typ = _f32(token_embeddings), _f32(position_embeddings), _f32(token_type_embeddings)
        eg, eb = _f32(embedding_ln_weight), _f32(embedding_ln_bias)
        keep += [tok, pos, typ, eg, eb]
        layers = len(layer_weights) // 16
        arr = (EncoderLayer * layers)()
        for l in range(layers):
            w = layer_weights[l * 16:(l + 1) * 16]
            L = arr[l]
            vec = {}
            for idx, name in ((1, "query_bias"), (3, "key_bias"), (5, "value_bias"), (7, "attn_out_bias"),
                              (8, "attn_ln_gamma"), (9, "attn_ln_beta"), (11, "inter_bias"), (13, "out_bias"),
                              (14, "out_ln_gamma"), (15, "out_ln_beta")):
                v = _f32(w[idx]).reshape(-1)
                keep.append(v)
                vec[name] = v
                setattr(L, name, v.ctypes.data)
            L.query, L.key, L.value = _matrix(w[0], keep), _matrix(w[2], keep), _matrix(w[4], keep)
            L.attn_out, L.inter, L.out = _matrix(w[6], keep), _matrix(w[10], keep), _matrix(w[12], keep)
            for name, mat in (("query_bias", L.query), ("key_bias", L.key), ("value_bias", L.value),
                              ("attn_out_bias", L.attn_out), ("inter_bias", L.inter), ("out_bias", L.out)):
                if vec[name].size != mat.rows:
                    raise ValueError(f"bert_encoder_layer {name} shape {vec[name].shape} does not match [out]=[{mat.rows}]")
        d = EncoderDesc()
        d.layers, d.hidden, d.heads = layers, tok.shape[1], int(num_attention_heads)
        d.intermediate = arr[0].inter.rows
        d.vocab, d.max_positions, d.type_vocab = tok.shape[0], pos.shape[0], typ.shape[0]
        d.activation = ACT_GELU_ERF if hidden_act == "gelu" else ACT_GELU_TANH
        d.pooling = 1 if pooling == "cls" else 0
        d.weight_mode = int(weight_mode)
        d.attention_window = int(attention_window)
        d.epsilon = float(epsilon)
        d.token_embeddings, d.position_embeddings, d.type_embeddings = tok.ctypes.data, pos.ctypes.data, typ.ctypes.data
        d.embedding_ln_gamma, d.embedding_ln_beta = eg.ctypes.data, eb.ctypes.data
        d.layer = arr
        self.out_dim = tok.shape[1]
        if head_weights is not None:
            hw = _f32(head_weights)
            if hw.ndim != 2 or hw.shape[0] != tok.shape[1]:
                raise ValueError("projection head input dimension mismatch")
            keep.append(hw)
            d.head_out, d.head_weights = hw.shape[1], hw.ctypes.data
            self.out_dim = hw.shape[1]
        if pos.shape[1] != tok.shape[1] or typ.shape[1] != tok.shape[1] or eg.size != tok.shape[1] or eb.size != tok.shape[1]:
            raise ValueError("bert_embeddings tables disagree on the hidden size")
        self.handle = C.c_void_p()
        _lib.call("eos_b200_encoder_bind", rt.handle, C.byref(d), C.byref(self.handle))
        rt._adopt(self)
        self.hidden, self.layers, self.heads, self.intermediate = d.hidden, layers, d.heads, d.intermediate
        self.last_stats = Stats()
        self._in_flight: list = []

    def reserve(self, batch: int, tokens: int) -> None:
        _lib.call("eos_b200_encoder_reserve", self.handle, int(batch), int(tokens))

    def run(self, input_ids, attention_mask, token_type_ids=None) -> np.ndarray:
        """Host buffers in, host buffer out ([B, E] fp32); copies are part of the call."""
        ids, mask = _i32(input_ids), _i32(attention_mask)
        if ids.ndim != 2:
            raise ValueError(f"bert_embedder input_ids must be rank-2 [B,T], got shape {ids.shape}")
        if mask.shape != ids.shape:
            raise ValueError(f"bert_embedder attention_mask shape {mask.shape} does not match input_ids shape {ids.shape}")
        types = None if token_type_ids is None else _i32(token_type_ids)
        if types is not None and types.shape != ids.shape:
            raise ValueError(f"bert_embedder token_type_ids shape {types.shape} does not match input_ids shape {ids.shape}")
        out = np.empty((ids.shape[0], self.out_dim), dtype=np.float32)
        _lib.call("eos_b200_encoder_run", self.handle, _ptr(ids), _ptr(mask), _ptr(types), ids.shape[0], ids.shape[1],
                  _ptr(out), C.byref(self.last_stats))
        return out

    def submit(self, input_ids, attention_mask, out: np.ndarray, token_type_ids=None) -> None:
        """Enqueues one batch (uploads, forward, download into `out` [B, E] fp32) and returns without waiting; `wait`
        completes every batch submitted since the last wait.  The arrays must be C-contiguous int32 / float32 (they are
        not copied), stay untouched until the wait, and be page-locked for the copies to overlap."""
        ids, mask = np.asarray(input_ids), np.asarray(attention_mask)
        types = None if token_type_ids is None else np.asarray(token_type_ids)
        for name, a in (("input_ids", ids), ("attention_mask", mask), ("token_type_ids", types)):
            if a is not None and (a.dtype != np.int32 or not a.flags.c_contiguous):
                raise ValueError(f"submit: {name} must be a C-contiguous int32 array (it is used in place)")
        if ids.ndim != 2 or mask.shape != ids.shape or (types is not None and types.shape != ids.shape):
            raise ValueError("submit: input_ids, attention_mask and token_type_ids must be [B,T] arrays of one shape")
        if out.dtype != np.float32 or not out.flags.c_contiguous or out.shape != (ids.shape[0], self.out_dim):
            raise ValueError(f"submit: out must be a C-contiguous float32 array [{ids.shape[0]}, {self.out_dim}]")
        _lib.call("eos_b200_encoder_submit", self.handle, _ptr(ids), _ptr(mask), _ptr(types), ids.shape[0], ids.shape[1],
                  _ptr(out))
        if not hasattr(self, "_in_flight"):
            self._in_flight = []
        self._in_flight.append((ids, mask, types, out))   # keeps the buffers alive until the wait

    def wait(self) -> None:
        try:
            _lib.call("eos_b200_encoder_wait", self.handle, C.byref(self.last_stats))
        finally:
            if hasattr(self, "_in_flight"):
                self._in_flight.clear()

    def run_device(self, d_ids: int, d_mask: int, d_types: Optional[int], batch: int, tokens: int, d_out: int,
                   stream: Optional[int] = None) -> int:
        """Device pointers in/out (ints), enqueued on `stream` without synchronising; returns kernels launched."""
        st = Stats()
        _lib.call("eos_b200_encoder_run_device", self.handle, d_ids, d_mask, d_types, int(batch), int(tokens), d_out,
                  stream, C.byref(st))
        return st.kernel_launches

    def set_token_head(self, weights) -> None:
        """Per-token output head [hidden, token_dim] (in-major, no bias): enables token_vectors_device."""
        w = _f32(weights)
        if w.ndim != 2:
            raise ValueError("token head weights must be [hidden, token_dim]")
        _lib.call("eos_b200_encoder_set_token_head", self.handle, _ptr(w), int(w.shape[1]))
        self.token_dim = int(w.shape[1])

    def token_vectors_device(self, d_ids: int, d_mask: int, d_types: Optional[int], batch: int, tokens: int,
                             d_vectors: int, d_row_count: Optional[int] = None, stream: Optional[int] = None) -> int:
        """L2-normalised per-token vectors of the valid tokens (sequence after sequence, token order) into
        d_vectors [rows, token_dim] fp32 on the device; returns kernels launched."""
        st = Stats()
        _lib.call("eos_b200_encoder_token_vectors_device", self.handle, d_ids, d_mask, d_types, int(batch), int(tokens),
                  d_vectors, d_row_count, stream, C.byref(st))
        return st.kernel_launches

    def sync(self, stream: Optional[int] = None) -> None:
        _lib.call("eos_b200_encoder_sync", self.handle, stream)

    def profile_begin(self, max_steps: int) -> None:
        """Record CUDA events around every kernel launch of the next `max_steps` forwards."""
        _lib.call("eos_b200_encoder_profile_begin", self.handle, int(max_steps))

    def profile_end(self, stream: Optional[int] = None) -> "_lib.EncoderTimes":
        out = _lib.EncoderTimes()
        _lib.call("eos_b200_encoder_profile_end", self.handle, stream, C.byref(out))
        return out

    def close(self) -> None:
        if self.handle:
            _lib.lib().eos_b200_encoder_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class CompactEmbedder(BertEmbedder):
    """The native compact q8 encoder profile (models/default_embedding.go:461-505): token + role embeddings, rotary
    positions, bias-free projections in [in, out] layout, non-affine LayerNorm (epsilon 1e-5), tanh-GELU FFN,
    per-token L2 normalize, optional output projection, masked mean pool.  `layer_weights` holds, per layer,
    (attn_q, attn_k, attn_v, attn_o, ffn_up, ffn_down); run(tokens, attention_mask, role_ids)."""

    def __init__(self, rt: Runtime, token_embedding, role_embedding, layer_weights: Sequence[Weight],
                 num_attention_heads: int, output_projection: Optional[Weight] = None,
                 weight_mode: int = WEIGHTS_F16_RESIDENT):
        from ._lib import CompactEncoderDesc, CompactLayer
        if len(layer_weights) == 0 or len(layer_weights) % 6 != 0:
            raise ValueError(f"compact encoder expects 6 tensors per layer, got {len(layer_weights)}")
        self.rt = rt
        keep: list = []
        tok, role = _f32(token_embedding), _f32(role_embedding)
        if tok.ndim != 2 or role.ndim != 2 or tok.shape[1] != role.shape[1]:
            raise ValueError("token and role embedding tables disagree on the hidden size")
        keep += [tok, role]
        layers = len(layer_weights) // 6
        arr = (CompactLayer * layers)()
        for l in range(layers):
            w = layer_weights[l * 6:(l + 1) * 6]
            for name, mat in zip(("attn_q", "attn_k", "attn_v", "attn_o", "ffn_up", "ffn_down"), w):
                setattr(arr[l], name, _matrix(mat, keep))
        d = CompactEncoderDesc()
        d.layers, d.hidden, d.heads = layers, tok.shape[1], int(num_attention_heads)
        d.intermediate = arr[0].ffn_up.cols
        d.vocab, d.role_vocab = tok.shape[0], role.shape[0]
        d.weight_mode = int(weight_mode)
        d.token_embedding, d.role_embedding = tok.ctypes.data, role.ctypes.data
        d.layer = arr
        self.out_dim = tok.shape[1]
        if output_projection is not None:
            d.output_projection = _matrix(output_projection, keep)
            d.output_dim = d.output_projection.cols
            self.out_dim = int(d.output_dim)
        self.handle = C.c_void_p()
        _lib.call("eos_b200_compact_encoder_bind", rt.handle, C.byref(d), C.byref(self.handle))
        rt._adopt(self)
        self.hidden, self.layers, self.heads, self.intermediate = d.hidden, layers, d.heads, d.intermediate
        self.last_stats = Stats()


class EmbedPooledPipeline:
    """gather -> matmul -> normalize -> masked mean_pool (examples/embed_masked_pooled.eos:11-16)."""

    def __init__(self, rt: Runtime, token_embedding, projection, matmul_scale="none"):
        """matmul_scale: the matmul step's `scale` attribute -- "none", "rsqrt_rhs_rows" (1 / sqrt of the projection's
        row count) or a number (matmulScale, runtime/backend/tensor_ops.go:1291-1315)."""
        table, proj = _f32(token_embedding), _f32(projection)
        if table.ndim != 2 or proj.ndim != 2 or proj.shape[0] != table.shape[1]:
            raise ValueError(f"matmul mismatch {table.shape} x {proj.shape}")
        if matmul_scale in (None, "", "none"):
            scale = 1.0
        elif matmul_scale == "rsqrt_rhs_rows":
            scale = float(np.float32(1.0 / np.sqrt(float(proj.shape[0]))))
        else:
            try:
                scale = float(np.float32(float(matmul_scale)))
            except (TypeError, ValueError):
                raise ValueError(f"unsupported matmul scale {matmul_scale!r}") from None
            if not np.isfinite(scale):
                raise ValueError(f"matmul scale must be finite, got {matmul_scale!r}")
        self.rt = rt
        self.out_dim = proj.shape[1]
        self.matmul_scale = scale
        self.handle = C.c_void_p()
        _lib.call("eos_b200_embed_pooled_bind", rt.handle, _ptr(table), table.shape[0], table.shape[1], _ptr(proj),
                  proj.shape[1], C.byref(self.handle))
        if scale != 1.0:
            _lib.call("eos_b200_embed_pooled_set_matmul_scale", self.handle, C.c_float(scale))
        rt._adopt(self)
        self.last_stats = Stats()

    def run(self, tokens, attention_mask, pool_then_l2: bool = False) -> np.ndarray:
        tok, mask = _i32(tokens), _i32(attention_mask)
        if tok.ndim != 2 or tok.size == 0:
            raise ValueError("embed_pooled_batch expects a non-empty [B,T] token tensor")
        if mask.shape != tok.shape:
            raise ValueError(f"mean_pool mask shape {mask.shape} does not match input {tok.shape}")
        out = np.empty((tok.shape[0], self.out_dim), dtype=np.float32)
        _lib.call("eos_b200_embed_pooled_run", self.handle, _ptr(tok), _ptr(mask), tok.shape[0], tok.shape[1],
                  1 if pool_then_l2 else 0, _ptr(out), C.byref(self.last_stats))
        return out

    def close(self) -> None:
        if self.handle:
            _lib.lib().eos_b200_embed_pooled_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def linear(rt: Runtime, x, weight: Weight, bias=None, epilogue: int = EPILOGUE_NONE, residual=None,
           weight_mode: int = WEIGHTS_Q8_SMEM_DEQUANT, stats: Optional[Stats] = None) -> np.ndarray:
    """y = epilogue(x W^T + b) through the tensor-core projection kernel; x, residual and y are f16-rounded."""
    keep: list = []
    xa = _f32(x)
    m = _matrix(weight, keep)
    if xa.shape[-1] != m.cols:
        raise ValueError(f"dense weight shape [{m.rows},{m.cols}] does not match input width {xa.shape[-1]}")
    rows = xa.size // m.cols
    b = None if bias is None else _f32(bias)
    r = None if residual is None else _f32(residual)
    out = np.empty(xa.shape[:-1] + (m.rows,), dtype=np.float32)
    st = stats if stats is not None else Stats()
    _lib.call("eos_b200_linear", rt.handle, _ptr(xa), rows, C.byref(m), _ptr(b), int(epilogue), _ptr(r),
              int(weight_mode), _ptr(out), C.byref(st))
    return out
