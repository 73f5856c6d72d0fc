"""Seeded synthetic weights and batches with the shapes and value distributions of the benchmark configurations.

No dataset or checkpoint is involved: weights are random-initialised, tokens are uniform, lengths are uniform in a
range.  The q8 rule is the reference's (runtime/embedding_trainer.go:11413-11446): symmetric abs-max, 127 levels,
round half away from zero, here with one scale per output channel, rounded to f16.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import numpy as np

from .encoder import Q8Weight


def f16_round(a: np.ndarray) -> np.ndarray:
    return np.asarray(a, dtype=np.float32).astype(np.float16).astype(np.float32)


def quantize_per_channel(w: np.ndarray) -> Q8Weight:
    """w [out, in] fp32 -> int8 codes + per-row f16-rounded scales; all-zero rows get scale 0 / codes 0."""
    w = np.asarray(w, dtype=np.float32)
    max_abs = np.abs(w).max(axis=1)
    scale = f16_round(max_abs / np.float32(127.0))
    safe = np.where(scale == 0, np.float32(1.0), scale).astype(np.float32)
    q = (w / safe[:, None]).astype(np.float32)
    q = np.sign(q) * np.floor(np.abs(q).astype(np.float64) + 0.5)
    q = np.clip(q, -127, 127)
    q[scale == 0] = 0
    return Q8Weight(q.astype(np.int8), scale.astype(np.float32))


def make_q8_encoder(layers: int, hidden: int, heads: int, inter: int, vocab: int, max_pos: int, seed: int,
                    head_out: int = 0, type_vocab: int = 2) -> Dict[str, object]:
    """Random-init q8 encoder: f16 tables ~N(0, 0.02), int8 per-channel dense weights from N(0, 0.02),
    small biases, LayerNorm gamma near 1.  Returns the constructor arguments of BertEmbedder."""
    rng = np.random.default_rng(seed)

    def normal(shape, std):
        return (rng.standard_normal(shape, dtype=np.float32) * np.float32(std)).astype(np.float32)

    out: Dict[str, object] = {
        "token_embeddings": f16_round(normal((vocab, hidden), 0.02)),
        "position_embeddings": f16_round(normal((max_pos, hidden), 0.02)),
        "token_type_embeddings": f16_round(normal((type_vocab, hidden), 0.02)),
        "embedding_ln_weight": 1.0 + normal((hidden,), 0.02),
        "embedding_ln_bias": normal((hidden,), 0.02),
        "num_attention_heads": heads,
    }
    lw: List[object] = []

    def dense(o, i):
        lw.append(quantize_per_channel(normal((o, i), 0.02)))
        lw.append(normal((o,), 0.02))

    def layernorm():
        lw.append(1.0 + normal((hidden,), 0.02))
        lw.append(normal((hidden,), 0.02))

    for _ in range(layers):
        dense(hidden, hidden)  # query
        dense(hidden, hidden)  # key
        dense(hidden, hidden)  # value
        dense(hidden, hidden)  # attention output
        layernorm()
        dense(inter, hidden)   # intermediate
        dense(hidden, inter)   # output
        layernorm()
    assert len(lw) == layers * 16
    out["layer_weights"] = lw
    if head_out > 0:
        out["head_weights"] = f16_round(normal((hidden, head_out), 0.05))
    return out


def dequantized_layer_weights(layer_weights) -> List[np.ndarray]:
    """The fp32 tensors the CPU oracle consumes (value = code * scale)."""
    return [w.dequantized() if isinstance(w, Q8Weight) else np.asarray(w, np.float32) for w in layer_weights]


def make_batch(batch: int, tokens: int, vocab: int, min_len: int, max_len: int, seed: int
               ) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """Uniform random tokens, lengths uniform in [min_len, max_len], mask 1 on t < len: (ids, mask, lengths)."""
    rng = np.random.default_rng(seed)
    ids = rng.integers(0, vocab, size=(batch, tokens), dtype=np.int32)
    lengths = rng.integers(min_len, max_len + 1, size=batch).astype(np.int32)
    mask = (np.arange(tokens, dtype=np.int32)[None, :] < lengths[:, None]).astype(np.int32)
    return ids, mask, lengths


def encoder_flops(lengths: np.ndarray, layers: int, hidden: int, inter: int, head_out: int = 0) -> float:
    """Algorithmic flops on valid tokens only: per sequence of length l and per layer
    2 l (4 D^2 + 2 D F) for the projections and 4 l^2 D for attention, plus 2 D E for the head."""
    l = lengths.astype(np.float64)
    per_layer = 2.0 * l * (4.0 * hidden * hidden + 2.0 * hidden * inter) + 4.0 * l * l * hidden
    return float((layers * per_layer + 2.0 * hidden * head_out).sum())


def gemm_flops(lengths: np.ndarray, layers: int, hidden: int, inter: int) -> float:
    l = lengths.astype(np.float64)
    return float((layers * 2.0 * l * (4.0 * hidden * hidden + 2.0 * hidden * inter)).sum())
