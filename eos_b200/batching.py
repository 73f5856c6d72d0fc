"""Host-side batch construction for the encoder entry points, with the reference's semantics.

    build_masked_token_inputs   buildMaskedTokenInputs, runtime/embedding_model.go:1457-1495
    pad_bert_batch              padPretrainedBERTBatchEncodings, runtime/pretrained_bert_retrieval_vector_export.go:615-646
    build_token_batch           buildTokenBatch, runtime/inference.go:323-339
    split_by_length             contiguous per-GPU slices of a length-sorted batch, so that the valid-token counts of
                                the data-parallel ranks balance (the reference groups by length before it batches:
                                runtime/embedding_model.go:798-881)
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np


def build_masked_token_inputs(batches: Sequence[Sequence[int]], pad_id: int) -> Tuple[np.ndarray, np.ndarray]:
    """Pads to the longest row with pad_id; mask = 1 on every token up to the last one that is not pad_id (trailing
    pad_id tokens that a row already carries are masked too), 0 elsewhere.  Returns int32 [B, T] tokens and mask."""
    if len(batches) == 0:
        raise ValueError("token batches are empty")
    for i, row in enumerate(batches):
        if len(row) == 0:
            raise ValueError(f"token batch {i} is empty")
    max_len = max(len(row) for row in batches)
    tokens = np.full((len(batches), max_len), pad_id, dtype=np.int32)
    mask = np.zeros((len(batches), max_len), dtype=np.int32)
    for i, row in enumerate(batches):
        r = np.asarray(row, dtype=np.int32)
        tokens[i, :r.size] = r
        active = r.size
        while active > 0 and r[active - 1] == pad_id:
            active -= 1
        mask[i, :active] = 1
    return tokens, mask


def pad_bert_batch(ids: Sequence[Sequence[int]], attention_masks: Sequence[Sequence[int]],
                   token_type_ids: Sequence[Sequence[int]], length: int, pad_id: int
                   ) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """Pads word-piece encodings to `length`: ids with pad_id, mask and token types with 0; a row longer than `length`
    or with inconsistent parts is an error, as in the reference."""
    if length <= 0:
        raise ValueError(f"pretrained BERT batch padded length must be positive, got {length}")
    b = len(ids)
    out_ids = np.full((b, length), pad_id, dtype=np.int32)
    out_mask = np.zeros((b, length), dtype=np.int32)
    out_types = np.zeros((b, length), dtype=np.int32)
    for row in range(b):
        n = len(ids[row])
        if n > length:
            raise ValueError(f"encoded row {row} length {n} exceeds padded length {length}")
        if len(attention_masks[row]) != n or len(token_type_ids[row]) != n:
            raise ValueError(f"encoded row {row} has inconsistent ids/masks/token types lengths: "
                             f"{n}/{len(attention_masks[row])}/{len(token_type_ids[row])}")
        out_ids[row, :n] = ids[row]
        out_mask[row, :n] = attention_masks[row]
        out_types[row, :n] = token_type_ids[row]
    return out_ids, out_mask, out_types


def build_token_batch(batches: Sequence[Sequence[int]]) -> np.ndarray:
    """Equal-length rows stacked into int32 [B, T]."""
    if len(batches) == 0:
        raise ValueError("token batches are empty")
    if len(batches[0]) == 0:
        raise ValueError("token batch 0 is empty")
    t = len(batches[0])
    for i, row in enumerate(batches):
        if len(row) != t:
            raise ValueError(f"token batch {i} size {len(row)} does not match {t}")
    return np.asarray(batches, dtype=np.int32).reshape(len(batches), t)


def split_by_length(lengths: Sequence[int], world: int) -> List[np.ndarray]:
    """Row indices for each of `world` ranks: rows sorted by valid length (stable), dealt round-robin, so every rank
    gets the same number of rows (+-1) and nearly the same number of valid tokens.  Concatenating the per-rank outputs
    and applying the inverse permutation (np.argsort(np.concatenate(result))) restores the original order."""
    if world <= 0:
        raise ValueError("world must be positive")
    order = np.argsort(np.asarray(lengths), kind="stable")
    return [order[r::world] for r in range(world)]
