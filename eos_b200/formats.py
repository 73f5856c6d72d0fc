"""On-disk payloads either side of the embed-and-score path, read without the Go host.

Tensor payloads of the weight container -- the bytes runtime/mll_export.go:902-1005 writes per tensor (packed q8 /
q4 codes with one `tensor_scales` entry each, f16, f32, i32, i64) -- and the JSONL vector caches of
runtime/retrieval_vector_export.go:83-88,424-523 as read by runtime/retrieval_eval.go:629-778.

The container's own framing (section table, string table, digests) belongs to the m31labs.dev/mll module, which the
reference tree does not carry; a caller that has split the container into (name, storage dtype, shape, raw bytes)
and the `tensor_scales` map hands those here.
"""
from __future__ import annotations

import json
import math
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np

from .encoder import Q8Weight, Q8WeightInOut

STORAGE_DTYPES = ("f32", "f16", "i32", "i64", "q8", "q4")


def _count(shape: Sequence[int]) -> int:
    n = 1
    for d in shape:
        if d < 0:
            raise ValueError(f"negative dim {d}")
        n *= int(d)
    return n


def pack_quantized_tensor(values, bits: int) -> Tuple[bytes, float]:
    """packQuantizedTensorStorage (runtime/mll_export.go:902-962): one scale = max|x| / (2^(bits-1) - 1), codes =
    round-half-away(x / scale) clamped; q8 one byte per code, q4 two offset-binary nibbles per byte, low first."""
    if bits not in (4, 8):
        raise ValueError(f"tensor bit width {bits} is not packable")
    x = np.ascontiguousarray(values, dtype=np.float32).reshape(-1)
    levels = np.float32((1 << (bits - 1)) - 1)
    max_abs = np.float32(np.abs(x).max()) if x.size else np.float32(0)
    scale = np.float32(max_abs / levels) if max_abs > 0 else np.float32(0)
    codes = np.zeros(x.size, dtype=np.int8)
    if scale > 0:
        ratio = (x / scale).astype(np.float64)
        q = np.sign(ratio) * np.floor(np.abs(ratio) + 0.5)          # math.Round: half away from zero
        codes = np.clip(q, -float(levels), float(levels)).astype(np.int8)
    if bits == 8:
        return codes.tobytes(), float(scale)
    nib = ((codes.astype(np.int16) + 8) & 0x0F).astype(np.uint8)
    if nib.size % 2:
        nib = np.concatenate([nib, np.zeros(1, np.uint8)])
    return (nib[0::2] | (nib[1::2] << 4)).astype(np.uint8).tobytes(), float(scale)


def unpack_quantized_codes(raw: bytes, shape: Sequence[int], bits: int) -> np.ndarray:
    """The int8 codes of a packed q8 / q4 payload, shaped."""
    n = _count(shape)
    data = np.frombuffer(raw, dtype=np.uint8)
    if bits == 8:
        if data.size != n:
            raise ValueError(f"q8 payload holds {data.size} codes, shape wants {n}")
        return data.view(np.int8).reshape(tuple(shape)).copy()
    if bits == 4:
        if data.size != (n + 1) // 2:
            raise ValueError(f"q4 payload holds {data.size} bytes, shape wants {(n + 1) // 2}")
        nib = np.empty(data.size * 2, dtype=np.int16)
        nib[0::2] = data & 0x0F
        nib[1::2] = data >> 4
        return (nib[:n] - 8).astype(np.int8).reshape(tuple(shape))
    raise ValueError(f"tensor bit width {bits} is not packable")


def decode_tensor_payload(storage: str, raw: bytes, shape: Sequence[int], scale: Optional[float] = None) -> np.ndarray:
    """One tensor's bytes -> values (fp32 for f32 / f16 / q8 / q4, int32 / int64 for the integer types), little endian
    as encodeTensorStorage writes them (runtime/mll_export.go:964-1005).  q8 / q4 need the tensor's scale."""
    shape = tuple(int(d) for d in shape)
    n = _count(shape)
    plain = {"f32": "<f4", "f16": "<f2", "i32": "<i4", "i64": "<i8"}
    if storage in plain:
        a = np.frombuffer(raw, dtype=plain[storage])
        if a.size != n:
            raise ValueError(f"{storage} payload holds {a.size} values, shape wants {n}")
        out = a.reshape(shape)
        return out.astype(np.float32) if storage in ("f32", "f16") else out.astype(a.dtype.newbyteorder("="))
    if storage in ("q8", "q4"):
        if scale is None or not math.isfinite(scale):
            raise ValueError(f"{storage} payload needs its tensor_scales entry")
        codes = unpack_quantized_codes(raw, shape, 8 if storage == "q8" else 4)
        return codes.astype(np.float32) * np.float32(scale)
    raise ValueError(f"unsupported tensor dtype {storage!r}")


def q8_weight_from_payload(raw: bytes, shape: Sequence[int], scale: float, layout: str = "out_in"):
    """A packed q8 matrix payload as a bind-ready weight: the codes go to the device as they are, the tensor's scale
    becomes the per-tensor scale of the projection (no dequantise / requantise round trip).  layout "out_in" is the
    encoder's dense layout [out, in] (Q8Weight), "in_out" the matmul layout [in, out] (Q8WeightInOut)."""
    if len(shape) != 2:
        raise ValueError("a projection weight is a matrix")
    codes = unpack_quantized_codes(raw, shape, 8)
    scales = np.array([scale], dtype=np.float32)
    if layout == "out_in":
        return Q8Weight(codes, scales)
    if layout == "in_out":
        return Q8WeightInOut(codes, scales)
    raise ValueError(f"unknown layout {layout!r}")


def load_tensor_payloads(tensors: Iterable[Tuple[str, str, Sequence[int], bytes]],
                         tensor_scales: Optional[Dict[str, float]] = None) -> Dict[str, np.ndarray]:
    """(name, storage dtype, shape, raw) entries + the `tensor_scales` metadata map -> name -> values."""
    scales = tensor_scales or {}
    out: Dict[str, np.ndarray] = {}
    for name, storage, shape, raw in tensors:
        try:
            out[name] = decode_tensor_payload(storage, raw, shape, scales.get(name))
        except ValueError as e:
            raise ValueError(f"tensor {name!r}: {e}") from None
    return out


# ---------------------------------------------------------------------------------------- JSONL vector caches
def _first_non_empty(*values) -> str:
    for v in values:
        v = (v or "").strip() if isinstance(v, str) else ""
        if v:
            return v
    return ""


def _first_vector(record: dict):
    for key in ("vector", "embedding", "values"):   # firstRetrievalVector, runtime/retrieval_eval.go:780-789
        v = record.get(key)
        if v:
            return v
    return []


def normalize_retrieval_vector(v) -> np.ndarray:
    """normalizeRetrievalVector (runtime/retrieval_eval.go:1040-1054): sum of squares in double, one fp32 scale."""
    out = np.array(v, dtype=np.float32)
    total = float((out.astype(np.float64) ** 2).sum())
    if total == 0:
        return out
    return out * np.float32(1.0 / math.sqrt(total))


def write_vector_cache(path: str, ids: Sequence[str], vectors) -> int:
    """One {"id", "embedding"} row per line (retrievalVectorExportRow, runtime/retrieval_vector_export.go:83-88)."""
    v = np.asarray(vectors, dtype=np.float32)
    if v.ndim != 2 or v.shape[0] != len(ids):
        raise ValueError("ids and vectors disagree")
    with open(path, "w", encoding="utf-8") as f:
        for i, vec in zip(ids, v):
            if vec.size == 0:
                raise ValueError(f"vector for {i!r} is empty")
            f.write(json.dumps({"id": i, "embedding": [float(x) for x in vec]}, separators=(",", ":")) + "\n")
    return v.shape[1]


def write_child_vector_cache(path: str, parent_ids: Sequence[str], child_ids: Sequence[str], vectors) -> int:
    v = np.asarray(vectors, dtype=np.float32)
    if v.ndim != 2 or v.shape[0] != len(parent_ids) or len(parent_ids) != len(child_ids):
        raise ValueError("ids and vectors disagree")
    with open(path, "w", encoding="utf-8") as f:
        for p, c, vec in zip(parent_ids, child_ids, v):
            f.write(json.dumps({"parent_id": p, "child_id": c, "embedding": [float(x) for x in vec]},
                               separators=(",", ":")) + "\n")
    return v.shape[1]


def read_vector_cache(path: str, ordered_ids: Sequence[str]) -> Tuple[List[str], np.ndarray, int, int]:
    """readRetrievalVectorCache (runtime/retrieval_eval.go:629-693): the vectors of the wanted ids in the wanted order
    (first occurrence wins, each L2-normalised), the count of wanted ids the file lacks, and the dimension."""
    needed = {i for i in ordered_ids if i}
    found: Dict[str, np.ndarray] = {}
    dim = 0
    with open(path, "r", encoding="utf-8") as f:
        for line_no, line in enumerate(f, 1):
            line = line.strip()
            if not line:
                continue
            try:
                rec = json.loads(line)
            except json.JSONDecodeError as e:
                raise ValueError(f"{path}:{line_no}: {e}") from None
            rid = _first_non_empty(rec.get("id"), rec.get("_id"))
            if not rid or rid not in needed:
                continue
            vec = _first_vector(rec)
            if len(vec) == 0:
                raise ValueError(f"{path}:{line_no}: vector for {rid!r} is empty")
            if dim == 0:
                dim = len(vec)
            elif len(vec) != dim:
                raise ValueError(f"{path}:{line_no}: vector for {rid!r} has dimension {len(vec)}, want {dim}")
            if rid not in found:
                found[rid] = normalize_retrieval_vector(vec)
    ids = [i for i in ordered_ids if i in found]
    missing = sum(1 for i in ordered_ids if i not in found)
    mat = np.stack([found[i] for i in ids]) if ids else np.zeros((0, dim), np.float32)
    return ids, mat, missing, dim


def read_child_vector_cache(path: str, ordered_parent_ids: Sequence[str]):
    """readRetrievalChildVectorCache (runtime/retrieval_eval.go:695-768): child vectors grouped by parent in the order
    of ordered_parent_ids (file order inside a parent), each L2-normalised.  Returns (parent_of_child int32 -- the
    index into ordered_parent_ids, which eos_b200_parent_topk takes --, child ids, vectors, missing parents, dim)."""
    needed = {p: i for i, p in enumerate(ordered_parent_ids) if p}
    by_parent: Dict[str, List[Tuple[str, np.ndarray]]] = {}
    dim = 0
    with open(path, "r", encoding="utf-8") as f:
        for line_no, line in enumerate(f, 1):
            line = line.strip()
            if not line:
                continue
            try:
                rec = json.loads(line)
            except json.JSONDecodeError as e:
                raise ValueError(f"{path}:{line_no}: {e}") from None
            rid = _first_non_empty(rec.get("id"), rec.get("_id"))
            parent = _first_non_empty(rec.get("parent_id"), rid)
            child = _first_non_empty(rec.get("child_id"), rid, parent)
            if not parent or parent not in needed:
                continue
            vec = _first_vector(rec)
            if len(vec) == 0:
                raise ValueError(f"{path}:{line_no}: vector for parent {parent!r} child {child!r} is empty")
            if dim == 0:
                dim = len(vec)
            elif len(vec) != dim:
                raise ValueError(f"{path}:{line_no}: vector for parent {parent!r} child {child!r} has dimension "
                                 f"{len(vec)}, want {dim}")
            by_parent.setdefault(parent, []).append((child, normalize_retrieval_vector(vec)))
    parent_of_child: List[int] = []
    child_ids: List[str] = []
    rows: List[np.ndarray] = []
    missing = 0
    for idx, parent in enumerate(ordered_parent_ids):
        children = by_parent.get(parent, [])
        if not children:
            missing += 1
            continue
        for child, vec in children:
            parent_of_child.append(idx)
            child_ids.append(child)
            rows.append(vec)
    mat = np.stack(rows) if rows else np.zeros((0, dim), np.float32)
    return np.asarray(parent_of_child, dtype=np.int32), child_ids, mat, missing, dim
