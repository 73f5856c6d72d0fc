"""Host-side readers of the on-disk payloads either side of the path (no device): the tensor payload rules of
runtime/mll_export.go:902-1005 and the JSONL vector caches of runtime/retrieval_eval.go:629-778."""
import json
import struct

import numpy as np
import pytest

from eos_b200 import formats as F


def test_packed_q8_payload_follows_the_export_rule():
    rng = np.random.default_rng(1)
    w = (rng.standard_normal((7, 12)) * 0.3).astype(np.float32)
    w[0, 0] = 0.5 * float(np.abs(w).max()) / 127 * 3    # a value that lands exactly between two codes
    raw, scale = F.pack_quantized_tensor(w, 8)
    assert len(raw) == w.size and scale == pytest.approx(float(np.abs(w).max()) / 127, rel=1e-7)
    codes = F.unpack_quantized_codes(raw, w.shape, 8)
    assert codes.dtype == np.int8 and np.abs(codes).max() == 127
    # round half away from zero, as math.Round
    r = w.astype(np.float32) / np.float32(scale)
    want = np.clip(np.sign(r) * np.floor(np.abs(r.astype(np.float64)) + 0.5), -127, 127)
    assert np.array_equal(codes, want.astype(np.int8))
    vals = F.decode_tensor_payload("q8", raw, w.shape, scale)
    assert np.abs(vals - w).max() <= scale / 2 + 1e-7
    wt = F.q8_weight_from_payload(raw, w.shape, scale)
    assert np.array_equal(wt.codes, codes) and wt.scales.tolist() == [np.float32(scale)]
    assert np.array_equal(wt.dequantized(), vals)
    assert isinstance(F.q8_weight_from_payload(raw, w.shape, scale, "in_out"), F.Q8WeightInOut)
    # the oracle's grid rule agrees (quantizeSymmetric, the same max / 127 grid)
    from oracle import oracle as O
    ocodes, oscales = O.quantize_symmetric(w.reshape(1, -1), 0, 8)
    assert np.array_equal(ocodes.reshape(w.shape), codes) and float(oscales[0]) == pytest.approx(scale, rel=1e-7)


def test_packed_q4_nibbles_low_first():
    vals = np.array([-7, 7, 0, 3, -3], np.float32)
    raw, scale = F.pack_quantized_tensor(vals, 4)
    assert scale == 1.0 and len(raw) == 3
    assert list(raw) == [(1) | (15 << 4), (8) | (11 << 4), 5]   # code + 8, low nibble first
    assert np.array_equal(F.unpack_quantized_codes(raw, (5,), 4), vals.astype(np.int8))
    assert np.array_equal(F.decode_tensor_payload("q4", raw, (5,), scale), vals)
    zr, zs = F.pack_quantized_tensor(np.zeros(4, np.float32), 8)
    assert zs == 0.0 and zr == bytes(4)


def test_plain_payloads_and_errors():
    a = np.arange(6, dtype=np.float32).reshape(2, 3) - 2.5
    assert np.array_equal(F.decode_tensor_payload("f32", a.astype("<f4").tobytes(), (2, 3)), a)
    assert np.array_equal(F.decode_tensor_payload("f16", a.astype("<f2").tobytes(), (2, 3)), a)
    assert np.array_equal(F.decode_tensor_payload("i32", struct.pack("<3i", 1, -2, 3), (3,)), [1, -2, 3])
    assert np.array_equal(F.decode_tensor_payload("i64", struct.pack("<2q", 1 << 40, -5), (2,)), [1 << 40, -5])
    with pytest.raises(ValueError):
        F.decode_tensor_payload("f32", b"\0" * 8, (3,))
    with pytest.raises(ValueError):
        F.decode_tensor_payload("q8", b"\0" * 4, (4,))          # no scale
    with pytest.raises(ValueError):
        F.decode_tensor_payload("bf16", b"", (0,))
    out = F.load_tensor_payloads([("w", "q8", (2, 2), bytes([1, 255, 127, 129])), ("b", "f32", (2,), a[0, :2].tobytes())],
                                 {"w": 0.5})
    assert np.array_equal(out["w"], np.array([[0.5, -0.5], [63.5, -63.5]], np.float32))
    with pytest.raises(ValueError, match="'w'"):
        F.load_tensor_payloads([("w", "q8", (2, 2), bytes(4))], {})


def test_vector_caches_round_trip(tmp_path):
    rng = np.random.default_rng(2)
    vecs = rng.standard_normal((5, 8)).astype(np.float32)
    ids = ["d3", "d1", "d4", "d0", "d2"]
    p = tmp_path / "doc-vectors.jsonl"
    assert F.write_vector_cache(str(p), ids, vecs) == 8
    with open(p, "a", encoding="utf-8") as f:
        f.write("\n")
        f.write(json.dumps({"_id": "d9", "vector": [3, 4, 0, 0, 0, 0, 0, 0]}) + "\n")     # other accepted field names
        f.write(json.dumps({"id": "d1", "values": [1] * 8}) + "\n")                        # duplicate: first wins
    got_ids, mat, missing, dim = F.read_vector_cache(str(p), ["d0", "d9", "nope", "d1"])
    assert got_ids == ["d0", "d9", "d1"] and missing == 1 and dim == 8
    assert np.allclose(np.linalg.norm(mat, axis=1), 1, atol=1e-6)
    assert np.allclose(mat[0], vecs[3] / np.linalg.norm(vecs[3]), atol=1e-6)
    assert np.allclose(mat[1], [0.6, 0.8, 0, 0, 0, 0, 0, 0], atol=1e-7)
    assert np.allclose(mat[2], vecs[1] / np.linalg.norm(vecs[1]), atol=1e-6)
    with open(p, "a", encoding="utf-8") as f:
        f.write(json.dumps({"id": "d0", "embedding": [1, 2]}) + "\n")
    with pytest.raises(ValueError, match="dimension 2"):
        F.read_vector_cache(str(p), ["d0"])


def test_child_vector_cache_groups_by_parent(tmp_path):
    p = tmp_path / "child-doc-vectors.jsonl"
    parents = ["b", "a", "b", "c", "a"]
    children = ["b#0", "a#0", "b#1", "c#0", "a#1"]
    vecs = np.eye(5, 4, dtype=np.float32) + 1
    F.write_child_vector_cache(str(p), parents, children, vecs)
    poc, cids, mat, missing, dim = F.read_child_vector_cache(str(p), ["a", "zz", "b"])
    assert poc.tolist() == [0, 0, 2, 2] and cids == ["a#0", "a#1", "b#0", "b#1"] and missing == 1 and dim == 4
    assert np.allclose(mat[1], vecs[4] / np.linalg.norm(vecs[4]), atol=1e-6)
    # a row with only an id is its own parent and child
    with open(p, "a", encoding="utf-8") as f:
        f.write(json.dumps({"id": "solo", "embedding": [0, 0, 2, 0]}) + "\n")
    poc, cids, mat, missing, dim = F.read_child_vector_cache(str(p), ["solo"])
    assert poc.tolist() == [0] and cids == ["solo"] and np.array_equal(mat[0], [0, 0, 1, 0])
