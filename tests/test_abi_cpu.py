"""CPU-only checks of the boundary: the library loads without a GPU, exports every symbol the header declares,
and fails loudly (no fallback) when asked to compute without a device."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "eos_b200.h")).read()
    return sorted(set(re.findall(r"EOS_B200_API\s+[\w\s\*]+?\b(eos_b200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from eos_b200 import _lib
    if not os.path.exists(_lib.LIB_PATH):
        from eos_b200 import build
        build.build()
    handle = _lib.lib()
    declared = _declared_symbols()
    assert len(declared) >= 30
    for name in declared:
        assert hasattr(handle, name), name
    assert sorted(_lib.SYMBOLS) == declared          # the Python binding covers the whole header
    assert handle.eos_b200_version().startswith(b"eos_b200")


def test_struct_layouts_match_the_header():
    from eos_b200 import _lib
    assert C.sizeof(_lib.Matrix) == 40
    assert C.sizeof(_lib.EncoderLayer) == 6 * 40 + 10 * 8
    assert _lib.EncoderDesc.epsilon.offset == 48
    assert C.sizeof(_lib.CompactLayer) == 6 * 40
    assert C.sizeof(_lib.CompactEncoderDesc) == 8 * 4 + 3 * 8 + 40
    assert C.sizeof(_lib.Stats) == 40
    assert C.sizeof(_lib.EncoderTimes) == 60


def test_no_cpu_fallback_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import eos_b200
    with pytest.raises(eos_b200.EosB200Error) as e:
        eos_b200.Runtime(0)
    assert "no CPU fallback" in str(e.value)


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "eos_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.replace("CPU oracle consumes", ""), f


def test_rotation_spec_and_lloyd_max_tables():
    import eos_b200
    c, b = eos_b200.lloyd_max_gaussian(16, 1.0)
    # textbook 16-level Lloyd-Max levels of the unit normal
    np.testing.assert_allclose(c[8:], [0.1284, 0.3881, 0.6568, 0.9424, 1.256, 1.618, 2.069, 2.733], atol=2e-3)
    assert np.array_equal(c, -c[::-1]) and np.all(np.diff(c) > 0)
    np.testing.assert_allclose(b, (c[:-1] + c[1:]) / 2, atol=1e-7)
    c4, _ = eos_b200.lloyd_max_gaussian(4, 1.0)
    np.testing.assert_allclose(c4, [-1.510, -0.4528, 0.4528, 1.510], atol=2e-3)
    s = eos_b200.make_rotation_spec(768, 4, seed=402)
    assert sorted(s.perm.tolist()) == list(range(768)) and set(np.unique(s.signs1)) <= {-1.0, 1.0}
    assert s.vector_bytes == 388                      # 384 code bytes + f32 norm (config 4)
    assert eos_b200.make_rotation_spec(128, 2).vector_bytes == 36
    s2 = eos_b200.make_rotation_spec(768, 4, seed=402)
    assert np.array_equal(s.perm, s2.perm) and np.array_equal(s.signs2, s2.signs2)


def test_oracle_turboquant_round_trip_properties():
    """The oracle's own consistency (parity for TurboQuant is unpinned: these are structural checks)."""
    import eos_b200
    from oracle import oracle as O
    spec = eos_b200.make_rotation_spec(768, 4, seed=402)
    rng = np.random.default_rng(0)
    x = rng.standard_normal((50, 768)).astype(np.float32)
    # the rotation is orthogonal: norms and inner products are preserved
    r0 = O.tq_rotate(x[0], spec.perm, spec.signs1, spec.signs2)
    r1 = O.tq_rotate(x[1], spec.perm, spec.signs1, spec.signs2)
    assert abs(np.linalg.norm(r0) - np.linalg.norm(x[0])) < 1e-3
    assert abs(float(r0 @ r1) - float(x[0] @ x[1])) < 1e-2
    codes, norms = O.tq_encode(x, 4, spec.perm, spec.signs1, spec.signs2, spec.boundaries)
    assert codes.shape == (50, 384) and np.allclose(norms, np.linalg.norm(x, axis=1), rtol=1e-6)
    dec = O.tq_decode(codes, norms, 768, 4, spec.perm, spec.signs1, spec.signs2, spec.centroids)
    cos = (dec * x).sum(1) / (np.linalg.norm(dec, axis=1) * np.linalg.norm(x, axis=1))
    assert cos.min() > 0.99                            # 16 levels: about 1 % distortion
    # score(query, doc) == <query, decode(doc)> up to float rounding
    prep = O.tq_prepare_query(x[3], spec.perm, spec.signs1, spec.signs2)
    sc = O.tq_score(codes, norms, 768, 4, spec.centroids, prep)
    np.testing.assert_allclose(sc, dec @ x[3], rtol=0, atol=2e-3 * float(np.abs(sc).max()))
    # zero vector: norm 0, score 0 (runtime/turboquant_quantized_vector.go:15-19)
    zc, zn = O.tq_encode(np.zeros((1, 768), np.float32), 4, spec.perm, spec.signs1, spec.signs2, spec.boundaries)
    assert zn[0] == 0 and O.tq_score(zc, zn, 768, 4, spec.centroids, prep)[0] == 0
    # multi-vector parents: max aggregation equals the per-parent maximum
    parent = rng.integers(0, 7, size=50).astype(np.int32)
    ids, ps = O.parent_topk(sc, parent, 7, 7)
    for i, p in zip(ids, ps):
        assert p == sc[parent == i].max()


def test_sparse_attention_plan_matches_oracle_knobs():
    """PlanSparseAttention (runtime/backend/attention_ops.go:78-141): the host mirror normalises the knobs like the
    oracle's restatement of sparseAttentionBudget / normalizeSparseAttentionRoute."""
    from eos_b200.attention import plan_sparse_attention
    from oracle import oracle as O
    for kl, tk, bs, tb in [(50, 0, 0, 0), (1000, 32, 64, 4), (1000, 0, 37, 128), (3, 10, 0, 0), (0, 5, 4, 4)]:
        plan = plan_sparse_attention(8, kl, tk, bs, tb)
        assert plan.top_k == (O.sparse_attention_budget(tk, kl) if kl > 0 else tk)
        assert (plan.route_block_size, plan.route_top_blocks) == O.sparse_attention_route(kl, bs, tb)


def test_log8_norm_sidecar_matches_the_oracle():
    """Host arithmetic of the C ABI (no device): the 8-bit log-scale norm codes of the reference's encode
    (runtime/backends/cuda/native_linux.go:1879-1904) against the oracle's restatement, edge values included."""
    from eos_b200.turboquant import norm_decode_log8, norm_encode_log8
    from oracle import oracle as O
    rng = np.random.default_rng(3)
    norms = np.concatenate([np.exp(rng.uniform(-20, 20, 5000)).astype(np.float32),
                            np.array([0.0, -1.0, np.inf, np.nan, 1.0, 1e-7, 8886110.0, 1e7], np.float32)])
    codes = norm_encode_log8(norms)
    assert np.array_equal(codes, O.tq_norm_code(norms))
    allc = np.arange(256, dtype=np.uint8)
    assert np.array_equal(norm_decode_log8(allc).view(np.uint32), O.tq_norm_value(allc).view(np.uint32))
    assert codes[-8] == 0 and codes[-7] == 0 and codes[-6] == 255 and codes[-5] == 0


def test_token_spans_follow_the_oracle():
    """sparseTokenPoolTokenSpans (runtime/sparse_token_pool_vector_export.go:1561-1595): host mirror vs the oracle."""
    from eos_b200.token_pool import token_spans
    from oracle import oracle as O
    for args in [(10, 4, 1, 2), (3, 4, 1, 2), (3, 4, 1, 5), (10, 4, 4, 1), (0, 4, 0, 1), (100, 16, 4, 3), (17, 16, 0, 2),
                 (33, 16, 0, 0), (64, 64, 8, 1)]:
        assert token_spans(*args) == O.token_spans(*args), args
