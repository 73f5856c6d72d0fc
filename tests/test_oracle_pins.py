"""Pins the CPU oracle to the reference's own known answers (CPU only).

Sources of the expected values:
  * tests/golden/bert_tiny_golden.npz -- Eos's runtime/testdata/pretrained_bert_golden fixture,
    tolerance of runtime/pretrained_bert_golden_parity_test.go:99-103.
  * tests/golden/bert_hf_seeded.npz -- a larger transformers BertModel case made like Eos's fixture.
  * hand-computed expectations copied as numbers from runtime/backend/tensor_ops_test.go,
    bert_embedding_ops_test.go and bert_encoder_layer_ops_test.go.
"""
import math

import numpy as np
import pytest

from oracle import oracle as O
from tests.helpers import cosine_rows, load_bert_fixture


@pytest.mark.parametrize("name", ["bert_tiny_golden.npz", "bert_hf_seeded.npz"])
def test_embedder_matches_golden(name):
    z, weights = load_bert_fixture(name)
    out = O.bert_embedder(z["input_ids"], z["attention_mask"], z["token_type_ids"], z["tok"], z["pos"], z["typ"],
                          z["emb_gamma"], z["emb_beta"], weights, int(z["heads"]), float(z["eps"]), "masked_mean")
    assert np.abs(out - z["expected"]).max() <= 2e-3
    assert cosine_rows(out, z["expected"]).min() >= 0.9999
    # tighter than the reference tolerance: the restatement is f64-accumulating like the reference
    assert np.abs(out - z["expected"]).max() <= 2e-5


def test_embedder_cls_pooling_matches_hf():
    z, weights = load_bert_fixture("bert_hf_seeded.npz")
    out = O.bert_embedder(z["input_ids"], z["attention_mask"], z["token_type_ids"], z["tok"], z["pos"], z["typ"],
                          z["emb_gamma"], z["emb_beta"], weights, int(z["heads"]), float(z["eps"]), "cls")
    assert np.abs(out - z["expected_cls"]).max() <= 2e-5


def test_embedder_threads_match_serial():
    z, weights = load_bert_fixture("bert_hf_seeded.npz")
    args = (z["input_ids"], z["attention_mask"], z["token_type_ids"], z["tok"], z["pos"], z["typ"], z["emb_gamma"],
            z["emb_beta"], weights, int(z["heads"]), float(z["eps"]), "masked_mean")
    a = O.bert_embedder(*args, workers=1)
    b = O.bert_embedder(*args, workers=4)
    assert np.array_equal(a, b)


# ---- runtime/backend/tensor_ops_test.go -------------------------------------------------
def test_gather_known_answer():  # TestGatherTensorRank2WithRank2Indices shape family / TestGatherTensor values
    table = np.array([[1, 0], [0, 1], [1, 1]], np.float32)
    out = O.gather(table, np.array([[2, 0]], np.int32))
    assert np.array_equal(out[0], [[1, 1], [1, 0]])
    with pytest.raises(IndexError):
        O.gather(table, np.array([[3]], np.int32))


def test_matmul_known_answer():  # TestMatmulTensor, TestMatmulTensorAppliesScaleAttribute
    out = O.matmul(np.array([[1, 2], [3, 4]], np.float32), np.array([[5, 6], [7, 8]], np.float32))
    assert np.array_equal(out, [[19, 22], [43, 50]])
    out = O.matmul(np.array([[1, 2], [3, 4]], np.float32), np.array([[5, 6], [7, 8]], np.float32), scale=0.5)
    assert np.array_equal(out, [[9.5, 11], [21.5, 25]])


def test_normalize_rows_known_answer():  # TestNormalizeRows (+ zero row untouched)
    out = O.normalize_rows(np.array([[3, 4], [1, 0], [0, 0]], np.float32))
    np.testing.assert_allclose(out, [[0.6, 0.8], [1, 0], [0, 0]], atol=1e-6)


def test_mean_pool_masked_known_answer():  # TestMeanPoolMaskedTensorBatched
    x = np.array([[[1, 0], [0.70710677, 0.70710677]], [[0, 1], [1, 0]]], np.float32)
    out = O.mean_pool_masked(x, np.array([[1, 1], [1, 0]], np.int32))
    np.testing.assert_allclose(out, [[0.8535534, 0.35355338], [0, 1]], atol=1e-6)
    out = O.mean_pool_masked(x, np.array([[0, 0], [1, 1]], np.int32))
    assert np.array_equal(out[0], [0, 0])  # count 0 -> zeros, never NaN


def test_topk_tie_rule_known_answer():  # TestTopKTensor / TestTopKTensorRank2: ties -> lower index
    ids, sc = O.topk(np.array([0.25, 0.9, 0.5, 0.9], np.float32), 3)
    assert ids.tolist() == [1, 3, 2]
    assert sc.tolist() == [np.float32(0.9), np.float32(0.9), 0.5]
    ids, _ = O.topk(np.array([0.9, 0.1, 0.9], np.float32), 2)
    assert ids.tolist() == [0, 2]


# ---- runtime/backend/bert_embedding_ops_test.go ------------------------------------------
def test_bert_embeddings_known_answer():  # TestBERTEmbeddingReferenceRank2LayerNormAffine
    tok = np.array([[1, 2], [10, 20]], np.float32)
    pos = np.array([[0, 1], [1, 0]], np.float32)
    typ = np.array([[0, 0], [2, -2]], np.float32)
    out = O.bert_embeddings(tok, pos, typ, [2, 3], [0.5, -0.5], [[0, 1], [0, 1]], [[0, 1], [1, 0]], [[1, 0], [0, 1]],
                            eps=3)
    want = [1.5, -2, -9.0 / math.sqrt(23.25) + 0.5, 13.5 / math.sqrt(23.25) - 0.5,
            0.5, -0.5, -7.0 / math.sqrt(15.25) + 0.5, 10.5 / math.sqrt(15.25) - 0.5]
    np.testing.assert_allclose(out.ravel(), np.array(want, np.float32), atol=1e-6)
    with pytest.raises(IndexError):
        O.bert_embeddings(tok, pos, typ, [2, 3], [0.5, -0.5], [[2]], [[0]], [[0]])


# ---- runtime/backend/bert_encoder_layer_ops_test.go ---------------------------------------
def _layer_fixture():
    return dict(
        hs=np.array([[[2, -1], [1, 3]]], np.float32),
        w=[np.array(a, np.float32) for a in (
            [[2, -1], [0.5, 3]], [0.25, -0.5], [[1, 4], [-2, 0.5]], [-0.25, 0.75], [[1.5, -0.25], [0.75, 2]],
            [0.1, -0.2], [[0.5, -1.25], [1.5, 0.25]], [0.3, -0.4], [1.2, -0.7], [0.05, 0.15],
            [[0.25, -0.5], [1.25, 0.75], [-1.5, 0.5]], [0.1, -0.2, 0.3], [[0.4, -0.8, 1.2], [-1.1, 0.6, 0.2]],
            [-0.05, 0.25], [0.9, 1.4], [-0.2, 0.4])])


def _manual_layer(hs, mask, w, heads, eps):
    """Independent float64 numpy re-derivation (the role manualBERTEncoderLayer plays in the reference test)."""
    x = hs.astype(np.float64)[0]
    q, k, v = (x @ w[i].T.astype(np.float64) + w[i + 1] for i in (0, 2, 4))
    t, h = x.shape
    hd = h // heads
    ctx = np.zeros_like(x)
    keys = [j for j in range(t) if mask[0, j] != 0]
    for i in range(t):
        for hh in range(heads):
            if not keys:
                continue
            sl = slice(hh * hd, (hh + 1) * hd)
            lg = np.array([q[i, sl] @ k[j, sl] / math.sqrt(hd) for j in keys])
            p = np.exp(lg - lg.max())
            p /= p.sum()
            ctx[i, sl] = sum(pj * v[j, sl] for pj, j in zip(p, keys))

    def ln(a, g, b):
        mu = a.mean(-1, keepdims=True)
        var = ((a - mu) ** 2).mean(-1, keepdims=True)
        return (a - mu) / np.sqrt(var + eps) * g + b

    a = ln(ctx @ w[6].T.astype(np.float64) + w[7] + x, w[8], w[9])
    mid = a @ w[10].T.astype(np.float64) + w[11]
    mid = 0.5 * mid * (1 + np.vectorize(math.erf)(mid / math.sqrt(2)))
    return ln(mid @ w[12].T.astype(np.float64) + w[13] + a, w[14], w[15])[None]


@pytest.mark.parametrize("mask", [[[1, 0]], [[0, 0]], [[1, 1]]])
def test_bert_layer_tiny_deterministic(mask):
    # TestBERTEncoderLayerReferenceTinyDeterministic / ...MaskAllKeysProducesZeroContext (heads 1, eps 0.25)
    f = _layer_fixture()
    m = np.array(mask, np.int32)
    out = O.bert_layer(f["hs"], m, f["w"], heads=1, eps=0.25)
    assert np.isfinite(out).all()
    np.testing.assert_allclose(out, _manual_layer(f["hs"], m, f["w"], 1, 0.25), atol=1e-5)


def test_attention_parallel_matches_serial():  # TestBERTSelfAttentionContextParallelMatchesSerial
    rng = np.random.default_rng(7)
    q, k, v = (rng.standard_normal((3, 20, 16)).astype(np.float32) for _ in range(3))
    mask = (rng.random((3, 20)) > 0.3).astype(np.int32)
    mask[1] = 0
    a = O.bert_attention(q, k, v, mask, heads=4, workers=1)
    b = O.bert_attention(q, k, v, mask, heads=4, workers=5)
    assert np.array_equal(a, b)
    assert np.array_equal(a[1], np.zeros_like(a[1]))


# ---- quant grid and f16 conversion ---------------------------------------------------------
def test_quant_grid_rule():  # runtime/embedding_trainer.go:11413-11446
    data = np.array([0.5, -1.27, 0.005, 1.0, -0.015, 0.0], np.float32)
    codes, scales = O.quantize_symmetric(data)
    scale = np.float32(1.27) / np.float32(127)
    assert scales[0] == scale
    want = np.clip(np.sign(data) * np.floor(np.abs(data / scale).astype(np.float64) + 0.5), -127, 127)
    assert codes.tolist() == want.astype(np.int8).tolist()
    np.testing.assert_array_equal(O.dequantize(codes, scales), codes.astype(np.float32) * scale)
    codes, scales = O.quantize_symmetric(np.zeros(4, np.float32))
    assert codes.tolist() == [0, 0, 0, 0]
    w = np.array([[1.0, -0.5], [0.1, 0.2]], np.float32)
    codes, scales = O.quantize_symmetric(w, group=2)
    assert codes.tolist() == [[127, -64], [64, 127]]  # round half away: 63.5 -> 64


def test_f16_roundtrip_matches_numpy_off_ties():
    rng = np.random.default_rng(3)
    xs = np.concatenate([rng.standard_normal(2000).astype(np.float32) * s for s in (1e-6, 1e-3, 1.0, 300.0)])
    for x in xs[::7]:
        bits = O.f32_to_f16_bits(float(x))
        assert bits == int(np.float16(x).view(np.uint16)) or abs(O.f16_bits_to_f32(bits) - float(np.float16(x))) > 0
        assert O.f16_bits_to_f32(bits) == float(np.uint16(bits).view(np.float16))
    n_equal = sum(O.f32_to_f16_bits(float(x)) == int(np.float16(x).view(np.uint16)) for x in xs[::7])
    assert n_equal >= len(xs[::7]) - 2  # differs from IEEE only on exact ties (round half up)


def test_dense_rows_and_rerank_restatement():
    """dotRows / cosineRows (runtime/backend/tensor_ops.go:1967-2057) on hand-checked values, and the rerank loop's
    order (retrieval_turboquant.go:1610-1635: score descending, then id ascending; candidates without a vector skipped)."""
    from oracle import oracle as O
    docs = np.array([[1, 0, 0], [0, 2, 0], [3, 4, 0], [0, 0, 0], [1, 0, 0]], np.float32)
    q = np.array([3, 4, 0], np.float32)
    assert O.dot_rows(q, docs).tolist() == [3.0, 8.0, 25.0, 0.0, 3.0]
    cos = O.cosine_rows(q, docs)
    assert np.allclose(cos, [0.6, 0.8, 1.0, 0.0, 0.6], atol=1e-7) and cos[3] == 0.0   # zero row -> 0, not NaN
    ids, scores = O.rerank(q, docs, [4, 0, 3, -1, 9, 1], 3)
    assert ids.tolist() == [1, 0, 4] and scores.tolist() == [8.0, 3.0, 3.0]             # tie 0 / 4: smaller id first
    ids, _ = O.rerank(q, docs, [-1, 17], 3)
    assert ids.size == 0


def test_compact_path_rows_match_reference_expectations():
    """Expected values copied from runtime/backend/tensor_ops_test.go: TestLayerNormRows(:465-475),
    TestLayerNormRowsBatched (:477-491), TestRoPERows (:646-656), TestRoPERowsBatchedResetsPositionPerBatch (:658-672)."""
    from oracle import oracle as O
    ln = O.layernorm_rows(np.array([[2, 4], [6, 8]], np.float32))
    assert np.allclose(ln, [[-0.999995, 0.999995], [-0.999995, 0.999995]], atol=1e-6)
    ln3 = O.layernorm_rows(np.array([[[2, 4], [6, 8]], [[1, 3], [5, 7]]], np.float32))
    assert np.allclose(ln3, np.tile([-0.999995, 0.999995], (2, 2, 1)), atol=1e-6)
    r = O.rope_rows(np.array([[1, 0], [0, 1]], np.float32))
    assert np.allclose(r, [[1, 0], [-0.84147096, 0.5403023]], atol=1e-7)
    r3 = O.rope_rows(np.array([[[1, 0], [0, 1]], [[1, 0], [0, 1]]], np.float32))
    assert np.allclose(r3, np.tile([[1, 0], [-0.84147096, 0.5403023]], (2, 1, 1)), atol=1e-7)


# ---- TurboQuant: the restatement against the reference's own device code compiled for the host ---------------------
def _turboq_ref():
    """oracle/_ref/libturboq_ref.so: the reference's turboQKernelSource string
    (runtime/backends/cuda/native_linux.go:1812-2003) compiled as C++ by oracle/build_ref.py."""
    import ctypes as C
    from oracle import build_ref
    path = build_ref.build()
    if path is None:
        pytest.skip("neither the reference tree nor a prebuilt oracle/_ref is present")
    return C.CDLL(path)


@pytest.mark.parametrize("dim,bits,n", [(768, 4, 400), (128, 2, 300), (96, 4, 65), (384, 4, 33), (40, 8, 20)])
def test_tq_encode_decode_match_the_reference_device_code(dim, bits, n):
    """Codes of eos_oracle_tq_encode == codes of manta_turboq_encode, and the decoded vectors agree, for a caller
    supplied rotation spec (the seed -> spec generator of the third-party module stays unpinned).  dim 96 / 40:
    several Hadamard blocks (64 + 32, 32 + 8)."""
    import ctypes as C
    import eos_b200
    ref = _turboq_ref()
    spec = eos_b200.make_rotation_spec(dim, bits, seed=402)
    rng = np.random.default_rng(dim * 7 + bits)
    x = rng.standard_normal((n, dim)).astype(np.float32)
    x /= np.linalg.norm(x, axis=1, keepdims=True).astype(np.float32)
    x *= np.linspace(0.25, 4.0, n, dtype=np.float32)[:, None]
    x[n // 3] = 0   # zero vector: scale stays 1, codes of the all-zero rotation
    levels = 1 << bits

    def fp(a):
        return np.ascontiguousarray(a, np.float32).ctypes.data_as(C.c_void_p)

    coords = np.zeros((n, dim), np.float32)
    norm_codes = np.zeros(n, np.float32)
    permf = spec.perm.astype(np.float32)
    ref.ref_turboq_encode(fp(x), fp(coords), fp(norm_codes), fp(permf), fp(spec.signs1), fp(spec.signs2),
                          fp(spec.centroids), fp(spec.boundaries), C.c_int(n), C.c_int(dim), C.c_int(levels))
    codes, norms = O.tq_encode(x, bits, spec.perm, spec.signs1, spec.signs2, spec.boundaries)
    per_byte = 8 // bits
    idx = np.zeros((n, dim), np.int32)
    for c in range(dim):
        idx[:, c] = (codes[:, c // per_byte] >> ((c % per_byte) * bits)) & (levels - 1)
    assert np.array_equal(idx, coords.astype(np.int32))          # bit-exact code assignment
    # the reference stores the norm as an 8-bit log code; the restatement keeps the f32 norm (stated deviation):
    # the f32 norm must map to exactly the reference's code
    ref.ref_turboq_norm_code.restype = C.c_int
    ref.ref_turboq_norm_value.restype = C.c_float
    got_codes = np.array([ref.ref_turboq_norm_code(C.c_float(float(v))) for v in norms], np.float32)
    assert np.array_equal(got_codes, norm_codes)
    assert np.array_equal(O.tq_norm_code(norms), norm_codes.astype(np.uint8))
    # decode: same centroids -> signs2 -> FWHT -> signs1, times the norm the reference would use (its 8-bit one)
    out_ref = np.zeros((n, dim), np.float32)
    ref.ref_turboq_decode(fp(coords), fp(norm_codes), fp(out_ref), fp(permf), fp(spec.signs1), fp(spec.signs2),
                          fp(spec.centroids), C.c_int(n), C.c_int(dim), C.c_int(levels))
    norm8 = np.array([ref.ref_turboq_norm_value(C.c_int(int(c))) for c in norm_codes], np.float32)
    assert np.array_equal(O.tq_norm_value(norm_codes.astype(np.uint8)), norm8)
    out = O.tq_decode(codes, norm8, dim, bits, spec.perm, spec.signs1, spec.signs2, spec.centroids)
    assert np.array_equal(out.view(np.uint32), out_ref.view(np.uint32))   # bit-exact reconstruction


# ---- sparse attention: known answers of runtime/backend/tensor_ops_test.go:898-1001 --------------------------------
def test_sparse_attention_known_answers():
    # TestSparseAttentionReferenceSelectsTopKValues
    q = np.array([[1, 0], [0, 1]], np.float32)
    k = np.array([[1, 0], [0, 1], [-1, 0]], np.float32)
    v = np.array([[10, 0], [0, 20], [-10, 0]], np.float32)
    np.testing.assert_allclose(O.sparse_attention(q, k, v, top_k=1), [[10, 0], [0, 20]], atol=1e-6)
    # TestSparseAttentionReferenceRoutesThroughSelectedBlocks: anchors are keys 1, 3, 5 -> block 1 wins, key 2 in it
    q = np.array([[1, 0]], np.float32)
    k = np.array([[0, 10], [0, 0], [3, 0], [2, 0], [10, 0], [0, 0]], np.float32)
    v = np.array([[10], [20], [30], [40], [50], [60]], np.float32)
    np.testing.assert_allclose(O.sparse_attention(q, k, v, top_k=1, route_block_size=2, route_top_blocks=1), [[30]],
                               atol=1e-6)
    # budget / route normalisation (PlanSparseAttention, TestSparseAttentionPlanTracksRoutedBudget)
    assert O.sparse_attention_budget(0, 64) == 8 and O.sparse_attention_budget(4, 64) == 4
    assert O.sparse_attention_budget(100, 64) == 64 and O.sparse_attention_budget(0, 0) == 0
    assert O.sparse_attention_route(64, 8, 2) == (8, 2) and O.sparse_attention_route(64, 100, 5) == (64, 1)
    assert O.sparse_attention_route(64, 0, 2) == (0, 0)
    # softmax over the selected keys only: two equal best scores share the weight
    k2 = np.array([[1, 0], [1, 0], [0, 1]], np.float32)
    v2 = np.array([[2, 0], [4, 0], [100, 100]], np.float32)
    np.testing.assert_allclose(O.sparse_attention(np.array([[1, 0]], np.float32), k2, v2, top_k=2), [[3, 0]], atol=1e-6)
