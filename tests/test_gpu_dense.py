"""GPU parity of the dense candidate operators (C ABI: eos_b200_dense_*) against the oracle's restatement of
dotRows / cosineRows + topKTensor (runtime/backend/tensor_ops.go:1967-2057, 2124-2193) and of the rerank loops
topDenseRerankScores / topFP16RerankScores (runtime/retrieval_turboquant.go:1610-1662)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    import eos_b200
    r = eos_b200.Runtime(0)
    yield r
    r.close()


def _check_ranked(ids, scores, ref_scores, k, tol):
    """ids/scores: one query's result; ref_scores: oracle score of every row."""
    from oracle import oracle as O
    ref_ids, ref_top = O.topk(ref_scores, k)
    assert np.abs(scores - ref_scores[ids]).max() <= tol
    assert np.abs(scores - ref_top).max() <= tol
    assert (np.diff(scores) <= 0).all()
    same = np.diff(scores) == 0
    assert (np.diff(ids)[same] > 0).all()
    sep = np.abs(np.diff(ref_top)) > 2 * tol
    clear = np.concatenate([[True], sep]) & np.concatenate([sep, [True]])
    cut = ref_top[-1]
    clear &= np.abs(ref_top - cut) > 2 * tol
    assert np.array_equal(ids[clear], ref_ids[clear])


@pytest.mark.parametrize("n,dim,nq,k", [(3000, 768, 5, 100), (257, 96, 9, 10), (40, 1000, 3, 40)])
@pytest.mark.parametrize("metric", [0, 1])
def test_dense_score_topk(rt, n, dim, nq, k, metric):
    import eos_b200
    from oracle import oracle as O
    rng = np.random.default_rng(n + dim + metric)
    docs = rng.standard_normal((n, dim)).astype(np.float32)
    docs[n // 2] = 0.0  # a zero row: cosine must give 0, not NaN
    docs[7] = docs[3]   # duplicate rows: equal scores, the smaller row wins
    q = rng.standard_normal((nq, dim)).astype(np.float32)
    ix = eos_b200.DenseIndex(rt, docs)
    ids, scores = ix.score_topk(q, k, metric)
    assert np.isfinite(scores).all()
    for i in range(nq):
        ref = O.cosine_rows(q[i], docs) if metric == 1 else O.dot_rows(q[i], docs)
        tol = 2e-5 * max(1.0, float(np.abs(ref).max()))
        _check_ranked(ids[i], scores[i], ref, k, tol)
    ix.close()


@pytest.mark.parametrize("store_f16", [False, True])
def test_dense_rerank_matches_oracle(rt, store_f16):
    import eos_b200
    from oracle import oracle as O
    rng = np.random.default_rng(5 + store_f16)
    n, dim, nq, cand, k = 5000, 768, 7, 200, 100
    docs = rng.standard_normal((n, dim)).astype(np.float32)
    docs /= np.linalg.norm(docs, axis=1, keepdims=True)
    q = rng.standard_normal((nq, dim)).astype(np.float32)
    candidates = np.stack([rng.choice(n, size=cand, replace=False) for _ in range(nq)]).astype(np.int64)
    candidates[0, 5] = -1          # a candidate without a vector is skipped
    candidates[1, :150] = -1       # fewer valid candidates than k: the tail of the result is empty
    candidates[2, 9] = n + 3       # out of range counts as absent
    ix = eos_b200.DenseIndex(rt, docs, store_f16=store_f16)
    ids, scores = ix.rerank(q, candidates, k)
    stored = docs.astype(np.float16).astype(np.float32) if store_f16 else docs
    for i in range(nq):
        ref_ids, ref_scores = O.rerank(q[i], stored, candidates[i], k)
        m = len(ref_ids)
        assert (ids[i, m:] == -1).all() and np.isneginf(scores[i, m:]).all()
        tol = 2e-5 * float(np.abs(ref_scores).max())
        assert np.abs(scores[i, :m] - ref_scores).max() <= tol
        sep = np.abs(np.diff(ref_scores)) > 2 * tol
        clear = np.concatenate([[True], sep]) & np.concatenate([sep, [True]])
        assert np.array_equal(ids[i, :m][clear], ref_ids[clear])
        assert set(ids[i, :m].tolist()) <= set(candidates[i].tolist())
    ix.close()


def test_rerank_after_turboquant_topk_recovers_exact_order(rt):
    """The pipeline the reference runs (retrieval_turboquant.go:1306-1331 + :1610-1635): over-fetch 200 candidates with
    the 4-bit scores, rerank them with the dense vectors, keep 100; the result must equal the exact dense top-100
    wherever the exact top-100 lies inside the candidate set."""
    import eos_b200
    from oracle import oracle as O
    rng = np.random.default_rng(77)
    n, dim, nq = 20000, 768, 4
    docs = rng.standard_normal((n, dim)).astype(np.float32)
    docs /= np.linalg.norm(docs, axis=1, keepdims=True)
    q = docs[rng.choice(n, nq)] + 0.5 * rng.standard_normal((nq, dim)).astype(np.float32) / np.sqrt(dim)
    spec = eos_b200.make_rotation_spec(dim, 4, seed=402)
    qz = eos_b200.Quantizer(rt, spec)
    codes, norms = qz.quantize(docs)
    corpus = eos_b200.Corpus(qz, codes, norms)
    cand_ids, _ = corpus.score_topk(q, 128)
    ix = eos_b200.DenseIndex(rt, docs)
    ids, scores = ix.rerank(q, cand_ids, 100)
    for i in range(nq):
        exact = O.dot_rows(q[i], docs)
        ref_ids, ref_scores = O.rerank(q[i], docs, cand_ids[i], 100)
        assert np.array_equal(ids[i], ref_ids) or np.abs(scores[i] - ref_scores).max() <= 2e-5
        best = int(np.argmax(exact))
        assert ids[i, 0] == best
    ix.close()
    corpus.close()
    qz.close()


def test_dense_argument_errors(rt):
    import eos_b200
    docs = np.ones((10, 16), np.float32)
    ix = eos_b200.DenseIndex(rt, docs)
    with pytest.raises(eos_b200.EosB200Error):
        ix.score_topk(np.ones((1, 16), np.float32), 11)          # k > rows
    with pytest.raises(eos_b200.EosB200Error):
        ix.score_topk(np.ones((1, 16), np.float32), 5, metric=7)  # unknown metric
    with pytest.raises(eos_b200.EosB200Error):
        eos_b200.DenseIndex(rt, np.ones((4, 2000), np.float32))   # dim > 1024
    ix.close()
