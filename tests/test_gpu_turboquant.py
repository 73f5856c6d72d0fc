"""GPU parity of TurboQuant packing, scoring and exact top-k (C ABI: eos_b200_quantize, _corpus_bind,
_score_topk, _topk_merge_device, _parent_topk) against the CPU oracle.

Bars: packed codes and norms bit-exact; scores within 1e-3 relative (of the score scale); top-k ids identical
wherever score gaps exceed that tolerance, ties by ascending id (runtime/retrieval_eval.go:1153-1161)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    import eos_b200
    r = eos_b200.Runtime(0)
    yield r
    r.close()


def _unit_rows(n, dim, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n, dim)).astype(np.float32)
    return x / np.linalg.norm(x, axis=1, keepdims=True).astype(np.float32)


def _oracle_pack(x, spec):
    from oracle import oracle as O
    return O.tq_encode(x, spec.bits, spec.perm, spec.signs1, spec.signs2, spec.boundaries)


@pytest.mark.parametrize("dim,bits,n", [(768, 4, 1500), (128, 2, 700), (96, 4, 33), (384, 4, 16)])
def test_pack_bit_exact(rt, dim, bits, n):
    import eos_b200
    spec = eos_b200.make_rotation_spec(dim, bits, seed=402)
    x = _unit_rows(n, dim, 401) * np.linspace(0.5, 3.0, n, dtype=np.float32)[:, None]
    x[n // 2] = 0  # zero vector: norm 0, codes of the all-zero rotation
    qz = eos_b200.Quantizer(rt, spec)
    codes, norms = qz.quantize(x)
    ref_codes, ref_norms = _oracle_pack(x, spec)
    assert np.array_equal(norms.view(np.uint32), ref_norms.view(np.uint32))
    assert np.array_equal(codes, ref_codes)
    assert codes.shape[1] + 4 == spec.vector_bytes
    assert norms[n // 2] == 0
    qz.close()


def _setup(rt, dim, bits, n, nq, seed=1):
    import eos_b200
    spec = eos_b200.make_rotation_spec(dim, bits, seed=402)
    x = _unit_rows(n, dim, seed)
    q = _unit_rows(nq, dim, seed + 1).astype(np.float16).astype(np.float32)
    codes, norms = _oracle_pack(x, spec)
    qz = eos_b200.Quantizer(rt, spec)
    return spec, qz, codes, norms, q


def _oracle_scores(spec, codes, norms, q):
    from oracle import oracle as O
    out = np.empty((q.shape[0], codes.shape[0]), np.float32)
    for i in range(q.shape[0]):
        prep = O.tq_prepare_query(q[i], spec.perm, spec.signs1, spec.signs2)
        out[i] = O.tq_score(codes, norms, spec.dim, spec.bits, spec.centroids, prep)
    return out


def _check_topk(ids, scores, ref_scores, k, id_base, tol):
    """ids/scores: GPU result of one query; ref_scores: oracle scores of every row."""
    from oracle import oracle as O
    n = ref_scores.size
    kk = min(k, n)
    ref_ids, ref_top = O.topk(ref_scores, k, id_base)
    assert (ids[kk:] == -1).all()
    got = ids[:kk] - id_base
    assert len(set(got.tolist())) == kk and got.min() >= 0 and got.max() < n
    assert np.abs(scores[:kk] - ref_scores[got]).max() <= tol        # reported score = that row's score
    # per score, not only against the score scale: 1e-3 relative for every returned score near the scale (operands
    # are f16, so a score that is itself a hundredth of the scale cannot carry a 1e-3 relative bound)
    big = np.abs(ref_scores[got]) >= 500 * tol                       # >= half of the scale
    if big.any():
        assert (np.abs(scores[:kk] - ref_scores[got])[big] / np.abs(ref_scores[got])[big]).max() <= 1e-3
    assert np.abs(scores[:kk] - ref_top).max() <= tol                # rank-wise agreement with the oracle
    assert (np.diff(scores[:kk]) <= 0).all()                         # descending
    same = np.diff(scores[:kk]) == 0
    assert (np.diff(ids[:kk])[same] > 0).all()                       # ties: ascending id
    # membership is exact wherever the score gap to the cut-off exceeds the tolerance
    cut = ref_top[-1]
    must = set((np.nonzero(ref_scores > cut + 2 * tol)[0]).tolist())
    may = set((np.nonzero(ref_scores >= cut - 2 * tol)[0]).tolist())
    assert must <= set(got.tolist()) <= may
    # and the ordered ids are identical wherever neighbouring oracle scores are separated by more than tol
    sep = np.abs(np.diff(ref_top)) > 2 * tol
    clear = np.concatenate([[True], sep]) & np.concatenate([sep, [True]])
    clear &= np.abs(ref_top - cut) > 2 * tol
    assert np.array_equal(ids[:kk][clear], ref_ids[clear])


@pytest.mark.parametrize("dim,bits,n,nq,k,per_pass", [
    (768, 4, 5000, 11, 100, 8), (768, 4, 2051, 40, 100, 32), (128, 2, 3000, 16, 10, 16), (96, 4, 50, 3, 100, 8),
    (96, 4, 140000, 9, 100, 8),   # large enough for the thresholds to be seeded from a sample of the first rows
    # 128 queries per launch: the tensor-core batch kernel
    (768, 4, 5000, 11, 100, 128), (768, 4, 2051, 140, 100, 128), (128, 2, 3000, 16, 10, 128), (96, 4, 50, 3, 100, 128),
    (96, 4, 140000, 9, 100, 128),  # unseeded, several tiles per CTA: every list is cut
    (96, 4, 310000, 9, 100, 128),  # thresholds seeded from the first 148 x 256 rows
    # 256 queries per launch: documents as the MMA rows
    (768, 4, 5000, 11, 100, 256), (768, 4, 2051, 300, 100, 256), (128, 2, 3000, 16, 10, 256), (96, 4, 50, 3, 100, 256),
    (96, 4, 140000, 9, 100, 256), (96, 4, 310000, 9, 100, 256),
])
def test_scores_and_topk_match_oracle(rt, dim, bits, n, nq, k, per_pass):
    import eos_b200
    spec, qz, codes, norms, q = _setup(rt, dim, bits, n, nq)
    corpus = eos_b200.Corpus(qz, codes, norms, id_base=1000)
    ref = _oracle_scores(spec, codes, norms, q)
    scale = float(np.abs(ref).max())
    tol = 1e-3 * scale
    allsc = corpus.score_all(q)
    assert np.abs(allsc - ref).max() <= tol, float(np.abs(allsc - ref).max() / scale)
    ids, scores = corpus.score_topk(q, k, queries_per_pass=per_pass)
    for i in range(nq):
        _check_topk(ids[i], scores[i], ref[i], k, 1000, tol)
    assert corpus.vector_bytes == spec.vector_bytes
    corpus.close()
    qz.close()


@pytest.mark.parametrize("per_pass", [8, 128, 256])
def test_ties_resolve_to_lower_id(rt, per_pass):
    import eos_b200
    spec, qz, codes, norms, q = _setup(rt, 768, 4, 640, 4)
    codes = np.tile(codes[:64], (10, 1))   # every vector appears 10 times: exact score ties
    norms = np.tile(norms[:64], 10)
    corpus = eos_b200.Corpus(qz, codes, norms)
    ids, scores = corpus.score_topk(q, 100, queries_per_pass=per_pass)
    for i in range(4):
        groups = ids[i].reshape(10, 10)
        assert (np.diff(scores[i].reshape(10, 10), axis=1) == 0).all()
        assert (np.diff(groups, axis=1) == 64).all()        # the 10 copies, ascending id
        assert (groups[:, 0] < 64).all()
    corpus.close()
    qz.close()


def test_sharded_merge_equals_single_corpus(rt):
    import torch
    import eos_b200
    from eos_b200 import turboquant as tq
    spec, qz, codes, norms, q = _setup(rt, 768, 4, 6000, 24)
    whole = eos_b200.Corpus(qz, codes, norms)
    ref_ids, ref_scores = whole.score_topk(q, 100, queries_per_pass=8)
    bounds = [0, 1500, 1516, 6000]
    dq = torch.from_numpy(q).cuda()
    keys = torch.zeros((3, 24, 100), dtype=torch.int64, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    shards = []
    for s in range(3):
        lo, hi = bounds[s], bounds[s + 1]
        c = eos_b200.Corpus(qz, codes[lo:hi], norms[lo:hi], id_base=lo)
        shards.append(c)
        c.score_topk_device(dq.data_ptr(), 24, 100, 8, None, None, keys[s].data_ptr(), stream)
    out_ids = torch.empty((24, 100), dtype=torch.int64, device="cuda")
    out_sc = torch.empty((24, 100), dtype=torch.float32, device="cuda")
    tq.topk_merge_device(rt, keys.data_ptr(), 3, 24, 100, out_ids.data_ptr(), out_sc.data_ptr(), stream)
    torch.cuda.synchronize()
    assert np.array_equal(out_ids.cpu().numpy(), ref_ids)
    assert np.array_equal(out_sc.cpu().numpy(), ref_scores)
    for c in shards + [whole]:
        c.close()
    qz.close()


def test_device_quantize_and_synthetic_corpus_round_trip(rt):
    """Corpus generated and packed on the device (the path the 10M-vector benchmark uses): a slice copied back
    must pack to the same bytes on the CPU, and a planted near-duplicate of a query must come back first."""
    import torch
    import eos_b200
    from eos_b200 import turboquant as tq
    spec = eos_b200.make_rotation_spec(768, 4, seed=402)
    qz = eos_b200.Quantizer(rt, spec)
    n = 20000
    x = torch.empty((n, 768), dtype=torch.float32, device="cuda")
    codes = torch.empty((n, 384), dtype=torch.uint8, device="cuda")
    norms = torch.empty((n,), dtype=torch.float32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    tq.synth_gaussian_device(rt, 401, 0, n, 768, True, x.data_ptr(), stream)
    qz.quantize_device(x.data_ptr(), n, codes.data_ptr(), norms.data_ptr(), stream)
    torch.cuda.synchronize()
    xs = x[5000:5300].cpu().numpy()
    assert np.abs(np.linalg.norm(xs, axis=1) - 1).max() < 1e-5
    assert abs(float(xs.mean())) < 2e-3 and abs(float(xs.std()) - 768 ** -0.5) < 2e-3
    ref_codes, ref_norms = _oracle_pack(xs, spec)
    assert np.array_equal(codes[5000:5300].cpu().numpy(), ref_codes)
    assert np.array_equal(norms[5000:5300].cpu().numpy(), ref_norms)
    # rows are a function of (seed, row) only: regenerating a window reproduces it
    y = torch.empty((300, 768), dtype=torch.float32, device="cuda")
    tq.synth_gaussian_device(rt, 401, 5000, 300, 768, True, y.data_ptr(), stream)
    torch.cuda.synchronize()
    assert torch.equal(y, x[5000:5300])
    corpus = eos_b200.Corpus(qz, device_ptrs=(codes.data_ptr(), norms.data_ptr(), n), id_base=0)
    queries = x[[17, 9999, 19999]].cpu().numpy()
    ids, scores = corpus.score_topk(queries, 10)
    assert ids[:, 0].tolist() == [17, 9999, 19999]       # encode -> score round trip finds the source row
    assert (scores[:, 0] > 0.9).all() and (scores[:, 1] < 0.5).all()
    corpus.close()
    qz.close()


def test_parent_aggregation_matches_oracle(rt):
    import eos_b200
    from oracle import oracle as O
    spec, qz, codes, norms, q = _setup(rt, 128, 2, 4000, 8)
    rng = np.random.default_rng(3)
    parents = 300
    parent_of_child = rng.integers(0, parents - 5, size=4000).astype(np.int32)  # last 5 parents have no children
    corpus = eos_b200.Corpus(qz, codes, norms)
    ref = _oracle_scores(spec, codes, norms, q)
    gpu_all = corpus.score_all(q)
    for top_n, penalty in ((1, 0.0), (3, 0.0), (5, 0.01)):
        ids, scores = corpus.parent_topk(parent_of_child, parents, q, 20, 1, top_n, penalty)
        for i in range(8):
            # aggregation is exact given the child scores: check it on the GPU's own child scores
            rid, rsc = O.parent_topk(gpu_all[i], parent_of_child, parents, 20, top_n, penalty)
            assert np.array_equal(ids[i], rid)
            np.testing.assert_allclose(scores[i], rsc, rtol=0, atol=1e-6)
            # and against the oracle's child scores within the score tolerance
            _, osc = O.parent_topk(ref[i], parent_of_child, parents, 20, top_n, penalty)
            assert np.abs(scores[i] - osc).max() <= 1e-3 * float(np.abs(ref).max())
    # late-interaction sum over a group of query vectors (extension): equals the sum of the per-vector maxima
    ids, scores = corpus.parent_topk(parent_of_child, parents, q, 20, query_group=8)
    per = np.full((8, parents), 0.0, np.float64)
    for i in range(8):
        for p in range(parents - 5):
            per[i, p] = gpu_all[i][parent_of_child == p].max()
    tot = per.astype(np.float32).sum(0, dtype=np.float32)
    order = np.lexsort((np.arange(parents - 5), -tot[:parents - 5]))[:20]
    np.testing.assert_allclose(scores[0], tot[order], atol=1e-5)
    corpus.close()
    qz.close()


def test_argument_validation(rt):
    import eos_b200
    spec, qz, codes, norms, q = _setup(rt, 768, 4, 64, 2)
    bad = norms.copy()
    bad[3] = 0
    with pytest.raises(eos_b200.EosB200Error):   # norm <= 0 rejected unless confirmed (turboquant_quantized_vector.go:25-49)
        eos_b200.Corpus(qz, codes, bad)
    c = eos_b200.Corpus(qz, codes, bad, allow_zero_norm=True)
    ids, scores = c.score_topk(q, 5)
    assert np.isfinite(scores).all()
    with pytest.raises(eos_b200.EosB200Error):
        c.score_topk(q, 257)                      # the host call takes k up to 256
    with pytest.raises(eos_b200.EosB200Error):
        c.score_topk(q, 5, queries_per_pass=12)
    c.close()
    asym = eos_b200.make_rotation_spec(768, 4)
    asym.centroids = asym.centroids.copy()
    asym.centroids[0] *= 1.5
    with pytest.raises(eos_b200.EosB200Error):
        eos_b200.Quantizer(rt, asym)
    qz.close()


def test_batch_kernel_ascending_scores(rt):
    """Worst case for the candidate lists of the batch kernel: every vector is the same code row with a norm that
    grows with its index, so every document beats the running threshold and every list is cut before every tile.
    The result must still be the exact top-k (the last k rows for queries with a positive score)."""
    import eos_b200
    spec, qz, codes, norms, q = _setup(rt, 96, 4, 64, 5)
    n = 60000
    codes = np.tile(codes[:1], (n, 1))
    norms = np.linspace(0.5, 2.0, n, dtype=np.float32)
    corpus = eos_b200.Corpus(qz, codes, norms)
    ref = _oracle_scores(spec, codes[:1], np.ones(1, np.float32), q)[:, 0:1] * norms[None, :]
    ids8, sc8 = corpus.score_topk(q, 100, queries_per_pass=8)
    tol = 1e-3 * float(np.abs(ref).max())
    for per_pass in (128, 256):
        ids, sc = corpus.score_topk(q, 100, queries_per_pass=per_pass)
        for i in range(q.shape[0]):
            _check_topk(ids[i], sc[i], ref[i], 100, 0, tol)
            assert np.array_equal(ids[i], ids8[i])
    corpus.close()
    qz.close()


_TMEM_SCRIPT = r"""
import numpy as np, sys
sys.path.insert(0, "tests")
import eos_b200
import test_gpu_turboquant as T
rt = eos_b200.Runtime(0)
bad = 0
for dim, bits, n, nq, k in ((768, 4, 5000, 11, 100), (768, 4, 2051, 140, 100), (128, 2, 3000, 16, 10), (96, 4, 50, 3, 100),
                            (96, 4, 140000, 9, 100), (96, 4, 310000, 9, 100)):
    spec, qz, codes, norms, q = T._setup(rt, dim, bits, n, nq)
    corpus = eos_b200.Corpus(qz, codes, norms, id_base=1000)
    ref = T._oracle_scores(spec, codes, norms, q)
    tol = 1e-3 * float(np.abs(ref).max())
    ids, scores = corpus.score_topk(q, k, queries_per_pass=128)
    for i in range(nq):
        T._check_topk(ids[i], scores[i], ref[i], k, 1000, tol)
    corpus.close()
    qz.close()
print("TMEM_RESULT ok")
rt.close()
"""


def test_batch_kernel_with_queries_in_tensor_memory():
    """The opt-in variant of the batch kernel (EOS_B200_TQ_QUERIES_IN_TMEM=1: queries written once to tensor memory,
    tcgen05.mma with A from tensor memory, 128-document tiles) against the oracle.  Child process: the switch is read
    when a corpus first allocates its batch workspace."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, EOS_B200_TQ_QUERIES_IN_TMEM="1", PYTHONPATH=root)
    out = subprocess.run([sys.executable, "-c", _TMEM_SCRIPT], env=env, cwd=root, capture_output=True, text=True,
                         timeout=900)
    assert out.returncode == 0, out.stderr[-2000:]
    assert "TMEM_RESULT ok" in out.stdout


def test_automatic_queries_per_pass_and_argument_errors(rt):
    """queries_per_pass = 0 picks the kernel from the batch size; every choice returns the same exact top-k.
    Values outside {0, 8, 16, 32, 128, 256} are rejected, and the allocation-free entry takes the scan only."""
    import torch
    import eos_b200
    spec, qz, codes, norms, q = _setup(rt, 128, 4, 6000, 300)
    corpus = eos_b200.Corpus(qz, codes, norms)
    ref_ids, ref_sc = corpus.score_topk(q, 20, queries_per_pass=8)
    for nq in (5, 40, 300):
        ids, sc = corpus.score_topk(q[:nq], 20)            # 8, 128 and 256 queries per pass respectively
        scale = float(np.abs(ref_sc).max())
        assert np.abs(sc - ref_sc[:nq]).max() <= 1e-5 * scale          # same f16 operands, fp32 accumulation
        differ = ids != ref_ids[:nq]                                     # only exact-to-rounding ties may swap
        assert differ.mean() < 0.01
    with pytest.raises(Exception, match="queries_per_pass"):
        corpus.score_topk(q[:4], 20, queries_per_pass=64)
    dq = torch.from_numpy(q[:8]).cuda()
    d_ids = torch.empty((8, 20), dtype=torch.int64, device="cuda")
    d_sc = torch.empty((8, 20), dtype=torch.float32, device="cuda")
    with pytest.raises(Exception, match="queries_per_pass"):
        corpus.score_topk_noalloc(dq.data_ptr(), 8, 20, 128, d_ids.data_ptr(), d_sc.data_ptr())
    # ids and scores come together or not at all (a lone pointer would make the merge store through null)
    with pytest.raises(Exception, match="together"):
        corpus.score_topk_device(dq.data_ptr(), 8, 20, 8, d_ids.data_ptr(), None)
    with pytest.raises(Exception, match="no output"):
        corpus.score_topk_device(dq.data_ptr(), 8, 20, 8, None, None)
    keys = torch.zeros((8, 20), dtype=torch.int64, device="cuda")
    corpus.score_topk_device(dq.data_ptr(), 8, 20, 8, None, None, keys.data_ptr())   # keys only is fine
    corpus.sync()
    assert int((keys != 0).sum()) == 8 * 20
    corpus.close()
    qz.close()


@pytest.mark.parametrize("per_pass", [8, 128, 256])
@pytest.mark.parametrize("dim,n,nq,k", [(1024, 3000, 20, 128), (64, 2000, 7, 1), (768, 40000, 130, 128)])
def test_extreme_k_and_dims(rt, dim, n, nq, k, per_pass):
    """Largest and smallest k, the widest supported dimension (1024: 16 k-blocks, queries cannot stay in tensor
    memory) and a narrow one (64: half a code chunk is padding), for every scoring kernel."""
    import eos_b200
    spec, qz, codes, norms, q = _setup(rt, dim, 4, n, nq)
    corpus = eos_b200.Corpus(qz, codes, norms, id_base=7)
    ref = _oracle_scores(spec, codes, norms, q)
    tol = 1e-3 * float(np.abs(ref).max())
    ids, scores = corpus.score_topk(q, k, queries_per_pass=per_pass)
    for i in range(nq):
        _check_topk(ids[i], scores[i], ref[i], k, 7, tol)
    corpus.close()
    qz.close()


def test_thresholds_seeded_on_other_shards(rt):
    """Two shards of one corpus on one GPU, as two ranks would hold them: each seeds the thresholds of half of the
    queries from its own sample, the halves are concatenated (the all-gather), both shards score with all
    thresholds, and the merge of the two partial lists is the exact top-k of the whole corpus."""
    import torch
    import eos_b200
    from eos_b200 import turboquant as tq
    dim, n, nq, k = 96, 640000, 300, 100
    spec, qz, codes, norms, q = _setup(rt, dim, 4, n, nq)
    half = n // 2
    shards = [eos_b200.Corpus(qz, codes[:half], norms[:half], id_base=0),
              eos_b200.Corpus(qz, codes[half:], norms[half:], id_base=half)]
    whole = eos_b200.Corpus(qz, codes, norms)
    ref_ids, ref_sc = whole.score_topk(q, k, queries_per_pass=256)
    dq = torch.from_numpy(q).cuda()
    tau = torch.zeros((nq,), dtype=torch.int64, device="cuda")
    cut = 150
    keys = torch.zeros((2, nq, k), dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()                                # the library works on its own stream
    shards[0].score_seed_device(dq.data_ptr(), cut, k, tau.data_ptr())
    shards[1].score_seed_device(dq[cut:].data_ptr(), nq - cut, k, tau[cut:].data_ptr())
    torch.cuda.synchronize()
    assert int((tau != 0).sum()) == nq                      # both shards are large enough to seed
    for r in range(2):
        shards[r].score_topk_seeded_device(dq.data_ptr(), nq, k, tau.data_ptr(), None, None, keys[r].data_ptr())
    ids = torch.empty((nq, k), dtype=torch.int64, device="cuda")
    sc = torch.empty((nq, k), dtype=torch.float32, device="cuda")
    tq.topk_merge_device(rt, keys.data_ptr(), 2, nq, k, ids.data_ptr(), sc.data_ptr())
    torch.cuda.synchronize()
    assert np.array_equal(ids.cpu().numpy(), ref_ids)
    assert np.array_equal(sc.cpu().numpy(), ref_sc)
    for c in shards + [whole]:
        c.close()
    qz.close()


@pytest.mark.parametrize("per_pass", [8, 256])
def test_sharded_call_through_the_library_communicator(rt, per_pass):
    """eos_b200_score_topk_sharded on a one-rank communicator (NCCL inside the library, world = 1): the same exact
    top-k as the unsharded call.  Ranks > 1 run the same code; bench.py checks them against the streaming scan."""
    import torch
    import eos_b200
    from eos_b200 import dist as edist
    spec, qz, codes, norms, q = _setup(rt, 96, 4, 400000, 300)
    corpus = eos_b200.Corpus(qz, codes, norms, id_base=5)
    ref_ids, ref_sc = corpus.score_topk(q, 50, queries_per_pass=per_pass)
    comm = edist.Comm(rt, 0, 1, edist.new_comm_id())
    dq = torch.from_numpy(q).cuda()
    ids = torch.empty((300, 50), dtype=torch.int64, device="cuda")
    sc = torch.empty((300, 50), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    for _ in range(2):   # the second call reuses the communicator's buffers
        launches = corpus.score_topk_sharded(comm, dq.data_ptr(), 300, 50, per_pass, ids.data_ptr(), sc.data_ptr())
        corpus.sync()
        assert launches > 0
        assert np.array_equal(ids.cpu().numpy(), ref_ids)
        assert np.array_equal(sc.cpu().numpy(), ref_sc)
    comm.close()
    corpus.close()
    qz.close()


@pytest.mark.parametrize("children,group,parents,nq", [(128, 32, 60, 9), (16, 8, 500, 40), (64, 1, 100, 130), (32, 32, 37, 4)])
def test_maxsim_over_fixed_size_parents(rt, children, group, parents, nq):
    """Late interaction on the tensor-core batch kernel: for each query (group consecutive query vectors) and parent
    (children consecutive rows) the sum over the query's vectors of the best child score, exact top-k over parents.
    Checked against the aggregation of the GPU's own child scores (exact up to fp32 summation order) and against the
    oracle's child scores within the score tolerance; one parent has only missing children (NaN norms)."""
    import torch
    import eos_b200
    from oracle import oracle as O
    dim, bits, k = 128, 2, 20
    n = parents * children
    spec, qz, codes, norms, q = _setup(rt, dim, bits, n, nq * group, seed=11)
    norms = norms * np.linspace(0.5, 1.5, n, dtype=np.float32)
    norms[3 * children:4 * children] = np.nan             # parent 3 has no children
    norms[5 * children + 1:6 * children] = np.nan          # parent 5 has one child
    d_codes = torch.from_numpy(codes).cuda()
    d_norms = torch.from_numpy(norms).cuda()
    id_base = 7 * children
    corpus = eos_b200.Corpus(qz, device_ptrs=(d_codes.data_ptr(), d_norms.data_ptr(), n), id_base=id_base)
    dq = torch.from_numpy(q).cuda()
    kk = min(k, parents - 1)
    ids = torch.empty((nq, kk), dtype=torch.int64, device="cuda")
    sc = torch.empty((nq, kk), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    corpus.maxsim_topk_device(dq.data_ptr(), nq * group, group, children, kk, ids.data_ptr(), sc.data_ptr())
    corpus.sync()
    ids, sc = ids.cpu().numpy(), sc.cpu().numpy()
    finite = np.where(np.isnan(norms), 1.0, norms).astype(np.float32)
    ref_child = _oracle_scores(spec, codes, finite, q)                      # [nq * group, n]
    ref_child[:, np.isnan(norms)] = -np.inf
    best = ref_child.reshape(nq, group, parents, children).max(axis=3)      # [nq, group, parents]
    total = best.sum(axis=1, dtype=np.float64)                              # [nq, parents]
    tol = 1e-3 * float(np.abs(total[np.isfinite(total)]).max())
    for i in range(nq):
        t = total[i].copy()
        t[~np.isfinite(t)] = -np.inf
        order = np.lexsort((np.arange(parents), -t))[:kk]
        assert (sc[i][:-1] >= sc[i][1:]).all()
        got = ids[i] - 7
        assert got.min() >= 0 and got.max() < parents and len(set(got.tolist())) == kk and 3 not in got.tolist()
        assert np.abs(sc[i] - t[got]).max() <= tol
        sep = np.abs(np.diff(t[order])) > 2 * tol
        clear = np.concatenate([[True], sep]) & np.concatenate([sep, [True]])
        clear &= np.abs(t[order] - t[order][-1]) > 2 * tol
        assert np.array_equal(got[clear], order[clear])
    corpus.close()
    qz.close()


def test_maxsim_argument_errors(rt):
    import torch
    import eos_b200
    spec, qz, codes, norms, q = _setup(rt, 128, 2, 640, 64)
    corpus = eos_b200.Corpus(qz, codes, norms)
    dq = torch.from_numpy(q).cuda()
    ids = torch.empty((2, 5), dtype=torch.int64, device="cuda")
    sc = torch.empty((2, 5), dtype=torch.float32, device="cuda")
    for args, msg in (((64, 32, 48, 5), "children_per_parent"), ((64, 24, 64, 5), "query_group"),
                      ((60, 32, 64, 5), "multiple of query_group"), ((64, 32, 128, 200), "k must")):
        with pytest.raises(Exception, match=msg):
            corpus.maxsim_topk_device(dq.data_ptr(), args[0], args[1], args[2], args[3], ids.data_ptr(), sc.data_ptr())
    corpus.close()
    qz.close()


def _ip_quantise(x, spec3, proj_seed):
    """Test-side producer of IPQuantized fields by the published two-stage scheme: MSE stage (spec3), then the signs
    of a seeded Gaussian projection of the residual in the rotated space and the residual's norm."""
    from oracle import oracle as O
    dim = x.shape[1]
    norms = np.linalg.norm(x, axis=1).astype(np.float32)
    unit = (x / np.maximum(norms, 1e-30)[:, None]).astype(np.float32)
    rot = np.stack([O.tq_rotate(u, spec3.perm, spec3.signs1, spec3.signs2) for u in unit])
    idx = np.searchsorted(spec3.boundaries, rot).astype(np.uint8)
    resid = rot - spec3.centroids[idx]
    proj = np.random.default_rng(proj_seed).standard_normal((dim, dim)).astype(np.float32)
    signs = np.packbits((resid @ proj.T) >= 0, axis=1, bitorder="little")
    return idx, signs, np.linalg.norm(resid, axis=1).astype(np.float32), norms, proj


@pytest.mark.parametrize("dim,levels,n,nq,k", [(768, 8, 3000, 11, 100), (128, 4, 5000, 5, 200), (96, 2, 700, 3, 256)])
def test_ip_quantised_rows(rt, dim, levels, n, nq, k):
    """Rows carrying MSE codes + QJL signs + ResNorm + Norm: GPU scores and top-k vs the oracle's restatement of the
    two-stage estimator.  392 bytes per vector at dim 768, bit width 4, as the reference accounts them."""
    import math
    import eos_b200
    from eos_b200.turboquant import IpCorpus, RotationSpec, lloyd_max_gaussian
    from oracle import oracle as O
    base = eos_b200.make_rotation_spec(dim, 2, seed=402)
    cent, bound = lloyd_max_gaussian(levels, 1.0 / math.sqrt(dim))
    spec = RotationSpec(dim, int(math.log2(levels)), base.perm, base.signs1, base.signs2, cent, bound)
    rng = np.random.default_rng(5)
    x = _unit_rows(n, dim, 31) * rng.uniform(0.5, 2.0, (n, 1)).astype(np.float32)
    q = _unit_rows(nq, dim, 32).astype(np.float16).astype(np.float32)
    idx, signs, resn, norms, proj = _ip_quantise(x, spec, 77)
    prepared = np.stack([O.tq_prepare_query(qi, spec.perm, spec.signs1, spec.signs2) for qi in q])
    sketch = (prepared @ proj.T).astype(np.float32)
    qjl = math.sqrt(math.pi / 2.0) / dim
    ref = np.stack([O.tq_ip_score(idx, signs, resn, norms, cent, prepared[i], sketch[i], qjl) for i in range(nq)])
    assert IpCorpus.vector_bytes(768, 4) == 392
    corpus = IpCorpus(rt, dim, spec.perm, spec.signs1, spec.signs2, cent, idx, signs, resn, norms, id_base=1000)
    ids, scores = corpus.score_topk(q, sketch, qjl, k)
    tol = 1e-3 * float(np.abs(ref).max())
    for i in range(nq):
        _check_topk(ids[i], scores[i], ref[i], k, 1000, tol)
    # what the sign stage buys is an unbiased estimate: the MSE stage alone shrinks inner products (slope < 1 against
    # the true values), the two-stage estimate does not
    true = q @ x.T
    mse_only = np.stack([O.tq_ip_score(idx, signs, resn * 0, norms, cent, prepared[i], sketch[i], qjl) for i in range(nq)])
    slope_ip = float((ref * true).sum() / (true * true).sum())
    slope_mse = float((mse_only * true).sum() / (true * true).sum())
    assert abs(slope_ip - 1.0) < 0.1 and abs(slope_ip - 1.0) <= abs(slope_mse - 1.0) + 0.02, (slope_ip, slope_mse)
    with pytest.raises(RuntimeError, match="256"):
        corpus.score_topk(q, sketch, qjl, 257)
    corpus.close()
    bad = idx.copy()
    bad[0, 0] = levels
    with pytest.raises(RuntimeError, match="out of range"):
        IpCorpus(rt, dim, spec.perm, spec.signs1, spec.signs2, cent, bad, signs, resn, norms)


def test_wide_k_overfetch(rt):
    """k = 200 (the over-fetch before a rerank to 100, runtime/retrieval_turboquant.go:1610-1662) through the host
    call, against the oracle's scores; the first 100 of it equal the fused kernels' top-100."""
    spec, qz, codes, norms, q = _setup(rt, 768, 4, 9000, 19, seed=61)
    import eos_b200
    corpus = eos_b200.Corpus(qz, codes, norms, id_base=5)
    ref = _oracle_scores(spec, codes, norms, q)
    tol = 1e-3 * float(np.abs(ref).max())
    ids, scores = corpus.score_topk(q, 200)
    for i in range(q.shape[0]):
        _check_topk(ids[i], scores[i], ref[i], 200, 5, tol)
    ids100, _ = corpus.score_topk(q, 100)
    # two kernels, two summation orders: rows whose scores differ in the last bits may swap places
    assert np.mean([len(set(ids[i, :100]) & set(ids100[i])) for i in range(q.shape[0])]) >= 99.0
    ids256, scores256 = corpus.score_topk(q[:3], 256)
    for i in range(3):
        _check_topk(ids256[i], scores256[i], ref[i], 256, 5, tol)
    with pytest.raises(RuntimeError):
        corpus.score_topk(q, 257)
    corpus.close()
    qz.close()


def test_wide_k_single_pass_and_fallback(rt):
    """k in (128, 256] on a corpus large enough for seeded thresholds: one pass of the 256-query batch kernel answers
    every query whose candidate lists were never cut (random data: all of them, `reserved` = 0 fallbacks); on data
    built to cut every list (scores ascending with the row index) every query falls back to the all-scores path and
    the answer is the same exact top-k."""
    import eos_b200
    spec, qz, codes, norms, q = _setup(rt, 96, 4, 320000, 7, seed=71)
    corpus = eos_b200.Corpus(qz, codes, norms, id_base=11)
    ref = _oracle_scores(spec, codes, norms, q)
    tol = 1e-3 * float(np.abs(ref).max())
    for k in (200, 256, 129):
        ids, scores = corpus.score_topk(q, k)
        assert corpus.last_stats.reserved == 0, corpus.last_stats.reserved
        for i in range(q.shape[0]):
            _check_topk(ids[i], scores[i], ref[i], k, 11, tol)
    corpus.close()
    n = 320000
    codes1 = np.tile(codes[:1], (n, 1))
    norms1 = np.linspace(0.5, 2.0, n, dtype=np.float32)
    corpus = eos_b200.Corpus(qz, codes1, norms1)
    ref = _oracle_scores(spec, codes1[:1], np.ones(1, np.float32), q)[:, 0:1] * norms1[None, :]
    tol = 1e-3 * float(np.abs(ref).max())
    ids, scores = corpus.score_topk(q, 200)
    assert corpus.last_stats.reserved > 0
    for i in range(q.shape[0]):
        _check_topk(ids[i], scores[i], ref[i], 200, 0, tol)
    corpus.close()
    qz.close()
