"""GPU parity at the shapes the benchmark configurations run (C ABI against the CPU oracle).

Encoder: the 12-layer D=768 / 12 heads / FFN 3072 / 768->768 head model at T=512 with sequence lengths from 64
to 512 (3-4 key tiles and up to 4 query tiles per head, K=3072 with real activations), and the 4-layer D=384
model at T=256; bars of runtime/pretrained_bert_golden_parity_test.go:99-103 (max-abs <= 2e-3 after L2,
cosine >= 0.9999).  Attention alone: sequences far above 512 tokens and local windows, on the tensor-memory kernel.
TurboQuant: a shard large enough (>= 64 x 148 x 256 rows) for the batch kernel's second threshold sample, generated
and packed on the device; the 256-query kernel against the 8-query scan on every query and against the oracle on a
1 M-row slice."""
import numpy as np
import pytest

from tests.helpers import cosine_rows

pytestmark = pytest.mark.gpu

MAX_ABS = 2e-3
MIN_COS = 0.9999


@pytest.fixture(scope="module")
def rt():
    import eos_b200
    r = eos_b200.Runtime(0)
    yield r
    r.close()


def _oracle_embed(args, ids, mask, heads, window=0):
    from eos_b200 import synth
    from oracle import oracle as O
    return O.bert_embedder(ids, mask, np.zeros_like(ids), args["token_embeddings"], args["position_embeddings"],
                           args["token_type_embeddings"], args["embedding_ln_weight"], args["embedding_ln_bias"],
                           synth.dequantized_layer_weights(args["layer_weights"]), heads, 1e-12, "masked_mean",
                           head_w=args.get("head_weights"), window=window, workers=O.default_workers())


def _check(out, ref):
    assert np.isfinite(out).all()
    err = float(np.abs(out - ref).max())
    assert err <= MAX_ABS, err
    assert cosine_rows(out, ref).min() >= MIN_COS
    return err


def test_c3_shape_both_weight_modes(rt):
    """Configuration 3's model (BERT-base shape, int8 per-channel weights) on 6 sequences whose lengths span
    64 .. 512 at T = 512, f16-resident and dequantise-in-shared-memory weights."""
    import eos_b200
    from eos_b200 import synth
    args = synth.make_q8_encoder(12, 768, 12, 3072, vocab=30522, max_pos=512, seed=3, head_out=768)
    rng = np.random.default_rng(33)
    lengths = np.array([64, 129, 255, 300, 448, 512])
    ids = rng.integers(0, 30522, size=(6, 512), dtype=np.int32)
    mask = (np.arange(512)[None, :] < lengths[:, None]).astype(np.int32)
    ref = _oracle_embed(args, ids, mask, 12)
    outs = []
    for mode in (0, 1):
        enc = eos_b200.BertEmbedder(rt, weight_mode=mode, **args)
        out = enc.run(ids, mask)
        _check(out, ref)
        outs.append(out)
        enc.close()
    assert np.array_equal(outs[0], outs[1])   # same arithmetic in both weight modes


def test_c2_shape(rt):
    """Configuration 2's model (4 layers, D = 384, 6 heads, FFN 1536) at T = 256 on 40 sequences of 32 .. 256 tokens."""
    import eos_b200
    from eos_b200 import synth
    args = synth.make_q8_encoder(4, 384, 6, 1536, vocab=30522, max_pos=512, seed=2)
    ids, mask, _ = synth.make_batch(40, 256, 30522, 32, 256, seed=22)
    enc = eos_b200.BertEmbedder(rt, **args)
    out = enc.run(ids, mask)
    _check(out, _oracle_embed(args, ids, mask, 6))
    enc.close()


def _peaked_encoder(hidden, heads, max_pos, seed, layers=1):
    """Weights large enough for attention to be far from uniform (a wrong mask, window or running maximum shows
    up well above the tolerance); dense fp32 weights."""
    rng = np.random.default_rng(seed)
    inter = 2 * hidden

    def mat(o, i, std=0.12):
        return (rng.standard_normal((o, i)) * std).astype(np.float32)

    def vec(n, base=0.0):
        return (base + rng.standard_normal(n) * 0.05).astype(np.float32)

    lw = []
    for _ in range(layers):
        lw += [mat(hidden, hidden), vec(hidden), mat(hidden, hidden), vec(hidden), mat(hidden, hidden), vec(hidden),
               mat(hidden, hidden), vec(hidden), vec(hidden, 1.0), vec(hidden), mat(inter, hidden), vec(inter),
               mat(hidden, inter), vec(hidden), vec(hidden, 1.0), vec(hidden)]
    return dict(token_embeddings=mat(100, hidden, 0.5), position_embeddings=mat(max_pos, hidden, 0.5),
                token_type_embeddings=mat(2, hidden, 0.5), embedding_ln_weight=vec(hidden, 1.0),
                embedding_ln_bias=vec(hidden), layer_weights=lw, num_attention_heads=heads)


@pytest.mark.parametrize("window", [0, 512, 130])
def test_long_sequences_and_windows_on_the_tensor_core_kernel(rt, window):
    """head_dim 64, T = 2304: 18 key tiles without a window (the running maximum moves many times with these
    weights), 5 / 3 key tiles per query tile with one, edge tiles masked per element; one sequence has holes in
    its mask (positions differ from packed row indices) and one ends inside a tile."""
    import eos_b200
    T = 2304
    args = _peaked_encoder(128, 2, T, seed=77)
    rng = np.random.default_rng(78)
    ids = rng.integers(0, 100, size=(4, T), dtype=np.int32)
    lengths = np.array([T, 1500, 700, 1])
    mask = (np.arange(T)[None, :] < lengths[:, None]).astype(np.int32)
    mask[1, 300:900:3] = 0
    enc = eos_b200.BertEmbedder(rt, attention_window=window, **args)
    out = enc.run(ids, mask)
    _check(out, _oracle_embed(args, ids, mask, 2, window=window))
    enc.close()


def test_bounded_wait_reports_a_status_not_a_result(rt):
    """A wait inside a kernel that runs out must surface as the device-status error (return code 2), and the
    runtime must stay usable.  The wait here is the library's own self-test: one warp waits about half a
    millisecond on a barrier that nothing completes."""
    import eos_b200
    with pytest.raises(eos_b200.EosB200DeviceStatusError, match="timeout"):
        rt.selftest_bounded_wait(1_000_000)
    assert rt.info()["sm_count"] > 0
    spec = eos_b200.make_rotation_spec(96, 4, seed=402)
    qz = eos_b200.Quantizer(rt, spec)
    x = np.random.default_rng(0).standard_normal((64, 96)).astype(np.float32)
    codes, norms = qz.quantize(x)
    c = eos_b200.Corpus(qz, codes, norms)
    ids, _ = c.score_topk(x[:3], 5)          # the status word was cleared when it was reported
    assert ids[:, 0].tolist() == [0, 1, 2]
    c.close()
    qz.close()


def test_c4_path_large_shard(rt):
    """2.6 M x 768 4-bit rows generated and packed on the device (above 64 x 148 x 256 rows: the batch kernel takes
    its second threshold sample), 300 queries, top-100."""
    import torch
    import eos_b200
    from eos_b200 import turboquant as tq
    from oracle import oracle as O
    dim, n, nq, k = 768, 2_600_000, 300, 100
    spec = eos_b200.make_rotation_spec(dim, 4, seed=402)
    qz = eos_b200.Quantizer(rt, spec)
    codes = torch.empty((n, dim // 2), dtype=torch.uint8, device="cuda")
    norms = torch.empty((n,), dtype=torch.float32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    chunk = 400_000
    x = torch.empty((chunk, dim), dtype=torch.float32, device="cuda")
    for r0 in range(0, n, chunk):
        m = min(chunk, n - r0)
        tq.synth_gaussian_device(rt, 401, r0, m, dim, True, x.data_ptr(), stream)
        qz.quantize_device(x.data_ptr(), m, codes[r0:].data_ptr(), norms[r0:].data_ptr(), stream)
    torch.cuda.synchronize()
    del x
    corpus = eos_b200.Corpus(qz, device_ptrs=(codes.data_ptr(), norms.data_ptr(), n), id_base=0)
    q = torch.empty((nq, dim), dtype=torch.float32, device="cuda")
    tq.synth_gaussian_device(rt, 977, 0, nq, dim, True, q.data_ptr(), stream)
    torch.cuda.synchronize()
    qh = q.cpu().numpy().astype(np.float16).astype(np.float32)
    ids_b, sc_b = corpus.score_topk(qh, k, queries_per_pass=256)
    ids_s, sc_s = corpus.score_topk(qh, k, queries_per_pass=8)
    scale = float(np.abs(sc_s).max())
    assert np.abs(sc_b - sc_s).max() <= 1e-5 * scale            # same f16 operands, fp32 accumulation
    assert (ids_b != ids_s).mean() < 0.002                      # only exact-to-rounding ties may swap
    assert (np.diff(sc_b, axis=1) <= 0).all() and (ids_b >= 0).all() and (ids_b < n).all()
    # oracle on the first 1 M rows for 4 queries: the GPU's top-k restricted to those rows must be the oracle's
    m = 1_000_000
    h_codes = codes[:m].cpu().numpy()
    h_norms = norms[:m].cpu().numpy()
    sub = eos_b200.Corpus(qz, device_ptrs=(codes.data_ptr(), norms.data_ptr(), m), id_base=0)
    ids_m, sc_m = sub.score_topk(qh[:4], k, queries_per_pass=256)
    worst_rel = 0.0
    for i in range(4):
        prep = O.tq_prepare_query(qh[i], spec.perm, spec.signs1, spec.signs2)
        ref = O.tq_score(h_codes, h_norms, dim, 4, spec.centroids, prep)
        rid, rsc = O.topk(ref, k, 0)
        tol = 1e-3 * float(np.abs(ref).max())
        assert np.abs(sc_m[i] - ref[ids_m[i]]).max() <= tol
        worst_rel = max(worst_rel, float((np.abs(sc_m[i] - ref[ids_m[i]]) / np.abs(ref[ids_m[i]])).max()))
        sep = np.abs(np.diff(rsc)) > 2 * tol
        clear = np.concatenate([[True], sep]) & np.concatenate([sep, [True]])
        assert np.array_equal(ids_m[i][clear], rid[clear])
        assert set(ids_m[i].tolist()) >= set(np.nonzero(ref > rsc[-1] + 2 * tol)[0].tolist())
    assert worst_rel <= 1e-3, worst_rel                          # per-score relative error of the returned scores
    sub.close()
    corpus.close()
    qz.close()


@pytest.mark.parametrize("T,layers,lengths", [(1536, 2, (1536, 700, 130)), (8192, 6, (8192, 3000, 257))])
def test_per_token_vectors_long_context(rt, T, layers, lengths):
    """The document side of the long-context multi-vector configuration: D = 512, 8 heads, FFN 2048, a 512-token
    window, a 512 -> 128 per-token head; at reduced depth and length, and at the configuration's own 6 layers and
    T = 8192 (64 key tiles per sequence, 5 of them per query tile under the window).  The GPU's per-token vectors
    against the oracle's, and their 2-bit packing bit-exact against the oracle's packing of the GPU vectors."""
    import torch
    import eos_b200
    from eos_b200 import synth
    from oracle import oracle as O
    D, heads, window, tdim = 512, 8, 512, 128
    args = synth.make_q8_encoder(layers, D, heads, 2048, vocab=2000, max_pos=T, seed=55)
    rng = np.random.default_rng(56)
    tw = synth.f16_round(rng.standard_normal((D, tdim), dtype=np.float32) * np.float32(0.05))
    lengths = np.array(lengths)
    B = len(lengths)
    ids = rng.integers(0, 2000, size=(B, T), dtype=np.int32)
    mask = (np.arange(T)[None, :] < lengths[:, None]).astype(np.int32)
    enc = eos_b200.BertEmbedder(rt, attention_window=window, **args)
    enc.set_token_head(tw)
    d_ids, d_mask = torch.from_numpy(ids).cuda(), torch.from_numpy(mask).cuda()
    rows = int(mask.sum())
    d_vec = torch.zeros((B * T, tdim), dtype=torch.float32, device="cuda")
    d_rows = torch.zeros((1,), dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    enc.token_vectors_device(d_ids.data_ptr(), d_mask.data_ptr(), None, B, T, d_vec.data_ptr(), d_rows.data_ptr())
    enc.sync()
    assert int(d_rows.item()) == rows
    got = d_vec[:rows].cpu().numpy()
    ref = O.bert_token_vectors(ids, mask, np.zeros_like(ids), args["token_embeddings"], args["position_embeddings"],
                               args["token_type_embeddings"], args["embedding_ln_weight"], args["embedding_ln_bias"],
                               synth.dequantized_layer_weights(args["layer_weights"]), heads, tw, window=window,
                               workers=O.default_workers())
    ref = ref[mask.astype(bool)]
    assert np.isfinite(got).all()
    assert np.abs(np.linalg.norm(got, axis=1) - 1).max() < 1e-3
    assert np.abs(got - ref).max() <= 3e-3           # per-token rows are 128-d unit vectors: entries ~0.09
    assert cosine_rows(got, ref).min() >= 0.9995
    # the pooled embedding of the same handle still works, and packing the vectors is bit-exact
    spec = eos_b200.make_rotation_spec(tdim, 2, seed=402)
    qz = eos_b200.Quantizer(rt, spec)
    codes = torch.empty((rows, tdim // 4), dtype=torch.uint8, device="cuda")
    norms = torch.empty((rows,), dtype=torch.float32, device="cuda")
    qz.quantize_device(d_vec.data_ptr(), rows, codes.data_ptr(), norms.data_ptr())
    torch.cuda.synchronize()
    rc, rn = O.tq_encode(got, 2, spec.perm, spec.signs1, spec.signs2, spec.boundaries)
    assert np.array_equal(codes.cpu().numpy(), rc) and np.array_equal(norms.cpu().numpy(), rn)
    pooled = enc.run(ids, mask)
    assert np.isfinite(pooled).all() and np.abs(np.linalg.norm(pooled[0]) - 1) < 1e-3
    qz.close()
    enc.close()
