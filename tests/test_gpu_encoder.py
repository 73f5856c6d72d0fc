"""GPU parity of the encoder forward (C ABI: eos_b200_encoder_bind / _run) against the CPU oracle and the
committed golden fixtures.  Tolerance: max-abs <= 2e-3 after L2 normalisation and cosine >= 0.9999
(runtime/pretrained_bert_golden_parity_test.go:99-103)."""
import numpy as np
import pytest

from tests.helpers import cosine_rows, load_bert_fixture

pytestmark = pytest.mark.gpu

MAX_ABS = 2e-3
MIN_COS = 0.9999


@pytest.fixture(scope="module")
def rt():
    import eos_b200
    r = eos_b200.Runtime(0)
    yield r
    r.close()


def _check(out, ref):
    assert np.isfinite(out).all()
    assert np.abs(out - ref).max() <= MAX_ABS, float(np.abs(out - ref).max())
    nz = np.linalg.norm(ref, axis=-1) > 0
    if nz.any():
        assert cosine_rows(out[nz], ref[nz]).min() >= MIN_COS


@pytest.mark.parametrize("name", ["bert_tiny_golden.npz", "bert_hf_seeded.npz"])
@pytest.mark.parametrize("pooling", ["masked_mean", "cls"])
def test_golden_fixture(rt, name, pooling):
    import eos_b200
    from oracle import oracle as O
    z, weights = load_bert_fixture(name)
    enc = eos_b200.BertEmbedder(rt, z["tok"], z["pos"], z["typ"], z["emb_gamma"], z["emb_beta"], weights,
                                int(z["heads"]), float(z["eps"]), pooling)
    out = enc.run(z["input_ids"], z["attention_mask"], z["token_type_ids"])
    ref = O.bert_embedder(z["input_ids"], z["attention_mask"], z["token_type_ids"], z["tok"], z["pos"], z["typ"],
                          z["emb_gamma"], z["emb_beta"], weights, int(z["heads"]), float(z["eps"]), pooling)
    _check(out, ref)
    if pooling == "masked_mean":
        _check(out, z["expected"])  # the reference's own known answer (PyTorch / transformers)
    elif "expected_cls" in z.files:
        _check(out, z["expected_cls"])
    enc.close()


def _ragged_mask(batch, tokens, rng):
    lengths = rng.integers(1, tokens + 1, size=batch)
    mask = (np.arange(tokens)[None, :] < lengths[:, None]).astype(np.int32)
    mask[1] = 0                       # all-masked sequence -> zero vector
    mask[2] = 1                       # full length
    mask[3, ::3] = 0                  # holes: not a prefix mask, token 0 masked
    return mask


@pytest.mark.parametrize("hidden,heads,inter,layers", [(128, 2, 256, 2), (96, 6, 192, 1), (384, 6, 1536, 4)])
@pytest.mark.parametrize("weight_mode", [0, 1])
@pytest.mark.parametrize("pooling", ["masked_mean", "cls"])
def test_q8_encoder_matches_oracle(rt, hidden, heads, inter, layers, weight_mode, pooling):
    import eos_b200
    from eos_b200 import synth
    from oracle import oracle as O
    if pooling == "cls" and (hidden != 128 or weight_mode != 0):
        pytest.skip("cls pooling covered on one configuration")
    rng = np.random.default_rng(hidden + layers)
    args = synth.make_q8_encoder(layers, hidden, heads, inter, vocab=500, max_pos=80, seed=hidden)
    batch, tokens = 6, 70
    ids = rng.integers(0, 500, size=(batch, tokens), dtype=np.int32)
    mask = _ragged_mask(batch, tokens, rng)
    types = rng.integers(0, 2, size=(batch, tokens), dtype=np.int32)
    enc = eos_b200.BertEmbedder(rt, pooling=pooling, weight_mode=weight_mode, **args)
    out = enc.run(ids, mask, types)
    ref = O.bert_embedder(ids, mask, types, args["token_embeddings"], args["position_embeddings"],
                          args["token_type_embeddings"], args["embedding_ln_weight"], args["embedding_ln_bias"],
                          synth.dequantized_layer_weights(args["layer_weights"]), heads, 1e-12, pooling, workers=8)
    _check(out, ref)
    if pooling == "masked_mean":
        assert np.array_equal(out[1], np.zeros_like(out[1]))  # all keys masked: zeros, never NaN
    assert enc.last_stats.valid_tokens == int(mask.sum()) + (int((mask[:, 0] == 0).sum()) if pooling == "cls" else 0)
    # the same call twice gives the same bits (no atomics on the data path)
    assert np.array_equal(out, enc.run(ids, mask, types))
    enc.close()


def test_projection_head_and_batch_independence(rt):
    import eos_b200
    from eos_b200 import synth
    from oracle import oracle as O
    args = synth.make_q8_encoder(2, 128, 2, 256, vocab=300, max_pos=64, seed=5, head_out=96)
    ids, mask, _ = synth.make_batch(9, 64, 300, 3, 64, seed=6)
    enc = eos_b200.BertEmbedder(rt, **args)
    out = enc.run(ids, mask)
    ref = O.bert_embedder(ids, mask, np.zeros_like(ids), args["token_embeddings"], args["position_embeddings"],
                          args["token_type_embeddings"], args["embedding_ln_weight"], args["embedding_ln_bias"],
                          synth.dequantized_layer_weights(args["layer_weights"]), 2, 1e-12, "masked_mean",
                          head_w=args["head_weights"], workers=8)
    _check(out, ref)
    np.testing.assert_allclose(np.linalg.norm(out, axis=1), 1.0, atol=1e-5)
    # a sequence's embedding does not depend on what else is in the batch, nor on padding width
    sub = enc.run(ids[3:5, :], mask[3:5, :])
    assert np.abs(sub - out[3:5]).max() <= 1e-6
    longest = int(mask[3:5].sum(1).max())
    sub2 = enc.run(ids[3:5, :longest], mask[3:5, :longest])
    assert np.abs(sub2 - out[3:5]).max() <= 1e-6
    enc.close()


def test_error_behaviour(rt):
    import eos_b200
    from eos_b200 import synth
    args = synth.make_q8_encoder(1, 64, 1, 128, vocab=50, max_pos=16, seed=9)
    enc = eos_b200.BertEmbedder(rt, **args)
    ids, mask, _ = synth.make_batch(2, 16, 50, 4, 16, seed=1)
    bad = ids.copy()
    bad[1, 2] = 50  # out of range: an error, not a clamp (runtime/backend/tensor_ops.go:1479-1487)
    with pytest.raises(eos_b200.EosB200DeviceStatusError):
        enc.run(bad, mask)
    bad[1, 2] = -1
    with pytest.raises(eos_b200.EosB200DeviceStatusError):
        enc.run(bad, mask)
    out = enc.run(ids, mask)  # the handle stays usable after a flagged run
    assert np.isfinite(out).all()
    with pytest.raises(eos_b200.EosB200Error):
        enc.run(np.zeros((2, 17), np.int32), np.ones((2, 17), np.int32))  # longer than max_positions
    with pytest.raises(ValueError):
        enc.run(ids, mask[:, :8])
    with pytest.raises(eos_b200.EosB200Error):
        enc.run(np.zeros((0, 16), np.int32), np.zeros((0, 16), np.int32))
    enc.close()
    with pytest.raises(eos_b200.EosB200Error):
        bad_args = dict(args)
        bad_args["num_attention_heads"] = 3  # hidden not divisible
        eos_b200.BertEmbedder(rt, **bad_args)


def test_device_resident_run_matches_host_run(rt):
    import torch
    import eos_b200
    from eos_b200 import synth
    args = synth.make_q8_encoder(2, 128, 2, 256, vocab=300, max_pos=128, seed=21)
    ids, mask, _ = synth.make_batch(16, 128, 300, 8, 128, seed=22)
    enc = eos_b200.BertEmbedder(rt, **args)
    ref = enc.run(ids, mask)
    d_ids = torch.from_numpy(ids).cuda()
    d_mask = torch.from_numpy(mask).cuda()
    d_out = torch.empty((16, 128), dtype=torch.float32, device="cuda")
    ts = torch.cuda.Stream()
    ts.wait_stream(torch.cuda.current_stream())
    stream = ts.cuda_stream  # non-null: the library launches on this stream
    launches = enc.run_device(d_ids.data_ptr(), d_mask.data_ptr(), None, 16, 128, d_out.data_ptr(), stream)
    enc.sync(stream)
    assert launches == 5 + 1 + 7 * 2 + 1
    assert np.array_equal(d_out.cpu().numpy(), ref)
    enc.close()


def test_local_window_attention_extension(rt):
    """Local-window attention (an extension: the reference has none).  Oracle = the reference attention with the
    band mask 2*|i - j| < W.  Weights are large enough for attention to be far from uniform, so a wrong band
    shows up well above the tolerance; covers the tensor-core (head_dim 64) and the generic kernel."""
    import eos_b200
    from oracle import oracle as O
    for hidden, heads in ((128, 2), (64, 4)):
        rng = np.random.default_rng(hidden)
        inter = 2 * hidden

        def mat(o, i, std=0.12):
            return (rng.standard_normal((o, i)) * std).astype(np.float32)

        def vec(n, base=0.0):
            return (base + rng.standard_normal(n) * 0.05).astype(np.float32)

        lw = [mat(hidden, hidden), vec(hidden), mat(hidden, hidden), vec(hidden), mat(hidden, hidden), vec(hidden),
              mat(hidden, hidden), vec(hidden), vec(hidden, 1.0), vec(hidden), mat(inter, hidden), vec(inter),
              mat(hidden, inter), vec(hidden), vec(hidden, 1.0), vec(hidden)]
        tok, pos, typ = mat(100, hidden, 0.5), mat(210, hidden, 0.5), mat(2, hidden, 0.5)
        eg, eb = vec(hidden, 1.0), vec(hidden)
        rng2 = np.random.default_rng(32)
        ids = rng2.integers(0, 100, size=(4, 210), dtype=np.int32)
        lengths = np.array([210, 150, 70, 1])
        mask = (np.arange(210)[None, :] < lengths[:, None]).astype(np.int32)
        mask[1, 40:90:2] = 0
        outs = {}
        for window in (0, 1000, 64, 16):
            enc = eos_b200.BertEmbedder(rt, tok, pos, typ, eg, eb, lw, heads, attention_window=window)
            outs[window] = enc.run(ids, mask)
            ref = O.bert_embedder(ids, mask, np.zeros_like(ids), tok, pos, typ, eg, eb, lw, heads, window=window,
                                  workers=8)
            _check(outs[window], ref)
            enc.close()
        # a window wider than the sequence is full attention (different kernels: tensor-memory vs mma.sync)
        assert np.abs(outs[0] - outs[1000]).max() <= 1e-4
        assert np.abs(outs[0][:3] - outs[16][:3]).max() > 5e-3  # and a narrow one is a different function


def test_submit_wait_reproduces_run(rt):
    """Batches submitted without waiting in between (eos_b200_encoder_submit / _wait) give the bits of the synchronous
    call, each in its own output buffer, in submission order; a bad token id in one of them surfaces at the wait and
    leaves the handle usable."""
    import eos_b200
    from eos_b200 import synth
    w = synth.make_q8_encoder(2, 128, 4, 256, vocab=500, max_pos=64, seed=77)
    enc = eos_b200.BertEmbedder(rt, **w)
    batches = [synth.make_batch(b, t, 500, 3, t, seed=90 + i)[:2] for i, (b, t) in enumerate(((5, 40), (9, 64), (2, 17)))]
    want = [enc.run(ids, mask) for ids, mask in batches]
    per_forward = enc.last_stats.kernel_launches
    outs = [np.full((ids.shape[0], enc.out_dim), np.nan, np.float32) for ids, _ in batches]
    for (ids, mask), out in zip(batches, outs):
        enc.submit(np.ascontiguousarray(ids, np.int32), np.ascontiguousarray(mask, np.int32), out)
    enc.wait()
    for got, ref in zip(outs, want):
        assert np.array_equal(got, ref)
    assert enc.last_stats.kernel_launches == 3 * per_forward
    bad = np.ascontiguousarray(batches[0][0], np.int32).copy()
    bad[0, 0] = 500
    enc.submit(bad, np.ascontiguousarray(batches[0][1], np.int32), outs[0])
    enc.submit(np.ascontiguousarray(batches[1][0], np.int32), np.ascontiguousarray(batches[1][1], np.int32), outs[1])
    with pytest.raises(eos_b200.EosB200DeviceStatusError):
        enc.wait()
    assert np.array_equal(enc.run(*batches[2]), want[2])
    with pytest.raises(ValueError):
        enc.submit(batches[0][0].astype(np.int64), batches[0][1], outs[0])
    enc.close()
