"""GPU parity of the token-pool encoder and its token-span child vectors (C ABI: eos_b200_token_pool_bind / _encode)
against the CPU oracle's restatement of sparseTokenPoolEncoder.embedTextFullEncoderRows and the span pooling
(runtime/sparse_token_pool_vector_export.go:1290-1335, 1534-1618).

The model is fp32 with fixed summation orders on both sides; the only steps that are not bit-specified are tanh and
exp in double (device library vs host library).  Rows are unit vectors (entries of the order of 0.1): the bar is
2e-6 absolute."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 2e-6


@pytest.fixture(scope="module")
def rt():
    import eos_b200
    r = eos_b200.Runtime(0)
    yield r
    r.close()


def _weights(vocab, dim, hidden, repeats, flags, seed):
    rng = np.random.default_rng(seed)

    def mat(i, o, std):
        return (rng.standard_normal((i, o)) * std).astype(np.float32)

    w = {"token_embedding": mat(vocab, dim, 1.0), "attention_query": mat(dim, dim, dim ** -0.5),
         "attention_key": mat(dim, dim, dim ** -0.5), "attention_value": mat(dim, dim, dim ** -0.5),
         "attention_output": mat(dim, dim, dim ** -0.5), "hidden_projection": mat(dim, hidden, dim ** -0.5),
         "projection": mat(hidden, dim, hidden ** -0.5), "encoder_repeats": repeats}
    w.update(dict(zip(("attention_residual", "attention_layer_norm", "ffn_residual", "ffn_layer_norm"), flags)))
    return w


def _encoder(rt, w):
    from eos_b200.token_pool import TokenPoolEncoder
    return TokenPoolEncoder(rt, **w)


@pytest.mark.parametrize("flags", [(True, True, True, True), (False, False, False, False), (True, False, False, True)])
def test_dense_rows_pooled_and_spans(rt, flags):
    from oracle import oracle as O
    w = _weights(300, 64, 160, 2, flags, seed=11)
    rng = np.random.default_rng(12)
    T = 75
    tokens = rng.integers(0, 300, T).astype(np.int32)
    tokens[5] = 300          # unknown ids gather a zero row
    tokens[6] = -1
    mask = np.ones(T, np.int32)
    mask[60:] = 0
    mask[10] = 0
    enc = _encoder(rt, w)
    rows = enc.token_rows(tokens)
    ref = O.token_pool_rows(w, tokens)
    assert np.abs(rows - ref).max() <= TOL
    assert np.abs(np.linalg.norm(rows, axis=1) - 1).max() < 1e-5
    pooled = enc.embed(tokens, mask)
    assert np.abs(pooled - O.token_span_pool(ref, mask, 0, T, fallback_all=True)[0]).max() <= TOL
    assert np.abs(enc.embed(tokens, np.zeros(T, np.int32)) - O.token_span_pool(ref, np.zeros(T, np.int32), 0, T, True)[0]).max() <= TOL
    spans = O.token_spans(T, 16, 4, 3)
    from eos_b200.token_pool import token_spans
    assert token_spans(T, 16, 4, 3) == spans
    # the last span lies in the masked tail: the reference refuses a span without an active token
    assert not mask[spans[-1][0]:spans[-1][1]].any()
    import eos_b200
    with pytest.raises(eos_b200.EosB200Error, match="no active tokens"):
        enc.span_child_vectors(tokens, mask, span_tokens=16, span_overlap=4, span_min_tokens=3)
    mask2 = mask.copy()
    mask2[60:] = 1
    children = enc.span_child_vectors(tokens, mask2, span_tokens=16, span_overlap=4, span_min_tokens=3)
    assert children.shape == (len(spans), 64)
    for i, (a, b) in enumerate(spans):
        vec, active = O.token_span_pool(ref, mask2, a, b)
        assert active > 0 and np.abs(children[i] - vec).max() <= TOL
    enc.close()


@pytest.mark.parametrize("key_bits,value_bits,top_k,rbs,rtb", [(4, 4, 8, 0, 0), (4, 2, 0, 0, 0), (2, 2, 12, 16, 3)])
def test_turbo_sparse_rows(rt, key_bits, value_bits, top_k, rbs, rtb):
    """Keys and values TurboQuant-encoded per layer (codes + 8-bit log norms), sparse attention over the decoded rows."""
    import eos_b200
    from eos_b200.token_pool import ATTENTION_TURBO_SPARSE
    from oracle import oracle as O
    w = _weights(200, 64, 96, 2, (True, True, True, True), seed=21)
    tokens = np.random.default_rng(22).integers(0, 200, 150).astype(np.int32)
    kspec = eos_b200.make_rotation_spec(64, key_bits, seed=402)
    vspec = kspec if value_bits == key_bits else eos_b200.make_rotation_spec(64, value_bits, seed=402)
    kq = eos_b200.Quantizer(rt, kspec)
    vq = kq if vspec is kspec else eos_b200.Quantizer(rt, vspec)
    enc = _encoder(rt, w)
    rows = enc.token_rows(tokens, ATTENTION_TURBO_SPARSE, kq, vq, top_k, rbs, rtb)
    ref = O.token_pool_rows(w, tokens, 1, kspec, vspec, top_k, rbs, rtb)
    assert np.abs(rows - ref).max() <= TOL
    with pytest.raises(eos_b200.EosB200Error):
        enc.token_rows(tokens, ATTENTION_TURBO_SPARSE)            # no quantizers
    enc.close()
    if vq is not kq:
        vq.close()
    kq.close()


def test_longer_sequence_and_bind_errors(rt):
    import eos_b200
    from eos_b200.token_pool import TokenPoolEncoder
    from oracle import oracle as O
    w = _weights(1000, 96, 192, 1, (True, True, True, True), seed=31)
    tokens = np.random.default_rng(32).integers(0, 1000, 700).astype(np.int32)
    enc = _encoder(rt, w)
    rows = enc.token_rows(tokens)
    assert np.abs(rows - O.token_pool_rows(w, tokens)).max() <= TOL
    assert enc.last_stats.kernel_launches > 0 and enc.last_stats.valid_tokens == 700
    enc.close()
    bad = dict(w)
    bad["projection"] = w["projection"][:, :50]
    with pytest.raises(ValueError):
        TokenPoolEncoder(rt, **bad)
    with pytest.raises(ValueError):
        _encoder(rt, w).token_rows(np.zeros(0, np.int32))
