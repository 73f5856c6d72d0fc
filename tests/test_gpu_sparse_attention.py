"""GPU parity of sparse attention (C ABI: eos_b200_sparse_attention, eos_b200_turbo_sparse_attention) against the
CPU oracle's restatement of sparseAttentionTensor / turboSparseAttentionTensor
(runtime/backend/attention_ops.go:218-300).

Bars: scores, selection and value mix are fp32 in the reference's order, so outputs agree to the last bits; the one
step that is not bit-specified is exp() in double (device libm vs host libm, each within 1 ulp of a double), which a
float output sees only when a weight lands on a rounding boundary.  The tolerance is therefore a few float ulps of the
largest output (4e-7 relative to it) and the tests also demand that almost every element is identical."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    import eos_b200
    r = eos_b200.Runtime(0)
    yield r
    r.close()


def _close(got, ref):
    assert got.shape == ref.shape
    assert np.abs(got - ref).max() <= 4e-7 * max(1e-30, float(np.abs(ref).max()))
    assert (got.view(np.uint32) == ref.view(np.uint32)).mean() >= 0.99


def test_known_answers(rt):
    """The two hand-checkable cases the reference's own tests hold (runtime/backend/attention_ops_test.go): a top-1
    pick returns that key's value; routing keeps the block whose middle key scores best."""
    from eos_b200.attention import sparse_attention
    q = np.array([[1, 0], [0, 1]], np.float32)
    k = np.array([[1, 0], [0, 1], [-1, 0]], np.float32)
    v = np.array([[10, 1], [20, 2], [30, 3]], np.float32)
    out = sparse_attention(rt, q, k, v, top_k=1)
    assert np.array_equal(out, np.array([[10, 1], [20, 2]], np.float32))
    q = np.array([[1, 0]], np.float32)
    k = np.array([[0, 0], [0, 0], [5, 0], [6, 0], [7, 0], [0, 0]], np.float32)
    v = np.array([[1], [2], [3], [4], [5], [6]], np.float32)
    out = sparse_attention(rt, q, k, v, top_k=1, route_block_size=2, route_top_blocks=1)
    from oracle import oracle as O
    assert np.array_equal(out, O.sparse_attention(q, k, v, 1, 2, 1))


@pytest.mark.parametrize("b,ql,kl,dim,vdim,top_k,rbs,rtb", [
    (1, 7, 50, 16, 16, 0, 0, 0),           # default budget ceil(sqrt(50)) = 8
    (3, 33, 1000, 64, 48, 32, 0, 0),
    (2, 5, 700, 96, 33, 128, 0, 0),        # the largest budget, odd value width
    (2, 9, 3, 8, 4, 10, 0, 0),             # budget clamped to the key count
    (2, 40, 2048, 64, 64, 16, 64, 4),      # routed: 32 blocks, 4 kept
    (1, 11, 1000, 32, 32, 0, 37, 128),     # routed, ragged last block, every block kept (clamped to 28)
    (1, 4, 300, 24, 8, 64, 5, 3),          # budget above the routed candidates (15)
    (1, 3, 9000, 128, 16, 96, 0, 0),       # many list cuts
])
def test_parity(rt, b, ql, kl, dim, vdim, top_k, rbs, rtb):
    from eos_b200.attention import sparse_attention
    from oracle import oracle as O
    rng = np.random.default_rng(1000 + kl + dim)
    q = rng.standard_normal((b, ql, dim)).astype(np.float32) * 0.5
    k = rng.standard_normal((b, kl, dim)).astype(np.float32)
    v = rng.standard_normal((b, kl, vdim)).astype(np.float32)
    _close(sparse_attention(rt, q, k, v, top_k, rbs, rtb), O.sparse_attention(q, k, v, top_k, rbs, rtb))


def test_ties_go_to_the_lower_index(rt):
    """Equal scores: the earlier key wins (attention_ops.go:418-443 orders by score, then index)."""
    from eos_b200.attention import sparse_attention
    from oracle import oracle as O
    rng = np.random.default_rng(7)
    q = rng.integers(-2, 3, (2, 6, 8)).astype(np.float32)
    k = rng.integers(-1, 2, (2, 400, 8)).astype(np.float32)       # small integers: many exact ties
    v = rng.standard_normal((2, 400, 12)).astype(np.float32)
    for top_k, rbs, rtb in [(5, 0, 0), (40, 0, 0), (7, 16, 5)]:
        _close(sparse_attention(rt, q, k, v, top_k, rbs, rtb), O.sparse_attention(q, k, v, top_k, rbs, rtb))


def test_rank2_and_empty_keys(rt):
    from eos_b200.attention import sparse_attention
    from oracle import oracle as O
    rng = np.random.default_rng(8)
    q = rng.standard_normal((5, 16)).astype(np.float32)
    k = rng.standard_normal((20, 16)).astype(np.float32)
    v = rng.standard_normal((20, 6)).astype(np.float32)
    _close(sparse_attention(rt, q, k, v, 4), O.sparse_attention(q, k, v, 4))
    out = sparse_attention(rt, q, k[:0], v[:0], 4)
    assert out.shape == (5, 6) and not out.any()


def test_argument_errors(rt):
    from eos_b200.attention import sparse_attention
    q = np.zeros((2, 4, 8), np.float32)
    k = np.zeros((2, 600, 8), np.float32)
    v = np.zeros((2, 600, 8), np.float32)
    with pytest.raises(ValueError):
        sparse_attention(rt, q, k[:1], v)                      # batch mismatch
    with pytest.raises(ValueError):
        sparse_attention(rt, q, k[:, :, :4], v)                # query / key widths
    with pytest.raises(ValueError):
        sparse_attention(rt, q, k, v[:, :10])                  # key / value lengths
    with pytest.raises(RuntimeError, match="128"):
        sparse_attention(rt, q, k, v, top_k=129)
    with pytest.raises(RuntimeError, match="128"):
        sparse_attention(rt, q, k, v, top_k=4, route_block_size=2, route_top_blocks=200)


def _unpack(codes, dim, bits):
    """Packed little-endian bit fields -> one code per byte (the layout of the reference's coords tensor)."""
    bitsarr = np.unpackbits(codes, axis=1, bitorder="little")[:, :dim * bits].reshape(codes.shape[0], dim, bits)
    return (bitsarr * (1 << np.arange(bits, dtype=np.uint8))).sum(axis=2).astype(np.uint8)


@pytest.mark.parametrize("dim,vdim,bits,kl,top_k,rbs,rtb", [(64, 64, 4, 500, 16, 0, 0), (96, 32, 2, 333, 0, 0, 0),
                                                         (128, 128, 4, 1024, 24, 32, 6)])
def test_turbo_parity(rt, dim, vdim, bits, kl, top_k, rbs, rtb):
    """Compressed K / V: codes and 8-bit log norms from the oracle's encoder; expected = oracle decode + oracle
    attention.  The device decode is fp32 in the oracle's order, so the attention sees identical K / V."""
    import eos_b200
    from eos_b200.attention import turbo_sparse_attention
    from oracle import oracle as O
    rng = np.random.default_rng(77 + dim)
    b, ql = 2, 9
    kspec = eos_b200.make_rotation_spec(dim, bits, seed=402)
    vspec = kspec if vdim == dim else eos_b200.make_rotation_spec(vdim, bits, seed=403)
    key = rng.standard_normal((b * kl, dim)).astype(np.float32) * np.exp(rng.uniform(-2, 2, (b * kl, 1))).astype(np.float32)
    val = rng.standard_normal((b * kl, vdim)).astype(np.float32)
    q = rng.standard_normal((b, ql, dim)).astype(np.float32) * 0.3
    kc, kn = O.tq_encode(key, bits, kspec.perm, kspec.signs1, kspec.signs2, kspec.boundaries)
    vc, vn = O.tq_encode(val, bits, vspec.perm, vspec.signs1, vspec.signs2, vspec.boundaries)
    knc, vnc = O.tq_norm_code(kn), O.tq_norm_code(vn)
    kd = O.tq_decode(kc, O.tq_norm_value(knc), dim, bits, kspec.perm, kspec.signs1, kspec.signs2, kspec.centroids)
    vd = O.tq_decode(vc, O.tq_norm_value(vnc), vdim, bits, vspec.perm, vspec.signs1, vspec.signs2, vspec.centroids)
    ref = O.sparse_attention(q, kd.reshape(b, kl, dim), vd.reshape(b, kl, vdim), top_k, rbs, rtb)
    kq = eos_b200.Quantizer(rt, kspec)
    vq = kq if vspec is kspec else eos_b200.Quantizer(rt, vspec)
    got = turbo_sparse_attention(kq, vq, q, _unpack(kc, dim, bits).reshape(b, kl, dim), knc.reshape(b, kl),
                                 _unpack(vc, vdim, bits).reshape(b, kl, vdim), vnc.reshape(b, kl), top_k, rbs, rtb)
    _close(got, ref)
    if vq is not kq:
        vq.close()
    kq.close()
