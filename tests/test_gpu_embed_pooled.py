"""GPU parity of the compiled pipeline gather -> matmul -> normalize -> masked mean_pool
(examples/embed_masked_pooled.eos) against the CPU oracle, at the CPU-runnable benchmark configuration."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    import eos_b200
    r = eos_b200.Runtime(0)
    yield r
    r.close()


def _config(vocab, dim, out_dim, batch, tokens, min_len, seed):
    from eos_b200 import synth
    rng = np.random.default_rng(seed)
    table = synth.f16_round(rng.standard_normal((vocab, dim), dtype=np.float32) * np.float32(0.02))
    proj = synth.f16_round(rng.standard_normal((dim, out_dim), dtype=np.float32) * np.float32(0.05))
    ids, mask, _ = synth.make_batch(batch, tokens, vocab, min_len, tokens, seed + 1)
    return table, proj, ids, mask


@pytest.mark.parametrize("pool_then_l2", [False, True])
def test_masked_mean_pooled_embed_config(rt, pool_then_l2):
    # table f16[30522,384] ~N(0,0.02), projection f16[384,384] ~N(0,0.05), batch 32 x T=128, lengths 16..128
    import eos_b200
    from oracle import oracle as O
    table, proj, ids, mask = _config(30522, 384, 384, 32, 128, 16, seed=101)
    pipe = eos_b200.EmbedPooledPipeline(rt, table, proj)
    out = pipe.run(ids, mask, pool_then_l2=pool_then_l2)
    ref = O.embed_pooled(table, proj, ids, mask, pool_then_l2=pool_then_l2)
    assert np.abs(out - ref).max() <= 2e-5, float(np.abs(out - ref).max())
    # the output dtype of the pipeline is f16: both sides agree after that rounding as well
    assert np.abs(out.astype(np.float16).astype(np.float32) - ref.astype(np.float16).astype(np.float32)).max() <= 1e-3
    pipe.close()


def test_edges(rt):
    import eos_b200
    from oracle import oracle as O
    table, proj, ids, mask = _config(97, 48, 40, 5, 19, 1, seed=7)
    mask[2] = 0          # nothing to pool: zeros
    mask[3, ::2] = 0     # holes
    pipe = eos_b200.EmbedPooledPipeline(rt, table, proj)
    out = pipe.run(ids, mask)
    ref = O.embed_pooled(table, proj, ids, mask)
    assert np.abs(out - ref).max() <= 2e-5
    assert np.array_equal(out[2], np.zeros(40, np.float32))
    bad = ids.copy()
    bad[0, 0] = 97
    with pytest.raises(eos_b200.EosB200DeviceStatusError):  # "gather index out of range"
        pipe.run(bad, mask)
    with pytest.raises(ValueError):
        pipe.run(ids[:0], mask[:0])
    pipe.close()


@pytest.mark.parametrize("scale", ["rsqrt_rhs_rows", -0.5, 0.0, "none"])
def test_matmul_scale_attribute(rt, scale):
    """The matmul step's `scale` attribute (runtime/backend/tensor_ops.go:1259-1315): a positive factor cancels under
    the normalisation up to rounding, a negative one flips the embedding, zero leaves nothing to normalise."""
    import eos_b200
    from oracle import oracle as O
    table, proj, ids, mask = _config(211, 64, 48, 6, 33, 3, seed=55)
    value = {"rsqrt_rhs_rows": float(np.float32(1.0 / np.sqrt(64.0))), "none": 1.0}.get(scale, scale)
    for pool_then_l2 in (False, True):
        pipe = eos_b200.EmbedPooledPipeline(rt, table, proj, matmul_scale=scale)
        out = pipe.run(ids, mask, pool_then_l2=pool_then_l2)
        ref = O.embed_pooled(table, proj, ids, mask, pool_then_l2=pool_then_l2, matmul_scale=float(value))
        assert np.abs(out - ref).max() <= 2e-5
        if value == 0.0:
            assert not out.any()
        pipe.close()
    with pytest.raises(ValueError):
        eos_b200.EmbedPooledPipeline(rt, table, proj, matmul_scale="sqrt")
    with pytest.raises(ValueError):
        eos_b200.EmbedPooledPipeline(rt, table, proj, matmul_scale=float("inf"))
