"""GPU parity of the compact encoder profile (C ABI: eos_b200_compact_encoder_bind + eos_b200_encoder_run) against the
oracle's step-by-step restatement of the graph models/default_embedding.go:461-505 emits (gather + gather, rope,
bias-free [in, out] projections, multi-head attention over the unmasked keys, non-affine LayerNorm, tanh GELU,
per-token normalize, optional output projection, masked mean pool).  Tolerance: the device-parity bar of the
reference's own embed_pooled tests (cosine >= 0.999, cuda_embed_pooled_parity_linux_test.go:124,241), tightened."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    import eos_b200
    r = eos_b200.Runtime(0)
    yield r
    r.close()


def _q8_in_out(rng, rows, cols, std, per_channel):
    """Weights on the reference's q8 grid (symmetric, 127 levels) in [in, out] layout."""
    import eos_b200
    w = (rng.standard_normal((rows, cols)) * std).astype(np.float32)
    if per_channel:
        scales = (np.abs(w).max(axis=0) / 127.0).astype(np.float32)
        codes = np.clip(np.rint(w / scales[None, :]), -127, 127).astype(np.int8)
    else:
        scales = np.array([np.abs(w).max() / 127.0], np.float32)
        codes = np.clip(np.rint(w / scales[0]), -127, 127).astype(np.int8)
    return eos_b200.Q8WeightInOut(codes, scales)


def _model(seed, layers, dim, heads, inter, vocab, roles, out_dim, per_channel):
    rng = np.random.default_rng(seed)
    f16 = lambda a: a.astype(np.float16).astype(np.float32)
    tok = f16(rng.standard_normal((vocab, dim)) * 0.5)
    role = f16(rng.standard_normal((roles, dim)) * 0.1)
    lw = []
    for _ in range(layers):
        lw += [_q8_in_out(rng, dim, dim, 0.08, per_channel) for _ in range(4)]
        lw += [_q8_in_out(rng, dim, inter, 0.08, per_channel), _q8_in_out(rng, inter, dim, 0.05, per_channel)]
    proj = _q8_in_out(rng, dim, out_dim, 0.1, per_channel) if out_dim else None
    return tok, role, lw, proj


def _batch(seed, batch, tokens, vocab, roles, min_len):
    rng = np.random.default_rng(seed)
    ids = rng.integers(0, vocab, size=(batch, tokens)).astype(np.int32)
    rid = rng.integers(0, roles, size=(batch, tokens)).astype(np.int32)
    lengths = rng.integers(min_len, tokens + 1, size=batch)
    mask = (np.arange(tokens)[None, :] < lengths[:, None]).astype(np.int32)
    return ids, mask, rid


@pytest.mark.parametrize("layers,dim,heads,inter,tokens,out_dim,per_channel", [
    (2, 128, 2, 256, 48, 0, False),      # head dim 64: tensor-memory attention kernel
    (2, 96, 4, 192, 40, 64, True),       # head dim 24: generic attention kernel, output projection
    (1, 64, 1, 128, 200, 0, False),      # single head, several query tiles
])
def test_compact_encoder_matches_oracle(rt, layers, dim, heads, inter, tokens, out_dim, per_channel):
    import eos_b200
    from oracle import oracle as O
    vocab, roles, batch = 500, 3, 6
    tok, role, lw, proj = _model(layers * 100 + dim, layers, dim, heads, inter, vocab, roles, out_dim, per_channel)
    ids, mask, rid = _batch(7, batch, tokens, vocab, roles, 3)
    mask[2] = 0                        # a sequence without valid tokens pools to zeros
    mask[3, 5] = 0                     # a hole in the mask: that key is invisible, positions stay absolute
    enc = eos_b200.CompactEmbedder(rt, tok, role, lw, heads, output_projection=proj)
    got = enc.run(ids, mask, rid)
    ref_layers = [tuple(w.dequantized() for w in lw[l * 6:(l + 1) * 6]) for l in range(layers)]
    ref = O.compact_encoder(ids, mask, rid, tok, role, ref_layers, heads,
                            output_projection=proj.dequantized() if proj is not None else None, workers=4)
    assert got.shape == ref.shape == (batch, out_dim or dim)
    assert np.isfinite(got).all()
    assert (got[2] == 0).all() and (ref[2] == 0).all()
    err = np.abs(got - ref).max()
    assert err <= 2e-3, float(err)
    for b in range(batch):
        if b == 2:
            continue
        cos = float(got[b] @ ref[b] / (np.linalg.norm(got[b]) * np.linalg.norm(ref[b])))
        assert cos >= 0.9999, (b, cos)
    enc.close()


def test_compact_encoder_weight_modes_agree_and_bad_ids_are_reported(rt):
    import eos_b200
    tok, role, lw, _ = _model(3, 1, 128, 2, 256, 300, 2, 0, True)
    ids, mask, rid = _batch(9, 4, 32, 300, 2, 5)
    a = eos_b200.CompactEmbedder(rt, tok, role, lw, 2, weight_mode=eos_b200.encoder.WEIGHTS_F16_RESIDENT)
    b = eos_b200.CompactEmbedder(rt, tok, role, lw, 2, weight_mode=eos_b200.encoder.WEIGHTS_Q8_SMEM_DEQUANT)
    assert np.array_equal(a.run(ids, mask, rid), b.run(ids, mask, rid))
    bad = ids.copy()
    bad[1, 0] = 300
    with pytest.raises(eos_b200.EosB200DeviceStatusError):
        a.run(bad, mask, rid)
    bad_role = rid.copy()
    bad_role[0, 1] = 2
    with pytest.raises(eos_b200.EosB200DeviceStatusError):
        a.run(ids, mask, bad_role)
    assert np.isfinite(a.run(ids, mask, rid)).all()   # the handle stays usable
    a.close()
    b.close()
