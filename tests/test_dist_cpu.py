"""Multi-rank host logic on CPU: world_size 2 over gloo.  The scoring on each rank is done by the CPU oracle
(this is a test of sharding, key exchange and merge order, not of the kernels)."""
import os
import socket

import numpy as np
import pytest


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, n_total, ret):
    import torch
    import torch.distributed as dist

    import eos_b200.dist as D
    from eos_b200.turboquant import make_rotation_spec
    from oracle import oracle as O

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        spec = make_rotation_spec(128, 4, seed=5)
        rng = np.random.default_rng(1)                      # same data on every rank, sharded by row range
        x = rng.standard_normal((n_total, 128)).astype(np.float32)
        q = rng.standard_normal((3, 128)).astype(np.float32)
        codes, norms = O.tq_encode(x, 4, spec.perm, spec.signs1, spec.signs2, spec.boundaries)
        if n_total >= 60:
            codes[40:60] = codes[0:20]                      # exact ties across the shard boundary
            norms[40:60] = norms[0:20]
        lo, hi = D.shard_bounds(n_total, world, rank)
        k = 10
        local = np.zeros((3, k), dtype=np.uint64)
        for i in range(3):
            prep = O.tq_prepare_query(q[i], spec.perm, spec.signs1, spec.signs2)
            if hi > lo:
                ids, sc = O.tq_score_topk(codes[lo:hi], norms[lo:hi], 128, 4, spec.centroids, prep, k, id_base=lo)
                pad = k - len(ids)
                ids = np.concatenate([ids, -np.ones(pad, np.int64)])
                sc = np.concatenate([sc, np.full(pad, -np.inf, np.float32)])
                local[i] = D.encode_keys(ids, sc)
        gathered = [torch.zeros((3, k), dtype=torch.int64) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(local.view(np.int64)))
        allk = np.stack([g.numpy().view(np.uint64) for g in gathered])        # [world, 3, k]
        ok = True
        for i in range(3):
            ids, sc = D.decode_keys(allk[:, i, :].ravel())
            keep = ids >= 0
            mid, msc = O.topk_merge(ids[keep], sc[keep], k)
            prep = O.tq_prepare_query(q[i], spec.perm, spec.signs1, spec.signs2)
            rid, rsc = O.tq_score_topk(codes, norms, 128, 4, spec.centroids, prep, k)
            ok &= bool(np.array_equal(mid, rid) and np.array_equal(msc, rsc))
            # descending keys are exactly "score desc, id asc"
            srt = np.sort(allk[:, i, :].ravel())[::-1][:k]
            sid, _ = D.decode_keys(srt)
            ok &= bool(np.array_equal(sid[:len(rid)], rid) and (sid[len(rid):] == -1).all())
        ret[rank] = ok
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_total", [101, 7])
def test_sharded_topk_merge_world2(n_total):
    import torch.multiprocessing as mp
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    procs = [mp.get_context("spawn").Process(target=_worker, args=(r, 2, port, n_total, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert ret[0] and ret[1]


def test_bounds_and_key_round_trip():
    import eos_b200.dist as D
    assert [D.shard_bounds(10, 4, r) for r in range(4)] == [(0, 3), (3, 6), (6, 9), (9, 10)]
    assert [D.shard_bounds(2, 4, r) for r in range(4)] == [(0, 1), (1, 2), (2, 2), (2, 2)]
    assert sum(hi - lo for lo, hi in (D.batch_bounds(1024, 8, r) for r in range(8))) == 1024
    with pytest.raises(ValueError):
        D.shard_bounds(10, 2, 2)
    rng = np.random.default_rng(0)
    sc = np.concatenate([rng.standard_normal(50).astype(np.float32), [0.0, -0.0, np.float32(1e-38), -np.inf]])
    ids = rng.integers(0, 2 ** 31, size=sc.size)
    keys = D.encode_keys(ids, sc)
    rid, rsc = D.decode_keys(keys)
    assert np.array_equal(rid, ids) and np.array_equal(rsc.view(np.uint32), sc.astype(np.float32).view(np.uint32))
    # order: score descending, then id ascending
    a = D.encode_keys(np.array([5, 9]), np.array([1.0, 1.0], np.float32))
    assert a[0] > a[1]
    b = D.encode_keys(np.array([5, 9]), np.array([-2.0, -1.0], np.float32))
    assert b[1] > b[0]
    e_ids, e_sc = D.decode_keys(D.encode_keys(np.array([-1]), np.array([3.0], np.float32)))
    assert e_ids[0] == -1 and e_sc[0] == -np.inf


def test_batching_helpers_follow_the_reference():
    """buildMaskedTokenInputs (runtime/embedding_model.go:1457-1495), padPretrainedBERTBatchEncodings
    (pretrained_bert_retrieval_vector_export.go:615-646), buildTokenBatch (inference.go:323-339)."""
    import pytest
    from eos_b200 import batching
    tok, mask = batching.build_masked_token_inputs([[5, 6, 0, 0], [7], [8, 0, 9]], pad_id=0)
    assert tok.tolist() == [[5, 6, 0, 0], [7, 0, 0, 0], [8, 0, 9, 0]]
    assert mask.tolist() == [[1, 1, 0, 0], [1, 0, 0, 0], [1, 1, 1, 0]]   # trailing pads masked, inner pad kept
    with pytest.raises(ValueError):
        batching.build_masked_token_inputs([], 0)
    with pytest.raises(ValueError):
        batching.build_masked_token_inputs([[1], []], 0)
    ids, m, ty = batching.pad_bert_batch([[101, 7, 102], [101, 102]], [[1, 1, 1], [1, 1]], [[0, 0, 0], [0, 1]], 4, pad_id=9)
    assert ids.tolist() == [[101, 7, 102, 9], [101, 102, 9, 9]]
    assert m.tolist() == [[1, 1, 1, 0], [1, 1, 0, 0]] and ty.tolist() == [[0, 0, 0, 0], [0, 1, 0, 0]]
    with pytest.raises(ValueError):
        batching.pad_bert_batch([[1, 2, 3]], [[1, 1, 1]], [[0, 0, 0]], 2, 0)
    with pytest.raises(ValueError):
        batching.pad_bert_batch([[1, 2]], [[1]], [[0, 0]], 4, 0)
    assert batching.build_token_batch([[1, 2], [3, 4]]).tolist() == [[1, 2], [3, 4]]
    with pytest.raises(ValueError):
        batching.build_token_batch([[1, 2], [3]])


def test_split_by_length_balances_valid_tokens():
    from eos_b200 import batching
    rng = np.random.default_rng(0)
    lengths = rng.integers(64, 513, size=1024)
    for world in (1, 2, 4, 8):
        parts = batching.split_by_length(lengths, world)
        assert sorted(np.concatenate(parts).tolist()) == list(range(1024))
        tokens = [int(lengths[p].sum()) for p in parts]
        assert max(len(p) for p in parts) - min(len(p) for p in parts) <= 1
        assert max(tokens) - min(tokens) <= 0.01 * sum(tokens) / world + 512
        inv = np.argsort(np.concatenate(parts))
        assert (np.concatenate(parts)[inv] == np.arange(1024)).all()
