"""The allocation-free scoring entry point (eos_b200_score_topk_noalloc) against the regular one.

Some hosts cannot call cudaMalloc while they serve queries: they own the GPU through a pre-sized arena, lock
allocation after start-up, or cannot afford the device-wide stall an allocation may cause on a latency path.
For them the library keeps the scan's scratch (query fragments, per-CTA candidate lists, counts) in a fixed
__device__ array.  This file is collected last on purpose, so a failure here cannot hide other results.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_noalloc_scoring_matches_regular_entry_point_twice():
    import torch

    import eos_b200
    from oracle import oracle as O
    rt = eos_b200.Runtime(0)
    spec = eos_b200.make_rotation_spec(768, 4, seed=402)
    rng = np.random.default_rng(77)
    x = rng.standard_normal((5000, 768)).astype(np.float32)
    x /= np.linalg.norm(x, axis=1, keepdims=True)
    codes, norms = O.tq_encode(x, 4, spec.perm, spec.signs1, spec.signs2, spec.boundaries)
    qz = eos_b200.Quantizer(rt, spec)
    corpus = eos_b200.Corpus(qz, codes, norms, id_base=100)
    stream = torch.cuda.Stream()
    handle = stream.cuda_stream
    k = 100
    for call, nq in enumerate((20, 7)):          # two calls in a row share the scratch array
        q = rng.standard_normal((nq, 768)).astype(np.float32)
        dq = torch.from_numpy(q).cuda()
        torch.cuda.synchronize()
        ref_ids = torch.empty((nq, k), dtype=torch.int64, device="cuda")
        ref_sc = torch.empty((nq, k), dtype=torch.float32, device="cuda")
        corpus.score_topk_device(dq.data_ptr(), nq, k, 8, ref_ids.data_ptr(), ref_sc.data_ptr(), None, handle)
        stream.synchronize()
        ids = torch.full((nq, k), -7, dtype=torch.int64, device="cuda")
        sc = torch.zeros((nq, k), dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        corpus.score_topk_noalloc(dq.data_ptr(), nq, k, 8 if call == 0 else 16, ids.data_ptr(), sc.data_ptr(), handle)
        stream.synchronize()
        if call == 1:  # once the first call has loaded what the driver loads lazily, free memory does not move
            assert torch.cuda.mem_get_info()[0] == free_before
        # same kernels on the same inputs: the tolerance of the scoring tests (1e-3 relative) is met exactly
        assert torch.equal(ids, ref_ids)
        assert torch.equal(sc, ref_sc)
        host_ids, host_sc = corpus.score_topk(q, k)
        assert np.array_equal(ids.cpu().numpy(), host_ids)
    with pytest.raises(eos_b200.EosB200Error):   # beyond the fixed scratch: rejected, never truncated
        big = torch.zeros((33, 768), dtype=torch.float32, device="cuda")
        out_i = torch.empty((33, k), dtype=torch.int64, device="cuda")
        out_s = torch.empty((33, k), dtype=torch.float32, device="cuda")
        corpus.score_topk_noalloc(big.data_ptr(), 33, k, 8, out_i.data_ptr(), out_s.data_ptr(), handle)
    corpus.close()
    qz.close()
    rt.close()
