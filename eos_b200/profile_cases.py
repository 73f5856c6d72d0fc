"""Small, self-contained launches of single kernels, sized for profiler captures that end by themselves.

    python -m eos_b200.profile_cases gemm        # projection kernel, 32768 x 768 -> 3072, erf-GELU epilogue
    python -m eos_b200.profile_cases gemm_res    # 32768 x 3072 -> 768 with residual epilogue
    python -m eos_b200.profile_cases layernorm   # two-layer forward over 512 sequences (capture layernorm_kernel)
    python -m eos_b200.profile_cases gemm_f16w / gemm_res_f16w / gemm_qkv_f16w / gemm_attn_out_f16w
                                                 # the four projections of a layer, weights resident as f16
    python -m eos_b200.profile_cases scan        # TurboQuant scan, 2,000,000 x 768 4-bit codes (776 MB), 8 / 16 / 32 queries per pass
    python -m eos_b200.profile_cases score_tc    # TurboQuant tensor-core batch scoring, 1,250,000 x 768 4-bit codes (485 MB), 512 queries
    python -m eos_b200.profile_cases attention   # 2-layer encoder forward, 128 x 512 tokens (attention + LN kernels)

Each case touches more than the 126 MB L2 but holds well under a few GB on the device.
"""
from __future__ import annotations

import sys

import numpy as np


def case_gemm(residual: bool = False, weight_mode: int = 0, rows: int = 32768, kn=None, epilogue=None) -> None:
    import eos_b200
    from eos_b200 import synth
    rt = eos_b200.Runtime(0)
    rng = np.random.default_rng(0)
    k, n = kn if kn is not None else ((3072, 768) if residual else (768, 3072))
    x = rng.standard_normal((rows, k), dtype=np.float32)
    w = synth.quantize_per_channel(rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))
    bias = (rng.standard_normal(n) * 0.02).astype(np.float32)
    res = rng.standard_normal((rows, n), dtype=np.float32) if residual else None
    for _ in range(3):
        st = eos_b200.Stats()
        epi = epilogue if epilogue is not None else (2 if residual else 1)
        eos_b200.linear(rt, x, w, bias, epilogue=epi, residual=res, weight_mode=weight_mode, stats=st)
        print(f"gemm {rows}x{k}->{n} weight_mode={weight_mode}: {st.device_ms:.3f} ms, {2.0 * rows * k * n / st.device_ms / 1e9:.1f} TFLOP/s")
    rt.close()


def case_scan(n: int = 2_000_000) -> None:
    import torch

    import eos_b200
    from eos_b200 import turboquant as tq
    rt = eos_b200.Runtime(0)
    spec = eos_b200.make_rotation_spec(768, 4, seed=402)
    qz = eos_b200.Quantizer(rt, spec)
    chunk = 500_000
    x = torch.empty((chunk, 768), dtype=torch.float32, device="cuda")
    codes = torch.empty((n, 384), dtype=torch.uint8, device="cuda")
    norms = torch.empty((n,), dtype=torch.float32, device="cuda")
    for c0 in range(0, n, chunk):
        c1 = min(n, c0 + chunk)
        tq.synth_gaussian_device(rt, 401, c0, c1 - c0, 768, True, x.data_ptr())
        qz.quantize_device(x.data_ptr(), c1 - c0, codes[c0:].data_ptr(), norms[c0:].data_ptr())
    torch.cuda.synchronize()
    corpus = eos_b200.Corpus(qz, device_ptrs=(codes.data_ptr(), norms.data_ptr(), n))
    q = x[:64].cpu().numpy()
    del x, codes
    torch.cuda.empty_cache()
    for per_pass in (8, 16, 32):
        corpus.score_topk(q, 100, queries_per_pass=per_pass)
        corpus.profile_begin(64)
        corpus.score_topk(q, 100, queries_per_pass=per_pass)
        ms, launches = corpus.profile_end()
        print(f"scan {n} rows, {per_pass} queries/pass: {ms / launches:.3f} ms per pass, "
              f"{n * spec.vector_bytes / (ms / launches) / 1e6:.0f} GB/s")
    corpus.close()
    qz.close()
    rt.close()


def case_score_tc(n: int = 1_250_000, nq: int = 512, per_pass: int = 128) -> None:
    import torch

    import eos_b200
    from eos_b200 import turboquant as tq
    rt = eos_b200.Runtime(0)
    spec = eos_b200.make_rotation_spec(768, 4, seed=402)
    qz = eos_b200.Quantizer(rt, spec)
    chunk = 250_000
    x = torch.empty((chunk, 768), dtype=torch.float32, device="cuda")
    codes = torch.empty((n, 384), dtype=torch.uint8, device="cuda")
    norms = torch.empty((n,), dtype=torch.float32, device="cuda")
    for c0 in range(0, n, chunk):
        c1 = min(n, c0 + chunk)
        tq.synth_gaussian_device(rt, 401, c0, c1 - c0, 768, True, x.data_ptr())
        qz.quantize_device(x.data_ptr(), c1 - c0, codes[c0:].data_ptr(), norms[c0:].data_ptr())
    torch.cuda.synchronize()
    corpus = eos_b200.Corpus(qz, device_ptrs=(codes.data_ptr(), norms.data_ptr(), n))
    queries = torch.empty((nq, 768), dtype=torch.float32, device="cuda")
    tq.synth_gaussian_device(rt, 403, 0, nq, 768, True, queries.data_ptr())
    ids = torch.empty((nq, 100), dtype=torch.int64, device="cuda")
    scores = torch.empty((nq, 100), dtype=torch.float32, device="cuda")
    del x, codes
    torch.cuda.empty_cache()
    ts = torch.cuda.Stream()
    stream = ts.cuda_stream
    for _ in range(2):
        corpus.score_topk_device(queries.data_ptr(), nq, 100, per_pass, ids.data_ptr(), scores.data_ptr(), None, stream)
    torch.cuda.synchronize()
    corpus.profile_begin(64)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(ts)
    corpus.score_topk_device(queries.data_ptr(), nq, 100, per_pass, ids.data_ptr(), scores.data_ptr(), None, stream)
    e1.record(ts)
    torch.cuda.synchronize()
    ms, launches = corpus.profile_end(stream)
    print(f"score_tc {n} rows x {nq} queries: {e0.elapsed_time(e1):.3f} ms in all, {ms / launches:.3f} ms per main launch "
          f"({launches} launches of {per_pass} queries), {2.0 * per_pass * n * 768 / (ms / launches) / 1e9:.0f} TFLOP/s")
    corpus.close()
    qz.close()
    rt.close()


def case_attention(sequences: int = 128) -> None:
    import eos_b200
    from eos_b200 import synth
    rt = eos_b200.Runtime(0)
    args = synth.make_q8_encoder(2, 768, 12, 3072, vocab=30522, max_pos=512, seed=301)
    ids, mask, lengths = synth.make_batch(sequences, 512, 30522, 64, 512, seed=303)
    enc = eos_b200.BertEmbedder(rt, **args)
    for _ in range(2):
        enc.run(ids, mask)
    enc.profile_begin(1)
    enc.run(ids, mask)
    t = enc.profile_end()
    print(f"tokens {int(lengths.sum())}: gemm {t.gemm_ms:.3f} ms, attention {t.attention_ms:.3f} ms, "
          f"layernorm {t.layernorm_ms:.3f} ms")
    enc.close()
    rt.close()


def case_maxsim(docs: int = 20000, children: int = 128, dim: int = 128, bits: int = 2, nq: int = 16, qt: int = 32) -> None:
    """Late interaction: nq queries x qt token vectors against docs x children packed vectors, top-100 documents."""
    import torch
    import eos_b200
    from eos_b200 import turboquant as tq
    rt = eos_b200.Runtime(0)
    ts = torch.cuda.Stream()
    stream = ts.cuda_stream
    spec = eos_b200.make_rotation_spec(dim, bits, seed=402)
    qz = eos_b200.Quantizer(rt, spec)
    n = docs * children
    with torch.cuda.stream(ts):
        x = torch.empty((n, dim), dtype=torch.float32, device="cuda")
        codes = torch.empty((n, spec.code_bytes), dtype=torch.uint8, device="cuda")
        norms = torch.empty((n,), dtype=torch.float32, device="cuda")
        queries = torch.empty((nq * qt, dim), dtype=torch.float32, device="cuda")
        ids = torch.empty((nq, 100), dtype=torch.int64, device="cuda")
        scores = torch.empty((nq, 100), dtype=torch.float32, device="cuda")
    tq.synth_gaussian_device(rt, 503, 0, n, dim, True, x.data_ptr(), stream)
    tq.synth_gaussian_device(rt, 504, 0, nq * qt, dim, True, queries.data_ptr(), stream)
    qz.quantize_device(x.data_ptr(), n, codes.data_ptr(), norms.data_ptr(), stream)
    torch.cuda.synchronize()
    corpus = eos_b200.Corpus(qz, device_ptrs=(codes.data_ptr(), norms.data_ptr(), n))
    for _ in range(2):
        corpus.maxsim_topk_device(queries.data_ptr(), nq * qt, qt, children, 100, ids.data_ptr(), scores.data_ptr(), None, stream)
    corpus.sync(stream)
    corpus.profile_begin(64)
    corpus.maxsim_topk_device(queries.data_ptr(), nq * qt, qt, children, 100, ids.data_ptr(), scores.data_ptr(), None, stream)
    ms, launches = corpus.profile_end(stream)
    print(f"maxsim {docs} docs x {children} x {dim}d {bits}-bit, {nq} x {qt} query vectors: {ms / launches:.3f} ms per main "
          f"launch ({launches} launches), {2.0 * 128 * n * dim / (ms / launches) / 1e9:.0f} TFLOP/s")
    corpus.close()
    qz.close()
    rt.close()


def case_pack(n: int = 1_000_000, dim: int = 768, bits: int = 4) -> None:
    import torch
    import eos_b200
    from eos_b200 import turboquant as tq
    rt = eos_b200.Runtime(0)
    ts = torch.cuda.Stream()
    stream = ts.cuda_stream
    spec = eos_b200.make_rotation_spec(dim, bits, seed=402)
    qz = eos_b200.Quantizer(rt, spec)
    with torch.cuda.stream(ts):
        x = torch.empty((n, dim), dtype=torch.float32, device="cuda")
        codes = torch.empty((n, spec.code_bytes), dtype=torch.uint8, device="cuda")
        norms = torch.empty((n,), dtype=torch.float32, device="cuda")
    tq.synth_gaussian_device(rt, 503, 0, n, dim, True, x.data_ptr(), stream)
    for _ in range(2):
        qz.quantize_device(x.data_ptr(), n, codes.data_ptr(), norms.data_ptr(), stream)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(ts)
    qz.quantize_device(x.data_ptr(), n, codes.data_ptr(), norms.data_ptr(), stream)
    e1.record(ts)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    print(f"pack {n} x {dim} at {bits} bits: {ms:.3f} ms, {n / ms / 1e3:.1f} M vectors/s, "
          f"{n * (dim * 4 + spec.vector_bytes) / ms / 1e6:.0f} GB/s")
    qz.close()
    rt.close()


def case_sparse_attention(batches: int = 8, q_len: int = 2048, k_len: int = 8192, dim: int = 64, top_k: int = 64,
                          block: int = 64, top_blocks: int = 16) -> None:
    import numpy as np
    import eos_b200
    from eos_b200.attention import sparse_attention
    rt = eos_b200.Runtime(0)
    rng = np.random.default_rng(1)
    q = rng.standard_normal((batches, q_len, dim)).astype(np.float32)
    k = rng.standard_normal((batches, k_len, dim)).astype(np.float32)
    v = rng.standard_normal((batches, k_len, dim)).astype(np.float32)
    for rbs, rtb, name in ((0, 0, "exact"), (block, top_blocks, "block_anchor")):
        st = eos_b200.Stats()
        sparse_attention(rt, q, k, v, top_k, rbs, rtb)
        sparse_attention(rt, q, k, v, top_k, rbs, rtb, stats=st)
        print(f"sparse attention {name}: {batches} x {q_len} queries x {k_len} keys x {dim}d, top {top_k}: "
              f"{st.device_ms:.3f} ms incl. copies")
    rt.close()


if __name__ == "__main__":
    name = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    {"gemm": case_gemm, "gemm_res": lambda: case_gemm(True), "scan": case_scan, "score_tc": case_score_tc, "score_tc256": lambda: case_score_tc(per_pass=256), "attention": case_attention,
     "layernorm": lambda: case_attention(512),   # the same two-layer forward at 512 sequences: rows larger than L2
     "maxsim": case_maxsim, "pack": case_pack, "sparse_attention": case_sparse_attention,
     "gemm_f16w": lambda: case_gemm(False, 1), "gemm_res_f16w": lambda: case_gemm(True, 1),
     "gemm_big": lambda: case_gemm(False, 0, 131072), "gemm_res_big": lambda: case_gemm(True, 0, 131072),
     "gemm_big_f16w": lambda: case_gemm(False, 1, 131072),
     "gemm_qkv_f16w": lambda: case_gemm(False, 1, 32768, (768, 2304), 0),
     "gemm_attn_out_f16w": lambda: case_gemm(True, 1, 32768, (768, 768)),
     "gemm_attn_out_big_f16w": lambda: case_gemm(True, 1, 131072, (768, 768)), "gemm_res_big_f16w": lambda: case_gemm(True, 1, 131072),
     }[name]()
