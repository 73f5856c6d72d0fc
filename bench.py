#!/usr/bin/env python3
"""Benchmark of the embed-and-score hot path.

    python bench.py --gpus N --steps K --warmup W            # this library on N B200s (torchrun for N > 1)
    python bench.py --impl reference --gpus N --steps K ...  # the CPU restatement of Eos's host path

One JSON line on rank 0.  Primary metric: q8 encoder embeddings/s on the 12-layer / T=512 configuration
(batch 1024 per GPU, uniform random tokens, lengths uniform 64..512, masked mean-pool + 768->768 head + L2;
random-init weights, synthetic tokens).  A step is one forward over the batch.  `value` has the inputs resident in
HBM; `e2e` goes through the host-buffer C-ABI call with the copies inside the timed region.  The TurboQuant
scoring workload (10M x 768 4-bit corpus, 4096 queries, top-100) is reported under "turboquant" in the same
line.  The CPU numbers come from oracle/ (the restatement of the reference's host loops), used here only as the
timed baseline.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ENC = dict(layers=12, hidden=768, heads=12, inter=3072, vocab=30522, max_pos=512, head_out=768)
ENC_BATCH, ENC_TOKENS, ENC_MIN_LEN = 1024, 512, 64
TQ = dict(dim=768, bits=4, corpus=10_000_000, queries=4096, k=100)
# DRAM traffic measured with ncu (dram__bytes_read.sum + dram__bytes_write.sum of one launch) on the small
# cases of eos_b200/profile_cases.py, per row of the launch; the summaries are under profiles/.
NCU_GEMM_DRAM_BYTES_PER_ROW = {"qkv": 157.73e6 / 32768, "attn_out": 122.71e6 / 32768, "ffn_up": 203.39e6 / 32768,
                               "ffn_down": 297.53e6 / 32768}
NCU_SCAN_DRAM_BYTES_PER_ROW = 780.13e6 / 2_000_000
NCU_TC_DRAM_BYTES_PER_ROW = {128: 493.16e6 / 1_250_000, 256: 494.45e6 / 1_250_000}  # profiles/tq_score_tc*_kernel_*.md


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "tflops": p["bf16_tflops_sustained"], "tflops_burst": p["bf16_tflops"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1400.0, "tflops_burst": 1590.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed regions run."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(prefix="clocks_", suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.gpu)], stdout=open(self.path, "w"),
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()  # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx.append(float(f[2]))
                    power.append(float(f[3]))
                except ValueError:
                    continue
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            # the samples under load are the ones with the highest power draw
            order = np.argsort(power)[len(power) // 2:]
            out.update(sm_mhz=float(np.median(np.array(sm)[order])), sm_max_mhz=float(max(mx)),
                       reasons=sorted(reasons), samples=len(sm), power_w_max=float(max(power)))
        return out


def dist_setup(n_gpus: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


# ------------------------------------------------------------------------------------------------ reference arm
def encoder_sample(n_seq: int, seed: int):
    """The first n_seq sequences of the seeded batch, padded to their own longest length (the reference pads a
    batch to its longest member, runtime/embedding_model.go:1457-1495)."""
    from eos_b200 import synth
    ids, mask, lengths = synth.make_batch(ENC_BATCH, ENC_TOKENS, ENC["vocab"], ENC_MIN_LEN, ENC_TOKENS, seed)
    t = int(lengths[:n_seq].max())
    return ids[:n_seq, :t].copy(), mask[:n_seq, :t].copy(), lengths[:n_seq]


def oracle_encoder_args(weights):
    from eos_b200 import synth
    return dict(tok=weights["token_embeddings"], pos=weights["position_embeddings"],
                typ=weights["token_type_embeddings"], emb_gamma=weights["embedding_ln_weight"],
                emb_beta=weights["embedding_ln_bias"],
                layer_weights=synth.dequantized_layer_weights(weights["layer_weights"]),
                heads=weights["num_attention_heads"], head_w=weights.get("head_weights"))


def time_oracle_encoder(oargs, n_seq: int, workers: int, steps: int, warmup: int, seed: int):
    from oracle import oracle as O
    ids, mask, lengths = encoder_sample(n_seq, seed)
    types = np.zeros_like(ids)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        time_oracle_encoder.last_output = O.bert_embedder(
            ids, mask, types, oargs["tok"], oargs["pos"], oargs["typ"], oargs["emb_gamma"], oargs["emb_beta"],
            oargs["layer_weights"], oargs["heads"], 1e-12, "masked_mean", head_w=oargs["head_w"], workers=workers)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    return n_seq * len(times) / sum(times), float(np.mean(times)), ids.shape[1], lengths


def run_reference(args, rank: int):
    if rank != 0:
        return
    from eos_b200 import synth
    cores = os.cpu_count() or 1
    weights = synth.make_q8_encoder(seed=301, **ENC)
    oargs = oracle_encoder_args(weights)
    # size the per-step sample so that warmup + steps stay within a few minutes
    rate1, t1, _, _ = time_oracle_encoder(oargs, 1, cores, 1, 0, 303)
    seconds_per_step = 150.0 / max(1, args.steps + args.warmup)
    n_seq = int(max(1, min(16, seconds_per_step / max(t1, 1e-3))))
    rate, t_step, t_len, lengths = time_oracle_encoder(oargs, n_seq, cores, args.steps, args.warmup, 303)
    sample = f"{n_seq} sequence(s) of the seeded batch padded to {t_len} tokens per step, all {cores} host threads"
    line = {
        "impl": "reference", "metric": "q8_encoder_embeddings_per_s_T512", "value": rate, "unit": "embeddings/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t_step * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64-accumulate/f32",
        "data": "synthetic", "config": dict(workload_config(args.gpus), weight_mode=args.weight_mode),
        "cpu_baseline": {"value": rate, "unit": "embeddings/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": rate, "unit": "embeddings/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(world: int) -> dict:
    return {"workload": "12-layer q8 encoder (BERT-base shape) D=768 heads=12 FFN=3072 vocab=30522, int8 per-channel "
                        "weights, f16 activations, fp32 accumulate; batch 1024 x T=512 per GPU, lengths uniform "
                        "64..512, masked mean-pool + 768->768 head + L2",
            "per_gpu_batch": ENC_BATCH, "global_batch": ENC_BATCH * world, "seq_len": ENC_TOKENS,
            "sharding": f"data-parallel x{world}: length-balanced slices of one seeded global batch, no collective on "
                        "the data path",
            "l2_policy": "inputs_larger_than_l2 (activations of one step exceed 126 MB many times over)"}


# ------------------------------------------------------------------------------------------------ this library
def run_ours(args, rank: int, world: int, local: int):
    import torch
    import torch.distributed as dist

    import eos_b200
    from eos_b200 import batching
    from eos_b200 import encoder as encoder_mod
    from eos_b200 import synth
    from eos_b200 import turboquant as tq

    torch.cuda.set_device(local)
    if world > 1:
        # NCCL writes its version banner to stdout when the communicator is created; stdout carries the one JSON
        # line only, so the banner goes to stderr
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    peaks = load_peaks()
    rt = eos_b200.Runtime(local)
    # an explicit stream: its handle is non-null, so the library launches on exactly the stream the timing
    # events are recorded on (a null handle would select the runtime's own stream)
    tstream = torch.cuda.Stream()
    torch.cuda.set_stream(tstream)
    stream = tstream.cuda_stream
    assert stream != 0
    K, W = args.steps, args.warmup

    # ------------------------------------------------------------------ encoder
    weights = synth.make_q8_encoder(seed=301, **ENC)
    wmode = encoder_mod.WEIGHTS_F16_RESIDENT if args.weight_mode == "f16_resident" else encoder_mod.WEIGHTS_Q8_SMEM_DEQUANT
    enc = eos_b200.BertEmbedder(rt, weight_mode=wmode, **weights)
    # one seeded global batch of 1024 x world sequences; ranks take length-balanced slices of it (sequences are
    # independent, so the split needs no collective and every rank sees nearly the same number of valid tokens)
    g_ids, g_mask, g_lengths = synth.make_batch(ENC_BATCH * world, ENC_TOKENS, ENC["vocab"], ENC_MIN_LEN, ENC_TOKENS, 303)
    rows = batching.split_by_length(g_lengths, world)[rank]
    ids, mask, lengths = np.ascontiguousarray(g_ids[rows]), np.ascontiguousarray(g_mask[rows]), g_lengths[rows]
    del g_ids, g_mask
    enc.reserve(ENC_BATCH, ENC_TOKENS)
    d_ids, d_mask = torch.from_numpy(ids).cuda(), torch.from_numpy(mask).cuda()
    d_out = torch.empty((ENC_BATCH, ENC["head_out"]), dtype=torch.float32, device="cuda")
    flops_total = synth.encoder_flops(lengths, ENC["layers"], ENC["hidden"], ENC["inter"], ENC["head_out"])
    flops_gemm = synth.gemm_flops(lengths, ENC["layers"], ENC["hidden"], ENC["inter"])

    def forward():
        return enc.run_device(d_ids.data_ptr(), d_mask.data_ptr(), None, ENC_BATCH, ENC_TOKENS, d_out.data_ptr(), stream)

    for _ in range(W):
        forward()
    enc.sync(stream)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    prof_steps = min(K, 4)
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    launches = 0
    for i in range(K):
        if i == K - prof_steps:
            enc.profile_begin(prof_steps)  # event pairs around every launch of the last steps
        launches += forward()
    ev1.record()
    barrier()
    enc.sync(stream)
    times = enc.profile_end(stream)
    ms_total = max_over_ranks(ev0.elapsed_time(ev1))
    ms_step = ms_total / K
    value = ENC_BATCH * world * K / (ms_total / 1e3)

    # ------------------------------------------------------------------ encoder, end to end (host buffers)
    h_ids = torch.from_numpy(ids).pin_memory().numpy()
    h_mask = torch.from_numpy(mask).pin_memory().numpy()
    enc.run(h_ids, h_mask)
    barrier()
    t0 = time.perf_counter()
    for _ in range(K):
        out_host = enc.run(h_ids, h_mask)
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    e2e_value = ENC_BATCH * world * K / e2e_s
    clocks = sampler.stop() if rank == 0 else {}
    # copied now: later calls on the same encoder (the self-check against the CPU port) reuse the stats object
    e2e_h2d, e2e_d2h = int(enc.last_stats.uploaded_bytes), int(enc.last_stats.downloaded_bytes)
    assert abs(float(np.linalg.norm(out_host[0])) - 1.0) < 1e-3

    gemm_ms_step = times.gemm_ms / max(1, times.steps)
    rows_step = int(lengths.sum())
    gemm_launches_step = times.gemm_launches // max(1, times.steps)
    # DRAM bytes per launch of the projection kernel: the ncu captures of the four projections of a layer
    # (dram__bytes_read.sum + dram__bytes_write.sum at 32768 rows, profiles/gemm_tc_kernel_*.md) scaled by
    # rows, averaged over the launches of a step; only quoted for the mode that was captured
    traffic = None
    if args.weight_mode == "f16_resident" and gemm_launches_step > 0:
        traffic = sum(NCU_GEMM_DRAM_BYTES_PER_ROW.values()) * ENC["layers"] * rows_step / gemm_launches_step
    roof = {
        "bound": "tensor",
        "kernel": "gemm_tc_kernel (q8 weights expanded to f16 at bind, scales in the fp32 epilogue)"
                  if args.weight_mode == "f16_resident" else "gemm_tc_kernel (8-bit weights dequantised in shared memory)",
        "achieved": flops_gemm / (gemm_ms_step / 1e3) / 1e12 if gemm_ms_step > 0 else None,
        "peak": peaks["tflops"], "unit": "TFLOP/s", "peak_source": f"{peaks['source']} (sustained cuBLAS bf16)",
        "traffic": traffic,
        "launches_per_step": gemm_launches_step,
        "avg_launch_ms": times.gemm_ms / max(1, times.gemm_launches),
        "per_step_ms": {"gemm": gemm_ms_step, "attention": times.attention_ms / max(1, times.steps),
                        "layernorm": times.layernorm_ms / max(1, times.steps),
                        "embed": times.embed_ms / max(1, times.steps), "pool": times.pool_ms / max(1, times.steps),
                        "layout": times.layout_ms / max(1, times.steps),
                        "gemm_qkv": times.gemm_kind_ms[0] / max(1, times.steps),
                        "gemm_attn_out": times.gemm_kind_ms[1] / max(1, times.steps),
                        "gemm_ffn_up": times.gemm_kind_ms[2] / max(1, times.steps),
                        "gemm_ffn_down": times.gemm_kind_ms[3] / max(1, times.steps)},
        "whole_step_tflops": flops_total / (ms_step / 1e3) / 1e12,
        "algorithmic_flops_per_step": flops_total, "gemm_flops_per_step": flops_gemm,
    }
    roof["frac"] = roof["achieved"] / roof["peak"] if roof["achieved"] else None

    # ------------------------------------------------------------------ CPU baseline (rank 0, one GPU only)
    cpu = None
    if rank == 0 and world == 1 and not args.skip_cpu:
        cores = os.cpu_count() or 1
        oargs = oracle_encoder_args(weights)
        _, t1, _, _ = time_oracle_encoder(oargs, 1, cores, 1, 0, 303)
        n_seq = int(max(1, min(8, 12.0 / max(t1, 1e-3))))
        rate, _, t_len, _ = time_oracle_encoder(oargs, n_seq, cores, 1, 0, 303)
        # outside every timed region: the GPU's embeddings of those same sequences against the CPU port's
        s_ids, s_mask, _ = encoder_sample(n_seq, 303)
        gpu_sample = enc.run(s_ids, s_mask)
        check_err = float(np.abs(gpu_sample - time_oracle_encoder.last_output).max())
        assert check_err <= 2e-3, f"encoder output differs from the CPU port by {check_err}"
        cpu = {"value": rate, "unit": "embeddings/s", "cores": cores, "kind": "port",
               "sample": f"{n_seq} sequence(s) of the seeded batch padded to {t_len} tokens, all {cores} host threads, "
                         "one pass",
               "gpu_vs_port_max_abs": check_err}
        del oargs
    # ------------------------------------------------------------------ the same encoder under strong scaling
    # configuration 3 words it as "batch 1024 ... sharded across 1/2/4/8 GPUs": one global batch of 1024 sequences,
    # 1024 / N per rank (length-balanced slices, no collective); reported beside the weak-scaling headline
    strong = None
    if world > 1:
        s_ids, s_mask, s_len = synth.make_batch(ENC_BATCH, ENC_TOKENS, ENC["vocab"], ENC_MIN_LEN, ENC_TOKENS, 303)
        rows_s = batching.split_by_length(s_len, world)[rank]
        nb = len(rows_s)
        ds_ids = torch.from_numpy(np.ascontiguousarray(s_ids[rows_s])).cuda()
        ds_mask = torch.from_numpy(np.ascontiguousarray(s_mask[rows_s])).cuda()
        for _ in range(3):
            enc.run_device(ds_ids.data_ptr(), ds_mask.data_ptr(), None, nb, ENC_TOKENS, d_out.data_ptr(), stream)
        enc.sync(stream)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(K):
            launches += enc.run_device(ds_ids.data_ptr(), ds_mask.data_ptr(), None, nb, ENC_TOKENS, d_out.data_ptr(), stream)
        e1.record()
        barrier()
        enc.sync(stream)
        ms_s = max_over_ranks(e0.elapsed_time(e1)) / K
        strong = {"scaling": "strong", "global_batch": ENC_BATCH, "per_gpu_batch": nb, "value": ENC_BATCH / (ms_s / 1e3),
                  "unit": "embeddings/s", "ms_per_step": ms_s, "steps": K}
        del ds_ids, ds_mask
    enc.close()
    # ------------------------------------------------------------------ configurations 1 and 2 (one GPU, rank 0's device)
    small = None
    if not args.skip_small_configs:
        small = run_small_configs(rt, stream, peaks, K)
        launches += small.pop("_launches", 0)
    # the other weight mode, timed the same way on fewer steps (reported beside the headline, not as it)
    other = None
    if not args.skip_other_mode:
        omode = (encoder_mod.WEIGHTS_Q8_SMEM_DEQUANT if args.weight_mode == "f16_resident"
                 else encoder_mod.WEIGHTS_F16_RESIDENT)
        enc2 = eos_b200.BertEmbedder(rt, weight_mode=omode, **weights)
        for _ in range(3):
            enc2.run_device(d_ids.data_ptr(), d_mask.data_ptr(), None, ENC_BATCH, ENC_TOKENS, d_out.data_ptr(), stream)
        enc2.sync(stream)
        k2 = min(K, 5)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(k2):
            launches += enc2.run_device(d_ids.data_ptr(), d_mask.data_ptr(), None, ENC_BATCH, ENC_TOKENS,
                                        d_out.data_ptr(), stream)
        e1.record()
        barrier()
        enc2.sync(stream)
        ms2 = max_over_ranks(e0.elapsed_time(e1)) / k2
        other = {"weight_mode": "q8_smem_dequant" if args.weight_mode == "f16_resident" else "f16_resident",
                 "value": ENC_BATCH * world / (ms2 / 1e3), "unit": "embeddings/s", "ms_per_step": ms2, "steps": k2}
        enc2.close()
    del d_ids, d_mask, d_out
    torch.cuda.empty_cache()

    # ------------------------------------------------------------------ TurboQuant scoring
    # N > 1: the library's own communicator (NCCL inside the C ABI); torch.distributed only carries the 128-byte id
    comm = None
    if world > 1:
        from eos_b200 import dist as edist
        id_t = torch.zeros((edist.NCCL_ID_BYTES,), dtype=torch.uint8, device="cuda")
        if rank == 0:
            id_t.copy_(torch.frombuffer(bytearray(edist.new_comm_id()), dtype=torch.uint8))
        dist.broadcast(id_t, src=0)
        comm = edist.Comm(rt, rank, world, bytes(id_t.cpu().numpy().tobytes()))
    tq_out = None
    if not args.skip_turboquant:
        tq_out = run_turboquant(args, rt, rank, world, stream, peaks, barrier, max_over_ranks, comm)
        launches += tq_out.pop("_launches", 0)
    lc_out = None
    if not args.skip_long_context:
        lc_out = run_long_context(args, rt, rank, world, stream, peaks, barrier, max_over_ranks, comm)
        launches += lc_out.pop("_launches", 0)
    if comm is not None:
        comm.close()

    if rank == 0:
        if clocks.get("sm_mhz"):   # time x clock: comparable between boxes whose power-capped clocks differ
            clocks["ms_per_step_x_sm_ghz"] = ms_step * clocks["sm_mhz"] / 1e3
        line = {
            "metric": "q8_encoder_embeddings_per_s_T512", "value": value, "unit": "embeddings/s", "n_gpus": world,
            "steps": K, "warmup": W, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16 x int8->f16, fp32 accumulate", "data": "synthetic",
            "config": dict(workload_config(world), weight_mode=args.weight_mode),
            "e2e": {"value": e2e_value, "unit": "embeddings/s", "h2d_bytes_per_step": e2e_h2d, "d2h_bytes_per_step": e2e_d2h},
            "gpu_launches": int(launches), "roofline": roof, "clocks": clocks,
            "valid_tokens_per_step": int(lengths.sum()),
        }
        if other is not None:
            line["other_weight_mode"] = other
        if strong is not None:
            line["encoder_strong_scaling"] = strong
        if small is not None:
            line["small_configs"] = small
        if cpu is not None:
            line["cpu_baseline"] = cpu
        if tq_out is not None:
            line["turboquant"] = tq_out
        if lc_out is not None:
            line["long_context_multivector"] = lc_out
        print(json.dumps(line), flush=True)
    rt.close()
    if world > 1:
        dist.destroy_process_group()


def run_small_configs(rt, stream, peaks, steps):
    """Configurations 1 and 2 of the benchmark list, per GPU (every rank runs them; rank 0's numbers are printed).
    C1: masked mean-pooled embed pipeline, table [30522, 384], batch 32 x 128, lengths 16..128: microseconds per batch
    through the host-buffer call (its device time from the call's own events beside it).
    C2: 4-layer q8 encoder D=384 / 6 heads / FFN 1536, batch 128 x 256, lengths 32..256: embeddings/s and TFLOP/s on
    valid tokens, inputs resident on the device."""
    import torch

    import eos_b200
    from eos_b200 import synth
    out = {}
    launches = 0
    rng = np.random.default_rng(101)
    table = synth.f16_round(rng.standard_normal((30522, 384), dtype=np.float32) * np.float32(0.02))
    proj = synth.f16_round(rng.standard_normal((384, 384), dtype=np.float32) * np.float32(0.05))
    tokens, mask, _ = synth.make_batch(32, 128, 30522, 16, 128, seed=102)
    pipe = eos_b200.EmbedPooledPipeline(rt, table, proj)
    for _ in range(5):
        pipe.run(tokens, mask)
    reps = max(20, steps * 5)
    dev_ms = 0.0
    t0 = time.perf_counter()
    for _ in range(reps):
        pipe.run(tokens, mask)
        dev_ms += pipe.last_stats.device_ms
    wall_us = (time.perf_counter() - t0) / reps * 1e6
    launches += reps
    st = pipe.last_stats
    out["c1_embed_pooled"] = {
        "workload": "gather [30522,384] f16 -> projection [384,384] -> per-token L2 -> masked mean, batch 32 x 128",
        "us_per_batch_e2e": wall_us, "us_per_batch_device": dev_ms / reps * 1e3, "batches_per_s": 1e6 / wall_us,
        "h2d_bytes_per_step": int(st.uploaded_bytes), "d2h_bytes_per_step": int(st.downloaded_bytes),
        "kernel_launches_per_batch": int(st.kernel_launches), "reps": reps}
    pipe.close()
    c2 = dict(layers=4, hidden=384, heads=6, inter=1536, vocab=30522, max_pos=512)
    w2 = synth.make_q8_encoder(seed=201, **c2)
    enc2 = eos_b200.BertEmbedder(rt, **w2)
    ids2, mask2, len2 = synth.make_batch(128, 256, 30522, 32, 256, seed=202)
    d_ids2, d_mask2 = torch.from_numpy(ids2).cuda(), torch.from_numpy(mask2).cuda()
    d_out2 = torch.empty((128, 384), dtype=torch.float32, device="cuda")
    for _ in range(5):
        enc2.run_device(d_ids2.data_ptr(), d_mask2.data_ptr(), None, 128, 256, d_out2.data_ptr(), stream)
    enc2.sync(stream)
    reps2 = max(20, steps * 5)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps2):
        launches += enc2.run_device(d_ids2.data_ptr(), d_mask2.data_ptr(), None, 128, 256, d_out2.data_ptr(), stream)
    e1.record()
    enc2.sync(stream)
    ms2 = e0.elapsed_time(e1) / reps2
    fl2 = synth.encoder_flops(len2, 4, 384, 1536)
    out["c2_encoder_4layer"] = {
        "workload": "4-layer q8 encoder D=384 heads=6 FFN=1536, batch 128 x T=256, lengths 32..256, masked mean + L2",
        "ms_per_batch": ms2, "embeddings_per_s": 128 / (ms2 / 1e3), "tflops_valid_tokens": fl2 / (ms2 / 1e3) / 1e12,
        "frac_of_sustained_tensor_peak": fl2 / (ms2 / 1e3) / 1e12 / peaks["tflops"], "valid_tokens": int(len2.sum()),
        "reps": reps2, "note": "3.2 GFLOP per batch: launch- and latency-bound (35 launches per forward), not tensor-bound"}
    enc2.close()
    out["_launches"] = launches
    return out


LC = dict(layers=6, hidden=512, heads=8, inter=2048, vocab=30522, max_pos=8192, tokens=8192, window=512, batch=16,
          token_dim=128, bits=2, docs=100_000, children=128, queries=256, query_tokens=32, k=100)


def run_long_context(args, rt, rank, world, stream, peaks, barrier, max_over_ranks, comm):
    """Configuration 5.  (a) Document side: 6-layer q8 encoder D=512 / 8 heads / FFN 2048 with a 512-token local
    window over 16 sequences of 8192 tokens -> 128-d L2-normalised per-token vectors -> 2-bit TurboQuant packing,
    per GPU (every rank encodes its own batch of 16: weak scaling, like the headline).  (b) Query side: late
    interaction of 256 queries x 32 token vectors against 100k documents x 128 packed vectors, documents sharded
    over the GPUs, per-shard parent lists merged through the library's communicator."""
    import torch

    import eos_b200
    from eos_b200 import synth
    from eos_b200 import turboquant as tq
    c = LC
    launches = 0
    # ---- (a) documents -> per-token vectors -> packed codes
    w = synth.make_q8_encoder(c["layers"], c["hidden"], c["heads"], c["inter"], vocab=c["vocab"], max_pos=c["max_pos"],
                              seed=501)
    enc = eos_b200.BertEmbedder(rt, attention_window=c["window"], **w)
    rng = np.random.default_rng(502)
    enc.set_token_head(synth.f16_round(rng.standard_normal((c["hidden"], c["token_dim"]), dtype=np.float32) * np.float32(0.05)))
    B, T = c["batch"], c["tokens"]
    ids = torch.from_numpy(rng.integers(0, c["vocab"], size=(B, T), dtype=np.int32)).cuda()
    mask = torch.ones((B, T), dtype=torch.int32, device="cuda")
    vec = torch.empty((B * T, c["token_dim"]), dtype=torch.float32, device="cuda")
    spec = eos_b200.make_rotation_spec(c["token_dim"], c["bits"], seed=402)
    qz = eos_b200.Quantizer(rt, spec)
    dcodes = torch.empty((B * T, spec.code_bytes), dtype=torch.uint8, device="cuda")
    dnorms = torch.empty((B * T,), dtype=torch.float32, device="cuda")

    def encode_step():
        n = enc.token_vectors_device(ids.data_ptr(), mask.data_ptr(), None, B, T, vec.data_ptr(), None, stream)
        qz.quantize_device(vec.data_ptr(), B * T, dcodes.data_ptr(), dnorms.data_ptr(), stream)
        return n + 1

    for _ in range(3):
        encode_step()
    enc.sync(stream)
    steps = max(1, min(args.steps, 10))
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        launches += encode_step()
    e1.record()
    barrier()
    enc.sync(stream)
    enc_ms = max_over_ranks(e0.elapsed_time(e1)) / steps
    D, F, L, W = c["hidden"], c["inter"], c["layers"], c["window"]
    flops_seq = T * L * (2.0 * (4 * D * D + 2 * D * F) + 4.0 * W * D) + 2.0 * T * D * c["token_dim"]
    enc_out = {"ms_per_batch": enc_ms, "sequences_per_s": B * world / (enc_ms / 1e3),
               "tokens_per_s": B * T * world / (enc_ms / 1e3), "tflops": B * flops_seq / (enc_ms / 1e3) / 1e12,
               "frac_of_sustained_tensor_peak": B * flops_seq / (enc_ms / 1e3) / 1e12 / peaks["tflops"],
               "algorithmic_gflop_per_sequence": flops_seq / 1e9, "per_gpu_batch": B, "steps": steps,
               "includes": "per-token head, L2 normalisation and 2-bit packing of 131072 vectors"}
    vnorm = float(torch.linalg.norm(vec[:64], dim=1).mean().item())
    assert abs(vnorm - 1.0) < 1e-2, vnorm
    enc.close()
    del vec, dcodes, dnorms, ids, mask
    torch.cuda.empty_cache()
    # ---- (b) late interaction over the sharded document set (synthetic unit-Gaussian child vectors)
    docs, ch = c["docs"], c["children"]
    shard = (docs + world - 1) // world
    lo = min(docs, rank * shard)
    n_docs = max(0, min(docs, lo + shard) - lo)
    n_child = n_docs * ch
    codes = torch.empty((max(1, n_child), spec.code_bytes), dtype=torch.uint8, device="cuda")
    norms = torch.empty((max(1, n_child),), dtype=torch.float32, device="cuda")
    chunk = 2_000_000
    xbuf = torch.empty((min(chunk, max(1, n_child)), c["token_dim"]), dtype=torch.float32, device="cuda")
    for c0 in range(0, n_child, chunk):
        c1 = min(n_child, c0 + chunk)
        tq.synth_gaussian_device(rt, 503, lo * ch + c0, c1 - c0, c["token_dim"], True, xbuf.data_ptr(), stream)
        qz.quantize_device(xbuf.data_ptr(), c1 - c0, codes[c0:].data_ptr(), norms[c0:].data_ptr(), stream)
    torch.cuda.synchronize()
    corpus = eos_b200.Corpus(qz, device_ptrs=(codes.data_ptr(), norms.data_ptr(), n_child), id_base=lo * ch)
    del xbuf
    nq, qt, k = c["queries"], c["query_tokens"], c["k"]
    queries = torch.empty((nq * qt, c["token_dim"]), dtype=torch.float32, device="cuda")
    tq.synth_gaussian_device(rt, 504, 0, nq * qt, c["token_dim"], True, queries.data_ptr(), stream)
    queries = queries.half().float().contiguous()
    out_ids = torch.empty((nq, k), dtype=torch.int64, device="cuda")
    out_sc = torch.empty((nq, k), dtype=torch.float32, device="cuda")
    keys = torch.empty((nq, k), dtype=torch.int64, device="cuda")

    def score_step():
        if world == 1:
            return corpus.maxsim_topk_device(queries.data_ptr(), nq * qt, qt, ch, k, out_ids.data_ptr(), out_sc.data_ptr(),
                                             None, stream)
        n = corpus.maxsim_topk_device(queries.data_ptr(), nq * qt, qt, ch, k, None, None, keys.data_ptr(), stream)
        comm.merge_keys(keys.data_ptr(), nq, k, out_ids.data_ptr(), out_sc.data_ptr(), stream)
        return n + 1

    for _ in range(2):
        score_step()
    corpus.sync(stream)
    barrier()
    corpus.profile_begin(steps * (nq * qt // 128) + 8)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        launches += score_step()
    e1.record()
    barrier()
    k_ms, k_launches = corpus.profile_end(stream)
    ms = max_over_ranks(e0.elapsed_time(e1)) / steps
    flops = 2.0 * nq * qt * docs * ch * c["token_dim"]
    dimp = (c["token_dim"] + 127) // 128 * 128
    k_flops = 2.0 * 128 * n_child * dimp
    k_avg = k_ms / max(1, k_launches)
    res = {"document_encoder": enc_out,
           "maxsim": {"ms_per_step": ms, "query_doc_pairs_per_s": nq * docs / (ms / 1e3), "tflops": flops / (ms / 1e3) / 1e12,
                      "scaling": "strong", "steps": steps,
                      "config": {"workload": f"{nq} queries x {qt} token vectors vs {docs} documents x {ch} vectors of "
                                             f"{c['token_dim']} dims at {c['bits']} bits, top-{k}; documents sharded over "
                                             f"{world} GPU(s)",
                                 "bytes_per_vector": spec.vector_bytes,
                                 "merge": "none" if world == 1 else "NCCL all-gather of per-shard parent lists + merge kernel "
                                                                    "(eos_b200_comm_merge_keys)"},
                      "roofline": {"bound": "tensor", "kernel": "tq_score_tc_kernel (late-interaction epilogue)",
                                   "achieved": k_flops / (k_avg / 1e3) / 1e12 if k_avg > 0 else None, "peak": peaks["tflops"],
                                   "unit": "TFLOP/s", "avg_launch_ms": k_avg, "launches_per_step": k_launches // max(1, steps),
                                   "algorithmic_flops_per_launch": k_flops,
                                   "frac": k_flops / (k_avg / 1e3) / 1e12 / peaks["tflops"] if k_avg > 0 else None,
                                   "traffic": None}},
           "_launches": launches}
    assert bool((out_ids[:, 0] >= 0).all().item()) and bool(torch.isfinite(out_sc).all().item())
    # outside the timed region: the fused kernel against the general parent aggregation (every child score written
    # out, then grouped by parent) on the first 2000 documents of this rank's shard, 4 queries
    if n_docs >= 2000:
        sub_docs, cq = 2000, 4
        sub = eos_b200.Corpus(qz, device_ptrs=(codes.data_ptr(), norms.data_ptr(), sub_docs * ch), id_base=0)
        s_ids = torch.empty((cq, k), dtype=torch.int64, device="cuda")
        s_sc = torch.empty((cq, k), dtype=torch.float32, device="cuda")
        sub.maxsim_topk_device(queries.data_ptr(), cq * qt, qt, ch, k, s_ids.data_ptr(), s_sc.data_ptr(), None, stream)
        sub.sync(stream)
        g_ids, g_sc = sub.parent_topk(np.repeat(np.arange(sub_docs, dtype=np.int32), ch), sub_docs,
                                      queries[:cq * qt].cpu().numpy(), k, query_group=qt)
        same = float((s_ids.cpu().numpy() == g_ids).mean())
        err = float(np.abs(s_sc.cpu().numpy() - g_sc).max() / np.abs(g_sc).max())
        assert same >= 0.98 and err <= 1e-4, f"late-interaction kernel and general aggregation disagree: {same}, {err}"
        res["maxsim"]["self_check"] = {"documents": sub_docs, "queries": cq, "ids_equal_fraction": same,
                                       "max_rel_score_diff": err, "against": "eos_b200_parent_topk (all child scores)"}
        sub.close()
    del codes
    corpus.close()
    qz.close()
    return res


def run_turboquant(args, rt, rank, world, stream, peaks, barrier, max_over_ranks, comm):
    import torch
    import torch.distributed as dist

    import eos_b200
    from eos_b200 import turboquant as tq

    dim, bits, k, nq = TQ["dim"], TQ["bits"], TQ["k"], TQ["queries"]
    n_total = args.tq_corpus
    per_pass = args.tq_queries_per_pass
    shard = (n_total + world - 1) // world
    lo = rank * shard
    n_local = max(0, min(n_total, lo + shard) - lo)
    spec = eos_b200.make_rotation_spec(dim, bits, seed=402)
    qz = eos_b200.Quantizer(rt, spec)
    codes = torch.empty((n_local, spec.code_bytes), dtype=torch.uint8, device="cuda")
    norms = torch.empty((n_local,), dtype=torch.float32, device="cuda")
    chunk = 1_000_000
    xbuf = torch.empty((min(chunk, n_local), dim), dtype=torch.float32, device="cuda")
    for c0 in range(0, n_local, chunk):
        c1 = min(n_local, c0 + chunk)
        tq.synth_gaussian_device(rt, 401, lo + c0, c1 - c0, dim, True, xbuf.data_ptr(), stream)
        qz.quantize_device(xbuf.data_ptr(), c1 - c0, codes[c0:].data_ptr(), norms[c0:].data_ptr(), stream)
    torch.cuda.synchronize()
    # the packer on its own: rows already on the device, one chunk re-packed (same bytes) under CUDA events
    pack_rows = min(chunk, n_local)
    pe0, pe1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    tq.synth_gaussian_device(rt, 401, lo, pack_rows, dim, True, xbuf.data_ptr(), stream)
    qz.quantize_device(xbuf.data_ptr(), pack_rows, codes.data_ptr(), norms.data_ptr(), stream)
    pe0.record()
    for _ in range(3):
        qz.quantize_device(xbuf.data_ptr(), pack_rows, codes.data_ptr(), norms.data_ptr(), stream)
    pe1.record()
    torch.cuda.synchronize()
    pack_ms = pe0.elapsed_time(pe1) / 3
    pack_bytes = dim * 4 + spec.vector_bytes
    pack = {"kernel": "tq_norms_kernel + tq_pack_kernel", "rows": pack_rows, "ms": pack_ms, "docs_per_s": pack_rows / (pack_ms / 1e3),
            "bound": "hbm", "algorithmic_bytes_per_vector": pack_bytes,
            "achieved_gbs": pack_rows * pack_bytes / (pack_ms / 1e3) / 1e9, "peak_gbs": peaks["hbm_gbs"],
            "frac": pack_rows * pack_bytes / (pack_ms / 1e3) / 1e9 / peaks["hbm_gbs"],
            "reference": "per-document q.Quantize loop, runtime/retrieval_turboquant.go:702-711 (host, one goroutine)"}
    corpus = eos_b200.Corpus(qz, device_ptrs=(codes.data_ptr(), norms.data_ptr(), n_local), id_base=lo)
    del xbuf, codes
    torch.cuda.empty_cache()
    queries = torch.empty((nq, dim), dtype=torch.float32, device="cuda")
    tq.synth_gaussian_device(rt, 403, 0, nq, dim, True, queries.data_ptr(), stream)
    queries = queries.half().float().contiguous()  # the configuration's queries are f16
    ids = torch.empty((nq, k), dtype=torch.int64, device="cuda")
    scores = torch.empty((nq, k), dtype=torch.float32, device="cuda")
    def measure(per_pass, steps, with_e2e):
        launches = 0

        def step():
            if world == 1:
                return corpus.score_topk_device(queries.data_ptr(), nq, k, per_pass, ids.data_ptr(), scores.data_ptr(), None,
                                                stream)
            # one C-ABI call per rank: seed slice -> all-gather of thresholds -> score -> all-gather of keys -> merge
            return corpus.score_topk_sharded(comm, queries.data_ptr(), nq, k, per_pass, ids.data_ptr(), scores.data_ptr(),
                                             stream)

        warm = max(1, min(args.warmup, 3))
        for _ in range(warm):
            step()
        barrier()
        passes = (nq + per_pass - 1) // per_pass
        corpus.profile_begin(passes * steps + 8)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(steps):
            launches += step()
        ev1.record()
        barrier()
        scan_ms, scan_launches = corpus.profile_end(stream)
        ms = max_over_ranks(ev0.elapsed_time(ev1)) / steps
        scored = float(nq) * n_total  # one vector scored = one (query, vector) inner product, as in the reference's loop
        # end to end: host queries in, host ids/scores out (single GPU); copies inside the timed region
        e2e = None
        if world == 1 and with_e2e:
            hq = queries.cpu().pin_memory().numpy()
            corpus.score_topk(hq[:64], k, per_pass)
            t0 = time.perf_counter()
            for _ in range(steps):
                h_ids, h_scores = corpus.score_topk(hq, k, per_pass)
            dt = (time.perf_counter() - t0) / steps
            st = corpus.last_stats
            e2e = {"value": scored / dt, "unit": "vectors/s", "h2d_bytes_per_step": int(st.uploaded_bytes),
                   "d2h_bytes_per_step": int(st.downloaded_bytes), "queries_per_s": nq / dt}
        bytes_per_vec = spec.vector_bytes
        scan_avg_ms = scan_ms / max(1, scan_launches)
        # a launch of the 256-query kernel walks the shard once per group of 256 queries (up to 4 groups per launch)
        passes_per_launch = passes * steps / max(1, scan_launches)
        achieved = (passes_per_launch * n_local * bytes_per_vec) / (scan_avg_ms / 1e3) / 1e9 if scan_avg_ms > 0 else None
        if per_pass >= 128:
            # the batch kernels are contractions on the tensor cores: 2 x queries x rows x padded dim flops per launch
            dimp = (dim + 127) // 128 * 128
            flops = 2.0 * per_pass * n_local * dimp * passes_per_launch
            tf = flops / (scan_avg_ms / 1e3) / 1e12 if scan_avg_ms > 0 else None
            roofline = {"bound": "tensor", "kernel": "tq_score_tc_kernel" if per_pass == 128 else "tq_score_tc256_kernel", "achieved": tf, "peak": peaks["tflops"],
                        "unit": "TFLOP/s", "frac": tf / peaks["tflops"] if tf else None,
                        "peak_source": f"{peaks['source']} (cuBLAS bf16, sustained)",
                        "traffic": n_local * NCU_TC_DRAM_BYTES_PER_ROW[per_pass] * passes_per_launch,
                        "shard_passes_per_launch": passes_per_launch,
                        "avg_launch_ms": scan_avg_ms, "algorithmic_flops_per_launch": flops,
                        "code_read_gbs": achieved}
        else:
            roofline = {"bound": "hbm",
                        "kernel": "tq_scan_stream_kernel" if per_pass == 8 else f"tq_scan_kernel<{per_pass // 8}>",
                        "achieved": achieved,
                        "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"] if achieved else None,
                        "peak_source": f"{peaks['source']} (copy bandwidth)",
                        # ncu DRAM traffic of one launch, scaled by rows (profiles/tq_scan_stream_kernel_*.md)
                        "traffic": n_local * NCU_SCAN_DRAM_BYTES_PER_ROW if per_pass == 8 else None,
                        "avg_launch_ms": scan_avg_ms, "algorithmic_bytes_per_launch": n_local * bytes_per_vec}
        res = {
            "metric": "turboquant_vectors_scored_per_s", "value": scored / (ms / 1e3), "unit": "vectors/s",
            "corpus_rows_streamed_per_s": float(passes) * n_total / (ms / 1e3), "ms_per_step": ms, "steps": steps,
            "scaling": "strong",
            "config": {"workload": f"TurboQuant 4-bit Hadamard/MSE, {n_total} x {dim} unit Gaussian corpus sharded over "
                                   f"{world} GPU(s), {nq} f16 queries, exact top-{k}, {per_pass} queries per corpus pass "
                                   f"({passes} passes); one vector scored = one (query, vector) inner product",
                       "bytes_per_vector": bytes_per_vec,
                       "merge": "none" if world == 1 else "NCCL all-gather of per-shard top-k + merge kernel",
                       "thresholds": "seeded per shard" if world == 1 or per_pass < 128 else
                                     f"each rank seeds its slice of the queries, NCCL all-gather of {nq} thresholds "
                                     "(eos_b200_score_topk_sharded)"},
            "roofline": roofline,
            "_launches": launches,
        }
        if e2e is not None:
            res["e2e"] = e2e
        return res

    steps = max(1, min(args.steps, args.tq_steps))
    sampler = ClockSampler(torch.cuda.current_device())
    if rank == 0:
        sampler.start()
    out = measure(per_pass, steps, True)
    out["pack"] = pack
    if rank == 0:
        out["clocks"] = sampler.stop()  # warm-up, timed steps and the end-to-end calls of the batch kernel
        if out["clocks"].get("sm_mhz"):   # time x clock: comparable between boxes whose power-capped clocks differ
            out["clocks"]["ms_per_step_x_sm_ghz"] = out["ms_per_step"] * out["clocks"]["sm_mhz"] / 1e3
    # outside the timed region: the job's result for the first 16 queries (ids / scores hold the last step's output,
    # merged over all shards) against the streaming scan of the same shards, merged the same way
    chk_q = 16
    batch_ids, batch_sc = ids[:chk_q].clone(), scores[:chk_q].clone()
    c_ids = torch.empty((chk_q, k), dtype=torch.int64, device="cuda")
    c_sc = torch.empty((chk_q, k), dtype=torch.float32, device="cuda")
    if world == 1:
        corpus.score_topk_device(queries.data_ptr(), chk_q, k, 8, c_ids.data_ptr(), c_sc.data_ptr(), None, stream)
    else:
        corpus.score_topk_sharded(comm, queries.data_ptr(), chk_q, k, 8, c_ids.data_ptr(), c_sc.data_ptr(), stream)
    corpus.sync(stream)
    same = float((batch_ids == c_ids).float().mean().item())
    sc_err = float(((batch_sc - c_sc).abs().max() / c_sc.abs().max()).item())
    assert same >= 0.99 and sc_err <= 1e-4, f"batch kernel and streaming scan disagree: ids {same}, scores {sc_err}"
    out["self_check"] = {"queries": chk_q, "ids_equal_fraction": same, "max_rel_score_diff": sc_err,
                         "against": "8-queries-per-pass streaming scan over the same shards"}
    if per_pass != 8 and not args.tq_skip_stream:
        # the 8-queries-per-pass streaming scan (the kernel small batches use) on the same shard: its HBM roofline
        st = measure(8, 1, False)
        out["stream_scan"] = {key: st[key] for key in ("value", "corpus_rows_streamed_per_s", "ms_per_step", "roofline")}
        out["_launches"] += st["_launches"]
    if rank == 0 and world == 1 and not args.skip_cpu:
        out["cpu_baseline"] = time_oracle_scoring(spec, rt, qz)
    corpus.close()
    qz.close()
    return out


def time_oracle_scoring(spec, rt, qz):
    """Per-query scoring loop + heap of the reference (single-threaded, as runtime/retrieval_turboquant.go:1306-1331
    runs it) on a bounded sample of the workload."""
    from oracle import oracle as O
    n, nq = 250_000, 8
    rng = np.random.default_rng(401)
    x = rng.standard_normal((n, spec.dim)).astype(np.float32)
    x /= np.linalg.norm(x, axis=1, keepdims=True)
    codes, norms = qz.quantize(x)  # packing is not what is timed
    q = rng.standard_normal((nq, spec.dim)).astype(np.float32)
    t0 = time.perf_counter()
    for i in range(nq):
        prep = O.tq_prepare_query(q[i], spec.perm, spec.signs1, spec.signs2)
        O.tq_score_topk(codes, norms, spec.dim, spec.bits, spec.centroids, prep, TQ["k"])
    dt = time.perf_counter() - t0
    return {"value": n * nq / dt, "unit": "vectors/s", "cores": 1, "kind": "port",
            "sample": f"{nq} queries x {n} packed vectors, one thread (the reference's scoring loop is serial)"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-cpu", action="store_true", help="omit the timed CPU baseline")
    ap.add_argument("--skip-turboquant", action="store_true", help="encoder only")
    ap.add_argument("--tq-corpus", type=int, default=TQ["corpus"])
    ap.add_argument("--tq-queries-per-pass", type=int, default=256, choices=[8, 16, 32, 128, 256],
                    help="128 = tensor-core batch kernel; 8 = streaming scan; 16 / 32 = the earlier register-blocked scan")
    ap.add_argument("--tq-skip-stream", action="store_true", help="do not also time the 8-queries-per-pass scan")
    ap.add_argument("--weight-mode", default="f16_resident", choices=["f16_resident", "q8_smem"],
                    help="how the projection kernel receives the 8-bit weights (results are bit-identical)")
    ap.add_argument("--skip-other-mode", action="store_true", help="do not also time the other weight mode")
    ap.add_argument("--skip-small-configs", action="store_true", help="do not also time configurations 1 and 2")
    ap.add_argument("--skip-long-context", action="store_true", help="do not also time configuration 5")
    ap.add_argument("--tq-steps", type=int, default=10)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank, world, local = dist_setup(args.gpus)
    if args.impl == "reference":
        run_reference(args, rank)
        return
    run_ours(args, rank, world, local)


if __name__ == "__main__":
    main()
