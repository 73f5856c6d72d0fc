"""eos_b200: the B200 (sm_100a) embed-and-score path of Eos behind its operator interfaces.

Host-side mirror of the reference's interfaces for this path; all compute happens in
libeos_b200.so (hand-written CUDA, C ABI in include/eos_b200.h).
"""
from ._lib import EosB200DeviceStatusError, EosB200Error, Stats
from .encoder import BertEmbedder, CompactEmbedder, EmbedPooledPipeline, Q8Weight, Q8WeightInOut, Runtime, linear
from .attention import plan_sparse_attention, sparse_attention, turbo_sparse_attention
from .token_pool import TokenPoolEncoder
from .turboquant import (Corpus, DenseIndex, IpCorpus, Quantizer, RotationSpec, lloyd_max_gaussian, make_rotation_spec,
                         norm_decode_log8, norm_encode_log8)

__all__ = [
    "BertEmbedder", "CompactEmbedder", "Corpus", "DenseIndex", "EmbedPooledPipeline", "EosB200DeviceStatusError",
    "EosB200Error", "IpCorpus", "Q8Weight", "Q8WeightInOut", "Quantizer", "RotationSpec", "Runtime", "Stats", "TokenPoolEncoder", "linear",
    "lloyd_max_gaussian", "make_rotation_spec", "norm_decode_log8", "norm_encode_log8", "plan_sparse_attention",
    "sparse_attention", "turbo_sparse_attention",
]
