"""eos_b200: the B200 (sm_100a) embed-and-score path of Eos behind its operator interfaces.

Host-side mirror of the reference's interfaces for this path; all compute happens in
libeos_b200.so (hand-written CUDA, C ABI in include/eos_b200.h).
"""
from ._lib import EosB200DeviceStatusError, EosB200Error, Stats
from .encoder import BertEmbedder, EmbedPooledPipeline, Q8Weight, Runtime, linear
from .turboquant import Corpus, DenseIndex, Quantizer, RotationSpec, lloyd_max_gaussian, make_rotation_spec

__all__ = [
    "BertEmbedder", "Corpus", "DenseIndex", "EmbedPooledPipeline", "EosB200DeviceStatusError", "EosB200Error", "Q8Weight",
    "Quantizer", "RotationSpec", "Runtime", "Stats", "linear", "lloyd_max_gaussian", "make_rotation_spec",
]
