"""Shared helpers for the tests: golden fixture loading."""
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_bert_fixture(name):
    z = np.load(os.path.join(GOLDEN, name))
    layers = int(z["layers"])
    weights = [z[f"l{l}_{i:02d}"] for l in range(layers) for i in range(16)]
    return z, weights


def cosine_rows(a, b):
    num = (a * b).sum(-1)
    den = np.linalg.norm(a, axis=-1) * np.linalg.norm(b, axis=-1)
    return num / np.maximum(den, 1e-30)
