"""GPU parity of the tensor-core projection (C ABI: eos_b200_linear) against float64 numpy on the same
f16-rounded inputs: y = epilogue(x W^T + b) with denseHF semantics
(runtime/backend/bert_encoder_layer_ops.go:452-462)."""
import math

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    import eos_b200
    r = eos_b200.Runtime(0)
    yield r
    r.close()


def _f16(a):
    return np.asarray(a, np.float32).astype(np.float16).astype(np.float32)


def _reference(x, w, bias, epilogue, residual):
    y = _f16(x).astype(np.float64) @ w.astype(np.float64).T
    if bias is not None:
        y = y + bias.astype(np.float64)
    if epilogue == 1:
        y = 0.5 * y * (1.0 + np.vectorize(math.erf)(y / math.sqrt(2.0)))
    elif epilogue == 3:
        y = 0.5 * y * (1.0 + np.tanh(0.7978845608028654 * (y + 0.044715 * y ** 3)))
    elif epilogue == 2:
        y = y + _f16(residual).astype(np.float64)
    return y


# (rows, in, out): tiny tiles, tails in every dimension, multi-tile M/N, long K
SHAPES = [(5, 16, 16), (300, 64, 48), (129, 96, 264), (1000, 768, 768), (257, 3072, 272), (4100, 384, 1152)]


@pytest.mark.parametrize("rows,k,n", SHAPES)
@pytest.mark.parametrize("weight_mode", [0, 1])
def test_linear_q8_matches_numpy(rt, rows, k, n, weight_mode):
    import eos_b200
    from eos_b200 import synth
    rng = np.random.default_rng(rows * 7 + k + n)
    x = rng.standard_normal((rows, k)).astype(np.float32)
    w = synth.quantize_per_channel((rng.standard_normal((n, k)) * 0.05).astype(np.float32))
    bias = (rng.standard_normal(n) * 0.1).astype(np.float32)
    y = eos_b200.linear(rt, x, w, bias, epilogue=0, weight_mode=weight_mode)
    ref = _reference(x, w.dequantized(), bias, 0, None)
    err = np.abs(y - ref)
    assert (err <= 1.5e-3 * np.abs(ref) + 1e-3).all(), float(err.max())


@pytest.mark.parametrize("epilogue", [1, 2, 3])
@pytest.mark.parametrize("weight_mode", [0, 1])
def test_linear_epilogues(rt, epilogue, weight_mode):
    import eos_b200
    from eos_b200 import synth
    rng = np.random.default_rng(epilogue)
    rows, k, n = 700, 256, 520
    x = rng.standard_normal((rows, k)).astype(np.float32)
    w = synth.quantize_per_channel((rng.standard_normal((n, k)) * 0.05).astype(np.float32))
    bias = (rng.standard_normal(n) * 0.1).astype(np.float32)
    res = rng.standard_normal((rows, n)).astype(np.float32) if epilogue == 2 else None
    y = eos_b200.linear(rt, x, w, bias, epilogue=epilogue, residual=res, weight_mode=weight_mode)
    ref = _reference(x, w.dequantized(), bias, epilogue, res)
    err = np.abs(y - ref)
    assert (err <= 1.5e-3 * np.abs(ref) + 1e-3).all(), float(err.max())


def test_linear_per_tensor_scale_and_dense_weights(rt):
    import eos_b200
    from oracle import oracle as O
    rng = np.random.default_rng(11)
    x = rng.standard_normal((200, 128)).astype(np.float32)
    wf = (rng.standard_normal((72, 128)) * 0.05).astype(np.float32)
    codes, scales = O.quantize_symmetric(wf)  # the reference's per-tensor rule
    y = eos_b200.linear(rt, x, eos_b200.Q8Weight(codes, scales), None)
    ref = _reference(x, O.dequantize(codes, scales), None, 0, None)
    assert (np.abs(y - ref) <= 1.5e-3 * np.abs(ref) + 1e-3).all()
    y = eos_b200.linear(rt, x, wf, None)
    ref = _reference(x, _f16(wf), None, 0, None)
    assert (np.abs(y - ref) <= 1.5e-3 * np.abs(ref) + 1e-3).all()
    # oracle's own dense (f64 accumulate) agrees too
    ref2 = O.dense_hf(_f16(x), _f16(wf), np.zeros(72, np.float32))
    assert (np.abs(y - ref2) <= 1.5e-3 * np.abs(ref2) + 1e-3).all()


def test_linear_from_packed_q8_payload(rt):
    """A packed q8 tensor payload + its tensor_scales entry (runtime/mll_export.go:902-949) binds as it is: the
    projection equals the one over the payload's decoded values."""
    import eos_b200
    from eos_b200 import formats
    rng = np.random.default_rng(12)
    x = rng.standard_normal((130, 96)).astype(np.float32)
    wf = (rng.standard_normal((40, 96)) * 0.07).astype(np.float32)
    raw, scale = formats.pack_quantized_tensor(wf, 8)
    weight = formats.q8_weight_from_payload(raw, wf.shape, scale)
    y = eos_b200.linear(rt, x, weight, None)
    ref = _reference(x, formats.decode_tensor_payload("q8", raw, wf.shape, scale), None, 0, None)
    assert (np.abs(y - ref) <= 1.5e-3 * np.abs(ref) + 1e-3).all()


def test_linear_rejects_bad_arguments(rt):
    import eos_b200
    x = np.zeros((4, 24), np.float32)
    with pytest.raises(eos_b200.EosB200Error):
        eos_b200.linear(rt, x, np.zeros((8, 24), np.float32))  # in width not a multiple of 16
    with pytest.raises(ValueError):
        eos_b200.linear(rt, x, np.zeros((8, 32), np.float32))


_PAIR_SCRIPT = r"""
import numpy as np, sys
import eos_b200
from eos_b200 import synth
rt = eos_b200.Runtime(0)
worst = 0.0
for rows, k, n, epi in ((5, 16, 16, 0), (129, 96, 264, 1), (1000, 768, 768, 2), (257, 3072, 272, 0), (4100, 384, 1152, 2),
                        (70000, 768, 768, 2)):
    rng = np.random.default_rng(rows + k + n)
    x = rng.standard_normal((rows, k)).astype(np.float32)
    w = synth.quantize_per_channel((rng.standard_normal((n, k)) * 0.05).astype(np.float32))
    bias = (rng.standard_normal(n) * 0.1).astype(np.float32)
    res = rng.standard_normal((rows, n)).astype(np.float32) if epi == 2 else None
    y1 = eos_b200.linear(rt, x, w, bias, epilogue=epi, residual=res, weight_mode=1)   # f16 weights: CTA pairs
    y0 = eos_b200.linear(rt, x, w, bias, epilogue=epi, residual=res, weight_mode=0)   # 8-bit weights: one CTA per tile
    if not np.array_equal(y0, y1):
        worst = max(worst, float(np.abs(y0 - y1).max()))
print("PAIR_RESULT", worst)
rt.close()
"""


def test_linear_cta_pair_mode_is_bit_identical():
    """The CTA-pair kernel (two CTAs of a cluster per 256 x 256 tile, tcgen05.mma.cta_group::2; by default it serves
    deep or wide projections, EOS_B200_GEMM_CTA_PAIR=1 makes it serve every f16-weight projection) must give exactly the bits of the
    one-CTA kernel: same products, same fp32
    accumulation order along K, same epilogue.  Runs in a child process because the mode is read once per process."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, EOS_B200_GEMM_CTA_PAIR="1", EOS_B200_DEBUG="1", PYTHONPATH=root)
    out = subprocess.run([sys.executable, "-c", _PAIR_SCRIPT], env=env, cwd=root, capture_output=True, text=True,
                         timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    assert "resident CTA pairs for the GEMM" in out.stderr and "pairs for the GEMM: 0" not in out.stderr, out.stderr[-500:]
    line = [l for l in out.stdout.splitlines() if l.startswith("PAIR_RESULT")][-1]
    assert float(line.split()[1]) == 0.0, line
