"""CPU oracle (test infrastructure, not product code): the reference's per-tensor
fake-quantiser restated in numpy fp32.

Follows ``_tensor_quant`` / ``FakeTensorQuantFunction``
(lightseq/training/pytorch_quantization/tensor_quant.py:349-409, 328-346) and the
learned-amax ``Clip`` that precedes it in ``TensorQuantizer._quant_forward``
(lightseq/training/pytorch_quantization/nn/modules/tensor_quantizer.py:340-368):

    scale = amax / 127                (unsigned: amax / 254)
    q     = clamp(floor(x / scale + 0.5), -127, 127)     (unsigned: subtract 127 first)
    fake  = q * scale                 (unsigned: (q + 127) * scale)

Every operation is a separately rounded fp32 operation, as in torch. The same
formula is restated in the reference's own tests (tests/util.py:70-87,
tests/quant_test.py:24-33).

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import
this package.
"""
from __future__ import annotations

import numpy as np

F32 = np.float32
QMAX = F32(127.0)


def scale_of(amax, unsigned: bool = False) -> np.float32:
    """tensor_quant.py:384-386 — ``amax / max_bound`` (``/ (2*max_bound)`` if unsigned)."""
    amax = F32(amax)
    return F32(amax / F32(254.0)) if unsigned else F32(amax / QMAX)


def quantize(x: np.ndarray, amax, unsigned: bool = False, clip: bool = True):
    """Returns (q int8 in [-127,127], scale fp32). For ``unsigned`` the stored q means q+127."""
    x = np.asarray(x, dtype=F32)
    amax = F32(amax)
    s = scale_of(amax, unsigned)
    if clip:  # learned-amax quantisers clamp to +-amax first (clip.py:75-78); a no-op for the result
        x = np.clip(x, -amax, amax)
    t = x / s
    if unsigned:
        t = t - QMAX
    t = np.floor(t + F32(0.5))
    t = np.clip(t, -QMAX, QMAX)
    return t.astype(np.int8), s


def dequantize(q: np.ndarray, scale, unsigned: bool = False) -> np.ndarray:
    q = q.astype(F32)
    if unsigned:
        q = q + QMAX
    return q * F32(scale)


def fake_quant(x: np.ndarray, amax, unsigned: bool = False) -> np.ndarray:
    q, s = quantize(x, amax, unsigned)
    return dequantize(q, s, unsigned)


def int_matmul(a_q: np.ndarray, w_q: np.ndarray) -> np.ndarray:
    """Exact integer A[M,K] . W[N,K]^T via float64 BLAS (|sum| < 2^53, so every partial sum is exact)."""
    acc = a_q.astype(np.float64) @ w_q.astype(np.float64).T
    return acc.astype(np.int64)


def gelu(x: np.ndarray) -> np.ndarray:
    """Exact-erf GELU in fp32 (lightseq/training/ops/pytorch/util.py:15-16)."""
    from scipy.special import erf

    x = np.asarray(x, dtype=F32)
    inner = erf((x * F32(0.70710678118654752440)).astype(np.float64)).astype(F32)
    return (F32(0.5) * x) * (F32(1.0) + inner)
