"""Known-answer cases restating the reference's own unit tests for the backend ops and
layers on the inference path (CpuBackendTest, LinearTest, RMSNorm1DTest,
RotaryEmbeddingTest, SiLUTest, MultiHeadSelfAttentionTest).  Every function uses the
process-wide `Tensor.backend()`, so the same cases pin the CPU oracle (not gpu) and the
CUDA runtime (gpu).  EPS follows the reference: 1e-6 for CPU literals.
"""
import math

import numpy as np
import pytest

from deepj_b200.layers import (HeadOps, Linear, MultiHeadSelfAttention, RMSNorm1D, RotaryEmbedding, SwiGLULayer,
                               TextGenerator)
from deepj_b200.tensor import Tensor

EPS = 1e-6


def eq(expected, t, eps=EPS):
    a = t.numpy() if isinstance(t, Tensor) else np.asarray(t)
    e = np.asarray(expected, dtype=np.float64)
    assert a.shape == e.shape, (a.shape, e.shape)
    assert np.all(np.abs(a - e) <= eps), (a, e)


A = [[1, 2, 3], [4, 5, 6]]


def case_matmul():                      # CpuBackendTest.java:85-102, MetalBackendTest.java:48-68
    eq([[58, 64], [139, 154]], Tensor.from2D(A).matmul(Tensor.from2D([[7, 8], [9, 10], [11, 12]])))
    with pytest.raises(ValueError):
        Tensor.from2D([[1, 2], [3, 4]]).matmul(Tensor.from2D([[1, 2, 3]]))


def case_causal_mask():                 # CpuBackendTest.java:72-81
    m = Tensor.causalMask(4).data
    for r in range(4):
        for c in range(4):
            assert m[r, c] == (np.float32(-1e9) if c > r else 0.0)


def case_elementwise():                 # CpuBackendTest.java add/subtract/multiply/divide
    a, b = Tensor.from2D([[1, 2], [3, 4]]), Tensor.from2D([[5, 6], [7, 8]])
    eq([[6, 8], [10, 12]], a.add(b))
    eq([[-4, -4], [-4, -4]], a.subtract(b))
    eq([[5, 12], [21, 32]], a.multiply(b))
    eq([[0.2, 1 / 3], [3 / 7, 0.5]], a.divide(b))
    with pytest.raises(ValueError):
        a.add(Tensor.from2D([[1, 2, 3]]))


def case_broadcasts():                  # CpuBackendTest.java:246-420
    a = Tensor.from2D(A)
    row, col = Tensor.from2D([[10, 20, 30]]), Tensor.from2D([[10], [20]])
    eq([[11, 22, 33], [14, 25, 36]], a.addRowVector(row))
    eq([[11, 22, 33], [14, 25, 36]], a.addBroadcastRows(row))
    eq([[10, 40, 90], [40, 100, 180]], a.multiplyBroadcastRows(row))
    eq([[11, 12, 13], [24, 25, 26]], a.addBroadcastCols(col))
    eq([[-9, -8, -7], [-16, -15, -14]], a.subtractBroadcastCols(col))
    eq([[10, 20, 30], [80, 100, 120]], a.multiplyBroadcastCols(col))
    eq([[0.1, 0.2, 0.3], [0.2, 0.25, 0.3]], a.divideBroadcastCols(col))
    bad = Tensor.from2D([[1, 2], [3, 4]])
    for f in (a.addRowVector, a.multiplyBroadcastRows, a.addBroadcastCols, a.divideBroadcastCols):
        with pytest.raises(ValueError):
            f(bad)


def case_scalars_and_unary():
    a = Tensor.from2D([[1, 4], [9, 16]])
    eq([[2, 8], [18, 32]], a.multiplyScalar(2.0))
    eq([[1.5, 4.5], [9.5, 16.5]], a.addScalar(0.5))
    eq([[0.5, 2], [4.5, 8]], a.divideScalar(2.0))
    eq([[1, 2], [3, 4]], a.sqrt())
    eq([[1, 16], [81, 256]], a.pow(2.0), 1e-4)
    eq([[-1, -4], [-9, -16]], a.neg())
    eq([[2, 4], [5, 5]], a.clamp(2.0, 5.0))
    eq([[1, 9], [4, 16]], a.transpose())
    x = Tensor.from2D([[0.0, 1.0, -1.0]])
    eq([[1.0, math.e, 1 / math.e]], x.exp(), 1e-6)
    eq([[0.0, math.log(2.0)]], Tensor.from2D([[1.0, 2.0]]).log(), 1e-6)
    eq([[0.0, math.tanh(1.0), -math.tanh(1.0)]], x.tanhActivation(), 1e-6)
    eq([[0.5, 1 / (1 + math.exp(-1)), 1 / (1 + math.e)]], x.sigmoidActivation(), 1e-6)
    eq([[0.0, 1.0, 0.0]], x.reluActivation())
    g = x.geluActivation().numpy()
    assert abs(g[0, 0]) < 1e-7 and abs(g[0, 1] - 0.8411919906) < 1e-5 and abs(g[0, 2] + 0.1588080094) < 1e-5


def case_reductions():                  # CpuBackendTest.java:430-652
    a = Tensor.from2D(A)
    eq([[5, 7, 9]], a.sumRows())
    eq([[5, 7, 9]], a.sumAlongCols())
    eq([[6], [15]], a.sumAlongRows())
    eq([[2], [5]], a.meanAlongRows())
    eq([[2 / 3], [2 / 3]], a.varianceAlongRows())          # variance of [1,2,3] is 2/3 (:514-526)
    eq([[3], [6]], a.maxAlongRows())
    assert abs(a.sum() - 21.0) < EPS
    assert abs(Tensor.from2D([[-1, 2], [-3, 4]]).sumAbs() - 10.0) < EPS
    s = Tensor.from2D([[1.0, 2.0, 3.0], [0.0, 0.0, 0.0]]).softmaxRows().numpy()
    e = np.exp([1.0, 2.0, 3.0]); e /= e.sum()
    assert np.allclose(s[0], e, atol=1e-6) and np.allclose(s[1], 1 / 3, atol=1e-6)


def case_linear():                      # LinearTest.java:17-41: y = [[5.5,1.5,0],[-0.5,-0.5,2]]
    lin = Linear(np.array([[1, 0, -1], [2, 1, 0]], dtype=np.float32), np.array([0.5, -0.5, 1.0], dtype=np.float32))
    eq([[5.5, 1.5, 0.0], [-0.5, -0.5, 2.0]], lin.forward(Tensor.from2D([[1, 2], [-1, 0]])))
    with pytest.raises(ValueError):
        lin.forward(Tensor.from2D([[1, 2, 3]]))


def case_rmsnorm():                     # RMSNorm1DTest.java:59-111,192-201
    x = Tensor.from2D([[3, 0, 4, 0]])
    y = RMSNorm1D(4).forward(x).numpy()
    assert abs(math.sqrt(float(np.mean(y ** 2))) - 1.0) < 1e-5                   # unit RMS
    eq([[1, 1, 1, 1]], RMSNorm1D(4).forward(Tensor.from2D([[5, 5, 5, 5]])), 1e-5)   # constant row → 1
    y2 = RMSNorm1D(4, np.full(4, 2.0, dtype=np.float32)).forward(x).numpy()
    assert np.allclose(y2, 2 * y, atol=1e-6)                                   # gain doubling
    y3 = RMSNorm1D(4).forward(Tensor.from2D([[30, 0, 40, 0]])).numpy()
    assert np.allclose(y3, y, atol=1e-6)                                       # scale invariance
    with pytest.raises(ValueError):
        RMSNorm1D(4).forward(Tensor.from2D([[1, 2, 3]]))
    with pytest.raises(ValueError):
        RMSNorm1D(0)


def case_rope():                        # RotaryEmbeddingTest.java:37-162
    rope = RotaryEmbedding(4, 8)
    t = Tensor.from2D([[1, 0, 1, 0], [1, 0, 1, 0]])
    out = rope.apply(t, 2, 1).numpy()
    assert np.allclose(out[0], [1, 0, 1, 0], atol=1e-7)                         # position 0 is the identity
    assert abs(out[1, 0] - math.cos(1.0)) < 1e-6 and abs(out[1, 1] - math.sin(1.0)) < 1e-6   # pair 0 at position 1
    x = np.random.default_rng(0).standard_normal((6, 4)).astype(np.float32)
    y = rope.apply(Tensor(6, 4, x), 3, 2).numpy()
    assert np.allclose(np.linalg.norm(y, axis=1), np.linalg.norm(x, axis=1), atol=1e-5)      # rotations keep the norm
    same = rope.apply(Tensor(6, 4, np.tile(x[:3], (2, 1))), 3, 2).numpy()
    assert np.array_equal(same[:3], same[3:])                                  # every head sees the same positions
    with pytest.raises(ValueError):
        RotaryEmbedding(3, 8)                                                   # odd headDim
    with pytest.raises(ValueError):
        RotaryEmbedding(4, 0)
    with pytest.raises(ValueError):
        rope.apply(Tensor(9, 4), 9, 1)                                          # seqLen > maxSeqLen


def case_silu_swiglu():                 # SiLUTest.java:34-58
    x = Tensor.from2D([[0.0, 1.0, -1.0]])
    s = x.multiply(x.sigmoidActivation()).numpy()
    sig1 = 1 / (1 + math.exp(-1.0))
    assert abs(s[0, 0]) < 1e-7 and abs(s[0, 1] - sig1) < 1e-6 and abs(s[0, 2] + (1 - sig1)) < 1e-6
    eye = np.eye(2, dtype=np.float32)
    sw = SwiGLULayer(Linear(eye), Linear(eye), Linear(eye))
    out = sw.forward(Tensor.from2D([[1.0, -1.0]])).numpy()
    assert abs(out[0, 0] - sig1) < 1e-6 and abs(out[0, 1] - (1 - sig1)) < 1e-6


def case_causal_no_leak():              # MultiHeadSelfAttentionTest.java:24-68
    d, n = 8, 5
    eye = np.eye(d, dtype=np.float32)
    attn = MultiHeadSelfAttention(d, 2, True, eye, eye, eye, eye)
    x = np.random.default_rng(1).standard_normal((n, d)).astype(np.float32)
    y1 = attn.forward(Tensor(n, d, x)).numpy().copy()
    x2 = x.copy()
    x2[-1] += 5.0                                                               # change only the last token
    y2 = attn.forward(Tensor(n, d, x2)).numpy()
    assert np.all(np.abs(y1[:-1] - y2[:-1]) <= 1e-7)
    assert np.abs(y1[-1] - y2[-1]).max() > 1e-3
    with pytest.raises(ValueError):
        MultiHeadSelfAttention(7, 2, True, eye, eye, eye, eye)


def case_head_ops_roundtrip():
    x = np.arange(24, dtype=np.float32).reshape(3, 8)
    sp = HeadOps.splitHeads(Tensor(3, 8, x), 3, 2, 4, 8)
    assert np.array_equal(sp.data[0], [0, 1, 2, 3]) and np.array_equal(sp.data[3], [4, 5, 6, 7])
    assert np.array_equal(HeadOps.mergeHeads(sp, 3, 2, 4, 8).data, x)


def case_greedy_semantics():            # TextGenerator.java:104-170; TextGeneratorTest.java:91-98
    logits = np.array([0.5, 2.0, 2.0, -1.0], dtype=np.float32)
    assert TextGenerator.argsortDescending(logits)[0] == 1                      # ties → lowest index
    assert TextGenerator.argsortDescending(np.array([-0.0, 0.0], dtype=np.float32))[0] == 1   # -0.0 < +0.0
    assert TextGenerator.argsortDescending(np.array([1.0, np.nan, 3.0], dtype=np.float32))[0] == 1   # NaN sorts largest
    fwd = lambda ids: Tensor.from2D([logits, logits])
    for r in (0.0, 0.3, 0.99):                                                  # topK = 1 ignores the random draw
        assert TextGenerator.generate(fwd, 8, [0], 3, 0.7, 1, lambda: r) == [0, 1, 1, 1]
    for bad in ((-1, 1.0, 1), (1, 0.0, 1), (1, 1.0, -1)):
        with pytest.raises(ValueError):
            TextGenerator.generate(fwd, 8, [0], *bad)


ALL_CASES = [case_matmul, case_causal_mask, case_elementwise, case_broadcasts, case_scalars_and_unary, case_reductions,
             case_linear, case_rmsnorm, case_rope, case_silu_swiglu, case_causal_no_leak, case_head_ops_roundtrip,
             case_greedy_semantics]
