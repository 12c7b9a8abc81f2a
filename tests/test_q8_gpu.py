"""GPU parity of the Q8 quantizer (bit-exact) and of the fused Q8 linear / SwiGLU ops
against the CPU oracle with dequantized weights."""
import ctypes

import numpy as np
import pytest

import oracle
from deepj_b200 import _lib
from deepj_b200.compute_graph import OP_Q8_LINEAR, OP_Q8_SWIGLU, float_bits

pytestmark = pytest.mark.gpu

ATOL, RTOL = 1e-4, 1e-4      # the reference's GPU-vs-CPU comparator: |e-a| <= atol + rtol*|e|
MANY_ROW_FLOOR = 1e-4        # of the largest |expected|, for five activation rows and more


def close(expected, actual, atol=ATOL, rtol=RTOL, floor=0.0):
    """|error| ≤ atol + rtol·|expected| + floor·max|expected|.  The floor term is for the several-row kernels: the
    5 … 16-row kernel multiplies 16-bit fixed-point activations (an error of up to 2^-16 of a 32-k block's largest
    value per element), the tensor-core GEMM accumulates fp16 products with ≈ 2^-18 of the output scale; the stated
    Q8 tolerance is 2e-3 of the output scale."""
    err = np.abs(expected - actual)
    bound = atol + rtol * np.abs(expected) + floor * float(np.abs(expected).max())
    worst = np.unravel_index(np.argmax(err - bound), err.shape)
    assert np.all(err <= bound), f"max err {err.max()} at {worst}: expected {expected[worst]}, got {actual[worst]} (bound {bound[worst]})"


class Dev:
    """Tiny helper over the C ABI: float buffers and Q8 objects by id."""

    def __init__(self, base):
        self.lib = _lib.load()
        _lib.check(self.lib.deepj_cuda_init(0))
        self.next = base
        self.owned = []

    def buf(self, n, data=None):
        i = self.next
        self.next += 1
        self.owned.append(i)
        _lib.check(self.lib.deepj_cuda_alloc_buffers((ctypes.c_int32 * 1)(i), (ctypes.c_int32 * 1)(n), 1))
        if data is not None:
            d = np.ascontiguousarray(data, dtype=np.float32)
            _lib.check(self.lib.deepj_cuda_upload_buffer(i, d.ctypes.data, d.size))
        return i

    def q8(self, W):
        K, N = W.shape
        src = self.buf(K * N, W)
        q = self.next
        self.next += 1
        self.owned.append(q)
        _lib.check(self.lib.deepj_cuda_q8_alloc(q, K, N))
        _lib.check(self.lib.deepj_cuda_q8_quantize_into(q, 0, src, 0, 0, N, N))
        return q

    def q8_download(self, q, K, N):
        codes = np.empty((N, K), dtype=np.int8)
        scales = np.empty((N, (K + 31) // 32), dtype=np.float32)
        _lib.check(self.lib.deepj_cuda_q8_download(q, codes.ctypes.data, scales.ctypes.data))
        return codes, scales

    def get(self, i, n):
        out = np.empty(n, dtype=np.float32)
        _lib.check(self.lib.deepj_cuda_download_buffer(i, out.ctypes.data, n))
        return out

    def flush(self, ints):
        cmd = np.asarray(ints, dtype=np.int32)
        _lib.check(self.lib.deepj_cuda_flush_ops(cmd.ctypes.data, cmd.size))

    def close(self):
        arr = (ctypes.c_int32 * len(self.owned))(*self.owned)
        _lib.check(self.lib.deepj_cuda_release_buffers(arr, len(self.owned)))
        self.owned = []


@pytest.fixture()
def dev():
    d = Dev(1 << 20)
    yield d
    d.close()


@pytest.mark.parametrize("K,N", [(32, 8), (64, 48), (100, 7), (688, 256), (4096, 96), (16, 3), (1, 5)])
def test_quantizer_is_bit_exact(dev, K, N):
    rng = np.random.default_rng(1000 + K + N)
    W = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    if K >= 64:
        W[:32, 0] = 0.0              # an all-zero block: scale 0, codes 0
        W[40, 1] = 3.0               # an outlier dominating its block
    codes_o, scales_o = oracle.q8_quantize(W)
    q = dev.q8(W)
    codes_g, scales_g = dev.q8_download(q, K, N)
    assert np.array_equal(scales_o.view(np.uint32), scales_g.view(np.uint32))
    assert np.array_equal(codes_o, codes_g)


def test_quantize_into_column_windows_and_upload_roundtrip(dev):
    rng = np.random.default_rng(5)
    K, N = 96, 40
    W = (rng.standard_normal((K + 8, N + 6)) * 0.05).astype(np.float32)    # a window inside a larger matrix
    src = dev.buf(W.size, W)
    q = dev.next; dev.next += 1; dev.owned.append(q)
    _lib.check(dev.lib.deepj_cuda_q8_alloc(q, K, N))
    _lib.check(dev.lib.deepj_cuda_q8_quantize_into(q, 0, src, 8, 6, N + 6, 16))
    _lib.check(dev.lib.deepj_cuda_q8_quantize_into(q, 16, src, 8, 22, N + 6, N - 16))
    codes_o, scales_o = oracle.q8_quantize(W[8:, 6:])
    codes_g, scales_g = dev.q8_download(q, K, N)
    assert np.array_equal(codes_o, codes_g) and np.array_equal(scales_o, scales_g)
    q2 = dev.next; dev.next += 1; dev.owned.append(q2)
    _lib.check(dev.lib.deepj_cuda_q8_alloc(q2, K, N))
    _lib.check(dev.lib.deepj_cuda_q8_upload(q2, codes_o.ctypes.data, scales_o.ctypes.data))
    c2, s2 = dev.q8_download(q2, K, N)
    assert np.array_equal(codes_o, c2) and np.array_equal(scales_o, s2)


def oracle_rmsnorm(x, gamma):
    """RMSNorm1D.forward in the reference's op order, fp32."""
    out = np.empty_like(x)
    for r in range(x.shape[0]):
        s = np.float32(0.0)
        for v in x[r]:
            s = np.float32(s + np.float32(v * v))
        mean = np.float32(s * np.float32(np.float32(1.0) / np.float32(x.shape[1])))
        rms = np.float32(np.sqrt(np.float64(np.float32(mean + np.float32(1e-6)))))
        out[r] = (x[r] / rms) * gamma
    return out


@pytest.mark.parametrize("M,K,N", [(1, 256, 256), (1, 688, 256), (3, 256, 688), (1, 4096, 512), (2, 2048, 100),
                                   (1, 11008, 64), (1, 100, 33), (1, 512, 2048), (1, 5632, 128), (6, 512, 40), (4, 4096, 24), (1, 1376, 64), (2, 96, 20), (1, 2752, 33),
                                   (5, 1376, 200), (16, 4096, 512), (16, 96, 20), (7, 2752, 33), (40, 512, 300), (9, 11008, 64),
                                   (17, 256, 128), (64, 4096, 512), (130, 512, 300), (512, 2048, 256), (40, 96, 20), (300, 64, 8),
                                   (257, 256, 128), (300, 512, 300), (640, 128, 520),
                                   # 17 … 128 rows at K = 4096: passes of the several-row kernel, then the split tensor-core form
                                   (17, 4096, 768), (24, 4096, 4096), (32, 4096, 768), (48, 4096, 1024), (96, 4096, 768), (128, 4096, 1280),
                                   (200, 11008, 512)])
@pytest.mark.parametrize("fused", ["plain", "norm_bias_res"])
def test_q8_linear_matches_oracle(dev, M, K, N, fused):
    rng = np.random.default_rng(K * 7 + N + M)
    x = rng.standard_normal((M, K)).astype(np.float32)
    W = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    Wq = oracle.q8_dequantize(*oracle.q8_quantize(W))
    q = dev.q8(W)
    xb = dev.buf(M * K, x)
    ob = dev.buf(M * N)
    if fused == "plain":
        expected = oracle.matmul(x, Wq)
        dev.flush([OP_Q8_LINEAR, xb, 0, K, -1, 0, q, -1, -1, 0, 0, ob, 0, N, M])
    else:
        gamma = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float32)
        bias = rng.standard_normal(N).astype(np.float32)
        res = rng.standard_normal((M, N)).astype(np.float32)
        expected = (oracle.matmul(oracle_rmsnorm(x, gamma), Wq) + bias) + res
        gb, bb, rb = dev.buf(K, gamma), dev.buf(N, bias), dev.buf(M * N, res)
        dev.flush([OP_Q8_LINEAR, xb, 0, K, gb, float_bits(1e-6), q, bb, rb, 0, N, ob, 0, N, M])
    close(expected, dev.get(ob, M * N).reshape(M, N), floor=MANY_ROW_FLOOR if M >= 5 else 0.0)


@pytest.mark.parametrize("M,K,F", [(1, 256, 688), (2, 256, 100), (1, 4096, 256), (1, 2048, 5632),
                                   (3, 256, 688), (16, 4096, 256), (5, 2048, 100), (20, 512, 72),
                                   (64, 512, 256), (200, 4096, 200), (300, 512, 256)])
def test_q8_swiglu_matches_oracle(dev, M, K, F):
    rng = np.random.default_rng(K + F)
    x = rng.standard_normal((M, K)).astype(np.float32)
    Wg = (rng.standard_normal((K, F)) * 0.05).astype(np.float32)
    Wu = (rng.standard_normal((K, F)) * 0.05).astype(np.float32)
    bg = (0.1 * rng.standard_normal(F)).astype(np.float32)
    bu = (0.1 * rng.standard_normal(F)).astype(np.float32)
    gamma = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float32)
    xn = oracle_rmsnorm(x, gamma)
    g = oracle.matmul(xn, oracle.q8_dequantize(*oracle.q8_quantize(Wg))) + bg
    u = oracle.matmul(xn, oracle.q8_dequantize(*oracle.q8_quantize(Wu))) + bu
    sig = (1.0 / (1.0 + np.exp(-g.astype(np.float64)).astype(np.float32))).astype(np.float32)
    expected = (g * sig) * u
    qg, qu = dev.q8(Wg), dev.q8(Wu)
    xb, gb, bgb, bub, ob = dev.buf(M * K, x), dev.buf(K, gamma), dev.buf(F, bg), dev.buf(F, bu), dev.buf(M * F)
    dev.flush([OP_Q8_SWIGLU, xb, 0, K, gb, float_bits(1e-6), qg, bgb, qu, bub, ob, 0, F, M])
    close(expected, dev.get(ob, M * F).reshape(M, F), floor=MANY_ROW_FLOOR if M >= 5 else 0.0)


def test_q8_linear_strided_windows(dev):
    """x_off / ldx / out_off / ldo address a window of a wider activation row (used by MLA)."""
    rng = np.random.default_rng(3)
    M, K, N, ldx, ldo = 2, 64, 48, 200, 160
    xw = rng.standard_normal((M, ldx)).astype(np.float32)
    W = (rng.standard_normal((K, N)) * 0.05).astype(np.float32)
    q = dev.q8(W)
    xb = dev.buf(xw.size, xw)
    out0 = rng.standard_normal((M, ldo)).astype(np.float32)
    ob = dev.buf(out0.size, out0)
    dev.flush([OP_Q8_LINEAR, xb, 100, ldx, -1, 0, q, -1, -1, 0, 0, ob, 32, ldo, M])
    got = dev.get(ob, out0.size).reshape(M, ldo)
    expected = oracle.matmul(np.ascontiguousarray(xw[:, 100:164]), oracle.q8_dequantize(*oracle.q8_quantize(W)))
    close(expected, got[:, 32:80])
    assert np.array_equal(got[:, :32], out0[:, :32]) and np.array_equal(got[:, 80:], out0[:, 80:])


def test_tc_correction_terms_trade_bits_for_products(dev):
    """deepj_cuda_tc_configure: the many-row kernel with both correction products (the default) sits at fp32-like error;
    each dropped product leaves an operand at 11 bits and the error rises by orders of magnitude; the setting is
    validated, takes effect on the next flush and is restored."""
    M, K, N = 512, 2048, 256
    rng = np.random.default_rng(99)
    x = rng.standard_normal((M, K)).astype(np.float32)
    W = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    Wq = oracle.q8_dequantize(*oracle.q8_quantize(W))
    expected = (x.astype(np.float64) @ Wq.astype(np.float64))
    q, xb, ob = dev.q8(W), dev.buf(M * K, x), dev.buf(M * N)
    errs = {}
    try:
        for terms in (3, 1, 2, 0):
            _lib.check(dev.lib.deepj_cuda_tc_configure(terms))
            dev.flush([OP_Q8_LINEAR, xb, 0, K, -1, 0, q, -1, -1, 0, 0, ob, 0, N, M])
            errs[terms] = float(np.abs(dev.get(ob, M * N).reshape(M, N) - expected).max() / np.abs(expected).max())
        assert dev.lib.deepj_cuda_tc_configure(4) != 0 and "correction_terms" in dev.lib.deepj_cuda_last_error().decode()
    finally:
        _lib.check(dev.lib.deepj_cuda_tc_configure(3))
    assert errs[3] < 2e-5, errs
    assert all(errs[t] > 8 * errs[3] for t in (1, 2, 0)), errs
    assert errs[0] < 2e-3, errs


@pytest.mark.parametrize("M,K,N,x_off", [(1, 256, 37, 101), (2, 1024, 50, 3), (1, 4096, 24, 7), (16, 512, 40, 5), (9, 1024, 21, 1)])
def test_q8_linear_unaligned_rows_and_ragged_tiles(dev, M, K, N, x_off):
    """Reduction lengths that take the TMA kernels, with activation rows that start off a 16-byte boundary (the staging
    falls back to scalar loads), a gain vector, bias and residual, an output window inside a wider row, and a last
    weight tile that is only partly there (the copy engine fills the missing rows with zeros)."""
    rng = np.random.default_rng(1000 + M + K + N)
    ldx, ldo, out_off = K + 2 * x_off + 3, N + 11, 5
    xw = rng.standard_normal((M, ldx)).astype(np.float32)
    W = (rng.standard_normal((K, N)) * 0.03).astype(np.float32)
    gamma = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    res = rng.standard_normal((M, N)).astype(np.float32)
    out0 = rng.standard_normal((M, ldo)).astype(np.float32)
    q = dev.q8(W)
    xb, gb, bb, rb, ob = dev.buf(xw.size, xw), dev.buf(K, gamma), dev.buf(N, bias), dev.buf(M * N, res), dev.buf(out0.size, out0)
    dev.flush([OP_Q8_LINEAR, xb, x_off, ldx, gb, float_bits(1e-6), q, bb, rb, 0, N, ob, out_off, ldo, M])
    got = dev.get(ob, out0.size).reshape(M, ldo)
    x = np.ascontiguousarray(xw[:, x_off:x_off + K])
    expected = (oracle.matmul(oracle_rmsnorm(x, gamma), oracle.q8_dequantize(*oracle.q8_quantize(W))) + bias) + res
    close(expected, got[:, out_off:out_off + N], floor=MANY_ROW_FLOOR if M >= 5 else 0.0)
    assert np.array_equal(got[:, :out_off], out0[:, :out_off]) and np.array_equal(got[:, out_off + N:], out0[:, out_off + N:])
