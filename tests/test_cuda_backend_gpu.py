"""The 42-op stream on the GPU: the reference's known answers through `CudaBackend`, and
GPU-vs-oracle parity at the shapes and tolerances of the reference's MetalBackendTest
(|e-a| <= atol + rtol*|e|; 1e-4 in general, 1e-3 for wide rows and atomics)."""
import ctypes

import numpy as np
import pytest

import oracle
import ref_cases
from deepj_b200 import _lib
from deepj_b200 import compute_graph as cg
from deepj_b200.decoder import DecoderConfig
from deepj_b200.layers import TextGenerator, build_model
from deepj_b200.tensor import CudaBackend, GraphBackend, Tensor

pytestmark = pytest.mark.gpu


@pytest.fixture()
def cuda():
    b = CudaBackend(0)
    Tensor.setBackend(b)
    yield b
    b.releaseResources()


def on_both(fn):
    """Run fn() under the oracle runtime and under CUDA; returns (expected, actual) arrays."""
    ob = GraphBackend(oracle.OracleRuntime())
    Tensor.setBackend(ob)
    e = fn()
    e = [np.array(x.numpy() if isinstance(x, Tensor) else x, copy=True) for x in (e if isinstance(e, (list, tuple)) else [e])]
    ob.releaseResources()
    cb = CudaBackend(0)
    Tensor.setBackend(cb)
    a = fn()
    a = [np.array(x.numpy() if isinstance(x, Tensor) else x, copy=True) for x in (a if isinstance(a, (list, tuple)) else [a])]
    cb.releaseResources()
    return e, a


def close(e, a, atol=1e-4, rtol=1e-4):
    for x, y in zip(e, a):
        assert x.shape == y.shape
        assert np.all(np.abs(x - y) <= atol + rtol * np.abs(x)), float(np.abs(x - y).max())


@pytest.mark.parametrize("case", ref_cases.ALL_CASES, ids=lambda c: c.__name__)
def test_reference_known_answers_on_cuda(cuda, case):
    case()


def rnd(shape, seed, scale=1.0):
    return (np.random.default_rng(seed).standard_normal(shape) * scale).astype(np.float32)


def test_matmul_128x192x64_is_bit_exact_with_the_ikj_loop():      # MetalBackendTest.java:71-78
    A, B = rnd((128, 192), 1), rnd((192, 64), 2)
    e, a = on_both(lambda: Tensor(128, 192, A).matmul(Tensor(192, 64, B)))
    assert np.array_equal(e[0].view(np.uint32), a[0].view(np.uint32))


@pytest.mark.parametrize("shape", [(7, 5), (33, 130), (4, 513), (3, 769), (2, 777), (1, 1)])
def test_elementwise_broadcast_reduction_parity(shape):           # MetalBackendTest.java:100-130,222-261
    r, c = shape
    X, Y = rnd(shape, 3), np.abs(rnd(shape, 4)) + 0.5
    row, col = rnd((1, c), 5), np.abs(rnd((r, 1), 6)) + 0.5

    def fn():
        x, y = Tensor(r, c, X), Tensor(r, c, Y)
        rv, cv = Tensor(1, c, row), Tensor(r, 1, col)
        return [x.add(y), x.subtract(y), x.multiply(y), x.divide(y), x.addRowVector(rv), x.multiplyBroadcastRows(rv),
                x.addBroadcastCols(cv), x.subtractBroadcastCols(cv), x.multiplyBroadcastCols(cv), x.divideBroadcastCols(cv),
                x.multiplyScalar(0.37), x.addScalar(-1.5), x.divideScalar(3.0), y.sqrt(), x.neg(), x.exp(), y.log(),
                x.tanhActivation(), x.sigmoidActivation(), x.reluActivation(), x.geluActivation(), x.clamp(-0.5, 0.5),
                y.pow(1.7), x.transpose(), x.sumRows(), x.sumAlongRows(), x.meanAlongRows(), x.varianceAlongRows(),
                x.maxAlongRows(), x.softmaxRows(), np.float32(x.sum()), np.float32(x.sumAbs())]
    e, a = on_both(fn)
    close(e, a, atol=1e-3 if c > 512 else 1e-4, rtol=1e-3 if c > 512 else 1e-4)


def test_training_ops_parity():                                   # MetalBackendTest.java:254-403
    G, S = rnd((6, 33), 7), np.abs(rnd((6, 33), 8))
    S /= S.sum(axis=1, keepdims=True)
    L = rnd((5, 17), 9, 2.0)
    tg = [0, 16, 3, 3, 9]
    W, Gr, M, V = rnd((4, 9), 10), rnd((4, 9), 11), rnd((4, 9), 12, 0.1), np.abs(rnd((4, 9), 13, 0.1))
    sd = np.abs(rnd((6, 1), 14)) + 0.5

    def fn():
        b = Tensor.backend()
        g, s = Tensor(6, 33, G), Tensor(6, 33, S)
        out = [b.softmaxBackward(g, s), b.layerNormBackward(g, s, Tensor(6, 1, sd), 33), b.reluBackward(g, s), b.geluBackward(g, s),
               np.float32(b.crossEntropyLoss(Tensor(5, 17, L), tg)), b.crossEntropyGradient(Tensor(5, 17, L), tg)]
        w, gr, m, v = Tensor(4, 9, W.copy()), Tensor(4, 9, Gr), Tensor(4, 9, M.copy()), Tensor(4, 9, V.copy())
        b.adamWUpdate(w, gr, m, v, 1e-2, 0.9, 0.999, 1e-8, 0.01, 0.1, 0.001)
        target = Tensor(7, 9, np.zeros((7, 9), dtype=np.float32))
        target.add(target).materialize()                      # put it on the device first
        b.scatterAddRows(target, [1, 3, 1, 6], Tensor(4, 9, Gr))
        return out + [w, m, v, target]
    e, a = on_both(fn)
    close(e[:4], a[:4])
    close(e[4:6], a[4:6], atol=1e-3, rtol=1e-2)                # softmax-derived: the reference's own tolerance
    close(e[6:], a[6:], atol=1e-3, rtol=1e-3)


@pytest.mark.parametrize("kind", ["llama", "deepseek"])
def test_unmodified_layer_stack_runs_on_cuda_backend(kind):
    """Drop-in: the reference's layer structure over CudaBackend gives the oracle's logits
    and greedy tokens (fp32 weights — the reference's true path)."""
    cfg = DecoderConfig(kind, 256, 24, 64, 4, 2, 176, q_rank=32 if kind == "deepseek" else 0, kv_rank=16 if kind == "deepseek" else 0)
    om = oracle.OracleModel(kind, 256, 24, 64, 4, 2, 176, cfg.q_rank, cfg.kv_rank, seed=3)
    from test_decoder_gpu import weight_getter
    ids = [5, 9, 200, 31, 7, 0, 255]
    expected = om.forward(ids)
    toks, _ = om.generate_greedy(ids, 4, use_cache=False)
    cb = CudaBackend(0)
    Tensor.setBackend(cb)
    model = build_model(cfg, weight_getter(om, cfg))
    got = model.forward(ids).numpy()
    rng_ = float(expected.max() - expected.min())
    assert float(np.abs(got - expected).max()) <= 2e-3 * rng_
    assert TextGenerator.generate(model.forward, 24, ids, 4, 1.0, 1)[7:] == list(toks)
    cb.releaseResources()


def test_gpt_layer_stack_runs_on_cuda_backend():
    """Drop-in for the GPT family: the same layer stack (LayerNorm, GELU MLP, learned positions, plain causal
    attention) over CudaBackend and over the oracle's interpreter — same logits, same greedy tokens."""
    import gpt_ref
    from deepj_b200.layers import build_gpt_model
    shape = dict(vocab=97, max_seq=16, d=32, heads=4, layers=2, d_ff=80)
    w, get = gpt_ref.make_weights(seed=6, **shape)
    ids = [3, 96, 0, 41, 41, 7, 12]
    ob = GraphBackend(oracle.OracleRuntime())
    Tensor.setBackend(ob)
    om = build_gpt_model(get=get, **shape)
    expected = om.forward(ids).numpy()
    exp_tokens = TextGenerator.generate(om.forward, 16, ids, 4, 1.0, 1)
    ob.releaseResources()
    cb = CudaBackend(0)
    Tensor.setBackend(cb)
    model = build_gpt_model(get=get, **shape)
    got = model.forward(ids).numpy()
    assert float(np.abs(got - expected).max()) <= 1e-5 * float(np.abs(expected).max())
    assert float(np.abs(got - gpt_ref.forward(w, ids, 32, 4, 2)).max()) <= 1e-4 * float(np.abs(expected).max())
    assert TextGenerator.generate(model.forward, 16, ids, 4, 1.0, 1) == exp_tokens
    cb.releaseResources()


# ── malformed streams are rejected before any launch ──
def flush_raw(ints):
    lib = _lib.load()
    _lib.check(lib.deepj_cuda_init(0))
    cmd = np.asarray(ints, dtype=np.int32)
    return lib.deepj_cuda_flush_ops(cmd.ctypes.data, cmd.size), lib.deepj_cuda_last_error().decode()


def test_malformed_streams_are_rejected(cuda):
    lib = _lib.load()
    ids, sizes = (ctypes.c_int32 * 2)(900001, 900002), (ctypes.c_int32 * 2)(8, 8)
    _lib.check(lib.deepj_cuda_alloc_buffers(ids, sizes, 2))
    one = np.ones(8, dtype=np.float32)
    _lib.check(lib.deepj_cuda_upload_buffer(900001, one.ctypes.data, 8))
    rc, msg = flush_raw([99, 900001, 900002, 8])
    assert rc != 0 and "Unknown op code" in msg
    rc, msg = flush_raw([cg.OP_ADD, 900001, 900002])
    assert rc != 0 and "Truncated" in msg
    rc, msg = flush_raw([cg.OP_NEG, 900001, 123456789, 8])
    assert rc != 0 and "missing GPU buffer" in msg
    rc, msg = flush_raw([cg.OP_NEG, 900001, 900002, 9])
    assert rc != 0 and "needs 9" in msg
    # a valid op first, an invalid one second: nothing may have run
    rc, msg = flush_raw([cg.OP_NEG, 900001, 900002, 8, cg.OP_NEG, 900001, 900002, 64])
    assert rc != 0
    out = np.empty(8, dtype=np.float32)
    _lib.check(lib.deepj_cuda_download_buffer(900002, out.ctypes.data, 8))
    assert not out.any()                                       # fresh buffers are zero-filled and were not written
    assert lib.deepj_cuda_upload_buffer(777777, one.ctypes.data, 8) != 0
    assert "Buffer not found for upload" in lib.deepj_cuda_last_error().decode()
    assert lib.deepj_cuda_download_buffer(777777, out.ctypes.data, 8) != 0
    _lib.check(lib.deepj_cuda_release_buffers((ctypes.c_int32 * 3)(900001, 900002, 424242), 3))   # unknown ids are ignored
    _lib.check(lib.deepj_cuda_alloc_buffers(ids, sizes, 2))
    _lib.check(lib.deepj_cuda_alloc_buffers(ids, sizes, 2))    # allocating an existing id is a no-op
    _lib.check(lib.deepj_cuda_release_buffers(ids, 2))


def test_repeated_stream_is_replayed_as_a_graph_and_survives_unrelated_releases(cuda):
    lib = _lib.load()
    ids = (ctypes.c_int32 * 3)(910001, 910002, 910003)
    _lib.check(lib.deepj_cuda_alloc_buffers(ids, (ctypes.c_int32 * 3)(16, 16, 16), 3))
    x = np.arange(16, dtype=np.float32)
    _lib.check(lib.deepj_cuda_upload_buffer(910001, x.ctypes.data, 16))
    stream = np.asarray([cg.OP_ADD_SCALAR, 910001, 910002, cg.float_bits(1.0), 16, cg.OP_MULTIPLY_SCALAR, 910002, 910003,
                         cg.float_bits(2.0), 16], dtype=np.int32)
    st = (ctypes.c_int64 * 6)()
    _lib.check(lib.deepj_cuda_stats(st, 6))
    replays0 = st[1]
    for i in range(4):
        _lib.check(lib.deepj_cuda_flush_ops(stream.ctypes.data, stream.size))
        if i == 2:      # an unrelated alloc/release in between must not invalidate the graph's buffers
            _lib.check(lib.deepj_cuda_alloc_buffers((ctypes.c_int32 * 1)(910009), (ctypes.c_int32 * 1)(4), 1))
            _lib.check(lib.deepj_cuda_release_buffers((ctypes.c_int32 * 1)(910009), 1))
    out = np.empty(16, dtype=np.float32)
    _lib.check(lib.deepj_cuda_download_buffer(910003, out.ctypes.data, 16))
    assert np.array_equal(out, (x + 1) * 2)
    _lib.check(lib.deepj_cuda_stats(st, 6))
    assert st[1] - replays0 >= 2 and st[5] == 0
    # releasing a buffer the graph uses invalidates it: the next flush must fail cleanly, not replay
    _lib.check(lib.deepj_cuda_release_buffers((ctypes.c_int32 * 1)(910002), 1))
    assert lib.deepj_cuda_flush_ops(stream.ctypes.data, stream.size) != 0
    _lib.check(lib.deepj_cuda_release_buffers(ids, 3))
