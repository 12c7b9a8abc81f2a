"""Pins the CPU oracle: the reference's known-answer tests, java.util.Random, RoPE tables,
Q8 format properties, and the equivalence of the oracle's two restatements of the model
(native C++ forward vs the Python layer stack over the oracle's op interpreter)."""
import numpy as np
import pytest

import oracle
import ref_cases
from deepj_b200.decoder import DecoderConfig, rope_tables
from deepj_b200.layers import TextGenerator, build_model
from deepj_b200.tensor import GraphBackend, Tensor


@pytest.fixture(autouse=True)
def oracle_backend():
    b = GraphBackend(oracle.OracleRuntime())
    Tensor.setBackend(b)
    yield b
    b.releaseResources()


@pytest.mark.parametrize("case", ref_cases.ALL_CASES, ids=lambda c: c.__name__)
def test_reference_known_answers_on_oracle(case):
    case()


def test_java_random_matches_documented_outputs():
    """java.util.Random per the Java SE specification; the Gaussian values need the fdlibm log."""
    r = oracle.JRandom(42)
    assert [r.next_int(10) for _ in range(10)] == [0, 3, 8, 4, 0, 5, 5, 8, 9, 3]
    assert oracle.JRandom(42).next_double() == 0.7275636800328681
    r = oracle.JRandom(42)
    assert [r.next_gaussian() for _ in range(3)] == [1.1419053154730547, 0.9194079489827879, -0.9498666368908959]
    assert oracle.JRandom(0).next_gaussian() == 0.8025330637390305
    a, b = oracle.JRandom(123).tensor_random(2, 3), oracle.JRandom(123).tensor_random(2, 3)   # CpuBackendTest.java:57-69
    assert np.array_equal(a, b)
    assert a[0, 0] == np.float32(-1.4380493091409068 * 0.1)
    r = oracle.JRandom(7)
    assert all(0 <= r.next_int(256) < 256 for _ in range(1000))
    assert 0.0 <= oracle.JRandom(5).next_float() < 1.0


def test_rope_tables_host_equals_oracle():
    for hd, n in ((32, 256), (128, 64), (2, 5)):
        c, s = rope_tables(hd, n)
        co, so = oracle.rope_tables(hd, n)
        assert np.array_equal(c.view(np.uint32), co.view(np.uint32)) and np.array_equal(s.view(np.uint32), so.view(np.uint32))
    assert np.all(rope_tables(8, 4)[0][0] == 1.0) and np.all(rope_tables(8, 4)[1][0] == 0.0)


def test_q8_format_properties():
    rng = np.random.default_rng(0)
    W = (rng.standard_normal((688, 40)) * 0.02).astype(np.float32)      # K = 688: 21 full blocks + one of 16
    W[:32, 0] = 0.0
    codes, scales = oracle.q8_quantize(W)
    assert codes.shape == (40, 688) and scales.shape == (40, 22)
    assert scales[0, 0] == 0.0 and not codes[0, :32].any()               # all-zero block → scale 0, codes 0
    assert np.abs(codes.astype(np.int32)).max() <= 127
    amax = np.abs(W[32:64, 3]).max()
    assert scales[3, 1] == np.float32(amax) / np.float32(127.0)
    assert np.abs(codes[3, 32:64]).max() == 127                          # the block's largest weight maps to ±127
    Wd = oracle.q8_dequantize(codes, scales)
    assert np.abs(Wd - W).max() <= scales.max() * 0.5 + 1e-9             # round to nearest: half a step
    c2, s2 = oracle.q8_quantize(Wd)                                      # quantizing the dequantized weights is stable
    assert np.array_equal(c2, codes)


def test_synthetic_generator_is_deterministic_and_gaussian_like():
    a = oracle.synth(9, 3, 0.02, 200000)
    assert np.array_equal(a, oracle.synth(9, 3, 0.02, 200000))
    assert np.array_equal(a[1000:1010], oracle.synth(9, 3, 0.02, 10, offset=1000))
    assert abs(float(a.std()) - 0.02) < 2e-4 and abs(float(a.mean())) < 2e-4
    assert not np.array_equal(a[:100], oracle.synth(9, 4, 0.02, 100))


def getter(om, cfg):
    from test_decoder_gpu import weight_getter
    return weight_getter(om, cfg)


@pytest.mark.parametrize("kind", ["llama", "deepseek"])
def test_native_oracle_model_equals_layer_stack_over_oracle_ops(kind):
    """Two independent restatements of DecoderOnlyModel.forward agree bit for bit, and the
    KV-cached step equals the reference's full re-forward of the context."""
    cfg = DecoderConfig(kind, 256, 24, 64, 4, 2, 176, q_rank=32 if kind == "deepseek" else 0, kv_rank=16 if kind == "deepseek" else 0)
    om = oracle.OracleModel(kind, 256, 24, 64, 4, 2, 176, cfg.q_rank, cfg.kv_rank, seed=3)
    model = build_model(cfg, getter(om, cfg))
    ids = [5, 9, 200, 31, 7, 0, 255]
    a, b = model.forward(ids).numpy(), om.forward(ids)
    assert a.shape == (7, 256) and np.all(np.isfinite(a))                    # LlamaModelTest.java:65-101
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    t_full, l_full = om.generate_greedy(ids, 6, use_cache=False)
    t_kv, l_kv = om.generate_greedy(ids, 6, use_cache=True)
    assert np.array_equal(t_full, t_kv) and np.array_equal(l_full.view(np.uint32), l_kv.view(np.uint32))
    assert TextGenerator.generate(model.forward, 24, ids, 6, 1.0, 1)[7:] == list(t_full)
    with pytest.raises(ValueError):
        model.forward([256])                                                 # Embedding range check
    with pytest.raises(oracle.OracleError):
        om.forward(list(range(25)))                                          # seqLen > maxSeqLen


def test_weight_draw_order_follows_the_reference_constructors():
    """Embedding and the stack both start from Random(seed); the LM head uses Random(seed+1)."""
    om = oracle.OracleModel("llama", 16, 8, 8, 2, 2, 24, seed=42)
    r = oracle.JRandom(42)
    assert np.array_equal(om.weight("emb"), r.tensor_random(16, 8).ravel())
    r = oracle.JRandom(42)
    for layer in range(2):
        for name, shape in (("Wq", (8, 8)), ("Wk", (8, 8)), ("Wv", (8, 8)), ("Wo", (8, 8)), ("Wg", (8, 24)), ("Wu", (8, 24)), ("Wd", (24, 8))):
            assert np.array_equal(om.weight(name, layer), r.tensor_random(*shape).ravel()), (name, layer)
    assert np.array_equal(om.weight("Wlm"), oracle.JRandom(43).tensor_random(8, 16).ravel())
    assert np.all(om.weight("g1", 0) == 1.0) and not om.weight("bd", 1).any() and not om.weight("blm").any()


def test_decoder_config_validation():
    with pytest.raises(ValueError):
        DecoderConfig("llama", 256, 16, 30, 4, 1, 64)          # dModel % nHeads
    with pytest.raises(ValueError):
        DecoderConfig("llama", 256, 16, 12, 4, 1, 64)          # odd head dim
    with pytest.raises(ValueError):
        DecoderConfig("deepseek", 256, 16, 32, 4, 1, 64)       # ranks missing
    with pytest.raises(ValueError):
        DecoderConfig("llama", 0, 16, 32, 4, 1, 64)
    c = DecoderConfig("llama", 32000, 2176, 4096, 32, 32, 11008)
    assert c.q8_weight_bytes() == 7432962048 and c.kv_bytes_per_position() == 1048576
