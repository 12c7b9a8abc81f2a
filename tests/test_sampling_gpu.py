"""Device sampling (op 74) against the oracle's restatement of TextGenerator.sampleFromLogits
(models/TextGenerator.java:104-151), and sampled generation end to end."""
import numpy as np
import pytest

import oracle
from deepj_b200.compute_graph import OP_ARGMAX_ROWS, OP_SAMPLE_TOPK, float_bits
from deepj_b200.decoder import DecoderConfig, Q8Decoder
from test_decoder_gpu import weight_getter
from test_q8_gpu import Dev

pytestmark = pytest.mark.gpu


@pytest.fixture()
def dev():
    d = Dev(3 << 20)
    yield d
    d.close()


@pytest.mark.parametrize("V,top_k,temperature", [(32000, 1, 1.0), (32000, 5, 0.7), (32000, 40, 1.0), (32000, 1024, 2.5),
                                                 (7, 40, 1.0), (1000, 1000, 0.3), (257, 64, 1.3),
                                                 # more than 1024 candidates, and the reference's topK = 0 = whole vocabulary
                                                 (32000, 0, 1.0), (32000, 2000, 0.9), (50257, 0, 1.3), (1500, 1025, 1.0), (7, 0, 0.5)])
def test_sample_topk_matches_oracle(dev, V, top_k, temperature):
    rng = np.random.default_rng(V + top_k)
    rows = 6
    logits = rng.standard_normal((rows, V)).astype(np.float32) * 3.0
    logits[1] = np.round(logits[1] * 2.0) / 2.0              # many exact ties: the stable order decides
    logits[2, :] = 0.25                                      # all equal: the lowest indices are the top k
    logits[3, ::3] = -0.0
    logits[3, 1::3] = 0.0                                    # Float.compare puts −0.0 below +0.0
    r = np.asarray([0.0, 0.37, 0.999999, 0.5, 0.81, 1.0 - 2.0 ** -24], dtype=np.float32)
    lb, rb, ob = dev.buf(rows * V, logits), dev.buf(rows, r), dev.buf(rows)
    dev.flush([OP_SAMPLE_TOPK, lb, rb, ob, rows, V, top_k, float_bits(temperature)])
    got = dev.get(ob, rows).astype(np.int64)
    want = np.asarray([oracle.sample_topk(logits[i], temperature, top_k, float(r[i])) for i in range(rows)])
    assert np.array_equal(got, want), (got, want)


@pytest.mark.parametrize("V", [7, 1000, 4096, 32000, 50257])
def test_argmax_rows_is_the_first_index_of_a_stable_descending_sort(dev, V):
    """Greedy pick (TextGenerator with topK = 1): lowest index among equal maxima, −0.0 below +0.0, NaN above
    everything — also when the row is reduced by several CTAs (long rows) and the maxima sit in different slices."""
    rng = np.random.default_rng(V)
    rows = 5
    x = rng.standard_normal((rows, V)).astype(np.float32)
    x[1, :] = 0.5                                                        # all equal → index 0
    x[2, V - 1] = 9.0; x[2, V // 2] = 9.0; x[2, 3] = 9.0                 # equal maxima in different slices → index 3
    x[3, :] = -1.0; x[3, V - 2] = -0.0; x[3, V // 3] = 0.0               # +0.0 beats −0.0
    x[4, V // 2 + 1] = np.nan                                            # NaN sorts above +inf
    xb, ob = dev.buf(rows * V, x), dev.buf(rows)
    dev.flush([OP_ARGMAX_ROWS, xb, ob, rows, V])
    got = dev.get(ob, rows).astype(np.int64)
    want = np.asarray([oracle.greedy_pick(x[i]) for i in range(rows)])
    assert np.array_equal(got, want), (got, want)
    assert list(got[1:]) == [0, 3, V // 3, V // 2 + 1]


def test_sampler_rejects_what_it_does_not_cover(dev):
    lb, rb, ob = dev.buf(8), dev.buf(1), dev.buf(1)
    for top_k, t in ((-1, 1.0), (4, 0.0), (4, -1.0)):
        with pytest.raises(Exception):
            dev.flush([OP_SAMPLE_TOPK, lb, rb, ob, 1, 8, top_k, float_bits(t)])


def test_sampled_generation_matches_oracle_loop():
    """generate(): Random(seed).nextFloat() per token on the host, everything else on the device; the same loop
    over the oracle's KV-cached logits picks the same tokens."""
    cfg = DecoderConfig("llama", 256, 64, 128, 4, 2, 352)
    om = oracle.OracleModel("llama", 256, 64, 128, 4, 2, 352, seed=17)
    dec = Q8Decoder(cfg, batch=1)
    dec.load_weights(weight_getter(om, cfg))
    om.apply_q8()
    prompt = list(np.random.default_rng(9).integers(0, 256, size=9))
    for temperature, top_k, seed in ((0.8, 20, 5), (1.5, 3, 11), (1.1, 0, 3)):
        got = dec.generate(prompt, 12, temperature=temperature, top_k=top_k, seed=seed)
        rnd = oracle.JRandom(seed)
        om.reset_cache()
        lg = None
        for t in prompt:
            lg = om.decode_step(int(t))
        want = []
        for i in range(12):
            tok = oracle.sample_topk(lg, temperature, top_k, rnd.next_float())
            want.append(tok)
            if i + 1 < 12:
                lg = om.decode_step(tok)
        assert np.array_equal(got, np.asarray(want)), (got, want)
    dec.close()
