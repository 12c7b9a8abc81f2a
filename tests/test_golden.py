"""Committed golden vectors of the tiny reference configuration (made by
tests/golden/make_golden.py from the CPU oracle): the oracle must keep reproducing them,
and the CUDA decoder must produce the same greedy tokens."""
import hashlib
import json
import os

import numpy as np
import pytest

import oracle

G = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "tiny_llama_c1.json")))


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def model():
    c = G["config"]
    return oracle.OracleModel("llama", c["vocab"], c["max_seq"], c["d_model"], c["heads"], c["layers"], c["d_ff"], seed=c["weight_seed"])


def test_oracle_reproduces_golden_vectors():
    r = oracle.JRandom(G["config"]["prompt_seed"])
    assert [r.next_int(256) for _ in range(32)] == G["prompt"]
    om = model()
    assert [float(x) for x in om.weight("emb")[:8]] == G["first_weights_emb"]
    cq, sq = oracle.q8_quantize(om.weight("Wq", 0).reshape(256, 256))
    cd, sd = oracle.q8_quantize(om.weight("Wd", 3).reshape(688, 256))
    assert (sha(cq), sha(sq), sha(cd), sha(sd)) == (G["q8_Wq0_codes_sha256"], G["q8_Wq0_scales_sha256"],
                                                    G["q8_Wd3_codes_sha256"], G["q8_Wd3_scales_sha256"])
    toks, logits = om.generate_greedy(G["prompt"], 64, use_cache=True)
    assert [int(t) for t in toks] == G["tokens_fp32"]
    assert [float(x) for x in logits[0, :8]] == G["logits_fp32_step0_head"]
    om.apply_q8()
    toks, logits = om.generate_greedy(G["prompt"], 64, use_cache=True)
    assert [int(t) for t in toks] == G["tokens_q8"] and sha(logits) == G["logits_q8_sha256"]


@pytest.mark.gpu
def test_cuda_decoder_reproduces_golden_tokens_and_q8_arrays():
    from deepj_b200.decoder import DecoderConfig, Q8Decoder
    from test_decoder_gpu import weight_getter
    c = G["config"]
    cfg = DecoderConfig("llama", c["vocab"], c["max_seq"], c["d_model"], c["heads"], c["layers"], c["d_ff"])
    om = model()
    dec = Q8Decoder(cfg, batch=1)
    try:
        dec.load_weights(weight_getter(om, cfg))
        codes, scales = dec.q8_arrays("Wqkv.0")
        assert sha(codes[:256]) == G["q8_Wq0_codes_sha256"] and sha(scales[:256]) == G["q8_Wq0_scales_sha256"]
        codes, scales = dec.q8_arrays("Wd.3")
        assert sha(codes) == G["q8_Wd3_codes_sha256"] and sha(scales) == G["q8_Wd3_scales_sha256"]
        toks, logits = dec.generate_greedy(G["prompt"], 64, keep_logits=True)
        assert [int(t) for t in toks] == G["tokens_q8"]
        assert np.abs(logits[0, :8] - np.asarray(G["logits_q8_step0_head"], dtype=np.float32)).max() <= 2e-3 * G["logits_q8_range"]
    finally:
        dec.close()


GG = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "tiny_gpt.json")))


def gpt_model():
    c = GG["config"]
    return oracle.OracleModel("gpt", c["vocab"], c["max_seq"], c["d_model"], c["heads"], c["layers"], c["d_ff"], seed=c["weight_seed"])


def test_oracle_reproduces_gpt_golden_vectors():
    om = gpt_model()
    assert [float(x) for x in om.weight("pos")[:8]] == GG["first_weights_pos"]
    c1, s1 = oracle.q8_quantize(om.weight("W1", 1).reshape(128, 512))
    assert (sha(c1), sha(s1)) == (GG["q8_W1_1_codes_sha256"], GG["q8_W1_1_scales_sha256"])
    toks, logits = om.generate_greedy(GG["prompt"], 32, use_cache=True)
    assert [int(t) for t in toks] == GG["tokens_fp32"]
    assert [float(x) for x in logits[0, :8]] == GG["logits_fp32_step0_head"]
    toks_full, _ = om.generate_greedy(GG["prompt"], 4, use_cache=False)         # the reference's own loop: full re-forward
    assert [int(t) for t in toks_full] == GG["tokens_fp32"][:4]
    om.apply_q8()
    toks, logits = om.generate_greedy(GG["prompt"], 32, use_cache=True)
    assert [int(t) for t in toks] == GG["tokens_q8"] and sha(logits) == GG["logits_q8_sha256"]


@pytest.mark.gpu
def test_cuda_decoder_reproduces_gpt_golden_tokens():
    from deepj_b200.decoder import DecoderConfig, Q8Decoder
    from test_decoder_gpu import weight_getter
    c = GG["config"]
    cfg = DecoderConfig("gpt", c["vocab"], c["max_seq"], c["d_model"], c["heads"], c["layers"], c["d_ff"])
    dec = Q8Decoder(cfg, batch=1)
    try:
        dec.load_weights(weight_getter(gpt_model(), cfg))
        codes, scales = dec.q8_arrays("W1.1")
        assert sha(codes) == GG["q8_W1_1_codes_sha256"] and sha(scales) == GG["q8_W1_1_scales_sha256"]
        toks, logits = dec.generate_greedy(GG["prompt"], 32, keep_logits=True)
        assert [int(t) for t in toks] == GG["tokens_q8"]
        assert np.abs(logits[0, :8] - np.asarray(GG["logits_q8_step0_head"], dtype=np.float32)).max() <= 2e-3 * GG["logits_q8_range"]
    finally:
        dec.close()
