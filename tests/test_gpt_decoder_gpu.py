"""The GPT family on the fused Q8 path: op 75 (LayerNorm → Q8 projection → GELU) against a numpy
restatement, and `Q8Decoder(kind="gpt")` against the numpy GPT forward pass of tests/gpt_ref.py run
with the same dequantized Q8 weights (full re-forward per token, as the reference's TextGenerator does)."""
import numpy as np
import pytest

import gpt_ref
import oracle
from deepj_b200.compute_graph import OP_Q8_LINEAR_LN, float_bits
from deepj_b200.decoder import DecoderConfig, Q8Decoder
from test_q8_gpu import MANY_ROW_FLOOR, Dev, close

pytestmark = pytest.mark.gpu

LOGIT_TOL = 2e-3
MATMULS = ("Wq", "Wk", "Wv", "Wo", "W1", "W2", "Wlm")


@pytest.fixture()
def dev():
    d = Dev(5 << 20)
    yield d
    d.close()


# rows 1-4: the GEMV with the norm and the activation fused; 6, 16 and 40: the 16-row kernel behind a
# normalising pass; 300: the tcgen05 path; K = 100: the FMA fallback (no 32-element blocks)
@pytest.mark.parametrize("M,K,N", [(1, 256, 96), (2, 512, 40), (4, 4096, 64), (3, 768, 33), (6, 512, 72), (16, 256, 128),
                                   (40, 256, 300), (300, 256, 300), (1, 100, 24), (5, 100, 24)])
@pytest.mark.parametrize("act", [0, 1])
def test_layernorm_q8_linear_gelu(dev, M, K, N, act):
    rng = np.random.default_rng(M * 1000 + K + N + act)
    x = (rng.standard_normal((M, K)) * 1.5 + 0.3).astype(np.float32)
    W = (rng.standard_normal((K, N)) * 0.05).astype(np.float32)
    gamma = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float32)
    beta = (0.1 * rng.standard_normal(K)).astype(np.float32)
    bias = (0.2 * rng.standard_normal(N)).astype(np.float32)
    Wq = oracle.q8_dequantize(*oracle.q8_quantize(W))
    expected = oracle.matmul(gpt_ref.layer_norm(x, gamma, beta).astype(np.float32), Wq) + bias
    if act:
        expected = gpt_ref.gelu(expected)
    q, xb, ob = dev.q8(W), dev.buf(M * K, x), dev.buf(M * N)
    gb, bb, cb = dev.buf(K, gamma), dev.buf(K, beta), dev.buf(N, bias)
    dev.flush([OP_Q8_LINEAR_LN, xb, 0, K, gb, bb, float_bits(1e-5), q, cb, -1, 0, 0, ob, 0, N, M, act])
    close(expected, dev.get(ob, M * N).reshape(M, N), floor=MANY_ROW_FLOOR if M >= 5 else 0.0)


def test_op75_without_norm_and_with_residual(dev):
    """gamma = beta = −1 is a plain projection; a residual is added after the bias; an activation together with a
    residual, or a norm with only one of its two vectors, is refused before anything is launched."""
    rng = np.random.default_rng(9)
    M, K, N = 2, 128, 48
    x = rng.standard_normal((M, K)).astype(np.float32)
    W = (rng.standard_normal((K, N)) * 0.05).astype(np.float32)
    res = rng.standard_normal((M, N)).astype(np.float32)
    Wq = oracle.q8_dequantize(*oracle.q8_quantize(W))
    q, xb, ob, rb = dev.q8(W), dev.buf(M * K, x), dev.buf(M * N), dev.buf(M * N, res)
    dev.flush([OP_Q8_LINEAR_LN, xb, 0, K, -1, -1, 0, q, -1, rb, 0, N, ob, 0, N, M, 0])
    close(oracle.matmul(x, Wq) + res, dev.get(ob, M * N).reshape(M, N))
    dev.flush([OP_Q8_LINEAR_LN, xb, 0, K, -1, -1, 0, q, -1, -1, 0, 0, ob, 0, N, M, 1])
    close(gpt_ref.gelu(oracle.matmul(x, Wq)), dev.get(ob, M * N).reshape(M, N))
    gb = dev.buf(K, np.ones(K))
    for bad in ([OP_Q8_LINEAR_LN, xb, 0, K, -1, -1, 0, q, -1, rb, 0, N, ob, 0, N, M, 1],
                [OP_Q8_LINEAR_LN, xb, 0, K, gb, -1, float_bits(1e-5), q, -1, -1, 0, 0, ob, 0, N, M, 0],
                [OP_Q8_LINEAR_LN, xb, 0, K, -1, -1, 0, q, -1, -1, 0, 0, ob, 0, N, M, 2]):
        with pytest.raises(RuntimeError):
            dev.flush(bad)


def q8_weights(w):
    """The reference weights with every matmul matrix replaced by dequant(Q8(W)) — what the device computes with."""
    out = dict(w)
    for (name, layer), a in w.items():
        if name in MATMULS:
            out[(name, layer)] = oracle.q8_dequantize(*oracle.q8_quantize(a)).astype(np.float32)
    return out


def reference_greedy(wq, prompt, n_new, d, heads, layers):
    ids, rows = list(prompt), []
    for _ in range(n_new):
        logits = gpt_ref.forward(wq, ids, d, heads, layers)[-1]
        rows.append(logits)
        ids.append(int(np.argmax(logits)))
    return np.asarray(ids[len(prompt):]), np.stack(rows)


def test_gpt_decoder_matches_the_numpy_forward():
    V, S, d, H, L, F = 160, 48, 64, 4, 2, 160
    cfg = DecoderConfig("gpt", V, S, d, H, L, F)
    w, get = gpt_ref.make_weights(V, S, d, H, L, F, seed=21)
    wq = q8_weights(w)
    prompt = list(np.random.default_rng(3).integers(0, V, size=9))
    toks_ref, logits_ref = reference_greedy(wq, prompt, 12, d, H, L)
    dec = Q8Decoder(cfg, batch=1)
    try:
        dec.load_weights(get)
        codes, scales = dec.q8_arrays("W1.1")
        co, so = oracle.q8_quantize(w[("W1", 1)])
        assert np.array_equal(codes, co) and np.array_equal(scales.view(np.uint32), so.view(np.uint32))
        toks, logits = dec.generate_greedy(prompt, 12, keep_logits=True)
        span = float(logits_ref.max() - logits_ref.min())
        assert float(np.abs(logits - logits_ref).max()) <= LOGIT_TOL * span
        assert np.array_equal(toks, toks_ref)
        st = dec.stats()
        assert st["graph_replays"] > 0 and st["device_error"] == 0
    finally:
        dec.close()


def test_gpt_chunked_prefill_equals_token_by_token_and_the_reference():
    """Prompt chunks (tcgen05 GEMMs behind the normalising pass, chunk attention, position rows per token) leave the
    same cache and logits as one step per position; two sequences, three chunks with a ragged last one."""
    V, S, d, H, L, F = 256, 360, 128, 4, 2, 256
    cfg = DecoderConfig("gpt", V, S, d, H, L, F)
    w, get = gpt_ref.make_weights(V, S, d, H, L, F, seed=8)
    prompts = np.random.default_rng(6).integers(0, V, size=(2, 330))     # chunks of 150, 150, 30: 300 rows, then 60

    def run(chunked):
        dec = Q8Decoder(cfg, batch=2)
        dec.PREFILL_CHUNK = 150
        dec.load_weights(get)
        dec.reset()
        nxt = dec.prefill(prompts, chunked=chunked)
        toks, rows = [nxt.copy()], [dec.logits().copy()]
        for _ in range(5):
            nxt = dec.step(nxt)
            toks.append(nxt.copy())
            rows.append(dec.logits().copy())
        st = dec.stats()
        dec.close()
        assert st["device_error"] == 0
        return np.stack(toks, axis=1), np.stack(rows, axis=1)

    tok_a, log_a = run(False)
    tok_b, log_b = run(True)
    span = float(log_a.max() - log_a.min())
    assert float(np.abs(log_a - log_b).max()) <= 2e-4 * span
    assert np.array_equal(tok_a, tok_b)
    wq = q8_weights(w)
    for b in range(2):
        toks_ref, logits_ref = reference_greedy(wq, list(prompts[b]), 6, d, H, L)
        assert np.array_equal(toks_ref, tok_b[b])
        assert float(np.abs(logits_ref - log_b[b]).max()) <= LOGIT_TOL * span


def test_gpt_checkpoint_import(tmp_path):
    """A GPT model written in ModelSerializer's format (GPTModel.parameters() order) loads through
    deepj_b200.checkpoint and decodes like the weights it was written from."""
    from deepj_b200 import checkpoint
    V, S, d, H, L, F = 96, 32, 64, 2, 2, 96
    cfg = DecoderConfig("gpt", V, S, d, H, L, F)
    w, get = gpt_ref.make_weights(V, S, d, H, L, F, seed=4)
    params = [np.asarray(get(name, layer), dtype=np.float32).reshape(shape) for name, layer, shape in checkpoint.parameter_layout(cfg)]
    path = tmp_path / "gpt.bin"
    checkpoint.write_parameters(path, params)
    prompt = [5, 17, 80, 3]
    outs = []
    for g in (get, checkpoint.weight_getter(cfg, path)):
        dec = Q8Decoder(cfg, batch=1)
        dec.load_weights(g)
        outs.append(np.asarray(dec.generate_greedy(prompt, 8)))
        dec.close()
    assert np.array_equal(outs[0], outs[1])


def test_gpt_decoder_matches_the_cpp_oracle_with_java_exact_weights():
    """`new GPTModel(cfg, seed)` as the oracle builds it (java.util.Random draw order, initScale 0.2): Q8 codes bit-exact,
    logits within 2e-3 of their range and the same greedy tokens over a 20-token prompt and 24 new tokens."""
    from test_decoder_gpu import run_parity
    cfg = DecoderConfig("gpt", 256, 64, 128, 4, 3, 352)
    prompt = list(np.random.default_rng(12).integers(0, 256, size=20))
    run_parity(cfg, seed=17, prompt=prompt, n_new=24)


def test_gpt_synthetic_weights_match_the_oracle_generator():
    """Device-generated synthetic GPT weights (token and position tables, the blocks' matrices) are the oracle's
    generator bit for bit, and the model decodes to the oracle's logits."""
    from test_decoder_gpu import check_q8_bit_exact
    cfg = DecoderConfig("gpt", 384, 48, 256, 4, 2, 640)
    om = oracle.OracleModel("gpt", 384, 48, 256, 4, 2, 640, seed=6, init_mode=1, std=0.05)
    dec = Q8Decoder(cfg, batch=1)
    try:
        dec.load_synthetic(6, 0.05)
        for name, dev_name, n in (("emb", "emb", 384 * 256), ("pos", "posemb", 48 * 256)):
            got = dec._download(dec.ids[dev_name], n)
            assert np.array_equal(got.view(np.uint32), om.weight(name).view(np.uint32)), name
        check_q8_bit_exact(dec, om, cfg, 1)
        om.apply_q8()
        prompt = list(np.random.default_rng(1).integers(0, 384, size=16))
        toks_o, logits_o = om.generate_greedy(prompt, 8, use_cache=True)
        toks_g, logits_g = dec.generate_greedy(prompt, 8, keep_logits=True)
        span = float(logits_o.max() - logits_o.min())
        assert float(np.abs(logits_o - logits_g).max()) <= LOGIT_TOL * span
        assert np.array_equal(toks_o, toks_g)
    finally:
        dec.close()


def test_gpt_runs_on_one_gpu_only():
    with pytest.raises(ValueError):
        Q8Decoder(DecoderConfig("gpt", 64, 32, 64, 2, 1, 64), tp_rank=0, tp_world=2)
