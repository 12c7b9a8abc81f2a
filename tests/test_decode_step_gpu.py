"""The whole-token decode kernel (op 76, `deepj_cuda_decode_plan`) against the per-operator stream.

The single kernel runs the arithmetic of the cp.async projection kernel and of the split attention kernel at the
same tile, warp and split assignments.  The per-operator path takes the TMA projection kernel wherever the
reduction length is a multiple of 128, which sums the 32-k blocks in another order and applies RMSNorm's 1/rms
after the sums, so the two paths agree to fp32 rounding (a few 1e-6 of the logit range), not bit for bit; both
are held to the CPU oracle at the tolerance of the other decoder tests, and the greedy tokens must be equal."""
import ctypes

import numpy as np
import pytest

import oracle
from deepj_b200 import _lib
from deepj_b200.compute_graph import OP_DECODE_STEP
from deepj_b200.decoder import DecoderConfig, Q8Decoder
from test_decoder_gpu import weight_getter

pytestmark = pytest.mark.gpu

PATH_TOL = 2e-5      # of the logit range: two fp32 summation orders of the same products


def run_steps(cfg, get, prompt, n_new, fused, chunked_prompt):
    dec = Q8Decoder(cfg, batch=1, fused_step=fused)
    try:
        dec.load_weights(get)
        dec.reset()
        nxt = dec.prefill(np.asarray(prompt).reshape(1, -1), chunked=chunked_prompt)
        toks, rows = [int(nxt[0])], [dec.logits()[0].copy()]
        for _ in range(n_new - 1):
            nxt = dec.step(nxt)
            toks.append(int(nxt[0]))
            rows.append(dec.logits()[0].copy())
        st = dec.stats()
        assert st["device_error"] == 0, st
        return np.asarray(toks), np.stack(rows), st
    finally:
        dec.close()


@pytest.mark.parametrize("d,heads,d_ff,layers,vocab,prompt_len", [
    (256, 4, 1024, 2, 512, 20),        # head dim 64
    (256, 2, 512, 3, 300, 9),          # head dim 128, a vocabulary that is not a multiple of the row tile
    (128, 4, 352, 2, 256, 40),         # head dim 32; odd 32-block count (K = 352 → 11 blocks) in the down projection
    (512, 8, 1408, 2, 1000, 70),       # more tiles than virtual CTAs in no phase, more warps than 64-k pairs in none
])
def test_single_kernel_step_agrees_with_the_per_operator_stream(d, heads, d_ff, layers, vocab, prompt_len):
    cfg = DecoderConfig("llama", vocab, 128, d, heads, layers, d_ff)
    assert Q8Decoder.fused_step_eligible(cfg, 1)
    om = oracle.OracleModel("llama", vocab, 128, d, heads, layers, d_ff, seed=77 + d)
    get = weight_getter(om, cfg)
    prompt = list(np.random.default_rng(d + heads).integers(0, vocab, size=prompt_len))
    # token by token from position 0: every step of the fused run is the single kernel
    tok_a, log_a, st_a = run_steps(cfg, get, prompt, 10, fused=False, chunked_prompt=False)
    tok_b, log_b, st_b = run_steps(cfg, get, prompt, 10, fused=True, chunked_prompt=False)
    span_a = float(log_a.max() - log_a.min())
    assert np.array_equal(tok_a, tok_b)
    assert float(np.abs(log_a - log_b).max()) <= PATH_TOL * span_a, float(np.abs(log_a - log_b).max()) / span_a
    # and behind a chunked prompt pass (prompts of 32 tokens or more), whose cache rows the many-row kernels wrote
    if prompt_len >= 32:
        tok_c, log_c, _ = run_steps(cfg, get, prompt, 10, fused=False, chunked_prompt=True)
        tok_d, log_d, _ = run_steps(cfg, get, prompt, 10, fused=True, chunked_prompt=True)
        assert np.array_equal(tok_c, tok_d)
        assert float(np.abs(log_c[1:] - log_d[1:]).max()) <= PATH_TOL * span_a
    # the oracle agrees with both
    om.apply_q8()
    toks_o, logits_o = om.generate_greedy(prompt, 10, use_cache=True)
    span = float(logits_o.max() - logits_o.min())
    assert np.array_equal(toks_o, tok_b)
    assert float(np.abs(logits_o - log_b).max()) <= 2e-3 * span


def test_device_feedback_with_the_single_kernel_step():
    """step_device: the pick is fed back by the kernel itself (feed_back = 1); same tokens as the host loop."""
    cfg = DecoderConfig("llama", 256, 96, 256, 4, 2, 512)
    om = oracle.OracleModel("llama", 256, 96, 256, 4, 2, 512, seed=5)
    dec = Q8Decoder(cfg, batch=1, fused_step=True)
    try:
        dec.load_weights(weight_getter(om, cfg))
        prompt = [3, 9, 250, 77, 1]
        host = dec.generate_greedy(prompt, 24)
        dec.reset()
        nxt = dec.prefill(np.asarray(prompt).reshape(1, -1))
        dec.set_tokens(nxt)
        dec.step_device(23)
        assert int(dec.next_tokens()[0]) == int(host[-1])
        st = dec.stats()
        assert st["device_error"] == 0
        assert dec.position == len(prompt) + 23
    finally:
        dec.close()


def test_plan_is_validated_and_dies_with_what_it_references():
    lib = _lib.load()
    cfg = DecoderConfig("llama", 256, 32, 128, 4, 1, 352)
    om = oracle.OracleModel("llama", 256, 32, 128, 4, 1, 352, seed=2)
    dec = Q8Decoder(cfg, batch=1, fused_step=True)
    try:
        dec.load_weights(weight_getter(om, cfg))
        dec.reset()
        dec.step([7])
        I = dec.ids
        good = [1, 1, 4, 32, 0, I["tok"], I["pos"], I["emb"], I["cos"], I["sin"], I["kv"], I["x"], I["x2"], I["qkv"], I["att"], I["h"],
                I["logits"], I["next"], I["gF"], I["Wlm"], I["blm"],
                I["g1.0"], I["Wqkv.0"], I["Wo.0"], I["g2.0"], I["Wg.0"], I["bg.0"], I["Wu.0"], I["bu.0"], I["Wd.0"], I["bd.0"]]

        def plan(desc, pid):
            a = np.asarray(desc, dtype=np.int32)
            return lib.deepj_cuda_decode_plan(pid, a.ctypes.data, a.size)

        base = 9 << 24
        assert plan(good[:-1], base) != 0 and "length" in lib.deepj_cuda_last_error().decode()
        bad = list(good); bad[22], bad[23] = good[23], good[22]                 # Wqkv and Wo swapped: shapes do not fit
        assert plan(bad, base) != 0 and "expected" in lib.deepj_cuda_last_error().decode()
        bad = list(good); bad[3] = 48                                           # a head dim the kernel has no form for
        assert plan(bad, base) != 0
        assert plan(good, base) == 0
        assert plan(good, base) != 0 and "already exists" in lib.deepj_cuda_last_error().decode()
        cmd = np.asarray([OP_DECODE_STEP, base, 0], dtype=np.int32)
        _lib.check(lib.deepj_cuda_flush_ops(cmd.ctypes.data, cmd.size))
        # an id that is not a plan, a bad flag
        cmd2 = np.asarray([OP_DECODE_STEP, I["x"], 0], dtype=np.int32)
        assert lib.deepj_cuda_flush_ops(cmd2.ctypes.data, cmd2.size) != 0
        cmd3 = np.asarray([OP_DECODE_STEP, base, 2], dtype=np.int32)
        assert lib.deepj_cuda_flush_ops(cmd3.ctypes.data, cmd3.size) != 0
        # releasing something the plan references: the next flush fails before anything is launched
        _lib.check(lib.deepj_cuda_release_buffers((ctypes.c_int32 * 1)(I["bd.0"]), 1))
        dec._owned.remove(I["bd.0"])
        assert lib.deepj_cuda_flush_ops(cmd.ctypes.data, cmd.size) != 0
        assert "released" in lib.deepj_cuda_last_error().decode()
        _lib.check(lib.deepj_cuda_release_buffers((ctypes.c_int32 * 1)(base), 1))
        st = dec.stats()
        assert st["device_error"] == 0
    finally:
        dec.close()
