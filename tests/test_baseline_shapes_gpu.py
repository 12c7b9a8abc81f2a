"""Parity at the BASELINE configurations' real widths.

C2 (the Q8 matmul operator sweep): K = 4096, N in {4096, 11008}, M in {1, 4, 16, 64, 512, 2048}, x ~ N(0,1) and
W ~ N(0, 0.02) drawn from ONE generator seeded 1 (x first, then W), against the oracle's matmul on the dequantized
weights — on 320 sampled output columns per case (the first 64, the last 64 and 192 spread between), which keeps
the CPU side to seconds; the sampled columns see every kernel the dispatcher picks for the row count.

C3 / C4 / C5 (Llama-1B, DeepSeek and Llama-7B shapes) at reduced depth: 2 blocks, full width, synthetic weights
that the oracle generates bit-identically; a 48-token prompt through the chunked prefill path, then 8 greedy
decode steps; Q8 codes bit-exact on one block, logits within 2e-3 of the logit range, identical tokens — for the
fp32 and the fp16 K/V cache, and (Llama shapes) for the whole-token kernel."""
import numpy as np
import pytest

import oracle
from deepj_b200.compute_graph import OP_Q8_LINEAR
from parity_util import LOGIT_TOL, reduced_depth_parity_variants
from test_q8_gpu import MANY_ROW_FLOOR, Dev, close

pytestmark = pytest.mark.gpu

BASELINE_SHAPES = {
    "llama1b": dict(kind="llama", vocab=32000, d=2048, heads=32, layers=22, d_ff=5632, seed=3, std=0.02),
    "deepseek": dict(kind="deepseek", vocab=32000, d=2048, heads=16, layers=16, d_ff=5632, seed=5, std=0.02, q_rank=1024, kv_rank=512),
    "llama7b": dict(kind="llama", vocab=32000, d=4096, heads=32, layers=32, d_ff=11008, seed=9, std=0.02),
}


@pytest.fixture()
def dev():
    d = Dev(11 << 20)
    yield d
    d.close()


@pytest.fixture(scope="module")
def sweep_weights():
    """One draw per N, shared by the M cases: seed 1, x for the largest M first, then W."""
    cache = {}

    def get(N):
        if N not in cache:
            rng = np.random.default_rng(1)
            x = rng.standard_normal((2048, 4096)).astype(np.float32)
            W = (rng.standard_normal((4096, N)) * 0.02).astype(np.float32)
            cols = np.unique(np.concatenate([np.arange(64), N - 64 + np.arange(64), np.linspace(64, N - 65, 192).astype(np.int64)]))
            codes, scales = oracle.q8_quantize(np.ascontiguousarray(W[:, cols]))
            cache[N] = (x, W, cols, oracle.q8_dequantize(codes, scales))
        return cache[N]
    return get


@pytest.mark.parametrize("N", [4096, 11008])
@pytest.mark.parametrize("M", [1, 4, 16, 64, 512, 2048])
def test_operator_sweep_shapes_match_oracle(dev, sweep_weights, M, N):
    K = 4096
    x_all, W, cols, Wq_cols = sweep_weights(N)
    x = np.ascontiguousarray(x_all[:M])
    q = dev.q8(W)
    xb, ob = dev.buf(M * K, x), dev.buf(M * N)
    dev.flush([OP_Q8_LINEAR, xb, 0, K, -1, 0, q, -1, -1, 0, 0, ob, 0, N, M])
    got = dev.get(ob, M * N).reshape(M, N)[:, cols]
    expected = oracle.matmul(x, Wq_cols)          # quantization is per output column: a column subset quantizes to the same codes
    close(expected, got, floor=MANY_ROW_FLOOR if M >= 5 else 0.0)


@pytest.mark.parametrize("name", ["llama1b", "deepseek", "llama7b"])
def test_reduced_depth_baseline_config_matches_oracle(name):
    # the per-operator step with the fp32 and the fp16 K/V cache; Llama shapes also as the single whole-token kernel
    variants = [dict(kv_dtype="f32"), dict(kv_dtype="f16")]
    if BASELINE_SHAPES[name]["kind"] == "llama":
        variants.append(dict(kv_dtype="f32", fused_step=True))
    for res in reduced_depth_parity_variants(BASELINE_SHAPES[name], variants, layers=2, prompt_len=48, n_new=8):
        assert res["tokens_equal"], res
        assert res["max_err_over_range"] <= LOGIT_TOL, res
