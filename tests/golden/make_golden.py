"""Generates tests/golden/tiny_llama_c1.json and tests/golden/tiny_gpt.json from the CPU oracle.

The reference (Java) cannot run in the build environment and its own tests hold no
logits or token goldens, so these vectors pin the ORACLE's output for the tiny reference
configuration (vocab 256, dModel 256, 8 heads, 4 blocks, dFF 688, context 256,
java.util.Random(42) weights x0.1, prompt = 32 draws of Random(7).nextInt(256), 64 greedy
tokens).  Run from the repository root:  python tests/golden/make_golden.py
"""
import hashlib
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import oracle  # noqa: E402


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main():
    om = oracle.OracleModel("llama", 256, 256, 256, 8, 4, 688, seed=42)
    r = oracle.JRandom(7)
    prompt = [r.next_int(256) for _ in range(32)]
    toks_a, logits_a = om.generate_greedy(prompt, 64, use_cache=True)          # oracle A: fp32 weights
    wq = om.weight("Wq", 0).reshape(256, 256)
    wd = om.weight("Wd", 3).reshape(688, 256)
    cq, sq = oracle.q8_quantize(wq)
    cd, sd = oracle.q8_quantize(wd)
    om.apply_q8()
    toks_b, logits_b = om.generate_greedy(prompt, 64, use_cache=True)          # oracle B: dequantized Q8 weights
    out = {
        "config": {"kind": "llama", "vocab": 256, "max_seq": 256, "d_model": 256, "heads": 8, "layers": 4, "d_ff": 688,
                   "weight_seed": 42, "prompt_seed": 7},
        "prompt": prompt,
        "first_weights_emb": [float(x) for x in oracle.JRandom(42).tensor_random(1, 8).ravel()],
        "tokens_fp32": [int(t) for t in toks_a],
        "tokens_q8": [int(t) for t in toks_b],
        "logits_fp32_step0_head": [float(x) for x in logits_a[0, :8]],
        "logits_q8_step0_head": [float(x) for x in logits_b[0, :8]],
        "logits_q8_sha256": sha(logits_b),
        "logits_q8_range": float(logits_b.max() - logits_b.min()),
        "q8_Wq0_codes_sha256": sha(cq), "q8_Wq0_scales_sha256": sha(sq),
        "q8_Wd3_codes_sha256": sha(cd), "q8_Wd3_scales_sha256": sha(sd),
        "q8_vs_fp32_max_logit_diff": float(np.abs(logits_a - logits_b).max()),
    }
    with open(os.path.join(HERE, "tiny_llama_c1.json"), "w") as f:
        json.dump(out, f, indent=1)
    print("wrote tiny_llama_c1.json; q8 tokens == fp32 tokens:", out["tokens_fp32"] == out["tokens_q8"])


def main_gpt():
    """A small GPT as `new GPTModel(cfg, 42)` builds it (vocab 256, context 128, dModel 128, 4 heads, 2 blocks, dFF 512,
    initScale 0.2), prompt = 16 draws of Random(7).nextInt(256), 32 greedy tokens."""
    cfg = dict(vocab=256, max_seq=128, d_model=128, heads=4, layers=2, d_ff=512)
    om = oracle.OracleModel("gpt", 256, 128, 128, 4, 2, 512, seed=42)
    r = oracle.JRandom(7)
    prompt = [r.next_int(256) for _ in range(16)]
    toks_a, logits_a = om.generate_greedy(prompt, 32, use_cache=True)
    c1, s1 = oracle.q8_quantize(om.weight("W1", 1).reshape(128, 512))
    pos_head = [float(x) for x in om.weight("pos")[:8]]
    om.apply_q8()
    toks_b, logits_b = om.generate_greedy(prompt, 32, use_cache=True)
    out = {
        "config": dict(cfg, kind="gpt", weight_seed=42, prompt_seed=7, init_scale=0.2),
        "prompt": prompt,
        "first_weights_pos": pos_head,
        "tokens_fp32": [int(t) for t in toks_a],
        "tokens_q8": [int(t) for t in toks_b],
        "logits_fp32_step0_head": [float(x) for x in logits_a[0, :8]],
        "logits_q8_step0_head": [float(x) for x in logits_b[0, :8]],
        "logits_q8_sha256": sha(logits_b),
        "logits_q8_range": float(logits_b.max() - logits_b.min()),
        "q8_W1_1_codes_sha256": sha(c1), "q8_W1_1_scales_sha256": sha(s1),
    }
    with open(os.path.join(HERE, "tiny_gpt.json"), "w") as f:
        json.dump(out, f, indent=1)
    print("wrote tiny_gpt.json; q8 tokens == fp32 tokens:", out["tokens_fp32"] == out["tokens_q8"])


if __name__ == "__main__":
    main()
    main_gpt()
