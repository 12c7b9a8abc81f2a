"""Reduced-depth parity check of a BASELINE configuration against the CPU oracle.

Full width (dModel, heads, dFF, vocab, qRank / kvRank as the configuration names them), a few blocks deep,
synthetic weights that the oracle and the device generate bit-identically: the prompt goes through the
product's prefill path, then greedy decode steps follow; the logits row behind every new token and the
tokens themselves are compared with the oracle's KV-cached decode of the same model with dequantized Q8
weights.  Used by tests/test_baseline_shapes_gpu.py and, before the timed region, by bench.py at every
number of GPUs (tensor-parallel ranks all compare their tokens; rank 0 alone holds the oracle).

Test infrastructure: imports the oracle, so the package never imports this module.
"""
from __future__ import annotations

import time

import numpy as np

import oracle
from deepj_b200.decoder import DecoderConfig, Q8Decoder

LOGIT_TOL = 2e-3      # max-abs-err relative to the logit range


def reduced_config(w: dict, layers: int, max_seq: int) -> DecoderConfig:
    return DecoderConfig(w["kind"], w["vocab"], max_seq, w["d"], w["heads"], layers, w["d_ff"], w.get("q_rank", 0), w.get("kv_rank", 0))


def check_q8_codes(dec: Q8Decoder, om, cfg: DecoderConfig, layer: int) -> None:
    """Device Q8 codes and scales of one block equal the oracle quantizer's, bit for bit (one GPU only)."""
    shapes = {n: (k, w) for n, k, w in cfg.matmul_shapes()}
    for obj, K, names in dec._layer_plan():
        codes, scales = dec.q8_arrays(f"{obj}.{layer}")
        col = 0
        for nm in names:
            k, n = shapes[nm]
            co, so = oracle.q8_quantize(om.weight(nm, layer).reshape(k, n))
            assert np.array_equal(codes[col:col + n], co), f"{nm} codes differ"
            assert np.array_equal(scales[col:col + n].view(np.uint32), so.view(np.uint32)), f"{nm} scales differ"
            col += n


def reduced_depth_parity(w: dict, layers: int = 2, prompt_len: int = 48, n_new: int = 8, rank: int = 0, world: int = 1,
                         device: int = 0, tp_slot_floats: int = 0, id_base: int = 3 << 24, check_codes: bool = True,
                         kv_dtype: str = "f32", fused_step=None) -> dict:
    """One variant of the product against the oracle; see `reduced_depth_parity_variants`."""
    return reduced_depth_parity_variants(w, [dict(kv_dtype=kv_dtype, fused_step=bool(fused_step))], layers, prompt_len, n_new, rank, world,
                                         device, tp_slot_floats, id_base, check_codes)[0]


def reduced_depth_parity_variants(w: dict, variants, layers: int = 2, prompt_len: int = 48, n_new: int = 8, rank: int = 0,
                                  world: int = 1, device: int = 0, tp_slot_floats: int = 0, id_base: int = 3 << 24,
                                  check_codes: bool = True):
    """Runs every variant of the product (dicts of `kv_dtype`, `fused_step`) on the GPU, then the oracle once, and
    returns one {"max_err_over_range", "tokens_equal", "tolerance", "checked", "seconds"} per variant.  Under tensor
    parallelism (world > 1) the exchange buffers must already be connected (`deepj_b200.tp.connect`) with slots of at
    least prompt_len × dModel floats; every rank calls this, rank 0 alone holds the oracle."""
    t_start = time.perf_counter()
    max_seq = prompt_len + n_new + 8
    cfg = reduced_config(w, layers, max_seq)
    prompt = np.random.default_rng(w["seed"] + 1000).integers(0, w["vocab"], size=prompt_len)
    runs = []
    dec = None
    try:
        for i, v in enumerate(variants):
            if dec is not None:
                dec.close()
            dec = Q8Decoder(cfg, batch=1, device=device, id_base=id_base + (i << 20), tp_rank=rank, tp_world=world,
                            tp_slot_floats=tp_slot_floats, fused_step=v.get("fused_step", False), kv_dtype=v.get("kv_dtype", "f32"))
            dec.load_synthetic(w["seed"], w["std"])
            if world > 1:
                from deepj_b200 import tp
                tp.barrier()          # waits for a peer are bounded: start stepping together
            toks_g, logits_g = dec.generate_greedy(prompt, n_new, keep_logits=True)
            runs.append((toks_g, logits_g, dec.stats()["device_error"], dec.fused_step, dec.kv_dtype))
        toks_o = np.zeros(n_new, dtype=np.int64)
        errs = [0.0] * len(runs)
        if rank == 0:
            om = oracle.OracleModel(cfg.kind, cfg.vocab_size, cfg.max_seq_len, cfg.d_model, cfg.n_heads, cfg.n_layers, cfg.d_ff,
                                    cfg.q_rank, cfg.kv_rank, seed=w["seed"], init_mode=1, std=w["std"])
            if check_codes and world == 1:
                check_q8_codes(dec, om, cfg, layers - 1)
            om.apply_q8()
            t, logits_o = om.generate_greedy(list(prompt), n_new, use_cache=True)
            toks_o = np.asarray(t, dtype=np.int64)
            span = float(logits_o.max() - logits_o.min())
            errs = [float(np.abs(logits_o - lg).max()) / span for _, lg, _, _, _ in runs]
            del om
        if world > 1:
            from deepj_b200 import tp
            toks_o = np.frombuffer(tp.all_gather_bytes(toks_o.tobytes())[0], dtype=np.int64)      # rank 0 holds the oracle's tokens
        out = []
        for (toks_g, _, dev_err, fused, kvd), err in zip(runs, errs):
            equal = bool(np.array_equal(toks_o, toks_g)) and dev_err == 0
            if world > 1:
                mine = np.asarray([int(equal)], dtype=np.int64)
                equal = all(np.frombuffer(b, dtype=np.int64)[0] == 1 for b in tp.all_gather_bytes(mine.tobytes()))
                err = tp.max_over_ranks(err)
            what = (f"{cfg.kind} d={cfg.d_model} heads={cfg.n_heads} dFF={cfg.d_ff} vocab={cfg.vocab_size}"
                    + (f" qRank={cfg.q_rank} kvRank={cfg.kv_rank}" if cfg.kind == "deepseek" else "")
                    + f", {layers} of {w['layers']} blocks, synthetic weights seed {w['seed']}, {prompt_len}-token prompt through prefill"
                    + f" + {n_new} greedy steps ({'one whole-token kernel per step' if fused else 'one kernel per operator'}), tp{world}, kv {kvd}:"
                    + " logits of every new token and the tokens vs the CPU oracle with dequantized Q8 weights"
                    + ("; Q8 codes and scales of one block bit-exact" if check_codes and world == 1 else ""))
            out.append({"max_err_over_range": err, "tokens_equal": bool(equal), "tolerance": LOGIT_TOL, "checked": what,
                        "seconds": time.perf_counter() - t_start})
        return out
    finally:
        if dec is not None:
            dec.close()
