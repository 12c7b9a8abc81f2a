"""Operator benchmark: `python -m deepj_b200.opbench --m 1 --k 4096 --n 11008` (Q8 matmul),
`python -m deepj_b200.opbench --attn-prefill --heads 32 --head-dim 128 --tokens 1024 --pos0 1024` (prompt-chunk attention) or
`python -m deepj_b200.opbench --decode-step --d 4096 --heads 32 --d-ff 11008 --vocab 32000 --layers 4 --context 2048`
(token steps of a reduced-depth Llama-shaped model: the whole-token kernel, or with --per-op one kernel per operator).

Times the fused Q8 linear op (y = x·W, W quantized to Q8) through the C ABI.  The
weights of one GEMV (19-51 MB) fit in the B200's L2, so the stream cycles through
`--copies` distinct weight objects (≥ 8, more than L2 in total) and every launch
streams its weights from HBM.  Prints one JSON line with the algorithmic GB/s
(K·N·1.125 + 4·M·(K+N) bytes per launch) and TFLOP/s (2·M·K·N).
"""
from __future__ import annotations

import argparse
import ctypes
import json

import numpy as np

from . import _lib
from .compute_graph import OP_Q8_LINEAR, OP_Q8_SWIGLU, float_bits


def run(m: int, k: int, n: int, copies: int, iters: int, warmup: int, swiglu: bool = False, norm: bool = False,
        device: int = 0, seed: int = 1):
    lib = _lib.load()
    _lib.check(lib.deepj_cuda_init(device))
    base = 1 << 26
    nid = [base]

    def new_id():
        nid[0] += 1
        return nid[0]

    def f32(count, data=None):
        i = new_id()
        _lib.check(lib.deepj_cuda_alloc_buffers((ctypes.c_int32 * 1)(i), (ctypes.c_int32 * 1)(count), 1))
        if data is not None:
            d = np.ascontiguousarray(data, dtype=np.float32)
            _lib.check(lib.deepj_cuda_upload_buffer(i, d.ctypes.data, d.size))
        return i

    rng = np.random.default_rng(seed)
    x = f32(m * k, rng.standard_normal((m, k)).astype(np.float32))
    out = f32(m * n)
    gamma = f32(k, np.ones(k, dtype=np.float32)) if norm else -1
    tmp = f32(k * n)
    per_op = 2 if swiglu else 1
    ws = []
    for c in range(copies * per_op):
        q = new_id()
        _lib.check(lib.deepj_cuda_synth_fill(tmp, seed, c, 0.02, 0, k * n))
        _lib.check(lib.deepj_cuda_q8_alloc(q, k, n))
        _lib.check(lib.deepj_cuda_q8_quantize_into(q, 0, tmp, 0, 0, n, n))
        ws.append(q)
    _lib.check(lib.deepj_cuda_release_buffers((ctypes.c_int32 * 1)(tmp), 1))
    eps = float_bits(1e-6)
    s = []
    for c in range(copies):
        if swiglu:
            s += [OP_Q8_SWIGLU, x, 0, k, gamma, eps, ws[2 * c], -1, ws[2 * c + 1], -1, out, 0, n, m]
        else:
            s += [OP_Q8_LINEAR, x, 0, k, gamma, eps, ws[c], -1, -1, 0, 0, out, 0, n, m]
    cmd = np.asarray(s, dtype=np.int32)
    for _ in range(max(warmup, 3)):
        _lib.check(lib.deepj_cuda_flush_ops(cmd.ctypes.data, cmd.size))
    _lib.check(lib.deepj_cuda_timer_begin())
    for _ in range(iters):
        _lib.check(lib.deepj_cuda_flush_ops_async(cmd.ctypes.data, cmd.size))
    ms = ctypes.c_float(0)
    _lib.check(lib.deepj_cuda_timer_end(ctypes.byref(ms)))
    launches = iters * copies
    us = ms.value * 1e3 / launches
    nb = (k + 31) // 32
    bytes_per = per_op * (k * n + nb * n * 4) + 4 * m * (k + n)
    flops = 2.0 * m * k * n * per_op
    res = {"op": "q8_swiglu" if swiglu else "q8_linear", "m": m, "k": k, "n": n, "copies": copies, "launches": launches,
           "us_per_launch": us, "algorithmic_bytes": bytes_per, "gb_per_s": bytes_per / (us * 1e-6) / 1e9,
           "tflop_per_s": flops / (us * 1e-6) / 1e12, "rmsnorm_fused": norm}
    import os
    if os.environ.get("DEEPJ_CUDA_TRACE") == "1":
        tr = np.zeros((4096, 8), dtype=np.uint64)
        cnt = ctypes.c_int32(0)
        _lib.check(lib.deepj_cuda_trace_read(tr.ctypes.data, 4096, ctypes.byref(cnt)))
        t = tr[cnt.value // 2: cnt.value].astype(np.int64)
        if len(t) > 1:
            d = np.diff(t[:, :6], axis=1)
            gap = t[1:, 0] - t[:-1, 5]
            res["trace_ns_median"] = {"prefetch_issue": float(np.median(d[:, 0])), "wait_prev": float(np.median(d[:, 1])),
                                      "stage_x": float(np.median(d[:, 2])), "first_tile": float(np.median(d[:, 3])),
                                      "rest": float(np.median(d[:, 4])), "start_minus_prev_end": float(np.median(gap)),
                                      "start_to_start": float(np.median(np.diff(t[:, 0]))),
                                      "last_cta_end_minus_cta0_end": float(np.median(t[:, 6] - t[:, 5])),
                                      "wait_return_minus_prev_last_end": float(np.median(t[1:, 2] - t[:-1, 6]))}
    ids = list(range(base + 1, nid[0] + 1))
    _lib.check(lib.deepj_cuda_release_buffers((ctypes.c_int32 * len(ids))(*ids), len(ids)))
    return res


def run_attn_prefill(heads: int, hd: int, tokens: int, pos0: int, batch: int, iters: int, warmup: int, device: int = 0, seed: int = 1):
    """Times op 73 (prompt-chunk attention: append + causal attention of `tokens` rows per sequence behind
    `pos0` cached positions).  Useful flops = 4·hd per (query, visible key) pair and head."""
    from .compute_graph import OP_ATTN_PREFILL
    from .decoder import rope_tables
    lib = _lib.load()
    _lib.check(lib.deepj_cuda_init(device))
    base = 1 << 26
    ids = []

    def f32(count, data=None):
        i = base + 1 + len(ids)
        ids.append(i)
        _lib.check(lib.deepj_cuda_alloc_buffers((ctypes.c_int32 * 1)(i), (ctypes.c_int32 * 1)(count), 1))
        if data is not None:
            d = np.ascontiguousarray(data, dtype=np.float32)
            _lib.check(lib.deepj_cuda_upload_buffer(i, d.ctypes.data, d.size))
        return i

    d, max_seq = heads * hd, pos0 + tokens
    rng = np.random.default_rng(seed)
    cos, sin = rope_tables(hd, max_seq)
    cb, sb = f32(cos.size, cos), f32(sin.size, sin)
    kv = base + 1 + len(ids)
    ids.append(kv)
    _lib.check(lib.deepj_cuda_kv_alloc(kv, 1, batch, heads, max_seq, hd))
    xb = f32(batch * tokens * 3 * d, rng.standard_normal((batch * tokens, 3 * d)).astype(np.float32))
    ob, pb = f32(batch * tokens * d), f32(batch, np.full(batch, float(pos0)))
    if pos0 > 0:       # fill the cache below pos0 with one earlier chunk of the same rows (timing only)
        fill = [OP_ATTN_PREFILL, xb, 0, d, 2 * d, 3 * d, kv, 0, f32(batch, np.zeros(batch)), cb, sb, ob, 0, d, batch, heads, hd, min(pos0, tokens)]
        c0 = np.asarray(fill, dtype=np.int32)
        _lib.check(lib.deepj_cuda_flush_ops(c0.ctypes.data, c0.size))
    cmd = np.asarray([OP_ATTN_PREFILL, xb, 0, d, 2 * d, 3 * d, kv, 0, pb, cb, sb, ob, 0, d, batch, heads, hd, tokens], dtype=np.int32)
    for _ in range(max(warmup, 3)):
        _lib.check(lib.deepj_cuda_flush_ops(cmd.ctypes.data, cmd.size))
    _lib.check(lib.deepj_cuda_timer_begin())
    for _ in range(iters):
        _lib.check(lib.deepj_cuda_flush_ops_async(cmd.ctypes.data, cmd.size))
    ms = ctypes.c_float(0)
    _lib.check(lib.deepj_cuda_timer_end(ctypes.byref(ms)))
    us = ms.value * 1e3 / iters
    pairs = batch * heads * (tokens * pos0 + tokens * (tokens + 1) // 2)
    res = {"op": "attn_prefill", "heads": heads, "head_dim": hd, "tokens": tokens, "pos0": pos0, "batch": batch, "us_per_launch": us,
           "useful_tflop_per_s": 4.0 * hd * pairs / (us * 1e-6) / 1e12}
    _lib.check(lib.deepj_cuda_release_buffers((ctypes.c_int32 * len(ids))(*ids), len(ids)))
    return res


def run_decode_step(d: int, heads: int, d_ff: int, vocab: int, layers: int, context: int, iters: int, warmup: int, per_op: bool,
                    device: int = 0, seed: int = 9):
    """Times greedy token steps (token fed back on the device) of a Llama-shaped Q8 model with synthetic weights, the
    cache positioned at `context` (its rows hold zeros below that: the attention still streams them).  Algorithmic bytes per
    step = Q8 weight bytes + K/V rows of the context."""
    from .decoder import DecoderConfig, Q8Decoder
    steps = warmup + iters
    cfg = DecoderConfig("llama", vocab, context + steps + 8, d, heads, layers, d_ff)
    dec = Q8Decoder(cfg, batch=1, device=device, fused_step=not per_op)
    dec.load_synthetic(seed, 0.02)
    dec.reset()
    dec.set_position(context)
    dec.set_tokens([1])
    dec.step_device(max(warmup, 3))
    _lib.check(dec.lib.deepj_cuda_timer_begin())
    dec.step_device(iters, sync=False)
    ms = ctypes.c_float(0)
    _lib.check(dec.lib.deepj_cuda_timer_end(ctypes.byref(ms)))
    us = ms.value * 1e3 / iters
    ctx = context + max(warmup, 3) + iters // 2
    step_bytes = cfg.q8_weight_bytes() + ctx * cfg.kv_bytes_per_position()
    st = dec.stats()
    res = {"op": "decode_step", "kernel": "k_decode_step" if dec.fused_step else "one kernel per operator", "d": d, "heads": heads, "d_ff": d_ff,
           "vocab": vocab, "layers": layers, "context": ctx, "us_per_step": us, "algorithmic_bytes": step_bytes,
           "gb_per_s": step_bytes / (us * 1e-6) / 1e9, "device_error": st["device_error"], "graph_replays": st["graph_replays"]}
    import os
    if os.environ.get("DEEPJ_CUDA_TRACE") == "1" and dec.fused_step:
        # CTA 0's %globaltimer stamps at the phase boundaries of block 1 (last launch): differences in ns
        tr = np.zeros((4, 8), dtype=np.uint64)
        cnt = ctypes.c_int32(0)
        _lib.check(dec.lib.deepj_cuda_trace_read(tr.ctypes.data, 4, ctypes.byref(cnt)))
        t = tr.reshape(-1).astype(np.int64)
        names = ["stage_qkv", "gemv_qkv", "barrier", "attention", "barrier", "stage_att", "gemv_wo", "barrier", "(gap)", "stage_x2",
                 "gemv_swiglu", "barrier", "stage_h", "gemv_down", "barrier"]
        t = t[t > 0]
        res["trace_ns"] = [[names[i] if i < len(names) else str(i), int(t[i + 1] - t[i])] for i in range(len(t) - 1)]
    dec.close()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--copies", type=int, default=8)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--swiglu", action="store_true")
    ap.add_argument("--norm", action="store_true")
    ap.add_argument("--attn-prefill", action="store_true", help="time op 73 instead: --heads --head-dim --tokens --pos0 --batch")
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--tokens", type=int, default=1024)
    ap.add_argument("--pos0", type=int, default=1024)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--decode-step", action="store_true", help="time token steps of a reduced-depth model: --d --d-ff --vocab --layers --context")
    ap.add_argument("--per-op", action="store_true", help="with --decode-step: one kernel per operator instead of the whole-token kernel")
    ap.add_argument("--d", type=int, default=4096)
    ap.add_argument("--d-ff", type=int, default=11008)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--context", type=int, default=2048)
    a = ap.parse_args()
    if a.decode_step:
        print(json.dumps(run_decode_step(a.d, a.heads, a.d_ff, a.vocab, a.layers, a.context, a.iters, a.warmup, a.per_op)))
        return
    if a.attn_prefill:
        print(json.dumps(run_attn_prefill(a.heads, a.head_dim, a.tokens, a.pos0, a.batch, a.iters, a.warmup)))
        return
    print(json.dumps(run(a.m, a.k, a.n, a.copies, a.iters, a.warmup, a.swiglu, a.norm)))


if __name__ == "__main__":
    main()
