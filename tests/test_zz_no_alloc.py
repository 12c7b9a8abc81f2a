"""deepj_cuda_attn_decode_static — decode attention for callers that cannot allocate.

A host that has given all device memory to its own arena, or a thread that must never
block in cudaMalloc, cannot use the stream form of the attention op: its scratch comes
from a workspace the library grows on demand.  The static entry point keeps that scratch
inside the library image.  This test drives it through the C ABI on two consecutive decode
positions and checks every output three ways: against the stream form (op 67 through
deepj_cuda_flush_ops, each side appending to its own KV cache), against a float64
restatement of the reference's attention chain (HeadOps.java:90-140, RotaryEmbedding.java:81-122,
Softmax.java:16-19), and that the library's growable workspace did not change size across
the static calls.  The history is long enough for the split-KV merge to run with ten
partials per head inside the static array.  It is collected last on purpose.
"""
import ctypes

import numpy as np
import pytest

from deepj_b200 import _lib
from deepj_b200.compute_graph import OP_ATTN_DECODE, OP_ATTN_PREFILL
from deepj_b200.decoder import rope_tables
from test_attn_prefill_gpu import rope

pytestmark = pytest.mark.gpu

ATOL, RTOL = 1e-4, 1e-4


def reference_last_row(q, k, v, cos, sin, pos):
    """The attention output of the token at `pos` over keys 0..pos: q [H × hd] of that token,
    k, v [pos+1 × H × hd] (un-rotated), float64."""
    H, hd = q.shape
    qr = rope(q[None], cos, sin, pos)[0].astype(np.float64)
    kr = rope(k, cos, sin, 0).astype(np.float64)
    out = np.zeros(H * hd)
    for h in range(H):
        s = (kr[:, h] @ qr[h]) / np.sqrt(hd)
        p = np.exp(s - s.max())
        out[h * hd:(h + 1) * hd] = (p / p.sum()) @ v[:, h].astype(np.float64)
    return out


def test_static_scratch_attention_matches_stream_attention_twice_in_a_row():
    lib = _lib.load()
    _lib.check(lib.deepj_cuda_init(0))
    B, H, hd, max_seq, layers, layer = 2, 4, 64, 640, 2, 1
    hist = (600, 500)                      # ragged histories: tokens already cached per sequence
    T = max(hist)
    d = H * hd
    base = 1 << 27
    ids = {n: base + i for i, n in enumerate(["qkv", "pos", "cos", "sin", "out_a", "out_b", "kv_a", "kv_b", "hist", "hout"])}

    def alloc(name, n, data=None):
        _lib.check(lib.deepj_cuda_alloc_buffers((ctypes.c_int32 * 1)(ids[name]), (ctypes.c_int32 * 1)(n), 1))
        if data is not None:
            upload(name, data)

    def upload(name, data):
        a = np.ascontiguousarray(data, dtype=np.float32)
        _lib.check(lib.deepj_cuda_upload_buffer(ids[name], a.ctypes.data, a.size))

    def download(name, n):
        out = np.empty(n, dtype=np.float32)
        _lib.check(lib.deepj_cuda_download_buffer(ids[name], out.ctypes.data, n))
        return out

    def stats():
        st = (ctypes.c_int64 * 6)()
        _lib.check(lib.deepj_cuda_stats(st, 6))
        return list(st)

    cos, sin = rope_tables(hd, max_seq)
    alloc("qkv", B * 3 * d); alloc("pos", B); alloc("cos", cos.size, cos); alloc("sin", sin.size, sin)
    alloc("out_a", B * d); alloc("out_b", B * d)
    alloc("hist", B * T * 3 * d); alloc("hout", B * T * d)
    _lib.check(lib.deepj_cuda_kv_alloc(ids["kv_a"], layers, B, H, max_seq, hd))
    _lib.check(lib.deepj_cuda_kv_alloc(ids["kv_b"], layers, B, H, max_seq, hd))
    rng = np.random.default_rng(12)
    try:
        # the same history in both caches, written by the prompt-chunk op (positions 0..T-1 of every sequence; the
        # decode positions below overwrite what lies beyond a sequence's own history)
        history = rng.standard_normal((B, T, 3, H, hd)).astype(np.float32)
        upload("hist", history.reshape(B * T, 3 * d))
        upload("pos", np.zeros(B, dtype=np.float32))
        for kv in ("kv_a", "kv_b"):
            chunk = np.asarray([OP_ATTN_PREFILL, ids["hist"], 0, d, 2 * d, 3 * d, ids[kv], layer, ids["pos"], ids["cos"], ids["sin"],
                                ids["hout"], 0, d, B, H, hd, T], dtype=np.int32)
            _lib.check(lib.deepj_cuda_flush_ops(chunk.ctypes.data, chunk.size))
        keys = [list(history[b, :hist[b], 1]) for b in range(B)]
        vals = [list(history[b, :hist[b], 2]) for b in range(B)]
        stream_a = np.asarray([OP_ATTN_DECODE, ids["qkv"], 0, d, 2 * d, 3 * d, ids["kv_a"], layer, ids["pos"], ids["cos"],
                               ids["sin"], ids["out_a"], 0, d, B, H, hd], dtype=np.int32)
        for step in range(2):              # two calls in a row: the second finds the first's partials and counters in the array
            qkv = rng.standard_normal((B, 3, H, hd)).astype(np.float32)
            upload("qkv", qkv.reshape(B, 3 * d))
            upload("pos", np.asarray([hist[b] + step for b in range(B)], dtype=np.float32))
            _lib.check(lib.deepj_cuda_flush_ops(stream_a.ctypes.data, stream_a.size))
            ws_before = stats()[4]
            _lib.check(lib.deepj_cuda_attn_decode_static(ids["qkv"], 0, d, 2 * d, 3 * d, ids["kv_b"], layer, ids["pos"],
                                                         ids["cos"], ids["sin"], ids["out_b"], 0, d, B, H, hd))
            assert stats()[4] == ws_before, "the static entry point must leave the growable workspace alone"
            a, b_ = download("out_a", B * d).reshape(B, d), download("out_b", B * d).reshape(B, d)
            assert np.all(np.isfinite(b_)) and np.abs(b_).max() > 0
            assert np.all(np.abs(a - b_) <= ATOL + RTOL * np.abs(a)), float(np.abs(a - b_).max())
            for b in range(B):
                keys[b].append(qkv[b, 1]); vals[b].append(qkv[b, 2])
                want = reference_last_row(qkv[b, 0], np.stack(keys[b]), np.stack(vals[b]), cos, sin, hist[b] + step)
                assert np.all(np.abs(want - b_[b]) <= ATOL + RTOL * np.abs(want)), (step, b, float(np.abs(want - b_[b]).max()))
        # a layer that does not exist is refused before anything runs
        rc = lib.deepj_cuda_attn_decode_static(ids["qkv"], 0, d, 2 * d, 3 * d, ids["kv_b"], 7, ids["pos"], ids["cos"], ids["sin"],
                                               ids["out_b"], 0, d, B, H, hd)
        assert rc != 0 and "layer out of range" in lib.deepj_cuda_last_error().decode()
        # a shape beyond the fixed array (batch·heads = 8192 counters > 4096) with consistent strides and buffers: the
        # refusal is the scratch limit itself, with both numbers in the message
        Bb, Hb, hdb, seqb = 64, 128, 16, 64
        db = Hb * hdb
        big = {n: base + 100 + i for i, n in enumerate(["kv", "qkv", "pos", "cos", "sin", "out"])}
        _lib.check(lib.deepj_cuda_kv_alloc(big["kv"], 1, Bb, Hb, seqb, hdb))
        sizes = {"qkv": Bb * 3 * db, "pos": Bb, "cos": seqb * hdb // 2, "sin": seqb * hdb // 2, "out": Bb * db}
        for name, n in sizes.items():
            _lib.check(lib.deepj_cuda_alloc_buffers((ctypes.c_int32 * 1)(big[name]), (ctypes.c_int32 * 1)(n), 1))
        rc = lib.deepj_cuda_attn_decode_static(big["qkv"], 0, db, 2 * db, 3 * db, big["kv"], 0, big["pos"], big["cos"], big["sin"],
                                               big["out"], 0, db, Bb, Hb, hdb)
        assert rc != 0
        msg = lib.deepj_cuda_last_error().decode()
        assert "static scratch holds" in msg and "4096" in msg, msg
        _lib.check(lib.deepj_cuda_release_buffers((ctypes.c_int32 * len(big))(*big.values()), len(big)))
        assert stats()[5] == 0
    finally:
        arr = (ctypes.c_int32 * len(ids))(*ids.values())
        _lib.check(lib.deepj_cuda_release_buffers(arr, len(ids)))
