"""deepj_cuda_attn_decode_static — decode attention for callers that cannot allocate.

A host that has given all device memory to its own arena, or a thread that must never
block in cudaMalloc, cannot use the stream form of the attention op: its scratch comes
from a workspace the library grows on demand.  The static entry point keeps that scratch
inside the library image.  This test drives it through the C ABI and checks it against
the stream form (op 67 through deepj_cuda_flush_ops) on two consecutive decode positions,
each side appending to its own KV cache.  It is collected last on purpose.
"""
import ctypes

import numpy as np
import pytest

from deepj_b200 import _lib
from deepj_b200.compute_graph import OP_ATTN_DECODE
from deepj_b200.decoder import rope_tables

pytestmark = pytest.mark.gpu

ATOL, RTOL = 1e-4, 1e-4


def test_static_scratch_attention_matches_stream_attention_twice_in_a_row():
    lib = _lib.load()
    _lib.check(lib.deepj_cuda_init(0))
    B, H, hd, max_seq, layers, layer = 2, 4, 64, 96, 2, 1
    d = H * hd
    base = 1 << 27
    ids = {n: base + i for i, n in enumerate(["qkv", "pos", "cos", "sin", "out_a", "out_b", "kv_a", "kv_b"])}

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

    cos, sin = rope_tables(hd, max_seq)
    alloc("qkv", B * 3 * d); alloc("pos", B); alloc("cos", cos.size, cos); alloc("sin", sin.size, sin)
    alloc("out_a", B * d); alloc("out_b", B * d)
    _lib.check(lib.deepj_cuda_kv_alloc(ids["kv_a"], layers, B, H, max_seq, hd))
    _lib.check(lib.deepj_cuda_kv_alloc(ids["kv_b"], layers, B, H, max_seq, hd))
    rng = np.random.default_rng(12)
    try:
        # fill both caches with the same history through the stream form, then compare the two forms
        for step in range(70):
            qkv = rng.standard_normal((B, 3 * d)).astype(np.float32)
            upload("qkv", qkv)
            upload("pos", np.asarray([step, max(step - 3, 0)], dtype=np.float32))      # ragged positions
            stream_a = np.asarray([OP_ATTN_DECODE, ids["qkv"], 0, d, 2 * d, 3 * d, ids["kv_a"], layer, ids["pos"], ids["cos"],
                                   ids["sin"], ids["out_a"], 0, d, B, H, hd], dtype=np.int32)
            _lib.check(lib.deepj_cuda_flush_ops(stream_a.ctypes.data, stream_a.size))
            if step < 68:
                stream_b = stream_a.copy()
                stream_b[6], stream_b[11] = ids["kv_b"], ids["out_b"]
                _lib.check(lib.deepj_cuda_flush_ops(stream_b.ctypes.data, stream_b.size))
            else:
                # the last two positions go through the entry point that allocates nothing
                _lib.check(lib.deepj_cuda_attn_decode_static(ids["qkv"], 0, d, 2 * d, 3 * d, ids["kv_b"], layer, ids["pos"],
                                                             ids["cos"], ids["sin"], ids["out_b"], 0, d, B, H, hd))
                a, b = download("out_a", B * d), download("out_b", B * d)
                assert np.all(np.isfinite(a)) and np.abs(a).max() > 0
                assert np.all(np.abs(a - b) <= ATOL + RTOL * np.abs(a)), float(np.abs(a - b).max())
        # shapes beyond the static scratch are refused with a clear message, nothing runs
        rc = lib.deepj_cuda_attn_decode_static(ids["qkv"], 0, d, 2 * d, 3 * d, ids["kv_b"], 7, ids["pos"], ids["cos"], ids["sin"],
                                               ids["out_b"], 0, d, B, H, hd)
        assert rc != 0 and "layer out of range" in lib.deepj_cuda_last_error().decode()
        big = base + 100
        _lib.check(lib.deepj_cuda_kv_alloc(big, 1, 64, 128, 64, 16))
        rc = lib.deepj_cuda_attn_decode_static(ids["qkv"], 0, d, 2 * d, 3 * d, big, 0, ids["pos"], ids["cos"], ids["sin"],
                                               ids["out_b"], 0, 128 * 16, 64, 128, 16)
        assert rc != 0
        msg = lib.deepj_cuda_last_error().decode()
        assert "static scratch holds" in msg or "smaller than the op needs" in msg or "row stride" in msg
        _lib.check(lib.deepj_cuda_release_buffers((ctypes.c_int32 * 1)(big), 1))
        st = (ctypes.c_int64 * 6)()
        _lib.check(lib.deepj_cuda_stats(st, 6))
        assert st[5] == 0
    finally:
        arr = (ctypes.c_int32 * len(ids))(*ids.values())
        _lib.check(lib.deepj_cuda_release_buffers(arr, len(ids)))
