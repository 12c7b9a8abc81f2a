"""Prompt-chunk attention (op 73) against a numpy restatement of the reference's attention chain
(HeadOps.java:90-140 + RotaryEmbedding.java:81-122 + Softmax.java:16-19): two chunks back to back, so the second
one attends over cached keys it did not write itself.  The default path is the tensor-core kernel; the fp32 tiled
and row-wise kernels behind their environment switches are checked in a child process each."""
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

CASES = [(64, 32, 70), (128, 64, 64), (128, 130, 33), (64, 200, 40), (128, 33, 150)]      # head dim, first chunk, second chunk


def rope(x, cos, sin, pos0):
    """x [T × H × hd], interleaved pairs rotated at positions pos0 + t."""
    T = x.shape[0]
    c, s = cos[pos0:pos0 + T, None, :], sin[pos0:pos0 + T, None, :]
    out = np.empty_like(x)
    out[..., 0::2] = x[..., 0::2] * c - x[..., 1::2] * s
    out[..., 1::2] = x[..., 0::2] * s + x[..., 1::2] * c
    return out


def reference(q, k, v, cos, sin):
    """Causal attention over the whole sequence: q, k, v [L × H × hd] → [L × H·hd]."""
    L, H, hd = q.shape
    q, k = rope(q, cos, sin, 0).astype(np.float64), rope(k, cos, sin, 0).astype(np.float64)
    out = np.zeros((L, H * hd))
    mask = np.triu(np.ones((L, L), dtype=bool), 1)
    for h in range(H):
        s = (q[:, h] @ k[:, h].T) / np.sqrt(hd)
        s[mask] = -np.inf
        p = np.exp(s - s.max(axis=1, keepdims=True))
        out[:, h * hd:(h + 1) * hd] = (p / p.sum(axis=1, keepdims=True)) @ v[:, h].astype(np.float64)
    return out


def run_case(hd, T1, T2, B=2, H=3, seed=0):
    import ctypes
    from deepj_b200 import _lib
    from deepj_b200.compute_graph import OP_ATTN_PREFILL
    from deepj_b200.decoder import rope_tables
    from test_q8_gpu import Dev
    dev = Dev(9 << 20)
    try:
        d, L = H * hd, T1 + T2
        max_seq = L + 5
        rng = np.random.default_rng(seed + hd + T1)
        qkv = rng.standard_normal((B, L, 3, H, hd)).astype(np.float32)
        qkv[:, :, 0] *= 2.0                                               # sharper softmax rows
        cos, sin = rope_tables(hd, max_seq)
        cb, sb = dev.buf(cos.size, cos), dev.buf(sin.size, sin)
        kv = dev.next; dev.next += 1; dev.owned.append(kv)
        _lib.check(dev.lib.deepj_cuda_kv_alloc(kv, 1, B, H, max_seq, hd))
        got = np.zeros((B, L, d), dtype=np.float32)
        for pos0, T in ((0, T1), (T1, T2)):
            rows = qkv[:, pos0:pos0 + T].reshape(B * T, 3 * d)
            xb, ob, pb = dev.buf(rows.size, rows), dev.buf(B * T * d), dev.buf(B, np.full(B, float(pos0)))
            dev.flush([OP_ATTN_PREFILL, xb, 0, d, 2 * d, 3 * d, kv, 0, pb, cb, sb, ob, 0, d, B, H, hd, T])
            got[:, pos0:pos0 + T] = dev.get(ob, B * T * d).reshape(B, T, d)
        worst = 0.0
        for b in range(B):
            want = reference(qkv[b, :, 0], qkv[b, :, 1], qkv[b, :, 2], cos, sin)
            worst = max(worst, float(np.abs(want - got[b]).max()))
        st = (ctypes.c_int64 * 6)()
        _lib.check(dev.lib.deepj_cuda_stats(st, 6))
        assert st[5] == 0
        return worst
    finally:
        dev.close()


@pytest.mark.gpu
@pytest.mark.parametrize("hd,T1,T2", CASES)
def test_chunk_attention_matches_the_reference_chain(hd, T1, T2):
    assert run_case(hd, T1, T2) <= 2e-5          # outputs are convex combinations of N(0,1) values; fp32-grade error


@pytest.mark.gpu
@pytest.mark.parametrize("switch", ["DEEPJ_CUDA_NO_MMA_PREFILL", "DEEPJ_CUDA_NO_TILED_PREFILL"])
def test_fp32_kernels_behind_their_switches(switch):
    env = dict(os.environ, **{switch: "1"})
    res = subprocess.run([sys.executable, os.path.abspath(__file__)], env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr


if __name__ == "__main__":
    for case in CASES[:3]:
        err = run_case(*case)
        print(case, err)
        assert err <= 2e-5, (case, err)
