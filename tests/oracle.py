"""ctypes binding of the CPU oracle (oracle/libdeepj_oracle.so) for the tests.

Test infrastructure only: the product package never imports this module.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
LIB_PATH = os.path.join(ORACLE_DIR, "libdeepj_oracle.so")

_lib = None
_vp = ctypes.c_void_p
_i32 = ctypes.c_int32
_i64 = ctypes.c_int64


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    src = os.path.join(ORACLE_DIR, "deepj_oracle.cpp")
    if not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", ORACLE_DIR], check=True, capture_output=True)
    L = ctypes.CDLL(LIB_PATH)
    L.oracle_last_error.restype = ctypes.c_char_p
    L.oracle_jrandom_new.restype = _vp
    L.oracle_jrandom_new.argtypes = [_i64]
    L.oracle_jrandom_free.argtypes = [_vp]
    L.oracle_jrandom_next_int.restype = _i32
    L.oracle_jrandom_next_int.argtypes = [_vp, _i32]
    L.oracle_jrandom_next_float.restype = ctypes.c_float
    L.oracle_jrandom_next_float.argtypes = [_vp]
    L.oracle_jrandom_next_double.restype = ctypes.c_double
    L.oracle_jrandom_next_double.argtypes = [_vp]
    L.oracle_jrandom_next_gaussian.restype = ctypes.c_double
    L.oracle_jrandom_next_gaussian.argtypes = [_vp]
    L.oracle_jrandom_fill_gaussian.argtypes = [_vp, _vp, _i64, ctypes.c_double]
    L.oracle_synth_fill.argtypes = [ctypes.c_uint64, ctypes.c_uint64, ctypes.c_float, _i64, _i64, _vp]
    L.oracle_q8_quantize.argtypes = [_vp, _i32, _i32, _vp, _vp]
    L.oracle_q8_dequantize.argtypes = [_vp, _vp, _i32, _i32, _vp]
    L.oracle_matmul.argtypes = [_vp, _vp, _vp, _i32, _i32, _i32]
    L.oracle_rope_tables.argtypes = [_i32, _i32, _vp, _vp]
    L.oracle_model_new.restype = _vp
    L.oracle_model_new.argtypes = [_i32] * 9 + [_i64, _i32, ctypes.c_double, _i32]
    L.oracle_model_free.argtypes = [_vp]
    L.oracle_model_weight_size.restype = _i64
    L.oracle_model_weight_size.argtypes = [_vp, ctypes.c_char_p, _i32]
    L.oracle_model_get_weight.argtypes = [_vp, ctypes.c_char_p, _i32, _vp]
    L.oracle_model_set_weight.argtypes = [_vp, ctypes.c_char_p, _i32, _vp, _i64]
    L.oracle_model_apply_q8.argtypes = [_vp]
    L.oracle_model_forward.argtypes = [_vp, _vp, _i32, _vp, _i32]
    L.oracle_model_reset_cache.argtypes = [_vp]
    L.oracle_model_decode_step.argtypes = [_vp, _i32, _vp]
    L.oracle_greedy_pick.restype = _i32
    L.oracle_greedy_pick.argtypes = [_vp, _i32]
    L.oracle_generate_greedy.argtypes = [_vp, _vp, _i32, _i32, _i32, _vp, _vp]
    L.oracle_sample_topk.restype = _i32
    L.oracle_sample_topk.argtypes = [_vp, _i32, ctypes.c_float, _i32, ctypes.c_float]
    L.oracle_alloc_buffers.argtypes = [_vp, _vp, _i32]
    L.oracle_upload_buffer.argtypes = [_i32, _vp, _i32]
    L.oracle_download_buffer.argtypes = [_i32, _vp, _i32]
    L.oracle_release_buffers.argtypes = [_vp, _i32]
    L.oracle_flush_ops.argtypes = [_vp, _i32]
    L.oracle_set_threads.argtypes = [_i32]
    _lib = L
    return L


class OracleError(RuntimeError):
    pass


def _check(rc: int) -> None:
    if rc != 0:
        raise OracleError(lib().oracle_last_error().decode())


class JRandom:
    """java.util.Random as restated in the oracle."""

    def __init__(self, seed: int):
        self.h = lib().oracle_jrandom_new(seed)

    def __del__(self):
        if getattr(self, "h", None):
            lib().oracle_jrandom_free(self.h)
            self.h = None

    def next_int(self, bound: int) -> int:
        return lib().oracle_jrandom_next_int(self.h, bound)

    def next_float(self) -> float:
        return lib().oracle_jrandom_next_float(self.h)

    def next_double(self) -> float:
        return lib().oracle_jrandom_next_double(self.h)

    def next_gaussian(self) -> float:
        return lib().oracle_jrandom_next_gaussian(self.h)

    def tensor_random(self, rows: int, cols: int, mult: float = 0.1) -> np.ndarray:
        """Tensor.random: (float)(nextGaussian() * mult), row-major."""
        out = np.empty((rows, cols), dtype=np.float32)
        lib().oracle_jrandom_fill_gaussian(self.h, out.ctypes.data, out.size, mult)
        return out


def synth(seed: int, ordinal: int, std: float, n: int, offset: int = 0) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    lib().oracle_synth_fill(seed, ordinal, std, offset, n, out.ctypes.data)
    return out


def q8_quantize(W: np.ndarray):
    W = np.ascontiguousarray(W, dtype=np.float32)
    K, N = W.shape
    codes = np.empty((N, K), dtype=np.int8)
    scales = np.empty((N, (K + 31) // 32), dtype=np.float32)
    _check(lib().oracle_q8_quantize(W.ctypes.data, K, N, codes.ctypes.data, scales.ctypes.data))
    return codes, scales


def q8_dequantize(codes: np.ndarray, scales: np.ndarray) -> np.ndarray:
    N, K = codes.shape
    W = np.empty((K, N), dtype=np.float32)
    _check(lib().oracle_q8_dequantize(np.ascontiguousarray(codes).ctypes.data, np.ascontiguousarray(scales).ctypes.data, K, N, W.ctypes.data))
    return W


def matmul(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    out = np.empty((a.shape[0], b.shape[1]), dtype=np.float32)
    _check(lib().oracle_matmul(a.ctypes.data, b.ctypes.data, out.ctypes.data, a.shape[0], b.shape[1], a.shape[1]))
    return out


def rope_tables(head_dim: int, max_seq: int):
    cos = np.empty((max_seq, max(head_dim // 2, 1)), dtype=np.float32)
    sin = np.empty_like(cos)
    _check(lib().oracle_rope_tables(head_dim, max_seq, cos.ctypes.data, sin.ctypes.data))
    return cos, sin


KIND = {"llama": 0, "deepseek": 1, "gpt": 2}


class OracleModel:
    """The reference model restated on the CPU.  init_mode 0 = java.util.Random in the
    reference's construction order; 1 = the counter-based synthetic generator."""

    def __init__(self, kind, vocab, max_seq, d, heads, layers, d_ff, q_rank=0, kv_rank=0, seed=42,
                 init_mode=0, std=0.1, layers_built=0):
        self.kind, self.V, self.max_seq, self.d, self.H, self.L, self.F = kind, vocab, max_seq, d, heads, layers, d_ff
        self.q_rank, self.kv_rank = q_rank, kv_rank
        self.h = lib().oracle_model_new(KIND[kind], vocab, max_seq, d, heads, layers, d_ff, q_rank, kv_rank,
                                        seed, init_mode, std, layers_built)
        if not self.h:
            raise OracleError(lib().oracle_last_error().decode())

    def __del__(self):
        if getattr(self, "h", None):
            lib().oracle_model_free(self.h)
            self.h = None

    def weight(self, name: str, layer: int = -1) -> np.ndarray:
        n = lib().oracle_model_weight_size(self.h, name.encode(), layer)
        if n < 0:
            raise KeyError(name)
        out = np.empty(n, dtype=np.float32)
        _check(lib().oracle_model_get_weight(self.h, name.encode(), layer, out.ctypes.data))
        return out

    def set_weight(self, name: str, layer: int, data: np.ndarray) -> None:
        data = np.ascontiguousarray(data, dtype=np.float32).reshape(-1)
        _check(lib().oracle_model_set_weight(self.h, name.encode(), layer, data.ctypes.data, data.size))

    def apply_q8(self) -> None:
        """Replace every matmul weight by dequant(Q8(W)) ("oracle B")."""
        _check(lib().oracle_model_apply_q8(self.h))

    def forward(self, ids, last_row_only=False) -> np.ndarray:
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        rows = 1 if last_row_only else ids.size
        out = np.empty((rows, self.V), dtype=np.float32)
        _check(lib().oracle_model_forward(self.h, ids.ctypes.data, ids.size, out.ctypes.data, int(last_row_only)))
        return out

    def reset_cache(self) -> None:
        lib().oracle_model_reset_cache(self.h)

    def decode_step(self, token: int) -> np.ndarray:
        out = np.empty(self.V, dtype=np.float32)
        _check(lib().oracle_model_decode_step(self.h, int(token), out.ctypes.data))
        return out

    def generate_greedy(self, prompt, max_new, use_cache=True, keep_logits=True):
        prompt = np.ascontiguousarray(prompt, dtype=np.int32)
        toks = np.empty(max_new, dtype=np.int32)
        logits = np.empty((max_new, self.V), dtype=np.float32) if keep_logits else None
        _check(lib().oracle_generate_greedy(self.h, prompt.ctypes.data, prompt.size, max_new, int(use_cache),
                                            toks.ctypes.data, logits.ctypes.data if keep_logits else None))
        return toks, logits


def greedy_pick(logits: np.ndarray) -> int:
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    return lib().oracle_greedy_pick(logits.ctypes.data, logits.size)


def sample_topk(logits: np.ndarray, temperature: float, top_k: int, r: float) -> int:
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    return lib().oracle_sample_topk(logits.ctypes.data, logits.size, temperature, top_k, r)


class OracleRuntime:
    """GpuRuntime over host memory: the command stream executed with CpuBackend arithmetic."""

    def alloc_buffers(self, ids, sizes, count):
        a = np.asarray(ids[:count], dtype=np.int32)
        s = np.asarray(sizes[:count], dtype=np.int32)
        _check(lib().oracle_alloc_buffers(a.ctypes.data, s.ctypes.data, count))

    def upload_buffer(self, buf_id, data):
        data = np.ascontiguousarray(data, dtype=np.float32)
        _check(lib().oracle_upload_buffer(buf_id, data.ctypes.data, data.size))

    def download_buffer(self, buf_id, out):
        _check(lib().oracle_download_buffer(buf_id, out.ctypes.data, out.size))

    def release_buffers(self, ids, count):
        a = np.asarray(ids[:count], dtype=np.int32)
        lib().oracle_release_buffers(a.ctypes.data, count)

    def flush_ops(self, cmd_stream, length):
        cmd = np.ascontiguousarray(cmd_stream[:length], dtype=np.int32)
        _check(lib().oracle_flush_ops(cmd.ctypes.data, length))
