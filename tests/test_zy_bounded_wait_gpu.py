"""Failure detection without a fault: an exchange whose peer never shows up.

`deepj_cuda_tp_connect(NULL, world)` gives every other rank a private buffer that nobody fills.  The exchange
kernel's wait for that rank's words is bounded (about a second); when it runs out the kernel records
100 + rank in the device error word, finishes, and the context stays usable — no trap, no hang.  While the
word is set every later wait gives up at once, and a synchronous flush reports the failure."""
import ctypes
import time

import numpy as np
import pytest

from deepj_b200 import _lib
from deepj_b200.compute_graph import OP_ADD, OP_TP_ALLREDUCE

pytestmark = pytest.mark.gpu


def _stats(lib):
    st = (ctypes.c_int64 * 6)()
    _lib.check(lib.deepj_cuda_stats(st, 6))
    return list(st)


def test_exchange_wait_expires_with_a_status_and_the_context_survives():
    lib = _lib.load()
    _lib.check(lib.deepj_cuda_init(0))
    ids = [(5 << 20) + i for i in range(4)]
    n = 64
    _lib.check(lib.deepj_cuda_alloc_buffers((ctypes.c_int32 * 4)(*ids), (ctypes.c_int32 * 4)(n, n, n, n), 4))
    x = np.arange(n, dtype=np.float32)
    _lib.check(lib.deepj_cuda_upload_buffer(ids[0], x.ctypes.data, n))
    _lib.check(lib.deepj_cuda_upload_buffer(ids[1], x.ctypes.data, n))
    handle = ctypes.create_string_buffer(64)
    _lib.check(lib.deepj_cuda_clear_device_error())
    _lib.check(lib.deepj_cuda_tp_create(0, 2, 64, handle))
    try:
        _lib.check(lib.deepj_cuda_tp_connect(None, 2))          # rank 1 never connects
        cmd = np.asarray([OP_TP_ALLREDUCE, ids[0], -1, ids[1], ids[2], 1, n], dtype=np.int32)
        # the flush comes back (the wait gave up) and says what happened
        assert lib.deepj_cuda_flush_ops(cmd.ctypes.data, cmd.size) != 0
        msg = lib.deepj_cuda_last_error().decode()
        assert "bounded wait" in msg and "rank 1" in msg, msg
        assert _stats(lib)[5] == 101                             # 100 + the rank whose data did not arrive
        # with the error word set, the next exchanges do not wait again: a dead peer costs one bounded wait
        t0 = time.perf_counter()
        for _ in range(3):
            assert lib.deepj_cuda_flush_ops(cmd.ctypes.data, cmd.size) != 0
        assert time.perf_counter() - t0 < 0.5, "later exchanges must give up at once"
        assert _stats(lib)[5] == 101                             # the first expiry keeps its rank
        # the context is intact: an ordinary op still runs and is right
        add = np.asarray([OP_ADD, ids[0], ids[1], ids[3], n], dtype=np.int32)
        _lib.check(lib.deepj_cuda_flush_ops(add.ctypes.data, add.size))
        out = np.empty(n, dtype=np.float32)
        _lib.check(lib.deepj_cuda_download_buffer(ids[3], out.ctypes.data, n))
        assert np.array_equal(out, 2 * x)
    finally:
        _lib.check(lib.deepj_cuda_tp_destroy())
        _lib.check(lib.deepj_cuda_clear_device_error())
        _lib.check(lib.deepj_cuda_release_buffers((ctypes.c_int32 * 4)(*ids), 4))
    assert _stats(lib)[5] == 0


def test_reconnecting_drops_the_graphs_that_hold_the_old_exchange_buffer():
    """A cached CUDA graph of an exchange holds the addresses of the exchange buffers.  After tp_destroy + tp_create +
    tp_connect the same stream must be captured afresh (graphs-captured counter rises) and still be right."""
    lib = _lib.load()
    _lib.check(lib.deepj_cuda_init(0))
    ids = [(6 << 20) + i for i in range(3)]
    n = 256
    _lib.check(lib.deepj_cuda_alloc_buffers((ctypes.c_int32 * 3)(*ids), (ctypes.c_int32 * 3)(n, n, n), 3))
    x = np.arange(n, dtype=np.float32)
    r = np.full(n, 0.5, dtype=np.float32)
    _lib.check(lib.deepj_cuda_upload_buffer(ids[0], x.ctypes.data, n))
    _lib.check(lib.deepj_cuda_upload_buffer(ids[1], r.ctypes.data, n))
    cmd = np.asarray([OP_TP_ALLREDUCE, ids[0], -1, ids[1], ids[2], 1, n], dtype=np.int32)
    out = np.empty(n, dtype=np.float32)
    captured = []
    try:
        for round_ in range(2):
            handle = ctypes.create_string_buffer(64)
            _lib.check(lib.deepj_cuda_tp_create(0, 1, 1024, handle))          # a world of one: the rank exchanges with itself
            _lib.check(lib.deepj_cuda_tp_connect(handle, 1))
            for _ in range(3):                                                 # second sighting captures, third replays
                _lib.check(lib.deepj_cuda_flush_ops(cmd.ctypes.data, cmd.size))
            _lib.check(lib.deepj_cuda_download_buffer(ids[2], out.ctypes.data, n))
            assert np.array_equal(out, x + r)
            captured.append(_stats(lib)[2])
            _lib.check(lib.deepj_cuda_tp_destroy())
        assert captured[1] == captured[0] + 1, captured
        assert _stats(lib)[5] == 0
    finally:
        lib.deepj_cuda_tp_destroy()
        _lib.check(lib.deepj_cuda_release_buffers((ctypes.c_int32 * 3)(*ids), 3))
