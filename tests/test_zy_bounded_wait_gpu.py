"""Failure detection without a fault: an exchange whose peer never shows up.

`deepj_cuda_tp_connect(NULL, world)` gives every other rank a private buffer that nobody fills.  The exchange
kernel's wait for that rank's words is bounded (about a second); when it runs out the kernel records
100 + rank in the device error word, finishes, and the context stays usable — no trap, no hang."""
import ctypes

import numpy as np
import pytest

from deepj_b200 import _lib
from deepj_b200.compute_graph import OP_ADD, OP_TP_ALLREDUCE

pytestmark = pytest.mark.gpu


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
        _lib.check(lib.deepj_cuda_flush_ops(cmd.ctypes.data, cmd.size))      # returns: the wait gave up
        st = (ctypes.c_int64 * 6)()
        _lib.check(lib.deepj_cuda_stats(st, 6))
        assert st[5] == 101                                      # 100 + the rank whose data did not arrive
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
    st = (ctypes.c_int64 * 6)()
    _lib.check(lib.deepj_cuda_stats(st, 6))
    assert st[5] == 0
