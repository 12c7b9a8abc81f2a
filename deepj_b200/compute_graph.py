"""Host-side mirror of DeepJ's lazy graph recorder and its five-call runtime SPI.

`ComputeGraph` reproduces what tensor/ComputeGraph.java emits: a flat int32 command
stream `[opCode, bufferIds..., shape ints / float bits...]` (op codes :19-60, strides
and buffer slots :89-147, encoders :261-518), batched allocation → uploads → one
flush (:528-538), orphan release through weak references (:566-598) and id restart
after `release_all` (:691-740).  `GpuRuntime` is tensor/GpuRuntime.java:9-28;
`CudaGpuRuntime` forwards the five calls to libdeepj_cuda_jni exactly as
tensor/metal/MetalGpuRuntime.java:9-35 forwards them to the Metal library.
"""
from __future__ import annotations

import ctypes
import struct
import weakref
from typing import Dict, List, Optional, Protocol, Sequence

import numpy as np

from . import _lib

# ── op codes: tensor/ComputeGraph.java:19-60 ──
OP_ADD, OP_SUBTRACT, OP_MULTIPLY, OP_DIVIDE, OP_MATMUL, OP_MULTIPLY_SCALAR = 1, 2, 3, 4, 5, 6
OP_SQRT, OP_NEG, OP_EXP, OP_LOG, OP_TANH, OP_SIGMOID, OP_RELU = 7, 8, 9, 10, 11, 12, 13
OP_RELU_BACKWARD, OP_GELU, OP_GELU_BACKWARD, OP_SOFTMAX_ROWS, OP_SOFTMAX_BACKWARD = 14, 15, 16, 17, 18
OP_LAYERNORM_BACKWARD, OP_ADAMW_UPDATE, OP_ADD_SCALAR, OP_DIVIDE_SCALAR, OP_TRANSPOSE = 19, 20, 21, 22, 23
OP_ADD_ROW_VECTOR, OP_ADD_BROADCAST_COLS, OP_SUBTRACT_BROADCAST_COLS, OP_DIVIDE_BROADCAST_COLS = 24, 25, 26, 27
OP_MULTIPLY_BROADCAST_ROWS, OP_SUM_ROWS, OP_MEAN_ALONG_ROWS, OP_VARIANCE_ALONG_ROWS = 28, 29, 30, 31
OP_MULTIPLY_BROADCAST_COLS, OP_SUM_ALONG_ROWS, OP_MAX_ALONG_ROWS, OP_CLAMP, OP_POW = 32, 33, 34, 35, 36
OP_SCATTER_ADD_ROWS, OP_SUM_ABS, OP_CROSS_ENTROPY_LOSS, OP_CROSS_ENTROPY_GRADIENT = 37, 38, 39, 40
OP_SUM_SCALAR, OP_SCATTER_ADD_ROWS_ATOMIC = 41, 42
# fused decode op codes of include/deepj_cuda.h (not in the reference)
OP_EMBED_GATHER, OP_Q8_LINEAR, OP_Q8_SWIGLU, OP_ATTN_DECODE = 64, 65, 66, 67
OP_ARGMAX_ROWS, OP_ADD_SCALAR_INPLACE, OP_COPY = 68, 69, 70
OP_TP_ALLREDUCE, OP_TP_ALLGATHER = 71, 72
OP_ATTN_PREFILL, OP_SAMPLE_TOPK, OP_Q8_LINEAR_LN, OP_DECODE_STEP = 73, 74, 75, 76

# op → (stride, offsets of the slots that hold buffer ids); ComputeGraph.java:89-147
OP_METADATA: Dict[int, tuple] = {}
for _op in (OP_SQRT, OP_NEG, OP_EXP, OP_LOG, OP_TANH, OP_SIGMOID, OP_RELU, OP_GELU):
    OP_METADATA[_op] = (4, (1, 2))
for _op in (OP_ADD, OP_SUBTRACT, OP_MULTIPLY, OP_DIVIDE, OP_RELU_BACKWARD, OP_GELU_BACKWARD):
    OP_METADATA[_op] = (5, (1, 2, 3))
for _op in (OP_MULTIPLY_SCALAR, OP_ADD_SCALAR, OP_DIVIDE_SCALAR, OP_TRANSPOSE, OP_SUM_ROWS, OP_MEAN_ALONG_ROWS,
            OP_VARIANCE_ALONG_ROWS, OP_SUM_ALONG_ROWS, OP_MAX_ALONG_ROWS, OP_SOFTMAX_ROWS, OP_POW, OP_SUM_ABS,
            OP_SUM_SCALAR):
    OP_METADATA[_op] = (5, (1, 2))
OP_METADATA[OP_CLAMP] = (6, (1, 2))
for _op in (OP_SCATTER_ADD_ROWS, OP_SCATTER_ADD_ROWS_ATOMIC, OP_MATMUL):
    OP_METADATA[_op] = (7, (1, 2, 3))
for _op in (OP_CROSS_ENTROPY_LOSS, OP_CROSS_ENTROPY_GRADIENT, OP_SOFTMAX_BACKWARD, OP_ADD_ROW_VECTOR,
            OP_ADD_BROADCAST_COLS, OP_SUBTRACT_BROADCAST_COLS, OP_DIVIDE_BROADCAST_COLS,
            OP_MULTIPLY_BROADCAST_ROWS, OP_MULTIPLY_BROADCAST_COLS):
    OP_METADATA[_op] = (6, (1, 2, 3))
OP_METADATA[OP_LAYERNORM_BACKWARD] = (7, (1, 2, 3, 4))
OP_METADATA[OP_ADAMW_UPDATE] = (13, (1, 2, 3, 4))
# fused ops extend the reference's table: the recorder
# must know their strides or orphan detection treats them as "references everything"
OP_METADATA[OP_EMBED_GATHER] = (7, (1, 2, 3))
OP_METADATA[OP_Q8_LINEAR] = (15, (1, 4, 6, 7, 8, 11))
OP_METADATA[OP_Q8_SWIGLU] = (14, (1, 4, 6, 7, 8, 9, 10))
OP_METADATA[OP_ATTN_DECODE] = (17, (1, 6, 8, 9, 10, 11))
OP_METADATA[OP_ARGMAX_ROWS] = (5, (1, 2))
OP_METADATA[OP_ADD_SCALAR_INPLACE] = (4, (1,))
OP_METADATA[OP_COPY] = (6, (1, 3))
OP_METADATA[OP_TP_ALLREDUCE] = (7, (1, 2, 3, 4))
OP_METADATA[OP_TP_ALLGATHER] = (5, (1, 2))
OP_METADATA[OP_ATTN_PREFILL] = (18, (1, 6, 8, 9, 10, 11))
OP_METADATA[OP_SAMPLE_TOPK] = (8, (1, 2, 3))
OP_METADATA[OP_Q8_LINEAR_LN] = (17, (1, 4, 5, 7, 8, 9, 12))
OP_METADATA[OP_DECODE_STEP] = (3, (1,))


def float_bits(value: float) -> int:
    """Float.floatToRawIntBits: the int32 that carries a float through the stream
    (ComputeGraph.java:252-254)."""
    return struct.unpack("<i", struct.pack("<f", float(np.float32(value))))[0]


class GpuRuntime(Protocol):
    """tensor/GpuRuntime.java:9-28."""

    def alloc_buffers(self, ids: Sequence[int], sizes: Sequence[int], count: int) -> None: ...
    def upload_buffer(self, buf_id: int, data: np.ndarray) -> None: ...
    def download_buffer(self, buf_id: int, out: np.ndarray) -> None: ...
    def release_buffers(self, ids: Sequence[int], count: int) -> None: ...
    def flush_ops(self, cmd_stream: np.ndarray, length: int) -> None: ...


class CudaGpuRuntime:
    """The five GpuRuntime calls over libdeepj_cuda_jni (MetalGpuRuntime.java:9-35 twin)."""

    def __init__(self, device: int = 0):
        self.lib = _lib.load()
        _lib.check(self.lib.deepj_cuda_init(device))

    def alloc_buffers(self, ids, sizes, count):
        a = (ctypes.c_int32 * count)(*ids[:count])
        s = (ctypes.c_int32 * count)(*sizes[:count])
        _lib.check(self.lib.deepj_cuda_alloc_buffers(a, s, count))

    def upload_buffer(self, buf_id, data):
        data = np.ascontiguousarray(data, dtype=np.float32)
        _lib.check(self.lib.deepj_cuda_upload_buffer(buf_id, data.ctypes.data, data.size))

    def download_buffer(self, buf_id, out):
        assert out.dtype == np.float32 and out.flags.c_contiguous
        _lib.check(self.lib.deepj_cuda_download_buffer(buf_id, out.ctypes.data, out.size))

    def release_buffers(self, ids, count):
        a = (ctypes.c_int32 * count)(*ids[:count])
        _lib.check(self.lib.deepj_cuda_release_buffers(a, count))

    def flush_ops(self, cmd_stream, length):
        cmd = np.ascontiguousarray(cmd_stream[:length], dtype=np.int32)
        _lib.check(self.lib.deepj_cuda_flush_ops(cmd.ctypes.data, length))


class GpuBuffer:
    """tensor/GpuBuffer.java:9-33."""

    __slots__ = ("id", "rows", "cols", "needs_upload", "cpu_stale", "allocated_on_gpu")

    def __init__(self, id_: int, rows: int, cols: int, needs_upload: bool):
        self.id, self.rows, self.cols = id_, rows, cols
        self.needs_upload = needs_upload
        self.cpu_stale = not needs_upload
        self.allocated_on_gpu = False

    def float_count(self) -> int:
        return self.rows * self.cols


class ComputeGraph:
    """Lazy recorder: ops accumulate in an int32 stream and run in one flush."""

    INITIAL_CAPACITY = 4096          # ComputeGraph.java:71

    def __init__(self, runtime: GpuRuntime):
        if runtime is None:
            raise ValueError("runtime")
        self.runtime = runtime
        self.next_buf_id = 0
        self.cmd = np.zeros(self.INITIAL_CAPACITY, dtype=np.int32)
        self.cmd_pos = 0
        self.op_count = 0
        self.pending_allocs: List[tuple] = []
        self.pending_uploads: List[tuple] = []
        self.buf_to_tensor: Dict[int, weakref.ref] = {}

    # ── buffers ──
    def ensure_gpu_buffer(self, t) -> GpuBuffer:
        buf = t.gpu_tag
        if isinstance(buf, GpuBuffer):
            self._track(buf.id, t)
            if buf.needs_upload:
                self.pending_uploads.append((buf.id, t.data.reshape(-1).copy()))
                buf.needs_upload = False
                buf.cpu_stale = False
            return buf
        buf = GpuBuffer(self._new_id(), t.rows, t.cols, True)
        self.pending_allocs.append((buf.id, buf.float_count()))
        self.pending_uploads.append((buf.id, t.data.reshape(-1).copy()))
        t.gpu_tag = buf
        self._track(buf.id, t)
        return buf

    def new_output_buffer(self, rows: int, cols: int) -> GpuBuffer:
        buf = GpuBuffer(self._new_id(), rows, cols, False)
        buf.cpu_stale = True
        self.pending_allocs.append((buf.id, buf.float_count()))
        return buf

    def bind_tensor_to_buffer(self, t, buf: GpuBuffer) -> None:
        t.gpu_tag = buf
        self._track(buf.id, t)

    def _new_id(self) -> int:
        i = self.next_buf_id
        self.next_buf_id += 1
        return i

    def _track(self, buf_id: int, t) -> None:
        self.buf_to_tensor[buf_id] = weakref.ref(t)

    # ── recording ──
    def emit(self, *ints: int) -> None:
        """Append one op (already encoded) to the stream, growing it by doubling
        (ComputeGraph.java:238-242)."""
        need = len(ints)
        if self.cmd_pos + need > self.cmd.size:
            grown = np.zeros(max(self.cmd.size * 2, self.cmd_pos + need), dtype=np.int32)
            grown[: self.cmd_pos] = self.cmd[: self.cmd_pos]
            self.cmd = grown
        self.cmd[self.cmd_pos: self.cmd_pos + need] = ints
        self.cmd_pos += need
        self.op_count += 1

    def record_binary(self, op, a, b, out):
        self.emit(op, a.id, b.id, out.id, out.float_count())

    def record_matmul(self, a, b, out, m, n, k):
        self.emit(OP_MATMUL, a.id, b.id, out.id, m, n, k)

    def record_unary(self, op, inp, out):
        self.emit(op, inp.id, out.id, out.float_count())

    def record_scalar(self, op, inp, out, scalar):
        self.emit(op, inp.id, out.id, float_bits(scalar), out.float_count())

    def record_clamp(self, inp, out, lo, hi):
        self.emit(OP_CLAMP, inp.id, out.id, float_bits(lo), float_bits(hi), out.float_count())

    def record_shaped(self, op, inp, out, rows, cols):
        """transpose, reductions, softmax, sum_abs, sum_scalar: [op, in, out, rows, cols]."""
        self.emit(op, inp.id, out.id, rows, cols)

    def record_broadcast(self, op, a, vec, out, rows, cols):
        self.emit(op, a.id, vec.id, out.id, rows, cols)

    def record_three_shaped(self, op, a, b, out, rows, cols):
        """softmax backward and the two cross-entropy ops: [op, a, b, out, rows, cols]."""
        self.emit(op, a.id, b.id, out.id, rows, cols)

    def record_scatter_add_rows(self, op, target, indices, grad, t_rows, t_cols, n_idx):
        self.emit(op, target.id, indices.id, grad.id, t_rows, t_cols, n_idx)

    def record_layernorm_backward(self, dxhat, xhat, std, out, rows, cols):
        self.emit(OP_LAYERNORM_BACKWARD, dxhat.id, xhat.id, std.id, out.id, rows, cols)

    def record_adamw_update(self, w, g, mt, vt, lr, beta1, beta2, eps, weight_decay, bc1, bc2, n):
        self.emit(OP_ADAMW_UPDATE, w.id, g.id, mt.id, vt.id, float_bits(lr), float_bits(beta1), float_bits(beta2),
                  float_bits(eps), float_bits(weight_decay), float_bits(bc1), float_bits(bc2), n)

    def is_empty(self) -> bool:
        return self.op_count == 0

    # ── flush ──
    def flush(self) -> None:
        if self.op_count == 0 and not self.pending_allocs:
            self._release_orphans()
            return
        if self.pending_allocs:
            ids = [a[0] for a in self.pending_allocs]
            sizes = [a[1] for a in self.pending_allocs]
            self.runtime.alloc_buffers(ids, sizes, len(ids))
            for ref in self.buf_to_tensor.values():
                t = ref()
                if t is not None and isinstance(t.gpu_tag, GpuBuffer):
                    t.gpu_tag.allocated_on_gpu = True
            self.pending_allocs.clear()
        for buf_id, data in self.pending_uploads:
            self.runtime.upload_buffer(buf_id, data)
        self.pending_uploads.clear()
        if self.op_count > 0:
            self.runtime.flush_ops(self.cmd, self.cmd_pos)
        self.cmd_pos = 0
        self.op_count = 0
        self._release_orphans()

    def _referenced_by_pending_ops(self, buf_id: int) -> bool:
        pos = 0
        while pos < self.cmd_pos:
            meta = OP_METADATA.get(int(self.cmd[pos]))
            if meta is None:
                return True      # unknown op: be conservative
            stride, slots = meta
            if any(int(self.cmd[pos + s]) == buf_id for s in slots):
                return True
            pos += stride
        return False

    def _release_orphans(self) -> None:
        orphans = []
        for buf_id, ref in self.buf_to_tensor.items():
            t = ref()
            gone = t is None or not isinstance(t.gpu_tag, GpuBuffer) or t.gpu_tag.id != buf_id
            if gone and not self._referenced_by_pending_ops(buf_id):
                orphans.append(buf_id)
        if not orphans:
            return
        dead = set(orphans)
        for buf_id in orphans:
            del self.buf_to_tensor[buf_id]
        self.pending_allocs = [a for a in self.pending_allocs if a[0] not in dead]
        self.pending_uploads = [u for u in self.pending_uploads if u[0] not in dead]
        self.runtime.release_buffers(orphans, len(orphans))

    def materialize(self, t) -> None:
        buf = t.gpu_tag
        if not isinstance(buf, GpuBuffer) or not buf.cpu_stale:
            return
        self.flush()
        flat = np.empty(buf.float_count(), dtype=np.float32)
        self.runtime.download_buffer(buf.id, flat)
        t.data[...] = flat.reshape(t.rows, t.cols)
        buf.cpu_stale = False

    def release_all(self) -> None:
        self.flush()
        live = []
        for ref in self.buf_to_tensor.values():
            t = ref()
            if t is None or not isinstance(t.gpu_tag, GpuBuffer):
                continue
            live.append(t)
            gb = t.gpu_tag
            if gb.cpu_stale:
                flat = np.empty(gb.float_count(), dtype=np.float32)
                self.runtime.download_buffer(gb.id, flat)
                t.data[...] = flat.reshape(t.rows, t.cols)
                gb.cpu_stale = False
                gb.needs_upload = False
        for t in live:
            t.gpu_tag = None
        if self.buf_to_tensor:
            ids = list(self.buf_to_tensor.keys())
            self.runtime.release_buffers(ids, len(ids))
        self.buf_to_tensor.clear()
        self.pending_allocs.clear()
        self.pending_uploads.clear()
        self.cmd_pos = 0
        self.op_count = 0
        self.next_buf_id = 0
