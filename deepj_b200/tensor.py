"""Host-side mirror of DeepJ's tensor façade and its lazy GPU backend.

`Tensor` is tensor/Tensor.java (2-D fp32, row-major, a process-wide backend).
`GraphBackend` implements the `TensorBackend` SPI (tensor/TensorBackend.java:3-113)
the way tensor/metal/MetalBackend.java does: every op takes GPU buffers for its
inputs, allocates an output buffer, records one op in the `ComputeGraph` and
returns a tensor whose data is stale until it is materialised.  Method names and
argument meaning are the reference's; shape errors raise ValueError where the
reference throws IllegalArgumentException, before anything is recorded.

`CudaBackend()` is the drop-in: `Tensor.setBackend(CudaBackend())`.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import numpy as np

from . import compute_graph as cg
from .compute_graph import ComputeGraph, CudaGpuRuntime, GpuBuffer, GpuRuntime


class Tensor:
    """tensor/Tensor.java:8 — rows × cols floats, row-major."""

    _backend: Optional["GraphBackend"] = None

    def __init__(self, rows: int, cols: int, data: Optional[np.ndarray] = None):
        if rows < 0 or cols < 0:
            raise ValueError("negative tensor dimension")
        self.rows, self.cols = int(rows), int(cols)
        if data is None:
            self.data = np.zeros((self.rows, self.cols), dtype=np.float32)
        else:
            self.data = np.ascontiguousarray(data, dtype=np.float32).reshape(self.rows, self.cols)
        self.gpu_tag: Optional[GpuBuffer] = None

    # ── backend switch: Tensor.java:24,34-37 ──
    @classmethod
    def setBackend(cls, backend: "GraphBackend") -> None:
        if backend is None:
            raise ValueError("backend must not be null")
        cls._backend = backend

    @classmethod
    def backend(cls) -> "GraphBackend":
        if cls._backend is None:
            raise RuntimeError("no backend set: call Tensor.setBackend(CudaBackend()) first (there is no CPU fallback)")
        return cls._backend

    # ── factories ──
    @staticmethod
    def from2D(values) -> "Tensor":
        a = np.asarray(values, dtype=np.float32)
        if a.ndim != 2:
            raise ValueError("from2D needs a 2-D array")
        return Tensor(a.shape[0], a.shape[1], a)

    @staticmethod
    def zeros(rows: int, cols: int) -> "Tensor":
        return Tensor(rows, cols)

    @staticmethod
    def ones(rows: int, cols: int) -> "Tensor":
        return Tensor(rows, cols, np.ones((rows, cols), dtype=np.float32))

    @staticmethod
    def causalMask(size: int) -> "Tensor":
        # CpuBackend.causalMask (tensor/cpu/CpuBackend.java:154-161): 0 on/below the diagonal, -1e9f above
        m = np.where(np.arange(size)[None, :] > np.arange(size)[:, None], np.float32(-1e9), np.float32(0.0))
        return Tensor(size, size, m.astype(np.float32))

    @staticmethod
    def requireSameShape(a: "Tensor", b: "Tensor", op: str) -> None:
        if a.rows != b.rows or a.cols != b.cols:
            raise ValueError(f"Shape mismatch for {op}: {a.rows}x{a.cols} vs {b.rows}x{b.cols}")

    @staticmethod
    def requireTargetsMatchRows(logits: "Tensor", targets: Sequence[int]) -> None:
        if len(targets) != logits.rows:
            raise ValueError(f"targets length {len(targets)} must match logits rows {logits.rows}")

    # ── lazy execution ──
    def materialize(self) -> "Tensor":
        Tensor.backend().materializeTensor(self)
        return self

    def numpy(self) -> np.ndarray:
        """Materialised contents as a [rows × cols] array."""
        return self.materialize().data

    # ── instance ops: delegate to the backend (Tensor.java:80-173) ──
    def matmul(self, o): return Tensor.backend().matmul(self, o)
    def add(self, o): return Tensor.backend().add(self, o)
    def subtract(self, o): return Tensor.backend().subtract(self, o)
    def multiply(self, o): return Tensor.backend().multiply(self, o)
    def divide(self, o): return Tensor.backend().divide(self, o)
    def addRowVector(self, v): return Tensor.backend().addRowVector(self, v)
    def addBroadcastRows(self, v): return Tensor.backend().addBroadcastRows(self, v)
    def multiplyBroadcastRows(self, v): return Tensor.backend().multiplyBroadcastRows(self, v)
    def addBroadcastCols(self, v): return Tensor.backend().addBroadcastCols(self, v)
    def subtractBroadcastCols(self, v): return Tensor.backend().subtractBroadcastCols(self, v)
    def multiplyBroadcastCols(self, v): return Tensor.backend().multiplyBroadcastCols(self, v)
    def divideBroadcastCols(self, v): return Tensor.backend().divideBroadcastCols(self, v)
    def multiplyScalar(self, s): return Tensor.backend().multiplyScalar(self, s)
    def addScalar(self, s): return Tensor.backend().addScalar(self, s)
    def divideScalar(self, s): return Tensor.backend().divideScalar(self, s)
    def sumRows(self): return Tensor.backend().sumRows(self)
    def sumAlongRows(self): return Tensor.backend().sumAlongRows(self)
    def sumAlongCols(self): return Tensor.backend().sumAlongCols(self)
    def meanAlongRows(self): return Tensor.backend().meanAlongRows(self)
    def varianceAlongRows(self): return Tensor.backend().varianceAlongRows(self)
    def maxAlongRows(self): return Tensor.backend().maxAlongRows(self)
    def sum(self): return Tensor.backend().sum(self)
    def sumAbs(self): return Tensor.backend().sumAbs(self)
    def transpose(self): return Tensor.backend().transpose(self)
    def clamp(self, lo, hi): return Tensor.backend().clamp(self, lo, hi)
    def sqrt(self): return Tensor.backend().sqrt(self)
    def pow(self, e): return Tensor.backend().pow(self, e)
    def neg(self): return Tensor.backend().neg(self)
    def exp(self): return Tensor.backend().exp(self)
    def log(self): return Tensor.backend().log(self)
    def tanhActivation(self): return Tensor.backend().tanh(self)
    def sigmoidActivation(self): return Tensor.backend().sigmoid(self)
    def reluActivation(self): return Tensor.backend().relu(self)
    def geluActivation(self): return Tensor.backend().gelu(self)
    def softmaxRows(self): return Tensor.backend().softmaxRows(self)
    def multiplyScalarInPlace(self, s): Tensor.backend().multiplyScalarInPlace(self, s)
    def addInPlace(self, o): Tensor.backend().addInPlace(self, o)

    @staticmethod
    def sliceRows(t: "Tensor", row_indices: Sequence[int], cols: int) -> "Tensor":
        """Tensor.sliceRows (Tensor.java:231-234): a CPU row gather after materialising."""
        t.materialize()
        idx = np.asarray(row_indices, dtype=np.int64)
        return Tensor(len(idx), cols, t.data[idx, :cols].copy())


def _require_row_vector(v: Tensor, target: Tensor) -> None:
    if v.rows != 1 or v.cols != target.cols:
        raise ValueError(f"Expected row vector 1x{target.cols} but got {v.rows}x{v.cols}")


def _require_col_vector(v: Tensor, target: Tensor) -> None:
    if v.rows != target.rows or v.cols != 1:
        raise ValueError(f"Expected col vector {target.rows}x1 but got {v.rows}x{v.cols}")


class GraphBackend:
    """TensorBackend over a ComputeGraph; the recording calls are those of
    tensor/metal/MetalBackend.java (gpuIn → newOutputBuffer → record* → gpuOut, :66-73).
    In-place variants allocate a new output buffer and rebind the tensor (:400-526)."""

    def __init__(self, runtime: GpuRuntime):
        self.graph = ComputeGraph(runtime)
        self._int_columns: Dict[int, Tensor] = {}

    # ── helpers ──
    def _in(self, t: Tensor) -> GpuBuffer:
        return self.graph.ensure_gpu_buffer(t)

    def _out(self, rows: int, cols: int) -> GpuBuffer:
        return self.graph.new_output_buffer(rows, cols)

    def _wrap(self, buf: GpuBuffer) -> Tensor:
        t = Tensor(buf.rows, buf.cols)
        self.graph.bind_tensor_to_buffer(t, buf)
        return t

    def _int_column(self, values: Sequence[int]) -> Tensor:
        """Index/target vectors travel as floats holding integers (MetalBackend.java:43-54)."""
        t = self._int_columns.get(len(values))
        if t is None:
            t = Tensor(len(values), 1)
            self._int_columns[len(values)] = t
        t.data[:, 0] = np.asarray(values, dtype=np.float32)
        if isinstance(t.gpu_tag, GpuBuffer):
            t.gpu_tag.needs_upload = True
            t.gpu_tag.cpu_stale = False
        return t

    def _binary(self, op: int, a: Tensor, b: Tensor, name: str) -> Tensor:
        Tensor.requireSameShape(a, b, name)
        ga, gb = self._in(a), self._in(b)
        out = self._out(a.rows, a.cols)
        self.graph.record_binary(op, ga, gb, out)
        return self._wrap(out)

    def _unary(self, op: int, a: Tensor) -> Tensor:
        ga = self._in(a)
        out = self._out(a.rows, a.cols)
        self.graph.record_unary(op, ga, out)
        return self._wrap(out)

    def _scalar(self, op: int, a: Tensor, s: float) -> Tensor:
        ga = self._in(a)
        out = self._out(a.rows, a.cols)
        self.graph.record_scalar(op, ga, out, s)
        return self._wrap(out)

    def _reduce(self, op: int, a: Tensor, rows: int, cols: int) -> Tensor:
        ga = self._in(a)
        out = self._out(rows, cols)
        self.graph.record_shaped(op, ga, out, a.rows, a.cols)
        return self._wrap(out)

    def _broadcast(self, op: int, a: Tensor, v: Tensor) -> Tensor:
        ga, gv = self._in(a), self._in(v)
        out = self._out(a.rows, a.cols)
        self.graph.record_broadcast(op, ga, gv, out, a.rows, a.cols)
        return self._wrap(out)

    def _rebind(self, target: Tensor, result: Tensor) -> None:
        self.graph.bind_tensor_to_buffer(target, result.gpu_tag)

    # ── lazy execution ──
    def materializeTensor(self, t: Tensor) -> None:
        self.graph.materialize(t)

    def releaseResources(self) -> None:
        self.graph.release_all()
        self._int_columns.clear()

    # ── binary / matmul ──
    def matmul(self, a: Tensor, b: Tensor) -> Tensor:
        if a.cols != b.rows:
            raise ValueError(f"Shape mismatch for matmul: {a.rows}x{a.cols} vs {b.rows}x{b.cols}")
        ga, gb = self._in(a), self._in(b)
        out = self._out(a.rows, b.cols)
        self.graph.record_matmul(ga, gb, out, a.rows, b.cols, a.cols)
        return self._wrap(out)

    def add(self, a, b): return self._binary(cg.OP_ADD, a, b, "add")
    def subtract(self, a, b): return self._binary(cg.OP_SUBTRACT, a, b, "subtract")
    def multiply(self, a, b): return self._binary(cg.OP_MULTIPLY, a, b, "multiply")
    def divide(self, a, b): return self._binary(cg.OP_DIVIDE, a, b, "divide")
    def reluBackward(self, x, g): return self._binary(cg.OP_RELU_BACKWARD, x, g, "reluBackward")
    def geluBackward(self, x, g): return self._binary(cg.OP_GELU_BACKWARD, x, g, "geluBackward")

    # ── broadcasts ──
    def addRowVector(self, a, v):
        _require_row_vector(v, a)
        return self._broadcast(cg.OP_ADD_ROW_VECTOR, a, v)

    def addBroadcastRows(self, a, v): return self.addRowVector(a, v)

    def multiplyBroadcastRows(self, a, v):
        _require_row_vector(v, a)
        return self._broadcast(cg.OP_MULTIPLY_BROADCAST_ROWS, a, v)

    def addBroadcastCols(self, a, v):
        _require_col_vector(v, a)
        return self._broadcast(cg.OP_ADD_BROADCAST_COLS, a, v)

    def subtractBroadcastCols(self, a, v):
        _require_col_vector(v, a)
        return self._broadcast(cg.OP_SUBTRACT_BROADCAST_COLS, a, v)

    def multiplyBroadcastCols(self, a, v):
        _require_col_vector(v, a)
        return self._broadcast(cg.OP_MULTIPLY_BROADCAST_COLS, a, v)

    def divideBroadcastCols(self, a, v):
        _require_col_vector(v, a)
        return self._broadcast(cg.OP_DIVIDE_BROADCAST_COLS, a, v)

    # ── scalar ──
    def multiplyScalar(self, a, s): return self._scalar(cg.OP_MULTIPLY_SCALAR, a, s)
    def addScalar(self, a, s): return self._scalar(cg.OP_ADD_SCALAR, a, s)
    def divideScalar(self, a, s): return self._scalar(cg.OP_DIVIDE_SCALAR, a, s)
    def pow(self, a, e): return self._scalar(cg.OP_POW, a, e)

    def clamp(self, a, lo, hi):
        ga = self._in(a)
        out = self._out(a.rows, a.cols)
        self.graph.record_clamp(ga, out, lo, hi)
        return self._wrap(out)

    # ── reductions ──
    def sumRows(self, a): return self._reduce(cg.OP_SUM_ROWS, a, 1, a.cols)
    def sumAlongCols(self, a): return self.sumRows(a)
    def sumAlongRows(self, a): return self._reduce(cg.OP_SUM_ALONG_ROWS, a, a.rows, 1)
    def meanAlongRows(self, a): return self._reduce(cg.OP_MEAN_ALONG_ROWS, a, a.rows, 1)
    def varianceAlongRows(self, a): return self._reduce(cg.OP_VARIANCE_ALONG_ROWS, a, a.rows, 1)
    def maxAlongRows(self, a): return self._reduce(cg.OP_MAX_ALONG_ROWS, a, a.rows, 1)

    def sum(self, a) -> float:
        # MetalBackend.sum (:247-254): one sum_scalar op, then a 1×1 download
        s = self._reduce(cg.OP_SUM_SCALAR, a, 1, 1)
        return float(s.numpy()[0, 0])

    def sumAbs(self, a) -> float:
        # MetalBackend.sumAbs (:257-266): per-row |x| sums, then sumRows
        rows = self._reduce(cg.OP_SUM_ABS, a, a.rows, 1)
        return float(self.sumRows(rows).numpy()[0, 0])

    # ── unary ──
    def transpose(self, a): return self._reduce(cg.OP_TRANSPOSE, a, a.cols, a.rows)
    def sqrt(self, a): return self._unary(cg.OP_SQRT, a)
    def neg(self, a): return self._unary(cg.OP_NEG, a)
    def exp(self, a): return self._unary(cg.OP_EXP, a)
    def log(self, a): return self._unary(cg.OP_LOG, a)
    def tanh(self, a): return self._unary(cg.OP_TANH, a)
    def sigmoid(self, a): return self._unary(cg.OP_SIGMOID, a)
    def relu(self, a): return self._unary(cg.OP_RELU, a)
    def gelu(self, a): return self._unary(cg.OP_GELU, a)
    def softmaxRows(self, a): return self._reduce(cg.OP_SOFTMAX_ROWS, a, a.rows, a.cols)

    def softmaxBackward(self, grad, sm):
        Tensor.requireSameShape(grad, sm, "softmaxBackward")
        gg, gs = self._in(grad), self._in(sm)
        out = self._out(grad.rows, grad.cols)
        self.graph.record_three_shaped(cg.OP_SOFTMAX_BACKWARD, gg, gs, out, grad.rows, grad.cols)
        return self._wrap(out)

    # ── fused ──
    def crossEntropyLoss(self, logits, targets) -> float:
        Tensor.requireTargetsMatchRows(logits, targets)
        t = self._int_column(targets)
        gl, gt = self._in(logits), self._in(t)
        out = self._out(logits.rows, 1)
        self.graph.record_three_shaped(cg.OP_CROSS_ENTROPY_LOSS, gl, gt, out, logits.rows, logits.cols)
        losses = self._wrap(out)
        return float(self.divideScalar(self.sumRows(losses), logits.rows).numpy()[0, 0])

    def crossEntropyGradient(self, logits, targets):
        Tensor.requireTargetsMatchRows(logits, targets)
        t = self._int_column(targets)
        gl, gt = self._in(logits), self._in(t)
        out = self._out(logits.rows, logits.cols)
        self.graph.record_three_shaped(cg.OP_CROSS_ENTROPY_GRADIENT, gl, gt, out, logits.rows, logits.cols)
        return self._wrap(out)

    def adamWUpdate(self, w, g, mt, vt, lr, beta1, beta2, eps, weightDecay, bc1, bc2) -> None:
        for o in (g, mt, vt):
            Tensor.requireSameShape(w, o, "adamWUpdate")
        gw, gg, gm, gv = self._in(w), self._in(g), self._in(mt), self._in(vt)
        self.graph.record_adamw_update(gw, gg, gm, gv, lr, beta1, beta2, eps, weightDecay, bc1, bc2, w.rows * w.cols)
        for b in (gw, gm, gv):
            b.cpu_stale, b.needs_upload = True, False

    def layerNormBackward(self, dXHat, xHat, std, dim):
        Tensor.requireSameShape(dXHat, xHat, "layerNormBackward")
        if dim != dXHat.cols:
            raise ValueError(f"layerNormBackward: dim={dim} must equal tensor cols={dXHat.cols}")
        if std.rows != dXHat.rows or std.cols != 1:
            raise ValueError(f"layerNormBackward: std must be {dXHat.rows}x1 but got {std.rows}x{std.cols}")
        a, b, c = self._in(dXHat), self._in(xHat), self._in(std)
        out = self._out(dXHat.rows, dXHat.cols)
        self.graph.record_layernorm_backward(a, b, c, out, dXHat.rows, dXHat.cols)
        return self._wrap(out)

    def scatterAddRows(self, target, indices, grad) -> None:
        if len(indices) != grad.rows:
            raise ValueError(f"scatterAddRows: indices length {len(indices)} must match grad rows {grad.rows}")
        if target.cols != grad.cols:
            raise ValueError(f"scatterAddRows: target cols {target.cols} must match grad cols {grad.cols}")
        if len(indices) == 0:
            return
        idx = self._int_column(indices)
        gt, gg, gi = self._in(target), self._in(grad), self._in(idx)
        self.graph.record_scatter_add_rows(cg.OP_SCATTER_ADD_ROWS_ATOMIC, gt, gi, gg, target.rows, target.cols, len(indices))
        gt.cpu_stale, gt.needs_upload = True, False

    # ── in-place: new buffer + rebind ──
    def addInPlace(self, a, b): self._rebind(a, self.add(a, b))
    def subtractInPlace(self, a, b): self._rebind(a, self.subtract(a, b))
    def multiplyInPlace(self, a, b): self._rebind(a, self.multiply(a, b))
    def divideInPlace(self, a, b): self._rebind(a, self.divide(a, b))
    def multiplyScalarInPlace(self, a, s): self._rebind(a, self.multiplyScalar(a, s))
    def addScalarInPlace(self, a, s): self._rebind(a, self.addScalar(a, s))
    def divideScalarInPlace(self, a, s): self._rebind(a, self.divideScalar(a, s))
    def sqrtInPlace(self, a): self._rebind(a, self.sqrt(a))
    def negInPlace(self, a): self._rebind(a, self.neg(a))
    def expInPlace(self, a): self._rebind(a, self.exp(a))
    def logInPlace(self, a): self._rebind(a, self.log(a))
    def reluInPlace(self, a): self._rebind(a, self.relu(a))
    def geluInPlace(self, a): self._rebind(a, self.gelu(a))
    def tanhInPlace(self, a): self._rebind(a, self.tanh(a))
    def sigmoidInPlace(self, a): self._rebind(a, self.sigmoid(a))


class CudaBackend(GraphBackend):
    """`Tensor.setBackend(CudaBackend())` — the B200 twin of `new MetalBackend()`."""

    def __init__(self, device: int = 0):
        super().__init__(CudaGpuRuntime(device))
