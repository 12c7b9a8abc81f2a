package io.github.kirstenali.deepj.tensor.cuda;

import io.github.kirstenali.deepj.tensor.ComputeGraph;
import io.github.kirstenali.deepj.tensor.GpuBuffer;
import io.github.kirstenali.deepj.tensor.Tensor;
import io.github.kirstenali.deepj.tensor.TensorBackend;

import java.util.HashMap;
import java.util.Map;

/**
 * {@code Tensor.setBackend(new CudaBackend())}: the lazy, graph-recording {@link TensorBackend} over a
 * {@link ComputeGraph} whose runtime is {@link CudaGpuRuntime} (libdeepj_cuda_jni on an NVIDIA B200).
 *
 * <p>It records exactly the command stream the Metal backend records for the same calls (same op codes, same
 * operand order, same shape checks and messages), so models, layers and {@code TextGenerator} run unchanged.
 * Every method reduces to one of a few recording shapes, kept as private helpers here: element-wise unary /
 * binary, scalar, row / column broadcast, row reduction.  In-place variants allocate a fresh output buffer and
 * rebind the tensor to it, so the native side never sees aliased operands; AdamW and scatter-add are the two
 * true read-modify-write ops.
 *
 * <p>There is no CPU fallback: constructing the runtime fails when the native library is missing.
 */
public final class CudaBackend implements TensorBackend {

    private final ComputeGraph graph;
    private final CudaGpuRuntime runtime;
    /** index / target vectors travel as floats holding integers; one reusable column per length */
    private final Map<Integer, Tensor> indexColumns = new HashMap<>();

    public CudaBackend() {
        this(0);
    }

    public CudaBackend(int device) {
        this.runtime = new CudaGpuRuntime(device);
        this.graph = new ComputeGraph(runtime);
    }

    /** The runtime behind the graph: Q8 objects, KV caches, decode plans and the fused decode op codes go through it. */
    public CudaGpuRuntime runtime() {
        return runtime;
    }

    public ComputeGraph graph() {
        return graph;
    }

    // ── recording shapes ──────────────────────────────────────────────────────────────────────────

    private interface Recorder {
        void into(GpuBuffer out);
    }

    /** allocate [rows x cols], let {@code r} record into it, hand back a tracked tensor */
    private Tensor produce(int rows, int cols, Recorder r) {
        GpuBuffer out = graph.newOutputBuffer(rows, cols);
        r.into(out);
        return graph.createOutputTensor(out);
    }

    /** the same, but the result replaces {@code target}'s storage */
    private void produceInto(Tensor target, Recorder r) {
        GpuBuffer out = graph.newOutputBuffer(target.rows, target.cols);
        r.into(out);
        graph.bindTensorToBuffer(target, out);
    }

    private GpuBuffer in(Tensor t) {
        return graph.ensureGpuBuffer(t);
    }

    private Recorder unaryOp(int op, Tensor a) {
        GpuBuffer ga = in(a);
        return out -> graph.recordUnary(op, ga, out);
    }

    private Recorder binaryOp(int op, Tensor a, Tensor b, String what) {
        if (what != null) Tensor.requireSameShape(a, b, what);
        GpuBuffer ga = in(a), gb = in(b);
        return out -> graph.recordBinary(op, ga, gb, out);
    }

    private Recorder scalarOp(int op, Tensor a, float s) {
        GpuBuffer ga = in(a);
        if (op == ComputeGraph.OP_MULTIPLY_SCALAR) return out -> graph.recordMultiplyScalar(ga, out, s);
        return out -> graph.recordScalarUnary(op, ga, out, s);
    }

    private Tensor rowBroadcast(int op, Tensor a, Tensor v) {
        if (v.rows != 1 || v.cols != a.cols) {
            throw new IllegalArgumentException("Expected row vector 1x" + a.cols + " but got " + v.rows + "x" + v.cols);
        }
        GpuBuffer ga = in(a), gv = in(v);
        return produce(a.rows, a.cols, out -> graph.recordRowBroadcast(op, ga, gv, out, a.rows, a.cols));
    }

    private Tensor colBroadcast(int op, Tensor a, Tensor v) {
        if (v.rows != a.rows || v.cols != 1) {
            throw new IllegalArgumentException("Expected col vector " + a.rows + "x1 but got " + v.rows + "x" + v.cols);
        }
        GpuBuffer ga = in(a), gv = in(v);
        return produce(a.rows, a.cols, out -> graph.recordColBroadcast(op, ga, gv, out, a.rows, a.cols));
    }

    private Tensor reduce(int op, Tensor a, int outRows, int outCols) {
        GpuBuffer ga = in(a);
        return produce(outRows, outCols, out -> graph.recordReduction(op, ga, out, a.rows, a.cols));
    }

    private static float firstValue(Tensor t) {
        t.materialize();
        return t.data[0];
    }

    private Tensor indexColumn(int[] values) {
        Tensor t = indexColumns.computeIfAbsent(values.length, n -> new Tensor(n, 1));
        for (int i = 0; i < values.length; i++) t.data[i] = values[i];
        if (t.getGpuTag() instanceof GpuBuffer gb) {      // the device copy is stale now
            gb.needsUpload = true;
            gb.cpuStale = false;
        }
        return t;
    }

    private static void deviceCopyIsNewer(GpuBuffer b) {
        b.cpuStale = true;
        b.needsUpload = false;
    }

    // ── matmul, element-wise, broadcast ───────────────────────────────────────────────────────────

    @Override
    public Tensor matmul(Tensor a, Tensor b) {
        if (a.cols != b.rows) {
            throw new IllegalArgumentException("Shape mismatch for matmul: " + a.rows + "x" + a.cols + " vs " + b.rows + "x" + b.cols);
        }
        GpuBuffer ga = in(a), gb = in(b);
        return produce(a.rows, b.cols, out -> graph.recordMatmul(ga, gb, out, a.rows, b.cols, a.cols));
    }

    @Override public Tensor add(Tensor a, Tensor b) { return produce(a.rows, a.cols, binaryOp(ComputeGraph.OP_ADD, a, b, "add")); }
    @Override public Tensor subtract(Tensor a, Tensor b) { return produce(a.rows, a.cols, binaryOp(ComputeGraph.OP_SUBTRACT, a, b, "subtract")); }
    @Override public Tensor multiply(Tensor a, Tensor b) { return produce(a.rows, a.cols, binaryOp(ComputeGraph.OP_MULTIPLY, a, b, "multiply")); }
    @Override public Tensor divide(Tensor a, Tensor b) { return produce(a.rows, a.cols, binaryOp(ComputeGraph.OP_DIVIDE, a, b, "divide")); }

    @Override public Tensor addRowVector(Tensor a, Tensor v) { return rowBroadcast(ComputeGraph.OP_ADD_ROW_VECTOR, a, v); }
    @Override public Tensor addBroadcastRows(Tensor a, Tensor v) { return addRowVector(a, v); }
    @Override public Tensor multiplyBroadcastRows(Tensor a, Tensor v) { return rowBroadcast(ComputeGraph.OP_MULTIPLY_BROADCAST_ROWS, a, v); }
    @Override public Tensor addBroadcastCols(Tensor a, Tensor v) { return colBroadcast(ComputeGraph.OP_ADD_BROADCAST_COLS, a, v); }
    @Override public Tensor subtractBroadcastCols(Tensor a, Tensor v) { return colBroadcast(ComputeGraph.OP_SUBTRACT_BROADCAST_COLS, a, v); }
    @Override public Tensor multiplyBroadcastCols(Tensor a, Tensor v) { return colBroadcast(ComputeGraph.OP_MULTIPLY_BROADCAST_COLS, a, v); }
    @Override public Tensor divideBroadcastCols(Tensor a, Tensor v) { return colBroadcast(ComputeGraph.OP_DIVIDE_BROADCAST_COLS, a, v); }

    // ── scalars ───────────────────────────────────────────────────────────────────────────────────

    @Override public Tensor multiplyScalar(Tensor a, float s) { return produce(a.rows, a.cols, scalarOp(ComputeGraph.OP_MULTIPLY_SCALAR, a, s)); }
    @Override public Tensor addScalar(Tensor a, float s) { return produce(a.rows, a.cols, scalarOp(ComputeGraph.OP_ADD_SCALAR, a, s)); }
    @Override public Tensor divideScalar(Tensor a, float s) { return produce(a.rows, a.cols, scalarOp(ComputeGraph.OP_DIVIDE_SCALAR, a, s)); }

    // ── reductions ────────────────────────────────────────────────────────────────────────────────

    @Override public Tensor sumRows(Tensor a) { return reduce(ComputeGraph.OP_SUM_ROWS, a, 1, a.cols); }
    @Override public Tensor sumAlongCols(Tensor a) { return sumRows(a); }
    @Override public Tensor sumAlongRows(Tensor a) { return reduce(ComputeGraph.OP_SUM_ALONG_ROWS, a, a.rows, 1); }
    @Override public Tensor meanAlongRows(Tensor a) { return reduce(ComputeGraph.OP_MEAN_ALONG_ROWS, a, a.rows, 1); }
    @Override public Tensor varianceAlongRows(Tensor a) { return reduce(ComputeGraph.OP_VARIANCE_ALONG_ROWS, a, a.rows, 1); }
    @Override public Tensor maxAlongRows(Tensor a) { return reduce(ComputeGraph.OP_MAX_ALONG_ROWS, a, a.rows, 1); }

    @Override
    public float sum(Tensor a) {
        GpuBuffer ga = in(a);
        return firstValue(produce(1, 1, out -> graph.recordSumScalar(ga, out, a.rows, a.cols)));
    }

    @Override
    public float sumAbs(Tensor a) {
        GpuBuffer ga = in(a);
        Tensor perRow = produce(a.rows, 1, out -> graph.recordSumAbs(ga, out, a.rows, a.cols));
        return firstValue(sumRows(perRow));
    }

    // ── unary math and activations ────────────────────────────────────────────────────────────────

    @Override
    public Tensor transpose(Tensor a) {
        GpuBuffer ga = in(a);
        return produce(a.cols, a.rows, out -> graph.recordTranspose(ga, out, a.rows, a.cols));
    }

    @Override
    public Tensor clamp(Tensor a, float min, float max) {
        GpuBuffer ga = in(a);
        return produce(a.rows, a.cols, out -> graph.recordClamp(ga, out, min, max));
    }

    @Override
    public Tensor pow(Tensor a, float exponent) {
        GpuBuffer ga = in(a);
        return produce(a.rows, a.cols, out -> graph.recordPow(ga, out, exponent));
    }

    @Override public Tensor sqrt(Tensor a) { return produce(a.rows, a.cols, unaryOp(ComputeGraph.OP_SQRT, a)); }
    @Override public Tensor neg(Tensor a) { return produce(a.rows, a.cols, unaryOp(ComputeGraph.OP_NEG, a)); }
    @Override public Tensor exp(Tensor a) { return produce(a.rows, a.cols, unaryOp(ComputeGraph.OP_EXP, a)); }
    @Override public Tensor log(Tensor a) { return produce(a.rows, a.cols, unaryOp(ComputeGraph.OP_LOG, a)); }
    @Override public Tensor tanh(Tensor a) { return produce(a.rows, a.cols, unaryOp(ComputeGraph.OP_TANH, a)); }
    @Override public Tensor sigmoid(Tensor a) { return produce(a.rows, a.cols, unaryOp(ComputeGraph.OP_SIGMOID, a)); }
    @Override public Tensor relu(Tensor a) { return produce(a.rows, a.cols, unaryOp(ComputeGraph.OP_RELU, a)); }
    @Override public Tensor gelu(Tensor a) { return produce(a.rows, a.cols, unaryOp(ComputeGraph.OP_GELU, a)); }

    @Override
    public Tensor reluBackward(Tensor input, Tensor gradOutput) {
        return produce(input.rows, input.cols, binaryOp(ComputeGraph.OP_RELU_BACKWARD, input, gradOutput, null));
    }

    @Override
    public Tensor geluBackward(Tensor input, Tensor gradOutput) {
        return produce(input.rows, input.cols, binaryOp(ComputeGraph.OP_GELU_BACKWARD, input, gradOutput, null));
    }

    // ── softmax ───────────────────────────────────────────────────────────────────────────────────

    @Override
    public Tensor softmaxRows(Tensor logits) {
        GpuBuffer g = in(logits);
        return produce(logits.rows, logits.cols, out -> graph.recordSoftmaxRows(g, out, logits.rows, logits.cols));
    }

    @Override
    public Tensor softmaxBackward(Tensor gradOutput, Tensor softmaxOut) {
        Tensor.requireSameShape(gradOutput, softmaxOut, "softmaxBackward");
        GpuBuffer gg = in(gradOutput), gs = in(softmaxOut);
        return produce(gradOutput.rows, gradOutput.cols,
                out -> graph.recordSoftmaxBackward(gg, gs, out, gradOutput.rows, gradOutput.cols));
    }

    // ── loss, optimiser, normalisation backward, scatter ──────────────────────────────────────────

    @Override
    public float crossEntropyLoss(Tensor logits, int[] targets) {
        Tensor.requireTargetsMatchRows(logits, targets);
        GpuBuffer gl = in(logits), gt = in(indexColumn(targets));
        Tensor perRow = produce(logits.rows, 1, out -> graph.recordCrossEntropyLoss(gl, gt, out, logits.rows, logits.cols));
        return firstValue(sumRows(perRow).divideScalar(logits.rows));
    }

    @Override
    public Tensor crossEntropyGradient(Tensor logits, int[] targets) {
        Tensor.requireTargetsMatchRows(logits, targets);
        GpuBuffer gl = in(logits), gt = in(indexColumn(targets));
        return produce(logits.rows, logits.cols, out -> graph.recordCrossEntropyGradient(gl, gt, out, logits.rows, logits.cols));
    }

    @Override
    public void adamWUpdate(Tensor w, Tensor g, Tensor mt, Tensor vt, float lr, float beta1, float beta2, float eps,
                            float weightDecay, float bc1, float bc2) {
        Tensor.requireSameShape(w, g, "adamWUpdate");
        Tensor.requireSameShape(w, mt, "adamWUpdate");
        Tensor.requireSameShape(w, vt, "adamWUpdate");
        GpuBuffer gw = in(w), gg = in(g), gm = in(mt), gv = in(vt);
        graph.recordAdamWUpdate(gw, gg, gm, gv, lr, beta1, beta2, eps, weightDecay, bc1, bc2, w.rows * w.cols);
        deviceCopyIsNewer(gw);
        deviceCopyIsNewer(gm);
        deviceCopyIsNewer(gv);
    }

    @Override
    public Tensor layerNormBackward(Tensor dXHat, Tensor xHat, Tensor std, int dim) {
        Tensor.requireSameShape(dXHat, xHat, "layerNormBackward");
        if (dim != dXHat.cols) {
            throw new IllegalArgumentException("layerNormBackward: dim=" + dim + " must equal tensor cols=" + dXHat.cols);
        }
        if (std.rows != dXHat.rows || std.cols != 1) {
            throw new IllegalArgumentException("layerNormBackward: std must be " + dXHat.rows + "x1 but got " + std.rows + "x" + std.cols);
        }
        GpuBuffer gd = in(dXHat), gx = in(xHat), gs = in(std);
        return produce(dXHat.rows, dXHat.cols, out -> graph.recordLayerNormBackward(gd, gx, gs, out, dXHat.rows, dXHat.cols));
    }

    @Override
    public void scatterAddRows(Tensor target, int[] indices, Tensor grad) {
        if (indices.length != grad.rows) {
            throw new IllegalArgumentException("scatterAddRows: indices length " + indices.length + " must match grad rows " + grad.rows);
        }
        if (target.cols != grad.cols) {
            throw new IllegalArgumentException("scatterAddRows: target cols " + target.cols + " must match grad cols " + grad.cols);
        }
        if (indices.length == 0) return;
        GpuBuffer gt = in(target), gg = in(grad), gi = in(indexColumn(indices));
        // duplicate indices accumulate with atomic adds on the device
        graph.recordScatterAddRowsAtomic(gt, gi, gg, target.rows, target.cols, indices.length);
        deviceCopyIsNewer(gt);
    }

    // ── in-place variants: a new output buffer, then rebind ───────────────────────────────────────

    @Override public void addInPlace(Tensor a, Tensor b) { produceInto(a, binaryOp(ComputeGraph.OP_ADD, a, b, "addInPlace")); }
    @Override public void subtractInPlace(Tensor a, Tensor b) { produceInto(a, binaryOp(ComputeGraph.OP_SUBTRACT, a, b, "subtractInPlace")); }
    @Override public void multiplyInPlace(Tensor a, Tensor b) { produceInto(a, binaryOp(ComputeGraph.OP_MULTIPLY, a, b, "multiplyInPlace")); }
    @Override public void divideInPlace(Tensor a, Tensor b) { produceInto(a, binaryOp(ComputeGraph.OP_DIVIDE, a, b, "divideInPlace")); }

    @Override public void multiplyScalarInPlace(Tensor a, float s) { produceInto(a, scalarOp(ComputeGraph.OP_MULTIPLY_SCALAR, a, s)); }
    @Override public void addScalarInPlace(Tensor a, float s) { produceInto(a, scalarOp(ComputeGraph.OP_ADD_SCALAR, a, s)); }
    @Override public void divideScalarInPlace(Tensor a, float s) { produceInto(a, scalarOp(ComputeGraph.OP_DIVIDE_SCALAR, a, s)); }

    @Override public void sqrtInPlace(Tensor a) { produceInto(a, unaryOp(ComputeGraph.OP_SQRT, a)); }
    @Override public void negInPlace(Tensor a) { produceInto(a, unaryOp(ComputeGraph.OP_NEG, a)); }
    @Override public void expInPlace(Tensor a) { produceInto(a, unaryOp(ComputeGraph.OP_EXP, a)); }
    @Override public void logInPlace(Tensor a) { produceInto(a, unaryOp(ComputeGraph.OP_LOG, a)); }
    @Override public void reluInPlace(Tensor a) { produceInto(a, unaryOp(ComputeGraph.OP_RELU, a)); }
    @Override public void geluInPlace(Tensor a) { produceInto(a, unaryOp(ComputeGraph.OP_GELU, a)); }
    @Override public void tanhInPlace(Tensor a) { produceInto(a, unaryOp(ComputeGraph.OP_TANH, a)); }
    @Override public void sigmoidInPlace(Tensor a) { produceInto(a, unaryOp(ComputeGraph.OP_SIGMOID, a)); }

    // ── lazy execution ────────────────────────────────────────────────────────────────────────────

    @Override
    public void materializeTensor(Tensor t) {
        graph.materialize(t);
    }

    @Override
    public void releaseResources() {
        graph.releaseAll();
        indexColumns.clear();
    }
}
