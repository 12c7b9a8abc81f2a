package io.github.kirstenali.deepj.tensor.cuda;

import io.github.kirstenali.deepj.tensor.GpuRuntime;

/**
 * {@link GpuRuntime} over libdeepj_cuda_jni: hand an instance to {@code ComputeGraph} and every
 * graph-recording backend runs on the CUDA device.
 */
public final class CudaGpuRuntime implements GpuRuntime {

    public CudaGpuRuntime() {
        this(0);
    }

    public CudaGpuRuntime(int device) {
        if (!CudaNative.AVAILABLE) {
            throw new IllegalStateException("libdeepj_cuda_jni is not available; there is no CPU fallback behind this runtime");
        }
        CudaNative.nativeInit(device);
    }

    @Override
    public void allocBuffers(int[] ids, int[] sizes, int count) {
        CudaNative.nativeAllocBuffers(ids, sizes, count);
    }

    @Override
    public void uploadBuffer(int bufId, float[] data) {
        CudaNative.nativeUploadBuffer(bufId, data);
    }

    @Override
    public void downloadBuffer(int bufId, float[] out) {
        CudaNative.nativeDownloadBuffer(bufId, out);
    }

    @Override
    public void releaseBuffers(int[] ids, int count) {
        CudaNative.nativeReleaseBuffers(ids, count);
    }

    @Override
    public void flushOps(int[] cmdStream, int cmdStreamLength) {
        CudaNative.nativeFlushOps(cmdStream, cmdStreamLength);
    }

    // ── what the fused Q8 decode stream needs besides the five calls ──

    public void flushOpsAsync(int[] cmdStream, int cmdStreamLength) {
        CudaNative.nativeFlushOpsAsync(cmdStream, cmdStreamLength);
    }

    public void synchronize() {
        CudaNative.nativeSynchronize();
    }

    public void allocQ8(int q8Id, int k, int n) {
        CudaNative.nativeQ8Alloc(q8Id, k, n);
    }

    /** Quantizes a whole row-major K×N float buffer into the Q8 object. */
    public void quantize(int q8Id, int srcId, int n) {
        CudaNative.nativeQ8QuantizeInto(q8Id, 0, srcId, 0, 0, n, n);
    }

    public void quantizeInto(int q8Id, int dstCol0, int srcId, int srcRow0, int srcCol0, int srcLd, int nCols) {
        CudaNative.nativeQ8QuantizeInto(q8Id, dstCol0, srcId, srcRow0, srcCol0, srcLd, nCols);
    }

    public void allocKvCache(int kvId, int layers, int batch, int heads, int maxSeq, int headDim) {
        CudaNative.nativeKvAlloc(kvId, layers, batch, heads, maxSeq, headDim);
    }

    /** A K/V cache that stores fp16 (same op codes, half the cache bytes per step; logits within the Q8 tolerance of the fp32 cache). */
    public void allocKvCacheF16(int kvId, int layers, int batch, int heads, int maxSeq, int headDim) {
        CudaNative.nativeKvAllocF16(kvId, layers, batch, heads, maxSeq, headDim);
    }

    /** Everything one batch-1 token step touches, resolved once; afterwards the stream {@code [76, planId, feedBack]} runs the step. */
    public void decodePlan(int planId, int[] desc) {
        CudaNative.nativeDecodePlan(planId, desc, desc.length);
    }

    /** Step 1 of the tensor-parallel set-up: this rank's 64-byte handle, to be sent to every other rank. */
    public byte[] tpCreate(int rank, int world, long slotFloats) {
        return CudaNative.nativeTpCreate(rank, world, slotFloats);
    }

    /** Step 2: every rank's handle concatenated in rank order; afterwards op codes 71 / 72 may be recorded. */
    public void tpConnect(byte[] handles, int world) {
        CudaNative.nativeTpConnect(handles, world);
    }

    public void tpDestroy() {
        CudaNative.nativeTpDestroy();
    }

    public long[] stats() {
        long[] out = new long[8];
        CudaNative.nativeStats(out);
        return out;
    }

    public void shutdown() {
        CudaNative.nativeShutdown();
    }
}
