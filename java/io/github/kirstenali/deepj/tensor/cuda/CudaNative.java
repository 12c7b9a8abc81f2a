package io.github.kirstenali.deepj.tensor.cuda;

import java.io.InputStream;
import java.nio.file.Files;
import java.nio.file.Path;
import java.nio.file.StandardCopyOption;

/**
 * Natives of libdeepj_cuda_jni (NVIDIA B200, sm_100a). The first five have the contract of the
 * Metal natives they stand in for; the rest reach the Q8 weight objects, the KV cache and the
 * device binding that the fused decode op codes (64 and up) work on.
 *
 * <p>Every native raises {@link RuntimeException} with the library's message when a call fails.
 */
final class CudaNative {

    /** True when the native library was found on the class path (or java.library.path) and loaded. */
    static final boolean AVAILABLE = loadLibrary();

    private CudaNative() {}

    private static boolean loadLibrary() {
        final String resource = "/native/linux/libdeepj_cuda_jni.so";
        try (InputStream in = CudaNative.class.getResourceAsStream(resource)) {
            if (in != null) {
                // System.load wants a file; a jar entry is not one.
                Path file = Files.createTempFile("deepj_cuda_jni_", ".so");
                file.toFile().deleteOnExit();
                Files.copy(in, file, StandardCopyOption.REPLACE_EXISTING);
                System.load(file.toAbsolutePath().toString());
                return true;
            }
            System.loadLibrary("deepj_cuda_jni");
            return true;
        } catch (Throwable t) {
            System.err.println("[DeepJ/CUDA] native library not loaded: " + t);
            return false;
        }
    }

    // ── the GpuRuntime contract ──

    /** ids[i] gets a zero-filled device buffer of sizes[i] floats; an id that exists is left alone. */
    static native void nativeAllocBuffers(int[] ids, int[] sizes, int count);

    /** Copies data.length floats into the buffer. */
    static native void nativeUploadBuffer(int bufId, float[] data);

    /** Waits for queued work, then copies out.length floats out of the buffer. */
    static native void nativeDownloadBuffer(int bufId, float[] out);

    /** Frees the buffers (float buffers, Q8 objects and KV caches share the id space). */
    static native void nativeReleaseBuffers(int[] ids, int count);

    /**
     * Runs a ComputeGraph command stream and returns when its results are readable. A stream
     * seen for the second time is replayed as a CUDA graph.
     */
    static native void nativeFlushOps(int[] cmdStream, int cmdStreamLength);

    // ── additions ──

    /** Like nativeFlushOps but returns once the work is queued; pair with nativeSynchronize. */
    static native void nativeFlushOpsAsync(int[] cmdStream, int cmdStreamLength);

    static native void nativeSynchronize();

    /** Binds the library to a CUDA device (device 0 at first use otherwise). */
    static native void nativeInit(int device);

    /** Frees every buffer, graph and workspace. */
    static native void nativeShutdown();

    /** A Q8 weight object for a K×N matrix: int8 codes and one fp32 scale per 32 rows of a column. */
    static native void nativeQ8Alloc(int q8Id, int k, int n);

    /**
     * Quantizes rows [srcRow0, srcRow0+K) and columns [srcCol0, srcCol0+nCols) of the row-major
     * float buffer srcId (srcLd columns wide) into columns [dstCol0, dstCol0+nCols) of the Q8 object.
     */
    static native void nativeQ8QuantizeInto(int q8Id, int dstCol0, int srcId, int srcRow0, int srcCol0, int srcLd, int nCols);

    /** K and V planes of [layers][batch][heads][maxSeq][headDim] floats, zero-filled. */
    static native void nativeKvAlloc(int kvId, int layers, int batch, int heads, int maxSeq, int headDim);

    /** The same cache with fp16 planes: keys rounded after the rotation, values rounded, fp32 arithmetic; half the K/V bytes per step. */
    static native void nativeKvAllocF16(int kvId, int layers, int batch, int heads, int maxSeq, int headDim);

    /** Registers the plan object behind op 76 (one whole token step as one kernel); desc as include/deepj_cuda.h lists it. */
    static native void nativeDecodePlan(int planId, int[] desc, int len);

    /** Tensor parallelism, one JVM per GPU: allocates this rank's exchange buffer, returns its 64-byte IPC handle. */
    static native byte[] nativeTpCreate(int rank, int world, long slotFloats);

    /** All ranks' handles (world × 64 bytes, rank order), exchanged by the host's own means. */
    static native void nativeTpConnect(byte[] handles, int world);

    static native void nativeTpDestroy();

    /** Library counters into out (launches, graph replays, device-side error code at index 5, …). */
    static native void nativeStats(long[] out);
}
