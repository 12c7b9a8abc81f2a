// JNI natives of io.github.kirstenali.deepj.tensor.cuda.CudaNative over the C ABI of
// include/deepj_cuda.h.  The five graph natives have the signatures and the error behaviour of
// the reference's Metal natives (tensor/metal/MetalNative.java:41-57,
// native/deepj_metal_jni.mm:1480-1560): inputs are released with JNI_ABORT, the download array
// is committed, and a failed call raises java.lang.RuntimeException carrying the library's
// message.  The remaining natives expose the Q8 / KV-cache objects and the device binding.
//
// The file compiles to nothing when no <jni.h> is on the include path (the library is then
// driven through its C ABI alone); building with a JDK adds the natives to the same library,
// which is why it is called libdeepj_cuda_jni.
//
// Uploads and downloads pin the Java array (GetPrimitiveArrayCritical) instead of asking for a
// copy: a 7B model's projection is 180 MB of floats, and the copy would double the host traffic
// of the slowest step of loading.  Nothing between pin and release calls back into the VM.
#if __has_include(<jni.h>)
#include <jni.h>

#include <cstdint>

#include "deepj_cuda.h"

#define CUDA_NATIVE(name) Java_io_github_kirstenali_deepj_tensor_cuda_CudaNative_##name

namespace {

void raise(JNIEnv* env, const char* msg) {
    if (env->ExceptionCheck()) return;                      // keep the first exception
    jclass cls = env->FindClass("java/lang/RuntimeException");
    if (cls != nullptr) env->ThrowNew(cls, msg);
}

void raise_last(JNIEnv* env) { raise(env, deepj_cuda_last_error()); }

// A read-only view of an int[] argument; released with JNI_ABORT (nothing to write back).
struct IntsIn {
    JNIEnv* env; jintArray arr; jint* p; jsize len;
    IntsIn(JNIEnv* e, jintArray a) : env(e), arr(a), p(nullptr), len(0) {
        if (a == nullptr) return;
        len = e->GetArrayLength(a);
        p = e->GetIntArrayElements(a, nullptr);
    }
    ~IntsIn() { if (p != nullptr) env->ReleaseIntArrayElements(arr, p, JNI_ABORT); }
    bool ok(jint need) const { return p != nullptr && need >= 0 && need <= len; }
};

static_assert(sizeof(jint) == sizeof(int32_t) && sizeof(jfloat) == sizeof(float), "JNI scalar sizes");

}  // namespace

extern "C" {

JNIEXPORT void JNICALL CUDA_NATIVE(nativeAllocBuffers)(JNIEnv* env, jclass, jintArray idsArr, jintArray sizesArr, jint count) {
    int rc;
    {
        IntsIn ids(env, idsArr), sizes(env, sizesArr);
        if (!ids.ok(count) || !sizes.ok(count)) { rc = -1; }
        else rc = deepj_cuda_alloc_buffers(reinterpret_cast<const int32_t*>(ids.p), reinterpret_cast<const int32_t*>(sizes.p), count);
    }                                                        // arrays released before any throw
    if (rc == -1) raise(env, "nativeAllocBuffers: count exceeds the id or size array");
    else if (rc != 0) raise_last(env);
}

JNIEXPORT void JNICALL CUDA_NATIVE(nativeUploadBuffer)(JNIEnv* env, jclass, jint bufId, jfloatArray dataArr) {
    if (dataArr == nullptr) { raise(env, "nativeUploadBuffer: null array"); return; }
    const jsize len = env->GetArrayLength(dataArr);          // the Java array's length, as the reference copies
    void* p = env->GetPrimitiveArrayCritical(dataArr, nullptr);
    if (p == nullptr) { raise(env, "nativeUploadBuffer: array could not be pinned"); return; }
    const int rc = deepj_cuda_upload_buffer(bufId, static_cast<const float*>(p), len);
    env->ReleasePrimitiveArrayCritical(dataArr, p, JNI_ABORT);
    if (rc != 0) raise_last(env);
}

JNIEXPORT void JNICALL CUDA_NATIVE(nativeDownloadBuffer)(JNIEnv* env, jclass, jint bufId, jfloatArray outArr) {
    if (outArr == nullptr) { raise(env, "nativeDownloadBuffer: null array"); return; }
    const jsize len = env->GetArrayLength(outArr);
    // wait for the queued work BEFORE the array is pinned: a critical region must be short and must not block
    // (it holds off the collector), so it covers the device-to-host copy only
    if (deepj_cuda_synchronize() != 0) { raise_last(env); return; }
    void* p = env->GetPrimitiveArrayCritical(outArr, nullptr);
    if (p == nullptr) { raise(env, "nativeDownloadBuffer: array could not be pinned"); return; }
    const int rc = deepj_cuda_download_buffer(bufId, static_cast<float*>(p), len);
    env->ReleasePrimitiveArrayCritical(outArr, p, rc == 0 ? 0 : JNI_ABORT);   // commit only what was written
    if (rc != 0) raise_last(env);
}

JNIEXPORT void JNICALL CUDA_NATIVE(nativeReleaseBuffers)(JNIEnv* env, jclass, jintArray idsArr, jint count) {
    int rc;
    {
        IntsIn ids(env, idsArr);
        rc = ids.ok(count) ? deepj_cuda_release_buffers(reinterpret_cast<const int32_t*>(ids.p), count) : -1;
    }
    if (rc == -1) raise(env, "nativeReleaseBuffers: count exceeds the id array");
    else if (rc != 0) raise_last(env);
}

JNIEXPORT void JNICALL CUDA_NATIVE(nativeFlushOps)(JNIEnv* env, jclass, jintArray cmdArr, jint cmdLength) {
    int rc;
    {
        IntsIn cmd(env, cmdArr);
        rc = cmd.ok(cmdLength) ? deepj_cuda_flush_ops(reinterpret_cast<const int32_t*>(cmd.p), cmdLength) : -1;
    }
    if (rc == -1) raise(env, "nativeFlushOps: cmdStreamLength exceeds the command array");
    else if (rc != 0) raise_last(env);
}

// ───────────── additions: enqueue-only flush, device binding, Q8 and KV objects ─────────────

JNIEXPORT void JNICALL CUDA_NATIVE(nativeFlushOpsAsync)(JNIEnv* env, jclass, jintArray cmdArr, jint cmdLength) {
    int rc;
    {
        IntsIn cmd(env, cmdArr);                             // the stream is copied or matched to a cached graph before the call returns
        rc = cmd.ok(cmdLength) ? deepj_cuda_flush_ops_async(reinterpret_cast<const int32_t*>(cmd.p), cmdLength) : -1;
    }
    if (rc == -1) raise(env, "nativeFlushOpsAsync: cmdStreamLength exceeds the command array");
    else if (rc != 0) raise_last(env);
}

JNIEXPORT void JNICALL CUDA_NATIVE(nativeSynchronize)(JNIEnv* env, jclass) {
    if (deepj_cuda_synchronize() != 0) raise_last(env);
}

JNIEXPORT void JNICALL CUDA_NATIVE(nativeInit)(JNIEnv* env, jclass, jint device) {
    if (deepj_cuda_init(device) != 0) raise_last(env);
}

JNIEXPORT void JNICALL CUDA_NATIVE(nativeShutdown)(JNIEnv* env, jclass) {
    if (deepj_cuda_shutdown() != 0) raise_last(env);
}

JNIEXPORT void JNICALL CUDA_NATIVE(nativeQ8Alloc)(JNIEnv* env, jclass, jint q8Id, jint K, jint N) {
    if (deepj_cuda_q8_alloc(q8Id, K, N) != 0) raise_last(env);
}

JNIEXPORT void JNICALL CUDA_NATIVE(nativeQ8QuantizeInto)(JNIEnv* env, jclass, jint q8Id, jint dstCol0, jint srcId,
                                                         jint srcRow0, jint srcCol0, jint srcLd, jint nCols) {
    if (deepj_cuda_q8_quantize_into(q8Id, dstCol0, srcId, srcRow0, srcCol0, srcLd, nCols) != 0) raise_last(env);
}

JNIEXPORT void JNICALL CUDA_NATIVE(nativeKvAlloc)(JNIEnv* env, jclass, jint kvId, jint layers, jint batch, jint heads,
                                                  jint maxSeq, jint headDim) {
    if (deepj_cuda_kv_alloc(kvId, layers, batch, heads, maxSeq, headDim) != 0) raise_last(env);
}

// The same cache with fp16 planes (keys rounded after the rotation, values rounded; fp32 arithmetic in every kernel).
JNIEXPORT void JNICALL CUDA_NATIVE(nativeKvAllocF16)(JNIEnv* env, jclass, jint kvId, jint layers, jint batch, jint heads,
                                                     jint maxSeq, jint headDim) {
    if (deepj_cuda_kv_alloc_f16(kvId, layers, batch, heads, maxSeq, headDim) != 0) raise_last(env);
}

// Decode plan behind op 76 (the whole-token kernel): desc as deepj_cuda_decode_plan documents it.
JNIEXPORT void JNICALL CUDA_NATIVE(nativeDecodePlan)(JNIEnv* env, jclass, jint planId, jintArray descArr, jint len) {
    int rc;
    {
        IntsIn desc(env, descArr);
        rc = desc.ok(len) ? deepj_cuda_decode_plan(planId, reinterpret_cast<const int32_t*>(desc.p), len) : -1;
    }
    if (rc == -1) raise(env, "nativeDecodePlan: len exceeds the descriptor array");
    else if (rc != 0) raise_last(env);
}

// ───────────── tensor parallelism: one JVM per GPU, the host exchanges the 64-byte handles ─────────────

// Allocates this rank's exchange buffer and returns its CUDA IPC handle (64 bytes), or null with an exception pending.
JNIEXPORT jbyteArray JNICALL CUDA_NATIVE(nativeTpCreate)(JNIEnv* env, jclass, jint rank, jint world, jlong slotFloats) {
    jbyte handle[64];
    if (deepj_cuda_tp_create(rank, world, slotFloats, handle) != 0) { raise_last(env); return nullptr; }
    jbyteArray out = env->NewByteArray(64);
    if (out == nullptr) { raise(env, "nativeTpCreate: could not allocate the handle array"); return nullptr; }
    env->SetByteArrayRegion(out, 0, 64, handle);
    return out;
}

// handles: world × 64 bytes in rank order.
JNIEXPORT void JNICALL CUDA_NATIVE(nativeTpConnect)(JNIEnv* env, jclass, jbyteArray handles, jint world) {
    if (handles == nullptr) { raise(env, "nativeTpConnect: null handles"); return; }
    const jsize len = env->GetArrayLength(handles);
    if (world < 1 || (jlong)len != (jlong)world * 64) { raise(env, "nativeTpConnect: expected world x 64 handle bytes"); return; }
    jbyte* p = env->GetByteArrayElements(handles, nullptr);
    if (p == nullptr) { raise(env, "nativeTpConnect: handles could not be read"); return; }
    const int rc = deepj_cuda_tp_connect(p, world);
    env->ReleaseByteArrayElements(handles, p, JNI_ABORT);
    if (rc != 0) raise_last(env);
}

JNIEXPORT void JNICALL CUDA_NATIVE(nativeTpDestroy)(JNIEnv* env, jclass) {
    if (deepj_cuda_tp_destroy() != 0) raise_last(env);
}

// Library counters (launches, graph replays, device error code, …) into out[0 .. out.length).
JNIEXPORT void JNICALL CUDA_NATIVE(nativeStats)(JNIEnv* env, jclass, jlongArray outArr) {
    if (outArr == nullptr) { raise(env, "nativeStats: null array"); return; }
    const jsize n = env->GetArrayLength(outArr);
    int64_t tmp[16] = {0};
    const int m = n < 16 ? static_cast<int>(n) : 16;
    if (deepj_cuda_stats(tmp, m) != 0) { raise_last(env); return; }
    static_assert(sizeof(jlong) == sizeof(int64_t), "jlong is 64 bits");
    env->SetLongArrayRegion(outArr, 0, m, reinterpret_cast<const jlong*>(tmp));
}

}  // extern "C"
#endif  // __has_include(<jni.h>)
