// A stand-in for the JDK's <jni.h>, for tests on machines without a JDK: just the types and the
// JNIEnv members the CUDA natives use, backed by plain host arrays, and a log of what the natives
// did with them (which arrays were released in which mode, which exception was thrown).  It makes
// no attempt to be a JVM; it exists so that the shim's own logic is compiled and exercised.
#ifndef DEEPJ_FAKE_JNI_H
#define DEEPJ_FAKE_JNI_H

#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#define JNIEXPORT __attribute__((visibility("default")))
#define JNICALL
#define JNI_COMMIT 1
#define JNI_ABORT 2

typedef int32_t jint;
typedef int64_t jlong;
typedef float jfloat;
typedef jint jsize;
typedef uint8_t jboolean;
typedef int8_t jbyte;

struct _jobject { virtual ~_jobject() {} };
struct _jclass : _jobject { std::string name; };
struct _jarray : _jobject {
    std::vector<uint8_t> bytes;   // the "Java heap" copy
    jsize length = 0;
    int pins = 0;                 // outstanding Get*/GetPrimitiveArrayCritical
};
struct _jintArray : _jarray {};
struct _jfloatArray : _jarray {};
struct _jlongArray : _jarray {};
struct _jbyteArray : _jarray {};
typedef _jobject* jobject;
typedef _jclass* jclass;
typedef _jarray* jarray;
typedef _jintArray* jintArray;
typedef _jfloatArray* jfloatArray;
typedef _jlongArray* jlongArray;
typedef _jbyteArray* jbyteArray;

struct JNIEnv {
    struct Release { const void* array; int mode; };
    std::vector<Release> releases;
    std::string thrown_class, thrown_message;
    bool pending = false;
    bool in_critical = false;
    int calls_in_critical = 0;    // JNI calls made while an array was pinned (must stay 0)
    _jclass runtime_exception;
    // Elements handed out by Get<T>ArrayElements are copies, as a moving collector would make them.
    std::vector<std::vector<uint8_t>> copies;
    std::vector<_jarray*> created;
    ~JNIEnv() { for (auto* a : created) delete a; }

    void note() { if (in_critical) ++calls_in_critical; }

    jsize GetArrayLength(jarray a) { note(); return a->length; }
    jint* GetIntArrayElements(jintArray a, jboolean* is_copy) {
        note();
        copies.emplace_back(a->bytes);
        ++a->pins;
        if (is_copy) *is_copy = 1;
        return reinterpret_cast<jint*>(copies.back().data());
    }
    void ReleaseIntArrayElements(jintArray a, jint* p, jint mode) {
        note();
        if (mode != JNI_ABORT) std::memcpy(a->bytes.data(), p, a->bytes.size());
        if (mode != JNI_COMMIT) --a->pins;
        releases.push_back({a, mode});
    }
    void* GetPrimitiveArrayCritical(jarray a, jboolean* is_copy) {
        note();
        in_critical = true;
        ++a->pins;
        if (is_copy) *is_copy = 0;
        return a->bytes.data();
    }
    void ReleasePrimitiveArrayCritical(jarray a, void*, jint mode) {
        in_critical = false;
        if (mode != JNI_COMMIT) --a->pins;
        releases.push_back({a, mode});
    }
    jbyte* GetByteArrayElements(jbyteArray a, jboolean* is_copy) {
        note();
        copies.emplace_back(a->bytes);
        ++a->pins;
        if (is_copy) *is_copy = 1;
        return reinterpret_cast<jbyte*>(copies.back().data());
    }
    void ReleaseByteArrayElements(jbyteArray a, jbyte* p, jint mode) {
        note();
        if (mode != JNI_ABORT) std::memcpy(a->bytes.data(), p, a->bytes.size());
        if (mode != JNI_COMMIT) --a->pins;
        releases.push_back({a, mode});
    }
    jbyteArray NewByteArray(jsize n) {            // owned by the env, like a local reference
        note();
        auto* a = new _jbyteArray();
        a->length = n;
        a->bytes.resize(static_cast<size_t>(n));
        created.push_back(a);
        return a;
    }
    void SetByteArrayRegion(jbyteArray a, jsize start, jsize n, const jbyte* src) {
        note();
        std::memcpy(a->bytes.data() + start, src, static_cast<size_t>(n));
    }
    jclass FindClass(const char* name) {
        note();
        runtime_exception.name = name;
        return &runtime_exception;
    }
    jint ThrowNew(jclass c, const char* msg) {
        note();
        thrown_class = c->name;
        thrown_message = msg ? msg : "";
        pending = true;
        return 0;
    }
    jboolean ExceptionCheck() { note(); return pending ? 1 : 0; }
    void SetLongArrayRegion(jlongArray a, jsize start, jsize n, const jlong* src) {
        note();
        std::memcpy(a->bytes.data() + sizeof(jlong) * start, src, sizeof(jlong) * n);
    }
};

#endif
