// Constructors and accessors for the stand-in JNI objects of jni.h in this directory, with C
// linkage so that a test can drive the natives through ctypes: it builds arrays and an env here,
// calls the Java_… symbols directly with them, and reads back what the native did.
#include <cstring>

#include "jni.h"

extern "C" {

JNIEXPORT void* fj_env_new() { return new JNIEnv(); }
JNIEXPORT void fj_env_free(void* e) { delete static_cast<JNIEnv*>(e); }
JNIEXPORT int fj_pending(void* e) { return static_cast<JNIEnv*>(e)->pending ? 1 : 0; }
JNIEXPORT const char* fj_thrown_class(void* e) { return static_cast<JNIEnv*>(e)->thrown_class.c_str(); }
JNIEXPORT const char* fj_thrown_message(void* e) { return static_cast<JNIEnv*>(e)->thrown_message.c_str(); }
JNIEXPORT void fj_clear(void* e) {
    JNIEnv* env = static_cast<JNIEnv*>(e);
    env->pending = false;
    env->thrown_class.clear();
    env->thrown_message.clear();
    env->releases.clear();
}
JNIEXPORT int fj_release_count(void* e) { return static_cast<int>(static_cast<JNIEnv*>(e)->releases.size()); }
JNIEXPORT int fj_release_mode(void* e, int i) { return static_cast<JNIEnv*>(e)->releases[i].mode; }
JNIEXPORT const void* fj_release_array(void* e, int i) { return static_cast<JNIEnv*>(e)->releases[i].array; }
JNIEXPORT int fj_calls_in_critical(void* e) { return static_cast<JNIEnv*>(e)->calls_in_critical; }

static void fill(_jarray* a, const void* data, int n, size_t elem) {
    a->length = n;
    a->bytes.resize(static_cast<size_t>(n) * elem);
    if (data != nullptr && n > 0) std::memcpy(a->bytes.data(), data, a->bytes.size());
}
JNIEXPORT void* fj_ints_new(const int32_t* data, int n) { auto* a = new _jintArray(); fill(a, data, n, 4); return a; }
JNIEXPORT void* fj_floats_new(const float* data, int n) { auto* a = new _jfloatArray(); fill(a, data, n, 4); return a; }
JNIEXPORT void* fj_bytes_new(const int8_t* data, int n) { auto* a = new _jbyteArray(); fill(a, data, n, 1); return a; }
JNIEXPORT int fj_array_length(void* a) { return static_cast<_jarray*>(a)->length; }
JNIEXPORT void* fj_longs_new(int n) { auto* a = new _jlongArray(); fill(a, nullptr, n, 8); return a; }
JNIEXPORT void fj_array_read(void* a, void* out) {
    auto* arr = static_cast<_jarray*>(a);
    std::memcpy(out, arr->bytes.data(), arr->bytes.size());
}
JNIEXPORT int fj_array_pins(void* a) { return static_cast<_jarray*>(a)->pins; }
JNIEXPORT void fj_array_free(void* a) { delete static_cast<_jarray*>(a); }

}  // extern "C"
