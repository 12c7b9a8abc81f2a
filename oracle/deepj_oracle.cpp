// TEST INFRASTRUCTURE — CPU oracle for the DeepJ decoder-inference path.
//
// A C++17 restatement of the reference's own CPU arithmetic (Java, fp32 scalar
// loops).  It is the checker the CUDA path is compared against and the timed CPU
// baseline; it is never linked into, imported by or called from the product
// library.  Build: g++ -O2 -ffp-contract=off -fno-fast-math (Java never fuses a
// multiply-add and never reassociates).
//
// Parity status.  The fp32 ops are pinned by the reference's known-answer unit
// tests (tests/test_oracle_known_answers.py restates them).  Everything Q8 and
// everything KV-cache is this build's own definition (the reference has neither):
// "parity unpinned" for those.  java.util.Random and the java.lang.Math
// transcendental functions live in the JDK, which is not part of the reference
// tree; they are restated here from the Java SE API specification and glibc's
// correctly-rounded-in-practice double functions — unverified against a JVM.
//
// Each section cites the reference file:line it follows (paths relative to
// src/main/java/io/github/kirstenali/deepj/ unless stated).

#include <algorithm>
#include <atomic>
#include <cmath>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <functional>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

namespace {

thread_local std::string g_err;

// ───────────────────────────────────────────────────────────────────────────
// Row-range threading — concurrent/DeepJExecutor.java:80-112.
// forRange(start,end,body): chunks = min(threads, n), chunkSize = ceil(n/chunks),
// default threads = max(1, cores-1) (:22-24).  Sequential when threads <= 1.
// ───────────────────────────────────────────────────────────────────────────
int g_threads = std::max(1u, std::thread::hardware_concurrency() > 1
                                 ? std::thread::hardware_concurrency() - 1 : 1u);

class Pool {
public:
    explicit Pool(int n) : stop_(false) {
        for (int i = 0; i < n; i++) workers_.emplace_back([this] { loop(); });
    }
    ~Pool() {
        { std::lock_guard<std::mutex> l(m_); stop_ = true; }
        cv_.notify_all();
        for (auto& t : workers_) t.join();
    }
    void submit(std::function<void()> f) {
        { std::lock_guard<std::mutex> l(m_); q_.push_back(std::move(f)); }
        cv_.notify_one();
    }
    int size() const { return (int)workers_.size(); }
private:
    void loop() {
        for (;;) {
            std::function<void()> f;
            {
                std::unique_lock<std::mutex> l(m_);
                cv_.wait(l, [this] { return stop_ || !q_.empty(); });
                if (stop_ && q_.empty()) return;
                f = std::move(q_.front());
                q_.erase(q_.begin());
            }
            f();
        }
    }
    std::vector<std::thread> workers_;
    std::vector<std::function<void()>> q_;
    std::mutex m_;
    std::condition_variable cv_;
    bool stop_;
};
std::unique_ptr<Pool> g_pool;

template <class F>
void forRange(int start, int end, F body) {
    int n = end - start;
    if (n <= 0) return;
    int threads = g_threads;
    if (threads <= 1 || n == 1) {
        for (int i = start; i < end; i++) body(i);
        return;
    }
    if (!g_pool || g_pool->size() != threads) g_pool.reset(new Pool(threads));
    int chunks = std::min(threads, n);
    int chunkSize = (n + chunks - 1) / chunks;
    std::mutex m;
    std::condition_variable cv;
    int left = chunks;
    for (int t = 0; t < chunks; t++) {
        int s = start + t * chunkSize;
        int e = std::min(end, s + chunkSize);
        g_pool->submit([&, s, e] {
            for (int i = s; i < e; i++) body(i);
            std::lock_guard<std::mutex> l(m);
            if (--left == 0) cv.notify_one();
        });
    }
    std::unique_lock<std::mutex> l(m);
    cv.wait(l, [&] { return left == 0; });
}

// ───────────────────────────────────────────────────────────────────────────
// Scalar helpers — tensor/cpu/CpuBackend.java:24-28: transcendental functions are
// evaluated in double and rounded to float.
// ───────────────────────────────────────────────────────────────────────────
inline float fSqrt(float x) { return (float)std::sqrt((double)x); }
inline float fPow(float x, float e) { return (float)std::pow((double)x, (double)e); }
inline float fExp(float x) { return (float)std::exp((double)x); }
inline float fLog(float x) { return (float)std::log((double)x); }
inline float fTanh(float x) { return (float)std::tanh((double)x); }
inline float fSigmoid(float x) { return 1.0f / (1.0f + fExp(-x)); }   // CpuBackend.java:322
// CpuBackend.java:338-343
inline float geluScalar(float x) {
    float c = fSqrt(2.0f / (float)M_PI);
    float x3 = x * x * x;
    float t = c * (x + 0.044715f * x3);
    return 0.5f * x * (1.0f + fTanh(t));
}
// CpuBackend.java:345-354
inline float geluDerivScalar(float x) {
    float c = fSqrt(2.0f / (float)M_PI);
    float x2 = x * x;
    float x3 = x2 * x;
    float t = c * (x + 0.044715f * x3);
    float th = fTanh(t);
    float sech2 = 1.0f - th * th;
    float dtDx = c * (1.0f + 3.0f * 0.044715f * x2);
    return 0.5f * (1.0f + th) + 0.5f * x * sech2 * dtDx;
}
// Math.max / Math.min on floats (NaN-propagating, -0 < +0) as used by clamp/relu
// (CpuBackend.java:311,324).
inline float jmax(float a, float b) {
    if (a != a) return a;
    if (b != b) return b;
    if (a == 0.0f && b == 0.0f) return std::signbit(a) ? b : a;
    return a > b ? a : b;
}
inline float jmin(float a, float b) {
    if (a != a) return a;
    if (b != b) return b;
    if (a == 0.0f && b == 0.0f) return std::signbit(a) ? a : b;
    return a < b ? a : b;
}

inline float rowSum(const float* d, int cols) {        // CpuBackend.java:366-370
    float s = 0.0f;
    for (int c = 0; c < cols; c++) s += d[c];
    return s;
}
inline float rowMax(const float* d, int cols) {        // CpuBackend.java:360-364
    float m = -INFINITY;
    for (int c = 0; c < cols; c++) if (d[c] > m) m = d[c];
    return m;
}
// CpuBackend.java:378-398 (max, write exp(x-max), re-sum exp(x-max), divide)
inline void rowSoftmax(const float* in, float* out, int cols) {
    float mx = rowMax(in, cols);
    for (int c = 0; c < cols; c++) out[c] = fExp(in[c] - mx);
    float sumExp = 0.0f;
    for (int c = 0; c < cols; c++) sumExp += fExp(in[c] - mx);
    for (int c = 0; c < cols; c++) out[c] /= sumExp;
}

// CpuBackend.java:168-188 — ikj loop, fp32 accumulate in k order, rows in parallel.
void matmul(const float* a, const float* b, float* out, int m, int n, int k) {
    forRange(0, m, [&](int r) {
        const float* ar = a + (size_t)r * k;
        float* o = out + (size_t)r * n;
        for (int c = 0; c < n; c++) o[c] = 0.0f;
        for (int kk = 0; kk < k; kk++) {
            float aVal = ar[kk];
            const float* br = b + (size_t)kk * n;
            for (int c = 0; c < n; c++) o[c] += aVal * br[c];
        }
    });
}

// ───────────────────────────────────────────────────────────────────────────
// java.util.Random — restated from the Java SE API "general contract" text
// (48-bit LCG, polar-method nextGaussian with a cached second value).
// ───────────────────────────────────────────────────────────────────────────
// StrictMath.log is specified as the fdlibm algorithm; restated here from its
// published description (argument reduction x = 2^k·(1+f), s = f/(2+f), a degree-14
// even polynomial in s, ln2 split in hi/lo) so that nextGaussian matches a JVM in
// the last bit.  Only called with 0 < x < 1.
double strictLog(double x) {
    static const double ln2_hi = 6.93147180369123816490e-01, ln2_lo = 1.90821492927058770002e-10,
        Lg1 = 6.666666666666735130e-01, Lg2 = 3.999999999940941908e-01, Lg3 = 2.857142874366239149e-01,
        Lg4 = 2.222219843214978396e-01, Lg5 = 1.818357216161805012e-01, Lg6 = 1.531383769920937332e-01,
        Lg7 = 1.479819860511658591e-01;
    uint64_t bits; std::memcpy(&bits, &x, 8);
    int32_t hx = (int32_t)(bits >> 32);
    uint32_t lx = (uint32_t)bits;
    int32_t k = 0;
    if (hx < 0x00100000) {
        if (((hx & 0x7fffffff) | lx) == 0) return -INFINITY;
        if (hx < 0) return NAN;
        k -= 54; x *= 1.80143985094819840000e+16;
        std::memcpy(&bits, &x, 8); hx = (int32_t)(bits >> 32);
    }
    if (hx >= 0x7ff00000) return x + x;
    k += (hx >> 20) - 1023;
    hx &= 0x000fffff;
    int32_t i = (hx + 0x95f64) & 0x100000;
    bits = (bits & 0xffffffffULL) | ((uint64_t)(uint32_t)(hx | (i ^ 0x3ff00000)) << 32);
    std::memcpy(&x, &bits, 8);
    k += (i >> 20);
    double f = x - 1.0, dk;
    if ((0x000fffff & (2 + hx)) < 3) {
        if (f == 0.0) { if (k == 0) return 0.0; dk = (double)k; return dk * ln2_hi + dk * ln2_lo; }
        double R = f * f * (0.5 - 0.33333333333333333 * f);
        if (k == 0) return f - R;
        dk = (double)k; return dk * ln2_hi - ((R - dk * ln2_lo) - f);
    }
    double s = f / (2.0 + f);
    dk = (double)k;
    double z = s * s;
    i = hx - 0x6147a;
    double w = z * z;
    int32_t j = 0x6b851 - hx;
    double t1 = w * (Lg2 + w * (Lg4 + w * Lg6));
    double t2 = z * (Lg1 + w * (Lg3 + w * (Lg5 + w * Lg7)));
    i |= j;
    double R = t2 + t1;
    if (i > 0) {
        double hfsq = 0.5 * f * f;
        if (k == 0) return f - (hfsq - s * (hfsq + R));
        return dk * ln2_hi - ((hfsq - (s * (hfsq + R) + dk * ln2_lo)) - f);
    }
    if (k == 0) return f - s * (f - R);
    return dk * ln2_hi - ((s * (f - R) - dk * ln2_lo) - f);
}

struct JRandom {
    int64_t seed;
    bool haveNext = false;
    double nextNext = 0.0;
    explicit JRandom(int64_t s) : seed((s ^ 0x5DEECE66DLL) & ((1LL << 48) - 1)) {}
    int32_t next(int bits) {
        seed = (seed * 0x5DEECE66DLL + 0xBLL) & ((1LL << 48) - 1);
        return (int32_t)(seed >> (48 - bits));
    }
    int32_t nextInt(int32_t bound) {
        int32_t r = next(31);
        int32_t m = bound - 1;
        if ((bound & m) == 0) return (int32_t)(((int64_t)bound * (int64_t)r) >> 31);
        for (int32_t u = r; ; u = next(31)) {
            r = u % bound;
            // overflow test of u - r + m in 32-bit signed arithmetic
            int64_t t = (int64_t)u - r + m;
            if (t <= INT32_MAX) break;
        }
        return r;
    }
    float nextFloat() { return next(24) / (float)(1 << 24); }
    double nextDouble() {
        return (double)(((int64_t)next(26) << 27) + next(27)) * 0x1.0p-53;
    }
    double nextGaussian() {
        if (haveNext) { haveNext = false; return nextNext; }
        double v1, v2, s;
        do {
            v1 = 2 * nextDouble() - 1;
            v2 = 2 * nextDouble() - 1;
            s = v1 * v1 + v2 * v2;
        } while (s >= 1 || s == 0);
        double mul = std::sqrt(-2 * strictLog(s) / s);
        nextNext = v2 * mul;
        haveNext = true;
        return v1 * mul;
    }
};

// ───────────────────────────────────────────────────────────────────────────
// Counter-based generator for the large synthetic configs (this build's own; the
// reference has no such thing).  Integer-only until one final float multiply, so
// CPU and GPU produce identical bits: the sum of eight 16-bit uniform fields of
// two splitmix64 outputs (Irwin–Hall, variance 8·(65536²−1)/12), centred, times
// a float constant.
// ───────────────────────────────────────────────────────────────────────────
inline uint64_t splitmix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ULL;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}
inline uint64_t tensorKey(uint64_t seed, uint64_t ordinal) {
    return splitmix64(seed ^ (ordinal * 0xD1342543DE82EF95ULL));
}
inline float synthScale(float std_) {
    // std of (2·Σfields − 8·65535) is 2·sqrt(8·(65536²−1)/12)
    double sd = 2.0 * std::sqrt(8.0 * (65536.0 * 65536.0 - 1.0) / 12.0);
    return (float)((double)std_ / sd);
}
inline float synthValue(uint64_t key, uint64_t idx, float scale) {
    uint64_t a = splitmix64(key + 2 * idx);
    uint64_t b = splitmix64(key + 2 * idx + 1);
    int32_t s = 0;
    for (int i = 0; i < 4; i++) { s += (int32_t)((a >> (16 * i)) & 0xFFFF); s += (int32_t)((b >> (16 * i)) & 0xFFFF); }
    int32_t centred = 2 * s - 8 * 65535;
    return (float)centred * scale;
}

// ───────────────────────────────────────────────────────────────────────────
// Q8 — this build's own format (the reference has no quantization; parity
// unpinned).  For W [K×N] row-major (K = reduction dim), per output column n and
// per block of 32 consecutive k (last block shorter when K % 32 != 0):
//   amax = max|w|;  scale = amax / 127.0f;  q = clamp(lrintf(w / scale), -127, 127),
//   scale == 0 → q = 0.   Canonical arrays: codes[N][K] int8, scales[N][ceil(K/32)].
// ───────────────────────────────────────────────────────────────────────────
void q8Quantize(const float* W, int K, int N, int8_t* codes, float* scales) {
    int nb = (K + 31) / 32;
    forRange(0, N, [&](int n) {
        for (int b = 0; b < nb; b++) {
            int k0 = b * 32, k1 = std::min(K, k0 + 32);
            float amax = 0.0f;
            for (int k = k0; k < k1; k++) amax = std::max(amax, std::fabs(W[(size_t)k * N + n]));
            float scale = amax / 127.0f;
            scales[(size_t)n * nb + b] = scale;
            for (int k = k0; k < k1; k++) {
                int q = 0;
                if (scale != 0.0f) {
                    q = (int)lrintf(W[(size_t)k * N + n] / scale);
                    q = std::max(-127, std::min(127, q));
                }
                codes[(size_t)n * K + k] = (int8_t)q;
            }
        }
    });
}
void q8Dequantize(const int8_t* codes, const float* scales, int K, int N, float* W) {
    int nb = (K + 31) / 32;
    forRange(0, N, [&](int n) {
        for (int k = 0; k < K; k++)
            W[(size_t)k * N + n] = (float)codes[(size_t)n * K + k] * scales[(size_t)n * nb + k / 32];
    });
}

// ───────────────────────────────────────────────────────────────────────────
// Buffer pool + command-stream interpreter.  Stream layout follows
// tensor/ComputeGraph.java:19-60 (op codes) and :89-147 (strides / buffer slots);
// per-op arithmetic follows tensor/cpu/CpuBackend.java.
// ───────────────────────────────────────────────────────────────────────────
std::unordered_map<int, std::vector<float>> g_bufs;

inline float bitsToFloat(int32_t b) { float f; std::memcpy(&f, &b, 4); return f; }

std::vector<float>& need(int id, size_t n, const char* what) {
    auto it = g_bufs.find(id);
    if (it == g_bufs.end()) throw std::runtime_error(std::string(what) + ": missing buffer id=" + std::to_string(id));
    if (it->second.size() < n) throw std::runtime_error(std::string(what) + ": buffer id=" + std::to_string(id) + " too small");
    return it->second;
}

template <class F> void unary(const int32_t* c, F f) {
    int n = c[3];
    auto& in = need(c[1], n, "unary"); auto& out = need(c[2], n, "unary");
    for (int i = 0; i < n; i++) out[i] = f(in[i]);
}
template <class F> void binary(const int32_t* c, F f) {
    int n = c[4];
    auto& a = need(c[1], n, "binary"); auto& b = need(c[2], n, "binary"); auto& out = need(c[3], n, "binary");
    for (int i = 0; i < n; i++) out[i] = f(a[i], b[i]);
}
template <class F> void scalarOp(const int32_t* c, F f) {
    int n = c[4]; float s = bitsToFloat(c[3]);
    auto& in = need(c[1], n, "scalar"); auto& out = need(c[2], n, "scalar");
    for (int i = 0; i < n; i++) out[i] = f(in[i], s);
}
template <class F> void rowBroadcast(const int32_t* c, F f) {     // vec is [1×cols]
    int rows = c[4], cols = c[5];
    auto& a = need(c[1], (size_t)rows * cols, "rowBroadcast"); auto& v = need(c[2], cols, "rowBroadcast");
    auto& out = need(c[3], (size_t)rows * cols, "rowBroadcast");
    for (int r = 0; r < rows; r++) for (int k = 0; k < cols; k++) out[(size_t)r * cols + k] = f(a[(size_t)r * cols + k], v[k]);
}
template <class F> void colBroadcast(const int32_t* c, F f) {     // vec is [rows×1]
    int rows = c[4], cols = c[5];
    auto& a = need(c[1], (size_t)rows * cols, "colBroadcast"); auto& v = need(c[2], rows, "colBroadcast");
    auto& out = need(c[3], (size_t)rows * cols, "colBroadcast");
    for (int r = 0; r < rows; r++) for (int k = 0; k < cols; k++) out[(size_t)r * cols + k] = f(a[(size_t)r * cols + k], v[r]);
}

int opStride(int op) {
    switch (op) {
        case 7: case 8: case 9: case 10: case 11: case 12: case 13: case 15: return 4;
        case 1: case 2: case 3: case 4: case 14: case 16: return 5;
        case 6: case 21: case 22: case 23: case 29: case 30: case 31: case 33: case 34: case 17: case 36: case 38: case 41: return 5;
        case 35: case 39: case 40: case 18: case 24: case 25: case 26: case 27: case 28: case 32: return 6;
        case 5: case 19: case 37: case 42: return 7;
        case 20: return 13;
        default: return -1;
    }
}

void execOp(const int32_t* c) {
    int op = c[0];
    switch (op) {
        case 1: binary(c, [](float x, float y) { return x + y; }); break;
        case 2: binary(c, [](float x, float y) { return x - y; }); break;
        case 3: binary(c, [](float x, float y) { return x * y; }); break;
        case 4: binary(c, [](float x, float y) { return x / y; }); break;
        case 5: {   // [5,a,b,out,m,n,k]
            int m = c[4], n = c[5], k = c[6];
            auto& a = need(c[1], (size_t)m * k, "matmul"); auto& b = need(c[2], (size_t)k * n, "matmul");
            auto& out = need(c[3], (size_t)m * n, "matmul");
            matmul(a.data(), b.data(), out.data(), m, n, k);
            break;
        }
        case 6: scalarOp(c, [](float x, float s) { return x * s; }); break;
        case 7: unary(c, fSqrt); break;
        case 8: unary(c, [](float x) { return -x; }); break;
        case 9: unary(c, fExp); break;
        case 10: unary(c, fLog); break;
        case 11: unary(c, fTanh); break;
        case 12: unary(c, fSigmoid); break;
        case 13: unary(c, [](float x) { return jmax(0.0f, x); }); break;
        case 14: binary(c, [](float x, float g) { return x > 0.0f ? g : 0.0f; }); break;        // CpuBackend.java:328-331
        case 15: unary(c, geluScalar); break;
        case 16: binary(c, [](float x, float g) { return g * geluDerivScalar(x); }); break;   // :333-336
        case 17: {  // softmax rows
            int rows = c[3], cols = c[4];
            auto& in = need(c[1], (size_t)rows * cols, "softmax"); auto& out = need(c[2], (size_t)rows * cols, "softmax");
            forRange(0, rows, [&](int r) { rowSoftmax(in.data() + (size_t)r * cols, out.data() + (size_t)r * cols, cols); });
            break;
        }
        case 18: {  // softmax backward — CpuBackend.java:411-427
            int rows = c[4], cols = c[5];
            auto& g = need(c[1], (size_t)rows * cols, "softmaxBackward"); auto& s = need(c[2], (size_t)rows * cols, "softmaxBackward");
            auto& out = need(c[3], (size_t)rows * cols, "softmaxBackward");
            for (int r = 0; r < rows; r++) {
                size_t base = (size_t)r * cols;
                float dot = 0.0f;
                for (int k = 0; k < cols; k++) dot += g[base + k] * s[base + k];
                for (int k = 0; k < cols; k++) out[base + k] = s[base + k] * (g[base + k] - dot);
            }
            break;
        }
        case 19: {  // layernorm backward — CpuBackend.java:489-516
            int rows = c[5], cols = c[6];
            auto& dXHat = need(c[1], (size_t)rows * cols, "layerNormBackward"); auto& xHat = need(c[2], (size_t)rows * cols, "layerNormBackward");
            auto& sd = need(c[3], rows, "layerNormBackward"); auto& out = need(c[4], (size_t)rows * cols, "layerNormBackward");
            for (int r = 0; r < rows; r++) {
                size_t base = (size_t)r * cols;
                float invStd = 1.0f / sd[r];
                float sumD = 0.0f, sumDX = 0.0f;
                for (int k = 0; k < cols; k++) { float d = dXHat[base + k]; sumD += d; sumDX += d * xHat[base + k]; }
                for (int k = 0; k < cols; k++) {
                    float d = dXHat[base + k], xh = xHat[base + k];
                    out[base + k] = invStd * (d - sumD / cols - xh * (sumDX / cols));
                }
            }
            break;
        }
        case 20: {  // AdamW — CpuBackend.java:461-487
            int n = c[12];
            auto& w = need(c[1], n, "adamW"); auto& g = need(c[2], n, "adamW");
            auto& mt = need(c[3], n, "adamW"); auto& vt = need(c[4], n, "adamW");
            float lr = bitsToFloat(c[5]), b1 = bitsToFloat(c[6]), b2 = bitsToFloat(c[7]), eps = bitsToFloat(c[8]);
            float wd = bitsToFloat(c[9]), bc1 = bitsToFloat(c[10]), bc2 = bitsToFloat(c[11]);
            for (int i = 0; i < n; i++) {
                float grad = g[i];
                float mNew = b1 * mt[i] + (1.0f - b1) * grad;
                float vNew = b2 * vt[i] + (1.0f - b2) * (grad * grad);
                mt[i] = mNew; vt[i] = vNew;
                float mHat = mNew / bc1, vHat = vNew / bc2;
                float update = (lr * mHat) / (fSqrt(vHat) + eps);
                if (wd != 0.0f) update += lr * wd * w[i];
                w[i] -= update;
            }
            break;
        }
        case 21: scalarOp(c, [](float x, float s) { return x + s; }); break;
        case 22: scalarOp(c, [](float x, float s) { return x / s; }); break;
        case 23: {  // transpose — CpuBackend.java:301-308
            int rows = c[3], cols = c[4];
            auto& in = need(c[1], (size_t)rows * cols, "transpose"); auto& out = need(c[2], (size_t)rows * cols, "transpose");
            for (int r = 0; r < rows; r++) for (int k = 0; k < cols; k++) out[(size_t)k * rows + r] = in[(size_t)r * cols + k];
            break;
        }
        case 24: rowBroadcast(c, [](float x, float y) { return x + y; }); break;
        case 25: colBroadcast(c, [](float x, float y) { return x + y; }); break;
        case 26: colBroadcast(c, [](float x, float y) { return x - y; }); break;
        case 27: colBroadcast(c, [](float x, float y) { return x / y; }); break;
        case 28: rowBroadcast(c, [](float x, float y) { return x * y; }); break;
        case 32: colBroadcast(c, [](float x, float y) { return x * y; }); break;
        case 29: {  // sumRows [rows×cols] → [1×cols] — CpuBackend.java:219-227
            int rows = c[3], cols = c[4];
            auto& in = need(c[1], (size_t)rows * cols, "sumRows"); auto& out = need(c[2], cols, "sumRows");
            for (int k = 0; k < cols; k++) out[k] = 0.0f;
            for (int r = 0; r < rows; r++) for (int k = 0; k < cols; k++) out[k] += in[(size_t)r * cols + k];
            break;
        }
        case 30: case 31: case 33: case 34: case 38: {   // per-row reductions → [rows×1]
            int rows = c[3], cols = c[4];
            auto& in = need(c[1], (size_t)rows * cols, "rowReduce"); auto& out = need(c[2], rows, "rowReduce");
            float invCols = 1.0f / cols;
            for (int r = 0; r < rows; r++) {
                const float* d = in.data() + (size_t)r * cols;
                if (op == 33) out[r] = rowSum(d, cols);
                else if (op == 30) out[r] = rowSum(d, cols) * invCols;                 // CpuBackend.java:242-251
                else if (op == 34) out[r] = rowMax(d, cols);
                else if (op == 38) { float s = 0.0f; for (int k = 0; k < cols; k++) s += std::fabs(d[k]); out[r] = s; }
                else {                                                                // variance :253-268
                    float mean = rowSum(d, cols) * invCols, acc = 0.0f;
                    for (int k = 0; k < cols; k++) { float diff = d[k] - mean; acc += diff * diff; }
                    out[r] = acc * invCols;
                }
            }
            break;
        }
        case 35: {  // clamp [op,in,out,minBits,maxBits,n] — CpuBackend.java:311
            int n = c[5]; float lo = bitsToFloat(c[3]), hi = bitsToFloat(c[4]);
            auto& in = need(c[1], n, "clamp"); auto& out = need(c[2], n, "clamp");
            for (int i = 0; i < n; i++) out[i] = jmin(hi, jmax(lo, in[i]));
            break;
        }
        case 36: scalarOp(c, fPow); break;
        case 37: case 42: {   // scatter-add rows [op,target,indices,grad,tRows,tCols,nIdx] — CpuBackend.java:542-549
            int tRows = c[4], tCols = c[5], nIdx = c[6];
            auto& tgt = need(c[1], (size_t)tRows * tCols, "scatterAdd"); auto& idx = need(c[2], nIdx, "scatterAdd");
            auto& g = need(c[3], (size_t)nIdx * tCols, "scatterAdd");
            for (int i = 0; i < nIdx; i++) {
                int row = (int)idx[i];
                if (row < 0 || row >= tRows) continue;   // native side skips out-of-range rows (native/deepj_metal_jni.mm:574)
                for (int k = 0; k < tCols; k++) tgt[(size_t)row * tCols + k] += g[(size_t)i * tCols + k];
            }
            break;
        }
        case 39: {  // CE row losses [op,logits,targets,out,rows,cols] — CpuBackend.java:433-444 per row
            int rows = c[4], cols = c[5];
            auto& lg = need(c[1], (size_t)rows * cols, "ceLoss"); auto& tg = need(c[2], rows, "ceLoss"); auto& out = need(c[3], rows, "ceLoss");
            for (int r = 0; r < rows; r++) {
                const float* d = lg.data() + (size_t)r * cols;
                int t = (int)tg[r];
                if (t < 0 || t >= cols) { out[r] = NAN; continue; }   // native/deepj_metal_jni.mm:472-476
                float mx = rowMax(d, cols), se = 0.0f;
                for (int k = 0; k < cols; k++) se += fExp(d[k] - mx);
                out[r] = fLog(se) + mx - d[t];
            }
            break;
        }
        case 40: {  // CE gradient — CpuBackend.java:446-459
            int rows = c[4], cols = c[5];
            auto& lg = need(c[1], (size_t)rows * cols, "ceGrad"); auto& tg = need(c[2], rows, "ceGrad"); auto& out = need(c[3], (size_t)rows * cols, "ceGrad");
            for (int r = 0; r < rows; r++) {
                float* o = out.data() + (size_t)r * cols;
                int t = (int)tg[r];
                if (t < 0 || t >= cols) { for (int k = 0; k < cols; k++) o[k] = NAN; continue; }
                rowSoftmax(lg.data() + (size_t)r * cols, o, cols);
                o[t] -= 1.0f;
                for (int k = 0; k < cols; k++) o[k] /= (float)rows;
            }
            break;
        }
        case 41: {  // sum of all elements → [1×1] — CpuBackend.java:283-287
            int rows = c[3], cols = c[4];
            auto& in = need(c[1], (size_t)rows * cols, "sum"); auto& out = need(c[2], 1, "sum");
            float s = 0.0f;
            for (size_t i = 0; i < (size_t)rows * cols; i++) s += in[i];
            out[0] = s;
            break;
        }
        default:
            throw std::runtime_error("unknown op code " + std::to_string(op));
    }
}

// ───────────────────────────────────────────────────────────────────────────
// Layers and models.
// ───────────────────────────────────────────────────────────────────────────
struct Mat { int rows = 0, cols = 0; std::vector<float> d; Mat() {} Mat(int r, int c) : rows(r), cols(c), d((size_t)r * c, 0.0f) {} };

// transformer/embeddings/RotaryEmbedding.java:52-71 — float exponent, double pow,
// float theta, double cos/sin rounded to float.
void ropeTables(int headDim, int maxSeq, float* cosT, float* sinT) {
    int half = headDim / 2;
    for (int pos = 0; pos < maxSeq; pos++)
        for (int i = 0; i < half; i++) {
            float expo = (2.0f * i) / headDim;
            float theta = (float)(pos / std::pow((double)10000.0f, (double)expo));
            cosT[(size_t)pos * half + i] = (float)std::cos((double)theta);
            sinT[(size_t)pos * half + i] = (float)std::sin((double)theta);
        }
}

// layers/transformer/norm/RMSNorm1D.java:46-57 as six backend ops:
// x*x → meanAlongRows → +1e-6 → sqrt → x / rms (col broadcast) → * gamma (row broadcast)
void rmsNorm(const Mat& x, const std::vector<float>& gamma, Mat& out) {
    out = Mat(x.rows, x.cols);
    float invCols = 1.0f / x.cols;
    for (int r = 0; r < x.rows; r++) {
        const float* xr = &x.d[(size_t)r * x.cols];
        float s = 0.0f;
        for (int c = 0; c < x.cols; c++) { float sq = xr[c] * xr[c]; s += sq; }
        float meanSq = s * invCols;
        float rms = fSqrt(meanSq + 1e-6f);
        for (int c = 0; c < x.cols; c++) out.d[(size_t)r * x.cols + c] = (xr[c] / rms) * gamma[c];
    }
}
// layers/transformer/norm/LayerNorm1D.java:34-42 (GPT): mean, biased variance
// (CpuBackend.java:253-268), std = sqrt(var + 1e-5), (x - mean)/std * gamma + beta.
void layerNorm(const Mat& x, const std::vector<float>& gamma, const std::vector<float>& beta, Mat& out) {
    out = Mat(x.rows, x.cols);
    float invCols = 1.0f / x.cols;
    for (int r = 0; r < x.rows; r++) {
        const float* xr = &x.d[(size_t)r * x.cols];
        float mean = rowSum(xr, x.cols) * invCols;
        float acc = 0.0f;
        for (int c = 0; c < x.cols; c++) { float diff = xr[c] - mean; acc += diff * diff; }
        float var = acc * invCols;
        float sd = fSqrt(var + 1e-5f);
        for (int c = 0; c < x.cols; c++)
            out.d[(size_t)r * x.cols + c] = ((xr[c] - mean) / sd) * gamma[c] + beta[c];
    }
}

// layers/Linear.java:31-36: x.matmul(W).addRowVector(b); bias == nullptr → bare matmul
void linear(const Mat& x, const float* W, const float* b, int dIn, int dOut, Mat& out) {
    out = Mat(x.rows, dOut);
    matmul(x.d.data(), W, out.d.data(), x.rows, dOut, dIn);
    if (b) for (int r = 0; r < x.rows; r++) for (int c = 0; c < dOut; c++) out.d[(size_t)r * dOut + c] += b[c];
}

enum Kind { LLAMA = 0, DEEPSEEK = 1, GPT = 2 };

struct Block {
    std::vector<float> g1, g2, b1n, b2n;          // norm gammas (+ betas for GPT)
    std::vector<float> Wq, Wk, Wv, Wo;            // MHSA [d×d]
    std::vector<float> Wdq, Wuq, Wdkv, Wuk, Wuv;  // MLA
    std::vector<float> Wg, bg, Wu, bu, Wd, bd;    // SwiGLU (GPT FNN: Wg=fc1, Wd=fc2)
};

struct Model {
    int kind, V, maxSeq, d, H, L, F, qRank, kvRank;
    std::vector<float> emb, pos, gF, bF, Wlm, blm;
    std::vector<Block> blocks;
    std::vector<float> cosT, sinT;
    // KV cache for incremental decode: [layer][pos][d]
    std::vector<std::vector<float>> kc, vc;
    int cachePos = 0;
};

void fillJava(JRandom& r, std::vector<float>& w, size_t n, double mult) {
    w.resize(n);
    for (size_t i = 0; i < n; i++) w[i] = (float)(r.nextGaussian() * mult);   // CpuBackend.java:148-152
}
void fillSynth(uint64_t seed, uint64_t& ordinal, std::vector<float>& w, size_t n, float std_) {
    w.resize(n);
    uint64_t key = tensorKey(seed, ordinal++);
    float sc = synthScale(std_);
    float* p = w.data();
    int chunks = 64;
    forRange(0, chunks, [&](int ci) {
        size_t s = n * ci / chunks, e = n * (ci + 1) / chunks;
        for (size_t i = s; i < e; i++) p[i] = synthValue(key, i, sc);
    });
}

// Weight init.  initMode 0: java.util.Random draw order of the reference
// constructors (models/llama/LlamaModel.java:27-42, transformer/LlamaTransformerBuilder.java:45-55,
// layers/transformer/attention/MultiHeadSelfAttention.java:47-50,
// MultiHeadLatentAttention.java:82-87, layers/transformer/SwiGLULayer.java:56-58);
// values are (float)(nextGaussian()*mult), mult = 0.1 in the reference.
// initMode 1: counter-based generator above, one ordinal per matrix in the same order.
Model* buildModel(int kind, int V, int maxSeq, int d, int H, int L, int F, int qRank, int kvRank,
                  int64_t seed, int initMode, double std_, int nLayersBuilt) {
    auto* m = new Model();
    m->kind = kind; m->V = V; m->maxSeq = maxSeq; m->d = d; m->H = H; m->L = L; m->F = F; m->qRank = qRank; m->kvRank = kvRank;
    int built = nLayersBuilt > 0 ? std::min(nLayersBuilt, L) : L;
    uint64_t ord = 0;
    JRandom rEmb(seed), rStack(seed), rHead(seed + 1), rPos(seed + 2);
    auto fill = [&](JRandom& r, std::vector<float>& w, size_t n) {
        if (initMode == 0) fillJava(r, w, n, std_); else fillSynth((uint64_t)seed, ord, w, n, (float)std_);
    };
    fill(rEmb, m->emb, (size_t)V * d);
    m->blocks.resize(built);
    for (int l = 0; l < built; l++) {
        Block& b = m->blocks[l];
        b.g1.assign(d, 1.0f); b.g2.assign(d, 1.0f);
        if (kind == GPT) {
            // blocks/GPTTransformerBlock.java:61-64: ln1, ln2 (no draws), attention, then FNN's two Linear layers
            // (layers/FNN.java:56-61; biases are zeros).  Wg / bg hold the hidden layer, Wd / bd the output layer.
            b.b1n.assign(d, 0.0f); b.b2n.assign(d, 0.0f);
            fill(rStack, b.Wq, (size_t)d * d); fill(rStack, b.Wk, (size_t)d * d);
            fill(rStack, b.Wv, (size_t)d * d); fill(rStack, b.Wo, (size_t)d * d);
            fill(rStack, b.Wg, (size_t)d * F); b.bg.assign(F, 0.0f);
            fill(rStack, b.Wd, (size_t)F * d); b.bd.assign(d, 0.0f);
            continue;
        }
        if (kind == LLAMA) {
            fill(rStack, b.Wq, (size_t)d * d); fill(rStack, b.Wk, (size_t)d * d);
            fill(rStack, b.Wv, (size_t)d * d); fill(rStack, b.Wo, (size_t)d * d);
        } else {
            fill(rStack, b.Wdq, (size_t)d * qRank); fill(rStack, b.Wuq, (size_t)qRank * d);
            fill(rStack, b.Wdkv, (size_t)d * kvRank); fill(rStack, b.Wuk, (size_t)kvRank * d);
            fill(rStack, b.Wuv, (size_t)kvRank * d); fill(rStack, b.Wo, (size_t)d * d);
        }
        fill(rStack, b.Wg, (size_t)d * F); b.bg.assign(F, 0.0f);
        fill(rStack, b.Wu, (size_t)d * F); b.bu.assign(F, 0.0f);
        fill(rStack, b.Wd, (size_t)F * d); b.bd.assign(d, 0.0f);
    }
    // Skipped layers still consume their ordinals so that the LM head is the same
    // tensor whether or not every layer is materialised (synthetic mode only).
    if (initMode == 1) ord += (uint64_t)(L - built) * (kind == LLAMA ? 7 : (kind == GPT ? 6 : 9));
    m->gF.assign(d, 1.0f);
    fill(rHead, m->Wlm, (size_t)d * V); m->blm.assign(V, 0.0f);
    if (kind == GPT) {
        // models/gpt/GPTModel.java:31-46: position table from Random(seed + 2), drawn after the LM head; then every
        // parameter, gains included, is multiplied by initScale (GPTConfig's default 0.2f; :78-83).  In synthetic mode
        // the table takes the ordinal after the LM head and nothing is rescaled (std is given directly).
        m->bF.assign(d, 0.0f);
        fill(rPos, m->pos, (size_t)maxSeq * d);
        if (initMode == 0) {
            const float f = 0.2f;
            auto sc = [&](std::vector<float>& w) { for (auto& v : w) v = v * f; };
            sc(m->emb); sc(m->pos); sc(m->gF); sc(m->bF); sc(m->Wlm); sc(m->blm);
            for (auto& b : m->blocks) {
                sc(b.g1); sc(b.b1n); sc(b.g2); sc(b.b2n); sc(b.Wq); sc(b.Wk); sc(b.Wv); sc(b.Wo);
                sc(b.Wg); sc(b.bg); sc(b.Wd); sc(b.bd);
            }
        }
    }
    int hd = d / H;
    m->cosT.resize((size_t)maxSeq * (hd / 2)); m->sinT.resize((size_t)maxSeq * (hd / 2));
    ropeTables(hd, maxSeq, m->cosT.data(), m->sinT.data());
    return m;
}

// transformer/embeddings/RotaryEmbedding.java:112-122 on one row of headDim floats
inline void ropeRow(const Model& m, float* row, int pos, int hd) {
    if (m.kind == GPT) return;                      // plain MultiHeadSelfAttention: transformQueryKey is the identity
    int half = hd / 2;
    for (int i = 0; i < half; i++) {
        float c = m.cosT[(size_t)pos * half + i], s = m.sinT[(size_t)pos * half + i];
        float x0 = row[2 * i], x1 = row[2 * i + 1];
        row[2 * i] = x0 * c - x1 * s;
        row[2 * i + 1] = x0 * s + x1 * c;
    }
}

// The attention tail shared by MHSA and MLA, restating HeadOps.java:33-140 +
// MultiHeadSelfAttention.java:60-86: split heads, RoPE on Q and K, per head
// S = (Q·Kᵀ)·scale via transpose + ikj matmul, + causal mask (0 / -1e9f), row
// softmax, P·V, merge heads.  Q, K, V are [seq×d]; result merged [seq×d].
void attentionTail(const Model& m, Mat& Q, Mat& K, const Mat& V, Mat& merged) {
    int seq = Q.rows, d = m.d, H = m.H, hd = d / H;
    float scale = (float)(1.0 / std::sqrt((double)hd));
    merged = Mat(seq, d);
    forRange(0, H, [&](int h) {
        std::vector<float> q((size_t)seq * hd), k((size_t)seq * hd), v((size_t)seq * hd), kT((size_t)seq * hd);
        for (int i = 0; i < seq; i++) {
            std::memcpy(&q[(size_t)i * hd], &Q.d[(size_t)i * d + h * hd], hd * 4);
            std::memcpy(&k[(size_t)i * hd], &K.d[(size_t)i * d + h * hd], hd * 4);
            std::memcpy(&v[(size_t)i * hd], &V.d[(size_t)i * d + h * hd], hd * 4);
            ropeRow(m, &q[(size_t)i * hd], i, hd);
            ropeRow(m, &k[(size_t)i * hd], i, hd);
        }
        for (int i = 0; i < seq; i++) for (int j = 0; j < hd; j++) kT[(size_t)j * seq + i] = k[(size_t)i * hd + j];
        std::vector<float> s((size_t)seq * seq, 0.0f), p((size_t)seq * seq), y((size_t)seq * hd, 0.0f);
        for (int r = 0; r < seq; r++) {
            float* sr = &s[(size_t)r * seq];
            for (int kk = 0; kk < hd; kk++) {
                float a = q[(size_t)r * hd + kk];
                const float* br = &kT[(size_t)kk * seq];
                for (int c = 0; c < seq; c++) sr[c] += a * br[c];
            }
            for (int c = 0; c < seq; c++) sr[c] = sr[c] * scale;
            for (int c = 0; c < seq; c++) sr[c] = sr[c] + ((c > r) ? -1e9f : 0.0f);
            rowSoftmax(sr, &p[(size_t)r * seq], seq);
            float* yr = &y[(size_t)r * hd];
            for (int kk = 0; kk < seq; kk++) {
                float a = p[(size_t)r * seq + kk];
                const float* vr = &v[(size_t)kk * hd];
                for (int c = 0; c < hd; c++) yr[c] += a * vr[c];
            }
            std::memcpy(&merged.d[(size_t)r * d + h * hd], yr, hd * 4);
        }
    });
}

// models/DecoderOnlyModel.java:58-64 full forward: ids[seq] → logits [seq×V].
// Blocks: layers/transformer/blocks/LlamaTransformerBlock.java:50-53,
// DeepSeekTransformerBlock.java:54-57; SwiGLU: layers/transformer/SwiGLULayer.java:63-70.
void forwardFull(Model& m, const int* ids, int seq, float* logits, int lastRowOnly) {
    int d = m.d;
    Mat x(seq, d);
    for (int i = 0; i < seq; i++) {
        if (ids[i] < 0 || ids[i] >= m.V) throw std::runtime_error("Token id out of range: " + std::to_string(ids[i]));
        std::memcpy(&x.d[(size_t)i * d], &m.emb[(size_t)ids[i] * d], d * 4);
    }
    if (seq > m.maxSeq) throw std::runtime_error("seqLen " + std::to_string(seq) + " exceeds maxSeqLen " + std::to_string(m.maxSeq));
    if (m.kind == GPT)      // GPTModel.embed: tokEmb.forward(ids).add(posEmb.forward(seq)) (embeddings/PositionalEmbedding.java:26-33)
        for (int i = 0; i < seq; i++) for (int c = 0; c < d; c++) x.d[(size_t)i * d + c] = x.d[(size_t)i * d + c] + m.pos[(size_t)i * d + c];
    for (auto& b : m.blocks) {
        Mat n1, Q, K, V, merged, att;
        if (m.kind == GPT) layerNorm(x, b.g1, b.b1n, n1); else rmsNorm(x, b.g1, n1);
        if (m.kind == LLAMA || m.kind == GPT) {
            linear(n1, b.Wq.data(), nullptr, d, d, Q);
            linear(n1, b.Wk.data(), nullptr, d, d, K);
            linear(n1, b.Wv.data(), nullptr, d, d, V);
        } else {   // MultiHeadLatentAttention.java:93-124
            Mat cQ, cKV;
            linear(n1, b.Wdq.data(), nullptr, d, m.qRank, cQ);
            linear(cQ, b.Wuq.data(), nullptr, m.qRank, d, Q);
            linear(n1, b.Wdkv.data(), nullptr, d, m.kvRank, cKV);
            linear(cKV, b.Wuk.data(), nullptr, m.kvRank, d, K);
            linear(cKV, b.Wuv.data(), nullptr, m.kvRank, d, V);
        }
        attentionTail(m, Q, K, V, merged);
        linear(merged, b.Wo.data(), nullptr, d, d, att);
        Mat x2(seq, d);
        for (size_t i = 0; i < x2.d.size(); i++) x2.d[i] = x.d[i] + att.d[i];
        Mat n2, g, u, dn;
        if (m.kind == GPT) {        // blocks/GPTTransformerBlock.java:66-74, layers/FNN.java:70-88: Linear → GELU → Linear
            layerNorm(x2, b.g2, b.b2n, n2);
            linear(n2, b.Wg.data(), b.bg.data(), d, m.F, g);
            for (size_t i = 0; i < g.d.size(); i++) g.d[i] = geluScalar(g.d[i]);
        } else {
            rmsNorm(x2, b.g2, n2);
            linear(n2, b.Wg.data(), b.bg.data(), d, m.F, g);
            linear(n2, b.Wu.data(), b.bu.data(), d, m.F, u);
            for (size_t i = 0; i < g.d.size(); i++) { float sg = fSigmoid(g.d[i]); float si = g.d[i] * sg; g.d[i] = si * u.d[i]; }
        }
        linear(g, b.Wd.data(), b.bd.data(), m.F, d, dn);
        for (size_t i = 0; i < x.d.size(); i++) x.d[i] = x2.d[i] + dn.d[i];
    }
    Mat nf, lg;
    if (lastRowOnly) {
        Mat last(1, d);
        std::memcpy(last.d.data(), &x.d[(size_t)(seq - 1) * d], d * 4);
        if (m.kind == GPT) layerNorm(last, m.gF, m.bF, nf); else rmsNorm(last, m.gF, nf);
        linear(nf, m.Wlm.data(), m.blm.data(), d, m.V, lg);
        std::memcpy(logits, lg.d.data(), (size_t)m.V * 4);
    } else {
        if (m.kind == GPT) layerNorm(x, m.gF, m.bF, nf); else rmsNorm(x, m.gF, nf);
        linear(nf, m.Wlm.data(), m.blm.data(), d, m.V, lg);
        std::memcpy(logits, lg.d.data(), (size_t)seq * m.V * 4);
    }
}

// Incremental step with a K/V cache (this build's addition; the reference
// re-forwards the whole context, models/TextGenerator.java:91-100).  Every
// reference op is row-wise independent and masked softmax terms are exactly +0,
// so this reproduces the last logits row of forwardFull bit for bit as long as
// the window never slides.
void decodeStep(Model& m, int token, float* logits) {
    int d = m.d, H = m.H, hd = d / H, pos = m.cachePos;
    if (pos >= m.maxSeq) throw std::runtime_error("KV cache full");
    if (token < 0 || token >= m.V) throw std::runtime_error("Token id out of range: " + std::to_string(token));
    if (m.kc.empty()) { m.kc.assign(m.blocks.size(), std::vector<float>((size_t)m.maxSeq * d)); m.vc = m.kc; }
    float scale = (float)(1.0 / std::sqrt((double)hd));
    Mat x(1, d);
    std::memcpy(x.d.data(), &m.emb[(size_t)token * d], d * 4);
    if (m.kind == GPT) for (int c = 0; c < d; c++) x.d[c] = x.d[c] + m.pos[(size_t)pos * d + c];
    for (size_t l = 0; l < m.blocks.size(); l++) {
        Block& b = m.blocks[l];
        Mat n1, Q, K, V, att;
        if (m.kind == GPT) layerNorm(x, b.g1, b.b1n, n1); else rmsNorm(x, b.g1, n1);
        if (m.kind == LLAMA || m.kind == GPT) {
            linear(n1, b.Wq.data(), nullptr, d, d, Q);
            linear(n1, b.Wk.data(), nullptr, d, d, K);
            linear(n1, b.Wv.data(), nullptr, d, d, V);
        } else {
            Mat cQ, cKV;
            linear(n1, b.Wdq.data(), nullptr, d, m.qRank, cQ);
            linear(cQ, b.Wuq.data(), nullptr, m.qRank, d, Q);
            linear(n1, b.Wdkv.data(), nullptr, d, m.kvRank, cKV);
            linear(cKV, b.Wuk.data(), nullptr, m.kvRank, d, K);
            linear(cKV, b.Wuv.data(), nullptr, m.kvRank, d, V);
        }
        for (int h = 0; h < H; h++) { ropeRow(m, &Q.d[(size_t)h * hd], pos, hd); ropeRow(m, &K.d[(size_t)h * hd], pos, hd); }
        std::memcpy(&m.kc[l][(size_t)pos * d], K.d.data(), d * 4);
        std::memcpy(&m.vc[l][(size_t)pos * d], V.d.data(), d * 4);
        Mat merged(1, d);
        int seq = pos + 1;
        forRange(0, H, [&](int h) {
            std::vector<float> s(seq), p(seq);
            for (int c = 0; c < seq; c++) {
                const float* kr = &m.kc[l][(size_t)c * d + h * hd];
                float acc = 0.0f;
                for (int kk = 0; kk < hd; kk++) acc += Q.d[(size_t)h * hd + kk] * kr[kk];
                s[c] = (acc * scale) + 0.0f;
            }
            rowSoftmax(s.data(), p.data(), seq);
            float* yr = &merged.d[(size_t)h * hd];
            for (int j = 0; j < hd; j++) yr[j] = 0.0f;
            for (int c = 0; c < seq; c++) {
                const float* vr = &m.vc[l][(size_t)c * d + h * hd];
                for (int j = 0; j < hd; j++) yr[j] += p[c] * vr[j];
            }
        });
        linear(merged, b.Wo.data(), nullptr, d, d, att);
        Mat x2(1, d);
        for (int i = 0; i < d; i++) x2.d[i] = x.d[i] + att.d[i];
        Mat n2, g, u, dn;
        if (m.kind == GPT) {
            layerNorm(x2, b.g2, b.b2n, n2);
            linear(n2, b.Wg.data(), b.bg.data(), d, m.F, g);
            for (size_t i = 0; i < g.d.size(); i++) g.d[i] = geluScalar(g.d[i]);
        } else {
            rmsNorm(x2, b.g2, n2);
            linear(n2, b.Wg.data(), b.bg.data(), d, m.F, g);
            linear(n2, b.Wu.data(), b.bu.data(), d, m.F, u);
            for (size_t i = 0; i < g.d.size(); i++) { float sg = fSigmoid(g.d[i]); float si = g.d[i] * sg; g.d[i] = si * u.d[i]; }
        }
        linear(g, b.Wd.data(), b.bd.data(), m.F, d, dn);
        for (int i = 0; i < d; i++) x.d[i] = x2.d[i] + dn.d[i];
    }
    Mat nf, lg;
    if (m.kind == GPT) layerNorm(x, m.gF, m.bF, nf); else rmsNorm(x, m.gF, nf);
    linear(nf, m.Wlm.data(), m.blm.data(), d, m.V, lg);
    std::memcpy(logits, lg.d.data(), (size_t)m.V * 4);
    m.cachePos++;
}

// Greedy pick = models/TextGenerator.java:104-170 with topK = 1: a stable
// descending sort under Float.compare(a[j], a[i]) keeps the lowest index among
// equal values, orders -0.0 below +0.0 and NaN above everything.
int javaFloatCompare(float a, float b) {
    if (a < b) return -1;
    if (a > b) return 1;
    int32_t ia, ib;
    std::memcpy(&ia, &a, 4); std::memcpy(&ib, &b, 4);
    if (a != a) ia = 0x7fc00000;
    if (b != b) ib = 0x7fc00000;
    return ia == ib ? 0 : (ia < ib ? -1 : 1);
}
int greedyPick(const float* logits, int n) {
    int best = 0;
    for (int i = 1; i < n; i++) if (javaFloatCompare(logits[i], logits[best]) > 0) best = i;
    return best;
}

std::vector<float>* weightByName(Model& m, const std::string& name, int layer) {
    if (name == "emb") return &m.emb;
    if (name == "pos" && m.kind == GPT) return &m.pos;
    if (name == "bF" && m.kind == GPT) return &m.bF;
    if (name == "gF") return &m.gF;
    if (name == "Wlm") return &m.Wlm;
    if (name == "blm") return &m.blm;
    if (layer < 0 || layer >= (int)m.blocks.size()) return nullptr;
    Block& b = m.blocks[layer];
    if (m.kind == GPT) {              // the names Q8Decoder and the checkpoint layout use for the GPT family
        if (name == "b1") return &b.b1n; if (name == "b2") return &b.b2n;
        if (name == "W1") return &b.Wg;  if (name == "c1") return &b.bg;  if (name == "W2") return &b.Wd;  if (name == "c2") return &b.bd;
    }
    if (name == "g1") return &b.g1;   if (name == "g2") return &b.g2;
    if (name == "Wq") return &b.Wq;   if (name == "Wk") return &b.Wk;   if (name == "Wv") return &b.Wv;   if (name == "Wo") return &b.Wo;
    if (name == "Wdq") return &b.Wdq; if (name == "Wuq") return &b.Wuq; if (name == "Wdkv") return &b.Wdkv;
    if (name == "Wuk") return &b.Wuk; if (name == "Wuv") return &b.Wuv;
    if (name == "Wg") return &b.Wg;   if (name == "bg") return &b.bg;   if (name == "Wu") return &b.Wu;   if (name == "bu") return &b.bu;
    if (name == "Wd") return &b.Wd;   if (name == "bd") return &b.bd;
    return nullptr;
}

}  // namespace

#define ORACLE_TRY try {
#define ORACLE_CATCH } catch (const std::exception& e) { g_err = e.what(); return -1; } return 0;

extern "C" {

const char* oracle_last_error() { return g_err.c_str(); }
int oracle_set_threads(int n) { g_threads = n > 0 ? n : std::max(1, (int)std::thread::hardware_concurrency() - 1); g_pool.reset(); return g_threads; }
int oracle_get_threads() { return g_threads; }

// ── the five runtime calls of tensor/GpuRuntime.java:9-28 over host memory ──
int oracle_alloc_buffers(const int32_t* ids, const int32_t* sizes, int32_t count) {
    ORACLE_TRY
    for (int i = 0; i < count; i++) if (!g_bufs.count(ids[i])) g_bufs[ids[i]].assign((size_t)sizes[i], 0.0f);
    ORACLE_CATCH
}
int oracle_upload_buffer(int32_t id, const float* data, int32_t len) {
    ORACLE_TRY
    auto it = g_bufs.find(id);
    if (it == g_bufs.end()) throw std::runtime_error("Buffer not found for upload");
    if ((size_t)len > it->second.size()) throw std::runtime_error("upload larger than buffer");
    std::memcpy(it->second.data(), data, (size_t)len * 4);
    ORACLE_CATCH
}
int oracle_download_buffer(int32_t id, float* out, int32_t len) {
    ORACLE_TRY
    auto it = g_bufs.find(id);
    if (it == g_bufs.end()) throw std::runtime_error("Buffer not found for download");
    if ((size_t)len > it->second.size()) throw std::runtime_error("download larger than buffer");
    std::memcpy(out, it->second.data(), (size_t)len * 4);
    ORACLE_CATCH
}
int oracle_release_buffers(const int32_t* ids, int32_t count) {
    for (int i = 0; i < count; i++) g_bufs.erase(ids[i]);
    return 0;
}
int oracle_flush_ops(const int32_t* cmd, int32_t len) {
    ORACLE_TRY
    int pos = 0;
    while (pos < len) {
        int stride = opStride(cmd[pos]);
        if (stride < 0) throw std::runtime_error("unknown op code " + std::to_string(cmd[pos]));
        if (pos + stride > len) throw std::runtime_error("truncated command stream");
        execOp(cmd + pos);
        pos += stride;
    }
    ORACLE_CATCH
}

// ── java.util.Random ──
void* oracle_jrandom_new(int64_t seed) { return new JRandom(seed); }
void oracle_jrandom_free(void* r) { delete (JRandom*)r; }
int32_t oracle_jrandom_next_int(void* r, int32_t bound) { return ((JRandom*)r)->nextInt(bound); }
float oracle_jrandom_next_float(void* r) { return ((JRandom*)r)->nextFloat(); }
double oracle_jrandom_next_double(void* r) { return ((JRandom*)r)->nextDouble(); }
double oracle_jrandom_next_gaussian(void* r) { return ((JRandom*)r)->nextGaussian(); }
// Tensor.random: (float)(nextGaussian() * mult), row-major fill
void oracle_jrandom_fill_gaussian(void* r, float* out, int64_t n, double mult) {
    for (int64_t i = 0; i < n; i++) out[i] = (float)(((JRandom*)r)->nextGaussian() * mult);
}
// counter-based synthetic tensor
void oracle_synth_fill(uint64_t seed, uint64_t ordinal, float std_, int64_t offset, int64_t n, float* out) {
    uint64_t key = tensorKey(seed, ordinal);
    float sc = synthScale(std_);
    for (int64_t i = 0; i < n; i++) out[i] = synthValue(key, (uint64_t)(offset + i), sc);
}

// ── Q8 ──
int oracle_q8_quantize(const float* W, int32_t K, int32_t N, int8_t* codes, float* scales) {
    ORACLE_TRY q8Quantize(W, K, N, codes, scales); ORACLE_CATCH
}
int oracle_q8_dequantize(const int8_t* codes, const float* scales, int32_t K, int32_t N, float* W) {
    ORACLE_TRY q8Dequantize(codes, scales, K, N, W); ORACLE_CATCH
}
int oracle_matmul(const float* a, const float* b, float* out, int32_t m, int32_t n, int32_t k) {
    ORACLE_TRY matmul(a, b, out, m, n, k); ORACLE_CATCH
}
int oracle_rope_tables(int32_t headDim, int32_t maxSeq, float* cosT, float* sinT) {
    ORACLE_TRY
    if (headDim <= 0 || headDim % 2 != 0) throw std::runtime_error("headDim must be a positive even number, got " + std::to_string(headDim));
    if (maxSeq <= 0) throw std::runtime_error("maxSeqLen must be > 0");
    ropeTables(headDim, maxSeq, cosT, sinT);
    ORACLE_CATCH
}

// ── models ──
void* oracle_model_new(int32_t kind, int32_t V, int32_t maxSeq, int32_t d, int32_t H, int32_t L, int32_t F,
                       int32_t qRank, int32_t kvRank, int64_t seed, int32_t initMode, double std_, int32_t nLayersBuilt) {
    try { return buildModel(kind, V, maxSeq, d, H, L, F, qRank, kvRank, seed, initMode, std_, nLayersBuilt); }
    catch (const std::exception& e) { g_err = e.what(); return nullptr; }
}
void oracle_model_free(void* m) { delete (Model*)m; }
int64_t oracle_model_weight_size(void* m, const char* name, int32_t layer) {
    auto* w = weightByName(*(Model*)m, name, layer);
    return w ? (int64_t)w->size() : -1;
}
int oracle_model_get_weight(void* m, const char* name, int32_t layer, float* out) {
    ORACLE_TRY
    auto* w = weightByName(*(Model*)m, name, layer);
    if (!w) throw std::runtime_error(std::string("no such weight: ") + name);
    std::memcpy(out, w->data(), w->size() * 4);
    ORACLE_CATCH
}
int oracle_model_set_weight(void* m, const char* name, int32_t layer, const float* in, int64_t n) {
    ORACLE_TRY
    auto* w = weightByName(*(Model*)m, name, layer);
    if (!w) throw std::runtime_error(std::string("no such weight: ") + name);
    if ((int64_t)w->size() != n) throw std::runtime_error(std::string("size mismatch for weight: ") + name);
    std::memcpy(w->data(), in, (size_t)n * 4);
    ORACLE_CATCH
}
// Replace every matmul weight by dequant(Q8(W)) — "oracle B".
int oracle_model_apply_q8(void* mp) {
    ORACLE_TRY
    Model& m = *(Model*)mp;
    auto rq = [&](std::vector<float>& W, int K, int N) {
        if (W.empty()) return;
        std::vector<int8_t> codes((size_t)K * N);
        std::vector<float> scales((size_t)N * ((K + 31) / 32));
        q8Quantize(W.data(), K, N, codes.data(), scales.data());
        q8Dequantize(codes.data(), scales.data(), K, N, W.data());
    };
    for (auto& b : m.blocks) {
        rq(b.Wq, m.d, m.d); rq(b.Wk, m.d, m.d); rq(b.Wv, m.d, m.d); rq(b.Wo, m.d, m.d);
        rq(b.Wdq, m.d, m.qRank); rq(b.Wuq, m.qRank, m.d); rq(b.Wdkv, m.d, m.kvRank);
        rq(b.Wuk, m.kvRank, m.d); rq(b.Wuv, m.kvRank, m.d);
        rq(b.Wg, m.d, m.F); rq(b.Wu, m.d, m.F); rq(b.Wd, m.F, m.d);
    }
    rq(m.Wlm, m.d, m.V);
    ORACLE_CATCH
}
int oracle_model_forward(void* m, const int32_t* ids, int32_t seq, float* logits, int32_t lastRowOnly) {
    ORACLE_TRY forwardFull(*(Model*)m, ids, seq, logits, lastRowOnly); ORACLE_CATCH
}
int oracle_model_reset_cache(void* m) { ((Model*)m)->cachePos = 0; return 0; }
int oracle_model_decode_step(void* m, int32_t token, float* logits) {
    ORACLE_TRY decodeStep(*(Model*)m, token, logits); ORACLE_CATCH
}
int32_t oracle_greedy_pick(const float* logits, int32_t n) { return greedyPick(logits, n); }
// TextGenerator.sampleFromLogits (models/TextGenerator.java:104-151): stable descending order under Float.compare,
// the first topK indices (0 = all), p_i = (float) Math.exp(logit_i / T - max) with max over the scaled logits,
// a sequential float sum, p_i /= sum, then the first i with r <= running sum (r = Random.nextFloat()).
int32_t oracle_sample_topk(const float* logits, int32_t n, float temperature, int32_t topK, float r) {
    std::vector<int32_t> order(n);
    for (int i = 0; i < n; i++) order[i] = i;
    auto key = [&](int i) {            // Float.compare's total order as a signed integer
        float v = logits[i];
        int32_t b;
        if (v != v) b = 0x7fc00000; else std::memcpy(&b, &v, 4);
        return b ^ ((b >> 31) & 0x7fffffff);
    };
    std::stable_sort(order.begin(), order.end(), [&](int i, int j) { return key(i) > key(j); });
    int k = topK == 0 ? n : std::min(topK, n);
    float mx = -INFINITY;
    for (int i = 0; i < k; i++) { float v = logits[order[i]] / temperature; if (v > mx) mx = v; }
    std::vector<float> p(k);
    float sum = 0.0f;
    for (int i = 0; i < k; i++) { p[i] = (float)std::exp((double)(logits[order[i]] / temperature - mx)); sum += p[i]; }
    for (int i = 0; i < k; i++) p[i] /= sum;
    float cum = 0.0f;
    for (int i = 0; i < k; i++) { cum += p[i]; if (r <= cum) return order[i]; }
    return order[k - 1];
}
// Reference-faithful greedy generation: full re-forward of the context per token
// (models/TextGenerator.java:81-100), window = last maxSeq ids (:172-175).
int oracle_generate_greedy(void* mp, const int32_t* prompt, int32_t nPrompt, int32_t maxNew,
                           int32_t useCache, int32_t* outTokens, float* outLogits) {
    ORACLE_TRY
    Model& m = *(Model*)mp;
    std::vector<int32_t> ids(prompt, prompt + nPrompt);
    std::vector<float> lg(m.V);
    if (useCache) {
        m.cachePos = 0;
        for (int i = 0; i < nPrompt; i++) decodeStep(m, ids[i], lg.data());
    }
    for (int t = 0; t < maxNew; t++) {
        if (!useCache) {
            int n = (int)ids.size();
            int start = n > m.maxSeq ? n - m.maxSeq : 0;
            forwardFull(m, ids.data() + start, n - start, lg.data(), 1);
        }
        int next = greedyPick(lg.data(), m.V);
        if (outLogits) std::memcpy(outLogits + (size_t)t * m.V, lg.data(), (size_t)m.V * 4);
        outTokens[t] = next;
        ids.push_back(next);
        if (useCache && t + 1 < maxNew) decodeStep(m, next, lg.data());
    }
    ORACLE_CATCH
}

}  // extern "C"
