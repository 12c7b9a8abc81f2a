// Small decode-path kernels: embedding row gather, greedy argmax, position advance,
// device copy, and the counter-based synthetic weight generator.
#include "kernels.h"

namespace dj {

namespace {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Embedding.forward → Tensor.sliceRows (transformer/embeddings/Embedding.java:28-34):
// out[r] = table[ids[r]].  The reference throws on an out-of-range id before any
// work; the runtime cannot see device-resident ids, so such a row is filled with NaN.
__global__ void k_embed_gather(const float* __restrict__ table, const float* __restrict__ ids, float* __restrict__ out,
                               int rows, int d, int vocab) {
    pdl_wait();
    pdl_launch_dependents();
    int r = blockIdx.x;
    int id = (int)ids[r];
    bool ok = id >= 0 && id < vocab;
    for (int c = threadIdx.x; c < d; c += blockDim.x)
        out[(size_t)r * d + c] = ok ? table[(size_t)id * d + c] : NAN;
}

// Total order of Float.compare (models/TextGenerator.java:163-170): -0.0 < +0.0,
// NaN above +inf.  Map the bits to a signed key with the same order.
__device__ __forceinline__ int order_key(float v) {
    int b = (v != v) ? 0x7fc00000 : __float_as_int(v);
    return b ^ ((b >> 31) & 0x7fffffff);
}

// Greedy pick: the first index of the largest value (a stable descending sort
// keeps the lowest index among equals).  grid (parts, rows): every CTA reduces its slice of the row to one
// (key, index) pair; the CTA that arrives last at the row (a self-resetting ticket) reduces the parts.  One CTA
// per row costs a full load round trip per 1024 columns — 18 µs for a 32000-entry row.
constexpr int kArgmaxParts = 16;
__global__ void __launch_bounds__(256) k_argmax_rows(const float* __restrict__ in, float* __restrict__ out, int rows, int cols,
                                                      int* __restrict__ scratch, int* __restrict__ tickets) {
    __shared__ int s_key[8];
    __shared__ int s_idx[8];
    __shared__ int s_last;
    pdl_wait();
    pdl_launch_dependents();
    const int part = blockIdx.x, parts = gridDim.x, r = blockIdx.y;
    const float* d = in + (size_t)r * cols;
    const int per = ((cols + parts - 1) / parts + 3) & ~3;
    const int lo = min(cols, part * per), hi = min(cols, lo + per);
    int bestKey = INT_MIN, bestIdx = INT_MAX;
    for (int c = lo + (int)threadIdx.x; c < hi; c += blockDim.x) {
        int k = order_key(d[c]);
        if (k > bestKey || (k == bestKey && c < bestIdx)) { bestKey = k; bestIdx = c; }
    }
    auto warp_best = [&]() {
        for (int o = 16; o > 0; o >>= 1) {
            int k2 = __shfl_xor_sync(0xffffffffu, bestKey, o), i2 = __shfl_xor_sync(0xffffffffu, bestIdx, o);
            if (k2 > bestKey || (k2 == bestKey && i2 < bestIdx)) { bestKey = k2; bestIdx = i2; }
        }
    };
    warp_best();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if (lane == 0) { s_key[warp] = bestKey; s_idx[warp] = bestIdx; }
    __syncthreads();
    if (warp == 0) {
        bestKey = lane < nw ? s_key[lane] : INT_MIN;
        bestIdx = lane < nw ? s_idx[lane] : INT_MAX;
        warp_best();
        if (parts == 1) { if (lane == 0) out[r] = (float)bestIdx; return; }
        if (lane == 0) {
            scratch[((size_t)r * parts + part) * 2] = bestKey;
            scratch[((size_t)r * parts + part) * 2 + 1] = bestIdx;
            __threadfence();
            const int t = atomicAdd(&tickets[r], 1);
            s_last = t == parts - 1;
            if (s_last) tickets[r] = 0;
        }
        __syncwarp();
        if (__shfl_sync(0xffffffffu, lane == 0 ? s_last : 0, 0)) {
            __threadfence();
            bestKey = lane < parts ? __ldcg(scratch + ((size_t)r * parts + lane) * 2) : INT_MIN;
            bestIdx = lane < parts ? __ldcg(scratch + ((size_t)r * parts + lane) * 2 + 1) : INT_MAX;
            warp_best();
            if (lane == 0) out[r] = (float)bestIdx;
        }
    }
}

// Temperature / top-k sampling with the reference's semantics (models/TextGenerator.java:104-151): indices in
// stable descending order of the logits (Float.compare, lowest index first among equals), the first k of them,
// p_i = (float) exp((double)(logit_i / T − max)), a sequential float sum, p_i /= sum, and the first i whose running
// sum reaches r (r = Random.nextFloat(), drawn by the host and passed per row).  One CTA of 1024 threads per row;
// k ≤ 1024.  The k-th largest key is found by an 8-bit radix select (four passes over the row), the candidates are
// gathered (equal keys by ascending index) and sorted by (key, −index) with a bitonic network in shared memory.
constexpr int kSampleMaxK = 1024;

__global__ void __launch_bounds__(1024) k_sample_topk(const float* __restrict__ logits, const float* __restrict__ rbuf,
                                                       float* __restrict__ out, int rows, int cols, int topK, float temperature) {
    __shared__ unsigned s_hist[256];
    __shared__ unsigned long long s_cand[kSampleMaxK];
    __shared__ float s_p[kSampleMaxK];
    __shared__ unsigned s_scan[1024];
    __shared__ unsigned s_prefix, s_need, s_cnt;
    __shared__ float s_red[32];
    pdl_wait();
    pdl_launch_dependents();
    const int tid = threadIdx.x;
    const float* d = logits + (size_t)blockIdx.x * cols;
    const int k = topK < cols ? topK : cols;
    auto ukey = [&](int c) { return (unsigned)order_key(d[c]) ^ 0x80000000u; };      // ascending unsigned = Float.compare order

    // ── the k-th largest key ──
    unsigned prefix = 0, mask = 0, need = (unsigned)k;
    for (int shift = 24; shift >= 0; shift -= 8) {
        if (tid < 256) s_hist[tid] = 0;
        __syncthreads();
        for (int c = tid; c < cols; c += blockDim.x) {
            const unsigned key = ukey(c);
            if ((key & mask) == prefix) atomicAdd(&s_hist[(key >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (tid == 0) {
            unsigned acc = 0; int chosen = 0;
            for (int b = 255; b >= 0; b--) {
                if (acc + s_hist[b] >= need) { chosen = b; break; }
                acc += s_hist[b];
            }
            s_prefix = prefix | ((unsigned)chosen << shift);
            s_need = need - acc;
        }
        __syncthreads();
        prefix = s_prefix; need = s_need; mask |= 255u << shift;
        __syncthreads();
    }
    const unsigned T = prefix;                       // need = how many of the keys equal to T belong to the top k
    const unsigned nGreater = (unsigned)k - need;

    // ── candidates: every key above T, and the `need` lowest indices among the keys equal to T ──
    if (tid == 0) s_cnt = 0;
    __syncthreads();
    for (int c = tid; c < cols; c += blockDim.x) {
        const unsigned key = ukey(c);
        if (key > T) {
            const unsigned pos = atomicAdd(&s_cnt, 1u);
            if (pos < (unsigned)kSampleMaxK) s_cand[pos] = ((unsigned long long)key << 32) | (0xFFFFFFFFu - (unsigned)c);
        }
    }
    const int chunk = (cols + (int)blockDim.x - 1) / (int)blockDim.x;
    const int lo = min(cols, tid * chunk), hi = min(cols, lo + chunk);
    unsigned mine = 0;
    for (int c = lo; c < hi; c++) mine += ukey(c) == T;
    s_scan[tid] = mine;
    __syncthreads();
    for (int o = 1; o < (int)blockDim.x; o <<= 1) {      // inclusive scan over the threads, in index order
        const unsigned v = tid >= o ? s_scan[tid - o] : 0u;
        __syncthreads();
        s_scan[tid] += v;
        __syncthreads();
    }
    unsigned rank = s_scan[tid] - mine;
    for (int c = lo; c < hi && rank < need; c++) {
        if (ukey(c) == T) {
            s_cand[nGreater + rank] = ((unsigned long long)T << 32) | (0xFFFFFFFFu - (unsigned)c);
            rank++;
        }
    }
    int P = 1;
    while (P < k) P <<= 1;
    for (int i = k + tid; i < P; i += blockDim.x) s_cand[i] = 0ull;
    // ── descending bitonic sort of (key, −index) ──
    for (int size = 2; size <= P; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            __syncthreads();
            const int i = tid, j = tid ^ stride;
            if (j > i && j < P) {
                const unsigned long long a = s_cand[i], b = s_cand[j];
                const bool desc = (i & size) == 0;
                if (desc ? a < b : a > b) { s_cand[i] = b; s_cand[j] = a; }
            }
        }
    }
    __syncthreads();
    // ── probabilities of the k candidates, then the sequential sums of the reference ──
    float v = -INFINITY;
    int idx = 0;
    if (tid < k) {
        idx = (int)(0xFFFFFFFFu - (unsigned)(s_cand[tid] & 0xFFFFFFFFull));
        v = d[idx] / temperature;
    }
    float mx = (tid < k && v == v) ? v : -INFINITY;      // `if (v > max) max = v` never takes a NaN
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if ((tid & 31) == 0) s_red[tid >> 5] = mx;
    __syncthreads();
    mx = s_red[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); w++) mx = fmaxf(mx, s_red[w]);
    if (tid < k) s_p[tid] = (float)exp((double)(v - mx));
    __syncthreads();
    if (tid == 0) {
        float sum = 0.0f;
        for (int i = 0; i < k; i++) sum += s_p[i];
        const float r = rbuf[blockIdx.x];
        float cum = 0.0f;
        int pick = k - 1;
        for (int i = 0; i < k; i++) {
            cum += s_p[i] / sum;
            if (r <= cum) { pick = i; break; }
        }
        out[blockIdx.x] = (float)(int)(0xFFFFFFFFu - (unsigned)(s_cand[pick] & 0xFFFFFFFFull));
    }
}

// The same draw when more than kSampleMaxK candidates take part — topK above 1024, or the reference's topK = 0,
// which means the whole vocabulary (models/TextGenerator.java:111-115).  One CTA per row sorts ALL (key, −index)
// pairs of the row, descending, with a bitonic network in global scratch (P = cols rounded up to a power of two,
// 8 bytes each), turns the first k into probabilities (4 bytes each, behind the pairs) and lets one thread run the
// reference's two sequential float loops.  Not a hot path: a 32000-entry row takes a fraction of a millisecond.
__global__ void __launch_bounds__(1024) k_sample_sorted(const float* __restrict__ logits, const float* __restrict__ rbuf,
                                                         float* __restrict__ out, int cols, int k, int P, float temperature,
                                                         unsigned long long* __restrict__ scratch) {
    __shared__ float s_red[32];
    pdl_wait();
    pdl_launch_dependents();
    const int tid = threadIdx.x;
    const float* d = logits + (size_t)blockIdx.x * cols;
    unsigned long long* cand = scratch + (size_t)blockIdx.x * ((size_t)P + (size_t)(P + 1) / 2);
    float* prob = reinterpret_cast<float*>(cand + P);
    for (int c = tid; c < P; c += blockDim.x)
        cand[c] = c < cols ? (((unsigned long long)((unsigned)order_key(d[c]) ^ 0x80000000u) << 32) | (0xFFFFFFFFu - (unsigned)c)) : 0ull;
    for (int size = 2; size <= P; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            __syncthreads();
            for (int t = tid; t < (P >> 1); t += blockDim.x) {
                const int i = 2 * t - (t & (stride - 1)), j = i + stride;
                const unsigned long long a = cand[i], b = cand[j];
                const bool desc = (i & size) == 0;
                if (desc ? a < b : a > b) { cand[i] = b; cand[j] = a; }
            }
        }
    }
    __syncthreads();
    float mx = -INFINITY;
    for (int i = tid; i < k; i += blockDim.x) {
        const float v = d[(int)(0xFFFFFFFFu - (unsigned)(cand[i] & 0xFFFFFFFFull))] / temperature;
        if (v == v) mx = fmaxf(mx, v);               // `if (v > max) max = v` never takes a NaN
    }
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if ((tid & 31) == 0) s_red[tid >> 5] = mx;
    __syncthreads();
    mx = s_red[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); w++) mx = fmaxf(mx, s_red[w]);
    for (int i = tid; i < k; i += blockDim.x) {
        const float v = d[(int)(0xFFFFFFFFu - (unsigned)(cand[i] & 0xFFFFFFFFull))] / temperature;
        prob[i] = (float)exp((double)(v - mx));
    }
    __syncthreads();
    if (tid == 0) {
        float sum = 0.0f;
        for (int i = 0; i < k; i++) sum += prob[i];
        const float r = rbuf[blockIdx.x];
        float cum = 0.0f;
        int pick = k - 1;
        for (int i = 0; i < k; i++) {
            cum += prob[i] / sum;
            if (r <= cum) { pick = i; break; }
        }
        out[blockIdx.x] = (float)(int)(0xFFFFFFFFu - (unsigned)(cand[pick] & 0xFFFFFFFFull));
    }
}

__global__ void k_add_scalar_inplace(float* __restrict__ buf, float v, int n) {
    pdl_wait();
    pdl_launch_dependents();
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) buf[i] = buf[i] + v;
}

__global__ void k_copy(const float* __restrict__ src, float* __restrict__ dst, long long n) {
    pdl_wait();
    pdl_launch_dependents();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) dst[i] = src[i];
}

// Integer-exact generator: two splitmix64 outputs give eight 16-bit uniform fields;
// their centred sum (Irwin–Hall) times one float constant.  Same bits on any device.
__device__ __forceinline__ unsigned long long splitmix64(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ULL;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}
__global__ void k_synth_fill(float* __restrict__ out, unsigned long long key, float scale, long long first, long long n) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        unsigned long long idx = (unsigned long long)(first + i);
        unsigned long long a = splitmix64(key + 2 * idx), b = splitmix64(key + 2 * idx + 1);
        int s = 0;
#pragma unroll
        for (int f = 0; f < 4; f++) { s += (int)((a >> (16 * f)) & 0xFFFF); s += (int)((b >> (16 * f)) & 0xFFFF); }
        int centred = 2 * s - 8 * 65535;
        out[i] = __fmul_rn((float)centred, scale);
    }
}

unsigned long long h_splitmix64(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ULL;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}

}  // namespace

void launch_embed_gather(const float* table, const float* ids, float* out, int rows, int d, int vocab, cudaStream_t s) {
    if (rows <= 0) return;
    launch_k(k_embed_gather, dim3(rows), dim3(256), 0, s, true, table, ids, out, rows, d, vocab);
}
void launch_argmax_rows(const float* in, float* out, int rows, int cols, int* scratch, int* tickets, cudaStream_t s) {
    if (rows <= 0) return;
    // short rows, or more rows than ticket counters: one CTA per row
    const int parts = (cols >= 4096 && rows <= kArgmaxRowsMax && scratch != nullptr) ? kArgmaxParts : 1;
    launch_k(k_argmax_rows, dim3(parts, rows), dim3(256), 0, s, true, in, out, rows, cols, scratch, tickets);
}
static int sample_pow2(int cols) { int P = 2; while (P < cols) P <<= 1; return P; }
size_t sample_topk_ws_floats(int rows, int cols, int topK) {
    const int k = (topK == 0 || topK > cols) ? cols : topK;
    if (k <= kSampleMaxK) return 0;
    const size_t P = (size_t)sample_pow2(cols);
    return (size_t)rows * (P + (P + 1) / 2) * 2;          // pairs of 8 bytes, then the probabilities
}
void launch_sample_topk(const float* logits, const float* r, float* out, int rows, int cols, int topK, float temperature, float* ws,
                        cudaStream_t s) {
    if (rows <= 0) return;
    if (topK < 0) throw std::runtime_error("sampleTopK: topK must be >= 0 (0 = the whole vocabulary)");
    if (!(temperature > 0.0f)) throw std::runtime_error("temperature must be > 0");
    const int k = (topK == 0 || topK > cols) ? cols : topK;      // models/TextGenerator.java:111-115
    if (k <= kSampleMaxK) {
        launch_k(k_sample_topk, dim3(rows), dim3(1024), 0, s, true, logits, r, out, rows, cols, k, temperature);
        return;
    }
    if (ws == nullptr) throw std::runtime_error("sampleTopK: more than 1024 candidates need the workspace");
    launch_k(k_sample_sorted, dim3(rows), dim3(1024), 0, s, true, logits, r, out, cols, k, sample_pow2(cols), temperature,
             reinterpret_cast<unsigned long long*>(ws));
}
void launch_add_scalar_inplace(float* buf, float v, int n, cudaStream_t s) {
    if (n <= 0) return;
    launch_k(k_add_scalar_inplace, dim3((n + 127) / 128), dim3(128), 0, s, true, buf, v, n);
}
void launch_copy(const float* src, float* dst, long long n, cudaStream_t s) {
    if (n <= 0) return;
    long long g = (n + 255) / 256;
    if (g > (long long)g_num_sms * 8) g = (long long)g_num_sms * 8;
    launch_k(k_copy, dim3((unsigned)g), dim3(256), 0, s, true, src, dst, n);
}
void launch_synth_fill(float* out, unsigned long long seed, unsigned long long ordinal, float std_dev,
                       long long first, long long n, cudaStream_t s) {
    if (n <= 0) return;
    unsigned long long key = h_splitmix64(seed ^ (ordinal * 0xD1342543DE82EF95ULL));
    double sd = 2.0 * sqrt(8.0 * (65536.0 * 65536.0 - 1.0) / 12.0);
    float scale = (float)((double)std_dev / sd);
    long long g = (n + 255) / 256;
    if (g > (long long)g_num_sms * 16) g = (long long)g_num_sms * 16;
    launch_k(k_synth_fill, dim3((unsigned)g), dim3(256), 0, s, false, out, key, scale, first, n);
}

}  // namespace dj
