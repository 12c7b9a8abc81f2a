// fp32 kernels for ComputeGraph op codes 1-42 (tensor/ComputeGraph.java:19-60).
// These keep the whole 42-op stream executable under the unmodified reference
// layer classes; they are not the decode hot path.  Arithmetic follows
// tensor/cpu/CpuBackend.java: transcendental functions are evaluated in double and
// rounded to float (:24-28), multiply and add are never fused (this file is built
// with -fmad=false), matmul accumulates in ascending k (:168-188).
#include "kernels.h"
#include <cmath>

namespace dj {

namespace {

constexpr int kEwBlock = 256;
inline int ew_grid(long long n) {
    long long g = (n + kEwBlock - 1) / kEwBlock;
    long long cap = (long long)g_num_sms * 16;
    return (int)(g < cap ? (g > 0 ? g : 1) : cap);
}

__device__ __forceinline__ float d_sqrt(float x) { return (float)sqrt((double)x); }
__device__ __forceinline__ float d_exp(float x) { return (float)exp((double)x); }
__device__ __forceinline__ float d_log(float x) { return (float)log((double)x); }
__device__ __forceinline__ float d_tanh(float x) { return (float)tanh((double)x); }
__device__ __forceinline__ float d_pow(float x, float e) { return (float)pow((double)x, (double)e); }
__device__ __forceinline__ float d_sigmoid(float x) { return 1.0f / (1.0f + d_exp(-x)); }
// Math.max / Math.min semantics: NaN propagates, -0.0 < +0.0
__device__ __forceinline__ float j_max(float a, float b) {
    if (a != a) return a;
    if (b != b) return b;
    if (a == 0.0f && b == 0.0f) return signbit(a) ? b : a;
    return a > b ? a : b;
}
__device__ __forceinline__ float j_min(float a, float b) {
    if (a != a) return a;
    if (b != b) return b;
    if (a == 0.0f && b == 0.0f) return signbit(a) ? a : b;
    return a < b ? a : b;
}
__device__ __forceinline__ float d_gelu(float x) {
    float c = d_sqrt(2.0f / 3.14159274101257324f);
    float x3 = x * x * x;
    float t = c * (x + 0.044715f * x3);
    return 0.5f * x * (1.0f + d_tanh(t));
}
__device__ __forceinline__ float d_gelu_deriv(float x) {
    float c = d_sqrt(2.0f / 3.14159274101257324f);
    float x2 = x * x;
    float x3 = x2 * x;
    float t = c * (x + 0.044715f * x3);
    float th = d_tanh(t);
    float sech2 = 1.0f - th * th;
    float dtDx = c * (1.0f + 3.0f * 0.044715f * x2);
    return 0.5f * (1.0f + th) + 0.5f * x * sech2 * dtDx;
}

__global__ void k_binary(int op, const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out, int n) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        float x = a[i], y = b[i], r;
        switch (op) {
            case 1: r = x + y; break;
            case 2: r = x - y; break;
            case 3: r = x * y; break;
            case 4: r = x / y; break;
            case 14: r = x > 0.0f ? y : 0.0f; break;          // relu backward (input, grad)
            default: r = y * d_gelu_deriv(x); break;          // 16: gelu backward
        }
        out[i] = r;
    }
}

__global__ void k_unary(int op, const float* __restrict__ in, float* __restrict__ out, int n) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        float x = in[i], r;
        switch (op) {
            case 7: r = d_sqrt(x); break;
            case 8: r = -x; break;
            case 9: r = d_exp(x); break;
            case 10: r = d_log(x); break;
            case 11: r = d_tanh(x); break;
            case 12: r = d_sigmoid(x); break;
            case 13: r = j_max(0.0f, x); break;
            default: r = d_gelu(x); break;                    // 15
        }
        out[i] = r;
    }
}

__global__ void k_scalar(int op, const float* __restrict__ in, float* __restrict__ out, float v, int n) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        float x = in[i], r;
        switch (op) {
            case 6: r = x * v; break;
            case 21: r = x + v; break;
            case 22: r = x / v; break;
            default: r = d_pow(x, v); break;                  // 36
        }
        out[i] = r;
    }
}

__global__ void k_clamp(const float* __restrict__ in, float* __restrict__ out, float lo, float hi, int n) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        out[i] = j_min(hi, j_max(lo, in[i]));
}

// C[m×n] = A[m×k]·B[k×n]; 32×32 output tile, ascending-k accumulation with separate
// multiply and add so the result equals the reference's ikj loop bit for bit.
__global__ void k_matmul_f32(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C, int m, int n, int k) {
    __shared__ float sa[32][33];
    __shared__ float sb[32][33];
    int tx = threadIdx.x, ty = threadIdx.y;
    int row = blockIdx.y * 32 + ty, col = blockIdx.x * 32 + tx;
    float acc = 0.0f;
    for (int k0 = 0; k0 < k; k0 += 32) {
        sa[ty][tx] = (row < m && k0 + tx < k) ? A[(size_t)row * k + k0 + tx] : 0.0f;
        sb[ty][tx] = (k0 + ty < k && col < n) ? B[(size_t)(k0 + ty) * n + col] : 0.0f;
        __syncthreads();
        int kmax = min(32, k - k0);
        for (int kk = 0; kk < kmax; kk++) acc = acc + sa[ty][kk] * sb[kk][tx];
        __syncthreads();
    }
    if (row < m && col < n) C[(size_t)row * n + col] = acc;
}

__global__ void k_transpose(const float* __restrict__ in, float* __restrict__ out, int rows, int cols) {
    __shared__ float t[32][33];
    int c = blockIdx.x * 32 + threadIdx.x, r = blockIdx.y * 32 + threadIdx.y;
    if (r < rows && c < cols) t[threadIdx.y][threadIdx.x] = in[(size_t)r * cols + c];
    __syncthreads();
    int oc = blockIdx.y * 32 + threadIdx.x, orow = blockIdx.x * 32 + threadIdx.y;   // out is [cols × rows]
    if (orow < cols && oc < rows) out[(size_t)orow * rows + oc] = t[threadIdx.x][threadIdx.y];
}

__global__ void k_row_broadcast(int op, const float* __restrict__ a, const float* __restrict__ v, float* __restrict__ out, int rows, int cols) {
    long long n = (long long)rows * cols;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        float y = v[i % cols];
        out[i] = op == 24 ? a[i] + y : a[i] * y;              // 24 add row vector, 28 multiply
    }
}
__global__ void k_col_broadcast(int op, const float* __restrict__ a, const float* __restrict__ v, float* __restrict__ out, int rows, int cols) {
    long long n = (long long)rows * cols;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        float x = a[i], y = v[i / cols], r;
        switch (op) {
            case 25: r = x + y; break;
            case 26: r = x - y; break;
            case 27: r = x / y; break;
            default: r = x * y; break;                        // 32
        }
        out[i] = r;
    }
}

template <int OP>   // 0 sum, 1 max
__device__ __forceinline__ float block_reduce(float v, float* sh) {
    for (int o = 16; o > 0; o >>= 1) {
        float u = __shfl_xor_sync(0xffffffffu, v, o);
        v = OP == 0 ? v + u : fmaxf(v, u);
    }
    int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();
    if (l == 0) sh[w] = v;
    __syncthreads();
    v = l < nw ? sh[l] : (OP == 0 ? 0.0f : -INFINITY);
    for (int o = 16; o > 0; o >>= 1) {
        float u = __shfl_xor_sync(0xffffffffu, v, o);
        v = OP == 0 ? v + u : fmaxf(v, u);
    }
    return v;
}

// One block per row.  op: 30 mean, 31 variance, 33 sum, 34 max, 38 sum of |x|.
__global__ void k_row_reduce(int op, const float* __restrict__ in, float* __restrict__ out, int rows, int cols) {
    __shared__ float sh[32];
    int r = blockIdx.x;
    const float* d = in + (size_t)r * cols;
    float invCols = 1.0f / cols;
    if (op == 34) {
        float m = -INFINITY;
        for (int c = threadIdx.x; c < cols; c += blockDim.x) m = fmaxf(m, d[c]);
        m = block_reduce<1>(m, sh);
        if (threadIdx.x == 0) out[r] = m;
        return;
    }
    float s = 0.0f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) s += (op == 38 ? fabsf(d[c]) : d[c]);
    s = block_reduce<0>(s, sh);
    if (op == 33 || op == 38) { if (threadIdx.x == 0) out[r] = s; return; }
    float mean = s * invCols;
    if (op == 30) { if (threadIdx.x == 0) out[r] = mean; return; }
    float acc = 0.0f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) { float diff = d[c] - mean; acc += diff * diff; }
    acc = block_reduce<0>(acc, sh);
    if (threadIdx.x == 0) out[r] = acc * invCols;
}

// [rows×cols] → [1×cols], ascending-row accumulation per column like the reference.
__global__ void k_sum_rows(const float* __restrict__ in, float* __restrict__ out, int rows, int cols) {
    int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    float s = 0.0f;
    for (int r = 0; r < rows; r++) s += in[(size_t)r * cols + c];
    out[c] = s;
}

__global__ void k_sum_scalar(const float* __restrict__ in, float* __restrict__ out, long long n) {
    __shared__ float sh[32];
    float s = 0.0f;
    for (long long i = threadIdx.x; i < n; i += blockDim.x) s += in[i];
    s = block_reduce<0>(s, sh);
    if (threadIdx.x == 0) out[0] = s;
}

__global__ void k_softmax_rows(const float* __restrict__ in, float* __restrict__ out, int rows, int cols) {
    __shared__ float sh[32];
    int r = blockIdx.x;
    const float* d = in + (size_t)r * cols;
    float* o = out + (size_t)r * cols;
    float m = -INFINITY;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) m = fmaxf(m, d[c]);
    m = block_reduce<1>(m, sh);
    float s = 0.0f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) { float e = d_exp(d[c] - m); o[c] = e; s += e; }
    s = block_reduce<0>(s, sh);
    for (int c = threadIdx.x; c < cols; c += blockDim.x) o[c] = o[c] / s;
}

__global__ void k_softmax_backward(const float* __restrict__ g, const float* __restrict__ sm, float* __restrict__ out, int rows, int cols) {
    __shared__ float sh[32];
    size_t base = (size_t)blockIdx.x * cols;
    float dot = 0.0f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) dot += g[base + c] * sm[base + c];
    dot = block_reduce<0>(dot, sh);
    for (int c = threadIdx.x; c < cols; c += blockDim.x) out[base + c] = sm[base + c] * (g[base + c] - dot);
}

__global__ void k_layernorm_backward(const float* __restrict__ dxh, const float* __restrict__ xh, const float* __restrict__ sd,
                                     float* __restrict__ out, int rows, int cols) {
    __shared__ float sh[32];
    size_t base = (size_t)blockIdx.x * cols;
    float invStd = 1.0f / sd[blockIdx.x];
    float a = 0.0f, b = 0.0f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) { float d = dxh[base + c]; a += d; b += d * xh[base + c]; }
    a = block_reduce<0>(a, sh);
    b = block_reduce<0>(b, sh);
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        float d = dxh[base + c], x = xh[base + c];
        out[base + c] = invStd * (d - a / cols - x * (b / cols));
    }
}

__global__ void k_adamw(float* __restrict__ w, const float* __restrict__ g, float* __restrict__ mt, float* __restrict__ vt,
                        float lr, float b1, float b2, float eps, float wd, float bc1, float bc2, int n) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        float grad = g[i];
        float mNew = b1 * mt[i] + (1.0f - b1) * grad;
        float vNew = b2 * vt[i] + (1.0f - b2) * (grad * grad);
        mt[i] = mNew; vt[i] = vNew;
        float mHat = mNew / bc1, vHat = vNew / bc2;
        float update = (lr * mHat) / (d_sqrt(vHat) + eps);
        if (wd != 0.0f) update += lr * wd * w[i];
        w[i] -= update;
    }
}

__global__ void k_scatter_add_rows(float* __restrict__ target, const float* __restrict__ idx, const float* __restrict__ grad,
                                   int tRows, int tCols, int nIdx) {
    long long total = (long long)nIdx * tCols;
    for (long long id = blockIdx.x * (long long)blockDim.x + threadIdx.x; id < total; id += (long long)gridDim.x * blockDim.x) {
        int i = (int)(id / tCols), c = (int)(id % tCols);
        int row = (int)idx[i];
        if (row < 0 || row >= tRows) continue;
        atomicAdd(&target[(size_t)row * tCols + c], grad[(size_t)i * tCols + c]);
    }
}

template <bool GRAD>
__global__ void k_cross_entropy(const float* __restrict__ logits, const float* __restrict__ targets, float* __restrict__ out, int rows, int cols) {
    __shared__ float sh[32];
    int r = blockIdx.x;
    const float* d = logits + (size_t)r * cols;
    int t = (int)targets[r];
    bool bad = t < 0 || t >= cols;
    if (bad) {
        if (GRAD) { for (int c = threadIdx.x; c < cols; c += blockDim.x) out[(size_t)r * cols + c] = NAN; }
        else if (threadIdx.x == 0) out[r] = NAN;
        return;
    }
    float m = -INFINITY;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) m = fmaxf(m, d[c]);
    m = block_reduce<1>(m, sh);
    float s = 0.0f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) s += d_exp(d[c] - m);
    s = block_reduce<0>(s, sh);
    if (GRAD) {
        for (int c = threadIdx.x; c < cols; c += blockDim.x) {
            float p = d_exp(d[c] - m) / s;
            if (c == t) p -= 1.0f;
            out[(size_t)r * cols + c] = p / (float)rows;
        }
    } else if (threadIdx.x == 0) {
        out[r] = d_log(s) + m - d[t];
    }
}

}  // namespace

void launch_binary(int op, const float* a, const float* b, float* out, int n, cudaStream_t s) {
    if (n <= 0) return;
    launch_k(k_binary, dim3(ew_grid(n)), dim3(kEwBlock), 0, s, false, op, a, b, out, n);
}
void launch_unary(int op, const float* in, float* out, int n, cudaStream_t s) {
    if (n <= 0) return;
    launch_k(k_unary, dim3(ew_grid(n)), dim3(kEwBlock), 0, s, false, op, in, out, n);
}
void launch_scalar(int op, const float* in, float* out, float v, int n, cudaStream_t s) {
    if (n <= 0) return;
    launch_k(k_scalar, dim3(ew_grid(n)), dim3(kEwBlock), 0, s, false, op, in, out, v, n);
}
void launch_clamp(const float* in, float* out, float lo, float hi, int n, cudaStream_t s) {
    if (n <= 0) return;
    launch_k(k_clamp, dim3(ew_grid(n)), dim3(kEwBlock), 0, s, false, in, out, lo, hi, n);
}
void launch_matmul_f32(const float* a, const float* b, float* out, int m, int n, int k, cudaStream_t s) {
    if (m <= 0 || n <= 0) return;
    launch_k(k_matmul_f32, dim3((n + 31) / 32, (m + 31) / 32), dim3(32, 32), 0, s, false, a, b, out, m, n, k);
}
void launch_transpose(const float* in, float* out, int rows, int cols, cudaStream_t s) {
    if (rows <= 0 || cols <= 0) return;
    launch_k(k_transpose, dim3((cols + 31) / 32, (rows + 31) / 32), dim3(32, 32), 0, s, false, in, out, rows, cols);
}
void launch_row_broadcast(int op, const float* a, const float* v, float* out, int rows, int cols, cudaStream_t s) {
    if ((long long)rows * cols <= 0) return;
    launch_k(k_row_broadcast, dim3(ew_grid((long long)rows * cols)), dim3(kEwBlock), 0, s, false, op, a, v, out, rows, cols);
}
void launch_col_broadcast(int op, const float* a, const float* v, float* out, int rows, int cols, cudaStream_t s) {
    if ((long long)rows * cols <= 0) return;
    launch_k(k_col_broadcast, dim3(ew_grid((long long)rows * cols)), dim3(kEwBlock), 0, s, false, op, a, v, out, rows, cols);
}
void launch_row_reduce(int op, const float* in, float* out, int rows, int cols, cudaStream_t s) {
    if (rows <= 0) return;
    launch_k(k_row_reduce, dim3(rows), dim3(256), 0, s, false, op, in, out, rows, cols);
}
void launch_sum_rows(const float* in, float* out, int rows, int cols, cudaStream_t s) {
    if (cols <= 0) return;
    launch_k(k_sum_rows, dim3((cols + 127) / 128), dim3(128), 0, s, false, in, out, rows, cols);
}
void launch_sum_scalar(const float* in, float* out, long long n, cudaStream_t s) {
    launch_k(k_sum_scalar, dim3(1), dim3(1024), 0, s, false, in, out, n);
}
void launch_softmax_rows(const float* in, float* out, int rows, int cols, cudaStream_t s) {
    if (rows <= 0) return;
    launch_k(k_softmax_rows, dim3(rows), dim3(256), 0, s, false, in, out, rows, cols);
}
void launch_softmax_backward(const float* g, const float* sm, float* out, int rows, int cols, cudaStream_t s) {
    if (rows <= 0) return;
    launch_k(k_softmax_backward, dim3(rows), dim3(256), 0, s, false, g, sm, out, rows, cols);
}
void launch_layernorm_backward(const float* dxh, const float* xh, const float* sd, float* out, int rows, int cols, cudaStream_t s) {
    if (rows <= 0) return;
    launch_k(k_layernorm_backward, dim3(rows), dim3(256), 0, s, false, dxh, xh, sd, out, rows, cols);
}
void launch_adamw(float* w, const float* g, float* mt, float* vt, float lr, float b1, float b2, float eps,
                  float wd, float bc1, float bc2, int n, cudaStream_t s) {
    if (n <= 0) return;
    launch_k(k_adamw, dim3(ew_grid(n)), dim3(kEwBlock), 0, s, false, w, g, mt, vt, lr, b1, b2, eps, wd, bc1, bc2, n);
}
void launch_scatter_add_rows(float* target, const float* idx, const float* grad, int tRows, int tCols, int nIdx, cudaStream_t s) {
    if ((long long)nIdx * tCols <= 0) return;
    launch_k(k_scatter_add_rows, dim3(ew_grid((long long)nIdx * tCols)), dim3(kEwBlock), 0, s, false, target, idx, grad, tRows, tCols, nIdx);
}
void launch_ce_loss(const float* logits, const float* targets, float* out, int rows, int cols, cudaStream_t s) {
    if (rows <= 0) return;
    launch_k(k_cross_entropy<false>, dim3(rows), dim3(256), 0, s, false, logits, targets, out, rows, cols);
}
void launch_ce_grad(const float* logits, const float* targets, float* out, int rows, int cols, cudaStream_t s) {
    if (rows <= 0) return;
    launch_k(k_cross_entropy<true>, dim3(rows), dim3(256), 0, s, false, logits, targets, out, rows, cols);
}

}  // namespace dj
