// Q8 weights: quantizer and the decode-time dequant-GEMV.
//
// HBM layout of a Q8 weight for y = x·W, W[K×N]: codes[N][Kp] int8 (one output
// column's K-vector contiguous, Kp = K rounded up to 16 with zero padding) and
// scales[N][nb] fp32, nb = ceil(K/32).  1.125 bytes per weight.
//
// GEMV (M small): HBM-bound.  A CTA of BLOCK threads owns the whole K extent:
// thread t keeps the activations of its 16-wide K chunks (t, t+BLOCK, ...) in
// registers for the life of the CTA, so the inner loop is one 128-bit streaming
// load of codes + one scale per chunk, a byte-permute/subtract dequant and fp32
// FMAs.  CTAs are persistent and walk row tiles round-robin; a tile is 4 output
// rows (or 2 gate + 2 up rows for the fused SwiGLU form) reduced across the CTA
// through shuffles and a double-buffered shared-memory slot.  RMSNorm is fused
// into the activation load, bias / residual / SiLU-gate into the epilogue.
#include "kernels.h"
#include "q8_common.cuh"
#include <cuda_fp16.h>

namespace dj {

int g_gemv_mode = 2;   // 2: tensor-pipe kernels (TMA GEMV, cp.async GEMV, batched, tcgen05) with the FMA kernel as the fallback, 1: the same without the TMA GEMV, 0: FMA kernel only

namespace {

// ───────────── quantizer ─────────────
// One thread per (column, 32-block).  Follows the format definition literally:
// IEEE division for the scale and for w/scale, round-half-even, clamp to ±127.
__global__ void k_q8_quantize(const float* __restrict__ src, int src_ld, int K, int n_cols,
                              int8_t* __restrict__ codes, float* __restrict__ scales, int Kp, int nb) {
    long long id = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    long long total = (long long)n_cols * nb;
    if (id >= total) return;
    int n = (int)(id % n_cols), b = (int)(id / n_cols);
    int k0 = b * 32, k1 = min(K, k0 + 32);
    float amax = 0.0f;
    for (int k = k0; k < k1; k++) amax = fmaxf(amax, fabsf(src[(size_t)k * src_ld + n]));
    float scale = __fdiv_rn(amax, 127.0f);
    scales[(size_t)n * nb + b] = scale;
    for (int k = k0; k < k1; k++) {
        int q = 0;
        if (scale != 0.0f) {
            q = __float2int_rn(__fdiv_rn(src[(size_t)k * src_ld + n], scale));
            q = max(-127, min(127, q));
        }
        codes[(size_t)n * Kp + k] = (int8_t)q;
    }
}

// ───────────── GEMV ─────────────
struct GemvParams {
    const float* x; int ldx;
    const float* gamma; float eps;
    const int8_t* codes; const float* scales; const float* bias;
    const int8_t* codes2; const float* scales2; const float* bias2;
    const float* residual; int ldr;
    float* out; int ldo;
    int K, N, Kp, nb;
};

__device__ __forceinline__ uint4 ld_stream_u4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// Σ_j float(code_j)·x_j for the 16 int8 codes of one 128-bit word group.
// int8 → fp32 without a convert instruction: flip the sign bit (code+128 as an
// unsigned byte), drop the byte into the mantissa of 2^23 and subtract 2^23+128.
__device__ __forceinline__ float dot16(const uint4& w, const float* x) {
    float acc = 0.0f;
    const uint32_t words[4] = {w.x ^ 0x80808080u, w.y ^ 0x80808080u, w.z ^ 0x80808080u, w.w ^ 0x80808080u};
#pragma unroll
    for (int q = 0; q < 4; q++) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            float f = __int_as_float(__byte_perm(words[q], 0x4B000000u, 0x7650 + j)) - 8388736.0f;
            acc = fmaf(f, x[q * 4 + j], acc);
        }
    }
    return acc;
}

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <int BLOCK, int NI, bool SWIGLU>
__global__ void __launch_bounds__(BLOCK) k_q8_gemv(const GemvParams p) {
    constexpr int R = (NI <= 2) ? 4 : 2;   // row slots per tile (fewer when a thread holds many K chunks)
    constexpr int RH = R / 2;
    constexpr int NW = BLOCK / 32;
    __shared__ float s_part[2][NW][R];
    __shared__ float s_red[NW];

    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int m = blockIdx.y;
    const int nChunks = p.Kp >> 4;
    const int rowsPerTile = SWIGLU ? RH : R;
    const int nTiles = (p.N + rowsPerTile - 1) / rowsPerTile;

    auto load_tile = [&](int tile, uint4 (&w)[R][NI], float (&sc)[R][NI]) {
#pragma unroll
        for (int r = 0; r < R; r++) {
            int n = SWIGLU ? tile * RH + (r % RH) : tile * R + r;
            const int8_t* cbase = (SWIGLU && r >= RH) ? p.codes2 : p.codes;
            const float* sbase = (SWIGLU && r >= RH) ? p.scales2 : p.scales;
#pragma unroll
            for (int i = 0; i < NI; i++) {
                int chunk = t + BLOCK * i;
                if (n < p.N && chunk < nChunks) {
                    w[r][i] = ld_stream_u4(cbase + (size_t)n * p.Kp + (size_t)chunk * 16);
                    sc[r][i] = __ldg(sbase + (size_t)n * p.nb + (chunk >> 1));
                } else {
                    w[r][i] = make_uint4(0x0u, 0x0u, 0x0u, 0x0u);
                    sc[r][i] = 0.0f;
                }
            }
        }
    };

    auto finish_tile = [&](int tile, const uint4 (&w)[R][NI], const float (&sc)[R][NI], const float (&xr)[NI][16], int buf) {
        float acc[R];
#pragma unroll
        for (int r = 0; r < R; r++) {
            acc[r] = 0.0f;
#pragma unroll
            for (int i = 0; i < NI; i++) acc[r] = fmaf(sc[r][i], dot16(w[r][i], xr[i]), acc[r]);
        }
#pragma unroll
        for (int r = 0; r < R; r++)
            for (int o = 16; o > 0; o >>= 1) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], o);
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < R; r++) s_part[buf][warp][r] = acc[r];
        }
        __syncthreads();
        if (SWIGLU) {
            if (t < RH) {
                int n = tile * RH + t;
                if (n < p.N) {
                    float g = 0.0f, u = 0.0f;
#pragma unroll
                    for (int q = 0; q < NW; q++) { g += s_part[buf][q][t]; u += s_part[buf][q][RH + t]; }
                    if (p.bias) g += p.bias[n];
                    if (p.bias2) u += p.bias2[n];
                    float sig = 1.0f / (1.0f + expf(-g));
                    p.out[(size_t)m * p.ldo + n] = (g * sig) * u;      // SiLU(gate) ⊙ up
                }
            }
        } else {
            if (t < R) {
                int n = tile * R + t;
                if (n < p.N) {
                    float v = 0.0f;
#pragma unroll
                    for (int q = 0; q < NW; q++) v += s_part[buf][q][t];
                    if (p.bias) v += p.bias[n];
                    if (p.residual) v += p.residual[(size_t)m * p.ldr + n];
                    p.out[(size_t)m * p.ldo + n] = v;
                }
            }
        }
    };

    // Weights do not depend on the previous kernel: issue the first tile's loads
    // before waiting for it.
    uint4 wa[R][NI], wb[R][NI];
    float sa[R][NI], sb[R][NI];
    int tile = blockIdx.x;
    const int stride = gridDim.x;
    if (tile < nTiles) load_tile(tile, wa, sa);
    pdl_wait();
    pdl_launch_dependents();

    // Activations of this thread's chunks, kept in registers.
    float xr[NI][16];
    const float* xrow = p.x + (size_t)m * p.ldx;
#pragma unroll
    for (int i = 0; i < NI; i++) {
        int k0 = (t + BLOCK * i) * 16;
#pragma unroll
        for (int j = 0; j < 16; j++) xr[i][j] = (k0 + j < p.K) ? xrow[k0 + j] : 0.0f;
    }
    if (p.gamma != nullptr) {
        // RMSNorm: x / sqrt(mean(x²) + eps) · gamma  (RMSNorm1D.forward)
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < NI; i++)
#pragma unroll
            for (int j = 0; j < 16; j++) ss = fmaf(xr[i][j], xr[i][j], ss);
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) s_red[warp] = ss;
        __syncthreads();
        float tot = 0.0f;
#pragma unroll
        for (int q = 0; q < NW; q++) tot += s_red[q];
        float rms = sqrtf(tot * (1.0f / (float)p.K) + p.eps);
#pragma unroll
        for (int i = 0; i < NI; i++) {
            int k0 = (t + BLOCK * i) * 16;
#pragma unroll
            for (int j = 0; j < 16; j++)
                xr[i][j] = (k0 + j < p.K) ? __fdiv_rn(xr[i][j], rms) * p.gamma[k0 + j] : 0.0f;
        }
    }

    // Two register sets: the loads of tile t+1 are in flight while tile t is reduced.
    while (tile < nTiles) {
        int next = tile + stride;
        if (next < nTiles) load_tile(next, wb, sb);
        finish_tile(tile, wa, sa, xr, 0);
        tile = next;
        if (tile >= nTiles) break;
        next = tile + stride;
        if (next < nTiles) load_tile(next, wa, sa);
        finish_tile(tile, wb, sb, xr, 1);
        tile = next;
    }
}

template <int BLOCK, int NI, bool SWIGLU>
void launch_gemv_inst(const GemvParams& p, int M, cudaStream_t s) {
    static int ctasPerSM = 0;
    if (ctasPerSM == 0) {
        DJ_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&ctasPerSM, k_q8_gemv<BLOCK, NI, SWIGLU>, BLOCK, 0));
        if (ctasPerSM < 1) ctasPerSM = 1;
    }
    int R = (NI <= 2) ? 4 : 2;
    int rowsPerTile = SWIGLU ? R / 2 : R;
    int nTiles = (p.N + rowsPerTile - 1) / rowsPerTile;
    int cap = g_num_sms * ctasPerSM;
    if (M > 1) cap = (cap + M - 1) / M;
    int gx = nTiles < cap ? nTiles : cap;
    if (gx < 1) gx = 1;
    launch_k(k_q8_gemv<BLOCK, NI, SWIGLU>, dim3(gx, M), dim3(BLOCK), 0, s, true, p);
}


template <bool SWIGLU>
void launch_gemv_dispatch(const GemvParams& p, int M, cudaStream_t s) {
    int chunks = p.Kp / 16;
    // smallest BLOCK·NI ≥ chunks with NI ≤ 4, preferring the widest block on ties
    int bestB = 0, bestNI = 0, bestWaste = 1 << 30;
    const int blocks[4] = {256, 128, 64, 32};
    for (int b : blocks) {
        int ni = (chunks + b - 1) / b;
        if (ni > 4) continue;
        int waste = b * ni - chunks;
        if (waste < bestWaste) { bestWaste = waste; bestB = b; bestNI = ni; }
    }
    if (bestB == 0) throw std::runtime_error("Q8 linear: K=" + std::to_string(p.K) + " exceeds the supported maximum of 16384");
#define DJ_GEMV_CASE(B, NI_) if (bestB == B && bestNI == NI_) { launch_gemv_inst<B, NI_, SWIGLU>(p, M, s); return; }
    DJ_GEMV_CASE(256, 1) DJ_GEMV_CASE(256, 2) DJ_GEMV_CASE(256, 3) DJ_GEMV_CASE(256, 4)
    DJ_GEMV_CASE(128, 1) DJ_GEMV_CASE(128, 2) DJ_GEMV_CASE(128, 3) DJ_GEMV_CASE(128, 4)
    DJ_GEMV_CASE(64, 1) DJ_GEMV_CASE(64, 2) DJ_GEMV_CASE(64, 3) DJ_GEMV_CASE(64, 4)
    DJ_GEMV_CASE(32, 1) DJ_GEMV_CASE(32, 2) DJ_GEMV_CASE(32, 3) DJ_GEMV_CASE(32, 4)
#undef DJ_GEMV_CASE
    throw std::runtime_error("Q8 linear: no kernel instance for this K");
}

}  // namespace

void launch_q8_quantize(const float* src, int src_ld, int K, int n_cols, int8_t* codes, float* scales,
                        int Kp, int nb, cudaStream_t s) {
    long long total = (long long)n_cols * nb;
    if (total <= 0) return;
    launch_k(k_q8_quantize, dim3((unsigned)((total + 127) / 128)), dim3(128), 0, s, false, src, src_ld, K, n_cols, codes, scales, Kp, nb);
}

namespace {

// LayerNorm1D.forward row by row (norm/LayerNorm1D.java:34-71 over CpuBackend.meanAlongRows /
// varianceAlongRows, tensor/cpu/CpuBackend.java:242-268): one CTA per row, two block reductions.
__global__ void __launch_bounds__(256) k_layernorm_rows(const float* __restrict__ x, int ldx, const float* __restrict__ gamma,
                                                        const float* __restrict__ beta, float eps, float* __restrict__ out, int K) {
    __shared__ float red[8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* row = x + (size_t)blockIdx.x * ldx;
    float* o = out + (size_t)blockIdx.x * K;
    auto block_sum = [&](float v) {
        for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
        __syncthreads();
        if (lane == 0) red[warp] = v;
        __syncthreads();
        float t = 0.0f;
#pragma unroll
        for (int q = 0; q < 8; q++) t += red[q];
        return t;
    };
    float sm = 0.0f;
    for (int k = tid; k < K; k += 256) sm += row[k];
    const float mean = block_sum(sm) * (1.0f / (float)K);
    float ss = 0.0f;
    for (int k = tid; k < K; k += 256) { const float d = row[k] - mean; ss = fmaf(d, d, ss); }
    const float stdv = sqrtf(block_sum(ss) * (1.0f / (float)K) + eps);
    for (int k = tid; k < K; k += 256) o[k] = __fdiv_rn(row[k] - mean, stdv) * gamma[k] + beta[k];
}

__global__ void k_gelu_rows(float* __restrict__ buf, int ld, int N, long long total) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    float* p = buf + (size_t)(i / N) * ld + (i % N);
    *p = gelu_ref(*p);
}

}  // namespace

void launch_layernorm_rows(const float* x, int ldx, const float* gamma, const float* beta, float eps, float* out, int K, int M, cudaStream_t s) {
    if (M <= 0 || K <= 0) return;
    launch_k(k_layernorm_rows, dim3(M), dim3(256), 0, s, false, x, ldx, gamma, beta, eps, out, K);
}

void launch_gelu_rows(float* buf, int ld, int N, int M, cudaStream_t s) {
    const long long total = (long long)M * N;
    if (total <= 0) return;
    launch_k(k_gelu_rows, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, s, false, buf, ld, N, total);
}

namespace {
void dispatch_q8_linear(const Q8LinearArgs& a, cudaStream_t s);
}

void launch_q8_linear(const Q8LinearArgs& a0, cudaStream_t s) {
    if (a0.M <= 0 || a0.w.N <= 0) return;
    if (a0.beta == nullptr && a0.act == 0) { dispatch_q8_linear(a0, s); return; }
    // GPT blocks: up to four rows go through the GEMV, which takes LayerNorm and GELU itself; the many-row
    // kernels see already normalised rows and get the activation applied to their output afterwards
    if (g_gemv_mode >= 1 && a0.M < 5 && q8_gemv_i8_fuses_gpt(a0)) { dispatch_q8_linear(a0, s); return; }
    Q8LinearArgs a = a0;
    if (a.beta != nullptr) {
        if (a.ln_ws == nullptr) throw std::runtime_error("Q8 linear: LayerNorm needs its workspace");
        launch_layernorm_rows(a.x, a.ldx, a.gamma, a.beta, a.eps, a.ln_ws, a.w.K, a.M, s);
        a.x = a.ln_ws; a.ldx = a.w.K; a.gamma = nullptr; a.beta = nullptr;
    }
    a.act = 0;
    dispatch_q8_linear(a, s);
    if (a0.act == 1) launch_gelu_rows(a.out, a.ldo, a.w.N, a.M, s);
}

namespace {

void dispatch_q8_linear(const Q8LinearArgs& a, cudaStream_t s) {

    if (a.M <= 0 || a.w.N <= 0) return;
    GemvParams p;
    p.x = a.x; p.ldx = a.ldx; p.gamma = a.gamma; p.eps = a.eps;
    p.codes = a.w.codes; p.scales = a.w.scales; p.bias = a.bias;
    p.codes2 = a.w2.codes; p.scales2 = a.w2.scales; p.bias2 = a.bias2;
    p.residual = a.residual; p.ldr = a.ldr;
    p.out = a.out; p.ldo = a.ldo;
    p.K = a.w.K; p.N = a.w.N; p.Kp = a.w.Kp; p.nb = a.w.nb;
    const bool swiglu = a.w2.codes != nullptr;
    static const bool noTc = getenv("DEEPJ_CUDA_NO_TC") != nullptr;
    const bool batchOk = g_gemv_mode >= 1 && a.M >= 5 && a.ws != nullptr && a.w.K % 32 == 0 && a.w.Kp == a.w.K;
    // A few dozen rows leave most SMs without a 128 × 256 tile: passes of the 16-row kernel (≈ 3 µs + 0.5 ps per weight
    // and pass with the TMA kernel, 0.9 ps with the cp.async one; measured on 4096 × 12288, 11008 × 4096 and 4096 × 4096)
    // win until the tensor-core grid fills up.
    bool preferBatch = false;
    if (batchOk && a.M >= kTcMinRows && a.M <= 256) {
        const bool tmaKernel = g_gemv_mode == 2 && a.w.K % 128 == 0;
        const double perPassUs = tmaKernel ? 3.0 + 0.5e-6 * (double)a.w.K * (double)a.w.N : 0.9e-6 * (double)a.w.K * (double)a.w.N;
        const int rem = a.M % 16;
        const double passes = (double)(a.M / 16) + (rem == 0 ? 0.0 : rem <= 8 ? 0.75 : 1.0);      // a last pass of up to eight rows issues half the MMAs
        preferBatch = passes * perPassUs < q8_tc_estimate_us(a.M, a.w.K, a.w.N);
    }
    if (g_gemv_mode >= 1 && !noTc && !preferBatch && a.M >= kTcMinRows && a.ws != nullptr && launch_q8_linear_tc(a, a.ws, s)) return;
    if (batchOk) {
        // five or more rows share one pass over the weights, 16 at a time (up to four are two GEMV passes, which is as fast)
        bool ok = true;
        for (int m0 = 0; m0 < a.M && ok; m0 += 16) {
            const int rows = a.M - m0 < 16 ? a.M - m0 : 16;
            ok = (g_gemv_mode == 2 && launch_q8_linear_batch_tma(a, m0, rows, a.ws, a.tickets, s)) || launch_q8_linear_batch(a, m0, rows, a.ws, a.tickets, s);
        }
        if (ok) return;
    }
    if (g_gemv_mode == 2 && launch_q8_gemv_tma(a, s)) return;
    if (g_gemv_mode >= 1 && launch_q8_gemv_i8(a, s)) return;
    if (swiglu) launch_gemv_dispatch<true>(p, a.M, s);
    else launch_gemv_dispatch<false>(p, a.M, s);
}

}  // namespace

}  // namespace dj
