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
#include <cuda_fp16.h>

namespace dj {

int g_gemv_mode = 2;   // 2: bulk-copy pipelined mma kernel, 1: register-pipelined mma kernel, 0: FMA kernel

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


// ───────────── GEMV on the tensor pipe (M ≤ 4, K % 256 == 0) ─────────────
// The FMA kernel above spends ~6 issue slots per weight (byte-permute, subtract,
// FMA, reduction), which is as expensive as the HBM stream itself.  Here the dot
// products go through mma.sync m16n8k16 (fp16 in, fp32 accumulate) purely to make
// the dequant cheap: one byte-permute turns two codes into two fp16 integers
// (0x6400|u = 1024+u, minus 1152 = the code, exact), and a 16-row × 32-k block costs
// two MMAs.  Activations stay fp32-accurate: each x is split into fp16 hi + fp16 lo
// (lo scaled by 2^11, the row pre-scaled by a power of two so |x| ≤ 1), which occupy
// two of the eight MMA columns; up to four activation rows share one weight pass.
// One MMA pair covers exactly one 32-k block of each row, so the block's fp32 scale
// multiplies the block's fp32 partial sum, as the format defines.
//   warp w of a CTA handles blocks w, w+8, …  of the CTA's 16-row tile; lane (g,t)
//   loads 8 codes of row g and of row g+8 (or gate row g / up row g for SwiGLU).
constexpr int kMmaWarps = 8;
constexpr int kMmaU = 4;            // blocks per load group (two groups in flight)
constexpr int kXsPad = 32;          // fp16 elements of padding per activation column

__device__ __forceinline__ uint2 ld_stream_u2(const void* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t codes_to_half2(uint32_t flipped, uint32_t selector) {
    // two bytes → two fp16 (1024+u), then −1152 → the signed codes as exact fp16 integers
    uint32_t h = __byte_perm(flipped, 0x64646464u, selector);
    uint32_t r;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(h), "r"(0x64806480u));
    return r;
}
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct MmaFrag { uint2 r0, r1; float s0, s1; };

template <bool SWIGLU>
__global__ void __launch_bounds__(kMmaWarps * 32) k_q8_gemv_mma(const GemvParams p, const int M) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int ldxs = p.K + kXsPad;
    const int NC = 2 * M;
    __half* xs = reinterpret_cast<__half*>(smem_raw);                        // [NC][ldxs]: col 2m = hi, 2m+1 = lo·2^11
    float* s_part = reinterpret_cast<float*>(smem_raw + (size_t)NC * ldxs * 2);   // [2][warps][16][8]
    __shared__ float s_red[3][kMmaWarps];
    __shared__ float s_xscale[4];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int rowsPerTile = SWIGLU ? 8 : 16;
    const int nTiles = (p.N + rowsPerTile - 1) / rowsPerTile;
    const int blocksPerWarp = (p.K >> 5) / kMmaWarps;
    const int groups = (blocksPerWarp + kMmaU - 1) / kMmaU;

    auto load_group = [&](int tile, int grp, MmaFrag (&f)[kMmaU]) {
        const int row0 = tile * rowsPerTile + g;
        const int row1 = SWIGLU ? row0 : row0 + 8;
        const int8_t* c1 = SWIGLU ? p.codes2 : p.codes;
        const float* sc1 = SWIGLU ? p.scales2 : p.scales;
#pragma unroll
        for (int u = 0; u < kMmaU; u++) {
            const int i = grp * kMmaU + u;
            const int blk = warp + kMmaWarps * i;
            const bool vb = i < blocksPerWarp;
            if (vb && row0 < p.N) {
                f[u].r0 = ld_stream_u2(p.codes + (size_t)row0 * p.Kp + blk * 32 + t * 8);
                f[u].s0 = __ldg(p.scales + (size_t)row0 * p.nb + blk);
            } else { f[u].r0 = make_uint2(0u, 0u); f[u].s0 = 0.0f; }
            if (vb && row1 < p.N) {
                f[u].r1 = ld_stream_u2(c1 + (size_t)row1 * p.Kp + blk * 32 + t * 8);
                f[u].s1 = __ldg(sc1 + (size_t)row1 * p.nb + blk);
            } else { f[u].r1 = make_uint2(0u, 0u); f[u].s1 = 0.0f; }
        }
    };

    MmaFrag fa[kMmaU], fb[kMmaU];
    int tile = blockIdx.x;
    const int stride = gridDim.x;
    if (tile < nTiles) load_group(tile, 0, fa);
    pdl_wait();
    pdl_launch_dependents();

    // ── activations → fp16 hi/lo columns in shared memory (RMSNorm fused) ──
    for (int m = 0; m < M; m++) {
        const float* xrow = p.x + (size_t)m * p.ldx;
        float ss = 0.0f, amax = 0.0f, gmax = 0.0f;
        for (int k = tid; k < p.K; k += blockDim.x) {
            float v = xrow[k];
            ss = fmaf(v, v, ss);
            amax = fmaxf(amax, fabsf(v));
            if (p.gamma) gmax = fmaxf(gmax, fabsf(p.gamma[k]));
        }
        for (int o = 16; o > 0; o >>= 1) {
            ss += __shfl_xor_sync(0xffffffffu, ss, o);
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            gmax = fmaxf(gmax, __shfl_xor_sync(0xffffffffu, gmax, o));
        }
        __syncthreads();
        if (lane == 0) { s_red[0][warp] = ss; s_red[1][warp] = amax; s_red[2][warp] = gmax; }
        __syncthreads();
        ss = 0.0f; amax = 0.0f; gmax = 0.0f;
#pragma unroll
        for (int q = 0; q < kMmaWarps; q++) { ss += s_red[0][q]; amax = fmaxf(amax, s_red[1][q]); gmax = fmaxf(gmax, s_red[2][q]); }
        float rms = 1.0f, bound = amax;
        if (p.gamma) {
            rms = sqrtf(ss * (1.0f / (float)p.K) + p.eps);
            bound = __fdiv_rn(amax, rms) * gmax;
        }
        // power of two ≥ bound (1 when the row is all zero or not finite)
        float sx = 1.0f;
        if (bound > 0.0f && bound < 1e37f) sx = __int_as_float((__float_as_int(bound) & 0x7f800000) + 0x00800000);
        const float inv_sx = 1.0f / sx;
        if (tid == 0) s_xscale[m] = sx;
        for (int k = tid; k < p.K; k += blockDim.x) {
            float v = xrow[k];
            if (p.gamma) v = __fdiv_rn(v, rms) * p.gamma[k];
            v *= inv_sx;
            __half hi = __float2half_rn(v);
            __half lo = __float2half_rn((v - __half2float(hi)) * 2048.0f);
            xs[(size_t)(2 * m) * ldxs + k] = hi;
            xs[(size_t)(2 * m + 1) * ldxs + k] = lo;
        }
    }
    __syncthreads();

    const uint4* xcol = reinterpret_cast<const uint4*>(xs + (size_t)(g < NC ? g : 0) * ldxs);
    const bool hasCol = g < NC;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};

    auto compute_group = [&](int grp, const MmaFrag (&f)[kMmaU]) {
#pragma unroll
        for (int u = 0; u < kMmaU; u++) {
            const int i = grp * kMmaU + u;
            const int blk = warp + kMmaWarps * i;
            if (i >= blocksPerWarp) break;
            uint4 xb = make_uint4(0u, 0u, 0u, 0u);
            if (hasCol) xb = xcol[(blk * 32 + t * 8) >> 3];
            const uint32_t w0 = f[u].r0.x ^ 0x80808080u, w1 = f[u].r0.y ^ 0x80808080u;
            const uint32_t v0 = f[u].r1.x ^ 0x80808080u, v1 = f[u].r1.y ^ 0x80808080u;
            float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            mma_16816(c, codes_to_half2(w0, 0x4140), codes_to_half2(v0, 0x4140),
                         codes_to_half2(w0, 0x4342), codes_to_half2(v0, 0x4342), xb.x, xb.y);
            mma_16816(c, codes_to_half2(w1, 0x4140), codes_to_half2(v1, 0x4140),
                         codes_to_half2(w1, 0x4342), codes_to_half2(v1, 0x4342), xb.z, xb.w);
            acc[0] = fmaf(f[u].s0, c[0], acc[0]);
            acc[1] = fmaf(f[u].s0, c[1], acc[1]);
            acc[2] = fmaf(f[u].s1, c[2], acc[2]);
            acc[3] = fmaf(f[u].s1, c[3], acc[3]);
        }
    };

    auto epilogue = [&](int tile, int buf) {
        float* part = s_part + (size_t)buf * kMmaWarps * 128;
        // c0,c1 → (row g, cols 2t,2t+1); c2,c3 → (row g+8, cols 2t,2t+1)
        float* mine = part + warp * 128;
        mine[g * 8 + 2 * t] = acc[0];       mine[g * 8 + 2 * t + 1] = acc[1];
        mine[(g + 8) * 8 + 2 * t] = acc[2]; mine[(g + 8) * 8 + 2 * t + 1] = acc[3];
        acc[0] = acc[1] = acc[2] = acc[3] = 0.0f;
        __syncthreads();
        const int r = tid % rowsPerTile, m = tid / rowsPerTile;
        if (m < M) {
            const int n = tile * rowsPerTile + r;
            if (n < p.N) {
                float hi = 0.0f, lo = 0.0f, hi2 = 0.0f, lo2 = 0.0f;
#pragma unroll
                for (int q = 0; q < kMmaWarps; q++) {
                    hi += part[q * 128 + r * 8 + 2 * m];
                    lo += part[q * 128 + r * 8 + 2 * m + 1];
                    if (SWIGLU) { hi2 += part[q * 128 + (r + 8) * 8 + 2 * m]; lo2 += part[q * 128 + (r + 8) * 8 + 2 * m + 1]; }
                }
                const float sx = s_xscale[m];
                float v = fmaf(lo, 1.0f / 2048.0f, hi) * sx;
                if (SWIGLU) {
                    float u = fmaf(lo2, 1.0f / 2048.0f, hi2) * sx;
                    if (p.bias) v += p.bias[n];
                    if (p.bias2) u += p.bias2[n];
                    float sig = 1.0f / (1.0f + expf(-v));
                    p.out[(size_t)m * p.ldo + n] = (v * sig) * u;          // SiLU(gate) ⊙ up
                } else {
                    if (p.bias) v += p.bias[n];
                    if (p.residual) v += p.residual[(size_t)m * p.ldr + n];
                    p.out[(size_t)m * p.ldo + n] = v;
                }
            }
        }
    };

    // Flat sequence of (tile, group) items; the loads of item i+1 are in flight
    // while item i goes through the tensor pipe.
    int grp = 0, buf = 0;
    while (tile < nTiles) {
        int ntile = tile, ngrp = grp + 1;
        if (ngrp == groups) { ngrp = 0; ntile = tile + stride; }
        if (ntile < nTiles) load_group(ntile, ngrp, fb);
        compute_group(grp, fa);
        if (grp == groups - 1) { epilogue(tile, buf); buf ^= 1; }
        tile = ntile; grp = ngrp;
        if (tile >= nTiles) break;
        ntile = tile; ngrp = grp + 1;
        if (ngrp == groups) { ngrp = 0; ntile = tile + stride; }
        if (ntile < nTiles) load_group(ntile, ngrp, fa);
        compute_group(grp, fb);
        if (grp == groups - 1) { epilogue(tile, buf); buf ^= 1; }
        tile = ntile; grp = ngrp;
    }
}

size_t gemv_mma_smem(int K, int M) {
    return (size_t)2 * M * (K + kXsPad) * 2 + (size_t)2 * kMmaWarps * 128 * 4;
}

template <bool SWIGLU>
void launch_gemv_mma(const GemvParams& p, int M, cudaStream_t s) {
    static size_t maxSmemSet = 0;
    static int lastSmemForOcc = -1, ctasPerSM = 1;
    size_t smem = gemv_mma_smem(p.K, M);
    if (smem > maxSmemSet) {
        DJ_CUDA_CHECK(cudaFuncSetAttribute(k_q8_gemv_mma<SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        maxSmemSet = 200 * 1024;
    }
    if (lastSmemForOcc != (int)smem) {
        DJ_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&ctasPerSM, k_q8_gemv_mma<SWIGLU>, kMmaWarps * 32, smem));
        if (ctasPerSM < 1) ctasPerSM = 1;
        lastSmemForOcc = (int)smem;
    }
    int rowsPerTile = SWIGLU ? 8 : 16;
    int nTiles = (p.N + rowsPerTile - 1) / rowsPerTile;
    int cap = g_num_sms * ctasPerSM;
    int gx = nTiles < cap ? nTiles : cap;
    launch_k(k_q8_gemv_mma<SWIGLU>, dim3(gx), dim3(kMmaWarps * 32), smem, s, true, p, M);
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

void launch_q8_linear(const Q8LinearArgs& a, cudaStream_t s) {
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
    if (g_gemv_mode == 2 && !noTc && a.M >= kTcMinRows && a.ws != nullptr && launch_q8_linear_tc(a, a.ws, s)) return;
    if (g_gemv_mode == 2 && a.M >= 5 && a.ws != nullptr && a.w.K % 32 == 0 && a.w.Kp == a.w.K) {
        // five or more rows share one pass over the weights, 16 at a time (up to four are two GEMV passes, which is as fast)
        bool ok = true;
        for (int m0 = 0; m0 < a.M && ok; m0 += 16) ok = launch_q8_linear_batch(a, m0, a.M - m0 < 16 ? a.M - m0 : 16, a.ws, a.tickets, s);
        if (ok) return;
    }
    if (g_gemv_mode == 2 && launch_q8_linear_tma(a, s)) return;
    if (g_gemv_mode >= 1 && p.K % 256 == 0 && gemv_mma_smem(p.K, 1) <= 200 * 1024) {
        // up to four activation rows share one pass over the weights
        int maxRows = 4;
        while (maxRows > 1 && gemv_mma_smem(p.K, maxRows) > 200 * 1024) maxRows--;
        for (int m0 = 0; m0 < a.M; m0 += maxRows) {
            GemvParams q = p;
            int rows = a.M - m0 < maxRows ? a.M - m0 : maxRows;
            q.x = p.x + (size_t)m0 * p.ldx;
            q.out = p.out + (size_t)m0 * p.ldo;
            if (p.residual) q.residual = p.residual + (size_t)m0 * p.ldr;
            if (swiglu) launch_gemv_mma<true>(q, rows, s); else launch_gemv_mma<false>(q, rows, s);
        }
        return;
    }
    if (swiglu) launch_gemv_dispatch<true>(p, a.M, s);
    else launch_gemv_dispatch<false>(p, a.M, s);
}

}  // namespace dj
