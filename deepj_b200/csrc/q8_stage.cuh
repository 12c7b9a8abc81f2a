// Activation staging and tile epilogue of the two Q8 GEMV kernels (cp.async rings in q8_gemv_i8.cu: CTA-wide
// staging, RMSNorm / LayerNorm fused; TMA rings in q8_gemv_tma.cu: per-warp staging, RMSNorm split between staging and
// epilogue): fp32 rows → three int8 digit columns + one power-of-two scale per 32-k block, and the cross-warp reduction
// with bias / GELU / residual / SiLU-gate fused.
#pragma once
#include "q8_common.cuh"

namespace dj {

constexpr int kGemvWarps = 8;
constexpr int kGemvThreads = kGemvWarps * 32;
constexpr int kGemvStageRounds = 3;         // rows of up to 3·256·16 = 12288 values are staged from registers
constexpr int kGemvXsPad = 32;              // bytes of padding per activation digit column
constexpr int kGemvColsPerRow = 3;          // digit columns per activation row in shared memory: d2, d1, d0

// Cross-warp sum of one value per thread (all threads of the CTA call it; s_red holds kGemvWarps floats).
__device__ __forceinline__ float gemv_block_sum(float v, float* s_red, int lane, int warp) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) s_red[warp] = v;
    __syncthreads();
    v = 0.0f;
#pragma unroll
    for (int q = 0; q < kGemvWarps; q++) v += s_red[q];
    return v;
}

// M activation rows → digit columns xd [3M][ldxs] and block scales xsc [M][K/32].  A thread converts 16
// consecutive values (half a block) per round; all rounds of a row are loaded before anything is converted, so a
// row costs one load round trip.  `after_first_loads` runs once, behind the first row's loads (the callers queue
// more weight copies there).  GPT adds LayerNorm1D (norm/LayerNorm1D.java:34-71: mean, biased variance,
// (x − mean)/√(var + eps)·γ + β); otherwise gamma != nullptr means RMSNorm1D (x / rms · γ).
template <bool GPT, class F>
__device__ __forceinline__ void gemv_stage_rows(const float* x, int ldx, const float* gamma, const float* beta, float eps, int K, int M,
                                                int8_t* xd, int ldxs, float* xsc, float* s_red, const float (&gpre)[16], bool gammaEarly,
                                                F&& after_first_loads) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nBlocks = K >> 5, nHalf = K >> 4;
    const int rounds = (nHalf + kGemvThreads - 1) / kGemvThreads;
    for (int m = 0; m < M; m++) {
        const float* xrow = x + (size_t)m * ldx;
        bool vec = ((reinterpret_cast<uintptr_t>(xrow) | (gamma ? reinterpret_cast<uintptr_t>(gamma) : 0)) & 15) == 0;
        if (GPT && beta) vec = vec && (reinterpret_cast<uintptr_t>(beta) & 15) == 0;
        int8_t* dcol = xd + (size_t)(kGemvColsPerRow * m) * ldxs;
        float* xscRow = xsc + (size_t)m * nBlocks;
        if (rounds <= kGemvStageRounds) {
            float xv[kGemvStageRounds][16];
#pragma unroll
            for (int r = 0; r < kGemvStageRounds; r++) {
                const int hb = r * kGemvThreads + tid;
                if (r < rounds && hb < nHalf) load16(xrow + hb * 16, vec, xv[r]);
                else {
#pragma unroll
                    for (int j = 0; j < 16; j++) xv[r][j] = 0.0f;
                }
            }
            if (m == 0) after_first_loads();
            float inv = 1.0f;
            const bool layerNorm = GPT && gamma && beta;
            if (layerNorm) {
                // padding lanes hold zeros: they add nothing to the sum, and are masked out of the squared deviations
                float sm = 0.0f;
#pragma unroll
                for (int r = 0; r < kGemvStageRounds; r++)
#pragma unroll
                    for (int j = 0; j < 16; j++) sm += xv[r][j];
                const float mean = gemv_block_sum(sm, s_red, lane, warp) * (1.0f / (float)K);
                float ss = 0.0f;
#pragma unroll
                for (int r = 0; r < kGemvStageRounds; r++) {
                    const bool on = r < rounds && r * kGemvThreads + tid < nHalf;
#pragma unroll
                    for (int j = 0; j < 16; j++) { xv[r][j] = on ? xv[r][j] - mean : 0.0f; ss = fmaf(xv[r][j], xv[r][j], ss); }
                }
                ss = gemv_block_sum(ss, s_red, lane, warp);
                inv = __frcp_rn(sqrtf(ss * (1.0f / (float)K) + eps));
            } else if (gamma) {
                float ss = 0.0f;
#pragma unroll
                for (int r = 0; r < kGemvStageRounds; r++)
#pragma unroll
                    for (int j = 0; j < 16; j++) ss = fmaf(xv[r][j], xv[r][j], ss);
                ss = gemv_block_sum(ss, s_red, lane, warp);
                inv = __frcp_rn(sqrtf(ss * (1.0f / (float)K) + eps));      // RMSNorm1D.forward: x / rms · γ
            }
#pragma unroll
            for (int r = 0; r < kGemvStageRounds; r++) {
                const int hb = r * kGemvThreads + tid;
                const bool on = r < rounds && hb < nHalf;
                if (gamma) {
                    float gv[16];
                    if (gammaEarly) {
#pragma unroll
                        for (int j = 0; j < 16; j++) gv[j] = gpre[j];
                    } else if (on) load16(gamma + hb * 16, vec, gv);
                    else {
#pragma unroll
                        for (int j = 0; j < 16; j++) gv[j] = 1.0f;
                    }
#pragma unroll
                    for (int j = 0; j < 16; j++) xv[r][j] = (xv[r][j] * inv) * gv[j];
                    if (layerNorm && on) {
                        load16(beta + hb * 16, vec, gv);
#pragma unroll
                        for (int j = 0; j < 16; j++) xv[r][j] += gv[j];
                    }
                }
                if (r < rounds) digits16(xv[r], on, dcol, ldxs, hb, xscRow);
            }
        } else {
            // very wide rows: one pass for the sum of squares, then round by round
            float inv = 1.0f;
            if (gamma) {
                float ss = 0.0f;
                for (int k = tid; k < K; k += kGemvThreads) { float v = xrow[k]; ss = fmaf(v, v, ss); }
                ss = gemv_block_sum(ss, s_red, lane, warp);
                inv = __frcp_rn(sqrtf(ss * (1.0f / (float)K) + eps));
            }
            if (m == 0) after_first_loads();
            for (int r = 0; r < rounds; r++) {
                const int hb = r * kGemvThreads + tid;
                const bool on = hb < nHalf;
                float xv[16], gv[16];
                if (on) load16(xrow + hb * 16, vec, xv);
                else {
#pragma unroll
                    for (int j = 0; j < 16; j++) xv[j] = 0.0f;
                }
                if (gamma) {
                    if (on) load16(gamma + hb * 16, vec, gv);
                    else {
#pragma unroll
                        for (int j = 0; j < 16; j++) gv[j] = 1.0f;
                    }
#pragma unroll
                    for (int j = 0; j < 16; j++) xv[j] = (xv[j] * inv) * gv[j];
                }
                digits16(xv, on, dcol, ldxs, hb, xscRow);
            }
        }
    }
}

__device__ __forceinline__ float4 gemv_load4(const float* src, bool vec) {
    if (vec) return *reinterpret_cast<const float4*>(src);
    return make_float4(src[0], src[1], src[2], src[3]);
}

// Staging for kernels whose warp w consumes only the 128-k groups w, w+8, … of the reduction: the warp converts exactly
// those groups of every row into its own part of the digit columns, so nothing but the warp itself waits for it — no
// block-wide barrier stands between the wait for the previous kernel and the first MMA.  RMSNorm is split: the gain
// is folded into the digits (x·γ), the warp's part of Σx² goes to ss_part[m][warp], and the tile epilogue multiplies
// the finished sums by 1/rms (Σ_k w_k·(x_k·γ_k)/rms = Σ_k w_k·(x_k/rms·γ_k)).  A lane converts four consecutive
// values of a group; eight lanes share a 32-k block.  Digits are stored in the order of the int8 MMA's B fragment, so that
// lane t fetches both of its registers (k = 4t … 4t+3 and k = 16+4t … 16+4t+3) with one 8-byte load at offset 8t: value k
// of a block sits at 8·((k mod 16)/4) + 4·(k/16) + k mod 4.
constexpr int kGemvWarpGroups = 12;         // groups a warp keeps in registers per load round trip: rows of up to 12288 values in one
template <class F>
__device__ __forceinline__ void gemv_stage_warp_groups(const float* x, int ldx, const float* gamma, int K, int M, int8_t* xd, int ldxs,
                                                       float* xsc, float* ss_part, const float4 (&gpre)[4], bool gammaEarly,
                                                       F&& after_first_loads) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nGroups = K >> 7, nBlocks = K >> 5;
    const int j8 = lane & 7;
    const int pos = j8 < 4 ? 8 * j8 : 8 * (j8 - 4) + 4;          // where the lane's four values sit inside the permuted block
    for (int m = 0; m < M; m++) {
        const float* xrow = x + (size_t)m * ldx;
        const bool vec = ((reinterpret_cast<uintptr_t>(xrow) | (gamma ? reinterpret_cast<uintptr_t>(gamma) : 0)) & 15) == 0;
        int8_t* dcol = xd + (size_t)(kGemvColsPerRow * m) * ldxs;
        float* xscRow = xsc + (size_t)m * nBlocks;
        float ss = 0.0f;
        for (int g0 = warp; g0 < nGroups; g0 += kGemvWarps * kGemvWarpGroups) {
            float4 xv[kGemvWarpGroups];
#pragma unroll
            for (int i = 0; i < kGemvWarpGroups; i++) {
                const int grp = g0 + kGemvWarps * i;
                xv[i] = grp < nGroups ? gemv_load4(xrow + grp * 128 + lane * 4, vec) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
            if (m == 0 && g0 == warp) after_first_loads();
#pragma unroll
            for (int i = 0; i < kGemvWarpGroups; i++) {
                const int grp = g0 + kGemvWarps * i;
                if (grp >= nGroups) break;                           // warp-uniform
                float v[4] = {xv[i].x, xv[i].y, xv[i].z, xv[i].w};
                ss = fmaf(v[0], v[0], ss); ss = fmaf(v[1], v[1], ss); ss = fmaf(v[2], v[2], ss); ss = fmaf(v[3], v[3], ss);
                if (gamma) {
                    const float4 gv = (gammaEarly && g0 == warp && i < 4) ? gpre[i & 3] : gemv_load4(gamma + grp * 128 + lane * 4, vec);
                    v[0] *= gv.x; v[1] *= gv.y; v[2] *= gv.z; v[3] *= gv.w;
                }
                float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
                int sbits = 0x3f800000;                              // as digits16: s = 2^(exponent(amax)+2), q = rne(v·2^23/s)
                if (amax > 0.0f && amax < 1e36f) sbits = (__float_as_int(amax) & 0x7f800000) + 0x01000000;
                const float mul = __int_as_float(0x7f000000 - sbits) * 8388608.0f;
                uint32_t u[4];
#pragma unroll
                for (int e = 0; e < 4; e++) u[e] = (uint32_t)(__float2int_rn(v[e] * mul) + 0x808080);
                const uint32_t t0 = __byte_perm(u[0], u[1], 0x5140), t1 = __byte_perm(u[2], u[3], 0x5140);
                const uint32_t t2 = __byte_perm(u[0], u[1], 0x7362), t3 = __byte_perm(u[2], u[3], 0x7362);
                const int blk = grp * 4 + (lane >> 3);
                int8_t* b = dcol + blk * 32 + pos;
                *reinterpret_cast<uint32_t*>(b) = __byte_perm(t2, t3, 0x5410) ^ 0x80808080u;
                *reinterpret_cast<uint32_t*>(b + ldxs) = __byte_perm(t0, t1, 0x7632) ^ 0x80808080u;
                *reinterpret_cast<uint32_t*>(b + 2 * ldxs) = __byte_perm(t0, t1, 0x5410) ^ 0x80808080u;
                if (j8 == 0) xscRow[blk] = __int_as_float(sbits) * (1.0f / 8388608.0f);
            }
        }
        if (gamma) {
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (lane == 0) ss_part[m * kGemvWarps + warp] = ss;
        }
    }
    __syncwarp();
}

// Operands of a tile's epilogue, fetched before the tile so that their latency hides behind it: thread `tid`
// finishes output (row em = tid / rowsPerTile of the activations, column en = tile·rowsPerTile + tid % rowsPerTile).
struct GemvEpilogueOperands { float bias, bias2, res; };

template <bool SWIGLU>
__device__ __forceinline__ GemvEpilogueOperands gemv_epilogue_fetch(int tile, int M, int N, const float* bias, const float* bias2,
                                                                    const float* residual, int ldr) {
    constexpr int rowsPerTile = SWIGLU ? 8 : 16;
    const int er = threadIdx.x % rowsPerTile, em = threadIdx.x / rowsPerTile, en = tile * rowsPerTile + er;
    GemvEpilogueOperands o = {0.0f, 0.0f, 0.0f};
    if (em < M && en < N) {
        if (bias) o.bias = bias[en];
        if (SWIGLU && bias2) o.bias2 = bias2[en];
        if (!SWIGLU && residual) o.res = residual[(size_t)em * ldr + en];
    }
    return o;
}

// Reduces the warps' partial sums of one tile (part: [warps][NM][16 rows][8 columns], column 4(m%2) + d = digit
// 2 − d of activation row m), recombines the digits and stores the fused result.  acc is zeroed for the next tile.
// ss_part != nullptr: the sums are of x·γ and get the row's 1/rms here.
template <bool SWIGLU, bool GPT, int NM>
__device__ __forceinline__ void gemv_tile_epilogue(float (&acc)[NM][4], float* part, int tile, int M, int N, const GemvEpilogueOperands& o,
                                                   bool hasBias, bool hasBias2, bool hasRes, int act, float* out, int ldo,
                                                   const float* ss_part = nullptr, float eps = 0.0f, int K = 1) {
    constexpr int rowsPerTile = SWIGLU ? 8 : 16;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int er = tid % rowsPerTile, em = tid / rowsPerTile, en = tile * rowsPerTile + er;
#pragma unroll
    for (int q = 0; q < NM; q++) {
        float* mine = part + (warp * NM + q) * 128;
        mine[g * 8 + 2 * t] = acc[q][0];       mine[g * 8 + 2 * t + 1] = acc[q][1];
        mine[(g + 8) * 8 + 2 * t] = acc[q][2]; mine[(g + 8) * 8 + 2 * t + 1] = acc[q][3];
        acc[q][0] = acc[q][1] = acc[q][2] = acc[q][3] = 0.0f;
    }
    __syncthreads();
    if (em < M && en < N) {
        float a2 = 0.0f, a1 = 0.0f, a0 = 0.0f, b2 = 0.0f, b1 = 0.0f, b0 = 0.0f;
#pragma unroll
        for (int q = 0; q < kGemvWarps; q++) {
            const float* pr = part + (q * NM + (em >> 1)) * 128 + er * 8 + 4 * (em & 1);      // MMA em/2, columns 4(em%2) .. +2
            a2 += pr[0]; a1 += pr[1]; a0 += pr[2];
            if (SWIGLU) { b2 += pr[64]; b1 += pr[65]; b0 += pr[66]; }
        }
        float v = fmaf(a2, 65536.0f, fmaf(a1, 256.0f, a0));
        float inv = 1.0f;
        if (ss_part) {                                   // RMSNorm left to the epilogue (gemv_stage_warp_groups): the warps' parts of Σx² in a fixed order
            float ss = 0.0f;
#pragma unroll
            for (int q = 0; q < kGemvWarps; q++) ss += ss_part[em * kGemvWarps + q];
            inv = __frcp_rn(sqrtf(ss * (1.0f / (float)K) + eps));
            v *= inv;
        }
        if (SWIGLU) {
            float u = fmaf(b2, 65536.0f, fmaf(b1, 256.0f, b0)) * inv;
            if (hasBias) v += o.bias;
            if (hasBias2) u += o.bias2;
            float sig = 1.0f / (1.0f + expf(-v));
            out[(size_t)em * ldo + en] = (v * sig) * u;          // SiLU(gate) ⊙ up
        } else {
            if (hasBias) v += o.bias;
            if (GPT && act == 1) v = gelu_ref(v);
            if (hasRes) v += o.res;
            out[(size_t)em * ldo + en] = v;
        }
    }
}

}  // namespace dj
