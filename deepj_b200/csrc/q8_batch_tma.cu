// Q8 linear for a small batch of activation rows (5 … 16 per launch) on the integer tensor pipe with warp-private
// TMA rings — the decode step of several concurrent sequences, for reduction lengths that are multiples of 128.
//
// HBM-bound: every weight byte is read once per launch and used for all rows.  The work decomposition is the
// fp16 kernel's (q8_batch.cu): K is cut into slices of 512, a work item is (group of 8 row tiles, slice), each warp
// owns one 16-row tile of the group, partial sums meet in a global workspace in records of the same layout.  What
// changed is everything inside a work item, and who adds the slices:
//   * weights reach shared memory as tiled bulk copies of the native [N][K] / [N][K/32] layout (two 8-row × 128-byte
//     boxes of codes, 128-byte swizzle, and two 8-row × 4 boxes of scales per 128-k item) on a warp-private
//     mbarrier; the MMA's A operand is one ldmatrix.x4 per 32-k block — no dequantisation instruction at all;
//   * the activations are the B operand as 16-bit fixed point per 32-k block: x · 32767 / (the block's largest |x|),
//     rounded to an integer q in [−32767, 32767] and split into a signed high byte and an unsigned low byte.  High bytes and low bytes sit in separate MMAs (s8 × s8 and s8 × u8), eight activation
//     rows per MMA, so that a lane holds both sums of one (weight row, activation row) pair: 256·S_hi + S_lo is the
//     exact integer block sum, and (weight scale × block maximum / 32767) × sum is accumulated in fp32.  The
//     activation error is at most 2^-16 of the block's largest |x| (the fp16 kernel carried 22 bits).  Measured on
//     the 32-block 7B model at context 2048, 16 sequences: logits within 3e-4 of the logit range of the single-row
//     path, tokens equal — the stated tolerance is 2e-3, and the bench line carries this check on every run;
//   * no tickets: the slices of a tile are added by a second, small kernel (k_q8_batch_reduce), so the main kernel's
//     warps never wait on a fence or an atomic;
//   * RMSNorm as before: the digits are taken from x ⊙ γ, Σx² of every slice is left in the workspace by the CTAs
//     that stage it, and the row factor 1/rms is applied in the epilogue.
#include <cuda.h>

#include "kernels.h"
#include "q8_batch_tail.cuh"
#include "q8_common.cuh"
#include "q8_tma.cuh"

namespace dj {
namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kSlice = 512;                          // reduction length per work item; must equal the fp16 kernel's (same workspace layout)
constexpr int kCodeBytes = 16 * kTmaItemK;           // 16 rows × 128 code bytes, two 1024-byte swizzle atoms
constexpr int kScaleBytes = 16 * 16;                 // 16 rows × 4 block scales
constexpr int kItemBytes = kCodeBytes + kScaleBytes;
// Ring slots per warp (two items in flight).  Measured in the 16-sequence decode step of the 7B model: 3 slots 8.75 ms,
// 4 slots 8.83 ms, 5 slots 11.1 ms per step with identical times back to back — the shared memory a deeper ring takes is
// L1 capacity that the attention kernel beside it (two thirds of that step) uses.
constexpr int kRingDepth = 3;
constexpr int kPre = 2;                              // of which fetched before the previous kernel has finished
constexpr int kLdx = kSlice + 32;                    // bytes per activation byte column (32 mod 128: conflict-free 8-byte reads)
constexpr int kCols = 2 * kBatchMaxRows;             // high-byte columns of rows 0..15, then low-byte columns
constexpr int kSliceBlocks = kSlice / 32;
constexpr int kXsLd = kSliceBlocks + 4;               // floats per row of the activation block scales: rows 2t, 2t+1 of the four lanes t hit different banks
constexpr int kSpinLimit = 1 << 22;
constexpr int kErrTmaWait = 331;                     // device error code: an item never arrived

struct BatchTmaParams {
    CUtensorMap codes, scales, codes2, scales2;
    const float* x; int ldx;
    const float* gamma;
    int K, N, M;
    int nSlices, nGroups, nTiles;
    BatchTail tail;
    int* error;
    unsigned long long* trace;
};

__device__ __forceinline__ void mma_s8u8_16832(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NP = MMA pairs per block: activation rows 0..7 (NP = 1) or 0..15 (NP = 2)
template <bool SWIGLU, int NP, int kDepth>
__global__ void __launch_bounds__(kThreads, 2) k_q8_gemm_i8(const __grid_constant__ BatchTmaParams p) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long s_bar[kWarps * kDepth];
    // layout from a 1024-byte boundary: code rings [warps][kDepth][2048] | scale rings [warps][kDepth][256] |
    // activation byte columns [32][kLdx] | activation block scales fp32 [16 rows][kXsLd]
    const uint32_t raw_s = smem_u32(smem_raw);
    unsigned char* const smem = smem_raw + (((raw_s + 1023u) & ~1023u) - raw_s);
    unsigned char* const ringC = smem;
    unsigned char* const ringS = smem + (size_t)kWarps * kDepth * kCodeBytes;
    unsigned char* const xd = ringS + (size_t)kWarps * kDepth * kScaleBytes;
    float* const xs = reinterpret_cast<float*>(xd + (size_t)kCols * kLdx);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    constexpr int rowsPerTile = SWIGLU ? 8 : 16;
    const int nItems = p.nGroups * p.nSlices;
    const bool tracing = p.trace != nullptr && blockIdx.x == 0 && tid == 0;
    if (tracing) { p.trace[0] = gtime(); p.trace[6] = 0ull; }

    const uint32_t myC = smem_u32(ringC) + (uint32_t)warp * kDepth * kCodeBytes;
    const uint32_t myS = smem_u32(ringS) + (uint32_t)warp * kDepth * kScaleBytes;
    const uint32_t myBar = smem_u32(&s_bar[warp * kDepth]);
    if (lane == 0) {
#pragma unroll
        for (int d = 0; d < kDepth; d++) mbar_init(myBar + 8 * d, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();

    // flat (work item, 128-k group) sequence of this warp with a cursor running kDepth-1 items ahead; rows past N
    // (a warp whose tile lies past the last row included) are filled with zeros by the copy engine
    int iitem = blockIdx.x, igi = 0, islot = 0;
    auto groups_of = [&](int item) { return (min(kSlice, p.K - (item % p.nSlices) * kSlice)) / kTmaItemK; };
    auto issue_next = [&]() {
        if (iitem < nItems) {
            if (lane == 0) {
                const int slice = iitem % p.nSlices, grp = iitem / p.nSlices;
                const int row0 = (grp * kWarps + warp) * rowsPerTile;
                const int k = slice * kSlice + igi * kTmaItemK;
                const uint32_t bar = myBar + 8 * islot;
                const uint32_t dc = myC + (uint32_t)islot * kCodeBytes, ds = myS + (uint32_t)islot * kScaleBytes;
                mbar_arrive_expect_tx(bar, kItemBytes);
                tma_box(dc, &p.codes, k, row0, bar);
                tma_box(dc + kCodeBytes / 2, SWIGLU ? &p.codes2 : &p.codes, k, SWIGLU ? row0 : row0 + 8, bar);
                tma_box(ds, &p.scales, k >> 5, row0, bar);
                tma_box(ds + kScaleBytes / 2, SWIGLU ? &p.scales2 : &p.scales, k >> 5, SWIGLU ? row0 : row0 + 8, bar);
            }
            if (++igi >= groups_of(iitem)) { igi = 0; iitem += gridDim.x; }
        }
        islot = islot + 1 == kDepth ? 0 : islot + 1;
    };
    for (int d = 0; d < kPre; d++) issue_next();
    pdl_launch_dependents();
    if (tracing) p.trace[1] = gtime();
    pdl_wait();
    if (tracing) p.trace[2] = gtime();
    for (int d = kPre; d < kDepth - 1; d++) issue_next();

    // columns of rows ≥ M stay zero
    for (int i = tid; i < (kCols * kLdx + kBatchMaxRows * kXsLd * 4) / 4; i += kThreads) reinterpret_cast<uint32_t*>(xd)[i] = 0u;

    // B fragments: MMA pair j covers activation rows 8j … 8j+7, lane (g,t) feeds row 8j + g; its two registers of a
    // block (k = 4t … 4t+3 and 16+4t … 16+4t+3) are the 8 bytes at 8t of the permuted block
    const unsigned char* xhi = xd + (size_t)g * kLdx + t * 8;
    const unsigned char* xlo = xd + (size_t)(kBatchMaxRows + g) * kLdx + t * 8;
    // ldmatrix.x4 addresses (see q8_gemv_tma.cu)
    const int lrow = (lane & 7) + ((lane >> 3) & 1) * 8;
    const uint32_t lmBase = (uint32_t)lrow * 128u;
    const uint32_t lmChunk = (uint32_t)((lane >> 4) ^ (lrow & 7));
    int staged = -1, cslot = 0, limit = kSpinLimit;
    uint32_t phases = 0;
    for (int item = blockIdx.x; item < nItems; item += gridDim.x) {
        const int slice = item % p.nSlices, grp = item / p.nSlices;
        const int k0 = slice * kSlice;
        const int nGrp = groups_of(item);
        if (slice != staged) {
            __syncthreads();            // every warp is done with the previous slice's columns (and with the clearing above)
            // one warp pass per activation row: 512 values; a lane converts 16 (half a block)
            for (int m0 = warp; m0 < p.M; m0 += 2 * kWarps) {
                float xv[2][16], gv[2][16];
                bool on[2];
#pragma unroll
                for (int u = 0; u < 2; u++) {
                    const int m = m0 + u * kWarps;
                    on[u] = m < p.M && k0 + lane * 16 < p.K;
                    const float* xrow = p.x + (size_t)m * p.ldx + k0;
                    const bool vec = ((reinterpret_cast<uintptr_t>(xrow) | (p.gamma ? reinterpret_cast<uintptr_t>(p.gamma + k0) : 0)) & 15) == 0;
                    if (on[u]) {
                        load16(xrow + lane * 16, vec, xv[u]);
                        if (p.gamma) load16(p.gamma + k0 + lane * 16, vec, gv[u]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; j++) { xv[u][j] = 0.0f; gv[u][j] = 1.0f; }
                    }
                }
#pragma unroll
                for (int u = 0; u < 2; u++) {
                    const int m = m0 + u * kWarps;
                    if (m >= p.M) break;                               // warp-uniform
                    if (p.gamma) {
                        float ss = 0.0f;
#pragma unroll
                        for (int j = 0; j < 16; j++) ss = fmaf(xv[u][j], xv[u][j], ss);
                        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                        if (lane == 0) p.tail.ssq[slice * kBatchMaxRows + m] = ss;      // every CTA that stages this slice writes the same bits
#pragma unroll
                        for (int j = 0; j < 16; j++) xv[u][j] *= gv[u][j];
                    }
                    float amax = 0.0f;
#pragma unroll
                    for (int j = 0; j < 16; j++) amax = fmaxf(amax, fabsf(xv[u][j]));
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));          // the other half of the 32-k block
                    // q = rne(x · 32767 / amax) uses the whole 16-bit range; blocks whose largest value is below 2^-100 count as zero
                    const bool live = amax >= 7.8886e-31f && amax <= 3.0e38f;
                    const float mul = live ? __fdividef(32767.0f, amax) : 0.0f;
                    uint32_t whi[4], wlo[4];
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        uint32_t q[4];
#pragma unroll
                        for (int i = 0; i < 4; i++) q[i] = (uint32_t)min(__float2int_rn(xv[u][4 * j + i] * mul), 32767);
                        const uint32_t t0 = __byte_perm(q[0], q[1], 0x5140), t1 = __byte_perm(q[2], q[3], 0x5140);
                        wlo[j] = __byte_perm(t0, t1, 0x5410);          // bits 0-7 of the four values
                        whi[j] = __byte_perm(t0, t1, 0x7632);          // bits 8-15: the signed high byte
                    }
                    if (on[u]) {
                        // the block order of the MMA's B fragment (as gemv_stage_warp_groups): the lane's values 4j … 4j+3 sit at 8j + 4·(half of the block)
                        unsigned char* bh = xd + (size_t)m * kLdx + (lane >> 1) * 32 + (lane & 1) * 4;
                        unsigned char* bl = bh + (size_t)kBatchMaxRows * kLdx;
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            *reinterpret_cast<uint32_t*>(bh + 8 * j) = whi[j];
                            *reinterpret_cast<uint32_t*>(bl + 8 * j) = wlo[j];
                        }
                        if ((lane & 1) == 0) xs[m * kXsLd + (lane >> 1)] = live ? amax * (1.0f / 32767.0f) : 0.0f;
                    }
                }
            }
            staged = slice;
            __syncthreads();
            if (tracing && item == blockIdx.x) p.trace[3] = gtime();
        }

        // the lane's results of pair j: weight rows g, g+8 × activation rows 8j + 2t, 8j + 2t + 1
        float acc[NP][4];
#pragma unroll
        for (int j = 0; j < NP; j++) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f; }
        for (int gi = 0; gi < nGrp; gi++) {
            issue_next();
            const uint32_t bar = myBar + 8 * cslot;
            const uint32_t parity = (phases >> cslot) & 1u;
            bool ready = mbar_try_wait(bar, parity);
            for (int spin = 0; !ready && spin < limit; spin++) ready = mbar_try_wait(bar, parity);
            if (!ready) {                               // never on a healthy device: flag it, stop waiting long, keep the control flow
                if (lane == 0) atomicCAS(p.error, 0, kErrTmaWait);
                limit = 64;
            }
            phases ^= 1u << cslot;
            const uint32_t sc = myC + (uint32_t)cslot * kCodeBytes;
            const unsigned char* ss = ringS + ((size_t)warp * kDepth + cslot) * kScaleBytes;
            const float4 w0 = *reinterpret_cast<const float4*>(ss + g * 16);            // weight row g: its four block scales
            const float4 w1 = *reinterpret_cast<const float4*>(ss + (g + 8) * 16);      // row g+8
            const float w0v[4] = {w0.x, w0.y, w0.z, w0.w}, w1v[4] = {w1.x, w1.y, w1.z, w1.w};
            float xsv[NP][2][4];
#pragma unroll
            for (int j = 0; j < NP; j++)
#pragma unroll
                for (int r = 0; r < 2; r++) {
                    const float4 v = *reinterpret_cast<const float4*>(xs + (8 * j + 2 * t + r) * kXsLd + gi * 4);
                    xsv[j][r][0] = v.x; xsv[j][r][1] = v.y; xsv[j][r][2] = v.z; xsv[j][r][3] = v.w;
                }
#pragma unroll
            for (int b = 0; b < 4; b++) {
                uint32_t a[4];
                ldmatrix_x4(a, sc + lmBase + ((lmChunk ^ (uint32_t)(2 * b)) << 4));
                const int boff = (gi * 4 + b) * 32;
#pragma unroll
                for (int j = 0; j < NP; j++) {
                    const uint2 bh = *reinterpret_cast<const uint2*>(xhi + (size_t)j * 8 * kLdx + boff);
                    const uint2 bl = *reinterpret_cast<const uint2*>(xlo + (size_t)j * 8 * kLdx + boff);
                    int ch[4] = {0, 0, 0, 0}, cl[4] = {0, 0, 0, 0};
                    mma_s8_16832(ch, a[0], a[1], a[2], a[3], bh.x, bh.y);
                    mma_s8u8_16832(cl, a[0], a[1], a[2], a[3], bl.x, bl.y);
                    acc[j][0] = fmaf(w0v[b] * xsv[j][0][b], (float)(ch[0] * 256 + cl[0]), acc[j][0]);
                    acc[j][1] = fmaf(w0v[b] * xsv[j][1][b], (float)(ch[1] * 256 + cl[1]), acc[j][1]);
                    acc[j][2] = fmaf(w1v[b] * xsv[j][0][b], (float)(ch[2] * 256 + cl[2]), acc[j][2]);
                    acc[j][3] = fmaf(w1v[b] * xsv[j][1][b], (float)(ch[3] * 256 + cl[3]), acc[j][3]);
                }
            }
            __syncwarp();           // every lane has read the slot before lane 0 hands it to the copy engine again
            cslot = cslot + 1 == kDepth ? 0 : cslot + 1;
        }
        if (tracing && item == blockIdx.x) p.trace[4] = gtime();
        const int tile = grp * kWarps + warp;
        if (tile >= p.nTiles) continue;                     // warp-uniform: nothing to deliver
        float* rec = p.tail.ws + ((size_t)tile * p.nSlices + slice) * kBatchTileFloats;
#pragma unroll
        for (int j = 0; j < NP; j++)
#pragma unroll
            for (int r = 0; r < 2; r++) {
                const int m = 8 * j + 2 * t + r;
                if (m < p.M) {
                    rec[m * 16 + g] = acc[j][r];
                    rec[m * 16 + g + 8] = acc[j][2 + r];
                }
            }
    }
    if (tracing) p.trace[5] = gtime();
    if (p.trace != nullptr && lane == 0) atomicMax(p.trace + 6, gtime());
}

// The slices of every tile meet here: one thread per (activation row, weight row) of a tile adds the tile's records
// in slice order (deterministic), applies RMSNorm's 1/rms from the Σx² the staging CTAs left per slice, and runs the
// epilogue (bias, residual, SiLU-gate).  A kernel of its own instead of tickets inside the main one: the records of a
// launch are a few MB in L2, the sums run fully parallel, and no warp of the main kernel ever waits on a fence or an
// atomic (measured with last-arriver merges: the main kernel's CTAs streamed for 16 µs and merged for 13 µs).
template <bool SWIGLU>
__global__ void __launch_bounds__(256) k_q8_batch_reduce(const BatchTail t, int nTiles, int nChunksK) {
    __shared__ float s_inv[kBatchMaxRows];
    constexpr int rowsPerTile = SWIGLU ? 8 : 16;
    const int tid = threadIdx.x, m = tid >> 4, r = tid & 15;
    pdl_wait();
    pdl_launch_dependents();
    // the first tile's records are requested together with the Σx² parts: one load round trip before the first sum
    const bool live = m < t.M;
    auto fetch = [&](int tile, float (&rec)[8], int s0) {
        const float* base = t.ws + (size_t)tile * t.nSlices * kBatchTileFloats + tid;
#pragma unroll
        for (int q = 0; q < 8; q++) rec[q] = (live && s0 + q < t.nSlices) ? __ldcg(base + (size_t)(s0 + q) * kBatchTileFloats) : 0.0f;
    };
    float rec[8];
    int tile = blockIdx.x;
    if (tile < nTiles) fetch(tile, rec, 0);
    {
        // row m's Σx²: the 16 threads of the row take the chunks r, r+16, … and meet in a fixed shuffle tree
        float ss = 0.0f;
        if (t.gamma && live)
            for (int c = r; c < nChunksK; c += 16) ss += __ldcg(t.ssq + c * kBatchMaxRows + m);
        for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (r == 0) s_inv[m] = (t.gamma && live) ? __frcp_rn(sqrtf(ss * (1.0f / (float)t.K) + t.eps)) : 1.0f;
    }
    __syncthreads();
    const float inv = s_inv[m];
    for (; tile < nTiles; tile += gridDim.x) {
        float v = 0.0f;
        for (int s0 = 0; s0 < t.nSlices; s0 += 8) {           // eight loads in flight, added in slice order
            if (s0 > 0) fetch(tile, rec, s0);
#pragma unroll
            for (int q = 0; q < 8; q++) v += rec[q];
        }
        v *= inv;
        const int next = tile + gridDim.x;
        if (next < nTiles) fetch(next, rec, 0);
        if (SWIGLU) {
            const float u = __shfl_down_sync(0xffffffffu, v, 8);      // the up projection's row sits 8 lanes on
            const int n = tile * rowsPerTile + r;
            if (m < t.M && r < 8 && n < t.N) {
                float vv = v, uu = u;
                if (t.bias) vv += t.bias[n];
                if (t.bias2) uu += t.bias2[n];
                const float sig = 1.0f / (1.0f + expf(-vv));
                t.out[(size_t)m * t.ldo + n] = (vv * sig) * uu;
            }
        } else {
            const int n = tile * rowsPerTile + r;
            if (m < t.M && n < t.N) {
                float vv = v;
                if (t.bias) vv += t.bias[n];
                if (t.residual) vv += t.residual[(size_t)m * t.ldr + n];
                t.out[(size_t)m * t.ldo + n] = vv;
            }
        }
    }
}

constexpr size_t batch_tma_smem(int kDepth) {
    return 1024 + (size_t)kWarps * kDepth * kItemBytes + (size_t)kCols * kLdx + (size_t)kBatchMaxRows * kXsLd * 4;
}

template <bool SWIGLU, int NP, int kDepth>
void launch_batch_tma(const BatchTmaParams& p, cudaStream_t s) {
    static bool attrSet = false;
    if (!attrSet) {
        DJ_CUDA_CHECK(cudaFuncSetAttribute(k_q8_gemm_i8<SWIGLU, NP, kDepth>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)batch_tma_smem(kDepth)));
        attrSet = true;
    }
    const int nItems = p.nGroups * p.nSlices;
    int cap = 2 * g_num_sms;
    if (p.nSlices <= cap) cap -= cap % p.nSlices;       // a CTA then keeps its slice from item to item
    const int gx = nItems < cap ? nItems : cap;
    launch_k(k_q8_gemm_i8<SWIGLU, NP, kDepth>, dim3(gx), dim3(kThreads), batch_tma_smem(kDepth), s, true, p);
    const int nChunksK = (p.K + kSlice - 1) / kSlice;
    launch_k(k_q8_batch_reduce<SWIGLU>, dim3(p.nTiles < 4 * g_num_sms ? p.nTiles : 4 * g_num_sms), dim3(256), 0, s, true, p.tail, p.nTiles, nChunksK);
}

}  // namespace

// Rows m0 … m0+rows−1 (rows ≤ 16) of a Q8 linear / SwiGLU with the workspace layout of launch_q8_linear_batch.
// Returns false when the shape is outside this kernel's domain (K a multiple of 128).
bool launch_q8_linear_batch_tma(const Q8LinearArgs& a, int m0, int rows, float* ws, int* tickets, cudaStream_t s) {
    const int K = a.w.K;
    if (K % kTmaItemK != 0 || a.w.Kp != K || rows < 1 || rows > kBatchMaxRows || g_dev_error == nullptr) return false;
    if (a.beta != nullptr || a.act != 0) return false;
    const bool swiglu = a.w2.codes != nullptr;
    if (swiglu && (a.w2.K != K || a.w2.Kp != K || a.w2.N != a.w.N)) return false;
    BatchTmaParams p;
    if (!q8_encode_weight_maps(a.w, &p.codes, &p.scales)) return false;
    if (swiglu) {
        if (!q8_encode_weight_maps(a.w2, &p.codes2, &p.scales2)) return false;
    } else {
        p.codes2 = p.codes; p.scales2 = p.scales;
    }
    const int rowsPerTile = swiglu ? 8 : 16;
    p.x = a.x + (size_t)m0 * a.ldx; p.ldx = a.ldx; p.gamma = a.gamma;
    p.K = K; p.N = a.w.N; p.M = rows;
    p.nTiles = (a.w.N + rowsPerTile - 1) / rowsPerTile;
    p.nGroups = (p.nTiles + kWarps - 1) / kWarps;
    p.nSlices = (K + kSlice - 1) / kSlice;
    p.tail.gamma = a.gamma; p.tail.eps = a.eps;
    p.tail.bias = a.bias; p.tail.bias2 = a.bias2;
    p.tail.residual = a.residual ? a.residual + (size_t)m0 * a.ldr : nullptr; p.tail.ldr = a.ldr;
    p.tail.out = a.out + (size_t)m0 * a.ldo; p.tail.ldo = a.ldo;
    p.tail.K = K; p.tail.N = a.w.N; p.tail.M = rows; p.tail.nSlices = p.nSlices;
    p.tail.ws = ws;
    p.tail.ssq = ws + (size_t)p.nSlices * p.nTiles * kBatchTileFloats;
    p.tail.tickets = nullptr;      // the reduce kernel needs none
    p.error = g_dev_error;
    p.trace = trace_slot();
    if (swiglu) {
        if (rows <= 8) launch_batch_tma<true, 1, kRingDepth>(p, s); else launch_batch_tma<true, 2, kRingDepth>(p, s);
    } else {
        if (rows <= 8) launch_batch_tma<false, 1, kRingDepth>(p, s); else launch_batch_tma<false, 2, kRingDepth>(p, s);
    }
    return true;
}

}  // namespace dj
