// Q8 linear for a small batch of activation rows (5 … 16 per launch) with cp.async rings and fp16 MMAs, for
// reduction lengths that are multiples of 32: the decode step of several concurrent sequences, and the short-prompt
// end of the operator sweep.  Reduction lengths that are multiples of 128 take the TMA / int8 kernel
// (q8_batch_tma.cu, ≈ 1.7 × faster at 16 bits of activation precision instead of 22); this one serves the rest.
//
// Still HBM-bound — every weight byte is read once per launch and used for all rows — so the
// streaming side is the GEMV's: warp-private cp.async rings of 16 weight rows × 64 codes (+ 32
// scales) per item.  The arithmetic is fp16 mma.sync m16n8k16 with fp32 accumulation:
//   * the int8 codes become fp16 exactly (sign flip, byte under the exponent 0x64, subtract
//     1152 — five instructions per four codes) and are the A operand;
//   * the activations are the B operand as fp16 hi + lo halves of x · 2^-e, e taken from the
//     largest |x| of the 512-k slice a work item covers: two MMAs per 32-k block and group of
//     eight rows, and `weight scale · block sum` is accumulated in fp32, so the per-block scale
//     semantics of the format are kept;
//   * K is cut into slices of 512: a work item is (group of 8 row tiles, slice), a CTA stages
//     only its slice of the activations, and each warp owns one 16-row tile of the group;
//   * partial sums of the slices meet in a global workspace: the WARP that arrives last at a
//     row tile (a ticket counter per tile) adds the slices in slice order — deterministic —
//     and runs the epilogue (RMSNorm scale, bias, residual, SiLU-gate).  No CTA-wide
//     barrier after the activations are staged: warps drift apart freely.
// RMSNorm: the halves are taken from x ⊙ γ and the row factor 1/rms is applied in the
// epilogue; Σx² of every 512-chunk of a row is left in the workspace by the CTAs that stage it.
#include "kernels.h"
#include "q8_common.cuh"
#include "q8_batch_tail.cuh"
#include <cuda_fp16.h>
#include <cstdlib>

namespace dj {
namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kRows = 16;
constexpr int kRowStride = 64;
constexpr int kSlotBytes = kRows * kRowStride + kRows * 2 * 4;
constexpr int kSlice = 512;                 // reduction length per work item = one warp pass over an activation row
constexpr int kLdx = kSlice * 2 + 64;       // bytes per fp16 activation column (64 mod 128: conflict-free 16-byte reads)
constexpr int kDepth = 6;                   // ring slots per warp
constexpr int kPre = 2;                     // of which fetched before the previous kernel has finished
constexpr int kMaxRows = kBatchMaxRows;
constexpr int kTileFloats = kBatchTileFloats;

struct BatchParams {
    const float* x; int ldx;
    const float* gamma; float eps;
    const int8_t* codes; const float* scales; const float* bias;
    const int8_t* codes2; const float* scales2; const float* bias2;
    const float* residual; int ldr;
    float* out; int ldo;
    int K, N, Kp, nb, M;
    int nSlices, nGroups, nTiles;
    float* ws;              // [nTiles · nSlices][kTileFloats] partial sums, then Σx² [⌈K/512⌉][16]
    float* ssq;
    int* tickets;           // [nTiles], zero between launches
    unsigned long long* trace;      // optional phase stamps of CTA 0 (see trace_slot)
};

__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// The same with a zero accumulator input: starts a block's sum without clearing registers first.
__device__ __forceinline__ void mma_f16_16816_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}
// Four int8 codes → two fp16x2 registers, exactly: flipping the sign bit gives u = code + 128, the
// byte under exponent 0x64 is the half 1024 + u, and 1152 comes off again.
__device__ __forceinline__ void codes_to_half2(uint32_t w, uint32_t& lo, uint32_t& hi) {
    const uint32_t u = w ^ 0x80808080u;
    uint32_t p0 = __byte_perm(u, 0x64646464u, 0x4140);      // {u.b0 | 0x64<<8, u.b1 | 0x64<<8}
    uint32_t p1 = __byte_perm(u, 0x64646464u, 0x4342);      // bytes 2 and 3
    const uint32_t k1152 = 0x64806480u;                     // half2(1152, 1152)
    asm("sub.f16x2 %0, %1, %2;" : "=r"(lo) : "r"(p0), "r"(k1152));
    asm("sub.f16x2 %0, %1, %2;" : "=r"(hi) : "r"(p1), "r"(k1152));
}
__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));      // first source → upper half
    return r;
}

template <bool SWIGLU, int NT>
__global__ void __launch_bounds__(kThreads, 2) k_q8_gemm_f16(const BatchParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    // layout: rings [warps][kDepth][kSlotBytes] | activation columns fp16 [8·NT][kLdx] (hi, lo per row) | row scales fp32 [4·NT]
    constexpr int kColsX = 8 * NT;
    unsigned char* xh = smem + (size_t)kWarps * kDepth * kSlotBytes;
    float* xscale = reinterpret_cast<float*>(xh + (size_t)kColsX * kLdx);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int nItems = p.nGroups * p.nSlices;
    unsigned char* myring = smem + (size_t)warp * kDepth * kSlotBytes;
    const uint32_t ring_s = smem_u32(myring);
    const int rowsPerTile = SWIGLU ? 8 : 16;
    const bool tracing = p.trace != nullptr && blockIdx.x == 0 && tid == 0;
    if (tracing) { p.trace[0] = gtime(); p.trace[6] = 0ull; }

    // ── copy issue (the GEMV's scheme): two 16-byte pieces and one scale per lane and pair ──
    uint32_t dstoff[2]; int rloc[2]; const int8_t* cbase[2];
#pragma unroll
    for (int j = 0; j < 2; j++) {
        const int q = lane + 32 * j, r = q >> 2, piece = q & 3;
        dstoff[j] = (uint32_t)(r * kRowStride + ((piece ^ (((r >> 1) & 1) << 1)) * 16));
        rloc[j] = SWIGLU ? (r & 7) : r;
        cbase[j] = ((SWIGLU && r >= 8) ? p.codes2 : p.codes) + piece * 16;
    }
    const int srow = lane >> 1;
    const int sloc = SWIGLU ? (srow & 7) : srow;
    const float* sbase = (SWIGLU && srow >= 8) ? p.scales2 : p.scales;
    const uint32_t sdst = (uint32_t)(kRows * kRowStride + lane * 4);

    // a warp whose tile lies past the last row still walks the sequence (clamped rows), it only skips the outputs
    int iitem = blockIdx.x, ipi = 0, islot = 0, ipairs = 0, ik0 = 0;
    const int8_t* csrc[2]; const float* ssrc;
    auto set_issue_item = [&]() {
        if (iitem >= nItems) return;
        const int slice = iitem % p.nSlices, grp = iitem / p.nSlices;
        const int row0 = (grp * kWarps + warp) * rowsPerTile;
        ik0 = slice * kSlice;
        ipairs = ((min(kSlice, p.K - ik0) >> 5) + 1) >> 1;
#pragma unroll
        for (int j = 0; j < 2; j++) csrc[j] = cbase[j] + (size_t)min(row0 + rloc[j], p.N - 1) * p.Kp + ik0;
        ssrc = sbase + (size_t)min(row0 + sloc, p.N - 1) * p.nb;
    };
    set_issue_item();
    auto issue_next = [&]() {
        if (iitem < nItems) {
            const uint32_t dst = ring_s + (uint32_t)islot * kSlotBytes;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + dstoff[0]), "l"(csrc[0] + ipi * 64) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + dstoff[1]), "l"(csrc[1] + ipi * 64) : "memory");
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + sdst), "l"(ssrc + min((ik0 >> 5) + ipi * 2 + (lane & 1), p.nb - 1)) : "memory");
            if (++ipi >= ipairs) { ipi = 0; iitem += gridDim.x; set_issue_item(); }
        }
        cp_async_commit();
        islot = islot + 1 == kDepth ? 0 : islot + 1;
    };
    for (int d = 0; d < kPre; d++) issue_next();
    pdl_launch_dependents();
    if (tracing) p.trace[1] = gtime();
    pdl_wait();
    if (tracing) p.trace[2] = gtime();
    for (int d = kPre; d < kDepth - 1; d++) issue_next();

    // columns of rows ≥ M stay zero
    for (int i = tid; i < kColsX * kLdx / 4; i += kThreads) reinterpret_cast<uint32_t*>(xh)[i] = 0u;
    if (tid < 4 * NT) xscale[tid] = 0.0f;

    // the lane's MMA column in n-tile j is 8j + g: activation row 4j + g/2, hi (g even) or lo (g odd) part;
    // its 8 reduction indices of a 32-k block are the 16 bytes at t·16 — the permutation the A side uses too
    const unsigned char* xcol0 = xh + (size_t)g * kLdx + t * 16;
    int aoff[2];
#pragma unroll
    for (int h = 0; h < 2; h++) aoff[h] = g * kRowStride + (h ^ ((g >> 1) & 1)) * 32 + t * 8;
    const int soff = kRows * kRowStride + g * 8;
    const int nChunksK = (p.K + kSlice - 1) / kSlice;

    const BatchTail tail = {p.gamma, p.eps, p.bias, p.bias2, p.residual, p.ldr, p.out, p.ldo, p.K, p.N, p.M, p.nSlices, p.ws, p.ssq, p.tickets};
    int staged = -1, cslot = 0;
    for (int item = blockIdx.x; item < nItems; item += gridDim.x) {
        const int slice = item % p.nSlices, grp = item / p.nSlices;
        const int k0 = slice * kSlice;
        const int sliceLen = min(kSlice, p.K - k0);
        const int nBlk = sliceLen >> 5;
        const int nPairs = (nBlk + 1) >> 1;
        if (slice != staged) {
            __syncthreads();            // every warp is done with the previous slice's columns (and with the clearing above)
            // one warp pass per activation row: 512 values → hi and lo halves of x · 2^-e, e from the slice's largest |x|
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
                    float amax = 0.0f;
                    if (p.gamma) {
                        float ss = 0.0f;
#pragma unroll
                        for (int j = 0; j < 16; j++) ss = fmaf(xv[u][j], xv[u][j], ss);
                        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                        if (lane == 0) p.ssq[slice * kMaxRows + m] = ss;      // every CTA that stages this slice writes the same bits
#pragma unroll
                        for (int j = 0; j < 16; j++) xv[u][j] *= gv[u][j];
                    }
#pragma unroll
                    for (int j = 0; j < 16; j++) amax = fmaxf(amax, fabsf(xv[u][j]));
                    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                    // 2^-e brings the largest value into [1024, 2048): the lo halves keep 2^-24 absolute steps far below it
                    int ebits = 0x3f800000;
                    if (amax > 0.0f && amax < 1e30f) ebits = (__float_as_int(amax) & 0x7f800000);
                    const float down = __int_as_float(0x7f000000 - ebits) * 1024.0f;    // 2^10 / 2^exponent(amax)
                    uint32_t hi[8], lo[8];
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const float a = xv[u][2 * j] * down, b = xv[u][2 * j + 1] * down;
                        hi[j] = pack_half2(a, b);
                        const float2 back = __half22float2(*reinterpret_cast<const __half2*>(&hi[j]));
                        lo[j] = pack_half2(a - back.x, b - back.y);
                    }
                    if (on[u]) {
                        uint4* dh = reinterpret_cast<uint4*>(xh + (size_t)(2 * m) * kLdx + lane * 32);
                        uint4* dl = reinterpret_cast<uint4*>(xh + (size_t)(2 * m + 1) * kLdx + lane * 32);
                        dh[0] = make_uint4(hi[0], hi[1], hi[2], hi[3]); dh[1] = make_uint4(hi[4], hi[5], hi[6], hi[7]);
                        dl[0] = make_uint4(lo[0], lo[1], lo[2], lo[3]); dl[1] = make_uint4(lo[4], lo[5], lo[6], lo[7]);
                    }
                    if (lane == 0) xscale[m] = __int_as_float(ebits) * (1.0f / 1024.0f);
                }
            }
            staged = slice;
            __syncthreads();
            if (tracing && item == blockIdx.x) p.trace[3] = gtime();
        }

        float acc[NT][4];
#pragma unroll
        for (int j = 0; j < NT; j++) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f; }
        for (int pi = 0; pi < nPairs; pi++) {
            issue_next();
            cp_async_wait<kDepth - 1>();
            __syncwarp();
            const unsigned char* slot = myring + (size_t)cslot * kSlotBytes;
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const int blk = pi * 2 + h;
                if (blk < nBlk) {
                    const uint2 a = *reinterpret_cast<const uint2*>(slot + aoff[h]);                    // row g: 8 codes
                    const uint2 d = *reinterpret_cast<const uint2*>(slot + aoff[h] + 8 * kRowStride);   // row g+8
                    const float s0 = *reinterpret_cast<const float*>(slot + soff + h * 4);
                    const float s1 = *reinterpret_cast<const float*>(slot + soff + 64 + h * 4);
                    uint32_t ag[4], ad[4];
                    codes_to_half2(a.x, ag[0], ag[1]); codes_to_half2(a.y, ag[2], ag[3]);
                    codes_to_half2(d.x, ad[0], ad[1]); codes_to_half2(d.y, ad[2], ad[3]);
                    // all fragment loads, then all MMAs of the first k-step, then the second: the n-tiles'
                    // chains are independent and are laid out so that they overlap
                    uint4 xb[NT];
#pragma unroll
                    for (int j = 0; j < NT; j++) xb[j] = *reinterpret_cast<const uint4*>(xcol0 + (size_t)j * 8 * kLdx + blk * 64);
                    float c[NT][4], e[NT][4];
#pragma unroll
                    for (int j = 0; j < NT; j++) mma_f16_16816_first(c[j], ag[0], ad[0], ag[1], ad[1], xb[j].x, xb[j].y);
#pragma unroll
                    for (int j = 0; j < NT; j++) mma_f16_16816_first(e[j], ag[2], ad[2], ag[3], ad[3], xb[j].z, xb[j].w);
#pragma unroll
                    for (int j = 0; j < NT; j++) {
                        acc[j][0] = fmaf(s0, c[j][0] + e[j][0], acc[j][0]);
                        acc[j][1] = fmaf(s0, c[j][1] + e[j][1], acc[j][1]);
                        acc[j][2] = fmaf(s1, c[j][2] + e[j][2], acc[j][2]);
                        acc[j][3] = fmaf(s1, c[j][3] + e[j][3], acc[j][3]);
                    }
                }
            }
            __syncwarp();
            cslot = cslot + 1 == kDepth ? 0 : cslot + 1;
        }
        if (tracing && item == blockIdx.x) p.trace[4] = gtime();
        const int tile = grp * kWarps + warp;
        if (tile >= p.nTiles) continue;                     // warp-uniform: nothing to deliver
        // the lane's two columns of n-tile j are the hi and lo parts of activation row 4j + t
        float* rec = p.ws + ((size_t)tile * p.nSlices + slice) * kTileFloats;
#pragma unroll
        for (int j = 0; j < NT; j++) {
            const int m = 4 * j + t;
            if (m < p.M) {
                const float up = xscale[m];
                rec[m * 16 + g] = (acc[j][0] + acc[j][1]) * up;
                rec[m * 16 + g + 8] = (acc[j][2] + acc[j][3]) * up;
            }
        }
        batch_finish_tile<SWIGLU>(tail, tile, nChunksK);
    }
    cp_async_wait<0>();
    if (tracing) p.trace[5] = gtime();
    if (p.trace != nullptr && lane == 0) atomicMax(p.trace + 6, gtime());
}

template <int NT> constexpr size_t batch_smem() {
    return (size_t)kWarps * kDepth * kSlotBytes + (size_t)8 * NT * kLdx + (size_t)4 * NT * 4;
}

template <bool SWIGLU, int NT>
void launch_batch(const BatchParams& p, cudaStream_t s) {
    static bool attrSet = false;
    if (!attrSet) {
        DJ_CUDA_CHECK(cudaFuncSetAttribute(k_q8_gemm_f16<SWIGLU, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)batch_smem<NT>()));
        attrSet = true;
    }
    const int nItems = p.nGroups * p.nSlices;
    int cap = 2 * g_num_sms;
    if (p.nSlices <= cap) cap -= cap % p.nSlices;       // a CTA then keeps its slice from item to item
    const int gx = nItems < cap ? nItems : cap;
    launch_k(k_q8_gemm_f16<SWIGLU, NT>, dim3(gx), dim3(kThreads), batch_smem<NT>(), s, true, p);
}

}  // namespace

// Workspace: the tile records of every slice, then Σx² per slice and activation row.
size_t q8_batch_ws_floats(int K, int N, bool swiglu) {
    const int nSlices = (K + kSlice - 1) / kSlice;
    const int nTiles = (N + (swiglu ? 8 : 16) - 1) / (swiglu ? 8 : 16);
    return (size_t)nSlices * nTiles * kTileFloats + (size_t)nSlices * kMaxRows;
}

// Rows m0 … m0+rows−1 (rows ≤ 16) of a Q8 linear / SwiGLU.  Returns false when the shape is outside
// this kernel's domain.
bool launch_q8_linear_batch(const Q8LinearArgs& a, int m0, int rows, float* ws, int* tickets, cudaStream_t s) {
    const int K = a.w.K;
    if (K % 32 != 0 || a.w.Kp != K || rows < 1 || rows > kMaxRows) return false;
    const bool swiglu = a.w2.codes != nullptr;
    BatchParams p;
    p.x = a.x + (size_t)m0 * a.ldx; p.ldx = a.ldx; p.gamma = a.gamma; p.eps = a.eps;
    p.codes = a.w.codes; p.scales = a.w.scales; p.bias = a.bias;
    p.codes2 = a.w2.codes; p.scales2 = a.w2.scales; p.bias2 = a.bias2;
    p.residual = a.residual ? a.residual + (size_t)m0 * a.ldr : nullptr; p.ldr = a.ldr;
    p.out = a.out + (size_t)m0 * a.ldo; p.ldo = a.ldo;
    p.K = K; p.N = a.w.N; p.Kp = a.w.Kp; p.nb = a.w.nb; p.M = rows;
    const int rowsPerTile = swiglu ? 8 : 16;
    p.nTiles = (a.w.N + rowsPerTile - 1) / rowsPerTile;
    p.nGroups = (p.nTiles + kWarps - 1) / kWarps;
    p.nSlices = (K + kSlice - 1) / kSlice;
    if (p.nTiles > kAttnTickets / 2) return false;
    p.ws = ws;
    p.ssq = ws + (size_t)p.nSlices * p.nTiles * kTileFloats;
    p.tickets = tickets + kAttnTickets / 2;
    p.trace = trace_slot();
    const int nt = rows <= 4 ? 1 : rows <= 8 ? 2 : 4;      // rows ≤ 4 only as the tail of a longer batch
    if (swiglu) {
        if (nt == 1) launch_batch<true, 1>(p, s); else if (nt == 2) launch_batch<true, 2>(p, s); else launch_batch<true, 4>(p, s);
    } else {
        if (nt == 1) launch_batch<false, 1>(p, s); else if (nt == 2) launch_batch<false, 2>(p, s); else launch_batch<false, 4>(p, s);
    }
    return true;
}

}  // namespace dj
