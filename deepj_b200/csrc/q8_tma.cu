// Q8 GEMV on the integer tensor pipe with warp-private cp.async rings — the decode
// hot kernel for up to two activation rows per pass.
//
// HBM-bound: 1.125 bytes per weight, read exactly once.  Two persistent CTAs of 8
// warps per SM walk 16-row weight tiles (two, so that the next kernel's CTAs can move
// in and prefetch while this kernel drains).  Inside a tile warp w owns the 64-k column
// pairs w, w+8, …; it streams its own 16 rows × 64 B (+ 32 scales) per pair into a
// private shared-memory ring with cp.async (three instructions per pair), DEPTH−1
// pairs ahead, so the bytes in flight per SM are set by the ring depth and not by
// registers, and no warp ever waits on another one until the tile epilogue.
// Each 32-k block is reduced by ONE mma.sync m16n8k32 (int8 × int8 → int32): the Q8
// codes ARE the A operand, no dequantisation instruction is spent on them.  The
// activations become the B operand as fixed point: every 32-k block of x is scaled
// by a power of two and rounded to 23 bits, which are split into three signed
// base-256 digits = three int8 columns; the integer block sums are exact, and
// 65536·S2 + 256·S1 + S0 times (weight scale × activation block scale) is accumulated
// in fp32 — the activation error is ≤ 2^-24 of the block's largest |x|, the same
// order as an fp32 FMA chain.  One MMA covers exactly one 32-k block of 16 weight
// rows, so the per-block scale semantics of the format are kept.  RMSNorm is fused
// into the activation staging; bias, residual and SiLU-gate into the epilogue.
//
// Measured dead ends, kept out of the code: a producer warp feeding a shared ring
// through mbarriers reached 1.0 TB/s with cp.async and 1.6 TB/s with 1-D
// cp.async.bulk row segments of 1 KB (per-copy cost of the bulk engine); fp16
// mma.sync with byte-permute dequant was no faster than the FMA kernel.
#include "kernels.h"
#include <cuda_fp16.h>
#include <cstdlib>

namespace dj {

int* g_dev_error = nullptr;     // device int, 0 = no bounded wait has ever expired

// Phase tracing (environment DEEPJ_CUDA_TRACE=1): every traced launch gets eight
// 64-bit slots in a device ring; CTA 0 stamps %globaltimer at its phase boundaries.
unsigned long long* g_trace = nullptr;
long long g_trace_launches = 0;
unsigned long long* trace_slot() {
    if (!g_trace) return nullptr;
    unsigned long long* p = g_trace + (size_t)(g_trace_launches % kTraceSlots) * 8;
    g_trace_launches++;
    return p;
}

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kRows = 16;                   // weight rows per tile (MMA M)
constexpr int kRowStride = 64;              // 64 code bytes per row per pair; 32-byte halves swizzled by row for conflict-free reads
constexpr int kSlotBytes = kRows * kRowStride + kRows * 2 * 4;    // + 32 scales
constexpr int kXsPad = 32;                  // bytes of padding per activation digit column
constexpr int kPreMax = 2;                  // items a warp prefetches before it waits for the previous kernel
constexpr int kColsPerRow = 3;              // digit columns per activation row in shared memory: d2, d1, d0

struct TmaParams {
    const float* x; int ldx;
    const float* gamma; float eps;
    const int8_t* codes; const float* scales; const float* bias;
    const int8_t* codes2; const float* scales2; const float* bias2;
    const float* residual; int ldr;
    float* out; int ldo;
    int K, N, Kp, nb, M;
    unsigned long long* trace;      // optional: six %globaltimer stamps of CTA 0 (phase tracing)
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ unsigned long long gtime() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void mma_s8_16832(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <bool SWIGLU, int DEPTH>
__global__ void __launch_bounds__(kThreads, 2) k_q8_gemv_i8(const TmaParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    // layout: rings [warps][DEPTH][kSlotBytes], digits int8 [3M][K+pad], block scales fp32 [M][K/32], partials [2][warps][16][8]
    const int ldxs = p.K + kXsPad;
    int8_t* xd = reinterpret_cast<int8_t*>(smem + (size_t)kWarps * DEPTH * kSlotBytes);
    float* xsc = reinterpret_cast<float*>(smem + (size_t)kWarps * DEPTH * kSlotBytes + (size_t)kColsPerRow * p.M * ldxs);
    float* s_part = xsc + (size_t)p.M * (p.K >> 5);
    __shared__ float s_red[kWarps];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int rowsPerTile = SWIGLU ? 8 : 16;
    const int nTiles = (p.N + rowsPerTile - 1) / rowsPerTile;
    const int nBlocks = p.K >> 5;
    const int nPairs = (nBlocks + 1) >> 1;      // an odd block count leaves the last pair half empty
    unsigned char* myring = smem + (size_t)warp * DEPTH * kSlotBytes;
    const bool tracing = p.trace != nullptr && blockIdx.x == 0 && tid == 0;
    if (tracing) p.trace[0] = gtime();

    // ── copy issue: per-lane constants are hoisted; rows past N are clamped to the last row
    // (their results are never written), so the copy path carries no predicates ──
    const uint32_t ring_s = smem_u32(myring);
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
    const float* sbase = ((SWIGLU && srow >= 8) ? p.scales2 : p.scales) + (lane & 1);
    const uint32_t sdst = (uint32_t)(kRows * kRowStride + lane * 4);

    // flat (tile, pair) sequence of this warp, with a cursor running DEPTH-1 items ahead
    int itile = blockIdx.x, ipi = warp, islot = 0;
    const int8_t* csrc[2]; const float* ssrc;
    auto set_issue_tile = [&]() {
#pragma unroll
        for (int j = 0; j < 2; j++) csrc[j] = cbase[j] + (size_t)min(itile * rowsPerTile + rloc[j], p.N - 1) * p.Kp;
        ssrc = sbase + (size_t)min(itile * rowsPerTile + sloc, p.N - 1) * p.nb;
    };
    set_issue_tile();
    auto issue_next = [&]() {
        if (itile < nTiles && ipi < nPairs) {
            const uint32_t dst = ring_s + (uint32_t)islot * kSlotBytes;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + dstoff[0]), "l"(csrc[0] + ipi * 64) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + dstoff[1]), "l"(csrc[1] + ipi * 64) : "memory");
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + sdst), "l"(ssrc + min(ipi * 2, nBlocks - 1 - (lane & 1))) : "memory");
            ipi += kWarps;
            if (ipi >= nPairs) { ipi = warp; itile += gridDim.x; set_issue_tile(); }
        }
        cp_async_commit();
        islot = islot + 1 == DEPTH ? 0 : islot + 1;
    };
    // Weights never depend on the previous kernel, so streaming starts before the wait — but
    // only kPre items deep: every byte in flight on this SM queues ahead of the activation
    // loads that follow the wait (latency = bytes in flight / bandwidth).
    constexpr int kPre = DEPTH - 1 < kPreMax ? DEPTH - 1 : kPreMax;
    const bool haveWork = warp < nPairs;
    if (haveWork) {
#pragma unroll
        for (int d = 0; d < kPre; d++) issue_next();
    }
    pdl_launch_dependents();
    if (tracing) p.trace[1] = gtime();
    pdl_wait();
    if (tracing) p.trace[2] = gtime();

    // activations → three int8 digit columns + one power-of-two scale per 32-k block (RMSNorm
    // fused).  A thread converts 16 consecutive values (half a block) per round.
    const int nHalf = p.K >> 4;
    for (int m = 0; m < p.M; m++) {
        const float* xrow = p.x + (size_t)m * p.ldx;
        const bool vec = ((reinterpret_cast<uintptr_t>(xrow) | (p.gamma ? reinterpret_cast<uintptr_t>(p.gamma) : 0)) & 15) == 0;
        float rms = 1.0f;
        const bool oneRound = nHalf <= kThreads;
        if (p.gamma && !oneRound) {
            // wide rows: the sum of squares needs its own pass
            float ss = 0.0f;
            for (int k = tid; k < p.K; k += kThreads) { float v = xrow[k]; ss = fmaf(v, v, ss); }
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            __syncthreads();
            if (lane == 0) s_red[warp] = ss;
            __syncthreads();
            ss = 0.0f;
#pragma unroll
            for (int q = 0; q < kWarps; q++) ss += s_red[q];
            rms = sqrtf(ss * (1.0f / (float)p.K) + p.eps);
        }
        int8_t* dcol = xd + (size_t)(kColsPerRow * m) * ldxs;
        for (int hb0 = 0; hb0 < nHalf; hb0 += kThreads) {
            const int hb = hb0 + tid;
            const bool on = hb < nHalf;
            float xv[16], gv[16];
            if (on) {
                if (vec) {
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        float4 v4 = reinterpret_cast<const float4*>(xrow + hb * 16)[j];
                        xv[4 * j] = v4.x; xv[4 * j + 1] = v4.y; xv[4 * j + 2] = v4.z; xv[4 * j + 3] = v4.w;
                        if (p.gamma) {
                            float4 g4 = reinterpret_cast<const float4*>(p.gamma + hb * 16)[j];
                            gv[4 * j] = g4.x; gv[4 * j + 1] = g4.y; gv[4 * j + 2] = g4.z; gv[4 * j + 3] = g4.w;
                        }
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 16; j++) { xv[j] = xrow[hb * 16 + j]; if (p.gamma) gv[j] = p.gamma[hb * 16 + j]; }
                }
            } else {
#pragma unroll
                for (int j = 0; j < 16; j++) { xv[j] = 0.0f; gv[j] = 1.0f; }
            }
            if (m == 0 && hb0 == 0 && haveWork) {
#pragma unroll
                for (int d = kPre; d < DEPTH - 1; d++) issue_next();      // now fill the ring behind the activation loads
            }
            if (p.gamma && oneRound) {
                float ss = 0.0f;
#pragma unroll
                for (int j = 0; j < 16; j++) ss = fmaf(xv[j], xv[j], ss);
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                __syncthreads();
                if (lane == 0) s_red[warp] = ss;
                __syncthreads();
                ss = 0.0f;
#pragma unroll
                for (int q = 0; q < kWarps; q++) ss += s_red[q];
                rms = sqrtf(ss * (1.0f / (float)p.K) + p.eps);      // RMSNorm1D.forward
            }
            float amax = 0.0f;
#pragma unroll
            for (int j = 0; j < 16; j++) {
                if (p.gamma) xv[j] = __fdiv_rn(xv[j], rms) * gv[j];
                amax = fmaxf(amax, fabsf(xv[j]));
            }
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));      // the other half of the 32-k block
            // s = 2^(exponent(amax)+2): |v|/s < 1/2, so the 23-bit fixed-point value fits three signed digits
            int sbits = 0x3f800000;
            if (amax > 0.0f && amax < 1e36f) sbits = (__float_as_int(amax) & 0x7f800000) + 0x01000000;
            const float mul = __int_as_float(0x7f000000 - sbits) * 8388608.0f;     // 2^23 / s, exact
            uint32_t w2[4], w1[4], w0[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                w2[j] = 0u; w1[j] = 0u; w0[j] = 0u;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int q = __float2int_rn(xv[4 * j + i] * mul);
                    const int e0 = ((q + 128) & 255) - 128;
                    const int q1 = (q - e0) >> 8;
                    const int e1 = ((q1 + 128) & 255) - 128;
                    const int e2 = (q1 - e1) >> 8;
                    w2[j] |= (uint32_t)(e2 & 255) << (8 * i);
                    w1[j] |= (uint32_t)(e1 & 255) << (8 * i);
                    w0[j] |= (uint32_t)(e0 & 255) << (8 * i);
                }
            }
            if (on) {
                *reinterpret_cast<uint4*>(dcol + hb * 16) = make_uint4(w2[0], w2[1], w2[2], w2[3]);
                *reinterpret_cast<uint4*>(dcol + ldxs + hb * 16) = make_uint4(w1[0], w1[1], w1[2], w1[3]);
                *reinterpret_cast<uint4*>(dcol + 2 * ldxs + hb * 16) = make_uint4(w0[0], w0[1], w0[2], w0[3]);
                if ((hb & 1) == 0) xsc[(size_t)m * nBlocks + (hb >> 1)] = __int_as_float(sbits) * (1.0f / 8388608.0f);
            }
        }
    }
    __syncthreads();
    if (tracing) p.trace[3] = gtime();

    // lane (g,t) feeds MMA column g: activation row g/4, digit g%4 (digit 3 does not exist)
    const bool hasCol = (g >> 2) < p.M && (g & 3) != 3;
    const unsigned char* xcol = reinterpret_cast<const unsigned char*>(xd) + (size_t)(hasCol ? kColsPerRow * (g >> 2) + (g & 3) : 0) * ldxs + t * 8;
    // the lane's two result columns 2t, 2t+1 belong to activation row t/2
    const float* myxsc = xsc + (size_t)((t >> 1) < p.M ? (t >> 1) : 0) * nBlocks;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    int cslot = 0, buf = 0;
    int aoff[2];
#pragma unroll
    for (int h = 0; h < 2; h++) aoff[h] = g * kRowStride + (h ^ ((g >> 1) & 1)) * 32 + t * 8;
    const int soff = kRows * kRowStride + g * 8;      // scales of row g: two floats; row g+8 is 64 bytes on
    for (int tile = blockIdx.x; tile < nTiles; tile += gridDim.x) {
        // epilogue operands are fetched now so that their latency hides behind the tile
        const int er = tid % rowsPerTile, em = tid / rowsPerTile, en = tile * rowsPerTile + er;
        float ebias = 0.0f, ebias2 = 0.0f, eres = 0.0f;
        if (em < p.M && en < p.N) {
            if (p.bias) ebias = p.bias[en];
            if (SWIGLU && p.bias2) ebias2 = p.bias2[en];
            if (!SWIGLU && p.residual) eres = p.residual[(size_t)em * p.ldr + en];
        }
        for (int pi = warp; pi < nPairs; pi += kWarps) {
            issue_next();
            cp_async_wait<DEPTH - 1>();
            __syncwarp();
            const unsigned char* slot = myring + (size_t)cslot * kSlotBytes;
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const uint2 a = *reinterpret_cast<const uint2*>(slot + aoff[h]);
                const uint2 d = *reinterpret_cast<const uint2*>(slot + aoff[h] + 8 * kRowStride);   // row g+8: same swizzle bit
                const float s0 = *reinterpret_cast<const float*>(slot + soff + h * 4);
                const float s1 = *reinterpret_cast<const float*>(slot + soff + 64 + h * 4);
                const int blk = pi * 2 + h;
                uint2 xb = make_uint2(0u, 0u);
                if (hasCol) xb = *reinterpret_cast<const uint2*>(xcol + blk * 32);
                int cc[4] = {0, 0, 0, 0};
                mma_s8_16832(cc, a.x, d.x, a.y, d.y, xb.x, xb.y);
                const float xs_ = blk < nBlocks ? myxsc[blk] : 0.0f;     // the empty half of an odd last pair adds nothing
                const float f0 = s0 * xs_, f1 = s1 * xs_;
                acc[0] = fmaf(f0, (float)cc[0], acc[0]);
                acc[1] = fmaf(f0, (float)cc[1], acc[1]);
                acc[2] = fmaf(f1, (float)cc[2], acc[2]);
                acc[3] = fmaf(f1, (float)cc[3], acc[3]);
            }
            __syncwarp();
            cslot = cslot + 1 == DEPTH ? 0 : cslot + 1;
        }
        if (tracing && tile == blockIdx.x) p.trace[4] = gtime();
        // ── tile epilogue: reduce the warps' column subsets, recombine the digits ──
        float* part = s_part + (size_t)buf * kWarps * 128;
        float* mine = part + warp * 128;
        mine[g * 8 + 2 * t] = acc[0];       mine[g * 8 + 2 * t + 1] = acc[1];
        mine[(g + 8) * 8 + 2 * t] = acc[2]; mine[(g + 8) * 8 + 2 * t + 1] = acc[3];
        acc[0] = acc[1] = acc[2] = acc[3] = 0.0f;
        __syncthreads();
        if (em < p.M && en < p.N) {
            float a2 = 0.0f, a1 = 0.0f, a0 = 0.0f, b2 = 0.0f, b1 = 0.0f, b0 = 0.0f;
#pragma unroll
            for (int q = 0; q < kWarps; q++) {
                const float* pr = part + q * 128 + er * 8 + 4 * em;      // MMA columns 4m .. 4m+2
                a2 += pr[0]; a1 += pr[1]; a0 += pr[2];
                if (SWIGLU) { b2 += pr[64]; b1 += pr[65]; b0 += pr[66]; }
            }
            float v = fmaf(a2, 65536.0f, fmaf(a1, 256.0f, a0));
            if (SWIGLU) {
                float u = fmaf(b2, 65536.0f, fmaf(b1, 256.0f, b0));
                if (p.bias) v += ebias;
                if (p.bias2) u += ebias2;
                float sig = 1.0f / (1.0f + expf(-v));
                p.out[(size_t)em * p.ldo + en] = (v * sig) * u;          // SiLU(gate) ⊙ up
            } else {
                if (p.bias) v += ebias;
                if (p.residual) v += eres;
                p.out[(size_t)em * p.ldo + en] = v;
            }
        }
        buf ^= 1;
    }
    cp_async_wait<0>();
    if (tracing) p.trace[5] = gtime();
}

size_t i8_smem_bytes(int K, int M, int depth) {
    return (size_t)kWarps * depth * kSlotBytes + (size_t)kColsPerRow * M * (K + kXsPad) + (size_t)M * (K / 32) * 4 +
           (size_t)2 * kWarps * 128 * 4;
}

template <bool SWIGLU, int DEPTH>
void launch_i8(const TmaParams& p, cudaStream_t s) {
    static bool attrSet = false;
    if (!attrSet) {
        DJ_CUDA_CHECK(cudaFuncSetAttribute(k_q8_gemv_i8<SWIGLU, DEPTH>, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024));
        attrSet = true;
    }
    int rowsPerTile = SWIGLU ? 8 : 16;
    int nTiles = (p.N + rowsPerTile - 1) / rowsPerTile;
    int cap = 2 * g_num_sms;
    int gx = nTiles < cap ? nTiles : cap;
    launch_k(k_q8_gemv_i8<SWIGLU, DEPTH>, dim3(gx), dim3(kThreads), i8_smem_bytes(p.K, p.M, DEPTH), s, true, p);
}

template <bool SWIGLU>
void launch_i8_depth(const TmaParams& p, int depth, cudaStream_t s) {
    switch (depth) {
        case 3: launch_i8<SWIGLU, 3>(p, s); break;
        case 4: launch_i8<SWIGLU, 4>(p, s); break;
        case 5: launch_i8<SWIGLU, 5>(p, s); break;
        case 6: launch_i8<SWIGLU, 6>(p, s); break;
        case 7: launch_i8<SWIGLU, 7>(p, s); break;
        case 8: launch_i8<SWIGLU, 8>(p, s); break;
        default: launch_i8<SWIGLU, 9>(p, s); break;
    }
}

}  // namespace

// Returns false when the shape is outside this kernel's domain (the caller falls
// back to the FMA kernel).  Two CTAs share an SM, so a CTA may use half of its
// shared memory: the ring takes what the activation digits leave.
bool launch_q8_linear_tma(const Q8LinearArgs& a, cudaStream_t s) {
    const int K = a.w.K;
    if (K % 32 != 0 || a.w.Kp != K) return false;
    const bool swiglu = a.w2.codes != nullptr;
    const size_t budget = 111 * 1024;
    if (i8_smem_bytes(K, 1, 3) > budget) return false;
    for (int m0 = 0; m0 < a.M;) {
        int rows = a.M - m0 < 2 ? a.M - m0 : 2;      // 8 MMA columns = 2 activation rows × (3 digits + 1 unused)
        while (rows > 1 && i8_smem_bytes(K, rows, 3) > budget) rows--;
        static int wantDepth = 0;
        if (wantDepth == 0) { const char* e = getenv("DEEPJ_CUDA_GEMV_DEPTH"); wantDepth = e ? atoi(e) : 5; if (wantDepth < 3) wantDepth = 3; if (wantDepth > 9) wantDepth = 9; }
        int depth = wantDepth;      // default: four items (4 KB) per warp in flight, 64 KB per SM
        while (depth > 3 && i8_smem_bytes(K, rows, depth) > budget) depth--;
        TmaParams p;
        p.x = a.x + (size_t)m0 * a.ldx; p.ldx = a.ldx; p.gamma = a.gamma; p.eps = a.eps;
        p.codes = a.w.codes; p.scales = a.w.scales; p.bias = a.bias;
        p.codes2 = a.w2.codes; p.scales2 = a.w2.scales; p.bias2 = a.bias2;
        p.residual = a.residual ? a.residual + (size_t)m0 * a.ldr : nullptr; p.ldr = a.ldr;
        p.out = a.out + (size_t)m0 * a.ldo; p.ldo = a.ldo;
        p.K = K; p.N = a.w.N; p.Kp = a.w.Kp; p.nb = a.w.nb; p.M = rows;
        p.trace = trace_slot();
        if (swiglu) launch_i8_depth<true>(p, depth, s); else launch_i8_depth<false>(p, depth, s);
        m0 += rows;
    }
    return true;
}

}  // namespace dj
