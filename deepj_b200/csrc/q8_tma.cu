// Q8 GEMV, bulk-copy (TMA) pipelined, integer tensor-core dot products — the decode
// hot kernel for up to two activation rows per pass.
//
// HBM-bound: 1.125 bytes per weight, read exactly once.  One persistent CTA per SM.
// A producer warp streams the weights into a ring of shared-memory stages with
// cp.async (16 bytes per lane, 512 contiguous bytes per instruction, completion
// counted on an mbarrier), so the bytes in flight per SM are set by the ring depth,
// not by registers.  (1-D cp.async.bulk copies of 1 KB row segments were measured at
// a quarter of this: the per-copy cost of the bulk engine dominates at that size.)  Sixteen consumer warps reduce each stage with mma.sync m16n8k32
// (int8 × int8 → int32): the Q8 codes ARE the A operand, no dequantisation
// instruction is spent on them.  The activations become the B operand as fixed
// point: every 32-k block of x is scaled by a power of two and rounded to 23 bits,
// which are split into three signed base-256 digits = three int8 columns; the
// integer block sums are exact, and 65536·S2 + 256·S1 + S0 times (weight scale ×
// activation block scale) is accumulated in fp32 — the activation error is ≤ 2^-24 of
// the block's largest |x|, the same order as an fp32 FMA chain.  One MMA covers
// exactly one 32-k block of 16 weight rows, so the per-block scale semantics of the
// format are kept.  RMSNorm is fused into the activation staging; bias, residual
// and SiLU-gate into the epilogue.
//
// Every mbarrier wait is bounded: when the bound is hit the CTA records an error
// code in device memory and stops computing, so a fault can never turn into a hang.
#include "kernels.h"
#include <cuda_fp16.h>

namespace dj {

int* g_dev_error = nullptr;     // device int, 0 = no bounded wait has ever expired

namespace {

constexpr int kConsumerWarps = 16;
constexpr int kThreads = (kConsumerWarps + 1) * 32;     // + one producer warp
constexpr int kRows = 16;                               // weight rows per stage (MMA M)
constexpr int kChunk = 1024;                            // k per stage (bytes per row)
constexpr int kRowStride = kChunk + 32;                 // +32 B: conflict-free 8-byte reads across rows
constexpr int kScaleBytes = kChunk / 32 * 4;            // 128 B of scales per row per stage
constexpr int kStageBytes = kRows * kRowStride + kRows * kScaleBytes;
constexpr int kXsPad = 32;                               // bytes of padding per activation digit column
constexpr int kColsPerRow = 4;                          // digit columns per activation row: d2, d1, d0, (unused)
constexpr unsigned kSpinLimit = 1u << 22;

struct TmaParams {
    const float* x; int ldx;
    const float* gamma; float eps;
    const int8_t* codes; const float* scales; const float* bias;
    const int8_t* codes2; const float* scales2; const float* bias2;
    const float* residual; int ldr;
    float* out; int ldo;
    int K, N, Kp, nb, M, stages;
    int* error;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait for the phase with the given parity; false when the bound expired.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity) {
    for (unsigned i = 0; i < kSpinLimit; i++) {
        unsigned ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
// The barrier receives one arrival from this thread once all its earlier cp.async have landed.
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void mma_s8_16832(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <bool SWIGLU>
__global__ void __launch_bounds__(kThreads, 1) k_q8_gemv_tma(const TmaParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    // layout: [stages × kStageBytes] ring | digits int8 [4M][K+pad] | block scales fp32 [M][K/32] | partials [2][16][16][8] fp32
    unsigned char* ring = smem;
    const int ldxs = p.K + kXsPad;
    int8_t* xd = reinterpret_cast<int8_t*>(smem + (size_t)p.stages * kStageBytes);
    float* xsc = reinterpret_cast<float*>(smem + (size_t)p.stages * kStageBytes + (size_t)kColsPerRow * p.M * ldxs);
    float* s_part = xsc + (size_t)p.M * (p.K >> 5);
    __shared__ __align__(8) uint64_t s_full[8], s_empty[8];
    __shared__ float s_red[kConsumerWarps];
    __shared__ volatile int s_abort;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int rowsPerTile = SWIGLU ? 8 : 16;
    const int nTiles = (p.N + rowsPerTile - 1) / rowsPerTile;
    const int nChunks = (p.K + kChunk - 1) / kChunk;

    if (tid == 0) {
        for (int s = 0; s < p.stages; s++) { mbar_init(&s_full[s], 32); mbar_init(&s_empty[s], kConsumerWarps); }
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == kConsumerWarps) {
        // ───────────── producer warp: weights never depend on the previous kernel ─────────────
        pdl_launch_dependents();
        int it = 0;
        for (int tile = blockIdx.x; tile < nTiles; tile += gridDim.x) {
            for (int c = 0; c < nChunks; c++, it++) {
                const int s = it % p.stages;
                const unsigned round = (unsigned)(it / p.stages);
                if (round > 0) {
                    bool ok = true;
                    if (lane == 0) ok = mbar_wait(&s_empty[s], (round - 1) & 1);
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) { if (lane == 0) { atomicExch(p.error, 1); s_abort = 1; } return; }
                }
                const int k0 = c * kChunk;
                const int kbytes = min(kChunk, p.K - k0);
                const int sbytes = kbytes / 32 * 4;
                unsigned char* stage = ring + (size_t)s * kStageBytes;
                // codes: 16 rows × kbytes, 512 contiguous bytes of one row per warp instruction
                for (int r = 0; r < kRows; r++) {
                    int row; const int8_t* cbase;
                    if (SWIGLU) { row = tile * 8 + (r & 7); cbase = r < 8 ? p.codes : p.codes2; }
                    else { row = tile * 16 + r; cbase = p.codes; }
                    if (row >= p.N) continue;
                    const int8_t* src = cbase + (size_t)row * p.Kp + k0;
                    unsigned char* dst = stage + (size_t)r * kRowStride;
                    for (int off = lane * 16; off < kbytes; off += 512) cp_async16(dst + off, src + off);
                }
                // scales: four rows per warp instruction
                for (int r4 = 0; r4 < kRows; r4 += 4) {
                    const int r = r4 + (lane >> 3), off = (lane & 7) * 16;
                    int row; const float* sbase;
                    if (SWIGLU) { row = tile * 8 + (r & 7); sbase = r < 8 ? p.scales : p.scales2; }
                    else { row = tile * 16 + r; sbase = p.scales; }
                    if (row < p.N && off < sbytes)
                        cp_async16(stage + (size_t)kRows * kRowStride + (size_t)r * kScaleBytes + off,
                                   reinterpret_cast<const unsigned char*>(sbase + (size_t)row * p.nb + (k0 >> 5)) + off);
                }
                cp_async_arrive(&s_full[s]);
            }
        }
        return;
    }

    // ───────────── consumer warps ─────────────
    const int g = lane >> 2, t = lane & 3;
    const int nBlocks = p.K >> 5;
    pdl_wait();
    // activations → three int8 digit columns + one power-of-two scale per 32-k block (RMSNorm fused)
    for (int m = 0; m < p.M; m++) {
        const float* xrow = p.x + (size_t)m * p.ldx;
        float rms = 1.0f;
        if (p.gamma) {
            float ss = 0.0f;
            for (int k = tid; k < p.K; k += kConsumerWarps * 32) { float v = xrow[k]; ss = fmaf(v, v, ss); }
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            consumer_sync();
            if (lane == 0) s_red[warp] = ss;
            consumer_sync();
            ss = 0.0f;
#pragma unroll
            for (int q = 0; q < kConsumerWarps; q++) ss += s_red[q];
            rms = sqrtf(ss * (1.0f / (float)p.K) + p.eps);      // RMSNorm1D.forward
        }
        int8_t* d2 = xd + (size_t)(kColsPerRow * m) * ldxs;
        int8_t* d1 = d2 + ldxs;
        int8_t* d0 = d1 + ldxs;
        for (int blk = warp; blk < nBlocks; blk += kConsumerWarps) {
            const int k = blk * 32 + lane;
            float v = xrow[k];
            if (p.gamma) v = __fdiv_rn(v, rms) * p.gamma[k];
            float amax = fabsf(v);
            for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            // s = 2^(exponent(amax)+2): |v|/s < 1/2, so the 23-bit fixed-point value fits three signed digits
            float sblk = 1.0f;
            if (amax > 0.0f && amax < 1e36f) sblk = __int_as_float((__float_as_int(amax) & 0x7f800000) + 0x01000000);
            int q = __float2int_rn(v * (1.0f / sblk) * 8388608.0f);
            int e0 = ((q + 128) & 255) - 128;
            int q1 = (q - e0) >> 8;
            int e1 = ((q1 + 128) & 255) - 128;
            int e2 = (q1 - e1) >> 8;
            d2[k] = (int8_t)e2; d1[k] = (int8_t)e1; d0[k] = (int8_t)e0;
            if (lane == 0) xsc[(size_t)m * nBlocks + blk] = sblk * (1.0f / 8388608.0f);
        }
    }
    consumer_sync();

    // lane (g,t) feeds MMA column g: activation row g/4, digit g%4 (digit 3 does not exist)
    const bool hasCol = (g >> 2) < p.M && (g & 3) != 3;
    const unsigned char* xcol = reinterpret_cast<const unsigned char*>(xd) + (size_t)(hasCol ? g : 0) * ldxs + t * 8;
    // the lane's two result columns 2t, 2t+1 belong to activation row t/2
    const float* myxsc = xsc + (size_t)((t >> 1) < p.M ? (t >> 1) : 0) * nBlocks;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    int it = 0, buf = 0;
    bool dead = false;
    for (int tile = blockIdx.x; tile < nTiles; tile += gridDim.x) {
        for (int c = 0; c < nChunks; c++, it++) {
            const int s = it % p.stages;
            const unsigned round = (unsigned)(it / p.stages);
            // A warp whose wait expired stops computing but keeps walking the loop, so
            // the tile barriers of the other consumer warps still match.
            if (!dead) {
                bool ok = true;
                if (lane == 0) ok = !s_abort && mbar_wait(&s_full[s], round & 1);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) { dead = true; if (lane == 0) { atomicExch(p.error, 2); s_abort = 1; } }
            }
            if (dead) continue;
            const int k0 = c * kChunk;
            const int blocksHere = min(kChunk, p.K - k0) >> 5;
            const unsigned char* stage = ring + (size_t)s * kStageBytes;
            const unsigned char* r0 = stage + (size_t)g * kRowStride + t * 8;
            const unsigned char* r1 = stage + (size_t)(g + 8) * kRowStride + t * 8;
            const float* sc0 = reinterpret_cast<const float*>(stage + (size_t)kRows * kRowStride + (size_t)g * kScaleBytes);
            const float* sc1 = reinterpret_cast<const float*>(stage + (size_t)kRows * kRowStride + (size_t)(g + 8) * kScaleBytes);
            // rows beyond N were not copied: their stage bytes are stale, mask them
            const int row0 = tile * rowsPerTile + g;
            const bool v0ok = row0 < p.N, v1ok = SWIGLU ? v0ok : (row0 + 8 < p.N);
#pragma unroll 2
            for (int b = warp; b < blocksHere; b += kConsumerWarps) {
                uint2 a = *reinterpret_cast<const uint2*>(r0 + b * 32);
                uint2 d = *reinterpret_cast<const uint2*>(r1 + b * 32);
                float s0 = sc0[b], s1 = sc1[b];
                if (!v0ok) { a = make_uint2(0u, 0u); s0 = 0.0f; }
                if (!v1ok) { d = make_uint2(0u, 0u); s1 = 0.0f; }
                uint2 xb = make_uint2(0u, 0u);
                if (hasCol) xb = *reinterpret_cast<const uint2*>(xcol + k0 + b * 32);
                int cc[4] = {0, 0, 0, 0};
                mma_s8_16832(cc, a.x, d.x, a.y, d.y, xb.x, xb.y);
                const float xs_ = myxsc[(k0 >> 5) + b];
                const float f0 = s0 * xs_, f1 = s1 * xs_;
                acc[0] = fmaf(f0, (float)cc[0], acc[0]);
                acc[1] = fmaf(f0, (float)cc[1], acc[1]);
                acc[2] = fmaf(f1, (float)cc[2], acc[2]);
                acc[3] = fmaf(f1, (float)cc[3], acc[3]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_empty[s]);
        }
        // ── tile epilogue: reduce the warps' block subsets, recombine the digits ──
        float* part = s_part + (size_t)buf * kConsumerWarps * 128;
        float* mine = part + warp * 128;
        mine[g * 8 + 2 * t] = acc[0];       mine[g * 8 + 2 * t + 1] = acc[1];
        mine[(g + 8) * 8 + 2 * t] = acc[2]; mine[(g + 8) * 8 + 2 * t + 1] = acc[3];
        acc[0] = acc[1] = acc[2] = acc[3] = 0.0f;
        consumer_sync();
        const int r = tid % rowsPerTile, m = tid / rowsPerTile;
        if (m < p.M) {
            const int n = tile * rowsPerTile + r;
            if (n < p.N) {
                float a2 = 0.0f, a1 = 0.0f, a0 = 0.0f, b2 = 0.0f, b1 = 0.0f, b0 = 0.0f;
#pragma unroll
                for (int q = 0; q < kConsumerWarps; q++) {
                    const float* pr = part + q * 128 + r * 8 + kColsPerRow * m;
                    a2 += pr[0]; a1 += pr[1]; a0 += pr[2];
                    if (SWIGLU) { b2 += pr[64]; b1 += pr[65]; b0 += pr[66]; }
                }
                float v = fmaf(a2, 65536.0f, fmaf(a1, 256.0f, a0));
                if (SWIGLU) {
                    float u = fmaf(b2, 65536.0f, fmaf(b1, 256.0f, b0));
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
        buf ^= 1;
    }
}

size_t tma_smem_bytes(int K, int M, int stages) {
    return (size_t)stages * kStageBytes + (size_t)kColsPerRow * M * (K + kXsPad) + (size_t)M * (K / 32) * 4 +
           (size_t)2 * kConsumerWarps * 128 * 4;
}

template <bool SWIGLU>
void launch_tma(const TmaParams& p, cudaStream_t s) {
    static bool attrSet = false;
    if (!attrSet) {
        DJ_CUDA_CHECK(cudaFuncSetAttribute(k_q8_gemv_tma<SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
        attrSet = true;
    }
    int rowsPerTile = SWIGLU ? 8 : 16;
    int nTiles = (p.N + rowsPerTile - 1) / rowsPerTile;
    int gx = nTiles < g_num_sms ? nTiles : g_num_sms;
    launch_k(k_q8_gemv_tma<SWIGLU>, dim3(gx), dim3(kThreads), tma_smem_bytes(p.K, p.M, p.stages), s, true, p);
}

}  // namespace

// Returns false when the shape is outside this kernel's domain (the caller falls
// back to the register-pipelined kernels).
bool launch_q8_linear_tma(const Q8LinearArgs& a, cudaStream_t s) {
    const int K = a.w.K;
    if (K % 256 != 0 || a.w.Kp != K || g_dev_error == nullptr) return false;
    const bool swiglu = a.w2.codes != nullptr;
    const size_t budget = 200 * 1024;
    if (tma_smem_bytes(K, 1, 3) > budget) return false;
    for (int m0 = 0; m0 < a.M;) {
        int rows = a.M - m0 < 2 ? a.M - m0 : 2;      // 8 MMA columns = 2 activation rows × (3 digits + 1 unused)
        while (rows > 1 && tma_smem_bytes(K, rows, 3) > budget) rows--;
        int stages = 8;
        while (stages > 3 && tma_smem_bytes(K, rows, stages) > budget) stages--;
        TmaParams p;
        p.x = a.x + (size_t)m0 * a.ldx; p.ldx = a.ldx; p.gamma = a.gamma; p.eps = a.eps;
        p.codes = a.w.codes; p.scales = a.w.scales; p.bias = a.bias;
        p.codes2 = a.w2.codes; p.scales2 = a.w2.scales; p.bias2 = a.bias2;
        p.residual = a.residual ? a.residual + (size_t)m0 * a.ldr : nullptr; p.ldr = a.ldr;
        p.out = a.out + (size_t)m0 * a.ldo; p.ldo = a.ldo;
        p.K = K; p.N = a.w.N; p.Kp = a.w.Kp; p.nb = a.w.nb; p.M = rows; p.stages = stages;
        p.error = g_dev_error;
        if (swiglu) launch_tma<true>(p, s); else launch_tma<false>(p, s);
        m0 += rows;
    }
    return true;
}

}  // namespace dj
