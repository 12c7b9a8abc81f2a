// Q8 GEMV on the integer tensor pipe with warp-private cp.async rings — up to four activation rows
// per pass, for reduction lengths that are multiples of 32.  Reduction lengths that are multiples of 128
// take the TMA kernel (q8_gemv_tma.cu, same arithmetic); this one serves the rest (tensor maps want
// 16-byte row pitches, i.e. K/32 scales per row a multiple of 4) and row counts whose digits do not fit
// beside the TMA kernel's ring.
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
#include "kernels.h"
#include "q8_common.cuh"
#include "q8_stage.cuh"

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

constexpr int kWarps = kGemvWarps;
constexpr int kThreads = kGemvThreads;
constexpr int kRows = 16;                   // weight rows per tile (MMA M)
constexpr int kRowStride = 64;              // 64 code bytes per row per pair; 32-byte halves swizzled by row for conflict-free reads
constexpr int kSlotBytes = kRows * kRowStride + kRows * 2 * 4;    // + 32 scales
constexpr int kXsPad = kGemvXsPad;
constexpr int kPreMax = 2;                  // items a warp prefetches before it waits for the previous kernel
constexpr int kColsPerRow = kGemvColsPerRow;

struct GemvI8Params {
    const float* x; int ldx;
    const float* gamma; float eps;
    const float* beta; int act;     // GPT instantiation only: LayerNorm shift (null = RMSNorm / none) and 1 = GELU after the bias
    const int8_t* codes; const float* scales; const float* bias;
    const int8_t* codes2; const float* scales2; const float* bias2;
    const float* residual; int ldr;
    float* out; int ldo;
    int K, N, Kp, nb, M;
    int pre;                        // ring items a warp fetches before it waits for the previous kernel
    int mid;                        // ring items in flight while the activations are staged; the rest of the ring fills afterwards
    unsigned long long* trace;      // optional: six %globaltimer stamps of CTA 0 (phase tracing)
};


constexpr int kStageRounds = kGemvStageRounds;

// GPT = true adds LayerNorm1D (norm/LayerNorm1D.java:34-71: mean, biased variance, (x − mean)/√(var + eps)·γ + β)
// to the staging and GELU to the epilogue; the Llama / DeepSeek instantiation carries neither.
// NM = 2 takes three or four activation rows in one pass over the weights: a second MMA per block whose eight
// columns are the digits of rows 2 and 3.
template <bool SWIGLU, int DEPTH, bool GPT, int NM>
__global__ void __launch_bounds__(kThreads, 2) k_q8_gemv_i8(const GemvI8Params p) {
    extern __shared__ __align__(128) unsigned char smem[];
    // layout: rings [warps][DEPTH][kSlotBytes], digits int8 [3M][K+pad], block scales fp32 [M][K/32], partials [2][warps][NM][16][8]
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
    if (tracing) { p.trace[0] = gtime(); p.trace[6] = 0ull; }

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
    const int kPre = p.pre < DEPTH - 1 ? p.pre : DEPTH - 1;
    const int kMid = p.mid < DEPTH - 1 ? (p.mid > kPre ? p.mid : kPre) : DEPTH - 1;
    const bool haveWork = warp < nPairs;
    if (haveWork) {
        for (int d = 0; d < kPre; d++) issue_next();
    }
    pdl_launch_dependents();
    if (tracing) p.trace[1] = gtime();
    // the RMSNorm gain is a weight as well: fetch it before the wait when one round covers the row
    const int nHalf = p.K >> 4;
    const int rounds = (nHalf + kThreads - 1) / kThreads;
    const bool gammaEarly = p.gamma != nullptr && rounds == 1;
    float gpre[16];
#pragma unroll
    for (int j = 0; j < 16; j++) gpre[j] = 1.0f;
    if (gammaEarly && tid < nHalf) load16(p.gamma + tid * 16, (reinterpret_cast<uintptr_t>(p.gamma) & 15) == 0, gpre);
    pdl_wait();
    if (tracing) p.trace[2] = gtime();

    // activations → three int8 digit columns + one power-of-two scale per 32-k block (norm fused); more of the
    // ring is queued behind the first row's loads
    gemv_stage_rows<GPT>(p.x, p.ldx, p.gamma, p.beta, p.eps, p.K, p.M, xd, ldxs, xsc, s_red, gpre, gammaEarly, [&]() {
        if (haveWork) {
            for (int d = kPre; d < kMid; d++) issue_next();
        }
    });
    __syncthreads();
    if (haveWork) {
        for (int d = kMid; d < DEPTH - 1; d++) issue_next();      // the rest of the ring: nothing latency-critical queues behind it now
    }
    if (tracing) p.trace[3] = gtime();

    // lane (g,t) feeds column g of MMA q: activation row 2q + g/4, digit g%4 (digit 3 does not exist)
    bool hasCol[NM]; const unsigned char* xcol[NM]; const float* myxsc[NM];
    float acc[NM][4];
#pragma unroll
    for (int q = 0; q < NM; q++) {
        const int mrow = 2 * q + (g >> 2);
        hasCol[q] = mrow < p.M && (g & 3) != 3;
        xcol[q] = reinterpret_cast<const unsigned char*>(xd) + (size_t)(hasCol[q] ? kColsPerRow * mrow + (g & 3) : 0) * ldxs + t * 8;
        // the lane's two result columns 2t, 2t+1 belong to activation row 2q + t/2
        const int rrow = 2 * q + (t >> 1);
        myxsc[q] = xsc + (size_t)(rrow < p.M ? rrow : 0) * nBlocks;
        acc[q][0] = acc[q][1] = acc[q][2] = acc[q][3] = 0.0f;
    }
    int cslot = 0, buf = 0;
    int aoff[2];
#pragma unroll
    for (int h = 0; h < 2; h++) aoff[h] = g * kRowStride + (h ^ ((g >> 1) & 1)) * 32 + t * 8;
    const int soff = kRows * kRowStride + g * 8;      // scales of row g: two floats; row g+8 is 64 bytes on
    for (int tile = blockIdx.x; tile < nTiles; tile += gridDim.x) {
        // epilogue operands are fetched now so that their latency hides behind the tile
        const GemvEpilogueOperands eo = gemv_epilogue_fetch<SWIGLU>(tile, p.M, p.N, p.bias, p.bias2, p.residual, p.ldr);
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
#pragma unroll
                for (int q = 0; q < NM; q++) {
                    uint2 xb = make_uint2(0u, 0u);
                    if (hasCol[q]) xb = *reinterpret_cast<const uint2*>(xcol[q] + blk * 32);
                    int cc[4] = {0, 0, 0, 0};
                    mma_s8_16832(cc, a.x, d.x, a.y, d.y, xb.x, xb.y);
                    const float xs_ = blk < nBlocks ? myxsc[q][blk] : 0.0f;     // the empty half of an odd last pair adds nothing
                    const float f0 = s0 * xs_, f1 = s1 * xs_;
                    acc[q][0] = fmaf(f0, (float)cc[0], acc[q][0]);
                    acc[q][1] = fmaf(f0, (float)cc[1], acc[q][1]);
                    acc[q][2] = fmaf(f1, (float)cc[2], acc[q][2]);
                    acc[q][3] = fmaf(f1, (float)cc[3], acc[q][3]);
                }
            }
            __syncwarp();
            cslot = cslot + 1 == DEPTH ? 0 : cslot + 1;
        }
        if (tracing && tile == blockIdx.x) p.trace[4] = gtime();
        // ── tile epilogue: reduce the warps' column subsets, recombine the digits ──
        gemv_tile_epilogue<SWIGLU, GPT, NM>(acc, s_part + (size_t)buf * kWarps * NM * 128, tile, p.M, p.N, eo, p.bias != nullptr,
                                            p.bias2 != nullptr, p.residual != nullptr, p.act, p.out, p.ldo);
        buf ^= 1;
    }
    cp_async_wait<0>();
    if (tracing) p.trace[5] = gtime();
    if (p.trace != nullptr && tid == 0) atomicMax(p.trace + 6, gtime());
}

size_t i8_smem_bytes(int K, int M, int depth) {
    return (size_t)kWarps * depth * kSlotBytes + (size_t)kColsPerRow * M * (K + kXsPad) + (size_t)M * (K / 32) * 4 +
           (size_t)2 * kWarps * (M > 2 ? 2 : 1) * 128 * 4;
}

template <bool SWIGLU, int DEPTH, bool GPT, int NM>
void launch_i8(const GemvI8Params& p, cudaStream_t s) {
    static bool attrSet = false;
    if (!attrSet) {
        DJ_CUDA_CHECK(cudaFuncSetAttribute(k_q8_gemv_i8<SWIGLU, DEPTH, GPT, NM>, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024));
        attrSet = true;
    }
    int rowsPerTile = SWIGLU ? 8 : 16;
    int nTiles = (p.N + rowsPerTile - 1) / rowsPerTile;
    // every CTA gets the same number of tiles (±1 only in the last round): the grid is the
    // smallest one that keeps the rounds of the full grid
    int cap = 2 * g_num_sms;
    int rounds = (nTiles + cap - 1) / cap;
    int gx = (nTiles + rounds - 1) / rounds;
    launch_k(k_q8_gemv_i8<SWIGLU, DEPTH, GPT, NM>, dim3(gx), dim3(kThreads), i8_smem_bytes(p.K, p.M, DEPTH), s, true, p);
}

template <bool SWIGLU, bool GPT>
void launch_i8_depth(const GemvI8Params& p, int depth, cudaStream_t s) {
    if (p.M > 2) {      // two MMAs per block; the digits of four rows leave room for a ring of at most five items
        switch (depth) {
            case 3: launch_i8<SWIGLU, 3, GPT, 2>(p, s); break;
            case 4: launch_i8<SWIGLU, 4, GPT, 2>(p, s); break;
            default: launch_i8<SWIGLU, 5, GPT, 2>(p, s); break;
        }
        return;
    }
    switch (depth) {
        case 3: launch_i8<SWIGLU, 3, GPT, 1>(p, s); break;
        case 4: launch_i8<SWIGLU, 4, GPT, 1>(p, s); break;
        default: launch_i8<SWIGLU, 5, GPT, 1>(p, s); break;
    }
}

}  // namespace

// Returns false when the shape is outside this kernel's domain (the caller falls
// back to the FMA kernel).  Two CTAs share an SM, so a CTA may use half of its
// shared memory: the ring takes what the activation digits leave.
bool q8_gemv_i8_fuses_gpt(const Q8LinearArgs& a) {
    const int K = a.w.K;
    if (K % 32 != 0 || a.w.Kp != K || a.w2.codes != nullptr) return false;
    if (i8_smem_bytes(K, 1, 3) > 111 * 1024) return false;
    return (K >> 4) <= kStageRounds * kThreads;      // LayerNorm lives in the register staging path only
}

bool launch_q8_gemv_i8(const Q8LinearArgs& a, cudaStream_t s) {
    const int K = a.w.K;
    if (K % 32 != 0 || a.w.Kp != K) return false;
    const bool swiglu = a.w2.codes != nullptr;
    const bool gpt = a.beta != nullptr || a.act != 0;
    if (gpt && !q8_gemv_i8_fuses_gpt(a)) return false;
    const size_t budget = 111 * 1024;
    if (i8_smem_bytes(K, 1, 3) > budget) return false;
    for (int m0 = 0; m0 < a.M;) {
        constexpr int maxRows = 4;
        int rows = a.M - m0 < maxRows ? a.M - m0 : maxRows;      // 8 MMA columns = 2 activation rows × (3 digits + 1 unused); 3-4 rows take a second MMA
        while (rows > 1 && i8_smem_bytes(K, rows, 3) > budget) rows--;
        int depth = 5;      // four items (4 KB) per warp in flight, 64 KB per SM
        while (depth > 3 && i8_smem_bytes(K, rows, depth) > budget) depth--;
        GemvI8Params p;
        p.x = a.x + (size_t)m0 * a.ldx; p.ldx = a.ldx; p.gamma = a.gamma; p.eps = a.eps;
        p.beta = a.beta; p.act = a.act;
        p.codes = a.w.codes; p.scales = a.w.scales; p.bias = a.bias;
        p.codes2 = a.w2.codes; p.scales2 = a.w2.scales; p.bias2 = a.bias2;
        p.residual = a.residual ? a.residual + (size_t)m0 * a.ldr : nullptr; p.ldr = a.ldr;
        p.out = a.out + (size_t)m0 * a.ldo; p.ldo = a.ldo;
        p.K = K; p.N = a.w.N; p.Kp = a.w.Kp; p.nb = a.w.nb; p.M = rows;
        p.pre = kPreMax;
        p.mid = 4;
        p.trace = trace_slot();
        if (swiglu) launch_i8_depth<true, false>(p, depth, s);
        else if (gpt) launch_i8_depth<false, true>(p, depth, s);
        else launch_i8_depth<false, false>(p, depth, s);
        m0 += rows;
    }
    return true;
}

}  // namespace dj
