// Q8 GEMV on the integer tensor pipe with warp-private TMA rings — the decode hot kernel for up to two
// activation rows per pass, for reduction lengths that are multiples of 128.
//
// Same arithmetic as the cp.async kernel (q8_gemv_i8.cu: one int8 MMA m16n8k32 per 32-k block of 16 weight
// rows, activations as three base-256 digit columns with a power-of-two block scale, exact integer block sums,
// fp32 accumulation of (weight scale × activation scale) × sum), but the weights reach shared memory through the
// tensor-memory accelerator instead of the load/store unit: one lane of a warp issues four tiled bulk copies per
// item (two 8-row × 128-byte boxes of codes, two 8-row × 4 boxes of scales, straight from the [N][K] / [N][K/32]
// layout of the format, 128-byte swizzle) that complete on a warp-private mbarrier, and the warp reads its MMA
// operands with one ldmatrix.x4 per block.  Measured on the cp.async kernel: its copies landed in shared memory
// sector by sector (≈ 11 wavefronts per 512-byte instruction, 58 % of all shared-memory wavefronts of the kernel)
// and held the load/store pipe near saturation in the streaming phase, so the kernel ran at the same speed from
// L2 as from HBM; here the pipe carries the operand reads only, and the conversion of the block sums to fp32 is
// an integer add and a subtraction on the main pipes instead of a conversion-unit instruction.
//
// Two CTAs of 8 warps per SM as before (the next kernel's CTAs move in while this one drains); warp w owns the
// 128-k groups w, w+8, … of every tile of its CTA and stages exactly those groups of the activations itself;
// two items (2304 bytes each) per warp in flight.  Projections with a fused LayerNorm or GELU (GPT blocks) stay on
// the cp.async kernel.
#include <cuda.h>

#include "kernels.h"
#include "q8_common.cuh"
#include "q8_stage.cuh"
#include "q8_tma.cuh"

namespace dj {

namespace {

constexpr int kWarps = kGemvWarps;
constexpr int kThreads = kGemvThreads;
constexpr int kItemK = kTmaItemK;
constexpr int kCodeBytes = 16 * kItemK;             // 16 rows × 128 code bytes, two 1024-byte swizzle atoms
constexpr int kScaleBytes = 16 * 16;                // 16 rows × 4 block scales
constexpr int kItemBytes = kCodeBytes + kScaleBytes;
// Three items per warp: a deeper ring measured no faster back to back (the kernel waits on the handoff and on the
// activations, not on bytes in flight) and slower inside the decode step, where a CTA pair of 2 × 96 KB and more takes
// the L1 capacity that the attention kernel beside it uses.
constexpr int kDepth = 3;
constexpr int kSpinLimit = 1 << 22;                 // polls of one item's barrier before the kernel gives up on it
constexpr int kErrTmaWait = 330;                    // device error code: an item never arrived

struct GemvTmaParams {
    CUtensorMap codes, scales, codes2, scales2;     // boxes of 8 rows; the second pair is the SwiGLU up projection
    const float* x; int ldx;
    const float* gamma; float eps;
    const float* bias; const float* bias2;
    const float* residual; int ldr;
    float* out; int ldo;
    int K, N, M;
    int pre;                        // ring items a warp fetches before it waits for the previous kernel
    int* error;
    unsigned long long* trace;
};

// NM = 2 takes three or four activation rows in one pass over the weights (a second MMA per block).
template <bool SWIGLU, int DEPTH, int NM>
__global__ void __launch_bounds__(kThreads, 2) k_q8_gemv_tma(const __grid_constant__ GemvTmaParams p) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long s_bar[kWarps * DEPTH];
    __shared__ float s_ss[4 * kWarps];               // the warps' parts of Σx² per activation row (RMSNorm in the epilogue)
    // layout (from a 1024-byte boundary, which the swizzle pattern wants): code rings [warps][DEPTH][2048], scale rings
    // [warps][DEPTH][256], digits int8 [3M][K+pad], block scales fp32 [M][K/32], partials [2][warps][NM][16][8]
    const uint32_t raw_s = smem_u32(smem_raw);
    unsigned char* const smem = smem_raw + (((raw_s + 1023u) & ~1023u) - raw_s);
    const int ldxs = p.K + kGemvXsPad;
    unsigned char* const ringC = smem;
    unsigned char* const ringS = smem + (size_t)kWarps * DEPTH * kCodeBytes;
    int8_t* xd = reinterpret_cast<int8_t*>(ringS + (size_t)kWarps * DEPTH * kScaleBytes);
    float* xsc = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(xd) + (size_t)kGemvColsPerRow * p.M * ldxs);
    float* s_part = xsc + (size_t)p.M * (p.K >> 5);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    constexpr int rowsPerTile = SWIGLU ? 8 : 16;
    const int nTiles = (p.N + rowsPerTile - 1) / rowsPerTile;
    const int nGroups = p.K / kItemK;
    const bool tracing = p.trace != nullptr && blockIdx.x == 0 && tid == 0;
    if (tracing) { p.trace[0] = gtime(); p.trace[6] = 0ull; }

    const uint32_t myC = smem_u32(ringC) + (uint32_t)warp * DEPTH * kCodeBytes;
    const uint32_t myS = smem_u32(ringS) + (uint32_t)warp * DEPTH * kScaleBytes;
    const uint32_t myBar = smem_u32(&s_bar[warp * DEPTH]);
    if (lane == 0) {
#pragma unroll
        for (int d = 0; d < DEPTH; d++) mbar_init(myBar + 8 * d, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();

    // flat (tile, group) sequence of this warp, with a cursor running DEPTH-1 items ahead; rows past N and the
    // second half of a tile that does not exist are filled with zeros by the copy engine and never stored
    int itile = blockIdx.x, igrp = warp, islot = 0;
    auto issue_next = [&]() {
        if (itile < nTiles && igrp < nGroups) {
            if (lane == 0) {
                const uint32_t bar = myBar + 8 * islot;
                const uint32_t dc = myC + (uint32_t)islot * kCodeBytes, ds = myS + (uint32_t)islot * kScaleBytes;
                const int row0 = itile * rowsPerTile;
                mbar_arrive_expect_tx(bar, kItemBytes);
                tma_box(dc, &p.codes, igrp * kItemK, row0, bar);
                tma_box(dc + kCodeBytes / 2, SWIGLU ? &p.codes2 : &p.codes, igrp * kItemK, SWIGLU ? row0 : row0 + 8, bar);
                tma_box(ds, &p.scales, igrp * 4, row0, bar);
                tma_box(ds + kScaleBytes / 2, SWIGLU ? &p.scales2 : &p.scales, igrp * 4, SWIGLU ? row0 : row0 + 8, bar);
            }
            igrp += kWarps;
            if (igrp >= nGroups) { igrp = warp; itile += gridDim.x; }
        }
        islot = islot + 1 == DEPTH ? 0 : islot + 1;
    };
    // Weights never depend on the previous kernel, so streaming starts before the wait.
    const int kPre = p.pre < DEPTH - 1 ? p.pre : DEPTH - 1;
    for (int d = 0; d < kPre; d++) issue_next();
    pdl_launch_dependents();
    if (tracing) p.trace[1] = gtime();
    // the norm's gain is a weight as well: fetch it before the wait when four groups per warp cover the row
    const bool gammaEarly = p.gamma != nullptr && nGroups <= 4 * kWarps && (reinterpret_cast<uintptr_t>(p.gamma) & 15) == 0;
    float4 gpre4[4];
#pragma unroll
    for (int j = 0; j < 4; j++) gpre4[j] = make_float4(1.0f, 1.0f, 1.0f, 1.0f);
    if (gammaEarly) {
#pragma unroll
        for (int j = 0; j < 4; j++)
            if (warp + kWarps * j < nGroups) gpre4[j] = gemv_load4(p.gamma + (warp + kWarps * j) * 128 + lane * 4, true);
    }
    pdl_wait();
    if (tracing) p.trace[2] = gtime();

    // activations → digit columns in the MMA fragment's order; the rest of the ring is queued behind the first loads.
    // Every warp converts the groups it consumes and goes on by itself; RMSNorm's 1/rms is applied in the epilogue.
    gemv_stage_warp_groups(p.x, p.ldx, p.gamma, p.K, p.M, xd, ldxs, xsc, s_ss, gpre4, gammaEarly, [&]() {
        for (int d = kPre; d < DEPTH - 1; d++) issue_next();
    });
    if (warp >= nGroups) {                               // a warp without groups still owes the ring its issue slots
        for (int d = kPre; d < DEPTH - 1; d++) issue_next();
    }
    if (tracing) p.trace[3] = gtime();

    // lane (g,t) feeds column g of MMA q: activation row 2q + g/4, digit g%4 (digit 3 does not exist)
    bool hasCol[NM]; const unsigned char* xcol[NM]; const float* myxsc[NM];
    float acc[NM][4];
#pragma unroll
    for (int q = 0; q < NM; q++) {
        const int mrow = 2 * q + (g >> 2);
        hasCol[q] = mrow < p.M && (g & 3) != 3;
        xcol[q] = reinterpret_cast<const unsigned char*>(xd) + (size_t)(hasCol[q] ? kGemvColsPerRow * mrow + (g & 3) : 0) * ldxs + t * 8;
        // the lane's two result columns 2t, 2t+1 belong to activation row 2q + t/2
        const int rrow = 2 * q + (t >> 1);
        myxsc[q] = xsc + (size_t)(rrow < p.M ? rrow : 0) * (p.K >> 5);
        acc[q][0] = acc[q][1] = acc[q][2] = acc[q][3] = 0.0f;
    }
    // ldmatrix.x4 addresses: lanes 0-7 rows 0-7 of the block's first 16-byte chunk, 8-15 rows 8-15 of it, 16-23 and
    // 24-31 the same rows of the second chunk; chunk c of row r sits at r·128 + ((c ^ (r & 7)) · 16)
    const int lrow = (lane & 7) + ((lane >> 3) & 1) * 8;
    const uint32_t lmBase = (uint32_t)lrow * 128u;
    const uint32_t lmChunk = (uint32_t)((lane >> 4) ^ (lrow & 7));
    int cslot = 0, buf = 0, limit = kSpinLimit;
    uint32_t phases = 0;
    for (int tile = blockIdx.x; tile < nTiles; tile += gridDim.x) {
        const GemvEpilogueOperands eo = gemv_epilogue_fetch<SWIGLU>(tile, p.M, p.N, p.bias, p.bias2, p.residual, p.ldr);
        for (int grp = warp; grp < nGroups; grp += kWarps) {
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
            const unsigned char* ss = ringS + ((size_t)warp * DEPTH + cslot) * kScaleBytes;
            const float4 s0 = *reinterpret_cast<const float4*>(ss + g * 16);            // row g: its four block scales
            const float4 s1 = *reinterpret_cast<const float4*>(ss + (g + 8) * 16);      // row g+8
            const float s0v[4] = {s0.x, s0.y, s0.z, s0.w}, s1v[4] = {s1.x, s1.y, s1.z, s1.w};
            float xsv[NM][4];
#pragma unroll
            for (int q = 0; q < NM; q++) {
                const float4 v = *reinterpret_cast<const float4*>(myxsc[q] + grp * 4);
                xsv[q][0] = v.x; xsv[q][1] = v.y; xsv[q][2] = v.z; xsv[q][3] = v.w;
            }
#pragma unroll
            for (int b = 0; b < 4; b++) {
                uint32_t a[4];
                ldmatrix_x4(a, sc + lmBase + ((lmChunk ^ (uint32_t)(2 * b)) << 4));
                const int blk = grp * 4 + b;
#pragma unroll
                for (int q = 0; q < NM; q++) {
                    uint2 xb = make_uint2(0u, 0u);
                    if (hasCol[q]) xb = *reinterpret_cast<const uint2*>(xcol[q] + blk * 32);
                    int cc[4] = {0, 0, 0, 0};
                    mma_s8_16832(cc, a[0], a[1], a[2], a[3], xb.x, xb.y);
                    const float f0 = s0v[b] * xsv[q][b], f1 = s1v[b] * xsv[q][b];
                    acc[q][0] = fmaf(f0, int_to_float_exact(cc[0]), acc[q][0]);
                    acc[q][1] = fmaf(f0, int_to_float_exact(cc[1]), acc[q][1]);
                    acc[q][2] = fmaf(f1, int_to_float_exact(cc[2]), acc[q][2]);
                    acc[q][3] = fmaf(f1, int_to_float_exact(cc[3]), acc[q][3]);
                }
            }
            __syncwarp();           // every lane has read the slot before lane 0 hands it to the copy engine again
            cslot = cslot + 1 == DEPTH ? 0 : cslot + 1;
        }
        if (tracing && tile == blockIdx.x) p.trace[4] = gtime();
        gemv_tile_epilogue<SWIGLU, false, NM>(acc, s_part + (size_t)buf * kWarps * NM * 128, tile, p.M, p.N, eo, p.bias != nullptr,
                                            p.bias2 != nullptr, p.residual != nullptr, 0, p.out, p.ldo,
                                            p.gamma ? s_ss : nullptr, p.eps, p.K);
        buf ^= 1;
    }
    if (tracing) p.trace[5] = gtime();
    if (p.trace != nullptr && tid == 0) atomicMax(p.trace + 6, gtime());
}

size_t tma_smem_bytes(int K, int M, int depth) {
    return 1024 + (size_t)kWarps * depth * kItemBytes + (size_t)kGemvColsPerRow * M * (K + kGemvXsPad) + (size_t)M * (K / 32) * 4 +
           (size_t)2 * kWarps * (M > 2 ? 2 : 1) * 128 * 4;
}
constexpr size_t kSmemBudget = 112 * 1024;       // two CTAs per SM

template <bool SWIGLU, int DEPTH, int NM>
void launch_tma(const GemvTmaParams& p, cudaStream_t s) {
    static bool attrSet = false;
    if (!attrSet) {
        DJ_CUDA_CHECK(cudaFuncSetAttribute(k_q8_gemv_tma<SWIGLU, DEPTH, NM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget));
        attrSet = true;
    }
    const int rowsPerTile = SWIGLU ? 8 : 16;
    const int nTiles = (p.N + rowsPerTile - 1) / rowsPerTile;
    // every CTA gets the same number of tiles (±1 only in the last round): the grid is the smallest one that
    // keeps the rounds of the full grid
    const int cap = 2 * g_num_sms;
    const int rounds = (nTiles + cap - 1) / cap;
    const int gx = (nTiles + rounds - 1) / rounds;
    launch_k(k_q8_gemv_tma<SWIGLU, DEPTH, NM>, dim3(gx), dim3(kThreads), tma_smem_bytes(p.K, p.M, DEPTH), s, true, p);
}

}  // namespace

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, looked up through the runtime so that the library carries no link-time
// dependency on the driver (it must load on machines without one).
static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        return reinterpret_cast<EncodeTiledFn>(sym);
    }();
    return fn;
}

// Tensor maps over one Q8 weight: codes [N][Kp] bytes in boxes of 8 rows × 128 bytes (128-byte swizzle) and
// scales [N][nb] floats in boxes of 8 rows × 4.
bool q8_encode_weight_maps(const Q8View& w, CUtensorMap* codes, CUtensorMap* scales) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return false;
    if ((reinterpret_cast<uintptr_t>(w.codes) & 15) != 0 || (reinterpret_cast<uintptr_t>(w.scales) & 15) != 0) return false;
    if (w.Kp % 16 != 0 || (w.nb * 4) % 16 != 0) return false;
    {
        const cuuint64_t dims[2] = {(cuuint64_t)w.Kp, (cuuint64_t)w.N};
        const cuuint64_t strides[1] = {(cuuint64_t)w.Kp};
        const cuuint32_t box[2] = {(cuuint32_t)kItemK, 8u};
        const cuuint32_t estr[2] = {1u, 1u};
        if (enc(codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(w.codes), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return false;
    }
    {
        const cuuint64_t dims[2] = {(cuuint64_t)w.nb, (cuuint64_t)w.N};
        const cuuint64_t strides[1] = {(cuuint64_t)w.nb * 4};
        const cuuint32_t box[2] = {4u, 8u};
        const cuuint32_t estr[2] = {1u, 1u};
        if (enc(scales, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(w.scales), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return false;
    }
    return true;
}

// Returns false when the shape is outside this kernel's domain (K a multiple of 128, no LayerNorm / GELU, the
// digits of all rows of the call — up to four — beside the ring in shared memory); the caller then takes the cp.async
// kernel.
bool launch_q8_gemv_tma(const Q8LinearArgs& a, cudaStream_t s) {
    const int K = a.w.K;
    if (K % kItemK != 0 || a.w.Kp != K || g_dev_error == nullptr) return false;
    const bool swiglu = a.w2.codes != nullptr;
    // LayerNorm needs the row's mean before any digit, i.e. CTA-wide staging: the cp.async kernel has it (and measured
    // 1.5 % faster per GPT-2 XL token than this kernel with the same staging)
    if (a.beta != nullptr || a.act != 0) return false;
    if (swiglu && (a.w2.K != K || a.w2.Kp != K || a.w2.N != a.w.N)) return false;
    // all rows (up to four) in one pass, or not at all: where the digits of the rows do not fit beside the ring, the
    // cp.async kernel with its smaller ring items takes them in fewer passes
    if (tma_smem_bytes(K, a.M < 4 ? a.M : 4, kDepth) > kSmemBudget) return false;
    GemvTmaParams p;
    if (!q8_encode_weight_maps(a.w, &p.codes, &p.scales)) return false;
    if (swiglu) {
        if (!q8_encode_weight_maps(a.w2, &p.codes2, &p.scales2)) return false;
    } else {
        p.codes2 = p.codes; p.scales2 = p.scales;
    }
    for (int m0 = 0; m0 < a.M;) {
        int rows = a.M - m0 < 4 ? a.M - m0 : 4;      // 8 MMA columns = 2 activation rows × (3 digits + 1 unused); 3-4 rows take a second MMA
        while (rows > 1 && tma_smem_bytes(K, rows, kDepth) > kSmemBudget) rows--;
        p.x = a.x + (size_t)m0 * a.ldx; p.ldx = a.ldx; p.gamma = a.gamma; p.eps = a.eps;
        p.bias = a.bias; p.bias2 = a.bias2;
        p.residual = a.residual ? a.residual + (size_t)m0 * a.ldr : nullptr; p.ldr = a.ldr;
        p.out = a.out + (size_t)m0 * a.ldo; p.ldo = a.ldo;
        p.K = K; p.N = a.w.N; p.M = rows;
        p.pre = 2;
        p.error = g_dev_error;
        p.trace = trace_slot();
        if (rows > 2) {
            if (swiglu) launch_tma<true, kDepth, 2>(p, s); else launch_tma<false, kDepth, 2>(p, s);
        } else {
            if (swiglu) launch_tma<true, kDepth, 1>(p, s); else launch_tma<false, kDepth, 1>(p, s);
        }
        m0 += rows;
    }
    return true;
}

}  // namespace dj
