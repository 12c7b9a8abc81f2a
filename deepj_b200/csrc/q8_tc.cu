// Q8 linear for many activation rows (prefill): tcgen05 tensor-core tiles with the
// accumulator in tensor memory.
//
// With M in the hundreds the work is a dense contraction, 2·M·K·N flops against K·N weight
// bytes, and belongs on the 5th-generation tensor cores.  The Q8 format keeps one fp32 scale per
// 32 weights, so the weights cannot stay int8 inside one long accumulation; instead each
// 256 × 32 weight tile is dequantised on the fly, exactly once per CTA, into two fp16 tiles with
//     w_hi + w_lo = code · scale   to ≈ 22 bits  (packed fp16 arithmetic, see the conversion loop)
// and the activations are split the same way by a pre-pass (x_hi, x_lo, after a power-of-two row
// scaling that keeps fp16 in range; RMSNorm is applied there too).  Three MMAs per k-step,
//     D += X_hi·W_hi + X_lo·W_hi + X_hi·W_lo,
// carry ≈ 22 bits of each operand into the fp32 accumulator — the dropped lo·lo term is 2^-22
// relative — so the prefill path stays inside the decode path's tolerance at one third of the
// fp16 tensor peak.
//
// One CTA per 128 (activation rows) × 256 (weight rows) output tile, or — when the launch has enough tiles to
// keep every SM busy that way — per pair of them: two 128 × 256 accumulators fill the SM's tensor memory and
// share every dequantised weight tile, which halves the conversion work per flop.  k-tiles of 32, ten warps:
//   warps 0-7  dequantise, as two groups of four that take the k-tiles in turn (a thread owns two weight rows of
//              the tile: 32 code bytes + a scale each per k-tile from global memory, its next three k-tiles
//              already in registers) and write the W_hi / W_lo tiles in the 64-byte-swizzled K-major layout the
//              MMA reads; afterwards they are the epilogue: tcgen05.ld of a 32 × 128 piece of the accumulator
//              each, row scale, bias, residual or SiLU-gate, 128-byte row stores through a shared-memory transpose;
//   warp 8     one thread streams the activation tiles: the pre-pass leaves every 128 × 32 tile as a ready
//              shared-memory image (hi and lo adjacent, 16 KB), so a stage is ONE plain bulk copy completing
//              on an mbarrier — no tensor map;
//   warp 9     one thread issues the MMAs (128 × 256 × 16, three per accumulator and 16-k step, each accumulator
//              256 columns of tensor memory) and commits each stage back to its "empty" barriers.
// 64 KB of activation stages (four of one 128-row tile, or two of a pair) and three weight stages of 32 KB.  Every wait is bounded: when a bound
// expires the CTA records an error code, stops waiting for anything, frees its tensor memory and returns.
#include "kernels.h"
#include "q8_common.cuh"
#include <cuda_fp16.h>

namespace dj {
namespace {

constexpr int kTileM = 128, kTileN = 256, kTileK = 32;
constexpr int kStagesA = 4, kStagesB = 3;                // activation stages: four of one 128-row tile, or two of a pair of tiles
constexpr int kATileBytes = kTileM * kTileK * 2;         // one fp16 activation tile: 8 KB
constexpr int kBTileBytes = kTileN * kTileK * 2;         // one fp16 weight tile: 16 KB
constexpr int kAImageBytes = 2 * kATileBytes;            // X_hi, X_lo of one 128-row tile, as the pre-pass lays them down
constexpr int kARegionBytes = kStagesA * kAImageBytes;   // 64 KB of activation stages either way
constexpr int kStageBBytes = 2 * kBTileBytes;            // W_hi, W_lo
constexpr int kDqWarps = 8;                              // dequantising (later: epilogue) warps, one weight row per thread; then one copy warp, one MMA warp
constexpr int kTcThreads = (kDqWarps + 2) * 32;
constexpr unsigned kTcWaitLimit = 1u << 22;              // try_wait rounds before a wait gives up
constexpr int kTmemCols = 512;                            // two 128 × 256 fp32 accumulators: all of tensor memory
constexpr int kRawRow = 144;                             // bytes per weight row in the raw-code buffer: 4 k-tiles of codes + their scales

// byte offset of 16-byte chunk c (0-3) of row r inside a 64-byte-swizzled K-major tile of 32 halves per row:
// 8-row groups of 512 bytes, the chunk index XORed with bits 1-2 of the row
__host__ __device__ __forceinline__ int swz_off(int r, int c) { return (r >> 3) * 512 + (r & 7) * 64 + ((c ^ ((r >> 1) & 3)) << 4); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait; `abort_flag` (shared) short-circuits every later wait of the CTA once one has expired.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* error, int code) {
    for (unsigned it = 0; it < kTcWaitLimit; it++) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    atomicExch(error, code);
    return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
          "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
          "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// K-major, 64-byte swizzle: 8-row groups 512 bytes apart (stride byte offset), leading offset unused (1),
// descriptor version 1, layout type 4.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3fff);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(512 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)4 << 61;
    return d;
}
// fp16 × fp16 → fp32, both operands K-major, M = 128, N = 256
constexpr uint32_t kIdesc = (1u << 4) | ((uint32_t)(kTileN >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));      // first source → upper half
    return r;
}

// ───────────── pre-pass: fp32 activations → hi/lo fp16 tile images ─────────────
// One warp per activation row.  Output tiles [m-tile][k-tile]{hi 16 KB, lo 16 KB}; rowscale[m] undoes the
// power-of-two scaling in the GEMM epilogue.  Rows ≥ M of the last m-tile are written as zeros.
__global__ void __launch_bounds__(256) k_x_to_f16_tiles(const float* __restrict__ x, int ldx, const float* __restrict__ gamma, float eps,
                                                         int M, int K, unsigned char* __restrict__ tiles, float* __restrict__ rowscale) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int m = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int mPad = (M + kTileM - 1) / kTileM * kTileM;
    if (m >= mPad) return;
    const int nK = K / kTileK;
    unsigned char* mt = tiles + (size_t)(m / kTileM) * nK * (2 * kATileBytes);
    const int r = m % kTileM;
    if (m >= M) {
        for (int c = lane; c < nK * 4; c += 32) {
            unsigned char* t = mt + (size_t)(c >> 2) * (2 * kATileBytes) + swz_off(r, c & 3);
            *reinterpret_cast<uint4*>(t) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(t + kATileBytes) = make_uint4(0, 0, 0, 0);
        }
        if (lane == 0) rowscale[m] = 0.0f;
        return;
    }
    const float* xr = x + (size_t)m * ldx;
    float ss = 0.0f, amax = 0.0f;
    for (int k = lane * 4; k < K; k += 128) {
        const float4 v = *reinterpret_cast<const float4*>(xr + k);
        ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        float4 g = make_float4(1.f, 1.f, 1.f, 1.f);
        if (gamma) g = *reinterpret_cast<const float4*>(gamma + k);
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x * g.x), fabsf(v.y * g.y)), fmaxf(fabsf(v.z * g.z), fabsf(v.w * g.w))));
    }
    for (int o = 16; o > 0; o >>= 1) { ss += __shfl_xor_sync(0xffffffffu, ss, o); amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o)); }
    float inv = 1.0f;
    if (gamma) inv = __frcp_rn(sqrtf(ss * (1.0f / (float)K) + eps));      // RMSNorm1D.forward: x / rms · γ
    amax *= inv;
    // 2^-e brings the row's largest value into [512, 1024)
    int ebits = 0x3f800000;
    if (amax > 0.0f && amax < 1e30f) ebits = __float_as_int(amax) & 0x7f800000;
    const float down = __int_as_float(0x7f000000 - ebits) * 512.0f;
    if (lane == 0) rowscale[m] = __int_as_float(ebits) * (1.0f / 512.0f);
    for (int c = lane; c < nK * 4; c += 32) {          // chunk c: values 8c … 8c+7
        const float4 a = *reinterpret_cast<const float4*>(xr + c * 8), b = *reinterpret_cast<const float4*>(xr + c * 8 + 4);
        float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        if (gamma) {
            const float4 ga = *reinterpret_cast<const float4*>(gamma + c * 8), gb = *reinterpret_cast<const float4*>(gamma + c * 8 + 4);
            const float g[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
#pragma unroll
            for (int j = 0; j < 8; j++) v[j] = (v[j] * inv) * g[j];
        }
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float p = v[2 * j] * down, q = v[2 * j + 1] * down;
            hi[j] = pack_h2(p, q);
            const float2 back = __half22float2(*reinterpret_cast<const __half2*>(&hi[j]));
            lo[j] = pack_h2(p - back.x, q - back.y);
        }
        unsigned char* t = mt + (size_t)(c >> 2) * (2 * kATileBytes) + swz_off(r, c & 3);
        *reinterpret_cast<uint4*>(t) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<uint4*>(t + kATileBytes) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    }
}

struct TcParams {
    const unsigned char* xtiles; const float* rowscale;
    const int8_t* codes; const float* scales; const float* bias;
    const float* residual; int ldr;
    float* out; int ldo;
    int M, N, K, Kp, nb;
    int mTiles;             // 128-row activation tiles
    int pair;               // 1: a CTA takes tiles 2·blockIdx.y and 2·blockIdx.y + 1 (the second may not exist), two accumulators; 0: tile blockIdx.y
    int mode;               // 0: out = acc + bias (+ residual);  1: out = SiLU(out) · (acc + bias)   (SwiGLU's second GEMM)
    int ktPer;              // k-tiles per K split (blockIdx.z); a multiple of 4.  One split = the whole reduction
    size_t splitStride;     // floats between the partial outputs of consecutive splits (0 when there is one split)
    int terms;              // correction products on top of x_hi · w_hi: bit 0 adds x_lo · w_hi, bit 1 adds x_hi · w_lo
    int* error;
    unsigned long long* trace;      // optional: thread 0 of CTA (0,0) sums the time it spends waiting / converting / fencing
};

__global__ void __launch_bounds__(kTcThreads, 1) k_q8_gemm_tc(const TcParams p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ __align__(8) unsigned long long s_bar[2 * kStagesA + 2 * kStagesB + 5];
    __shared__ uint32_t s_tmem;
    __shared__ volatile int s_abort;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile0 = p.pair ? 2 * (int)blockIdx.y : (int)blockIdx.y;
    const int n0 = blockIdx.x * kTileN, m0 = tile0 * kTileM;
    const bool has1 = p.pair && tile0 + 1 < p.mTiles;           // a second 128-row tile for the second accumulator
    const int nStA = p.pair ? kStagesA / 2 : kStagesA;          // activation stages in use, and their size
    const uint32_t stABytes = p.pair ? 2 * kAImageBytes : kAImageBytes;
    // K split blockIdx.z covers k-tiles kt0 … kt0 + nK − 1 of the nKfull of the reduction; everything below counts
    // k-tiles from 0 within the split and only the global addresses know kt0
    const int nKfull = p.K / kTileK;
    const int kt0 = (int)blockIdx.z * p.ktPer;
    const int nK = min(p.ktPer, nKfull - kt0);
    const int8_t* const codes = p.codes + (size_t)kt0 * kTileK;
    const float* const scales = p.scales + kt0;
    float* const outp = p.out + (size_t)blockIdx.z * p.splitStride;
    // the swizzled tiles want 1024-byte alignment: the dynamic segment carries 1 KB of slack for it
    const uint32_t smem_raw = smem_u32(smem);
    const uint32_t smem_s = (smem_raw + 1023u) & ~1023u;
    unsigned char* const smem_al = smem + (smem_s - smem_raw);
    // layout: activation stages [kStagesA][tile 0: X_hi 8 KB | X_lo 8 KB][tile 1: the same], then weight stages [kStagesB][W_hi 16 KB | W_lo 16 KB]
    const uint32_t smemB_s = smem_s + kARegionBytes;
    unsigned char* const smemB = smem_al + kARegionBytes;
    auto bar_fullA = [&](int s) { return smem_u32(&s_bar[s]); };
    auto bar_emptyA = [&](int s) { return smem_u32(&s_bar[kStagesA + s]); };
    auto bar_fullB = [&](int s) { return smem_u32(&s_bar[2 * kStagesA + s]); };
    auto bar_emptyB = [&](int s) { return smem_u32(&s_bar[2 * kStagesA + kStagesB + s]); };
    const uint32_t bar_acc = smem_u32(&s_bar[2 * kStagesA + 2 * kStagesB]);
    const uint32_t bar_rawFull = smem_u32(&s_bar[2 * kStagesA + 2 * kStagesB + 1]);
    const uint32_t bar_rawEmpty = smem_u32(&s_bar[2 * kStagesA + 2 * kStagesB + 2]);
    unsigned char* const raw = smemB + kStagesB * kStageBBytes;          // [256 rows][128 code bytes + 4 scales]

    if (tid == 0) {
        for (int s = 0; s < kStagesA; s++) { mbar_init(bar_fullA(s), 1); mbar_init(bar_emptyA(s), 1); }
        for (int s = 0; s < kStagesB; s++) { mbar_init(bar_fullB(s), 128); mbar_init(bar_emptyB(s), 1); }
        mbar_init(bar_acc, 1);
        mbar_init(bar_rawFull, kDqWarps * 32);
        mbar_init(bar_rawEmpty, kDqWarps * 32);
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kDqWarps) tmem_alloc(smem_u32(&s_tmem), kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = s_tmem;
    pdl_wait();
    pdl_launch_dependents();

    if (warp < kDqWarps) {
        // ── dequantise: two groups of four warps take the k-tiles in turn (group g: k-tiles g, g+2, …); thread r of a
        // group owns weight rows n0 + r and n0 + r + 128 of the 256-row tile.  The raw codes and scales of four
        // k-tiles at a time (256 rows × 128 code bytes + 4 scales) come through a shared-memory buffer filled with
        // cp.async in row-contiguous runs — a warp's copy instruction touches 4 lines, where a load per row owner
        // touched 32 and kept L1TEX saturated; every thread lifts its own pieces into registers, the buffer is
        // refilled for the next four k-tiles behind a barrier, and the conversion runs from registers. ──
        const int r = tid & 127, grp = tid >> 7;
        const int nG = nK / 4;
        auto issue_group = [&](int G) {
            // chunk q = tid + 256·i → row q / 8 (clamped: rows past N are never stored), 16-byte piece q % 8
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int row = (tid >> 3) + 32 * i, c = tid & 7;
                const int n = min(n0 + row, p.N - 1);
                cp_async16(raw + row * kRawRow + c * 16, codes + (size_t)n * p.Kp + (size_t)G * 128 + c * 16);
            }
            const int n = min(n0 + tid, p.N - 1);
            cp_async16(raw + tid * kRawRow + 128, scales + (size_t)n * p.nb + (size_t)G * 4);
            asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar_rawFull) : "memory");
        };
        issue_group(0);
        const bool tracing = p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && tid == 0;
        unsigned long long tWait = 0, tConv = 0, tFence = 0, tStart = tracing ? gtime() : 0;
        const bool wantLo = (p.terms & 2) != 0;              // without the x_hi · w_lo product the low halves are never read
        for (int G = 0; G < nG; G++) {
            uint4 cur4[2][2][2]; float scl4[2][2];            // [own k-tile of the group][row][16-byte half]
            mbar_wait(bar_rawFull, G & 1, &s_abort, p.error, 206);
#pragma unroll
            for (int o = 0; o < 2; o++)
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const unsigned char* src = raw + (r + 128 * h) * kRawRow;
                    const int j = grp + 2 * o;                   // k-tile inside the group
                    cur4[o][h][0] = *reinterpret_cast<const uint4*>(src + 32 * j);
                    cur4[o][h][1] = *reinterpret_cast<const uint4*>(src + 32 * j + 16);
                    scl4[o][h] = *reinterpret_cast<const float*>(src + 128 + 4 * j);
                }
            mbar_arrive(bar_rawEmpty);
            if (G + 1 < nG) {
                mbar_wait(bar_rawEmpty, G & 1, &s_abort, p.error, 207);      // every thread has lifted its pieces
                issue_group(G + 1);
            }
#pragma unroll
            for (int o = 0; o < 2; o++) {
                const int kt = 4 * G + grp + 2 * o;
                const int s = kt % kStagesB;
                uint4 cur[2][2]; float scl[2];
#pragma unroll
                for (int h = 0; h < 2; h++) { cur[h][0] = cur4[o][h][0]; cur[h][1] = cur4[o][h][1]; scl[h] = scl4[o][h]; }
                unsigned long long t0 = tracing ? gtime() : 0;
                if (kt >= kStagesB) mbar_wait(bar_emptyB(s), ((kt / kStagesB) - 1) & 1, &s_abort, p.error, 201);
                unsigned long long t1 = tracing ? gtime() : 0;
                unsigned char* bhi = smemB + (size_t)s * kStageBBytes;
                unsigned char* blo = bhi + kBTileBytes;
                // The block's scale (times 2^12, undone in the epilogue, so that it sits in fp16's normal range) as
                // s_hi + s_lo, both fp16.  Per pair of codes, all in packed fp16 arithmetic:
                //   c    = the codes as fp16, exactly (sign flip, byte under exponent 0x64, subtract 1152)
                //   w_hi = rn(c · s_hi)
                //   w_lo = rn(c · s_lo + (c · s_hi − w_hi))      — the product's rounding error is exact in one fma
                // so w_hi + w_lo carries ≈ 22 bits of c · scale at 2.75 instructions per weight.
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const int row = r + 128 * h;
                    const float sv = scl[h] * 4096.0f;
                    const __half sh1 = __float2half_rn(sv);
                    const __half sl1 = __float2half_rn(sv - __half2float(sh1));
                    const __half2 sh = __half2half2(sh1), sl = __half2half2(sl1);
#pragma unroll
                    for (int j = 0; j < 2; j++) {                  // 16 codes → two 16-byte chunks of hi and of lo
                        const uint32_t w4[4] = {cur[h][j].x, cur[h][j].y, cur[h][j].z, cur[h][j].w};
                        uint32_t hi[8], lo[8];
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            const uint32_t u = w4[q] ^ 0x80808080u;
                            uint32_t c01 = __byte_perm(u, 0x64646464u, 0x4140), c23 = __byte_perm(u, 0x64646464u, 0x4342);
                            const uint32_t k1152 = 0x64806480u;
                            asm("sub.f16x2 %0, %1, %2;" : "=r"(c01) : "r"(c01), "r"(k1152));
                            asm("sub.f16x2 %0, %1, %2;" : "=r"(c23) : "r"(c23), "r"(k1152));
#pragma unroll
                            for (int e = 0; e < 2; e++) {
                                const __half2 c = *reinterpret_cast<const __half2*>(e == 0 ? &c01 : &c23);
                                const __half2 wh = __hmul2(c, sh);
                                hi[2 * q + e] = *reinterpret_cast<const uint32_t*>(&wh);
                                if (wantLo) {
                                    const __half2 er = __hfma2(c, sh, __hneg2(wh));
                                    const __half2 wl = __hfma2(c, sl, er);
                                    lo[2 * q + e] = *reinterpret_cast<const uint32_t*>(&wl);
                                }
                            }
                        }
                        const int o0 = swz_off(row, 2 * j), o1 = swz_off(row, 2 * j + 1);
                        *reinterpret_cast<uint4*>(bhi + o0) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                        *reinterpret_cast<uint4*>(bhi + o1) = make_uint4(hi[4], hi[5], hi[6], hi[7]);
                        if (wantLo) {
                            *reinterpret_cast<uint4*>(blo + o0) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                            *reinterpret_cast<uint4*>(blo + o1) = make_uint4(lo[4], lo[5], lo[6], lo[7]);
                        }
                    }
                }
                unsigned long long t2 = tracing ? gtime() : 0;
                fence_proxy_async_smem();                      // generic-proxy stores → visible to the tensor-core (async) proxy
                mbar_arrive(bar_fullB(s));
                if (tracing) { const unsigned long long t3 = gtime(); tWait += t1 - t0; tConv += t2 - t1; tFence += t3 - t2; }
            }
        }
        if (tracing) { p.trace[0] = tStart; p.trace[1] = tStart + tWait; p.trace[2] = p.trace[1] + tConv; p.trace[3] = p.trace[2] + tFence; p.trace[4] = gtime(); }
        // ── epilogue: warp w reads accumulator rows 32(w%4) … +31, columns 128(w/4) … +127; each 32 × 32 block goes
        // through a padded shared-memory square so that a warp stores 128 contiguous bytes of one output row ──
        const bool ok = __all_sync(0xffffffffu, mbar_wait(bar_acc, 0, &s_abort, p.error, 202));
        tc_fence_after();
        const int q4 = warp & 3, chalf = warp >> 2;
        float* stg = reinterpret_cast<float*>(smem_al) + warp * (32 * 33);       // the pipeline stages are idle by now
#pragma unroll 1
        for (int acc = 0; acc < (has1 ? 2 : 1); acc++) {
        const int mbase = m0 + acc * kTileM + q4 * 32;
        const int mrow = mbase + lane;
        const float rs = (ok && mrow < p.M) ? p.rowscale[mrow] * (1.0f / 4096.0f) : 0.0f;       // the weights carry 2^12
#pragma unroll 1
        for (int c0 = chalf * 128; c0 < chalf * 128 + 128; c0 += 32) {
            uint32_t v[32];
            if (ok) tmem_ld32(tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(acc * kTileN + c0), v);      // warp-uniform
            else {
#pragma unroll
                for (int j = 0; j < 32; j++) v[j] = 0u;
            }
#pragma unroll
            for (int j = 0; j < 32; j++) stg[lane * 33 + j] = __uint_as_float(v[j]) * rs;
            __syncwarp();
            const int nn = n0 + c0 + lane;
            const float bv = (p.bias && nn < p.N) ? p.bias[nn] : 0.0f;
            for (int i = 0; i < 32; i++) {
                const int m = mbase + i;
                if (!ok || m >= p.M || nn >= p.N) continue;
                float val = stg[i * 33 + lane] + bv;
                float* o = outp + (size_t)m * p.ldo + nn;
                if (p.mode == 0) {
                    if (p.residual) val += p.residual[(size_t)m * p.ldr + nn];
                    *o = val;
                } else {
                    const float gte = *o;
                    const float sig = 1.0f / (1.0f + expf(-gte));
                    *o = (gte * sig) * val;
                }
            }
            __syncwarp();
        }
        }
        if (tracing) { p.trace[5] = gtime(); p.trace[6] = p.trace[5]; }
        tc_fence_before();
    } else if (warp == kDqWarps) {
        // ── activation tiles: one bulk copy of 16 KB (hi + lo) per 128-row tile and stage ──
        if (lane == 0) {
            const unsigned char* src = p.xtiles + ((size_t)tile0 * nKfull + kt0) * kAImageBytes;
            for (int kt = 0; kt < nK; kt++) {
                const int s = kt % nStA;
                if (kt >= nStA && !mbar_wait(bar_emptyA(s), ((kt / nStA) - 1) & 1, &s_abort, p.error, 203)) break;
                mbar_arrive_expect_tx(bar_fullA(s), has1 ? 2 * kAImageBytes : kAImageBytes);
                bulk_g2s(smem_s + (uint32_t)s * stABytes, src + (size_t)kt * kAImageBytes, kAImageBytes, bar_fullA(s));
                if (has1)
                    bulk_g2s(smem_s + (uint32_t)s * stABytes + kAImageBytes, src + (size_t)(nKfull + kt) * kAImageBytes, kAImageBytes, bar_fullA(s));
            }
        }
        __syncwarp();
    } else {
        // ── MMA issue: one thread ──
        if (lane == 0) {
            bool ok = true;
            const bool xLo = (p.terms & 1) != 0, wLo = (p.terms & 2) != 0;
            for (int kt = 0; kt < nK && ok; kt++) {
                const int sa = kt % nStA, sb = kt % kStagesB;
                ok = mbar_wait(bar_fullA(sa), (kt / nStA) & 1, &s_abort, p.error, 204) &&
                     mbar_wait(bar_fullB(sb), (kt / kStagesB) & 1, &s_abort, p.error, 205);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_hi = smem_s + (uint32_t)sa * stABytes, a_lo = a_hi + kATileBytes;
                const uint32_t b_hi = smemB_s + (uint32_t)sb * kStageBBytes, b_lo = b_hi + kBTileBytes;
#pragma unroll
                for (int ks = 0; ks < kTileK / 16; ks++) {
                    const uint32_t off = ks * 32;          // 16 halves along K inside the swizzled row
                    umma_f16(tmem_base, umma_desc(a_hi + off), umma_desc(b_hi + off), kIdesc, (kt | ks) != 0);
                    if (xLo) umma_f16(tmem_base, umma_desc(a_lo + off), umma_desc(b_hi + off), kIdesc, 1);
                    if (wLo) umma_f16(tmem_base, umma_desc(a_hi + off), umma_desc(b_lo + off), kIdesc, 1);
                    if (has1) {                            // the same weight tile against the second 128 rows → accumulator 2
                        umma_f16(tmem_base + kTileN, umma_desc(a_hi + kAImageBytes + off), umma_desc(b_hi + off), kIdesc, (kt | ks) != 0);
                        if (xLo) umma_f16(tmem_base + kTileN, umma_desc(a_lo + kAImageBytes + off), umma_desc(b_hi + off), kIdesc, 1);
                        if (wLo) umma_f16(tmem_base + kTileN, umma_desc(a_hi + kAImageBytes + off), umma_desc(b_lo + off), kIdesc, 1);
                    }
                }
                umma_commit(bar_emptyA(sa));               // both arrive when the MMAs above have finished reading the stages
                umma_commit(bar_emptyB(sb));
            }
            if (ok) umma_commit(bar_acc);
        }
        __syncwarp();
    }
    __syncthreads();
    if (warp == kDqWarps) { tc_fence_after(); tmem_dealloc(tmem_base, kTmemCols); }
}

constexpr size_t kTcSmem = (size_t)kARegionBytes + (size_t)kStagesB * kStageBBytes + (size_t)kTileN * kRawRow + 1024;

// Adds the partial outputs of a K-split launch in split order and runs the epilogue that the GEMM kernel runs itself
// when the reduction is not split: out = Σ + bias (+ residual), or out = SiLU(out) · (Σ + bias) for SwiGLU's second GEMM.
__global__ void __launch_bounds__(256) k_q8_tc_split_reduce(const float* __restrict__ part, size_t splitStride, int splits, int M, int N,
                                                            const float* __restrict__ bias, const float* __restrict__ residual, int ldr,
                                                            float* __restrict__ out, int ldo, int mode) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t total = (size_t)M * N;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int m = (int)(i / N), n = (int)(i - (size_t)m * N);
        float v = 0.0f;
        for (int z = 0; z < splits; z++) v += __ldcg(part + (size_t)z * splitStride + i);
        if (bias) v += bias[n];
        float* o = out + (size_t)m * ldo + n;
        if (mode == 0) {
            if (residual) v += residual[(size_t)m * ldr + n];
            *o = v;
        } else {
            const float gte = *o;
            const float sig = 1.0f / (1.0f + expf(-gte));
            *o = (gte * sig) * v;
        }
    }
}

// How a launch is laid out: CTAs take one 128-row tile or a pair, and when that leaves most SMs without a tile (a few
// dozen to a few hundred rows) the reduction is split over up to four CTAs whose partial outputs a small kernel adds.
struct TcPlan { bool pair; int splits, ktPer; long ctas; };
TcPlan tc_plan(int M, int K, int N) {
    const long mTiles = (M + kTileM - 1) / kTileM, nTiles = (N + kTileN - 1) / kTileN;
    const int nK = K / kTileK;
    // Two accumulators per CTA halve the conversion work per flop but also the number of CTAs, and a paired CTA
    // takes 1.55–1.7 × as long as a single one: pair when the rounds of CTAs over the SMs it saves outweigh that.
    const long single = nTiles * mTiles, paired = nTiles * ((mTiles + 1) / 2);
    const long roundsSingle = (single + g_num_sms - 1) / g_num_sms, roundsPaired = (paired + g_num_sms - 1) / g_num_sms;
    TcPlan pl;
    pl.pair = mTiles >= 2 && 1.7 * (double)roundsPaired < (double)roundsSingle;
    pl.ctas = pl.pair ? paired : single;
    pl.splits = 1;
    if (M <= 256 && 2 * pl.ctas <= g_num_sms) {
        int sp = (int)(g_num_sms / pl.ctas);
        if (sp > 4) sp = 4;
        while (sp > 1 && nK / sp < 16) sp--;              // at least 16 k-tiles (512 k) per split
        pl.splits = sp;
    }
    pl.ktPer = ((nK + pl.splits - 1) / pl.splits + 3) / 4 * 4;      // whole groups of four k-tiles (the raw-code buffer's unit)
    pl.splits = (nK + pl.ktPer - 1) / pl.ktPer;
    return pl;
}

}  // namespace

int g_tc_terms = 3;

// Rough duration of launch_q8_linear_tc in µs, for the choice between this path and passes of the 16-row kernel
// when M is small: a CTA needs ≈ 0.75 µs per 32-k tile (1.2 µs when it carries two accumulators), CTAs run in
// rounds over the SMs, the activation pre-pass costs a few µs, and a split reduction adds its small second kernel.
double q8_tc_estimate_us(int M, int K, int N) {
    const TcPlan pl = tc_plan(M, K, N);
    const long rounds = (pl.ctas * pl.splits + g_num_sms - 1) / g_num_sms;
    // 0.75 µs per k-tile measured with one wave of a few dozen CTAs, 0.95 µs with the ≈ 144 CTAs of a split launch
    const double perCta = (pl.pair ? 1.2 : pl.splits > 1 ? 0.95 : 0.75) * pl.ktPer;
    double t = perCta * rounds + 5.0;
    if (pl.splits > 1) t += 4.0 + (double)pl.splits * M * N * 8.0 / 3.0e6;      // partial outputs written and read back at ≈ 3 TB/s
    return t;
}

size_t q8_tc_ws_floats(int M, int K, int N) {
    const size_t mPad = (size_t)(M + kTileM - 1) / kTileM * kTileM;
    const TcPlan pl = tc_plan(M, K, N);
    return mPad * K + mPad + (pl.splits > 1 ? (size_t)pl.splits * M * N : 0);          // hi + lo halves = 4 bytes per value, the row scales, the splits' partial outputs
}

// out = x · W (+ fused norm / bias / residual / SiLU-gate) for M ≥ 1 rows on the tensor cores.
// Returns false when the shape is outside the kernel's domain (K must be a multiple of 128).
bool launch_q8_linear_tc(const Q8LinearArgs& a, float* ws, cudaStream_t s) {
    const int K = a.w.K, N = a.w.N, M = a.M;
    if (K % 128 != 0 || a.w.Kp != K || ws == nullptr || M < 1) return false;      // raw codes travel four k-tiles (and their 4 scales = 16 bytes) at a time
    if (((uintptr_t)a.x & 15) != 0 || a.ldx % 4 != 0 || (a.gamma && ((uintptr_t)a.gamma & 15) != 0)) return false;
    static bool attrSet = false;
    if (!attrSet) {
        DJ_CUDA_CHECK(cudaFuncSetAttribute(k_q8_gemm_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmem));
        attrSet = true;
    }
    const int mTiles = (M + kTileM - 1) / kTileM, nTiles = (N + kTileN - 1) / kTileN;
    const size_t mPad = (size_t)mTiles * kTileM;
    unsigned char* tiles = reinterpret_cast<unsigned char*>(ws);
    float* rowscale = ws + mPad * K;
    float* part = rowscale + mPad;
    launch_k(k_x_to_f16_tiles, dim3((unsigned)(mPad / 8)), dim3(256), 0, s, true, a.x, a.ldx, a.gamma, a.eps, M, K, tiles, rowscale);
    const TcPlan pl = tc_plan(M, K, N);
    const bool split = pl.splits > 1;
    const dim3 grid(nTiles, pl.pair ? (mTiles + 1) / 2 : mTiles, pl.splits);
    const int redBlocks = (int)(((size_t)M * N + 255) / 256 < (size_t)(4 * g_num_sms) ? ((size_t)M * N + 255) / 256 : (size_t)(4 * g_num_sms));
    TcParams p;
    p.xtiles = tiles; p.rowscale = rowscale;
    p.M = M; p.N = N; p.K = K; p.Kp = a.w.Kp; p.nb = a.w.nb; p.mTiles = mTiles; p.pair = pl.pair ? 1 : 0;
    p.ktPer = pl.ktPer; p.splitStride = split ? (size_t)M * N : 0;
    p.terms = g_tc_terms; p.error = g_dev_error; p.trace = trace_slot();
    auto run = [&](const Q8View& w, const float* bias, const float* residual, int mode) {
        p.codes = w.codes; p.scales = w.scales;
        if (split) {
            // raw partial sums per split, the epilogue in the reduce kernel
            p.bias = nullptr; p.residual = nullptr; p.ldr = 0; p.out = part; p.ldo = N; p.mode = 0;
            launch_k(k_q8_gemm_tc, grid, dim3(kTcThreads), kTcSmem, s, true, p);
            launch_k(k_q8_tc_split_reduce, dim3(redBlocks), dim3(256), 0, s, true, (const float*)part, p.splitStride, pl.splits, M, N, bias,
                     residual, a.ldr, a.out, a.ldo, mode);
        } else {
            p.bias = bias; p.residual = residual; p.ldr = a.ldr; p.out = a.out; p.ldo = a.ldo; p.mode = mode;
            launch_k(k_q8_gemm_tc, grid, dim3(kTcThreads), kTcSmem, s, true, p);
        }
    };
    run(a.w, a.bias, a.residual, 0);
    // SwiGLU: the gate projection is in `out`; the up projection's epilogue multiplies SiLU(gate) into it
    if (a.w2.codes != nullptr) run(a.w2, a.bias2, nullptr, 1);
    return true;
}

}  // namespace dj

// Which of the two fp16 correction products the tensor-core GEMM issues on top of x_hi · w_hi: bit 0 = x_lo · w_hi,
// bit 1 = x_hi · w_lo.  3 (the default) carries ≈ 22 bits of both operands; 1, 2 and 0 trade bits for tensor-pipe time
// (and, without bit 1, for half of the dequantisation stores).  Drops the cached CUDA graphs, which hold the old value.
extern "C" int deepj_cuda_tc_configure(int32_t correction_terms) {
    if (correction_terms < 0 || correction_terms > 3) { dj::set_last_error("tc_configure: correction_terms must be 0..3"); return 1; }
    if (dj::g_tc_terms != correction_terms) { dj::g_tc_terms = correction_terms; dj::invalidate_graphs(); }
    return 0;
}
