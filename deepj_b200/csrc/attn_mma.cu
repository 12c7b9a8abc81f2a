// Prompt-chunk attention on the tensor cores.
//
// For a chunk of T tokens every query row of a head attends to the cached keys 0 … pos + t.  The
// fp32 kernel in attn.cu spends four FMA per (query, key, dim) triple on the CUDA cores; this one
// runs S = Q·Kᵀ and O += P·V as mma.sync.m16n8k16 (fp16 inputs, fp32 accumulate) while keeping
// fp32-grade accuracy: every fp32 operand x is split into hi = fp16(x) and lo = fp16(x − hi), and a
// product a·b is accumulated as a_hi·b_hi + a_lo·b_hi + a_hi·b_lo (the dropped lo·lo term is
// ≈ 2^-22 of the product) — the same split the many-row Q8 projection uses.
//
// grid (ceil(T / 64), heads, sequences), 128 threads.  Warp w owns query rows 16w … 16w+15 of the
// tile; the CTA walks the keys in tiles of 32: K and V rows come from the fp32 cache, are split and
// laid down in shared memory as fp16 [key][dim] (row stride dim + 8 halves, so the eight rows an
// ldmatrix fetches fall into different banks) — into the stage that is not being multiplied, the
// global loads of the next tile's K issued before this tile's Q·Kᵀ and those of its V before the
// softmax and P·V, so that their latency is covered by tensor work — S stays in registers, the online softmax is the
// usual running max / sum per row in fp32, and P goes back into the tensor cores straight from the
// S registers (an S accumulator pair is exactly an A-operand pair of the next MMA).
// V is consumed through ldmatrix.trans, so no transposed copy is needed.
//
// The arithmetic it restates: HeadOps.scaledDotProductScores / applyCausalMask / Softmax /
// applyAttentionToValues (layers/transformer/attention/HeadOps.java:90-140, activations/Softmax.java:16-19);
// masked terms contribute exactly 0, as exp(−1e9 − max) does in fp32.
#include "kernels.h"
#include "kv_cache.cuh"
#include "q8_common.cuh"
#include <cuda_fp16.h>

namespace dj {

namespace {

constexpr int kMQ = 64;     // query rows per CTA
constexpr int kMK = 32;     // keys per tile (two tiles are resident: one being multiplied, one being filled)

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(__half a, __half b) {
    return (uint32_t)__half_as_ushort(a) | ((uint32_t)__half_as_ushort(b) << 16);
}
// x0, x1 → packed hi halves and packed lo halves
__device__ __forceinline__ void split2(float x0, float x1, uint32_t& hi, uint32_t& lo) {
    const __half h0 = __float2half_rn(x0), h1 = __float2half_rn(x1);
    hi = pack_h2(h0, h1);
    lo = pack_h2(__float2half_rn(x0 - __half2float(h0)), __float2half_rn(x1 - __half2float(h1)));
}

template <int HD, typename KT>
__global__ void __launch_bounds__(128, 2) k_attn_prefill_mma(
        const float* __restrict__ qkv, int q_off, int ld, const KT* __restrict__ kcache, const KT* __restrict__ vcache,
        int maxSeq, const float* __restrict__ posbuf, const float* __restrict__ cosT, const float* __restrict__ sinT,
        float* __restrict__ out, int ldo, int H, float scale, int T) {
    constexpr int LDS = HD + 8;                     // halves per shared-memory row
    constexpr int KS = HD / 16;                     // k-steps of Q·Kᵀ, and pairs of output n-tiles
    extern __shared__ __align__(16) __half smh[];
    __half* Qh = smh;                               // [64][LDS] each
    __half* Ql = Qh + kMQ * LDS;
    __half* Kh = Ql + kMQ * LDS;
    __half* Kl = Kh + kMK * LDS;
    __half* Vh = Kl + kMK * LDS;
    __half* Vl = Vh + kMK * LDS;
    pdl_wait();
    pdl_launch_dependents();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int t0 = qt * kMQ;
    int pos0 = (int)posbuf[b];
    pos0 = pos0 < 0 ? 0 : pos0;
    constexpr int half_ = HD >> 1;

    // Q tile: rotate the interleaved pairs at position pos0 + t, fold in 1/sqrt(hd), split
    for (int i = tid; i < kMQ * half_; i += 128) {
        const int r = i / half_, pr = i % half_;
        const int t = t0 + r;
        float x0 = 0.0f, x1 = 0.0f;
        if (t < T && pos0 + t < maxSeq) {
            const float2 v = *reinterpret_cast<const float2*>(qkv + (size_t)(b * T + t) * ld + q_off + h * HD + 2 * pr);
            const float c = cosT[(size_t)(pos0 + t) * half_ + pr], s = sinT[(size_t)(pos0 + t) * half_ + pr];
            x0 = (v.x * c - v.y * s) * scale;
            x1 = (v.x * s + v.y * c) * scale;
        }
        uint32_t hi, lo;
        split2(x0, x1, hi, lo);
        *reinterpret_cast<uint32_t*>(Qh + r * LDS + 2 * pr) = hi;
        *reinterpret_cast<uint32_t*>(Ql + r * LDS + 2 * pr) = lo;
    }
    const KT* kb = kcache + ((size_t)b * H + h) * maxSeq * HD;
    const KT* vb = vcache + ((size_t)b * H + h) * maxSeq * HD;
    const int lastKey = min(maxSeq - 1, pos0 + min(T, t0 + kMQ) - 1);       // newest key any row of this tile may see
    const int row0 = warp * 16 + g, row1 = row0 + 8;                         // this lane's two query rows within the tile
    const int lim0 = pos0 + t0 + row0, lim1 = pos0 + t0 + row1;              // row r attends to keys ≤ lim

    // ldmatrix lane addresses (bytes, shared window)
    const uint32_t qAddr = smem_u32(Qh) + (uint32_t)(((warp * 16 + (lane & 15)) * LDS + (lane >> 4) * 8) * 2);
    const uint32_t qlDelta = (uint32_t)(kMQ * LDS * 2);                      // Ql − Qh
    const uint32_t kAddr = smem_u32(Kh) + (uint32_t)((((lane & 7) + ((lane >> 4) << 3)) * LDS + ((lane >> 3) & 1) * 8) * 2);
    const uint32_t klDelta = (uint32_t)(kMK * LDS * 2);
    const uint32_t vAddr = smem_u32(Vh) + (uint32_t)((((lane & 7) + (((lane >> 3) & 1) << 3)) * LDS + (lane >> 4) * 8) * 2);

    float o[2 * KS][4];
#pragma unroll
    for (int j = 0; j < 2 * KS; j++) { o[j][0] = 0.0f; o[j][1] = 0.0f; o[j][2] = 0.0f; o[j][3] = 0.0f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;

    // A thread's share of one 32-key tile of K (or of V): kPer float4 pieces, piece u = tid + 128·u.
    constexpr int kPer = kMK * (HD / 4) / 128;
    float4 pre[kPer];
    auto fetch = [&](const KT* base, int k0) {
#pragma unroll
        for (int u = 0; u < kPer; u++) {
            const int i = tid + u * 128;
            const int key = i / (HD / 4), d4 = i % (HD / 4);
            pre[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (k0 + key <= lastKey) pre[u] = KvIo<KT>::ld4(base + (size_t)(k0 + key) * HD + 4 * d4);
        }
    };
    auto put = [&](__half* hiT, __half* loT) {      // split what `fetch` brought and lay it down as fp16 [key][dim]
#pragma unroll
        for (int u = 0; u < kPer; u++) {
            const int i = tid + u * 128;
            const int key = i / (HD / 4), d4 = i % (HD / 4);
            uint2 hi, lo;
            split2(pre[u].x, pre[u].y, hi.x, lo.x); split2(pre[u].z, pre[u].w, hi.y, lo.y);
            *reinterpret_cast<uint2*>(hiT + key * LDS + 4 * d4) = hi;
            *reinterpret_cast<uint2*>(loT + key * LDS + 4 * d4) = lo;
        }
    };
    constexpr int kStageHalves = 4 * kMK * LDS;     // K_hi, K_lo, V_hi, V_lo of one tile
    constexpr uint32_t kStageBytes = kStageHalves * 2;

    // first tile into stage 0
    fetch(kb, 0); put(Kh, Kl);
    fetch(vb, 0); put(Vh, Vl);
    __syncthreads();
    const int nTiles = lastKey / kMK + 1;
    for (int it = 0; it < nTiles; it++) {
        const int k0 = it * kMK;
        const uint32_t cur = (uint32_t)(it & 1) * kStageBytes;
        __half* const nKh = Kh + ((it + 1) & 1) * kStageHalves;
        const bool more = it + 1 < nTiles;
        if (more) fetch(kb, k0 + kMK);              // the next tile's keys travel while this tile's Q·Kᵀ runs

        // S = Q·Kᵀ: 16 rows × 32 keys per warp, four n-tiles of eight keys
        float s[4][4];
#pragma unroll
        for (int j = 0; j < 4; j++) { s[j][0] = 0.0f; s[j][1] = 0.0f; s[j][2] = 0.0f; s[j][3] = 0.0f; }
#pragma unroll
        for (int kk = 0; kk < KS; kk++) {
            uint32_t ah[4], al[4], bh[2][4], bl[2][4];
            ldsm_x4(ah, qAddr + kk * 32);
            ldsm_x4(al, qAddr + qlDelta + kk * 32);
#pragma unroll
            for (int np = 0; np < 2; np++) {        // two n-tiles (16 keys) per ldmatrix
                const uint32_t a = kAddr + cur + (uint32_t)(np * 16 * LDS * 2) + kk * 32;
                ldsm_x4(bh[np], a);
                ldsm_x4(bl[np], a + klDelta);
            }
            // three passes over the four accumulators: consecutive MMAs never wait on each other's result
#pragma unroll
            for (int np = 0; np < 2; np++) { mma_f16(s[2 * np], ah, bh[np][0], bh[np][1]); mma_f16(s[2 * np + 1], ah, bh[np][2], bh[np][3]); }
#pragma unroll
            for (int np = 0; np < 2; np++) { mma_f16(s[2 * np], al, bh[np][0], bh[np][1]); mma_f16(s[2 * np + 1], al, bh[np][2], bh[np][3]); }
#pragma unroll
            for (int np = 0; np < 2; np++) { mma_f16(s[2 * np], ah, bl[np][0], bl[np][1]); mma_f16(s[2 * np + 1], ah, bl[np][2], bl[np][3]); }
        }
        if (more) { put(nKh, nKh + kMK * LDS); fetch(vb, k0 + kMK); }      // … and its values while the softmax and P·V run

        // causal mask, running max
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 4; j++) {
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int key = k0 + j * 8 + 2 * t4 + e;
                if (key > lim0 || key > lastKey) s[j][e] = -INFINITY;
                if (key > lim1 || key > lastKey) s[j][2 + e] = -INFINITY;
                mx0 = fmaxf(mx0, s[j][e]); mx1 = fmaxf(mx1, s[j][2 + e]);
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float c0 = mn0 > -INFINITY ? expf(m0 - mn0) : 1.0f, c1 = mn1 > -INFINITY ? expf(m1 - mn1) : 1.0f;
        float ps0 = 0.0f, ps1 = 0.0f;
#pragma unroll
        for (int j = 0; j < 4; j++) {
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const float p0 = s[j][e] > -INFINITY ? expf(s[j][e] - mn0) : 0.0f;
                const float p1 = s[j][2 + e] > -INFINITY ? expf(s[j][2 + e] - mn1) : 0.0f;
                s[j][e] = p0; s[j][2 + e] = p1;
                ps0 += p0; ps1 += p1;
            }
        }
        l0 = l0 * c0 + ps0; l1 = l1 * c1 + ps1;     // per-lane partial sums: the four lanes of a row are added at the end
        m0 = mn0; m1 = mn1;
        if (c0 != 1.0f || c1 != 1.0f) {             // the running maxima rarely move after the first tiles
#pragma unroll
            for (int j = 0; j < 2 * KS; j++) { o[j][0] *= c0; o[j][1] *= c0; o[j][2] *= c1; o[j][3] *= c1; }
        }

        // O += P·V: the S registers of n-tiles 2kk, 2kk+1 are the A operand of key step kk
#pragma unroll
        for (int kk = 0; kk < kMK / 16; kk++) {
            uint32_t ph[4], pl[4];
            split2(s[2 * kk][0], s[2 * kk][1], ph[0], pl[0]);
            split2(s[2 * kk][2], s[2 * kk][3], ph[1], pl[1]);
            split2(s[2 * kk + 1][0], s[2 * kk + 1][1], ph[2], pl[2]);
            split2(s[2 * kk + 1][2], s[2 * kk + 1][3], ph[3], pl[3]);
#pragma unroll
            for (int c4 = 0; c4 < KS; c4 += 4) {    // eight n-tiles (64 output columns) per round, two per ldmatrix
                uint32_t bh[4][4], bl[4][4];
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const uint32_t a = vAddr + cur + (uint32_t)(kk * 16 * LDS * 2) + (c4 + q) * 32;
                    ldsm_x4_t(bh[q], a);
                    ldsm_x4_t(bl[q], a + klDelta);
                }
#pragma unroll
                for (int q = 0; q < 4; q++) { mma_f16(o[2 * (c4 + q)], ph, bh[q][0], bh[q][1]); mma_f16(o[2 * (c4 + q) + 1], ph, bh[q][2], bh[q][3]); }
#pragma unroll
                for (int q = 0; q < 4; q++) { mma_f16(o[2 * (c4 + q)], pl, bh[q][0], bh[q][1]); mma_f16(o[2 * (c4 + q) + 1], pl, bh[q][2], bh[q][3]); }
#pragma unroll
                for (int q = 0; q < 4; q++) { mma_f16(o[2 * (c4 + q)], ph, bl[q][0], bl[q][1]); mma_f16(o[2 * (c4 + q) + 1], ph, bl[q][2], bl[q][3]); }
            }
        }
        if (more) put(nKh + 2 * kMK * LDS, nKh + 3 * kMK * LDS);
        __syncthreads();                            // the next stage is complete, and nobody still reads this one
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    if (t0 + row0 < T && l0 > 0.0f) {
        float* dst = out + (size_t)(b * T + t0 + row0) * ldo + h * HD + 2 * t4;
#pragma unroll
        for (int j = 0; j < 2 * KS; j++) *reinterpret_cast<float2*>(dst + j * 8) = make_float2(o[j][0] / l0, o[j][1] / l0);
    }
    if (t0 + row1 < T && l1 > 0.0f) {
        float* dst = out + (size_t)(b * T + t0 + row1) * ldo + h * HD + 2 * t4;
#pragma unroll
        for (int j = 0; j < 2 * KS; j++) *reinterpret_cast<float2*>(dst + j * 8) = make_float2(o[j][2] / l1, o[j][3] / l1);
    }
}

template <int HD> constexpr size_t prefill_mma_smem() { return (size_t)(2 * kMQ + 2 * 4 * kMK) * (HD + 8) * sizeof(__half); }

template <int HD, typename KT>
void launch_mma(const AttnDecodeArgs& a, int T, cudaStream_t s) {
    static bool attr = false;
    if (!attr) {
        DJ_CUDA_CHECK(cudaFuncSetAttribute(k_attn_prefill_mma<HD, KT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)prefill_mma_smem<HD>()));
        attr = true;
    }
    dim3 grid((T + kMQ - 1) / kMQ, a.H, a.B);
    launch_k(k_attn_prefill_mma<HD, KT>, grid, dim3(128), prefill_mma_smem<HD>(), s, true, (const float*)a.qkv, a.q_off, a.ld,
             (const KT*)a.kcache, (const KT*)a.vcache, a.maxSeq, a.pos, a.cosT, a.sinT, a.out, a.ldo, a.H, a.scale, T);
}

}  // namespace

// The chunk's keys and values must already be in the cache (k_kv_append).  Returns false for head dims
// this kernel has no instance for.
bool launch_attn_prefill_mma(const AttnDecodeArgs& a, cudaStream_t s) {
    const int T = a.T < 1 ? 1 : a.T;
    if (a.ldo % 2 != 0 || (reinterpret_cast<uintptr_t>(a.out) & 7) != 0) return false;      // float2 stores
    if (a.hd != 128 && a.hd != 64) return false;
    if (a.kvHalf) { if (a.hd == 128) launch_mma<128, __half>(a, T, s); else launch_mma<64, __half>(a, T, s); }
    else { if (a.hd == 128) launch_mma<128, float>(a, T, s); else launch_mma<64, float>(a, T, s); }
    return true;
}

}  // namespace dj
