// Single-token causal attention over a K/V cache resident in HBM — one kernel.
//
// Replaces, for one new token per sequence, the reference's split-heads / RoPE /
// per-head QKᵀ / mask / softmax / PV / merge chain (HeadOps.java:33-140,
// RotaryEmbedding.java:81-122).  Masked positions contribute exactly +0 to the
// reference's softmax, so attending over 0..pos only is the same function.
//
// grid (splits, heads, batch), flash-decoding: a CTA rotates its head's q in
// registers (interleaved pairs, x0·c − x1·s, x0·s + x1·c), streams its slice of the
// cache once — hd/16 lanes per position, 128-bit loads, online softmax in fp32 — and
// leaves (acc[hd], m, l) in a workspace.  The lane group that meets the newest
// position takes k and v from the projection buffer instead, rotates k and appends
// both to the cache.  The last CTA of a head to finish (a ticket counter that it
// resets) merges the split partials into the merged-heads row, so no second launch
// is needed.  HBM-bound: the algorithmic traffic is the K and V rows of 0..pos.
#include "../../include/deepj_cuda.h"
#include "kernels.h"
#include "kv_cache.cuh"
#include "q8_common.cuh"
#include <algorithm>
#include <cmath>
#include <cstdlib>

namespace dj {

namespace {

constexpr int kAttnWarps = 4;
constexpr int kMaxSplits = 256;             // split partials a head can have (the merge keeps their weights in shared memory)

// Prompt chunk: row z = (sequence b, token t) of the projection buffer holds k and v of position pos[b] + t.
// One thread per interleaved pair: rotate k (x0·c − x1·s, x0·s + x1·c — RotaryEmbedding.java:81-122), copy v.
template <typename KT>
__global__ void k_kv_append(const float* __restrict__ qkv, int k_off, int v_off, int ld, KT* __restrict__ kcache,
                            KT* __restrict__ vcache, int maxSeq, const float* __restrict__ posbuf,
                            const float* __restrict__ cosT, const float* __restrict__ sinT, int H, int hd, int T) {
    pdl_wait();
    pdl_launch_dependents();
    const int h = blockIdx.x, z = blockIdx.y, i = threadIdx.x;
    const int b = z / T, tok = z - b * T;
    const int p = (int)posbuf[b] + tok;
    if (p < 0 || p >= maxSeq) return;
    const float* row = qkv + (size_t)z * ld;
    const float2 k2 = *reinterpret_cast<const float2*>(row + k_off + h * hd + 2 * i);
    const float2 v2 = *reinterpret_cast<const float2*>(row + v_off + h * hd + 2 * i);
    const float c = cosT[(size_t)p * (hd >> 1) + i], s = sinT[(size_t)p * (hd >> 1) + i];
    const size_t dst = (((size_t)b * H + h) * maxSeq + p) * hd + 2 * i;
    KvIo<KT>::st2(kcache + dst, k2.x * c - k2.y * s, k2.x * s + k2.y * c);
    KvIo<KT>::st2(vcache + dst, v2.x, v2.y);
}

template <int LPP, typename KT>   // lanes per position = hd / 16; cache element type
__global__ void __launch_bounds__(kAttnWarps * 32, 4) k_attn_decode(
        const float* __restrict__ qkv, int q_off, int k_off, int v_off, int ld,
        KT* __restrict__ kcache, KT* __restrict__ vcache, int maxSeq,
        const float* __restrict__ posbuf, const float* __restrict__ cosT, const float* __restrict__ sinT,
        float* __restrict__ ws, int* __restrict__ tickets, float* __restrict__ out, int ldo, int H, float scale,
        int T, int append) {
    constexpr int HD = LPP * 16;
    constexpr int PPW = 32 / LPP;                 // positions per warp iteration
    constexpr int G = kAttnWarps * PPW;           // position groups per CTA
    constexpr int kStages = 3;                    // ring stages per warp: two groups of positions in flight, one being folded in
    constexpr int kStageElems = 2 * PPW * HD;     // a stage: K rows of PPW consecutive positions, then their V rows (1024 elements)
    // dynamic shared memory: warp-private K/V rings [warps][kStages][kStageElems] of the cache type while the slice
    // streams; afterwards the same bytes hold the CTA's partial rows (s_acc [G][HD], s_m [G], s_l [G])
    extern __shared__ __align__(16) unsigned char dynsm[];
    float (*s_acc)[HD] = reinterpret_cast<float (*)[HD]>(dynsm);
    float* s_m = reinterpret_cast<float*>(dynsm) + G * HD;
    float* s_l = s_m + G;
    __shared__ int s_last;

    // row z of the projection / output buffers is token t of sequence b: T = 1 (and append) for a decode step;
    // T > 1 for a prompt chunk, whose k/v rows the append kernel has already written
    const int split = blockIdx.x, splits = gridDim.x, h = blockIdx.y, z = blockIdx.z;
    const int b = z / T, tok = z - b * T;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int group = lane / LPP, gl = lane % LPP;
    // The cache rows below the current position were written by earlier steps, not by the kernel this one depends
    // on, so the first two groups of K/V rows are requested BEFORE the wait and stream in while the projection kernel
    // drains.  The position read here is re-read after the wait; in the (never observed) case that it moved, the
    // speculative rows are dropped and requested again.
    const int half = HD >> 1;
    auto read_pos = [&]() {
        int v = (int)__ldcg(posbuf + b) + tok;
        return v < 0 ? 0 : (v >= maxSeq ? maxSeq - 1 : v);
    };
    int pos = read_pos();
    int seq = pos + 1;
    int chunk = (seq + splits - 1) / splits;
    int start = split * chunk;
    int end = min(seq, start + chunk);
    KT* khead = kcache + ((size_t)b * H + h) * maxSeq * HD;      // this head's rows [maxSeq][HD]
    KT* vhead = vcache + ((size_t)b * H + h) * maxSeq * HD;
    KT* kbase = khead + gl * 16;
    KT* vbase = vhead + gl * 16;
    KT* ring = reinterpret_cast<KT*>(dynsm) + (size_t)warp * kStages * kStageElems;
    // Stage `st` ← the K and V rows of positions pb … pb+PPW−1 (consecutive rows are contiguous): 16-byte pieces, lane by
    // lane.  Rows past the end of the cache are clamped to its last row (their lanes are masked out below).
    constexpr int kPieces = PPW * HD * (int)sizeof(KT) / 16;       // per plane: 128 (fp32) or 64 (fp16)
    constexpr int kPerRow = HD * (int)sizeof(KT) / 16;
    auto issue = [&](int st, int pb) {
        KT* dst = ring + (size_t)st * kStageElems;
#pragma unroll
        for (int c0 = 0; c0 < kPieces; c0 += 32) {
            const int c = c0 + lane;
            const int prow = min(pb + c / kPerRow, maxSeq - 1);
            const size_t src = (size_t)prow * HD + (size_t)(c % kPerRow) * (16 / sizeof(KT));
            cp_async16(reinterpret_cast<unsigned char*>(dst) + (size_t)c * 16, khead + src);
            cp_async16(reinterpret_cast<unsigned char*>(dst + PPW * HD) + (size_t)c * 16, vhead + src);
        }
    };
    // iteration `it` of this warp covers positions start + warp·PPW + it·G … + PPW − 1
    int nIter = 0;
    auto count_iters = [&]() { const int first = start + warp * PPW; nIter = first < end ? (end - first + G - 1) / G : 0; };
    count_iters();
    const bool spec = T == 1;                     // a chunk's own rows were written by the kernel before this one: no early requests
    if (spec) {
#pragma unroll
        for (int i = 0; i < kStages - 1; i++) {
            if (i < nIter) issue(i, start + warp * PPW + i * G);
            cp_async_commit();
        }
    }
    // the rotation tables are constants: the row of the speculative position is fetched before the wait too
    float cs[8], sn[8];
    auto load_tables = [&](float (&cs)[8], float (&sn)[8]) {
        const float4* cp = reinterpret_cast<const float4*>(cosT + (size_t)pos * half + gl * 8);
        const float4* sp = reinterpret_cast<const float4*>(sinT + (size_t)pos * half + gl * 8);
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const float4 c4 = cp[j], s4 = sp[j];
            cs[4 * j] = c4.x; cs[4 * j + 1] = c4.y; cs[4 * j + 2] = c4.z; cs[4 * j + 3] = c4.w;
            sn[4 * j] = s4.x; sn[4 * j + 1] = s4.y; sn[4 * j + 2] = s4.z; sn[4 * j + 3] = s4.w;
        }
    };
    load_tables(cs, sn);
    const int specPos = pos;
    pdl_wait();
    pdl_launch_dependents();
    // the query row does not depend on the position: its loads go out together with the position's
    const float* rowp = qkv + (size_t)z * ld;
    float q[16];
    {
        const float4* qp = reinterpret_cast<const float4*>(rowp + q_off + h * HD + gl * 16);
#pragma unroll
        for (int j = 0; j < 4; j++) { float4 v = qp[j]; q[4 * j] = v.x; q[4 * j + 1] = v.y; q[4 * j + 2] = v.z; q[4 * j + 3] = v.w; }
    }
    pos = read_pos();
    if (pos != specPos || !spec) {
        if (pos != specPos) load_tables(cs, sn);
        seq = pos + 1;
        chunk = (seq + splits - 1) / splits;
        start = split * chunk;
        end = min(seq, start + chunk);
        cp_async_wait<0>();                       // whatever was requested for the old position is dropped
        __syncwarp();
        count_iters();
#pragma unroll
        for (int i = 0; i < kStages - 1; i++) {
            if (i < nIter) issue(i, start + warp * PPW + i * G);
            cp_async_commit();
        }
    }

    // rotate 8 interleaved pairs held in v[16] by the table row of the current position (cs, sn)
    auto rotate = [&](float (&v)[16], const float (&cs)[8], const float (&sn)[8]) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float x0 = v[2 * i], x1 = v[2 * i + 1];
            v[2 * i] = x0 * cs[i] - x1 * sn[i];
            v[2 * i + 1] = x0 * sn[i] + x1 * cs[i];
        }
    };
    rotate(q, cs, sn);

    float m = -INFINITY, l = 0.0f, acc[16];
#pragma unroll
    for (int j = 0; j < 16; j++) acc[j] = 0.0f;
    for (int it = 0; it < nIter; it++) {
        // keep two groups in flight: the stage freed by the previous iteration takes the group two ahead
        if (it + kStages - 1 < nIter) issue((it + kStages - 1) % kStages, start + warp * PPW + (it + kStages - 1) * G);
        cp_async_commit();
        cp_async_wait<kStages - 1>();
        __syncwarp();
        const int p = start + warp * PPW + it * G + group;
        const bool valid = p < end;
        float kf[16], vf[16];
        if (valid && p == pos && append) {
            // the new token: k and v come from the projections; rotate k, append both to the cache
            const float4* kp = reinterpret_cast<const float4*>(rowp + k_off + h * HD + gl * 16);
            const float4* vp = reinterpret_cast<const float4*>(rowp + v_off + h * HD + gl * 16);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float4 a = kp[j], c = vp[j];
                kf[4 * j] = a.x; kf[4 * j + 1] = a.y; kf[4 * j + 2] = a.z; kf[4 * j + 3] = a.w;
                vf[4 * j] = c.x; vf[4 * j + 1] = c.y; vf[4 * j + 2] = c.z; vf[4 * j + 3] = c.w;
            }
            float ck[8], sk[8];              // fetched again here (a cache hit) rather than kept live through the loop
            load_tables(ck, sk);
            rotate(kf, ck, sk);
            KvIo<KT>::st16(kbase + (size_t)p * HD, kf);
            KvIo<KT>::st16(vbase + (size_t)p * HD, vf);
            // this step attends to what later steps will read back (the rounded values of an fp16 cache)
#pragma unroll
            for (int j = 0; j < 16; j++) { kf[j] = KvIo<KT>::stored(kf[j]); vf[j] = KvIo<KT>::stored(vf[j]); }
        } else if (valid) {
            const KT* st = ring + (size_t)(it % kStages) * kStageElems + group * HD + gl * 16;
            KvIo<KT>::ld16_shared(st, kf);
            KvIo<KT>::ld16_shared(st + PPW * HD, vf);
        } else {
#pragma unroll
            for (int j = 0; j < 16; j++) { kf[j] = 0.0f; vf[j] = 0.0f; }
        }
        float dot = 0.0f;
#pragma unroll
        for (int j = 0; j < 16; j++) dot = fmaf(q[j], kf[j], dot);
#pragma unroll
        for (int o = LPP / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        if (valid) {
            const float s = dot * scale;
            const float mn = fmaxf(m, s);
            const float corr = expf(m - mn);
            const float pe = expf(s - mn);
            l = l * corr + pe;
#pragma unroll
            for (int j = 0; j < 16; j++) acc[j] = fmaf(pe, vf[j], acc[j] * corr);
            m = mn;
        }
        __syncwarp();                             // the stage is read out before a later request may overwrite it
    }
    cp_async_wait<0>();
    __syncthreads();                              // every warp is done with its ring: the bytes become the partial rows
    const int g = warp * PPW + group;
#pragma unroll
    for (int j = 0; j < 16; j++) s_acc[g][gl * 16 + j] = acc[j];
    if (gl == 0) { s_m[g] = m; s_l[g] = l; }
    __syncthreads();
    float* mine = ws + (((size_t)z * H + h) * splits + split) * (HD + 2);
    for (int j = threadIdx.x; j < HD; j += blockDim.x) {
        float M = -INFINITY;
        for (int gg = 0; gg < G; gg++) M = fmaxf(M, s_m[gg]);
        float a = 0.0f, L = 0.0f;
        if (M > -INFINITY) {
            for (int gg = 0; gg < G; gg++) {
                const float e = expf(s_m[gg] - M);
                a = fmaf(s_acc[gg][j], e, a);
                L = fmaf(s_l[gg], e, L);
            }
        }
        mine[j] = a;
        if (j == 0) { mine[HD] = M; mine[HD + 1] = L; }
    }
    if (splits == 1) {
        // nothing to merge
        __syncthreads();
        for (int j = threadIdx.x; j < HD; j += blockDim.x) out[(size_t)z * ldo + h * HD + j] = mine[j] / mine[HD + 1];
        return;
    }
    // ── the last CTA of this head merges the split partials ──
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int ticket = atomicAdd(&tickets[z * H + h], 1);
        s_last = ticket == splits - 1;
        if (s_last) tickets[z * H + h] = 0;          // ready for the next launch
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // Every thread requests its own column of up to 24 split partials together with the (m, l) pairs, so the
    // merge costs one load round trip (more splits: further rounds of 24).
    const float* pbase = ws + ((size_t)z * H + h) * splits * (HD + 2);
    float* s_m2 = &s_acc[0][0];                 // reused: the CTA's own partial has been written out
    float* s_l2 = s_m2 + kMaxSplits;
    for (int sp = threadIdx.x; sp < splits; sp += blockDim.x) {
        s_m2[sp] = __ldcg(pbase + (size_t)sp * (HD + 2) + HD);
        s_l2[sp] = __ldcg(pbase + (size_t)sp * (HD + 2) + HD + 1);
    }
    constexpr int kBatch = 24;
    const int j0 = threadIdx.x;                 // HD ≤ 512 = 4 columns per thread at most; the first one is prefetched here
    float first[kBatch];
#pragma unroll
    for (int q = 0; q < kBatch; q++) first[q] = (j0 < HD && q < splits) ? __ldcg(pbase + (size_t)q * (HD + 2) + j0) : 0.0f;
    __syncthreads();
    float M = -INFINITY;
    for (int sp = 0; sp < splits; sp++) M = fmaxf(M, s_m2[sp]);
    float L = 0.0f;
    for (int sp = 0; sp < splits; sp++) L = fmaf(s_l2[sp], expf(s_m2[sp] - M), L);
    __syncthreads();
    for (int sp = threadIdx.x; sp < splits; sp += blockDim.x) s_m2[sp] = expf(s_m2[sp] - M);
    __syncthreads();
    for (int j = threadIdx.x; j < HD; j += blockDim.x) {
        float a = 0.0f;
        for (int s0 = 0; s0 < splits; s0 += kBatch) {
            float part[kBatch];
            if (j == j0 && s0 == 0) {
#pragma unroll
                for (int q = 0; q < kBatch; q++) part[q] = first[q];
            } else {
#pragma unroll
                for (int q = 0; q < kBatch; q++) part[q] = s0 + q < splits ? __ldcg(pbase + (size_t)(s0 + q) * (HD + 2) + j) : 0.0f;
            }
#pragma unroll
            for (int q = 0; q < kBatch; q++) if (s0 + q < splits) a = fmaf(part[q], s_m2[s0 + q], a);
        }
        out[(size_t)z * ldo + h * HD + j] = a / L;
    }
}


// The same step with the K/V rows travelling through registers, one group of positions ahead: the form the fp32 cache
// keeps — its 48 KB of rings per CTA would leave no room for this kernel's CTAs to move in beside the projection kernel
// they follow, and measured slower (0.55 against 0.51 ms per 7B token at context 2063).
template <int LPP, typename KT>   // lanes per position = hd / 16; cache element type
__global__ void __launch_bounds__(kAttnWarps * 32, 4) k_attn_decode_regs(
        const float* __restrict__ qkv, int q_off, int k_off, int v_off, int ld,
        KT* __restrict__ kcache, KT* __restrict__ vcache, int maxSeq,
        const float* __restrict__ posbuf, const float* __restrict__ cosT, const float* __restrict__ sinT,
        float* __restrict__ ws, int* __restrict__ tickets, float* __restrict__ out, int ldo, int H, float scale,
        int T, int append) {
    constexpr int HD = LPP * 16;
    constexpr int PPW = 32 / LPP;                 // positions per warp iteration
    constexpr int G = kAttnWarps * PPW;           // position groups per CTA
    __shared__ float s_acc[G][HD];
    __shared__ float s_m[G], s_l[G];
    __shared__ int s_last;

    // row z of the projection / output buffers is token t of sequence b: T = 1 (and append) for a decode step;
    // T > 1 for a prompt chunk, whose k/v rows the append kernel has already written
    const int split = blockIdx.x, splits = gridDim.x, h = blockIdx.y, z = blockIdx.z;
    const int b = z / T, tok = z - b * T;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int group = lane / LPP, gl = lane % LPP;
    // The cache rows below the current position were written by earlier steps, not by the kernel
    // this one depends on, so the first group of K/V rows is fetched BEFORE the wait and streams in
    // while the projection kernel drains.  The position read here is re-read after the wait; in the
    // (never observed) case that it moved, the speculative rows are dropped and fetched again.
    const int half = HD >> 1;
    auto read_pos = [&]() {
        int v = (int)__ldcg(posbuf + b) + tok;
        return v < 0 ? 0 : (v >= maxSeq ? maxSeq - 1 : v);
    };
    int pos = read_pos();
    int seq = pos + 1;
    int chunk = (seq + splits - 1) / splits;
    int start = split * chunk;
    int end = min(seq, start + chunk);
    KT* kbase = kcache + ((size_t)b * H + h) * maxSeq * HD + gl * 16;
    KT* vbase = vcache + ((size_t)b * H + h) * maxSeq * HD + gl * 16;
    float kf[16], vf[16], kn[16], vn[16];
    auto fetch_cached = [&](int p, bool valid, float (&kx)[16], float (&vx)[16]) {
        if (valid) {
            KvIo<KT>::ld16_stream(kbase + (size_t)p * HD, kx);
            KvIo<KT>::ld16_stream(vbase + (size_t)p * HD, vx);
        } else {
#pragma unroll
            for (int j = 0; j < 16; j++) { kx[j] = 0.0f; vx[j] = 0.0f; }
        }
    };
    {
        const int p0 = start + warp * PPW + group;
        fetch_cached(p0, T == 1 && p0 < end && p0 != pos, kf, vf);      // a chunk's own rows were written by the kernel before this one
    }
    // the rotation tables are constants: the row of the speculative position is fetched before the wait too
    float cs[8], sn[8];
    auto load_tables = [&](float (&cs)[8], float (&sn)[8]) {
        const float4* cp = reinterpret_cast<const float4*>(cosT + (size_t)pos * half + gl * 8);
        const float4* sp = reinterpret_cast<const float4*>(sinT + (size_t)pos * half + gl * 8);
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const float4 c4 = cp[j], s4 = sp[j];
            cs[4 * j] = c4.x; cs[4 * j + 1] = c4.y; cs[4 * j + 2] = c4.z; cs[4 * j + 3] = c4.w;
            sn[4 * j] = s4.x; sn[4 * j + 1] = s4.y; sn[4 * j + 2] = s4.z; sn[4 * j + 3] = s4.w;
        }
    };
    load_tables(cs, sn);
    const int specPos = pos;
    pdl_wait();
    pdl_launch_dependents();
    // the query row does not depend on the position: its loads go out together with the position's
    const float* rowp = qkv + (size_t)z * ld;
    float q[16];
    {
        const float4* qp = reinterpret_cast<const float4*>(rowp + q_off + h * HD + gl * 16);
#pragma unroll
        for (int j = 0; j < 4; j++) { float4 v = qp[j]; q[4 * j] = v.x; q[4 * j + 1] = v.y; q[4 * j + 2] = v.z; q[4 * j + 3] = v.w; }
    }
    pos = read_pos();
    if (pos != specPos) load_tables(cs, sn);
    seq = pos + 1;
    chunk = (seq + splits - 1) / splits;
    start = split * chunk;
    end = min(seq, start + chunk);

    // rotate 8 interleaved pairs held in v[16] by the table row of the current position (cs, sn)
    auto rotate = [&](float (&v)[16], const float (&cs)[8], const float (&sn)[8]) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float x0 = v[2 * i], x1 = v[2 * i + 1];
            v[2 * i] = x0 * cs[i] - x1 * sn[i];
            v[2 * i + 1] = x0 * sn[i] + x1 * cs[i];
        }
    };
    rotate(q, cs, sn);

    // K or V slice of a cached position p for this lane (zeros when the lane has no position)
    auto load_k = [&](int p, bool valid, float (&kx)[16]) {
        if (valid) KvIo<KT>::ld16_stream(kbase + (size_t)p * HD, kx);
        else {
#pragma unroll
            for (int j = 0; j < 16; j++) kx[j] = 0.0f;
        }
    };
    auto load_v = [&](int p, bool valid, float (&vx)[16]) {
        if (valid) KvIo<KT>::ld16_stream(vbase + (size_t)p * HD, vx);
        else {
#pragma unroll
            for (int j = 0; j < 16; j++) vx[j] = 0.0f;
        }
    };

    float m = -INFINITY, l = 0.0f, acc[16];
#pragma unroll
    for (int j = 0; j < 16; j++) acc[j] = 0.0f;
    auto fold = [&](bool valid, float dot, const float (&vx)[16]) {
#pragma unroll
        for (int o = LPP / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        if (valid) {
            const float s = dot * scale;
            const float mn = fmaxf(m, s);
            const float corr = expf(m - mn);
            const float pe = expf(s - mn);
            l = l * corr + pe;
#pragma unroll
            for (int j = 0; j < 16; j++) acc[j] = fmaf(pe, vx[j], acc[j] * corr);
            m = mn;
        }
    };

    // The cached rows: two groups of positions travel in two register sets.  A set's K registers are reloaded (two
    // groups ahead) as soon as the dot product has read them, its V registers as soon as the accumulation has: between
    // one and two groups of rows are in flight per warp at any time, with no register copies.  The new token's own
    // position (the last one of the last split) is not in the cache yet and is folded in after the loop.
    const bool ownsNew = append && pos >= start && pos < end;
    const int endc = ownsNew ? pos : end;
    int base = start + warp * PPW;
    if (base < endc) {
        const int p0 = base + group;
        if (T > 1 || pos != specPos) {                                   // a prompt chunk, or a dropped speculation
            load_k(p0, p0 < endc, kf);
            load_v(p0, p0 < endc, vf);
        }
        if (base + G < endc) {
            load_k(base + G + group, base + G + group < endc, kn);
            load_v(base + G + group, base + G + group < endc, vn);
        }
    }
    auto consume = [&](float (&kx)[16], float (&vx)[16], int at, int reload) {
        float dot = 0.0f;
#pragma unroll
        for (int j = 0; j < 16; j++) dot = fmaf(q[j], kx[j], dot);
        if (reload < endc) load_k(reload + group, reload + group < endc, kx);
        fold(at + group < endc, dot, vx);
        if (reload < endc) load_v(reload + group, reload + group < endc, vx);
    };
    for (; base < endc; base += 2 * G) {
        consume(kf, vf, base, base + 2 * G);
        if (base + G >= endc) break;
        consume(kn, vn, base + G, base + 3 * G);
    }
    if (ownsNew && warp == 0) {                                          // warp-uniform
        // the new token: k and v come from the projections; k is rotated, both are appended to the cache, and this step
        // attends to what later steps will read back (the rounded values of an fp16 cache).  Lane group 0 does it.
        const bool mine = group == 0;
        if (mine) {
            const float4* kp = reinterpret_cast<const float4*>(rowp + k_off + h * HD + gl * 16);
            const float4* vp = reinterpret_cast<const float4*>(rowp + v_off + h * HD + gl * 16);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float4 a = kp[j], c = vp[j];
                kf[4 * j] = a.x; kf[4 * j + 1] = a.y; kf[4 * j + 2] = a.z; kf[4 * j + 3] = a.w;
                vf[4 * j] = c.x; vf[4 * j + 1] = c.y; vf[4 * j + 2] = c.z; vf[4 * j + 3] = c.w;
            }
            float ck[8], sk[8];              // fetched again here (a cache hit) rather than kept live through the loop
            load_tables(ck, sk);
            rotate(kf, ck, sk);
            KvIo<KT>::st16(kbase + (size_t)pos * HD, kf);
            KvIo<KT>::st16(vbase + (size_t)pos * HD, vf);
#pragma unroll
            for (int j = 0; j < 16; j++) { kf[j] = KvIo<KT>::stored(kf[j]); vf[j] = KvIo<KT>::stored(vf[j]); }
        }
        float dot = 0.0f;
#pragma unroll
        for (int j = 0; j < 16; j++) dot = fmaf(q[j], kf[j], dot);
        fold(mine, dot, vf);
    }
    const int g = warp * PPW + group;
#pragma unroll
    for (int j = 0; j < 16; j++) s_acc[g][gl * 16 + j] = acc[j];
    if (gl == 0) { s_m[g] = m; s_l[g] = l; }
    __syncthreads();
    float* mine = ws + (((size_t)z * H + h) * splits + split) * (HD + 2);
    for (int j = threadIdx.x; j < HD; j += blockDim.x) {
        float M = -INFINITY;
        for (int gg = 0; gg < G; gg++) M = fmaxf(M, s_m[gg]);
        float a = 0.0f, L = 0.0f;
        if (M > -INFINITY) {
            for (int gg = 0; gg < G; gg++) {
                const float e = expf(s_m[gg] - M);
                a = fmaf(s_acc[gg][j], e, a);
                L = fmaf(s_l[gg], e, L);
            }
        }
        mine[j] = a;
        if (j == 0) { mine[HD] = M; mine[HD + 1] = L; }
    }
    if (splits == 1) {
        // nothing to merge
        __syncthreads();
        for (int j = threadIdx.x; j < HD; j += blockDim.x) out[(size_t)z * ldo + h * HD + j] = mine[j] / mine[HD + 1];
        return;
    }
    // ── the last CTA of this head merges the split partials ──
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int ticket = atomicAdd(&tickets[z * H + h], 1);
        s_last = ticket == splits - 1;
        if (s_last) tickets[z * H + h] = 0;          // ready for the next launch
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // Every thread requests its own column of up to 24 split partials together with the (m, l) pairs, so the
    // merge costs one load round trip (more splits: further rounds of 24).
    const float* pbase = ws + ((size_t)z * H + h) * splits * (HD + 2);
    float* s_m2 = &s_acc[0][0];                 // reused: the CTA's own partial has been written out
    float* s_l2 = s_m2 + kMaxSplits;
    for (int sp = threadIdx.x; sp < splits; sp += blockDim.x) {
        s_m2[sp] = __ldcg(pbase + (size_t)sp * (HD + 2) + HD);
        s_l2[sp] = __ldcg(pbase + (size_t)sp * (HD + 2) + HD + 1);
    }
    constexpr int kBatch = 24;
    const int j0 = threadIdx.x;                 // HD ≤ 512 = 4 columns per thread at most; the first one is prefetched here
    float first[kBatch];
#pragma unroll
    for (int q = 0; q < kBatch; q++) first[q] = (j0 < HD && q < splits) ? __ldcg(pbase + (size_t)q * (HD + 2) + j0) : 0.0f;
    __syncthreads();
    float M = -INFINITY;
    for (int sp = 0; sp < splits; sp++) M = fmaxf(M, s_m2[sp]);
    float L = 0.0f;
    for (int sp = 0; sp < splits; sp++) L = fmaf(s_l2[sp], expf(s_m2[sp] - M), L);
    __syncthreads();
    for (int sp = threadIdx.x; sp < splits; sp += blockDim.x) s_m2[sp] = expf(s_m2[sp] - M);
    __syncthreads();
    for (int j = threadIdx.x; j < HD; j += blockDim.x) {
        float a = 0.0f;
        for (int s0 = 0; s0 < splits; s0 += kBatch) {
            float part[kBatch];
            if (j == j0 && s0 == 0) {
#pragma unroll
                for (int q = 0; q < kBatch; q++) part[q] = first[q];
            } else {
#pragma unroll
                for (int q = 0; q < kBatch; q++) part[q] = s0 + q < splits ? __ldcg(pbase + (size_t)(s0 + q) * (HD + 2) + j) : 0.0f;
            }
#pragma unroll
            for (int q = 0; q < kBatch; q++) if (s0 + q < splits) a = fmaf(part[q], s_m2[s0 + q], a);
        }
        out[(size_t)z * ldo + h * HD + j] = a / L;
    }
}



// ───────────── prompt chunks: tiled causal attention ─────────────
// Row-wise decode attention re-reads every key once per query row.  For a chunk of T ≥ 32 tokens this kernel
// lets 32 consecutive query rows of one head share each 64-key tile of K and V through shared memory (fp32 on the
// CUDA cores, online softmax per row):  S = Q·Kᵀ (Q rotated and pre-scaled at load, the K tile's 16-byte chunks
// XOR-swizzled so that the 16-byte reads of a quarter warp never share a bank), mask, running max / sum, P through
// shared memory, O += P·V.
// grid (query tiles, heads, sequences), 256 threads: thread (rg, cg) = (t / 16, t % 16) owns rows 2rg, 2rg+1 —
// the 16 lanes of a row pair are contiguous, row reductions are half-warp shuffles.
constexpr int kPQ = 32, kPK = 64;

template <int HD, typename KT>
__global__ void __launch_bounds__(256, 2) k_attn_prefill_tiled(
        const float* __restrict__ qkv, int q_off, int ld, const KT* __restrict__ kcache, const KT* __restrict__ vcache,
        int maxSeq, const float* __restrict__ posbuf, const float* __restrict__ cosT, const float* __restrict__ sinT,
        float* __restrict__ out, int ldo, int H, float scale, int T) {
    extern __shared__ __align__(16) float sm[];
    float* Qs = sm;                                 // [32][HD]
    float* Ks = Qs + kPQ * HD;                      // [64][HD], 16-byte chunks XOR-swizzled by (key / 4) % 8
    float* Vs = Ks + kPK * HD;                      // [64][HD]
    float* Ps = Vs + kPK * HD;                      // [32][68]
    constexpr int kPsStride = kPK + 4;
    pdl_wait();
    pdl_launch_dependents();
    const int tid = threadIdx.x, rg = tid >> 4, cg = tid & 15;
    const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int t0 = qt * kPQ;
    int pos0 = (int)posbuf[b];
    pos0 = pos0 < 0 ? 0 : pos0;
    const int half = HD >> 1;
    // Q tile: rotate (interleaved pairs) at position pos0 + t and fold in the 1/sqrt(hd) scale
    for (int i = tid; i < kPQ * half; i += 256) {
        const int r = i / half, pr = i % half;
        const int t = t0 + r;
        float x0 = 0.0f, x1 = 0.0f;
        if (t < T && pos0 + t < maxSeq) {
            const float2 v = *reinterpret_cast<const float2*>(qkv + (size_t)(b * T + t) * ld + q_off + h * HD + 2 * pr);
            const float c = cosT[(size_t)(pos0 + t) * half + pr], s = sinT[(size_t)(pos0 + t) * half + pr];
            x0 = (v.x * c - v.y * s) * scale;
            x1 = (v.x * s + v.y * c) * scale;
        }
        Qs[r * HD + 2 * pr] = x0;
        Qs[r * HD + 2 * pr + 1] = x1;
    }
    const KT* kb = kcache + ((size_t)b * H + h) * maxSeq * HD;
    const KT* vb = vcache + ((size_t)b * H + h) * maxSeq * HD;
    const int lastKey = min(maxSeq - 1, pos0 + min(T, t0 + kPQ) - 1);       // newest key any row of this tile may see
    const int r0 = 2 * rg, r1 = 2 * rg + 1;
    const int lim0 = pos0 + t0 + r0, lim1 = pos0 + t0 + r1;                  // row r attends to keys ≤ lim
    constexpr int kOC = HD / 16;                                             // output columns per thread
    float o0[kOC], o1[kOC];
#pragma unroll
    for (int j = 0; j < kOC; j++) { o0[j] = 0.0f; o1[j] = 0.0f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;
    for (int k0 = 0; k0 <= lastKey; k0 += kPK) {
        __syncthreads();                            // the previous tile's K, V and P are no longer read (first round: Q is written)
        // K tile, transposed, and V tile
        for (int i = tid; i < kPK * (HD / 4); i += 256) {
            const int key = i / (HD / 4), d4 = i % (HD / 4);
            float4 kv = make_float4(0.f, 0.f, 0.f, 0.f), vv = kv;
            if (k0 + key <= lastKey) {
                kv = KvIo<KT>::ld4(kb + (size_t)(k0 + key) * HD + 4 * d4);
                vv = KvIo<KT>::ld4(vb + (size_t)(k0 + key) * HD + 4 * d4);
            }
            *reinterpret_cast<float4*>(Ks + key * HD + 4 * (d4 ^ ((key >> 2) & 7))) = kv;
            *reinterpret_cast<float4*>(Vs + key * HD + 4 * d4) = vv;
        }
        __syncthreads();
        // S = Q·Kᵀ for rows r0, r1 and keys 4cg … 4cg+3
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
        const int sw = cg & 7;                      // (key / 4) % 8 of this thread's four keys
#pragma unroll 4
        for (int c = 0; c < HD / 4; c++) {
            const float4 q0 = *reinterpret_cast<const float4*>(Qs + r0 * HD + 4 * c);
            const float4 q1 = *reinterpret_cast<const float4*>(Qs + r1 * HD + 4 * c);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float4 k4 = *reinterpret_cast<const float4*>(Ks + (4 * cg + j) * HD + 4 * (c ^ sw));
                s0[j] = fmaf(q0.x, k4.x, s0[j]); s0[j] = fmaf(q0.y, k4.y, s0[j]); s0[j] = fmaf(q0.z, k4.z, s0[j]); s0[j] = fmaf(q0.w, k4.w, s0[j]);
                s1[j] = fmaf(q1.x, k4.x, s1[j]); s1[j] = fmaf(q1.y, k4.y, s1[j]); s1[j] = fmaf(q1.z, k4.z, s1[j]); s1[j] = fmaf(q1.w, k4.w, s1[j]);
            }
        }
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int key = k0 + 4 * cg + j;
            if (key > lim0 || key > lastKey) s0[j] = -INFINITY;
            if (key > lim1 || key > lastKey) s1[j] = -INFINITY;
            mx0 = fmaxf(mx0, s0[j]); mx1 = fmaxf(mx1, s1[j]);
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) { mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o)); }
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float c0 = mn0 > -INFINITY ? expf(m0 - mn0) : 1.0f, c1 = mn1 > -INFINITY ? expf(m1 - mn1) : 1.0f;
        float ps0 = 0.0f, ps1 = 0.0f;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float p0 = s0[j] > -INFINITY ? expf(s0[j] - mn0) : 0.0f, p1 = s1[j] > -INFINITY ? expf(s1[j] - mn1) : 0.0f;
            Ps[r0 * kPsStride + 4 * cg + j] = p0; Ps[r1 * kPsStride + 4 * cg + j] = p1;
            ps0 += p0; ps1 += p1;
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) { ps0 += __shfl_xor_sync(0xffffffffu, ps0, o); ps1 += __shfl_xor_sync(0xffffffffu, ps1, o); }
        l0 = l0 * c0 + ps0; l1 = l1 * c1 + ps1;
        m0 = mn0; m1 = mn1;
#pragma unroll
        for (int j = 0; j < kOC; j++) { o0[j] *= c0; o1[j] *= c1; }
        __syncthreads();
        // O += P·V for rows r0, r1 and columns kOC·cg … kOC·cg + kOC − 1
        const int nk = min(kPK, lastKey - k0 + 1);
        for (int key = 0; key < nk; key++) {
            const float p0 = Ps[r0 * kPsStride + key], p1 = Ps[r1 * kPsStride + key];
            const float* vr = Vs + key * HD + kOC * cg;
#pragma unroll
            for (int j = 0; j < kOC; j += 4) {
                const float4 v4 = *reinterpret_cast<const float4*>(vr + j);
                o0[j] = fmaf(p0, v4.x, o0[j]); o0[j + 1] = fmaf(p0, v4.y, o0[j + 1]); o0[j + 2] = fmaf(p0, v4.z, o0[j + 2]); o0[j + 3] = fmaf(p0, v4.w, o0[j + 3]);
                o1[j] = fmaf(p1, v4.x, o1[j]); o1[j + 1] = fmaf(p1, v4.y, o1[j + 1]); o1[j + 2] = fmaf(p1, v4.z, o1[j + 2]); o1[j + 3] = fmaf(p1, v4.w, o1[j + 3]);
            }
        }
    }
    if (t0 + r0 < T && l0 > 0.0f) {
        float* dst = out + (size_t)(b * T + t0 + r0) * ldo + h * HD + kOC * cg;
#pragma unroll
        for (int j = 0; j < kOC; j++) dst[j] = o0[j] / l0;
    }
    if (t0 + r1 < T && l1 > 0.0f) {
        float* dst = out + (size_t)(b * T + t0 + r1) * ldo + h * HD + kOC * cg;
#pragma unroll
        for (int j = 0; j < kOC; j++) dst[j] = o1[j] / l1;
    }
}

template <int HD> constexpr size_t prefill_tiled_smem() { return (size_t)(kPQ * HD + kPK * HD + kPK * HD + kPQ * (kPK + 4)) * 4; }

}  // namespace

int attn_decode_splits(int B, int H, int maxSeq) {
    int want = (4 * g_num_sms) / (B * H);           // every CTA resident at once: a second, nearly empty wave would double the time
    int cap = (maxSeq + 63) / 64;
    int s = want < cap ? want : cap;
    if (s > 256) s = 256;                           // the merge keeps one weight per split in shared memory
    return s < 1 ? 1 : s;
}
size_t attn_decode_ws_floats(int B, int H, int hd, int splits) {
    return (size_t)B * H * splits * (hd + 2);
}

namespace {

template <typename KT>
void launch_attn_decode_t(const AttnDecodeArgs& a, cudaStream_t s) {
    int lpp = a.hd / 16;
    if (a.hd % 16 != 0 || (lpp != 1 && lpp != 2 && lpp != 4 && lpp != 8 && lpp != 16 && lpp != 32))
        throw std::runtime_error("attention: head dim " + std::to_string(a.hd) + " is not one of 16,32,64,128,256,512");
    const int T = a.T < 1 ? 1 : a.T;
    const long rows = (long)a.B * T;
    if (rows > 65535) throw std::runtime_error("attention: more than 65535 rows in one launch");
    dim3 grid(a.splits, a.H, (unsigned)rows), block(kAttnWarps * 32);
    if (a.splits > 1 && rows * a.H > kAttnTickets / 2) throw std::runtime_error("attention: rows × heads exceeds " + std::to_string(kAttnTickets / 2));
    KT* kc = static_cast<KT*>(a.kcache);
    KT* vc = static_cast<KT*>(a.vcache);
    if (T > 1) {
        // the chunk's keys (rotated) and values go into the cache first; the attention kernel then only reads
        dim3 ag(a.H, (unsigned)rows);
        launch_k(k_kv_append<KT>, ag, dim3(a.hd / 2), 0, s, true, (const float*)a.qkv, a.k_off, a.v_off, a.ld, kc, vc, a.maxSeq,
                 a.pos, a.cosT, a.sinT, a.H, a.hd, T);
    }
    static const bool noTiled = getenv("DEEPJ_CUDA_NO_TILED_PREFILL") != nullptr;
    static const bool noMma = getenv("DEEPJ_CUDA_NO_MMA_PREFILL") != nullptr;
    if (T >= kPQ && !noTiled && !noMma && launch_attn_prefill_mma(a, s)) return;      // tensor-core tiles (attn_mma.cu)
    if (T >= kPQ && !noTiled && (a.hd == 64 || a.hd == 128)) {
        dim3 tg((T + kPQ - 1) / kPQ, a.H, a.B);
        if (a.hd == 128) {
            static bool attr = false;
            if (!attr) { DJ_CUDA_CHECK(cudaFuncSetAttribute(k_attn_prefill_tiled<128, KT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)prefill_tiled_smem<128>())); attr = true; }
            launch_k(k_attn_prefill_tiled<128, KT>, tg, dim3(256), prefill_tiled_smem<128>(), s, true, (const float*)a.qkv, a.q_off, a.ld,
                     (const KT*)kc, (const KT*)vc, a.maxSeq, a.pos, a.cosT, a.sinT, a.out, a.ldo, a.H, a.scale, T);
        } else {
            static bool attr = false;
            if (!attr) { DJ_CUDA_CHECK(cudaFuncSetAttribute(k_attn_prefill_tiled<64, KT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)prefill_tiled_smem<64>())); attr = true; }
            launch_k(k_attn_prefill_tiled<64, KT>, tg, dim3(256), prefill_tiled_smem<64>(), s, true, (const float*)a.qkv, a.q_off, a.ld,
                     (const KT*)kc, (const KT*)vc, a.maxSeq, a.pos, a.cosT, a.sinT, a.out, a.ldo, a.H, a.scale, T);
        }
        return;
    }
    const int append = T == 1 ? 1 : 0;
    int* tickets = a.tickets;
    // fp16 cache: K/V stream through warp-private rings in dynamic shared memory (3 stages × 1024 elements each, reused for
    // the partial rows afterwards); fp32 cache: through registers (k_attn_decode_regs)
    const size_t smem = std::max<size_t>((size_t)kAttnWarps * 3 * 1024 * sizeof(KT), (size_t)(4 * 512 + 2 * 4 * 32) * sizeof(float));
#define DJ_ATTN_CASE(L)                                                                                              \
    case L: {                                                                                                        \
        static bool attr = false;                                                                                    \
        if (!attr) { DJ_CUDA_CHECK(cudaFuncSetAttribute(k_attn_decode<L, KT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024)); attr = true; } \
        if (sizeof(KT) == 2)                                                                                         \
            launch_k(k_attn_decode<L, KT>, grid, block, smem, s, true, (const float*)a.qkv, a.q_off, a.k_off, a.v_off, a.ld, \
                     kc, vc, a.maxSeq, a.pos, a.cosT, a.sinT, a.ws, tickets, a.out, a.ldo, a.H, a.scale, T, append); \
        else                                                                                                         \
            launch_k(k_attn_decode_regs<L, KT>, grid, block, 0, s, true, (const float*)a.qkv, a.q_off, a.k_off, a.v_off, a.ld, \
                     kc, vc, a.maxSeq, a.pos, a.cosT, a.sinT, a.ws, tickets, a.out, a.ldo, a.H, a.scale, T, append); \
    } break;
    switch (lpp) {
        DJ_ATTN_CASE(1) DJ_ATTN_CASE(2) DJ_ATTN_CASE(4) DJ_ATTN_CASE(8) DJ_ATTN_CASE(16) DJ_ATTN_CASE(32)
    }
#undef DJ_ATTN_CASE
}

}  // namespace

void launch_attn_decode(const AttnDecodeArgs& a, cudaStream_t s) {
    if (a.kvHalf) launch_attn_decode_t<__half>(a, s);
    else launch_attn_decode_t<float>(a, s);
}

}  // namespace dj

// ───────────── attention without any allocation ─────────────
// Scratch for deepj_cuda_attn_decode_static: the split partials and the ticket counters
// live in this fixed array instead of the runtime's growable workspace.  Every GPU that
// loads the library holds these 2 MiB + 16 KiB until the process exits.
namespace {
constexpr size_t kStaticPartialFloats = 512 * 1024;     // 2 MiB of (acc[hd], m, l) records
constexpr size_t kStaticTickets = 4096;                 // batch × heads
static __device__ __align__(256) float g_attn_static_scratch[kStaticPartialFloats + kStaticTickets];

// The array's name is only a host-side handle; the device address comes from
// cudaGetSymbolAddress, asked once per device with that device current.
float* g_static_scratch_addr[64] = {};
}  // namespace

extern "C" int deepj_cuda_attn_decode_static(int32_t qkv, int32_t q_off, int32_t k_off, int32_t v_off, int32_t ld,
                                             int32_t kv, int32_t layer, int32_t pos, int32_t cos_table, int32_t sin_table,
                                             int32_t out, int32_t out_off, int32_t ldo, int32_t B, int32_t H, int32_t hd) {
    using namespace dj;
    try {
        cudaStream_t stream = runtime_stream();
        if (stream == nullptr) throw std::runtime_error("attn_decode_static: the library holds no buffers yet (nothing was allocated through it)");
        const int dev = runtime_device();
        if (dev < 0 || dev >= 64) throw std::runtime_error("attn_decode_static: device index out of range");
        // the library's device is made current for the length of this call and the caller's is put back on every way out
        struct DeviceGuard {
            int prev = -1; bool switched = false;
            ~DeviceGuard() { if (switched) cudaSetDevice(prev); }
        } guard;
        DJ_CUDA_CHECK(cudaGetDevice(&guard.prev));
        if (guard.prev != dev) { DJ_CUDA_CHECK(cudaSetDevice(dev)); guard.switched = true; }
        if (g_static_scratch_addr[dev] == nullptr) {
            // first call on this device: resolve the scratch array's device address
            float* p = nullptr;
            DJ_CUDA_CHECK(cudaGetSymbolAddress((void**)&p, g_attn_static_scratch));
            if (p == nullptr) throw std::runtime_error("attn_decode_static: scratch address is null");
            g_static_scratch_addr[dev] = p;
        }
        float* scratch = g_static_scratch_addr[dev];

        PoolKV kvb; PoolF32 bq, bp, bc, bs, bo;
        if (!pool_kv(kv, &kvb)) throw std::runtime_error("attn_decode_static: missing KV cache id=" + std::to_string(kv));
        if (!pool_f32(qkv, &bq) || !pool_f32(pos, &bp) || !pool_f32(cos_table, &bc) || !pool_f32(sin_table, &bs) || !pool_f32(out, &bo))
            throw std::runtime_error("attn_decode_static: missing GPU buffer");
        if (B < 1 || H < 1 || hd < 2 || B > kvb.B || H != kvb.H || hd != kvb.hd) throw std::runtime_error("attn_decode_static: shape does not match the KV cache");
        if (layer < 0 || layer >= kvb.layers) throw std::runtime_error("attn_decode_static: layer out of range");
        if (q_off < 0 || k_off < 0 || v_off < 0 || out_off < 0 || ld % 4 || q_off % 4 || k_off % 4 || v_off % 4)
            throw std::runtime_error("attn_decode_static: offsets and stride must be non-negative multiples of 4 floats");
        const int d = H * hd;
        const int maxOff = std::max(q_off, std::max(k_off, v_off));
        if (ld < maxOff + d || ldo < d) throw std::runtime_error("attn_decode_static: row stride smaller than the row");
        if (bq.floats < (size_t)(B - 1) * ld + maxOff + d || bp.floats < (size_t)B || bo.floats < (size_t)out_off + (size_t)(B - 1) * ldo + d ||
            bc.floats < (size_t)kvb.maxSeq * (hd / 2) || bs.floats < (size_t)kvb.maxSeq * (hd / 2))
            throw std::runtime_error("attn_decode_static: a buffer is smaller than the op needs");
        const int splits = attn_decode_splits(B, H, kvb.maxSeq);
        const size_t need = attn_decode_ws_floats(B, H, hd, splits);
        if (need > kStaticPartialFloats || (size_t)B * H > kStaticTickets)
            throw std::runtime_error("attn_decode_static: needs " + std::to_string(need) + " scratch floats and " + std::to_string((size_t)B * H) +
                                     " counters; the static scratch holds " + std::to_string(kStaticPartialFloats) + " and " +
                                     std::to_string(kStaticTickets) + " (use op 67 through deepj_cuda_flush_ops for larger shapes)");
        int* tickets = reinterpret_cast<int*>(scratch + kStaticPartialFloats);
        // the array keeps whatever the last call left: the counters must start at zero
        DJ_CUDA_CHECK(cudaMemsetAsync(tickets, 0, (size_t)B * H * sizeof(int), stream));
        AttnDecodeArgs a = {};
        a.qkv = bq.ptr; a.q_off = q_off; a.k_off = k_off; a.v_off = v_off; a.ld = ld;
        const size_t esz = kvb.half ? 2 : 4;
        const size_t plane = (size_t)kvb.layers * kvb.B * kvb.H * kvb.maxSeq * kvb.hd;
        const size_t layerOff = (size_t)layer * kvb.B * kvb.H * kvb.maxSeq * kvb.hd;
        a.kcache = static_cast<char*>(kvb.ptr) + layerOff * esz; a.vcache = static_cast<char*>(kvb.ptr) + (plane + layerOff) * esz;
        a.maxSeq = kvb.maxSeq; a.kvHalf = kvb.half;
        a.pos = bp.ptr; a.cosT = bc.ptr; a.sinT = bs.ptr;
        a.out = bo.ptr + out_off; a.ldo = ldo; a.B = B; a.H = H; a.hd = hd;
        a.scale = (float)(1.0 / std::sqrt((double)hd));
        a.splits = splits; a.ws = scratch; a.tickets = tickets;
        launch_attn_decode(a, stream);
        DJ_CUDA_CHECK(cudaStreamSynchronize(stream));
        return 0;
    } catch (const std::exception& e) {
        set_last_error(e.what());
        return 1;
    }
}

