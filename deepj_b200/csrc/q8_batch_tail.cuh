// The end of a work item of the small-batch Q8 kernels (q8_batch.cu, q8_batch_tma.cu): a warp has left the partial
// sums of its 16-row tile and K slice in the workspace record; the warp that arrives last at the tile (a ticket
// counter per tile) adds the slices in slice order — deterministic — and runs the epilogue (RMSNorm's 1/rms from the
// Σx² the staging CTAs left per slice, bias, residual, SiLU-gate).
#pragma once
#include "kernels.h"

namespace dj {

constexpr int kBatchMaxRows = 16;                       // activation rows per launch
constexpr int kBatchTileFloats = kBatchMaxRows * 16;    // one (tile, slice) record: partial sums [16 activation rows][16 weight rows]

struct BatchTail {
    const float* gamma; float eps;
    const float* bias; const float* bias2;
    const float* residual; int ldr;
    float* out; int ldo;
    int K, N, M, nSlices;
    float* ws; float* ssq; int* tickets;
};

// The merge and epilogue of one tile, run by the warp whose ticket was the last one (after a __threadfence()).
template <bool SWIGLU>
__device__ __forceinline__ void batch_merge_tile(const BatchTail& t, int tile, int nChunksK) {
    constexpr int rowsPerTile = SWIGLU ? 8 : 16;
    constexpr int kTileFloats = kBatchTileFloats;
    constexpr int kMaxRows = kBatchMaxRows;
    const int lane = threadIdx.x & 31;
    float inv = 1.0f;
    if (t.gamma && lane < t.M) {
        float ss = 0.0f;
        for (int c = 0; c < nChunksK; c++) ss += __ldcg(t.ssq + c * kMaxRows + lane);
        inv = __frcp_rn(sqrtf(ss * (1.0f / (float)t.K) + t.eps));
    }
    // every lane owns up to 8 outputs (SwiGLU: 4 gate/up pairs); the partials of 4 slices × all of them
    // are requested before any is added, so a tile costs one load round trip per 4 slices
    const float* base = t.ws + (size_t)tile * t.nSlices * kTileFloats;
    const int nOut = t.M * rowsPerTile;
    constexpr int kIdx = SWIGLU ? 4 : 8;
    constexpr int kSliceBatch = 4;
    float v[kIdx], u[kIdx];
#pragma unroll
    for (int i = 0; i < kIdx; i++) { v[i] = 0.0f; u[i] = 0.0f; }
    for (int s0 = 0; s0 < t.nSlices; s0 += kSliceBatch) {
        float tv[kIdx][kSliceBatch], tu[SWIGLU ? kIdx : 1][kSliceBatch];
#pragma unroll
        for (int i = 0; i < kIdx; i++) {
            const int idx = lane + 32 * i;
            const int m = idx / rowsPerTile, r = idx % rowsPerTile;
#pragma unroll
            for (int q = 0; q < kSliceBatch; q++) {
                const bool ok = idx < nOut && s0 + q < t.nSlices;
                const float* src = base + (size_t)(s0 + q) * kTileFloats + m * 16 + r;
                tv[i][q] = ok ? __ldcg(src) : 0.0f;
                if (SWIGLU) tu[i][q] = ok ? __ldcg(src + 8) : 0.0f;
            }
        }
#pragma unroll
        for (int i = 0; i < kIdx; i++)
#pragma unroll
            for (int q = 0; q < kSliceBatch; q++) { v[i] += tv[i][q]; if (SWIGLU) u[i] += tu[i][q]; }
    }
#pragma unroll
    for (int i = 0; i < kIdx; i++) {
        const int idx = lane + 32 * i;
        const int m = idx / rowsPerTile, r = idx % rowsPerTile;
        const float invm = __shfl_sync(0xffffffffu, inv, m & 31);
        const int n = tile * rowsPerTile + r;
        if (idx >= nOut || n >= t.N) continue;
        float vv = v[i] * invm;
        if (SWIGLU) {
            float uu = u[i] * invm;
            if (t.bias) vv += t.bias[n];
            if (t.bias2) uu += t.bias2[n];
            const float sig = 1.0f / (1.0f + expf(-vv));
            t.out[(size_t)m * t.ldo + n] = (vv * sig) * uu;
        } else {
            if (t.bias) vv += t.bias[n];
            if (t.residual) vv += t.residual[(size_t)m * t.ldr + n];
            t.out[(size_t)m * t.ldo + n] = vv;
        }
    }
}

// One tile at a time: publish the record, take a ticket, merge if it was the last.
template <bool SWIGLU>
__device__ __forceinline__ void batch_finish_tile(const BatchTail& t, int tile, int nChunksK) {
    const int lane = threadIdx.x & 31;
    // ── the warp that arrives last at this tile adds the slices, in slice order, and finishes the outputs ──
    __threadfence();
    __syncwarp();
    int last = 0;
    if (lane == 0) {
        const int ticket = atomicAdd(&t.tickets[tile], 1);
        last = ticket == t.nSlices - 1;
        if (last) t.tickets[tile] = 0;                  // ready for the next launch
    }
    last = __shfl_sync(0xffffffffu, last, 0);
    if (!last) return;
    __threadfence();
    batch_merge_tile<SWIGLU>(t, tile, nChunksK);
}

}  // namespace dj
