// One decode step of a Llama-shaped Q8 model as ONE persistent kernel (op 76).
//
// Replaces, for batch 1, the per-operator launches of a token step (embedding gather, per block
// RMSNorm → QKV projection, RoPE + KV append + attention, Wo + residual, RMSNorm → SwiGLU, down +
// residual, then final norm → LM head → greedy pick → position advance): what
// DecoderOnlyModel.forward (models/DecoderOnlyModel.java:58-64) and LlamaTransformerBlock.forward
// (layers/transformer/blocks/LlamaTransformerBlock.java:50-53) compute for the last row, and
// TextGenerator's topK = 1 pick (models/TextGenerator.java:91-100).
//
// Why one kernel: a batch-1 token is ≈ 160 dependent operators of 3–25 µs; launched one by one,
// each pays ≈ 5 µs around its streaming phase (dependency release, activation staging, tail).
// Here one cooperative grid of one 16-warp CTA per SM walks the phases and meets at device-side
// barriers.  The Q8 weights of ALL phases form one static sequence of ring items per warp (16 weight
// rows × 64 codes + 32 scales = 1152 bytes, cp.async into a warp-private shared-memory ring, 8
// deep), and the producer side of a ring runs ahead of the consumer ACROSS phase boundaries: while a
// CTA waits at a barrier, stages activations or runs attention, its rings fill with the next
// projection's weights, so HBM keeps streaming through the dependency chain.
//
// The arithmetic is the per-operator kernels' (q8_gemv_i8.cu, attn.cu), instruction for
// instruction: int8 codes as the A operand of mma.sync m16n8k32, activations as three base-256
// digit columns with a power-of-two scale per 32-k block, split-KV attention with a ticket merge —
// at the same tile, warp and split assignments, so one GPU produces the same bits either way.
//
// A CTA's 16 warps work as two halves of 8 (each half owns a weight-row tile at a time, like one
// CTA of the GEMV kernel; the halves share the staged activations) and, in the attention phase,
// as four groups of 4 warps (each takes one (head, split) item).
//
// Tensor parallelism: the row-parallel projections (Wo, down) leave partial sums; their epilogue
// pushes them as {bits, epoch} words into every rank's exchange buffer over NVLink (plain peer
// stores), the CTAs then add the ranks' words in rank order for a slice of the row each (+ residual,
// + bias), and the next phase stages the sum — the exchange is part of this kernel.  The LM head is
// split by vocabulary columns; every rank publishes its best (key, index) pair and all ranks pick
// the same token.
//
// Every wait (grid barrier, peer words) is bounded: when the bound expires the CTA records a code
// in the device error word (300 + phase for a barrier, 100 + rank for a peer), stops waiting for the
// rest of the launch, drains its copies and runs to the end.  The results of such a launch are
// garbage; the context stays usable.
#include "../../include/deepj_cuda.h"
#include "kernels.h"
#include "q8_common.cuh"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <unordered_map>

namespace dj {

namespace {

constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
constexpr int kHalfWarps = 8;                   // warps that share a weight-row tile
constexpr int kRows = 16;
constexpr int kRowStride = 64;
constexpr int kSlotBytes = kRows * kRowStride + kRows * 2 * 4;      // 1152: 16 rows × 64 codes, then 32 scales
constexpr int kDepth = 8;                       // ring slots per warp
constexpr int kXsPad = 32;
constexpr int kStageRounds = 2;                 // rows of up to 2·512·16 = 16384 values are staged from registers
constexpr int kMaxSplits = 256;
constexpr int kSubWarps = 4;                    // warps of an attention group
constexpr int kAttnScratchFloats = 2048 + 128;  // per group: G × HD partial rows, then m and l per position group
constexpr unsigned kSpinLimit = 1u << 22;
constexpr int kMaxWorld = 8;

struct DsLayer {                // one block's device pointers (a table in global memory)
    const float* g1; const int8_t* qkv_c; const float* qkv_s;
    const int8_t* wo_c; const float* wo_s;
    const float* g2; const int8_t* wg_c; const float* wg_s; const float* bg;
    const int8_t* wu_c; const float* wu_s; const float* bu;
    const int8_t* wd_c; const float* wd_s; const float* bd;
    float* kcache; float* vcache;
};

struct DsPhase {                // a projection's weight stream as the ring producer sees it
    const int8_t* codes; const float* scales; const int8_t* codes2; const float* scales2;
    int K, N, swiglu, pad;
};

struct DsPeers { unsigned long long* words[kMaxWorld]; };

struct DsParams {
    const DsLayer* layers; int n_layers;
    const float* emb; float* tok; float* pos; const float* cosT; const float* sinT;
    float* x; float* x2; float* qkv; float* att; float* h; float* part; float* logits; float* next;
    const float* gF; const int8_t* lm_c; const float* lm_s; const float* blm;
    int d, H, hd, F, V, vocab, maxSeq, splits, kmax;
    float eps, scale;
    float* attn_ws; int* tickets; unsigned* bar; int* pick; int* error;
    int feed_back;
    // tensor parallelism (world == 1: unused)
    int rank, world;
    DsPeers peers;                      // every rank's exchange words (mine included)
    unsigned* epoch;                    // the last exchange tag handed out (device counter, advanced by CTA 0 at the end)
};

// ── small device helpers ──
__device__ __forceinline__ void bar_sync(int id, int nthreads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory"); }
__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void cp_async_wait_dyn(int n) {
    switch (n) {
        case 0: cp_async_wait<0>(); break;
        case 1: cp_async_wait<1>(); break;
        case 2: cp_async_wait<2>(); break;
        case 3: cp_async_wait<3>(); break;
        case 4: cp_async_wait<4>(); break;
        case 5: cp_async_wait<5>(); break;
        case 6: cp_async_wait<6>(); break;
        default: cp_async_wait<7>(); break;
    }
}
static_assert(kDepth == 8, "cp_async_wait_dyn covers ring depths up to 8");
__device__ __forceinline__ void load16_cg(const float* src, float (&v)[16]) {       // rows written by other SMs in this launch: L2, never a stale L1 line
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float4 v4 = __ldcg(reinterpret_cast<const float4*>(src) + j);
        v[4 * j] = v4.x; v[4 * j + 1] = v4.y; v[4 * j + 2] = v4.z; v[4 * j + 3] = v4.w;
    }
}
// Float.compare's total order as a signed key (models/TextGenerator.java:163-170): -0.0 < +0.0, NaN above +inf.
__device__ __forceinline__ int order_key(float v) {
    int b = (v != v) ? 0x7fc00000 : __float_as_int(v);
    return b ^ ((b >> 31) & 0x7fffffff);
}
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint2 ld_volatile_v2(const void* p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_volatile_v2(void* p, uint2 v) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}

template <int LPP>      // lanes per cached position = head dim / 16
__global__ void __launch_bounds__(kThreads, 1) k_decode_step(const DsParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int HD = LPP * 16;
    constexpr int PPW = 32 / LPP;
    constexpr int G = kSubWarps * PPW;              // position groups of an attention group
    // layout: rings [16][kDepth][1152] | activation digits (3 columns) + block scales, overlaid by the attention scratch |
    //         tile partials [2 halves][2][8 warps][128] | phase descriptors [2 layers][4] | reductions
    unsigned char* rings = smem;
    unsigned char* actRegion = rings + (size_t)kWarps * kDepth * kSlotBytes;
    const int actBytes = max(3 * (p.kmax + kXsPad) + (p.kmax >> 5) * 4, 4 * kAttnScratchFloats * 4);
    float* s_part = reinterpret_cast<float*>(actRegion + ((actBytes + 127) & ~127));
    DsPhase* s_desc = reinterpret_cast<DsPhase*>(s_part + 2 * 2 * kHalfWarps * 128);
    float* s_red = reinterpret_cast<float*>(s_desc + 8);             // [16]
    int* s_flags = reinterpret_cast<int*>(s_red + kWarps);           // [0] dead, [1..4] attention group "last" flags, [8..] pick scratch
    int8_t* xd = reinterpret_cast<int8_t*>(actRegion);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int half = warp >> 3, hw = warp & 7, htid = tid & 255;
    const int g = lane >> 2, t = lane & 3;
    const int nCtas = gridDim.x;
    const int vcta = 2 * blockIdx.x + half, nV = 2 * nCtas;           // a half = one virtual CTA of the GEMV tiling
    const int L = p.n_layers;
    const int nWp = 4 * L + 1;                                         // weight phases: 4 per block, then the LM head
    const bool tp = p.world > 1;

    if (tid == 0) s_flags[0] = 0;
    // token and position of this step (they change only at the very end of the launch)
    const int tokId = (int)__ldcg(p.tok);
    const bool tokOk = tokId >= 0 && tokId < p.vocab;
    int pos = (int)__ldcg(p.pos);
    pos = pos < 0 ? 0 : (pos >= p.maxSeq ? p.maxSeq - 1 : pos);
    const float* embRow = p.emb + (size_t)(tokOk ? tokId : 0) * p.d;
    // Exchange e of this launch (Wo of block l: 2l, down: 2l + 1, the pick: 2L) travels under tag epochBase + 1 + e.  All
    // ranks run the same launches, so their counters agree; words of exchange e − 2 (same slot parity) carry an older tag.
    const unsigned epochBase = tp ? ld_acquire(p.epoch) : 0u;

    // ── phase descriptors ──
    auto load_desc = [&](int layer) {          // threads 0..3 fill the four descriptors of `layer` (layer == L: the LM head)
        if (tid < 4) {
            DsPhase d; d.codes = nullptr; d.scales = nullptr; d.codes2 = nullptr; d.scales2 = nullptr; d.K = 32; d.N = 0; d.swiglu = 0; d.pad = 0;
            if (layer < L) {
                const DsLayer* ly = p.layers + layer;
                const int dl = p.H * HD;
                if (tid == 0) { d.codes = ly->qkv_c; d.scales = ly->qkv_s; d.K = p.d; d.N = 3 * dl; }
                if (tid == 1) { d.codes = ly->wo_c; d.scales = ly->wo_s; d.K = dl; d.N = p.d; }
                if (tid == 2) { d.codes = ly->wg_c; d.scales = ly->wg_s; d.codes2 = ly->wu_c; d.scales2 = ly->wu_s; d.K = p.d; d.N = p.F; d.swiglu = 1; }
                if (tid == 3) { d.codes = ly->wd_c; d.scales = ly->wd_s; d.K = p.F; d.N = p.d; }
            } else if (layer == L && tid == 0) {
                d.codes = p.lm_c; d.scales = p.lm_s; d.K = p.d; d.N = p.V;
            }
            s_desc[(layer & 1) * 4 + tid] = d;
        }
    };
    load_desc(0);
    load_desc(1);
    __syncthreads();

    // ── ring producer: this warp's static sequence of (phase, tile, 64-k pair) items ──
    unsigned char* myring = rings + (size_t)warp * kDepth * kSlotBytes;
    const uint32_t ring_s = smem_u32(myring);
    uint32_t dstoff[2]; int rsel[2], pieceOff[2];
#pragma unroll
    for (int j = 0; j < 2; j++) {
        const int q = lane + 32 * j, r = q >> 2, piece = q & 3;
        dstoff[j] = (uint32_t)(r * kRowStride + ((piece ^ (((r >> 1) & 1) << 1)) * 16));
        rsel[j] = r; pieceOff[j] = piece * 16;
    }
    const int srow = lane >> 1;
    const uint32_t sdst = (uint32_t)(kRows * kRowStride + lane * 4);
    int wp = 0, itile = 0, ipi = 0, islot = 0, ahead = 0, cslot = 0;
    int cl = 0;                                   // the block the consumer side is in: the producer may be one block ahead
    int pN = 0, pK = 0, pnb = 0, pnPairs = 0, pnTiles = 0, pnBlocks = 0, prpt = 16;
    int rloc[2], sloc = 0;
    const int8_t* cbase[2]; const float* sbase = nullptr;
    const int8_t* csrc[2]; const float* ssrc = nullptr;
    auto set_issue_tile = [&]() {
#pragma unroll
        for (int j = 0; j < 2; j++) csrc[j] = cbase[j] + (size_t)min(itile * prpt + rloc[j], pN - 1) * pK;
        ssrc = sbase + (size_t)min(itile * prpt + sloc, pN - 1) * pnb;
    };
    auto set_phase = [&](int w) {
        const DsPhase& d = s_desc[((w >> 2) & 1) * 4 + (w & 3)];
        const bool sw = d.swiglu != 0;
        prpt = sw ? 8 : 16; pN = d.N; pK = d.K; pnb = d.K >> 5; pnBlocks = d.K >> 5; pnPairs = (pnBlocks + 1) >> 1;
        pnTiles = (pN + prpt - 1) / prpt;
#pragma unroll
        for (int j = 0; j < 2; j++) {
            rloc[j] = sw ? (rsel[j] & 7) : rsel[j];
            cbase[j] = ((sw && rsel[j] >= 8) ? d.codes2 : d.codes) + pieceOff[j];
        }
        sloc = sw ? (srow & 7) : srow;
        sbase = ((sw && srow >= 8) ? d.scales2 : d.scales) + (lane & 1);
        itile = vcta; ipi = hw;
        if (itile < pnTiles) set_issue_tile();
    };
    set_phase(0);
    auto can_issue = [&]() -> bool {
        while (true) {
            if (wp >= nWp) return false;
            if (itile < pnTiles && ipi < pnPairs) return true;
            if (((wp + 1) >> 2) > cl + 1) return false;       // descriptors exist for the consumer's block and the next one
            wp++;
            if (wp < nWp) set_phase(wp);
        }
    };
    auto top_up = [&]() {
        while (ahead < kDepth && can_issue()) {
            const uint32_t dst = ring_s + (uint32_t)islot * kSlotBytes;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + dstoff[0]), "l"(csrc[0] + ipi * 64) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + dstoff[1]), "l"(csrc[1] + ipi * 64) : "memory");
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + sdst), "l"(ssrc + min(ipi * 2, pnBlocks - 1 - (lane & 1))) : "memory");
            cp_async_commit();
            ipi += kHalfWarps;
            if (ipi >= pnPairs) { ipi = hw; itile += nV; if (itile < pnTiles) set_issue_tile(); }
            islot = islot + 1 == kDepth ? 0 : islot + 1;
            ahead++;
        }
    };
    top_up();

    // ── grid barrier (bounded) ──
    unsigned barGen = 0;
    auto grid_barrier = [&](int code) {
        __syncthreads();
        if (tid == 0 && s_flags[0] == 0) {
            barGen++;
            const unsigned target = barGen * (unsigned)nCtas;
            __threadfence();
            atomicAdd(p.bar, 1u);
            unsigned it = 0;
            while (ld_acquire(p.bar) < target) {
                if (++it > kSpinLimit) { atomicCAS(p.error, 0, code); s_flags[0] = 1; break; }
                if (it > 4096u) __nanosleep(64);
                if ((it & 0xffffu) == 0u && *reinterpret_cast<volatile int*>(p.error) != 0) { s_flags[0] = 1; break; }
            }
            __threadfence();
        }
        __syncthreads();
    };

    // ── activation staging: one row → three int8 digit columns + a power-of-two scale per 32-k block (RMSNorm fused) ──
    auto stage = [&](const float* xrow, bool nanRow, const float* gamma, int K) {
        const int ldxs = K + kXsPad;
        float* xsc = reinterpret_cast<float*>(xd + (size_t)3 * ldxs);
        const int nHalf = K >> 4;
        const int rounds = (nHalf + kThreads - 1) / kThreads;
        float xv[kStageRounds][16];
#pragma unroll
        for (int r = 0; r < kStageRounds; r++) {
            const int hb = r * kThreads + tid;
            if (r < rounds && hb < nHalf && !nanRow) load16_cg(xrow + hb * 16, xv[r]);
            else {
#pragma unroll
                for (int j = 0; j < 16; j++) xv[r][j] = (nanRow && r < rounds && hb < nHalf) ? NAN : 0.0f;
            }
        }
        float inv = 1.0f;
        if (gamma) {
            float ss = 0.0f;
#pragma unroll
            for (int r = 0; r < kStageRounds; r++)
#pragma unroll
                for (int j = 0; j < 16; j++) ss = fmaf(xv[r][j], xv[r][j], ss);
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (lane == 0) s_red[warp] = ss;
            __syncthreads();
            ss = 0.0f;
#pragma unroll
            for (int q = 0; q < kWarps; q++) ss += s_red[q];
            inv = __frcp_rn(sqrtf(ss * (1.0f / (float)K) + p.eps));      // RMSNorm1D.forward: x / rms · γ
        }
#pragma unroll
        for (int r = 0; r < kStageRounds; r++) {
            const int hb = r * kThreads + tid;
            const bool on = r < rounds && hb < nHalf;
            if (gamma) {
                float gv[16];
                if (on) load16(gamma + hb * 16, true, gv);
                else {
#pragma unroll
                    for (int j = 0; j < 16; j++) gv[j] = 1.0f;
                }
#pragma unroll
                for (int j = 0; j < 16; j++) xv[r][j] = (xv[r][j] * inv) * gv[j];
            }
            if (r < rounds) digits16(xv[r], on, xd, ldxs, hb, xsc);
        }
        __syncthreads();
    };

    // ── one projection: this half's tiles of the current weight phase against the staged row ──
    // mode 0: out = v (+bias) (+residual); 1: SiLU(gate + bias) ⊙ (up + bias2); 2: logits (+bias) and the running greedy pick;
    // 3: partial sum pushed to every rank's exchange words (tensor parallelism)
    int bestKey = INT_MIN, bestIdx = INT_MAX;
    auto gemv = [&](int cp, int mode, const float* bias, const float* bias2, const float* residual, bool resNan, float* out,
                    unsigned long long wordBase, unsigned tag) {
        if (wp < cp) { wp = cp; set_phase(cp); }          // a warp without items in earlier phases catches up
        const DsPhase& d = s_desc[((cp >> 2) & 1) * 4 + (cp & 3)];
        const int K = d.K, N = d.N;
        const bool sw = d.swiglu != 0;
        const int rowsPerTile = sw ? 8 : 16;
        const int nTiles = (N + rowsPerTile - 1) / rowsPerTile;
        const int nBlocks = K >> 5, nPairs = (nBlocks + 1) >> 1;
        const int ldxs = K + kXsPad;
        const float* xsc = reinterpret_cast<const float*>(xd + (size_t)3 * ldxs);
        // lane (g,t) feeds MMA column g: digit g (g < 3) of the one activation row; columns 3..7 stay zero
        const bool hasCol = g < 3;
        const unsigned char* xcol = reinterpret_cast<const unsigned char*>(xd) + (size_t)(hasCol ? g : 0) * ldxs + t * 8;
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        int aoff[2];
#pragma unroll
        for (int hh = 0; hh < 2; hh++) aoff[hh] = g * kRowStride + (hh ^ ((g >> 1) & 1)) * 32 + t * 8;
        const int soff = kRows * kRowStride + g * 8;
        float* partBase = s_part + (size_t)half * 2 * kHalfWarps * 128;
        int buf = 0;
        for (int tile = vcta; tile < nTiles; tile += nV) {
            const int er = htid, en = tile * rowsPerTile + er;          // htid < rowsPerTile: the thread that finishes output en
            float ebias = 0.0f, ebias2 = 0.0f, eres = 0.0f;
            if (er < rowsPerTile && en < N) {
                if (bias) ebias = bias[en];
                if (sw && bias2) ebias2 = bias2[en];
                if (residual) eres = resNan ? NAN : __ldcg(residual + en);
            }
            for (int pi = hw; pi < nPairs; pi += kHalfWarps) {
                top_up();
                cp_async_wait_dyn(ahead - 1);
                __syncwarp();
                const unsigned char* slot = myring + (size_t)cslot * kSlotBytes;
#pragma unroll
                for (int hh = 0; hh < 2; hh++) {
                    const uint2 a = *reinterpret_cast<const uint2*>(slot + aoff[hh]);
                    const uint2 dd = *reinterpret_cast<const uint2*>(slot + aoff[hh] + 8 * kRowStride);
                    const float s0 = *reinterpret_cast<const float*>(slot + soff + hh * 4);
                    const float s1 = *reinterpret_cast<const float*>(slot + soff + 64 + hh * 4);
                    const int blk = pi * 2 + hh;
                    uint2 xb = make_uint2(0u, 0u);
                    if (hasCol) xb = *reinterpret_cast<const uint2*>(xcol + blk * 32);
                    int cc[4] = {0, 0, 0, 0};
                    mma_s8_16832(cc, a.x, dd.x, a.y, dd.y, xb.x, xb.y);
                    const float xs_ = blk < nBlocks ? xsc[blk] : 0.0f;
                    const float f0 = s0 * xs_, f1 = s1 * xs_;
                    acc[0] = fmaf(f0, (float)cc[0], acc[0]);
                    acc[1] = fmaf(f0, (float)cc[1], acc[1]);
                    acc[2] = fmaf(f1, (float)cc[2], acc[2]);
                    acc[3] = fmaf(f1, (float)cc[3], acc[3]);
                }
                __syncwarp();
                cslot = cslot + 1 == kDepth ? 0 : cslot + 1;
                ahead--;
            }
            // tile epilogue: reduce the half's warps, recombine the digits
            float* part = partBase + (size_t)buf * kHalfWarps * 128;
            float* mine = part + hw * 128;
            mine[g * 8 + 2 * t] = acc[0];       mine[g * 8 + 2 * t + 1] = acc[1];
            mine[(g + 8) * 8 + 2 * t] = acc[2]; mine[(g + 8) * 8 + 2 * t + 1] = acc[3];
            acc[0] = acc[1] = acc[2] = acc[3] = 0.0f;
            bar_sync(1 + half, 256);
            if (er < rowsPerTile && en < N) {
                float a2 = 0.0f, a1 = 0.0f, a0 = 0.0f, b2 = 0.0f, b1 = 0.0f, b0 = 0.0f;
#pragma unroll
                for (int q = 0; q < kHalfWarps; q++) {
                    const float* pr = part + q * 128 + er * 8;
                    a2 += pr[0]; a1 += pr[1]; a0 += pr[2];
                    if (sw) { b2 += pr[64]; b1 += pr[65]; b0 += pr[66]; }
                }
                float v = fmaf(a2, 65536.0f, fmaf(a1, 256.0f, a0));
                if (mode == 1) {
                    float u = fmaf(b2, 65536.0f, fmaf(b1, 256.0f, b0));
                    if (bias) v += ebias;
                    if (bias2) u += ebias2;
                    const float sig = 1.0f / (1.0f + expf(-v));
                    out[en] = (v * sig) * u;                 // SiLU(gate) ⊙ up
                } else if (mode == 3) {
                    // the partial sum travels with the launch's epoch in one 8-byte word, to every rank (this one included)
                    const uint2 w = make_uint2(__float_as_uint(v), tag);
#pragma unroll 1
                    for (int r = 0; r < p.world; r++) st_volatile_v2(p.peers.words[r] + wordBase + (size_t)p.rank * p.d + en, w);
                } else {
                    if (bias) v += ebias;
                    if (residual) v += eres;
                    out[en] = v;
                    if (mode == 2) {
                        const int k = order_key(v);
                        if (k > bestKey || (k == bestKey && en < bestIdx)) { bestKey = k; bestIdx = en; }
                    }
                }
            }
            buf ^= 1;
        }
        top_up();          // whatever the next phases allow: these copies run through the barrier that follows
    };

    // ── sum of the ranks' partial words for a slice of the row: out = residual + bias + Σ_r part_r, rank order ──
    auto tp_reduce = [&](unsigned long long wordBase, unsigned epochNow, const float* bias, const float* residual, bool resNan, float* out) {
        // two values (16 bytes) per thread; CTA c takes pairs c·512 + tid, …
        const int pairs = p.d >> 1;
        for (int pr = blockIdx.x * kThreads + tid; pr < pairs; pr += nCtas * kThreads) {
            float sa = 0.0f, sb = 0.0f;
            bool gaveUp = s_flags[0] != 0;
            for (int r = 0; r < p.world; r++) {
                const unsigned long long* src = p.peers.words[p.rank] + wordBase + (size_t)r * p.d + 2 * pr;
                uint4 v = ld_volatile_v4(src);
                if (v.y != epochNow || v.w != epochNow) {
                    gaveUp = gaveUp || *reinterpret_cast<volatile int*>(p.error) != 0;
                    for (unsigned it = 0; !gaveUp && (v.y != epochNow || v.w != epochNow) && it < kSpinLimit; it++) {
                        if (it > 1024u) __nanosleep(32);
                        v = ld_volatile_v4(src);
                        if ((it & 1023u) == 1023u) gaveUp = *reinterpret_cast<volatile int*>(p.error) != 0;
                    }
                    if (v.y != epochNow || v.w != epochNow) {
                        if (!gaveUp) atomicCAS(p.error, 0, 100 + r);
                        gaveUp = true;
                    }
                }
                sa += __uint_as_float(v.x); sb += __uint_as_float(v.z);
            }
            float ra = 0.0f, rb = 0.0f;
            if (residual) { if (resNan) { ra = NAN; rb = NAN; } else { const float2 rr = __ldcg(reinterpret_cast<const float2*>(residual) + pr); ra = rr.x; rb = rr.y; } }
            if (bias) { ra += bias[2 * pr]; rb += bias[2 * pr + 1]; }
            out[2 * pr] = ra + sa;
            out[2 * pr + 1] = rb + sb;
            if (gaveUp) s_flags[0] = 1;          // the CTA stops waiting at barriers too
        }
    };

    // ── attention of one block: 4-warp groups take (head, split) items ──
    const int sub = warp >> 2, w4 = warp & 3, st = tid & 127;
    const int group = lane / LPP, gl = lane % LPP;
    const int item = sub * nCtas + blockIdx.x;
    const bool attnOn = item < p.H * p.splits;
    const int ah = attnOn ? item / p.splits : 0, asplit = attnOn ? item % p.splits : 0;
    const int seq = pos + 1;
    const int achunk = (seq + p.splits - 1) / p.splits;
    const int astart = asplit * achunk, aend = min(seq, astart + achunk);
    const int halfHd = HD >> 1;
    float* s_acc = reinterpret_cast<float*>(actRegion) + (size_t)sub * kAttnScratchFloats;      // [G][HD]
    float* s_m = s_acc + 2048;                                                                    // [G], then s_l [G]
    float* s_l = s_m + G;

    auto fetch_cached = [&](const float* kb, const float* vb, int pp, bool valid, float (&kx)[16], float (&vx)[16]) {
        if (valid) {
            const float4* kp = reinterpret_cast<const float4*>(kb + (size_t)pp * HD);
            const float4* vp = reinterpret_cast<const float4*>(vb + (size_t)pp * HD);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float4 a = __ldcs(kp + j), c = __ldcs(vp + j);
                kx[4 * j] = a.x; kx[4 * j + 1] = a.y; kx[4 * j + 2] = a.z; kx[4 * j + 3] = a.w;
                vx[4 * j] = c.x; vx[4 * j + 1] = c.y; vx[4 * j + 2] = c.z; vx[4 * j + 3] = c.w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; j++) { kx[j] = 0.0f; vx[j] = 0.0f; }
        }
    };

    for (int l = 0; l < L; l++) {
        const DsLayer* ly = p.layers + l;
        if (l > 0) load_desc(l + 1);        // into the slot block l−1 used; nobody reads it any more (visible after the staging barriers)
        cl = l;
        const float* xin = l == 0 ? embRow : p.x;
        const bool xinNan = l == 0 && !tokOk;

        // ── RMSNorm → QKV projection ──
        stage(xin, xinNan, ly->g1, p.d);
        gemv(4 * l, 0, nullptr, nullptr, nullptr, false, p.qkv, 0ull, 0u);

        // ── attention: the cached rows below `pos` do not depend on this launch, so the first group is requested
        //    before the barrier that publishes q, k, v ──
        float* kbase = ly->kcache + (size_t)ah * p.maxSeq * HD + gl * 16;
        float* vbase = ly->vcache + (size_t)ah * p.maxSeq * HD + gl * 16;
        float kf[16], vf[16];
        float cs[8], sn[8];
        if (attnOn) {
            const int p0 = astart + w4 * PPW + group;
            fetch_cached(kbase, vbase, p0, p0 < aend && p0 != pos, kf, vf);
            const float4* cp4 = reinterpret_cast<const float4*>(p.cosT + (size_t)pos * halfHd + gl * 8);
            const float4* sp4 = reinterpret_cast<const float4*>(p.sinT + (size_t)pos * halfHd + gl * 8);
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const float4 c4 = cp4[j], s4 = sp4[j];
                cs[4 * j] = c4.x; cs[4 * j + 1] = c4.y; cs[4 * j + 2] = c4.z; cs[4 * j + 3] = c4.w;
                sn[4 * j] = s4.x; sn[4 * j + 1] = s4.y; sn[4 * j + 2] = s4.z; sn[4 * j + 3] = s4.w;
            }
        }
        grid_barrier(300 + 0);
        if (attnOn) {
            const int dl = p.H * HD;
            float q[16];
            load16_cg(p.qkv + ah * HD + gl * 16, q);
            auto rotate = [&](float (&v)[16]) {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const float x0 = v[2 * i], x1 = v[2 * i + 1];
                    v[2 * i] = x0 * cs[i] - x1 * sn[i];
                    v[2 * i + 1] = x0 * sn[i] + x1 * cs[i];
                }
            };
            rotate(q);
            auto fetch = [&](int pp, bool valid, float (&kx)[16], float (&vx)[16]) {
                if (valid && pp == pos) {
                    // the new token: k and v come from the projections; rotate k, append both to the cache
                    load16_cg(p.qkv + dl + ah * HD + gl * 16, kx);
                    load16_cg(p.qkv + 2 * dl + ah * HD + gl * 16, vx);
                    rotate(kx);
                    float4* kd = reinterpret_cast<float4*>(kbase + (size_t)pp * HD);
                    float4* vd = reinterpret_cast<float4*>(vbase + (size_t)pp * HD);
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        kd[j] = make_float4(kx[4 * j], kx[4 * j + 1], kx[4 * j + 2], kx[4 * j + 3]);
                        vd[j] = make_float4(vx[4 * j], vx[4 * j + 1], vx[4 * j + 2], vx[4 * j + 3]);
                    }
                } else fetch_cached(kbase, vbase, pp, valid, kx, vx);
            };
            float m = -INFINITY, lsum = 0.0f, acc[16];
#pragma unroll
            for (int j = 0; j < 16; j++) acc[j] = 0.0f;
            int base = astart + w4 * PPW;
            if (base < aend) {
                const int p0 = base + group;
                if (p0 == pos && p0 < aend) fetch(p0, true, kf, vf);
            }
            float kn[16], vn[16];
            for (; base < aend; base += G) {
                const bool valid = base + group < aend;
                const int nbase = base + G;
                if (nbase < aend) fetch(nbase + group, nbase + group < aend, kn, vn);
                float dot = 0.0f;
#pragma unroll
                for (int j = 0; j < 16; j++) dot = fmaf(q[j], kf[j], dot);
#pragma unroll
                for (int o = LPP / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                if (valid) {
                    const float s = dot * p.scale;
                    const float mn = fmaxf(m, s);
                    const float corr = expf(m - mn);
                    const float pe = expf(s - mn);
                    lsum = lsum * corr + pe;
#pragma unroll
                    for (int j = 0; j < 16; j++) acc[j] = fmaf(pe, vf[j], acc[j] * corr);
                    m = mn;
                }
#pragma unroll
                for (int j = 0; j < 16; j++) { kf[j] = kn[j]; vf[j] = vn[j]; }
            }
            const int gg0 = w4 * PPW + group;
#pragma unroll
            for (int j = 0; j < 16; j++) s_acc[gg0 * HD + gl * 16 + j] = acc[j];
            if (gl == 0) { s_m[gg0] = m; s_l[gg0] = lsum; }
            bar_sync(3 + sub, 128);
            float* mine = p.attn_ws + ((size_t)ah * p.splits + asplit) * (HD + 2);
            for (int j = st; j < HD; j += 128) {
                float M = -INFINITY;
                for (int gg = 0; gg < G; gg++) M = fmaxf(M, s_m[gg]);
                float a = 0.0f, Ls = 0.0f;
                if (M > -INFINITY) {
                    for (int gg = 0; gg < G; gg++) {
                        const float e = expf(s_m[gg] - M);
                        a = fmaf(s_acc[gg * HD + j], e, a);
                        Ls = fmaf(s_l[gg], e, Ls);
                    }
                }
                mine[j] = a;
                if (j == 0) { mine[HD] = M; mine[HD + 1] = Ls; }
            }
            if (p.splits == 1) {
                bar_sync(3 + sub, 128);
                for (int j = st; j < HD; j += 128) p.att[ah * HD + j] = mine[j] / mine[HD + 1];
            } else {
                // the last group of this head merges the split partials
                __threadfence();
                bar_sync(3 + sub, 128);
                if (st == 0) {
                    const int ticket = atomicAdd(&p.tickets[ah], 1);
                    const int last = ticket == p.splits - 1;
                    s_flags[1 + sub] = last;
                    if (last) p.tickets[ah] = 0;
                }
                bar_sync(3 + sub, 128);
                if (s_flags[1 + sub]) {
                    __threadfence();
                    const float* pbase = p.attn_ws + (size_t)ah * p.splits * (HD + 2);
                    float* s_m2 = s_acc;
                    float* s_l2 = s_m2 + kMaxSplits;
                    for (int sp = st; sp < p.splits; sp += 128) {
                        s_m2[sp] = __ldcg(pbase + (size_t)sp * (HD + 2) + HD);
                        s_l2[sp] = __ldcg(pbase + (size_t)sp * (HD + 2) + HD + 1);
                    }
                    constexpr int kBatch = 24;
                    const int j0 = st;
                    float first[kBatch];
#pragma unroll
                    for (int q2 = 0; q2 < kBatch; q2++) first[q2] = (j0 < HD && q2 < p.splits) ? __ldcg(pbase + (size_t)q2 * (HD + 2) + j0) : 0.0f;
                    bar_sync(3 + sub, 128);
                    float M = -INFINITY;
                    for (int sp = 0; sp < p.splits; sp++) M = fmaxf(M, s_m2[sp]);
                    float Lt = 0.0f;
                    for (int sp = 0; sp < p.splits; sp++) Lt = fmaf(s_l2[sp], expf(s_m2[sp] - M), Lt);
                    bar_sync(3 + sub, 128);
                    for (int sp = st; sp < p.splits; sp += 128) s_m2[sp] = expf(s_m2[sp] - M);
                    bar_sync(3 + sub, 128);
                    for (int j = st; j < HD; j += 128) {
                        float a = 0.0f;
                        for (int s0 = 0; s0 < p.splits; s0 += kBatch) {
                            float part[kBatch];
                            if (j == j0 && s0 == 0) {
#pragma unroll
                                for (int q2 = 0; q2 < kBatch; q2++) part[q2] = first[q2];
                            } else {
#pragma unroll
                                for (int q2 = 0; q2 < kBatch; q2++) part[q2] = s0 + q2 < p.splits ? __ldcg(pbase + (size_t)(s0 + q2) * (HD + 2) + j) : 0.0f;
                            }
#pragma unroll
                            for (int q2 = 0; q2 < kBatch; q2++) if (s0 + q2 < p.splits) a = fmaf(part[q2], s_m2[s0 + q2], a);
                        }
                        p.att[ah * HD + j] = a / Lt;
                    }
                }
            }
        }
        grid_barrier(300 + 1);

        // ── Wo + residual ──
        stage(p.att, false, nullptr, p.H * HD);
        if (!tp) {
            gemv(4 * l + 1, 0, nullptr, nullptr, xin, xinNan, p.x2, 0ull, 0u);
            grid_barrier(300 + 2);
        } else {
            const unsigned long long wb = 0ull;                                            // even exchanges: slot parity 0
            gemv(4 * l + 1, 3, nullptr, nullptr, nullptr, false, nullptr, wb, epochBase + 1u + 2u * l);
            tp_reduce(wb, epochBase + 1u + 2u * l, nullptr, xin, xinNan, p.x2);
            grid_barrier(300 + 2);
        }

        // ── RMSNorm → SwiGLU ──
        stage(p.x2, false, ly->g2, p.d);
        gemv(4 * l + 2, 1, ly->bg, ly->bu, nullptr, false, p.h, 0ull, 0u);
        grid_barrier(300 + 3);

        // ── down + bias + residual ──
        stage(p.h, false, nullptr, p.F);
        if (!tp) {
            gemv(4 * l + 3, 0, ly->bd, nullptr, p.x2, false, p.x, 0ull, 0u);
            grid_barrier(300 + 4);
        } else {
            const unsigned long long wb = (unsigned long long)p.world * p.d;               // odd exchanges: slot parity 1
            gemv(4 * l + 3, 3, nullptr, nullptr, nullptr, false, nullptr, wb, epochBase + 2u + 2u * l);
            tp_reduce(wb, epochBase + 2u + 2u * l, ly->bd, p.x2, false, p.x);
            grid_barrier(300 + 4);
        }
    }

    // ── final RMSNorm → LM head → greedy pick ──
    cl = L;
    stage(L == 0 ? embRow : p.x, L == 0 && !tokOk, p.gF, p.d);
    gemv(4 * L, 2, p.blm, nullptr, nullptr, false, p.logits, 0ull, 0u);
    cp_async_wait<0>();
    {
        // CTA-wide best (key, index) of the outputs this CTA finished; lowest index among equal keys
        for (int o = 16; o > 0; o >>= 1) {
            const int k2 = __shfl_xor_sync(0xffffffffu, bestKey, o), i2 = __shfl_xor_sync(0xffffffffu, bestIdx, o);
            if (k2 > bestKey || (k2 == bestKey && i2 < bestIdx)) { bestKey = k2; bestIdx = i2; }
        }
        int* s_pick = s_flags + 8;
        __syncthreads();
        if (lane == 0) { s_pick[2 * warp] = bestKey; s_pick[2 * warp + 1] = bestIdx; }
        __syncthreads();
        if (warp == 0) {
            bestKey = lane < kWarps ? s_pick[2 * lane] : INT_MIN;
            bestIdx = lane < kWarps ? s_pick[2 * lane + 1] : INT_MAX;
            for (int o = 16; o > 0; o >>= 1) {
                const int k2 = __shfl_xor_sync(0xffffffffu, bestKey, o), i2 = __shfl_xor_sync(0xffffffffu, bestIdx, o);
                if (k2 > bestKey || (k2 == bestKey && i2 < bestIdx)) { bestKey = k2; bestIdx = i2; }
            }
            if (lane == 0) {
                // global column index under tensor parallelism: this rank's vocabulary shard starts at rank · V
                p.pick[2 * blockIdx.x] = bestKey;
                p.pick[2 * blockIdx.x + 1] = bestIdx == INT_MAX ? INT_MAX : bestIdx + p.rank * p.V;
            }
        }
    }
    grid_barrier(300 + 5);
    if (blockIdx.x == 0 && warp == 0) {
        bestKey = INT_MIN; bestIdx = INT_MAX;
        for (int c = lane; c < nCtas; c += 32) {
            const int k2 = __ldcg(p.pick + 2 * c), i2 = __ldcg(p.pick + 2 * c + 1);
            if (k2 > bestKey || (k2 == bestKey && i2 < bestIdx)) { bestKey = k2; bestIdx = i2; }
        }
        for (int o = 16; o > 0; o >>= 1) {
            const int k2 = __shfl_xor_sync(0xffffffffu, bestKey, o), i2 = __shfl_xor_sync(0xffffffffu, bestIdx, o);
            if (k2 > bestKey || (k2 == bestKey && i2 < bestIdx)) { bestKey = k2; bestIdx = i2; }
        }
        if (tp) {
            // every rank publishes its best pair in every rank's buffer, then takes the best of all (lowest global index on ties)
            const unsigned epochNow = epochBase + 1u + 2u * (unsigned)L;
            const unsigned long long pb = (unsigned long long)2 * p.world * p.d;       // behind the two parities of partial sums
            if (lane == 0) {
                for (int r = 0; r < p.world; r++) {
                    unsigned long long* dst = p.peers.words[r] + pb + 2 * (size_t)p.rank;
                    st_volatile_v2(dst, make_uint2((unsigned)bestKey, epochNow));
                    st_volatile_v2(dst + 1, make_uint2((unsigned)bestIdx, epochNow));
                }
            }
            int k2 = INT_MIN, i2 = INT_MAX;
            if (lane < p.world) {
                const unsigned long long* src = p.peers.words[p.rank] + pb + 2 * (size_t)lane;
                uint4 v = ld_volatile_v4(src);
                bool gaveUp = *reinterpret_cast<volatile int*>(p.error) != 0;
                for (unsigned it = 0; !gaveUp && (v.y != epochNow || v.w != epochNow) && it < kSpinLimit; it++) {
                    if (it > 1024u) __nanosleep(32);
                    v = ld_volatile_v4(src);
                    if ((it & 1023u) == 1023u) gaveUp = *reinterpret_cast<volatile int*>(p.error) != 0;
                }
                if (v.y != epochNow || v.w != epochNow) { if (!gaveUp) atomicCAS(p.error, 0, 100 + lane); }
                else { k2 = (int)v.x; i2 = (int)v.z; }
            }
            bestKey = k2; bestIdx = i2;
            for (int o = 16; o > 0; o >>= 1) {
                const int k3 = __shfl_xor_sync(0xffffffffu, bestKey, o), i3 = __shfl_xor_sync(0xffffffffu, bestIdx, o);
                if (k3 > bestKey || (k3 == bestKey && i3 < bestIdx)) { bestKey = k3; bestIdx = i3; }
            }
        }
        if (lane == 0) {
            const float pickF = (float)(bestIdx == INT_MAX ? 0 : bestIdx);
            p.next[0] = pickF;
            p.pos[0] = __ldcg(p.pos) + 1.0f;
            if (p.feed_back) p.tok[0] = pickF;
            if (tp) *p.epoch = epochBase + 2u * (unsigned)L + 2u;
        }
    }
    // the last CTA out re-arms the barrier counter for the next launch
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        const unsigned done = atomicAdd(p.bar + 1, 1u);
        if (done == (unsigned)nCtas - 1u) { p.bar[0] = 0u; p.bar[1] = 0u; __threadfence(); }
    }
}

// ───────────── host side: plans ─────────────

struct Plan {
    unsigned long long serial = 0;                 // of the pool object that owns the device block
    std::vector<std::pair<int, unsigned long long>> refs;
    DsParams prm = {};
    int lpp = 0;
    size_t smem = 0;
    bool uses_tp = false;
};
std::unordered_map<int, Plan> g_plans;

size_t ds_smem_bytes(int kmax) {
    const size_t act = std::max<size_t>((size_t)3 * (kmax + kXsPad) + (size_t)(kmax >> 5) * 4, (size_t)4 * kAttnScratchFloats * 4);
    return (size_t)kWarps * kDepth * kSlotBytes + ((act + 127) & ~(size_t)127) + (size_t)2 * 2 * kHalfWarps * 128 * 4 + 8 * sizeof(DsPhase) +
           kWarps * 4 + (8 + 2 * kWarps) * 4;
}

}  // namespace

// Exchange words of the decode-step kernel inside the tensor-parallel buffer (tp.cu): returns null when no buffer is connected.
unsigned long long* tp_step_words(int rank_index);
unsigned* tp_step_epoch();
size_t tp_step_floats();
int tp_rank();

void decode_step_check(int plan_id, std::vector<std::pair<int, unsigned long long>>* refs) {
    auto it = g_plans.find(plan_id);
    if (it == g_plans.end() || it->second.serial != pool_serial(plan_id))
        throw std::runtime_error("decodeStep: id " + std::to_string(plan_id) + " is not a decode plan");
    for (auto& r : it->second.refs) {
        if (pool_serial(r.first) != r.second)
            throw std::runtime_error("decodeStep: the plan references buffer id=" + std::to_string(r.first) + ", which has been released");
        if (refs) refs->push_back(r);
    }
    if (it->second.uses_tp && (!tp_ready() || tp_world() != it->second.prm.world))
        throw std::runtime_error("decodeStep: the plan was made for a tensor-parallel connection that no longer exists");
}

void launch_decode_step(int plan_id, int feed_back, cudaStream_t s) {
    Plan& pl = g_plans.at(plan_id);
    DsParams prm = pl.prm;
    prm.feed_back = feed_back;
    if (pl.uses_tp) {
        for (int r = 0; r < prm.world; r++) prm.peers.words[r] = tp_step_words(r);
        prm.epoch = tp_step_epoch();
    }
    g_launches++;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(g_num_sms); cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = pl.smem; cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;          // all CTAs resident at once: they meet at device-side barriers
    attr[0].val.cooperative = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    switch (pl.lpp) {
        case 2: DJ_CUDA_CHECK(cudaLaunchKernelEx(&cfg, k_decode_step<2>, prm)); break;
        case 4: DJ_CUDA_CHECK(cudaLaunchKernelEx(&cfg, k_decode_step<4>, prm)); break;
        default: DJ_CUDA_CHECK(cudaLaunchKernelEx(&cfg, k_decode_step<8>, prm)); break;
    }
}

}  // namespace dj

using namespace dj;

// desc: [version = 1, n_layers, heads (this rank's), head_dim, epsBits,
//        tok, pos, emb, cos, sin, kv, x, x2, qkv, att, h, logits, next, gF, Wlm, blm,
//        then per block: g1, Wqkv, Wo, g2, Wg, bg, Wu, bu, Wd, bd]
extern "C" int deepj_cuda_decode_plan(int32_t plan_id, const int32_t* desc, int32_t len) {
    try {
        if (runtime_stream() == nullptr) throw std::runtime_error("decode_plan: call deepj_cuda_init first");
        constexpr int kHead = 21, kPerLayer = 10;
        if (desc == nullptr || len < kHead) throw std::runtime_error("decode_plan: descriptor too short");
        if (desc[0] != 1) throw std::runtime_error("decode_plan: unknown descriptor version");
        const int L = desc[1], H = desc[2], hd = desc[3];
        if (L < 0 || len != kHead + L * kPerLayer) throw std::runtime_error("decode_plan: descriptor length does not match the block count");
        if (H < 1 || (hd != 32 && hd != 64 && hd != 128)) throw std::runtime_error("decode_plan: head dim must be 32, 64 or 128");
        if (pool_serial(plan_id) != 0) throw std::runtime_error("decode_plan: id " + std::to_string(plan_id) + " already exists");
        Plan pl;
        auto f32 = [&](int id, size_t need, const char* what) -> float* {
            PoolF32 b;
            if (!pool_f32(id, &b)) throw std::runtime_error(std::string("decode_plan: missing float buffer for ") + what);
            if (b.floats < need) throw std::runtime_error(std::string("decode_plan: buffer too small for ") + what);
            pl.refs.push_back({id, pool_serial(id)});
            return b.ptr;
        };
        auto q8 = [&](int id, int K, int N, const char* what) -> Q8View {
            Q8View v;
            if (!pool_q8(id, &v)) throw std::runtime_error(std::string("decode_plan: missing Q8 object for ") + what);
            if ((K > 0 && v.K != K) || (N > 0 && v.N != N))
                throw std::runtime_error(std::string("decode_plan: ") + what + " is " + std::to_string(v.K) + "x" + std::to_string(v.N) + ", expected " +
                                         std::to_string(K) + "x" + std::to_string(N));
            if (v.K % 32 != 0 || v.Kp != v.K) throw std::runtime_error(std::string("decode_plan: the reduction length of ") + what + " must be a multiple of 32");
            pl.refs.push_back({id, pool_serial(id)});
            return v;
        };
        const int world = tp_ready() ? tp_world() : 1;
        const int dl = H * hd;
        DsParams& P = pl.prm;
        float epsF; std::memcpy(&epsF, &desc[4], 4);
        P.eps = epsF; P.n_layers = L; P.H = H; P.hd = hd;
        Q8View lm = q8(desc[19], 0, 0, "the LM head");
        const int d = lm.K, V = lm.N;
        if (d != dl * world) throw std::runtime_error("decode_plan: dModel must equal heads x head_dim x tensor-parallel ranks");
        if (d % 32 != 0 || d % 2 != 0) throw std::runtime_error("decode_plan: dModel must be a multiple of 32");
        P.d = d; P.V = V; P.lm_c = lm.codes; P.lm_s = lm.scales;
        PoolKV kv;
        if (!pool_kv(desc[10], &kv)) throw std::runtime_error("decode_plan: missing KV cache");
        pl.refs.push_back({desc[10], pool_serial(desc[10])});
        if (kv.layers < L || kv.H != H || kv.hd != hd || kv.B < 1) throw std::runtime_error("decode_plan: the KV cache does not match the model");
        P.maxSeq = kv.maxSeq;
        P.tok = f32(desc[5], 1, "token"); P.pos = f32(desc[6], 1, "position");
        PoolF32 emb;
        if (!pool_f32(desc[7], &emb) || emb.floats % (size_t)d != 0 || emb.floats < (size_t)d) throw std::runtime_error("decode_plan: the embedding table is not [vocab x dModel]");
        pl.refs.push_back({desc[7], pool_serial(desc[7])});
        P.emb = emb.ptr; P.vocab = (int)(emb.floats / (size_t)d);
        P.cosT = f32(desc[8], (size_t)kv.maxSeq * (hd / 2), "cos table"); P.sinT = f32(desc[9], (size_t)kv.maxSeq * (hd / 2), "sin table");
        P.x = f32(desc[11], d, "x"); P.x2 = f32(desc[12], d, "x2"); P.qkv = f32(desc[13], (size_t)3 * dl, "qkv"); P.att = f32(desc[14], dl, "att");
        P.logits = f32(desc[16], V, "logits"); P.next = f32(desc[17], 1, "next");
        P.gF = f32(desc[18], d, "final norm gain"); P.blm = f32(desc[20], V, "LM head bias");
        int F = 0;
        std::vector<DsLayer> table(L);
        const size_t plane = (size_t)kv.layers * kv.B * kv.H * kv.maxSeq * kv.hd;
        for (int l = 0; l < L; l++) {
            const int32_t* e = desc + kHead + l * kPerLayer;
            DsLayer& y = table[l];
            y.g1 = f32(e[0], d, "norm gain 1");
            Q8View w = q8(e[1], d, 3 * dl, "Wqkv"); y.qkv_c = w.codes; y.qkv_s = w.scales;
            w = q8(e[2], dl, d, "Wo"); y.wo_c = w.codes; y.wo_s = w.scales;
            y.g2 = f32(e[3], d, "norm gain 2");
            w = q8(e[4], d, F, "gate"); if (l == 0) F = w.N; y.wg_c = w.codes; y.wg_s = w.scales;
            y.bg = f32(e[5], F, "gate bias");
            w = q8(e[6], d, F, "up"); y.wu_c = w.codes; y.wu_s = w.scales;
            y.bu = f32(e[7], F, "up bias");
            w = q8(e[8], F, d, "down"); y.wd_c = w.codes; y.wd_s = w.scales;
            y.bd = f32(e[9], d, "down bias");
            const size_t layerOff = (size_t)l * kv.B * kv.H * kv.maxSeq * kv.hd;
            y.kcache = kv.ptr + layerOff; y.vcache = kv.ptr + plane + layerOff;
        }
        if (L > 0 && F < 32) throw std::runtime_error("decode_plan: dFF must be at least 32");
        P.F = F;
        P.h = f32(desc[15], std::max(F, 1), "h");
        P.kmax = std::max(std::max(d, dl), F);
        if ((P.kmax >> 4) > kStageRounds * kThreads) throw std::runtime_error("decode_plan: rows longer than " + std::to_string(kStageRounds * kThreads * 16) + " values are not covered");
        P.scale = (float)(1.0 / std::sqrt((double)hd));
        int splits = std::max(1, (4 * g_num_sms) / H);
        splits = std::min(splits, std::min((kv.maxSeq + 63) / 64, kMaxSplits));
        P.splits = std::max(1, splits);
        P.rank = 0; P.world = world;
        if (world > 1) {
            if (world > kMaxWorld) throw std::runtime_error("decode_plan: more than 8 tensor-parallel ranks");
            if (tp_step_floats() < (size_t)2 * world * d + 2 * (size_t)world + 8)
                throw std::runtime_error("decode_plan: the tensor-parallel exchange buffer is too small for the decode-step kernel (connect with a slot of at least dModel floats)");
            P.rank = tp_rank();
            pl.uses_tp = true;
        }
        pl.lpp = hd / 16;
        pl.smem = ds_smem_bytes(P.kmax);
        if (pl.smem > 227 * 1024) throw std::runtime_error("decode_plan: the model's rows do not fit the kernel's shared memory");
        // one device block: the layer table, then scratch (attention partials, tickets, barrier words, pick pairs)
        const size_t tableBytes = ((size_t)L * sizeof(DsLayer) + 255) & ~(size_t)255;
        const size_t wsFloats = (size_t)H * P.splits * (hd + 2);
        const size_t scratchBytes = wsFloats * 4 + (size_t)H * 4 + 16 * 4 + (size_t)2 * g_num_sms * 4 + 256;
        char* block = nullptr;
        DJ_CUDA_CHECK(cudaMalloc((void**)&block, tableBytes + scratchBytes));
        DJ_CUDA_CHECK(cudaMemset(block, 0, tableBytes + scratchBytes));
        if (L > 0) DJ_CUDA_CHECK(cudaMemcpy(block, table.data(), (size_t)L * sizeof(DsLayer), cudaMemcpyHostToDevice));
        P.layers = reinterpret_cast<const DsLayer*>(block);
        P.attn_ws = reinterpret_cast<float*>(block + tableBytes);
        P.tickets = reinterpret_cast<int*>(P.attn_ws + wsFloats);
        P.bar = reinterpret_cast<unsigned*>(P.tickets + H);
        P.pick = reinterpret_cast<int*>(P.bar + 16);
        P.error = g_dev_error;
        static bool attrSet[3] = {false, false, false};
        const int ai = pl.lpp == 2 ? 0 : (pl.lpp == 4 ? 1 : 2);
        if (!attrSet[ai]) {
            if (pl.lpp == 2) DJ_CUDA_CHECK(cudaFuncSetAttribute(k_decode_step<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
            else if (pl.lpp == 4) DJ_CUDA_CHECK(cudaFuncSetAttribute(k_decode_step<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
            else DJ_CUDA_CHECK(cudaFuncSetAttribute(k_decode_step<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
            attrSet[ai] = true;
        }
        pool_add_plan(plan_id, block, tableBytes + scratchBytes);
        pl.serial = pool_serial(plan_id);
        g_plans[plan_id] = std::move(pl);
        return 0;
    } catch (const std::exception& e) { set_last_error(e.what()); return 1; }
}
