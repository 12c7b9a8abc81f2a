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
// barriers.  The Q8 weights of ALL phases form one static sequence of ring items per warp, and the
// producer side of a ring runs ahead of the consumer ACROSS phase boundaries: while a CTA waits at a
// barrier, stages activations or runs attention, its rings fill with the next projection's weights,
// so HBM keeps streaming through the dependency chain.
//
// The weights are read from a tile-major copy made once per plan (k_pack_phase): the 16 weight rows ×
// 64 codes + 32 scales of a (tile, 64-k pair) are one contiguous 1152-byte image of what the MMA
// fragments read from shared memory (32-byte halves already XOR-swizzled by row), and a tile's pairs
// follow each other, so a ring item — 16 pairs, two for each of the eight warps that share a tile,
// 18 KB — is ONE cp.async.bulk on an mbarrier, issued by one lane of the half (full / empty
// barriers per slot, as in any bulk-copy pipeline).  With the canonical row-major layout every lane
// spent ≈ 100 instructions per 1152 bytes on copy addresses and group bookkeeping, and with one
// small bulk copy per warp the issuing warp stalled ≈ 450 cycles per copy.  The tile-major copy
// costs the plan as much memory again as the Q8 weights it covers.
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
constexpr int kPairBytes = kRows * kRowStride + kRows * 2 * 4;      // 1152: 16 rows × 64 codes, then 32 scales
constexpr int kWarpPairs = 2;                   // 64-k pairs of one warp in a ring item
constexpr int kItemPairs = 8 * kWarpPairs;      // a ring item: 16 consecutive pairs of a tile, two for each warp of the half (18 KB)
constexpr int kSlotBytes = kItemPairs * kPairBytes;
constexpr int kDepth = 4;                       // ring slots per half: three items (55 KB) in flight, one being read
constexpr int kPartBufs = 4;                    // tile partial buffers per half: a warp may run this many tiles ahead of the slowest
constexpr int kPartFloats = 48;                 // 16 weight rows × 3 digit sums per warp and tile
constexpr int kXsPad = 32;
constexpr int kStageRounds = 2;                 // rows of up to 2·512·16 = 16384 values are staged from registers
constexpr int kMaxSplits = 256;
constexpr int kSubWarps = 4;                    // warps of an attention group
constexpr int kAttnScratchFloats = 2048 + 128;  // per group: G × HD partial rows, then m and l per position group
constexpr unsigned kSpinLimit = 1u << 22;
constexpr int kMaxWorld = 8;

struct DsLayer {                // one block's device pointers (a table in global memory)
    const float* g1; const float* g2; const float* bg; const float* bu; const float* bd;
    const unsigned char* w[4];  // tile-major weight streams: Wq‖Wk‖Wv, Wo, gate‖up (8 + 8 rows per tile), down
    float* kcache; float* vcache;
};

struct DsPhase {                // a projection's weight stream as the ring producer sees it
    const unsigned char* packed; int K, N, swiglu, pad;
};

struct DsPeers { unsigned long long* words[kMaxWorld]; };

struct DsParams {
    const DsLayer* layers; int n_layers;
    const float* emb; float* tok; float* pos; const float* cosT; const float* sinT;
    float* x; float* x2; float* qkv; float* att; float* h; float* logits; float* next;
    const float* gF; const unsigned char* lm_w; const float* blm;      // lm_w: the LM head's tile-major stream
    int d, H, hd, F, V, vocab, maxSeq, splits, kmax;
    float eps, scale;
    float* attn_ws; int* tickets; unsigned* bar; int* pick; int* error;
    int feed_back;
    // tensor parallelism (world == 1: unused)
    int rank, world;
    DsPeers peers;                      // every rank's exchange words (mine included)
    unsigned* epoch;                    // the last exchange tag handed out (device counter, advanced by CTA 0 at the end)
    unsigned long long* trace;          // phase tracing (DEEPJ_CUDA_TRACE=1): CTA 0 stamps %globaltimer at the phase boundaries of block 1
};

// ── small device helpers ──
__device__ __forceinline__ void bar_sync(int id, int nthreads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory"); }
__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// Shared-memory loads by 32-bit shared address: the out-of-line phases get their pointers as plain arguments, so the
// compiler cannot prove the address space and would otherwise emit (slower) generic loads.
__device__ __forceinline__ uint2 lds_u2(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ float lds_f(uint32_t a) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
    return v;
}
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
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
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
__device__ __forceinline__ void st_volatile_v2(void* p, uint2 v) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}

// ── shared-memory layout ──
// rings [2 halves][kDepth][18432] | activation digits (3 columns) + block scales, overlaid by the attention scratch |
// tile partials [2 halves][4][8 warps][16 rows × 3 digits] | weight-phase descriptors [2 blocks][4] | block tables [2] | reductions | flags | peers
struct DsSmem {
    unsigned char* rings; unsigned char* act; float* part; DsPhase* desc; DsLayer* lay; float* red; int* flags;
    unsigned long long** peers; unsigned long long* mbar;      // mbar: [2 halves][full | empty][kDepth]
};
__device__ __forceinline__ DsSmem ds_layout(unsigned char* smem, int kmax) {
    DsSmem m;
    m.rings = smem;
    m.act = smem + (size_t)2 * kDepth * kSlotBytes;
    const int actBytes = max(3 * (kmax + kXsPad) + (kmax >> 5) * 4, 4 * kAttnScratchFloats * 4);
    m.part = reinterpret_cast<float*>(m.act + ((actBytes + 127) & ~127));
    m.desc = reinterpret_cast<DsPhase*>(m.part + 2 * kPartBufs * kHalfWarps * kPartFloats);
    m.lay = reinterpret_cast<DsLayer*>(m.desc + 8);
    m.red = reinterpret_cast<float*>(m.lay + 2);
    m.flags = reinterpret_cast<int*>(m.red + kWarps);       // [0] dead, [1..4] attention groups' "last" flags, [5] barrier generation, [8..39] pick pairs,
                                                            // [40..47] tile arrivals [half][buffer], [48..55] tile reductions done [half][buffer]
    m.peers = reinterpret_cast<unsigned long long**>(m.flags + 64);
    m.mbar = reinterpret_cast<unsigned long long*>(m.peers + kMaxWorld);
    return m;
}

// Grid barrier over the cooperative launch, bounded: the generation lives in shared memory (flags[5]); a CTA whose wait
// ran out, or that finds the error word set, marks itself dead (flags[0]) and stops waiting for the rest of the launch.
__device__ __noinline__ void ds_grid_barrier(unsigned* bar, int* error, int* flags, int nCtas, int code) {
    __syncthreads();
    if (threadIdx.x == 0 && flags[0] == 0) {
        const unsigned gen = (unsigned)flags[5] + 1u;
        flags[5] = (int)gen;
        const unsigned target = gen * (unsigned)nCtas;
        __threadfence();
        atomicAdd(bar, 1u);
        unsigned it = 0;
        while (ld_acquire(bar) < target) {
            if (++it > kSpinLimit) { atomicCAS(error, 0, code); flags[0] = 1; break; }
            if (it > 4096u) __nanosleep(64);
            if ((it & 0xffffu) == 0u && *reinterpret_cast<volatile int*>(error) != 0) { flags[0] = 1; break; }
        }
        __threadfence();
    }
    __syncthreads();
}

// A warp's cursors over its static sequence of ring items (weight phase, tile, 64-k pair): the producer side runs up to
// kDepth items ahead of the consumer side, across phase boundaries.  Warp-uniform; lives in the kernel's frame and is
// handed to the out-of-line phases by reference.
struct DsRing {
    int wp, itile, ipi, islot, ahead, cslot;      // producer (warp 0 of a half): phase / tile / next item of the tile / next slot; items issued and not yet consumed; consumer slot
    unsigned par;                                 // bit s: the parity a consumer waits for on full[s] next; bit 16+s: the parity the producer waits for on empty[s] next
    unsigned used;                                // bit s: slot s has been filled before (its empty barrier must complete before the next fill)
    unsigned tileSeq;                             // tiles this half has finished so far (the same in its eight warps)
    int cl;                                       // the block the consumer is in (the producer may be one block ahead)
    int bestKey, bestIdx;                         // running greedy pick of the LM-head outputs this thread finished
};

struct DsCtx {                                    // what every phase needs from the launch
    unsigned char* smem; int kmax, nCtas, nWp;
    int rank, world, d;
    float eps;
};

// The producer of a half's ring — lane 0 of the half's first warp: where the next item of the half's static sequence lies in
// the phase's tile-major stream, and the issue loop.  A slot is refilled once all eight warps have released its previous
// content (its empty barrier); the wait for that is taken only when the producer's own warp has nothing left to consume.
struct DsProducer {
    uint32_t ring_s, full_s, empty_s;
    int vcta, nV, hw, lane;
    int pnTiles, pnPairs, pnItems;                // this phase: tiles, pairs per tile, items per tile
    size_t tileBytes;
    const unsigned char* base;
    const DsPhase* desc; int nWp;
    volatile int* dead; int* error;

    __device__ __forceinline__ void init(const DsSmem& m, int nCtas, int nWp_, int* error_) {
        const int tid = threadIdx.x, warp = tid >> 5, half = warp >> 3;
        lane = tid & 31; hw = warp & 7;
        vcta = 2 * blockIdx.x + half; nV = 2 * nCtas;
        desc = m.desc; nWp = nWp_;
        ring_s = smem_u32(m.rings + (size_t)half * kDepth * kSlotBytes);
        full_s = smem_u32(m.mbar + half * 2 * kDepth);
        empty_s = full_s + kDepth * 8u;
        dead = m.flags; error = error_;
    }
    __device__ __forceinline__ void load_phase(int w) {
        const DsPhase& d = desc[((w >> 2) & 1) * 4 + (w & 3)];
        const int rpt = d.swiglu ? 8 : 16;
        pnTiles = (d.N + rpt - 1) / rpt;
        pnPairs = ((d.K >> 5) + 1) >> 1;
        pnItems = (pnPairs + kItemPairs - 1) / kItemPairs;
        tileBytes = (size_t)pnPairs * kPairBytes;
        base = d.packed;
    }
    __device__ __forceinline__ bool can_issue(DsRing& r) {
        while (true) {
            if (r.wp >= nWp) return false;
            if (r.itile < pnTiles && r.ipi < pnItems) return true;
            if (((r.wp + 1) >> 2) > r.cl + 1) return false;       // descriptors exist for the consumer's block and the next one
            r.wp++;
            r.itile = vcta; r.ipi = 0;
            if (r.wp < nWp) load_phase(r.wp);
        }
    }
    // only the producer warp (hw == 0) calls this; warp-uniform
    __device__ __forceinline__ void top_up(DsRing& r) {
        while (r.ahead < kDepth && can_issue(r)) {
            const uint32_t ebar = empty_s + (uint32_t)r.islot * 8u;
            if ((r.used >> r.islot) & 1u) {
                // the slot's previous content must have been released by all eight warps
                const uint32_t eparity = (r.par >> (16 + r.islot)) & 1u;
                bool ok = mbar_try_wait(ebar, eparity);
                if (!ok) {
                    if (r.ahead > 0) return;                 // this warp still has items to consume: come back later
                    unsigned it = 0;
                    while (!(ok = mbar_try_wait(ebar, eparity))) {
                        if (*dead) break;
                        if (++it > kSpinLimit) { atomicCAS(error, 0, 312); *dead = 1; break; }
                    }
                }
                r.par ^= 1u << (16 + r.islot);
            }
            r.used |= 1u << r.islot;
            const int pairs = min(kItemPairs, pnPairs - r.ipi * kItemPairs);
            if (lane == 0) {
                const uint32_t bar = full_s + (uint32_t)r.islot * 8u;
                const uint32_t bytes = (uint32_t)pairs * kPairBytes;
                mbar_arrive_expect_tx(bar, bytes);
                bulk_g2s(ring_s + (uint32_t)r.islot * kSlotBytes, base + (size_t)r.itile * tileBytes + (size_t)r.ipi * kSlotBytes, bytes, bar);
            }
            r.ipi++;
            if (r.ipi >= pnItems) { r.ipi = 0; r.itile += nV; }
            r.islot = r.islot + 1 == kDepth ? 0 : r.islot + 1;
            r.ahead++;
        }
    }
};

// Fill the rings as far as the descriptors allow (launch start).
__device__ __noinline__ void ds_prefetch(const DsCtx c, DsRing& ring, int* error) {
    const DsSmem m = ds_layout(c.smem, c.kmax);
    DsProducer P;
    P.init(m, c.nCtas, c.nWp, error);
    if (P.hw != 0) return;
    DsRing r = ring;
    P.load_phase(r.wp);
    P.top_up(r);
    ring = r;
}

// Activation staging: one row → three int8 digit columns + a power-of-two scale per 32-k block (RMSNorm fused).
// The gain is a weight: its loads go out together with the row's.
__device__ __noinline__ void ds_stage(const DsCtx c, const float* xrow, int nanRow, const float* gamma, int K) {
    const DsSmem m = ds_layout(c.smem, c.kmax);
    int8_t* xd = reinterpret_cast<int8_t*>(m.act);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int ldxs = K + kXsPad;
    float* xsc = reinterpret_cast<float*>(xd + (size_t)3 * ldxs);
    const int nHalf = K >> 4;
    const int rounds = (nHalf + kThreads - 1) / kThreads;
    float xv[kStageRounds][16], gv[kStageRounds][16];
#pragma unroll
    for (int r = 0; r < kStageRounds; r++) {
        const int hb = r * kThreads + tid;
        const bool on = r < rounds && hb < nHalf;
        if (on && !nanRow) load16_cg(xrow + hb * 16, xv[r]);
        else {
#pragma unroll
            for (int j = 0; j < 16; j++) xv[r][j] = (nanRow && on) ? NAN : 0.0f;
        }
        if (gamma != nullptr && on) load16(gamma + hb * 16, true, gv[r]);
        else {
#pragma unroll
            for (int j = 0; j < 16; j++) gv[r][j] = 1.0f;
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
        if (lane == 0) m.red[warp] = ss;
        __syncthreads();
        ss = 0.0f;
#pragma unroll
        for (int q = 0; q < kWarps; q++) ss += m.red[q];
        inv = __frcp_rn(sqrtf(ss * (1.0f / (float)K) + c.eps));      // RMSNorm1D.forward: x / rms · γ
    }
#pragma unroll
    for (int r = 0; r < kStageRounds; r++) {
        const int hb = r * kThreads + tid;
        const bool on = r < rounds && hb < nHalf;
        if (gamma) {
#pragma unroll
            for (int j = 0; j < 16; j++) xv[r][j] = (xv[r][j] * inv) * gv[r][j];
        }
        if (r < rounds) digits16(xv[r], on, xd, ldxs, hb, xsc);
    }
    __syncthreads();
}

struct DsGemv {
    int cp, mode;                     // weight phase; 0: out = v (+bias) (+residual); 1: SiLU(gate + bias) ⊙ (up + bias2);
                                      // 2: logits (+bias) and the running greedy pick; 3: partial sums pushed to every rank's exchange words
    const float* bias; const float* bias2; const float* residual; int resNan; float* out;
    unsigned long long wordBase; unsigned tag;
};

// One projection: this half's tiles of weight phase `cp` against the staged row.  Warp hw of a half owns the 64-k pairs
// hw, hw+8, … of a tile; every 32-k block of 16 weight rows is ONE int8 MMA whose B operand holds the row's three digits.
__device__ __noinline__ void ds_gemv(const DsCtx c, const DsGemv a, DsRing& ring, int* error) {
    const DsSmem m = ds_layout(c.smem, c.kmax);
    const int8_t* xd = reinterpret_cast<const int8_t*>(m.act);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int half = warp >> 3, hw = warp & 7;
    const int g = lane >> 2, t = lane & 3;
    DsProducer P;
    P.init(m, c.nCtas, c.nWp, error);
    const bool producer = hw == 0;                                           // this warp also feeds the half's ring
    DsRing r = ring;
    if (r.wp < a.cp) { r.wp = a.cp; r.itile = P.vcta; r.ipi = 0; }          // a half without items in earlier phases catches up
    P.load_phase(r.wp);
    const uint32_t myring = P.ring_s + (uint32_t)hw * kPairBytes;            // this warp's first pair inside a slot; its second lies 8 pairs on
    const DsPhase& d = m.desc[((a.cp >> 2) & 1) * 4 + (a.cp & 3)];
    const int K = d.K, N = d.N;
    const bool sw = d.swiglu != 0;
    const int rowsPerTile = sw ? 8 : 16;
    const int nTiles = (N + rowsPerTile - 1) / rowsPerTile;
    const int nBlocks = K >> 5, nPairs = (nBlocks + 1) >> 1;
    const int nItems = (nPairs + kItemPairs - 1) / kItemPairs;               // ring items of a tile; pairs hw, hw+8, … are this warp's
    const int ldxs = K + kXsPad;
    const uint32_t xsc = smem_u32(xd + (size_t)3 * ldxs);
    // lane (g,t) feeds MMA column g: digit g (g < 3) of the one activation row; columns 3..7 stay zero
    const bool hasCol = g < 3;
    const uint32_t xcol = smem_u32(xd) + (uint32_t)((hasCol ? g : 0) * ldxs + t * 8);
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    int aoff[2];
#pragma unroll
    for (int hh = 0; hh < 2; hh++) aoff[hh] = g * kRowStride + (hh ^ ((g >> 1) & 1)) * 32 + t * 8;
    const int soff = kRows * kRowStride + g * 8;
    float* partBase = m.part + (size_t)half * kPartBufs * kHalfWarps * kPartFloats;
    volatile int* arrivals = m.flags + 40 + half * kPartBufs;
    volatile int* reduced = m.flags + 48 + half * kPartBufs;
    int bestKey = r.bestKey, bestIdx = r.bestIdx;
    volatile int* dead = m.flags;
    for (int tile = P.vcta; tile < nTiles; tile += P.nV) {
        // epilogue operands of output row `lane` of the tile, in every warp: whichever arrives last finishes the tile
        const int er = lane, en = tile * rowsPerTile + er;
        float ebias = 0.0f, ebias2 = 0.0f, eres = 0.0f;
        if (er < rowsPerTile && en < N) {
            if (a.bias) ebias = a.bias[en];
            if (sw && a.bias2) ebias2 = a.bias2[en];
            if (a.residual) eres = a.resNan ? NAN : __ldcg(a.residual + en);
        }
        for (int it_ = 0; it_ < nItems; it_++) {
            if (producer) P.top_up(r);
            const uint32_t fbar = P.full_s + (uint32_t)r.cslot * 8u;
            {
                // the item's bytes have landed when its slot's full barrier completes the phase armed for it (bounded wait)
                const uint32_t parity = (r.par >> r.cslot) & 1u;
                if (!mbar_try_wait(fbar, parity) && !*dead) {
                    unsigned it = 0;
                    while (!mbar_try_wait(fbar, parity)) {
                        if (++it > kSpinLimit) { atomicCAS(error, 0, 310); *dead = 1; break; }
                        if ((it & 0xfffu) == 0u && *dead) break;
                    }
                }
                r.par ^= 1u << r.cslot;
            }
            const uint32_t slot = myring + (uint32_t)r.cslot * kSlotBytes;
            // this warp's pairs of the item: hw + 16·it_ and hw + 16·it_ + 8, where they exist
            const int pi0 = it_ * kItemPairs + hw;
            // all fragments first (independent shared-memory loads), then the MMAs, then the fp32 folds
            uint2 av[2 * kWarpPairs], dd[2 * kWarpPairs], xb[2 * kWarpPairs];
            float s0[2 * kWarpPairs], s1[2 * kWarpPairs], xs[2 * kWarpPairs];
#pragma unroll
            for (int q = 0; q < 2 * kWarpPairs; q++) {
                const int pp = q >> 1, hh = q & 1;
                const uint32_t ps = slot + pp * (kHalfWarps * kPairBytes);
                const int pi = pi0 + kHalfWarps * pp, blk = pi * 2 + hh;
                const bool on = pi < nPairs && blk < nBlocks;      // a short last item, or the empty half of an odd last pair
                av[q] = lds_u2(ps + aoff[hh]);
                dd[q] = lds_u2(ps + aoff[hh] + 8 * kRowStride);
                s0[q] = lds_f(ps + soff + hh * 4);
                s1[q] = lds_f(ps + soff + 64 + hh * 4);
                xb[q] = (hasCol && on) ? lds_u2(xcol + blk * 32) : make_uint2(0u, 0u);
                xs[q] = on ? lds_f(xsc + blk * 4) : 0.0f;
            }
            __syncwarp();          // every lane has its fragments: this warp releases the slot
            if (lane == 0) mbar_arrive(P.empty_s + (uint32_t)r.cslot * 8u);
            r.cslot = r.cslot + 1 == kDepth ? 0 : r.cslot + 1;
            r.ahead--;
#pragma unroll
            for (int q = 0; q < 2 * kWarpPairs; q++) {
                int cc[4] = {0, 0, 0, 0};
                mma_s8_16832(cc, av[q].x, dd[q].x, av[q].y, dd[q].y, xb[q].x, xb[q].y);
                // a pair that is not there was not copied either: its slot bytes are stale (possibly NaN patterns), so its fold is skipped
                if (pi0 + kHalfWarps * (q >> 1) < nPairs) {
                    const float f0 = s0[q] * xs[q], f1 = s1[q] * xs[q];
                    // |block sum| ≤ 32·127·128 < 2^22: the integer drops exactly into the mantissa of 1.5·2^23 (one add instead of a convert)
                    acc[0] = fmaf(f0, __int_as_float(0x4B400000 + cc[0]) - 12582912.0f, acc[0]);
                    acc[1] = fmaf(f0, __int_as_float(0x4B400000 + cc[1]) - 12582912.0f, acc[1]);
                    acc[2] = fmaf(f1, __int_as_float(0x4B400000 + cc[2]) - 12582912.0f, acc[2]);
                    acc[3] = fmaf(f1, __int_as_float(0x4B400000 + cc[3]) - 12582912.0f, acc[3]);
                }
            }
        }
        // ── tile epilogue without a barrier: every warp leaves its 16 × 3 digit sums and moves on; the warp that arrives
        //    last adds the eight in warp order (deterministic) and finishes the outputs ──
        const unsigned useNo = r.tileSeq / kPartBufs;
        const int pbuf = (int)(r.tileSeq % kPartBufs);
        r.tileSeq++;
        if ((unsigned)reduced[pbuf] < useNo && !*dead) {          // the buffer's previous tile has not been reduced yet (a warp ran four tiles ahead)
            unsigned it = 0;
            while ((unsigned)reduced[pbuf] < useNo) {
                if (++it > kSpinLimit) { atomicCAS(error, 0, 311); *dead = 1; break; }
                if ((it & 0xfffu) == 0u && *dead) break;
            }
        }
        float* part = partBase + (size_t)pbuf * kHalfWarps * kPartFloats;
        float* mine = part + hw * kPartFloats;
        if (t == 0) {
            mine[g * 3] = acc[0]; mine[g * 3 + 1] = acc[1];
            mine[(g + 8) * 3] = acc[2]; mine[(g + 8) * 3 + 1] = acc[3];
        } else if (t == 1) {
            mine[g * 3 + 2] = acc[0];
            mine[(g + 8) * 3 + 2] = acc[2];
        }
        acc[0] = acc[1] = acc[2] = acc[3] = 0.0f;
        __syncwarp();
        int last = 0;
        if (lane == 0) {
            __threadfence_block();
            const int old = atomicAdd(const_cast<int*>(arrivals + pbuf), 1);
            last = ((old + 1) % kHalfWarps) == 0;
        }
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last) {
            __threadfence_block();
            if (er < rowsPerTile && en < N) {
                float a2 = 0.0f, a1 = 0.0f, a0 = 0.0f, b2 = 0.0f, b1 = 0.0f, b0 = 0.0f;
                const volatile float* vp = part;
#pragma unroll
                for (int q = 0; q < kHalfWarps; q++) {
                    const volatile float* pr = vp + q * kPartFloats + er * 3;
                    a2 += pr[0]; a1 += pr[1]; a0 += pr[2];
                    if (sw) { b2 += pr[24]; b1 += pr[25]; b0 += pr[26]; }
                }
                float v = fmaf(a2, 65536.0f, fmaf(a1, 256.0f, a0));
                if (a.mode == 1) {
                    float u = fmaf(b2, 65536.0f, fmaf(b1, 256.0f, b0));
                    if (a.bias) v += ebias;
                    if (a.bias2) u += ebias2;
                    const float sig = 1.0f / (1.0f + expf(-v));
                    a.out[en] = (v * sig) * u;                 // SiLU(gate) ⊙ up
                } else if (a.mode == 3) {
                    // the partial sum travels with its exchange tag in one 8-byte word, to every rank (this one included)
                    const uint2 w = make_uint2(__float_as_uint(v), a.tag);
#pragma unroll 1
                    for (int q = 0; q < c.world; q++) st_volatile_v2(m.peers[q] + a.wordBase + (size_t)c.rank * c.d + en, w);
                } else {
                    if (a.bias) v += ebias;
                    if (a.residual) v += eres;
                    a.out[en] = v;
                    if (a.mode == 2) {
                        const int k = order_key(v);
                        if (k > bestKey || (k == bestKey && en < bestIdx)) { bestKey = k; bestIdx = en; }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) { __threadfence_block(); reduced[pbuf] = (int)useNo + 1; }
        }
    }
    if (producer) P.top_up(r);          // whatever the next phases allow: these copies run through the barrier that follows
    r.bestKey = bestKey; r.bestIdx = bestIdx;
    ring = r;
}

// Sum of the ranks' partial words for a slice of the row: out = residual + bias + Σ_r part_r, in rank order.
__device__ __noinline__ void ds_tp_reduce(const DsCtx c, unsigned long long wordBase, unsigned tag, const float* bias, const float* residual,
                                          int resNan, float* out, int* error) {
    const DsSmem m = ds_layout(c.smem, c.kmax);
    const int tid = threadIdx.x;
    const int pairs = c.d >> 1;          // two values (16 bytes) per thread; CTA b takes pairs b·512 + tid, …
    for (int pr = blockIdx.x * kThreads + tid; pr < pairs; pr += c.nCtas * kThreads) {
        float sa = 0.0f, sb = 0.0f;
        bool gaveUp = m.flags[0] != 0;
        for (int q = 0; q < c.world; q++) {
            const unsigned long long* src = m.peers[c.rank] + wordBase + (size_t)q * c.d + 2 * pr;
            uint4 v = ld_volatile_v4(src);
            if (v.y != tag || v.w != tag) {
                gaveUp = gaveUp || *reinterpret_cast<volatile int*>(error) != 0;
                for (unsigned it = 0; !gaveUp && (v.y != tag || v.w != tag) && it < kSpinLimit; it++) {
                    if (it > 1024u) __nanosleep(32);
                    v = ld_volatile_v4(src);
                    if ((it & 1023u) == 1023u) gaveUp = *reinterpret_cast<volatile int*>(error) != 0;
                }
                if (v.y != tag || v.w != tag) {
                    if (!gaveUp) atomicCAS(error, 0, 100 + q);
                    gaveUp = true;
                }
            }
            sa += __uint_as_float(v.x); sb += __uint_as_float(v.z);
        }
        float ra = 0.0f, rb = 0.0f;
        if (residual) {
            if (resNan) { ra = NAN; rb = NAN; }
            else { const float2 rr = __ldcg(reinterpret_cast<const float2*>(residual) + pr); ra = rr.x; rb = rr.y; }
        }
        if (bias) { ra += bias[2 * pr]; rb += bias[2 * pr + 1]; }
        out[2 * pr] = ra + sa;
        out[2 * pr + 1] = rb + sb;
        if (gaveUp) m.flags[0] = 1;          // the CTA stops waiting at barriers too
    }
}

struct DsAttn {
    const float* qkv; float* att; float* ws; int* tickets; const float* cosT; const float* sinT;
    float* kcache; float* vcache; unsigned* bar; int* error; float* scratch; int* flags;
    int pos, maxSeq, H, splits, nCtas; float scale;
};

// Attention of one block for the one new token: 4-warp groups of the CTA take (head, split) items.  The cached rows
// below `pos` do not depend on this launch, so a group requests its first rows BEFORE the grid barrier that publishes
// q, k and v, then rotates q, folds its slice of the cache in (the group that meets `pos` takes k and v from the
// projections, rotates k and appends both), and the last group of a head to finish merges the split partials.
template <int LPP>
__device__ __noinline__ void ds_attention(const DsAttn p) {
    constexpr int HD = LPP * 16;
    constexpr int PPW = 32 / LPP;
    constexpr int G = kSubWarps * PPW;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nCtas = p.nCtas, pos = p.pos;
    int* s_flags = p.flags;
    const int sub = warp >> 2, w4 = warp & 3, st = tid & 127;
    const int group = lane / LPP, gl = lane % LPP;
    const int item = sub * nCtas + blockIdx.x;
    const bool attnOn = item < p.H * p.splits;
    const int ah = attnOn ? item / p.splits : 0, asplit = attnOn ? item % p.splits : 0;
    const int seq = pos + 1;
    const int achunk = (seq + p.splits - 1) / p.splits;
    const int astart = asplit * achunk, aend = min(seq, astart + achunk);
    const int halfHd = HD >> 1;
    float* s_acc = p.scratch + (size_t)sub * kAttnScratchFloats;      // [G][HD]
    float* s_m = s_acc + 2048;                                        // [G], then s_l [G]
    float* s_l = s_m + G;
    float* kbase = p.kcache + (size_t)ah * p.maxSeq * HD + gl * 16;
    float* vbase = p.vcache + (size_t)ah * p.maxSeq * HD + gl * 16;

    auto fetch_cached = [&](int pp, bool valid, float (&kx)[16], float (&vx)[16]) {
        if (valid) {
            const float4* kp = reinterpret_cast<const float4*>(kbase + (size_t)pp * HD);
            const float4* vp = reinterpret_cast<const float4*>(vbase + (size_t)pp * HD);
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
    // rotate 8 interleaved pairs by the table row of the current position; the row is fetched where it is used
    // (twice per launch and lane, cache hits) rather than kept live through the loop
    auto rotate = [&](float (&v)[16]) {
        const float4* cp4 = reinterpret_cast<const float4*>(p.cosT + (size_t)pos * halfHd + gl * 8);
        const float4* sp4 = reinterpret_cast<const float4*>(p.sinT + (size_t)pos * halfHd + gl * 8);
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const float4 c4 = cp4[j], s4 = sp4[j];
            const float cs[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float x0 = v[8 * j + 2 * i], x1 = v[8 * j + 2 * i + 1];
                v[8 * j + 2 * i] = x0 * cs[i] - x1 * sn[i];
                v[8 * j + 2 * i + 1] = x0 * sn[i] + x1 * cs[i];
            }
        }
    };

    float kf[16], vf[16];
    if (attnOn) {
        const int p0 = astart + w4 * PPW + group;
        fetch_cached(p0, p0 < aend && p0 != pos, kf, vf);
    }
    ds_grid_barrier(p.bar, p.error, s_flags, nCtas, 300);
    if (!attnOn) return;

    const int dl = p.H * HD;
    float q[16];
    load16_cg(p.qkv + ah * HD + gl * 16, q);
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
        } else fetch_cached(pp, valid, kx, vx);
    };
    float mx = -INFINITY, lsum = 0.0f, acc[16];
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
            const float mn = fmaxf(mx, s);
            const float corr = expf(mx - mn);
            const float pe = expf(s - mn);
            lsum = lsum * corr + pe;
#pragma unroll
            for (int j = 0; j < 16; j++) acc[j] = fmaf(pe, vf[j], acc[j] * corr);
            mx = mn;
        }
#pragma unroll
        for (int j = 0; j < 16; j++) { kf[j] = kn[j]; vf[j] = vn[j]; }
    }
    const int gg0 = w4 * PPW + group;
#pragma unroll
    for (int j = 0; j < 16; j++) s_acc[gg0 * HD + gl * 16 + j] = acc[j];
    if (gl == 0) { s_m[gg0] = mx; s_l[gg0] = lsum; }
    bar_sync(3 + sub, 128);
    float* mine = p.ws + ((size_t)ah * p.splits + asplit) * (HD + 2);
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
        return;
    }
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
    if (!s_flags[1 + sub]) return;
    __threadfence();
    const float* pbase = p.ws + (size_t)ah * p.splits * (HD + 2);
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

template <int LPP>      // lanes per cached position = head dim / 16
__global__ void __launch_bounds__(kThreads, 1) k_decode_step(const DsParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    const DsSmem m = ds_layout(smem, p.kmax);
    int* s_flags = m.flags;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nCtas = gridDim.x;
    const int L = p.n_layers;
    const bool tp = p.world > 1;
    DsCtx c;
    c.smem = smem; c.kmax = p.kmax; c.nCtas = nCtas; c.nWp = 4 * L + 1;      // weight phases: 4 per block, then the LM head
    c.rank = p.rank; c.world = p.world; c.d = p.d; c.eps = p.eps;

    if (tid < 64 && (tid < 8 || tid >= 40)) s_flags[tid] = 0;
    if (tid < kMaxWorld) m.peers[tid] = p.peers.words[tid];
    // full barriers: one arrival (the issuing lane's, with the byte count) per use; empty barriers: one arrival per warp of the half
    if (tid < 2 * 2 * kDepth) mbar_init(smem_u32(m.mbar + tid), ((tid / kDepth) & 1) ? kHalfWarps : 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // token and position of this step (they change only at the very end of the launch)
    const int tokId = (int)__ldcg(p.tok);
    const bool tokOk = tokId >= 0 && tokId < p.vocab;
    int pos = (int)__ldcg(p.pos);
    pos = pos < 0 ? 0 : (pos >= p.maxSeq ? p.maxSeq - 1 : pos);
    const float* embRow = p.emb + (size_t)(tokOk ? tokId : 0) * p.d;
    // Exchange e of this launch (Wo of block l: 2l, down: 2l + 1, the pick: 2L) travels under tag epochBase + 1 + e.  All
    // ranks run the same launches, so their counters agree; words of exchange e − 2 (same slot parity) carry an older tag.
    const unsigned epochBase = tp ? ld_acquire(p.epoch) : 0u;

    // ── block tables and weight-phase descriptors of two blocks at a time (block == L: the LM head) ──
    auto load_block = [&](int layer) {
        // the table entry: a handful of pointers, one per thread
        if (layer < L && tid < (int)(sizeof(DsLayer) / sizeof(void*)))
            reinterpret_cast<const void**>(m.lay + (layer & 1))[tid] = reinterpret_cast<const void* const*>(p.layers + layer)[tid];
        if (tid >= 32 && tid < 36) {
            const int ph = tid - 32;
            DsPhase d; d.packed = nullptr; d.K = 32; d.N = 0; d.swiglu = 0; d.pad = 0;
            if (layer < L) {
                const DsLayer* ly = p.layers + layer;
                const int dl = p.H * LPP * 16;
                d.packed = ly->w[ph];
                if (ph == 0) { d.K = p.d; d.N = 3 * dl; }
                if (ph == 1) { d.K = dl; d.N = p.d; }
                if (ph == 2) { d.K = p.d; d.N = p.F; d.swiglu = 1; }
                if (ph == 3) { d.K = p.F; d.N = p.d; }
            } else if (layer == L && ph == 0) {
                d.packed = p.lm_w; d.K = p.d; d.N = p.V;
            }
            m.desc[(layer & 1) * 4 + ph] = d;
        }
    };
    load_block(0);
    load_block(1);
    __syncthreads();

    DsRing ring;
    ring.wp = 0; ring.itile = 2 * blockIdx.x + (warp >> 3); ring.ipi = 0; ring.islot = 0; ring.ahead = 0; ring.cslot = 0; ring.cl = 0; ring.par = 0u; ring.used = 0u; ring.tileSeq = 0u;
    ring.bestKey = INT_MIN; ring.bestIdx = INT_MAX;
    ds_prefetch(c, ring, p.error);

    auto grid_barrier = [&](int code) { ds_grid_barrier(p.bar, p.error, s_flags, nCtas, code); };
    int stampAt = 0;
    auto stamp = [&](int l) {
        if (p.trace != nullptr && blockIdx.x == 0 && tid == 0 && l == (L > 1 ? 1 : 0) && stampAt < 32) p.trace[stampAt++] = gtime();
    };
    auto gemv = [&](int cp, int mode, const float* bias, const float* bias2, const float* residual, bool resNan, float* out,
                    unsigned long long wordBase, unsigned tag) {
        DsGemv a;
        a.cp = cp; a.mode = mode; a.bias = bias; a.bias2 = bias2; a.residual = residual; a.resNan = resNan ? 1 : 0; a.out = out;
        a.wordBase = wordBase; a.tag = tag;
        ds_gemv(c, a, ring, p.error);
    };

    for (int l = 0; l < L; l++) {
        const DsLayer* ly = m.lay + (l & 1);          // this block's table, in shared memory since the block before
        stamp(l);
        if (l > 0) load_block(l + 1);                 // into the slots block l−1 used; nobody reads them any more (visible after the staging barriers)
        ring.cl = l;
        const float* xin = l == 0 ? embRow : p.x;
        const bool xinNan = l == 0 && !tokOk;

        // ── RMSNorm → QKV projection ──
        ds_stage(c, xin, xinNan, ly->g1, p.d);
        stamp(l);
        gemv(4 * l, 0, nullptr, nullptr, nullptr, false, p.qkv, 0ull, 0u);
        stamp(l);

        // ── attention (RoPE, KV append, split-KV softmax attention, ticket merge; it holds the barrier that publishes q, k, v) ──
        {
            DsAttn aa;
            aa.qkv = p.qkv; aa.att = p.att; aa.ws = p.attn_ws; aa.tickets = p.tickets; aa.cosT = p.cosT; aa.sinT = p.sinT;
            aa.kcache = ly->kcache; aa.vcache = ly->vcache; aa.bar = p.bar; aa.error = p.error;
            aa.scratch = reinterpret_cast<float*>(m.act); aa.flags = s_flags;
            aa.pos = pos; aa.maxSeq = p.maxSeq; aa.H = p.H; aa.splits = p.splits; aa.nCtas = nCtas; aa.scale = p.scale;
            ds_attention<LPP>(aa);
        }
        stamp(l);
        grid_barrier(300 + 1);
        stamp(l);

        // ── Wo + residual ──
        ds_stage(c, p.att, 0, nullptr, p.H * LPP * 16);
        stamp(l);
        if (!tp) {
            gemv(4 * l + 1, 0, nullptr, nullptr, xin, xinNan, p.x2, 0ull, 0u);
            stamp(l);
            grid_barrier(300 + 2);
        } else {
            const unsigned long long wb = 0ull;                                            // even exchanges: slot parity 0
            gemv(4 * l + 1, 3, nullptr, nullptr, nullptr, false, nullptr, wb, epochBase + 1u + 2u * l);
            ds_tp_reduce(c, wb, epochBase + 1u + 2u * l, nullptr, xin, xinNan, p.x2, p.error);
            grid_barrier(300 + 2);
        }

        // ── RMSNorm → SwiGLU ──
        stamp(l);
        ds_stage(c, p.x2, 0, ly->g2, p.d);
        stamp(l);
        gemv(4 * l + 2, 1, ly->bg, ly->bu, nullptr, false, p.h, 0ull, 0u);
        stamp(l);
        grid_barrier(300 + 3);
        stamp(l);

        // ── down + bias + residual ──
        ds_stage(c, p.h, 0, nullptr, p.F);
        stamp(l);
        if (!tp) {
            gemv(4 * l + 3, 0, ly->bd, nullptr, p.x2, false, p.x, 0ull, 0u);
            stamp(l);
            grid_barrier(300 + 4);
            stamp(l);
        } else {
            const unsigned long long wb = (unsigned long long)p.world * p.d;               // odd exchanges: slot parity 1
            gemv(4 * l + 3, 3, nullptr, nullptr, nullptr, false, nullptr, wb, epochBase + 2u + 2u * l);
            ds_tp_reduce(c, wb, epochBase + 2u + 2u * l, ly->bd, p.x2, 0, p.x, p.error);
            grid_barrier(300 + 4);
        }
    }

    // ── final RMSNorm → LM head → greedy pick ──
    ring.cl = L;
    ds_stage(c, L == 0 ? embRow : p.x, L == 0 && !tokOk, p.gF, p.d);
    gemv(4 * L, 2, p.blm, nullptr, nullptr, false, p.logits, 0ull, 0u);
    // nothing lies behind the LM head in a warp's sequence, so no copy of this launch is in flight any more
    int bestKey = ring.bestKey, bestIdx = ring.bestIdx;
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
        for (int cc = lane; cc < nCtas; cc += 32) {
            const int k2 = __ldcg(p.pick + 2 * cc), i2 = __ldcg(p.pick + 2 * cc + 1);
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
    // A CTA that gave up a wait may still have copies in flight (it stopped waiting for them): give them time to land
    // before its shared memory is handed on.  A healthy CTA has consumed every item it issued.
    if (s_flags[0] != 0) {
        for (int i = 0; i < 100; i++) __nanosleep(2000);
    }
    // the last CTA out re-arms the barrier counter for the next launch
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        const unsigned done = atomicAdd(p.bar + 1, 1u);
        if (done == (unsigned)nCtas - 1u) { p.bar[0] = 0u; p.bar[1] = 0u; __threadfence(); }
    }
}

// ───────────── tile-major weight stream ─────────────
// One CTA per (tile, 64-k pair): 72 threads move 16 bytes each — 64 code pieces (row r, 16-byte piece c at
// r·64 + (c ^ ((r>>1 & 1)·2))·16, the swizzle the MMA fragment reads expect) and 8 × 4 scales (row r, block b at
// 1024 + (2r + b)·4).  Rows past N repeat the last row (their results are never written); the missing second block
// of an odd last pair is zeros with scale 0.  With codes2 != null a tile is 8 gate rows then 8 up rows.
__global__ void k_pack_phase(const int8_t* __restrict__ codes, const float* __restrict__ scales, const int8_t* __restrict__ codes2,
                             const float* __restrict__ scales2, int K, int N, unsigned char* __restrict__ out) {
    const int nBlocks = K >> 5, nPairs = (nBlocks + 1) >> 1, nb = nBlocks;
    const int tile = blockIdx.y, pi = blockIdx.x, i = threadIdx.x;
    const bool sw = codes2 != nullptr;
    const int rpt = sw ? 8 : 16;
    const size_t dstPair = ((size_t)tile * nPairs + pi) * kPairBytes;          // a tile's pairs in order: 16 consecutive ones are a ring item
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (i < 64) {
        const int r = i >> 2, c = i & 3;
        const int row = min(tile * rpt + (sw ? (r & 7) : r), N - 1);
        const int8_t* src = (sw && r >= 8) ? codes2 : codes;
        if (pi * 2 + (c >> 1) < nBlocks) v = *reinterpret_cast<const uint4*>(src + (size_t)row * K + pi * 64 + c * 16);
        *reinterpret_cast<uint4*>(out + dstPair + r * kRowStride + ((c ^ (((r >> 1) & 1) << 1)) * 16)) = v;
    } else if (i < 72) {
        float f[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int idx = (i - 64) * 4 + e, r = idx >> 1, b = idx & 1;
            const int row = min(tile * rpt + (sw ? (r & 7) : r), N - 1);
            const float* src = (sw && r >= 8) ? scales2 : scales;
            f[e] = pi * 2 + b < nBlocks ? src[(size_t)row * nb + pi * 2 + b] : 0.0f;
        }
        *reinterpret_cast<float4*>(out + dstPair + kRows * kRowStride + (i - 64) * 16) = make_float4(f[0], f[1], f[2], f[3]);
    }
}

size_t packed_bytes(int K, int N, bool swiglu) {
    const int rpt = swiglu ? 8 : 16;
    const size_t nTiles = (size_t)(N + rpt - 1) / rpt, nPairs = (size_t)((K >> 5) + 1) >> 1;
    return nTiles * nPairs * kPairBytes;
}

void pack_phase(const Q8View& w, const Q8View* w2, unsigned char* out, cudaStream_t s) {
    const int rpt = w2 ? 8 : 16;
    const dim3 grid((unsigned)(((w.K >> 5) + 1) >> 1), (unsigned)((w.N + rpt - 1) / rpt));
    k_pack_phase<<<grid, 96, 0, s>>>(w.codes, w.scales, w2 ? w2->codes : nullptr, w2 ? w2->scales : nullptr, w.K, w.N, out);
    DJ_CUDA_CHECK(cudaGetLastError());
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
    return (size_t)2 * kDepth * kSlotBytes + ((act + 127) & ~(size_t)127) + (size_t)2 * kPartBufs * kHalfWarps * kPartFloats * 4 + 8 * sizeof(DsPhase) +
           2 * sizeof(DsLayer) + kWarps * 4 + 64 * 4 + kMaxWorld * sizeof(void*) + (size_t)2 * 2 * kDepth * 8;
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
    prm.trace = g_trace;                 // null unless DEEPJ_CUDA_TRACE=1; the stamps of the last launch stay in the first 32 slots
    if (g_trace && g_trace_launches < 4) g_trace_launches = 4;
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
        P.d = d; P.V = V;
        PoolKV kv;
        if (!pool_kv(desc[10], &kv)) throw std::runtime_error("decode_plan: missing KV cache");
        pl.refs.push_back({desc[10], pool_serial(desc[10])});
        if (kv.layers < L || kv.H != H || kv.hd != hd || kv.B < 1) throw std::runtime_error("decode_plan: the KV cache does not match the model");
        if (kv.half) throw std::runtime_error("decode_plan: the whole-token kernel reads an fp32 KV cache");
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
        struct Src { Q8View w, w2; bool sw; };
        std::vector<Src> srcs;                       // 4 per block in phase order, then the LM head
        const size_t plane = (size_t)kv.layers * kv.B * kv.H * kv.maxSeq * kv.hd;
        for (int l = 0; l < L; l++) {
            const int32_t* e = desc + kHead + l * kPerLayer;
            DsLayer& y = table[l];
            y.g1 = f32(e[0], d, "norm gain 1");
            const Q8View wqkv = q8(e[1], d, 3 * dl, "Wqkv");
            const Q8View wo = q8(e[2], dl, d, "Wo");
            y.g2 = f32(e[3], d, "norm gain 2");
            const Q8View wg = q8(e[4], d, F, "gate");
            if (l == 0) F = wg.N;
            y.bg = f32(e[5], F, "gate bias");
            const Q8View wu = q8(e[6], d, F, "up");
            y.bu = f32(e[7], F, "up bias");
            const Q8View wd = q8(e[8], F, d, "down");
            y.bd = f32(e[9], d, "down bias");
            srcs.push_back({wqkv, {}, false}); srcs.push_back({wo, {}, false}); srcs.push_back({wg, wu, true}); srcs.push_back({wd, {}, false});
            const size_t layerOff = (size_t)l * kv.B * kv.H * kv.maxSeq * kv.hd;
            y.kcache = static_cast<float*>(kv.ptr) + layerOff; y.vcache = static_cast<float*>(kv.ptr) + plane + layerOff;
        }
        srcs.push_back({lm, {}, false});
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
        // one device block: the layer table, scratch (attention partials, tickets, barrier words, pick pairs), then the
        // tile-major copies of every weight the step streams (as many bytes again as the Q8 objects they are made from)
        const size_t tableBytes = ((size_t)L * sizeof(DsLayer) + 255) & ~(size_t)255;
        const size_t wsFloats = (size_t)H * P.splits * (hd + 2);
        const size_t scratchBytes = (wsFloats * 4 + (size_t)H * 4 + 16 * 4 + (size_t)2 * g_num_sms * 4 + 511) & ~(size_t)255;
        std::vector<size_t> wOff(srcs.size());
        size_t weightBytes = 0;
        for (size_t i = 0; i < srcs.size(); i++) {
            wOff[i] = weightBytes;
            weightBytes += (packed_bytes(srcs[i].w.K, srcs[i].w.N, srcs[i].sw) + 255) & ~(size_t)255;
        }
        char* block = nullptr;
        DJ_CUDA_CHECK(cudaMalloc((void**)&block, tableBytes + scratchBytes + weightBytes));
        DJ_CUDA_CHECK(cudaMemset(block, 0, tableBytes + scratchBytes));
        unsigned char* wbase = reinterpret_cast<unsigned char*>(block + tableBytes + scratchBytes);
        for (size_t i = 0; i < srcs.size(); i++) pack_phase(srcs[i].w, srcs[i].sw ? &srcs[i].w2 : nullptr, wbase + wOff[i], runtime_stream());
        for (int l = 0; l < L; l++)
            for (int ph = 0; ph < 4; ph++) table[l].w[ph] = wbase + wOff[(size_t)4 * l + ph];
        P.lm_w = wbase + wOff[(size_t)4 * L];
        DJ_CUDA_CHECK(cudaStreamSynchronize(runtime_stream()));
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
        pool_add_plan(plan_id, block, tableBytes + scratchBytes + weightBytes);
        pl.serial = pool_serial(plan_id);
        g_plans[plan_id] = std::move(pl);
        return 0;
    } catch (const std::exception& e) { set_last_error(e.what()); return 1; }
}
