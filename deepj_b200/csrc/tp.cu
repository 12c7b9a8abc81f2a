// Tensor-parallel exchange over NVLink peer memory — one process per GPU.
//
// A transformer block needs two sum-exchanges of [B × d] floats (after the row-parallel
// Wo and down projections) and the LM head one gather of [B × V/g] logits.  At batch 1
// these are 16 KB messages: latency, not bandwidth.  Each rank owns a communication
// buffer (two parities × world slots) that every peer maps through CUDA IPC.  One kernel
// per exchange, no fence and no separate flag on the critical path:
//   push   every value travels as an 8-byte word {bits, epoch}; a thread stores two of them
//          (16 bytes) into slot[parity][my rank] of EVERY rank with plain peer stores;
//   wait   the same thread polls its own words in all slots until their epoch fields show
//          the current epoch (8-byte stores arrive whole, so a word whose epoch matches
//          carries its value) — a bounded poll: when the bound expires the kernel records
//          an error code and carries on, it never hangs;
//   finish add the slots in rank order (+ residual + bias) — every rank computes the same
//          bits — or place them side by side for the gather.
// The cost is one NVLink one-way latency instead of store → system fence → flag.
// Parity flips every exchange of a grid class; a rank can be at most one exchange ahead of a
// peer (it needs the peer's words to finish), so two parities are enough and a stale word
// (epoch − 2) can never be taken for a fresh one.  That argument holds per grid class only —
// a decode-sized exchange directly after a chunk-sized one could share a parity with it —
// so the two classes own separate slot regions of the buffer and never touch each other's
// words.  Epochs live in device memory, which makes the kernels replayable inside a
// captured CUDA graph.
// Once a wait has expired (the device error word is non-zero) every later wait, in this
// launch and in the following ones, gives up at once: a dead peer costs one bounded wait,
// not one per word.
#include "../../include/deepj_cuda.h"
#include "kernels.h"

#include <algorithm>
#include <cstring>
#include <vector>

namespace dj {

namespace {

constexpr int kMaxWorld = 8;
constexpr int kTpCtas = 32;                   // CTAs of a decode-sized exchange (one pass for one sequence, eight for sixteen)
constexpr int kTpCtasLarge = 296;             // CTAs of a chunk-sized exchange (a fixed number: the per-CTA counters depend on it)
constexpr long kTpLargePairs = 1L << 14;      // messages above 2^15 floats take the large grid (16 sequences of a 4096-wide model: 2.73 → 2.80 k tokens/s at 2 GPUs against a threshold of 2^17)
constexpr unsigned kTpSpinLimit = 1u << 21;   // polls of one word (≈ a second), then give up
long g_large_pairs = kTpLargePairs;           // deepj_cuda_tp_configure; the same on every rank

struct TpState {
    bool ready = false;
    int rank = 0, world = 1;
    size_t slot_floats = 0;         // values one exchange may carry per rank
    size_t small_floats = 0;        // … of which the decode-sized class can see at most this many
    // layout of one rank's buffer, {bits, epoch} words of 8 bytes: the decode-sized class's region
    // words[2][world][small_floats], then the chunk-sized class's words[2][world][slot_floats], then the region of the
    // whole-token decode kernel (decode_step.cu: words[2][world][small_floats] of partial sums + [world][2] pick pairs),
    // then the exchange counters (u32; kTpCtas for the small grid, kTpCtasLarge for the large one, one tag counter of
    // the decode kernel; private to this rank)
    void* local = nullptr;
    size_t bytes = 0;
    float* peer_data[kMaxWorld] = {};
    unsigned* epochs = nullptr;
    void* opened[kMaxWorld] = {};
    void* absent[kMaxWorld] = {};      // stand-ins for ranks that never connect (tp_connect without handles)
} T;

struct TpPtrs {
    float* data[kMaxWorld];
};

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_volatile_v4(void* p, uint4 v) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}


// mode 0: out[m][n] = residual[m][n] + bias[n] + Σ_r contribution_r[m][n]   (n_local == N)
// mode 1: out[m][r·n_local + j] = contribution_r[m][j]
__global__ void __launch_bounds__(256) k_tp_exchange(TpPtrs P, int rank, int world, size_t region_words, size_t slot_floats, unsigned* epochs, unsigned tag,
                                                      const float* __restrict__ in, const float* __restrict__ bias,
                                                      const float* __restrict__ residual, float* __restrict__ out,
                                                      int M, int n_local, int mode, int* error) {
    pdl_wait();
    pdl_launch_dependents();
    const int cta = blockIdx.x, tid = threadIdx.x;
    // Every CTA counts the exchanges it has taken part in; all ranks run the same sequence of exchanges with the same
    // grids, so CTA i of every rank agrees on the count without communicating it.  The two grid sizes (decode-sized
    // and chunk-sized messages) keep separate counters, and `tag` keeps their words apart in the shared slots.
    const unsigned count = (epochs[cta] + 1) & 0x7fffffffu;
    const unsigned epoch = count | tag;
    const unsigned parity = count & 1u;
    const int total = M * n_local;                       // floats this rank contributes
    const int pairs = (total + 1) >> 1;
    const size_t slotWords = region_words + (size_t)parity * world * slot_floats;      // in 8-byte words
    bool gaveUp = false;                                  // a wait of this thread has expired, or the error word was already set
    // push first, for ALL of this thread's pairs: my values into my slot on every rank (myself included).  Only then wait —
    // a thread with several passes (16 sequences, a prompt chunk) pays one NVLink latency, not one per pass.
    const int stride = gridDim.x * blockDim.x;
    for (int p0 = cta * blockDim.x + tid; p0 < pairs; p0 += stride) {
        const int i = 2 * p0;
        const float a = i < total ? in[i] : 0.0f, b = i + 1 < total ? in[i + 1] : 0.0f;
        const uint4 w = make_uint4(__float_as_uint(a), epoch, __float_as_uint(b), epoch);
        for (int r = 0; r < world; r++) {
            uint4* dst = reinterpret_cast<uint4*>(P.data[r]) + (slotWords + (size_t)rank * slot_floats) / 2;
            st_volatile_v4(dst + p0, w);
        }
    }
    // wait + finish: the same pairs from every rank's slot in my own buffer, in rank order
    for (int p0 = cta * blockDim.x + tid; p0 < pairs; p0 += stride) {
        float sa = 0.0f, sb = 0.0f;
        const int i = 2 * p0;
        for (int r = 0; r < world; r++) {
            const uint4* src = reinterpret_cast<const uint4*>(P.data[rank]) + (slotWords + (size_t)r * slot_floats) / 2;
            uint4 v = ld_volatile_v4(src + p0);
            if (v.y != epoch || v.w != epoch) {
                // not there yet: poll, unless some wait has already run out (here or in an earlier launch)
                gaveUp = gaveUp || *reinterpret_cast<volatile int*>(error) != 0;
                for (unsigned it = 0; !gaveUp && (v.y != epoch || v.w != epoch) && it < kTpSpinLimit; it++) {
                    __nanosleep(32);
                    v = ld_volatile_v4(src + p0);
                    if ((it & 63u) == 63u) gaveUp = *reinterpret_cast<volatile int*>(error) != 0;
                }
                if (v.y != epoch || v.w != epoch) {
                    if (!gaveUp) atomicCAS(error, 0, 100 + r);      // the first expiry names the rank
                    gaveUp = true;
                }
            }
            const float a = __uint_as_float(v.x), b = __uint_as_float(v.z);
            if (mode == 0) { sa += a; sb += b; }
            else {
                if (i < total) out[(size_t)(i / n_local) * n_local * world + (size_t)r * n_local + i % n_local] = a;
                if (i + 1 < total) out[(size_t)((i + 1) / n_local) * n_local * world + (size_t)r * n_local + (i + 1) % n_local] = b;
            }
        }
        if (mode == 0) {
            if (i < total) {
                float v = residual ? residual[i] : 0.0f;
                if (bias) v += bias[i % n_local];
                out[i] = v + sa;
            }
            if (i + 1 < total) {
                float v = residual ? residual[i + 1] : 0.0f;
                if (bias) v += bias[(i + 1) % n_local];
                out[i + 1] = v + sb;
            }
        }
    }
    __syncthreads();
    if (tid == 0) epochs[cta] = count;
}

}  // namespace

size_t tp_exchange_bytes() {
    // a chunk-sized region only when a message can exceed the decode-sized class
    const size_t largeFloats = T.slot_floats > T.small_floats ? T.slot_floats : 0;
    return (size_t)2 * T.world * (T.small_floats + largeFloats) * 8;
}
size_t tp_step_words_count() { return (size_t)2 * T.world * T.small_floats + 2 * (size_t)T.world + 8; }
size_t tp_data_bytes() { return tp_exchange_bytes() + tp_step_words_count() * 8; }

// The decode-step kernel's view of the connection: rank r's word region, the tag counter, the region's size in words.
unsigned long long* tp_step_words(int r) {
    return T.ready ? reinterpret_cast<unsigned long long*>(reinterpret_cast<char*>(T.peer_data[r]) + tp_exchange_bytes()) : nullptr;
}
unsigned* tp_step_epoch() { return T.ready ? T.epochs + kTpCtas + kTpCtasLarge : nullptr; }
size_t tp_step_floats() { return T.ready ? tp_step_words_count() : 0; }
int tp_rank() { return T.rank; }

bool tp_ready() { return T.ready; }
int tp_world() { return T.ready ? T.world : 1; }

void launch_tp_exchange(const float* in, const float* bias, const float* residual, float* out, int M, int n_local, int mode,
                        cudaStream_t s) {
    if (!T.ready) throw std::runtime_error("tensor-parallel exchange recorded but deepj_cuda_tp_connect was never called");
    if ((size_t)M * n_local > T.slot_floats)
        throw std::runtime_error("tensor-parallel exchange of " + std::to_string((size_t)M * n_local) + " floats exceeds the slot size " +
                                 std::to_string(T.slot_floats));
    TpPtrs P;
    for (int r = 0; r < kMaxWorld; r++) { P.data[r] = T.peer_data[r]; }
    // a decode step's message (16 KB … 256 KB) spreads over kTpCtas CTAs; a prompt chunk's megabytes over kTpCtasLarge
    const long pairs = ((long)M * n_local + 1) / 2;
    const bool large = pairs > g_large_pairs;
    const size_t smallRegionWords = (size_t)2 * T.world * T.small_floats;
    launch_k(k_tp_exchange, dim3(large ? kTpCtasLarge : kTpCtas), dim3(256), 0, s, true, P, T.rank, T.world,
             large ? smallRegionWords : (size_t)0, large ? T.slot_floats : T.small_floats,
             large ? T.epochs + kTpCtas : T.epochs, large ? 0x80000000u : 0u, in, bias, residual, out,
             M, n_local, mode, g_dev_error);
}

}  // namespace dj

using namespace dj;

extern "C" {

// The message size (in floats per rank) above which an exchange takes the chunk-sized grid and its own slot
// region.  Call before tp_create, with the same value on every rank; 0 restores the default (2^15).
int deepj_cuda_tp_configure(int64_t large_message_floats) {
    try {
        if (T.local) throw std::runtime_error("tp_configure: call before tp_create");
        if (large_message_floats < 0) throw std::runtime_error("tp_configure: negative threshold");
        g_large_pairs = large_message_floats == 0 ? kTpLargePairs : (long)((large_message_floats + 1) / 2);
        return 0;
    } catch (const std::exception& e) { set_last_error(e.what()); return 1; }
}

// Step 1: allocate this rank's communication buffer and return its IPC handle (64 bytes).
int deepj_cuda_tp_create(int32_t rank, int32_t world, int64_t slot_floats, void* handle_out64) {
    try {
        if (runtime_stream() == nullptr) throw std::runtime_error("tp_create: call deepj_cuda_init first");
        if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world) throw std::runtime_error("tp_create: bad rank/world");
        if (slot_floats <= 0 || slot_floats % 4 != 0) throw std::runtime_error("tp_create: slot size must be a positive multiple of 4 floats");
        if (T.local) throw std::runtime_error("tp_create: already created");
        T.rank = rank; T.world = world; T.slot_floats = (size_t)slot_floats;
        T.small_floats = std::min((size_t)slot_floats, (size_t)(2 * g_large_pairs + 3) / 4 * 4);
        const size_t dataBytes = tp_data_bytes();       // {bits, epoch} per value, both regions
        T.bytes = dataBytes + (size_t)(kTpCtas + kTpCtasLarge + 4) * sizeof(unsigned);
        DJ_CUDA_CHECK(cudaMalloc(&T.local, T.bytes));
        DJ_CUDA_CHECK(cudaMemset(T.local, 0, T.bytes));
        DJ_CUDA_CHECK(cudaDeviceSynchronize());
        cudaIpcMemHandle_t h;
        DJ_CUDA_CHECK(cudaIpcGetMemHandle(&h, T.local));
        static_assert(sizeof(h) == 64, "IPC handle size");
        std::memcpy(handle_out64, &h, 64);
        return 0;
    } catch (const std::exception& e) { set_last_error(e.what()); return 1; }
}

// Step 2: hand over the handles of all ranks (world × 64 bytes, rank order).
int deepj_cuda_tp_connect(const void* handles, int32_t world) {
    try {
        if (!T.local || world != T.world) throw std::runtime_error("tp_connect: call tp_create first, with the same world size");
        const size_t dataBytes = tp_data_bytes();
        for (int r = 0; r < T.world; r++) {
            void* base = T.local;
            if (r != T.rank && handles == nullptr) {
                // nobody will ever write here: this rank's pushes land in it, and its own buffer never sees rank r
                DJ_CUDA_CHECK(cudaMalloc(&base, T.bytes));
                DJ_CUDA_CHECK(cudaMemset(base, 0, T.bytes));
                T.absent[r] = base;
            } else if (r != T.rank) {
                cudaIpcMemHandle_t h;
                std::memcpy(&h, (const char*)handles + (size_t)r * 64, 64);
                DJ_CUDA_CHECK(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
                T.opened[r] = base;
            }
            T.peer_data[r] = (float*)base;
        }
        T.epochs = (unsigned*)((char*)T.local + dataBytes);
        T.ready = true;
        invalidate_graphs();        // a graph captured against an earlier connection holds its peer addresses
        return 0;
    } catch (const std::exception& e) { set_last_error(e.what()); return 1; }
}

int deepj_cuda_clear_device_error(void) {
    try {
        if (runtime_stream() == nullptr || g_dev_error == nullptr) return 0;
        DJ_CUDA_CHECK(cudaStreamSynchronize(runtime_stream()));
        DJ_CUDA_CHECK(cudaMemset(g_dev_error, 0, sizeof(int)));
        return 0;
    } catch (const std::exception& e) { set_last_error(e.what()); return 1; }
}

int deepj_cuda_tp_destroy(void) {
    try {
        if (runtime_stream()) cudaStreamSynchronize(runtime_stream());
        for (int r = 0; r < kMaxWorld; r++) if (T.opened[r]) { cudaIpcCloseMemHandle(T.opened[r]); T.opened[r] = nullptr; }
        for (int r = 0; r < kMaxWorld; r++) if (T.absent[r]) { cudaFree(T.absent[r]); T.absent[r] = nullptr; }
        if (T.local) cudaFree(T.local);
        T = TpState();
        invalidate_graphs();        // captured exchanges point into the buffers just unmapped
        return 0;
    } catch (const std::exception& e) { set_last_error(e.what()); return 1; }
}

}  // extern "C"
