// Tensor-parallel exchange over NVLink peer memory — one process per GPU.
//
// A transformer block needs two sum-exchanges of [B × d] floats (after the row-parallel
// Wo and down projections) and the LM head one gather of [B × V/g] logits.  At batch 1
// these are 16 KB messages: latency, not bandwidth.  Each rank owns a communication
// buffer (two parities × world slots) that every peer maps through CUDA IPC.  One kernel
// per exchange:
//   push   every rank stores its contribution into slot[parity][my rank] of EVERY peer
//          (plain peer stores over NVLink), then publishes an epoch
//          number in the peer's flag word;
//   wait   until all ranks' flags for this epoch have arrived locally (bounded spin: when
//          the bound expires the kernel records an error code and carries on, it never hangs);
//   finish sum the slots in rank order (+ residual + bias) — every rank computes the same
//          bits — or copy them side by side for the gather.
// Parity flips every exchange; a rank can be at most one exchange ahead of a peer (it needs
// the peer's flag to finish), so two parities are enough.  Epochs live in device memory,
// which makes the kernels replayable inside a captured CUDA graph.
#include "../../include/deepj_cuda.h"
#include "kernels.h"

#include <cstring>
#include <vector>

namespace dj {

namespace {

constexpr int kMaxWorld = 8;
constexpr int kTpCtas = 8;                    // CTAs per exchange; each owns a contiguous chunk
constexpr unsigned kTpSpinLimit = 1u << 24;   // ≈ seconds, then give up

struct TpState {
    bool ready = false;
    int rank = 0, world = 1;
    size_t slot_floats = 0;
    // layout of one rank's buffer: data[2][world][slot_floats] floats, then flags[world][kTpCtas] u32, then epochs[kTpCtas] u32
    void* local = nullptr;
    size_t bytes = 0;
    float* peer_data[kMaxWorld] = {};
    unsigned* peer_flags[kMaxWorld] = {};
    unsigned* epochs = nullptr;
    void* opened[kMaxWorld] = {};
} T;

struct TpPtrs {
    float* data[kMaxWorld];
    unsigned* flags[kMaxWorld];
};

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ unsigned ld_volatile_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys_u32(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// mode 0: out[m][n] = residual[m][n] + bias[n] + Σ_r contribution_r[m][n]   (n_local == N)
// mode 1: out[m][r·n_local + j] = contribution_r[m][j]
__global__ void __launch_bounds__(256) k_tp_exchange(TpPtrs P, int rank, int world, size_t slot_floats, unsigned* epochs,
                                                      const float* __restrict__ in, const float* __restrict__ bias,
                                                      const float* __restrict__ residual, float* __restrict__ out,
                                                      int M, int n_local, int mode, int* error) {
    __shared__ int s_ok;
    pdl_wait();
    pdl_launch_dependents();
    const int cta = blockIdx.x, tid = threadIdx.x;
    const unsigned epoch = epochs[cta] + 1;
    const unsigned parity = epoch & 1u;
    const int total = M * n_local;                                   // floats this rank contributes
    const int per = ((total + kTpCtas - 1) / kTpCtas + 3) & ~3;       // chunk, multiple of 4 floats
    const int lo = min(total, cta * per), hi = min(total, lo + per);

    // push my chunk into slot[parity][rank] of every rank (myself included)
    const size_t slot = ((size_t)parity * world + rank) * slot_floats;
    for (int r = 0; r < world; r++) {
        float* dst = P.data[r] + slot;
        for (int i = lo + tid * 4; i < hi; i += blockDim.x * 4) {
            if (i + 3 < hi) *reinterpret_cast<float4*>(dst + i) = *reinterpret_cast<const float4*>(in + i);
            else for (int j = i; j < hi; j++) dst[j] = in[j];
        }
    }
    __threadfence_system();
    __syncthreads();
    if (tid == 0) {
        for (int r = 0; r < world; r++) st_release_sys_u32(P.flags[r] + rank * kTpCtas + cta, epoch);
    }
    // wait for every rank's chunk of this epoch
    if (tid < world) {
        const unsigned* f = P.flags[rank] + tid * kTpCtas + cta;
        bool ok = false;
        for (unsigned it = 0; it < kTpSpinLimit; it++) {
            if ((int)(ld_volatile_u32(f) - epoch) >= 0) { ok = true; break; }
            __nanosleep(64);
        }
        if (!ok) atomicExch(error, 100 + tid);
    }
    __syncthreads();
    __threadfence_system();
    (void)s_ok;
    const float* mine = P.data[rank] + (size_t)parity * world * slot_floats;
    if (mode == 0) {
        for (int i = lo + tid; i < hi; i += blockDim.x) {
            const int n = i % n_local;
            float v = residual ? residual[i] : 0.0f;
            if (bias) v += bias[n];
            float s = 0.0f;
            for (int r = 0; r < world; r++) s += __ldcv(mine + (size_t)r * slot_floats + i);     // rank order: same bits everywhere
            out[i] = v + s;
        }
    } else {
        for (int i = lo + tid; i < hi; i += blockDim.x) {
            const int m = i / n_local, j = i % n_local;
            for (int r = 0; r < world; r++)
                out[(size_t)m * n_local * world + (size_t)r * n_local + j] = __ldcv(mine + (size_t)r * slot_floats + i);
        }
    }
    __syncthreads();
    if (tid == 0) epochs[cta] = epoch;
}

}  // namespace

bool tp_ready() { return T.ready; }
int tp_world() { return T.ready ? T.world : 1; }

void launch_tp_exchange(const float* in, const float* bias, const float* residual, float* out, int M, int n_local, int mode,
                        cudaStream_t s) {
    if (!T.ready) throw std::runtime_error("tensor-parallel exchange recorded but deepj_cuda_tp_connect was never called");
    if ((size_t)M * n_local > T.slot_floats)
        throw std::runtime_error("tensor-parallel exchange of " + std::to_string((size_t)M * n_local) + " floats exceeds the slot size " +
                                 std::to_string(T.slot_floats));
    TpPtrs P;
    for (int r = 0; r < kMaxWorld; r++) { P.data[r] = T.peer_data[r]; P.flags[r] = T.peer_flags[r]; }
    launch_k(k_tp_exchange, dim3(kTpCtas), dim3(256), 0, s, true, P, T.rank, T.world, T.slot_floats, T.epochs, in, bias, residual, out,
             M, n_local, mode, g_dev_error);
}

}  // namespace dj

using namespace dj;

extern "C" {

// Step 1: allocate this rank's communication buffer and return its IPC handle (64 bytes).
int deepj_cuda_tp_create(int32_t rank, int32_t world, int64_t slot_floats, void* handle_out64) {
    try {
        if (runtime_stream() == nullptr) throw std::runtime_error("tp_create: call deepj_cuda_init first");
        if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world) throw std::runtime_error("tp_create: bad rank/world");
        if (slot_floats <= 0 || slot_floats % 4 != 0) throw std::runtime_error("tp_create: slot size must be a positive multiple of 4 floats");
        if (T.local) throw std::runtime_error("tp_create: already created");
        T.rank = rank; T.world = world; T.slot_floats = (size_t)slot_floats;
        const size_t dataBytes = (size_t)2 * world * slot_floats * sizeof(float);
        T.bytes = dataBytes + (size_t)(world + 1) * kTpCtas * sizeof(unsigned);
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
        const size_t dataFloats = (size_t)2 * T.world * T.slot_floats;
        for (int r = 0; r < T.world; r++) {
            void* base = T.local;
            if (r != T.rank) {
                cudaIpcMemHandle_t h;
                std::memcpy(&h, (const char*)handles + (size_t)r * 64, 64);
                DJ_CUDA_CHECK(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
                T.opened[r] = base;
            }
            T.peer_data[r] = (float*)base;
            T.peer_flags[r] = (unsigned*)((float*)base + dataFloats);
        }
        T.epochs = T.peer_flags[T.rank] + (size_t)T.world * kTpCtas;
        T.ready = true;
        return 0;
    } catch (const std::exception& e) { set_last_error(e.what()); return 1; }
}

int deepj_cuda_tp_destroy(void) {
    try {
        if (runtime_stream()) cudaStreamSynchronize(runtime_stream());
        for (int r = 0; r < kMaxWorld; r++) if (T.opened[r]) { cudaIpcCloseMemHandle(T.opened[r]); T.opened[r] = nullptr; }
        if (T.local) cudaFree(T.local);
        T = TpState();
        return 0;
    } catch (const std::exception& e) { set_last_error(e.what()); return 1; }
}

}  // extern "C"
