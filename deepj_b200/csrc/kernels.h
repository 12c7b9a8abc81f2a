// Launcher declarations shared by the runtime (runtime.cu) and the kernel files.
// Every launcher enqueues on the given stream and never synchronises.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdlib>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#define DJ_CUDA_CHECK(expr)                                                                  \
    do {                                                                                     \
        cudaError_t _e = (expr);                                                             \
        if (_e != cudaSuccess)                                                               \
            throw std::runtime_error(std::string("CUDA error: ") + cudaGetErrorString(_e) + \
                                     " at " + __FILE__ + ":" + std::to_string(__LINE__));   \
    } while (0)

namespace dj {

// Counts kernel launches issued by this library (eager path and capture).
extern long long g_launches;
extern int g_num_sms;
// When true, launchers attach the programmatic-dependent-launch attribute so that
// a kernel's weight prefetch overlaps the tail of its predecessor.
extern bool g_use_pdl;
// Q8 GEMV kernel choice (environment DEEPJ_CUDA_GEMV = cpasync | fma to step down); shapes outside a
// kernel's domain fall through to the next one.
extern int g_gemv_mode;
extern int g_tc_terms;      // deepj_cuda_tc_configure
// Device int set non-zero when a bounded wait inside a kernel expired.
extern int* g_dev_error;
// Phase-trace ring (null unless tracing is on) and the number of traced launches so far.
constexpr int kTraceSlots = 4096;
extern unsigned long long* g_trace;
extern long long g_trace_launches;
unsigned long long* trace_slot();

// A Q8 weight as laid out in HBM: codes[N][Kp] int8 (Kp = K rounded up to 16, zero
// padded) followed by scales[N][nb] fp32, nb = ceil(K/32).
struct Q8View {
    const int8_t* codes;
    const float* scales;
    int K, N, Kp, nb;
};

// ── base ops (ComputeGraph op codes 1-42) ──
void launch_binary(int op, const float* a, const float* b, float* out, int n, cudaStream_t s);
void launch_unary(int op, const float* in, float* out, int n, cudaStream_t s);
void launch_scalar(int op, const float* in, float* out, float v, int n, cudaStream_t s);
void launch_clamp(const float* in, float* out, float lo, float hi, int n, cudaStream_t s);
void launch_matmul_f32(const float* a, const float* b, float* out, int m, int n, int k, cudaStream_t s);
void launch_transpose(const float* in, float* out, int rows, int cols, cudaStream_t s);
void launch_row_broadcast(int op, const float* a, const float* v, float* out, int rows, int cols, cudaStream_t s);
void launch_col_broadcast(int op, const float* a, const float* v, float* out, int rows, int cols, cudaStream_t s);
void launch_row_reduce(int op, const float* in, float* out, int rows, int cols, cudaStream_t s);
void launch_sum_rows(const float* in, float* out, int rows, int cols, cudaStream_t s);
void launch_sum_scalar(const float* in, float* out, long long n, cudaStream_t s);
void launch_softmax_rows(const float* in, float* out, int rows, int cols, cudaStream_t s);
void launch_softmax_backward(const float* g, const float* sm, float* out, int rows, int cols, cudaStream_t s);
void launch_layernorm_backward(const float* dxh, const float* xh, const float* sd, float* out, int rows, int cols, cudaStream_t s);
void launch_adamw(float* w, const float* g, float* mt, float* vt, float lr, float b1, float b2, float eps,
                  float wd, float bc1, float bc2, int n, cudaStream_t s);
void launch_scatter_add_rows(float* target, const float* idx, const float* grad, int tRows, int tCols, int nIdx, cudaStream_t s);
void launch_ce_loss(const float* logits, const float* targets, float* out, int rows, int cols, cudaStream_t s);
void launch_ce_grad(const float* logits, const float* targets, float* out, int rows, int cols, cudaStream_t s);

// ── Q8 ──
void launch_q8_quantize(const float* src, int src_ld, int K, int n_cols, int8_t* codes, float* scales,
                        int Kp, int nb, cudaStream_t s);
struct Q8LinearArgs {
    const float* x; int ldx;            // activations [M × K], row stride ldx
    const float* gamma; float eps;      // RMSNorm fused into the activation load when gamma != nullptr
    Q8View w;                           // plain linear / SwiGLU gate
    const float* bias;
    Q8View w2;                          // SwiGLU up projection (codes == nullptr → plain linear)
    const float* bias2;
    const float* residual; int ldr;
    float* out; int ldo;
    int M;
    float* ws = nullptr; int* tickets = nullptr;    // workspace (q8_batch_ws_floats) and counters for the batched kernel (M ≥ 3)
    // GPT blocks: beta != nullptr turns the fused norm into LayerNorm1D (mean and biased variance, γ and β);
    // act == 1 applies GELU after the bias.  The GEMV fuses both; the many-row kernels get them from a
    // normalising pass into ln_ws ([M × K] floats) before and an activation pass over `out` after.
    const float* beta = nullptr; int act = 0; float* ln_ws = nullptr;
};
void launch_q8_linear(const Q8LinearArgs& a, cudaStream_t s);
bool launch_q8_gemv_i8(const Q8LinearArgs& a, cudaStream_t s);
bool launch_q8_gemv_tma(const Q8LinearArgs& a, cudaStream_t s);     // K a multiple of 128; false = outside its domain
bool q8_gemv_i8_fuses_gpt(const Q8LinearArgs& a);     // true when launch_q8_gemv_i8 can take beta / act itself
void launch_layernorm_rows(const float* x, int ldx, const float* gamma, const float* beta, float eps, float* out, int K, int M, cudaStream_t s);
void launch_gelu_rows(float* buf, int ld, int N, int M, cudaStream_t s);
bool launch_q8_linear_batch(const Q8LinearArgs& a, int m0, int rows, float* ws, int* tickets, cudaStream_t s);
bool launch_q8_linear_batch_tma(const Q8LinearArgs& a, int m0, int rows, float* ws, int* tickets, cudaStream_t s);   // K a multiple of 128; same workspace
size_t q8_batch_ws_floats(int K, int N, bool swiglu);
bool launch_q8_linear_tc(const Q8LinearArgs& a, float* ws, cudaStream_t s);
size_t q8_tc_ws_floats(int M, int K, int N);     // activation tiles, row scales and, when the reduction is split, the partial outputs
double q8_tc_estimate_us(int M, int K, int N);
constexpr int kTcMinRows = 17;            // from this many activation rows on, a Q8 linear runs on the tcgen05 path

// ── decode attention ──
struct AttnDecodeArgs {
    float* qkv; int q_off, k_off, v_off, ld;   // current token's projections, one row per sequence
    void* kcache; void* vcache;                // this layer's planes [B][H][maxSeq][hd], fp32 or (kvHalf) fp16
    int maxSeq;
    const float* pos;                          // [B] floats holding the write position
    const float* cosT; const float* sinT;      // [maxSeq × hd/2]
    float* out; int ldo;                       // merged heads [B × H·hd]
    int B, H, hd;
    float scale;
    float* ws;                                 // split partials: [B][H][splits][hd + 2]
    int* tickets;                              // [B·H] zero-initialised, self-resetting counters
    int kvHalf = 0;                            // 1: the cache holds fp16 (keys rounded after the rotation, values rounded; fp32 arithmetic)
    int T = 1;                                 // tokens per sequence in this call: 1 = decode step, > 1 = prompt chunk (rows b·T + t)
    int splits;
};
constexpr int kAttnTickets = 1 << 16;
size_t attn_decode_ws_floats(int B, int H, int hd, int splits);
int attn_decode_splits(int B, int H, int maxSeq);
void launch_attn_decode(const AttnDecodeArgs& a, cudaStream_t s);
bool launch_attn_prefill_mma(const AttnDecodeArgs& a, cudaStream_t s);     // prompt chunks on the tensor cores (head dim 64 / 128)

// ── misc ──
void launch_embed_gather(const float* table, const float* ids, float* out, int rows, int d, int vocab, cudaStream_t s);
// scratch: 2·16·rows ints of partial (key, index) pairs, tickets: rows zeroed self-resetting counters (rows ≤ kArgmaxRowsMax)
constexpr int kArgmaxRowsMax = 4096;
void launch_argmax_rows(const float* in, float* out, int rows, int cols, int* scratch, int* tickets, cudaStream_t s);
// topK = 0 means the whole row (the reference's convention); more than 1024 candidates sort the row in `ws`
// (sample_topk_ws_floats floats, 8-byte aligned).
void launch_sample_topk(const float* logits, const float* r, float* out, int rows, int cols, int topK, float temperature, float* ws,
                        cudaStream_t s);
size_t sample_topk_ws_floats(int rows, int cols, int topK);
void launch_add_scalar_inplace(float* buf, float v, int n, cudaStream_t s);
void launch_copy(const float* src, float* dst, long long n, cudaStream_t s);
void launch_synth_fill(float* out, unsigned long long seed, unsigned long long ordinal, float std_dev,
                       long long first, long long n, cudaStream_t s);

// ── tensor-parallel exchange over peer memory (tp.cu) ──
bool tp_ready();
int tp_world();
// mode 0: out = residual + bias + Σ_ranks in (all-reduce); mode 1: out[m][r·n_local + j] = in_r[m][j] (all-gather)
void launch_tp_exchange(const float* in, const float* bias, const float* residual, float* out, int M, int n_local, int mode,
                        cudaStream_t s);

// Read-only views of the runtime's buffer pool for entry points that live beside their kernels.
struct PoolF32 { float* ptr; size_t floats; };
struct PoolKV { void* ptr; int layers, B, H, maxSeq, hd, half; };
bool pool_f32(int id, PoolF32* out);
bool pool_kv(int id, PoolKV* out);
bool pool_q8(int id, Q8View* out);
// Serial number of a pool object (0 when the id does not exist); a released and re-created id gets a new serial.
unsigned long long pool_serial(int id);
// Registers device memory owned by a decode plan under `id` in the pool (released with the other objects).
void pool_add_plan(int id, void* dev_ptr, size_t bytes);

// ── whole-token decode kernel (decode_step.cu) ──
// Validates the plan object behind op 76 and appends the (id, serial) of everything it references to `refs`.
void decode_step_check(int plan_id, std::vector<std::pair<int, unsigned long long>>* refs);
void launch_decode_step(int plan_id, int feed_back, cudaStream_t s);
// The library's stream and device; the stream is null until the library has been initialised.
cudaStream_t runtime_stream();
int runtime_device();
// Drops every captured graph: called when addresses baked into kernel parameters (peer mappings, exchange
// buffers) stop being valid, so that the next flush of a cached stream is captured afresh.
void invalidate_graphs();
void set_last_error(const std::string& msg);

// Launch helper: plain <<<>>> or cudaLaunchKernelEx with the PDL attribute.
template <typename... KArgs, typename... Args>
inline void launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, bool pdl, Args... args) {
    g_launches++;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = s;
    cudaLaunchAttribute attr[1];
    if (pdl && g_use_pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
    }
    DJ_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...));
}

}  // namespace dj
