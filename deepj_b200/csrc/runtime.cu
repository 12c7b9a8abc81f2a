// Runtime behind the C ABI of include/deepj_cuda.h: the id → device-buffer pool,
// the ComputeGraph command-stream interpreter (validate everything, then launch),
// and the CUDA-graph cache that turns a repeated stream into one graph replay.
//
// Stream format: tensor/ComputeGraph.java:89-147 (strides and buffer slots) and
// :261-518 (the record* encoders); the Metal twin of the interpreter is
// native/deepj_metal_jni.mm:1554-2140.
#include "../../include/deepj_cuda.h"
#include "kernels.h"

#include <cmath>
#include <cstring>
#include <memory>
#include <unordered_map>
#include <vector>

namespace dj {
long long g_launches = 0;
int g_num_sms = 148;
bool g_use_pdl = true;
}  // namespace dj

namespace {

using namespace dj;

thread_local std::string g_err;

enum BufKind { kF32 = 0, kQ8 = 1, kKV = 2, kPlan = 3 };
struct Buf {
    BufKind kind = kF32;
    void* ptr = nullptr;
    size_t bytes = 0;
    size_t floats = 0;                 // kF32
    int K = 0, N = 0, Kp = 0, nb = 0;  // kQ8
    int layers = 0, B = 0, H = 0, maxSeq = 0, hd = 0, kvHalf = 0;   // kKV (kvHalf: fp16 elements)
    unsigned long long serial = 0;
};

struct GraphEntry {
    std::vector<int32_t> stream;
    int seen = 0;
    bool no_graph = false;
    cudaGraphExec_t exec = nullptr;
    size_t kernel_nodes = 0;
    unsigned long long epoch = 0;
    std::vector<std::pair<int, unsigned long long>> refs;
};

struct Runtime {
    bool inited = false;
    int device = 0;
    cudaStream_t stream = nullptr;
    std::unordered_map<int, Buf> pool;
    unsigned long long next_serial = 1;
    unsigned long long epoch = 1;          // bumped whenever a pointer baked into a graph may have died
    float* ws = nullptr;
    size_t ws_floats = 0;
    int* tickets = nullptr;
    std::unordered_map<unsigned long long, GraphEntry> graphs;
    cudaEvent_t t0 = nullptr, t1 = nullptr;
    long long replays = 0, captured = 0, last_nodes = 0;
    bool graphs_enabled = true;
} R;

void ensure_init() {
    if (R.inited) return;
    DJ_CUDA_CHECK(cudaSetDevice(R.device));
    cudaDeviceProp prop;
    DJ_CUDA_CHECK(cudaGetDeviceProperties(&prop, R.device));
    if (prop.major < 10)
        throw std::runtime_error(std::string("libdeepj_cuda_jni is built for sm_100a only; device is ") + prop.name);
    g_num_sms = prop.multiProcessorCount;
    DJ_CUDA_CHECK(cudaStreamCreateWithFlags(&R.stream, cudaStreamNonBlocking));
    DJ_CUDA_CHECK(cudaEventCreate(&R.t0));
    DJ_CUDA_CHECK(cudaEventCreate(&R.t1));
    const char* e = getenv("DEEPJ_CUDA_NO_GRAPH");
    if (e && e[0] == '1') R.graphs_enabled = false;
    e = getenv("DEEPJ_CUDA_NO_PDL");
    if (e && e[0] == '1') g_use_pdl = false;
    e = getenv("DEEPJ_CUDA_GEMV");
    if (e && std::string(e) == "fma") g_gemv_mode = 0;
    if (e && std::string(e) == "cpasync") g_gemv_mode = 1;
    if (e && std::string(e) == "cpasync") g_gemv_mode = 1;
    e = getenv("DEEPJ_CUDA_TRACE");
    if (e && e[0] == '1') {
        DJ_CUDA_CHECK(cudaMalloc((void**)&g_trace, (size_t)kTraceSlots * 8 * sizeof(unsigned long long)));
        DJ_CUDA_CHECK(cudaMemset(g_trace, 0, (size_t)kTraceSlots * 8 * sizeof(unsigned long long)));
        R.graphs_enabled = false;      // slots are handed out per launch, which a replayed graph would not do
    }
    // ticket counters of the split-attention merge and the batched linear, then the greedy pick's (kArgmaxRowsMax)
    // and its partial pairs (2 · 16 per row)
    DJ_CUDA_CHECK(cudaMalloc((void**)&R.tickets, (kAttnTickets + kArgmaxRowsMax * 33) * sizeof(int)));
    DJ_CUDA_CHECK(cudaMemset(R.tickets, 0, (kAttnTickets + kArgmaxRowsMax * 33) * sizeof(int)));
    DJ_CUDA_CHECK(cudaMalloc((void**)&g_dev_error, sizeof(int)));
    DJ_CUDA_CHECK(cudaMemset(g_dev_error, 0, sizeof(int)));
    R.inited = true;
}

void drop_graphs() {
    for (auto& kv : R.graphs) if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
    R.graphs.clear();
}

void free_buf(Buf& b) {
    if (b.ptr) cudaFree(b.ptr);
    b.ptr = nullptr;
}

// ───────────── stream decoding ─────────────

struct Ctx {
    bool execute;
    cudaStream_t s;
    size_t ws_need = 0;
    bool bounded_waits = false;        // the stream holds an op whose kernel waits on a peer (tensor-parallel exchange)
    std::vector<std::pair<int, unsigned long long>>* refs = nullptr;
};

inline float bits_to_float(int32_t b) { float f; std::memcpy(&f, &b, 4); return f; }

Buf& find_buf(Ctx& c, int id, BufKind kind, const char* what) {
    auto it = R.pool.find(id);
    if (it == R.pool.end() || it->second.ptr == nullptr)
        throw std::runtime_error(std::string(what) + ": missing GPU buffer id=" + std::to_string(id));
    if (it->second.kind != kind)
        throw std::runtime_error(std::string(what) + ": buffer id=" + std::to_string(id) + " has the wrong kind");
    if (c.refs) c.refs->push_back({id, it->second.serial});
    return it->second;
}
float* f32(Ctx& c, int id, size_t need, const char* what) {
    Buf& b = find_buf(c, id, kF32, what);
    if (b.floats < need)
        throw std::runtime_error(std::string(what) + ": buffer id=" + std::to_string(id) + " holds " +
                                 std::to_string(b.floats) + " floats, op needs " + std::to_string(need));
    return (float*)b.ptr;
}
float* f32_opt(Ctx& c, int id, size_t need, const char* what) { return id < 0 ? nullptr : f32(c, id, need, what); }
void require(bool ok, const char* what, const char* msg) {
    if (!ok) throw std::runtime_error(std::string(what) + ": " + msg);
}
Q8View q8view(const Buf& b) {
    Q8View v;
    v.codes = (const int8_t*)b.ptr;
    size_t codeBytes = ((size_t)b.N * b.Kp + 255) / 256 * 256;
    v.scales = (const float*)((const char*)b.ptr + codeBytes);
    v.K = b.K; v.N = b.N; v.Kp = b.Kp; v.nb = b.nb;
    return v;
}

int op_stride(int op) {
    switch (op) {
        case 7: case 8: case 9: case 10: case 11: case 12: case 13: case 15: return 4;
        case 1: case 2: case 3: case 4: case 14: case 16: return 5;
        case 6: case 21: case 22: case 36: return 5;
        case 17: case 23: case 29: case 30: case 31: case 33: case 34: case 38: case 41: return 5;
        case 18: case 24: case 25: case 26: case 27: case 28: case 32: case 35: case 39: case 40: return 6;
        case 5: case 19: case 37: case 42: return 7;
        case 20: return 13;
        case DEEPJ_OP_EMBED_GATHER: return 7;
        case DEEPJ_OP_Q8_LINEAR: return 15;
        case DEEPJ_OP_Q8_LINEAR_LN: return 17;
        case DEEPJ_OP_Q8_SWIGLU: return 14;
        case DEEPJ_OP_ATTN_DECODE: return 17;
        case DEEPJ_OP_ATTN_PREFILL: return 18;
        case DEEPJ_OP_SAMPLE_TOPK: return 8;
        case DEEPJ_OP_ARGMAX_ROWS: return 5;
        case DEEPJ_OP_ADD_SCALAR_INPLACE: return 4;
        case DEEPJ_OP_COPY: return 6;
        case DEEPJ_OP_TP_ALLREDUCE: return 7;
        case DEEPJ_OP_TP_ALLGATHER: return 5;
        case DEEPJ_OP_DECODE_STEP: return 3;
        default: return -1;
    }
}

inline size_t sz(int a, int b) { return (size_t)a * (size_t)b; }

// Decode one op at c; validate; launch when ctx.execute.
void do_op(Ctx& ctx, const int32_t* c) {
    const int op = c[0];
    cudaStream_t s = ctx.s;
    const bool go = ctx.execute;
    switch (op) {
        case 1: case 2: case 3: case 4: case 14: case 16: {
            int n = c[4]; require(n >= 0, "binary op", "negative element count");
            const float* a = f32(ctx, c[1], n, "binary op"); const float* b = f32(ctx, c[2], n, "binary op");
            float* o = f32(ctx, c[3], n, "binary op");
            if (go) launch_binary(op, a, b, o, n, s);
            break;
        }
        case 7: case 8: case 9: case 10: case 11: case 12: case 13: case 15: {
            int n = c[3]; require(n >= 0, "unary op", "negative element count");
            const float* a = f32(ctx, c[1], n, "unary op"); float* o = f32(ctx, c[2], n, "unary op");
            if (go) launch_unary(op, a, o, n, s);
            break;
        }
        case 6: case 21: case 22: case 36: {
            int n = c[4]; require(n >= 0, "scalar op", "negative element count");
            const float* a = f32(ctx, c[1], n, "scalar op"); float* o = f32(ctx, c[2], n, "scalar op");
            if (go) launch_scalar(op, a, o, bits_to_float(c[3]), n, s);
            break;
        }
        case 35: {
            int n = c[5]; require(n >= 0, "clamp", "negative element count");
            const float* a = f32(ctx, c[1], n, "clamp"); float* o = f32(ctx, c[2], n, "clamp");
            if (go) launch_clamp(a, o, bits_to_float(c[3]), bits_to_float(c[4]), n, s);
            break;
        }
        case 5: {   // [5, a, b, out, m, n, k]
            int m = c[4], n = c[5], k = c[6];
            require(m >= 0 && n >= 0 && k >= 0, "matmul", "negative dimension");
            const float* a = f32(ctx, c[1], sz(m, k), "matmul"); const float* b = f32(ctx, c[2], sz(k, n), "matmul");
            float* o = f32(ctx, c[3], sz(m, n), "matmul");
            if (go) launch_matmul_f32(a, b, o, m, n, k, s);
            break;
        }
        case 17: case 23: case 29: case 30: case 31: case 33: case 34: case 38: case 41: {
            int rows = c[3], cols = c[4];
            require(rows >= 0 && cols >= 0, "row/col op", "negative dimension");
            size_t outN = (op == 17 || op == 23) ? sz(rows, cols) : (op == 29 ? (size_t)cols : (op == 41 ? 1 : (size_t)rows));
            const float* a = f32(ctx, c[1], sz(rows, cols), "row/col op"); float* o = f32(ctx, c[2], outN, "row/col op");
            if (!go) break;
            if (op == 17) launch_softmax_rows(a, o, rows, cols, s);
            else if (op == 23) launch_transpose(a, o, rows, cols, s);
            else if (op == 29) launch_sum_rows(a, o, rows, cols, s);
            else if (op == 41) launch_sum_scalar(a, o, (long long)rows * cols, s);
            else launch_row_reduce(op, a, o, rows, cols, s);
            break;
        }
        case 24: case 28: case 25: case 26: case 27: case 32: {
            int rows = c[4], cols = c[5];
            require(rows >= 0 && cols >= 0, "broadcast op", "negative dimension");
            bool rowVec = (op == 24 || op == 28);
            const float* a = f32(ctx, c[1], sz(rows, cols), "broadcast op");
            const float* v = f32(ctx, c[2], rowVec ? cols : rows, "broadcast op");
            float* o = f32(ctx, c[3], sz(rows, cols), "broadcast op");
            if (!go) break;
            if (rowVec) launch_row_broadcast(op, a, v, o, rows, cols, s); else launch_col_broadcast(op, a, v, o, rows, cols, s);
            break;
        }
        case 18: {
            int rows = c[4], cols = c[5]; require(rows >= 0 && cols >= 0, "softmaxBackward", "negative dimension");
            const float* g = f32(ctx, c[1], sz(rows, cols), "softmaxBackward"); const float* sm = f32(ctx, c[2], sz(rows, cols), "softmaxBackward");
            float* o = f32(ctx, c[3], sz(rows, cols), "softmaxBackward");
            if (go) launch_softmax_backward(g, sm, o, rows, cols, s);
            break;
        }
        case 19: {
            int rows = c[5], cols = c[6]; require(rows >= 0 && cols >= 0, "layerNormBackward", "negative dimension");
            const float* a = f32(ctx, c[1], sz(rows, cols), "layerNormBackward"); const float* b = f32(ctx, c[2], sz(rows, cols), "layerNormBackward");
            const float* sd = f32(ctx, c[3], rows, "layerNormBackward"); float* o = f32(ctx, c[4], sz(rows, cols), "layerNormBackward");
            if (go) launch_layernorm_backward(a, b, sd, o, rows, cols, s);
            break;
        }
        case 20: {
            int n = c[12]; require(n >= 0, "adamW", "negative element count");
            float* w = f32(ctx, c[1], n, "adamW"); const float* g = f32(ctx, c[2], n, "adamW");
            float* mt = f32(ctx, c[3], n, "adamW"); float* vt = f32(ctx, c[4], n, "adamW");
            if (go) launch_adamw(w, g, mt, vt, bits_to_float(c[5]), bits_to_float(c[6]), bits_to_float(c[7]), bits_to_float(c[8]),
                                 bits_to_float(c[9]), bits_to_float(c[10]), bits_to_float(c[11]), n, s);
            break;
        }
        case 37: case 42: {
            int tRows = c[4], tCols = c[5], nIdx = c[6];
            require(tRows >= 0 && tCols >= 0 && nIdx >= 0, "scatterAddRows", "negative dimension");
            float* t = f32(ctx, c[1], sz(tRows, tCols), "scatterAddRows"); const float* idx = f32(ctx, c[2], nIdx, "scatterAddRows");
            const float* g = f32(ctx, c[3], sz(nIdx, tCols), "scatterAddRows");
            if (go) launch_scatter_add_rows(t, idx, g, tRows, tCols, nIdx, s);
            break;
        }
        case 39: case 40: {
            int rows = c[4], cols = c[5]; require(rows >= 0 && cols >= 0, "crossEntropy", "negative dimension");
            const float* lg = f32(ctx, c[1], sz(rows, cols), "crossEntropy"); const float* tg = f32(ctx, c[2], rows, "crossEntropy");
            float* o = f32(ctx, c[3], op == 39 ? (size_t)rows : sz(rows, cols), "crossEntropy");
            if (!go) break;
            if (op == 39) launch_ce_loss(lg, tg, o, rows, cols, s); else launch_ce_grad(lg, tg, o, rows, cols, s);
            break;
        }
        case DEEPJ_OP_EMBED_GATHER: {   // [op, table, ids, out, rows, d, vocab]
            int rows = c[4], d = c[5], vocab = c[6];
            require(rows >= 0 && d > 0 && vocab > 0, "embedGather", "bad dimension");
            const float* table = f32(ctx, c[1], sz(vocab, d), "embedGather"); const float* ids = f32(ctx, c[2], rows, "embedGather");
            float* o = f32(ctx, c[3], sz(rows, d), "embedGather");
            if (go) launch_embed_gather(table, ids, o, rows, d, vocab, s);
            break;
        }
        case DEEPJ_OP_Q8_LINEAR:
        case DEEPJ_OP_Q8_LINEAR_LN: {
            // 65: [op, x, x_off, ldx, gamma, epsBits, w, bias, residual, res_off, ldr, out, out_off, ldo, M]
            // 75: [op, x, x_off, ldx, gamma, beta, epsBits, w, bias, residual, res_off, ldr, out, out_off, ldo, M, act]
            const bool ln = op == DEEPJ_OP_Q8_LINEAR_LN;
            const int32_t* e = ln ? c + 1 : c;          // fields from epsBits on sit one slot later in op 75
            int x_off = c[2], ldx = c[3], res_off = e[9], ldr = e[10], out_off = e[12], ldo = e[13], M = e[14];
            Buf& wb = find_buf(ctx, e[6], kQ8, "q8Linear");
            require(M >= 1 && x_off >= 0 && out_off >= 0 && res_off >= 0, "q8Linear", "bad M or offset");
            require(ldx >= wb.K && ldo >= wb.N, "q8Linear", "row stride smaller than the row");
            Q8LinearArgs a = {};
            a.x = f32(ctx, c[1], (size_t)x_off + sz(M - 1, ldx) + wb.K, "q8Linear") + x_off; a.ldx = ldx;
            a.gamma = f32_opt(ctx, c[4], wb.K, "q8Linear"); a.eps = bits_to_float(e[5]);
            a.w = q8view(wb);
            a.bias = f32_opt(ctx, e[7], wb.N, "q8Linear");
            if (e[8] >= 0) {
                require(ldr >= wb.N, "q8Linear", "residual stride smaller than the row");
                a.residual = f32(ctx, e[8], (size_t)res_off + sz(M - 1, ldr) + wb.N, "q8Linear") + res_off; a.ldr = ldr;
            }
            a.out = f32(ctx, e[11], (size_t)out_off + sz(M - 1, ldo) + wb.N, "q8Linear") + out_off; a.ldo = ldo;
            a.M = M;
            size_t need = 0;
            if (M >= 3) {
                need = q8_batch_ws_floats(wb.K, wb.N, false);
                if (M >= kTcMinRows) need = std::max(need, q8_tc_ws_floats(M, wb.K, wb.N));
                a.ws = R.ws; a.tickets = R.tickets;
            }
            if (ln) {
                a.act = c[16];
                require(a.act == 0 || a.act == 1, "q8LinearLN", "activation must be 0 (none) or 1 (GELU)");
                require(a.act == 0 || a.residual == nullptr, "q8LinearLN", "an activation and a residual cannot be combined");
                a.beta = f32_opt(ctx, c[5], wb.K, "q8LinearLN");
                require((a.beta == nullptr) == (a.gamma == nullptr), "q8LinearLN", "LayerNorm needs both gamma and beta (or neither)");
                if (a.beta != nullptr) {             // room for the normalised rows when the kernel chosen cannot fuse the norm
                    need = (need + 31) & ~(size_t)31;      // 128-byte aligned rows for the vector loads that follow
                    a.ln_ws = R.ws + need;
                    need += sz(M, wb.K);
                }
            }
            if (need > ctx.ws_need) ctx.ws_need = need;
            if (go) launch_q8_linear(a, s);
            break;
        }
        case DEEPJ_OP_Q8_SWIGLU: {
            // [op, x, x_off, ldx, gamma, epsBits, w_gate, b_gate, w_up, b_up, out, out_off, ldo, M]
            int x_off = c[2], ldx = c[3], out_off = c[11], ldo = c[12], M = c[13];
            Buf& wg = find_buf(ctx, c[6], kQ8, "q8SwiGLU");
            Buf& wu = find_buf(ctx, c[8], kQ8, "q8SwiGLU");
            require(wg.K == wu.K && wg.N == wu.N, "q8SwiGLU", "gate and up projections differ in shape");
            require(M >= 1 && x_off >= 0 && out_off >= 0, "q8SwiGLU", "bad M or offset");
            require(ldx >= wg.K && ldo >= wg.N, "q8SwiGLU", "row stride smaller than the row");
            Q8LinearArgs a = {};
            a.x = f32(ctx, c[1], (size_t)x_off + sz(M - 1, ldx) + wg.K, "q8SwiGLU") + x_off; a.ldx = ldx;
            a.gamma = f32_opt(ctx, c[4], wg.K, "q8SwiGLU"); a.eps = bits_to_float(c[5]);
            a.w = q8view(wg); a.bias = f32_opt(ctx, c[7], wg.N, "q8SwiGLU");
            a.w2 = q8view(wu); a.bias2 = f32_opt(ctx, c[9], wu.N, "q8SwiGLU");
            a.out = f32(ctx, c[10], (size_t)out_off + sz(M - 1, ldo) + wg.N, "q8SwiGLU") + out_off; a.ldo = ldo;
            a.M = M;
            if (M >= 3) {
                size_t need = q8_batch_ws_floats(wg.K, wg.N, true);
                if (M >= kTcMinRows) need = std::max(need, q8_tc_ws_floats(M, wg.K, wg.N));
                if (need > ctx.ws_need) ctx.ws_need = need;
                a.ws = R.ws; a.tickets = R.tickets;
            }
            if (go) launch_q8_linear(a, s);
            break;
        }
        case DEEPJ_OP_ATTN_DECODE:
        case DEEPJ_OP_ATTN_PREFILL: {
            // [op, qkv, q_off, k_off, v_off, ld, kv, layer, pos, cos, sin, out, out_off, ldo, B, H, hd (, T)]
            // prefill: rows b·T + t of qkv / out are tokens pos[b] + t, t < T, of sequence b
            int q_off = c[2], k_off = c[3], v_off = c[4], ld = c[5], layer = c[7], out_off = c[12], ldo = c[13];
            int B = c[14], H = c[15], hd = c[16];
            const int T = op == DEEPJ_OP_ATTN_PREFILL ? c[17] : 1;
            require(T >= 1 && (long)B * T <= 65535, "attnPrefill", "bad token count");
            const int rows = B * T;
            Buf& kv = find_buf(ctx, c[6], kKV, "attnDecode");
            require(B >= 1 && H >= 1 && hd >= 2, "attnDecode", "bad dimension");
            require(B <= kv.B && H == kv.H && hd == kv.hd, "attnDecode", "shape does not match the KV cache");
            require(layer >= 0 && layer < kv.layers, "attnDecode", "layer out of range");
            require(q_off >= 0 && k_off >= 0 && v_off >= 0 && out_off >= 0, "attnDecode", "negative offset");
            require(ld % 4 == 0 && q_off % 4 == 0 && k_off % 4 == 0 && v_off % 4 == 0, "attnDecode", "offsets and stride must be multiples of 4 floats");
            int d = H * hd;
            int maxOff = std::max(q_off, std::max(k_off, v_off));
            require(ld >= maxOff + d && ldo >= d, "attnDecode", "row stride smaller than the row");
            AttnDecodeArgs a = {};
            a.qkv = f32(ctx, c[1], sz(rows - 1, ld) + maxOff + d, "attnDecode"); a.q_off = q_off; a.k_off = k_off; a.v_off = v_off; a.ld = ld;
            size_t plane = (size_t)kv.layers * kv.B * kv.H * kv.maxSeq * kv.hd;
            size_t layerOff = (size_t)layer * kv.B * kv.H * kv.maxSeq * kv.hd;
            const size_t esz = kv.kvHalf ? 2 : 4;
            a.kcache = (char*)kv.ptr + layerOff * esz; a.vcache = (char*)kv.ptr + (plane + layerOff) * esz;
            a.maxSeq = kv.maxSeq; a.kvHalf = kv.kvHalf;
            a.pos = f32(ctx, c[8], B, "attnDecode");
            a.cosT = f32(ctx, c[9], sz(kv.maxSeq, hd / 2), "attnDecode"); a.sinT = f32(ctx, c[10], sz(kv.maxSeq, hd / 2), "attnDecode");
            a.out = f32(ctx, c[11], (size_t)out_off + sz(rows - 1, ldo) + d, "attnDecode") + out_off; a.ldo = ldo;
            a.B = B; a.H = H; a.hd = hd; a.T = T;
            a.scale = (float)(1.0 / std::sqrt((double)hd));     // MultiHeadSelfAttention.java:44
            a.splits = attn_decode_splits(rows, H, kv.maxSeq);
            size_t need = attn_decode_ws_floats(rows, H, hd, a.splits);
            if (need > ctx.ws_need) ctx.ws_need = need;
            a.ws = R.ws;
            a.tickets = R.tickets;
            if (go) launch_attn_decode(a, s);
            break;
        }
        case DEEPJ_OP_ARGMAX_ROWS: {
            int rows = c[3], cols = c[4]; require(rows >= 0 && cols >= 1, "argmaxRows", "bad dimension");
            const float* a = f32(ctx, c[1], sz(rows, cols), "argmaxRows"); float* o = f32(ctx, c[2], rows, "argmaxRows");
            if (go) launch_argmax_rows(a, o, rows, cols, R.tickets + kAttnTickets + kArgmaxRowsMax, R.tickets + kAttnTickets, s);
            break;
        }
        case DEEPJ_OP_SAMPLE_TOPK: {     // [op, logits, r, out, rows, cols, topK, temperatureBits]
            int rows = c[4], cols = c[5], topK = c[6];
            require(rows >= 0 && cols >= 1, "sampleTopK", "bad dimension");
            require(topK >= 0, "sampleTopK", "topK must be >= 0 (0 = the whole vocabulary)");
            const float temperature = bits_to_float(c[7]);
            require(temperature > 0.0f, "sampleTopK", "temperature must be > 0");
            const float* lg = f32(ctx, c[1], sz(rows, cols), "sampleTopK");
            const float* rr = f32(ctx, c[2], rows, "sampleTopK");
            float* o = f32(ctx, c[3], rows, "sampleTopK");
            const size_t need = sample_topk_ws_floats(rows, cols, topK);
            if (need > ctx.ws_need) ctx.ws_need = need;
            if (go) launch_sample_topk(lg, rr, o, rows, cols, topK, temperature, R.ws, s);
            break;
        }
        case DEEPJ_OP_ADD_SCALAR_INPLACE: {
            int n = c[3]; require(n >= 0, "addScalarInPlace", "negative element count");
            float* b = f32(ctx, c[1], n, "addScalarInPlace");
            if (go) launch_add_scalar_inplace(b, bits_to_float(c[2]), n, s);
            break;
        }
        case DEEPJ_OP_COPY: {   // [op, src, src_off, dst, dst_off, n]
            int so = c[2], dof = c[4], n = c[5]; require(so >= 0 && dof >= 0 && n >= 0, "copy", "bad offset or count");
            const float* src = f32(ctx, c[1], (size_t)so + n, "copy") + so; float* dst = f32(ctx, c[3], (size_t)dof + n, "copy") + dof;
            if (go) launch_copy(src, dst, n, s);
            break;
        }
        case DEEPJ_OP_TP_ALLREDUCE: {   // [op, in, bias, residual, out, M, N]
            int M = c[5], N = c[6]; require(M >= 1 && N >= 1, "tpAllReduce", "bad dimension");
            require(tp_ready(), "tpAllReduce", "deepj_cuda_tp_connect has not been called");
            const float* in = f32(ctx, c[1], sz(M, N), "tpAllReduce");
            const float* bias = f32_opt(ctx, c[2], N, "tpAllReduce");
            const float* res = f32_opt(ctx, c[3], sz(M, N), "tpAllReduce");
            float* o = f32(ctx, c[4], sz(M, N), "tpAllReduce");
            ctx.bounded_waits = true;
            if (go) launch_tp_exchange(in, bias, res, o, M, N, 0, s);
            break;
        }
        case DEEPJ_OP_TP_ALLGATHER: {   // [op, in, out, M, n_local]
            int M = c[3], nl = c[4]; require(M >= 1 && nl >= 1, "tpAllGather", "bad dimension");
            require(tp_ready(), "tpAllGather", "deepj_cuda_tp_connect has not been called");
            const float* in = f32(ctx, c[1], sz(M, nl), "tpAllGather");
            float* o = f32(ctx, c[2], sz(M, nl) * tp_world(), "tpAllGather");
            ctx.bounded_waits = true;
            if (go) launch_tp_exchange(in, nullptr, nullptr, o, M, nl, 1, s);
            break;
        }
        case DEEPJ_OP_DECODE_STEP: {   // [op, plan, feed_back]
            require(c[2] == 0 || c[2] == 1, "decodeStep", "feed_back must be 0 or 1");
            find_buf(ctx, c[1], kPlan, "decodeStep");
            decode_step_check(c[1], ctx.refs);
            if (tp_world() > 1) ctx.bounded_waits = true;
            if (go) launch_decode_step(c[1], c[2], s);
            break;
        }
        default:
            throw std::runtime_error("Unknown op code in command stream: " + std::to_string(op));
    }
}

int walk(Ctx& ctx, const int32_t* cmd, int len) {
    int pos = 0, nops = 0;

    while (pos < len) {
        int stride = op_stride(cmd[pos]);
        if (stride < 0) throw std::runtime_error("Unknown op code in command stream: " + std::to_string(cmd[pos]));
        if (pos + stride > len) throw std::runtime_error("Truncated command stream at int " + std::to_string(pos));
        do_op(ctx, cmd + pos);
        pos += stride;
        nops++;
    }
    return nops;
}

void ensure_ws(size_t floats) {
    if (floats <= R.ws_floats) return;
    DJ_CUDA_CHECK(cudaStreamSynchronize(R.stream));
    if (R.ws) cudaFree(R.ws);
    R.ws = nullptr; R.ws_floats = 0;
    DJ_CUDA_CHECK(cudaMalloc((void**)&R.ws, floats * sizeof(float)));
    R.ws_floats = floats;
    R.epoch++;
    drop_graphs();
}

unsigned long long hash_stream(const int32_t* cmd, int len) {
    unsigned long long h = 1469598103934665603ULL;
    for (int i = 0; i < len; i++) { h ^= (unsigned int)cmd[i]; h *= 1099511628211ULL; }
    return h ^ (unsigned long long)len;
}

bool graph_still_valid(GraphEntry& g) {
    if (g.epoch == R.epoch) return true;
    for (auto& r : g.refs) {
        auto it = R.pool.find(r.first);
        if (it == R.pool.end() || it->second.serial != r.second) return false;
    }
    g.epoch = R.epoch;
    return true;
}

void flush(const int32_t* cmd, int len, bool sync) {
    ensure_init();
    if (len < 0) throw std::runtime_error("negative command stream length");
    if (len > 0 && cmd == nullptr) throw std::runtime_error("null command stream");
    std::vector<std::pair<int, unsigned long long>> refs;
    Ctx v; v.execute = false; v.s = R.stream; v.refs = &refs;
    walk(v, cmd, len);
    ensure_ws(v.ws_need);

    GraphEntry* ge = nullptr;
    if (R.graphs_enabled && len > 0) {
        unsigned long long h = hash_stream(cmd, len);
        auto it = R.graphs.find(h);
        if (it == R.graphs.end()) {
            if (R.graphs.size() >= 512) {      // streams that never repeated
                for (auto i = R.graphs.begin(); i != R.graphs.end();) { if (!i->second.exec) i = R.graphs.erase(i); else ++i; }
            }
            GraphEntry e; e.seen = 0;
            it = R.graphs.emplace(h, std::move(e)).first;
        }
        ge = &it->second;
        if (ge->exec) {
            bool same = (int)ge->stream.size() == len && std::memcmp(ge->stream.data(), cmd, (size_t)len * 4) == 0;
            if (!same || !graph_still_valid(*ge)) { cudaGraphExecDestroy(ge->exec); ge->exec = nullptr; ge->seen = 0; ge->stream.clear(); }
        }
    }

    if (ge && ge->exec) {
        DJ_CUDA_CHECK(cudaGraphLaunch(ge->exec, R.stream));
        R.replays++; R.last_nodes = (long long)ge->kernel_nodes;
    } else if (ge && ge->seen >= 1 && !ge->no_graph) {
        // second sighting: capture, instantiate, replay
        cudaGraph_t graph = nullptr;
        long long before = g_launches;
        DJ_CUDA_CHECK(cudaStreamBeginCapture(R.stream, cudaStreamCaptureModeRelaxed));
        bool ok = true; std::string why;
        try {
            Ctx x; x.execute = true; x.s = R.stream;
            walk(x, cmd, len);
        } catch (const std::exception& e) { ok = false; why = e.what(); }
        cudaError_t ce = cudaStreamEndCapture(R.stream, &graph);
        size_t nodes = (size_t)(g_launches - before);
        g_launches = before;            // captured launches are counted when replayed
        if (ok && ce == cudaSuccess && graph) {
            cudaGraphExec_t exec = nullptr;
            ce = cudaGraphInstantiate(&exec, graph, 0);
            cudaGraphDestroy(graph);
            if (ce == cudaSuccess) {
                ge->exec = exec; ge->stream.assign(cmd, cmd + len); ge->refs = refs; ge->epoch = R.epoch; ge->kernel_nodes = nodes;
                R.captured++;
                DJ_CUDA_CHECK(cudaGraphLaunch(ge->exec, R.stream));
                R.replays++; R.last_nodes = (long long)nodes;
            } else { ok = false; why = cudaGetErrorString(ce); }
        } else if (ok) { ok = false; why = cudaGetErrorString(ce); if (graph) cudaGraphDestroy(graph); }
        if (!ok) {
            cudaGetLastError();
            ge->no_graph = true;
            Ctx x; x.execute = true; x.s = R.stream;
            walk(x, cmd, len);
        }
    } else {
        Ctx x; x.execute = true; x.s = R.stream;
        walk(x, cmd, len);
        if (ge) ge->seen++;
    }
    if (sync) {
        DJ_CUDA_CHECK(cudaStreamSynchronize(R.stream));
        if (v.bounded_waits) {
            // a wait on a peer that ran out leaves a code in the device error word; the results of this flush are
            // then incomplete, which a synchronous caller learns here (an asynchronous one from deepj_cuda_stats)
            int code = 0;
            DJ_CUDA_CHECK(cudaMemcpy(&code, g_dev_error, sizeof(int), cudaMemcpyDeviceToHost));
            if (code != 0)
                throw std::runtime_error("a bounded wait inside a kernel expired (device error word " + std::to_string(code) +
                                         (code >= 100 && code < 200 ? ": no data from tensor-parallel rank " + std::to_string(code - 100) : std::string()) +
                                         "); the results of this flush are incomplete, the context stays usable");
        }
    }
}

}  // namespace

namespace dj {
bool pool_f32(int id, PoolF32* out) {
    auto it = R.pool.find(id);
    if (it == R.pool.end() || it->second.kind != kF32 || it->second.ptr == nullptr) return false;
    out->ptr = (float*)it->second.ptr; out->floats = it->second.floats;
    return true;
}
bool pool_kv(int id, PoolKV* out) {
    auto it = R.pool.find(id);
    if (it == R.pool.end() || it->second.kind != kKV || it->second.ptr == nullptr) return false;
    const Buf& b = it->second;
    out->ptr = b.ptr; out->layers = b.layers; out->B = b.B; out->H = b.H; out->maxSeq = b.maxSeq; out->hd = b.hd; out->half = b.kvHalf;
    return true;
}
void invalidate_graphs() { R.epoch++; drop_graphs(); }
bool pool_q8(int id, Q8View* out) {
    auto it = R.pool.find(id);
    if (it == R.pool.end() || it->second.kind != kQ8 || it->second.ptr == nullptr) return false;
    *out = q8view(it->second);
    return true;
}
unsigned long long pool_serial(int id) {
    auto it = R.pool.find(id);
    return it == R.pool.end() ? 0ull : it->second.serial;
}
void pool_add_plan(int id, void* dev_ptr, size_t bytes) {
    Buf b; b.kind = kPlan; b.ptr = dev_ptr; b.bytes = bytes;
    b.serial = R.next_serial++;
    R.pool[id] = b;
}
cudaStream_t runtime_stream() { return R.inited ? R.stream : nullptr; }
int runtime_device() { return R.device; }
void set_last_error(const std::string& msg) { g_err = msg; }
}  // namespace dj

#define DJ_TRY try {
#define DJ_CATCH } catch (const std::exception& e) { g_err = e.what(); return 1; } catch (...) { g_err = "unknown error"; return 1; } return 0;

extern "C" {

const char* deepj_cuda_last_error(void) { return g_err.c_str(); }

int deepj_cuda_init(int32_t device) {
    DJ_TRY
    if (R.inited && R.device != device) throw std::runtime_error("already bound to device " + std::to_string(R.device));
    R.device = device;
    ensure_init();
    DJ_CATCH
}

int deepj_cuda_shutdown(void) {
    DJ_TRY
    if (!R.inited) return 0;
    cudaStreamSynchronize(R.stream);
    drop_graphs();
    for (auto& kv : R.pool) free_buf(kv.second);
    R.pool.clear();
    if (R.ws) cudaFree(R.ws);
    R.ws = nullptr; R.ws_floats = 0;
    R.epoch++;
    DJ_CATCH
}

int deepj_cuda_alloc_buffers(const int32_t* ids, const int32_t* sizes, int32_t count) {
    DJ_TRY
    ensure_init();
    if (count < 0) throw std::runtime_error("negative buffer count");
    for (int i = 0; i < count; i++) {
        if (sizes[i] < 0) throw std::runtime_error("negative buffer size for id=" + std::to_string(ids[i]));
        if (R.pool.count(ids[i])) continue;                    // native/deepj_metal_jni.mm:1489
        Buf b; b.kind = kF32; b.floats = (size_t)sizes[i]; b.bytes = std::max<size_t>(b.floats * 4, 4);
        DJ_CUDA_CHECK(cudaMalloc(&b.ptr, b.bytes));
        DJ_CUDA_CHECK(cudaMemsetAsync(b.ptr, 0, b.bytes, R.stream));
        b.serial = R.next_serial++;
        R.pool[ids[i]] = b;
    }
    DJ_CATCH
}

int deepj_cuda_upload_buffer(int32_t id, const float* data, int32_t len) {
    DJ_TRY
    ensure_init();
    auto it = R.pool.find(id);
    if (it == R.pool.end() || it->second.kind != kF32) throw std::runtime_error("Buffer not found for upload");
    if (len < 0 || (size_t)len > it->second.floats) throw std::runtime_error("upload of " + std::to_string(len) + " floats exceeds buffer id=" + std::to_string(id));
    if (len > 0) DJ_CUDA_CHECK(cudaMemcpyAsync(it->second.ptr, data, (size_t)len * 4, cudaMemcpyHostToDevice, R.stream));
    DJ_CATCH
}

int deepj_cuda_download_buffer(int32_t id, float* out, int32_t len) {
    DJ_TRY
    ensure_init();
    auto it = R.pool.find(id);
    if (it == R.pool.end() || it->second.kind != kF32) throw std::runtime_error("Buffer not found for download");
    if (len < 0 || (size_t)len > it->second.floats) throw std::runtime_error("download of " + std::to_string(len) + " floats exceeds buffer id=" + std::to_string(id));
    if (len > 0) DJ_CUDA_CHECK(cudaMemcpyAsync(out, it->second.ptr, (size_t)len * 4, cudaMemcpyDeviceToHost, R.stream));
    DJ_CUDA_CHECK(cudaStreamSynchronize(R.stream));
    DJ_CATCH
}

int deepj_cuda_release_buffers(const int32_t* ids, int32_t count) {
    DJ_TRY
    if (!R.inited) return 0;
    bool any = false;
    for (int i = 0; i < count; i++) {
        auto it = R.pool.find(ids[i]);
        if (it == R.pool.end()) continue;                      // native/deepj_metal_jni.mm:1545-1547
        if (!any) { DJ_CUDA_CHECK(cudaStreamSynchronize(R.stream)); any = true; }
        free_buf(it->second);
        R.pool.erase(it);
    }
    if (any) R.epoch++;
    DJ_CATCH
}

int deepj_cuda_flush_ops(const int32_t* cmd, int32_t len) { DJ_TRY flush(cmd, len, true); DJ_CATCH }
int deepj_cuda_flush_ops_async(const int32_t* cmd, int32_t len) { DJ_TRY flush(cmd, len, false); DJ_CATCH }
int deepj_cuda_synchronize(void) { DJ_TRY ensure_init(); DJ_CUDA_CHECK(cudaStreamSynchronize(R.stream)); DJ_CATCH }

// Page-locked host memory for the per-step token / result staging: uploads from and downloads into it are true
// asynchronous DMA transfers on the library's stream.
int deepj_cuda_pinned_alloc(void** out, int64_t bytes) {
    DJ_TRY
    ensure_init();
    if (out == nullptr || bytes <= 0) throw std::runtime_error("pinned_alloc: bad arguments");
    DJ_CUDA_CHECK(cudaMallocHost(out, (size_t)bytes));
    DJ_CATCH
}
int deepj_cuda_pinned_free(void* p) { DJ_TRY if (p) DJ_CUDA_CHECK(cudaFreeHost(p)); DJ_CATCH }

int deepj_cuda_timer_begin(void) { DJ_TRY ensure_init(); DJ_CUDA_CHECK(cudaEventRecord(R.t0, R.stream)); DJ_CATCH }
int deepj_cuda_timer_end(float* ms) {
    DJ_TRY
    ensure_init();
    DJ_CUDA_CHECK(cudaEventRecord(R.t1, R.stream));
    DJ_CUDA_CHECK(cudaEventSynchronize(R.t1));
    DJ_CUDA_CHECK(cudaEventElapsedTime(ms, R.t0, R.t1));
    DJ_CATCH
}

int deepj_cuda_profile_ops(const int32_t* cmd, int32_t len, float* ms_per_op, int32_t max_ops, int32_t* n_ops) {
    DJ_TRY
    ensure_init();
    Ctx v; v.execute = false; v.s = R.stream;
    int nops = walk(v, cmd, len);
    ensure_ws(v.ws_need);
    if (n_ops) *n_ops = nops;
    if (nops > max_ops) throw std::runtime_error("profile buffer too small: stream has " + std::to_string(nops) + " ops");
    std::vector<cudaEvent_t> ev(nops + 1);
    for (auto& e : ev) DJ_CUDA_CHECK(cudaEventCreate(&e));
    Ctx x; x.execute = true; x.s = R.stream;
    int pos = 0, i = 0;
    DJ_CUDA_CHECK(cudaEventRecord(ev[0], R.stream));
    while (pos < len) {
        do_op(x, cmd + pos);
        pos += op_stride(cmd[pos]);
        DJ_CUDA_CHECK(cudaEventRecord(ev[++i], R.stream));
    }
    DJ_CUDA_CHECK(cudaStreamSynchronize(R.stream));
    for (int k = 0; k < nops; k++) DJ_CUDA_CHECK(cudaEventElapsedTime(&ms_per_op[k], ev[k], ev[k + 1]));
    for (auto& e : ev) cudaEventDestroy(e);
    DJ_CATCH
}

int deepj_cuda_stats(int64_t* counters, int32_t n) {
    DJ_TRY
    int dev_err = 0;
    if (R.inited && g_dev_error) {
        DJ_CUDA_CHECK(cudaStreamSynchronize(R.stream));
        DJ_CUDA_CHECK(cudaMemcpy(&dev_err, g_dev_error, sizeof(int), cudaMemcpyDeviceToHost));
    }
    int64_t v[6] = {g_launches, R.replays, R.captured, R.last_nodes, (int64_t)(R.ws_floats * 4), dev_err};
    for (int i = 0; i < n && i < 6; i++) counters[i] = v[i];
    DJ_CATCH
}

int deepj_cuda_trace_read(uint64_t* out, int32_t max_launches, int32_t* n_launches) {
    DJ_TRY
    ensure_init();
    if (!g_trace) throw std::runtime_error("tracing is off (set DEEPJ_CUDA_TRACE=1 before the first call)");
    DJ_CUDA_CHECK(cudaStreamSynchronize(R.stream));
    long long n = g_trace_launches < kTraceSlots ? g_trace_launches : kTraceSlots;
    if (n > max_launches) n = max_launches;
    if (n_launches) *n_launches = (int32_t)n;
    if (n > 0) DJ_CUDA_CHECK(cudaMemcpy(out, g_trace, (size_t)n * 8 * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
    DJ_CATCH
}

int deepj_cuda_q8_alloc(int32_t id, int32_t K, int32_t N) {
    DJ_TRY
    ensure_init();
    if (K <= 0 || N <= 0) throw std::runtime_error("q8_alloc: K and N must be positive");
    if (R.pool.count(id)) throw std::runtime_error("q8_alloc: id " + std::to_string(id) + " already exists");
    Buf b; b.kind = kQ8; b.K = K; b.N = N; b.Kp = (K + 15) / 16 * 16; b.nb = (K + 31) / 32;
    size_t codeBytes = ((size_t)N * b.Kp + 255) / 256 * 256;
    b.bytes = codeBytes + (size_t)N * b.nb * 4;
    DJ_CUDA_CHECK(cudaMalloc(&b.ptr, b.bytes));
    DJ_CUDA_CHECK(cudaMemsetAsync(b.ptr, 0, b.bytes, R.stream));
    b.serial = R.next_serial++;
    R.pool[id] = b;
    DJ_CATCH
}

int deepj_cuda_q8_quantize_into(int32_t q8_id, int32_t dst_col0, int32_t src_id, int32_t src_row0, int32_t src_col0,
                                int32_t src_ld, int32_t n_cols) {
    DJ_TRY
    ensure_init();
    Ctx c; c.execute = false; c.s = R.stream;
    Buf& q = find_buf(c, q8_id, kQ8, "q8_quantize_into");
    if (dst_col0 < 0 || n_cols < 0 || dst_col0 + n_cols > q.N) throw std::runtime_error("q8_quantize_into: destination columns out of range");
    if (src_row0 < 0 || src_col0 < 0 || src_ld < src_col0 + n_cols) throw std::runtime_error("q8_quantize_into: source window out of range");
    const float* src = f32(c, src_id, (size_t)(src_row0 + q.K - 1) * src_ld + src_col0 + n_cols, "q8_quantize_into");
    Q8View v = q8view(q);
    launch_q8_quantize(src + (size_t)src_row0 * src_ld + src_col0, src_ld, q.K, n_cols,
                       (int8_t*)v.codes + (size_t)dst_col0 * q.Kp, (float*)v.scales + (size_t)dst_col0 * q.nb, q.Kp, q.nb, R.stream);
    DJ_CATCH
}

int deepj_cuda_q8_upload(int32_t q8_id, const int8_t* codes, const float* scales) {
    DJ_TRY
    ensure_init();
    Ctx c; c.execute = false; c.s = R.stream;
    Buf& q = find_buf(c, q8_id, kQ8, "q8_upload");
    Q8View v = q8view(q);
    DJ_CUDA_CHECK(cudaMemcpy2DAsync((void*)v.codes, q.Kp, codes, q.K, q.K, q.N, cudaMemcpyHostToDevice, R.stream));
    DJ_CUDA_CHECK(cudaMemcpyAsync((void*)v.scales, scales, (size_t)q.N * q.nb * 4, cudaMemcpyHostToDevice, R.stream));
    DJ_CUDA_CHECK(cudaStreamSynchronize(R.stream));
    DJ_CATCH
}

int deepj_cuda_q8_download(int32_t q8_id, int8_t* codes, float* scales) {
    DJ_TRY
    ensure_init();
    Ctx c; c.execute = false; c.s = R.stream;
    Buf& q = find_buf(c, q8_id, kQ8, "q8_download");
    Q8View v = q8view(q);
    DJ_CUDA_CHECK(cudaMemcpy2DAsync(codes, q.K, v.codes, q.Kp, q.K, q.N, cudaMemcpyDeviceToHost, R.stream));
    DJ_CUDA_CHECK(cudaMemcpyAsync(scales, v.scales, (size_t)q.N * q.nb * 4, cudaMemcpyDeviceToHost, R.stream));
    DJ_CUDA_CHECK(cudaStreamSynchronize(R.stream));
    DJ_CATCH
}

int deepj_cuda_synth_fill(int32_t id, uint64_t seed, uint64_t ordinal, float std_dev, int64_t first_index, int64_t n) {
    DJ_TRY
    ensure_init();
    Ctx c; c.execute = false; c.s = R.stream;
    if (n < 0) throw std::runtime_error("synth_fill: negative count");
    float* p = f32(c, id, (size_t)n, "synth_fill");
    launch_synth_fill(p, seed, ordinal, std_dev, first_index, n, R.stream);
    DJ_CATCH
}

static int kv_alloc_impl(int32_t id, int32_t layers, int32_t batch, int32_t heads, int32_t max_seq, int32_t head_dim, int half) {
    DJ_TRY
    ensure_init();
    if (layers <= 0 || batch <= 0 || heads <= 0 || max_seq <= 0 || head_dim <= 0) throw std::runtime_error("kv_alloc: dimensions must be positive");
    if (R.pool.count(id)) throw std::runtime_error("kv_alloc: id " + std::to_string(id) + " already exists");
    Buf b; b.kind = kKV; b.layers = layers; b.B = batch; b.H = heads; b.maxSeq = max_seq; b.hd = head_dim;
    size_t plane = (size_t)layers * batch * heads * max_seq * head_dim;
    b.kvHalf = half;
    if (half && head_dim % 16 != 0) throw std::runtime_error("kv_alloc: an fp16 cache needs a head dim that is a multiple of 16");
    b.bytes = plane * 2 * (half ? 2 : 4);
    DJ_CUDA_CHECK(cudaMalloc(&b.ptr, b.bytes));
    DJ_CUDA_CHECK(cudaMemsetAsync(b.ptr, 0, b.bytes, R.stream));
    b.serial = R.next_serial++;
    R.pool[id] = b;
    DJ_CATCH
}

int deepj_cuda_kv_alloc(int32_t id, int32_t layers, int32_t batch, int32_t heads, int32_t max_seq, int32_t head_dim) {
    return kv_alloc_impl(id, layers, batch, heads, max_seq, head_dim, 0);
}
int deepj_cuda_kv_alloc_f16(int32_t id, int32_t layers, int32_t batch, int32_t heads, int32_t max_seq, int32_t head_dim) {
    return kv_alloc_impl(id, layers, batch, heads, max_seq, head_dim, 1);
}

}  // extern "C"
