/*
 * deepj_cuda.h — C ABI of libdeepj_cuda_jni, a CUDA (sm_100a) GpuRuntime for
 * DeepJ's lazy ComputeGraph command stream.
 *
 * The first five entry points are one-to-one twins of the five `static native`
 * methods DeepJ binds for its Metal runtime; a JNI shim (or any other FFI) forwards
 * to them with plain pointers and lengths.  Everything returns 0 on success and a
 * non-zero status on failure; the message is available from deepj_cuda_last_error()
 * (the JNI shim turns it into java.lang.RuntimeException, as the Metal library does
 * in native/deepj_metal_jni.mm:888-893).
 *
 * Threading: one caller thread per process, like the reference runtime
 * (unsynchronised singletons, native/deepj_metal_jni.mm:63,1358).
 */
#ifndef DEEPJ_CUDA_H
#define DEEPJ_CUDA_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ───────────── the reference's five natives ───────────── */

/* Replaces MetalNative.nativeAllocBuffers (tensor/metal/MetalNative.java:41,
 * native/deepj_metal_jni.mm:1480-1507).  ids[i] gets sizes[i] floats; an id that
 * already exists is left untouched.  New buffers are zero-filled. */
int deepj_cuda_alloc_buffers(const int32_t* ids, const int32_t* sizes_in_floats, int32_t count);

/* Replaces MetalNative.nativeUploadBuffer (MetalNative.java:44,
 * native/deepj_metal_jni.mm:1509-1523).  Copies len floats from host memory;
 * unknown id → error "Buffer not found for upload". */
int deepj_cuda_upload_buffer(int32_t id, const float* data, int32_t len);

/* Replaces MetalNative.nativeDownloadBuffer (MetalNative.java:47,
 * native/deepj_metal_jni.mm:1525-1539).  Waits for all queued work, then copies
 * len floats to host memory. */
int deepj_cuda_download_buffer(int32_t id, float* out, int32_t len);

/* Replaces MetalNative.nativeReleaseBuffers (MetalNative.java:50,
 * native/deepj_metal_jni.mm:1541-1550).  Unknown ids are ignored. */
int deepj_cuda_release_buffers(const int32_t* ids, int32_t count);

/* Replaces MetalNative.nativeFlushOps (MetalNative.java:57,
 * native/deepj_metal_jni.mm:1554-2140).  Executes a ComputeGraph command stream
 * (op codes 1-42 of tensor/ComputeGraph.java:19-60 plus the fused decode op codes
 * listed below) and returns when the results are readable.  The whole stream is
 * validated before the first launch.  A stream seen for the second time is
 * captured as a CUDA graph and replayed from then on. */
int deepj_cuda_flush_ops(const int32_t* cmd, int32_t len);

/* Message of the last failed call on this thread (never NULL). */
const char* deepj_cuda_last_error(void);

/* ───────────── additions (no counterpart in the reference) ───────────── */

/* Bind the library to a CUDA device (default: device 0 at first use). */
int deepj_cuda_init(int32_t device);
/* Free every buffer, graph and workspace. */
int deepj_cuda_shutdown(void);

/* Same as deepj_cuda_flush_ops but returns after enqueueing. */
int deepj_cuda_flush_ops_async(const int32_t* cmd, int32_t len);
int deepj_cuda_synchronize(void);
/* Page-locked host memory for staging buffers that are uploaded / downloaded every step. */
int deepj_cuda_pinned_alloc(void** out, int64_t bytes);
int deepj_cuda_pinned_free(void* p);

/* Device-time measurement on the library's stream (CUDA events). */
int deepj_cuda_timer_begin(void);
int deepj_cuda_timer_end(float* elapsed_ms);

/* Run a stream op by op (no graph) and report the device time of every op, in
 * stream order; n_ops receives the number of ops. */
int deepj_cuda_profile_ops(const int32_t* cmd, int32_t len, float* ms_per_op, int32_t max_ops, int32_t* n_ops);

/* Phase tracing of the Q8 GEMV kernel.  With DEEPJ_CUDA_TRACE=1 in the environment at
 * the first call, graphs are off and every GEMV launch records six device timestamps
 * (ns): start, weights prefetch issued, previous kernel finished, activations staged,
 * first tile reduced, end.  Reads up to max_launches records of eight uint64 each. */
int deepj_cuda_trace_read(uint64_t* out, int32_t max_launches, int32_t* n_launches);

/* counters[0]=kernel launches issued eagerly, [1]=graph replays, [2]=graphs
 * captured, [3]=kernel nodes in the last replayed graph, [4]=workspace bytes,
 * [5]=device-side error flag of bounded waits (0 = none; 100 + rank: a tensor-parallel peer's data
 * never arrived; 201-207: a barrier of the tensor-core GEMM; 300-312: the whole-token kernel's grid barrier
 * or rings; 330 / 331: a bulk-copy item of the GEMV / several-row kernel never arrived). */
int deepj_cuda_stats(int64_t* counters, int32_t n);

/* Q8 weights.  Format (defined by this library; DeepJ has no quantization): for a
 * weight W[K×N] (row-major, K = reduction dimension), every output column n is cut
 * into blocks of 32 consecutive k (the last block is shorter when K % 32 != 0);
 * scale = max|w| / 127.0f, code = clamp(round-half-even(w / scale), -127, 127),
 * scale == 0 → code 0.  Canonical arrays: codes[N][K] int8, scales[N][ceil(K/32)]
 * float.  A Q8 object lives in the same id space as float buffers. */
int deepj_cuda_q8_alloc(int32_t q8_id, int32_t K, int32_t N);
/* Quantize columns [src_col0, src_col0+n_cols) and rows [src_row0, src_row0+K) of
 * the float buffer src_id (a row-major matrix with src_ld columns) into columns
 * [dst_col0, dst_col0+n_cols) of the Q8 object. */
int deepj_cuda_q8_quantize_into(int32_t q8_id, int32_t dst_col0, int32_t src_id,
                                int32_t src_row0, int32_t src_col0, int32_t src_ld, int32_t n_cols);
int deepj_cuda_q8_upload(int32_t q8_id, const int8_t* codes, const float* scales);
int deepj_cuda_q8_download(int32_t q8_id, int8_t* codes, float* scales);

/* Fill a float buffer with the library's counter-based synthetic weights (the same
 * integer-exact generator the CPU oracle restates): element i of the buffer gets
 * generator index first_index + i. */
int deepj_cuda_synth_fill(int32_t id, uint64_t seed, uint64_t ordinal, float std_dev,
                          int64_t first_index, int64_t n);

/* KV cache object: K and V planes of [layers][batch][heads][max_seq][head_dim]
 * floats, zero-filled. */
int deepj_cuda_kv_alloc(int32_t kv_id, int32_t layers, int32_t batch, int32_t heads,
                        int32_t max_seq, int32_t head_dim);
/* The same object with fp16 elements (half the bytes a token's attention reads).  Keys are rotated in fp32 and
 * rounded to nearest-even when appended, values are rounded when appended; scores, softmax and the weighted sum
 * stay fp32.  The reference keeps everything in fp32 (tensor/cpu/CpuBackend.java), so this is an option that has to
 * pass the same logit and token gates against the oracle; head_dim must be a multiple of 16.  Ops 67 and 73 and
 * deepj_cuda_attn_decode_static take either kind; decode plans (op 76) take the fp32 kind only. */
int deepj_cuda_kv_alloc_f16(int32_t kv_id, int32_t layers, int32_t batch, int32_t heads,
                            int32_t max_seq, int32_t head_dim);

/* Decode plan: everything one batch-1 token step of a Llama-shaped Q8 model touches, resolved once, for op 76
 * (DECODE_STEP), which runs the whole step — embedding row, every block, final norm, LM head, greedy pick, position
 * advance — as ONE persistent kernel.  No counterpart in the reference (its step is DecoderOnlyModel.forward over the
 * whole context, models/DecoderOnlyModel.java:58-64).  The plan lives in the same id space as the buffers and is
 * released with deepj_cuda_release_buffers; releasing anything it references makes later flushes of op 76 fail cleanly.
 * desc = [1 (version), n_layers, heads on this rank, head_dim (32 | 64 | 128), epsBits,
 *         tok, pos, emb, cos, sin, kv, x, x2, qkv, att, h, logits, next, gF, Wlm, blm,                 (buffer ids)
 *         then per block: g1, Wqkv, Wo, g2, Wgate, bgate, Wup, bup, Wdown, bdown]
 * Shapes are checked against the Q8 objects (every reduction length a multiple of 32).  With a tensor-parallel
 * connection in place (tp_connect before this call) the plan is made for this rank's shard: Wo and down are row shards
 * whose partial sums the kernel exchanges itself, `logits` holds this rank's vocabulary columns, and every rank ends up
 * with the same pick. */
int deepj_cuda_decode_plan(int32_t plan_id, const int32_t* desc, int32_t len);

/* Tensor parallelism, one process per GPU of one node.  No counterpart in the reference
 * (DeepJ is single-device).  Every rank calls tp_create (allocates its exchange buffer:
 * 2 x world slots of slot_floats values, 8 bytes each, returns a 64-byte CUDA IPC handle; one exchange
 * carries at most slot_floats values per rank: M x N of op 71, M x n_local of op 72 - batch x dModel for decode
 * steps, rows x dModel for prompt chunks),
 * the host exchanges the handles by any means (the Python runner uses torch.distributed),
 * then every rank calls tp_connect with all handles in rank order.  After that op codes 71
 * and 72 may appear in streams; every rank must flush the same sequence of them.  Waits
 * inside the exchange kernel are bounded; an expired wait sets stats counter [5] to
 * 100 + the rank whose data did not arrive, the kernel finishes and the context stays usable; while the counter
 * is non-zero every later wait gives up at once, and a synchronous flush whose stream held an exchange returns
 * non-zero with a message naming the rank.  tp_connect and tp_destroy drop the cached CUDA graphs (they hold peer
 * addresses).
 * tp_connect(NULL, world) maps every other rank to a private buffer that nobody fills: the
 * way to see the bounded wait expire (a peer that never shows up) without a second process.
 * deepj_cuda_clear_device_error() zeroes counter [5] again. */
int deepj_cuda_tp_create(int32_t rank, int32_t world, int64_t slot_floats, void* handle_out64);
/* Optional, before tp_create and with the same value on every rank: the message size (floats per rank) above
 * which an exchange takes the chunk-sized grid and its own slot region; 0 = the default of 2^15. */
int deepj_cuda_tp_configure(int64_t large_message_floats);
int deepj_cuda_tp_connect(const void* handles, int32_t world);
int deepj_cuda_tp_destroy(void);
int deepj_cuda_clear_device_error(void);

/* Precision of the many-row (tcgen05) Q8 projection, which multiplies fp16 halves x = x_hi + x_lo and
 * w = w_hi + w_lo: x_hi * w_hi is always issued; bit 0 of correction_terms adds x_lo * w_hi, bit 1 adds x_hi * w_lo.
 * 3 is the default (both operands at about 22 bits); fewer products are faster and coarser (11 bits in the dropped
 * operand).  Takes effect on the next flush; cached CUDA graphs are dropped.  No counterpart in the reference, whose
 * Q8 matmul is fp32 throughout (native/deepj_metal_jni.mm:828-889). */
int deepj_cuda_tc_configure(int32_t correction_terms);

/* Decode attention for callers that must not allocate.  No counterpart in the reference.
 *
 * Some hosts of this library cannot let a call reach cudaMalloc: a JVM thread inside a
 * latency-critical section, a serving loop that has handed all device memory to its own
 * arena, a process whose memory budget was fixed at start-up.  The stream form of this op
 * (code 67) takes its split-partial scratch from a workspace that the library grows on
 * demand, so its first use, or a larger shape, allocates.  This entry point runs the same
 * kernel with the scratch in a fixed 2 MiB + 16 KiB array inside the library image (held
 * by every GPU that loads the library until the process exits) and calls no allocating
 * routine.  Arguments are those of op 67: buffer ids of objects that already exist, float
 * offsets, strides and shapes; it returns when `out` is readable.
 * Limits: batch·heads·splits·(head_dim+2) <= 524288 floats and batch·heads <= 4096;
 * anything larger is rejected with a message naming both numbers.
 * The first call on a device resolves the array's device address (cudaGetSymbolAddress), and the
 * first call for a given head dimension may make the CUDA runtime load that kernel's code, which can
 * allocate inside the driver: make one warm-up call per head dimension at start-up, before any stream
 * capture begins and before the section that must not allocate.  The caller's current device is left
 * as it was found.  Every call shares the one
 * array: calls that overlap on the GPU race on it, so keep them on one thread, one after
 * the other (the call is synchronous, which does that for a single caller). */
int deepj_cuda_attn_decode_static(int32_t qkv, int32_t q_off, int32_t k_off, int32_t v_off, int32_t ld,
                                  int32_t kv, int32_t layer, int32_t pos, int32_t cos_table, int32_t sin_table,
                                  int32_t out, int32_t out_off, int32_t ldo, int32_t batch, int32_t heads, int32_t head_dim);

/* ───────────── fused decode op codes (extend ComputeGraph.java:19-60) ─────────────
 * Buffer-id slots may hold -1 where an operand is optional.  Integers that the
 * reference would keep in an int[] (token ids, positions) travel as floats holding
 * integers, like its index tensors (tensor/metal/MetalBackend.java:43-54).
 *
 *  64 EMBED_GATHER      [op, table, ids, out, rows, d, vocab]
 *  65 Q8_LINEAR         [op, x, x_off, ldx, gamma, epsBits, w, bias, residual, res_off, ldr, out, out_off, ldo, M]
 *                        out = (gamma>=0 ? rmsnorm(x) : x) · W (+bias) (+residual)
 *  66 Q8_SWIGLU         [op, x, x_off, ldx, gamma, epsBits, w_gate, b_gate, w_up, b_up, out, out_off, ldo, M]
 *                        out = silu(xn·Wg + bg) ⊙ (xn·Wu + bu)
 *  67 ATTN_DECODE       [op, qkv, q_off, k_off, v_off, ld, kv, layer, pos, cos, sin, out, out_off, ldo, B, H, hd]
 *                        RoPE(q,k) at pos[b]; append k,v; causal softmax attention over 0..pos[b]
 *  68 ARGMAX_ROWS       [op, in, out, rows, cols]      lowest index among equal maxima
 *  69 ADD_SCALAR_INPLACE[op, buf, valueBits, n]         buf[i] += value (advances positions)
 *  70 COPY              [op, src, src_off, dst, dst_off, n]
 *  71 TP_ALLREDUCE      [op, in, bias, residual, out, M, N]   out = residual + bias + sum over ranks of in (rank order)
 *  72 TP_ALLGATHER      [op, in, out, M, n_local]             out[m][r*n_local + j] = in of rank r
 *  73 ATTN_PREFILL      [op, qkv, q_off, k_off, v_off, ld, kv, layer, pos, cos, sin, out, out_off, ldo, B, H, hd, T]
 *                        a prompt chunk: row b*T + t is token pos[b] + t of sequence b; the chunk's k (rotated)
 *                        and v are appended first, then every row attends causally over 0..pos[b]+t
 *  74 SAMPLE_TOPK       [op, logits, r, out, rows, cols, topK, temperatureBits]
 *                        TextGenerator.sampleFromLogits per row (stable descending order, first topK — 0 = the whole
 *                        row, models/TextGenerator.java:111-115 — float softmax of logit/T, first index whose running
 *                        sum reaches r[row]); r = Random.nextFloat().  Up to 1024 candidates are selected and sorted in
 *                        shared memory; more sort the whole row in the workspace
 *  76 DECODE_STEP       [op, plan, feed_back]   one whole batch-1 token step of the plan's model as one kernel:
 *                        next = greedy pick of the logits at pos, pos += 1, and tok = next when feed_back = 1
 *  75 Q8_LINEAR_LN      [op, x, x_off, ldx, gamma, beta, epsBits, w, bias, residual, res_off, ldr, out, out_off, ldo, M, act]
 *                        the GPT blocks' projection: out = act(layernorm(x; gamma, beta, eps) · W + bias) (+residual),
 *                        LayerNorm1D semantics (mean, biased variance); act 0 = none, 1 = GELU (tanh form);
 *                        gamma = beta = -1 skips the norm
 */
#define DEEPJ_OP_EMBED_GATHER        64
#define DEEPJ_OP_Q8_LINEAR           65
#define DEEPJ_OP_Q8_SWIGLU           66
#define DEEPJ_OP_ATTN_DECODE         67
#define DEEPJ_OP_ARGMAX_ROWS         68
#define DEEPJ_OP_ADD_SCALAR_INPLACE  69
#define DEEPJ_OP_COPY                70
#define DEEPJ_OP_TP_ALLREDUCE        71
#define DEEPJ_OP_TP_ALLGATHER        72
#define DEEPJ_OP_ATTN_PREFILL        73
#define DEEPJ_OP_SAMPLE_TOPK         74
#define DEEPJ_OP_Q8_LINEAR_LN       75
#define DEEPJ_OP_DECODE_STEP        76

#ifdef __cplusplus
}
#endif
#endif /* DEEPJ_CUDA_H */
