/*
 * rq.h -- C ABI of the B200 (sm_100a) GGUF quantised matrix-vector library.
 *
 * This is the boundary a recipe host binds in place of the LLVM-IR GPU lowering of its
 * quantised contraction nodes. Plain pointers and sizes only; every entry point returns
 * 0 on success or a negative rq_status, and rq_last_error() gives thread-local text.
 * The library owns prepared weights and its context; the caller owns every other buffer.
 *
 * Streams. The device-pointer entry points enqueue on the caller's stream and return without
 * synchronising. A context keeps work areas (the int8 activation records, the batched product's
 * activation image, an expert bank's plans) that successive calls reuse: calls on ONE stream are
 * ordered by the stream; when a call arrives on a different stream than the previous call on the
 * context, the library makes the new stream wait for the work enqueued on the previous one (an
 * event), so the two never overlap on the work areas. Inside a stream capture no such event is
 * recorded: calls captured into one graph must share one stream. A stream handed to a call must
 * stay alive until the next call on the context. One host thread at a time per context.
 * No entry point aborts on bad arguments, none falls back to the CPU.
 *
 * Each declaration names the reference interface (nm-z/recipe-dev, file:line) it replaces.
 */
#ifndef RQ_H
#define RQ_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct rq_ctx rq_ctx;       /* one per device; replaces the per-device Gpu + arenas, recipe.rs:28014, :24795-24801 */
typedef struct rq_weight rq_weight; /* a stored weight resident in HBM; replaces StoredWeight in the device arena, recipe.rs:16032-16045, :2107-2126 */

enum rq_status {
    RQ_OK = 0,
    RQ_ERR_INVALID = -1,     /* null pointer, bad shape, K not a multiple of the block, bad enum */
    RQ_ERR_CUDA = -2,        /* a CUDA runtime call failed; text names it */
    RQ_ERR_ALLOC = -3,       /* device or host allocation failed */
    RQ_ERR_UNSUPPORTED = -4, /* valid request this build does not serve */
    RQ_ERR_LIMIT = -5,       /* size beyond a documented fixed maximum */
    RQ_ERR_WAIT = -6         /* rq_check: a kernel gave up one of its bounded waits; text names which */
};

/* GGML tensor types on this path (recipe.rs:9925-9962). */
enum { RQ_Q4_0 = 2, RQ_Q8_0 = 8, RQ_Q4_K = 12, RQ_Q6_K = 14,
       /* The other stored formats the same bodies serve (recipe.rs:15812-15824; the IQ1 / IQ2 / IQ3 grid formats are not among them): bound, decoded bit-exactly (rq_dequant,
        * rq_gather_rows), dotted with fp32 activations (RQ_ACT_FLOAT: the run decoders, recipe.rs:7826-7917) and re-encoded
        * to Q8_0 by rq_weight_requantize, which is what `.int(8)` does to them at load (recipe.rs:22345-22369). They have
        * no int8 dot here (Q4_1 excepted: it is the storage of int4 sums and RQ_ACT_INT8 over it is what `.int(4)` runs), so
        * RQ_ACT_INT8 on the others returns RQ_ERR_UNSUPPORTED and names the re-encode; rq_quantize (no encoder) and expert
        * banks do not take them. */
       RQ_Q4_1 = 3, RQ_Q5_0 = 6, RQ_Q5_1 = 7, RQ_Q5_K = 13, RQ_IQ4_NL = 20,
       RQ_Q8_1 = 9, RQ_Q2_K = 10, RQ_Q3_K = 11, RQ_Q8_K = 15, RQ_IQ4_XS = 23 };

/* Activation handling, what `.fp(32)` / `.int(8)` select (recipe.rs:14027-14054, :22326-22369):
 * FLOAT keeps the activations as they are (run decoders, recipe.rs:7826-7917);
 * INT8 rounds them to int8 records with one fp32 step per `step` inputs (amd-nv-cpu.ll:1381-1517). */
enum { RQ_ACT_FLOAT = 0, RQ_ACT_INT8 = 1,
       /* INT8 where the caller states that x is the same column, token count and step as the previous
        * RQ_ACT_INT8 call on this context (q/k/v, or gate/up, read one activation): the library may
        * reuse the records it derived then instead of deriving them again. The results are the same
        * bits either way. Fails if the previous INT8 call was of another width, token count or step. */
       RQ_ACT_INT8_CACHED = 2 };

/* Routing (Scoring, recipe.rs:13955). */
enum { RQ_SCORE_SOFTMAX = 0, RQ_SCORE_SIGMOID = 1 };

/* ---- context ------------------------------------------------------------------- */

/* Binds a context to CUDA device `device`. Replaces native_prepare / module load for this
 * path (recipe.rs:28155, :27843). */
int rq_init(int device, rq_ctx** out);
void rq_destroy(rq_ctx* ctx);
/* Synchronises the device and reports whether any kernel of this context gave up one of its
 * bounded waits since the last check (the device code never traps and never spins unbounded;
 * the reference's hand PTX waits return a status the same way, barrier.ptx:1653-1748). */
int rq_check(rq_ctx* ctx);
/* How long a kernel of this context waits on a barrier (a copy that has not landed, a ring slot, a peer's
 * flag) before it records a code, stops waiting and returns: 2 s unless set. 1 us .. 60 s. */
int rq_set_wait_limit(rq_ctx* ctx, uint64_t nanoseconds);
/* Runs the give-up path on purpose: one warp waits, with the context's limit (which must have been set to
 * 100 ms or less), on a barrier nothing arrives on, gives up and returns; the next rq_check reports
 * RQ_ERR_WAIT. No fault, no trap, no endless loop: the kernel ends by itself after the limit. */
int rq_wait_selftest(rq_ctx* ctx, void* stream);
/* Sizes the context's work areas ahead of time for weights of up to max_rows x max_cols and calls of up
 * to max_tokens tokens. Growing a work area frees and allocates device memory, which synchronises the
 * device: a call wider than anything seen or reserved so far does that on demand, inside the call, and
 * cannot do it while its stream is being captured. After rq_reserve no matvec / matmul call within the
 * reserved sizes allocates, frees or synchronises. (The reference sizes its arenas once, at place():
 * recipe.rs:24795-24801.) */
int rq_reserve(rq_ctx* ctx, int64_t max_rows, int64_t max_cols, int max_tokens);
/* Thread-local text of the last failure on the calling thread (RecipeError, recipe.rs:13416-13433). */
const char* rq_last_error(void);
/* Block geometry of a type: values per block and bytes per block (QUANTIZATIONS, recipe.rs:15811-15822). 0 if unknown. */
int rq_block_values(int ggml_type);
int rq_block_bytes(int ggml_type);

/* ---- weights -------------------------------------------------------------------- */

/* Uploads rows [row_first, row_first + row_count) of a host tensor of GGUF blocks
 * ([rows][cols / block] blocks, rows contiguous) and lays them out for the kernels.
 * Replaces range_tape's weight upload + recipe_model_load (recipe.rs:22200, :8128-8165);
 * the row range is a die's share of a row split (lone_split, recipe.rs:21010-21020). */
int rq_weight_prepare(rq_ctx* ctx, int ggml_type, const void* host_blocks, int64_t rows, int64_t cols,
                      int64_t row_first, int64_t row_count, rq_weight** out);
/* Same, from blocks already in device memory (e.g. written by rq_quantize): all `rows`. */
int rq_weight_prepare_device(rq_ctx* ctx, int ggml_type, const void* dev_blocks, int64_t rows, int64_t cols,
                             rq_weight** out, void* stream);
/* Writes the weight back as GGUF blocks into host memory (round-trip check of the layout). */
int rq_weight_export(rq_ctx* ctx, const rq_weight* w, void* host_blocks);
/* The load-time re-encode of a bound tensor: decodes `src` with its own decoder and encodes it as
 * `target_type` (RQ_Q8_0 or RQ_Q4_1) with the load kernel's encoder, byte-exact with what the reference's
 * recipe_model_load writes (requantize_bound recipe.rs:22373-22431, emit_requantize :8016-8127).
 * This is what `.int(8)` (target Q8_0) and `.int(4)` (target Q4_1) do to a tensor bound in a format
 * they do not keep. `src` stays valid. */
int rq_weight_requantize(rq_ctx* ctx, const rq_weight* src, int target_type, rq_weight** out, void* stream);
/* 1 when `.int(8)` dots a lone tensor of this type as stored (Q8_0, Q4_K), 0 when the reference
 * re-encodes it to Q8_0 at load first (Q6_K, Q4_0): finish_int_sums, recipe.rs:22345-22369. */
int rq_int8_keeps(int ggml_type);
/* The same question for `.int(4)`, whose storage is Q4_1 (recipe.rs:22348): 1 for Q4_1, 0 for everything else -- re-encode
 * with rq_weight_requantize(ctx, w, RQ_Q4_1, ..) (the load kernel's Q4_1 encoder, recipe.rs:8088-8094) and run RQ_ACT_INT8
 * over the result: int8 activation records against the four-bit codes, q8_d * (d * dot + m * sum) per 16-value slice
 * (block32 slice kind 3, build.rs:777-796). */
int rq_int4_keeps(int ggml_type);
void rq_weight_free(rq_ctx* ctx, rq_weight* w);
int64_t rq_weight_rows(const rq_weight* w);
int64_t rq_weight_cols(const rq_weight* w);
int rq_weight_type(const rq_weight* w);
/* Bytes the weight occupies in HBM (equal to its GGUF size). */
int64_t rq_weight_bytes(const rq_weight* w);

/* Dequantises every value to fp32, bit-exact with the reference unpacking
 * (dequant_scalar / dequant_q45k / dequant_q6k, recipe.rs:3687-3833). dev_out: rows*cols floats. */
int rq_dequant(rq_ctx* ctx, const rq_weight* w, float* dev_out, void* stream);

/* Embedding-row gather from a packed table: y[k * y_k_stride + t * y_t_stride] = value k of row dev_ids[t] of `table`,
 * decoded with rq_dequant's arithmetic (the same bits). dev_ids: `tokens` int32 in device memory; an id outside the table
 * is clamped into it. Replaces Primitive::Gather over a stored table (recipe.rs:4632-4651). */
int rq_gather_rows(rq_ctx* ctx, const rq_weight* table, const int32_t* dev_ids, int tokens, float* y, int64_t y_k_stride, int64_t y_t_stride, void* stream);

/* Quantises `count` fp32 device values into GGUF blocks in device memory, byte-exact with
 * Integer::compress (recipe.rs:16191-16242 Q8_0/Q4_0, :16325-16375 Q4_K, :16376-16414 Q6_K).
 * count must be a whole number of blocks. */
int rq_quantize(rq_ctx* ctx, int ggml_type, const float* dev_values, int64_t count, void* dev_blocks, void* stream);

/* ---- matvec ---------------------------------------------------------------------- */

/* y[n*y_n_stride + t*y_t_stride] = sum_k W[n][k] * x[k*x_k_stride + t*x_t_stride], t < tokens.
 * Device pointers. Replaces contraction_forward_body for blocked weights
 * (amd-nv-cpu.ll:2242-2300 -> :1231-2241) and packed_rows_body mode 0 (amd-nv-cpu.ll:3136-3508).
 * The reference's channel-major planes are x_k_stride = tokens, x_t_stride = 1.
 * act_mode RQ_ACT_INT8 takes step 32 or 256 (recipe.model.int.step); FLOAT ignores step.
 * RQ_ACT_INT8 dots the blocks of `w` as they are stored. The reference does that for Q8_0 and Q4_K
 * only; a lone Q6_K or Q4_0 tensor under `.int(8)` is first re-encoded to Q8_0 (rq_int8_keeps,
 * rq_weight_requantize): pass the re-encoded weight to reproduce recipe's `.int(8)`, the stored one
 * for the direct dot over the file's own blocks (fewer bytes, a different rounding of the weights).
 * Enqueues on `stream` (a cudaStream_t, may be NULL) and returns without synchronising. */
int rq_matvec(rq_ctx* ctx, const rq_weight* w, const float* x, int64_t x_k_stride, int64_t x_t_stride, int tokens,
              float* y, int64_t y_n_stride, int64_t y_t_stride, int act_mode, int step, void* stream);

/* n matrices of one format and width against the SAME activations (q/k/v, gate/up): the column
 * is quantised once and, where the shape allows, one launch walks all n row sets. ys[i] receives
 * matrix i's rows with the strides of rq_matvec. The reference runs such sibling nodes inside
 * one persistent kernel (recipe_model_forward, recipe.rs:8235-8276); this is that grouping. */
int rq_matvec_multi(rq_ctx* ctx, int n, const rq_weight* const* ws, const float* x, int64_t x_k_stride, int64_t x_t_stride, int tokens,
                    float* const* ys, int64_t y_n_stride, int64_t y_t_stride, int act_mode, int step, void* stream);

/* The dense gated feed-forward's first half in one launch: y[n] = silu(gate[n] . x) * (up[n] . x), both matrices streamed
 * as one virtual row set, the activation and the product applied as the launch's epilogue (lower_gated,
 * recipe.rs:23279-23286; silu with recipe's portable transcendentals). gate and up: one format, one shape, rows of whole
 * 256-value units. Arguments as rq_matvec. */
int rq_matvec_glu(rq_ctx* ctx, const rq_weight* gate, const rq_weight* up, const float* x, int64_t x_k_stride, int64_t x_t_stride, int tokens, float* y,
                  int64_t y_n_stride, int64_t y_t_stride, int act_mode, int step, void* stream);

/* The steps either side of a projection in a decode layer, device pointers, enqueued on `stream`:
 * RMS normalisation of `tokens` positions of n values, y = (x / sqrt(mean(x^2) + epsilon)) * gain (gain may be null),
 *   emit_normalize_stats in Rms mode, recipe.rs:6836-7120;
 * the residual add y = a + b over n values;
 * the logit soft-cap y = cap * tanh(x / cap) with recipe's portable tanh (scale, tanh, scale: rnj-1.rs:47-51). */
int rq_rmsnorm(rq_ctx* ctx, const float* x, int64_t x_k_stride, int64_t x_t_stride, int64_t n, int tokens, const float* gain, float epsilon, float* y,
               int64_t y_k_stride, int64_t y_t_stride, void* stream);
int rq_add(rq_ctx* ctx, const float* a, const float* b, int64_t n, float* y, void* stream);
int rq_softcap(rq_ctx* ctx, const float* x, int64_t n, double cap, float* y, void* stream);

/* The batched product (prefill, multi-sequence decode): the same contraction as rq_matvec for many
 * tokens, on the tensor cores (tcgen05.mma, fp32 accumulation in tensor memory) where a kernel serves
 * the case. Q4_K / Q6_K weights: exact-integer weight operands, activations as fp16 hi + lo pairs,
 * for RQ_ACT_FLOAT and for RQ_ACT_INT8 windows of twelve and more positions (the int8 answer is the
 * product over the records' code * step). Q8_0 / Q4_0 with RQ_ACT_FLOAT: weights dequantised a tile at
 * a time, both operands as hi + lo pairs. Everything else (shorter int8 windows, int8 over the 32-value
 * formats, the decode-only formats) runs the matvec kernels. Replaces contraction_forward_body's
 * position loop and contraction_forward_gemm_body (amd-nv-cpu.ll:1231-2241, :3509-3649). Same
 * arguments as rq_matvec.
 * Range on the tensor-core routes: operands pass through fp16, so an activation of magnitude above
 * 65504 overflows (the result row is inf / NaN) and one below 6e-8 counts as zero; on the Q8_0 / Q4_0
 * route a dequantised weight of magnitude 256 or more overflows as well. rq_matvec has no such limit. */
int rq_matmul(rq_ctx* ctx, const rq_weight* w, const float* x, int64_t x_k_stride, int64_t x_t_stride, int tokens,
              float* y, int64_t y_n_stride, int64_t y_t_stride, int act_mode, int step, void* stream);

/* The same call with HOST buffers: copies x in, runs, copies y out, synchronises. This is the
 * call a host without device buffers makes (Placed::infer, recipe.rs:21314-21490). */
int rq_matvec_host(rq_ctx* ctx, const rq_weight* w, const float* host_x, int64_t x_k_stride, int64_t x_t_stride, int tokens,
                   float* host_y, int64_t y_n_stride, int64_t y_t_stride, int act_mode, int step);

/* rq_matvec_multi with HOST buffers: x goes in once, the n matrices run as one launch, the outputs come
 * back in one copy, one synchronisation. What a host without device buffers calls for sibling
 * projections (q/k/v, gate/up; Placed::infer, recipe.rs:21314-21490). */
int rq_matvec_multi_host(rq_ctx* ctx, int n, const rq_weight* const* ws, const float* host_x, int64_t x_k_stride, int64_t x_t_stride,
                         int tokens, float* const* host_ys, int64_t y_n_stride, int64_t y_t_stride, int act_mode, int step);

/* The INT8 product of one contiguous column (x[cols] -> y[rows]) for callers that cannot allocate.
 * No counterpart in the reference: there the host owns every arena and kernels never allocate, so
 * the question does not arise; here rq_matvec grows a scratch buffer with cudaMalloc on demand.
 * After one warm-up call per device (which looks up the array's address and lets the runtime load
 * the kernels), no call of this entry point allocates, frees or synchronises. Its activation scratch
 * is a fixed array in the library's device image, held by every GPU that loads the library until
 * the process exits; the context's own scratch is not touched.
 * Who needs it: a host that has given all device memory to its own pre-planned arenas, and a decode
 * loop that must never stall on the device-wide synchronisation an allocation or free brings.
 *  - at most RQ_STATIC_MAX_COLS inputs per row; wider weights are refused with RQ_ERR_LIMIT;
 *  - the first call on a device looks up the array's device address; make that first call before
 *    any stream capture begins;
 *  - all calls on a device share the array: calls that overlap on the GPU race (one stream is safe);
 *    nothing in it needs clearing between calls, every byte that is read is written first.
 * Same results as rq_matvec(..., RQ_ACT_INT8, step, ...) with tokens = 1 and unit strides. */
#define RQ_STATIC_MAX_COLS 32768
int rq_matvec_int8_static(rq_ctx* ctx, const rq_weight* w, const float* x, float* y, int step, void* stream);

/* Writes the int8 activation records the INT8 path derives from x (36 bytes per 32 inputs:
 * fp32 step, 32 codes; build.rs:332-337) for `tokens` columns into dev_records
 * ([tokens][cols/32][36]). Exposes amd-nv-cpu.ll:1381-1517 for bit-exact checks. */
int rq_quantize_activations(rq_ctx* ctx, const float* x, int64_t x_k_stride, int64_t x_t_stride, int64_t cols, int tokens,
                            int step, void* dev_records, void* stream);

/* ---- gguf_moe: routing and expert banks ------------------------------------------------ */

typedef struct rq_moe rq_moe; /* the expert tables of one gguf_moe block resident in HBM (MoeTensors / SharedTensors, recipe.rs:14382-14420) */

/* Routing weights of `tokens` positions from their router scores: softmax or sigmoid scoring, the
 * top_k experts by score (ties to the lower index; with a selection bias, by probability + bias),
 * renormalised over the kept experts or not. Writes the dense plane the expert bodies read:
 * weights[e * weight_e_stride + t * weight_t_stride], zero for experts not taken.
 * Replaces topk_forward_body (amd-nv-cpu.ll:4666-4716), same bits (its exp is build.rs:1079-1120). */
int rq_moe_route(rq_ctx* ctx, const float* scores, int64_t score_e_stride, int64_t score_t_stride, int experts, int top_k, int scoring,
                 int renormalize, const float* selection_bias, int tokens, float* weights, int64_t weight_e_stride, int64_t weight_t_stride,
                 void* stream);

/* Uploads experts [expert_first, expert_first + expert_count) of the three expert tables (host GGUF
 * blocks: gate and up are [experts][ffn][hidden], down is [experts][hidden][ffn]) and, optionally, a
 * gated shared expert (one expert of the same shape and its [hidden] fp32 gate vector; all four
 * null for none). The expert range is this GPU's share of an expert-parallel split; the reference
 * instead slices every expert's rows across dies (recipe.rs:4764-4766, :21015-21016). */
int rq_moe_prepare(rq_ctx* ctx, int ggml_type, const void* gate, const void* up, const void* down, int experts, int expert_first,
                   int expert_count, int hidden, int ffn, const void* shared_gate, const void* shared_up, const void* shared_down,
                   const float* shared_gate_vector, rq_moe** out);
/* The block's routed scale: the routing weights are multiplied by it before the experts add up (gguf_moe's `scale`,
 * lower_scale after the top-k, recipe.rs:23426-23428). 1 unless set. */
int rq_moe_set_routed_scale(rq_moe* moe, float scale);
/* Attaches the block's shared expert to a bank made without one (SharedExpert, recipe.rs:13855-13862, :23430-23457):
 * `count` merged experts, so its banks are gate / up [count * ffn][hidden] and down [hidden][count * ffn], host GGUF blocks
 * of the bank's format; gated != 0: weight sigmoid(gate_vector . x) (Gated), else weight one at every position (Ungated,
 * gate_vector ignored). top_k + count may not exceed 16. */
int rq_moe_attach_shared(rq_ctx* ctx, rq_moe* moe, int gated, int count, const void* shared_gate, const void* shared_up, const void* shared_down,
                         const float* shared_gate_vector);
void rq_moe_free(rq_ctx* ctx, rq_moe* moe);
int64_t rq_moe_bytes(const rq_moe* moe);

/* y[n * y_n_stride + t * y_t_stride] = sum over the experts of this bank that token t routes to of
 * w_e * down_e( silu(gate_e x) * up_e x ), plus (include_shared != 0) the shared expert at weight
 * sigmoid(gate_vector . x). Activations stay fp32 (expert tables are never int sums in the
 * reference, recipe.rs:24284-24294). Tokens nothing here is routed to get zeros, so the outputs of
 * the ranks of an expert-parallel split add up to the block's output.
 * Replaces lower_experts over the packed bodies, modes 1 and 2 (recipe.rs:23386-23459,
 * amd-nv-cpu.ll:2304-2365, :3136-3508). At most 64 tokens per call; top_k plus the shared expert's count at most 16.
 * A bank's plans and hidden activations are work areas shared by every call on it: calls on one stream are ordered, a call
 * on another stream waits for the previous one (see "Streams" at the top). */
int rq_moe_forward(rq_ctx* ctx, rq_moe* moe, const float* x, int64_t x_k_stride, int64_t x_t_stride, const float* routing,
                   int64_t routing_e_stride, int64_t routing_t_stride, int top_k, int tokens, int include_shared, float* y,
                   int64_t y_n_stride, int64_t y_t_stride, void* stream);
/* rq_moe_route followed by rq_moe_forward over the same tokens, as one call: the block's router -> TopK -> experts chain
 * (lower_gguf_moe, recipe.rs:23415-23459) with one launch less, the CTA that routes a token also writing its plan. `weights`
 * receives the dense routing plane exactly as rq_moe_route writes it (the bank's whole expert count gives its height); the
 * remaining arguments are those of the two calls. */
int rq_moe_route_forward(rq_ctx* ctx, rq_moe* moe, const float* scores, int64_t score_e_stride, int64_t score_t_stride, int top_k, int scoring,
                         int renormalize, const float* selection_bias, float* weights, int64_t weight_e_stride, int64_t weight_t_stride, const float* x,
                         int64_t x_k_stride, int64_t x_t_stride, int tokens, int include_shared, float* y, int64_t y_n_stride, int64_t y_t_stride,
                         void* stream);

/* ---- recorded sequences: one boundary crossing per step ------------------------------------------ */

/* The reference crosses its host / device boundary once per step: recipe_model_step is one launch that
 * walks every node of the step, with the planes between nodes resident on the device
 * (recipe.rs:8262-8276). The same here: between rq_sequence_begin and rq_sequence_end the
 * device-pointer entry points (rq_matvec, rq_matvec_multi, rq_matmul, rq_moe_route, rq_moe_forward, ...)
 * called with the stream that rq_sequence_begin returns are recorded instead of run; rq_sequence_run
 * replays the whole list as one submission, rq_sequence_run_host adds one copy in (host_in -> dev_in),
 * one copy out (dev_out -> host_out) and one synchronisation. The planes between the calls are device
 * buffers of the caller (rq_device_alloc for a host that has no allocator of its own).
 * A recording cannot allocate: call rq_reserve for the widest recorded call first. Pointers, shapes
 * and modes are fixed at recording time; the data in the planes is not. */
typedef struct rq_sequence rq_sequence;
int rq_device_alloc(rq_ctx* ctx, int64_t bytes, void** out);
void rq_device_free(rq_ctx* ctx, void* ptr);
int rq_sequence_begin(rq_ctx* ctx, void** stream_out);
int rq_sequence_end(rq_ctx* ctx, rq_sequence** out);
int rq_sequence_run(rq_sequence* seq, void* stream);
int rq_sequence_run_host(rq_sequence* seq, const float* host_in, float* dev_in, int64_t in_floats, const float* dev_out, float* host_out, int64_t out_floats);
void rq_sequence_free(rq_sequence* seq);

/* ---- GGUF files: reader and tensor binding --------------------------------------------------- */

/* A GGUF v3 file (or the complete split model its first shard names), mapped read-only. Replaces
 * Gguf::open and the descriptors it yields (recipe.rs:9786-10326): little-endian header, metadata of
 * the thirteen value kinds, tensor descriptors, data section at general.alignment (default 32), every
 * tensor checked to lie inside its file. Needs no GPU. */
typedef struct rq_gguf rq_gguf;
int rq_gguf_open(const char* path, rq_gguf** out);
void rq_gguf_close(rq_gguf* gguf);
/* Tensor descriptors in file order (GgufTensor, recipe.rs:9846-9853): name, GGML type id, shape
 * (dims[0] = the row length k, as GGUF stores it), bytes, and the bytes themselves in the mapping. */
int rq_gguf_tensor_count(const rq_gguf* gguf);
int rq_gguf_find(const rq_gguf* gguf, const char* name); /* index, or -1 */
const char* rq_gguf_tensor_name(const rq_gguf* gguf, int index);
int rq_gguf_tensor_type(const rq_gguf* gguf, int index);
int rq_gguf_tensor_dims(const rq_gguf* gguf, int index, int64_t* shape, int capacity); /* returns the number of dimensions */
int64_t rq_gguf_tensor_bytes(const rq_gguf* gguf, int index);
const void* rq_gguf_tensor_data(const rq_gguf* gguf, int index);
/* First-shard metadata (Gguf::value / integer_at / float_at, recipe.rs:10127-10160). kind: the GGUF value
 * kind 0..12, -1 when absent. Integers of any width (and bools) come back as u64, floats as f64. */
int rq_gguf_meta_count(const rq_gguf* gguf);
const char* rq_gguf_meta_key(const rq_gguf* gguf, int index);
int rq_gguf_meta_kind(const rq_gguf* gguf, const char* key);
int rq_gguf_meta_integer(const rq_gguf* gguf, const char* key, uint64_t* out);
int rq_gguf_meta_float(const rq_gguf* gguf, const char* key, double* out);
const char* rq_gguf_meta_text(const rq_gguf* gguf, const char* key);
int64_t rq_gguf_meta_array_length(const rq_gguf* gguf, const char* key);
const char* rq_gguf_meta_array_text(const rq_gguf* gguf, const char* key, int64_t index);
/* Binds rows [row_first, row_first + row_count) of a stored [k, n] (or [k, n, experts]: every expert's rows,
 * one after another) tensor as a resident weight; row_count <= 0 binds every row. Replaces Gguf::stored +
 * the tape's weight upload (recipe.rs:10196-10203, :22200) and GgufTensor::rows (:9873-9880). */
int rq_gguf_bind(rq_ctx* ctx, const rq_gguf* gguf, const char* name, int64_t row_first, int64_t row_count, rq_weight** out);
/* Binds experts [expert_first, expert_first + expert_count) of a gguf_moe block from its three [k, n, experts]
 * tensors (GgufTensor::expert, recipe.rs:9862-9869; MoeTensors, :14382-14420) and, when named, a gated shared
 * expert (three [k, n] tensors of the bank's format and an F32 gate vector). expert_count <= 0: every expert. */
int rq_gguf_bind_experts(rq_ctx* ctx, const rq_gguf* gguf, const char* gate, const char* up, const char* down, int expert_first, int expert_count,
                         const char* shared_gate, const char* shared_up, const char* shared_down, const char* shared_gate_vector, rq_moe** out);

/* ---- the exchange of the sharded configs ---------------------------------------------------- */

/* The exchange through the host's own NCCL communicator (`nccl_comm` is its ncclComm_t): the ranks'
 * slices of a row-split plane are gathered rank after rank (gathered: [nranks][count_per_rank]), or
 * the ranks' planes are summed. Device pointers; enqueued on `stream`. Replaces Primitive::Exchange
 * after a row split (gather, recipe.rs:5386-5394) and after a term split (die-order sum,
 * recipe.rs:5395-5441; buffers :20412-20486). libnccl.so.2 is looked up at run time: RQ_ERR_UNSUPPORTED
 * when the process has none. */
int rq_allgather_rows(rq_ctx* ctx, void* nccl_comm, const float* local, float* gathered, int64_t count_per_rank, void* stream);
int rq_allreduce_sum(rq_ctx* ctx, void* nccl_comm, const float* local, float* summed, int64_t count, void* stream);
/* For a host without a communicator of its own: rank 0 makes an id (128 bytes, ncclUniqueId), hands it to
 * the other ranks by whatever channel it has, and every rank creates its communicator from it. */
int rq_nccl_unique_id(void* id128);
int rq_nccl_comm_create(rq_ctx* ctx, const void* id128, int nranks, int rank, void** nccl_comm_out);
void rq_nccl_comm_destroy(void* nccl_comm);

/* The library's own exchange over NVLink peer memory: no collective library on the path, one kernel
 * per exchange. Every rank owns a buffer of per-rank slots which its peers map; the kernel stores this
 * rank's slice into its slot on every rank (plain peer stores), raises a flag on each peer, waits for
 * the peers' flags (bounded: a peer that never arrives makes rq_check report RQ_ERR_WAIT) and then
 * writes the result: the slots one after another (gather), or their sum in rank order (reduce: the same
 * bits on every rank and every run, as the reference's die-order sum, recipe.rs:5395-5441).
 * Set-up, once: every rank creates its exchange (slot_bytes = the largest slice it will ever send),
 * exports a 64-byte handle (a CUDA IPC handle) to every other rank, and connects with all ranks' handles
 * in rank order ([nranks][64]; its own entry is ignored). Ranks that share one process pass their
 * buffers (rq_exchange_buffer) as `same_process_buffers` instead and `handles` null.
 * Every rank must make the same sequence of gather / reduce calls with the same counts. Calls may be
 * captured into a CUDA graph and replayed. At most 16 ranks. */
typedef struct rq_exchange rq_exchange;
int rq_exchange_create(rq_ctx* ctx, int rank, int nranks, int64_t slot_bytes, rq_exchange** out);
int rq_exchange_handle(rq_exchange* ex, void* handle64);
void* rq_exchange_buffer(rq_exchange* ex);
int rq_exchange_connect(rq_exchange* ex, const void* handles, const void* const* same_process_buffers);
int rq_exchange_gather(rq_exchange* ex, const float* local, int64_t count, float* gathered, void* stream);
int rq_exchange_reduce(rq_exchange* ex, const float* local, int64_t count, float* summed, void* stream);
void rq_exchange_free(rq_exchange* ex);

#ifdef __cplusplus
}
#endif
#endif
