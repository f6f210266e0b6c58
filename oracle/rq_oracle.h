/*
 * CPU oracle for the GGUF quantised matrix-vector path -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the reference's (nm-z/recipe-dev) algorithm for this path:
 * block formats, per-value dequantisation, the weight quantisers, the int8 activation
 * quantiser, the three dot-product semantics, top-k routing and the MoE block. Each
 * function cites the reference file:line it follows (recipe.rs, amd-nv-cpu.ll, build.rs).
 *
 * The product library never links, loads or calls this file: only the test suite, the
 * smoke check and the benchmark's CPU-baseline leg do, and only as the checker.
 *
 * Pinning: the reference's own tests hold two vectors for this path -- the Q8_0 table of
 * .github/runtime/suite.rs:191-194 and the Q4_K x Q8_1 scalar check of
 * evidence/2026-10-10-m60-p2p/bench.rs:177-228 -- and both are reproduced in the test
 * suite. Q6_K, Q4_0, the quantisers, top-k and the int8 activation codes have no vector
 * in the reference: for those, PARITY IS UNPINNED by the reference and rests on this
 * restatement plus an independent NumPy restatement of the unpacking.
 */
#ifndef RQ_ORACLE_H
#define RQ_ORACLE_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* GGML type ids, recipe.rs:9925-9962 */
#define RQO_Q4_0 2
#define RQO_Q8_0 8
#define RQO_Q4_K 12
#define RQO_Q6_K 14
/* stored formats the same bodies serve beside the four above (recipe.rs:15812-15821, IQ4_NL :15823):
 * decoded per value, dotted by the run decoders, re-encoded to Q8_0 under `.int(8)` */
#define RQO_Q4_1 3
#define RQO_Q5_0 6
#define RQO_Q5_1 7
#define RQO_Q5_K 13
#define RQO_IQ4_NL 20
#define RQO_Q8_1 9
#define RQO_Q2_K 10
#define RQO_Q3_K 11
#define RQO_Q8_K 15
#define RQO_IQ4_XS 23

/* activation handling, as a layer gets it from its precision (recipe.rs:22326-22369) */
#define RQO_ACT_FLOAT_RUN 0   /* packed bodies + run decoders: recipe.rs:7826-7917, ll:3136-3508 */
#define RQO_ACT_FLOAT_EXACT 1 /* contraction body exact branch: ll:1734-1811, build.rs:923-1022 */
#define RQO_ACT_INT8 2        /* int8 records: ll:1381-1517 and the slice/block dots */

int rqo_block_values(int type);  /* 32 or 256, 0 if unknown */
int rqo_block_bytes(int type);   /* 18, 34, 144, 210; 20, 22, 24, 176, 18; 36, 84, 110, 292, 136 */

uint16_t rqo_fp16(float value);      /* recipe.rs:15098-15112 */
float rqo_unfp16(uint16_t value);    /* recipe.rs:15114-15126 */
float rqo_qround(float value);       /* recipe.rs:15133-15135 */

/* Dequantise `count` values (whole blocks) to fp32: f32(HostQuantOps value). */
int rqo_dequantize(int type, const uint8_t* blocks, int64_t count, float* out, int threads);
/* Quantise `count` fp32 values (padded with zeros to whole blocks) into blocks. */
int rqo_quantize(int type, const float* values, int64_t count, uint8_t* blocks, int threads);

/* The load-time re-encode `.int(8)` applies to a tensor bound in a format it does not keep
 * (a lone Q6_K or Q4_0 tensor): decode with the source decoder, encode as Q8_0 with the load
 * kernel's encoder (recipe.rs:22345-22431, :8016-8127). out: ceil(count / 32) * 34 bytes. */
int rqo_requantize_q8_0(int type, const uint8_t* blocks, int64_t count, uint8_t* out, int threads);
/* `.int(4)`: storage Q4_1 (recipe.rs:22348); a tensor not stored as Q4_1 is decoded and encoded as Q4_1 by the load
 * kernel (recipe.rs:8088-8094). out: ceil(count / 32) * 20 bytes. rqo_matvec with RQO_ACT_INT8 over Q4_1 blocks is the
 * int dot such a layer then runs (block32 slice kind 3, build.rs:777-796). */
int rqo_requantize_q4_1(int type, const uint8_t* blocks, int64_t count, uint8_t* out, int threads);

/* int8 activation records (36 bytes each: fp32 d, 32 codes) for one column of `terms`
 * inputs read at x[k * x_stride]; `step` is 32 or 256. ll:1381-1517, CPU wave width 1. */
int rqo_quantize_activations(const float* x, int64_t x_stride, int64_t terms, int step, uint8_t* records);

/* y[n * y_stride + t] = sum_k W[n][k] * x[k * x_stride + t] for t < tokens.
 * The reference's layout is channel-major (x_stride = y_stride = tokens).
 * act_mode selects the dot semantics; step (32|256) matters for RQO_ACT_INT8 only.
 * Rows are dealt to threads as row r -> thread r mod T (recipe.rs:29264-29292). */
int rqo_matvec(int type, const uint8_t* blocks, int64_t rows, int64_t cols,
               const float* x, int64_t x_stride, int tokens,
               float* y, int64_t y_stride, int act_mode, int step, int threads);

/* Portable transcendentals, build.rs:1079-1176 (math = "portable"). */
float rqo_exp(float x);
float rqo_tanh(float x);
float rqo_sigmoid(float x);  /* 0.5 * (tanh(0.5 x) + 1), recipe.rs:22662-22668 */
float rqo_silu(float x);

/* Routing weights of `tokens` positions: scores and weights are [experts][tokens].
 * scoring 0 = softmax, 1 = sigmoid. selection_bias may be NULL. ll:4666-4716. */
int rqo_topk(const float* scores, int experts, int tokens, int top, int scoring, int renormalize,
             const float* selection_bias, float* weights);

/* gguf_moe forward for `tokens` positions (recipe.rs:23386-23459, ll:2304-2365 modes 1/2):
 * gate/up banks are [experts][ffn][hidden] rows of `type` blocks, down is [experts][hidden][ffn].
 * routing is the dense [experts][tokens] plane. x and y are [hidden][tokens] channel-major.
 * Shared expert (optional, shared_gate_w != NULL): gate scalar sigmoid(w . x), then the same
 * pipeline with one expert; y = routed + shared. */
int rqo_moe_forward(int type, const uint8_t* gate, const uint8_t* up, const uint8_t* down,
                    int experts, int top, int hidden, int ffn,
                    const float* x, const float* routing, int tokens,
                    const uint8_t* sh_gate, const uint8_t* sh_up, const uint8_t* sh_down,
                    const float* shared_gate_w, float* y, int threads);

/* The same with the rest of gguf_moe's arguments: routed weights times `routed_scale`; shared_kind 0 none, 1 ungated
 * (weight one), 2 gated; the shared expert is shared_count * ffn wide (its banks: gate/up [count*ffn][hidden], down
 * [hidden][count*ffn]). recipe.rs:23415-23459, SharedExpert :13855-13862. */
int rqo_moe_forward_ex(int type, const uint8_t* gate, const uint8_t* up, const uint8_t* down,
                       int experts, int top, int hidden, int ffn,
                       const float* x, const float* routing, int tokens, float routed_scale,
                       int shared_kind, int shared_count,
                       const uint8_t* sh_gate, const uint8_t* sh_up, const uint8_t* sh_down,
                       const float* shared_gate_w, float* y, int threads);

/* The steps either side of a projection in a decode layer: RMS norm (recipe.rs:6836-7120, Rms mode), the logit soft-cap
 * (scale, tanh, scale: rnj-1.rs:47-51) and the gated product silu(gate) * up (lower_gated, recipe.rs:23279-23286). */
void rqo_rmsnorm(const float* x, int64_t x_stride, int64_t n, const float* gain, float epsilon, float* y, int64_t y_stride);
void rqo_softcap(const float* x, int64_t n, double cap, float* y);
void rqo_glu(const float* gate, const float* up, int64_t n, float* y);

/* Counter-based synthetic inputs: splitmix64 -> Box-Muller (f64) -> scale -> f32.
 * Value i of stream (seed, stream) depends only on (seed, stream, i). */
void rqo_normal(uint64_t seed, uint64_t stream, int64_t first, int64_t count, double sigma, float* out);

#ifdef __cplusplus
}
#endif
#endif
