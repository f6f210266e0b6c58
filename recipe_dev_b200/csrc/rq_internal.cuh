// Internal declarations shared by the translation units of librq_b200.so.
// Device layouts of the four stored formats, the context, and small device helpers.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "rq.h"

// ---------------------------------------------------------------------------------
// Data layout in HBM.
//
// Q4_K keeps its GGUF blocks as they are: 144 bytes = nine 16-byte lines, the first the
// header (d, dmin, twelve scale bytes), the other eight the nibbles, so every line of a
// row is a 128-bit load.
// The other three formats have strides that are only 2-byte aligned (18, 34, 210), so
// they are split into planes at load, the same bytes in aligned places:
//   Q6_K : body  [rows][blocks][208] = ql(128) | qh(64) | scales(16)   + d [rows][blocks] fp16
//   Q8_0 : codes [rows][cols] int8                                      + d [rows][cols/32] fp16
//   Q4_0 : qs    [rows][cols/32][16]                                    + d [rows][cols/32] fp16
// No plane is padded: device bytes equal GGUF bytes.
// ---------------------------------------------------------------------------------
struct rq_weight {
    int type;
    int64_t rows, cols;
    uint8_t* main;   // Q4_K blocks | Q6_K bodies | Q8_0 codes | Q4_0 nibbles
    uint16_t* scale; // fp16 d plane (null for Q4_K)
    int64_t bytes;   // total device bytes
    int device;
    // K-quant weights of whole superblocks: a TMA descriptor of the main plane as a [rows][row bytes] byte matrix, fetched in
    // tiles of 128 rows x one superblock (144 / 208 bytes) by the batched kernel
    alignas(64) CUtensorMap tile_map;
    int has_tile_map;
};

struct rq_ctx {
    int device;
    int sm_count;
    // scratch the INT8 path writes its activation records into (grown on demand)
    uint8_t* act_scratch;
    size_t act_scratch_bytes;
    int64_t act_cols; int act_tokens; int act_step;  // what the scratch holds (0 = nothing)
    int* error_flag;  // device word a kernel sets when a bounded wait ran out
    unsigned long long wait_limit_ns;  // how long a kernel of this context waits on a barrier before it gives up
    int* pin_flag;    // pinned host copy, refreshed by the host-buffer entry points
    // pinned + device staging for the host-buffer entry points
    float* stage_x; float* stage_y; size_t stage_x_bytes, stage_y_bytes;
    float* pin_x; float* pin_y; size_t pin_x_bytes, pin_y_bytes;
    cudaStream_t stream; // used by the host-buffer entry points
    // the stream of the last call that used the context's work areas (the activation scratch, a bank's plans), and the event
    // a call on another stream waits for before it touches them
    cudaStream_t work_stream; bool work_stream_set; cudaEvent_t work_event;
    bool recording;  // between rq_sequence_begin and rq_sequence_end: the context's stream is capturing, nothing may allocate
};

int rq_fail(int status, const char* fmt, ...);
#define RQ_CUDA(call)                                                                         \
    do {                                                                                      \
        cudaError_t e_ = (call);                                                              \
        if (e_ != cudaSuccess) return rq_fail(RQ_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e_)); \
    } while (0)

struct DeviceGuard {
    int prev;
    bool ok;
    explicit DeviceGuard(int dev) : prev(-1), ok(false) {
        if (cudaGetDevice(&prev) != cudaSuccess) return;
        ok = (prev == dev) || cudaSetDevice(dev) == cudaSuccess;
    }
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

// Device-side activation scratch, per token (INT8 path).
// Inputs that are whole 256-value units use one padded record per unit, the layout the streaming
// kernel keeps in shared memory:
//   codes[256] int8 | d[8] fp32 @256 | sum16[16] int16 @288 | sum32[8] int16 @320   (336 bytes)
// Other widths use three planes: codes [cols] int8 | d [cols/32] fp32 | sum16 [cols/16] int16.
// d = the step of a 32-value group, sum16 = the sum of the 16 codes of a slice.
#define RQ_ACT_RECORD_INT8 336
#define RQ_ACT_RECORD_FLOAT 1104
__host__ __device__ inline bool rq_act_unit_layout(int64_t cols) { return cols % 256 == 0; }
__host__ __device__ inline size_t rq_act_token_bytes(int64_t cols) {
    return rq_act_unit_layout(cols) ? (size_t)(cols / 256) * RQ_ACT_RECORD_INT8
                                    : (size_t)cols + (size_t)(cols / 32) * 4 + (size_t)(cols / 16) * 2;
}

// Orders this call's use of the context's work areas after the previous call's when the two were given different streams.
int rq_order_work_areas(rq_ctx* ctx, cudaStream_t s);
// Makes the activation scratch at least `bytes` large (growing it synchronises the device: rq_reserve does that ahead of
// time) and orders its use on `s` after the previous call's.
int rq_ensure_act_scratch(rq_ctx* ctx, size_t bytes, cudaStream_t s);

// launchers (defined in the .cu files)
int rq_launch_repack(const rq_weight* w, const uint8_t* dev_blocks, cudaStream_t s);
int rq_launch_export(const rq_weight* w, uint8_t* dev_blocks, cudaStream_t s);
int rq_launch_dequant(const rq_weight* w, float* out, cudaStream_t s);
int rq_launch_gemv_generic(rq_ctx* ctx, const rq_weight* w, const float* x, int64_t sk, int64_t st, int tokens, float* y, int64_t yn, int64_t yt, cudaStream_t s);
int rq_launch_gather(const rq_weight* w, const int32_t* ids, int tokens, float* y, int64_t yn, int64_t yt, cudaStream_t s);
// fills w->tile_map for Q4_K / Q6_K weights (no-op for the others)
int rq_make_tile_map(rq_weight* w);
int rq_launch_requant_q8_0(const rq_weight* src, rq_weight* dst, cudaStream_t s);
int rq_launch_requant_q4_1(const rq_weight* src, rq_weight* dst, cudaStream_t s);
int rq_launch_gemv_q41_int8(rq_ctx* ctx, const rq_weight* w, const uint8_t* records, int tokens, float* y, int64_t yn, int64_t yt, cudaStream_t s);
int rq_launch_act_quant(const float* x, int64_t sk, int64_t st, int64_t cols, int tokens, int step,
                        uint8_t* scratch, uint8_t* records36, cudaStream_t s);
int rq_launch_gemv(rq_ctx* ctx, const rq_weight* w, const float* x, int64_t sk, int64_t st, int tokens,
                   float* y, int64_t yn, int64_t yt, int act_mode, int step, cudaStream_t s);
int rq_launch_gemv_multi(rq_ctx* ctx, int n, const rq_weight* const* ws, const float* x, int64_t sk, int64_t st, int tokens,
                         float* const* ys, int64_t yn, int64_t yt, int act_mode, int step, cudaStream_t s);
int rq_launch_gemv_tiled_int8(rq_ctx* ctx, const rq_weight* w, int tokens, float* y, int64_t yn, int64_t yt, const uint8_t* act, cudaStream_t s);
// RQ_ERR_UNSUPPORTED (no error text) = width not served by the tensor-core kernel
int rq_launch_matmul(rq_ctx* ctx, const rq_weight* w, const float* x, int64_t sk, int64_t st, int tokens, float* y, int64_t yn, int64_t yt, cudaStream_t s);
// The K-quant batched product with integer weight operands (rq_matmul_kq.cu): FLOAT or INT8 activations.
// RQ_ERR_UNSUPPORTED (no error text) = not a Q4_K / Q6_K weight.
int rq_launch_matmul_kq(rq_ctx* ctx, const rq_weight* w, const float* x, int64_t sk, int64_t st, int tokens, float* y, int64_t yn, int64_t yt, int act_mode,
                        int step, cudaStream_t s);
size_t rq_matmul_kq_scratch_bytes(const rq_ctx* ctx, int type, int64_t rows, int64_t cols, int tokens);
// y[row][token] = the splits' partial sums ([split][token][row]) added in split order
int rq_launch_sum_splits(const float* partial, int splits, int64_t rows, int tokens, float* y, int64_t yn, int64_t yt, cudaStream_t s);
// scratch bytes rq_launch_matmul takes for a weight of this shape and this many tokens (its activation image and split-K sums)
size_t rq_matmul_scratch_bytes(const rq_ctx* ctx, int64_t rows, int64_t cols, int tokens);
int rq_launch_quantize(int type, const float* values, int64_t count, uint8_t* blocks, cudaStream_t s);
// A run of virtual output rows of the streaming kernel (see rq_gemv_stream.cu).
#define RQ_MAX_SUB 16
#define RQ_INLINE_SEGMENTS 4
#define RQ_MAX_SEGMENTS 16
enum { RQ_EPI_PLAIN = 0, RQ_EPI_WSUM = 1, RQ_EPI_GLU = 2 };
struct RqSegment {
    int row_begin, rows;                 // virtual rows [row_begin, row_begin + rows)
    float* y;                            // y[local_row * yn + token * yt]
    const uint8_t* main[RQ_MAX_SUB];     // main plane of each sub-row's matrix, at this segment's first row
    const uint16_t* scale[RQ_MAX_SUB];   // its fp16 d plane there (null for Q4_K)
    int act[RQ_MAX_SUB];                 // the staged activation vector each sub-row dots
    float coef[RQ_MAX_SUB];              // RQ_EPI_WSUM: the coefficient of each sub-row
};
// A segment table in device memory, written by a kernel (the expert planner): the counts are read
// on the device, so the host launches without knowing how many experts a token routed here.
struct RqPlan {
    int n_segments;   // <= RQ_MAX_SEGMENTS
    int subs;         // sub-rows per virtual row in use, <= the launch's `subs`
    int total_rows;   // virtual rows of all segments
    int pad;
    RqSegment seg[RQ_MAX_SEGMENTS];
};
int rq_launch_stream_plan(rq_ctx* ctx, int type, int64_t cols, const RqPlan* plan, int plan_count, int plan_stride, int max_segments, int max_subs,
                          int epilogue, int64_t max_rows, const float* x, int64_t x_plan_stride, int64_t sk, int64_t st, int vectors, int64_t yn, int64_t yt,
                          cudaStream_t s);
int rq_launch_stream(rq_ctx* ctx, int type, int64_t cols, const RqSegment* table, const RqSegment* inline_seg, int n_segments, int subs,
                     int epilogue, int64_t total_rows, const float* x, int64_t sk, int64_t st, int tokens, int vectors_per_launch,
                     int64_t yn, int64_t yt, int act_mode, const uint8_t* act, int fuse_step, uint8_t* act_out, cudaStream_t s);
// RQ_ERR_UNSUPPORTED (no error text) = shape not served by the streaming kernel.
// fuse_step = 32 / 256: an INT8 launch quantises x itself in its prologue (single token; nothing is
// launched when the shape cannot be served that way) and leaves the records at act_out; 0: the
// records are read from `act`.
int rq_launch_gemv_stream(rq_ctx* ctx, const rq_weight* w, const float* x, int64_t sk, int64_t st, int tokens,
                          float* y, int64_t yn, int64_t yt, int act_mode, const uint8_t* act, int fuse_step, uint8_t* act_out, cudaStream_t s);

// ---------------------------------------------------------------------------------
// device helpers
// ---------------------------------------------------------------------------------
#ifdef __CUDACC__
__device__ __forceinline__ float rq_h2f(uint16_t h) { return __half2float(__ushort_as_half(h)); }

// Q8_0 / Q4_0 main planes of rows made of whole 256-value units keep each row's 16-byte chunks PERMUTED: logical chunk L
// of a row (a unit is 16 chunks of Q8_0, 8 of Q4_0) sits at L with its low three bits xor-ed with the low three bits of
// its unit index. In shared memory a thread's unit starts at a multiple of 128 bytes, so eight threads on adjacent
// units reading the same logical chunk would otherwise all hit one 16-byte bank group; permuted, they hit eight.
// The map is its own inverse. Rows that are not whole units (the tiled kernel's) are stored as they come.
// every format that is served by per-value decode alone, for switch statements over kernels templated on the type
#define RQ_DECODE_ONLY_TYPES(X) X(RQ_Q4_1) X(RQ_Q5_0) X(RQ_Q5_1) X(RQ_Q5_K) X(RQ_IQ4_NL) X(RQ_Q8_1) X(RQ_Q2_K) X(RQ_Q3_K) X(RQ_Q8_K) X(RQ_IQ4_XS)
// Q4_K and the formats served by per-value decode alone stay in HBM as their GGUF blocks (one plane, no scale plane)
__host__ __device__ __forceinline__ bool rq_type_keeps_blocks(int type) {
    return type == RQ_Q4_K || type == RQ_Q4_1 || type == RQ_Q5_0 || type == RQ_Q5_1 || type == RQ_Q5_K || type == RQ_IQ4_NL || type == RQ_Q8_1 || type == RQ_Q2_K ||
           type == RQ_Q3_K || type == RQ_Q8_K || type == RQ_IQ4_XS;
}
// the formats with streaming / tensor-core kernels and int8 slice dots of their own; the rest go through rq_gemv_generic.cu
__host__ __device__ __forceinline__ bool rq_type_has_fast_path(int type) { return type == RQ_Q4_0 || type == RQ_Q8_0 || type == RQ_Q4_K || type == RQ_Q6_K; }
__host__ __device__ __forceinline__ bool rq_plane_permuted(int type, int64_t cols) { return (type == RQ_Q8_0 || type == RQ_Q4_0) && cols % 256 == 0; }
__host__ __device__ __forceinline__ int64_t rq_plane_chunk(int type, int64_t logical) { return logical ^ ((logical >> (type == RQ_Q8_0 ? 4 : 3)) & 7); }

// Six-bit scale and minimum of sub-block j from the twelve scale bytes held as three words
// (little-endian bytes 0..11).
__device__ __forceinline__ void rq_q4k_scale_min(uint32_t s0, uint32_t s1, uint32_t s2, int j, int& sc, int& mn) {
    // byte(i) of the 12: i<4 -> s0, i<8 -> s1, else s2
    if (j < 4) {
        sc = (s0 >> (8 * j)) & 63;
        mn = (s1 >> (8 * j)) & 63;
    } else {
        int i = j - 4;
        uint32_t hi = (s2 >> (8 * i)) & 0xff; // byte j+4
        uint32_t a = (s0 >> (8 * i)) & 0xff;  // byte j-4
        uint32_t b = (s1 >> (8 * i)) & 0xff;  // byte j
        sc = (hi & 15) | ((a >> 6) << 4);
        mn = (hi >> 4) | ((b >> 6) << 4);
    }
}
#endif
