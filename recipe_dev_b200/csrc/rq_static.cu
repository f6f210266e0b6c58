// rq_matvec_int8_static: the INT8 matrix-vector product for callers that cannot allocate.
//
// The ordinary INT8 path keeps the quantised activations in a scratch buffer that the context
// grows with cudaMalloc the first time a wider column arrives. Two kinds of caller cannot live
// with that: a host that has already handed every byte of device memory to arenas it planned up
// front (the way recipe itself places weights, values and contexts) has nothing left for a
// library to allocate from; and a decode loop that may not stall cannot take the device-wide
// synchronisation an allocation or a free implies. For them the scratch is this file-scope
// array, a fixed part of the library's image on every GPU that loads it, until the process exits.
//
// Limits and sharing: one token, a contiguous column of at most RQ_STATIC_MAX_COLS inputs.
// Every call on a device writes the same array, so two calls that overlap on the GPU (different
// streams, or threads) race; calls on one stream are ordered and safe. Nothing in the array has
// to start at zero: the quantiser overwrites every byte the product reads (codes, steps, slice and
// group sums) for the width of the call, and what an earlier, wider call left beyond that is never
// read.
#include "rq_internal.cuh"

// 128 units of 336 bytes (the widest column, 32768 inputs, in the unit-record layout); narrower
// plane layouts (widths that are not whole 256-value units) need less.
#define RQ_STATIC_SCRATCH_BYTES (RQ_STATIC_MAX_COLS / 256 * RQ_ACT_RECORD_INT8)

static __device__ __align__(256) uint8_t g_static_act[RQ_STATIC_SCRATCH_BYTES];

// In host code `g_static_act` is only a handle for the runtime, not a device address: the address
// each device gave the array is asked for once per device, with that device current, and kept.
static uint8_t* g_static_ptr[64] = {};

static int static_scratch(int device, uint8_t** out) {
    if (device < 0 || device >= 64) return rq_fail(RQ_ERR_LIMIT, "rq_matvec_int8_static: device %d beyond the 64 this entry point tracks", device);
    if (!g_static_ptr[device]) {
        void* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_act);
        if (e != cudaSuccess || !ptr) return rq_fail(RQ_ERR_CUDA, "rq_matvec_int8_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        g_static_ptr[device] = (uint8_t*)ptr;
    }
    *out = g_static_ptr[device];
    return RQ_OK;
}

extern "C" int rq_matvec_int8_static(rq_ctx* ctx, const rq_weight* w, const float* x, float* y, int step, void* stream) {
    if (!ctx || !w || !x || !y) return rq_fail(RQ_ERR_INVALID, "rq_matvec_int8_static: null argument");
    if (w->device != ctx->device) return rq_fail(RQ_ERR_INVALID, "rq_matvec_int8_static: weight lives on device %d, context on %d", w->device, ctx->device);
    if (step != 32 && step != 256) return rq_fail(RQ_ERR_INVALID, "rq_matvec_int8_static: int8 step=%d must be 32 or 256", step);
    if (!rq_type_has_fast_path(w->type)) return rq_fail(RQ_ERR_UNSUPPORTED, "rq_matvec_int8_static: type %d has no int8 dot; re-encode it with rq_weight_requantize first", w->type);
    if (w->cols > RQ_STATIC_MAX_COLS)
        return rq_fail(RQ_ERR_LIMIT, "rq_matvec_int8_static: %lld inputs per row, but the fixed scratch holds at most %d; use rq_matvec, which allocates",
                       (long long)w->cols, RQ_STATIC_MAX_COLS);
    if (rq_act_token_bytes(w->cols) > (size_t)RQ_STATIC_SCRATCH_BYTES)
        return rq_fail(RQ_ERR_LIMIT, "rq_matvec_int8_static: the records of %lld inputs do not fit the fixed scratch", (long long)w->cols);
    DeviceGuard guard(ctx->device);
    if (!guard.ok) return rq_fail(RQ_ERR_CUDA, "rq_matvec_int8_static: cannot select device %d", ctx->device);
    uint8_t* scratch = nullptr;
    int rc = static_scratch(ctx->device, &scratch);
    if (rc) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    rc = rq_launch_act_quant(x, 1, w->cols, w->cols, 1, step, scratch, nullptr, s);
    if (rc) return rc;
    rc = rq_launch_gemv_stream(ctx, w, x, 1, w->cols, 1, y, 1, w->rows, RQ_ACT_INT8, scratch, 0, nullptr, s);
    if (rc != RQ_ERR_UNSUPPORTED) return rc;
    return rq_launch_gemv_tiled_int8(ctx, w, 1, y, 1, w->rows, scratch, s);
}
