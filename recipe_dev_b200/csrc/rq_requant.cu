// Load-time re-encode of a bound tensor into Q8_0 (`.int(8)`) or Q4_1 (`.int(4)`), byte-exact with the reference's load kernel.
//
// In the reference `.int(8)` keeps a tensor only when it is Q8_0, Q4_K or a Q4_K + Q6_K mix
// (finish_int_sums, recipe.rs:22345-22369). Every other bound tensor -- a lone Q6_K or Q4_0
// one -- is decoded by its source decoder and encoded again as Q8_0, once, by the load kernel
// (requantize_bound recipe.rs:22373-22431, emit_requantize recipe.rs:8016-8127, dispatched per
// node by recipe_model_load :8128-8165), and the int8 dot then runs over those Q8_0 blocks.
//
// The encoder here is that kernel's, not the host's Integer::compress: the extreme is the FIRST
// value of strictly largest magnitude (a running value that starts at zero), the code is
// fptosi(q + 0.5) or fptosi(q - 0.5) by the sign of q (half away from zero by truncation; f32::round
// differs when q + 0.5 itself rounds up), the scale is narrowed to fp16 with round to nearest even.
//
// One warp takes one 32-value block: lane i decodes value i from the source planes, the lanes agree
// on the extreme by shuffles, and every lane writes its code straight into the Q8_0 planes of the
// new weight (permuted chunks and all), so no staging buffer of GGUF blocks or fp32 values exists.
#include "rq_decode.cuh"
#include "rq_internal.cuh"

namespace {

template <int SRC>
__global__ void rq_requant_q8_0_kernel(const uint8_t* __restrict__ src_main, const uint16_t* __restrict__ src_scale, int64_t rows, int64_t cols,
                                       uint8_t* __restrict__ dst_codes, uint16_t* __restrict__ dst_d) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int64_t blocks = rows * (cols >> 5);
    const bool permuted = rq_plane_permuted(RQ_Q8_0, cols);
    for (int64_t b = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; b < blocks; b += warps) {
        const int64_t i = b * 32 + lane;
        const float v = rq_decode_value<SRC>(src_main, src_scale, i, cols);
        // first value of strictly largest magnitude: the larger |v| wins, equal magnitudes go to the lower index
        float e = v == v ? v : 0.0f;  // a NaN is never "larger": the running extreme skips it
        int at = lane;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float oe = __shfl_xor_sync(0xffffffffu, e, off);
            const int oa = __shfl_xor_sync(0xffffffffu, at, off);
            if (fabsf(oe) > fabsf(e) || (fabsf(oe) == fabsf(e) && oa < at)) { e = oe; at = oa; }
        }
        const float scale = __fdiv_rn(fabsf(e), 127.0f);
        const float inverse = scale == 0.0f ? 0.0f : __fdiv_rn(1.0f, scale);
        const float q = __fmul_rn(v, inverse);
        const float r = q >= 0.0f ? __fadd_rn(q, 0.5f) : __fadd_rn(q, -0.5f);
        int code = __float2int_rz(r);
        code = code < -128 ? -128 : (code > 127 ? 127 : code);
        int64_t where = i;
        if (permuted) {
            const int64_t row = i / cols, off = i - row * cols;
            where = row * cols + ((rq_plane_chunk(RQ_Q8_0, off >> 4) << 4) | (off & 15));
        }
        dst_codes[where] = (uint8_t)(int8_t)code;
        if (lane == 0) dst_d[b] = __half_as_ushort(__float2half_rn(scale));
    }
}

// The same for `.int(4)`, whose storage is Q4_1 (recipe.rs:22348): emit_requantize's DeviceQuantizer::Q4_1 arm
// (recipe.rs:8037-8047, :8088-8094, :8099-8112). Minimum and maximum of the block (the first of equal values is kept, which
// matters for the sign of a zero), step = (max - min) / 15, code = fptoui(clamp((v - min) * (1 / step) + 0.5, 0, 15)); step
// and minimum narrowed to fp16 with round to nearest even; codes two to a byte, value i low and value i + 16 high. The new
// weight keeps its GGUF blocks (20 bytes each).
template <int SRC>
__global__ void rq_requant_q4_1_kernel(const uint8_t* __restrict__ src_main, const uint16_t* __restrict__ src_scale, int64_t rows, int64_t cols,
                                       uint8_t* __restrict__ dst_blocks) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int64_t blocks = rows * (cols >> 5);
    for (int64_t b = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; b < blocks; b += warps) {
        const float v = rq_decode_value<SRC>(src_main, src_scale, b * 32 + lane, cols);
        float mn = v, mx = v;
        int mn_at = lane, mx_at = lane;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float on = __shfl_xor_sync(0xffffffffu, mn, off), ox = __shfl_xor_sync(0xffffffffu, mx, off);
            const int an = __shfl_xor_sync(0xffffffffu, mn_at, off), ax = __shfl_xor_sync(0xffffffffu, mx_at, off);
            if (on < mn || (on == mn && an < mn_at)) { mn = on; mn_at = an; }
            if (ox > mx || (ox == mx && ax < mx_at)) { mx = ox; mx_at = ax; }
        }
        const float scale = __fdiv_rn(__fsub_rn(mx, mn), 15.0f);
        const float inverse = scale == 0.0f ? 0.0f : __fdiv_rn(1.0f, scale);
        float sh = __fadd_rn(__fmul_rn(__fsub_rn(v, mn), inverse), 0.5f);
        sh = sh < 0.0f ? 0.0f : sh;
        sh = sh > 15.0f ? 15.0f : sh;
        const unsigned code = __float2uint_rz(sh);
        const unsigned high = __shfl_down_sync(0xffffffffu, code, 16);
        uint8_t* blk = dst_blocks + b * 20;
        if (lane < 16) blk[4 + lane] = (uint8_t)(code | (high << 4));
        if (lane == 0) {
            *(uint16_t*)blk = __half_as_ushort(__float2half_rn(scale));
            *(uint16_t*)(blk + 2) = __half_as_ushort(__float2half_rn(mn));
        }
    }
}

}  // namespace

int rq_launch_requant_q4_1(const rq_weight* src, rq_weight* dst, cudaStream_t s) {
    const int64_t blocks = src->rows * (src->cols / 32);
    const int threads = 256;
    int64_t want = (blocks * 32 + threads - 1) / threads;
    const int grid = (int)(want < 148 * 32 ? (want < 1 ? 1 : want) : 148 * 32);
    switch (src->type) {
#define RQ_CASE(T) case T: rq_requant_q4_1_kernel<T><<<grid, threads, 0, s>>>(src->main, src->scale, src->rows, src->cols, dst->main); break;
        RQ_CASE(RQ_Q4_K) RQ_CASE(RQ_Q6_K) RQ_CASE(RQ_Q8_0) RQ_CASE(RQ_Q4_0) RQ_DECODE_ONLY_TYPES(RQ_CASE)
#undef RQ_CASE
        default: return rq_fail(RQ_ERR_INVALID, "requantize: source type %d", src->type);
    }
    RQ_CUDA(cudaGetLastError());
    return RQ_OK;
}

int rq_launch_requant_q8_0(const rq_weight* src, rq_weight* dst, cudaStream_t s) {
    const int64_t blocks = src->rows * (src->cols / 32);
    const int threads = 256;
    int64_t want = (blocks * 32 + threads - 1) / threads;
    const int grid = (int)(want < 148 * 32 ? (want < 1 ? 1 : want) : 148 * 32);
    switch (src->type) {
        case RQ_Q4_K: rq_requant_q8_0_kernel<RQ_Q4_K><<<grid, threads, 0, s>>>(src->main, src->scale, src->rows, src->cols, dst->main, dst->scale); break;
        case RQ_Q6_K: rq_requant_q8_0_kernel<RQ_Q6_K><<<grid, threads, 0, s>>>(src->main, src->scale, src->rows, src->cols, dst->main, dst->scale); break;
        case RQ_Q8_0: rq_requant_q8_0_kernel<RQ_Q8_0><<<grid, threads, 0, s>>>(src->main, src->scale, src->rows, src->cols, dst->main, dst->scale); break;
        case RQ_Q4_0: rq_requant_q8_0_kernel<RQ_Q4_0><<<grid, threads, 0, s>>>(src->main, src->scale, src->rows, src->cols, dst->main, dst->scale); break;
#define RQ_CASE(T) case T: rq_requant_q8_0_kernel<T><<<grid, threads, 0, s>>>(src->main, src->scale, src->rows, src->cols, dst->main, dst->scale); break;
        RQ_DECODE_ONLY_TYPES(RQ_CASE)
#undef RQ_CASE
        default: return rq_fail(RQ_ERR_INVALID, "requantize: source type %d", src->type);
    }
    RQ_CUDA(cudaGetLastError());
    return RQ_OK;
}
