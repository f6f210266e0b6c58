// Matrix-vector product over the stored formats that have no streaming kernel of their own (Q4_1, Q5_0,
// Q5_1, Q5_K, IQ4_NL): fp32 activations against per-value decoded weights, the reference's run decoders
// (recipe.rs:7826-7917: one fused-multiply-add chain per unit of 32 values in index order; the units of a
// row add up, ll:3451-3492). HBM-bound by design: a warp owns a row and walks it in units of 32 values,
// lane l taking units l, l + 32, ..; the lanes' sums meet in a fixed xor tree, so every run gives the same
// bits. `.int(8)` never reaches these formats: the reference re-encodes them to Q8_0 at load
// (rq_weight_requantize), and that weight takes the streaming kernel.
#include "rq_decode.cuh"

namespace {

constexpr int kWarps = 8;  // rows per CTA

template <int TYPE>
__global__ void __launch_bounds__(kWarps * 32) rq_gemv_generic_kernel(const uint8_t* __restrict__ main_plane, int64_t rows, int64_t cols, const float* __restrict__ x,
                                                                        int64_t sk, int64_t st, float* __restrict__ y, int64_t yn, int64_t yt) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, token = blockIdx.y;
    const float* xt = x + (int64_t)token * st;
    const int64_t units = cols >> 5;
    for (int64_t row = (int64_t)blockIdx.x * kWarps + warp; row < rows; row += (int64_t)gridDim.x * kWarps) {
        float sum = 0.f;
        for (int64_t u = lane; u < units; u += 32) {
            float unit = 0.f;
            const int64_t first = row * cols + (u << 5);
#pragma unroll 8
            for (int j = 0; j < 32; ++j) unit = fmaf(rq_decode_value<TYPE>(main_plane, nullptr, first + j, cols), __ldg(xt + ((u << 5) + j) * sk), unit);
            sum += unit;
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
        if (lane == 0) y[row * yn + (int64_t)token * yt] = sum;
    }
}

template <int TYPE>
int launch_generic(const rq_weight* w, const float* x, int64_t sk, int64_t st, int tokens, float* y, int64_t yn, int64_t yt, int sm_count, cudaStream_t s) {
    const int64_t ctas = (w->rows + kWarps - 1) / kWarps;
    const int64_t cap = (int64_t)sm_count * 8;  // eight resident CTAs of 256 threads per SM
    dim3 grid((unsigned)(ctas < cap ? ctas : cap), (unsigned)tokens);
    rq_gemv_generic_kernel<TYPE><<<grid, kWarps * 32, 0, s>>>(w->main, w->rows, w->cols, x, sk, st, y, yn, yt);
    RQ_CUDA(cudaGetLastError());
    return RQ_OK;
}

}  // namespace

int rq_launch_gemv_generic(rq_ctx* ctx, const rq_weight* w, const float* x, int64_t sk, int64_t st, int tokens, float* y, int64_t yn, int64_t yt, cudaStream_t s) {
    if (tokens > 65535) return rq_fail(RQ_ERR_LIMIT, "matvec: %d tokens over a %d-type weight, at most 65535 per call", tokens, w->type);
    switch (w->type) {
        case RQ_Q4_1: return launch_generic<RQ_Q4_1>(w, x, sk, st, tokens, y, yn, yt, ctx->sm_count, s);
        case RQ_Q5_0: return launch_generic<RQ_Q5_0>(w, x, sk, st, tokens, y, yn, yt, ctx->sm_count, s);
        case RQ_Q5_1: return launch_generic<RQ_Q5_1>(w, x, sk, st, tokens, y, yn, yt, ctx->sm_count, s);
        case RQ_Q5_K: return launch_generic<RQ_Q5_K>(w, x, sk, st, tokens, y, yn, yt, ctx->sm_count, s);
        case RQ_IQ4_NL: return launch_generic<RQ_IQ4_NL>(w, x, sk, st, tokens, y, yn, yt, ctx->sm_count, s);
        default: return rq_fail(RQ_ERR_INVALID, "matvec: type %d", w->type);
    }
}
