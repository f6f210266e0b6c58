// The steps either side of a projection in a decode layer: RMS normalisation, residual add, the logit soft-cap, and the
// dense gated feed-forward's silu(gate x) * (up x) as the epilogue of ONE matvec launch over both matrices.
//
// Semantics follow the reference: RMS norm = emit_normalize_stats in Rms mode (recipe.rs:6836-7120): sum of squares,
// variance = sum / n, scale = 1 / sqrt(variance + epsilon), y = (x * scale) * gain, every step a separate fp32 operation;
// the soft-cap is scale(1 / cap), tanh, scale(cap) with recipe's portable tanh (rnj-1.rs:47-51, build.rs:1146-1166);
// the gated product is lower_gated (recipe.rs:23279-23286). The sum of squares is added by a fixed tree (the same bits
// on every run); the reference's CPU path adds in index order, so the two agree to fp32 rounding of the sum, not bit for bit.
#include <string.h>

#include "rq_internal.cuh"

namespace {

__global__ void __launch_bounds__(256) rq_rmsnorm_kernel(const float* __restrict__ x, int64_t sk, int64_t st, int64_t n, const float* __restrict__ gain,
                                                          float epsilon, float* __restrict__ y, int64_t yk, int64_t yt) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float red[256];
    const int t = blockIdx.x, tid = threadIdx.x;
    const float* xt = x + (int64_t)t * st;
    float acc = 0.0f;
    for (int64_t k = tid; k < n; k += 256) { const float v = xt[k * sk]; acc = __fadd_rn(acc, __fmul_rn(v, v)); }
    red[tid] = acc;
    __syncthreads();
    for (int off = 128; off > 0; off >>= 1) { if (tid < off) red[tid] = __fadd_rn(red[tid], red[tid + off]); __syncthreads(); }
    const float variance = __fdiv_rn(red[0], (float)n);
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(variance, epsilon)));
    float* yo = y + (int64_t)t * yt;
    for (int64_t k = tid; k < n; k += 256) {
        const float v = __fmul_rn(xt[k * sk], scale);
        yo[k * yk] = gain ? __fmul_rn(v, gain[k]) : v;
    }
}

__global__ void __launch_bounds__(256) rq_add_kernel(const float* __restrict__ a, const float* __restrict__ b, int64_t n, float* __restrict__ y) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) y[i] = __fadd_rn(a[i], b[i]);
}

// recipe's portable tanh: u / (u + 2), u = expm1(2x), evaluated in double and rounded once (build.rs:1146-1166)
__device__ double exp_wide(double x) {
    if (x != x) return x;
    if (x > 709.782712893383973096) return __longlong_as_double(0x7ff0000000000000LL);
    if (x < -745.133219101941108420) return 0.0;
    const double kf = floor(x * 1.4426950408889634074 + 0.5);
    const int k = (int)kf;
    const double r = (x - kf * __longlong_as_double(0x3FE62E42FEE00000LL)) - kf * 1.90821492927058770002e-10;
    double factorial = 1.0, coeff[13];
#pragma unroll
    for (int t = 1; t <= 13; ++t) { factorial *= (double)t; coeff[t - 1] = 1.0 / factorial; }
    double cur = coeff[12];
#pragma unroll
    for (int t = 11; t >= 0; --t) cur = fma(cur, r, coeff[t]);
    const double expanded = 1.0 + r * cur;
    const int half = k >> 1, rest = k - half;
    auto p2 = [](int e) { int b = e + 1023; b = b < 0 ? 0 : (b > 2046 ? 2046 : b); return __longlong_as_double((long long)b << 52); };
    return expanded * p2(half) * p2(rest);
}
__device__ float tanh_portable(float xf) {
    const double x = (double)xf;
    if (x != x) return xf;
    if (fabs(x) >= 20.0) return x < 0.0 ? -1.0f : 1.0f;
    const double z = 2.0 * x;
    double u;
    if (fabs(z) < 0.35) {
        double factorial = 1.0, coeff[16];
#pragma unroll
        for (int t = 1; t <= 16; ++t) { factorial *= (double)t; coeff[t - 1] = 1.0 / factorial; }
        double cur = coeff[15];
#pragma unroll
        for (int t = 14; t >= 0; --t) cur = fma(cur, z, coeff[t]);
        u = z * cur;
    } else {
        u = exp_wide(z) - 1.0;
    }
    return (float)(u / (u + 2.0));
}

__global__ void __launch_bounds__(256) rq_softcap_kernel(const float* __restrict__ x, int64_t n, float down, float up, float* __restrict__ y) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        y[i] = __fmul_rn(tanh_portable(__fmul_rn(x[i], down)), up);
}

template <typename... Args>
int launch_pdl(void (*kernel)(Args...), unsigned grid, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(256);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    RQ_CUDA(cudaLaunchKernelEx(&cfg, kernel, args...));
    return RQ_OK;
}

unsigned grid_for(int64_t n) { const int64_t want = (n + 255) / 256; return (unsigned)(want < 1 ? 1 : (want > 148 * 8 ? 148 * 8 : want)); }

}  // namespace

extern "C" int rq_rmsnorm(rq_ctx* ctx, const float* x, int64_t x_k_stride, int64_t x_t_stride, int64_t n, int tokens, const float* gain, float epsilon, float* y,
                          int64_t y_k_stride, int64_t y_t_stride, void* stream) {
    if (!ctx || !x || !y) return rq_fail(RQ_ERR_INVALID, "rq_rmsnorm: null argument");
    if (n <= 0 || tokens <= 0 || x_k_stride <= 0 || y_k_stride <= 0) return rq_fail(RQ_ERR_INVALID, "rq_rmsnorm: n, tokens and strides must be positive");
    if (!(epsilon >= 0.0f)) return rq_fail(RQ_ERR_INVALID, "rq_rmsnorm: epsilon must be non-negative");
    DeviceGuard guard(ctx->device);
    return launch_pdl(rq_rmsnorm_kernel, (unsigned)tokens, (cudaStream_t)stream, x, x_k_stride, x_t_stride, n, gain, epsilon, y, y_k_stride, y_t_stride);
}

extern "C" int rq_add(rq_ctx* ctx, const float* a, const float* b, int64_t n, float* y, void* stream) {
    if (!ctx || !a || !b || !y) return rq_fail(RQ_ERR_INVALID, "rq_add: null argument");
    if (n <= 0) return rq_fail(RQ_ERR_INVALID, "rq_add: n must be positive");
    DeviceGuard guard(ctx->device);
    return launch_pdl(rq_add_kernel, grid_for(n), (cudaStream_t)stream, a, b, n, y);
}

extern "C" int rq_softcap(rq_ctx* ctx, const float* x, int64_t n, double cap, float* y, void* stream) {
    if (!ctx || !x || !y) return rq_fail(RQ_ERR_INVALID, "rq_softcap: null argument");
    if (n <= 0) return rq_fail(RQ_ERR_INVALID, "rq_softcap: n must be positive");
    if (!(cap > 0.0) || cap > 1e300) return rq_fail(RQ_ERR_INVALID, "final logit softcap must be finite and positive");
    DeviceGuard guard(ctx->device);
    return launch_pdl(rq_softcap_kernel, grid_for(n), (cudaStream_t)stream, x, n, (float)(1.0 / cap), (float)cap, y);
}

// y = silu(gate x) * (up x): one launch of the streaming kernel, a virtual row = (gate row, up row), joined by the gated epilogue
extern "C" int rq_matvec_glu(rq_ctx* ctx, const rq_weight* gate, const rq_weight* up, const float* x, int64_t sk, int64_t st, int tokens, float* y, int64_t yn,
                             int64_t yt, int act_mode, int step, void* stream) {
    if (!ctx || !gate || !up || !x || !y) return rq_fail(RQ_ERR_INVALID, "rq_matvec_glu: null argument");
    if (gate->device != ctx->device || up->device != ctx->device) return rq_fail(RQ_ERR_INVALID, "rq_matvec_glu: a weight lives on another device than the context");
    if (gate->type != up->type || gate->rows != up->rows || gate->cols != up->cols)
        return rq_fail(RQ_ERR_INVALID, "rq_matvec_glu: gate and up must have one format and one shape");
    if (tokens <= 0 || sk <= 0 || yn <= 0 || (tokens > 1 && (st <= 0 || yt <= 0))) return rq_fail(RQ_ERR_INVALID, "rq_matvec_glu: tokens and strides must be positive");
    if (act_mode != RQ_ACT_FLOAT && act_mode != RQ_ACT_INT8) return rq_fail(RQ_ERR_INVALID, "rq_matvec_glu: act_mode=%d is neither FLOAT(0) nor INT8(1)", act_mode);
    if (act_mode == RQ_ACT_INT8 && step != 32 && step != 256) return rq_fail(RQ_ERR_INVALID, "rq_matvec_glu: int8 step=%d must be 32 or 256", step);
    if (!rq_type_has_fast_path(gate->type)) return rq_fail(RQ_ERR_UNSUPPORTED, "rq_matvec_glu: type %d has no fused form; run rq_matvec on gate and up", gate->type);
    if (gate->cols % 256) return rq_fail(RQ_ERR_UNSUPPORTED, "rq_matvec_glu: %lld inputs per row; the fused form serves rows of whole 256-value units", (long long)gate->cols);
    DeviceGuard guard(ctx->device);
    cudaStream_t s = (cudaStream_t)stream;
    RqSegment seg;
    memset(&seg, 0, sizeof(seg));
    seg.row_begin = 0; seg.rows = (int)gate->rows; seg.y = y;
    seg.main[0] = gate->main; seg.scale[0] = gate->scale; seg.main[1] = up->main; seg.scale[1] = up->scale;
    seg.act[0] = 0; seg.act[1] = 0; seg.coef[0] = 1.0f; seg.coef[1] = 1.0f;
    int rc;
    if (act_mode == RQ_ACT_INT8) {
        rc = rq_ensure_act_scratch(ctx, rq_act_token_bytes(gate->cols) * (size_t)tokens, s);
        if (rc) return rc;
        rc = rq_launch_act_quant(x, sk, st, gate->cols, tokens, step, ctx->act_scratch, nullptr, s);
        if (rc) return rc;
        ctx->act_cols = gate->cols; ctx->act_tokens = tokens; ctx->act_step = step;
    }
    rc = rq_launch_stream(ctx, gate->type, gate->cols, nullptr, &seg, 1, 2, RQ_EPI_GLU, gate->rows, x, sk, st, tokens, 0, yn, yt, act_mode, ctx->act_scratch, 0, nullptr, s);
    if (rc == RQ_ERR_UNSUPPORTED) return rq_fail(RQ_ERR_LIMIT, "rq_matvec_glu: %lld inputs per row are beyond what the streaming kernel holds for two sub-rows", (long long)gate->cols);
    return rc;
}
