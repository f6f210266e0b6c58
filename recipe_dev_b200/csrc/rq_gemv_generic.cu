// Matrix-vector product over the stored formats that have no streaming kernel of their own (Q4_1, Q5_0, Q5_1, Q5_K,
// IQ4_NL, Q8_1, Q2_K, Q3_K, Q8_K, IQ4_XS): fp32 activations against per-value decoded weights, the reference's run
// decoders (recipe.rs:7826-7917: one fused-multiply-add chain per unit of 32 values in index order; the units of a row
// add up, ll:3451-3492; here the additions are regrouped, within the 1e-3 band). A warp owns a row and walks it in units
// of 32 values, lane l taking value l of every unit, so that a unit's activations are one coalesced line and its weight
// bytes one block; the lanes' sums meet in a fixed xor tree, so every run gives the same bits. `.int(8)` never reaches
// these formats: the reference re-encodes them to Q8_0 at load (rq_weight_requantize), and that weight takes the
// streaming kernel. `.int(4)` stores Q4_1 and dots it with int8 activation records: rq_gemv_q41_int8_kernel below.
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
        // lane l takes value l of every unit: the warp's activation loads are one line, its weight bytes one block
        float sum = 0.f;
        const int64_t first = row * cols + lane;
#pragma unroll 4
        for (int64_t u = 0; u < units; ++u) sum = fmaf(rq_decode_value<TYPE>(main_plane, nullptr, first + (u << 5), cols), __ldg(xt + ((u << 5) + lane) * sk), sum);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
        if (lane == 0) y[row * yn + (int64_t)token * yt] = sum;
    }
}

// `.int(4)`: int8 activation records against Q4_1 blocks (block32 slice kind 3, build.rs:777-796). Per 16-value slice
// r = q8_d * (d * f32(dot) + m * f32(sum of the slice's activation codes)); slice 0 takes the low nibbles, slice 1 the high
// ones. A warp owns a row, lane l the blocks l, l + 32, ..; dots by dp4a over the nibbles in place; fixed xor tree.
__global__ void __launch_bounds__(kWarps * 32) rq_gemv_q41_int8_kernel(const uint8_t* __restrict__ blocks, int64_t rows, int64_t cols, const uint8_t* __restrict__ records,
                                                                         size_t token_bytes, float* __restrict__ y, int64_t yn, int64_t yt) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, token = blockIdx.y;
    const uint8_t* tok = records + (size_t)token * token_bytes;
    const bool unit = rq_act_unit_layout(cols);
    const int64_t nb = cols >> 5;
    // Programmatic dependent launch: the records come from the quantiser launched before this kernel; the weights are
    // constants of the model, so the first round's weight loads go out before the wait for that kernel.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    bool records_ready = false;
    for (int64_t row = (int64_t)blockIdx.x * kWarps + warp; row < rows; row += (int64_t)gridDim.x * kWarps) {
        float sum = 0.f;
        // four blocks per lane and round, their twenty weight words loaded before the first is used: the row is read once,
        // from HBM, and a round trip per block would leave the warp waiting on latency
        for (int64_t b0 = 0; b0 < nb; b0 += 128) {
            uint32_t wq[4][5];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int64_t b = b0 + 32 * i + lane;
                const uint32_t* blk = (const uint32_t*)(blocks + (row * nb + (b < nb ? b : nb - 1)) * 20);  // 20-byte stride from a 256-byte aligned base: words are aligned
#pragma unroll
                for (int w = 0; w < 5; ++w) wq[i][w] = __ldcs(blk + w);
            }
            if (!records_ready) {
                asm volatile("griddepcontrol.wait;" ::: "memory");
                records_ready = true;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int64_t b = b0 + 32 * i + lane;
                if (b >= nb) break;
                const float d = rq_h2f((uint16_t)(wq[i][0] & 0xffff)), m = rq_h2f((uint16_t)(wq[i][0] >> 16));
                int cl[4], ch[4];
                float q8_d; uint32_t sums;
                if (unit) {
                    const uint8_t* rec = tok + (size_t)(b >> 3) * RQ_ACT_RECORD_INT8;  // records are 16-byte aligned
                    const uint4 lo = __ldg((const uint4*)(rec + 32 * (b & 7))), hi = __ldg((const uint4*)(rec + 32 * (b & 7)) + 1);
                    cl[0] = (int)lo.x; cl[1] = (int)lo.y; cl[2] = (int)lo.z; cl[3] = (int)lo.w;
                    ch[0] = (int)hi.x; ch[1] = (int)hi.y; ch[2] = (int)hi.z; ch[3] = (int)hi.w;
                    q8_d = ((const float*)(rec + 256))[b & 7];
                    sums = ((const uint32_t*)(rec + 288))[b & 7];
                } else {
                    const int* codes = (const int*)(tok + b * 32);  // a token's planes start on a multiple of 8 bytes
#pragma unroll
                    for (int w = 0; w < 4; ++w) { cl[w] = __ldg(codes + w); ch[w] = __ldg(codes + 4 + w); }
                    q8_d = ((const float*)(tok + cols))[b];
                    sums = ((const uint32_t*)(tok + cols + nb * 4))[b];
                }
                int dot_lo = 0, dot_hi = 0;
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const uint32_t q = wq[i][1 + w];
                    dot_lo = __dp4a((int)(q & 0x0F0F0F0Fu), cl[w], dot_lo);
                    dot_hi = __dp4a((int)((q >> 4) & 0x0F0F0F0Fu), ch[w], dot_hi);
                }
                const float r0 = __fmul_rn(q8_d, __fadd_rn(__fmul_rn(d, (float)dot_lo), __fmul_rn(m, (float)(int16_t)(sums & 0xffff))));
                const float r1 = __fmul_rn(q8_d, __fadd_rn(__fmul_rn(d, (float)dot_hi), __fmul_rn(m, (float)(int16_t)(sums >> 16))));
                sum += r0;
                sum += r1;
            }
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
#define RQ_CASE(T) case T: return launch_generic<T>(w, x, sk, st, tokens, y, yn, yt, ctx->sm_count, s);
        RQ_DECODE_ONLY_TYPES(RQ_CASE)
#undef RQ_CASE
        default: return rq_fail(RQ_ERR_INVALID, "matvec: type %d", w->type);
    }
}

int rq_launch_gemv_q41_int8(rq_ctx* ctx, const rq_weight* w, const uint8_t* records, int tokens, float* y, int64_t yn, int64_t yt, cudaStream_t s) {
    if (tokens > 65535) return rq_fail(RQ_ERR_LIMIT, "matvec: %d tokens over a Q4_1 weight, at most 65535 per call", tokens);
    const int64_t ctas = (w->rows + kWarps - 1) / kWarps;
    const int64_t cap = (int64_t)ctx->sm_count * 8;
    dim3 grid((unsigned)(ctas < cap ? ctas : cap), (unsigned)tokens);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kWarps * 32);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    RQ_CUDA(cudaLaunchKernelEx(&cfg, rq_gemv_q41_int8_kernel, (const uint8_t*)w->main, w->rows, w->cols, records, rq_act_token_bytes(w->cols), y, yn, yt));
    return RQ_OK;
}
