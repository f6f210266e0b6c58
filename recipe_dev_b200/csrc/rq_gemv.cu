// Batch-1 (and few-token) quantised matrix-vector kernels and the int8 activation quantiser.
//
// The matvec is bound by HBM: every weight byte is read once with 128-bit loads, the
// activation column sits in shared memory (fp32 for FLOAT, int8 records for INT8), nibbles
// and 6-bit codes unpack in registers and a row's partial sums meet by warp shuffles.
//
// Work decomposition: an ITEM is one 16-byte line of quantised codes of one row
//   Q4_K : line c of block b  -> 16 values of sub-block 2p (low nibbles) + 16 of 2p+1 (high)
//   Q6_K : ql line c of block b (+ its qh line) -> 16 values of group g and 16 of group g+2
//   Q8_0 : 16 codes            Q4_0 : one block (16 low + 16 high nibbles)
// LPR lanes share a row group and stride over its items; each group carries R rows at once
// so the activations a lane reads from shared memory serve R rows; T tokens ride along.
#include <string.h>

#include "rq_actquant.cuh"
#include "rq_internal.cuh"

namespace {

constexpr int kThreads = 256;

struct GemvParams {
    const uint8_t* main;
    const uint16_t* scale;
    int64_t rows, cols;
    const float* x; int64_t sk, st;      // FLOAT: activations in global memory, element strides
    const uint8_t* act;                  // INT8: per-token scratch (codes | d | sum16)
    float* y; int64_t yn, yt;
    int tokens;
};

__device__ __forceinline__ uint4 ldg128(const void* p) { return __ldg((const uint4*)p); }

// Four unsigned bytes of `w` as floats, exactly: 0x4B0000bb is 2^23 + bb.
__device__ __forceinline__ void bytes_to_float(uint32_t w, float* f) {
    f[0] = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7650)) - 8388608.0f;
    f[1] = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7651)) - 8388608.0f;
    f[2] = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7652)) - 8388608.0f;
    f[3] = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7653)) - 8388608.0f;
}

// sum_i f(byte i of w[0..3]) * x[i], i < 16, bytes unsigned
__device__ __forceinline__ float dot16_u8(const uint32_t* w, const float* x) {
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float f[4];
        bytes_to_float(w[j], f);
        s0 = fmaf(f[0], x[4 * j + 0], s0);
        s1 = fmaf(f[1], x[4 * j + 1], s1);
        s0 = fmaf(f[2], x[4 * j + 2], s0);
        s1 = fmaf(f[3], x[4 * j + 3], s1);
    }
    return s0 + s1;
}

__device__ __forceinline__ int dot16_i8(const uint32_t* w, const uint32_t* a) {
    int s = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) s = __dp4a((int)w[j], (int)a[j], s);
    return s;
}

template <int TYPE> __host__ __device__ constexpr int item_values() { return TYPE == RQ_Q8_0 ? 16 : 32; }

// One item of one row against T tokens. xs / codes are the shared-memory activations.
template <int TYPE, int MODE, int T>
struct Item {
    // FLOAT shared layout per token: x[cols] fp32 | xsum16[cols/16] fp32
    // INT8  shared layout per token: codes[cols] int8 | d[cols/32] fp32 | sum16[cols/16] int16
    __device__ __forceinline__ static void run(const GemvParams& p, int64_t row, int item, const uint8_t* smem, size_t tok_bytes, float* acc) {
        const int64_t cols = p.cols;
        if (TYPE == RQ_Q4_K) {
            const int b = item >> 3, c = item & 7, pr = c >> 1, h = c & 1;
            const uint8_t* blk = p.main + (row * (cols >> 8) + b) * 144;
            uint4 hdr = ldg128(blk);
            uint4 qs = ldg128(blk + 16 + 16 * c);
            int sc_lo, mn_lo, sc_hi, mn_hi;
            rq_q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * pr, sc_lo, mn_lo);
            rq_q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * pr + 1, sc_hi, mn_hi);
            const float d = rq_h2f((uint16_t)(hdr.x & 0xffff)), dmin = rq_h2f((uint16_t)(hdr.x >> 16));
            const float dsl = d * (float)sc_lo, dml = dmin * (float)mn_lo, dsh = d * (float)sc_hi, dmh = dmin * (float)mn_hi;
            const int k_lo = (b << 8) + 64 * pr + 16 * h, k_hi = k_lo + 32;
            uint32_t w[4] = {qs.x, qs.y, qs.z, qs.w}, lo[4], hi[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) { lo[j] = w[j] & 0x0F0F0F0Fu; hi[j] = (w[j] >> 4) & 0x0F0F0F0Fu; }
#pragma unroll
            for (int t = 0; t < T; ++t) {
                const uint8_t* tok = smem + t * tok_bytes;
                if (MODE == RQ_ACT_FLOAT) {
                    const float* xs = (const float*)tok;
                    const float* xsum = xs + cols;
                    float xl[16], xh[16];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        *(float4*)(xl + 4 * j) = *(const float4*)(xs + k_lo + 4 * j);
                        *(float4*)(xh + 4 * j) = *(const float4*)(xs + k_hi + 4 * j);
                    }
                    float dl = dot16_u8(lo, xl), dh = dot16_u8(hi, xh);
                    acc[t] += (dsl * dl - dml * xsum[k_lo >> 4]) + (dsh * dh - dmh * xsum[k_hi >> 4]);
                } else {
                    const uint8_t* codes = tok;
                    const float* d8 = (const float*)(tok + cols);
                    const int16_t* s16 = (const int16_t*)(tok + cols + (cols >> 5) * 4);
                    uint4 al = *(const uint4*)(codes + k_lo), ah = *(const uint4*)(codes + k_hi);
                    uint32_t a_lo[4] = {al.x, al.y, al.z, al.w}, a_hi[4] = {ah.x, ah.y, ah.z, ah.w};
                    int dl = dot16_i8(lo, a_lo), dh = dot16_i8(hi, a_hi);
                    float vl = dsl * (float)dl - dml * (float)s16[k_lo >> 4];
                    float vh = dsh * (float)dh - dmh * (float)s16[k_hi >> 4];
                    acc[t] += d8[k_lo >> 5] * vl + d8[k_hi >> 5] * vh;
                }
            }
        } else if (TYPE == RQ_Q6_K) {
            const int b = item >> 3, c = item & 7, ch = c >> 2, gl = (c >> 1) & 1, wh = c & 1;
            const int64_t nb = cols >> 8;
            const uint8_t* body = p.main + (row * nb + b) * 208;
            uint4 ql = ldg128(body + 64 * ch + 32 * gl + 16 * wh);
            uint4 qh = ldg128(body + 128 + 32 * ch + 16 * wh);
            const int sc_lo = (int8_t)__ldg(body + 192 + 8 * ch + 2 * gl + wh);
            const int sc_hi = (int8_t)__ldg(body + 192 + 8 * ch + 2 * (gl + 2) + wh);
            const float d = rq_h2f(__ldg(p.scale + row * nb + b));
            const int k_lo = (b << 8) + 128 * ch + 32 * gl + 16 * wh, k_hi = k_lo + 64;
            uint32_t l[4] = {ql.x, ql.y, ql.z, ql.w}, hq[4] = {qh.x, qh.y, qh.z, qh.w}, lo[4], hi[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                lo[j] = (l[j] & 0x0F0F0F0Fu) | (((hq[j] >> (2 * gl)) & 0x03030303u) << 4);
                hi[j] = ((l[j] >> 4) & 0x0F0F0F0Fu) | (((hq[j] >> (2 * gl + 4)) & 0x03030303u) << 4);
            }
#pragma unroll
            for (int t = 0; t < T; ++t) {
                const uint8_t* tok = smem + t * tok_bytes;
                if (MODE == RQ_ACT_FLOAT) {
                    const float* xs = (const float*)tok;
                    const float* xsum = xs + cols;
                    float xl[16], xh[16];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        *(float4*)(xl + 4 * j) = *(const float4*)(xs + k_lo + 4 * j);
                        *(float4*)(xh + 4 * j) = *(const float4*)(xs + k_hi + 4 * j);
                    }
                    float dl = dot16_u8(lo, xl) - 32.0f * xsum[k_lo >> 4];
                    float dh = dot16_u8(hi, xh) - 32.0f * xsum[k_hi >> 4];
                    acc[t] += d * ((float)sc_lo * dl + (float)sc_hi * dh);
                } else {
                    const uint8_t* codes = tok;
                    const float* d8 = (const float*)(tok + cols);
                    const int16_t* s16 = (const int16_t*)(tok + cols + (cols >> 5) * 4);
                    uint4 al = *(const uint4*)(codes + k_lo), ah = *(const uint4*)(codes + k_hi);
                    uint32_t a_lo[4] = {al.x, al.y, al.z, al.w}, a_hi[4] = {ah.x, ah.y, ah.z, ah.w};
                    int dl = dot16_i8(lo, a_lo) - 32 * (int)s16[k_lo >> 4];
                    int dh = dot16_i8(hi, a_hi) - 32 * (int)s16[k_hi >> 4];
                    acc[t] += d * (d8[k_lo >> 5] * (float)(sc_lo * dl) + d8[k_hi >> 5] * (float)(sc_hi * dh));
                }
            }
        } else if (TYPE == RQ_Q8_0) {
            uint4 q = ldg128(p.main + row * cols + 16 * (rq_plane_permuted(TYPE, cols) ? rq_plane_chunk(TYPE, item) : (int64_t)item));
            const float d = rq_h2f(__ldg(p.scale + row * (cols >> 5) + (item >> 1)));
            const int k0 = 16 * item;
            uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int t = 0; t < T; ++t) {
                const uint8_t* tok = smem + t * tok_bytes;
                if (MODE == RQ_ACT_FLOAT) {
                    const float* xs = (const float*)tok;
                    const float* xsum = xs + cols;
                    float xv[16];
                    uint32_t u[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) { *(float4*)(xv + 4 * j) = *(const float4*)(xs + k0 + 4 * j); u[j] = w[j] ^ 0x80808080u; }
                    // codes biased by 128 to unsigned bytes; the bias leaves through the slice's sum of x
                    acc[t] += d * (dot16_u8(u, xv) - 128.0f * xsum[k0 >> 4]);
                } else {
                    const uint8_t* codes = tok;
                    const float* d8 = (const float*)(tok + cols);
                    uint4 av = *(const uint4*)(codes + k0);
                    uint32_t a[4] = {av.x, av.y, av.z, av.w};
                    acc[t] += d8[k0 >> 5] * (d * (float)dot16_i8(w, a));
                }
            }
        } else {  // Q4_0
            uint4 q = ldg128(p.main + row * (cols >> 1) + 16 * (rq_plane_permuted(TYPE, cols) ? rq_plane_chunk(TYPE, item) : (int64_t)item));
            const float d = rq_h2f(__ldg(p.scale + row * (cols >> 5) + item));
            const int k_lo = 32 * item, k_hi = k_lo + 16;
            uint32_t w[4] = {q.x, q.y, q.z, q.w}, lo[4], hi[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) { lo[j] = w[j] & 0x0F0F0F0Fu; hi[j] = (w[j] >> 4) & 0x0F0F0F0Fu; }
#pragma unroll
            for (int t = 0; t < T; ++t) {
                const uint8_t* tok = smem + t * tok_bytes;
                if (MODE == RQ_ACT_FLOAT) {
                    const float* xs = (const float*)tok;
                    const float* xsum = xs + cols;
                    float xl[16], xh[16];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        *(float4*)(xl + 4 * j) = *(const float4*)(xs + k_lo + 4 * j);
                        *(float4*)(xh + 4 * j) = *(const float4*)(xs + k_hi + 4 * j);
                    }
                    float dot = dot16_u8(lo, xl) + dot16_u8(hi, xh);
                    acc[t] += d * (dot - 8.0f * (xsum[k_lo >> 4] + xsum[k_hi >> 4]));
                } else {
                    const uint8_t* codes = tok;
                    const float* d8 = (const float*)(tok + cols);
                    const int16_t* s16 = (const int16_t*)(tok + cols + (cols >> 5) * 4);
                    uint4 al = *(const uint4*)(codes + k_lo), ah = *(const uint4*)(codes + k_hi);
                    uint32_t a_lo[4] = {al.x, al.y, al.z, al.w}, a_hi[4] = {ah.x, ah.y, ah.z, ah.w};
                    int dot = dot16_i8(lo, a_lo) + dot16_i8(hi, a_hi) - 8 * ((int)s16[k_lo >> 4] + (int)s16[k_hi >> 4]);
                    acc[t] += d8[k_lo >> 5] * (d * (float)dot);
                }
            }
        }
    }
};

template <int TYPE, int MODE, int LPR, int R, int T>
__global__ void __launch_bounds__(kThreads) rq_gemv_kernel(GemvParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int64_t cols = p.cols;
    // every token's activations start on a 16-byte boundary: the rows read them with 128-bit loads
    const size_t tok_bytes = MODE == RQ_ACT_FLOAT ? (((size_t)(cols + (cols >> 4)) * 4 + 15) & ~(size_t)15) : ((rq_act_token_bytes(cols) + 15) & ~(size_t)15);
    const int tok0 = blockIdx.y * T;

    // ---- stage the activations of this CTA's tokens -------------------------------------
    if (MODE == RQ_ACT_FLOAT) {
        for (int t = 0; t < T; ++t) {
            float* xs = (float*)(smem + t * tok_bytes);
            const bool live = tok0 + t < p.tokens;
            const float* src = p.x + (int64_t)(live ? tok0 + t : tok0) * p.st;
            for (int64_t k = threadIdx.x; k < cols; k += kThreads) xs[k] = live ? __ldg(src + k * p.sk) : 0.0f;
        }
        __syncthreads();
        for (int t = 0; t < T; ++t) {
            float* xs = (float*)(smem + t * tok_bytes);
            float* xsum = xs + cols;
            for (int64_t s = threadIdx.x; s < (cols >> 4); s += kThreads) {
                float a = 0.f;
#pragma unroll
                for (int i = 0; i < 16; ++i) a += xs[16 * s + i];
                xsum[s] = a;
            }
        }
    } else {
        const size_t src_bytes = rq_act_token_bytes(cols);
        for (int t = 0; t < T; ++t) {
            const bool live = tok0 + t < p.tokens;
            const uint32_t* src = (const uint32_t*)(p.act + (size_t)(live ? tok0 + t : tok0) * src_bytes);
            uint32_t* dst = (uint32_t*)(smem + t * tok_bytes);
            // token scratch is a whole number of 4-byte words: cols is a multiple of 32
            for (size_t i = threadIdx.x; i < src_bytes / 4; i += kThreads) dst[i] = live ? __ldg(src + i) : 0u;
        }
    }
    __syncthreads();

    // ---- rows ---------------------------------------------------------------------------
    constexpr int GROUPS = kThreads / LPR;
    const int group = threadIdx.x / LPR, lane = threadIdx.x % LPR;
    const int items = (int)(cols / item_values<TYPE>());
    const int64_t row0 = ((int64_t)blockIdx.x * GROUPS + group) * R;
    float acc[R][T];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int t = 0; t < T; ++t) acc[r][t] = 0.f;

    if (row0 < p.rows) {
        for (int item = lane; item < items; item += LPR) {
#pragma unroll
            for (int r = 0; r < R; ++r) {
                int64_t row = row0 + r < p.rows ? row0 + r : p.rows - 1;  // clamped rows are computed and dropped
                Item<TYPE, MODE, T>::run(p, row, item, smem, tok_bytes, acc[r]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int t = 0; t < T; ++t) {
            float v = acc[r][t];
#pragma unroll
            for (int off = LPR / 2; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
            if (lane == 0 && row0 + r < p.rows && tok0 + t < p.tokens) p.y[(row0 + r) * p.yn + (int64_t)(tok0 + t) * p.yt] = v;
        }
}

// ---------------------------------------------------------------------------------------
// int8 activation quantiser: one warp per group of `step` inputs of one token.
// The extreme is the FIRST input of strictly largest magnitude, signed; inverse = -127/extreme
// and d = 1/inverse are IEEE fp32 divides; code = clamp(rint(x * inverse)).
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) rq_act_quant_kernel(const float* __restrict__ x, int64_t sk, int64_t st, int64_t cols, int tokens,
                                                               int step, uint8_t* __restrict__ scratch, uint8_t* __restrict__ records36) {
    // Programmatic dependent launch: the matvec behind this kernel may start streaming its weights
    // now; x may come from the kernel before this one, so wait for that one before reading it.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int span_shift = step == 256 ? 3 : 0;  // 32-value records per group: 8 or 1
    const int64_t recs = cols >> 5, groups = (recs + (1 << span_shift) - 1) >> span_shift;
    const int64_t g = (int64_t)blockIdx.x * (kThreads / 32) + warp;
    const int t = blockIdx.y;
    if (g >= groups || t >= tokens) return;
    const float* xt = x + (int64_t)t * st;
    uint8_t* tok = scratch + (size_t)t * rq_act_token_bytes(cols);
    const bool unit_layout = rq_act_unit_layout(cols);
    uint8_t* r36 = records36 ? records36 + (size_t)t * recs * 36 : nullptr;
    asm volatile("griddepcontrol.wait;" ::: "memory");  // after the index arithmetic: the wait is where the chain of launches passes through
    rq_quantise_group(xt, sk, cols, step, g, lane, tok, unit_layout, r36);
}

// The same for the common call -- groups of 32 contiguous inputs into unit records, no copy in the reference's record
// format -- as a short straight line of code: the kernel sits in the chain of a decode layer's launches (between gate/up and
// down), runs once per layer on an instruction cache that other kernels have filled, and what it costs there is the length of
// its instruction stream and its one trip to L2, not its arithmetic. Same operations in the same order as rq_quantise_group.
__global__ void __launch_bounds__(kThreads) rq_act_quant32_kernel(const float* __restrict__ x, int64_t st, int units, uint8_t* __restrict__ scratch) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int lane = threadIdx.x & 31;
    const int rec = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);  // 32-value record = group
    if (rec >= units * 8) return;
    const float* src = x + (int64_t)blockIdx.y * st + rec * 32 + lane;
    uint8_t* unit = scratch + ((size_t)blockIdx.y * units + (rec >> 3)) * RQ_ACT_RECORD_INT8;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const float v = __ldg(src);
    const unsigned key = __float_as_uint(fabsf(v)) <= 0x7f800000u ? __float_as_uint(fabsf(v)) : 0u;  // a NaN is never the extreme
    const unsigned top = __reduce_max_sync(0xffffffffu, key);
    const unsigned first = __reduce_min_sync(0xffffffffu, key == top && top != 0u ? (unsigned)lane : 0xffffffffu);
    const float best = first == 0xffffffffu ? 0.f : __shfl_sync(0xffffffffu, v, (int)(first & 31u));
    const bool nonzero = fabsf(best) > 0.f;
    const float inverse = nonzero ? __fdiv_rn(-127.0f, best) : 0.f;
    const float d = nonzero ? __fdiv_rn(1.0f, inverse) : 0.f;
    int code = __float2int_rn(__fmul_rn(v, inverse));
    code = code < -128 ? -128 : (code > 127 ? 127 : code);
    ((int8_t*)unit)[32 * (rec & 7) + lane] = (int8_t)code;
    const int s = __reduce_add_sync(lane < 16 ? 0x0000ffffu : 0xffff0000u, code);
    const int gs = s + __shfl_xor_sync(0xffffffffu, s, 16);
    if ((lane & 15) == 0) ((int16_t*)(unit + 288))[2 * (rec & 7) + (lane >> 4)] = (int16_t)s;
    if (lane == 0) {
        ((float*)(unit + 256))[rec & 7] = d;
        ((int16_t*)(unit + 320))[rec & 7] = (int16_t)gs;
    }
}

template <int TYPE, int MODE, int LPR, int R, int T>
int launch_one(const GemvParams& p, size_t smem_bytes, cudaStream_t s) {
    auto kernel = rq_gemv_kernel<TYPE, MODE, LPR, R, T>;
    if (smem_bytes > 48 * 1024) RQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes));
    constexpr int rows_per_cta = (kThreads / LPR) * R;
    dim3 grid((unsigned)((p.rows + rows_per_cta - 1) / rows_per_cta), (unsigned)((p.tokens + T - 1) / T));
    kernel<<<grid, kThreads, smem_bytes, s>>>(p);
    RQ_CUDA(cudaGetLastError());
    return RQ_OK;
}

template <int TYPE, int MODE, int LPR, int T>
int launch_r(const GemvParams& p, size_t smem, int r, cudaStream_t s) {
    switch (r) {
        case 4: return launch_one<TYPE, MODE, LPR, 4, T>(p, smem, s);
        case 2: return launch_one<TYPE, MODE, LPR, 2, T>(p, smem, s);
        default: return launch_one<TYPE, MODE, LPR, 1, T>(p, smem, s);
    }
}

template <int TYPE, int MODE>
int launch_tm(const GemvParams& p, int sm_count, cudaStream_t s) {
    const int items = (int)(p.cols / item_values<TYPE>());
    const int lpr = items % 32 == 0 ? 32 : 8;
    const size_t tok = MODE == RQ_ACT_FLOAT ? (((size_t)(p.cols + (p.cols >> 4)) * 4 + 15) & ~(size_t)15) : ((rq_act_token_bytes(p.cols) + 15) & ~(size_t)15);
    const size_t limit = 200 * 1024;
    if (tok > limit) return rq_fail(RQ_ERR_LIMIT, "matvec: %lld inputs per row exceed the %zu bytes of shared memory one token may take", (long long)p.cols, limit);
    const int t = (p.tokens >= 2 && 4 * tok <= limit) ? 4 : 1;
    // rows per group: as many as keep at least ~2 CTAs per SM in flight
    const int groups = kThreads / lpr;
    int r = 4;
    while (r > 1 && (p.rows + (int64_t)groups * r - 1) / ((int64_t)groups * r) < 2 * (int64_t)sm_count) r >>= 1;
    const size_t smem = tok * t;
    if (lpr == 32) return t == 4 ? launch_r<TYPE, MODE, 32, 4>(p, smem, r, s) : launch_r<TYPE, MODE, 32, 1>(p, smem, r, s);
    return t == 4 ? launch_r<TYPE, MODE, 8, 4>(p, smem, r, s) : launch_r<TYPE, MODE, 8, 1>(p, smem, r, s);
}

template <int TYPE>
int launch_t(const GemvParams& p, int mode, int sm_count, cudaStream_t s) {
    return mode == RQ_ACT_FLOAT ? launch_tm<TYPE, RQ_ACT_FLOAT>(p, sm_count, s) : launch_tm<TYPE, RQ_ACT_INT8>(p, sm_count, s);
}

}  // namespace

int rq_launch_act_quant(const float* x, int64_t sk, int64_t st, int64_t cols, int tokens, int step,
                        uint8_t* scratch, uint8_t* records36, cudaStream_t s) {
    const int span = step / 32;
    const int64_t recs = cols / 32, groups = (recs + span - 1) / span;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((groups + kThreads / 32 - 1) / (kThreads / 32)), (unsigned)tokens);
    cfg.blockDim = dim3(kThreads);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (step == 32 && sk == 1 && records36 == nullptr && rq_act_unit_layout(cols) && cols <= ((int64_t)1 << 30)) {
        RQ_CUDA(cudaLaunchKernelEx(&cfg, rq_act_quant32_kernel, x, st, (int)(cols >> 8), scratch));
        return RQ_OK;
    }
    RQ_CUDA(cudaLaunchKernelEx(&cfg, rq_act_quant_kernel, x, sk, st, cols, tokens, step, scratch, records36));
    return RQ_OK;
}

// INT8 activations reach a matvec through the context's scratch: RQ_ACT_INT8 runs the quantiser
// kernel, RQ_ACT_INT8_CACHED reuses what the previous INT8 call left there. The quantiser and the
// matvec are both launched with programmatic stream serialization: the matvec's producer warp
// streams weights while the quantiser is still running, and only its consumers wait for it.
static int int8_records(rq_ctx* ctx, const char* who, const float* x, int64_t sk, int64_t st, int64_t cols, int tokens, int step, int act_mode,
                        cudaStream_t s) {
    if (act_mode == RQ_ACT_INT8) {
        int rc = rq_ensure_act_scratch(ctx, rq_act_token_bytes(cols) * (size_t)tokens, s);
        if (rc) return rc;
        rc = rq_launch_act_quant(x, sk, st, cols, tokens, step, ctx->act_scratch, nullptr, s);
        if (rc) return rc;
        ctx->act_cols = cols; ctx->act_tokens = tokens; ctx->act_step = step;
    } else if (act_mode == RQ_ACT_INT8_CACHED) {
        int rc = rq_order_work_areas(ctx, s);  // the records may have been written on another stream
        if (rc) return rc;
        if (ctx->act_cols != cols || ctx->act_tokens != tokens || ctx->act_step != step)
            return rq_fail(RQ_ERR_INVALID, "%s: no cached int8 records for %lld inputs x %d tokens at step %d (held: %lld x %d at %d)", who,
                           (long long)cols, tokens, step, (long long)ctx->act_cols, ctx->act_tokens, ctx->act_step);
    }
    return RQ_OK;
}

// A single-token INT8 call over whole 256-value units can quantise inside the matvec launch. True when
// that is to be tried (the scratch is then large enough for the records the launch leaves behind);
// *rc carries an allocation failure.
static bool fused_int8(rq_ctx* ctx, int act_mode, int tokens, int64_t cols, int* rc, cudaStream_t s) {
    *rc = RQ_OK;
    // Every CTA of a fused launch reads all of x: beyond 8192 inputs that traffic (some 300 CTAs x 4 bytes x inputs)
    // costs more than the quantiser launch it saves.
    if (act_mode != RQ_ACT_INT8 || tokens != 1 || cols % 256 || cols > 8192) return false;
    *rc = rq_ensure_act_scratch(ctx, rq_act_token_bytes(cols), s);
    return *rc == RQ_OK;
}

// Several matrices of one format and width against the same activations, as one launch when the
// streaming kernel serves the shape (one segment per matrix), else one launch per matrix.
int rq_launch_gemv_multi(rq_ctx* ctx, int n, const rq_weight* const* ws, const float* x, int64_t sk, int64_t st, int tokens,
                         float* const* ys, int64_t yn, int64_t yt, int act_mode, int step, cudaStream_t s) {
    const rq_weight* w0 = ws[0];
    const int mode = act_mode == RQ_ACT_FLOAT ? RQ_ACT_FLOAT : RQ_ACT_INT8;
    int rc;
    if (!rq_type_has_fast_path(w0->type)) {
        for (int i = 0; i < n; ++i) {
            rc = rq_launch_gemv(ctx, ws[i], x, sk, st, tokens, ys[i], yn, yt, act_mode, step, s);
            if (rc) return rc;
        }
        return RQ_OK;
    }
    RqSegment seg[RQ_INLINE_SEGMENTS];
    int64_t total = 0;
    if (n <= RQ_INLINE_SEGMENTS) {
        memset(seg, 0, sizeof(seg));
        for (int i = 0; i < n; ++i) {
            seg[i].row_begin = (int)total; seg[i].rows = (int)ws[i]->rows; seg[i].y = ys[i];
            seg[i].main[0] = ws[i]->main; seg[i].scale[0] = ws[i]->scale; seg[i].act[0] = 0; seg[i].coef[0] = 1.0f;
            total += ws[i]->rows;
        }
        if (fused_int8(ctx, act_mode, tokens, w0->cols, &rc, s)) {
            // one launch: the matvec quantises x in its prologue
            rc = rq_launch_stream(ctx, w0->type, w0->cols, nullptr, seg, n, 1, RQ_EPI_PLAIN, total, x, sk, st, tokens, 0, yn, yt, mode, ctx->act_scratch, step,
                                  ctx->act_scratch, s);
            if (rc == RQ_OK) { ctx->act_cols = w0->cols; ctx->act_tokens = tokens; ctx->act_step = step; }
            if (rc != RQ_ERR_UNSUPPORTED) return rc;
        } else if (rc) {
            return rc;
        }
    }
    rc = int8_records(ctx, "matvec_multi", x, sk, st, w0->cols, tokens, step, act_mode, s);
    if (rc) return rc;
    if (n <= RQ_INLINE_SEGMENTS) {
        rc = rq_launch_stream(ctx, w0->type, w0->cols, nullptr, seg, n, 1, RQ_EPI_PLAIN, total, x, sk, st, tokens, 0, yn, yt, mode, ctx->act_scratch, 0, nullptr, s);
        if (rc != RQ_ERR_UNSUPPORTED) return rc;
    }
    for (int i = 0; i < n; ++i) {
        rc = rq_launch_gemv(ctx, ws[i], x, sk, st, tokens, ys[i], yn, yt, mode == RQ_ACT_INT8 ? RQ_ACT_INT8_CACHED : mode, step, s);
        if (rc) return rc;
    }
    return RQ_OK;
}

int rq_launch_gemv(rq_ctx* ctx, const rq_weight* w, const float* x, int64_t sk, int64_t st, int tokens,
                   float* y, int64_t yn, int64_t yt, int act_mode, int step, cudaStream_t s) {
    const int mode = act_mode == RQ_ACT_FLOAT ? RQ_ACT_FLOAT : RQ_ACT_INT8;
    int rc;
    if (!rq_type_has_fast_path(w->type)) {
        // the other stored formats: run decoders over fp32 activations; int sums never see them (recipe.rs:22345-22369)
        if (mode != RQ_ACT_FLOAT && w->type == RQ_Q4_1) {
            // `.int(4)`: Q4_1 is the storage of int4 sums (recipe.rs:22348) and has an int8 dot of its own
            rc = int8_records(ctx, "matvec", x, sk, st, w->cols, tokens, step, act_mode, s);
            if (rc) return rc;
            return rq_launch_gemv_q41_int8(ctx, w, ctx->act_scratch, tokens, y, yn, yt, s);
        }
        if (mode != RQ_ACT_FLOAT)
            return rq_fail(RQ_ERR_UNSUPPORTED, "matvec: int8 activations over a type-%d weight; `.int(8)` re-encodes such a tensor to Q8_0 at load: call rq_weight_requantize(.., RQ_Q8_0, ..) and use the result", w->type);
        return rq_launch_gemv_generic(ctx, w, x, sk, st, tokens, y, yn, yt, s);
    }
    if (fused_int8(ctx, act_mode, tokens, w->cols, &rc, s)) {
        // one launch: the matvec quantises x in its prologue
        rc = rq_launch_gemv_stream(ctx, w, x, sk, st, tokens, y, yn, yt, mode, ctx->act_scratch, step, ctx->act_scratch, s);
        if (rc == RQ_OK) { ctx->act_cols = w->cols; ctx->act_tokens = tokens; ctx->act_step = step; }
        if (rc != RQ_ERR_UNSUPPORTED) return rc;
    } else if (rc) {
        return rc;
    }
    rc = int8_records(ctx, "matvec", x, sk, st, w->cols, tokens, step, act_mode, s);
    if (rc) return rc;
    rc = rq_launch_gemv_stream(ctx, w, x, sk, st, tokens, y, yn, yt, mode, ctx->act_scratch, 0, nullptr, s);
    if (rc != RQ_ERR_UNSUPPORTED) return rc;
    if (rq_act_unit_layout(w->cols) && mode == RQ_ACT_INT8)
        return rq_fail(RQ_ERR_LIMIT, "matvec: %lld inputs per row exceed what one CTA's shared memory holds", (long long)w->cols);
    GemvParams p;
    p.main = w->main; p.scale = w->scale; p.rows = w->rows; p.cols = w->cols;
    p.x = x; p.sk = sk; p.st = st; p.act = mode == RQ_ACT_INT8 ? ctx->act_scratch : nullptr;
    p.y = y; p.yn = yn; p.yt = yt; p.tokens = tokens;
    switch (w->type) {
        case RQ_Q4_K: return launch_t<RQ_Q4_K>(p, mode, ctx->sm_count, s);
        case RQ_Q6_K: return launch_t<RQ_Q6_K>(p, mode, ctx->sm_count, s);
        case RQ_Q8_0: return launch_t<RQ_Q8_0>(p, mode, ctx->sm_count, s);
        case RQ_Q4_0: return launch_t<RQ_Q4_0>(p, mode, ctx->sm_count, s);
        default: return rq_fail(RQ_ERR_INVALID, "matvec: type %d", w->type);
    }
}

// The tiled kernel over int8 records the caller already holds at `act` (plane layout).
int rq_launch_gemv_tiled_int8(rq_ctx* ctx, const rq_weight* w, int tokens, float* y, int64_t yn, int64_t yt, const uint8_t* act, cudaStream_t s) {
    if (rq_act_unit_layout(w->cols))
        return rq_fail(RQ_ERR_LIMIT, "matvec: %lld inputs per row exceed what one CTA's shared memory holds", (long long)w->cols);
    GemvParams p;
    p.main = w->main; p.scale = w->scale; p.rows = w->rows; p.cols = w->cols;
    p.x = nullptr; p.sk = 1; p.st = w->cols; p.act = act;
    p.y = y; p.yn = yn; p.yt = yt; p.tokens = tokens;
    switch (w->type) {
        case RQ_Q4_K: return launch_t<RQ_Q4_K>(p, RQ_ACT_INT8, ctx->sm_count, s);
        case RQ_Q6_K: return launch_t<RQ_Q6_K>(p, RQ_ACT_INT8, ctx->sm_count, s);
        case RQ_Q8_0: return launch_t<RQ_Q8_0>(p, RQ_ACT_INT8, ctx->sm_count, s);
        case RQ_Q4_0: return launch_t<RQ_Q4_0>(p, RQ_ACT_INT8, ctx->sm_count, s);
        default: return rq_fail(RQ_ERR_INVALID, "matvec: type %d", w->type);
    }
}
