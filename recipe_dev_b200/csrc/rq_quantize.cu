// Weight quantisers on the device, byte-exact with the reference's Integer::compress
// (recipe.rs:16191-16242 Q8_0 / Q4_0, :16325-16375 Q4_K with qkx2 :15140-15162,
// :16376-16414 Q6_K with qx :15183-15203).
//
// The reference's searches are sequential fp32 loops whose sums depend on their order, so
// one thread owns one sub-block and walks it in index order; the block-level steps read the
// sub-block results from shared memory, again in index order. This file is compiled with
// --fmad=false: every multiply and add below rounds on its own, as the host code does.
#include "rq_internal.cuh"

namespace {

__device__ __forceinline__ float qround(float v) {
    float shifted = v + 12582912.0f;
    return (float)((__float_as_int(shifted) & 0x007fffff) - 0x00400000);
}
// Rust `as u8` / `as i8` on a float: truncate toward zero, saturate, NaN -> 0
__device__ __forceinline__ uint8_t sat_u8(float v) { return !(v > 0.0f) ? 0 : (v >= 255.0f ? 255 : (uint8_t)(int)v); }
__device__ __forceinline__ int sat_i8(float v) { return v != v ? 0 : (v <= -128.0f ? -128 : (v >= 127.0f ? 127 : (int)v)); }
__device__ __forceinline__ float fmax32(float a, float b) { return (b > a || a != a) ? b : a; }
__device__ __forceinline__ float fmin32(float a, float b) { return (b < a || a != a) ? b : a; }

// fp32 -> fp16 bits, recipe.rs:15098-15112 (round to nearest even; overflow to infinity)
__device__ uint16_t to_half_bits(float value) {
    uint32_t bits = __float_as_uint(value);
    uint32_t sign = (bits >> 16) & 0x8000u;
    int exponent = (int)((bits >> 23) & 0xffu) - 112;
    uint32_t mantissa = bits & 0x7fffffu;
    if (exponent <= 0) {
        if (exponent < -10) return (uint16_t)sign;
        uint32_t wide = (mantissa | 0x800000u) >> (1 - exponent);
        return (uint16_t)(sign | ((wide + 0xfffu + ((wide >> 13) & 1u)) >> 13));
    }
    if (exponent >= 31) return (uint16_t)(sign | 0x7c00u | (mantissa != 0 ? 1u : 0u));
    uint32_t rounded = mantissa + 0xfffu + ((mantissa >> 13) & 1u);
    if (rounded & 0x800000u) {
        int up = exponent + 1 > 31 ? 31 : exponent + 1;
        return (uint16_t)(sign | (uint32_t)(up << 10));
    }
    return (uint16_t)(sign | (uint32_t)(exponent << 10) | (rounded >> 13));
}

__device__ __forceinline__ void put_half(uint8_t* p, uint16_t h) { p[0] = (uint8_t)(h & 0xff); p[1] = (uint8_t)(h >> 8); }

// ---- Q8_0 / Q4_0: one thread per 32-value block -----------------------------------------
template <int TYPE>
__global__ void quant_block32_kernel(const float* __restrict__ values, int64_t blocks, uint8_t* __restrict__ out) {
    int64_t b = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (b >= blocks) return;
    const float* v = values + b * 32;
    float extreme = v[0];
    for (int i = 1; i < 32; ++i) if (fabsf(v[i]) >= fabsf(extreme)) extreme = v[i];  // the last of equal maxima
    float scale = TYPE == RQ_Q8_0 ? fabsf(extreme) / 127.0f : extreme / -8.0f;
    float inverse = scale == 0.0f ? 0.0f : 1.0f / scale;
    uint8_t* o = out + b * (TYPE == RQ_Q8_0 ? 34 : 18);
    put_half(o, to_half_bits(scale));
    if (TYPE == RQ_Q8_0) {
        for (int i = 0; i < 32; ++i) {
            float shifted = roundf(v[i] * inverse) + 128.0f;
            uint8_t code = sat_u8(fmin32(fmax32(shifted, 0.0f), 255.0f));
            o[2 + i] = (uint8_t)(code - 128u);
        }
    } else {
        for (int i = 0; i < 16; ++i) {
            float lo = v[i] * inverse + 8.0f + 0.5f, hi = v[i + 16] * inverse + 8.0f + 0.5f;
            uint8_t cl = sat_u8(fmin32(fmax32(lo, 0.0f), 15.0f)), ch = sat_u8(fmin32(fmax32(hi, 0.0f), 15.0f));
            o[2 + i] = (uint8_t)((cl & 15) | ((ch & 15) << 4));
        }
    }
}

// ---- Q4_K: eight threads per 256-value block, one per 32-value sub-block ---------------------
constexpr int kQ4Blocks = 16;  // blocks per CTA -> 128 threads

__global__ void __launch_bounds__(kQ4Blocks * 8) quant_q4k_kernel(const float* __restrict__ values, int64_t blocks, uint8_t* __restrict__ out) {
    __shared__ float s_scale[kQ4Blocks][8], s_min[kQ4Blocks][8];
    __shared__ uint8_t s_sc[kQ4Blocks][8], s_mc[kQ4Blocks][8];
    __shared__ uint8_t s_codes[kQ4Blocks][256];
    const int lb = threadIdx.x >> 3, sub = threadIdx.x & 7;
    const int64_t b = (int64_t)blockIdx.x * kQ4Blocks + lb;
    const bool live = b < blocks;
    float x[32], wts[32];
    uint8_t codes[32], trial[32];
    float scale = 0.0f, minimum = 0.0f;
    if (live) {
        const float* v = values + b * 256 + sub * 32;
        float sum = 0.0f;
        for (int i = 0; i < 32; ++i) { x[i] = v[i]; sum += x[i] * x[i]; }
        float magnitude = __fsqrt_rn(sum / 32.0f);
        for (int i = 0; i < 32; ++i) wts[i] = magnitude + fabsf(x[i]);
        // qkx2(levels = 15, range = (-1.0, 0.1, 20), squared error)
        float lo = x[0], hi = x[0], sum_w = wts[0], sum_x = wts[0] * x[0];
        for (int i = 1; i < 32; ++i) {
            if (x[i] < lo) lo = x[i];
            if (x[i] > hi) hi = x[i];
            sum_w += wts[i];
            sum_x += wts[i] * x[i];
        }
        if (lo > 0.0f) lo = 0.0f;
        if (hi == lo) {
            for (int i = 0; i < 32; ++i) codes[i] = 0;
            scale = 0.0f; minimum = -lo;
        } else {
            float inverse = 15.0f / (hi - lo);
            scale = 1.0f / inverse;
            float best_error = 0.0f;
            for (int i = 0; i < 32; ++i) {
                codes[i] = sat_u8(fmin32(fmax32(qround(inverse * (x[i] - lo)), 0.0f), 15.0f));
                float diff = scale * (float)codes[i] + lo - x[i];
                best_error += wts[i] * (diff * diff);
            }
            for (int step = 0; step <= 20; ++step) {
                inverse = (-1.0f + 0.1f * (float)step + 15.0f) / (hi - lo);
                float sum_l = 0.0f, sum_l2 = 0.0f, sum_xl = 0.0f;
                for (int i = 0; i < 32; ++i) {
                    trial[i] = sat_u8(fmin32(fmax32(qround(inverse * (x[i] - lo)), 0.0f), 15.0f));
                    float code = (float)trial[i];
                    sum_l += wts[i] * code;
                    sum_l2 += wts[i] * code * code;
                    sum_xl += wts[i] * code * x[i];
                }
                float denominator = sum_w * sum_l2 - sum_l * sum_l;
                if (denominator > 0.0f) {
                    float cs = (sum_w * sum_xl - sum_x * sum_l) / denominator;
                    float cm = (sum_l2 * sum_x - sum_l * sum_xl) / denominator;
                    if (cm > 0.0f) { cm = 0.0f; cs = sum_xl / sum_l2; }
                    float error = 0.0f;
                    for (int i = 0; i < 32; ++i) {
                        float diff = cs * (float)trial[i] + cm - x[i];
                        error += wts[i] * (diff * diff);
                    }
                    if (error < best_error) {
                        for (int i = 0; i < 32; ++i) codes[i] = trial[i];
                        best_error = error; scale = cs; lo = cm;
                    }
                }
            }
            minimum = -lo;
        }
        s_scale[lb][sub] = scale;
        s_min[lb][sub] = minimum;
    }
    __syncthreads();
    float maximum = 0.0f, max_minimum = 0.0f, stored_scale = 0.0f, stored_minimum = 0.0f;
    uint16_t hs = 0, hm = 0;
    if (live) {
        for (int j = 0; j < 8; ++j) { if (s_scale[lb][j] > maximum) maximum = s_scale[lb][j]; if (s_min[lb][j] > max_minimum) max_minimum = s_min[lb][j]; }
        hs = to_half_bits(maximum / 63.0f);
        hm = to_half_bits(max_minimum / 63.0f);
        stored_scale = rq_h2f(hs);
        stored_minimum = rq_h2f(hm);
        uint8_t sc = maximum > 0.0f ? sat_u8(fmin32(qround(63.0f * scale / maximum), 63.0f)) : 0;
        uint8_t mc = max_minimum > 0.0f ? sat_u8(fmin32(qround(63.0f * minimum / max_minimum), 63.0f)) : 0;
        s_sc[lb][sub] = sc; s_mc[lb][sub] = mc;
        // the six-bit codes survive the packing unchanged, so the re-quantisation reads them directly
        float d = stored_scale * (float)sc, m = stored_minimum * (float)mc;
        if (d != 0.0f)
            for (int i = 0; i < 32; ++i) codes[i] = sat_u8(fmin32(fmax32(qround((x[i] + m) / d), 0.0f), 15.0f));
        for (int i = 0; i < 32; ++i) s_codes[lb][sub * 32 + i] = codes[i];
    }
    __syncthreads();
    if (live) {
        uint8_t* o = out + b * 144;
        if (sub == 0) {
            put_half(o, hs);
            put_half(o + 2, hm);
            uint8_t meta[12];
            for (int j = 0; j < 12; ++j) meta[j] = 0;
            for (int j = 0; j < 8; ++j) {
                uint8_t sc = s_sc[lb][j], mc = s_mc[lb][j];
                if (j < 4) { meta[j] = sc; meta[j + 4] = mc; }
                else { meta[j + 4] = (uint8_t)((sc & 15) | ((mc & 15) << 4)); meta[j - 4] |= (uint8_t)((sc >> 4) << 6); meta[j] |= (uint8_t)((mc >> 4) << 6); }
            }
            for (int j = 0; j < 12; ++j) o[4 + j] = meta[j];
        }
        // thread `sub` packs 16 of the 128 nibble bytes: pair p = sub / 2, half h = sub % 2
        const int p = sub >> 1, h = sub & 1;
        for (int i = 0; i < 16; ++i) {
            int w = 16 * h + i;
            o[16 + 32 * p + w] = (uint8_t)((s_codes[lb][64 * p + w] & 15) | ((s_codes[lb][64 * p + 32 + w] & 15) << 4));
        }
    }
}

// ---- Q6_K: sixteen threads per block, one per 16-value sub-block ------------------------------
constexpr int kQ6Blocks = 8;  // blocks per CTA -> 128 threads

__global__ void __launch_bounds__(kQ6Blocks * 16) quant_q6k_kernel(const float* __restrict__ values, int64_t blocks, uint8_t* __restrict__ out) {
    __shared__ float s_scale[kQ6Blocks][16];
    __shared__ int8_t s_sc[kQ6Blocks][16];
    __shared__ uint8_t s_codes[kQ6Blocks][256];
    const int lb = threadIdx.x >> 4, sub = threadIdx.x & 15;
    const int64_t b = (int64_t)blockIdx.x * kQ6Blocks + lb;
    const bool live = b < blocks;
    float x[16];
    int codes[16];
    if (live) {
        const float* v = values + b * 256 + sub * 16;
        for (int i = 0; i < 16; ++i) x[i] = v[i];
        // qx(levels = 32)
        float maximum = 0.0f, absolute = 0.0f, scale = 0.0f;
        for (int i = 0; i < 16; ++i) { float c = fabsf(x[i]); if (c > absolute) { absolute = c; maximum = x[i]; } }
        if (absolute < 1.0e-15f) {
            for (int i = 0; i < 16; ++i) codes[i] = 0;
        } else {
            float inverse = -32.0f / maximum;
            float sum_lx = 0.0f, sum_l2 = 0.0f;
            for (int i = 0; i < 16; ++i) {
                float sg = fmin32(fmax32(qround(inverse * x[i]), -32.0f), 31.0f);
                codes[i] = sat_i8(sg) + 32;
                float wt = x[i] * x[i];
                sum_lx += wt * x[i] * sg;
                sum_l2 += wt * sg * sg;
            }
            scale = sum_l2 == 0.0f ? 0.0f : sum_lx / sum_l2;
            float best = scale * sum_lx;
            for (int step = -9; step <= 9; ++step) {
                if (step == 0) continue;
                inverse = -(32.0f + 0.1f * (float)step) / maximum;
                sum_lx = 0.0f; sum_l2 = 0.0f;
                for (int i = 0; i < 16; ++i) {
                    float code = fmin32(fmax32(qround(inverse * x[i]), -32.0f), 31.0f);
                    float wt = x[i] * x[i];
                    sum_lx += wt * x[i] * code;
                    sum_l2 += wt * code * code;
                }
                if (sum_l2 > 0.0f && sum_lx * sum_lx > best * sum_l2) {
                    for (int i = 0; i < 16; ++i) codes[i] = sat_i8(fmin32(fmax32(qround(inverse * x[i]), -32.0f), 31.0f)) + 32;
                    scale = sum_lx / sum_l2;
                    best = scale * sum_lx;
                }
            }
        }
        s_scale[lb][sub] = scale;
    }
    __syncthreads();
    uint16_t hd = 0;
    if (live) {
        float maximum = 0.0f, extreme = 0.0f;
        for (int j = 0; j < 16; ++j) { float a = fabsf(s_scale[lb][j]); if (a > extreme) { extreme = a; maximum = s_scale[lb][j]; } }
        float inverse = extreme < 1.0e-15f ? 0.0f : -128.0f / maximum;
        float scale = inverse == 0.0f ? 0.0f : 1.0f / inverse;
        hd = to_half_bits(scale);
        float stored = rq_h2f(hd);
        int sc = sat_i8(fmin32(qround(inverse * s_scale[lb][sub]), 127.0f));
        s_sc[lb][sub] = (int8_t)sc;
        float d = stored * (float)sc;
        if (d != 0.0f)
            for (int i = 0; i < 16; ++i) codes[i] = sat_i8(fmin32(fmax32(qround(x[i] / d), -32.0f), 31.0f)) + 32;
        for (int i = 0; i < 16; ++i) s_codes[lb][sub * 16 + i] = (uint8_t)(int8_t)codes[i];
    }
    __syncthreads();
    if (live) {
        uint8_t* o = out + b * 210;
        const uint8_t* c = s_codes[lb];
        // 128 ql bytes + 64 qh bytes over sixteen threads: eight ql and four qh bytes each
        for (int i = 0; i < 8; ++i) {
            int at = sub * 8 + i;                    // ql byte index 0..127
            int group = (at >> 6) * 128, within = at & 63, first = within < 32;
            int off = within & 31;
            uint8_t a = first ? c[group + off] : c[group + off + 32];
            uint8_t bq = first ? c[group + off + 64] : c[group + off + 96];
            o[at] = (uint8_t)((a & 15) | ((bq & 15) << 4));
        }
        for (int i = 0; i < 4; ++i) {
            int at = sub * 4 + i;                    // qh byte index 0..63
            int group = (at >> 5) * 128, off = at & 31;
            o[128 + at] = (uint8_t)((c[group + off] >> 4) | ((c[group + off + 32] >> 4) << 2) | ((c[group + off + 64] >> 4) << 4) | ((c[group + off + 96] >> 4) << 6));
        }
        o[192 + sub] = (uint8_t)s_sc[lb][sub];
        if (sub == 0) put_half(o + 208, hd);
    }
}

}  // namespace

int rq_launch_quantize(int type, const float* values, int64_t count, uint8_t* blocks, cudaStream_t s) {
    if (type == RQ_Q4_K) {
        int64_t n = count / 256;
        quant_q4k_kernel<<<(unsigned)((n + kQ4Blocks - 1) / kQ4Blocks), kQ4Blocks * 8, 0, s>>>(values, n, blocks);
    } else if (type == RQ_Q6_K) {
        int64_t n = count / 256;
        quant_q6k_kernel<<<(unsigned)((n + kQ6Blocks - 1) / kQ6Blocks), kQ6Blocks * 16, 0, s>>>(values, n, blocks);
    } else if (type == RQ_Q8_0) {
        int64_t n = count / 32;
        quant_block32_kernel<RQ_Q8_0><<<(unsigned)((n + 127) / 128), 128, 0, s>>>(values, n, blocks);
    } else if (type == RQ_Q4_0) {
        int64_t n = count / 32;
        quant_block32_kernel<RQ_Q4_0><<<(unsigned)((n + 127) / 128), 128, 0, s>>>(values, n, blocks);
    } else {
        return rq_fail(RQ_ERR_INVALID, "quantize: type %d", type);
    }
    RQ_CUDA(cudaGetLastError());
    return RQ_OK;
}
