// The int8 activation quantiser as a warp-level device function, shared by the standalone
// kernel and the streaming matvec (which runs it in its prologue, into shared memory).
//
// One warp handles one group of `step` inputs (32 or 256) of one token:
// the extreme is the FIRST input of strictly largest magnitude, signed; inverse = -127/extreme
// and d = 1/inverse are IEEE fp32 divides; code = clamp(rint(x * inverse)) -- the arithmetic of
// the reference's template at wave width 1 (amd-nv-cpu.ll:1381-1517).
#pragma once
#include "rq_internal.cuh"

// `tok` = where this token's records go (unit-record layout when `unit_layout`, else planes);
// `records36` = optional [recs][36] copy in the reference's own record format, or null.
__device__ __forceinline__ void rq_quantise_group(const float* __restrict__ xt, int64_t sk, int64_t cols, int step, int64_t g, int lane,
                                                  uint8_t* __restrict__ tok, bool unit_layout, uint8_t* __restrict__ records36) {
    const int span = step >> 5;  // 32-value records per group
    const int64_t recs = cols >> 5;
    const int64_t rec0 = g * span;
    const int n = (int)((rec0 + span <= recs ? span : recs - rec0));
    float v[8];
    float best = 0.f;
    int best_at = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        v[j] = 0.f;
        if (j < n) {
            v[j] = __ldg(xt + ((rec0 + j) * 32 + lane) * sk);
            if (fabsf(v[j]) > fabsf(best)) { best = v[j]; best_at = j * 32 + lane; }
        }
    }
    {
        // The first input of largest magnitude over the warp, by integer reductions (one instruction each): magnitudes of finite
        // floats order as their bits do; among the lanes that hold the largest, the lowest input index wins; its lane (the index's
        // low five bits) hands out the signed value. A lane's own `best` is never a NaN (a NaN loses every comparison above).
        const unsigned key = __float_as_uint(fabsf(best));
        const unsigned top = __reduce_max_sync(0xffffffffu, key);
        const unsigned first = __reduce_min_sync(0xffffffffu, key == top ? (unsigned)best_at : 0xffffffffu);
        best = __shfl_sync(0xffffffffu, best, (int)(first & 31u));
        best_at = (int)first;
    }
    const bool nonzero = fabsf(best) > 0.f;
    const float inverse = nonzero ? __fdiv_rn(-127.0f, best) : 0.f;
    const float d = nonzero ? __fdiv_rn(1.0f, inverse) : 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        if (j < n) {
            int code = __float2int_rn(__fmul_rn(v[j], inverse));
            code = code < -128 ? -128 : (code > 127 ? 127 : code);
            const int64_t rec = rec0 + j;
            // where this 32-value group keeps its codes, its step and its two slice sums
            int8_t* codes; float* dp; int16_t* sp;
            if (unit_layout) {
                uint8_t* unit = tok + (size_t)(rec >> 3) * RQ_ACT_RECORD_INT8;
                codes = (int8_t*)unit + 32 * (rec & 7);
                dp = (float*)(unit + 256) + (rec & 7);
                sp = (int16_t*)(unit + 288) + 2 * (rec & 7);
            } else {
                codes = (int8_t*)tok + rec * 32;
                dp = (float*)(tok + cols) + rec;
                sp = (int16_t*)(tok + cols + recs * 4) + rec * 2;
            }
            codes[lane] = (int8_t)code;
            // the two slices' sums: one integer reduction over each half of the warp
            const int s = __reduce_add_sync(lane < 16 ? 0x0000ffffu : 0xffff0000u, code);
            if ((lane & 15) == 0) sp[lane >> 4] = (int16_t)s;
            if (lane == 0) *dp = d;
            if (unit_layout) {
                const int gs = s + __shfl_xor_sync(0xffffffffu, s, 16);  // the whole group's sum
                if (lane == 0) ((int16_t*)(tok + (size_t)(rec >> 3) * RQ_ACT_RECORD_INT8 + 320))[rec & 7] = (int16_t)gs;
            }
            if (records36) {
                uint8_t* r36 = records36 + (size_t)rec * 36;
                if (lane == 0) *(float*)r36 = d;
                r36[4 + lane] = (uint8_t)(int8_t)code;
            }
        }
    }
}
