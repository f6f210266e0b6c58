/*
 * CPU oracle for the GGUF quantised matrix-vector path -- TEST INFRASTRUCTURE ONLY.
 * See rq_oracle.h for scope, pinning status and who may call this.
 *
 * Every arithmetic step that the reference performs in fp32 is performed here in fp32
 * with no contraction (build with -ffp-contract=off, no fast-math); fused multiply-adds
 * appear only where the reference calls `recipe.state.madd` (= llvm.fma, build.rs:1200).
 */
#include "rq_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------------- formats */

/* recipe.rs:15811-15822: block / stride of the four formats on the path. */
int rqo_block_values(int type) {
    switch (type) {
        case RQO_Q4_0: case RQO_Q8_0: case RQO_Q4_1: case RQO_Q5_0: case RQO_Q5_1: case RQO_IQ4_NL: case RQO_Q8_1: return 32;
        case RQO_Q4_K: case RQO_Q6_K: case RQO_Q5_K: case RQO_Q2_K: case RQO_Q3_K: case RQO_Q8_K: case RQO_IQ4_XS: return 256;
        default: return 0;
    }
}
int rqo_block_bytes(int type) {
    switch (type) {
        case RQO_Q4_0: return 18;
        case RQO_Q8_0: return 34;
        case RQO_Q4_K: return 144;
        case RQO_Q6_K: return 210;
        case RQO_Q4_1: return 20;
        case RQO_Q5_0: return 22;
        case RQO_Q5_1: return 24;
        case RQO_Q5_K: return 176;
        case RQO_IQ4_NL: return 18;
        case RQO_Q8_1: return 36;
        case RQO_Q2_K: return 84;
        case RQO_Q3_K: return 110;
        case RQO_Q8_K: return 292;
        case RQO_IQ4_XS: return 136;
        default: return 0;
    }
}

static inline uint32_t f32_bits(float v) { uint32_t b; memcpy(&b, &v, 4); return b; }
static inline float bits_f32(uint32_t b) { float v; memcpy(&v, &b, 4); return v; }

/* recipe.rs:15098-15112. Round to nearest even through the 0xfff + lsb carry; an
 * exponent past the half range gives infinity, with the low bit set when the source
 * mantissa was non-zero (the reference does that for finite overflow too). */
uint16_t rqo_fp16(float value) {
    uint32_t bits = f32_bits(value);
    uint16_t sign = (uint16_t)((bits >> 16) & 0x8000u);
    int32_t exponent = (int32_t)((bits >> 23) & 0xffu) - 112;
    uint32_t mantissa = bits & 0x7fffffu;
    if (exponent <= 0) {
        if (exponent < -10) return sign;
        uint32_t wide = (mantissa | 0x800000u) >> (1 - exponent);
        return (uint16_t)(sign | (uint16_t)((wide + 0xfffu + ((wide >> 13) & 1u)) >> 13));
    }
    if (exponent >= 31) return (uint16_t)(sign | 0x7c00u | (mantissa != 0 ? 1u : 0u));
    uint32_t rounded = mantissa + 0xfffu + ((mantissa >> 13) & 1u);
    if (rounded & 0x800000u) {
        int32_t up = exponent + 1;
        if (up > 31) up = 31;
        return (uint16_t)(sign | (uint16_t)(up << 10));
    }
    return (uint16_t)(sign | (uint16_t)(exponent << 10) | (uint16_t)(rounded >> 13));
}

/* recipe.rs:15114-15126. */
float rqo_unfp16(uint16_t value) {
    uint32_t sign = ((uint32_t)value & 0x8000u) << 16;
    uint32_t exponent = (value >> 10) & 31u;
    uint32_t mantissa = value & 1023u;
    uint32_t bits;
    if (exponent == 0) {
        if (mantissa == 0) {
            bits = sign;
        } else {
            uint32_t shift = (uint32_t)__builtin_clz(mantissa) - 21u;
            bits = sign | ((113u - shift) << 23) | ((mantissa << (shift + 13u)) & 0x7fffffu);
        }
    } else if (exponent == 31) {
        bits = sign | 0x7f800000u | (mantissa << 13);
    } else {
        bits = sign | ((exponent + 112u) << 23) | (mantissa << 13);
    }
    return bits_f32(bits);
}

static inline float half_at(const uint8_t* p) { return rqo_unfp16((uint16_t)(p[0] | (p[1] << 8))); }
static inline void put_half(uint8_t* p, float v) { uint16_t h = rqo_fp16(v); p[0] = (uint8_t)(h & 0xff); p[1] = (uint8_t)(h >> 8); }

/* recipe.rs:15133-15135: round to nearest even through the 1.5 * 2^23 magic constant. */
float rqo_qround(float value) {
    float shifted = value + 12582912.0f;
    int32_t bits = (int32_t)f32_bits(shifted);
    return (float)((bits & 0x007fffff) - 0x00400000);
}

/* Rust's `as u8` / `as i8` on a float: truncate toward zero, saturate, NaN -> 0. */
static inline uint8_t sat_u8(float v) { if (!(v > 0.0f)) return 0; if (v >= 255.0f) return 255; return (uint8_t)v; }
static inline int8_t sat_i8(float v) { if (v != v) return 0; if (v <= -128.0f) return -128; if (v >= 127.0f) return 127; return (int8_t)v; }
/* f32::max / f32::min (NaN-ignoring; inputs here are never NaN for finite data). */
static inline float fmax32(float a, float b) { return (b > a || a != a) ? b : a; }
static inline float fmin32(float a, float b) { return (b < a || a != a) ? b : a; }

/* ------------------------------------------------------------------ per-value unpack */

/* recipe.rs:15204-15210 (k_scale) = recipe.rs:3710-3731 (dequant_q45k). `s` = the 12 bytes. */
static inline void q4k_scale_min(const uint8_t* s, int j, int* sc, int* mn) {
    if (j < 4) {
        *sc = s[j] & 63;
        *mn = s[j + 4] & 63;
    } else {
        *sc = (s[j + 4] & 15) | ((s[j - 4] >> 6) << 4);
        *mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}

/* recipe.rs:3687-3741 with man = 4: step = d*sc, base = dmin*m, value = step*q - base,
 * each a separate fp32 operation (NativeQuantOps, recipe.rs:4083-4231). */
static inline float q4k_value(const uint8_t* b, int i) {
    int sub = i / 32, within = i % 32;
    uint8_t packed = b[16 + (sub / 2) * 32 + within];
    int q = (packed >> ((sub % 2) * 4)) & 15;
    int sc, mn;
    q4k_scale_min(b + 4, sub, &sc, &mn);
    float step = half_at(b) * (float)sc;
    float base = half_at(b + 2) * (float)mn;
    float product = step * (float)q;
    return product - base;
}
static inline int q4k_code(const uint8_t* b, int i) {
    int sub = i / 32, within = i % 32;
    return (b[16 + (sub / 2) * 32 + within] >> ((sub % 2) * 4)) & 15;
}

/* recipe.rs:3743-3780. Returns the raw 0..63 code; the value is (d*scale)*(code-32). */
static inline int q6k_code(const uint8_t* b, int i) {
    int chunk = i / 128, local = i % 128, group = local / 32, within = local % 32;
    uint8_t low = b[64 * chunk + 32 * (group & 1) + within];
    uint8_t high = b[128 + 32 * chunk + within];
    int lo = (low >> (4 * (group / 2))) & 15;
    int hi = (high >> (2 * group)) & 3;
    return lo | (hi << 4);
}
static inline int q6k_scale_index(int i) {
    int chunk = i / 128, local = i % 128, group = local / 32, within = local % 32;
    return 8 * chunk + 2 * group + within / 16;
}
static inline float q6k_value(const uint8_t* b, int i) {
    int code = q6k_code(b, i) - 32;
    float scaled = half_at(b + 208) * (float)(int8_t)b[192 + q6k_scale_index(i)];
    return scaled * (float)code;
}

/* recipe.rs:3782-3833 (variant 0, man 8 / man 4): code * scale. */
static inline int q80_code(const uint8_t* b, int i) { return (int8_t)b[2 + i]; }
static inline int q40_code(const uint8_t* b, int i) { return ((b[2 + i % 16] >> ((i / 16) * 4)) & 15) - 8; }
static inline float q80_value(const uint8_t* b, int i) { return (float)q80_code(b, i) * half_at(b); }
static inline float q40_value(const uint8_t* b, int i) { return (float)q40_code(b, i) * half_at(b); }

/* recipe.rs:3782-3833, variant 1 (a block minimum after the step: header d, m) and man 5 (the
 * fifth bit of value i is bit i % 8 of byte header + i / 8; the nibbles follow those four bytes). */
static inline float q41_value(const uint8_t* b, int i) {
    int code = (b[4 + i % 16] >> ((i / 16) * 4)) & 15;
    float product = (float)code * half_at(b);
    return product + half_at(b + 2);
}
static inline float q50_value(const uint8_t* b, int i) {
    int low = (b[6 + i % 16] >> ((i / 16) * 4)) & 15;
    int high = (b[2 + i / 8] >> (i % 8)) & 1;
    return (float)((low | (high << 4)) - 16) * half_at(b);
}
static inline float q51_value(const uint8_t* b, int i) {
    int low = (b[8 + i % 16] >> ((i / 16) * 4)) & 15;
    int high = (b[4 + i / 8] >> (i % 8)) & 1;
    float product = (float)(low | (high << 4)) * half_at(b);
    return product + half_at(b + 2);
}
/* recipe.rs:3687-3741 with man = 5: the nibbles start at byte 48, the fifth bit of value i of
 * sub-block `sub` is bit `sub` of byte 16 + i % 32; scales and minima as Q4_K. */
static inline float q5k_value(const uint8_t* b, int i) {
    int sub = i / 32, within = i % 32;
    int low = (b[48 + (sub / 2) * 32 + within] >> ((sub % 2) * 4)) & 15;
    int high = (b[16 + within] >> sub) & 1;
    int sc, mn;
    q4k_scale_min(b + 4, sub, &sc, &mn);
    float step = half_at(b) * (float)sc;
    float base = half_at(b + 2) * (float)mn;
    float product = step * (float)(low | (high << 4));
    return product - base;
}
/* recipe.rs:3919-3958 without the per-sub-block exponent (xs = false): (d * 1) * IQ4[nibble];
 * levels recipe.rs:15211. */
static const int8_t IQ4_LEVELS[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
static inline float iq4nl_value(const uint8_t* b, int i) {
    int code = (b[2 + i % 16] >> (i < 16 ? 0 : 4)) & 15;
    float scaled = half_at(b) * 1.0f;
    return scaled * (float)IQ4_LEVELS[code];
}

/* recipe.rs:3782-3833, man 8 variant 1 (Q8_1): header d, s; the code times d (the stored sum s is not part of a value). */
static inline float q81_value(const uint8_t* b, int i) { return (float)(int8_t)b[4 + i] * half_at(b); }
/* recipe.rs:3835-3866: sixteen (scale | minimum << 4) bytes, 64 bytes of two-bit codes, d @80, dmin @82. Group `order` of
 * sixteen values reads metadata byte `order`; its codes sit in byte 16 + 32 (order / 8) + 16 (order % 2) + i % 16 at bit
 * 2 ((order % 8) / 2). */
static inline float q2k_value(const uint8_t* b, int i) {
    int order = i / 16, section = order / 8, shift = 2 * ((order % 8) / 2), half_index = order % 2;
    uint8_t metadata = b[section * 8 + shift + half_index];
    int code = (b[16 + section * 32 + half_index * 16 + i % 16] >> shift) & 3;
    float scaled = half_at(b + 80) * (float)(metadata & 15);
    float product = scaled * (float)code;
    float minimum = half_at(b + 82) * (float)(metadata >> 4);
    return product - minimum;
}
/* recipe.rs:3868-3907: high-bit mask 0..31, two-bit codes 32..95, twelve scale bytes 96..107 (four low bits per group in
 * bytes 96..103, two high bits in bytes 104..107), d @108. A clear mask bit subtracts four from the code. */
static inline float q3k_value(const uint8_t* b, int i) {
    int block = i / 16;
    int low = (b[96 + (block < 8 ? block : block - 8)] >> (block < 8 ? 0 : 4)) & 15;
    int high = (b[104 + block % 4] >> ((block / 4) * 2)) & 3;
    int scale_code = (low | (high << 4)) - 32;
    int code = (b[32 + (i / 128) * 32 + i % 32] >> (((i % 128) / 32) * 2)) & 3;
    int sign = (b[i % 32] >> (i / 32)) & 1;
    code -= sign ? 0 : 4;
    float scaled = half_at(b + 108) * (float)scale_code;
    return scaled * (float)code;
}
/* recipe.rs:3909-3917: an fp32 step, 256 int8 codes from byte 4 (the sixteen partial sums after them are not part of a value). */
static inline float q8k_value(const uint8_t* b, int i) {
    float d;
    memcpy(&d, b, 4);
    return d * (float)(int8_t)b[4 + i];
}
/* recipe.rs:3919-3958 with a six-bit exponent per 32 values (xs = true): two high bits from the u16 @2, four low bits
 * from bytes 4..7, less 32; (d * exponent) * IQ4[nibble], nibbles from byte 8. */
static inline float iq4xs_value(const uint8_t* b, int i) {
    int block = i / 32;
    int high = ((b[2] | (b[3] << 8)) >> (2 * block)) & 3;
    int low = (b[4 + block / 2] >> ((block % 2) * 4)) & 15;
    int exponent = (low | (high << 4)) - 32;
    int code = (b[8 + block * 16 + i % 16] >> (i % 32 < 16 ? 0 : 4)) & 15;
    float scaled = half_at(b) * (float)exponent;
    return scaled * (float)IQ4_LEVELS[code];
}

static inline float block_value(int type, const uint8_t* b, int i) {
    switch (type) {
        case RQO_Q4_0: return q40_value(b, i);
        case RQO_Q8_0: return q80_value(b, i);
        case RQO_Q4_K: return q4k_value(b, i);
        case RQO_Q4_1: return q41_value(b, i);
        case RQO_Q5_0: return q50_value(b, i);
        case RQO_Q5_1: return q51_value(b, i);
        case RQO_Q5_K: return q5k_value(b, i);
        case RQO_IQ4_NL: return iq4nl_value(b, i);
        case RQO_Q8_1: return q81_value(b, i);
        case RQO_Q2_K: return q2k_value(b, i);
        case RQO_Q3_K: return q3k_value(b, i);
        case RQO_Q8_K: return q8k_value(b, i);
        case RQO_IQ4_XS: return iq4xs_value(b, i);
        default: return q6k_value(b, i);
    }
}
/* the four formats with their own int8 slice helpers, exact-slice helpers and quantisers here */
static inline int type_has_slices(int type) { return type == RQO_Q4_0 || type == RQO_Q8_0 || type == RQO_Q4_K || type == RQO_Q6_K; }

/* ----------------------------------------------------------------------- threading */

typedef void (*span_fn)(void* ctx, int64_t first, int64_t last, int worker, int workers);
typedef struct { span_fn fn; void* ctx; int64_t first, last; int worker, workers; } span_job;
static void* span_entry(void* p) { span_job* j = (span_job*)p; j->fn(j->ctx, j->first, j->last, j->worker, j->workers); return NULL; }

/* One contiguous run of items per worker (recipe.rs:16141-16158, :16163-16185). */
static void run_spans(int64_t items, int threads, span_fn fn, void* ctx) {
    if (threads < 1) threads = 1;
    if (threads > 256) threads = 256;
    int64_t span = (items + threads - 1) / threads;
    if (span < 1) span = 1;
    int used = (int)((items + span - 1) / span);
    if (used <= 1) { fn(ctx, 0, items, 0, 1); return; }
    pthread_t ids[256];
    span_job jobs[256];
    for (int t = 0; t < used; ++t) {
        int64_t a = t * span, b = a + span > items ? items : a + span;
        jobs[t] = (span_job){fn, ctx, a, b, t, used};
        pthread_create(&ids[t], NULL, span_entry, &jobs[t]);
    }
    for (int t = 0; t < used; ++t) pthread_join(ids[t], NULL);
}

/* ------------------------------------------------------------------------ dequantise */

typedef struct { int type; const uint8_t* blocks; float* out; } dequant_ctx;
static void dequant_span(void* p, int64_t first, int64_t last, int worker, int workers) {
    (void)worker; (void)workers;
    dequant_ctx* c = (dequant_ctx*)p;
    int values = rqo_block_values(c->type), bytes = rqo_block_bytes(c->type);
    for (int64_t blk = first; blk < last; ++blk) {
        const uint8_t* b = c->blocks + blk * bytes;
        float* o = c->out + blk * values;
        for (int i = 0; i < values; ++i) o[i] = block_value(c->type, b, i);
    }
}
int rqo_dequantize(int type, const uint8_t* blocks, int64_t count, float* out, int threads) {
    int values = rqo_block_values(type);
    if (!values || count % values) return -1;
    dequant_ctx c = {type, blocks, out};
    run_spans(count / values, threads, dequant_span, &c);
    return 0;
}

/* ------------------------------------------------------------------------ quantisers */

/* recipe.rs:15136-15138 */
static float positive_max(const float* v, int n) { float m = 0.0f; for (int i = 0; i < n; ++i) if (v[i] > m) m = v[i]; return m; }

/* recipe.rs:15140-15162 (qkx2), squared-error form (mad = false). */
static void qkx2(const float* values, const float* weights, int n, int levels, float r0, float r1, int steps,
                 uint8_t* codes, float* out_scale, float* out_minimum) {
    float lv = (float)levels;
    float minimum = values[0], maximum = values[0], sum_w = weights[0], sum_x = weights[0] * values[0];
    for (int i = 1; i < n; ++i) {
        if (values[i] < minimum) minimum = values[i];
        if (values[i] > maximum) maximum = values[i];
        sum_w += weights[i];
        sum_x += weights[i] * values[i];
    }
    if (minimum > 0.0f) minimum = 0.0f;
    if (maximum == minimum) { memset(codes, 0, (size_t)n); *out_scale = 0.0f; *out_minimum = -minimum; return; }
    float inverse = lv / (maximum - minimum);
    float scale = 1.0f / inverse;
    float best_error = 0.0f;
    for (int i = 0; i < n; ++i) {
        codes[i] = sat_u8(fmin32(fmax32(rqo_qround(inverse * (values[i] - minimum)), 0.0f), lv));
        float difference = scale * (float)codes[i] + minimum - values[i];
        best_error += weights[i] * (difference * difference);
    }
    uint8_t trial[32];
    for (int step = 0; step <= steps; ++step) {
        inverse = (r0 + r1 * (float)step + lv) / (maximum - minimum);
        float sum_l = 0.0f, sum_l2 = 0.0f, sum_xl = 0.0f;
        for (int i = 0; i < n; ++i) {
            trial[i] = sat_u8(fmin32(fmax32(rqo_qround(inverse * (values[i] - minimum)), 0.0f), lv));
            float code = (float)trial[i];
            sum_l += weights[i] * code;
            sum_l2 += weights[i] * code * code;
            sum_xl += weights[i] * code * values[i];
        }
        float denominator = sum_w * sum_l2 - sum_l * sum_l;
        if (denominator > 0.0f) {
            float cand_scale = (sum_w * sum_xl - sum_x * sum_l) / denominator;
            float cand_minimum = (sum_l2 * sum_x - sum_l * sum_xl) / denominator;
            if (cand_minimum > 0.0f) { cand_minimum = 0.0f; cand_scale = sum_xl / sum_l2; }
            float error = 0.0f;
            for (int i = 0; i < n; ++i) {
                float difference = cand_scale * (float)trial[i] + cand_minimum - values[i];
                error += weights[i] * (difference * difference);
            }
            if (error < best_error) { memcpy(codes, trial, (size_t)n); best_error = error; scale = cand_scale; minimum = cand_minimum; }
        }
    }
    *out_scale = scale;
    *out_minimum = -minimum;
}

/* recipe.rs:15183-15203 (qx). */
static float qx(const float* values, int n, int levels, int8_t* codes) {
    float lv = (float)levels, top = (float)(levels - 1);
    float maximum = 0.0f, absolute = 0.0f;
    for (int i = 0; i < n; ++i) { float cand = fabsf(values[i]); if (cand > absolute) { absolute = cand; maximum = values[i]; } }
    if (absolute < 1.0e-15f) { memset(codes, 0, (size_t)n); return 0.0f; }
    float inverse = -lv / maximum;
    float sum_lx = 0.0f, sum_l2 = 0.0f;
    for (int i = 0; i < n; ++i) {
        float sgn = fmin32(fmax32(rqo_qround(inverse * values[i]), -lv), top);
        codes[i] = (int8_t)(sat_i8(sgn) + (int8_t)levels);
        float weight = values[i] * values[i];
        sum_lx += weight * values[i] * sgn;
        sum_l2 += weight * sgn * sgn;
    }
    float scale = sum_l2 == 0.0f ? 0.0f : sum_lx / sum_l2;
    float best = scale * sum_lx;
    for (int step = -9; step <= 9; ++step) {
        if (step == 0) continue;
        inverse = -(lv + 0.1f * (float)step) / maximum;
        sum_lx = 0.0f; sum_l2 = 0.0f;
        for (int i = 0; i < n; ++i) {
            float code = fmin32(fmax32(rqo_qround(inverse * values[i]), -lv), top);
            float weight = values[i] * values[i];
            sum_lx += weight * values[i] * code;
            sum_l2 += weight * code * code;
        }
        if (sum_l2 > 0.0f && sum_lx * sum_lx > best * sum_l2) {
            for (int i = 0; i < n; ++i)
                codes[i] = (int8_t)(sat_i8(fmin32(fmax32(rqo_qround(inverse * values[i]), -lv), top)) + (int8_t)levels);
            scale = sum_lx / sum_l2;
            best = scale * sum_lx;
        }
    }
    return scale;
}

/* recipe.rs:16191-16242, Scalar quantiser with (bits, variant) = (8, 0) and (4, 0). */
static void encode_block32(int type, const float* values, uint8_t* out) {
    /* max_by(|a| total_cmp |b|) keeps the LAST of equal maxima (recipe.rs:16195). */
    float extreme = values[0];
    for (int i = 1; i < 32; ++i) if (fabsf(values[i]) >= fabsf(extreme)) extreme = values[i];
    float scale = type == RQO_Q8_0 ? fabsf(extreme) / 127.0f : extreme / -8.0f;
    float inverse = scale == 0.0f ? 0.0f : 1.0f / scale;
    put_half(out, scale);
    uint8_t* data = out + 2;
    if (type == RQO_Q8_0) {
        for (int i = 0; i < 32; ++i) {
            float shifted = roundf(values[i] * inverse) + 128.0f;  /* f32::round: half away from zero */
            uint8_t code = sat_u8(fmin32(fmax32(shifted, 0.0f), 255.0f));
            data[i] = (uint8_t)(code - 128u);
        }
    } else {
        memset(data, 0, 16);
        for (int i = 0; i < 32; ++i) {
            float shifted = values[i] * inverse + 8.0f + 0.5f;
            uint8_t code = sat_u8(fmin32(fmax32(shifted, 0.0f), 15.0f));
            data[i % 16] |= (uint8_t)((code & 15) << (i / 16 * 4));
        }
    }
}

/* recipe.rs:16325-16375 with bits = 4. */
static void encode_q4k(const float* values, uint8_t* out) {
    uint8_t codes[256];
    float block_scales[8], minima[8];
    for (int blk = 0; blk < 8; ++blk) {
        const float* slice = values + blk * 32;
        float sum = 0.0f;
        for (int i = 0; i < 32; ++i) sum += slice[i] * slice[i];
        float magnitude = sqrtf(sum / 32.0f);
        float weights[32];
        for (int i = 0; i < 32; ++i) weights[i] = magnitude + fabsf(slice[i]);
        qkx2(slice, weights, 32, 15, -1.0f, 0.1f, 20, codes + blk * 32, &block_scales[blk], &minima[blk]);
    }
    float maximum = positive_max(block_scales, 8), max_minimum = positive_max(minima, 8);
    float scale = maximum / 63.0f, minimum = max_minimum / 63.0f;
    float stored_scale = rqo_unfp16(rqo_fp16(scale)), stored_minimum = rqo_unfp16(rqo_fp16(minimum));
    uint8_t metadata[12];
    memset(metadata, 0, 12);
    for (int blk = 0; blk < 8; ++blk) {
        uint8_t sc = maximum > 0.0f ? sat_u8(fmin32(rqo_qround(63.0f * block_scales[blk] / maximum), 63.0f)) : 0;
        uint8_t mc = max_minimum > 0.0f ? sat_u8(fmin32(rqo_qround(63.0f * minima[blk] / max_minimum), 63.0f)) : 0;
        if (blk < 4) {
            metadata[blk] = sc;
            metadata[blk + 4] = mc;
        } else {
            metadata[blk + 4] = (uint8_t)((sc & 15) | ((mc & 15) << 4));
            metadata[blk - 4] |= (uint8_t)((sc >> 4) << 6);
            metadata[blk] |= (uint8_t)((mc >> 4) << 6);
        }
    }
    for (int blk = 0; blk < 8; ++blk) {
        int sc, mc;
        q4k_scale_min(metadata, blk, &sc, &mc);
        float d = stored_scale * (float)sc, m = stored_minimum * (float)mc;
        if (d != 0.0f)
            for (int o = 0; o < 32; ++o)
                codes[blk * 32 + o] = sat_u8(fmin32(fmax32(rqo_qround((values[blk * 32 + o] + m) / d), 0.0f), 15.0f));
    }
    put_half(out, scale);
    put_half(out + 2, minimum);
    memcpy(out + 4, metadata, 12);
    uint8_t* packed = out + 16;
    for (int group = 0; group < 256; group += 64)
        for (int o = 0; o < 32; ++o)
            packed[group / 2 + o] = (uint8_t)((codes[group + o] & 15) | ((codes[group + o + 32] & 15) << 4));
}

/* recipe.rs:16376-16414. */
static void encode_q6k(const float* values, uint8_t* out) {
    int8_t codes[256];
    float block_scales[16];
    float maximum = 0.0f, extreme = 0.0f;
    for (int blk = 0; blk < 16; ++blk) {
        block_scales[blk] = qx(values + blk * 16, 16, 32, codes + blk * 16);
        if (fabsf(block_scales[blk]) > extreme) { extreme = fabsf(block_scales[blk]); maximum = block_scales[blk]; }
    }
    float inverse = extreme < 1.0e-15f ? 0.0f : -128.0f / maximum;
    float scale = inverse == 0.0f ? 0.0f : 1.0f / inverse;
    float stored_scale = rqo_unfp16(rqo_fp16(scale));
    int8_t scales[16];
    for (int blk = 0; blk < 16; ++blk) {
        scales[blk] = sat_i8(fmin32(rqo_qround(inverse * block_scales[blk]), 127.0f));
        float d = stored_scale * (float)scales[blk];
        if (d != 0.0f)
            for (int o = 0; o < 16; ++o)
                codes[blk * 16 + o] = (int8_t)(sat_i8(fmin32(fmax32(rqo_qround(values[blk * 16 + o] / d), -32.0f), 31.0f)) + 32);
    }
    uint8_t* low = out;
    uint8_t* high = out + 128;
    for (int group = 0; group < 256; group += 128)
        for (int o = 0; o < 32; ++o) {
            uint8_t c0 = (uint8_t)codes[group + o], c1 = (uint8_t)codes[group + o + 32];
            uint8_t c2 = (uint8_t)codes[group + o + 64], c3 = (uint8_t)codes[group + o + 96];
            low[group / 2 + o] = (uint8_t)((c0 & 15) | ((c2 & 15) << 4));
            low[group / 2 + o + 32] = (uint8_t)((c1 & 15) | ((c3 & 15) << 4));
            high[group / 4 + o] = (uint8_t)((c0 >> 4) | ((c1 >> 4) << 2) | ((c2 >> 4) << 4) | ((c3 >> 4) << 6));
        }
    for (int blk = 0; blk < 16; ++blk) out[192 + blk] = (uint8_t)scales[blk];
    put_half(out + 208, scale);
}

typedef struct { int type; const float* values; int64_t count; uint8_t* blocks; } quant_ctx;
static void quant_span(void* p, int64_t first, int64_t last, int worker, int workers) {
    (void)worker; (void)workers;
    quant_ctx* c = (quant_ctx*)p;
    int values = rqo_block_values(c->type), bytes = rqo_block_bytes(c->type);
    float staged[256];
    for (int64_t blk = first; blk < last; ++blk) {
        /* a trailing partial slice pads with zeros (recipe.rs:16171-16173) */
        for (int i = 0; i < values; ++i) {
            int64_t at = blk * values + i;
            staged[i] = at < c->count ? c->values[at] : 0.0f;
        }
        uint8_t* out = c->blocks + blk * bytes;
        if (c->type == RQO_Q4_K) encode_q4k(staged, out);
        else if (c->type == RQO_Q6_K) encode_q6k(staged, out);
        else encode_block32(c->type, staged, out);
    }
}
int rqo_quantize(int type, const float* values, int64_t count, uint8_t* blocks, int threads) {
    int per = rqo_block_values(type);
    if (!per || count < 0 || !type_has_slices(type)) return -1; /* encoders exist for the four formats of the path */
    quant_ctx c = {type, values, count, blocks};
    run_spans((count + per - 1) / per, threads, quant_span, &c);
    return 0;
}

/* -------------------------------------------- load-time re-encode of a bound tensor (a20) */

/* One 32-value block through the load kernel's encoder, emit_requantize recipe.rs:8016-8127.
 * The extreme is the FIRST value of strictly largest magnitude, found from a running value
 * that starts at zero (:8066-8081); Q8_0 (:8141-8155): scale = |extreme| / 127, inverse =
 * 1 / scale (0 when the scale is 0), code = fptosi(q + 0.5) or fptosi(q - 0.5) by the sign
 * of q = v * inverse (half away from zero by truncation, NOT f32::round), clamped to
 * [-128, 127]; the scale is stored with fptrunc (round to nearest even). */
static void requant_block_q8_0(const float* v, uint8_t* out) {
    float e = 0.0f;
    for (int i = 0; i < 32; ++i) if (fabsf(v[i]) > fabsf(e)) e = v[i];
    float ext = fabsf(e);
    float scale = ext / 127.0f;
    float inverse = scale == 0.0f ? 0.0f : 1.0f / scale;
    put_half(out, scale);
    for (int i = 0; i < 32; ++i) {
        float q = v[i] * inverse;
        float r = q >= 0.0f ? q + 0.5f : q + -0.5f;
        int32_t code = (int32_t)r; /* fptosi: toward zero */
        if (code < -128) code = -128;
        if (code > 127) code = 127;
        out[2 + i] = (uint8_t)(int8_t)code;
    }
}

/* emit_requantize, DeviceQuantizer::Q4_1 (recipe.rs:8037-8047, :8088-8094, :8099-8112): the block's minimum and maximum
 * (first of equals kept), step = (max - min) / 15, inverse guarded against a zero step, code = fptoui(clamp((v - min) *
 * inverse + 0.5, 0, 15)); step and minimum stored with fptrunc (round to nearest even), codes two to a byte (value i low,
 * value i + 16 high). */
static void requant_block_q4_1(const float* v, uint8_t* out) {
    float mn = v[0], mx = v[0];
    for (int i = 0; i < 32; ++i) {
        if (v[i] < mn) mn = v[i];
        if (v[i] > mx) mx = v[i];
    }
    float range = mx - mn;
    float scale = range / 15.0f;
    float inverse = scale == 0.0f ? 0.0f : 1.0f / scale;
    put_half(out, scale);
    put_half(out + 2, mn);
    uint8_t code[32];
    for (int i = 0; i < 32; ++i) {
        float off = v[i] - mn;
        float q = off * inverse;
        float sh = q + 0.5f;
        float cl = sh < 0.0f ? 0.0f : sh;
        cl = cl > 15.0f ? 15.0f : cl;
        code[i] = (uint8_t)(uint32_t)cl; /* fptoui: toward zero */
    }
    for (int i = 0; i < 16; ++i) out[4 + i] = (uint8_t)(code[i] | (code[i + 16] << 4));
}

typedef struct { int type; const uint8_t* blocks; int64_t count; uint8_t* out; int target; } requant_ctx;
static void requant_span(void* p, int64_t first, int64_t last, int worker, int workers) {
    (void)worker; (void)workers;
    requant_ctx* c = (requant_ctx*)p;
    int per = rqo_block_values(c->type), bytes = rqo_block_bytes(c->type);
    float v[32];
    for (int64_t blk = first; blk < last; ++blk) {
        for (int i = 0; i < 32; ++i) {
            /* a tail past the weight's end contributes zero (recipe.rs:8049-8063) */
            int64_t at = blk * 32 + i;
            v[i] = at < c->count ? block_value(c->type, c->blocks + (at / per) * bytes, (int)(at % per)) : 0.0f;
        }
        if (c->target == RQO_Q4_1) requant_block_q4_1(v, c->out + blk * 20);
        else requant_block_q8_0(v, c->out + blk * 34);
    }
}
/* finish_int_sums + requantize_bound (recipe.rs:22345-22431): a tensor bound in a format that
 * `.int(8)` does not keep (anything but Q8_0, Q4_K and the Q4_K + Q6_K mix) is decoded by its
 * source decoder and encoded again as Q8_0 by the load kernel, once, before any matvec. */
int rqo_requantize_q8_0(int type, const uint8_t* blocks, int64_t count, uint8_t* out, int threads) {
    if (!rqo_block_values(type) || count < 0) return -1;
    requant_ctx c = {type, blocks, count, out, RQO_Q8_0};
    run_spans((count + 31) / 32, threads, requant_span, &c);
    return 0;
}
/* The same for `.int(4)`: its storage is Q4_1 (recipe.rs:22348), kept only when the tensor is stored as Q4_1 already;
 * everything else is decoded and encoded as Q4_1 by the load kernel. out: ceil(count / 32) * 20 bytes. */
int rqo_requantize_q4_1(int type, const uint8_t* blocks, int64_t count, uint8_t* out, int threads) {
    if (!rqo_block_values(type) || count < 0) return -1;
    requant_ctx c = {type, blocks, count, out, RQO_Q4_1};
    run_spans((count + 31) / 32, threads, requant_span, &c);
    return 0;
}

/* ----------------------------------------------------- int8 activation records (a10) */

#define RQO_RECORD 36 /* fp32 step + 32 int8 codes: build.rs:332-337 */

/* ll:1381-1517 at wave width 1: one scan over the group's values keeps the first value
 * of strictly largest magnitude, signed; inverse = -127/extreme, d = 1/inverse (both
 * fp32 divides); code = clamp(fptosi(roundeven(x * inverse)), -128, 127). */
int rqo_quantize_activations(const float* x, int64_t x_stride, int64_t terms, int step, uint8_t* records) {
    if (terms % 32 || (step != 32 && step != 256)) return -1;
    int64_t blocks = terms / 32;
    int span = step / 32;
    for (int64_t first = 0; first < blocks; first += span) {
        int64_t stop = first + span > blocks ? blocks : first + span;
        float extreme = 0.0f;
        for (int64_t k = first * 32; k < stop * 32; ++k) {
            float v = x[k * x_stride];
            if (fabsf(v) > fabsf(extreme)) extreme = v;
        }
        int nonzero = fabsf(extreme) > 0.0f;
        float inverse = nonzero ? -127.0f / extreme : 0.0f;
        float d = nonzero ? 1.0f / inverse : 0.0f;
        for (int64_t b = first; b < stop; ++b) {
            uint8_t* rec = records + b * RQO_RECORD;
            memcpy(rec, &d, 4);
            for (int v = 0; v < 32; ++v) {
                float scaled = x[(b * 32 + v) * x_stride] * inverse;
                float even = nearbyintf(scaled); /* default rounding mode = ties to even */
                int32_t code = (int32_t)even;
                if (code < -128) code = -128;
                if (code > 127) code = 127;
                rec[4 + v] = (uint8_t)(int8_t)code;
            }
        }
    }
    return 0;
}

static inline float rec_d(const uint8_t* rec) { float d; memcpy(&d, rec, 4); return d; }
static inline const int8_t* rec_codes(const uint8_t* rec) { return (const int8_t*)(rec + 4); }

/* ------------------------------------------------------------- int8 dots, step 32 (a11-a13) */

/* build.rs:777-796: r = q8_d * (d * f32(dot) + m * f32(sum a)), m = 0 for Q8_0 / Q4_0, the block's minimum for Q4_1;
 * Q4_0 folds its offset of eight into the integer: dot -= 8 * sum a. */
static float b32_slice(int type, const uint8_t* block, const uint8_t* rec, int slice) {
    const int8_t* a = rec_codes(rec) + 16 * slice;
    int32_t dot = 0, sum = 0;
    for (int i = 0; i < 16; ++i) {
        int code = type == RQO_Q8_0 ? (int8_t)block[2 + 16 * slice + i] : ((block[(type == RQO_Q4_1 ? 4 : 2) + i] >> (4 * slice)) & 15);
        dot += code * a[i];
        sum += a[i];
    }
    if (type == RQO_Q4_0) dot -= 8 * sum;
    float d = half_at(block), m = type == RQO_Q4_1 ? half_at(block + 2) : 0.0f; /* kind 3: the block minimum times the activation sum */
    float value = d * (float)dot + m * (float)sum;
    return rec_d(rec) * value;
}

/* build.rs:799-846. `recs` = the block's eight records. */
static void q4k_slice_ints(const uint8_t* block, const uint8_t* recs, int slice, int* sc, int* mn, int32_t* dot, int32_t* sum) {
    int group = slice / 2, half = slice & 1;
    q4k_scale_min(block + 4, group, sc, mn);
    const uint8_t* q = block + 16 + (group / 2) * 32 + 16 * half;
    const int8_t* a = rec_codes(recs + group * RQO_RECORD) + 16 * half;
    int shift = (group & 1) * 4;
    int32_t d = 0, s = 0;
    for (int i = 0; i < 16; ++i) { d += ((q[i] >> shift) & 15) * a[i]; s += a[i]; }
    *dot = d; *sum = s;
}
static float q4k_slice(const uint8_t* block, const uint8_t* recs, int slice) {
    int sc, mn; int32_t dot, sum;
    q4k_slice_ints(block, recs, slice, &sc, &mn, &dot, &sum);
    float group_d = half_at(block) * (float)sc;
    float group_dmin = half_at(block + 2) * (float)mn;
    float value = group_d * (float)dot - group_dmin * (float)sum;
    return rec_d(recs + (slice / 2) * RQO_RECORD) * value;
}

/* build.rs:883-915: r = d * (q8_d * (scale * f32(dot - 32 * sum a))), codes raw 0..63. */
static void q6k_word_ints(const uint8_t* block, const uint8_t* recs, int slice, int word, int32_t* dot, int32_t* sum) {
    int chunk = slice / 8, group = slice / 2, local = group % 4, half = slice & 1;
    const uint8_t* ql = block + 64 * chunk + 32 * (local & 1) + 16 * half + 4 * word;
    const uint8_t* qh = block + 128 + 32 * chunk + 16 * half + 4 * word;
    const int8_t* a = rec_codes(recs + group * RQO_RECORD) + 16 * half + 4 * word;
    int32_t d = 0, s = 0;
    for (int i = 0; i < 4; ++i) {
        int code = ((ql[i] >> (4 * (local / 2))) & 15) | (((qh[i] >> (2 * local)) & 3) << 4);
        d += code * a[i];
        s += a[i];
    }
    *dot = d; *sum = s;
}
static float q6k_slice(const uint8_t* block, const uint8_t* recs, int slice) {
    int32_t dot = 0, sum = 0;
    for (int w = 0; w < 4; ++w) { int32_t d, s; q6k_word_ints(block, recs, slice, w, &d, &s); dot += d; sum += s; }
    float scale = (float)(int8_t)block[192 + slice];
    float scaled = scale * (float)(dot - 32 * sum);
    float value = rec_d(recs + (slice / 2) * RQO_RECORD) * scaled;
    return half_at(block + 208) * value;
}

/* ------------------------------------------------------------ int8 dots, step 256 (a14) */

/* ll:1558-1732. `quarters` selects four fmas per block (rows a llama.cpp gemm would take)
 * instead of one (its gemv); a single-token step always folds the block whole. */
static float q4k_row_block_order(const uint8_t* row, int64_t blocks, const uint8_t* recs, int quarters) {
    float acc = 0.0f, accmin = 0.0f;
    for (int64_t b = 0; b < blocks; ++b) {
        const uint8_t* block = row + b * 144;
        const uint8_t* brec = recs + b * 8 * RQO_RECORD;
        int32_t dotq[4] = {0, 0, 0, 0}, minq[4] = {0, 0, 0, 0};
        for (int s = 0; s < 16; ++s) {
            int sc, mn; int32_t dot, sum;
            q4k_slice_ints(block, brec, s, &sc, &mn, &dot, &sum);
            dotq[s >> 2] += sc * dot;
            minq[s >> 2] += mn * sum;
        }
        float d8 = rec_d(brec);
        float scale = half_at(block) * d8;
        float dscale = half_at(block + 2) * d8;
        if (quarters) {
            for (int q = 0; q < 4; ++q) {
                acc = fmaf((float)dotq[q], scale, acc);
                accmin = fmaf((float)minq[q], dscale, accmin);
            }
        } else {
            int32_t dot_all = (dotq[0] + dotq[1]) + (dotq[2] + dotq[3]);
            int32_t min_all = (minq[0] + minq[1]) + (minq[2] + minq[3]);
            acc = fmaf((float)dot_all, scale, acc);
            accmin = fmaf((float)min_all, dscale, accmin);
        }
    }
    return acc - accmin;
}

/* ll:1846-2030 with build.rs:871-879. */
static float q6k_row_block_order(const uint8_t* row, int64_t blocks, const uint8_t* recs) {
    float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int64_t b = 0; b < blocks; ++b) {
        const uint8_t* block = row + b * 210;
        const uint8_t* brec = recs + b * 8 * RQO_RECORD;
        int32_t lanes[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int p = 0; p < 16; ++p) {
            int l = p & 7, is_sub = p >> 3;
            int32_t gathered = 0;
            for (int k = 0; k < 8; ++k) {
                int slice = is_sub ? 2 * l + (k >> 2) : 2 * k + (l >> 2);
                int word = is_sub ? (k & 3) : (l & 3);
                int32_t dot, sum;
                q6k_word_ints(block, brec, slice, word, &dot, &sum);
                int32_t scale = (int8_t)block[192 + slice];
                gathered += is_sub ? (scale * sum) * -32 : scale * dot;
            }
            lanes[l] += gathered;
        }
        float scale = rec_d(brec) * half_at(block + 208);
        for (int l = 0; l < 8; ++l) f[l] = fmaf(scale, (float)lanes[l], f[l]);
    }
    float t0 = f[0] + f[4], t1 = f[1] + f[5], t2 = f[2] + f[6], t3 = f[3] + f[7];
    return (t0 + t2) + (t1 + t3);
}

/* ------------------------------------------------------------------- exact dots (a15) */

/* build.rs:923-1022 `sums`: four fma chains (value i on chain i % 4), joined (0+1)+(2+3). */
static void exact_chains(const int* codes, const float* x, int64_t x_stride, float* acc16, float* xsum16) {
    float acc[4] = {0, 0, 0, 0}, xs[4] = {0, 0, 0, 0};
    for (int i = 0; i < 16; ++i) {
        float xi = x[i * x_stride];
        acc[i % 4] = fmaf((float)codes[i], xi, acc[i % 4]);
        xs[i % 4] = xs[i % 4] + xi;
    }
    *acc16 = (acc[0] + acc[1]) + (acc[2] + acc[3]);
    *xsum16 = (xs[0] + xs[1]) + (xs[2] + xs[3]);
}
/* One 16-value slice of the row's 256-value chunk starting at value `base`. */
static float exact_slice(int type, const uint8_t* row, int64_t base, int slice, const float* x, int64_t x_stride) {
    int codes[16];
    float acc16, xsum16;
    const float* xs = x + (base + 16 * slice) * x_stride;
    if (type == RQO_Q4_K) {
        const uint8_t* block = row + (base / 256) * 144;
        int group = slice / 2, sc, mn;
        q4k_scale_min(block + 4, group, &sc, &mn);
        for (int i = 0; i < 16; ++i) codes[i] = q4k_code(block, 16 * slice + i);
        exact_chains(codes, xs, x_stride, &acc16, &xsum16);
        float group_d = half_at(block) * (float)sc, group_dmin = half_at(block + 2) * (float)mn;
        return group_d * acc16 - group_dmin * xsum16;
    }
    if (type == RQO_Q6_K) {
        const uint8_t* block = row + (base / 256) * 210;
        for (int i = 0; i < 16; ++i) codes[i] = q6k_code(block, 16 * slice + i) - 32;
        exact_chains(codes, xs, x_stride, &acc16, &xsum16);
        float scaled = (float)(int8_t)block[192 + slice] * acc16;
        return half_at(block + 208) * scaled;
    }
    int bytes = rqo_block_bytes(type);
    const uint8_t* block = row + ((base + 16 * slice) / 32) * bytes;
    int half = slice & 1;
    for (int i = 0; i < 16; ++i) codes[i] = type == RQO_Q8_0 ? q80_code(block, 16 * half + i) : q40_code(block, 16 * half + i);
    exact_chains(codes, xs, x_stride, &acc16, &xsum16);
    float m = 0.0f;
    return half_at(block) * acc16 + m * xsum16;
}
/* ll:1734-1811 + :2125-2158 at wave width 1: 32 logical partial lanes per 256-value chunk
 * (lane L takes slices L, L+32, ...), a fixed tree over the 32, and the chunk's sum meets
 * the earlier chunks through the output (ll:2211-2224). */
static float exact_row(int type, const uint8_t* row, int64_t cols, const float* x, int64_t x_stride) {
    float carried = 0.0f;
    for (int64_t base = 0; base < cols; base += 256) {
        int64_t chunk = cols - base < 256 ? cols - base : 256;
        int slices = (int)(chunk / 16);
        float partial[32];
        for (int lane = 0; lane < 32; ++lane) {
            float sum = 0.0f;
            for (int s = lane; s < slices; s += 32) sum = sum + exact_slice(type, row, base, s, x, x_stride);
            partial[lane] = sum;
        }
        for (int off = 16; off > 0; off /= 2)
            for (int i = 0; i < off; ++i) partial[i] = partial[i] + partial[i + off];
        carried = base == 0 ? partial[0] : partial[0] + carried;
    }
    return carried;
}

/* -------------------------------------------------------------- run decoders (a16, a17) */

/* recipe.rs:7870-7903: one unit (a 256-value block, or 32 values) as a single fma chain in
 * index order over the dequantised weights. */
static float run_unit(int type, const uint8_t* block, const float* x, int64_t x_stride) {
    int n = rqo_block_values(type);
    float sum = 0.0f;
    for (int j = 0; j < n; ++j) sum = fmaf(block_value(type, block, j), x[j * x_stride], sum);
    return sum;
}
/* ll:3451-3492 at wave width 1: the row's units add in order into a zeroed sum. */
static float run_row(int type, const uint8_t* row, int64_t cols, const float* x, int64_t x_stride) {
    int n = rqo_block_values(type), bytes = rqo_block_bytes(type);
    float sum = 0.0f;
    for (int64_t u = 0; u < cols / n; ++u) sum = sum + run_unit(type, row + u * bytes, x + u * n * x_stride, x_stride);
    return sum;
}

/* --------------------------------------------------------------------------- matvec */

typedef struct {
    int type; const uint8_t* blocks; int64_t rows, cols;
    const float* x; int64_t x_stride; int tokens;
    float* y; int64_t y_stride; int act_mode, step;
    const uint8_t* records; /* [tokens][cols/32] records, int8 mode */
} matvec_ctx;

static void matvec_span(void* p, int64_t first, int64_t last, int worker, int workers) {
    (void)first; (void)last;
    matvec_ctx* c = (matvec_ctx*)p;
    int per = rqo_block_values(c->type), bytes = rqo_block_bytes(c->type);
    int64_t row_bytes = c->cols / per * bytes, row_blocks = c->cols / per;
    int64_t rec_per_token = c->cols / 32 * RQO_RECORD;
    /* row r belongs to worker r mod workers (recipe.rs:29264-29292; ll:1522-1526 with one wave per group) */
    for (int t = 0; t < c->tokens; ++t) {
        const float* x = c->x + t;
        const uint8_t* recs = c->records ? c->records + t * rec_per_token : NULL;
        for (int64_t r = worker; r < c->rows; r += workers) {
            const uint8_t* row = c->blocks + r * row_bytes;
            float sum;
            if (c->act_mode == RQO_ACT_FLOAT_RUN) {
                sum = run_row(c->type, row, c->cols, x, c->x_stride);
            } else if (c->act_mode == RQO_ACT_FLOAT_EXACT) {
                sum = exact_row(c->type, row, c->cols, x, c->x_stride);
            } else if (c->step == 256 && c->type == RQO_Q4_K) {
                /* ll:1698-1722: positions inside the first 4*(span/4) of a batch take four fmas per block */
                int quarters = t < c->tokens - (c->tokens & 3);
                sum = q4k_row_block_order(row, row_blocks, recs, quarters);
            } else if (c->step == 256 && c->type == RQO_Q6_K) {
                sum = q6k_row_block_order(row, row_blocks, recs);
            } else {
                /* ll:1813-1834, :2032-2053, :2057-2091: slices in increasing order, one add each */
                sum = 0.0f;
                int64_t slices = c->cols / 16;
                for (int64_t s = 0; s < slices; ++s) {
                    float r16;
                    if (c->type == RQO_Q4_K) r16 = q4k_slice(row + (s / 16) * 144, recs + (s / 16) * 8 * RQO_RECORD, (int)(s % 16));
                    else if (c->type == RQO_Q6_K) r16 = q6k_slice(row + (s / 16) * 210, recs + (s / 16) * 8 * RQO_RECORD, (int)(s % 16));
                    else r16 = b32_slice(c->type, row + (s / 2) * bytes, recs + (s / 2) * RQO_RECORD, (int)(s % 2));
                    sum = sum + r16;
                }
            }
            c->y[r * c->y_stride + t] = sum;
        }
    }
}

int rqo_matvec(int type, const uint8_t* blocks, int64_t rows, int64_t cols,
               const float* x, int64_t x_stride, int tokens,
               float* y, int64_t y_stride, int act_mode, int step, int threads) {
    int per = rqo_block_values(type);
    if (!per || rows < 0 || cols <= 0 || cols % per || tokens < 0) return -1;
    if (act_mode < 0 || act_mode > 2) return -1;
    if (act_mode == RQO_ACT_INT8 && step != 32 && step != 256) return -1;
    /* the other stored formats are dotted by the run decoders only; `.int(8)` re-encodes them first */
    if (act_mode != RQO_ACT_FLOAT_RUN && !type_has_slices(type) && !(act_mode == RQO_ACT_INT8 && type == RQO_Q4_1)) return -1;
    matvec_ctx c = {type, blocks, rows, cols, x, x_stride, tokens, y, y_stride, act_mode, step, NULL};
    uint8_t* records = NULL;
    if (act_mode == RQO_ACT_INT8) {
        records = (uint8_t*)malloc((size_t)tokens * (size_t)(cols / 32) * RQO_RECORD + 1);
        if (!records) return -2;
        for (int t = 0; t < tokens; ++t)
            rqo_quantize_activations(x + t, x_stride, cols, step, records + (size_t)t * (size_t)(cols / 32) * RQO_RECORD);
        c.records = records;
    }
    if (threads < 1) threads = 1;
    if (threads > rows && rows > 0) threads = (int)rows;
    /* one span per worker; the span bounds are unused, the worker index deals the rows */
    run_spans(threads, threads, matvec_span, &c);
    free(records);
    return 0;
}

/* ------------------------------------------------------------------ portable math */

/* build.rs:1079-1120, exponential_math("float", ..., 127, 254, 23, 88.72283905206835,
 * -103.972084045410, 8): every constant is the fp32 rounding of the double literal. */
static float exp_pow2(int k) {
    int biased = k + 127;
    if (biased < 0) biased = 0;
    if (biased > 254) biased = 254;
    return bits_f32((uint32_t)biased << 23);
}
float rqo_exp(float x) {
    if (x != x) return x;
    if (x > (float)88.72283905206835) return INFINITY;
    if (x < (float)-103.972084045410) return 0.0f;
    float scaled = x * (float)1.4426950408889634074; /* LOG2_E */
    float shifted = scaled + 0.5f;
    float kf = floorf(shifted);
    int k = (int)kf;
    union { uint64_t u; double d; } hi = {0x3FE62E42FEE00000ull};
    float upper = kf * (float)hi.d;
    float partial = x - upper;
    float lower = kf * (float)1.90821492927058770002e-10;
    float r = partial - lower;
    /* Horner over 1/1!, 1/2!, ..., 1/8!, innermost coefficient first, one fma per term */
    double factorial = 1.0, coeff[8];
    for (int t = 1; t <= 8; ++t) { factorial *= (double)t; coeff[t - 1] = 1.0 / factorial; }
    float current = (float)coeff[7];
    for (int t = 6; t >= 0; --t) current = fmaf(current, r, (float)coeff[t]);
    float body = r * current;
    float expanded = 1.0f + body;
    int half = k >> 1, rest = k - half;
    float scaled_once = expanded * exp_pow2(half);
    return scaled_once * exp_pow2(rest);
}

/* build.rs:1079-1120 with "double": 13 terms. */
static double exp_pow2_wide(int k) {
    int biased = k + 1023;
    if (biased < 0) biased = 0;
    if (biased > 2046) biased = 2046;
    union { uint64_t u; double d; } v = {(uint64_t)biased << 52};
    return v.d;
}
static double exp_wide(double x) {
    if (x != x) return x;
    if (x > 709.782712893383973096) return INFINITY;
    if (x < -745.133219101941108420) return 0.0;
    double scaled = x * 1.4426950408889634074;
    double shifted = scaled + 0.5;
    double kf = floor(shifted);
    int k = (int)kf;
    union { uint64_t u; double d; } hi = {0x3FE62E42FEE00000ull};
    double upper = kf * hi.d;
    double partial = x - upper;
    double lower = kf * 1.90821492927058770002e-10;
    double r = partial - lower;
    double factorial = 1.0, coeff[13];
    for (int t = 1; t <= 13; ++t) { factorial *= (double)t; coeff[t - 1] = 1.0 / factorial; }
    double current = coeff[12];
    for (int t = 11; t >= 0; --t) current = fma(current, r, coeff[t]);
    double body = r * current;
    double expanded = 1.0 + body;
    int half = k >> 1, rest = k - half;
    return expanded * exp_pow2_wide(half) * exp_pow2_wide(rest);
}
/* build.rs:1128-1142 */
static double expm1_wide(double x) {
    if (fabs(x) < 0.35) {
        double factorial = 1.0, coeff[16];
        for (int t = 1; t <= 16; ++t) { factorial *= (double)t; coeff[t - 1] = 1.0 / factorial; }
        double current = coeff[15];
        for (int t = 14; t >= 0; --t) current = fma(current, x, coeff[t]);
        return x * current;
    }
    return exp_wide(x) - 1.0;
}
/* build.rs:1146-1166: tanh = u / (u + 2), u = expm1(2x), in double, rounded once. */
float rqo_tanh(float x) {
    double w = (double)x;
    if (w != w) return x;
    if (fabs(w) >= 20.0) return w < 0.0 ? -1.0f : 1.0f;
    double u = expm1_wide(w * 2.0);
    return (float)(u / (u + 2.0));
}
/* recipe.rs:22662-22668 */
float rqo_sigmoid(float x) {
    float half_x = 0.5f * x;
    float curved = rqo_tanh(half_x);
    float shifted = curved + 1.0f;
    return 0.5f * shifted;
}
float rqo_silu(float x) { return x * rqo_sigmoid(x); }

/* ------------------------------------------------------------------ top-k routing */

/* ll:5007-5009: the template's own logistic, 1 / (1 + exp(-x)) -- not the tanh form the
 * activation programs use. */
static float logistic(float x) {
    float exponential = rqo_exp(-x);
    float denominator = 1.0f + exponential;
    return 1.0f / denominator;
}
/* ll:4486-4488 */
static float topk_score(float score, float maximum, int sigmoid) { return sigmoid ? logistic(score) : rqo_exp(score - maximum); }

/* ll:4666-4716 (serial body). weights doubles as the mark plane, as in the reference. */
int rqo_topk(const float* scores, int experts, int tokens, int top, int scoring, int renormalize,
             const float* selection_bias, float* weights) {
    if (experts <= 0 || top <= 0 || top > experts || tokens < 0) return -1;
    int sigmoid = scoring != 0, every = !renormalize, divide = renormalize || !sigmoid;
    for (int p = 0; p < tokens; ++p) {
        const float* s = scores + p;
        float* w = weights + p;
        float all_max = 0.0f;
        for (int e = 0; e < experts; ++e) if (e == 0 || s[(int64_t)e * tokens] > all_max) all_max = s[(int64_t)e * tokens];
        float all_total = 0.0f;
        for (int e = 0; e < experts; ++e) all_total = all_total + topk_score(s[(int64_t)e * tokens], all_max, sigmoid);
        for (int e = 0; e < experts; ++e) w[(int64_t)e * tokens] = 0.0f;
        for (int pick = 0; pick < top; ++pick) {
            int best = -1;
            float best_score = 0.0f;
            for (int e = 0; e < experts; ++e) {
                if (w[(int64_t)e * tokens] != 0.0f) continue;
                float score = s[(int64_t)e * tokens];
                float key = score;
                if (selection_bias) {
                    /* ll:4656-4659: probability over every expert plus the expert's bias */
                    float raw = topk_score(score, all_max, sigmoid);
                    float probability = sigmoid ? raw : raw / all_total;
                    key = probability + selection_bias[e];
                }
                if (best == -1 || key > best_score) { best = e; best_score = key; }
            }
            w[(int64_t)best * tokens] = 1.0f;
        }
        float maximum = 0.0f;
        int first = 1;
        for (int e = 0; e < experts; ++e) {
            int member = w[(int64_t)e * tokens] == 1.0f || every;
            float score = s[(int64_t)e * tokens];
            if (member && (first || score > maximum)) { maximum = score; first = 0; }
        }
        float total = 0.0f;
        for (int e = 0; e < experts; ++e) {
            int member = w[(int64_t)e * tokens] == 1.0f || every;
            float raw = topk_score(s[(int64_t)e * tokens], maximum, sigmoid);
            total = total + (member ? raw : 0.0f);
        }
        float denominator = divide ? total : 1.0f;
        for (int e = 0; e < experts; ++e) {
            int marked = w[(int64_t)e * tokens] == 1.0f;
            float raw = topk_score(s[(int64_t)e * tokens], maximum, sigmoid);
            w[(int64_t)e * tokens] = marked ? raw / denominator : 0.0f;
        }
    }
    return 0;
}

/* ----------------------------------------------------------------------- MoE block */

typedef struct {
    int type; const uint8_t *gate, *up, *down;
    int experts, top, hidden, ffn, tokens;
    const float* x; const float* routing; float* y;
    int accumulate;
} moe_ctx;

/* One position of lower_experts (recipe.rs:23386-23399) over the packed bodies
 * (ll:2304-2365): slots list the routed experts in ascending index; unfilled slots read
 * expert 0 at weight zero (ll:3189-3191). Mode 1 rows: slot = row / ffn. Mode 2 units are
 * scaled by their slot's weight before they add (ll:2359-2362). */
static void moe_position(const moe_ctx* c, int p, float* hbuf, float* xcol) {
    int per = rqo_block_values(c->type), bytes = rqo_block_bytes(c->type);
    int ids[64];
    float scales[64];
    int filled = 0;
    for (int s = 0; s < c->top; ++s) { ids[s] = 0; scales[s] = 0.0f; }
    for (int e = 0; e < c->experts && filled < c->top; ++e) {
        float w = c->routing[(int64_t)e * c->tokens + p];
        if (w != 0.0f) { ids[filled] = e; scales[filled] = w; ++filled; }
    }
    for (int k = 0; k < c->hidden; ++k) xcol[k] = c->x[(int64_t)k * c->tokens + p];
    int64_t in_row_bytes = (int64_t)c->hidden / per * bytes;   /* gate/up rows of `hidden` values */
    int64_t down_row_bytes = (int64_t)c->ffn / per * bytes;    /* down rows of `ffn` values */
    for (int s = 0; s < c->top; ++s)
        for (int f = 0; f < c->ffn; ++f) {
            int64_t row = (int64_t)ids[s] * c->ffn + f;
            float g = run_row(c->type, c->gate + row * in_row_bytes, c->hidden, xcol, 1);
            float u = run_row(c->type, c->up + row * in_row_bytes, c->hidden, xcol, 1);
            hbuf[s * c->ffn + f] = rqo_silu(g) * u; /* lower_gated, recipe.rs:23279-23286 */
        }
    int units_per_slot = c->ffn / per;
    for (int r = 0; r < c->hidden; ++r) {
        float sum = 0.0f;
        for (int s = 0; s < c->top; ++s) {
            const uint8_t* row = c->down + ((int64_t)ids[s] * c->hidden + r) * down_row_bytes;
            for (int u = 0; u < units_per_slot; ++u) {
                float part = 0.0f + run_unit(c->type, row + (int64_t)u * bytes, hbuf + s * c->ffn + u * per, 1);
                sum = sum + part * scales[s];
            }
        }
        float* out = c->y + (int64_t)r * c->tokens + p;
        *out = c->accumulate ? *out + sum : sum; /* binary Add of routed and shared, recipe.rs:23457 */
    }
}
static void moe_span(void* p, int64_t first, int64_t last, int worker, int workers) {
    (void)worker; (void)workers;
    const moe_ctx* c = (const moe_ctx*)p;
    float* hbuf = (float*)malloc(sizeof(float) * (size_t)c->top * (size_t)c->ffn);
    float* xcol = (float*)malloc(sizeof(float) * (size_t)c->hidden);
    for (int64_t t = first; t < last; ++t) moe_position(c, (int)t, hbuf, xcol);
    free(hbuf); free(xcol);
}

/* lower_gguf_moe, recipe.rs:23415-23459. The routed weights are multiplied by `routed_scale` first when it is not 1
 * (lower_scale after the top-k, :23426-23428). The shared expert is one more expert of width shared_count * ffn that every
 * position takes: at weight one (SharedExpert::Ungated, :23447) or at sigmoid(gate_vector . x) (Gated, :23448-23454). */
int rqo_moe_forward_ex(int type, const uint8_t* gate, const uint8_t* up, const uint8_t* down,
                       int experts, int top, int hidden, int ffn,
                       const float* x, const float* routing, int tokens, float routed_scale,
                       int shared_kind, int shared_count,
                       const uint8_t* sh_gate, const uint8_t* sh_up, const uint8_t* sh_down,
                       const float* shared_gate_w, float* y, int threads) {
    int per = rqo_block_values(type);
    if (!per || hidden % per || ffn % per || top > 64 || top < 1) return -1;
    if (shared_kind < 0 || shared_kind > 2 || (shared_kind && shared_count < 1) || (shared_kind == 2 && !shared_gate_w)) return -1;
    float* scaled = NULL;
    if (routed_scale != 1.0f) {
        scaled = (float*)malloc(sizeof(float) * (size_t)experts * (size_t)tokens);
        for (int64_t i = 0; i < (int64_t)experts * tokens; ++i) scaled[i] = routing[i] * routed_scale;
        routing = scaled;
    }
    moe_ctx routed = {type, gate, up, down, experts, top, hidden, ffn, tokens, x, routing, y, 0};
    run_spans(tokens, threads, moe_span, &routed);
    free(scaled);
    if (shared_kind) {
        float* weight = (float*)malloc(sizeof(float) * (size_t)tokens);
        for (int p = 0; p < tokens; ++p) {
            if (shared_kind == 1) { weight[p] = 1.0f; continue; }
            /* recipe.rs:23450-23453: a one-row bias-free contraction (dense sum loop, ll:2094-2123:
             * product then add, unfused), the gate activation, then one expert at that weight. */
            float sum = 0.0f;
            for (int k = 0; k < hidden; ++k) { float product = shared_gate_w[k] * x[(int64_t)k * tokens + p]; sum = sum + product; }
            weight[p] = rqo_sigmoid(sum);
        }
        moe_ctx shared = {type, sh_gate, sh_up, sh_down, 1, 1, hidden, ffn * shared_count, tokens, x, weight, y, 1};
        run_spans(tokens, threads, moe_span, &shared);
        free(weight);
    }
    return 0;
}

int rqo_moe_forward(int type, const uint8_t* gate, const uint8_t* up, const uint8_t* down,
                    int experts, int top, int hidden, int ffn,
                    const float* x, const float* routing, int tokens,
                    const uint8_t* sh_gate, const uint8_t* sh_up, const uint8_t* sh_down,
                    const float* shared_gate_w, float* y, int threads) {
    return rqo_moe_forward_ex(type, gate, up, down, experts, top, hidden, ffn, x, routing, tokens, 1.0f, shared_gate_w ? 2 : 0, 1, sh_gate, sh_up, sh_down,
                              shared_gate_w, y, threads);
}

/* ------------------------------------------------- the steps either side of a projection */

/* RMS normalisation of one position (emit_normalize_stats, recipe.rs:6836-7120, NormalizeMode::Rms, fp32 state, CPU wave
 * width 1): the squares are added in index order (square, then add: two operations), variance = sum / n,
 * scale = 1 / sqrt(variance + epsilon), y = (x * scale) * gain. gain may be NULL (no per-channel gain). */
void rqo_rmsnorm(const float* x, int64_t x_stride, int64_t n, const float* gain, float epsilon, float* y, int64_t y_stride) {
    float sum = 0.0f;
    for (int64_t k = 0; k < n; ++k) { float v = x[k * x_stride]; float square = v * v; sum = sum + square; }
    float variance = sum / (float)n;
    float adjusted = variance + epsilon;
    float deviation = sqrtf(adjusted);
    float scale = 1.0f / deviation;
    for (int64_t k = 0; k < n; ++k) {
        float v = x[k * x_stride] * scale;
        y[k * y_stride] = gain ? v * gain[k] : v;
    }
}

/* Logit soft-cap as the model scripts spell it (rnj-1.rs:47-51): scale(1 / cap), tanh, scale(cap), with the portable tanh. */
void rqo_softcap(const float* x, int64_t n, double cap, float* y) {
    float down = (float)(1.0 / cap), up = (float)cap;
    for (int64_t k = 0; k < n; ++k) y[k] = rqo_tanh(x[k] * down) * up;
}

/* lower_gated (recipe.rs:23279-23286): act(gate) * up, elementwise, silu with the portable transcendentals. */
void rqo_glu(const float* gate, const float* up, int64_t n, float* y) {
    for (int64_t k = 0; k < n; ++k) y[k] = rqo_silu(gate[k]) * up[k];
}

/* ------------------------------------------------------------------ synthetic inputs */

static inline uint64_t splitmix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
/* value i: two 53-bit uniforms from counters (2i, 2i+1) of the (seed, stream) key. */
void rqo_normal(uint64_t seed, uint64_t stream, int64_t first, int64_t count, double sigma, float* out) {
    uint64_t key = splitmix64(seed * 0x100000001B3ull + stream);
    for (int64_t i = 0; i < count; ++i) {
        uint64_t n = (uint64_t)(first + i);
        uint64_t a = splitmix64(key ^ splitmix64(2 * n));
        uint64_t b = splitmix64(key ^ splitmix64(2 * n + 1));
        double u1 = ((double)(a >> 11) + 1.0) * (1.0 / 9007199254740992.0); /* (0, 1] */
        double u2 = (double)(b >> 11) * (1.0 / 9007199254740992.0);         /* [0, 1) */
        double z = sqrt(-2.0 * log(u1)) * cos(6.283185307179586476925 * u2);
        out[i] = (float)(z * sigma);
    }
}
