// Per-value decode of a stored weight from its device planes, shared by the dequantiser and the
// load-time re-encoder. Every fp32 step is a separate rounded operation (__fmul_rn / __fsub_rn never
// contract), which makes the result bit-equal to the reference's f64 unpacking rounded to fp32
// (dequant_scalar / dequant_q45k / dequant_q6k / dequant_q2k / dequant_q3k / dequant_q8k / dequant_iq4, recipe.rs:3687-3958): d*sc, dmin*m and step*q are
// exact in fp32, and the one inexact step, the final subtract, rounds the same exact difference.
#pragma once
#include "rq_internal.cuh"

// Value i (row-major over rows x cols) of a weight whose planes are main_plane / scale_plane.
template <int TYPE>
__device__ __forceinline__ float rq_decode_value(const uint8_t* __restrict__ main_plane, const uint16_t* __restrict__ scale_plane, int64_t i, int64_t cols) {
    float value;
    if (TYPE == RQ_Q4_K) {
        int64_t b = i >> 8;
        int v = (int)(i & 255), sub = v >> 5, within = v & 31;
        const uint8_t* blk = main_plane + b * 144;
        const uint32_t* hdr = (const uint32_t*)blk;
        uint32_t dd = hdr[0];
        int sc, mn;
        rq_q4k_scale_min(hdr[1], hdr[2], hdr[3], sub, sc, mn);
        int q = (blk[16 + (sub >> 1) * 32 + within] >> ((sub & 1) * 4)) & 15;
        float step = __fmul_rn(rq_h2f((uint16_t)(dd & 0xffff)), (float)sc);
        float base = __fmul_rn(rq_h2f((uint16_t)(dd >> 16)), (float)mn);
        value = __fsub_rn(__fmul_rn(step, (float)q), base);
    } else if (TYPE == RQ_Q6_K) {
        int64_t b = i >> 8;
        int v = (int)(i & 255), chunk = v >> 7, local = v & 127, group = local >> 5, within = local & 31;
        const uint8_t* body = main_plane + b * 208;
        int lo = (body[64 * chunk + 32 * (group & 1) + within] >> (4 * (group >> 1))) & 15;
        int hi = (body[128 + 32 * chunk + within] >> (2 * group)) & 3;
        int code = (lo | (hi << 4)) - 32;
        int scale = (int8_t)body[192 + 8 * chunk + 2 * group + (within >> 4)];
        float scaled = __fmul_rn(rq_h2f(scale_plane[b]), (float)scale);
        value = __fmul_rn(scaled, (float)code);
    } else if (TYPE == RQ_Q8_0) {
        int64_t at = i;
        if (rq_plane_permuted(TYPE, cols)) {
            const int64_t row = i / cols, off = i - row * cols;  // one byte per value
            at = row * cols + ((rq_plane_chunk(TYPE, off >> 4) << 4) | (off & 15));
        }
        value = __fmul_rn((float)(int8_t)main_plane[at], rq_h2f(scale_plane[i >> 5]));
    } else if (TYPE == RQ_Q4_1 || TYPE == RQ_Q5_0 || TYPE == RQ_Q5_1 || TYPE == RQ_IQ4_NL) {
        // GGUF blocks as stored (dequant_scalar variants and dequant_iq4, recipe.rs:3782-3833, :3919-3958). Strides are even
        // and the plane is 256-byte aligned, so the fp16 header fields are aligned 16-bit loads.
        constexpr int kStride = TYPE == RQ_Q4_1 ? 20 : (TYPE == RQ_Q5_0 ? 22 : (TYPE == RQ_Q5_1 ? 24 : 18));
        constexpr int kHeader = (TYPE == RQ_Q4_1 || TYPE == RQ_Q5_1) ? 4 : 2;
        const uint8_t* blk = main_plane + (i >> 5) * kStride;
        const int v = (int)(i & 31);
        const float d = rq_h2f(*(const uint16_t*)blk);
        if (TYPE == RQ_Q4_1) {
            const int code = (blk[kHeader + (v & 15)] >> ((v >> 4) * 4)) & 15;
            value = __fadd_rn(__fmul_rn((float)code, d), rq_h2f(*(const uint16_t*)(blk + 2)));
        } else if (TYPE == RQ_IQ4_NL) {
            const int code = (blk[kHeader + (v & 15)] >> ((v >> 4) * 4)) & 15;
            // the sixteen levels (recipe.rs:15211), two eight-byte words indexed by shifts: no table in memory
            const unsigned long long lo = 0xF6EADDCFBFAD9881ull, hi = 0x7159453526190D01ull;
            const int level = (int)(int8_t)(((code < 8 ? lo : hi) >> (8 * (code & 7))) & 0xff);
            value = __fmul_rn(__fmul_rn(d, 1.0f), (float)level);
        } else {
            const int low = (blk[kHeader + 4 + (v & 15)] >> ((v >> 4) * 4)) & 15;
            const int high = (blk[kHeader + (v >> 3)] >> (v & 7)) & 1;
            const int code = low | (high << 4);
            if (TYPE == RQ_Q5_0) value = __fmul_rn((float)(code - 16), d);
            else value = __fadd_rn(__fmul_rn((float)code, d), rq_h2f(*(const uint16_t*)(blk + 2)));
        }
    } else if (TYPE == RQ_Q8_1) {
        // dequant_scalar, man 8 variant 1 (recipe.rs:3782-3833): header d, s; the value is code * d
        const uint8_t* blk = main_plane + (i >> 5) * 36;
        value = __fmul_rn((float)(int8_t)blk[4 + (i & 31)], rq_h2f(*(const uint16_t*)blk));
    } else if (TYPE == RQ_Q2_K) {
        // dequant_q2k (recipe.rs:3835-3866): scale | minimum << 4 per sixteen values, two-bit codes from byte 16, d @80, dmin @82
        const uint8_t* blk = main_plane + (i >> 8) * 84;
        const int v = (int)(i & 255), order = v >> 4, section = order >> 3, shift = 2 * ((order & 7) >> 1), half_index = order & 1;
        const int metadata = blk[section * 8 + shift + half_index];
        const int code = (blk[16 + section * 32 + half_index * 16 + (v & 15)] >> shift) & 3;
        const uint32_t dd = *(const uint32_t*)(blk + 80);
        const float scaled = __fmul_rn(rq_h2f((uint16_t)(dd & 0xffff)), (float)(metadata & 15));
        value = __fsub_rn(__fmul_rn(scaled, (float)code), __fmul_rn(rq_h2f((uint16_t)(dd >> 16)), (float)(metadata >> 4)));
    } else if (TYPE == RQ_Q3_K) {
        // dequant_q3k (recipe.rs:3868-3907): mask 0..31, codes 32..95, scales 96..107, d @108; a clear mask bit takes four off the code
        const uint8_t* blk = main_plane + (i >> 8) * 110;
        const int v = (int)(i & 255), block = v >> 4;
        const int low = (blk[96 + (block < 8 ? block : block - 8)] >> (block < 8 ? 0 : 4)) & 15;
        const int high = (blk[104 + (block & 3)] >> ((block >> 2) * 2)) & 3;
        const int scale_code = (low | (high << 4)) - 32;
        int code = (blk[32 + (v >> 7) * 32 + (v & 31)] >> (((v & 127) >> 5) * 2)) & 3;
        code -= ((blk[v & 31] >> (v >> 5)) & 1) ? 0 : 4;
        value = __fmul_rn(__fmul_rn(rq_h2f(*(const uint16_t*)(blk + 108)), (float)scale_code), (float)code);
    } else if (TYPE == RQ_Q8_K) {
        // dequant_q8k (recipe.rs:3909-3917): an fp32 step and 256 int8 codes from byte 4
        const uint8_t* blk = main_plane + (i >> 8) * 292;
        value = __fmul_rn(*(const float*)blk, (float)(int8_t)blk[4 + (i & 255)]);
    } else if (TYPE == RQ_IQ4_XS) {
        // dequant_iq4 with a six-bit exponent per 32 values (recipe.rs:3919-3958): high bits in the u16 @2, low bits in bytes 4..7
        const uint8_t* blk = main_plane + (i >> 8) * 136;
        const int v = (int)(i & 255), block = v >> 5;
        const int high = (*(const uint16_t*)(blk + 2) >> (2 * block)) & 3;
        const int low = (blk[4 + (block >> 1)] >> ((block & 1) * 4)) & 15;
        const int exponent = (low | (high << 4)) - 32;
        const int code = (blk[8 + block * 16 + (v & 15)] >> ((v & 31) < 16 ? 0 : 4)) & 15;
        const unsigned long long lo8 = 0xF6EADDCFBFAD9881ull, hi8 = 0x7159453526190D01ull;  // the sixteen levels, recipe.rs:15211
        const int level = (int)(int8_t)(((code < 8 ? lo8 : hi8) >> (8 * (code & 7))) & 0xff);
        value = __fmul_rn(__fmul_rn(rq_h2f(*(const uint16_t*)blk), (float)exponent), (float)level);
    } else if (TYPE == RQ_Q5_K) {
        // dequant_q45k with man = 5 (recipe.rs:3687-3741): nibbles from byte 48, fifth bits in bytes 16..47
        const uint8_t* blk = main_plane + (i >> 8) * 176;
        const int v = (int)(i & 255), sub = v >> 5, within = v & 31;
        const uint32_t* hdr = (const uint32_t*)blk;
        const uint32_t dd = hdr[0];
        int sc, mn;
        rq_q4k_scale_min(hdr[1], hdr[2], hdr[3], sub, sc, mn);
        const int low = (blk[48 + (sub >> 1) * 32 + within] >> ((sub & 1) * 4)) & 15;
        const int high = (blk[16 + within] >> sub) & 1;
        const float step = __fmul_rn(rq_h2f((uint16_t)(dd & 0xffff)), (float)sc);
        const float base = __fmul_rn(rq_h2f((uint16_t)(dd >> 16)), (float)mn);
        value = __fsub_rn(__fmul_rn(step, (float)(low | (high << 4))), base);
    } else {
        int64_t b = i >> 5;
        int v = (int)(i & 31);
        int64_t at = b * 16 + (v & 15);
        if (rq_plane_permuted(TYPE, cols)) {
            const int64_t row_bytes = cols >> 1, row = at / row_bytes, off = at - row * row_bytes;
            at = row * row_bytes + ((rq_plane_chunk(TYPE, off >> 4) << 4) | (off & 15));
        }
        int code = ((main_plane[at] >> ((v >> 4) * 4)) & 15) - 8;
        value = __fmul_rn((float)code, rq_h2f(scale_plane[b]));
    }
    return value;
}
