// Streaming matrix-vector kernel for sm_100a: the main path for inputs that are whole
// 256-value units per row (every K-quant tensor; 32-value formats when cols % 256 == 0).
//
// One persistent CTA per SM owns a contiguous range of rows. Rows are contiguous in HBM, so
// the range is one byte stream; a producer warp moves it into a ring of shared-memory stages
// with bulk asynchronous copies (cp.async.bulk, completion counted on an mbarrier), far
// enough ahead that HBM stays busy whatever the consumers do. The consumer warps wait on a
// stage, and each thread takes one ITEM: half of a 256-value unit of one row (four sub-blocks
// of a Q4_K block with their six-bit scales, one 128-value chunk of a Q6_K body, four Q8_0 /
// Q4_0 blocks). Items are dealt flat (thread t takes items t, t + threads, ... of the stage),
// so any row length fills the lanes; an item's partial sum goes to shared memory and one thread
// per row adds the row's partials in item order: no floating-point atomics, the same bits on
// every run.
// The activation column sits in shared memory as one padded record per 256 inputs (int8 codes
// with their steps and slice sums, or fp32 with slice sums), padded so that threads on
// adjacent units read different banks; it is staged while the first weight stages are in flight.
//
// Every wait on an mbarrier is bounded in time: when the limit runs out a thread records an
// error code in the context's flag word and stops waiting (it keeps walking its loop, so the
// CTA's barriers still balance); the CTA drains the copies it issued before it exits. A set
// flag makes the next rq_check() fail.
#include <string.h>

#include "rq_internal.cuh"


namespace {

constexpr int kMaxStages = 12;

// What a launch computes is described by a table of SEGMENTS of virtual output rows. A virtual
// row is made of `subs` sub-rows, each a row of some stored matrix dotted with one activation
// vector, and an epilogue joins the sub-row sums:
//   plain matvec        : 1 segment, 1 sub-row
//   q/k/v or gate/up    : one segment per matrix (they read the same activations), 1 sub-row
//   expert gate and up  : one segment per routed slot, 2 sub-rows (gate row, up row), out = silu(g) * u
//   expert down         : 1 segment, one sub-row per slot (each with its slot's activations and
//                         routing weight), out = sum_s coef_s * dot_s in slot order
struct StreamParams {
    const RqSegment* table;    // device memory, or null: use `inline_seg`
    const RqPlan* plan;        // device memory written by an earlier kernel: table and counts come from it
    int plan_count;            // > 1: a batch of planned launches in one -- grid row y reads plan[y * plan_stride] and the
    int plan_stride;           //      activations at x + y * x_plan_stride (one token of an expert bank per grid row)
    int64_t x_plan_stride;
    RqSegment inline_seg[RQ_INLINE_SEGMENTS];
    int n_segments, subs, epilogue;
    int64_t rows;              // virtual rows of all segments
    int64_t rows_quot; int rows_rem;  // rows / CTAs and rows % CTAs (launches whose row count the host knows): CTA b takes
                               // rows_quot rows from b * rows_quot + min(b, rows_rem), one more when b < rows_rem
    int cols, units;           // units = cols / 256 per row
    int unit_bytes;            // bytes of one unit in the main plane: 144, 208, 256, 128
    int scales_per_unit;       // fp16 d values per unit in the scale plane: 0, 1, 8, 8
    int stage_rows, stages;    // virtual rows per stage, ring depth
    int units_shift;           // log2(units) when that is a power of two, else -1
    size_t sub_main_bytes, sub_scale_bytes, stage_bytes, act_bytes, partial_bytes;  // shared-memory sizes
    int act_vectors;           // activation vectors staged in shared memory
    int act_regs;              // INT8, one token, every sub-row on vector 0: each thread keeps its activations in registers
    int warp_rows;             // > 0: the warp scheme -- a row's 2 * units items are that many adjacent lanes (a power of two), a warp
                               // pass covers warp_rows = 32 / (2 * units) rows, and the lanes of a row join their sums by shuffles
    int rows_per_thread;       // warp scheme: passes per stage (1 or 2)
    int interleaved;           // warp-scheme launches with an inline table: CTA b takes stages b, b + CTAs, b + 2 CTAs, ... of the launch
                               // (at any moment the CTAs read one moving window of memory; measured a little faster than a contiguous
                               // range per CTA). Claiming stages from a global ticket counter instead was tried and is slower: under
                               // load an atomic's round trip outlasts a stage.
    int total_stages, seg_stage_begin[RQ_INLINE_SEGMENTS + 1];  // interleaved: stages of the launch, and where each segment's stages begin
    int pieces, piece_rows;    // a stage lands as `pieces` copies with a barrier each (2 in the warp scheme with two passes: one per pass), piece_rows rows each
    int window;                // the producer keeps at most this many pieces in flight: enough bytes to cover the memory latency at full
                               // bandwidth, not more -- a deeper queue only delays everything else that reads memory (the activations)
    int row_warps;             // warp scheme: 1 = a row lies inside one warp; NW = every warp holds 32 / warp_rows lanes' worth of
                               // each row of the pass, and the warps' sums meet in shared memory (the last warp to arrive adds them)
    int sum_group, sum_chunks; // the order a row's item sums are added in when the shape has a warp scheme (so that a multi-token
                               // launch gives each token the bits a single-token launch gives it): chunks of sum_group items, an
                               // xor tree inside a chunk, chunks in order. sum_group = 0: items strided over eight lanes, then a tree
    int fuse_step;             // act_regs launches: 32 or 256 = quantise x in the prologue (no quantiser launch before), 0 = read `act`
    uint8_t* act_out;          // fused launches: CTA 0 leaves the records here for later INT8_CACHED calls
    const float* x; int64_t sk, st;   // FLOAT: vector v is x + v * st, element stride sk
    const uint8_t* act;        // INT8 activation scratch, one token's records after another
    int64_t yn, yt;
    int tokens;
    int* error_flag;
    unsigned long long wait_ns;  // a wait on an mbarrier gives up after this long (the context's limit, two seconds unless set)
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count)); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory"); }
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait: false when the time limit ran out (the caller records the error and stops waiting). Reading
// %globaltimer costs about a microsecond, so the clock is looked at only every 256th unsuccessful try (a try itself
// suspends the thread for a short, system-chosen time).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, unsigned long long limit_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    unsigned long long t0 = 0;
    uint32_t tries = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++tries & 255u) == 0) {
            const unsigned long long now = global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit_ns) return false;
        }
    }
    return true;
}
// Weights are read once per launch: the copies carry an evict-first L2 policy, so the stream does not push
// the activations, the outputs and the kernel's own code out of L2 between launches.
__device__ __forceinline__ uint64_t evict_first_policy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(smem_u32(dst)), "l"(src),
                 "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
                 : "memory");
}
template <int THREADS>
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(THREADS) : "memory"); }
__device__ __forceinline__ int dp4a_us(uint32_t a_unsigned, uint32_t b_signed, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_unsigned), "r"(b_signed), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) { return __dp4a((int)a, (int)b, c); }

// Four unsigned bytes of `w` as floats, exactly: 0x4B0000bb is 2^23 + bb.
__device__ __forceinline__ void bytes_to_float4(uint32_t w, float* f) {
    f[0] = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7650)) - 8388608.0f;
    f[1] = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7651)) - 8388608.0f;
    f[2] = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7652)) - 8388608.0f;
    f[3] = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7653)) - 8388608.0f;
}
// sum over 16 unsigned bytes (four words) times 16 floats
__device__ __forceinline__ float dot16f(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3, const float* x) {
    float f[4], s0 = 0.f, s1 = 0.f;
    uint32_t w[4] = {w0, w1, w2, w3};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        bytes_to_float4(w[j], f);
        s0 = fmaf(f[0], x[4 * j + 0], s0);
        s1 = fmaf(f[1], x[4 * j + 1], s1);
        s0 = fmaf(f[2], x[4 * j + 2], s0);
        s1 = fmaf(f[3], x[4 * j + 3], s1);
    }
    return s0 + s1;
}
__device__ __forceinline__ void load16f(const float* src, float* dst) {
#pragma unroll
    for (int j = 0; j < 4; ++j) *(float4*)(dst + 4 * j) = *(const float4*)(src + 4 * j);
}

// Two spellings the compiler might otherwise contract differently at different call sites (a row must have
// the same bits whichever path computes it): a - b * c as one fused operation, and a * b - c * d with the
// products rounded first.
__device__ __forceinline__ float minus_scaled(float a, float b, float c) { return fmaf(-b, c, a); }
__device__ __forceinline__ float diff_of_products(float a, float b, float c, float d) { return __fsub_rn(__fmul_rn(a, b), __fmul_rn(c, d)); }

// Activations of one token in shared memory: one padded record per 256 inputs.
//   INT8  (336 bytes): codes[256] int8 | d[8] fp32 @256 | sum16[16] int16 @288 | sum32[8] int16 @320
//          d = the step of each 32-value group, sum16 / sum32 = the sum of the codes of each
//          16-value slice / 32-value group
//   FLOAT (1104 bytes): x[256] fp32 | xsum16[16] fp32 @1024 | pad
// 336 = 84 words and 1104 = 276 words are both 20 mod 32, so the 128-bit loads of eight threads
// on adjacent units fall in eight different bank groups.

// The int8 activations one item needs: the 128 codes of its half record, their four steps, and
// the sums of its eight slices / four groups. A thread's item always covers the same inputs
// (its unit and half never change from stage to stage), so a single-token launch loads this
// once, from global memory, and keeps it in registers for the whole kernel.
struct ActHalf {
    uint32_t c[32];
    float d8[4];
    uint32_t s16w[4];  // eight int16 slice sums
    uint32_t g32w[2];  // four int16 group sums
    float dg[4];       // step x group sum, per group (the Q4_K minimum term)
    __device__ __forceinline__ void load(const uint8_t* rec, int h) {
        const uint4* cp = (const uint4*)(rec + 128 * h);
#pragma unroll
        for (int i = 0; i < 8; ++i) { const uint4 v = cp[i]; c[4 * i] = v.x; c[4 * i + 1] = v.y; c[4 * i + 2] = v.z; c[4 * i + 3] = v.w; }
        const float4 dv = *(const float4*)(rec + 256 + 16 * h);
        d8[0] = dv.x; d8[1] = dv.y; d8[2] = dv.z; d8[3] = dv.w;
        const uint4 sv = *(const uint4*)(rec + 288 + 16 * h);
        s16w[0] = sv.x; s16w[1] = sv.y; s16w[2] = sv.z; s16w[3] = sv.w;
        const uint2 gv = *(const uint2*)(rec + 320 + 8 * h);
        g32w[0] = gv.x; g32w[1] = gv.y;
#pragma unroll
        for (int i = 0; i < 4; ++i) dg[i] = d8[i] * (float)g32(i);
    }
    __device__ __forceinline__ int s16(int i) const { return (int)(int16_t)(s16w[i >> 1] >> (16 * (i & 1))); }
    __device__ __forceinline__ int g32(int i) const { return (int)(int16_t)(g32w[i >> 1] >> (16 * (i & 1))); }
};

// ------------------------------------------------------------------------------------------
// One item = half `h` of a 256-value unit, against the activation record `ar` of the unit
// (FLOAT) or the item's int8 activations `ah` (INT8).
// `w` = the unit in shared memory, `sc` = its fp16 d values in shared memory (not Q4_K).
// ------------------------------------------------------------------------------------------
template <int TYPE, int MODE>
__device__ __forceinline__ float item_dot(const uint8_t* __restrict__ w, const uint16_t* __restrict__ sc, const uint8_t* __restrict__ ar, const ActHalf& ah8, const int h, const int u) {
    const float* xf = (const float*)ar + 128 * h;      // FLOAT: the half's 128 inputs
    const float* xsum = (const float*)ar + 256 + 8 * h;  // and its eight slice sums
    if (TYPE == RQ_Q4_K) {
        const uint4 hdr = *(const uint4*)w;
        const float d = rq_h2f((uint16_t)(hdr.x & 0xffff)), dmin = rq_h2f((uint16_t)(hdr.x >> 16));
        // the four six-bit scales and minimums of sub-blocks 4h .. 4h+3, one per byte
        const uint32_t scw = h == 0 ? (hdr.y & 0x3f3f3f3fu) : ((hdr.w & 0x0f0f0f0fu) | ((hdr.y >> 2) & 0x30303030u));
        const uint32_t mnw = h == 0 ? (hdr.z & 0x3f3f3f3fu) : (((hdr.w >> 4) & 0x0f0f0f0fu) | ((hdr.z >> 2) & 0x30303030u));
        float acc_s = 0.f, acc_m = 0.f;
#pragma unroll
        for (int pp = 0; pp < 2; ++pp) {  // 32 bytes: sub-block 4h+2pp in the low nibbles, 4h+2pp+1 in the high
            const uint8_t* qp = w + 16 + 64 * h + 32 * pp;
            const uint4 q0 = *(const uint4*)qp, q1 = *(const uint4*)(qp + 16);
            const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
            const int sc_lo = (scw >> (16 * pp)) & 0xff, sc_hi = (scw >> (16 * pp + 8)) & 0xff;
            const int mn_lo = (mnw >> (16 * pp)) & 0xff, mn_hi = (mnw >> (16 * pp + 8)) & 0xff;
            if (MODE == RQ_ACT_INT8) {
                const uint32_t* al = ah8.c + 16 * pp;      // the 32 codes of sub-block 4h+2pp
                const uint32_t* ah = ah8.c + 16 * pp + 8;  // and of sub-block 4h+2pp+1
                int dl0 = 0, dl1 = 0, dh0 = 0, dh1 = 0;
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    dl0 = dp4a_us(qw[j] & 0x0F0F0F0Fu, al[j], dl0);
                    dl1 = dp4a_us(qw[j + 1] & 0x0F0F0F0Fu, al[j + 1], dl1);
                    dh0 = dp4a_us(qw[j] & 0xF0F0F0F0u, ah[j], dh0);  // sixteen times the high-nibble dot
                    dh1 = dp4a_us(qw[j + 1] & 0xF0F0F0F0u, ah[j + 1], dh1);
                }
                const int dl = dl0 + dl1, dh = (dh0 + dh1) >> 4;
                acc_s = fmaf(ah8.d8[2 * pp], (float)(sc_lo * dl), acc_s);
                acc_s = fmaf(ah8.d8[2 * pp + 1], (float)(sc_hi * dh), acc_s);
                acc_m = fmaf(ah8.dg[2 * pp], (float)mn_lo, acc_m);  // the same roundings as dot_regs
                acc_m = fmaf(ah8.dg[2 * pp + 1], (float)mn_hi, acc_m);
            } else {
                float xl[16], dl, dh;
                const float* xs = xf + 64 * pp;
                load16f(xs, xl);
                dl = dot16f(qw[0] & 0x0F0F0F0Fu, qw[1] & 0x0F0F0F0Fu, qw[2] & 0x0F0F0F0Fu, qw[3] & 0x0F0F0F0Fu, xl);
                load16f(xs + 16, xl);
                dl += dot16f(qw[4] & 0x0F0F0F0Fu, qw[5] & 0x0F0F0F0Fu, qw[6] & 0x0F0F0F0Fu, qw[7] & 0x0F0F0F0Fu, xl);
                load16f(xs + 32, xl);
                dh = dot16f((qw[0] >> 4) & 0x0F0F0F0Fu, (qw[1] >> 4) & 0x0F0F0F0Fu, (qw[2] >> 4) & 0x0F0F0F0Fu, (qw[3] >> 4) & 0x0F0F0F0Fu, xl);
                load16f(xs + 48, xl);
                dh += dot16f((qw[4] >> 4) & 0x0F0F0F0Fu, (qw[5] >> 4) & 0x0F0F0F0Fu, (qw[6] >> 4) & 0x0F0F0F0Fu, (qw[7] >> 4) & 0x0F0F0F0Fu, xl);
                const float4 xs4 = *(const float4*)(xsum + 4 * pp);
                acc_s = fmaf((float)sc_lo, dl, acc_s);
                acc_s = fmaf((float)sc_hi, dh, acc_s);
                acc_m = fmaf((float)mn_lo, xs4.x + xs4.y, acc_m);
                acc_m = fmaf((float)mn_hi, xs4.z + xs4.w, acc_m);
            }
        }
        return diff_of_products(d, acc_s, dmin, acc_m);
    } else if (TYPE == RQ_Q6_K) {
        // half h = the 128-value chunk h: ql lines 64h.., qh lines 128 + 32h.., scales 8h..8h+7
        const float d = rq_h2f(sc[0]);
        const uint2 s2 = *(const uint2*)(w + 192 + 8 * h);
        const uint32_t scales[2] = {s2.x, s2.y};  // eight int8 scales
        float acc = 0.f;
#pragma unroll
        for (int wh = 0; wh < 2; ++wh) {  // sixteen-byte half of the 32-byte lines
            const uint4 qh4 = *(const uint4*)(w + 128 + 32 * h + 16 * wh);
            const uint32_t qh[4] = {qh4.x, qh4.y, qh4.z, qh4.w};
#pragma unroll
            for (int gl = 0; gl < 2; ++gl) {
                const uint4 ql4 = *(const uint4*)(w + 64 * h + 32 * gl + 16 * wh);
                const uint32_t ql[4] = {ql4.x, ql4.y, ql4.z, ql4.w};
                // slices within the chunk: low nibbles -> group gl, high nibbles -> group gl + 2; slice 2 g + wh
                const int s_lo = 2 * gl + wh, s_hi = s_lo + 4;
                const int sc_lo = (int)(int8_t)(scales[s_lo >> 2] >> (8 * (s_lo & 3)));
                const int sc_hi = (int)(int8_t)(scales[s_hi >> 2] >> (8 * (s_hi & 3)));
                const int k_lo = 32 * gl + 16 * wh, k_hi = k_lo + 64;  // within the chunk
                if (MODE == RQ_ACT_INT8) {
                    // The dot is linear in the code's bit fields, so the fields are dotted where they lie
                    // (nibbles of ql, bit pairs of qh, as unsigned bytes) and the sums scaled afterwards:
                    // no six-bit code is ever assembled.
                    const uint32_t* alw = ah8.c + (k_lo >> 2);
                    const uint32_t* ahw = ah8.c + (k_hi >> 2);
                    constexpr uint32_t kPairLo = 0x03030303u, kPairHi = 0x30303030u;
                    int nl = 0, nh = 0, pl = 0, ph = 0;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        nl = dp4a_us(ql[j] & 0x0F0F0F0Fu, alw[j], nl);            // low nibbles
                        nh = dp4a_us(ql[j] & 0xF0F0F0F0u, ahw[j], nh);            // 16 x high nibbles
                        pl = dp4a_us(qh[j] & (kPairLo << (2 * gl)), alw[j], pl);  // 4^gl x the pair of group gl
                        ph = dp4a_us(qh[j] & (kPairHi << (2 * gl)), ahw[j], ph);  // 16 * 4^gl x the pair of group gl + 2
                    }
                    // code = nibble + 16 * pair, less the offset of 32 through the slice's sum of activations
                    const int dl = nl + ((pl >> (2 * gl)) << 4) - 32 * ah8.s16(k_lo >> 4);
                    const int dh = (nh >> 4) + (ph >> (2 * gl)) - 32 * ah8.s16(k_hi >> 4);
                    acc = fmaf(ah8.d8[k_lo >> 5], (float)(sc_lo * dl), acc);
                    acc = fmaf(ah8.d8[k_hi >> 5], (float)(sc_hi * dh), acc);
                } else {
                    uint32_t lo[4], hi[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        lo[j] = (ql[j] & 0x0F0F0F0Fu) | (((qh[j] >> (2 * gl)) & 0x03030303u) << 4);
                        hi[j] = ((ql[j] >> 4) & 0x0F0F0F0Fu) | (((qh[j] >> (2 * gl + 4)) & 0x03030303u) << 4);
                    }
                    float xv[16];
                    load16f(xf + k_lo, xv);
                    float dl = minus_scaled(dot16f(lo[0], lo[1], lo[2], lo[3], xv), 32.0f, xsum[k_lo >> 4]);
                    load16f(xf + k_hi, xv);
                    float dh = minus_scaled(dot16f(hi[0], hi[1], hi[2], hi[3], xv), 32.0f, xsum[k_hi >> 4]);
                    acc = fmaf((float)sc_lo, dl, acc);
                    acc = fmaf((float)sc_hi, dh, acc);
                }
            }
        }
        return d * acc;
    } else if (TYPE == RQ_Q8_0) {
        const uint2 dd = *(const uint2*)(sc + 4 * h);  // four fp16 d values
        const uint32_t dw[2] = {dd.x, dd.y};
        float acc = 0.f;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const float d = rq_h2f((uint16_t)(dw[b >> 1] >> (16 * (b & 1))));
            // chunks 8h + 2b and 8h + 2b + 1 of the unit, at their permuted places (rq_plane_chunk)
            const uint4 q0 = *(const uint4*)(w + 16 * ((8 * h + 2 * b) ^ (u & 7))), q1 = *(const uint4*)(w + 16 * ((8 * h + 2 * b + 1) ^ (u & 7)));
            if (MODE == RQ_ACT_INT8) {
                const uint32_t* a0 = ah8.c + 8 * b;
                const uint32_t* a1 = a0 + 4;
                int dot = dp4a_ss(q0.x, a0[0], 0), dot1 = dp4a_ss(q1.x, a1[0], 0);
                dot = dp4a_ss(q0.y, a0[1], dot); dot1 = dp4a_ss(q1.y, a1[1], dot1);
                dot = dp4a_ss(q0.z, a0[2], dot); dot1 = dp4a_ss(q1.z, a1[2], dot1);
                dot = dp4a_ss(q0.w, a0[3], dot); dot1 = dp4a_ss(q1.w, a1[3], dot1);
                acc = fmaf(ah8.d8[b] * d, (float)(dot + dot1), acc);
            } else {
                float xv[16];
                load16f(xf + 32 * b, xv);
                // codes biased by 128 to unsigned bytes; the bias leaves through the slice sums of x
                float dot = dot16f(q0.x ^ 0x80808080u, q0.y ^ 0x80808080u, q0.z ^ 0x80808080u, q0.w ^ 0x80808080u, xv);
                load16f(xf + 32 * b + 16, xv);
                dot += dot16f(q1.x ^ 0x80808080u, q1.y ^ 0x80808080u, q1.z ^ 0x80808080u, q1.w ^ 0x80808080u, xv);
                acc = fmaf(d, minus_scaled(dot, 128.0f, xsum[2 * b] + xsum[2 * b + 1]), acc);
            }
        }
        return acc;
    } else {  // Q4_0: four blocks of sixteen bytes
        const uint2 dd = *(const uint2*)(sc + 4 * h);
        const uint32_t dw[2] = {dd.x, dd.y};
        float acc = 0.f;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const float d = rq_h2f((uint16_t)(dw[b >> 1] >> (16 * (b & 1))));
            const uint4 q = *(const uint4*)(w + 16 * ((4 * h + b) ^ (u & 7)));  // chunk 4h + b of the unit, at its permuted place
            const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
            if (MODE == RQ_ACT_INT8) {
                const uint32_t* alw = ah8.c + 8 * b;
                const uint32_t* ahw = alw + 4;
                int dl = 0, dh = 0;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    dl = dp4a_us(qw[j] & 0x0F0F0F0Fu, alw[j], dl);
                    dh = dp4a_us(qw[j] & 0xF0F0F0F0u, ahw[j], dh);
                }
                const int dot = dl + (dh >> 4) - 8 * ah8.g32(b);
                acc = fmaf(ah8.d8[b] * d, (float)dot, acc);
            } else {
                float xv[16];
                load16f(xf + 32 * b, xv);
                float dot = dot16f(qw[0] & 0x0F0F0F0Fu, qw[1] & 0x0F0F0F0Fu, qw[2] & 0x0F0F0F0Fu, qw[3] & 0x0F0F0F0Fu, xv);
                load16f(xf + 32 * b + 16, xv);
                dot += dot16f((qw[0] >> 4) & 0x0F0F0F0Fu, (qw[1] >> 4) & 0x0F0F0F0Fu, (qw[2] >> 4) & 0x0F0F0F0Fu, (qw[3] >> 4) & 0x0F0F0F0Fu, xv);
                acc = fmaf(d, minus_scaled(dot, 8.0f, xsum[2 * b] + xsum[2 * b + 1]), acc);
            }
        }
        return acc;
    }
}

// ------------------------------------------------------------------------------------------
// Four tokens against one item (INT8). The tokens' records of a unit are interleaved in shared memory
// (kRecord4 bytes per unit), so that one 128-bit load brings the same word of all four tokens:
//   word k of the codes (k < 64) of token t  at 16 k + 4 t
//   step of group g (g < 8)                  at 1024 + 16 g + 4 t
//   sum of slice s (s < 16), int16           at 1152 + 8 s + 2 t
//   sum of group g, int16                    at 1280 + 8 g + 2 t
// 1360 bytes = 85 sixteen-byte lines, an odd count: the loads of eight threads on adjacent units fall
// in eight different bank groups. A weight word is masked once and dotted with four tokens; every
// token's float operations are those of item_dot, in its order, so the sums are bit for bit the same.
// ------------------------------------------------------------------------------------------
constexpr int kRecord4 = 1360;
__device__ __forceinline__ uint32_t lane_of(const uint4& v, int t) { return t == 0 ? v.x : (t == 1 ? v.y : (t == 2 ? v.z : v.w)); }
__device__ __forceinline__ float lane_of(const float4& v, int t) { return t == 0 ? v.x : (t == 1 ? v.y : (t == 2 ? v.z : v.w)); }
__device__ __forceinline__ int short_of(const uint2& v, int t) { return (int)(int16_t)((t < 2 ? v.x : v.y) >> (16 * (t & 1))); }

template <int TYPE>
__device__ __forceinline__ void item_dot_tok4(const uint8_t* __restrict__ w, const uint16_t* __restrict__ sc, const uint8_t* __restrict__ rec, const int h, const int u, float (&out)[4]) {
    const uint4* codes = (const uint4*)rec + 32 * h;              // the half's 32 code words, four tokens each
    const float4* steps = (const float4*)(rec + 1024) + 4 * h;    // its four group steps
    const uint2* sum16 = (const uint2*)(rec + 1152) + 8 * h;      // its eight slice sums
    const uint2* sum32 = (const uint2*)(rec + 1280) + 4 * h;      // its four group sums
    if (TYPE == RQ_Q4_K) {
        const uint4 hdr = *(const uint4*)w;
        const float d = rq_h2f((uint16_t)(hdr.x & 0xffff)), dmin = rq_h2f((uint16_t)(hdr.x >> 16));
        const uint32_t scw = h == 0 ? (hdr.y & 0x3f3f3f3fu) : ((hdr.w & 0x0f0f0f0fu) | ((hdr.y >> 2) & 0x30303030u));
        const uint32_t mnw = h == 0 ? (hdr.z & 0x3f3f3f3fu) : (((hdr.w >> 4) & 0x0f0f0f0fu) | ((hdr.z >> 2) & 0x30303030u));
        float acc_s[4] = {0.f, 0.f, 0.f, 0.f}, acc_m[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int pp = 0; pp < 2; ++pp) {
            const uint8_t* qp = w + 16 + 64 * h + 32 * pp;
            const uint4 q0 = *(const uint4*)qp, q1 = *(const uint4*)(qp + 16);
            const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
            const int sc_lo = (scw >> (16 * pp)) & 0xff, sc_hi = (scw >> (16 * pp + 8)) & 0xff;
            const int mn_lo = (mnw >> (16 * pp)) & 0xff, mn_hi = (mnw >> (16 * pp + 8)) & 0xff;
            int dl[4] = {0, 0, 0, 0}, dh[4] = {0, 0, 0, 0};
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t lo = qw[j] & 0x0F0F0F0Fu, hi = qw[j] & 0xF0F0F0F0u;
                const uint4 al = codes[16 * pp + j], ah = codes[16 * pp + 8 + j];
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    dl[t] = dp4a_us(lo, lane_of(al, t), dl[t]);
                    dh[t] = dp4a_us(hi, lane_of(ah, t), dh[t]);  // sixteen times the high-nibble dot
                }
            }
            const float4 d_lo = steps[2 * pp], d_hi = steps[2 * pp + 1];
            const uint2 g_lo = sum32[2 * pp], g_hi = sum32[2 * pp + 1];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                acc_s[t] = fmaf(lane_of(d_lo, t), (float)(sc_lo * dl[t]), acc_s[t]);
                acc_s[t] = fmaf(lane_of(d_hi, t), (float)(sc_hi * (dh[t] >> 4)), acc_s[t]);
                acc_m[t] = fmaf(__fmul_rn(lane_of(d_lo, t), (float)short_of(g_lo, t)), (float)mn_lo, acc_m[t]);
                acc_m[t] = fmaf(__fmul_rn(lane_of(d_hi, t), (float)short_of(g_hi, t)), (float)mn_hi, acc_m[t]);
            }
        }
#pragma unroll
        for (int t = 0; t < 4; ++t) out[t] = diff_of_products(d, acc_s[t], dmin, acc_m[t]);
    } else if (TYPE == RQ_Q6_K) {
        const float d = rq_h2f(sc[0]);
        const uint2 s2 = *(const uint2*)(w + 192 + 8 * h);
        const uint32_t scales[2] = {s2.x, s2.y};
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int wh = 0; wh < 2; ++wh) {
            const uint4 qh4 = *(const uint4*)(w + 128 + 32 * h + 16 * wh);
            const uint32_t qh[4] = {qh4.x, qh4.y, qh4.z, qh4.w};
#pragma unroll
            for (int gl = 0; gl < 2; ++gl) {
                const uint4 ql4 = *(const uint4*)(w + 64 * h + 32 * gl + 16 * wh);
                const uint32_t ql[4] = {ql4.x, ql4.y, ql4.z, ql4.w};
                const int s_lo = 2 * gl + wh, s_hi = s_lo + 4;
                const int sc_lo = (int)(int8_t)(scales[s_lo >> 2] >> (8 * (s_lo & 3)));
                const int sc_hi = (int)(int8_t)(scales[s_hi >> 2] >> (8 * (s_hi & 3)));
                const int k_lo = 32 * gl + 16 * wh, k_hi = k_lo + 64;
                constexpr uint32_t kPairLo = 0x03030303u, kPairHi = 0x30303030u;
                int nl[4] = {0, 0, 0, 0}, nh[4] = {0, 0, 0, 0}, pl[4] = {0, 0, 0, 0}, ph[4] = {0, 0, 0, 0};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t m_nl = ql[j] & 0x0F0F0F0Fu, m_nh = ql[j] & 0xF0F0F0F0u;
                    const uint32_t m_pl = qh[j] & (kPairLo << (2 * gl)), m_ph = qh[j] & (kPairHi << (2 * gl));
                    const uint4 al = codes[(k_lo >> 2) + j], ah = codes[(k_hi >> 2) + j];
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        nl[t] = dp4a_us(m_nl, lane_of(al, t), nl[t]);
                        nh[t] = dp4a_us(m_nh, lane_of(ah, t), nh[t]);
                        pl[t] = dp4a_us(m_pl, lane_of(al, t), pl[t]);
                        ph[t] = dp4a_us(m_ph, lane_of(ah, t), ph[t]);
                    }
                }
                const float4 d_lo = steps[k_lo >> 5], d_hi = steps[k_hi >> 5];
                const uint2 a_lo = sum16[k_lo >> 4], a_hi = sum16[k_hi >> 4];
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const int dl = nl[t] + ((pl[t] >> (2 * gl)) << 4) - 32 * short_of(a_lo, t);
                    const int dh = (nh[t] >> 4) + (ph[t] >> (2 * gl)) - 32 * short_of(a_hi, t);
                    acc[t] = fmaf(lane_of(d_lo, t), (float)(sc_lo * dl), acc[t]);
                    acc[t] = fmaf(lane_of(d_hi, t), (float)(sc_hi * dh), acc[t]);
                }
            }
        }
#pragma unroll
        for (int t = 0; t < 4; ++t) out[t] = d * acc[t];
    } else if (TYPE == RQ_Q8_0) {
        const uint2 dd = *(const uint2*)(sc + 4 * h);
        const uint32_t dw[2] = {dd.x, dd.y};
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const float d = rq_h2f((uint16_t)(dw[b >> 1] >> (16 * (b & 1))));
            const uint4 q0 = *(const uint4*)(w + 16 * ((8 * h + 2 * b) ^ (u & 7))), q1 = *(const uint4*)(w + 16 * ((8 * h + 2 * b + 1) ^ (u & 7)));
            const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
            int dot[4] = {0, 0, 0, 0};
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint4 a = codes[8 * b + j];
#pragma unroll
                for (int t = 0; t < 4; ++t) dot[t] = dp4a_ss(qw[j], lane_of(a, t), dot[t]);
            }
            const float4 d8 = steps[b];
#pragma unroll
            for (int t = 0; t < 4; ++t) acc[t] = fmaf(__fmul_rn(lane_of(d8, t), d), (float)dot[t], acc[t]);
        }
#pragma unroll
        for (int t = 0; t < 4; ++t) out[t] = acc[t];
    } else {  // Q4_0
        const uint2 dd = *(const uint2*)(sc + 4 * h);
        const uint32_t dw[2] = {dd.x, dd.y};
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const float d = rq_h2f((uint16_t)(dw[b >> 1] >> (16 * (b & 1))));
            const uint4 q = *(const uint4*)(w + 16 * ((4 * h + b) ^ (u & 7)));
            const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
            int dl[4] = {0, 0, 0, 0}, dh[4] = {0, 0, 0, 0};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t lo = qw[j] & 0x0F0F0F0Fu, hi = qw[j] & 0xF0F0F0F0u;
                const uint4 al = codes[8 * b + j], ah = codes[8 * b + 4 + j];
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    dl[t] = dp4a_us(lo, lane_of(al, t), dl[t]);
                    dh[t] = dp4a_us(hi, lane_of(ah, t), dh[t]);
                }
            }
            const float4 d8 = steps[b];
            const uint2 g = sum32[b];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const int dot = dl[t] + (dh[t] >> 4) - 8 * short_of(g, t);
                acc[t] = fmaf(__fmul_rn(lane_of(d8, t), d), (float)dot, acc[t]);
            }
        }
#pragma unroll
        for (int t = 0; t < 4; ++t) out[t] = acc[t];
    }
}

// ------------------------------------------------------------------------------------------
// Register-resident items (single-token INT8 launches): a thread copies its item's weights out
// of the stage into registers and releases the stage at once, so the ring slot is busy only while
// the bytes are in flight, and works on two items at a time for instruction-level parallelism.
// ------------------------------------------------------------------------------------------
template <int TYPE> struct ItemRegs;
template <> struct ItemRegs<RQ_Q4_K> {
    uint4 hdr, q[4];
    __device__ __forceinline__ void load(const uint8_t* w, const uint16_t*, int h, int) {
        hdr = *(const uint4*)w;
        const uint4* qp = (const uint4*)(w + 16 + 64 * h);
        q[0] = qp[0]; q[1] = qp[1]; q[2] = qp[2]; q[3] = qp[3];
    }
};
template <> struct ItemRegs<RQ_Q6_K> {
    uint4 ql[4], qh[2];  // ql[2 * gl + wh], qh[wh]
    uint2 sc;
    uint32_t d16;
    __device__ __forceinline__ void load(const uint8_t* w, const uint16_t* scp, int h, int) {
        const uint4* lp = (const uint4*)(w + 64 * h);
        ql[0] = lp[0]; ql[1] = lp[1]; ql[2] = lp[2]; ql[3] = lp[3];
        const uint4* hp = (const uint4*)(w + 128 + 32 * h);
        qh[0] = hp[0]; qh[1] = hp[1];
        sc = *(const uint2*)(w + 192 + 8 * h);
        d16 = scp[0];
    }
};
template <> struct ItemRegs<RQ_Q8_0> {
    uint4 q[8];
    uint2 dd;
    __device__ __forceinline__ void load(const uint8_t* w, const uint16_t* scp, int h, int u) {
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = *(const uint4*)(w + 16 * ((8 * h + i) ^ (u & 7)));  // logical order in registers
        dd = *(const uint2*)(scp + 4 * h);
    }
};
template <> struct ItemRegs<RQ_Q4_0> {
    uint4 q[4];
    uint2 dd;
    __device__ __forceinline__ void load(const uint8_t* w, const uint16_t* scp, int h, int u) {
#pragma unroll
        for (int i = 0; i < 4; ++i) q[i] = *(const uint4*)(w + 16 * ((4 * h + i) ^ (u & 7)));  // logical order in registers
        dd = *(const uint2*)(scp + 4 * h);
    }
};

// An integer of magnitude below 2^22 as a float, exactly, without the conversion unit:
// 0x4B400000 is 1.5 * 2^23, whose mantissa takes the integer as it is.
__device__ __forceinline__ float small_int_to_float(int v) { return __int_as_float(0x4B400000 + v) - 12582912.0f; }

__device__ __forceinline__ float dot_regs(const ItemRegs<RQ_Q4_K>& r, const ActHalf& a, const int h) {
    const uint4 hdr = r.hdr;
    const float d = rq_h2f((uint16_t)(hdr.x & 0xffff)), dmin = rq_h2f((uint16_t)(hdr.x >> 16));
    const uint32_t scw = h == 0 ? (hdr.y & 0x3f3f3f3fu) : ((hdr.w & 0x0f0f0f0fu) | ((hdr.y >> 2) & 0x30303030u));
    const uint32_t mnw = h == 0 ? (hdr.z & 0x3f3f3f3fu) : (((hdr.w >> 4) & 0x0f0f0f0fu) | ((hdr.z >> 2) & 0x30303030u));
    float mn[4];
    bytes_to_float4(mnw, mn);
    float acc_s = 0.f, acc_m = 0.f;
#pragma unroll
    for (int pp = 0; pp < 2; ++pp) {
        const uint4 q0 = r.q[2 * pp], q1 = r.q[2 * pp + 1];
        const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        const int sc_lo = (int)__byte_perm(scw, 0, 0x4440 + 2 * pp), sc_hi = (int)__byte_perm(scw, 0, 0x4441 + 2 * pp);
        const uint32_t* al = a.c + 16 * pp;
        const uint32_t* ah = a.c + 16 * pp + 8;
        int dl0 = 0, dl1 = 0, dh0 = 0, dh1 = 0;
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
            dl0 = dp4a_us(qw[j] & 0x0F0F0F0Fu, al[j], dl0);
            dl1 = dp4a_us(qw[j + 1] & 0x0F0F0F0Fu, al[j + 1], dl1);
            dh0 = dp4a_us(qw[j] & 0xF0F0F0F0u, ah[j], dh0);  // sixteen times the high-nibble dot
            dh1 = dp4a_us(qw[j + 1] & 0xF0F0F0F0u, ah[j + 1], dh1);
        }
        // |scale * dot| <= 63 * 32 * 15 * 128 < 2^22
        acc_s = fmaf(a.d8[2 * pp], small_int_to_float(sc_lo * (dl0 + dl1)), acc_s);
        acc_s = fmaf(a.d8[2 * pp + 1], small_int_to_float(sc_hi * ((dh0 + dh1) >> 4)), acc_s);
        acc_m = fmaf(a.dg[2 * pp], mn[2 * pp], acc_m);
        acc_m = fmaf(a.dg[2 * pp + 1], mn[2 * pp + 1], acc_m);
    }
    return diff_of_products(d, acc_s, dmin, acc_m);
}

__device__ __forceinline__ float dot_regs(const ItemRegs<RQ_Q6_K>& r, const ActHalf& a, const int) {
    const float d = rq_h2f((uint16_t)r.d16);
    const uint32_t scales[2] = {r.sc.x, r.sc.y};
    float acc = 0.f;
#pragma unroll
    for (int wh = 0; wh < 2; ++wh) {
        const uint32_t qh[4] = {r.qh[wh].x, r.qh[wh].y, r.qh[wh].z, r.qh[wh].w};
#pragma unroll
        for (int gl = 0; gl < 2; ++gl) {
            const uint4 ql4 = r.ql[2 * gl + wh];
            const uint32_t ql[4] = {ql4.x, ql4.y, ql4.z, ql4.w};
            const int s_lo = 2 * gl + wh, s_hi = s_lo + 4;
            const int sc_lo = (int)(int8_t)(scales[s_lo >> 2] >> (8 * (s_lo & 3)));
            const int sc_hi = (int)(int8_t)(scales[s_hi >> 2] >> (8 * (s_hi & 3)));
            const int k_lo = 32 * gl + 16 * wh, k_hi = k_lo + 64;
            const uint32_t* alw = a.c + (k_lo >> 2);
            const uint32_t* ahw = a.c + (k_hi >> 2);
            constexpr uint32_t kPairLo = 0x03030303u, kPairHi = 0x30303030u;
            int nl = 0, nh = 0, pl = 0, ph = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                nl = dp4a_us(ql[j] & 0x0F0F0F0Fu, alw[j], nl);
                nh = dp4a_us(ql[j] & 0xF0F0F0F0u, ahw[j], nh);
                pl = dp4a_us(qh[j] & (kPairLo << (2 * gl)), alw[j], pl);
                ph = dp4a_us(qh[j] & (kPairHi << (2 * gl)), ahw[j], ph);
            }
            const int dl = nl + ((pl >> (2 * gl)) << 4) - 32 * a.s16(k_lo >> 4);
            const int dh = (nh >> 4) + (ph >> (2 * gl)) - 32 * a.s16(k_hi >> 4);
            acc = fmaf(a.d8[k_lo >> 5], (float)(sc_lo * dl), acc);
            acc = fmaf(a.d8[k_hi >> 5], (float)(sc_hi * dh), acc);
        }
    }
    return d * acc;
}

__device__ __forceinline__ float dot_regs(const ItemRegs<RQ_Q8_0>& r, const ActHalf& a, const int) {
    const uint32_t dw[2] = {r.dd.x, r.dd.y};
    float acc = 0.f;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        const float d = rq_h2f((uint16_t)(dw[b >> 1] >> (16 * (b & 1))));
        const uint4 q0 = r.q[2 * b], q1 = r.q[2 * b + 1];
        const uint32_t* a0 = a.c + 8 * b;
        const uint32_t* a1 = a0 + 4;
        int dot = dp4a_ss(q0.x, a0[0], 0), dot1 = dp4a_ss(q1.x, a1[0], 0);
        dot = dp4a_ss(q0.y, a0[1], dot); dot1 = dp4a_ss(q1.y, a1[1], dot1);
        dot = dp4a_ss(q0.z, a0[2], dot); dot1 = dp4a_ss(q1.z, a1[2], dot1);
        dot = dp4a_ss(q0.w, a0[3], dot); dot1 = dp4a_ss(q1.w, a1[3], dot1);
        acc = fmaf(a.d8[b] * d, (float)(dot + dot1), acc);
    }
    return acc;
}

__device__ __forceinline__ float dot_regs(const ItemRegs<RQ_Q4_0>& r, const ActHalf& a, const int) {
    const uint32_t dw[2] = {r.dd.x, r.dd.y};
    float acc = 0.f;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        const float d = rq_h2f((uint16_t)(dw[b >> 1] >> (16 * (b & 1))));
        const uint32_t qw[4] = {r.q[b].x, r.q[b].y, r.q[b].z, r.q[b].w};
        const uint32_t* alw = a.c + 8 * b;
        const uint32_t* ahw = alw + 4;
        int dl = 0, dh = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            dl = dp4a_us(qw[j] & 0x0F0F0F0Fu, alw[j], dl);
            dh = dp4a_us(qw[j] & 0xF0F0F0F0u, ahw[j], dh);
        }
        const int dot = dl + (dh >> 4) - 8 * a.g32(b);
        acc = fmaf(a.d8[b] * d, (float)dot, acc);
    }
    return acc;
}

// ------------------------------------------------------------------------------------------
// fp32 activations in the warp scheme: the weights of the thread's R rows sit in registers, the
// item's 128 inputs come from the unit record in shared memory sixteen at a time, and each
// sixteen serve all R rows. Per row the operations and their order are item_dot's, so a row has
// the same bits whichever path computes it.
// ------------------------------------------------------------------------------------------
template <int R>
__device__ __forceinline__ void dot_regs_float(const ItemRegs<RQ_Q4_K> (&r)[R], const bool (&have)[R], const uint8_t* __restrict__ ar, const int h, float (&out)[R]) {
    const float* xf = (const float*)ar + 128 * h;
    const float* xsum = (const float*)ar + 256 + 8 * h;
    float acc_s[R], acc_m[R];
    uint32_t scw[R], mnw[R];
#pragma unroll
    for (int k = 0; k < R; ++k) {
        const uint4 hdr = r[k].hdr;
        scw[k] = h == 0 ? (hdr.y & 0x3f3f3f3fu) : ((hdr.w & 0x0f0f0f0fu) | ((hdr.y >> 2) & 0x30303030u));
        mnw[k] = h == 0 ? (hdr.z & 0x3f3f3f3fu) : (((hdr.w >> 4) & 0x0f0f0f0fu) | ((hdr.z >> 2) & 0x30303030u));
        acc_s[k] = 0.f; acc_m[k] = 0.f;
    }
#pragma unroll
    for (int pp = 0; pp < 2; ++pp) {
        float dl[R], dh[R], xl[16];
        const float* xs = xf + 64 * pp;
        load16f(xs, xl);
#pragma unroll
        for (int k = 0; k < R; ++k) { const uint4 q = r[k].q[2 * pp]; dl[k] = dot16f(q.x & 0x0F0F0F0Fu, q.y & 0x0F0F0F0Fu, q.z & 0x0F0F0F0Fu, q.w & 0x0F0F0F0Fu, xl); }
        load16f(xs + 16, xl);
#pragma unroll
        for (int k = 0; k < R; ++k) { const uint4 q = r[k].q[2 * pp + 1]; dl[k] += dot16f(q.x & 0x0F0F0F0Fu, q.y & 0x0F0F0F0Fu, q.z & 0x0F0F0F0Fu, q.w & 0x0F0F0F0Fu, xl); }
        load16f(xs + 32, xl);
#pragma unroll
        for (int k = 0; k < R; ++k) { const uint4 q = r[k].q[2 * pp]; dh[k] = dot16f((q.x >> 4) & 0x0F0F0F0Fu, (q.y >> 4) & 0x0F0F0F0Fu, (q.z >> 4) & 0x0F0F0F0Fu, (q.w >> 4) & 0x0F0F0F0Fu, xl); }
        load16f(xs + 48, xl);
#pragma unroll
        for (int k = 0; k < R; ++k) { const uint4 q = r[k].q[2 * pp + 1]; dh[k] += dot16f((q.x >> 4) & 0x0F0F0F0Fu, (q.y >> 4) & 0x0F0F0F0Fu, (q.z >> 4) & 0x0F0F0F0Fu, (q.w >> 4) & 0x0F0F0F0Fu, xl); }
        const float4 xs4 = *(const float4*)(xsum + 4 * pp);
#pragma unroll
        for (int k = 0; k < R; ++k) {
            const int sc_lo = (scw[k] >> (16 * pp)) & 0xff, sc_hi = (scw[k] >> (16 * pp + 8)) & 0xff;
            const int mn_lo = (mnw[k] >> (16 * pp)) & 0xff, mn_hi = (mnw[k] >> (16 * pp + 8)) & 0xff;
            acc_s[k] = fmaf((float)sc_lo, dl[k], acc_s[k]);
            acc_s[k] = fmaf((float)sc_hi, dh[k], acc_s[k]);
            acc_m[k] = fmaf((float)mn_lo, xs4.x + xs4.y, acc_m[k]);
            acc_m[k] = fmaf((float)mn_hi, xs4.z + xs4.w, acc_m[k]);
        }
    }
#pragma unroll
    for (int k = 0; k < R; ++k) {
        const float d = rq_h2f((uint16_t)(r[k].hdr.x & 0xffff)), dmin = rq_h2f((uint16_t)(r[k].hdr.x >> 16));
        out[k] = have[k] ? diff_of_products(d, acc_s[k], dmin, acc_m[k]) : 0.f;
    }
}

template <int R>
__device__ __forceinline__ void dot_regs_float(const ItemRegs<RQ_Q6_K> (&r)[R], const bool (&have)[R], const uint8_t* __restrict__ ar, const int h, float (&out)[R]) {
    const float* xf = (const float*)ar + 128 * h;
    const float* xsum = (const float*)ar + 256 + 8 * h;
    float acc[R];
#pragma unroll
    for (int k = 0; k < R; ++k) acc[k] = 0.f;
#pragma unroll
    for (int wh = 0; wh < 2; ++wh) {
#pragma unroll
        for (int gl = 0; gl < 2; ++gl) {
            const int s_lo = 2 * gl + wh, s_hi = s_lo + 4;
            const int k_lo = 32 * gl + 16 * wh, k_hi = k_lo + 64;  // within the chunk
            float xv[16], dl[R], dh[R];
            load16f(xf + k_lo, xv);
#pragma unroll
            for (int k = 0; k < R; ++k) {
                const uint4 ql4 = r[k].ql[2 * gl + wh], qh4 = r[k].qh[wh];
                const uint32_t ql[4] = {ql4.x, ql4.y, ql4.z, ql4.w}, qh[4] = {qh4.x, qh4.y, qh4.z, qh4.w};
                uint32_t lo[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) lo[j] = (ql[j] & 0x0F0F0F0Fu) | (((qh[j] >> (2 * gl)) & 0x03030303u) << 4);
                dl[k] = minus_scaled(dot16f(lo[0], lo[1], lo[2], lo[3], xv), 32.0f, xsum[k_lo >> 4]);
            }
            load16f(xf + k_hi, xv);
#pragma unroll
            for (int k = 0; k < R; ++k) {
                const uint4 ql4 = r[k].ql[2 * gl + wh], qh4 = r[k].qh[wh];
                const uint32_t ql[4] = {ql4.x, ql4.y, ql4.z, ql4.w}, qh[4] = {qh4.x, qh4.y, qh4.z, qh4.w};
                uint32_t hi[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) hi[j] = ((ql[j] >> 4) & 0x0F0F0F0Fu) | (((qh[j] >> (2 * gl + 4)) & 0x03030303u) << 4);
                dh[k] = minus_scaled(dot16f(hi[0], hi[1], hi[2], hi[3], xv), 32.0f, xsum[k_hi >> 4]);
            }
#pragma unroll
            for (int k = 0; k < R; ++k) {
                const uint32_t scales[2] = {r[k].sc.x, r[k].sc.y};
                const int sc_lo = (int)(int8_t)(scales[s_lo >> 2] >> (8 * (s_lo & 3)));
                const int sc_hi = (int)(int8_t)(scales[s_hi >> 2] >> (8 * (s_hi & 3)));
                acc[k] = fmaf((float)sc_lo, dl[k], acc[k]);
                acc[k] = fmaf((float)sc_hi, dh[k], acc[k]);
            }
        }
    }
#pragma unroll
    for (int k = 0; k < R; ++k) out[k] = have[k] ? rq_h2f((uint16_t)r[k].d16) * acc[k] : 0.f;
}

template <int R>
__device__ __forceinline__ void dot_regs_float(const ItemRegs<RQ_Q8_0> (&r)[R], const bool (&have)[R], const uint8_t* __restrict__ ar, const int h, float (&out)[R]) {
    const float* xf = (const float*)ar + 128 * h;
    const float* xsum = (const float*)ar + 256 + 8 * h;
    float acc[R];
#pragma unroll
    for (int k = 0; k < R; ++k) acc[k] = 0.f;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        float xv[16], dot[R];
        load16f(xf + 32 * b, xv);
#pragma unroll
        for (int k = 0; k < R; ++k) { const uint4 q0 = r[k].q[2 * b]; dot[k] = dot16f(q0.x ^ 0x80808080u, q0.y ^ 0x80808080u, q0.z ^ 0x80808080u, q0.w ^ 0x80808080u, xv); }
        load16f(xf + 32 * b + 16, xv);
#pragma unroll
        for (int k = 0; k < R; ++k) {
            const uint4 q1 = r[k].q[2 * b + 1];
            dot[k] += dot16f(q1.x ^ 0x80808080u, q1.y ^ 0x80808080u, q1.z ^ 0x80808080u, q1.w ^ 0x80808080u, xv);
            const uint32_t dw[2] = {r[k].dd.x, r[k].dd.y};
            const float d = rq_h2f((uint16_t)(dw[b >> 1] >> (16 * (b & 1))));
            acc[k] = fmaf(d, minus_scaled(dot[k], 128.0f, xsum[2 * b] + xsum[2 * b + 1]), acc[k]);
        }
    }
#pragma unroll
    for (int k = 0; k < R; ++k) out[k] = have[k] ? acc[k] : 0.f;
}

template <int R>
__device__ __forceinline__ void dot_regs_float(const ItemRegs<RQ_Q4_0> (&r)[R], const bool (&have)[R], const uint8_t* __restrict__ ar, const int h, float (&out)[R]) {
    const float* xf = (const float*)ar + 128 * h;
    const float* xsum = (const float*)ar + 256 + 8 * h;
    float acc[R];
#pragma unroll
    for (int k = 0; k < R; ++k) acc[k] = 0.f;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        float xv[16], dot[R];
        load16f(xf + 32 * b, xv);
#pragma unroll
        for (int k = 0; k < R; ++k) { const uint4 q = r[k].q[b]; dot[k] = dot16f(q.x & 0x0F0F0F0Fu, q.y & 0x0F0F0F0Fu, q.z & 0x0F0F0F0Fu, q.w & 0x0F0F0F0Fu, xv); }
        load16f(xf + 32 * b + 16, xv);
#pragma unroll
        for (int k = 0; k < R; ++k) {
            const uint4 q = r[k].q[b];
            dot[k] += dot16f((q.x >> 4) & 0x0F0F0F0Fu, (q.y >> 4) & 0x0F0F0F0Fu, (q.z >> 4) & 0x0F0F0F0Fu, (q.w >> 4) & 0x0F0F0F0Fu, xv);
            const uint32_t dw[2] = {r[k].dd.x, r[k].dd.y};
            const float d = rq_h2f((uint16_t)(dw[b >> 1] >> (16 * (b & 1))));
            acc[k] = fmaf(d, minus_scaled(dot[k], 8.0f, xsum[2 * b] + xsum[2 * b + 1]), acc[k]);
        }
    }
#pragma unroll
    for (int k = 0; k < R; ++k) out[k] = have[k] ? acc[k] : 0.f;
}

// The int8 activation quantiser inside the matvec's prologue: the CTA's consumer threads turn the
// `cols` inputs of one token into unit records in shared memory. A thread owns slices of sixteen
// inputs, one slice per round, the next round's loads in flight while it works on this round's;
// the two threads of a 32-value group, or the sixteen of a 256-value group, agree on the extreme
// by shuffles. Same arithmetic as the standalone quantiser: the extreme is the FIRST input of
// strictly largest magnitude, inverse = -127 / extreme, d = 1 / inverse (IEEE divides),
// code = clamp(rint(x * inverse)).
template <int THREADS>
__device__ __forceinline__ void quantise_to_smem(const float* __restrict__ x, int64_t sk, int cols, int step, uint8_t* __restrict__ rec_base, int tid) {
    constexpr int kRecord = RQ_ACT_RECORD_INT8;
    const int slices = cols >> 4;
    const bool vec = sk == 1 && ((uintptr_t)x & 15) == 0;
    auto fetch = [&](int sl, float* v) {
        if (sl < slices) {
            if (vec) {
#pragma unroll
                for (int j = 0; j < 4; ++j) *(float4*)&v[4 * j] = __ldg((const float4*)(x + 16 * (int64_t)sl) + j);
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = __ldg(x + (16 * (int64_t)sl + j) * sk);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = 0.f;
        }
    };
    // one slice per thread per round; the next round's inputs are on their way while this round's are worked on
    float cur[16], nxt[16];
    fetch(tid, cur);
#pragma unroll 1
    for (int base = 0; base < slices; base += THREADS) {  // uniform over the CTA: every lane takes part in the shuffles
        const int sl = base + tid;
        fetch(sl + THREADS, nxt);
        const int slot = sl & 15;                 // slice within its unit
        float best = 0.f;
        int best_at = 0x7fffffff;
#pragma unroll
        for (int j = 0; j < 16; ++j)
            if (fabsf(cur[j]) > fabsf(best)) { best = cur[j]; best_at = 16 * slot + j; }
        const int reach = step == 32 ? 1 : 8;     // partners: lane ^ 1, or the sixteen lanes of the unit
        for (int off = 1; off <= reach; off <<= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, off);
            const int oa = __shfl_xor_sync(0xffffffffu, best_at, off);
            const bool take = fabsf(ob) > fabsf(best) || (fabsf(ob) == fabsf(best) && oa < best_at);
            if (take) { best = ob; best_at = oa; }
        }
        const bool nonzero = fabsf(best) > 0.f;
        const float inverse = nonzero ? __fdiv_rn(-127.0f, best) : 0.f;
        const float d = nonzero ? __fdiv_rn(1.0f, inverse) : 0.f;
        uint32_t cw[4];
        int sum = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t word = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                int code = __float2int_rn(__fmul_rn(cur[4 * j + b], inverse));
                code = code < -128 ? -128 : (code > 127 ? 127 : code);
                sum += code;
                word |= (uint32_t)(code & 0xff) << (8 * b);
            }
            cw[j] = word;
        }
        const int pair_sum = sum + __shfl_xor_sync(0xffffffffu, sum, 1);
        if (sl < slices) {
            uint8_t* rec = rec_base + (size_t)(sl >> 4) * kRecord;
            *(uint4*)(rec + 16 * slot) = make_uint4(cw[0], cw[1], cw[2], cw[3]);
            ((int16_t*)(rec + 288))[slot] = (int16_t)sum;
            if ((slot & 1) == 0) {
                ((float*)(rec + 256))[slot >> 1] = d;
                ((int16_t*)(rec + 320))[slot >> 1] = (int16_t)pair_sum;
            }
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) cur[j] = nxt[j];
    }
}

// recipe's portable transcendentals for the expert epilogue (build.rs:1079-1176, math = "portable"):
// tanh(x) = u / (u + 2), u = expm1(2x), evaluated in double and rounded once; sigmoid and silu as
// the activation programs spell them (recipe.rs:22662-22668).
__device__ double rq_exp_wide(double x) {
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
    auto pow2 = [](int e) { int b = e + 1023; b = b < 0 ? 0 : (b > 2046 ? 2046 : b); return __longlong_as_double((long long)b << 52); };
    return expanded * pow2(half) * pow2(rest);
}
__device__ float rq_tanh_portable(float xf) {
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
        u = rq_exp_wide(z) - 1.0;
    }
    return (float)(u / (u + 2.0));
}
__device__ __forceinline__ float rq_sigmoid_portable(float x) { return __fmul_rn(0.5f, __fadd_rn(rq_tanh_portable(__fmul_rn(0.5f, x)), 1.0f)); }
__device__ __forceinline__ float rq_silu_portable(float x) { return __fmul_rn(x, rq_sigmoid_portable(x)); }

// R = rows a thread takes per stage in the warp scheme (its weight registers): 2 only where the launch uses two
template <int TYPE, int MODE, int T, int NW, int R>
__global__ void __launch_bounds__(NW * 32 + 32, NW == 5 ? (T == 2 ? 2 : 3) : (NW <= 7 ? 2 : 1)) rq_gemv_stream_kernel(const __grid_constant__ StreamParams p) {
    constexpr int kConsumers = NW * 32;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t full_bar[2 * kMaxStages];  // [slot][piece]
    __shared__ __align__(8) uint64_t empty_bar[kMaxStages];
    constexpr int kRecord = MODE == RQ_ACT_INT8 ? RQ_ACT_RECORD_INT8 : RQ_ACT_RECORD_FLOAT;
    uint8_t* act_smem = smem;                                              // activation vectors x units records
    float* partial = (float*)(smem + p.act_bytes * p.act_vectors);         // [2][T][stage items]
    uint8_t* ring = smem + p.act_bytes * p.act_vectors + p.partial_bytes;  // stages

    const int tid = threadIdx.x;
    const int64_t row_bytes = (int64_t)p.units * p.unit_bytes;
    const int row_scales = p.units * p.scales_per_unit;
    const int stage_items = 2 * p.subs * p.stage_rows * p.units;
    // The segment table sits in shared memory for the whole kernel: the producer and the consumers
    // both index it with run-time values.
    __shared__ RqSegment table[RQ_MAX_SEGMENTS];
    __shared__ int plan_counts[4];
    // what the producer put into each ring slot: rows, segment, first row (local to the segment), and where the
    // first d value sits inside its 16-byte-aligned copy. Written before the copies are issued, read after they land.
    __shared__ int4 stage_info[kMaxStages];
    // warp scheme with rows split over the warps: per stage in flight, each warp's sum of each row, and how many warps have
    // delivered. A warp is never more than the ring's depth ahead of the slowest, so kMaxStages + 1 buffers never collide.
    constexpr int TR = T == 2 ? 2 : 1;  // tokens a thread keeps in registers (the warp schemes)
    __shared__ float cross_sum[kMaxStages + 1][TR][8][NW];
    __shared__ int cross_count[kMaxStages + 1];

    // Programmatic dependent launch: the next kernel in the stream may start its own prologue now.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int batch_row = p.plan_count > 1 ? (int)blockIdx.y : 0;
    const RqPlan* const plan = p.plan ? p.plan + (size_t)batch_row * p.plan_stride : nullptr;
    const float* const xbase = p.x + (size_t)batch_row * p.x_plan_stride;
    const int tok0 = p.plan_count > 1 ? 0 : blockIdx.y * T;
    // An inline table came with the launch and the weights are constants of the model: the producer of such a
    // launch streams weights from its first instruction on, whatever the previous kernel is doing. A table or
    // plan in device memory may have been written by the kernel before: it is read after griddepcontrol.wait.
    const bool direct = p.table == nullptr && p.plan == nullptr;
    // fused launches: every warp of the CTA, the producer's included, takes part in quantising x
    const bool fused = MODE == RQ_ACT_INT8 && p.act_regs && p.fuse_step != 0;
    constexpr int kThreads = NW * 32 + 32;
    int n_segments = p.n_segments, subs = p.subs;
    int64_t row_begin = 0, row_end = 0;
    auto split_rows = [&](int64_t rows) {
        if (p.plan) {
            row_begin = (rows * (int64_t)blockIdx.x) / gridDim.x;
            row_end = (rows * (int64_t)(blockIdx.x + 1)) / gridDim.x;
        } else {
            const int b = (int)blockIdx.x;
            row_begin = b * p.rows_quot + (b < p.rows_rem ? b : p.rows_rem);
            row_end = row_begin + p.rows_quot + (b < p.rows_rem ? 1 : 0);
        }
    };

    if (tid >= kConsumers) {
        // ---------------------------------------------------------------- producer warp (lane 0 works)
        int issued = 0, seg = 0, slot = 0, st = 0, n_pieces = 0;
        uint32_t phase = 1;  // parity of the slot's previous round: the first round of the ring waits for nothing
        int64_t r = 0;
        const RqSegment* segs = p.inline_seg;
        bool failed = false;
        const uint64_t policy = evict_first_policy();
        // issues stages until `limit` have been issued or the rows run out
        const int grid = (int)gridDim.x;
        int my_stage = (int)blockIdx.x;  // interleaved launches: the stage to issue next
        auto issue = [&](int limit) {
            for (; st < limit && !failed; ++st) {
                int nr;
                int64_t lr0;  // first row, local to the segment
                if (p.interleaved) {
                    if (my_stage >= p.total_stages) break;
                    seg = 0;
                    while (seg + 1 < n_segments && my_stage >= p.seg_stage_begin[seg + 1]) ++seg;
                    lr0 = (int64_t)(my_stage - p.seg_stage_begin[seg]) * p.stage_rows;
                    const int64_t left = segs[seg].rows - lr0;
                    nr = (int)(left < p.stage_rows ? left : p.stage_rows);
                    my_stage += grid;
                } else {
                    if (r >= row_end) break;
                    while (seg + 1 < n_segments && r >= segs[seg].row_begin + segs[seg].rows) ++seg;
                    const int64_t seg_end = segs[seg].row_begin + segs[seg].rows;
                    int64_t stop = r + p.stage_rows;
                    if (stop > seg_end) stop = seg_end;
                    if (stop > row_end) stop = row_end;
                    nr = (int)(stop - r);
                    lr0 = r - segs[seg].row_begin;
                    r = stop;
                }
                const RqSegment& sg = segs[seg];
                if (st >= p.stages && !mbar_wait(&empty_bar[slot], phase, p.wait_ns)) { atomicExch(p.error_flag, 1); failed = true; break; }
                uint8_t* dst = ring + (size_t)slot * p.stage_bytes;
                stage_info[slot] = make_int4(nr, seg, (int)lr0,
                                             TYPE != RQ_Q4_K ? (int)(((uintptr_t)sg.scale[0] + (uintptr_t)(lr0 * row_scales * 2)) & 15) : 0);
                for (int k = 0; k < p.pieces; ++k) {
                    // at most `window` pieces in flight: wait for the one issued `window` pieces ago
                    if (n_pieces >= p.window) {
                        const int old_piece = n_pieces - p.window, old_st = old_piece / p.pieces;
                        if (!mbar_wait(&full_bar[2 * (old_st % p.stages) + (old_piece - old_st * p.pieces)], (old_st / p.stages) & 1, p.wait_ns)) { atomicExch(p.error_flag, 4); failed = true; break; }
                    }
                    ++n_pieces;
                    uint64_t* bar = &full_bar[2 * slot + k];
                    int rows_k = nr - k * p.piece_rows;
                    rows_k = rows_k < 0 ? 0 : (rows_k > p.piece_rows ? p.piece_rows : rows_k);
                    if (p.pieces == 1) rows_k = nr;
                    const uint32_t main_bytes = (uint32_t)(rows_k * row_bytes);
                    // bytes first, then the copies: the barrier must expect them before any can complete.
                    // The d values of the whole stage travel with its first piece.
                    uint32_t total = main_bytes * subs;
                    if (TYPE != RQ_Q4_K && k == 0) {
                        for (int s = 0; s < subs; ++s) {
                            // the rows' d values, widened to whole 16-byte lines (the plane has slack past its end)
                            const uintptr_t first = (uintptr_t)sg.scale[s] + (uintptr_t)(lr0 * row_scales * 2);
                            const uintptr_t last = first + (uintptr_t)nr * row_scales * 2;
                            total += (uint32_t)(((last + 15) & ~(uintptr_t)15) - (first & ~(uintptr_t)15));
                        }
                    }
                    mbar_expect_tx(bar, total);
                    const int64_t piece_off = (int64_t)k * p.piece_rows * row_bytes;
                    for (int s = 0; s < subs; ++s) {
                        if (main_bytes) bulk_g2s(dst + (size_t)s * p.sub_main_bytes + piece_off, sg.main[s] + lr0 * row_bytes + piece_off, main_bytes, bar, policy);
                        if (TYPE != RQ_Q4_K && k == 0) {
                            const uintptr_t first = (uintptr_t)sg.scale[s] + (uintptr_t)(lr0 * row_scales * 2);
                            const uintptr_t last = first + (uintptr_t)nr * row_scales * 2;
                            const uintptr_t a0 = first & ~(uintptr_t)15, a1 = (last + 15) & ~(uintptr_t)15;
                            bulk_g2s(dst + (size_t)p.subs * p.sub_main_bytes + (size_t)s * p.sub_scale_bytes, (const void*)a0, (uint32_t)(a1 - a0), bar, policy);
                        }
                    }
                }
                if (failed) break;
                issued = st + 1;
                if (++slot == p.stages) { slot = 0; phase ^= 1; }
            }
        };
        if (tid == kConsumers) {
            for (int s = 0; s < p.stages; ++s) { mbar_init(&full_bar[2 * s], 1); mbar_init(&full_bar[2 * s + 1], 1); mbar_init(&empty_bar[s], NW); }
            for (int s = 0; s <= kMaxStages; ++s) cross_count[s] = 0;
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            if (!direct) {
                // the table or plan is in device memory and may come from the kernel before: wait for that one, then read it
                // from there (the consumers are copying it to shared memory meanwhile)
                asm volatile("griddepcontrol.wait;" ::: "memory");
                int64_t rows = p.rows;
                if (p.plan) {
                    segs = plan->seg;
                    n_segments = min(plan->n_segments, p.n_segments); subs = min(plan->subs, p.subs);
                    rows = min((int64_t)plan->total_rows, p.rows);
                } else {
                    segs = p.table;
                }
                split_rows(rows);
                r = row_begin;
                const int early = p.window / p.pieces;
                issue(early < 1 ? 1 : (early > p.stages ? p.stages : early));
            } else {
                // the first window of copies goes out before the CTA has even synchronised (no waiting here:
                // the consumers meet this thread at the barrier below)
                split_rows(p.rows);
                r = row_begin;
                const int early = p.window / p.pieces;
                issue(early < 1 ? 1 : (early > p.stages ? p.stages : early));
            }
        }
        __syncwarp();
        if (fused) {
            asm volatile("griddepcontrol.wait;" ::: "memory");  // x may come from the kernel before this one
            quantise_to_smem<kThreads>(p.x, p.sk, p.cols, p.fuse_step, smem, tid);
        }
        __syncthreads();  // barriers initialised; the consumers have staged the table and their activations
        if (tid == kConsumers) {
            if (!direct) segs = table;  // the same entries, now in shared memory
            issue(0x7fffffff);
            if (p.warp_rows && !failed) {
                // the warp scheme's consumers read what each slot holds from stage_info: a stage of no rows ends their loop
                if (st >= p.stages && !mbar_wait(&empty_bar[slot], phase, p.wait_ns)) { atomicExch(p.error_flag, 1); failed = true; }
                else {
                    stage_info[slot] = make_int4(0, 0, 0, 0);
                    for (int k = 0; k < p.pieces; ++k) mbar_expect_tx(&full_bar[2 * slot + k], 0);
                    issued = ++st;
                }
            }
            // leave only after every copy this CTA issued has landed (bounded)
            for (int w = (issued > p.stages ? issued - p.stages : 0); w < issued; ++w)
                for (int k = 0; k < p.pieces; ++k)
                    if (!mbar_wait(&full_bar[2 * (w % p.stages) + k], (w / p.stages) & 1, p.wait_ns)) { atomicExch(p.error_flag, 2); break; }
        }
    } else {
        // ---------------------------------------------------------------- consumers
        // Everything below reads what earlier kernels wrote (activations, tables) or writes what
        // they may still read (y): wait for them. The producer's weight copies are already running.
        // The segment table sits in shared memory for the whole kernel. One that came with the launch is
        // copied before the wait (it does not depend on the kernel before), one in device memory after.
        auto stage_table = [&]() {
            if (p.plan && tid == 0) { plan_counts[0] = plan->n_segments; plan_counts[1] = plan->subs; plan_counts[2] = plan->total_rows; }
            const int n_copy = p.n_segments;  // a planned launch copies its maximum: no trip to memory for the count first
            const uint32_t* src = (const uint32_t*)(p.plan ? plan->seg : (p.table ? p.table : p.inline_seg));
            uint32_t* dst = (uint32_t*)table;
            const int words = (n_copy < RQ_MAX_SEGMENTS ? n_copy : RQ_MAX_SEGMENTS) * (int)(sizeof(RqSegment) / 4);
            for (int i = tid; i < words; i += kConsumers) dst[i] = src[i];
        };
        if (direct) stage_table();
        // A thread's item is the same (half, sub-row, row slot, unit) in every stage: thread t takes
        // item t of the stage's grid [half][sub-row][row][unit]. Halves are outermost so that a warp
        // works on one half of adjacent units: no divergence, no bank conflicts.
        const int su_cap = p.stage_rows * p.units;          // units of one sub-row in a full stage
        const int items_cap = 2 * p.subs * su_cap;
        int my_h = tid / (p.subs * su_cap);
        const int my_rem = tid - my_h * (p.subs * su_cap);
        const int my_s = my_rem / su_cap, my_su = my_rem - my_s * su_cap;
        const int my_lr = my_su / p.units;
        int my_u = my_su - my_lr * p.units;
        bool act_owner = tid < items_cap;   // this thread has an item, hence activations to hold
        const int group = p.warp_rows ? 32 / p.warp_rows : 32;  // warp scheme: lanes per row, the power of two that holds its 2 * units items
        if (p.warp_rows) {
            const int item = ((tid & 31) & (group - 1)) + (p.row_warps > 1 ? (tid >> 5) * group : 0);
            act_owner = item < 2 * p.units;   // a row whose items are no power of two leaves the group's last lanes idle
            my_h = item >= p.units && act_owner ? 1 : 0;
            my_u = act_owner ? item - my_h * p.units : 0;
        }
        // (all of the above is arithmetic on the launch's parameters: done before the wait, it costs the chain nothing)
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (!direct) stage_table();
        ActHalf areg[TR];
        if (MODE == RQ_ACT_INT8 && p.act_regs) {
            // single token: this thread's 128 codes, steps and sums, kept in registers for the whole
            // kernel. They come from the records an earlier launch left in the scratch, or (fused
            // launches) from records this CTA makes of x right here, while its first weights fly.
            if (p.fuse_step) {
                quantise_to_smem<kThreads>(p.x, p.sk, p.cols, p.fuse_step, act_smem, tid);
                __syncthreads();  // with the producer warp: records complete, barriers initialised
                if (act_owner) areg[0].load(act_smem + (size_t)my_u * kRecord, my_h);
                if (blockIdx.x == 0 && p.act_out) {
                    const uint4* src = (const uint4*)act_smem;
                    uint4* dst = (uint4*)p.act_out;
                    for (int i = tid; i < p.units * (kRecord / 16); i += kConsumers) dst[i] = src[i];
                }
            } else if (act_owner) {
#pragma unroll
                for (int j = 0; j < TR; ++j) {
                    const int tok = tok0 + j < p.tokens ? tok0 + j : tok0;  // a pair past the last token dots the first again and stores nothing
                    areg[j].load(p.act + ((size_t)tok * p.units + my_u) * kRecord, my_h);
                }
            }
        } else if (MODE == RQ_ACT_FLOAT) {
            // stage the activations while the first weight stages are in flight
            // all vectors as one flat range, sixteen loads in flight per thread: the copy costs a few trips to L2, not one per
            // element. (vector, input) of a flat index advance by subtraction: no division in the loop.
            const int total = p.act_vectors * p.cols;
            int v0 = tid / p.cols, k0 = tid - v0 * p.cols;
            const int adv_v = kConsumers / p.cols, adv_k = kConsumers - adv_v * p.cols;  // one step of kConsumers
            for (int base_i = tid; base_i < total; base_i += 16 * kConsumers) {
                float got[16];
                int v = v0, k = k0;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    got[j] = 0.0f;
                    if (base_i + j * kConsumers < total) {
                        const int vec = tok0 + v;  // plain: token; expert banks: slot vector (one token per launch)
                        const bool live = p.act_vectors > T || vec < p.tokens;
                        if (live) got[j] = __ldg(xbase + (int64_t)vec * p.st + (int64_t)k * p.sk);
                    }
                    v += adv_v; k += adv_k;
                    if (k >= p.cols) { k -= p.cols; ++v; }
                }
                v = v0; k = k0;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    if (base_i + j * kConsumers < total) ((float*)(act_smem + v * p.act_bytes + (size_t)(k >> 8) * kRecord))[k & 255] = got[j];
                    v += adv_v; k += adv_k;
                    if (k >= p.cols) { k -= p.cols; ++v; }
                }
                v0 = v; k0 = k;
            }
            consumer_sync<kConsumers>();
            {
                // the sums of every 16-input slice of every vector, dealt flat over the threads
                const int per_vec = p.cols >> 4, slices = p.act_vectors * per_vec;
                for (int i = tid; i < slices; i += kConsumers) {
                    const int v = i / per_vec, s2 = i - v * per_vec;
                    float* rec = (float*)(act_smem + v * p.act_bytes + (size_t)(s2 >> 4) * kRecord);
                    float acc = 0.f;
#pragma unroll
                    for (int q = 0; q < 16; ++q) acc += rec[16 * (s2 & 15) + q];
                    rec[256 + (s2 & 15)] = acc;
                }
            }
            consumer_sync<kConsumers>();
        } else if (MODE == RQ_ACT_INT8 && T == 4) {
            // four tokens' records, interleaved unit by unit (the layout item_dot_tok4 reads); a token past
            // the end of the batch is staged as zeros
            const int per_vec = p.units * (kRecord / 16), total = 4 * per_vec;
            for (int base_i = tid; base_i < total; base_i += 4 * kConsumers) {  // four 16-byte loads in flight per thread
                uint4 got[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int i = base_i + j * kConsumers;
                    got[j] = make_uint4(0, 0, 0, 0);
                    if (i < total) {
                        const int v = i / per_vec, e = i - v * per_vec;
                        if (tok0 + v < p.tokens) got[j] = __ldg((const uint4*)(p.act + (size_t)(tok0 + v) * per_vec * 16) + e);
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int i = base_i + j * kConsumers;
                    if (i < total) {
                        const int v = i / per_vec, e = i - v * per_vec;
                        const int unit = e / (kRecord / 16), line = e - unit * (kRecord / 16);  // 16-byte line of the token's record
                        uint8_t* rec = act_smem + (size_t)unit * kRecord4;
                        const uint32_t wv[4] = {got[j].x, got[j].y, got[j].z, got[j].w};
                        if (line < 18) {
                            // code words (lines 0..15) and steps (16, 17, which follow the 64 code words at
                            // the same pitch): word by word, sixteen bytes apart
                            uint32_t* dst = (uint32_t*)rec + 16 * line + v;
#pragma unroll
                            for (int q = 0; q < 4; ++q) dst[4 * q] = wv[q];
                        } else {
                            // slice sums (lines 18, 19) and group sums (20): int16 by int16, eight bytes apart
                            uint16_t* dst = (uint16_t*)(rec + (line < 20 ? 1152 + 64 * (line - 18) : 1280)) + v;
#pragma unroll
                            for (int q = 0; q < 8; ++q) dst[4 * q] = (uint16_t)(wv[q >> 1] >> (16 * (q & 1)));
                        }
                    }
                }
            }
            consumer_sync<kConsumers>();
        } else {
            const size_t src_bytes = (size_t)p.units * kRecord;
            const int per_vec = (int)(src_bytes / 16), total = p.act_vectors * per_vec;
            for (int base_i = tid; base_i < total; base_i += 4 * kConsumers) {  // four 16-byte loads in flight per thread
                uint4 got[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int i = base_i + j * kConsumers;
                    got[j] = make_uint4(0, 0, 0, 0);
                    if (i < total) {
                        const int v = i / per_vec, e = i - v * per_vec;
                        const int vec = tok0 + v;
                        const bool live = p.act_vectors > T || vec < p.tokens;
                        if (live) got[j] = __ldg((const uint4*)(p.act + (size_t)vec * src_bytes) + e);
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int i = base_i + j * kConsumers;
                    if (i < total) {
                        const int v = i / per_vec, e = i - v * per_vec;
                        ((uint4*)(act_smem + v * p.act_bytes))[e] = got[j];
                    }
                }
            }
            consumer_sync<kConsumers>();
        }
        if (!fused) __syncthreads();  // the producer has initialised the barriers; table and plan counts are in place
        // counts: from the launch, or (planned launches) from the device-side plan, never above the launch's
        if (p.plan) { n_segments = min(plan_counts[0], p.n_segments); subs = min(plan_counts[1], p.subs); }
        split_rows(p.plan ? min((int64_t)plan_counts[2], p.rows) : p.rows);

        const int lane = tid & 31, warp = tid >> 5;
        bool dead = false;  // a wait ran out: no more waiting, the results are flagged invalid
        int seg = 0;
        int64_t r = row_begin;
        int slot = 0;
        uint32_t phase = 0;  // ring position and parity of the next stage
        // A row's partial sums (its items, in shared memory) are added by eight adjacent lanes: each strides
        // over the items, then a fixed xor tree joins the eight -- the same order, hence the same bits, on
        // every run; sub-rows are joined by the epilogue in sub-row order. `first` = the task of this
        // thread's lane group in the first sweep, `sweep` = tasks per sweep.
        auto reduce_rows = [&](const float* part, const RqSegment& sg, int nr, int64_t lr0, int first, int sweep) {
            const int l8 = lane & 7;
            const int tasks = nr * T;
            for (int base = 0; base < tasks; base += sweep) {  // uniform trip count: every lane takes part in the shuffles
                const int task = base + first;
                const bool live = task < tasks && tok0 + (task % T) < p.tokens;
                const int lr = live ? task / T : 0, t = live ? task - lr * T : 0;
                float out = 0.f, gate = 0.f;
                for (int s = 0; s < subs; ++s) {
                    const float* lo = part + t * stage_items + s * su_cap + lr * p.units;  // the row's half-0 partials
                    const float* hi = lo + p.subs * su_cap;                                // and its half-1 partials
                    float sum = 0.f;
                    if (p.sum_group) {
                        const int q = p.sum_group;
                        for (int c = 0; c < p.sum_chunks; ++c) {
                            float w4[4];
#pragma unroll
                            for (int m = 0; m < 4; ++m) {
                                const int idx = c * q + l8 + 8 * m;  // item of the row: half-0 items first, then half-1
                                w4[m] = (live && l8 + 8 * m < q && idx < 2 * p.units) ? (idx < p.units ? lo[idx] : hi[idx - p.units]) : 0.f;
                            }
                            if (q == 32) { w4[0] += w4[2]; w4[1] += w4[3]; }
                            if (q >= 16) w4[0] += w4[1];
                            float cs = w4[0];
                            if (q > 4) cs += __shfl_xor_sync(0xffffffffu, cs, 4);
                            if (q > 2) cs += __shfl_xor_sync(0xffffffffu, cs, 2);
                            cs += __shfl_xor_sync(0xffffffffu, cs, 1);
                            sum = p.sum_chunks == 1 ? cs : sum + cs;
                        }
                    } else {
                        if (live)
                            for (int j = l8; j < p.units; j += 8) sum += lo[j] + hi[j];
                        sum += __shfl_xor_sync(0xffffffffu, sum, 4);
                        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                    }
                    if (p.epilogue == RQ_EPI_GLU) { if (s == 0) gate = sum; else if (live && l8 == 0) out = rq_silu_portable(gate) * sum; }
                    else if (p.epilogue == RQ_EPI_WSUM) out += sum * sg.coef[s];
                    else out = sum;
                }
                if (live && l8 == 0) sg.y[(lr0 + lr) * p.yn + (int64_t)(tok0 + t) * p.yt] = out;
            }
        };
        constexpr int kSweep = kConsumers / 8;  // row tasks per sweep of the consumer threads
        if (T <= 2 && p.warp_rows) {
            // ---- the warp scheme: no partial sums in shared memory, no CTA-wide barrier. A row's items are
            // `group` adjacent lanes; a thread takes up to two rows of a stage (one per pass), holds their
            // weights in registers, releases the stage, and the lanes of a row join their sums by an xor tree.
            const bool split = p.row_warps > 1;
            const int row_in_pass = (split ? 0 : warp * p.warp_rows) + (lane / group);
            const int rows_per_pass = (split ? 1 : NW) * p.warp_rows;
            int cross_buf = 0;
            const size_t my_off = (size_t)row_in_pass * row_bytes + (size_t)my_u * p.unit_bytes;
            const size_t pass_bytes = (size_t)rows_per_pass * row_bytes;
            const bool writer = (lane & (group - 1)) == 0;
            while (true) {
                if (!mbar_wait(&full_bar[2 * slot], phase, p.wait_ns)) { atomicExch(p.error_flag, 3); dead = true; }
                if (dead) break;
                const int4 info = stage_info[slot];  // rows, segment, first local row, offset of the first d
                if (info.x == 0) break;               // the producer has no more rows for this CTA
                const uint8_t* stage = ring + (size_t)slot * p.stage_bytes;
                ItemRegs<TYPE> wr[R];
                bool have[R];
#pragma unroll
                for (int k = 0; k < R; ++k) {
                    const int lr = row_in_pass + k * rows_per_pass;
                    // the second pass's rows are the stage's second piece
                    if (k == 1 && p.pieces == 2 && !dead && !mbar_wait(&full_bar[2 * slot + 1], phase, p.wait_ns)) { atomicExch(p.error_flag, 3); dead = true; }
                    have[k] = lr < info.x && act_owner;
                    if (have[k]) {
                        const uint16_t* sc = nullptr;
                        if (TYPE != RQ_Q4_K) sc = (const uint16_t*)(stage + p.sub_main_bytes + info.w) + ((size_t)lr * p.units + my_u) * p.scales_per_unit;
                        wr[k].load(stage + my_off + k * pass_bytes, sc, my_h, my_u);
                    }
                }
                // the warp holds its weights in registers: the producer may refill the slot
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty_bar[slot]);
                if (++slot == p.stages) { slot = 0; phase ^= 1; }
                // v[j][k]: token tok0 + j (the tokens a thread holds in registers) against row k of the stage; every token's
                // dot and sums are the single-token ones, so a position gets the bits its own call gives
                float v[TR][R];
                if (MODE == RQ_ACT_INT8) {
#pragma unroll
                    for (int j = 0; j < TR; ++j)
#pragma unroll
                        for (int k = 0; k < R; ++k) v[j][k] = have[k] ? dot_regs(wr[k], areg[j], my_h) : 0.f;
                } else {
                    dot_regs_float<R>(wr, have, act_smem + (size_t)my_u * kRecord, my_h, v[0]);
                }
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) {
                    if (off < group) {  // uniform over the launch
#pragma unroll
                        for (int j = 0; j < TR; ++j)
#pragma unroll
                            for (int k = 0; k < R; ++k) v[j][k] += __shfl_xor_sync(0xffffffffu, v[j][k], off);
                    }
                }
                if (!split) {
                    if (writer) {
                        float* yb = table[info.y].y;
#pragma unroll
                        for (int j = 0; j < TR; ++j)
#pragma unroll
                            for (int k = 0; k < R; ++k)
                                if (have[k] && tok0 + j < p.tokens) yb[(int64_t)(info.z + row_in_pass + k * rows_per_pass) * p.yn + (int64_t)(tok0 + j) * p.yt] = v[j][k];
                    }
                } else {
                    // this warp's share of each row goes to shared memory; the warp that finds the others all
                    // there adds the shares in warp order (whichever warp that is, the order is the same)
                    if (writer) {
#pragma unroll
                        for (int j = 0; j < TR; ++j)
#pragma unroll
                            for (int k = 0; k < R; ++k)
                                cross_sum[cross_buf][j][row_in_pass + k * rows_per_pass][warp] = v[j][k];
                    }
                    __threadfence_block();
                    __syncwarp();
                    int arrived = 0;
                    if (lane == 0) arrived = atomicAdd(&cross_count[cross_buf], 1);
                    arrived = __shfl_sync(0xffffffffu, arrived, 0);
                    if (arrived == NW - 1) {
                        __threadfence_block();
                        const int rows_here = info.x;
                        // lanes 0..7 take the rows for the first token, lanes 8..15 for the second
                        const int row = lane & 7, j = lane >> 3;
                        if (row < rows_here && j < TR && tok0 + j < p.tokens) {
                            float out = 0.f;
#pragma unroll
                            for (int w = 0; w < NW; ++w) out += *(volatile float*)&cross_sum[cross_buf][j][row][w];
                            table[info.y].y[(int64_t)(info.z + row) * p.yn + (int64_t)(tok0 + j) * p.yt] = out;
                        }
                        __syncwarp();
                        if (lane == 0) cross_count[cross_buf] = 0;
                    }
                    if (++cross_buf > kMaxStages) cross_buf = 0;
                }
            }
        } else if (R == 2) {
            // two-row instantiations serve the warp scheme only
        } else if (MODE == RQ_ACT_INT8 && T == 1 && p.act_regs) {
            // ---- register items through shared-memory partial sums (rows the warp scheme does not take)
            constexpr int PAIR = 1;
            int buf = 0;
            while (r < row_end) {
                ItemRegs<TYPE> wr[PAIR];
                bool have[PAIR];
                int st_seg[PAIR], st_nr[PAIR];
                int64_t st_lr0[PAIR];
#pragma unroll
                for (int k = 0; k < PAIR; ++k) {
                    have[k] = false; st_nr[k] = 0; st_seg[k] = seg; st_lr0[k] = 0;
                    if (r < row_end) {
                        while (seg + 1 < n_segments && r >= table[seg].row_begin + table[seg].rows) ++seg;
                        const RqSegment& sg = table[seg];
                        const int64_t seg_end = sg.row_begin + sg.rows;
                        int64_t stop = r + p.stage_rows;
                        if (stop > seg_end) stop = seg_end;
                        if (stop > row_end) stop = row_end;
                        const int nr = (int)(stop - r);
                        const int64_t lr0 = r - sg.row_begin;
                        st_seg[k] = seg; st_nr[k] = nr; st_lr0[k] = lr0;
                        if (!dead && !mbar_wait(&full_bar[2 * slot], phase, p.wait_ns)) { atomicExch(p.error_flag, 3); dead = true; }
                        const uint8_t* stage = ring + (size_t)slot * p.stage_bytes;
                        have[k] = tid < items_cap && my_lr < nr && my_s < subs;
                        if (have[k]) {
                            const uint8_t* w = stage + (size_t)my_s * p.sub_main_bytes + (size_t)my_su * p.unit_bytes;
                            const uint16_t* sc = nullptr;
                            if (TYPE != RQ_Q4_K) {
                                const uintptr_t first = (uintptr_t)sg.scale[my_s] + (uintptr_t)(lr0 * row_scales * 2);
                                sc = (const uint16_t*)(stage + (size_t)p.subs * p.sub_main_bytes + (size_t)my_s * p.sub_scale_bytes + (first & 15)) + (size_t)my_su * p.scales_per_unit;
                            }
                            wr[k].load(w, sc, my_h, my_u);
                        }
                        // the warp holds its weights in registers: the producer may refill the slot
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&empty_bar[slot]);
                        if (++slot == p.stages) { slot = 0; phase ^= 1; }
                        r = stop;
                    }
                }
                float* part = partial + (size_t)buf * PAIR * stage_items;
                buf ^= 1;
#pragma unroll
                for (int k = 0; k < PAIR; ++k)
                    if (have[k]) part[k * stage_items + tid] = dot_regs(wr[k], areg[0], my_h);
                consumer_sync<kConsumers>();
                // the rows of both stages, dealt to the warps in turn
                reduce_rows(part, table[st_seg[0]], st_nr[0], st_lr0[0], tid >> 3, kSweep);
                if (PAIR == 2 && st_nr[PAIR - 1] > 0) {
                    const int shift = st_nr[0] % kSweep;  // carry the deal on where the first stage left it
                    reduce_rows(part + stage_items, table[st_seg[PAIR - 1]], st_nr[PAIR - 1], st_lr0[PAIR - 1], ((tid >> 3) + kSweep - shift) % kSweep, kSweep);
                }
            }
        } else {
            for (int st = 0; r < row_end; ++st) {
                while (seg + 1 < n_segments && r >= table[seg].row_begin + table[seg].rows) ++seg;
                const RqSegment& sg = table[seg];
                const int64_t seg_end = sg.row_begin + sg.rows;
                int64_t stop = r + p.stage_rows;
                if (stop > seg_end) stop = seg_end;
                if (stop > row_end) stop = row_end;
                const int nr = (int)(stop - r);
                const int64_t lr0 = r - sg.row_begin;
                if (!dead && !mbar_wait(&full_bar[2 * slot], phase, p.wait_ns)) { atomicExch(p.error_flag, 3); dead = true; }
                const uint8_t* stage = ring + (size_t)slot * p.stage_bytes;
                float* part = partial + (size_t)(st & 1) * T * stage_items;
                if (tid < items_cap && my_lr < nr && my_s < subs) {
                    const uint8_t* w = stage + (size_t)my_s * p.sub_main_bytes + (size_t)my_su * p.unit_bytes;
                    const uint16_t* sc = nullptr;
                    if (TYPE != RQ_Q4_K) {
                        // where this sub-row's first d value sits inside its 16-byte-aligned copy
                        const uintptr_t first = (uintptr_t)sg.scale[my_s] + (uintptr_t)(lr0 * row_scales * 2);
                        sc = (const uint16_t*)(stage + (size_t)p.subs * p.sub_main_bytes + (size_t)my_s * p.sub_scale_bytes + (first & 15)) + (size_t)my_su * p.scales_per_unit;
                    }
                    if constexpr (MODE == RQ_ACT_INT8 && T == 4) {
                        float v4[4];
                        item_dot_tok4<TYPE>(w, sc, act_smem + (size_t)my_u * kRecord4, my_h, my_u, v4);
#pragma unroll
                        for (int t = 0; t < 4; ++t) part[t * stage_items + tid] = v4[t];
                    } else {
                        const uint8_t* a0 = act_smem + (size_t)sg.act[my_s] * p.act_bytes + (size_t)my_u * kRecord;
#pragma unroll
                        for (int t = 0; t < T; ++t) {
                            const uint8_t* ar = a0 + t * p.act_bytes;
                            if (MODE == RQ_ACT_INT8) areg[0].load(ar, my_h);
                            part[t * stage_items + tid] = item_dot<TYPE, MODE>(w, sc, ar, areg[0], my_h, my_u);
                        }
                    }
                }
                // this warp is done with the stage's weights: the producer may refill the slot
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty_bar[slot]);
                if (++slot == p.stages) { slot = 0; phase ^= 1; }
                consumer_sync<kConsumers>();
                reduce_rows(part, sg, nr, lr0, tid >> 3, kSweep);
                r = stop;
            }
        }
    }
}

template <int TYPE, int MODE, int T, int NW, int R>
int launch_stream(const StreamParams& p, int grid_x, size_t smem, cudaStream_t s) {
    auto kernel = rq_gemv_stream_kernel<TYPE, MODE, T, NW, R>;
    static bool configured[64] = {};  // per instantiation and device: the opt-in to large dynamic shared memory
    int dev = 0;
    RQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        // everything a block may take (227 KB on sm_100), less this kernel's static shared memory
        cudaFuncAttributes fa;
        int optin = 0;
        RQ_CUDA(cudaFuncGetAttributes(&fa, kernel));
        RQ_CUDA(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        RQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, optin - (int)fa.sharedSizeBytes));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid_x, (unsigned)(p.plan_count > 1 ? p.plan_count : (p.tokens + T - 1) / T));
    cfg.blockDim = dim3(NW * 32 + 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    RQ_CUDA(cudaLaunchKernelEx(&cfg, kernel, p));
    return RQ_OK;
}

// How a row of `ipr` items is laid on lanes by the single-token int8 schemes (and hence the order its item sums are
// added in, whatever kernel runs): `group` adjacent lanes per row inside a warp, the row spread over `chunks` warps.
// chunks = 1: the row lies in one warp (a power of two of items, or padded up to one); 7 / 5 / 8: rows of 7, 5 or 8
// times a power of two of items (14336, 2560, 32768 inputs) with as many consumer warps. group = 0: no such layout.
static void row_layout(int ipr, int* group, int* chunks) {
    auto pow2 = [](int v) { return v > 0 && (v & (v - 1)) == 0; };
    *group = 0; *chunks = 1;
    if (ipr <= 32 && pow2(ipr)) { *group = ipr; return; }
    if (ipr % 7 == 0 && pow2(ipr / 7) && ipr / 7 >= 8 && ipr / 7 <= 32) { *group = ipr / 7; *chunks = 7; return; }
    if (ipr % 5 == 0 && pow2(ipr / 5) && ipr / 5 >= 4 && ipr / 5 <= 32) { *group = ipr / 5; *chunks = 5; return; }
    if (ipr == 256) { *group = 32; *chunks = 8; return; }
    if (ipr <= 32) { *group = 2; while (*group < ipr) *group <<= 1; }
}

template <int TYPE, int MODE, int NW>
int dispatch_stream_nw(StreamParams& p, int sm_count, int vectors_per_launch, cudaStream_t s, bool one_per_sm = false, bool token_pairs = false) {
    // Two CTAs share an SM (eight consumer warps and about 100 KB each): their barriers and waits
    // interleave, and when a CTA of one launch exits, a CTA of the next launch (programmatic
    // dependent launch) takes its place and prefetches weights while the other is still working.
    // five consumer warps: three CTAs of six warps per SM. one_per_sm: a single CTA with the whole SM's shared memory, for
    // launches whose staged activations leave two CTAs no room for a ring (fp32 records of 14336 inputs are 62 KB).
    // token_pairs (int8 windows over rows of five consumer warps): two tokens' records in every thread's registers, 170
    // registers a thread, so two CTAs per SM instead of three
    const int kCtasPerSm = one_per_sm ? 1 : (NW == 5 && !token_pairs ? 3 : 2);
    // dynamic; with the static tables (about 10 KB) and the 1 KB the system keeps per CTA, two (three) CTAs fit an SM's 228 KB
    const size_t kSmemBudget = one_per_sm ? 200 * 1024 : (NW == 5 && !token_pairs ? 64 * 1024 : 102 * 1024);
    constexpr int kRecord = MODE == RQ_ACT_INT8 ? RQ_ACT_RECORD_INT8 : RQ_ACT_RECORD_FLOAT;
    // NW = consumer warps: seven, so that with the producer warp a CTA is eight warps and two CTAs per SM leave each
    // thread 128 registers; eight (one CTA per SM then) only for rows too long for seven warps' worth of items.
    constexpr int kConsumers = NW * 32;
    p.act_bytes = ((size_t)p.units * kRecord + 127) & ~(size_t)127;
    int t = 1;
    if (vectors_per_launch > 0) {
        p.act_vectors = vectors_per_launch;  // expert banks: one token, a vector per slot
    } else {
        t = token_pairs ? 2 : ((p.tokens >= 2 && 4 * p.act_bytes <= 40 * 1024) ? 4 : 1);
        p.act_vectors = t;
        // four int8 tokens are staged interleaved, kRecord4 bytes per unit: a quarter of that per vector
        if (MODE == RQ_ACT_INT8 && t == 4) p.act_bytes = ((size_t)p.units * (kRecord4 / 4) + 127) & ~(size_t)127;
    }
    // single-token INT8 launches whose sub-rows all read vector 0 keep the activations in registers
    p.act_regs = (MODE == RQ_ACT_INT8 && (t == 1 || token_pairs) && vectors_per_launch == 0 && p.table == nullptr && p.plan == nullptr) ? 1 : 0;
    if (p.fuse_step && !p.act_regs) return RQ_ERR_UNSUPPORTED;  // the caller quantises with the standalone kernel instead
    if (p.act_regs) p.act_vectors = p.fuse_step ? 1 : 0;        // fused: one token's records are made in shared memory; else nothing is staged
    if (p.act_bytes * p.act_vectors > (size_t)(one_per_sm ? 128 : 64) * 1024) return RQ_ERR_UNSUPPORTED;  // the caller falls back to the tiled kernel
    const int64_t row_bytes = (int64_t)p.units * p.unit_bytes;
    int ctas = sm_count * kCtasPerSm;
    if (p.plan_count > 1) { ctas /= p.plan_count; if (ctas < 1) ctas = 1; }  // the batch's grid rows share the GPU
    const int64_t rows_per_cta = (p.rows + ctas - 1) / ctas;
    const int ipr = 2 * p.units * p.subs;  // items per virtual row
    p.units_shift = (p.units & (p.units - 1)) == 0 ? __builtin_ctz(p.units) : -1;
    // Stage: whole virtual rows that (nearly) fill one pass of the consumer threads, 48 KB at most.
    if (ipr > kConsumers) return RQ_ERR_UNSUPPORTED;  // a row must fit one pass of the consumer threads
    int stage_rows = kConsumers / ipr;
    while (stage_rows > 1 && (int64_t)stage_rows * row_bytes * p.subs > 32 * 1024) --stage_rows;
    if (stage_rows > rows_per_cta) stage_rows = (int)rows_per_cta;
    // The warp scheme: plain single-sub-row launches with register activations whose rows are a power
    // of two of items, at most a warp's worth.
    p.warp_rows = 0; p.rows_per_thread = 0;
    p.row_warps = 1;
    p.sum_group = 0; p.sum_chunks = 1;
    const bool warp_shape = vectors_per_launch == 0 && p.table == nullptr && p.plan == nullptr && p.subs == 1 && p.epilogue == RQ_EPI_PLAIN;
    // single-token launches that run a warp scheme: int8 with register activations, fp32 with the token's record in shared memory
    const bool warp_launch = warp_shape && (p.act_regs || (MODE == RQ_ACT_FLOAT && t == 1));
    int layout_group = 0, layout_chunks = 1;
    row_layout(ipr, &layout_group, &layout_chunks);
    const bool split_shape = layout_chunks > 1 && layout_chunks == NW;
    if (warp_shape && layout_group) { p.sum_group = layout_group; p.sum_chunks = layout_chunks; }
    if (warp_launch && layout_group && layout_chunks == 1) {
        const int group = layout_group;
        p.warp_rows = 32 / group;
        const int pass_rows = NW * p.warp_rows;
        p.rows_per_thread = (int64_t)2 * pass_rows * row_bytes <= 34 * 1024 && rows_per_cta > pass_rows ? 2 : 1;
        stage_rows = pass_rows * p.rows_per_thread;
    } else if (warp_launch && split_shape) {
        // longer rows whose items split evenly over the warps, a power of two of lanes each (14336 inputs: 7 x 16)
        const int group = layout_group;
        p.warp_rows = 32 / group;
        p.row_warps = NW;
        p.rows_per_thread = (int64_t)2 * p.warp_rows * row_bytes <= 34 * 1024 && rows_per_cta > p.warp_rows && 2 * p.warp_rows <= 8 ? 2 : 1;
        stage_rows = p.warp_rows * p.rows_per_thread;
    }
    if (token_pairs) {
        if (!p.warp_rows) return RQ_ERR_UNSUPPORTED;  // pairs run a warp scheme or not at all
        if (p.rows_per_thread == 2) { p.rows_per_thread = 1; stage_rows /= 2; }  // two tokens' records leave no registers for a second row
    }
    p.stage_rows = stage_rows;
    p.pieces = 1; p.piece_rows = stage_rows;
    if (p.warp_rows && p.rows_per_thread == 2) { p.pieces = 2; p.piece_rows = stage_rows / 2; }
    {
        // in flight per CTA: about 32 KB (two CTAs per SM: some 9 MB on the whole GPU, the memory latency at full bandwidth), two pieces at least
        const int64_t piece_bytes = (int64_t)p.piece_rows * row_bytes * p.subs;
        p.window = (int)((32 * 1024 + piece_bytes - 1) / piece_bytes);
        if (p.window < 2) p.window = 2;
    }
    p.sub_main_bytes = ((size_t)stage_rows * row_bytes + 127) & ~(size_t)127;
    p.sub_scale_bytes = p.scales_per_unit ? (((size_t)stage_rows * p.units * p.scales_per_unit * 2 + 32 + 127) & ~(size_t)127) : 0;
    p.stage_bytes = (p.sub_main_bytes + p.sub_scale_bytes) * p.subs;
    p.partial_bytes = ((size_t)2 * (t == 1 ? 2 : t) * stage_rows * ipr * 4 + 127) & ~(size_t)127;  // two buffers of T stages (of a pair of stages when T = 1)
    if (p.warp_rows) p.partial_bytes = 0;
    const size_t fixed = p.act_bytes * p.act_vectors + p.partial_bytes;
    if (fixed + 2 * p.stage_bytes > kSmemBudget) return RQ_ERR_UNSUPPORTED;
    int stages = (int)((kSmemBudget - fixed) / p.stage_bytes);
    if (stages > kMaxStages) stages = kMaxStages;
    p.stages = stages;
    if (p.window > stages * p.pieces - 1) p.window = stages * p.pieces - 1;  // the producer looks back at barriers of slots it has not re-armed yet
    if (p.window < 1) p.window = 1;
    const size_t smem = fixed + (size_t)stages * p.stage_bytes;
    const int grid_x = (int)(p.rows < ctas ? p.rows : ctas);
    p.rows_quot = p.rows / grid_x; p.rows_rem = (int)(p.rows % grid_x);
    p.interleaved = 0;
    if (p.warp_rows && p.table == nullptr && p.plan == nullptr && p.n_segments <= RQ_INLINE_SEGMENTS) {
        p.interleaved = 1;
        int at = 0;
        for (int i = 0; i < p.n_segments; ++i) { p.seg_stage_begin[i] = at; at += (p.inline_seg[i].rows + stage_rows - 1) / stage_rows; }
        for (int i = p.n_segments; i <= RQ_INLINE_SEGMENTS; ++i) p.seg_stage_begin[i] = at;
        p.total_stages = at;
    }
    if constexpr (NW == 5 && MODE == RQ_ACT_INT8) {
        if (token_pairs) return launch_stream<TYPE, MODE, 2, NW, 1>(p, grid_x, smem, s);
    }
    if (t == 4) return launch_stream<TYPE, MODE, 4, NW, 1>(p, grid_x, smem, s);
    if (p.rows_per_thread == 2) return launch_stream<TYPE, MODE, 1, NW, 2>(p, grid_x, smem, s);
    return launch_stream<TYPE, MODE, 1, NW, 1>(p, grid_x, smem, s);
}

template <int TYPE, int MODE>
int dispatch_stream(StreamParams& p, int sm_count, int vectors_per_launch, cudaStream_t s) {
    const int ipr = 2 * p.units * p.subs;
    if (ipr > 7 * 32) return dispatch_stream_nw<TYPE, MODE, 8>(p, sm_count, vectors_per_launch, s);
    if constexpr (MODE == RQ_ACT_INT8) {
        // rows of 5 x 2^k items (2560 inputs): single-token launches run five consumer warps, three CTAs per SM
        int group = 0, chunks = 1;
        row_layout(ipr, &group, &chunks);
        if (chunks == 5 && vectors_per_launch == 0 && p.table == nullptr && p.plan == nullptr && p.subs == 1 && p.epilogue == RQ_EPI_PLAIN) {
            if (p.tokens == 1) return dispatch_stream_nw<TYPE, MODE, 5>(p, sm_count, vectors_per_launch, s);
            // a window of positions: token pairs in registers (the weights are read once per pair, at the single-token rate)
            // where the staged four-token pass is bound by its shared-memory loads
            if (!p.fuse_step) {
                const int rc = dispatch_stream_nw<TYPE, MODE, 5>(p, sm_count, vectors_per_launch, s, false, true);
                if (rc != RQ_ERR_UNSUPPORTED) return rc;
            }
        }
    }
    int rc = dispatch_stream_nw<TYPE, MODE, 7>(p, sm_count, vectors_per_launch, s);
    if (rc == RQ_ERR_UNSUPPORTED) rc = dispatch_stream_nw<TYPE, MODE, 7>(p, sm_count, vectors_per_launch, s, true);
    return rc;
}

}  // namespace


// Launches the streaming kernel over a segment table. `table` is device memory, or null with the
// segments in `inline_seg` (at most RQ_INLINE_SEGMENTS, one sub-row each).
// vectors_per_launch = 0: the activation vectors are the tokens (x + t * st); > 0: one token, that
// many slot vectors. Returns RQ_ERR_UNSUPPORTED (without error text) when the shape is not served.
int rq_launch_stream(rq_ctx* ctx, int type, int64_t cols, const RqSegment* table, const RqSegment* inline_seg, int n_segments, int subs,
                     int epilogue, int64_t total_rows, const float* x, int64_t sk, int64_t st, int tokens, int vectors_per_launch,
                     int64_t yn, int64_t yt, int act_mode, const uint8_t* act, int fuse_step, uint8_t* act_out, cudaStream_t s) {
    if (cols % 256 || subs < 1 || subs > RQ_MAX_SUB) return RQ_ERR_UNSUPPORTED;
    if ((!table && n_segments > RQ_INLINE_SEGMENTS) || n_segments < 1 || n_segments > RQ_MAX_SEGMENTS) return RQ_ERR_UNSUPPORTED;
    StreamParams p;
    memset(&p, 0, sizeof(p));
    p.table = table;
    if (!table) for (int i = 0; i < n_segments; ++i) p.inline_seg[i] = inline_seg[i];
    p.n_segments = n_segments; p.subs = subs; p.epilogue = epilogue;
    p.rows = total_rows; p.cols = (int)cols; p.units = (int)(cols / 256);
    p.x = x; p.sk = sk; p.st = st; p.act = act; p.yn = yn; p.yt = yt; p.tokens = tokens;
    p.fuse_step = act_mode == RQ_ACT_INT8 ? fuse_step : 0; p.act_out = act_out;
    p.error_flag = ctx->error_flag; p.wait_ns = ctx->wait_limit_ns;
    switch (type) {
        case RQ_Q4_K: p.unit_bytes = 144; p.scales_per_unit = 0; break;
        case RQ_Q6_K: p.unit_bytes = 208; p.scales_per_unit = 1; break;
        case RQ_Q8_0: p.unit_bytes = 256; p.scales_per_unit = 8; break;
        case RQ_Q4_0: p.unit_bytes = 128; p.scales_per_unit = 8; break;
        default: return RQ_ERR_UNSUPPORTED;
    }
    const bool f = act_mode == RQ_ACT_FLOAT;
    const int v = vectors_per_launch, sm = ctx->sm_count;
    switch (type) {
        case RQ_Q4_K: return f ? dispatch_stream<RQ_Q4_K, RQ_ACT_FLOAT>(p, sm, v, s) : dispatch_stream<RQ_Q4_K, RQ_ACT_INT8>(p, sm, v, s);
        case RQ_Q6_K: return f ? dispatch_stream<RQ_Q6_K, RQ_ACT_FLOAT>(p, sm, v, s) : dispatch_stream<RQ_Q6_K, RQ_ACT_INT8>(p, sm, v, s);
        case RQ_Q8_0: return f ? dispatch_stream<RQ_Q8_0, RQ_ACT_FLOAT>(p, sm, v, s) : dispatch_stream<RQ_Q8_0, RQ_ACT_INT8>(p, sm, v, s);
        default: return f ? dispatch_stream<RQ_Q4_0, RQ_ACT_FLOAT>(p, sm, v, s) : dispatch_stream<RQ_Q4_0, RQ_ACT_INT8>(p, sm, v, s);
    }
}

// A launch whose segment table and counts a kernel wrote into `plan` (device memory): the host
// sizes the launch for the maxima. FLOAT activations only: vector v is x + v * st. plan_count > 1 runs
// that many planned launches as the grid rows of one: row y reads plan[y * plan_stride] and x + y * x_plan_stride.
int rq_launch_stream_plan(rq_ctx* ctx, int type, int64_t cols, const RqPlan* plan, int plan_count, int plan_stride, int max_segments, int max_subs,
                          int epilogue, int64_t max_rows, const float* x, int64_t x_plan_stride, int64_t sk, int64_t st, int vectors, int64_t yn, int64_t yt,
                          cudaStream_t s) {
    if (cols % 256 || max_subs < 1 || max_subs > RQ_MAX_SUB || max_segments < 1 || max_segments > RQ_MAX_SEGMENTS || vectors < 1) return RQ_ERR_UNSUPPORTED;
    StreamParams p;
    memset(&p, 0, sizeof(p));
    p.plan = plan; p.plan_count = plan_count; p.plan_stride = plan_stride; p.x_plan_stride = x_plan_stride;
    p.n_segments = max_segments; p.subs = max_subs; p.epilogue = epilogue;
    p.rows = max_rows; p.cols = (int)cols; p.units = (int)(cols / 256);
    p.x = x; p.sk = sk; p.st = st; p.yn = yn; p.yt = yt; p.tokens = 1;
    p.error_flag = ctx->error_flag; p.wait_ns = ctx->wait_limit_ns;
    switch (type) {
        case RQ_Q4_K: p.unit_bytes = 144; p.scales_per_unit = 0; break;
        case RQ_Q6_K: p.unit_bytes = 208; p.scales_per_unit = 1; break;
        case RQ_Q8_0: p.unit_bytes = 256; p.scales_per_unit = 8; break;
        case RQ_Q4_0: p.unit_bytes = 128; p.scales_per_unit = 8; break;
        default: return RQ_ERR_UNSUPPORTED;
    }
    const int sm = ctx->sm_count;
    switch (type) {
        case RQ_Q4_K: return dispatch_stream<RQ_Q4_K, RQ_ACT_FLOAT>(p, sm, vectors, s);
        case RQ_Q6_K: return dispatch_stream<RQ_Q6_K, RQ_ACT_FLOAT>(p, sm, vectors, s);
        case RQ_Q8_0: return dispatch_stream<RQ_Q8_0, RQ_ACT_FLOAT>(p, sm, vectors, s);
        default: return dispatch_stream<RQ_Q4_0, RQ_ACT_FLOAT>(p, sm, vectors, s);
    }
}

int rq_launch_gemv_stream(rq_ctx* ctx, const rq_weight* w, const float* x, int64_t sk, int64_t st, int tokens,
                          float* y, int64_t yn, int64_t yt, int act_mode, const uint8_t* act, int fuse_step, uint8_t* act_out, cudaStream_t s) {
    RqSegment seg;
    memset(&seg, 0, sizeof(seg));
    seg.row_begin = 0; seg.rows = (int)w->rows; seg.y = y;
    seg.main[0] = w->main; seg.scale[0] = w->scale; seg.act[0] = 0; seg.coef[0] = 1.0f;
    return rq_launch_stream(ctx, w->type, w->cols, nullptr, &seg, 1, 1, RQ_EPI_PLAIN, w->rows, x, sk, st, tokens, 0, yn, yt, act_mode, act, fuse_step, act_out, s);
}
