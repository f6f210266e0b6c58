// Batched product over Q4_K / Q6_K weights on the 5th-generation tensor cores, with EXACT INTEGER
// weight operands that live in TENSOR MEMORY.
//
//   Y[t][n] = sum_k W[n][k] * X[t][k]
//
// A K-quant value factors into a per-superblock fp16 scale and small integers:
//   Q4_K : w = d * (sc_g * q) - dmin * m_g        sc_g, m_g six bits, q four bits: sc_g * q <= 945
//   Q6_K : w = d * (s_j * (q - 32))               s_j int8, q six bits: |s_j * (q - 32)| <= 4096
// fp16 holds every integer up to 2048 exactly, so the tensor core is fed the integers themselves
// (Q4_K: one operand; Q6_K: the fp16 rounding of the integer plus its exact residual, -1 / 0 / 1)
// and `d` is applied outside it, when a sum leaves tensor memory.
//
// Data path of one CTA (128 weight rows x bn tokens):
//   * the stored bytes of 128 rows x one superblock arrive in shared memory by ONE TMA tensor copy
//     (a [rows][row bytes] byte matrix, box 144 or 208 bytes x 128 rows), two superblocks ahead;
//   * eight staging warps unpack a 64-wide slice at a time with integer and half2 arithmetic only
//     (a nibble pair becomes 1024 + q by an OR with 0x6400, one HFMA2 turns it into sc * q exactly)
//     and write the operand straight into tensor memory with tcgen05.st: the A operand of
//     tcgen05.mma is read from there, so the weights never cross shared memory a second time and
//     the tensor core's shared-memory reads are the activations' alone;
//   * the activations are fp32 and go in as fp16 pairs hi + lo (22 mantissa bits), prepared once per
//     call by rq_kq_prep_kernel in the tensor core's 128-byte-swizzled K-major image and fetched by
//     bulk copies; the two middle inputs of every four swap places there, because that is the order
//     the nibble pairs come out of a 32-bit word;
//   * per 16-wide slice Q4_K issues A x B_lo and A x B_hi (two instructions where split weights need
//     three), Q6_K issues A_hi x B_lo, A_lo x B_hi, A_hi x B_hi.
//
// The tensor core adds into its fp32 accumulator by TRUNCATION, a bias that grows with the length of
// the chain (measured: 7e-7 relative over 256 inputs, 1.2e-5 over 4096). So a sum stays in tensor
// memory for one 64-wide slice only, in one of a few accumulators in turn, the small cross terms
// issued first (while the accumulator is still small, their truncation is nothing); eight drain
// warps multiply each finished slice by the superblock's d and add it into fp32 registers with one
// round-to-nearest fma per value while the tensor core fills the next accumulator.
//
// A tcgen05.commit costs its issuing thread some 200 cycles (measured), so a slice has exactly one:
// its arrival says at once "the sum is complete" (drain warps), "the operand slot in tensor memory
// is free" (staging warps) and "the activation slot is free" (copy warp).
//
// The Q4_K minimum term, sum_g (dmin * m_g) * (sum of x over group g), is a second, 32 times smaller
// product. Its operands (dmin * m_g as fp16 hi + lo, scaled by 2^8; the group sums of x as hi + lo)
// are collected for eight superblocks at a time in one more pair of swizzled tiles in shared memory
// and multiplied into an accumulator that lives for the whole K.
//
// INT8 activations take the same kernel: rq_kq_prep_int8_kernel quantises them with the reference's
// arithmetic while it writes the image, which then holds code * step -- what the integer dot
// multiplies out to; only the order of the fp32 additions differs.
//
// Every wait is bounded; a wait that runs out records a code in the context's error word, the
// thread stops waiting and the CTA still frees its tensor memory before it exits.
#include "rq_internal.cuh"
#include "rq_mma.cuh"

using namespace rqmma;

namespace {

constexpr int kStageWarps = 8, kDrainWarps = 8;
constexpr int kStagers = kStageWarps * 32;
constexpr int kMmaWarps = 2;  // issuing threads (lane 0 of each): thread i takes the slices ks = i (mod kMmaWarps)
constexpr int kMmaWarp = kStageWarps + kDrainWarps, kCopyWarp = kMmaWarp + kMmaWarps;
constexpr int kThreadsKq = (kCopyWarp + 1) * 32;
constexpr int kTileBytes = BM * BK * 2;  // one fp16 tile of 128 rows x 64 inputs: 16 KB
constexpr int kMaxSlots = 8;   // ring depths (activation slots, operand slots in tensor memory, accumulators) and the ring of "slice done" barriers
constexpr int kRawSlots = 2;   // superblocks of stored bytes in flight per CTA
constexpr float kMinScale = 256.0f, kMinUnscale = 1.0f / 256.0f;  // the minimum term's weights are scaled so that their fp16 residuals are no subnormals

struct KqParams {
    CUtensorMap tile_map;  // the weight's main plane as a [rows][row bytes] byte matrix (TMA descriptor; first: 64-byte aligned)
    const uint8_t* main;
    const uint16_t* scale;
    int64_t rows;
    int cols;
    const uint8_t* xs;  // activations: [token tile][64-wide slice][hi | lo][bn rows x 128 bytes, swizzled]
    const uint8_t* xg;  // Q4_K: group sums of the activations: [token tile][window of 8 superblocks][hi | lo][bn rows x 128 bytes]
    int bn, tokens;
    float* y; int64_t yn, yt;
    int sb_per_split;   // superblocks per CTA along K (gridDim.z CTAs share a tile's K)
    float* partial;     // gridDim.z > 1: [split][token][row] sums, added in split order afterwards
    int b_slots;        // activation slots in shared memory
    int a_slots;        // operand slots in tensor memory (32 columns each for Q4_K, 64 for Q6_K)
    int accs;           // accumulators in rotation (bn columns each)
    int* error_flag;
    unsigned long long wait_ns;
};

__device__ __forceinline__ __half2 as_half2(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }
__device__ __forceinline__ uint32_t as_u32(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }

// ------------------------------------------------------------------------------------------
// The stored bytes behind 32 consecutive inputs of one row (`half` 0 or 1 of the 64-wide slice
// `kg`), read from the superblock tile in shared memory, and their integer operands as 32 fp16
// values (sixteen 32-bit words, four 16-byte groups), inputs in the order 0 2 1 3 within every four.
// ------------------------------------------------------------------------------------------
template <int TYPE> struct RawKq;
template <> struct RawKq<RQ_Q4_K> {
    uint4 hdr, q0, q1;
    // `tile`: 128 rows x 144 bytes of one superblock in shared memory; r: the row; pr: the 64-wide slice of the superblock
    __device__ __forceinline__ void load(const uint8_t* tile, int r, int pr, int) {
        const uint8_t* blk = tile + r * 144;
        hdr = *(const uint4*)blk;
        q0 = *(const uint4*)(blk + 16 + 32 * pr);
        q1 = *(const uint4*)(blk + 32 + 32 * pr);
    }
    // sc * (q - 8) of sub-block 2 pr + half (low nibbles hold sub-block 2 pr, high nibbles 2 pr + 1). The codes are centred
    // (the eight goes into the minimum term, which becomes dmin * m - 8 * d * sc: an order of magnitude smaller than dmin * m
    // for weights that are spread about zero), so the two sums that are subtracted at the end are small and what the tensor
    // core's truncating accumulation loses of them is small too.
    __device__ __forceinline__ void decode(int kg, int half, uint4* hi, uint4*) const {
        int sc, mn;
        rq_q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * (kg & 3) + half, sc, mn);
        const __half2 sc2 = __half2half2(__int2half_rn(sc));
        const __half2 k1032 = __half2half2(__float2half_rn(1032.0f));
        const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        const int shift = 4 * half;
        uint32_t o[16];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            // 0x6400 | n is the fp16 number 1024 + n; (1024 + q) - 1032 = q - 8 and (q - 8) * sc (at most 504) are both exact
            const uint32_t a = ((w[j] >> shift) & 0x000F000Fu) | 0x64006400u;        // inputs 4j, 4j + 2
            const uint32_t b = ((w[j] >> (shift + 8)) & 0x000F000Fu) | 0x64006400u;  // inputs 4j + 1, 4j + 3
            o[2 * j] = as_u32(__hmul2(__hsub2(as_half2(a), k1032), sc2));
            o[2 * j + 1] = as_u32(__hmul2(__hsub2(as_half2(b), k1032), sc2));
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) hi[c] = make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
    }
    // dmin * m_g - 8 * d * sc_g of the superblock's eight sub-blocks (what is left of the minimum once the codes are centred),
    // times 2^8, as fp16 hi and lo
    __device__ __forceinline__ void minimum_terms(uint4& hi, uint4& lo) const {
        const float dmin = rq_h2f((uint16_t)(hdr.x >> 16)), d8 = __fmul_rn(8.0f, rq_h2f((uint16_t)(hdr.x & 0xffff)));
        uint32_t hw[4], lw[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int s0, m0, s1, m1;
            rq_q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * j, s0, m0);
            rq_q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * j + 1, s1, m1);
            // both products are exact in fp32 (an fp16 times an integer below 64); their difference is rounded once
            const float a = __fmul_rn(__fsub_rn(__fmul_rn(dmin, (float)m0), __fmul_rn(d8, (float)s0)), kMinScale);
            const float b = __fmul_rn(__fsub_rn(__fmul_rn(dmin, (float)m1), __fmul_rn(d8, (float)s1)), kMinScale);
            const __half2 h2 = __floats2half2_rn(a, b);
            const float2 back = __half22float2(h2);
            const __half2 l2 = __floats2half2_rn(a - back.x, b - back.y);
            hw[j] = as_u32(h2);
            lw[j] = as_u32(l2);
        }
        hi = make_uint4(hw[0], hw[1], hw[2], hw[3]);
        lo = make_uint4(lw[0], lw[1], lw[2], lw[3]);
    }
};
template <> struct RawKq<RQ_Q6_K> {
    uint4 ql[2], qh[2];
    uint32_t scales;  // two int8 scales: inputs 0..15 and 16..31 of the group
    // `tile`: 128 rows x 208 bytes (ql | qh | scales) of one superblock in shared memory
    __device__ __forceinline__ void load(const uint8_t* tile, int r, int pr, int half) {
        const int ch = pr >> 1, sel = pr & 1, g = 2 * sel + half;
        const uint8_t* body = tile + r * 208;
        ql[0] = *(const uint4*)(body + 64 * ch + 32 * half);
        ql[1] = *(const uint4*)(body + 64 * ch + 32 * half + 16);
        qh[0] = *(const uint4*)(body + 128 + 32 * ch);
        qh[1] = *(const uint4*)(body + 128 + 32 * ch + 16);
        scales = *(const uint16_t*)(body + 192 + 8 * ch + 2 * g);
    }
    // s * (q - 32) of group g = 2 sel + half of the slice's chunk: the fp16 rounding and the exact residual
    __device__ __forceinline__ void decode(int kg, int half, uint4* hi, uint4* lo) const {
        const int sel = kg & 1, g = 2 * sel + half;
        const uint32_t lwv[8] = {ql[0].x, ql[0].y, ql[0].z, ql[0].w, ql[1].x, ql[1].y, ql[1].z, ql[1].w};
        const uint32_t hwv[8] = {qh[0].x, qh[0].y, qh[0].z, qh[0].w, qh[1].x, qh[1].y, qh[1].z, qh[1].w};
        const __half2 s_first = __half2half2(__int2half_rn((int)(int8_t)(scales & 0xff)));
        const __half2 s_second = __half2half2(__int2half_rn((int)(int8_t)(scales >> 8)));
        const __half2 k1056 = __half2half2(__float2half_rn(1056.0f));
        uint32_t oh[16], ol[16];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const __half2 s2 = j < 4 ? s_first : s_second;
            const uint32_t q4 = ((lwv[j] >> (4 * sel)) & 0x0F0F0F0Fu) | (((hwv[j] >> (2 * g)) & 0x03030303u) << 4);  // four six-bit codes
            const uint32_t a = (q4 & 0x00FF00FFu) | 0x64006400u;         // inputs 4j, 4j + 2 as 1024 + q
            const uint32_t b = ((q4 >> 8) & 0x00FF00FFu) | 0x64006400u;  // inputs 4j + 1, 4j + 3
            const __half2 ca = __hsub2(as_half2(a), k1056), cb = __hsub2(as_half2(b), k1056);  // q - 32, exact
            const __half2 ha = __hmul2(ca, s2), hb = __hmul2(cb, s2);
            oh[2 * j] = as_u32(ha);
            oh[2 * j + 1] = as_u32(hb);
            ol[2 * j] = as_u32(__hfma2(ca, s2, __hneg2(ha)));  // the product less its rounding: exact, -1, 0 or 1
            ol[2 * j + 1] = as_u32(__hfma2(cb, s2, __hneg2(hb)));
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            hi[c] = make_uint4(oh[4 * c], oh[4 * c + 1], oh[4 * c + 2], oh[4 * c + 3]);
            lo[c] = make_uint4(ol[4 * c], ol[4 * c + 1], ol[4 * c + 2], ol[4 * c + 3]);
        }
    }
    __device__ __forceinline__ void minimum_terms(uint4&, uint4&) const {}
};

// fp32 pair -> fp16 hi and lo words
__device__ __forceinline__ void split2(float a, float b, uint32_t& hi, uint32_t& lo) {
    const __half2 h2 = __floats2half2_rn(a, b);
    const float2 back = __half22float2(h2);
    hi = as_u32(h2);
    lo = as_u32(__floats2half2_rn(a - back.x, b - back.y));
}

// ------------------------------------------------------------------------------------------
// X -> the tensor core's operand images (fp32 activations). grid (64-wide slices, token tiles), one
// thread per token row of the tile; rows past the last token are zero.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) rq_kq_prep_kernel(const float* __restrict__ x, int64_t sk, int64_t st, int cols, int tokens, int bn,
                                                          uint8_t* __restrict__ xs, uint8_t* __restrict__ xg) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int kg = blockIdx.x, nt = blockIdx.y, r = threadIdx.x;
    if (r >= bn) return;
    const int token = nt * bn + r;
    uint8_t* hi = xs + ((size_t)nt * gridDim.x + kg) * 2 * (size_t)bn * 128;
    uint8_t* lo = hi + (size_t)bn * 128;
    float sums[2] = {0.f, 0.f};
    const bool vec = sk == 1 && (st & 3) == 0 && ((uintptr_t)x & 15) == 0;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        float v[8];
        if (token >= tokens) {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = 0.f;
        } else {
            const float* src = x + (int64_t)token * st + (int64_t)(kg * BK + 8 * c) * sk;
            if (vec) {
                *(float4*)v = __ldg((const float4*)src);
                *(float4*)(v + 4) = __ldg((const float4*)src + 1);
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = __ldg(src + j * sk);
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) sums[c >> 2] += v[j];
        uint32_t hw[4], lw[4];
        // inputs 0 2 1 3 | 4 6 5 7: the order the weights' nibble pairs come in
        split2(v[0], v[2], hw[0], lw[0]);
        split2(v[1], v[3], hw[1], lw[1]);
        split2(v[4], v[6], hw[2], lw[2]);
        split2(v[5], v[7], hw[3], lw[3]);
        *(uint4*)(hi + swizzled(r, c)) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
        *(uint4*)(lo + swizzled(r, c)) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
    }
    if (xg) {
        // the sums of this slice's two 32-input groups: elements 2 pr, 2 pr + 1 of the superblock's chunk
        const int sb = kg >> 2, pr = kg & 3;
        const int windows = ((cols >> 8) + 7) >> 3;
        uint8_t* ghi = xg + ((size_t)nt * windows + (sb >> 3)) * 2 * (size_t)bn * 128;
        uint8_t* glo = ghi + (size_t)bn * 128;
        uint32_t h, l;
        split2(sums[0], sums[1], h, l);
        *(uint32_t*)(ghi + swizzled(r, sb & 7) + 4 * pr) = h;
        *(uint32_t*)(glo + swizzled(r, sb & 7) + 4 * pr) = l;
    }
}

// ------------------------------------------------------------------------------------------
// INT8 activations: the reference's quantiser and the operand images in one pass, with no int8
// records in between. grid (superblocks, token tiles), block (bn, 4): thread (r, pr) holds the 64
// inputs of token row r in slice pr of the superblock. The extreme of a group is the FIRST input of
// strictly largest magnitude, signed: a serial scan in input order finds it (a 32-input group lies
// within one thread; a 256-input group is settled over the four threads of a row, slice by slice,
// through shared memory); inverse = -127 / extreme and d = 1 / inverse are IEEE divides,
// code = clamp(rint(x * inverse)), and the image holds code * d -- the standalone quantiser's
// arithmetic, bit for bit, so the sums equal the ones its records would give.
// ------------------------------------------------------------------------------------------
template <int STEP>
__global__ void __launch_bounds__(512) rq_kq_prep_int8_kernel(const float* __restrict__ x, int64_t sk, int64_t st, int tokens, int bn,
                                                              uint8_t* __restrict__ xs, uint8_t* __restrict__ xg) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float row_best[4][128];
    const int r = threadIdx.x, pr = threadIdx.y, sb = blockIdx.x, nt = blockIdx.y;
    const int kg = sb * 4 + pr;
    const int token = nt * bn + r;
    uint8_t* hi = xs + ((size_t)nt * gridDim.x * 4 + kg) * 2 * (size_t)bn * 128;
    uint8_t* lo = hi + (size_t)bn * 128;
    float v[64];
    if (token < tokens) {
        const float* src = x + (int64_t)token * st + (int64_t)kg * BK * sk;
        if (sk == 1 && (st & 3) == 0 && ((uintptr_t)x & 15) == 0) {
#pragma unroll
            for (int j = 0; j < 16; ++j) *(float4*)(v + 4 * j) = __ldg((const float4*)src + j);
        } else {
#pragma unroll
            for (int j = 0; j < 64; ++j) v[j] = __ldg(src + j * sk);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 64; ++j) v[j] = 0.f;
    }
    float best[2] = {0.f, 0.f};  // a NaN is never larger, so it never becomes the extreme
#pragma unroll
    for (int j = 0; j < 64; ++j)
        if (fabsf(v[j]) > fabsf(best[j >> 5])) best[j >> 5] = v[j];
    if (STEP == 256) {
        row_best[pr][r] = fabsf(best[1]) > fabsf(best[0]) ? best[1] : best[0];
        __syncthreads();
        float e = 0.f;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float c = row_best[q][r];
            if (fabsf(c) > fabsf(e)) e = c;
        }
        best[0] = best[1] = e;
    }
    float inverse[2], d[2];
#pragma unroll
    for (int g = 0; g < 2; ++g) {
        const bool nonzero = fabsf(best[g]) > 0.f;
        inverse[g] = nonzero ? __fdiv_rn(-127.0f, best[g]) : 0.f;
        d[g] = nonzero ? __fdiv_rn(1.0f, inverse[g]) : 0.f;
    }
    float sums[2] = {0.f, 0.f};
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        float q[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            int code = __float2int_rn(__fmul_rn(v[8 * c + j], inverse[c >> 2]));
            code = code < -128 ? -128 : (code > 127 ? 127 : code);
            q[j] = __fmul_rn((float)code, d[c >> 2]);
            sums[c >> 2] += q[j];
        }
        uint32_t hw[4], lw[4];
        split2(q[0], q[2], hw[0], lw[0]);
        split2(q[1], q[3], hw[1], lw[1]);
        split2(q[4], q[6], hw[2], lw[2]);
        split2(q[5], q[7], hw[3], lw[3]);
        *(uint4*)(hi + swizzled(r, c)) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
        *(uint4*)(lo + swizzled(r, c)) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
    }
    if (xg) {
        const int windows = ((int)gridDim.x + 7) >> 3;
        uint8_t* ghi = xg + ((size_t)nt * windows + (sb >> 3)) * 2 * (size_t)bn * 128;
        uint8_t* glo = ghi + (size_t)bn * 128;
        uint32_t h, l;
        split2(sums[0], sums[1], h, l);
        *(uint32_t*)(ghi + swizzled(r, sb & 7) + 4 * pr) = h;
        *(uint32_t*)(glo + swizzled(r, sb & 7) + 4 * pr) = l;
    }
}

template <int TYPE>
__global__ void __launch_bounds__(kThreadsKq, 1) rq_matmul_kq_kernel(const __grid_constant__ KqParams p) {
    constexpr bool kQ4 = TYPE == RQ_Q4_K;
    constexpr int kUnit = kQ4 ? 144 : 208;           // stored bytes of one row's superblock in the main plane
    constexpr int kRawBytes = 128 * kUnit;           // one TMA tile: 128 rows x one superblock
    constexpr int kACols = kQ4 ? 32 : 64;            // tensor-memory columns of one operand slot: 64 fp16 per row (and their residuals)
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);  // swizzled tiles want 1024-byte alignment
    // Every barrier array is indexed by the slice, ks % kMaxSlots, not by the slot the slice uses: a parity wait is only sound
    // while the waiter is less than one phase behind, and the issuing threads run up to kMmaWarps slices apart whatever the
    // number of slots or accumulators (kMaxSlots >= slots + kMmaWarps keeps every waiter within a phase).
    // done[]: the single tcgen05.commit of slice ks arrives on done[ks % kMaxSlots] when the slice's products have finished.
    // The drain warps wait for it (the sum is complete), the staging warps wait for the slice that used their operand slot
    // last, the copy warp for the slice that used its activation slot last.
    __shared__ __align__(8) uint64_t b_full[kMaxSlots], a_full[kMaxSlots], done[kMaxSlots], acc_empty[kMaxSlots], raw_full[kRawSlots], raw_empty[kRawSlots], done_bar,
        min_full, min_free;
    __shared__ uint32_t tmem_base_slot;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t m0 = (int64_t)blockIdx.x * BM;
    const int nt = blockIdx.y, bn = p.bn, n0 = nt * bn;
    const int nb = p.cols >> 8;                                   // superblocks per row
    const int sb_first = blockIdx.z * p.sb_per_split;            // this CTA's superblocks
    const int n_sb = min(p.sb_per_split, nb - sb_first);
    const int k_steps = 4 * n_sb, kg_first = 4 * sb_first;       // 64-wide slices
    const int b_slots = p.b_slots, a_slots = p.a_slots, accs = p.accs;
    const int b_bytes = 2 * bn * 128;                             // one slice's B_hi | B_lo
    uint8_t* raw = smem + (size_t)b_slots * b_bytes;              // kRawSlots tiles of stored bytes
    uint8_t* min_a = raw + (size_t)kRawSlots * kRawBytes;         // Q4_K: A' hi | A' lo (16 KB each), then B' hi | B' lo
    min_a = (uint8_t*)(((uintptr_t)min_a + 1023) & ~(uintptr_t)1023);
    uint8_t* min_b = min_a + 2 * kTileBytes;
    // tensor memory: the accumulators, for Q4_K one for the minimum term, then the operand slots; a power of two of columns
    const int acc_cols = (accs + (kQ4 ? 1 : 0)) * bn;
    const int want_cols = acc_cols + a_slots * kACols;
    uint32_t tmem_cols = 32;
    while ((int)tmem_cols < want_cols) tmem_cols <<= 1;

    if (tid == 0) {
        for (int s = 0; s < kMaxSlots; ++s) { mbar_init(&b_full[s], 1); mbar_init(&a_full[s], kStageWarps); mbar_init(&done[s], 1); mbar_init(&acc_empty[s], kDrainWarps); }
        for (int s = 0; s < kRawSlots; ++s) { mbar_init(&raw_full[s], 1); mbar_init(&raw_empty[s], kStageWarps); }
        mbar_init(&done_bar, 1);
        mbar_init(&min_full, 1);
        mbar_init(&min_free, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (kQ4 && warp < kStageWarps) {
        // the minimum term's weight tiles start as zeros: chunks this CTA never writes must multiply to nothing
        for (int i = tid; i < 2 * kTileBytes / 16; i += kStagers) ((uint4*)min_a)[i] = make_uint4(0, 0, 0, 0);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;
    const uint32_t acc_min = tmem_base + (uint32_t)(accs * bn);
    const uint32_t a_ring = tmem_base + (uint32_t)acc_cols;

    if (warp < kStageWarps) {
        // ------------------------------------------------------------ staging warps: stored bytes -> integer operands in tensor memory
        // thread = (row r of the tile, half of the slice's 64 inputs); a warp may write the 32 tensor-memory lanes 32 (warp % 4) ..,
        // so warps 0-3 take the rows' first halves and warps 4-7 their second halves
        const int r = tid & 127, half = tid >> 7;
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        bool dead = false;
        for (int s = 0; s < n_sb; ++s) {
            const int rslot = s % kRawSlots;
            if (!dead && !mbar_wait_warp(&raw_full[rslot], (s / kRawSlots) & 1, p.wait_ns)) { atomicExch(p.error_flag, 18); dead = true; }
            const uint8_t* tile = raw + (size_t)rslot * kRawBytes;
#pragma unroll 1
            for (int pr = 0; pr < 4; ++pr) {
                const int ks = 4 * s + pr, kg = kg_first + ks, aslot = ks % a_slots;
                RawKq<TYPE> cur;
                cur.load(tile, r, pr, half);
                uint4 hi[4], lo[4];
                cur.decode(kg, half, hi, lo);
                // the operand slot is free once the products of the slice that used it last have finished
                if (ks >= a_slots && !dead && !mbar_wait_warp(&done[(ks - a_slots) % kMaxSlots], ((ks - a_slots) / kMaxSlots) & 1, p.wait_ns)) { atomicExch(p.error_flag, 11); dead = true; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t at = a_ring + lane_base + (uint32_t)(aslot * kACols + 16 * half);
                tmem_st16(at, (const uint32_t*)hi);
                if (!kQ4) tmem_st16(at + 32, (const uint32_t*)lo);
                bool wrote_shared = false;
                if (kQ4 && half == 0 && pr == 3) {
                    // The superblock's minimum-term weights, one 16-byte chunk per row. The tiles are reused window after window
                    // (eight superblocks): the first chunk of a window waits until the previous window's products have read them.
                    const int sb_abs = kg >> 2, w_local = (sb_abs >> 3) - (sb_first >> 3);
                    if ((sb_abs & 7) == 0 && w_local >= 1 && !dead && !mbar_wait_warp(&min_free, (w_local - 1) & 1, p.wait_ns)) { atomicExch(p.error_flag, 11); dead = true; }
                    uint4 mh, ml;
                    cur.minimum_terms(mh, ml);
                    const int chunk = sb_abs & 7;
                    *(uint4*)(min_a + swizzled(r, chunk)) = mh;
                    *(uint4*)(min_a + kTileBytes + swizzled(r, chunk)) = ml;
                    if (ks == k_steps - 1 && chunk < 7) {
                        // the CTA's last superblock: the chunk after it shares a 16-wide slice with it when `chunk` is even
                        *(uint4*)(min_a + swizzled(r, chunk + 1)) = make_uint4(0, 0, 0, 0);
                        *(uint4*)(min_a + kTileBytes + swizzled(r, chunk + 1)) = make_uint4(0, 0, 0, 0);
                    }
                    wrote_shared = true;
                }
                tmem_st_wait();
                if (wrote_shared) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the tensor core reads those tiles through the async proxy
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(&a_full[ks % kMaxSlots]);  // one arrival per warp (an arrival is an atomic on the barrier)
            }
            // this warp has read the superblock's stored bytes: the copy warp may fetch another into the slot
            __syncwarp();
            if (lane == 0) mbar_arrive(&raw_empty[rslot]);
        }
    } else if (warp < kMmaWarp) {
        // ------------------------------------------------------------ drain warps: tensor memory -> d * sum -> fp32 registers -> Y
        // warp w may read accumulator rows 32 (w % 4) ..; the eight warps split the columns in two
        const int dw = warp - kStageWarps, quarter = warp & 3, chalf = dw >> 2;
        const int cols_here = bn >> 1 > 16 ? bn >> 1 : 16;       // bn = 16: both halves would be the same sixteen columns,
        const bool active = bn > 16 || chalf == 0;               // so only the first four warps drain
        const int col0 = active ? chalf * cols_here : 0;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const int64_t out_row = m0 + quarter * 32 + lane;
        const int64_t d_row = out_row < p.rows ? out_row : p.rows - 1;
        float acc[64];
#pragma unroll
        for (int i = 0; i < 64; ++i) acc[i] = 0.f;
        bool dead = false;
        auto d_of = [&](int sb) -> float {
            if (kQ4) return rq_h2f(__ldg((const uint16_t*)(p.main + (d_row * nb + sb) * 144)));
            return rq_h2f(__ldg(p.scale + d_row * nb + sb));
        };
        float d = d_of(sb_first);
        for (int ks = 0; ks < k_steps; ++ks) {
            const int a = ks % accs;
            // the next superblock's d is on its way while this superblock's last slice is drained
            float d_next = d;
            if ((ks & 3) == 3 && ks + 1 < k_steps) d_next = d_of(sb_first + (ks >> 2) + 1);
            if (!dead && !mbar_wait_warp(&done[ks % kMaxSlots], (ks / kMaxSlots) & 1, p.wait_ns)) { atomicExch(p.error_flag, 14); dead = true; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (active) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    if (16 * c < cols_here) {
                        uint32_t t[16];
                        tmem_ld16(tmem_base + lane_base + (uint32_t)(a * bn + col0 + 16 * c), t);
#pragma unroll
                        for (int j = 0; j < 16; ++j) acc[16 * c + j] = fmaf(d, __uint_as_float(t[j]), acc[16 * c + j]);
                    }
                }
            }
            // this warp has read the accumulator: the tensor core may overwrite it
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[ks % kMaxSlots]);
            d = d_next;
        }
        if (!dead && !mbar_wait_warp(&done_bar, 0, p.wait_ns)) { atomicExch(p.error_flag, 12); dead = true; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (active) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                if (16 * c < cols_here) {
                    uint32_t t[16];
                    if (kQ4) tmem_ld16(acc_min + lane_base + (uint32_t)(col0 + 16 * c), t);  // the minimum term
                    if (out_row < p.rows && !dead) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int token = n0 + col0 + 16 * c + j;
                            const float out = kQ4 ? fmaf(-kMinUnscale, __uint_as_float(t[j]), acc[16 * c + j]) : acc[16 * c + j];
                            if (token < p.tokens) {
                                if (gridDim.z == 1) p.y[out_row * p.yn + (int64_t)token * p.yt] = out;
                                else p.partial[((size_t)blockIdx.z * p.tokens + token) * p.rows + out_row] = out;
                            }
                        }
                    }
                }
            }
        }
    } else if (warp < kCopyWarp) {
        // ------------------------------------------------------------ MMA warps (lane 0 of each issues): warp i takes slices i, i + kMmaWarps, ..
        // One thread's loop of waits, instruction issue and commit is a chain of slow operations (a look at a barrier, a
        // tcgen05.mma, a commit each cost it on the order of a hundred cycles), some 2000 cycles a slice where the tensor core
        // needs 500. Several threads on interleaved slices, each slice with its own accumulator, overlap those chains. A commit
        // covers its own thread's products only, which is what a slice's barrier needs; the minimum term and the CTA's last
        // slice (ks = 3 mod 4 both, kMmaWarps dividing 4) belong to the last of the threads.
        static_assert(4 % kMmaWarps == 0, "window ends must all fall to one issuing thread");
        const int first_slice = warp - kMmaWarp;
        bool dead = false;
        const uint32_t idesc = instr_desc(bn);
        bool min_started = false;
        // one thread waits, issues and commits: nothing here needs the other lanes, and a warp-wide look at a barrier costs
        // thirty-two operations on its word
        for (int ks = first_slice; lane == 0 && ks < k_steps; ks += kMmaWarps) {
            const int aslot = ks % a_slots, bslot = ks % b_slots, a = ks % accs;
            const int sb_abs = sb_first + (ks >> 2);
            if (!dead && !mbar_wait(&a_full[ks % kMaxSlots], (ks / kMaxSlots) & 1, p.wait_ns)) { atomicExch(p.error_flag, 13); dead = true; }
            if (!dead && !mbar_wait(&b_full[ks % kMaxSlots], (ks / kMaxSlots) & 1, p.wait_ns)) { atomicExch(p.error_flag, 13); dead = true; }
            if (ks >= accs && !dead && !mbar_wait(&acc_empty[(ks - accs) % kMaxSlots], ((ks - accs) / kMaxSlots) & 1, p.wait_ns)) { atomicExch(p.error_flag, 15); dead = true; }
            // Q4_K: at the end of each window of eight superblocks (and at the CTA's last), the window's minimum-term product
            const bool window_end = kQ4 && (ks & 3) == 3 && ((sb_abs & 7) == 7 || ks == k_steps - 1);
            if (window_end && !dead) {
                // windows are numbered from the CTA's first: the copy warp arms min_full once per window, in order
                const int w_local = (sb_abs >> 3) - (sb_first >> 3);
                if (!mbar_wait(&min_full, w_local & 1, p.wait_ns)) { atomicExch(p.error_flag, 17); dead = true; }
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (!dead) {
                const uint32_t bbase = smem_u32(smem + (size_t)bslot * b_bytes);
                const uint64_t b_hi = smem_desc(bbase), b_lo = smem_desc(bbase + bn * 128);
                const uint32_t a_hi = a_ring + (uint32_t)(aslot * kACols), a_lo = a_hi + 32;
                const uint32_t acc_main = tmem_base + (uint32_t)(a * bn);
                // a fresh sum for every slice; the cross terms (2^-11 of the sum) first, the main term last
#pragma unroll
                for (int kk = 0; kk < BK / 16; ++kk) {
                    const uint64_t adv = (uint64_t)(kk * 2);  // 32 bytes along K, in 16-byte units of the descriptor's start address
                    mma_f16_ts(acc_main, a_hi + 8 * kk, b_lo + adv, idesc, kk ? 1u : 0u);
                    if (!kQ4) mma_f16_ts(acc_main, a_lo + 8 * kk, b_hi + adv, idesc, 1u);
                }
#pragma unroll
                for (int kk = 0; kk < BK / 16; ++kk) mma_f16_ts(acc_main, a_hi + 8 * kk, b_hi + (uint64_t)(kk * 2), idesc, 1u);
                if (window_end) {
                    // chunks [first, last] of the window belong to this CTA: the 16-wide slices that hold them
                    const int first_chunk = (sb_abs >> 3) == (sb_first >> 3) ? (sb_first & 7) : 0, last_chunk = sb_abs & 7;
                    const uint32_t mbase = smem_u32(min_a), mbb = smem_u32(min_b);
                    const uint64_t ma_hi = smem_desc(mbase), ma_lo = smem_desc(mbase + kTileBytes);
                    const uint64_t mb_hi = smem_desc(mbb), mb_lo = smem_desc(mbb + bn * 128);
                    for (int kk = first_chunk >> 1; kk <= last_chunk >> 1; ++kk) {
                        const uint64_t adv = (uint64_t)(kk * 2);
                        mma_f16(acc_min, ma_hi + adv, mb_hi + adv, idesc, min_started ? 1u : 0u);
                        mma_f16(acc_min, ma_hi + adv, mb_lo + adv, idesc, 1u);
                        mma_f16(acc_min, ma_lo + adv, mb_hi + adv, idesc, 1u);
                        min_started = true;
                    }
                    mma_commit(&min_free);  // the minimum tiles may be rewritten once these have finished
                }
                // one commit: the slice's sum is complete, and its operand and activation slots are free
                if (ks == k_steps - 1) mma_commit(&done_bar);
                mma_commit(&done[ks % kMaxSlots]);
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ copy warp: lane 0 the prepared X tiles, lane 1 the stored weight bytes
        if (lane == 1) {
            // weights are constants of the model: nothing to wait for before the first fetches
            for (int s = 0; s < n_sb; ++s) {
                const int rslot = s % kRawSlots;
                if (s >= kRawSlots && !mbar_wait(&raw_empty[rslot], ((s / kRawSlots) - 1) & 1, p.wait_ns)) { atomicExch(p.error_flag, 19); break; }
                mbar_expect_tx(&raw_full[rslot], kRawBytes);
                tma_load_2d(raw + (size_t)rslot * kRawBytes, &p.tile_map, (sb_first + s) * kUnit, (int)m0, &raw_full[rslot]);
            }
        } else if (lane == 0) {
            // the activation images were written by the kernel before this one
            asm volatile("griddepcontrol.wait;" ::: "memory");
            const uint32_t bytes = (uint32_t)b_bytes;
            const int k_total = p.cols / BK, windows = (nb + 7) >> 3;
            const uint8_t* src = p.xs + ((size_t)nt * k_total + kg_first) * bytes;
            int w_issue = 0;
            const int w_last = ((sb_first + n_sb - 1) >> 3) - (sb_first >> 3);  // windows of eight superblocks this CTA touches, counted from its first
            for (int ks = 0; ks < k_steps; ++ks) {
                const int bslot = ks % b_slots;
                if (ks >= b_slots && !mbar_wait(&done[(ks - b_slots) % kMaxSlots], ((ks - b_slots) / kMaxSlots) & 1, p.wait_ns)) { atomicExch(p.error_flag, 16); break; }
                mbar_expect_tx(&b_full[ks % kMaxSlots], bytes);
                bulk_g2s(smem + (size_t)bslot * b_bytes, src + (size_t)ks * bytes, bytes, &b_full[ks % kMaxSlots]);
                if (kQ4 && w_issue <= w_last) {
                    // The group sums of window `w_issue`: the CTA's first window at once; a later window a few slices into it (by
                    // then the previous window's products, which read this tile, have finished: min_free says so), or at the
                    // window's last slice when the window is shorter than that.
                    const int win = (sb_first >> 3) + w_issue;
                    const int win_first_sb = w_issue == 0 ? sb_first : win << 3;
                    const int win_last_sb = min(sb_first + n_sb - 1, (win << 3) + 7);
                    const int ks_begin = (win_first_sb - sb_first) * 4, ks_end = (win_last_sb - sb_first) * 4 + 3;
                    const int ks_issue = w_issue == 0 ? 0 : min(ks_begin + b_slots, ks_end);
                    if (ks == ks_issue) {
                        if (w_issue > 0 && !mbar_wait(&min_free, (w_issue - 1) & 1, p.wait_ns)) { atomicExch(p.error_flag, 16); break; }
                        mbar_expect_tx(&min_full, bytes);
                        bulk_g2s(min_b, p.xg + ((size_t)nt * windows + win) * bytes, bytes, &min_full);
                        ++w_issue;
                    }
                }
            }
        }
    }
    // free the tensor memory: everyone is past its use
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == kMmaWarp) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
}

template <int TYPE>
int launch_kq(const KqParams& p, int grid_m, int grid_n, int grid_k, size_t smem, cudaStream_t s) {
    auto kernel = rq_matmul_kq_kernel<TYPE>;
    static bool configured[64] = {};
    int dev = 0;
    RQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        RQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 225 * 1024));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid_m, (unsigned)grid_n, (unsigned)grid_k);
    cfg.blockDim = dim3(kThreadsKq);
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

// How a call is cut: tokens per tile, superblocks per CTA, CTAs along K, pipeline depth, shared memory and scratch.
struct KqCut {
    int bn, n_tiles, sb_per_split, splits, b_slots, a_slots, accs;
    size_t smem, xs_bytes, xg_bytes, partial_bytes;
};
KqCut kq_cut(int type, int sm_count, int64_t rows, int64_t cols, int tokens) {
    KqCut c;
    c.bn = tokens <= 16 ? 16 : (tokens <= 32 ? 32 : (tokens <= 64 ? 64 : 128));
    c.n_tiles = (tokens + c.bn - 1) / c.bn;
    const int nb = (int)(cols >> 8);
    const bool q4 = type == RQ_Q4_K;
    // tensor memory (512 columns): four operand slots, the minimum term's accumulator (Q4_K), the rest accumulators
    c.a_slots = 4;
    c.accs = (512 - c.a_slots * (q4 ? 32 : 64) - (q4 ? c.bn : 0)) / c.bn;
    if (c.accs > 4) c.accs = 4;
    // shared memory: the stored-byte tiles, the minimum term's tiles (Q4_K), the rest activation slots
    const size_t raw = (size_t)kRawSlots * 128 * (q4 ? 144 : 208) + 1024;
    const size_t fixed = q4 ? 2 * (size_t)kTileBytes + 2 * (size_t)c.bn * 128 : 0;
    const size_t slot = 2 * (size_t)c.bn * 128;
    c.b_slots = (int)((220 * 1024 - raw - fixed) / slot);
    if (c.b_slots > 6) c.b_slots = 6;
    c.smem = (size_t)c.b_slots * slot + raw + fixed + 1024;
    // CTAs along K: the cut that leaves the busiest SM the least work, counting about one superblock's time per CTA for
    // its prologue and drain, with at least two superblocks per CTA
    const int64_t tiles = ((rows + BM - 1) / BM) * c.n_tiles;
    int best = 1;
    double best_cost = 1e30;
    for (int s = 1; s <= 16 && s <= (nb + 1) / 2; ++s) {
        const int per = (nb + s - 1) / s, real = (nb + per - 1) / per;
        const double waves = (double)((tiles * real + sm_count - 1) / sm_count);
        const double cost = waves * (per + 1.0) + (real > 1 ? 0.5 : 0.0);
        if (cost < best_cost - 1e-9) { best_cost = cost; best = real; }
    }
    c.sb_per_split = (nb + best - 1) / best;
    c.splits = (nb + c.sb_per_split - 1) / c.sb_per_split;
    c.xs_bytes = (size_t)c.n_tiles * (size_t)(cols / BK) * 2 * c.bn * 128;
    c.xg_bytes = type == RQ_Q4_K ? (size_t)c.n_tiles * (size_t)((nb + 7) / 8) * 2 * c.bn * 128 : 0;
    c.partial_bytes = c.splits > 1 ? (size_t)c.splits * tokens * rows * 4 : 0;
    return c;
}

}  // namespace

size_t rq_matmul_kq_scratch_bytes(const rq_ctx* ctx, int type, int64_t rows, int64_t cols, int tokens) {
    const KqCut c = kq_cut(type, ctx->sm_count, rows, cols, tokens);
    return c.xs_bytes + c.xg_bytes + c.partial_bytes;
}

// RQ_ERR_UNSUPPORTED (no error text) = not a K-quant weight. act_mode FLOAT or INT8 (step 32 / 256).
int rq_launch_matmul_kq(rq_ctx* ctx, const rq_weight* w, const float* x, int64_t sk, int64_t st, int tokens, float* y, int64_t yn, int64_t yt, int act_mode,
                        int step, cudaStream_t s) {
    if ((w->type != RQ_Q4_K && w->type != RQ_Q6_K) || w->cols % 256 || !w->has_tile_map) return RQ_ERR_UNSUPPORTED;
    const bool int8 = act_mode != RQ_ACT_FLOAT;
    const KqCut cut = kq_cut(w->type, ctx->sm_count, w->rows, w->cols, tokens);
    int rc = rq_ensure_act_scratch(ctx, cut.xs_bytes + cut.xg_bytes + cut.partial_bytes, s);
    if (rc) return rc;
    ctx->act_cols = 0;  // whatever int8 records the scratch held for INT8_CACHED calls are gone
    uint8_t* xs = ctx->act_scratch;
    uint8_t* xg = cut.xg_bytes ? xs + cut.xs_bytes : nullptr;
    float* partial = cut.splits > 1 ? (float*)(xs + cut.xs_bytes + cut.xg_bytes) : nullptr;
    if (xg) RQ_CUDA(cudaMemsetAsync(xg, 0, cut.xg_bytes, s));  // groups past the last superblock of a window count as zeros
    {
        cudaLaunchConfig_t cfg = {};
        cfg.stream = s;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = int8 && !xg ? 1 : 0;  // after a memset node the kernel is launched the plain way
        if (int8) {
            cfg.gridDim = dim3((unsigned)(w->cols >> 8), (unsigned)cut.n_tiles);
            cfg.blockDim = dim3((unsigned)cut.bn, 4);
            if (step == 256) RQ_CUDA(cudaLaunchKernelEx(&cfg, rq_kq_prep_int8_kernel<256>, x, sk, st, tokens, cut.bn, xs, xg));
            else RQ_CUDA(cudaLaunchKernelEx(&cfg, rq_kq_prep_int8_kernel<32>, x, sk, st, tokens, cut.bn, xs, xg));
        } else {
            cfg.gridDim = dim3((unsigned)(w->cols / BK), (unsigned)cut.n_tiles);
            cfg.blockDim = dim3(128);
            RQ_CUDA(cudaLaunchKernelEx(&cfg, rq_kq_prep_kernel, x, sk, st, (int)w->cols, tokens, cut.bn, xs, xg));
        }
    }
    KqParams p;
    p.main = w->main; p.scale = w->scale; p.rows = w->rows; p.cols = (int)w->cols;
    p.xs = xs; p.xg = xg; p.bn = cut.bn; p.tokens = tokens; p.y = y; p.yn = yn; p.yt = yt;
    p.sb_per_split = cut.sb_per_split; p.partial = partial; p.b_slots = cut.b_slots; p.a_slots = cut.a_slots; p.accs = cut.accs;
    p.tile_map = w->tile_map;
    p.error_flag = ctx->error_flag; p.wait_ns = ctx->wait_limit_ns;
    const int grid_m = (int)((w->rows + BM - 1) / BM);
    rc = w->type == RQ_Q4_K ? launch_kq<RQ_Q4_K>(p, grid_m, cut.n_tiles, cut.splits, cut.smem, s) : launch_kq<RQ_Q6_K>(p, grid_m, cut.n_tiles, cut.splits, cut.smem, s);
    if (rc || cut.splits == 1) return rc;
    return rq_launch_sum_splits(partial, cut.splits, w->rows, tokens, y, yn, yt, s);
}
