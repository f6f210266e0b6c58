// Batched product over Q4_K / Q6_K weights on the 5th-generation tensor cores, with EXACT INTEGER
// weight operands.
//
//   Y[t][n] = sum_k W[n][k] * X[t][k]
//
// A K-quant value factors into a per-superblock fp16 scale and small integers:
//   Q4_K : w = d * (sc_g * q) - dmin * m_g        sc_g, m_g six bits, q four bits: sc_g * q <= 945
//   Q6_K : w = d * (s_j * (q - 32))               s_j int8, q six bits: |s_j * (q - 32)| <= 4096
// fp16 holds every integer up to 2048 exactly, so the tensor core is fed the integers themselves
// (Q4_K: one operand; Q6_K: the fp16 rounding of the integer plus its exact residual, -1 / 0 / 1)
// and `d` is applied outside it, when a sum leaves tensor memory.
// Unpacking is integer and half2 arithmetic only: a nibble pair becomes (1024 + q) by an OR with
// 0x6400, one HFMA2 turns it into sc * q exactly. The activations are fp32 and go in as fp16 pairs
// hi + lo (22 mantissa bits), prepared once per call by rq_kq_prep_kernel in the tensor core's
// 128-byte-swizzled K-major image; the two middle inputs of every four swap places there, because
// that is the order the nibble pairs come out of a 32-bit word.
//
// Per 16-wide slice: Q4_K issues A x B_hi and A x B_lo (two instructions where split weights need
// three), Q6_K issues A_hi x B_hi, A_hi x B_lo, A_lo x B_hi. The tensor core adds into its fp32
// accumulator by TRUNCATION, a bias that grows with the length of the chain (measured: 7e-7 relative
// over 256 inputs, 1.2e-5 over 4096). So a sum stays in tensor memory for one 64-wide slice only, in
// one of two accumulators in turn, the small cross terms issued first (while the accumulator is
// still small, their truncation is nothing); eight drain warps multiply each finished slice by the
// superblock's d and add it into fp32 registers with one round-to-nearest fma per value while the
// tensor core fills the other accumulator.
//
// The Q4_K minimum term, sum_g (dmin * m_g) * (sum of x over group g), is a second, 32 times smaller
// product. Its operands (dmin * m_g as fp16 hi + lo, scaled by 2^8; the group sums of x as hi + lo)
// are collected for eight superblocks at a time in one more pair of swizzled tiles and multiplied
// into a third accumulator that lives for the whole K.
//
// INT8 activations take the same kernel: the int8 records are made by the standalone quantiser
// (bit-exact with the reference's) and the prepared image holds code * step, which is what the
// integer dot multiplies out to; only the order of the fp32 additions differs.
//
// Every wait is bounded; a wait that runs out records a code in the context's error word, the
// thread stops waiting and the CTA still frees its tensor memory before it exits.
#include "rq_internal.cuh"
#include "rq_mma.cuh"

using namespace rqmma;

namespace {

constexpr int kStageWarps = 8, kDrainWarps = 8;
constexpr int kStagers = kStageWarps * 32;
constexpr int kMmaWarp = kStageWarps + kDrainWarps, kCopyWarp = kMmaWarp + 1;
constexpr int kThreadsKq = (kCopyWarp + 1) * 32;
constexpr int kTileBytes = BM * BK * 2;  // one fp16 tile of 128 rows x 64 inputs: 16 KB
constexpr int kMaxStages = 6;
constexpr float kMinScale = 256.0f, kMinUnscale = 1.0f / 256.0f;  // the minimum term's weights are scaled so that their fp16 residuals are no subnormals

struct KqParams {
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
    int stages;            // ring slots; each has its own accumulator of bn columns in tensor memory
    int slices_per_stage;  // 64-wide slices per stage: 1, 2 or 4 (fewer, larger stages when the token tile is narrow)
    int* error_flag;
    unsigned long long wait_ns;
};

__device__ __forceinline__ __half2 as_half2(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }
__device__ __forceinline__ uint32_t as_u32(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }

// ------------------------------------------------------------------------------------------
// The raw bytes behind 32 consecutive inputs of one row (`half` 0 or 1 of the 64-wide slice
// `kg`), and their integer operands as 32 fp16 values (four 16-byte chunks), inputs in the order
// 0 2 1 3 within every four.
// ------------------------------------------------------------------------------------------
template <int TYPE> struct RawKq;
template <> struct RawKq<RQ_Q4_K> {
    uint4 hdr, q0, q1;
    __device__ __forceinline__ void load(const KqParams& p, int64_t row, int kg, int) {
        const uint8_t* blk = p.main + (row * (p.cols >> 8) + (kg >> 2)) * 144;
        const int pr = kg & 3;
        hdr = __ldg((const uint4*)blk);
        q0 = __ldg((const uint4*)(blk + 16 + 32 * pr));
        q1 = __ldg((const uint4*)(blk + 32 + 32 * pr));
    }
    // sc * q of sub-block 2 pr + half (low nibbles hold sub-block 2 pr, high nibbles 2 pr + 1)
    __device__ __forceinline__ void decode(int kg, int half, uint4* hi, uint4*) const {
        int sc, mn;
        rq_q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * (kg & 3) + half, sc, mn);
        const __half2 sc2 = __half2half2(__int2half_rn(sc));
        const __half2 off2 = __half2half2(__float2half_rn(-1024.0f * (float)sc));  // at most 64512: exact
        const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        const int shift = 4 * half;
        uint32_t o[16];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            // 0x6400 | n is the fp16 number 1024 + n; (1024 + q) * sc - 1024 * sc is exact inside the fused operation
            const uint32_t a = ((w[j] >> shift) & 0x000F000Fu) | 0x64006400u;        // inputs 4j, 4j + 2
            const uint32_t b = ((w[j] >> (shift + 8)) & 0x000F000Fu) | 0x64006400u;  // inputs 4j + 1, 4j + 3
            o[2 * j] = as_u32(__hfma2(as_half2(a), sc2, off2));
            o[2 * j + 1] = as_u32(__hfma2(as_half2(b), sc2, off2));
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) hi[c] = make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
    }
    // dmin * m_g of the superblock's eight sub-blocks, times 2^8, as fp16 hi and lo
    __device__ __forceinline__ void minimum_terms(uint4& hi, uint4& lo) const {
        const float dmin = rq_h2f((uint16_t)(hdr.x >> 16));
        uint32_t hw[4], lw[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int s0, m0, s1, m1;
            rq_q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * j, s0, m0);
            rq_q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * j + 1, s1, m1);
            const float a = __fmul_rn(__fmul_rn(dmin, (float)m0), kMinScale), b = __fmul_rn(__fmul_rn(dmin, (float)m1), kMinScale);
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
    __device__ __forceinline__ void load(const KqParams& p, int64_t row, int kg, int half) {
        const int j64 = kg & 3, ch = j64 >> 1, sel = j64 & 1, g = 2 * sel + half;
        const uint8_t* body = p.main + (row * (p.cols >> 8) + (kg >> 2)) * 208;
        ql[0] = __ldg((const uint4*)(body + 64 * ch + 32 * half));
        ql[1] = __ldg((const uint4*)(body + 64 * ch + 32 * half + 16));
        qh[0] = __ldg((const uint4*)(body + 128 + 32 * ch));
        qh[1] = __ldg((const uint4*)(body + 128 + 32 * ch + 16));
        scales = __ldg((const uint16_t*)(body + 192 + 8 * ch + 2 * g));
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
// X -> the tensor core's operand images. grid (64-wide slices, token tiles), one thread per token
// row of the tile; rows past the last token are zero. With `records` the inputs are the int8
// activation records' code * step (unit records, one after another per token).
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) rq_kq_prep_kernel(const float* __restrict__ x, int64_t sk, int64_t st, const uint8_t* __restrict__ records, int cols,
                                                          int tokens, int bn, uint8_t* __restrict__ xs, uint8_t* __restrict__ xg) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int kg = blockIdx.x, nt = blockIdx.y, r = threadIdx.x;
    if (r >= bn) return;
    const int token = nt * bn + r;
    uint8_t* hi = xs + ((size_t)nt * gridDim.x + kg) * 2 * (size_t)bn * 128;
    uint8_t* lo = hi + (size_t)bn * 128;
    float sums[2] = {0.f, 0.f};
    const bool vec = !records && sk == 1 && (st & 3) == 0 && ((uintptr_t)x & 15) == 0;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        float v[8];
        if (token >= tokens) {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = 0.f;
        } else if (records) {
            const uint8_t* rec = records + ((size_t)token * (cols >> 8) + (kg >> 2)) * RQ_ACT_RECORD_INT8;
            const uint2 codes = *(const uint2*)(rec + 64 * (kg & 3) + 8 * c);
            const float d = ((const float*)(rec + 256))[2 * (kg & 3) + (c >> 2)];
            const uint32_t cw[2] = {codes.x, codes.y};
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = __fmul_rn((float)(int8_t)(cw[j >> 2] >> (8 * (j & 3))), d);
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

template <int TYPE>
__global__ void __launch_bounds__(kThreadsKq, 1) rq_matmul_kq_kernel(const __grid_constant__ KqParams p) {
    constexpr bool kQ4 = TYPE == RQ_Q4_K;
    constexpr int kATiles = kQ4 ? 1 : 2;  // A | A_hi, A_lo
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);  // swizzled tiles want 1024-byte alignment
    // One barrier says "stage filled" (the staging warps and the activation copy arrive), one says "stage done": the single
    // tcgen05.commit of a stage arrives on it when the stage's products have finished, and both the drain warps (the sum
    // is complete) and the staging and copy warps (the slot is free) wait on it. A commit costs the issuing thread some 200
    // cycles, so a stage has exactly one. acc_empty: the drain warps have read the stage's accumulator.
    __shared__ __align__(8) uint64_t full_bar[kMaxStages], stage_done[kMaxStages], acc_empty[kMaxStages], done_bar, min_full, min_free;
    __shared__ uint32_t tmem_base_slot;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t m0 = (int64_t)blockIdx.x * BM;
    const int nt = blockIdx.y, bn = p.bn, n0 = nt * bn;
    const int nb = p.cols >> 8;                                   // superblocks per row
    const int sb_first = blockIdx.z * p.sb_per_split;            // this CTA's superblocks
    const int n_sb = min(p.sb_per_split, nb - sb_first);
    const int k_steps = 4 * n_sb, kg_first = 4 * sb_first;       // 64-wide slices
    const int stages = p.stages;                                  // ring slots, each with its own accumulator
    const int per = p.slices_per_stage;                           // 64-wide slices per stage: 1, 2 or 4
    const int n_stages = k_steps / per;
    const int a_bytes = kATiles * kTileBytes, b_bytes = 2 * bn * 128;  // one slice's weight tile(s), and its B_hi | B_lo
    const int stage_bytes = per * (a_bytes + b_bytes);            // the slices' A tiles, then their B tiles
    uint8_t* min_a = smem + (size_t)stages * stage_bytes;         // Q4_K: A' hi | A' lo (16 KB each), then B' hi | B' lo
    uint8_t* min_b = min_a + 2 * kTileBytes;
    // tensor memory: one accumulator per ring slot and, for Q4_K, one for the minimum term; a power of two of columns
    const int want_cols = (stages + (kQ4 ? 1 : 0)) * bn;
    uint32_t tmem_cols = 32;
    while ((int)tmem_cols < want_cols) tmem_cols <<= 1;

    if (tid == 0) {
        for (int s = 0; s < stages; ++s) { mbar_init(&full_bar[s], kStageWarps + 1); mbar_init(&stage_done[s], 1); mbar_init(&acc_empty[s], kDrainWarps); }
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
    const uint32_t acc_min = tmem_base + (uint32_t)(stages * bn);

    if (warp < kStageWarps) {
        // ------------------------------------------------------------ staging warps: W -> integer operand tiles
        const int r = tid & 127, half = tid >> 7;  // a row of the tile, and which 32 of a slice's 64 inputs
        const int64_t row = m0 + r < p.rows ? m0 + r : p.rows - 1;  // rows past the end are computed and dropped
        bool dead = false;
        // Three sets of raw bytes rotate by NAME (the loop is unrolled by three), never by copy: copying a set whose loads
        // are still in flight would wait for them, and the point is to have two slices' bytes on their way while one is
        // being unpacked.
        RawKq<TYPE> raw0, raw1, raw2;
        raw0.load(p, row, kg_first, half);
        if (k_steps > 1) raw1.load(p, row, kg_first + 1, half);
        auto slice_one = [&](int ks, const RawKq<TYPE>& cur, RawKq<TYPE>& ahead) {
            const int st = ks / per, sub = ks - st * per, slot = st % stages, kg = kg_first + ks;
            if (ks + 2 < k_steps) ahead.load(p, row, kg + 2, half);
            uint4 hi[4], lo[4];
            cur.decode(kg, half, hi, lo);
            // the slot is free once the products of the stage that used it last have finished
            if (sub == 0 && st >= stages && !dead && !mbar_wait(&stage_done[slot], ((st / stages) - 1) & 1, p.wait_ns)) { atomicExch(p.error_flag, 11); dead = true; }
            uint8_t* a_hi = smem + (size_t)slot * stage_bytes + (size_t)sub * a_bytes;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int off = swizzled(r, 4 * half + c);
                *(uint4*)(a_hi + off) = hi[c];
                if (!kQ4) *(uint4*)(a_hi + kTileBytes + off) = lo[c];
            }
            if (kQ4 && half == 0 && (kg & 3) == 3) {
                // The superblock's minimum-term weights, one 16-byte chunk per row. The tiles are reused window after window
                // (eight superblocks): the first chunk of a window waits until the previous window's products have read them.
                const int sb_abs = kg >> 2, w_local = (sb_abs >> 3) - (sb_first >> 3);
                if ((sb_abs & 7) == 0 && w_local >= 1 && !dead && !mbar_wait(&min_free, (w_local - 1) & 1, p.wait_ns)) { atomicExch(p.error_flag, 11); dead = true; }
                uint4 mh, ml;
                cur.minimum_terms(mh, ml);
                const int chunk = (kg >> 2) & 7;
                *(uint4*)(min_a + swizzled(r, chunk)) = mh;
                *(uint4*)(min_a + kTileBytes + swizzled(r, chunk)) = ml;
                if (ks == k_steps - 1 && chunk < 7) {
                    // the CTA's last superblock: the chunk after it shares a 16-wide slice with it when `chunk` is even
                    *(uint4*)(min_a + swizzled(r, chunk + 1)) = make_uint4(0, 0, 0, 0);
                    *(uint4*)(min_a + kTileBytes + swizzled(r, chunk + 1)) = make_uint4(0, 0, 0, 0);
                }
            }
            if (sub == per - 1) {
                // the tensor core reads shared memory through the async proxy: every thread orders its own stores before it,
                // then one lane per warp counts the warp in (an arrival is an atomic on the barrier: 8 per stage, not 256)
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(&full_bar[slot]);
            }
        };
        for (int ks = 0; ks < k_steps; ks += 3) {
            slice_one(ks, raw0, raw2);
            if (ks + 1 < k_steps) slice_one(ks + 1, raw1, raw0);
            if (ks + 2 < k_steps) slice_one(ks + 2, raw2, raw1);
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
        const int stages_per_sb = 4 / per;
        float d = d_of(sb_first);
        for (int st = 0; st < n_stages; ++st) {
            const int slot = st % stages;
            // the next superblock's d is on its way while this superblock's last stage is drained
            float d_next = d;
            if ((st + 1) % stages_per_sb == 0 && st + 1 < n_stages) d_next = d_of(sb_first + (st + 1) / stages_per_sb);
            if (!dead && !mbar_wait(&stage_done[slot], (st / stages) & 1, p.wait_ns)) { atomicExch(p.error_flag, 14); dead = true; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (active) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    if (16 * c < cols_here) {
                        uint32_t t[16];
                        tmem_ld16(tmem_base + lane_base + (uint32_t)(slot * bn + col0 + 16 * c), t);
#pragma unroll
                        for (int j = 0; j < 16; ++j) acc[16 * c + j] = fmaf(d, __uint_as_float(t[j]), acc[16 * c + j]);
                    }
                }
            }
            // this warp has read the accumulator: the tensor core may overwrite it
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[slot]);
            d = d_next;
        }
        if (!dead && !mbar_wait(&done_bar, 0, p.wait_ns)) { atomicExch(p.error_flag, 12); dead = true; }
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
    } else if (warp == kMmaWarp) {
        // ------------------------------------------------------------ MMA warp (lane 0 issues)
        bool dead = false;
        const uint32_t idesc = instr_desc(bn);
        bool min_started = false;
        for (int st = 0; st < n_stages; ++st) {
            const int slot = st % stages;
            const int ks_last = st * per + per - 1;                     // the stage's last 64-wide slice
            const int sb_abs = sb_first + (ks_last >> 2);
            if (!dead && !mbar_wait(&full_bar[slot], (st / stages) & 1, p.wait_ns)) { atomicExch(p.error_flag, 13); dead = true; }
            if (st >= stages && !dead && !mbar_wait(&acc_empty[slot], ((st / stages) - 1) & 1, p.wait_ns)) { atomicExch(p.error_flag, 15); dead = true; }
            // Q4_K: at the end of each window of eight superblocks (and at the CTA's last), the window's minimum-term product
            const bool window_end = kQ4 && (ks_last & 3) == 3 && ((sb_abs & 7) == 7 || ks_last == k_steps - 1);
            if (window_end && !dead) {
                // windows are numbered from the CTA's first: the copy warp arms min_full once per window, in order
                const int w_local = (sb_abs >> 3) - (sb_first >> 3);
                if (!mbar_wait(&min_full, w_local & 1, p.wait_ns)) { atomicExch(p.error_flag, 17); dead = true; }
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (lane == 0 && !dead) {
                const uint32_t base = smem_u32(smem + (size_t)slot * stage_bytes);
                const uint32_t acc_main = tmem_base + (uint32_t)(slot * bn);
                // a fresh sum for every stage; the cross terms (2^-11 of the sum) first, the main term last
                for (int sub = 0; sub < per; ++sub) {
                    const uint64_t a_hi = smem_desc(base + sub * a_bytes), a_lo = smem_desc(base + sub * a_bytes + kTileBytes);
                    const uint64_t b_hi = smem_desc(base + per * a_bytes + sub * b_bytes), b_lo = smem_desc(base + per * a_bytes + sub * b_bytes + bn * 128);
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk) {
                        const uint64_t adv = (uint64_t)(kk * 2);  // 32 bytes along K, in 16-byte units of the start address
                        mma_f16(acc_main, a_hi + adv, b_lo + adv, idesc, (sub | kk) ? 1u : 0u);
                        if (!kQ4) mma_f16(acc_main, a_lo + adv, b_hi + adv, idesc, 1u);
                    }
                }
                for (int sub = 0; sub < per; ++sub) {
                    const uint64_t a_hi = smem_desc(base + sub * a_bytes), b_hi = smem_desc(base + per * a_bytes + sub * b_bytes);
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk) {
                        const uint64_t adv = (uint64_t)(kk * 2);
                        mma_f16(acc_main, a_hi + adv, b_hi + adv, idesc, 1u);
                    }
                }
                if (window_end) {
                    // chunks [first, last] of the window belong to this CTA: the 16-wide slices that hold them
                    const int first_chunk = (sb_abs >> 3) == (sb_first >> 3) ? (sb_first & 7) : 0, last_chunk = sb_abs & 7;
                    const uint32_t mbase = smem_u32(min_a), bbase = smem_u32(min_b);
                    const uint64_t ma_hi = smem_desc(mbase), ma_lo = smem_desc(mbase + kTileBytes);
                    const uint64_t mb_hi = smem_desc(bbase), mb_lo = smem_desc(bbase + bn * 128);
                    for (int kk = first_chunk >> 1; kk <= last_chunk >> 1; ++kk) {
                        const uint64_t adv = (uint64_t)(kk * 2);
                        mma_f16(acc_min, ma_hi + adv, mb_hi + adv, idesc, min_started ? 1u : 0u);
                        mma_f16(acc_min, ma_hi + adv, mb_lo + adv, idesc, 1u);
                        mma_f16(acc_min, ma_lo + adv, mb_hi + adv, idesc, 1u);
                        min_started = true;
                    }
                    mma_commit(&min_free);  // the minimum tiles may be rewritten once these have finished
                }
                // one commit: the stage's sum is complete, and its slot (and the minimum tiles, if read) are free
                mma_commit(st == n_stages - 1 ? &done_bar : &stage_done[slot]);
                if (st == n_stages - 1) mma_commit(&stage_done[slot]);
            }
            __syncwarp();
        }
    } else {
        // ------------------------------------------------------------ copy warp (lane 0): the prepared X tiles
        if (lane == 0) {
            // the activation images were written by the kernel before this one
            asm volatile("griddepcontrol.wait;" ::: "memory");
            const uint32_t slice_bytes = (uint32_t)b_bytes, bytes = slice_bytes * (uint32_t)per;
            const int k_total = p.cols / BK, windows = (nb + 7) >> 3;
            const uint8_t* src = p.xs + ((size_t)nt * k_total + kg_first) * slice_bytes;
            int w_issue = 0;
            const int w_last = ((sb_first + n_sb - 1) >> 3) - (sb_first >> 3);  // windows of eight superblocks this CTA touches, counted from its first
            for (int st = 0; st < n_stages; ++st) {
                const int slot = st % stages;
                if (st >= stages && !mbar_wait(&stage_done[slot], ((st / stages) - 1) & 1, p.wait_ns)) { atomicExch(p.error_flag, 16); break; }
                mbar_expect_tx(&full_bar[slot], bytes);
                bulk_g2s(smem + (size_t)slot * stage_bytes + per * a_bytes, src + (size_t)st * bytes, bytes, &full_bar[slot]);
                if (kQ4 && w_issue <= w_last) {
                    // The group sums of window `w_issue`: the CTA's first window at once; a later window `stages` stages into
                    // it (by then the slot wait above has seen the previous window's last stage finish, and with it the products
                    // that read this tile), or at the window's last stage when the window is shorter than that.
                    const int win = (sb_first >> 3) + w_issue;
                    const int win_first_sb = w_issue == 0 ? sb_first : win << 3;
                    const int win_last_sb = min(sb_first + n_sb - 1, (win << 3) + 7);
                    const int st_begin = ((win_first_sb - sb_first) * 4) / per, st_end = ((win_last_sb - sb_first) * 4 + 3) / per;
                    const int st_issue = w_issue == 0 ? 0 : min(st_begin + stages, st_end);
                    if (st == st_issue) {
                        if (w_issue > 0 && !mbar_wait(&min_free, (w_issue - 1) & 1, p.wait_ns)) { atomicExch(p.error_flag, 16); break; }
                        mbar_expect_tx(&min_full, slice_bytes);
                        bulk_g2s(min_b, p.xg + ((size_t)nt * windows + win) * slice_bytes, slice_bytes, &min_full);
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
    int bn, n_tiles, sb_per_split, splits, stages, slices;
    size_t smem, records_bytes, xs_bytes, xg_bytes, partial_bytes;
};
KqCut kq_cut(int type, int sm_count, int64_t rows, int64_t cols, int tokens, bool int8) {
    KqCut c;
    c.bn = tokens <= 16 ? 16 : (tokens <= 32 ? 32 : (tokens <= 64 ? 64 : 128));
    c.n_tiles = (tokens + c.bn - 1) / c.bn;
    const int nb = (int)(cols >> 8), a_tiles = type == RQ_Q4_K ? 1 : 2;
    // A stage costs a fixed few hundred cycles of hand-offs (fill, one commit, drain): narrow token tiles, whose products are
    // short, take two 64-wide slices per stage
    c.slices = c.bn <= 32 ? 2 : 1;
    const size_t stage = (size_t)c.slices * ((size_t)a_tiles * kTileBytes + 2 * (size_t)c.bn * 128);
    const size_t fixed = type == RQ_Q4_K ? 2 * (size_t)kTileBytes + 2 * (size_t)c.bn * 128 : 0;
    c.stages = (int)((220 * 1024 - fixed) / stage);
    const int acc_room = (512 - (type == RQ_Q4_K ? c.bn : 0)) / c.bn;  // an accumulator per stage
    if (c.stages > acc_room) c.stages = acc_room;
    if (c.stages > kMaxStages) c.stages = kMaxStages;
    c.smem = (size_t)c.stages * stage + fixed + 1024;
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
    c.records_bytes = int8 ? (((size_t)tokens * nb * RQ_ACT_RECORD_INT8 + 1023) & ~(size_t)1023) : 0;
    c.xs_bytes = (size_t)c.n_tiles * (size_t)(cols / BK) * 2 * c.bn * 128;
    c.xg_bytes = type == RQ_Q4_K ? (size_t)c.n_tiles * (size_t)((nb + 7) / 8) * 2 * c.bn * 128 : 0;
    c.partial_bytes = c.splits > 1 ? (size_t)c.splits * tokens * rows * 4 : 0;
    return c;
}

}  // namespace

size_t rq_matmul_kq_scratch_bytes(const rq_ctx* ctx, int type, int64_t rows, int64_t cols, int tokens) {
    const KqCut c = kq_cut(type, ctx->sm_count, rows, cols, tokens, true);
    return c.records_bytes + c.xs_bytes + c.xg_bytes + c.partial_bytes;
}

// RQ_ERR_UNSUPPORTED (no error text) = not a K-quant weight. act_mode FLOAT or INT8 (step 32 / 256).
int rq_launch_matmul_kq(rq_ctx* ctx, const rq_weight* w, const float* x, int64_t sk, int64_t st, int tokens, float* y, int64_t yn, int64_t yt, int act_mode,
                        int step, cudaStream_t s) {
    if ((w->type != RQ_Q4_K && w->type != RQ_Q6_K) || w->cols % 256) return RQ_ERR_UNSUPPORTED;
    const bool int8 = act_mode != RQ_ACT_FLOAT;
    const KqCut cut = kq_cut(w->type, ctx->sm_count, w->rows, w->cols, tokens, int8);
    int rc = rq_ensure_act_scratch(ctx, cut.records_bytes + cut.xs_bytes + cut.xg_bytes + cut.partial_bytes, s);
    if (rc) return rc;
    ctx->act_cols = 0;  // whatever int8 records the scratch held for INT8_CACHED calls are gone
    uint8_t* records = ctx->act_scratch;
    uint8_t* xs = records + cut.records_bytes;
    uint8_t* xg = cut.xg_bytes ? xs + cut.xs_bytes : nullptr;
    float* partial = cut.splits > 1 ? (float*)(xs + cut.xs_bytes + cut.xg_bytes) : nullptr;
    if (int8) {
        rc = rq_launch_act_quant(x, sk, st, w->cols, tokens, step, records, nullptr, s);
        if (rc) return rc;
    }
    if (xg) RQ_CUDA(cudaMemsetAsync(xg, 0, cut.xg_bytes, s));  // groups past the last superblock of a window count as zeros
    {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(w->cols / BK), (unsigned)cut.n_tiles);
        cfg.blockDim = dim3(128);
        cfg.stream = s;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = int8 ? 1 : 0;  // after a memset node the kernel is launched the plain way
        RQ_CUDA(cudaLaunchKernelEx(&cfg, rq_kq_prep_kernel, x, sk, st, (const uint8_t*)(int8 ? records : nullptr), (int)w->cols, tokens, cut.bn, xs, xg));
    }
    KqParams p;
    p.main = w->main; p.scale = w->scale; p.rows = w->rows; p.cols = (int)w->cols;
    p.xs = xs; p.xg = xg; p.bn = cut.bn; p.tokens = tokens; p.y = y; p.yn = yn; p.yt = yt;
    p.sb_per_split = cut.sb_per_split; p.partial = partial; p.stages = cut.stages; p.slices_per_stage = cut.slices;
    p.error_flag = ctx->error_flag; p.wait_ns = ctx->wait_limit_ns;
    const int grid_m = (int)((w->rows + BM - 1) / BM);
    rc = w->type == RQ_Q4_K ? launch_kq<RQ_Q4_K>(p, grid_m, cut.n_tiles, cut.splits, cut.smem, s) : launch_kq<RQ_Q6_K>(p, grid_m, cut.n_tiles, cut.splits, cut.smem, s);
    if (rc || cut.splits == 1) return rc;
    return rq_launch_sum_splits(partial, cut.splits, w->rows, tokens, y, yn, yt, s);
}
