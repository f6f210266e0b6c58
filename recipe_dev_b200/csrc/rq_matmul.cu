// Batched quantised matmul (prefill / multi-sequence decode) on the 5th-generation tensor cores.
//
// Y[t][n] = sum_k W[n][k] * X[t][k], W stored as GGUF blocks, fp32 activations kept as they are
// (the FLOAT handling of a stored sum).
//
// Operands reach the tensor core as fp16 PAIRS hi + lo with hi = fp16(v), lo = fp16(v - hi):
// together 22 mantissa bits, so nothing of the fp32 inputs that matters at the 1e-3 bar is lost.
// Three products are issued per 16-wide slice, A_hi B_hi + A_hi B_lo + A_lo B_hi (the dropped
// A_lo B_lo term is 2^-22 relative).
//
//   * a small kernel splits X once into hi and lo tiles, already in the 128-byte-swizzled K-major
//     image the tensor core reads, so the main kernel fetches a tile with one bulk copy;
//   * a CTA owns 128 weight rows x BN tokens (BN = 32, 64 or 128). Eight staging warps dequantise
//     128 x 64 slices of W (bit-exact values, as rq_dequant gives them; the next slice's bytes are
//     fetched while this one is converted) into swizzled hi / lo tiles in shared memory;
//   * one thread issues tcgen05.mma (kind::f16, M = 128, N = BN, K = 16). The tensor core adds
//     into its fp32 accumulator by TRUNCATION, a bias that grows with the length of the chain
//     (measured: 1.2e-5 relative at K = 4096). So the large term A_hi B_hi is accumulated in
//     tensor memory only over one 64-wide slice (four instructions), into one of two
//     accumulators in turn, and eight drain warps add each finished slice into fp32 registers
//     with round-to-nearest adds while the tensor core works on the next. The two cross terms,
//     2^-11 of the result, stay in a third accumulator for the whole K.
// Three stages of 64 KB keep dequantisation ahead of the tensor core.
//
// Every wait is bounded in time; a wait that runs out records a code in the context's error word,
// the thread stops waiting and the CTA still frees its tensor memory before it exits.
#include "rq_internal.cuh"
#include "rq_mma.cuh"

using namespace rqmma;

namespace {

constexpr int kStages = 3;
constexpr int kStageWarps = 8, kDrainWarps = 8;
constexpr int kStagers = kStageWarps * 32;
constexpr int kMmaWarp = kStageWarps + kDrainWarps, kCopyWarp = kMmaWarp + 1;
constexpr int kThreadsMM = (kCopyWarp + 1) * 32;
constexpr int kTileBytes = BM * BK * 2;            // one fp16 tile of 128 rows: 16 KB
constexpr int kStageBytes = 4 * kTileBytes;        // A_hi | A_lo | B_hi | B_lo (B tiles of BN rows, at most 128)

struct MatmulParams {
    const uint8_t* main;
    const uint16_t* scale;
    int64_t rows;
    int cols;
    const uint8_t* xs;  // the split activations: [token tile][k slice][hi | lo][bn rows x 128 bytes, swizzled]
    int bn;             // tokens per tile
    int tokens;
    float* y; int64_t yn, yt;
    int ks_per_split;   // 64-wide slices per CTA along K (gridDim.z CTAs share a tile's K)
    float* partial;     // gridDim.z > 1: [split][token][row] sums, added in split order by rq_sum_splits_kernel
    int* error_flag;
    unsigned long long wait_ns;  // bounded waits give up after this long
};

// Weights are scaled by 2^8 before the split and the accumulator by 2^-8 after: a weight of 0.02
// leaves a residual near 1e-5, which fp16 could only hold as a subnormal with a few bits; scaled, the
// residual keeps its eleven. (Weights of magnitude 255 and more would overflow fp16; GGUF model
// weights are orders of magnitude below that.)
constexpr float kWeightScale = 256.0f, kWeightUnscale = 1.0f / 256.0f;

// Eight fp32 values (times `scale`) as one 16-byte chunk of fp16 hi and one of fp16 lo.
__device__ __forceinline__ void split8(const float* v, float scale, uint4& hi, uint4& lo) {
    uint32_t hw[4], lw[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float a = v[2 * j] * scale, b = v[2 * j + 1] * scale;
        const __half2 h2 = __floats2half2_rn(a, b);
        const float2 back = __half22float2(h2);
        const __half2 l2 = __floats2half2_rn(a - back.x, b - back.y);
        hw[j] = *(const uint32_t*)&h2;
        lw[j] = *(const uint32_t*)&l2;
    }
    hi = make_uint4(hw[0], hw[1], hw[2], hw[3]);
    lo = make_uint4(lw[0], lw[1], lw[2], lw[3]);
}

// ------------------------------------------------------------------------------------------
// The raw bytes behind 32 consecutive values of one row (`half` 0 or 1 of a 64-wide slice at k0),
// fetched one slice ahead, and their dequantisation: the same bits rq_dequant gives.
// ------------------------------------------------------------------------------------------
template <int TYPE> struct RawHalf;
template <> struct RawHalf<RQ_Q4_K> {
    uint4 hdr, q0, q1;
    __device__ __forceinline__ void load(const MatmulParams& p, int64_t row, int k0, int) {
        const uint8_t* blk = p.main + (row * (p.cols >> 8) + (k0 >> 8)) * 144;
        const int pr = (k0 & 255) >> 6;
        hdr = __ldg((const uint4*)blk);
        q0 = __ldg((const uint4*)(blk + 16 + 32 * pr));
        q1 = __ldg((const uint4*)(blk + 32 + 32 * pr));
    }
    __device__ __forceinline__ void decode(int k0, int half, float* v) const {
        const int pr = (k0 & 255) >> 6;
        int sc, mn;
        rq_q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * pr + half, sc, mn);
        const float d = rq_h2f((uint16_t)(hdr.x & 0xffff)), dmin = rq_h2f((uint16_t)(hdr.x >> 16));
        const float step = __fmul_rn(d, (float)sc), base = __fmul_rn(dmin, (float)mn);
        const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        const int shift = 4 * half;  // sub-block 2 pr in the low nibbles, 2 pr + 1 in the high
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t nib = (w[j] >> shift) & 0x0F0F0F0Fu;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                // 0x4B0000nn is 2^23 + nn: the nibble as a float without the conversion unit
                const float q = __uint_as_float(__byte_perm(nib, 0x4B000000u, 0x7650 + i)) - 8388608.0f;
                v[4 * j + i] = __fsub_rn(__fmul_rn(step, q), base);
            }
        }
    }
};
template <> struct RawHalf<RQ_Q6_K> {
    uint4 ql[2], qh[2];
    uint32_t scales;  // two int8 scales
    uint32_t d16;
    __device__ __forceinline__ void load(const MatmulParams& p, int64_t row, int k0, int half) {
        const int64_t nb = p.cols >> 8;
        const int j64 = (k0 & 255) >> 6, ch = j64 >> 1, sel = j64 & 1, g = 2 * sel + half;
        const uint8_t* body = p.main + (row * nb + (k0 >> 8)) * 208;
        ql[0] = __ldg((const uint4*)(body + 64 * ch + 32 * half));
        ql[1] = __ldg((const uint4*)(body + 64 * ch + 32 * half + 16));
        qh[0] = __ldg((const uint4*)(body + 128 + 32 * ch));
        qh[1] = __ldg((const uint4*)(body + 128 + 32 * ch + 16));
        scales = __ldg((const uint16_t*)(body + 192 + 8 * ch + 2 * g));
        d16 = __ldg(p.scale + row * nb + (k0 >> 8));
    }
    __device__ __forceinline__ void decode(int k0, int half, float* v) const {
        const int j64 = (k0 & 255) >> 6, sel = j64 & 1, g = 2 * sel + half;  // group g of its chunk: ql line 32 * half, nibble sel
        const float d = rq_h2f((uint16_t)d16);
#pragma unroll
        for (int q4 = 0; q4 < 2; ++q4) {  // sixteen values at a time
            const uint32_t lw[4] = {ql[q4].x, ql[q4].y, ql[q4].z, ql[q4].w}, hw[4] = {qh[q4].x, qh[q4].y, qh[q4].z, qh[q4].w};
            const int scale = (int)(int8_t)(scales >> (8 * q4));
            const float scaled = __fmul_rn(d, (float)scale);
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int lo = (lw[j] >> (8 * i + 4 * sel)) & 15, hi = (hw[j] >> (8 * i + 2 * g)) & 3;
                    v[16 * q4 + 4 * j + i] = __fmul_rn(scaled, (float)((lo | (hi << 4)) - 32));
                }
        }
    }
};
template <> struct RawHalf<RQ_Q8_0> {
    uint4 a, c;
    uint32_t d16;
    __device__ __forceinline__ void load(const MatmulParams& p, int64_t row, int k0, int half) {
        const int64_t chunk = (k0 + 32 * half) >> 4;  // two 16-byte chunks of the row
        const bool perm = rq_plane_permuted(RQ_Q8_0, p.cols);
        a = __ldg((const uint4*)(p.main + row * p.cols + 16 * (perm ? rq_plane_chunk(RQ_Q8_0, chunk) : chunk)));
        c = __ldg((const uint4*)(p.main + row * p.cols + 16 * (perm ? rq_plane_chunk(RQ_Q8_0, chunk + 1) : chunk + 1)));
        d16 = __ldg(p.scale + row * (p.cols >> 5) + (k0 >> 5) + half);
    }
    __device__ __forceinline__ void decode(int, int, float* v) const {
        const float d = rq_h2f((uint16_t)d16);
        const uint32_t w[8] = {a.x, a.y, a.z, a.w, c.x, c.y, c.z, c.w};
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) v[4 * j + i] = __fmul_rn((float)(int8_t)(w[j] >> (8 * i)), d);
    }
};
template <> struct RawHalf<RQ_Q4_0> {
    uint4 a;
    uint32_t d16;
    __device__ __forceinline__ void load(const MatmulParams& p, int64_t row, int k0, int half) {
        const int64_t chunk = (k0 >> 5) + half;  // one 16-byte chunk per block of 32 values
        a = __ldg((const uint4*)(p.main + row * (p.cols >> 1) + 16 * (rq_plane_permuted(RQ_Q4_0, p.cols) ? rq_plane_chunk(RQ_Q4_0, chunk) : chunk)));
        d16 = __ldg(p.scale + row * (p.cols >> 5) + (k0 >> 5) + half);
    }
    __device__ __forceinline__ void decode(int, int, float* v) const {
        const float d = rq_h2f((uint16_t)d16);
        const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t byte = (w[j] >> (8 * i)) & 0xff;
                v[4 * j + i] = __fmul_rn((float)((int)(byte & 15) - 8), d);
                v[16 + 4 * j + i] = __fmul_rn((float)((int)(byte >> 4) - 8), d);
            }
    }
};

// ------------------------------------------------------------------------------------------
// X -> fp16 hi / lo tiles in the tensor core's swizzled image. grid (k slices, token tiles),
// one thread per token row of the tile; rows past the last token are zero.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) rq_split_x_kernel(const float* __restrict__ x, int64_t sk, int64_t st, int tokens, int bn, uint8_t* __restrict__ xs) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int ks = blockIdx.x, nt = blockIdx.y, r = threadIdx.x;
    if (r >= bn) return;
    const int token = nt * bn + r;
    uint8_t* hi = xs + ((size_t)nt * gridDim.x + ks) * 2 * (size_t)bn * 128;
    uint8_t* lo = hi + (size_t)bn * 128;
    const bool vec = sk == 1 && (st & 3) == 0 && ((uintptr_t)x & 15) == 0;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        float v[8];
        if (token < tokens) {
            const float* src = x + (int64_t)token * st + (int64_t)(ks * BK + 8 * c) * sk;
            if (vec) {
                *(float4*)v = __ldg((const float4*)src);
                *(float4*)(v + 4) = __ldg((const float4*)src + 1);
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = __ldg(src + j * sk);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = 0.f;
        }
        uint4 h, l;
        split8(v, 1.0f, h, l);
        *(uint4*)(hi + swizzled(r, c)) = h;
        *(uint4*)(lo + swizzled(r, c)) = l;
    }
}

// y[row][token] = the splits' sums added in split order (the same bits on every run). Grid row = token; a thread takes four
// adjacent rows at a time where the planes allow 16-byte accesses (the partial sums are [split][token][row]).
__global__ void __launch_bounds__(256) rq_sum_splits_kernel(const float* __restrict__ partial, int splits, int64_t rows, int tokens, float* __restrict__ y, int64_t yn, int64_t yt) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int64_t total = rows * tokens;
    const bool vec = yn == 1 && (rows & 3) == 0 && (yt & 3) == 0 && (((uintptr_t)partial | (uintptr_t)y) & 15) == 0;
    for (int token = blockIdx.y; token < tokens; token += gridDim.y) {
        const float* src = partial + (int64_t)token * rows;
        if (vec) {
            float4* dst = (float4*)(y + (int64_t)token * yt);
            for (int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; q < (rows >> 2); q += (int64_t)gridDim.x * blockDim.x) {
                float4 sum = __ldcs((const float4*)src + q);
                for (int z = 1; z < splits; ++z) {
                    const float4 v = __ldcs((const float4*)(src + (size_t)z * total) + q);
                    sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
                }
                dst[q] = sum;
            }
        } else {
            for (int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; row < rows; row += (int64_t)gridDim.x * blockDim.x) {
                float sum = src[row];
                for (int z = 1; z < splits; ++z) sum += src[(size_t)z * total + row];
                y[row * yn + (int64_t)token * yt] = sum;
            }
        }
    }
}

template <int TYPE>
__global__ void __launch_bounds__(kThreadsMM, 1) rq_matmul_kernel(const __grid_constant__ MatmulParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);  // swizzled tiles want 1024-byte alignment
    __shared__ __align__(8) uint64_t full_bar[kStages], empty_bar[kStages], acc_full[2], acc_empty[2], done_bar;
    __shared__ uint32_t tmem_base_slot;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t m0 = (int64_t)blockIdx.x * BM;
    const int nt = blockIdx.y, n0 = nt * p.bn;
    const int k_first = blockIdx.z * p.ks_per_split;  // this CTA's slices of K
    const int k_steps = min(p.ks_per_split, p.cols / BK - k_first);
    const int k_total = p.cols / BK;
    const int bn = p.bn;
    // tensor memory: two accumulators for the hi x hi term, one for the cross terms: 3 bn columns, allocated as a power of two
    const uint32_t tmem_cols = bn == 128 ? 512u : (bn == 64 ? 256u : 128u);

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], kStagers + 1); mbar_init(&empty_bar[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], kDrainWarps); }
        mbar_init(&done_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;

    if (warp < kStageWarps) {
        // ------------------------------------------------------------ staging warps: W -> hi / lo tiles
        const int r = tid & 127, half = tid >> 7;  // a row of the tile, and which 32 of the slice's 64 values
        const int64_t row = m0 + r < p.rows ? m0 + r : p.rows - 1;  // rows past the end are computed and dropped
        bool dead = false;
        RawHalf<TYPE> cur, nxt;
        cur.load(p, row, k_first * BK, half);
        for (int ks = 0; ks < k_steps; ++ks) {
            const int slot = ks % kStages;
            if (ks + 1 < k_steps) nxt.load(p, row, (k_first + ks + 1) * BK, half);
            float v[32];
            cur.decode((k_first + ks) * BK, half, v);
            if (ks >= kStages && !dead && !mbar_wait(&empty_bar[slot], ((ks / kStages) - 1) & 1, p.wait_ns)) { atomicExch(p.error_flag, 11); dead = true; }
            uint8_t* a_hi = smem + (size_t)slot * kStageBytes;
            uint8_t* a_lo = a_hi + kTileBytes;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint4 h, l;
                split8(v + 8 * c, kWeightScale, h, l);
                const int off = swizzled(r, 4 * half + c);
                *(uint4*)(a_hi + off) = h;
                *(uint4*)(a_lo + off) = l;
            }
            // the tensor core reads shared memory through the async proxy
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(&full_bar[slot]);
            cur = nxt;
        }
    } else if (warp < kMmaWarp) {
        // ------------------------------------------------------------ drain warps: tensor memory -> fp32 registers -> Y
        // warp w may read accumulator rows 32 (w % 4) ..; the eight warps split the columns in two
        const int dw = warp - kStageWarps, quarter = warp & 3, chalf = dw >> 2;
        const int cols_here = bn >> 1, col0 = chalf * cols_here;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        float acc[64];
#pragma unroll
        for (int i = 0; i < 64; ++i) acc[i] = 0.f;
        bool dead = false;
        for (int ks = 0; ks < k_steps; ++ks) {
            const int b = ks & 1;
            if (!dead && !mbar_wait(&acc_full[b], (ks >> 1) & 1, p.wait_ns)) { atomicExch(p.error_flag, 14); dead = true; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                if (16 * c < cols_here) {
                    uint32_t t[16];
                    tmem_ld16(tmem_base + lane_base + (uint32_t)(b * bn + col0 + 16 * c), t);
#pragma unroll
                    for (int j = 0; j < 16; ++j) acc[16 * c + j] += __uint_as_float(t[j]);
                }
            }
            // this warp has read the accumulator: the tensor core may overwrite it
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[b]);
        }
        if (!dead && !mbar_wait(&done_bar, 0, p.wait_ns)) { atomicExch(p.error_flag, 12); dead = true; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int64_t out_row = m0 + quarter * 32 + lane;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            if (16 * c < cols_here) {
                uint32_t t[16];
                tmem_ld16(tmem_base + lane_base + (uint32_t)(2 * bn + col0 + 16 * c), t);  // the cross terms
                if (out_row < p.rows && !dead) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int token = n0 + col0 + 16 * c + j;
                        const float out = (acc[16 * c + j] + __uint_as_float(t[j])) * kWeightUnscale;
                        if (token < p.tokens) {
                            if (gridDim.z == 1) p.y[out_row * p.yn + (int64_t)token * p.yt] = out;
                            else p.partial[((size_t)blockIdx.z * p.tokens + token) * p.rows + out_row] = out;
                        }
                    }
                }
            }
        }
    } else if (warp == kMmaWarp) {
        // ------------------------------------------------------------ MMA warp (lane 0 issues)
        bool dead = false;
        const uint32_t idesc = instr_desc(bn);
        for (int ks = 0; ks < k_steps; ++ks) {
            const int slot = ks % kStages, b = ks & 1;
            if (!dead && !mbar_wait(&full_bar[slot], (ks / kStages) & 1, p.wait_ns)) { atomicExch(p.error_flag, 13); dead = true; }
            if (ks >= 2 && !dead && !mbar_wait(&acc_empty[b], ((ks >> 1) - 1) & 1, p.wait_ns)) { atomicExch(p.error_flag, 15); dead = true; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (lane == 0 && !dead) {
                const uint32_t base = smem_u32(smem + (size_t)slot * kStageBytes);
                const uint64_t a_hi = smem_desc(base), a_lo = smem_desc(base + kTileBytes);
                const uint64_t b_hi = smem_desc(base + 2 * kTileBytes), b_lo = smem_desc(base + 2 * kTileBytes + bn * 128);
                const uint32_t acc_main = tmem_base + (uint32_t)(b * bn), acc_cross = tmem_base + (uint32_t)(2 * bn);
#pragma unroll
                for (int kk = 0; kk < BK / 16; ++kk) {
                    const uint64_t adv = (uint64_t)(kk * 2);  // 32 bytes along K, in 16-byte units of the start address
                    mma_f16(acc_main, a_hi + adv, b_hi + adv, idesc, kk ? 1u : 0u);       // a fresh sum for every slice
                    mma_f16(acc_cross, a_hi + adv, b_lo + adv, idesc, (ks | kk) ? 1u : 0u);
                    mma_f16(acc_cross, a_lo + adv, b_hi + adv, idesc, 1u);
                }
                mma_commit(&empty_bar[slot]);  // the stage is free once these have read it
                mma_commit(&acc_full[b]);      // and the slice's sum is complete
                if (ks == k_steps - 1) mma_commit(&done_bar);
            }
            __syncwarp();
        }
    } else {
        // ------------------------------------------------------------ copy warp (lane 0): the split X tiles
        if (lane == 0) {
            // the activation tiles were written by the kernel before this one
            asm volatile("griddepcontrol.wait;" ::: "memory");
            const uint32_t bytes = 2u * (uint32_t)bn * 128u;
            const uint8_t* src = p.xs + ((size_t)nt * k_total + k_first) * bytes;
            for (int ks = 0; ks < k_steps; ++ks) {
                const int slot = ks % kStages;
                if (ks >= kStages && !mbar_wait(&empty_bar[slot], ((ks / kStages) - 1) & 1, p.wait_ns)) { atomicExch(p.error_flag, 16); break; }
                mbar_expect_tx(&full_bar[slot], bytes);
                bulk_g2s(smem + (size_t)slot * kStageBytes + 2 * kTileBytes, src + (size_t)ks * bytes, bytes, &full_bar[slot]);
            }
        }
    }
    // free the tensor memory: everyone is past its use
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == kMmaWarp) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
}

template <int TYPE>
int launch_mm(const MatmulParams& p, cudaStream_t s) {
    auto kernel = rq_matmul_kernel<TYPE>;
    const size_t smem = (size_t)kStages * kStageBytes + 1024;
    static bool configured[64] = {};
    int dev = 0;
    RQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        RQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((p.rows + BM - 1) / BM), (unsigned)((p.tokens + p.bn - 1) / p.bn), (unsigned)((p.cols / BK + p.ks_per_split - 1) / p.ks_per_split));
    cfg.blockDim = dim3(kThreadsMM);
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

}  // namespace

// How a call is cut: tokens per tile, K slices per CTA, CTAs along K, and the scratch it takes.
struct MatmulCut { int bn, n_tiles, k_steps, ks_per_split, splits; size_t xs_bytes, partial_bytes; };
static MatmulCut matmul_cut(int sm_count, int64_t rows, int64_t cols, int tokens) {
    MatmulCut c;
    c.bn = tokens <= 32 ? 32 : (tokens <= 64 ? 64 : 128);
    c.n_tiles = (tokens + c.bn - 1) / c.bn; c.k_steps = (int)(cols / BK);
    c.xs_bytes = (size_t)c.n_tiles * c.k_steps * 2 * c.bn * 128;
    // Few tiles and a long K: several CTAs share a tile's K (at least sixteen slices each) so that the whole GPU
    // dequantises, and a second kernel adds their sums.
    const int64_t tiles = ((rows + BM - 1) / BM) * c.n_tiles;
    int splits = 1;
    if (tiles < sm_count) {
        splits = (int)(sm_count / tiles);
        if (splits > c.k_steps / 16) splits = c.k_steps / 16;
        if (splits < 1) splits = 1;
    }
    c.ks_per_split = (c.k_steps + splits - 1) / splits;
    c.splits = (c.k_steps + c.ks_per_split - 1) / c.ks_per_split;
    c.partial_bytes = c.splits > 1 ? (size_t)c.splits * tokens * rows * 4 : 0;
    return c;
}
size_t rq_matmul_scratch_bytes(const rq_ctx* ctx, int64_t rows, int64_t cols, int tokens) {
    const MatmulCut c = matmul_cut(ctx->sm_count, rows, cols, tokens);
    size_t want = c.xs_bytes + c.partial_bytes;
    if (cols % 256 == 0) {
        // the K-quant kernel's images (int8 records included), for either K-quant format
        const size_t a = rq_matmul_kq_scratch_bytes(ctx, RQ_Q4_K, rows, cols, tokens), b = rq_matmul_kq_scratch_bytes(ctx, RQ_Q6_K, rows, cols, tokens);
        if (a > want) want = a;
        if (b > want) want = b;
    }
    return want;
}

int rq_launch_matmul(rq_ctx* ctx, const rq_weight* w, const float* x, int64_t sk, int64_t st, int tokens, float* y, int64_t yn, int64_t yt, cudaStream_t s) {
    if (w->cols % BK) return RQ_ERR_UNSUPPORTED;
    MatmulParams p;
    p.main = w->main; p.scale = w->scale; p.rows = w->rows; p.cols = (int)w->cols;
    const MatmulCut cut = matmul_cut(ctx->sm_count, w->rows, w->cols, tokens);
    p.bn = cut.bn;
    p.tokens = tokens; p.y = y; p.yn = yn; p.yt = yt; p.error_flag = ctx->error_flag; p.wait_ns = ctx->wait_limit_ns;
    // the split activations live in the context's scratch (whatever int8 records it held are gone)
    const int n_tiles = cut.n_tiles, k_steps = cut.k_steps, splits = cut.splits;
    const size_t bytes = cut.xs_bytes, partial_bytes = cut.partial_bytes;
    p.ks_per_split = cut.ks_per_split;
    int rc = rq_ensure_act_scratch(ctx, bytes + partial_bytes, s);
    if (rc) return rc;
    ctx->act_cols = 0;
    p.xs = ctx->act_scratch;
    p.partial = splits > 1 ? (float*)(ctx->act_scratch + bytes) : nullptr;
    {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)k_steps, (unsigned)n_tiles);
        cfg.blockDim = dim3(128);
        cfg.stream = s;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        RQ_CUDA(cudaLaunchKernelEx(&cfg, rq_split_x_kernel, x, sk, st, tokens, p.bn, ctx->act_scratch));
    }
    switch (w->type) {
        case RQ_Q4_K: rc = launch_mm<RQ_Q4_K>(p, s); break;
        case RQ_Q6_K: rc = launch_mm<RQ_Q6_K>(p, s); break;
        case RQ_Q8_0: rc = launch_mm<RQ_Q8_0>(p, s); break;
        case RQ_Q4_0: rc = launch_mm<RQ_Q4_0>(p, s); break;
        default: return RQ_ERR_UNSUPPORTED;
    }
    if (rc || splits == 1) return rc;
    return rq_launch_sum_splits(p.partial, splits, w->rows, tokens, y, yn, yt, s);
}

int rq_launch_sum_splits(const float* partial, int splits, int64_t rows, int tokens, float* y, int64_t yn, int64_t yt, cudaStream_t s) {
    cudaLaunchConfig_t cfg = {};
    const int64_t per_token = (rows / 4 + 255) / 256;  // CTAs that cover a token's rows four at a time
    cfg.gridDim = dim3((unsigned)(per_token < 1 ? 1 : (per_token > 64 ? 64 : per_token)), (unsigned)(tokens < 65535 ? tokens : 65535));
    cfg.blockDim = dim3(256);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    RQ_CUDA(cudaLaunchKernelEx(&cfg, rq_sum_splits_kernel, partial, splits, rows, tokens, y, yn, yt));
    return RQ_OK;
}
