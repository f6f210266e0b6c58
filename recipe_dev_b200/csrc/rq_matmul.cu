// Batched quantised matmul (prefill / multi-sequence decode) on the 5th-generation tensor cores.
//
// Y[t][n] = sum_k W[n][k] * X[t][k], W stored as GGUF blocks, fp32 activations kept as they are
// (the FLOAT handling of a stored sum). A CTA owns a tile of 128 weight rows x 128 tokens:
//   * four staging warps dequantise a 128 x 64 slice of W (bit-exact values, as rq_dequant gives
//     them) and convert it, and the matching 128 x 64 slice of X, to fp16 PAIRS hi + lo with
//     hi = fp16(v), lo = fp16(v - hi): together 22 mantissa bits, so nothing of the fp32 inputs that
//     matters at the 1e-3 bar is lost. The four tiles go to shared memory in the 128-byte-swizzled
//     K-major layout the tensor core reads;
//   * one warp issues tcgen05.mma (kind::f16, M = 128, N = 128, K = 16) three times per 16-wide
//     slice: A_hi B_hi + A_hi B_lo + A_lo B_hi, accumulating in fp32 in TMEM (the dropped
//     A_lo B_lo term is 2^-22 relative); tcgen05.commit releases the stage and, at the end, signals
//     the epilogue;
//   * the staging warps read the 128 x 128 fp32 accumulator back with tcgen05.ld and store Y.
// Three stages of 64 KB keep dequantisation ahead of the tensor core.
//
// Every wait is bounded in time; a wait that runs out records a code in the context's error word,
// the thread stops waiting and the CTA still frees its TMEM before it exits.
#include "rq_internal.cuh"

namespace {

constexpr int BM = 128, BN = 128, BK = 64, kStages = 3;
constexpr int kStagers = 128, kThreadsMM = 160;
constexpr int kTileBytes = BM * BK * 2;            // one fp16 tile: 16 KB
constexpr int kStageBytes = 4 * kTileBytes;        // A_hi | A_lo | B_hi | B_lo
constexpr unsigned long long kWaitLimitNs = 2000000000ull;

struct MatmulParams {
    const uint8_t* main;
    const uint16_t* scale;
    int64_t rows;
    int cols;
    const float* x; int64_t sk, st;
    int x_vec;  // token rows are contiguous and 16-byte aligned: 128-bit loads
    int tokens;
    float* y; int64_t yn, yt;
    int* error_flag;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long global_ns() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count)); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory"); }
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    while (!mbar_try_wait(bar, parity))
        if (global_ns() - t0 > kWaitLimitNs) return false;
    return true;
}

// K-major, 128-byte-swizzled operand tile of 128-byte rows: rows 128 bytes apart, groups of eight
// rows 1024 bytes apart (stride byte offset), descriptor version 1, layout type SWIZZLE_128B.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    uint64_t d = (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;                 // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;       // stride byte offset
    d |= (uint64_t)1 << 46;                 // descriptor version
    d |= (uint64_t)2 << 61;                 // SWIZZLE_128B
    return d;
}
// kind::f16, fp16 x fp16 -> fp32, both operands K-major, M = 128, N = BN
constexpr uint32_t kInstrDesc = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

__device__ __forceinline__ void mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(kInstrDesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// 64 consecutive values of one row, starting at k0 (a multiple of 64): the same bits rq_dequant gives.
template <int TYPE>
__device__ __forceinline__ void row_values(const MatmulParams& p, int64_t row, int k0, float* v) {
    if (TYPE == RQ_Q4_K) {
        const int b = k0 >> 8, pr = (k0 & 255) >> 6;
        const uint8_t* blk = p.main + (row * (p.cols >> 8) + b) * 144;
        const uint4 hdr = __ldg((const uint4*)blk);
        const uint4 q0 = __ldg((const uint4*)(blk + 16 + 32 * pr)), q1 = __ldg((const uint4*)(blk + 32 + 32 * pr));
        int sc_lo, mn_lo, sc_hi, mn_hi;
        rq_q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * pr, sc_lo, mn_lo);
        rq_q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * pr + 1, sc_hi, mn_hi);
        const float d = rq_h2f((uint16_t)(hdr.x & 0xffff)), dmin = rq_h2f((uint16_t)(hdr.x >> 16));
        const float step_lo = __fmul_rn(d, (float)sc_lo), base_lo = __fmul_rn(dmin, (float)mn_lo);
        const float step_hi = __fmul_rn(d, (float)sc_hi), base_hi = __fmul_rn(dmin, (float)mn_hi);
        const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t byte = (w[j] >> (8 * i)) & 0xff;
                v[4 * j + i] = __fsub_rn(__fmul_rn(step_lo, (float)(byte & 15)), base_lo);
                v[32 + 4 * j + i] = __fsub_rn(__fmul_rn(step_hi, (float)(byte >> 4)), base_hi);
            }
    } else if (TYPE == RQ_Q6_K) {
        const int b = k0 >> 8, j64 = (k0 & 255) >> 6, ch = j64 >> 1, sel = j64 & 1;  // groups 2 sel, 2 sel + 1 of chunk ch
        const int64_t nb = p.cols >> 8;
        const uint8_t* body = p.main + (row * nb + b) * 208;
        const float d = rq_h2f(__ldg(p.scale + row * nb + b));
#pragma unroll
        for (int half = 0; half < 2; ++half) {   // group g = 2 sel + half: ql line 32 * (g & 1) = 32 * half, nibble g / 2 = sel
            const int g = 2 * sel + half;
#pragma unroll
            for (int q4 = 0; q4 < 2; ++q4) {     // sixteen values at a time
                const uint4 ql = __ldg((const uint4*)(body + 64 * ch + 32 * half + 16 * q4));
                const uint4 qh = __ldg((const uint4*)(body + 128 + 32 * ch + 16 * q4));
                const uint32_t lw[4] = {ql.x, ql.y, ql.z, ql.w}, hw[4] = {qh.x, qh.y, qh.z, qh.w};
                const int scale = (int8_t)__ldg(body + 192 + 8 * ch + 2 * g + q4);
                const float scaled = __fmul_rn(d, (float)scale);
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int lo = (lw[j] >> (8 * i + 4 * sel)) & 15, hi = (hw[j] >> (8 * i + 2 * g)) & 3;
                        v[32 * half + 16 * q4 + 4 * j + i] = __fmul_rn(scaled, (float)((lo | (hi << 4)) - 32));
                    }
            }
        }
    } else if (TYPE == RQ_Q8_0) {
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
            const float d = rq_h2f(__ldg(p.scale + row * (p.cols >> 5) + (k0 >> 5) + blk));
            const uint4 a = __ldg((const uint4*)(p.main + row * p.cols + k0 + 32 * blk)), c = __ldg((const uint4*)(p.main + row * p.cols + k0 + 32 * blk + 16));
            const uint32_t w[8] = {a.x, a.y, a.z, a.w, c.x, c.y, c.z, c.w};
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) v[32 * blk + 4 * j + i] = __fmul_rn((float)(int8_t)(w[j] >> (8 * i)), d);
        }
    } else {
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
            const float d = rq_h2f(__ldg(p.scale + row * (p.cols >> 5) + (k0 >> 5) + blk));
            const uint4 a = __ldg((const uint4*)(p.main + row * (p.cols >> 1) + ((k0 >> 5) + blk) * 16));
            const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t byte = (w[j] >> (8 * i)) & 0xff;
                    v[32 * blk + 4 * j + i] = __fmul_rn((float)((int)(byte & 15) - 8), d);
                    v[32 * blk + 16 + 4 * j + i] = __fmul_rn((float)((int)(byte >> 4) - 8), d);
                }
        }
    }
}

// Weights are scaled by 2^8 before the split and the accumulator by 2^-8 after: a weight of 0.02
// leaves a residual near 1e-5, which fp16 could only hold as a subnormal with a few bits; scaled, the
// residual keeps its eleven. (Weights of magnitude 255 and more would overflow fp16; GGUF model
// weights are orders of magnitude below that.)
constexpr float kWeightScale = 256.0f, kWeightUnscale = 1.0f / 256.0f;

// Splits 64 fp32 values (times `scale`) into fp16 hi and lo and writes the row into the two swizzled tiles.
__device__ __forceinline__ void store_row_split(const float* v, float scale, uint8_t* tile_hi, uint8_t* tile_lo, int row) {
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        uint32_t hw[4], lw[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float a = v[8 * c + 2 * j] * scale, b = v[8 * c + 2 * j + 1] * scale;
            const __half ha = __float2half_rn(a), hb = __float2half_rn(b);
            const __half la = __float2half_rn(a - __half2float(ha)), lb = __float2half_rn(b - __half2float(hb));
            hw[j] = (uint32_t)__half_as_ushort(ha) | ((uint32_t)__half_as_ushort(hb) << 16);
            lw[j] = (uint32_t)__half_as_ushort(la) | ((uint32_t)__half_as_ushort(lb) << 16);
        }
        const int off = row * 128 + ((c ^ (row & 7)) << 4);  // Swizzle<3,4,3>: the 16-byte chunk index xor the row within its group of eight
        *(uint4*)(tile_hi + off) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
        *(uint4*)(tile_lo + off) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
    }
}

template <int TYPE>
__global__ void __launch_bounds__(kThreadsMM, 1) rq_matmul_kernel(const __grid_constant__ MatmulParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);  // swizzled tiles want 1024-byte alignment
    __shared__ __align__(8) uint64_t full_bar[kStages], empty_bar[kStages], done_bar;
    __shared__ uint32_t tmem_base_slot;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t m0 = (int64_t)blockIdx.x * BM;
    const int n0 = blockIdx.y * BN;
    const int k_steps = p.cols / BK;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], kStagers); mbar_init(&empty_bar[s], 1); }
        mbar_init(&done_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 4) {
        // 128 fp32 accumulator columns of tensor memory for this CTA
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"((uint32_t)BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;

    if (warp < 4) {
        // ------------------------------------------------------------ staging warps
        const int64_t row = m0 + tid < p.rows ? m0 + tid : p.rows - 1;  // rows past the end are computed and dropped
        const int token = n0 + tid;
        const bool live_token = token < p.tokens;
        const float* xt = p.x + (int64_t)(live_token ? token : 0) * p.st;
        bool dead = false;
        for (int ks = 0; ks < k_steps; ++ks) {
            const int slot = ks % kStages;
            if (ks >= kStages && !dead && !mbar_wait(&empty_bar[slot], ((ks / kStages) - 1) & 1)) { atomicExch(p.error_flag, 11); dead = true; }
            uint8_t* stage = smem + (size_t)slot * kStageBytes;
            float v[64];
            row_values<TYPE>(p, row, ks * BK, v);
            store_row_split(v, kWeightScale, stage, stage + kTileBytes, tid);
            if (live_token) {
                if (p.x_vec) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) *(float4*)(v + 4 * j) = __ldg((const float4*)(xt + ks * BK) + j);
                } else {
#pragma unroll
                    for (int j = 0; j < 64; ++j) v[j] = __ldg(xt + (int64_t)(ks * BK + j) * p.sk);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 64; ++j) v[j] = 0.0f;
            }
            store_row_split(v, 1.0f, stage + 2 * kTileBytes, stage + 3 * kTileBytes, tid);
            // the tensor core reads shared memory through the async proxy
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(&full_bar[slot]);
        }
        // ------------------------------------------------------------ epilogue
        if (!dead && !mbar_wait(&done_bar, 0)) { atomicExch(p.error_flag, 12); dead = true; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int64_t out_row = m0 + warp * 32 + lane;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
            uint32_t r[32];
            const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0;
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, "
                "%23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
                : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
                  "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
                  "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
                  "=r"(r[31])
                : "r"(taddr));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (out_row < p.rows && !dead) {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int t = n0 + c0 + j;
                    if (t < p.tokens) p.y[out_row * p.yn + (int64_t)t * p.yt] = __uint_as_float(r[j]) * kWeightUnscale;
                }
            }
        }
    } else {
        // ------------------------------------------------------------ MMA warp
        bool dead = false;
        for (int ks = 0; ks < k_steps; ++ks) {
            const int slot = ks % kStages;
            if (!dead && !mbar_wait(&full_bar[slot], (ks / kStages) & 1)) { atomicExch(p.error_flag, 13); dead = true; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (lane == 0 && !dead) {
                const uint32_t base = smem_u32(smem + (size_t)slot * kStageBytes);
                const uint64_t a_hi = smem_desc(base), a_lo = smem_desc(base + kTileBytes);
                const uint64_t b_hi = smem_desc(base + 2 * kTileBytes), b_lo = smem_desc(base + 3 * kTileBytes);
#pragma unroll
                for (int kk = 0; kk < BK / 16; ++kk) {
                    const uint64_t adv = (uint64_t)(kk * 2);  // 32 bytes along K, in 16-byte units of the start address
                    mma_f16(tmem_base, a_hi + adv, b_hi + adv, (ks | kk) ? 1u : 0u);
                    mma_f16(tmem_base, a_hi + adv, b_lo + adv, 1u);
                    mma_f16(tmem_base, a_lo + adv, b_hi + adv, 1u);
                }
                mma_commit(&empty_bar[slot]);          // the stage is free once these have read it
                if (ks == k_steps - 1) mma_commit(&done_bar);
            }
            __syncwarp();
        }
    }
    // free the tensor memory: everyone is past its use
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 4) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)BN) : "memory");
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
    dim3 grid((unsigned)((p.rows + BM - 1) / BM), (unsigned)((p.tokens + BN - 1) / BN));
    kernel<<<grid, kThreadsMM, smem, s>>>(p);
    RQ_CUDA(cudaGetLastError());
    return RQ_OK;
}

}  // namespace

int rq_launch_matmul(rq_ctx* ctx, const rq_weight* w, const float* x, int64_t sk, int64_t st, int tokens, float* y, int64_t yn, int64_t yt, cudaStream_t s) {
    if (w->cols % BK) return RQ_ERR_UNSUPPORTED;
    MatmulParams p;
    p.main = w->main; p.scale = w->scale; p.rows = w->rows; p.cols = (int)w->cols;
    p.x = x; p.sk = sk; p.st = st; p.tokens = tokens; p.y = y;
    p.x_vec = (sk == 1 && (st % 4 == 0 || tokens == 1) && ((uintptr_t)x % 16) == 0) ? 1 : 0; p.yn = yn; p.yt = yt; p.error_flag = ctx->error_flag;
    switch (w->type) {
        case RQ_Q4_K: return launch_mm<RQ_Q4_K>(p, s);
        case RQ_Q6_K: return launch_mm<RQ_Q6_K>(p, s);
        case RQ_Q8_0: return launch_mm<RQ_Q8_0>(p, s);
        case RQ_Q4_0: return launch_mm<RQ_Q4_0>(p, s);
        default: return RQ_ERR_UNSUPPORTED;
    }
}
