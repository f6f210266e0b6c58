// gguf_moe on the device: top-k routing, the per-token plan and the expert bank forward.
//
// Routing follows the reference's serial body (amd-nv-cpu.ll:4666-4716) with its portable exp
// (build.rs:1079-1120): the values each expert contributes are computed in parallel, the sums
// that depend on their order are added by one thread in expert order, so the weights are the
// same bits as the CPU path's.
//
// The forward never brings routing decisions to the host. A small planner kernel turns a
// token's dense routing weights into two segment tables in device memory:
//   table A : one segment of `ffn` virtual rows per routed slot (ascending expert index, as
//             amd-nv-cpu.ll:3163-3230 lists them), two sub-rows (the expert's gate row and up
//             row, both against x), epilogue h = silu(g) * u          (lower_gated, recipe.rs:23279)
//   table B : one segment of `hidden` virtual rows, one sub-row per slot (the expert's down row
//             against that slot's h), epilogue y = sum_s w_s * dot_s in slot order
//             (amd-nv-cpu.ll:2359-2362)
// and the streaming matvec kernel walks them. The gated shared expert is one more slot whose
// weight is sigmoid(gate_vector . x) (recipe.rs:23450-23453).
#include <stdlib.h>
#include <string.h>

#include <new>

#include "rq_internal.cuh"

struct rq_moe {
    int type, experts, expert_first, expert_count, hidden, ffn, device;
    uint8_t* base;                      // one allocation
    uint8_t *gate, *up, *down;          // main planes of the local experts' banks
    uint16_t *gate_sc, *up_sc, *down_sc;
    bool has_shared;
    int sh_count;                       // the shared expert is sh_count * ffn wide: sh_count slots of the routed experts' shape
    bool sh_gated;                      // weight sigmoid(gate_vector . x); else weight one
    float routed_scale;                 // the routed weights are multiplied by this (gguf_moe's `scale`)
    uint8_t* sh_base;                   // a shared expert attached after the bank was made: its own allocation
    uint8_t *sh_gate, *sh_up, *sh_down; // gate / up: [sh_count * ffn][hidden]; down: sh_count matrices [hidden][ffn], one per column block
    uint16_t *sh_gate_sc, *sh_up_sc, *sh_down_sc;
    float* sh_vector;                   // [hidden] fp32 gate vector of the shared expert
    // per-token work areas (sized for RQ_MOE_MAX_TOKENS tokens at once)
    RqPlan* plans;                      // [tokens][2]
    float* h;                           // [tokens][slots][ffn]
    int64_t bytes;
};

namespace {

constexpr int kMaxTokens = 64;

// ---- portable transcendentals in fp32 (build.rs:1079-1120 with the fp32 parameters) ----------
__device__ __forceinline__ float pow2f(int k) {
    int b = k + 127;
    b = b < 0 ? 0 : (b > 254 ? 254 : b);
    return __int_as_float(b << 23);
}
__device__ float exp_narrow(float x) {
    if (x != x) return x;
    if (x > (float)88.72283905206835) return __int_as_float(0x7f800000);
    if (x < (float)-103.972084045410) return 0.0f;
    const float kf = floorf(__fadd_rn(__fmul_rn(x, (float)1.4426950408889634074), 0.5f));
    const int k = (int)kf;
    const float hi = (float)__longlong_as_double(0x3FE62E42FEE00000LL);
    const float r = __fsub_rn(__fsub_rn(x, __fmul_rn(kf, hi)), __fmul_rn(kf, (float)1.90821492927058770002e-10));
    // Horner over 1/1! .. 1/8!, innermost coefficient first, one fma per term
    float cur = (float)(1.0 / 40320.0);
    cur = fmaf(cur, r, (float)(1.0 / 5040.0));
    cur = fmaf(cur, r, (float)(1.0 / 720.0));
    cur = fmaf(cur, r, (float)(1.0 / 120.0));
    cur = fmaf(cur, r, (float)(1.0 / 24.0));
    cur = fmaf(cur, r, (float)(1.0 / 6.0));
    cur = fmaf(cur, r, (float)(1.0 / 2.0));
    cur = fmaf(cur, r, 1.0f);
    const float expanded = __fadd_rn(1.0f, __fmul_rn(r, cur));
    const int half = k >> 1, rest = k - half;
    return __fmul_rn(__fmul_rn(expanded, pow2f(half)), pow2f(rest));
}
// the template's own logistic, amd-nv-cpu.ll:5007-5009
__device__ __forceinline__ float logistic(float x) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, exp_narrow(-x))); }
__device__ __forceinline__ float topk_score(float s, float mx, bool sigmoid) { return sigmoid ? logistic(s) : exp_narrow(__fsub_rn(s, mx)); }

// double-precision tanh of build.rs:1146-1166 for the shared expert's gate
__device__ double exp_wide(double x) {
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
    auto p2 = [](int e) { int b = e + 1023; b = b < 0 ? 0 : (b > 2046 ? 2046 : b); return __longlong_as_double((long long)b << 52); };
    return expanded * p2(half) * p2(rest);
}
__device__ float tanh_portable(float xf) {
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
        u = exp_wide(z) - 1.0;
    }
    return (float)(u / (u + 2.0));
}
__device__ __forceinline__ float sigmoid_portable(float x) { return __fmul_rn(0.5f, __fadd_rn(tanh_portable(__fmul_rn(0.5f, x)), 1.0f)); }

// ---- routing: one CTA per token ------------------------------------------------------------
constexpr int kRouteThreads = 256;

// Sums are added in expert order by one thread (the order is part of the result's bits); maxima and the
// top-k picks do not depend on order and are found by the whole CTA. A NaN among the scores or keys makes
// "greater than" order-dependent, so such a token takes the one-thread path throughout.
__device__ __forceinline__ float block_max(float v, float* scratch, int tid) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    __syncthreads();
    if ((tid & 31) == 0) scratch[tid >> 5] = v;
    __syncthreads();
    float m = scratch[0];
    for (int w = 1; w < kRouteThreads / 32; ++w) m = fmaxf(m, scratch[w]);
    return m;
}

__device__ __forceinline__ void route_token(const float* __restrict__ scores, int64_t se, int64_t st, int experts, int top, int sigmoid, int renorm,
                                            const float* __restrict__ bias, float* __restrict__ weights, int64_t we, int64_t wt) {
    extern __shared__ float sm[];      // [experts] raw scores | [experts] values | [experts] keys | [experts] marks
    float* raw = sm;
    float* val = sm + experts;
    float* key = sm + 2 * experts;
    int* mark = (int*)(sm + 3 * experts);
    __shared__ float s_max, s_total, s_wmax[kRouteThreads / 32], s_wkey[kRouteThreads / 32];
    __shared__ int s_widx[kRouteThreads / 32];
    const int t = blockIdx.x, tid = threadIdx.x;
    const bool sig = sigmoid != 0, every = renorm == 0, divide = renorm != 0 || !sig;
    const float kLowest = __int_as_float(0xff800000);  // -inf
    int nan_here = 0;
    for (int e = tid; e < experts; e += kRouteThreads) {
        const float v = scores[e * se + t * st];
        raw[e] = v; mark[e] = 0;
        nan_here |= (v != v) || (bias && bias[e] != bias[e]);
    }
    const bool ordered = __syncthreads_or(nan_here) != 0;  // a NaN somewhere: every step in index order by one thread
    // the scores over every expert, which only a selection bias reads (its key is the score plus the bias): without one the
    // selection key is the raw score, and this pass -- a maximum, an exponential per expert, a total in expert order -- is skipped
    if (bias) {
        // the maximum over every expert
        if (ordered) {
            if (tid == 0) {
                float mx = raw[0];
                for (int e = 1; e < experts; ++e) if (raw[e] > mx) mx = raw[e];
                s_max = mx;
            }
            __syncthreads();
        } else {
            float mx = kLowest;
            for (int e = tid; e < experts; e += kRouteThreads) mx = fmaxf(mx, raw[e]);
            mx = block_max(mx, s_wmax, tid);
            if (tid == 0) s_max = mx;
            __syncthreads();
        }
        for (int e = tid; e < experts; e += kRouteThreads) val[e] = topk_score(raw[e], s_max, sig);
        __syncthreads();
        if (tid == 0) {
            float total = 0.0f;
#pragma unroll 8
            for (int e = 0; e < experts; ++e) total = __fadd_rn(total, val[e]);
            s_total = total;
        }
        __syncthreads();
    }
    // selection key: the raw score, or the probability over every expert plus the expert's bias
    int key_nan = 0;
    for (int e = tid; e < experts; e += kRouteThreads) {
        const float k = bias ? __fadd_rn(sig ? val[e] : __fdiv_rn(val[e], s_total), bias[e]) : raw[e];
        key[e] = k;
        key_nan |= k != k;
    }
    const bool ordered_pick = __syncthreads_or(key_nan) != 0 || ordered;
    // pick `top` times the unmarked expert of strictly greatest key; ties go to the lowest index
    const bool by_rank = !ordered_pick && experts <= 512;
    if (by_rank) {
        // Without NaNs that is the `top` first experts in the order "greater key first, equal keys by index": an expert's
        // place is the number of experts ahead of it, which every thread counts for its own expert with no barrier in between
        // (eight rounds of a block-wide argmax are sixteen barriers; this kernel is one CTA of latency per token).
        for (int e = tid; e < experts; e += kRouteThreads) {
            const float k = key[e];
            int ahead = 0;
#pragma unroll 8
            for (int o = 0; o < experts; ++o) {
                const float ko = key[o];
                ahead += (ko > k || (ko == k && o < e)) ? 1 : 0;
            }
            mark[e] = ahead < top ? 1 : 0;
        }
        __syncthreads();
    }
    for (int pick = 0; pick < top && !by_rank; ++pick) {
        if (ordered_pick) {
            if (tid == 0) {
                int best = -1;
                float best_key = 0.0f;
                for (int e = 0; e < experts; ++e)
                    if (!mark[e] && (best == -1 || key[e] > best_key)) { best = e; best_key = key[e]; }
                if (best >= 0) mark[best] = 1;
            }
            __syncthreads();
        } else {
            int best = 0x7fffffff;
            float best_key = kLowest;
            for (int e = tid; e < experts; e += kRouteThreads)
                if (!mark[e] && (best == 0x7fffffff || key[e] > best_key)) { best = e; best_key = key[e]; }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                const float ok = __shfl_xor_sync(0xffffffffu, best_key, off);
                const int oi = __shfl_xor_sync(0xffffffffu, best, off);
                if (oi != 0x7fffffff && (best == 0x7fffffff || ok > best_key || (ok == best_key && oi < best))) { best = oi; best_key = ok; }
            }
            if ((tid & 31) == 0) { s_wkey[tid >> 5] = best_key; s_widx[tid >> 5] = best; }
            __syncthreads();
            if (tid == 0) {
                for (int w = 1; w < kRouteThreads / 32; ++w) {
                    const float ok = s_wkey[w];
                    const int oi = s_widx[w];
                    if (oi != 0x7fffffff && (best == 0x7fffffff || ok > best_key || (ok == best_key && oi < best))) { best = oi; best_key = ok; }
                }
                if (best != 0x7fffffff) mark[best] = 1;
            }
            __syncthreads();
        }
    }
    // the maximum and the total over the kept experts (or every expert without renormalising)
    if (ordered) {
        if (tid == 0) {
            float mx = 0.0f;
            bool first = true;
            for (int e = 0; e < experts; ++e)
                if ((mark[e] || every) && (first || raw[e] > mx)) { mx = raw[e]; first = false; }
            s_max = mx;
        }
        __syncthreads();
    } else {
        float mx = kLowest;
        int any = 0;
        for (int e = tid; e < experts; e += kRouteThreads)
            if (mark[e] || every) { mx = fmaxf(mx, raw[e]); any = 1; }
        mx = block_max(mx, s_wmax, tid);
        const bool some = __syncthreads_or(any) != 0;
        if (tid == 0) s_max = some ? mx : 0.0f;
        __syncthreads();
    }
    for (int e = tid; e < experts; e += kRouteThreads) val[e] = topk_score(raw[e], s_max, sig);
    __syncthreads();
    if (tid == 0) {
        float total = 0.0f;
#pragma unroll 8
        for (int e = 0; e < experts; ++e)
            if (mark[e] || every) total = __fadd_rn(total, val[e]);  // (the reference adds 0.0 for the others, which leaves every total as it is)
        s_total = total;
    }
    __syncthreads();
    const float denom = divide ? s_total : 1.0f;
    for (int e = tid; e < experts; e += kRouteThreads) weights[e * we + t * wt] = mark[e] ? __fdiv_rn(val[e], denom) : 0.0f;
}

__global__ void __launch_bounds__(kRouteThreads) rq_route_kernel(const float* __restrict__ scores, int64_t se, int64_t st, int experts, int top,
                                                                int sigmoid, int renorm, const float* __restrict__ bias,
                                                                float* __restrict__ weights, int64_t we, int64_t wt) {
    route_token(scores, se, st, experts, top, sigmoid, renorm, bias, weights, we, wt);
}

// ---- planner: one CTA per token ------------------------------------------------------------
struct BankView {
    int type, experts, expert_first, expert_count, hidden, ffn;
    const uint8_t *gate, *up, *down;
    const uint16_t *gate_sc, *up_sc, *down_sc;
    int has_shared, sh_count, sh_gated;
    float routed_scale;
    const uint8_t *sh_gate, *sh_up, *sh_down;
    const uint16_t *sh_gate_sc, *sh_up_sc, *sh_down_sc;
    const float* sh_vector;
};

__device__ __forceinline__ void plan_token(const BankView& b, const float* __restrict__ routing, int64_t re, int64_t rt, const float* __restrict__ x, int64_t sk,
                                           int64_t st, int top, int include_shared, RqPlan* __restrict__ plans, float* __restrict__ h, float* __restrict__ y,
                                           int64_t yn, int64_t yt) {
    const int t = blockIdx.x, tid = threadIdx.x;
    __shared__ float red[256];
    __shared__ float s_gate;
    const int per = b.type == RQ_Q4_K || b.type == RQ_Q6_K ? 256 : 32;
    const int main_unit = b.type == RQ_Q4_K ? 144 : (b.type == RQ_Q6_K ? 208 : (b.type == RQ_Q8_0 ? 32 : 16));
    const int64_t in_row_main = (int64_t)(b.hidden / per) * main_unit, in_row_sc = b.hidden / per;   // gate / up rows (hidden inputs)
    const int64_t dn_row_main = (int64_t)(b.ffn / per) * main_unit, dn_row_sc = b.ffn / per;         // down rows (ffn inputs)
    // the shared expert's weight: sigmoid of a one-row bias-free contraction (partials in a fixed tree)
    if (b.has_shared && include_shared && b.sh_gated) {
        float acc = 0.0f;
        for (int k = tid; k < b.hidden; k += 256) acc = __fadd_rn(acc, __fmul_rn(b.sh_vector[k], x[k * sk + t * st]));
        red[tid] = acc;
        __syncthreads();
        // the fixed tree red[i] += red[i + off], off = 128 .. 1: across warps through shared memory, inside warp 0 by shuffles
        // (the same pairs in the same order, five barriers fewer)
        for (int off = 128; off >= 32; off >>= 1) { if (tid < off) red[tid] = __fadd_rn(red[tid], red[tid + off]); __syncthreads(); }
        if (tid < 32) {
            float v = red[tid];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) v = __fadd_rn(v, __shfl_down_sync(0xffffffffu, v, off));
            if (tid == 0) s_gate = sigmoid_portable(v);
        }
        __syncthreads();
    }
    RqPlan* pa = plans + 2 * t;
    RqPlan* pb = pa + 1;
    const int slots_max = top + (b.has_shared ? b.sh_count : 1);
    float* ht = h + (size_t)t * slots_max * b.ffn;
    // Routed experts that live here take slots in ascending expert index. Every thread looks at one expert
    // per sweep; a selected expert's slot is the number of selected experts before it (ballots and counts).
    __shared__ int s_warp_count[8];
    __shared__ int s_base;
    if (tid == 0) s_base = 0;
    __syncthreads();
    const int lane = tid & 31, warp = tid >> 5;
    for (int e0 = b.expert_first; e0 < b.expert_first + b.expert_count; e0 += 256) {
        const int e = e0 + tid;
        const bool in = e < b.expert_first + b.expert_count;
        const float w = in ? routing[e * re + t * rt] : 0.0f;
        const bool sel = in && w != 0.0f;
        const unsigned ballot = __ballot_sync(0xffffffffu, sel);
        if (lane == 0) s_warp_count[warp] = __popc(ballot);
        __syncthreads();
        int n = s_base + __popc(ballot & ((1u << lane) - 1u));
        for (int w2 = 0; w2 < warp; ++w2) n += s_warp_count[w2];
        if (sel && n < top) {
            const int le = e - b.expert_first;
            RqSegment& sa = pa->seg[n];
            sa.row_begin = n * b.ffn; sa.rows = b.ffn; sa.y = ht + (size_t)n * b.ffn;
            sa.main[0] = b.gate + (size_t)le * b.ffn * in_row_main; sa.main[1] = b.up + (size_t)le * b.ffn * in_row_main;
            sa.scale[0] = b.gate_sc ? b.gate_sc + (size_t)le * b.ffn * in_row_sc : nullptr;
            sa.scale[1] = b.up_sc ? b.up_sc + (size_t)le * b.ffn * in_row_sc : nullptr;
            sa.act[0] = 0; sa.act[1] = 0; sa.coef[0] = 1.0f; sa.coef[1] = 1.0f;
            RqSegment& sb = pb->seg[0];
            sb.main[n] = b.down + (size_t)le * b.hidden * dn_row_main;
            sb.scale[n] = b.down_sc ? b.down_sc + (size_t)le * b.hidden * dn_row_sc : nullptr;
            sb.act[n] = n; sb.coef[n] = b.routed_scale == 1.0f ? w : __fmul_rn(w, b.routed_scale);
        }
        __syncthreads();
        if (tid == 0) { int total = 0; for (int w2 = 0; w2 < 8; ++w2) total += s_warp_count[w2]; s_base += total; }
        __syncthreads();
    }
    if (tid == 0) {
        int n = s_base < top ? s_base : top;
        if (b.has_shared && include_shared) {
            // the shared expert: sh_count slots of the routed experts' shape (rows j * ffn .. of its gate / up banks, column
            // block j of its down bank), every one at the shared weight
            const float weight = b.sh_gated ? s_gate : 1.0f;
            for (int j = 0; j < b.sh_count; ++j, ++n) {
                RqSegment& sa = pa->seg[n];
                sa.row_begin = n * b.ffn; sa.rows = b.ffn; sa.y = ht + (size_t)n * b.ffn;
                sa.main[0] = b.sh_gate + (size_t)j * b.ffn * in_row_main; sa.main[1] = b.sh_up + (size_t)j * b.ffn * in_row_main;
                sa.scale[0] = b.sh_gate_sc ? b.sh_gate_sc + (size_t)j * b.ffn * in_row_sc : nullptr;
                sa.scale[1] = b.sh_up_sc ? b.sh_up_sc + (size_t)j * b.ffn * in_row_sc : nullptr;
                sa.act[0] = 0; sa.act[1] = 0; sa.coef[0] = 1.0f; sa.coef[1] = 1.0f;
                RqSegment& sb = pb->seg[0];
                sb.main[n] = b.sh_down + (size_t)j * b.hidden * dn_row_main;
                sb.scale[n] = b.sh_down_sc ? b.sh_down_sc + (size_t)j * b.hidden * dn_row_sc : nullptr;
                sb.act[n] = n; sb.coef[n] = weight;
            }
        }
        pa->n_segments = n; pa->subs = 2; pa->total_rows = n * b.ffn; pa->pad = 0;
        RqSegment& sb = pb->seg[0];
        sb.row_begin = 0; sb.rows = b.hidden; sb.y = y + (int64_t)t * yt;
        pb->n_segments = n > 0 ? 1 : 0; pb->subs = n; pb->total_rows = n > 0 ? b.hidden : 0; pb->pad = 0;
    }
    // a token nothing here is routed to still owes zeros (the caller sums the ranks' outputs)
    __syncthreads();
    if (pb->total_rows == 0)
        for (int r = tid; r < b.hidden; r += 256) y[r * yn + (int64_t)t * yt] = 0.0f;
}

__global__ void __launch_bounds__(256) rq_moe_plan_kernel(BankView b, const float* __restrict__ routing, int64_t re, int64_t rt,
                                                         const float* __restrict__ x, int64_t sk, int64_t st, int top, int include_shared,
                                                         RqPlan* __restrict__ plans, float* __restrict__ h, float* __restrict__ y, int64_t yn, int64_t yt) {
    plan_token(b, routing, re, rt, x, sk, st, top, include_shared, plans, h, y, yn, yt);
}

// Routing and planning of a token in one launch: the CTA that computed the token's routing weights (and wrote them to the
// dense plane, which stays the block's visible result) reads them back after a barrier and writes the token's two segment
// tables. One launch and one dependency less on the path of a decode step.
static_assert(kRouteThreads == 256, "the fused launch runs both bodies with the same CTA");
__global__ void __launch_bounds__(256) rq_moe_route_plan_kernel(BankView b, const float* __restrict__ scores, int64_t se, int64_t sst, int experts, int top, int sigmoid,
                                                               int renorm, const float* __restrict__ bias, float* __restrict__ weights, int64_t we, int64_t wt,
                                                               const float* __restrict__ x, int64_t sk, int64_t st, int include_shared, RqPlan* __restrict__ plans,
                                                               float* __restrict__ h, float* __restrict__ y, int64_t yn, int64_t yt) {
    route_token(scores, se, sst, experts, top, sigmoid, renorm, bias, weights, we, wt);
    __syncthreads();  // the CTA's own stores to the plane are visible to its threads after the barrier
    plan_token(b, weights, we, wt, x, sk, st, top, include_shared, plans, h, y, yn, yt);
}

static BankView view_of(const rq_moe* m) {
    BankView b;
    b.type = m->type; b.experts = m->experts; b.expert_first = m->expert_first; b.expert_count = m->expert_count; b.hidden = m->hidden; b.ffn = m->ffn;
    b.gate = m->gate; b.up = m->up; b.down = m->down; b.gate_sc = m->gate_sc; b.up_sc = m->up_sc; b.down_sc = m->down_sc;
    b.has_shared = m->has_shared ? 1 : 0; b.sh_count = m->sh_count; b.sh_gated = m->sh_gated ? 1 : 0; b.routed_scale = m->routed_scale;
    b.sh_gate = m->sh_gate; b.sh_up = m->sh_up; b.sh_down = m->sh_down; b.sh_gate_sc = m->sh_gate_sc; b.sh_up_sc = m->sh_up_sc; b.sh_down_sc = m->sh_down_sc;
    b.sh_vector = m->sh_vector;
    return b;
}

static int64_t main_bytes_of(int type, int64_t rows, int64_t cols) {
    const int per = rq_block_values(type), bytes = rq_block_bytes(type);
    return rows * (cols / per) * (type == RQ_Q4_K ? 144 : bytes - 2);
}
static int64_t scale_bytes_of(int type, int64_t rows, int64_t cols) { return type == RQ_Q4_K ? 0 : rows * (cols / rq_block_values(type)) * 2; }
static int64_t pad256(int64_t v) { return (v + 255) / 256 * 256; }

// Uploads `rows` rows of GGUF blocks and lays them out as planes at main / scale.
static int upload_bank(rq_ctx* ctx, int type, const void* host_blocks, int64_t rows, int64_t cols, uint8_t* main, uint16_t* scale) {
    rq_weight tmp;
    memset(&tmp, 0, sizeof(tmp));
    tmp.type = type; tmp.rows = rows; tmp.cols = cols; tmp.main = main; tmp.scale = scale; tmp.device = ctx->device;
    const int64_t total = rows * (cols / rq_block_values(type)) * rq_block_bytes(type);
    // in slices, so the staging copy stays small next to a large bank
    const int64_t row_gguf = cols / rq_block_values(type) * rq_block_bytes(type);
    int64_t rows_per = (256ll << 20) / row_gguf;
    if (rows_per < 1) rows_per = 1;
    uint8_t* staging = nullptr;
    const int64_t cap = (rows_per < rows ? rows_per : rows) * row_gguf;
    cudaError_t e = cudaMalloc(&staging, (size_t)cap + 16);
    if (e != cudaSuccess) return rq_fail(RQ_ERR_ALLOC, "expert bank staging of %lld bytes: %s", (long long)cap, cudaGetErrorString(e));
    int rc = RQ_OK;
    for (int64_t r0 = 0; r0 < rows && !rc; r0 += rows_per) {
        const int64_t nr = r0 + rows_per <= rows ? rows_per : rows - r0;
        e = cudaMemcpy(staging, (const uint8_t*)host_blocks + r0 * row_gguf, (size_t)(nr * row_gguf), cudaMemcpyHostToDevice);
        if (e != cudaSuccess) { rc = rq_fail(RQ_ERR_CUDA, "expert bank upload: %s", cudaGetErrorString(e)); break; }
        rq_weight part = tmp;
        part.rows = nr;
        part.main = main + main_bytes_of(type, r0, cols);
        part.scale = scale ? scale + scale_bytes_of(type, r0, cols) / 2 : nullptr;
        rc = rq_launch_repack(&part, staging, nullptr);
        if (!rc && cudaDeviceSynchronize() != cudaSuccess) rc = rq_fail(RQ_ERR_CUDA, "expert bank repack failed");
    }
    cudaFree(staging);
    (void)total;
    return rc;
}

}  // namespace

extern "C" void rq_moe_free(rq_ctx* ctx, rq_moe* m) {
    if (!m) return;
    DeviceGuard guard(ctx ? ctx->device : m->device);
    if (m->base) cudaFree(m->base);
    if (m->sh_base) cudaFree(m->sh_base);
    delete m;
}

extern "C" int rq_moe_prepare(rq_ctx* ctx, int type, const void* gate, const void* up, const void* down, int experts, int expert_first,
                              int expert_count, int hidden, int ffn, const void* sh_gate, const void* sh_up, const void* sh_down,
                              const float* sh_vector, rq_moe** out) {
    if (!ctx || !gate || !up || !down || !out) return rq_fail(RQ_ERR_INVALID, "rq_moe_prepare: null argument");
    *out = nullptr;
    const int per = rq_block_values(type);
    if (!per || !rq_type_has_fast_path(type)) return rq_fail(per ? RQ_ERR_UNSUPPORTED : RQ_ERR_INVALID, "rq_moe_prepare: GGML type %d is not served for expert banks (Q4_0, Q8_0, Q4_K, Q6_K are)", type);
    if (hidden <= 0 || ffn <= 0 || hidden % 256 || ffn % 256) return rq_fail(RQ_ERR_INVALID, "rq_moe_prepare: hidden=%d and ffn=%d must be positive multiples of 256", hidden, ffn);
    if (experts <= 0 || expert_first < 0 || expert_count <= 0 || expert_first + expert_count > experts)
        return rq_fail(RQ_ERR_INVALID, "rq_moe_prepare: experts [%d, %d) outside the bank's %d", expert_first, expert_first + expert_count, experts);
    const bool shared = sh_gate || sh_up || sh_down || sh_vector;
    if (shared && !(sh_gate && sh_up && sh_down && sh_vector)) return rq_fail(RQ_ERR_INVALID, "rq_moe_prepare: a shared expert needs its gate, up and down banks and its gate vector");
    DeviceGuard guard(ctx->device);
    rq_moe* m = new (std::nothrow) rq_moe();
    if (!m) return rq_fail(RQ_ERR_ALLOC, "out of host memory");
    memset(m, 0, sizeof(*m));
    m->type = type; m->experts = experts; m->expert_first = expert_first; m->expert_count = expert_count; m->hidden = hidden; m->ffn = ffn;
    m->device = ctx->device; m->has_shared = shared; m->sh_count = 1; m->sh_gated = true; m->routed_scale = 1.0f;
    const int64_t in_rows = (int64_t)expert_count * ffn, dn_rows = (int64_t)expert_count * hidden;
    const int64_t in_main = pad256(main_bytes_of(type, in_rows, hidden)), in_sc = pad256(scale_bytes_of(type, in_rows, hidden) + 64);
    const int64_t dn_main = pad256(main_bytes_of(type, dn_rows, ffn)), dn_sc = pad256(scale_bytes_of(type, dn_rows, ffn) + 64);
    const int64_t sh_in_main = shared ? pad256(main_bytes_of(type, ffn, hidden)) : 0, sh_in_sc = shared ? pad256(scale_bytes_of(type, ffn, hidden) + 64) : 0;
    const int64_t sh_dn_main = shared ? pad256(main_bytes_of(type, hidden, ffn)) : 0, sh_dn_sc = shared ? pad256(scale_bytes_of(type, hidden, ffn) + 64) : 0;
    const int64_t vec = shared ? pad256((int64_t)hidden * 4) : 0;
    const int64_t plans = pad256((int64_t)sizeof(RqPlan) * 2 * kMaxTokens);
    const int64_t hbytes = pad256((int64_t)kMaxTokens * (RQ_MAX_SUB) * ffn * 4);
    const int64_t total = 2 * (in_main + in_sc) + dn_main + dn_sc + 2 * (sh_in_main + sh_in_sc) + sh_dn_main + sh_dn_sc + vec + plans + hbytes + 256;
    cudaError_t e = cudaMalloc(&m->base, (size_t)total);
    if (e != cudaSuccess) { delete m; return rq_fail(RQ_ERR_ALLOC, "expert bank of %lld bytes: %s", (long long)total, cudaGetErrorString(e)); }
    m->bytes = total;
    uint8_t* at = m->base;
    auto take = [&](int64_t n) { uint8_t* p = at; at += n; return p; };
    const bool planes = type != RQ_Q4_K;
    m->gate = take(in_main); m->gate_sc = planes ? (uint16_t*)take(in_sc) : nullptr;
    m->up = take(in_main); m->up_sc = planes ? (uint16_t*)take(in_sc) : nullptr;
    m->down = take(dn_main); m->down_sc = planes ? (uint16_t*)take(dn_sc) : nullptr;
    if (shared) {
        m->sh_gate = take(sh_in_main); m->sh_gate_sc = planes ? (uint16_t*)take(sh_in_sc) : nullptr;
        m->sh_up = take(sh_in_main); m->sh_up_sc = planes ? (uint16_t*)take(sh_in_sc) : nullptr;
        m->sh_down = take(sh_dn_main); m->sh_down_sc = planes ? (uint16_t*)take(sh_dn_sc) : nullptr;
        m->sh_vector = (float*)take(vec);
    }
    m->plans = (RqPlan*)take(plans);
    m->h = (float*)take(hbytes);
    const int64_t in_gguf = (int64_t)ffn * (hidden / per) * rq_block_bytes(type), dn_gguf = (int64_t)hidden * (ffn / per) * rq_block_bytes(type);
    int rc = upload_bank(ctx, type, (const uint8_t*)gate + (int64_t)expert_first * in_gguf, in_rows, hidden, m->gate, m->gate_sc);
    if (!rc) rc = upload_bank(ctx, type, (const uint8_t*)up + (int64_t)expert_first * in_gguf, in_rows, hidden, m->up, m->up_sc);
    if (!rc) rc = upload_bank(ctx, type, (const uint8_t*)down + (int64_t)expert_first * dn_gguf, dn_rows, ffn, m->down, m->down_sc);
    if (!rc && shared) {
        rc = upload_bank(ctx, type, sh_gate, ffn, hidden, m->sh_gate, m->sh_gate_sc);
        if (!rc) rc = upload_bank(ctx, type, sh_up, ffn, hidden, m->sh_up, m->sh_up_sc);
        if (!rc) rc = upload_bank(ctx, type, sh_down, hidden, ffn, m->sh_down, m->sh_down_sc);
        if (!rc && cudaMemcpy(m->sh_vector, sh_vector, (size_t)hidden * 4, cudaMemcpyHostToDevice) != cudaSuccess) rc = rq_fail(RQ_ERR_CUDA, "shared gate vector upload failed");
    }
    if (rc) { rq_moe_free(ctx, m); return rc; }
    *out = m;
    return RQ_OK;
}

extern "C" int64_t rq_moe_bytes(const rq_moe* m) { return m ? m->bytes : 0; }

extern "C" int rq_moe_set_routed_scale(rq_moe* m, float scale) {
    if (!m) return rq_fail(RQ_ERR_INVALID, "rq_moe_set_routed_scale: null bank");
    if (!(scale == scale) || scale > 3.0e38f || scale < -3.0e38f) return rq_fail(RQ_ERR_INVALID, "moe routed scale must be finite");
    m->routed_scale = scale;
    return RQ_OK;
}

extern "C" int rq_moe_attach_shared(rq_ctx* ctx, rq_moe* m, int gated, int count, const void* sh_gate, const void* sh_up, const void* sh_down, const float* gate_vector) {
    if (!ctx || !m || !sh_gate || !sh_up || !sh_down) return rq_fail(RQ_ERR_INVALID, "rq_moe_attach_shared: null argument");
    if (m->has_shared) return rq_fail(RQ_ERR_INVALID, "rq_moe_attach_shared: the bank already has a shared expert");
    if (count <= 0) return rq_fail(RQ_ERR_INVALID, "shared expert count must be positive");
    if (count >= RQ_MAX_SUB) return rq_fail(RQ_ERR_LIMIT, "rq_moe_attach_shared: count=%d, at most %d", count, RQ_MAX_SUB - 1);
    if (gated && !gate_vector) return rq_fail(RQ_ERR_INVALID, "rq_moe_attach_shared: a gated shared expert needs its gate vector");
    DeviceGuard guard(ctx->device);
    const int type = m->type, hidden = m->hidden, ffn = m->ffn, per = rq_block_values(type), stride = rq_block_bytes(type);
    const int64_t width = (int64_t)count * ffn;
    const int64_t in_main = pad256(main_bytes_of(type, width, hidden)), in_sc = pad256(scale_bytes_of(type, width, hidden) + 64);
    const int64_t dn_main = pad256(main_bytes_of(type, (int64_t)count * hidden, ffn)), dn_sc = pad256(scale_bytes_of(type, (int64_t)count * hidden, ffn) + 64);
    const int64_t vec = pad256((int64_t)hidden * 4);
    const int64_t total = 2 * (in_main + in_sc) + dn_main + dn_sc + vec + 256;
    cudaError_t e = cudaMalloc(&m->sh_base, (size_t)total);
    if (e != cudaSuccess) return rq_fail(RQ_ERR_ALLOC, "shared expert of %lld bytes: %s", (long long)total, cudaGetErrorString(e));
    uint8_t* at = m->sh_base;
    auto take = [&](int64_t n) { uint8_t* p = at; at += n; return p; };
    const bool planes = type != RQ_Q4_K;
    m->sh_gate = take(in_main); m->sh_gate_sc = planes ? (uint16_t*)take(in_sc) : nullptr;
    m->sh_up = take(in_main); m->sh_up_sc = planes ? (uint16_t*)take(in_sc) : nullptr;
    m->sh_down = take(dn_main); m->sh_down_sc = planes ? (uint16_t*)take(dn_sc) : nullptr;
    m->sh_vector = (float*)take(vec);
    int rc = upload_bank(ctx, type, sh_gate, width, hidden, m->sh_gate, m->sh_gate_sc);
    if (!rc) rc = upload_bank(ctx, type, sh_up, width, hidden, m->sh_up, m->sh_up_sc);
    if (!rc) {
        // down is [hidden][count * ffn]: column block j of every row becomes matrix j, [hidden][ffn] (a block of ffn inputs is
        // whole GGUF blocks, so the split moves bytes, nothing is re-encoded)
        const int64_t block_row = (int64_t)ffn / per * stride, full_row = block_row * count;
        uint8_t* split = (uint8_t*)malloc((size_t)(full_row * hidden));
        if (!split) rc = rq_fail(RQ_ERR_ALLOC, "out of host memory");
        else {
            for (int j = 0; j < count; ++j)
                for (int64_t r = 0; r < hidden; ++r)
                    memcpy(split + ((int64_t)j * hidden + r) * block_row, (const uint8_t*)sh_down + r * full_row + (int64_t)j * block_row, (size_t)block_row);
            rc = upload_bank(ctx, type, split, (int64_t)count * hidden, ffn, m->sh_down, m->sh_down_sc);
            free(split);
        }
    }
    if (!rc && gated && cudaMemcpy(m->sh_vector, gate_vector, (size_t)hidden * 4, cudaMemcpyHostToDevice) != cudaSuccess) rc = rq_fail(RQ_ERR_CUDA, "shared gate vector upload failed");
    if (rc) { cudaFree(m->sh_base); m->sh_base = nullptr; return rc; }
    m->has_shared = true; m->sh_count = count; m->sh_gated = gated != 0;
    m->bytes += total;
    return RQ_OK;
}

extern "C" int rq_moe_route(rq_ctx* ctx, const float* scores, int64_t score_e_stride, int64_t score_t_stride, int experts, int top_k, int scoring,
                            int renormalize, const float* selection_bias, int tokens, float* weights, int64_t weight_e_stride,
                            int64_t weight_t_stride, void* stream) {
    if (!ctx || !scores || !weights) return rq_fail(RQ_ERR_INVALID, "rq_moe_route: null argument");
    if (experts <= 0 || top_k <= 0 || top_k > experts || tokens <= 0) return rq_fail(RQ_ERR_INVALID, "rq_moe_route: experts=%d top_k=%d tokens=%d", experts, top_k, tokens);
    if (experts > 8192) return rq_fail(RQ_ERR_LIMIT, "rq_moe_route: %d experts, at most 8192", experts);
    if (scoring != RQ_SCORE_SOFTMAX && scoring != RQ_SCORE_SIGMOID) return rq_fail(RQ_ERR_INVALID, "rq_moe_route: scoring=%d", scoring);
    DeviceGuard guard(ctx->device);
    if ((size_t)experts * 16 > 40 * 1024) {
        // beyond the default dynamic shared memory of a block: opt in once per device (8192 experts take 128 KB)
        static bool configured[64] = {};
        int dev = ctx->device;
        if (dev < 0 || dev >= 64 || !configured[dev]) {
            RQ_CUDA(cudaFuncSetAttribute(rq_route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 8192 * 16));
            if (dev >= 0 && dev < 64) configured[dev] = true;
        }
    }
    rq_route_kernel<<<tokens, kRouteThreads, (size_t)experts * 16, (cudaStream_t)stream>>>(scores, score_e_stride, score_t_stride, experts, top_k, scoring,
                                                                                        renormalize, selection_bias, weights, weight_e_stride,
                                                                                        weight_t_stride);
    RQ_CUDA(cudaGetLastError());
    return RQ_OK;
}

static int check_forward(const char* who, const rq_ctx* ctx, const rq_moe* m, const void* x, const void* routing, const void* y, int top_k, int tokens,
                         int64_t x_k_stride, int64_t y_n_stride) {
    if (!ctx || !m || !x || !routing || !y) return rq_fail(RQ_ERR_INVALID, "%s: null argument", who);
    if (m->device != ctx->device) return rq_fail(RQ_ERR_INVALID, "%s: bank lives on device %d, context on %d", who, m->device, ctx->device);
    if (tokens <= 0 || tokens > kMaxTokens) return rq_fail(RQ_ERR_LIMIT, "%s: tokens=%d, between 1 and %d per call", who, tokens, kMaxTokens);
    const int shared_slots = m->has_shared ? m->sh_count : 1;
    if (top_k <= 0 || top_k + shared_slots > RQ_MAX_SUB)
        return rq_fail(RQ_ERR_LIMIT, "%s: top_k=%d with a shared expert of %d x the expert width: at most %d slots together", who, top_k, shared_slots, RQ_MAX_SUB);
    if (x_k_stride <= 0 || y_n_stride <= 0) return rq_fail(RQ_ERR_INVALID, "%s: strides must be positive", who);
    return RQ_OK;
}

static int launch_banks(rq_ctx* ctx, rq_moe* m, const float* x, int64_t x_k_stride, int64_t x_t_stride, int top_k, int tokens, int64_t y_n_stride, cudaStream_t s);

// rq_moe_route and rq_moe_forward as one call: the routing weights land in `weights` as rq_moe_route writes them, and the
// token's plan is made by the same launch (three launches per call instead of four).
extern "C" int rq_moe_route_forward(rq_ctx* ctx, rq_moe* m, const float* scores, int64_t score_e_stride, int64_t score_t_stride, int top_k, int scoring,
                                    int renormalize, const float* selection_bias, float* weights, int64_t weight_e_stride, int64_t weight_t_stride,
                                    const float* x, int64_t x_k_stride, int64_t x_t_stride, int tokens, int include_shared, float* y, int64_t y_n_stride,
                                    int64_t y_t_stride, void* stream) {
    if (!scores) return rq_fail(RQ_ERR_INVALID, "rq_moe_route_forward: null argument");
    int rc = check_forward("rq_moe_route_forward", ctx, m, x, weights, y, top_k, tokens, x_k_stride, y_n_stride);
    if (rc) return rc;
    const int experts = m->experts;
    if (top_k > experts) return rq_fail(RQ_ERR_INVALID, "rq_moe_route_forward: top_k=%d of %d experts", top_k, experts);
    if (experts > 8192) return rq_fail(RQ_ERR_LIMIT, "rq_moe_route_forward: %d experts, at most 8192", experts);
    if (scoring != RQ_SCORE_SOFTMAX && scoring != RQ_SCORE_SIGMOID) return rq_fail(RQ_ERR_INVALID, "rq_moe_route_forward: scoring=%d", scoring);
    DeviceGuard guard(ctx->device);
    cudaStream_t s = (cudaStream_t)stream;
    rc = rq_order_work_areas(ctx, s);
    if (rc) return rc;
    if ((size_t)experts * 16 > 40 * 1024) {
        static bool configured[64] = {};
        int dev = ctx->device;
        if (dev < 0 || dev >= 64 || !configured[dev]) {
            RQ_CUDA(cudaFuncSetAttribute(rq_moe_route_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 8192 * 16));
            if (dev >= 0 && dev < 64) configured[dev] = true;
        }
    }
    rq_moe_route_plan_kernel<<<tokens, 256, (size_t)experts * 16, s>>>(view_of(m), scores, score_e_stride, score_t_stride, experts, top_k, scoring, renormalize,
                                                                       selection_bias, weights, weight_e_stride, weight_t_stride, x, x_k_stride, x_t_stride,
                                                                       include_shared, m->plans, m->h, y, y_n_stride, y_t_stride);
    RQ_CUDA(cudaGetLastError());
    return launch_banks(ctx, m, x, x_k_stride, x_t_stride, top_k, tokens, y_n_stride, s);
}

extern "C" int rq_moe_forward(rq_ctx* ctx, rq_moe* m, const float* x, int64_t x_k_stride, int64_t x_t_stride, const float* routing,
                              int64_t routing_e_stride, int64_t routing_t_stride, int top_k, int tokens, int include_shared, float* y,
                              int64_t y_n_stride, int64_t y_t_stride, void* stream) {
    int rc = check_forward("rq_moe_forward", ctx, m, x, routing, y, top_k, tokens, x_k_stride, y_n_stride);
    if (rc) return rc;
    DeviceGuard guard(ctx->device);
    cudaStream_t s = (cudaStream_t)stream;
    rc = rq_order_work_areas(ctx, s);  // the bank's plans and hidden activations are shared by every call on it
    if (rc) return rc;
    rq_moe_plan_kernel<<<tokens, 256, 0, s>>>(view_of(m), routing, routing_e_stride, routing_t_stride, x, x_k_stride, x_t_stride, top_k, include_shared,
                                              m->plans, m->h, y, y_n_stride, y_t_stride);
    RQ_CUDA(cudaGetLastError());
    return launch_banks(ctx, m, x, x_k_stride, x_t_stride, top_k, tokens, y_n_stride, s);
}

static int launch_banks(rq_ctx* ctx, rq_moe* m, const float* x, int64_t x_k_stride, int64_t x_t_stride, int top_k, int tokens, int64_t y_n_stride, cudaStream_t s) {
    const int shared_slots = m->has_shared ? m->sh_count : 1;
    const int slots = top_k + shared_slots;
    int rc;
    // All tokens in two launches: grid row t of each reads token t's plan and activations.
    // expert gate and up rows against the token's x, h = silu(g) * u per slot
    rc = rq_launch_stream_plan(ctx, m->type, m->hidden, m->plans, tokens, 2, slots, 2, RQ_EPI_GLU, (int64_t)slots * m->ffn, x, x_t_stride, x_k_stride, 0,
                                   1, 1, 0, s);
    if (rc == RQ_ERR_UNSUPPORTED) return rq_fail(RQ_ERR_LIMIT, "rq_moe_forward: hidden=%d is beyond what the streaming kernel holds", m->hidden);
    if (rc) return rc;
    // expert down rows, one sub-row per slot against that slot's h, summed with the routing weights
    rc = rq_launch_stream_plan(ctx, m->type, m->ffn, m->plans + 1, tokens, 2, 1, slots, RQ_EPI_WSUM, m->hidden, m->h, (int64_t)slots * m->ffn, 1, m->ffn, slots,
                               y_n_stride, 0, s);
    if (rc == RQ_ERR_UNSUPPORTED) return rq_fail(RQ_ERR_LIMIT, "rq_moe_forward: ffn=%d with %d slots is beyond what the streaming kernel holds", m->ffn, slots);
    if (rc) return rc;
    return RQ_OK;
}
