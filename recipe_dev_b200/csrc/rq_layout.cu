// Load-time layout kernels (GGUF blocks <-> device planes) and the bit-exact dequantiser.
#include "rq_decode.cuh"
#include "rq_internal.cuh"

// GGUF strides 18/34/210 are multiples of two, so blocks move as 16-bit words.
// mode 0: GGUF -> planes, mode 1: planes -> GGUF.
template <int TYPE>
__global__ void rq_plane_kernel(uint16_t* __restrict__ gguf, uint16_t* __restrict__ main_plane, uint16_t* __restrict__ scale_plane,
                                int64_t blocks, int to_gguf, int64_t cols) {
    constexpr int WORDS = TYPE == RQ_Q6_K ? 105 : (TYPE == RQ_Q8_0 ? 17 : 9);
    constexpr int BODY = WORDS - 1;                       // 16-bit words of the block that are not d
    constexpr int D_AT = TYPE == RQ_Q6_K ? 104 : 0;       // where d sits in the GGUF block
    int64_t total = blocks * WORDS;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t b = i / WORDS;
        int wd = (int)(i - b * WORDS);
        uint16_t* g = gguf + i;
        uint16_t* p;
        if (wd == D_AT) {
            p = scale_plane + b;
        } else if (rq_plane_permuted(TYPE, cols)) {
            // byte offset of this word in its row's plane, with the row's chunk permutation applied
            const int64_t per_row = cols >> 5, row = b / per_row, in_row = b - row * per_row;
            const int64_t off = in_row * (2 * BODY) + 2 * (wd - 1);
            const int64_t phys = (rq_plane_chunk(TYPE, off >> 4) << 4) | (off & 15);
            p = main_plane + (row * per_row * (2 * BODY) + phys) / 2;
        } else {
            p = main_plane + b * BODY + (TYPE == RQ_Q6_K ? wd : wd - 1);
        }
        if (to_gguf) *g = *p; else *p = *g;
    }
}

static int plane_launch(const rq_weight* w, uint8_t* blocks, int to_gguf, cudaStream_t s) {
    int64_t nblocks = w->rows * (w->cols / rq_block_values(w->type));
    if (rq_type_keeps_blocks(w->type)) {
        const size_t bytes = (size_t)nblocks * (size_t)rq_block_bytes(w->type);
        if (to_gguf) RQ_CUDA(cudaMemcpyAsync(blocks, w->main, bytes, cudaMemcpyDeviceToDevice, s));
        else RQ_CUDA(cudaMemcpyAsync(w->main, blocks, bytes, cudaMemcpyDeviceToDevice, s));
        return RQ_OK;
    }
    int threads = 256;
    int64_t words = nblocks * (rq_block_bytes(w->type) / 2);
    int grid = (int)((words + threads - 1) / threads < 148 * 16 ? (words + threads - 1) / threads : 148 * 16);
    if (grid < 1) grid = 1;
    uint16_t* g = (uint16_t*)blocks;
    uint16_t* m = (uint16_t*)w->main;
    switch (w->type) {
        case RQ_Q6_K: rq_plane_kernel<RQ_Q6_K><<<grid, threads, 0, s>>>(g, m, w->scale, nblocks, to_gguf, w->cols); break;
        case RQ_Q8_0: rq_plane_kernel<RQ_Q8_0><<<grid, threads, 0, s>>>(g, m, w->scale, nblocks, to_gguf, w->cols); break;
        case RQ_Q4_0: rq_plane_kernel<RQ_Q4_0><<<grid, threads, 0, s>>>(g, m, w->scale, nblocks, to_gguf, w->cols); break;
        default: return rq_fail(RQ_ERR_INVALID, "layout: type %d", w->type);
    }
    RQ_CUDA(cudaGetLastError());
    return RQ_OK;
}

int rq_launch_repack(const rq_weight* w, const uint8_t* dev_blocks, cudaStream_t s) { return plane_launch(w, (uint8_t*)dev_blocks, 0, s); }
int rq_launch_export(const rq_weight* w, uint8_t* dev_blocks, cudaStream_t s) { return plane_launch(w, dev_blocks, 1, s); }

// ---------------------------------------------------------------------------------------
// Dequantiser: one thread per value. Every fp32 step is a separate rounded operation
// (__fmul_rn / __fsub_rn never contract), which is what makes the result bit-equal to the
// reference's f64 unpacking rounded to fp32: d*sc, dmin*m and step*q are exact in fp32, and
// the one inexact step, the final subtract, rounds the same exact difference.
// ---------------------------------------------------------------------------------------
template <int TYPE>
__global__ void rq_dequant_kernel(const uint8_t* __restrict__ main_plane, const uint16_t* __restrict__ scale_plane, float* __restrict__ out, int64_t count, int64_t cols) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < count; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = rq_decode_value<TYPE>(main_plane, scale_plane, i, cols);
}

int rq_launch_dequant(const rq_weight* w, float* out, cudaStream_t s) {
    int64_t count = w->rows * w->cols;
    int threads = 256;
    int64_t want = (count + threads - 1) / threads;
    int grid = (int)(want < 148 * 32 ? want : 148 * 32);
    switch (w->type) {
        case RQ_Q4_K: rq_dequant_kernel<RQ_Q4_K><<<grid, threads, 0, s>>>(w->main, w->scale, out, count, w->cols); break;
        case RQ_Q6_K: rq_dequant_kernel<RQ_Q6_K><<<grid, threads, 0, s>>>(w->main, w->scale, out, count, w->cols); break;
        case RQ_Q8_0: rq_dequant_kernel<RQ_Q8_0><<<grid, threads, 0, s>>>(w->main, w->scale, out, count, w->cols); break;
        case RQ_Q4_0: rq_dequant_kernel<RQ_Q4_0><<<grid, threads, 0, s>>>(w->main, w->scale, out, count, w->cols); break;
#define RQ_CASE(T) case T: rq_dequant_kernel<T><<<grid, threads, 0, s>>>(w->main, w->scale, out, count, w->cols); break;
        RQ_DECODE_ONLY_TYPES(RQ_CASE)
#undef RQ_CASE
        default: return rq_fail(RQ_ERR_INVALID, "dequant: type %d", w->type);
    }
    RQ_CUDA(cudaGetLastError());
    return RQ_OK;
}

// ---------------------------------------------------------------------------------------
// Embedding-row gather from a packed table (Primitive::Gather, recipe.rs:4632-4651): position t takes row ids[t] of the
// stored table, decoded value by value with the dequantiser's arithmetic (the same bits), into y[channel * yn + t * yt].
// Ids live in device memory, so they cannot be checked before the launch: an id outside the table is clamped into it.
// ---------------------------------------------------------------------------------------
template <int TYPE>
__global__ void rq_gather_kernel(const uint8_t* __restrict__ main_plane, const uint16_t* __restrict__ scale_plane, int64_t rows, int64_t cols,
                                 const int32_t* __restrict__ ids, int tokens, float* __restrict__ y, int64_t yn, int64_t yt) {
    const int64_t total = (int64_t)tokens * cols;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / cols, k = i - t * cols;
        int64_t row = ids[t];
        row = row < 0 ? 0 : (row >= rows ? rows - 1 : row);
        y[k * yn + t * yt] = rq_decode_value<TYPE>(main_plane, scale_plane, row * cols + k, cols);
    }
}

int rq_launch_gather(const rq_weight* w, const int32_t* ids, int tokens, float* y, int64_t yn, int64_t yt, cudaStream_t s) {
    const int64_t total = (int64_t)tokens * w->cols;
    const int threads = 256;
    int64_t want = (total + threads - 1) / threads;
    const int grid = (int)(want < 148 * 16 ? (want < 1 ? 1 : want) : 148 * 16);
    switch (w->type) {
        case RQ_Q4_K: rq_gather_kernel<RQ_Q4_K><<<grid, threads, 0, s>>>(w->main, w->scale, w->rows, w->cols, ids, tokens, y, yn, yt); break;
        case RQ_Q6_K: rq_gather_kernel<RQ_Q6_K><<<grid, threads, 0, s>>>(w->main, w->scale, w->rows, w->cols, ids, tokens, y, yn, yt); break;
        case RQ_Q8_0: rq_gather_kernel<RQ_Q8_0><<<grid, threads, 0, s>>>(w->main, w->scale, w->rows, w->cols, ids, tokens, y, yn, yt); break;
        case RQ_Q4_0: rq_gather_kernel<RQ_Q4_0><<<grid, threads, 0, s>>>(w->main, w->scale, w->rows, w->cols, ids, tokens, y, yn, yt); break;
#define RQ_CASE(T) case T: rq_gather_kernel<T><<<grid, threads, 0, s>>>(w->main, w->scale, w->rows, w->cols, ids, tokens, y, yn, yt); break;
        RQ_DECODE_ONLY_TYPES(RQ_CASE)
#undef RQ_CASE
        default: return rq_fail(RQ_ERR_INVALID, "gather: type %d", w->type);
    }
    RQ_CUDA(cudaGetLastError());
    return RQ_OK;
}
