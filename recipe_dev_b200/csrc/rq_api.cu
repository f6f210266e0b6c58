// C ABI of librq_b200.so: context, weights, argument validation, error text.
// Every entry point validates, returns a status and never aborts; none has a CPU path.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <new>

#include "rq_internal.cuh"

static thread_local char g_error[512] = "";

int rq_fail(int status, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return status;
}

extern "C" const char* rq_last_error(void) { return g_error; }

extern "C" int rq_block_values(int t) {
    switch (t) {
        case RQ_Q4_0: case RQ_Q8_0: case RQ_Q4_1: case RQ_Q5_0: case RQ_Q5_1: case RQ_IQ4_NL: case RQ_Q8_1: return 32;
        case RQ_Q4_K: case RQ_Q6_K: case RQ_Q5_K: case RQ_Q2_K: case RQ_Q3_K: case RQ_Q8_K: case RQ_IQ4_XS: return 256;
        default: return 0;
    }
}
extern "C" int rq_block_bytes(int t) {
    switch (t) {
        case RQ_Q4_0: return 18;
        case RQ_Q8_0: return 34;
        case RQ_Q4_K: return 144;
        case RQ_Q6_K: return 210;
        case RQ_Q4_1: return 20;
        case RQ_Q5_0: return 22;
        case RQ_Q5_1: return 24;
        case RQ_Q5_K: return 176;
        case RQ_IQ4_NL: return 18;
        case RQ_Q8_1: return 36;
        case RQ_Q2_K: return 84;
        case RQ_Q3_K: return 110;
        case RQ_Q8_K: return 292;
        case RQ_IQ4_XS: return 136;
        default: return 0;
    }
}

extern "C" int rq_init(int device, rq_ctx** out) {
    if (!out) return rq_fail(RQ_ERR_INVALID, "rq_init: out is null");
    *out = nullptr;
    int count = 0;
    RQ_CUDA(cudaGetDeviceCount(&count));
    if (device < 0 || device >= count) return rq_fail(RQ_ERR_INVALID, "rq_init: device %d out of range (%d visible)", device, count);
    DeviceGuard guard(device);
    if (!guard.ok) return rq_fail(RQ_ERR_CUDA, "rq_init: cannot select device %d", device);
    cudaDeviceProp prop;
    RQ_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major < 10) return rq_fail(RQ_ERR_UNSUPPORTED, "rq_init: device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);
    rq_ctx* ctx = new (std::nothrow) rq_ctx();
    if (!ctx) return rq_fail(RQ_ERR_ALLOC, "rq_init: out of host memory");
    memset(ctx, 0, sizeof(*ctx));
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->wait_limit_ns = 2000000000ull;
    cudaError_t e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) { delete ctx; return rq_fail(RQ_ERR_CUDA, "cudaStreamCreate: %s", cudaGetErrorString(e)); }
    e = cudaMalloc(&ctx->error_flag, sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(ctx->error_flag, 0, sizeof(int));
    if (e == cudaSuccess) e = cudaMallocHost(&ctx->pin_flag, sizeof(int));
    if (e == cudaSuccess) *ctx->pin_flag = 0;
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ctx->work_event, cudaEventDisableTiming);
    if (e != cudaSuccess) { cudaStreamDestroy(ctx->stream); delete ctx; return rq_fail(RQ_ERR_CUDA, "error flag: %s", cudaGetErrorString(e)); }
    *out = ctx;
    return RQ_OK;
}

extern "C" void rq_destroy(rq_ctx* ctx) {
    if (!ctx) return;
    DeviceGuard guard(ctx->device);
    if (ctx->act_scratch) cudaFree(ctx->act_scratch);
    if (ctx->error_flag) cudaFree(ctx->error_flag);
    if (ctx->pin_flag) cudaFreeHost(ctx->pin_flag);
    if (ctx->stage_x) cudaFree(ctx->stage_x);
    if (ctx->stage_y) cudaFree(ctx->stage_y);
    if (ctx->pin_x) cudaFreeHost(ctx->pin_x);
    if (ctx->pin_y) cudaFreeHost(ctx->pin_y);
    if (ctx->work_event) cudaEventDestroy(ctx->work_event);
    if (ctx->stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
}

int rq_order_work_areas(rq_ctx* ctx, cudaStream_t s) {
    if (ctx->work_stream_set && ctx->work_stream != s) {
        // The previous call's kernels may still read or write the work areas on their stream: this call's stream waits
        // for everything enqueued there so far. Inside a stream capture nothing is recorded or waited for (an event
        // cannot cross a capture's boundary): calls captured into one graph must share a stream.
        cudaStreamCaptureStatus before = cudaStreamCaptureStatusNone, now = cudaStreamCaptureStatusNone;
        const bool known = cudaStreamIsCapturing(ctx->work_stream, &before) == cudaSuccess && cudaStreamIsCapturing(s, &now) == cudaSuccess;
        if (known && before == cudaStreamCaptureStatusNone && now == cudaStreamCaptureStatusNone) {
            RQ_CUDA(cudaEventRecord(ctx->work_event, ctx->work_stream));
            RQ_CUDA(cudaStreamWaitEvent(s, ctx->work_event, 0));
        } else if (!known) {
            cudaGetLastError();  // the earlier stream no longer exists: its work was finished or abandoned with it
        }
    }
    ctx->work_stream = s;
    ctx->work_stream_set = true;
    return RQ_OK;
}

static int grow_act_scratch(rq_ctx* ctx, size_t want) {
    if (ctx->recording)
        return rq_fail(RQ_ERR_INVALID, "a recorded call needs %zu bytes of work area and the context holds %zu: call rq_reserve for the widest call before rq_sequence_begin",
                       want, ctx->act_scratch_bytes);
    // the old buffer may still be read by kernels in flight
    RQ_CUDA(cudaDeviceSynchronize());
    if (ctx->act_scratch) RQ_CUDA(cudaFree(ctx->act_scratch));
    ctx->act_scratch = nullptr;
    ctx->act_scratch_bytes = 0;
    ctx->act_cols = 0;
    cudaError_t e = cudaMalloc(&ctx->act_scratch, want);
    if (e != cudaSuccess) return rq_fail(RQ_ERR_ALLOC, "activation scratch of %zu bytes: %s", want, cudaGetErrorString(e));
    ctx->act_scratch_bytes = want;
    return RQ_OK;
}

int rq_ensure_act_scratch(rq_ctx* ctx, size_t bytes, cudaStream_t s) {
    if (bytes > ctx->act_scratch_bytes) {
        // grow geometrically, so that a run of slightly wider calls does not allocate every time
        int rc = grow_act_scratch(ctx, bytes + bytes / 2 + 4096);
        if (rc) return rc;
    }
    return rq_order_work_areas(ctx, s);
}

extern "C" int rq_reserve(rq_ctx* ctx, int64_t max_rows, int64_t max_cols, int max_tokens) {
    if (!ctx) return rq_fail(RQ_ERR_INVALID, "rq_reserve: null context");
    if (max_rows <= 0 || max_cols <= 0 || max_tokens <= 0 || max_cols > (int64_t)1 << 24 || max_rows > (int64_t)1 << 31 || max_tokens > 1 << 20)
        return rq_fail(RQ_ERR_INVALID, "rq_reserve: max_rows=%lld max_cols=%lld max_tokens=%d out of range", (long long)max_rows, (long long)max_cols, max_tokens);
    DeviceGuard guard(ctx->device);
    // the int8 records of every token, or the batched product's activation image and split-K sums, whichever is larger
    const int64_t cols32 = (max_cols + 255) / 256 * 256;
    size_t want = rq_act_token_bytes(cols32) * (size_t)max_tokens;
    const size_t mm = rq_matmul_scratch_bytes(ctx, max_rows, cols32, max_tokens);
    if (mm > want) want = mm;
    if (want <= ctx->act_scratch_bytes) return RQ_OK;
    return grow_act_scratch(ctx, want);
}

static const char* wait_code_text(int code) {
    switch (code) {
        case 1: return "matvec producer: a ring slot never came free";
        case 2: return "matvec producer: a copy it issued never landed";
        case 3: return "matvec consumer: a stage never arrived";
        case 4: return "matvec producer: an earlier copy of its window never landed";
        case 11: return "batched product, staging warps: a stage never came free";
        case 12: return "batched product, drain warps: the last product never finished";
        case 13: return "batched product, issuing warp: a stage was never filled";
        case 14: return "batched product, drain warps: an accumulator never filled";
        case 15: return "batched product, issuing warp: an accumulator never came free";
        case 16: return "batched product, copy warp: a stage never came free";
        case 17: return "batched product: the activation sums never arrived";
        case 21: return "wait self-test: the barrier nothing arrives on";
        case 31: return "exchange: a peer's arrival flag never came";
        default: return "unknown wait";
    }
}

extern "C" int rq_check(rq_ctx* ctx) {
    if (!ctx) return rq_fail(RQ_ERR_INVALID, "rq_check: null context");
    DeviceGuard guard(ctx->device);
    RQ_CUDA(cudaDeviceSynchronize());
    int flag = 0;
    RQ_CUDA(cudaMemcpy(&flag, ctx->error_flag, sizeof(int), cudaMemcpyDeviceToHost));
    if (flag) {
        cudaMemset(ctx->error_flag, 0, sizeof(int));
        return rq_fail(RQ_ERR_WAIT, "a kernel gave up a bounded wait (code %d: %s); its outputs are not valid", flag, wait_code_text(flag));
    }
    return RQ_OK;
}

extern "C" int rq_set_wait_limit(rq_ctx* ctx, uint64_t nanoseconds) {
    if (!ctx) return rq_fail(RQ_ERR_INVALID, "rq_set_wait_limit: null context");
    if (nanoseconds < 1000 || nanoseconds > 60000000000ull) return rq_fail(RQ_ERR_INVALID, "rq_set_wait_limit: %llu ns is outside 1 us .. 60 s", (unsigned long long)nanoseconds);
    ctx->wait_limit_ns = nanoseconds;
    return RQ_OK;
}

// One warp waits, with the context's limit, on a barrier that nothing ever arrives on, gives up, records code 21 and
// returns: the same wait, the same give-up path and the same error word as the matvec and batched kernels use.
__global__ void rq_wait_selftest_kernel(int* error_flag, unsigned long long limit_ns) {
    __shared__ __align__(8) uint64_t bar;
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(&bar);
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(addr), "r"(1u));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long t0, now;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
        bool done = false;
        while (!done) {
            uint32_t ok;
            asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(ok) : "r"(addr), "r"(0u) : "memory");
            if (ok) break;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
            if (now - t0 > limit_ns) { atomicExch(error_flag, 21); done = true; }
        }
    }
}

extern "C" int rq_wait_selftest(rq_ctx* ctx, void* stream) {
    if (!ctx) return rq_fail(RQ_ERR_INVALID, "rq_wait_selftest: null context");
    if (ctx->wait_limit_ns > 100000000ull) return rq_fail(RQ_ERR_INVALID, "rq_wait_selftest: set a wait limit of at most 100 ms first (rq_set_wait_limit); it is %llu ns", (unsigned long long)ctx->wait_limit_ns);
    DeviceGuard guard(ctx->device);
    rq_wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(ctx->error_flag, ctx->wait_limit_ns);
    RQ_CUDA(cudaGetLastError());
    return RQ_OK;
}

// ---- weights ------------------------------------------------------------------------

static int check_shape(const char* who, int type, int64_t rows, int64_t cols) {
    int per = rq_block_values(type);
    if (!per) return rq_fail(RQ_ERR_INVALID, "%s: GGML type %d is not one of Q4_0(2) Q4_1(3) Q5_0(6) Q5_1(7) Q8_0(8) Q8_1(9) Q2_K(10) Q3_K(11) Q4_K(12) Q5_K(13) Q6_K(14) Q8_K(15) IQ4_NL(20) IQ4_XS(23)", who, type);
    if (rows <= 0 || cols <= 0) return rq_fail(RQ_ERR_INVALID, "%s: rows=%lld cols=%lld must be positive", who, (long long)rows, (long long)cols);
    if (cols % per) return rq_fail(RQ_ERR_INVALID, "%s: cols=%lld is not a multiple of the %d-value block", who, (long long)cols, per);
    if (cols > (int64_t)1 << 24 || rows > (int64_t)1 << 31) return rq_fail(RQ_ERR_LIMIT, "%s: shape %lld x %lld beyond the supported range", who, (long long)rows, (long long)cols);
    return RQ_OK;
}

static int alloc_weight(rq_ctx* ctx, int type, int64_t rows, int64_t cols, rq_weight** out) {
    rq_weight* w = new (std::nothrow) rq_weight();
    if (!w) return rq_fail(RQ_ERR_ALLOC, "out of host memory");
    memset(w, 0, sizeof(*w));
    w->type = type; w->rows = rows; w->cols = cols; w->device = ctx->device;
    int per = rq_block_values(type), bytes = rq_block_bytes(type);
    int64_t blocks = rows * (cols / per);
    // formats kept as their GGUF blocks have one plane; the others a body plane and an fp16 scale plane
    int64_t main_bytes = rq_type_keeps_blocks(type) ? blocks * bytes : blocks * (bytes - 2);
    int64_t scale_bytes = rq_type_keeps_blocks(type) ? 0 : blocks * 2;
    w->bytes = main_bytes + scale_bytes;
    // one allocation, scale plane after the main plane at a 256-byte boundary
    int64_t main_padded = (main_bytes + 255) / 256 * 256;
    uint8_t* base = nullptr;
    cudaError_t e = cudaMalloc(&base, (size_t)(main_padded + scale_bytes + 256));
    if (e != cudaSuccess) { delete w; return rq_fail(RQ_ERR_ALLOC, "weight of %lld bytes: %s", (long long)w->bytes, cudaGetErrorString(e)); }
    w->main = base;
    w->scale = scale_bytes ? (uint16_t*)(base + main_padded) : nullptr;
    *out = w;
    return RQ_OK;
}

int rq_make_tile_map(rq_weight* w) {
    w->has_tile_map = 0;
    if ((w->type != RQ_Q4_K && w->type != RQ_Q6_K) || w->cols % 256) return RQ_OK;
    typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                    CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeTiled encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult found;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &found) != cudaSuccess || found != cudaDriverEntryPointSuccess || !fn)
            return rq_fail(RQ_ERR_CUDA, "the driver does not export cuTensorMapEncodeTiled");
        encode = (EncodeTiled)fn;
    }
    const cuuint64_t unit = w->type == RQ_Q4_K ? 144 : 208, row_bytes = (cuuint64_t)(w->cols / 256) * unit;
    const cuuint64_t dims[2] = {row_bytes, (cuuint64_t)w->rows};
    const cuuint64_t strides[1] = {row_bytes};          // bytes between rows: a multiple of 16 (144 = 9 x 16, 208 = 13 x 16)
    const cuuint32_t box[2] = {(cuuint32_t)unit, 128};  // one superblock of 128 rows; rows past the end arrive as zeros
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = encode(&w->tile_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, w->main, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return rq_fail(RQ_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d for a %lld x %lld weight", (int)rc, (long long)w->rows, (long long)w->cols);
    w->has_tile_map = 1;
    return RQ_OK;
}

extern "C" void rq_weight_free(rq_ctx* ctx, rq_weight* w) {
    if (!w) return;
    DeviceGuard guard(ctx ? ctx->device : w->device);
    if (w->main) cudaFree(w->main);
    delete w;
}

extern "C" int rq_weight_prepare_device(rq_ctx* ctx, int type, const void* dev_blocks, int64_t rows, int64_t cols, rq_weight** out, void* stream) {
    if (!ctx || !dev_blocks || !out) return rq_fail(RQ_ERR_INVALID, "rq_weight_prepare_device: null argument");
    *out = nullptr;
    int rc = check_shape("rq_weight_prepare_device", type, rows, cols);
    if (rc) return rc;
    DeviceGuard guard(ctx->device);
    rq_weight* w = nullptr;
    rc = alloc_weight(ctx, type, rows, cols, &w);
    if (rc) return rc;
    rc = rq_launch_repack(w, (const uint8_t*)dev_blocks, (cudaStream_t)stream);
    if (!rc) rc = rq_make_tile_map(w);
    if (rc) { rq_weight_free(ctx, w); return rc; }
    *out = w;
    return RQ_OK;
}

extern "C" int rq_weight_prepare(rq_ctx* ctx, int type, const void* host_blocks, int64_t rows, int64_t cols,
                                 int64_t row_first, int64_t row_count, rq_weight** out) {
    if (!ctx || !host_blocks || !out) return rq_fail(RQ_ERR_INVALID, "rq_weight_prepare: null argument");
    *out = nullptr;
    int rc = check_shape("rq_weight_prepare", type, rows, cols);
    if (rc) return rc;
    if (row_first < 0 || row_count <= 0 || row_first + row_count > rows)
        return rq_fail(RQ_ERR_INVALID, "rq_weight_prepare: rows [%lld, %lld) outside the tensor's %lld rows", (long long)row_first, (long long)(row_first + row_count), (long long)rows);
    DeviceGuard guard(ctx->device);
    int64_t row_bytes = cols / rq_block_values(type) * rq_block_bytes(type);
    int64_t total = row_count * row_bytes;
    uint8_t* staging = nullptr;
    cudaError_t e = cudaMalloc(&staging, (size_t)total + 16);
    if (e != cudaSuccess) return rq_fail(RQ_ERR_ALLOC, "upload staging of %lld bytes: %s", (long long)total, cudaGetErrorString(e));
    e = cudaMemcpy(staging, (const uint8_t*)host_blocks + row_first * row_bytes, (size_t)total, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) { cudaFree(staging); return rq_fail(RQ_ERR_CUDA, "weight upload: %s", cudaGetErrorString(e)); }
    rc = rq_weight_prepare_device(ctx, type, staging, row_count, cols, out, nullptr);
    cudaError_t e2 = cudaDeviceSynchronize();
    cudaFree(staging);
    if (rc) return rc;
    if (e2 != cudaSuccess) { rq_weight_free(ctx, *out); *out = nullptr; return rq_fail(RQ_ERR_CUDA, "weight repack: %s", cudaGetErrorString(e2)); }
    return RQ_OK;
}

extern "C" int rq_weight_requantize(rq_ctx* ctx, const rq_weight* src, int target_type, rq_weight** out, void* stream) {
    if (!ctx || !src || !out) return rq_fail(RQ_ERR_INVALID, "rq_weight_requantize: null argument");
    *out = nullptr;
    if (target_type != RQ_Q8_0 && target_type != RQ_Q4_1)
        return rq_fail(RQ_ERR_UNSUPPORTED, "rq_weight_requantize: target type %d; the load kernel's encoders served are Q8_0(8), the storage of int8 sums, and Q4_1(3), that of int4 sums", target_type);
    if (src->device != ctx->device) return rq_fail(RQ_ERR_INVALID, "rq_weight_requantize: weight lives on device %d, context on %d", src->device, ctx->device);
    DeviceGuard guard(ctx->device);
    rq_weight* w = nullptr;
    int rc = alloc_weight(ctx, target_type, src->rows, src->cols, &w);
    if (rc) return rc;
    rc = target_type == RQ_Q8_0 ? rq_launch_requant_q8_0(src, w, (cudaStream_t)stream) : rq_launch_requant_q4_1(src, w, (cudaStream_t)stream);
    if (rc) { rq_weight_free(ctx, w); return rc; }
    *out = w;
    return RQ_OK;
}

extern "C" int rq_int8_keeps(int ggml_type) { return ggml_type == RQ_Q8_0 || ggml_type == RQ_Q4_K; }
extern "C" int rq_int4_keeps(int ggml_type) { return ggml_type == RQ_Q4_1; }

extern "C" int rq_weight_export(rq_ctx* ctx, const rq_weight* w, void* host_blocks) {
    if (!ctx || !w || !host_blocks) return rq_fail(RQ_ERR_INVALID, "rq_weight_export: null argument");
    DeviceGuard guard(ctx->device);
    int64_t total = w->rows * (w->cols / rq_block_values(w->type)) * rq_block_bytes(w->type);
    uint8_t* staging = nullptr;
    cudaError_t e = cudaMalloc(&staging, (size_t)total + 16);
    if (e != cudaSuccess) return rq_fail(RQ_ERR_ALLOC, "export staging: %s", cudaGetErrorString(e));
    int rc = rq_launch_export(w, staging, nullptr);
    if (!rc) {
        e = cudaMemcpy(host_blocks, staging, (size_t)total, cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) rc = rq_fail(RQ_ERR_CUDA, "export copy: %s", cudaGetErrorString(e));
    }
    cudaFree(staging);
    return rc;
}

extern "C" int64_t rq_weight_rows(const rq_weight* w) { return w ? w->rows : 0; }
extern "C" int64_t rq_weight_cols(const rq_weight* w) { return w ? w->cols : 0; }
extern "C" int rq_weight_type(const rq_weight* w) { return w ? w->type : 0; }
extern "C" int64_t rq_weight_bytes(const rq_weight* w) { return w ? w->bytes : 0; }

extern "C" int rq_dequant(rq_ctx* ctx, const rq_weight* w, float* dev_out, void* stream) {
    if (!ctx || !w || !dev_out) return rq_fail(RQ_ERR_INVALID, "rq_dequant: null argument");
    DeviceGuard guard(ctx->device);
    return rq_launch_dequant(w, dev_out, (cudaStream_t)stream);
}

extern "C" int rq_gather_rows(rq_ctx* ctx, const rq_weight* table, const int32_t* dev_ids, int tokens, float* y, int64_t y_k_stride, int64_t y_t_stride, void* stream) {
    if (!ctx || !table || !dev_ids || !y) return rq_fail(RQ_ERR_INVALID, "rq_gather_rows: null argument");
    if (table->device != ctx->device) return rq_fail(RQ_ERR_INVALID, "rq_gather_rows: table lives on device %d, context on %d", table->device, ctx->device);
    if (tokens <= 0 || y_k_stride <= 0 || (tokens > 1 && y_t_stride <= 0)) return rq_fail(RQ_ERR_INVALID, "rq_gather_rows: tokens and strides must be positive");
    DeviceGuard guard(ctx->device);
    return rq_launch_gather(table, dev_ids, tokens, y, y_k_stride, y_t_stride, (cudaStream_t)stream);
}

extern "C" int rq_quantize(rq_ctx* ctx, int type, const float* dev_values, int64_t count, void* dev_blocks, void* stream) {
    if (!ctx || !dev_values || !dev_blocks) return rq_fail(RQ_ERR_INVALID, "rq_quantize: null argument");
    int per = rq_block_values(type);
    if (!per) return rq_fail(RQ_ERR_INVALID, "rq_quantize: GGML type %d is not on this path", type);
    if (count <= 0 || count % per) return rq_fail(RQ_ERR_INVALID, "rq_quantize: count=%lld is not a positive multiple of %d", (long long)count, per);
    DeviceGuard guard(ctx->device);
    return rq_launch_quantize(type, dev_values, count, (uint8_t*)dev_blocks, (cudaStream_t)stream);
}

// ---- matvec ---------------------------------------------------------------------------

static int check_matvec(const char* who, const rq_ctx* ctx, const rq_weight* w, const void* x, const void* y, int tokens, int act_mode, int step) {
    if (!ctx || !w || !x || !y) return rq_fail(RQ_ERR_INVALID, "%s: null argument", who);
    if (w->device != ctx->device) return rq_fail(RQ_ERR_INVALID, "%s: weight lives on device %d, context on %d", who, w->device, ctx->device);
    if (tokens <= 0) return rq_fail(RQ_ERR_INVALID, "%s: tokens=%d must be positive", who, tokens);
    if (act_mode != RQ_ACT_FLOAT && act_mode != RQ_ACT_INT8 && act_mode != RQ_ACT_INT8_CACHED)
        return rq_fail(RQ_ERR_INVALID, "%s: act_mode=%d is none of FLOAT(0), INT8(1), INT8_CACHED(2)", who, act_mode);
    if (act_mode != RQ_ACT_FLOAT && step != 32 && step != 256) return rq_fail(RQ_ERR_INVALID, "%s: int8 step=%d must be 32 or 256", who, step);
    return RQ_OK;
}

extern "C" int rq_matvec(rq_ctx* ctx, const rq_weight* w, const float* x, int64_t sk, int64_t st, int tokens,
                         float* y, int64_t yn, int64_t yt, int act_mode, int step, void* stream) {
    int rc = check_matvec("rq_matvec", ctx, w, x, y, tokens, act_mode, step);
    if (rc) return rc;
    if (sk <= 0 || yn <= 0 || (tokens > 1 && (st <= 0 || yt <= 0))) return rq_fail(RQ_ERR_INVALID, "rq_matvec: strides must be positive");
    DeviceGuard guard(ctx->device);
    return rq_launch_gemv(ctx, w, x, sk, st, tokens, y, yn, yt, act_mode, step, (cudaStream_t)stream);
}

extern "C" int rq_matvec_multi(rq_ctx* ctx, int n, const rq_weight* const* ws, const float* x, int64_t sk, int64_t st, int tokens,
                               float* const* ys, int64_t yn, int64_t yt, int act_mode, int step, void* stream) {
    if (!ctx || !ws || !ys || n < 1) return rq_fail(RQ_ERR_INVALID, "rq_matvec_multi: null argument or no matrices");
    if (n > 16) return rq_fail(RQ_ERR_LIMIT, "rq_matvec_multi: %d matrices, at most 16", n);
    for (int i = 0; i < n; ++i) {
        int rc = check_matvec("rq_matvec_multi", ctx, ws[i], x, ys[i], tokens, act_mode, step);
        if (rc) return rc;
        if (ws[i]->type != ws[0]->type || ws[i]->cols != ws[0]->cols)
            return rq_fail(RQ_ERR_INVALID, "rq_matvec_multi: matrix %d differs from matrix 0 in format or width (they must read one activation column)", i);
    }
    if (sk <= 0 || yn <= 0 || (tokens > 1 && (st <= 0 || yt <= 0))) return rq_fail(RQ_ERR_INVALID, "rq_matvec_multi: strides must be positive");
    DeviceGuard guard(ctx->device);
    return rq_launch_gemv_multi(ctx, n, ws, x, sk, st, tokens, ys, yn, yt, act_mode, step, (cudaStream_t)stream);
}

extern "C" int rq_matmul(rq_ctx* ctx, const rq_weight* w, const float* x, int64_t sk, int64_t st, int tokens,
                         float* y, int64_t yn, int64_t yt, int act_mode, int step, void* stream) {
    int rc = check_matvec("rq_matmul", ctx, w, x, y, tokens, act_mode, step);
    if (rc) return rc;
    if (sk <= 0 || yn <= 0 || (tokens > 1 && (st <= 0 || yt <= 0))) return rq_fail(RQ_ERR_INVALID, "rq_matmul: strides must be positive");
    DeviceGuard guard(ctx->device);
    // K-quant weights: the integer-operand tensor-core kernel, for fp32 activations and for int8 windows of twelve and more
    // positions (measured: below that the matvec kernel's exact integer dots, four tokens a pass, are faster)
    if (act_mode == RQ_ACT_FLOAT || (act_mode == RQ_ACT_INT8 && tokens >= 12)) {
        rc = rq_launch_matmul_kq(ctx, w, x, sk, st, tokens, y, yn, yt, act_mode, step, (cudaStream_t)stream);
        if (rc != RQ_ERR_UNSUPPORTED) return rc;
    }
    if (act_mode == RQ_ACT_FLOAT) {
        rc = rq_launch_matmul(ctx, w, x, sk, st, tokens, y, yn, yt, (cudaStream_t)stream);
        if (rc != RQ_ERR_UNSUPPORTED) return rc;
    }
    // int8 activations over the 32-value formats and odd widths go through the matvec kernels, four tokens a pass
    return rq_launch_gemv(ctx, w, x, sk, st, tokens, y, yn, yt, act_mode, step, (cudaStream_t)stream);
}

// Host planes <-> the token-major pinned staging buffer: one memcpy per token when the plane's elements are adjacent.
static void gather_plane(float* dst, const float* src, int64_t n, int tokens, int64_t sn, int64_t st) {
    for (int t = 0; t < tokens; ++t) {
        if (sn == 1) memcpy(dst + (size_t)t * n, src + (int64_t)t * st, (size_t)n * 4);
        else for (int64_t k = 0; k < n; ++k) dst[(size_t)t * n + k] = src[k * sn + t * st];
    }
}
static void scatter_plane(float* dst, const float* src, int64_t n, int64_t src_token_stride, int tokens, int64_t sn, int64_t st) {
    for (int t = 0; t < tokens; ++t) {
        if (sn == 1) memcpy(dst + (int64_t)t * st, src + (size_t)t * src_token_stride, (size_t)n * 4);
        else for (int64_t k = 0; k < n; ++k) dst[k * sn + t * st] = src[(size_t)t * src_token_stride + k];
    }
}

static int ensure_buffer(float** dev, size_t* dev_bytes, float** pin, size_t* pin_bytes, size_t need) {
    if (need > *dev_bytes) {
        if (*dev) cudaFree(*dev);
        *dev = nullptr; *dev_bytes = 0;
        RQ_CUDA(cudaMalloc(dev, need));
        *dev_bytes = need;
    }
    if (need > *pin_bytes) {
        if (*pin) cudaFreeHost(*pin);
        *pin = nullptr; *pin_bytes = 0;
        RQ_CUDA(cudaMallocHost(pin, need));
        *pin_bytes = need;
    }
    return RQ_OK;
}

extern "C" int rq_matvec_host(rq_ctx* ctx, const rq_weight* w, const float* host_x, int64_t sk, int64_t st, int tokens,
                              float* host_y, int64_t yn, int64_t yt, int act_mode, int step) {
    int rc = check_matvec("rq_matvec_host", ctx, w, host_x, host_y, tokens, act_mode, step);
    if (rc) return rc;
    if (sk <= 0 || yn <= 0 || (tokens > 1 && (st <= 0 || yt <= 0))) return rq_fail(RQ_ERR_INVALID, "rq_matvec_host: strides must be positive");
    DeviceGuard guard(ctx->device);
    // The host planes are gathered token-major into pinned memory, so one copy moves them.
    size_t xb = (size_t)tokens * (size_t)w->cols * 4, yb = (size_t)tokens * (size_t)w->rows * 4;
    rc = ensure_buffer(&ctx->stage_x, &ctx->stage_x_bytes, &ctx->pin_x, &ctx->pin_x_bytes, xb);
    if (rc) return rc;
    rc = ensure_buffer(&ctx->stage_y, &ctx->stage_y_bytes, &ctx->pin_y, &ctx->pin_y_bytes, yb);
    if (rc) return rc;
    gather_plane(ctx->pin_x, host_x, w->cols, tokens, sk, st);
    RQ_CUDA(cudaMemcpyAsync(ctx->stage_x, ctx->pin_x, xb, cudaMemcpyHostToDevice, ctx->stream));
    rc = rq_launch_gemv(ctx, w, ctx->stage_x, 1, w->cols, tokens, ctx->stage_y, 1, w->rows, act_mode, step, ctx->stream);
    if (rc) return rc;
    RQ_CUDA(cudaMemcpyAsync(ctx->pin_y, ctx->stage_y, yb, cudaMemcpyDeviceToHost, ctx->stream));
    RQ_CUDA(cudaMemcpyAsync(ctx->pin_flag, ctx->error_flag, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    RQ_CUDA(cudaStreamSynchronize(ctx->stream));
    if (*ctx->pin_flag) return rq_check(ctx);
    scatter_plane(host_y, ctx->pin_y, w->rows, w->rows, tokens, yn, yt);
    return RQ_OK;
}

extern "C" int rq_matvec_multi_host(rq_ctx* ctx, int n, const rq_weight* const* ws, const float* host_x, int64_t sk, int64_t st, int tokens,
                                    float* const* host_ys, int64_t yn, int64_t yt, int act_mode, int step) {
    if (!ctx || !ws || !host_ys || n < 1) return rq_fail(RQ_ERR_INVALID, "rq_matvec_multi_host: null argument or no matrices");
    if (n > 16) return rq_fail(RQ_ERR_LIMIT, "rq_matvec_multi_host: %d matrices, at most 16", n);
    int64_t total_rows = 0;
    for (int i = 0; i < n; ++i) {
        int rc = check_matvec("rq_matvec_multi_host", ctx, ws[i], host_x, host_ys[i], tokens, act_mode, step);
        if (rc) return rc;
        if (ws[i]->type != ws[0]->type || ws[i]->cols != ws[0]->cols)
            return rq_fail(RQ_ERR_INVALID, "rq_matvec_multi_host: matrix %d differs from matrix 0 in format or width (they must read one activation column)", i);
        total_rows += ws[i]->rows;
    }
    if (sk <= 0 || yn <= 0 || (tokens > 1 && (st <= 0 || yt <= 0))) return rq_fail(RQ_ERR_INVALID, "rq_matvec_multi_host: strides must be positive");
    DeviceGuard guard(ctx->device);
    const int64_t cols = ws[0]->cols;
    // x token-major in pinned memory; the outputs as one [tokens, all rows] plane, matrix i at its row offset
    size_t xb = (size_t)tokens * (size_t)cols * 4, yb = (size_t)tokens * (size_t)total_rows * 4;
    int rc = ensure_buffer(&ctx->stage_x, &ctx->stage_x_bytes, &ctx->pin_x, &ctx->pin_x_bytes, xb);
    if (rc) return rc;
    rc = ensure_buffer(&ctx->stage_y, &ctx->stage_y_bytes, &ctx->pin_y, &ctx->pin_y_bytes, yb);
    if (rc) return rc;
    gather_plane(ctx->pin_x, host_x, cols, tokens, sk, st);
    RQ_CUDA(cudaMemcpyAsync(ctx->stage_x, ctx->pin_x, xb, cudaMemcpyHostToDevice, ctx->stream));
    float* dev_ys[16];
    int64_t at = 0;
    for (int i = 0; i < n; ++i) { dev_ys[i] = ctx->stage_y + at; at += ws[i]->rows; }
    rc = rq_launch_gemv_multi(ctx, n, ws, ctx->stage_x, 1, cols, tokens, dev_ys, 1, total_rows, act_mode, step, ctx->stream);
    if (rc) return rc;
    RQ_CUDA(cudaMemcpyAsync(ctx->pin_y, ctx->stage_y, yb, cudaMemcpyDeviceToHost, ctx->stream));
    RQ_CUDA(cudaMemcpyAsync(ctx->pin_flag, ctx->error_flag, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    RQ_CUDA(cudaStreamSynchronize(ctx->stream));
    if (*ctx->pin_flag) return rq_check(ctx);
    at = 0;
    for (int i = 0; i < n; ++i) {
        scatter_plane(host_ys[i], ctx->pin_y + at, ws[i]->rows, total_rows, tokens, yn, yt);
        at += ws[i]->rows;
    }
    return RQ_OK;
}

extern "C" int rq_quantize_activations(rq_ctx* ctx, const float* x, int64_t sk, int64_t st, int64_t cols, int tokens,
                                       int step, void* dev_records, void* stream) {
    if (!ctx || !x || !dev_records) return rq_fail(RQ_ERR_INVALID, "rq_quantize_activations: null argument");
    if (cols <= 0 || cols % 32) return rq_fail(RQ_ERR_INVALID, "rq_quantize_activations: cols=%lld is not a positive multiple of 32", (long long)cols);
    if (step != 32 && step != 256) return rq_fail(RQ_ERR_INVALID, "rq_quantize_activations: step=%d must be 32 or 256", step);
    if (tokens <= 0 || sk <= 0) return rq_fail(RQ_ERR_INVALID, "rq_quantize_activations: tokens and strides must be positive");
    DeviceGuard guard(ctx->device);
    int rc = rq_ensure_act_scratch(ctx, rq_act_token_bytes(cols) * (size_t)tokens, (cudaStream_t)stream);
    if (rc) return rc;
    rc = rq_launch_act_quant(x, sk, st, cols, tokens, step, ctx->act_scratch, (uint8_t*)dev_records, (cudaStream_t)stream);
    if (rc) return rc;
    ctx->act_cols = cols; ctx->act_tokens = tokens; ctx->act_step = step;
    return RQ_OK;
}

// ---- recorded sequences: one boundary crossing per step ----------------------------------------------

// Host <-> device planes of a recorded sequence, moved by a kernel rather than by the copy engines: the host buffer is pinned
// and mapped, one CTA reads (or writes) it across the bus, and the move is one more kernel of the same submission.
__global__ void __launch_bounds__(256) rq_plane_move_kernel(const float* __restrict__ src, float* __restrict__ dst, int64_t n, const int* flag_src, int* flag_dst) {
    const int64_t n4 = (((uintptr_t)src | (uintptr_t)dst) & 15) == 0 ? n >> 2 : 0;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) ((float4*)dst)[i] = ((const float4*)src)[i];
    for (int64_t i = 4 * n4 + blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) dst[i] = src[i];
    if (flag_src && blockIdx.x == 0 && threadIdx.x == 0) *flag_dst = *flag_src;
}

struct rq_sequence {
    rq_ctx* ctx;
    cudaGraph_t graph;
    cudaGraphExec_t exec;
    // rq_sequence_run_host: the copy in, the recorded calls, the copy out and the error word as ONE graph over the sequence's
    // own pinned buffers, built at the first call and rebuilt when the call's pointers or sizes change
    cudaGraphExec_t host_exec;
    float* pin_in; float* pin_out; size_t pin_in_bytes, pin_out_bytes;
    float* host_dev_in; const float* host_dev_out; int64_t host_in_floats, host_out_floats;
};

extern "C" int rq_device_alloc(rq_ctx* ctx, int64_t bytes, void** out) {
    if (!ctx || !out || bytes <= 0) return rq_fail(RQ_ERR_INVALID, "rq_device_alloc: null argument or no bytes");
    DeviceGuard guard(ctx->device);
    cudaError_t e = cudaMalloc(out, (size_t)bytes);
    if (e != cudaSuccess) { *out = nullptr; return rq_fail(RQ_ERR_ALLOC, "device buffer of %lld bytes: %s", (long long)bytes, cudaGetErrorString(e)); }
    return RQ_OK;
}
extern "C" void rq_device_free(rq_ctx* ctx, void* ptr) {
    if (!ctx || !ptr) return;
    DeviceGuard guard(ctx->device);
    cudaFree(ptr);
}

extern "C" int rq_sequence_begin(rq_ctx* ctx, void** stream_out) {
    if (!ctx || !stream_out) return rq_fail(RQ_ERR_INVALID, "rq_sequence_begin: null argument");
    if (ctx->recording) return rq_fail(RQ_ERR_INVALID, "rq_sequence_begin: the context is already recording");
    DeviceGuard guard(ctx->device);
    RQ_CUDA(cudaStreamSynchronize(ctx->stream));
    RQ_CUDA(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
    ctx->recording = true;
    ctx->work_stream = ctx->stream;  // the recorded calls share this stream: no event is needed between them
    ctx->work_stream_set = true;
    *stream_out = ctx->stream;
    return RQ_OK;
}

extern "C" int rq_sequence_end(rq_ctx* ctx, rq_sequence** out) {
    if (!ctx || !out) return rq_fail(RQ_ERR_INVALID, "rq_sequence_end: null argument");
    *out = nullptr;
    if (!ctx->recording) return rq_fail(RQ_ERR_INVALID, "rq_sequence_end: the context is not recording");
    DeviceGuard guard(ctx->device);
    ctx->recording = false;
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
    if (e != cudaSuccess || !graph) { cudaGetLastError(); return rq_fail(RQ_ERR_CUDA, "the recording was invalidated (a recorded call failed or did something a recording cannot hold): %s", cudaGetErrorString(e)); }
    rq_sequence* seq = new (std::nothrow) rq_sequence();
    if (!seq) { cudaGraphDestroy(graph); return rq_fail(RQ_ERR_ALLOC, "out of host memory"); }
    memset(seq, 0, sizeof(*seq));
    seq->ctx = ctx; seq->graph = graph; seq->exec = nullptr;
    e = cudaGraphInstantiate(&seq->exec, graph, 0);
    if (e != cudaSuccess) { cudaGraphDestroy(graph); delete seq; return rq_fail(RQ_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(e)); }
    e = cudaGraphUpload(seq->exec, ctx->stream);  // so that the first run is not the one that pays for the upload
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) { cudaGraphExecDestroy(seq->exec); cudaGraphDestroy(graph); delete seq; return rq_fail(RQ_ERR_CUDA, "cudaGraphUpload: %s", cudaGetErrorString(e)); }
    *out = seq;
    return RQ_OK;
}

extern "C" void rq_sequence_free(rq_sequence* seq) {
    if (!seq) return;
    DeviceGuard guard(seq->ctx->device);
    cudaStreamSynchronize(seq->ctx->stream);
    if (seq->host_exec) cudaGraphExecDestroy(seq->host_exec);
    if (seq->exec) cudaGraphExecDestroy(seq->exec);
    if (seq->graph) cudaGraphDestroy(seq->graph);
    if (seq->pin_in) cudaFreeHost(seq->pin_in);
    if (seq->pin_out) cudaFreeHost(seq->pin_out);
    delete seq;
}

extern "C" int rq_sequence_run(rq_sequence* seq, void* stream) {
    if (!seq) return rq_fail(RQ_ERR_INVALID, "rq_sequence_run: null sequence");
    DeviceGuard guard(seq->ctx->device);
    int rc = rq_order_work_areas(seq->ctx, (cudaStream_t)stream);
    if (rc) return rc;
    RQ_CUDA(cudaGraphLaunch(seq->exec, (cudaStream_t)stream));
    return RQ_OK;
}

extern "C" int rq_sequence_run_host(rq_sequence* seq, const float* host_in, float* dev_in, int64_t in_floats, const float* dev_out, float* host_out, int64_t out_floats) {
    if (!seq || !host_in || !dev_in || !dev_out || !host_out) return rq_fail(RQ_ERR_INVALID, "rq_sequence_run_host: null argument");
    if (in_floats <= 0 || out_floats <= 0) return rq_fail(RQ_ERR_INVALID, "rq_sequence_run_host: in_floats and out_floats must be positive");
    rq_ctx* ctx = seq->ctx;
    DeviceGuard guard(ctx->device);
    const size_t ib = (size_t)in_floats * 4, ob = (size_t)out_floats * 4;
    if (!seq->host_exec || seq->host_dev_in != dev_in || seq->host_dev_out != dev_out || seq->host_in_floats != in_floats || seq->host_out_floats != out_floats) {
        // (re)build the one-submission graph: pinned x -> dev_in, the recorded calls, dev_out -> pinned y and the error word
        RQ_CUDA(cudaStreamSynchronize(ctx->stream));
        if (seq->host_exec) { cudaGraphExecDestroy(seq->host_exec); seq->host_exec = nullptr; }
        if (ib > seq->pin_in_bytes) { if (seq->pin_in) cudaFreeHost(seq->pin_in); seq->pin_in = nullptr; seq->pin_in_bytes = 0; RQ_CUDA(cudaMallocHost(&seq->pin_in, ib)); seq->pin_in_bytes = ib; }
        if (ob > seq->pin_out_bytes) { if (seq->pin_out) cudaFreeHost(seq->pin_out); seq->pin_out = nullptr; seq->pin_out_bytes = 0; RQ_CUDA(cudaMallocHost(&seq->pin_out, ob)); seq->pin_out_bytes = ob; }
        RQ_CUDA(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
        const unsigned in_ctas = (unsigned)((in_floats + 4095) / 4096 < 8 ? (in_floats + 4095) / 4096 : 8), out_ctas = (unsigned)((out_floats + 4095) / 4096 < 8 ? (out_floats + 4095) / 4096 : 8);
        rq_plane_move_kernel<<<in_ctas, 256, 0, ctx->stream>>>(seq->pin_in, dev_in, in_floats, nullptr, nullptr);
        cudaError_t e = cudaGetLastError();
        cudaGraphNode_t child = nullptr;
        if (e == cudaSuccess) {
            // the recorded calls as a child graph, after whatever the capture holds so far
            cudaStreamCaptureStatus status;
            cudaGraph_t capturing = nullptr;
            const cudaGraphNode_t* deps = nullptr;
            size_t n_deps = 0;
            e = cudaStreamGetCaptureInfo(ctx->stream, &status, nullptr, &capturing, &deps, &n_deps);
            if (e == cudaSuccess) e = cudaGraphAddChildGraphNode(&child, capturing, deps, n_deps, seq->graph);
            if (e == cudaSuccess) e = cudaStreamUpdateCaptureDependencies(ctx->stream, &child, 1, cudaStreamSetCaptureDependencies);
        }
        if (e == cudaSuccess) {
            rq_plane_move_kernel<<<out_ctas, 256, 0, ctx->stream>>>(dev_out, seq->pin_out, out_floats, ctx->error_flag, ctx->pin_flag);
            e = cudaGetLastError();
        }
        cudaGraph_t whole = nullptr;
        const cudaError_t e_end = cudaStreamEndCapture(ctx->stream, &whole);
        if (e != cudaSuccess || e_end != cudaSuccess || !whole) {
            cudaGetLastError();
            if (whole) cudaGraphDestroy(whole);
            return rq_fail(RQ_ERR_CUDA, "building the one-submission graph: %s", cudaGetErrorString(e != cudaSuccess ? e : e_end));
        }
        e = cudaGraphInstantiate(&seq->host_exec, whole, 0);
        cudaGraphDestroy(whole);
        if (e != cudaSuccess) { seq->host_exec = nullptr; return rq_fail(RQ_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(e)); }
        e = cudaGraphUpload(seq->host_exec, ctx->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess) return rq_fail(RQ_ERR_CUDA, "cudaGraphUpload: %s", cudaGetErrorString(e));
        seq->host_dev_in = dev_in; seq->host_dev_out = dev_out; seq->host_in_floats = in_floats; seq->host_out_floats = out_floats;
    }
    memcpy(seq->pin_in, host_in, ib);
    int rc = rq_order_work_areas(ctx, ctx->stream);
    if (rc) return rc;
    RQ_CUDA(cudaGraphLaunch(seq->host_exec, ctx->stream));
    RQ_CUDA(cudaStreamSynchronize(ctx->stream));
    if (*ctx->pin_flag) return rq_check(ctx);
    memcpy(host_out, seq->pin_out, ob);
    return RQ_OK;
}
