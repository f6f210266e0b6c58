// The exchange step of the sharded configs, behind the C ABI.
//
// The reference has one exchange primitive (Primitive::Exchange, recipe.rs:5344-5441, buffers
// :20412-20486): after a row split the dies' slices of a plane are gathered, after a term split the
// dies' planes are summed in die order. Here the dies are the GPUs of one node, one process each:
//
//   * rq_allgather_rows / rq_allreduce_sum run the exchange through the host's own NCCL
//     communicator (an ncclComm_t handed in as a pointer). libnccl.so.2 is looked up at run time
//     (the copy already loaded into the process, else the system's): a host that never shards
//     needs no NCCL.
//   * rq_exchange_* is the library's own exchange over NVLink peer memory: every rank owns a
//     buffer of per-rank slots that its peers map (CUDA IPC); one kernel stores this rank's slice
//     into its slot of every peer with plain peer stores, raises a flag on each peer, waits (bounded)
//     for the peers' flags and, for a sum, adds the slots in rank order -- the same bits on every
//     rank and on every run. Loads never leave the GPU, and no library kernel ever sees peer memory.
//
// The count of calls so far lives in device memory and the kernel advances it itself, so a CUDA graph that holds
// exchange launches can be replayed: nothing about a call is baked into its launch parameters.
//
// Memory order of an exchange: a rank's stores to a peer are followed by __threadfence_system()
// and a release store of the flag; the peer acquires the flag before it reads. Slots are double
// buffered by the parity of the call count, so a rank that runs ahead writes the half its peers are
// not reading; it cannot run two calls ahead, because each call waits for every peer's flag.
#include <dlfcn.h>
#include <string.h>

#include <new>

#include "rq_internal.cuh"

// ---- NCCL, bound at run time --------------------------------------------------------------------
namespace {

struct NcclId { char internal[128]; };  // ncclUniqueId
typedef int (*fn_get_unique_id)(NcclId*);
typedef int (*fn_comm_init_rank)(void**, int, NcclId, int);
typedef int (*fn_comm_destroy)(void*);
typedef int (*fn_comm_count)(void*, int*);
typedef int (*fn_comm_user_rank)(void*, int*);
typedef int (*fn_all_gather)(const void*, void*, size_t, int, void*, cudaStream_t);
typedef int (*fn_all_reduce)(const void*, void*, size_t, int, int, void*, cudaStream_t);
typedef const char* (*fn_error_string)(int);

struct Nccl {
    void* lib;
    fn_get_unique_id get_unique_id;
    fn_comm_init_rank comm_init_rank;
    fn_comm_destroy comm_destroy;
    fn_comm_count comm_count;
    fn_comm_user_rank comm_user_rank;
    fn_all_gather all_gather;
    fn_all_reduce all_reduce;
    fn_error_string error_string;
};
constexpr int kNcclFloat = 7, kNcclSum = 0;  // ncclFloat32, ncclSum

int nccl_load(const Nccl** out) {
    static Nccl n = {};
    static bool tried = false;
    if (!tried) {
        tried = true;
        // the copy the host already uses (its communicator belongs to that copy), else whatever the loader finds
        void* lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
        if (!lib) lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!lib) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (lib) {
            n.get_unique_id = (fn_get_unique_id)dlsym(lib, "ncclGetUniqueId");
            n.comm_init_rank = (fn_comm_init_rank)dlsym(lib, "ncclCommInitRank");
            n.comm_destroy = (fn_comm_destroy)dlsym(lib, "ncclCommDestroy");
            n.comm_count = (fn_comm_count)dlsym(lib, "ncclCommCount");
            n.comm_user_rank = (fn_comm_user_rank)dlsym(lib, "ncclCommUserRank");
            n.all_gather = (fn_all_gather)dlsym(lib, "ncclAllGather");
            n.all_reduce = (fn_all_reduce)dlsym(lib, "ncclAllReduce");
            n.error_string = (fn_error_string)dlsym(lib, "ncclGetErrorString");
            if (n.get_unique_id && n.comm_init_rank && n.comm_destroy && n.comm_count && n.comm_user_rank && n.all_gather && n.all_reduce && n.error_string) n.lib = lib;
        }
    }
    if (!n.lib) return rq_fail(RQ_ERR_UNSUPPORTED, "libnccl.so.2 is not loaded and cannot be found: the NCCL exchange is unavailable in this process");
    *out = &n;
    return RQ_OK;
}

int nccl_fail(const Nccl* n, const char* what, int rc) { return rq_fail(RQ_ERR_CUDA, "%s: %s", what, n->error_string(rc)); }

}  // namespace

extern "C" int rq_nccl_unique_id(void* id128) {
    if (!id128) return rq_fail(RQ_ERR_INVALID, "rq_nccl_unique_id: null argument");
    const Nccl* n;
    int rc = nccl_load(&n);
    if (rc) return rc;
    NcclId id;
    rc = n->get_unique_id(&id);
    if (rc) return nccl_fail(n, "ncclGetUniqueId", rc);
    memcpy(id128, &id, sizeof(id));
    return RQ_OK;
}

extern "C" int rq_nccl_comm_create(rq_ctx* ctx, const void* id128, int nranks, int rank, void** comm_out) {
    if (!ctx || !id128 || !comm_out) return rq_fail(RQ_ERR_INVALID, "rq_nccl_comm_create: null argument");
    if (nranks < 1 || rank < 0 || rank >= nranks) return rq_fail(RQ_ERR_INVALID, "rq_nccl_comm_create: rank %d of %d", rank, nranks);
    *comm_out = nullptr;
    const Nccl* n;
    int rc = nccl_load(&n);
    if (rc) return rc;
    DeviceGuard guard(ctx->device);
    NcclId id;
    memcpy(&id, id128, sizeof(id));
    void* comm = nullptr;
    rc = n->comm_init_rank(&comm, nranks, id, rank);
    if (rc) return nccl_fail(n, "ncclCommInitRank", rc);
    *comm_out = comm;
    return RQ_OK;
}

extern "C" void rq_nccl_comm_destroy(void* comm) {
    const Nccl* n;
    if (comm && nccl_load(&n) == RQ_OK) n->comm_destroy(comm);
}

extern "C" int rq_allgather_rows(rq_ctx* ctx, void* nccl_comm, const float* local, float* gathered, int64_t count_per_rank, void* stream) {
    if (!ctx || !nccl_comm || !local || !gathered) return rq_fail(RQ_ERR_INVALID, "rq_allgather_rows: null argument");
    if (count_per_rank <= 0) return rq_fail(RQ_ERR_INVALID, "rq_allgather_rows: count_per_rank=%lld must be positive", (long long)count_per_rank);
    const Nccl* n;
    int rc = nccl_load(&n);
    if (rc) return rc;
    DeviceGuard guard(ctx->device);
    rc = n->all_gather(local, gathered, (size_t)count_per_rank, kNcclFloat, nccl_comm, (cudaStream_t)stream);
    return rc ? nccl_fail(n, "ncclAllGather", rc) : RQ_OK;
}

extern "C" int rq_allreduce_sum(rq_ctx* ctx, void* nccl_comm, const float* local, float* summed, int64_t count, void* stream) {
    if (!ctx || !nccl_comm || !local || !summed) return rq_fail(RQ_ERR_INVALID, "rq_allreduce_sum: null argument");
    if (count <= 0) return rq_fail(RQ_ERR_INVALID, "rq_allreduce_sum: count=%lld must be positive", (long long)count);
    const Nccl* n;
    int rc = nccl_load(&n);
    if (rc) return rc;
    DeviceGuard guard(ctx->device);
    rc = n->all_reduce(local, summed, (size_t)count, kNcclFloat, kNcclSum, nccl_comm, (cudaStream_t)stream);
    return rc ? nccl_fail(n, "ncclAllReduce", rc) : RQ_OK;
}

// ---- the library's own exchange over peer memory ------------------------------------------------------

#define RQ_EXCHANGE_MAX_RANKS 16

struct rq_exchange {
    rq_ctx* ctx;
    int rank, nranks;
    int64_t slot_bytes;             // one rank's slice, rounded up to 256 bytes
    uint8_t* local;                 // [2 halves][nranks slots][slot_bytes] | flags[RQ_EXCHANGE_MAX_RANKS] | arrivals | departures | calls so far
    uint8_t* peer[RQ_EXCHANGE_MAX_RANKS];  // every rank's buffer as this process maps it (peer[rank] == local)
    bool opened[RQ_EXCHANGE_MAX_RANKS];    // mapped through cudaIpcOpenMemHandle (to be closed)
    bool connected;
};

namespace {

struct ExchangeParams {
    uint8_t* peer[RQ_EXCHANGE_MAX_RANKS];
    int rank, nranks;
    int64_t slot_bytes, half_bytes;
    const float* src; int64_t count;  // this rank's slice
    float* out;                       // gather: [nranks][count], the slots one after another; sum: [count], the slots added in rank order
    int sum;
    int* error_flag;
    unsigned long long wait_ns;
};

__device__ __forceinline__ unsigned long long ex_now() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }

// grid of G CTAs: each stores its part of the slice into this rank's slot on every rank, the last CTA to finish raises
// the flags; every CTA then waits for the peers' flags and copies out (or adds, in rank order) its part of the slots.
// Call e (counted in device memory) uses half e & 1 of the slots and the flag value e + 1.
__global__ void __launch_bounds__(256) rq_exchange_kernel(const ExchangeParams p) {
    // the launch after this one may start its own prologue (a matvec's first weight copies) while this kernel exchanges
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int tid = threadIdx.x;
    uint32_t* flags = (uint32_t*)(p.peer[p.rank] + 2 * p.half_bytes);
    unsigned int* arrivals = (unsigned int*)(flags + RQ_EXCHANGE_MAX_RANKS);
    unsigned int* departures = arrivals + 1;
    volatile uint32_t* calls = flags + RQ_EXCHANGE_MAX_RANKS + 2;
    const uint32_t epoch = *calls;  // advanced by the last CTA of the previous call to leave, which this launch waited for
    const int64_t half_off = (int64_t)(epoch & 1) * p.half_bytes, slot_off = half_off + (int64_t)p.rank * p.slot_bytes;
    // 1. this rank's slice into its slot everywhere (16-byte stores when the slice allows)
    const int64_t stride = (int64_t)gridDim.x * blockDim.x, at0 = (int64_t)blockIdx.x * blockDim.x + tid;
    const bool vec = (((uintptr_t)p.src | (uintptr_t)p.out) & 15) == 0 && (p.count & 3) == 0;
    if (vec) {
        const int64_t n4 = p.count >> 2;
        for (int64_t i = at0; i < n4; i += stride) {
            const float4 v = __ldg((const float4*)p.src + i);
            for (int r = 0; r < p.nranks; ++r) ((float4*)(p.peer[r] + slot_off))[i] = v;
        }
    } else {
        for (int64_t i = at0; i < p.count; i += stride) {
            const float v = __ldg(p.src + i);
            for (int r = 0; r < p.nranks; ++r) ((float*)(p.peer[r] + slot_off))[i] = v;
        }
    }
    // One system-scope fence per CTA, not per thread: the barrier orders the CTA's stores before thread 0's fence, and the
    // fence is cumulative, so everything the CTA stored is ordered before what thread 0 does next.
    __syncthreads();
    __shared__ bool s_last;
    if (tid == 0) {
        __threadfence_system();
        s_last = gridDim.x == 1u || atomicAdd(arrivals, 1u) == gridDim.x - 1u;
        if (s_last && gridDim.x > 1u) {
            *arrivals = 0;            // nobody adds again before the next call
            __threadfence_system();   // the other CTAs' fenced stores, seen through their arrivals, go before the flags
        }
        if (s_last) {
            // 2. every CTA's stores are out and fenced: tell each peer that this rank's slot is complete. The fence above
            // already orders the stores before these, so the flag stores themselves are relaxed (a release store would
            // pay for one more system-scope fence each).
            for (int r = 0; r < p.nranks; ++r) {
                if (r == p.rank) continue;
                uint32_t* there = (uint32_t*)(p.peer[r] + 2 * p.half_bytes) + p.rank;
                asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(there), "r"(epoch + 1u) : "memory");
            }
        }
    }
    __syncthreads();
    // 3. wait for every peer's flag of this call (bounded)
    if (tid < p.nranks && tid != p.rank) {
        unsigned long long t0 = 0;
        uint32_t seen, tries = 0;
        while (true) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flags + tid) : "memory");
            if ((int32_t)(seen - (epoch + 1u)) >= 0) break;
            if ((++tries & 63u) == 0) {  // the clock is read at every 64th look at the flag
                const unsigned long long now = ex_now();
                if (t0 == 0) t0 = now;
                else if (now - t0 > p.wait_ns) { atomicExch(p.error_flag, 31); break; }
            }
        }
    }
    __syncthreads();
    // 4. out of the slots: one after another, or their sum in rank order
    const uint8_t* mine = p.peer[p.rank] + half_off;
    if (p.sum && vec) {
        const int64_t n4 = p.count >> 2;
        for (int64_t i = at0; i < n4; i += stride) {
            float4 total = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int r = 0; r < p.nranks; ++r) {  // rank order: the same bits on every rank
                const float4 v = __ldcg((const float4*)(mine + (int64_t)r * p.slot_bytes) + i);
                total.x += v.x; total.y += v.y; total.z += v.z; total.w += v.w;
            }
            ((float4*)p.out)[i] = total;
        }
    } else if (p.sum) {
        for (int64_t i = at0; i < p.count; i += stride) {
            float total = 0.f;
            for (int r = 0; r < p.nranks; ++r) total += __ldcg((const float*)(mine + (int64_t)r * p.slot_bytes) + i);
            p.out[i] = total;
        }
    } else if (vec) {
        const int64_t n4 = p.count >> 2;
        for (int r = 0; r < p.nranks; ++r)
            for (int64_t i = at0; i < n4; i += stride) ((float4*)(p.out + (int64_t)r * p.count))[i] = __ldcg((const float4*)(mine + (int64_t)r * p.slot_bytes) + i);
    } else {
        for (int r = 0; r < p.nranks; ++r)
            for (int64_t i = at0; i < p.count; i += stride) p.out[(int64_t)r * p.count + i] = __ldcg((const float*)(mine + (int64_t)r * p.slot_bytes) + i);
    }
    // 5. the last CTA to leave advances the call count
    __syncthreads();
    if (tid == 0 && atomicAdd(departures, 1u) == gridDim.x - 1u) {
        *departures = 0;
        *calls = epoch + 1u;
        __threadfence();
    }
}

}  // namespace

extern "C" int rq_exchange_create(rq_ctx* ctx, int rank, int nranks, int64_t slot_bytes, rq_exchange** out) {
    if (!ctx || !out) return rq_fail(RQ_ERR_INVALID, "rq_exchange_create: null argument");
    *out = nullptr;
    if (nranks < 1 || nranks > RQ_EXCHANGE_MAX_RANKS || rank < 0 || rank >= nranks) return rq_fail(RQ_ERR_INVALID, "rq_exchange_create: rank %d of %d (at most %d ranks)", rank, nranks, RQ_EXCHANGE_MAX_RANKS);
    if (slot_bytes <= 0 || slot_bytes > (int64_t)1 << 32) return rq_fail(RQ_ERR_INVALID, "rq_exchange_create: slot_bytes=%lld out of range", (long long)slot_bytes);
    DeviceGuard guard(ctx->device);
    rq_exchange* ex = new (std::nothrow) rq_exchange();
    if (!ex) return rq_fail(RQ_ERR_ALLOC, "out of host memory");
    memset(ex, 0, sizeof(*ex));
    ex->ctx = ctx; ex->rank = rank; ex->nranks = nranks;
    ex->slot_bytes = (slot_bytes + 255) / 256 * 256;
    const size_t total = (size_t)2 * nranks * ex->slot_bytes + 256;
    cudaError_t e = cudaMalloc(&ex->local, total);
    if (e == cudaSuccess) e = cudaMemset(ex->local, 0, total);
    if (e != cudaSuccess) { if (ex->local) cudaFree(ex->local); delete ex; return rq_fail(RQ_ERR_ALLOC, "exchange buffer of %zu bytes: %s", total, cudaGetErrorString(e)); }
    ex->peer[rank] = ex->local;
    ex->connected = nranks == 1;
    *out = ex;
    return RQ_OK;
}

extern "C" int rq_exchange_handle(rq_exchange* ex, void* handle64) {
    if (!ex || !handle64) return rq_fail(RQ_ERR_INVALID, "rq_exchange_handle: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is passed as 64 bytes");
    DeviceGuard guard(ex->ctx->device);
    cudaIpcMemHandle_t h;
    RQ_CUDA(cudaIpcGetMemHandle(&h, ex->local));
    memcpy(handle64, &h, 64);
    return RQ_OK;
}

extern "C" void* rq_exchange_buffer(rq_exchange* ex) { return ex ? ex->local : nullptr; }

extern "C" int rq_exchange_connect(rq_exchange* ex, const void* handles, const void* const* same_process_buffers) {
    if (!ex) return rq_fail(RQ_ERR_INVALID, "rq_exchange_connect: null exchange");
    if (ex->connected) return RQ_OK;
    if (!handles && !same_process_buffers) return rq_fail(RQ_ERR_INVALID, "rq_exchange_connect: neither handles nor buffers given");
    DeviceGuard guard(ex->ctx->device);
    for (int r = 0; r < ex->nranks; ++r) {
        if (r == ex->rank) continue;
        if (same_process_buffers) {
            // ranks that share this process (one thread or context per GPU): the peers' buffers are plain pointers
            cudaPointerAttributes attr;
            RQ_CUDA(cudaPointerGetAttributes(&attr, same_process_buffers[r]));
            if (attr.device != ex->ctx->device) {
                cudaError_t e = cudaDeviceEnablePeerAccess(attr.device, 0);
                if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
                else if (e != cudaSuccess) return rq_fail(RQ_ERR_CUDA, "peer access to device %d: %s", attr.device, cudaGetErrorString(e));
            }
            ex->peer[r] = (uint8_t*)same_process_buffers[r];
        } else {
            cudaIpcMemHandle_t h;
            memcpy(&h, (const uint8_t*)handles + 64 * (size_t)r, 64);
            void* ptr = nullptr;
            cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess) return rq_fail(RQ_ERR_CUDA, "mapping rank %d's exchange buffer: %s", r, cudaGetErrorString(e));
            ex->peer[r] = (uint8_t*)ptr;
            ex->opened[r] = true;
        }
    }
    ex->connected = true;
    return RQ_OK;
}

extern "C" void rq_exchange_free(rq_exchange* ex) {
    if (!ex) return;
    DeviceGuard guard(ex->ctx->device);
    cudaDeviceSynchronize();
    for (int r = 0; r < ex->nranks; ++r)
        if (ex->opened[r] && ex->peer[r]) cudaIpcCloseMemHandle(ex->peer[r]);
    if (ex->local) cudaFree(ex->local);
    delete ex;
}

static int exchange_launch(rq_exchange* ex, const char* who, const float* local, int64_t count, float* out, int sum, void* stream) {
    if (!ex || !local || !out) return rq_fail(RQ_ERR_INVALID, "%s: null argument", who);
    if (!ex->connected) return rq_fail(RQ_ERR_INVALID, "%s: the exchange is not connected to its peers yet (rq_exchange_connect)", who);
    if (count <= 0 || count * 4 > ex->slot_bytes) return rq_fail(RQ_ERR_LIMIT, "%s: %lld floats per rank, the slots hold %lld", who, (long long)count, (long long)(ex->slot_bytes / 4));
    DeviceGuard guard(ex->ctx->device);
    ExchangeParams p;
    memset(&p, 0, sizeof(p));
    for (int r = 0; r < ex->nranks; ++r) p.peer[r] = ex->peer[r];
    p.rank = ex->rank; p.nranks = ex->nranks; p.slot_bytes = ex->slot_bytes; p.half_bytes = (int64_t)ex->nranks * ex->slot_bytes;
    p.src = local; p.count = count; p.out = out; p.sum = sum;
    p.error_flag = ex->ctx->error_flag; p.wait_ns = ex->ctx->wait_limit_ns;
    // A CTA per 4 KB of slice (one 16-byte line per thread: the push is a chain of a load and a store per line, so its time
    // is the number of lines a thread moves one after another), at most 128: every CTA must be resident while it waits for
    // the peers' flags, and 128 CTAs of 256 threads and no shared memory fit the device beside anything else that runs.
    int64_t ctas = (count * 4 + 4095) / 4096;
    if (ctas < 1) ctas = 1;
    if (ctas > 128) ctas = 128;
    if (ctas > ex->ctx->sm_count) ctas = ex->ctx->sm_count;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctas);
    cfg.blockDim = dim3(256);
    cfg.stream = (cudaStream_t)stream;
    // Launched the plain way, after the kernel before it has finished: with programmatic serialization this kernel's
    // early trigger let the launch after it (the next step's matvec, itself programmatic) start while the matvec that
    // feeds this exchange was still running, and the step measured 17 us slower (LM head share of 131072 rows, two GPUs).
    cfg.attrs = nullptr;
    cfg.numAttrs = 0;
    RQ_CUDA(cudaLaunchKernelEx(&cfg, rq_exchange_kernel, p));
    return RQ_OK;
}

extern "C" int rq_exchange_gather(rq_exchange* ex, const float* local, int64_t count, float* gathered, void* stream) {
    return exchange_launch(ex, "rq_exchange_gather", local, count, gathered, 0, stream);
}

extern "C" int rq_exchange_reduce(rq_exchange* ex, const float* local, int64_t count, float* summed, void* stream) {
    return exchange_launch(ex, "rq_exchange_reduce", local, count, summed, 1, stream);
}
