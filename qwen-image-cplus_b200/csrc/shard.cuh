// Column (N) sharding of a packed linear over the GPUs of one box: rank r of R holds weight rows
// [r*N/R, (r+1)*N/R) (codes, scales, minimums are row-major per output, so a shard is a contiguous
// slice of each region), computes y[:, r*N/R:(r+1)*N/R] with the ordinary kernels, and the slices
// are all-gathered over NVLink with NCCL. The reference is single-GPU (runtime.cu:6-19 uses device
// 0 only); this is new work with no counterpart there.
//
// The W4A4 linear has a second form without the all-gather: every rank holds the whole [m, N]
// output, the ranks map one another's copy (CUDA IPC, qi_shard_peer_export / _open), and the GEMM's
// epilogue stores its slice into every copy itself (qi_w4a4_gemm_wide_scatter_ex). What is left of
// the collective is qi_shard_barrier: a kernel's stores are complete when it ends, so once every
// rank has passed a barrier placed after its GEMM in stream order, every copy is whole.
//
// One process per GPU. NCCL is not linked: it is looked up at run time (dlopen), so that a process
// that already carries an NCCL (a PyTorch process, for instance) shares that copy and a
// single-GPU user of this library needs none at all.
#pragma once
#include <dlfcn.h>

#include <mutex>

#include "../../include/qipack_b200.h"

namespace qi {
namespace shard {

constexpr int NCCL_ERROR_BASE = 10000;  // returned as NCCL_ERROR_BASE + ncclResult_t
constexpr int NCCL_MISSING = 10100;     // no libnccl could be loaded
constexpr int NCCL_UINT8 = 1, NCCL_FLOAT16 = 6, NCCL_FLOAT32 = 7;  // ncclDataType_t values (nccl.h)

struct UniqueId {
    char internal[QI_SHARD_ID_BYTES];
};

struct Nccl {
    void *handle = nullptr;
    int (*GetUniqueId)(UniqueId *) = nullptr;
    int (*CommInitRank)(void **, int, UniqueId, int) = nullptr;
    int (*CommDestroy)(void *) = nullptr;
    int (*CommAbort)(void *) = nullptr;
    int (*AllGather)(const void *, void *, size_t, int, void *, cudaStream_t) = nullptr;
    int (*AllReduce)(const void *, void *, size_t, int, int, void *, cudaStream_t) = nullptr;
    int (*ReduceScatter)(const void *, void *, size_t, int, int, void *, cudaStream_t) = nullptr;
    bool ok() const { return handle && GetUniqueId && CommInitRank && CommDestroy && AllGather; }
};

inline Nccl &nccl() {
    static Nccl api;
    static std::once_flag once;
    std::call_once(once, [] {
        const char *override_path = getenv("QI_NCCL_LIBRARY");
        const char *candidates[] = {override_path, "libnccl.so.2", "libnccl.so"};
        for (const char *name : candidates) {
            if (name == nullptr) continue;
            api.handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
            if (api.handle != nullptr) break;
        }
        if (api.handle != nullptr) {
            api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(api.handle, "ncclGetUniqueId"));
            api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(api.handle, "ncclCommInitRank"));
            api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(api.handle, "ncclCommDestroy"));
            api.CommAbort = reinterpret_cast<decltype(api.CommAbort)>(dlsym(api.handle, "ncclCommAbort"));
            api.AllGather = reinterpret_cast<decltype(api.AllGather)>(dlsym(api.handle, "ncclAllGather"));
            api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(dlsym(api.handle, "ncclAllReduce"));
            api.ReduceScatter = reinterpret_cast<decltype(api.ReduceScatter)>(dlsym(api.handle, "ncclReduceScatter"));
        }
    });
    return api;
}

constexpr int PUT_LANES = 4;

struct Context {
    uint32_t magic;
    int rank, ranks, device;
    void *comm;
    float *token;  // four bytes for the barrier's all-reduce
    // qi_shard_put_slice spreads its copies over these streams, so that several copy engines work at once
    int lanes_made, joins_made;
    bool fork_made;
    cudaStream_t lanes[PUT_LANES];
    cudaEvent_t fork, joins[PUT_LANES];
};

// Everything a context owns besides the communicator is made when it is created (nothing is allocated by the
// calls that run on a stream) and taken down here, whatever part of it exists.
inline void release(Context *c) {
    if (c->token != nullptr) cudaFree(c->token);
    for (int i = 0; i < c->lanes_made; ++i) cudaStreamDestroy(c->lanes[i]);
    for (int i = 0; i < c->joins_made; ++i) cudaEventDestroy(c->joins[i]);
    if (c->fork_made) cudaEventDestroy(c->fork);
    c->token = nullptr, c->lanes_made = c->joins_made = 0, c->fork_made = false;
}

inline cudaError_t equip(Context *c) {
    cudaError_t error = cudaMalloc(&c->token, sizeof(float));
    if (error == cudaSuccess) error = cudaMemset(c->token, 0, sizeof(float));
    for (int i = 0; i < PUT_LANES && error == cudaSuccess; ++i) {
        error = cudaStreamCreateWithFlags(&c->lanes[i], cudaStreamNonBlocking);
        if (error == cudaSuccess) c->lanes_made = i + 1, error = cudaEventCreateWithFlags(&c->joins[i], cudaEventDisableTiming);
        if (error == cudaSuccess) c->joins_made = i + 1;
    }
    if (error == cudaSuccess) error = cudaEventCreateWithFlags(&c->fork, cudaEventDisableTiming);
    if (error == cudaSuccess) c->fork_made = true;
    return error;
}

typedef CUresult (*AddressRange)(CUdeviceptr *, size_t *, CUdeviceptr);

inline AddressRange address_range() {
    static AddressRange function = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *entry = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &entry, cudaEnableDefault, &result) == cudaSuccess &&
            result == cudaDriverEntryPointSuccess)
            function = reinterpret_cast<AddressRange>(entry);
    });
    return function;
}
static_assert(sizeof(cudaIpcMemHandle_t) == QI_SHARD_PEER_HANDLE_BYTES, "size of an exported handle");
constexpr uint32_t CONTEXT_MAGIC = 0x51495348;  // "QISH"

inline Context *checked(void *context) {
    Context *c = static_cast<Context *>(context);
    return (c != nullptr && c->magic == CONTEXT_MAGIC) ? c : nullptr;
}

// Rows of an [n, ...] weight that rank `rank` of `ranks` owns. Every shard must itself be a legal
// GEMM (a multiple of 128 output rows), so n must divide into ranks * 128.
inline int plan(int n, int ranks, int rank, int *first_row, int *row_count) {
    if (n <= 0 || ranks <= 0 || rank < 0 || rank >= ranks) return static_cast<int>(cudaErrorInvalidValue);
    if (n % ranks != 0 || (n / ranks) % 128 != 0) return static_cast<int>(cudaErrorInvalidValue);
    if (first_row) *first_row = rank * (n / ranks);
    if (row_count) *row_count = n / ranks;
    return 0;
}

// Input columns of an [n, k] weight that rank `rank` of `ranks` owns when the linear is split along K (row-parallel).
// A slice must hold whole quantisation groups, and for scheme 6 whole 256-input Hadamard blocks, so that rotating
// and quantising a slice of the activations gives the same codes as slicing the unsharded ones.
inline int plan_inputs(int k, int scheme, int ranks, int rank, int *first_input, int *input_count) {
    if (k <= 0 || ranks <= 0 || rank < 0 || rank >= ranks) return static_cast<int>(cudaErrorInvalidValue);
    const int unit = scheme == QI_SCHEME_W4A4_H256 ? 256 : (scheme == QI_SCHEME_W4A16 ? 64 : 0);
    if (unit == 0 || k % ranks != 0 || (k / ranks) % unit != 0) return static_cast<int>(cudaErrorInvalidValue);
    if (first_input) *first_input = rank * (k / ranks);
    if (input_count) *input_count = k / ranks;
    return 0;
}

}  // namespace shard
}  // namespace qi

extern "C" {

int qi_shard_plan(int n, int ranks, int rank, int *first_row, int *row_count) {
    return qi::shard::plan(n, ranks, rank, first_row, row_count);
}

int qi_shard_unique_id(void *id) {
    using namespace qi::shard;
    if (id == nullptr) return static_cast<int>(cudaErrorInvalidValue);
    Nccl &api = nccl();
    if (!api.ok()) return NCCL_MISSING;
    const int result = api.GetUniqueId(static_cast<UniqueId *>(id));
    return result == 0 ? 0 : NCCL_ERROR_BASE + result;
}

int qi_shard_create(void **context, int rank, int ranks, const void *id) {
    using namespace qi::shard;
    if (context == nullptr || id == nullptr || ranks < 1 || rank < 0 || rank >= ranks)
        return static_cast<int>(cudaErrorInvalidValue);
    *context = nullptr;
    Nccl &api = nccl();
    if (!api.ok()) return NCCL_MISSING;
    int device = 0;
    cudaError_t error = cudaGetDevice(&device);
    if (error != cudaSuccess) return static_cast<int>(error);
    Context *c = new Context{};
    c->magic = CONTEXT_MAGIC, c->rank = rank, c->ranks = ranks, c->device = device;
    UniqueId unique;
    memcpy(&unique, id, sizeof(unique));
    const int result = api.CommInitRank(&c->comm, ranks, unique, rank);
    if (result != 0) {
        delete c;
        return NCCL_ERROR_BASE + result;
    }
    if (ranks > 1) {
        error = equip(c);
        if (error != cudaSuccess) {
            release(c);
            if (api.CommAbort != nullptr) api.CommAbort(c->comm);
            else api.CommDestroy(c->comm);
            delete c;
            return static_cast<int>(error);
        }
    }
    *context = c;
    return 0;
}

int qi_shard_destroy(void *context) {
    using namespace qi::shard;
    Context *c = checked(context);
    if (c == nullptr) return static_cast<int>(cudaErrorInvalidValue);
    const int result = c->comm ? nccl().CommDestroy(c->comm) : 0;
    release(c);
    c->magic = 0;
    delete c;
    return result == 0 ? 0 : NCCL_ERROR_BASE + result;
}

int qi_shard_rank(void *context, int *rank, int *ranks) {
    using namespace qi::shard;
    Context *c = checked(context);
    if (c == nullptr) return static_cast<int>(cudaErrorInvalidValue);
    if (rank) *rank = c->rank;
    if (ranks) *ranks = c->ranks;
    return 0;
}

int qi_shard_all_gather(void *context, const void *y_local, void *y_slabs, int output_dtype, int rows, int n_local,
                        void *stream) {
    using namespace qi::shard;
    Context *c = checked(context);
    if (c == nullptr || y_local == nullptr || y_slabs == nullptr || rows <= 0 || n_local <= 0)
        return static_cast<int>(cudaErrorInvalidValue);
    if (output_dtype != QI_DTYPE_F32 && output_dtype != QI_DTYPE_F16) return static_cast<int>(cudaErrorInvalidValue);
    const size_t count = static_cast<size_t>(rows) * n_local;
    const int result = nccl().AllGather(y_local, y_slabs, count, output_dtype == QI_DTYPE_F16 ? NCCL_FLOAT16 : NCCL_FLOAT32,
                                        c->comm, static_cast<cudaStream_t>(stream));
    return result == 0 ? 0 : NCCL_ERROR_BASE + result;
}

int qi_shard_all_reduce_f32(void *context, float *y, unsigned long long count, void *stream) {
    using namespace qi::shard;
    Context *c = checked(context);
    if (c == nullptr || y == nullptr || count == 0) return static_cast<int>(cudaErrorInvalidValue);
    if (c->ranks == 1) return 0;
    if (nccl().AllReduce == nullptr) return NCCL_MISSING;
    const int result = nccl().AllReduce(y, y, static_cast<size_t>(count), NCCL_FLOAT32, 0 /* ncclSum */, c->comm,
                                        static_cast<cudaStream_t>(stream));
    return result == 0 ? 0 : NCCL_ERROR_BASE + result;
}

int qi_shard_reduce_scatter_f32(void *context, const float *y, float *y_share, unsigned long long count_per_rank, void *stream) {
    using namespace qi::shard;
    Context *c = checked(context);
    if (c == nullptr || y == nullptr || y_share == nullptr || count_per_rank == 0) return static_cast<int>(cudaErrorInvalidValue);
    if (c->ranks == 1)
        return static_cast<int>(cudaMemcpyAsync(y_share, y, count_per_rank * sizeof(float), cudaMemcpyDeviceToDevice,
                                                static_cast<cudaStream_t>(stream)));
    if (nccl().ReduceScatter == nullptr) return NCCL_MISSING;
    const int result = nccl().ReduceScatter(y, y_share, static_cast<size_t>(count_per_rank), NCCL_FLOAT32, 0 /* ncclSum */, c->comm,
                                            static_cast<cudaStream_t>(stream));
    return result == 0 ? 0 : NCCL_ERROR_BASE + result;
}

int qi_shard_barrier(void *context, void *stream) {
    using namespace qi::shard;
    Context *c = checked(context);
    if (c == nullptr) return static_cast<int>(cudaErrorInvalidValue);
    if (c->ranks == 1) return 0;
    if (nccl().AllReduce == nullptr) return NCCL_MISSING;
    if (c->token == nullptr) return static_cast<int>(cudaErrorInvalidValue);
    const int result = nccl().AllReduce(c->token, c->token, 1, NCCL_FLOAT32, 0 /* ncclSum */, c->comm,
                                        static_cast<cudaStream_t>(stream));
    return result == 0 ? 0 : NCCL_ERROR_BASE + result;
}

int qi_shard_put_slice(void *context, void *const *y_copies, int copies, int output_dtype, long long ldy, int column,
                       int rows, int n_local, void *stream) {
    using namespace qi::shard;
    Context *c = checked(context);
    if (c == nullptr || y_copies == nullptr || copies != c->ranks || rows <= 0 || n_local <= 0 || column < 0 ||
        ldy < static_cast<long long>(column) + n_local)
        return static_cast<int>(cudaErrorInvalidValue);
    if (output_dtype != QI_DTYPE_F32 && output_dtype != QI_DTYPE_F16) return static_cast<int>(cudaErrorInvalidValue);
    for (int i = 0; i < copies; ++i)
        if (y_copies[i] == nullptr) return static_cast<int>(cudaErrorInvalidValue);
    if (copies == 1) return 0;
    if (c->lanes_made != PUT_LANES || !c->fork_made) return static_cast<int>(cudaErrorInvalidValue);
    cudaError_t error = cudaSuccess;
    cudaStream_t caller = static_cast<cudaStream_t>(stream);
    const size_t element = output_dtype == QI_DTYPE_F16 ? 2 : 4;
    const size_t pitch = static_cast<size_t>(ldy) * element, first_byte = static_cast<size_t>(column) * element;
    const char *source = static_cast<const char *>(y_copies[c->rank]) + first_byte;
    const int lanes = copies - 1 < PUT_LANES ? copies - 1 : PUT_LANES;
    error = cudaEventRecord(c->fork, caller);
    int forked = 0;  // lanes that wait for the caller's stream: they are joined back below whatever happens in between
    for (int i = 0; i < lanes && error == cudaSuccess; ++i) {
        error = cudaStreamWaitEvent(c->lanes[i], c->fork, 0);
        if (error == cudaSuccess) forked = i + 1;
    }
    for (int step = 1; step < copies && error == cudaSuccess; ++step) {
        const int peer = (c->rank + step) % copies;  // every rank starts with another GPU
        char *target = static_cast<char *>(y_copies[peer]) + first_byte;
        const size_t width = static_cast<size_t>(n_local) * element;
        if (width == pitch)  // the slice is the whole matrix (a slab): one contiguous block
            error = cudaMemcpyAsync(target, source, width * rows, cudaMemcpyDefault, c->lanes[(step - 1) % lanes]);
        else
            error = cudaMemcpy2DAsync(target, pitch, source, pitch, width, rows, cudaMemcpyDefault,
                                      c->lanes[(step - 1) % lanes]);
    }
    for (int i = 0; i < forked; ++i) {  // also after an error: copies already queued stay ordered before the caller's later work
        cudaError_t joined = cudaEventRecord(c->joins[i], c->lanes[i]);
        if (joined == cudaSuccess) joined = cudaStreamWaitEvent(caller, c->joins[i], 0);
        if (error == cudaSuccess) error = joined;
    }
    return static_cast<int>(error);
}

int qi_shard_peer_export(const void *pointer, void *handle, size_t *offset) {
    using namespace qi::shard;
    if (pointer == nullptr || handle == nullptr || offset == nullptr) return static_cast<int>(cudaErrorInvalidValue);
    AddressRange range = address_range();
    if (range == nullptr) return static_cast<int>(cudaErrorNotSupported);
    CUdeviceptr base = 0;
    size_t bytes = 0;
    if (range(&base, &bytes, reinterpret_cast<CUdeviceptr>(pointer)) != CUDA_SUCCESS)
        return static_cast<int>(cudaErrorInvalidValue);
    cudaIpcMemHandle_t exported;
    const cudaError_t error = cudaIpcGetMemHandle(&exported, reinterpret_cast<void *>(base));
    if (error != cudaSuccess) return static_cast<int>(error);
    memcpy(handle, &exported, sizeof(exported));
    *offset = reinterpret_cast<CUdeviceptr>(pointer) - base;
    return 0;
}

int qi_shard_peer_open(const void *handle, size_t offset, void **pointer) {
    if (handle == nullptr || pointer == nullptr) return static_cast<int>(cudaErrorInvalidValue);
    *pointer = nullptr;
    cudaIpcMemHandle_t imported;
    memcpy(&imported, handle, sizeof(imported));
    void *base = nullptr;
    const cudaError_t error = cudaIpcOpenMemHandle(&base, imported, cudaIpcMemLazyEnablePeerAccess);
    if (error != cudaSuccess) return static_cast<int>(error);
    *pointer = static_cast<char *>(base) + offset;
    return 0;
}

int qi_shard_peer_close(void *pointer, size_t offset) {
    if (pointer == nullptr) return static_cast<int>(cudaErrorInvalidValue);
    return static_cast<int>(cudaIpcCloseMemHandle(static_cast<char *>(pointer) - offset));
}

int qi_shard_plan_inputs(int k, int scheme, int ranks, int rank, int *first_input, int *input_count) {
    return qi::shard::plan_inputs(k, scheme, ranks, rank, first_input, input_count);
}

int qi_shard_linear_inputs(void *context, const qi_packed_linear *local_record, const qi_linear_work *work,
                           const void *input_local, int input_dtype, float *y, int rows, int reuse_input, void *stream) {
    using namespace qi::shard;
    Context *c = checked(context);
    if (c == nullptr || local_record == nullptr || y == nullptr) return static_cast<int>(cudaErrorInvalidValue);
    const int unit = local_record->scheme == QI_SCHEME_W4A4_H256 ? 256 : 64;
    if (local_record->k % unit != 0) return static_cast<int>(cudaErrorInvalidValue);
    if (c->ranks > 1 && local_record->bias != nullptr && c->rank != 0)
        return static_cast<int>(cudaErrorInvalidValue);  // the bias is added once: give it to rank 0 only
    const int status = qi_linear(local_record, work, input_local, input_dtype, y, QI_DTYPE_F32, local_record->n, rows,
                                 reuse_input, stream);
    if (status != 0 || c->ranks == 1) return status;
    if (nccl().AllReduce == nullptr) return NCCL_MISSING;
    const int result = nccl().AllReduce(y, y, static_cast<size_t>(rows) * local_record->n, NCCL_FLOAT32, 0 /* ncclSum */,
                                        c->comm, static_cast<cudaStream_t>(stream));
    return result == 0 ? 0 : NCCL_ERROR_BASE + result;
}

int qi_shard_linear(void *context, const qi_packed_linear *local_record, const qi_linear_work *work, const void *input,
                    int input_dtype, void *y_local, void *y_slabs, int output_dtype, int rows, int reuse_input,
                    void *stream) {
    using namespace qi::shard;
    Context *c = checked(context);
    if (c == nullptr || local_record == nullptr) return static_cast<int>(cudaErrorInvalidValue);
    if (local_record->n % 128 != 0) return static_cast<int>(cudaErrorInvalidValue);
    const int status = qi_linear(local_record, work, input, input_dtype, y_local, output_dtype, local_record->n, rows,
                                 reuse_input, stream);
    if (status != 0 || y_slabs == nullptr || c->ranks == 1) return status;
    return qi_shard_all_gather(context, y_local, y_slabs, output_dtype, rows, local_record->n, stream);
}

}  // extern "C"
