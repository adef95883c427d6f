// Tensor-parallel communicator over NCCL (NVLink 5 / NVSwitch), one process per GPU.
//
// Stands where the engine has its process-global `Communicator` (rank, world_size, all_reduce, barrier) and the
// `mynn_all_reduce(dst, src, num_elements, dtype)` helper its CPU code calls.  NCCL is resolved at run time with
// dlopen so that the library has no link-time dependency on it and shares the copy the host process already
// loaded (a torch process brings its own libnccl.so.2).  Only the calls declared below are used.
#include <dlfcn.h>
#include <nccl.h>

#include "common.cuh"
#include "comm.cuh"

namespace mynn {

struct NcclApi {
    void *handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
};

static NcclApi g_nccl;
static ncclComm_t g_comm = nullptr;
static int g_rank = 0, g_world = 1;
static float *g_barrier_buf = nullptr;

static int load_nccl() {
    if (g_nccl.handle) return MYNN_OK;
    const char *names[] = {"libnccl.so.2", "libnccl.so"};
    void *h = nullptr;
    for (const char *n : names) {
        h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (h) break;
    }
    if (!h) return fail(MYNN_E_COMM, "cannot load NCCL: %s", dlerror());
#define SYM(field, name)                                                        \
    g_nccl.field = reinterpret_cast<decltype(g_nccl.field)>(dlsym(h, name));    \
    if (!g_nccl.field) return fail(MYNN_E_COMM, "NCCL symbol %s not found", name);
    SYM(GetUniqueId, "ncclGetUniqueId")
    SYM(CommInitRank, "ncclCommInitRank")
    SYM(AllReduce, "ncclAllReduce")
    SYM(AllGather, "ncclAllGather")
    SYM(CommDestroy, "ncclCommDestroy")
    SYM(GetErrorString, "ncclGetErrorString")
#undef SYM
    g_nccl.handle = h;
    return MYNN_OK;
}

#define NCCL_OK(expr)                                                                                 \
    do {                                                                                              \
        ncclResult_t r__ = (expr);                                                                    \
        if (r__ != ncclSuccess) return fail(MYNN_E_COMM, "%s failed: %s", #expr, g_nccl.GetErrorString(r__)); \
    } while (0)

static int nccl_dtype(int dt, ncclDataType_t *out) {
    switch (dt) {
        case MYNN_F32: *out = ncclFloat32; return MYNN_OK;
        case MYNN_BF16: *out = ncclBfloat16; return MYNN_OK;
        case MYNN_F16: *out = ncclFloat16; return MYNN_OK;
    }
    return fail(MYNN_E_ARG, "all_reduce: bad dtype %d", dt);
}

int comm_world() { return g_world; }
int comm_rank() { return g_rank; }

int comm_all_reduce(cudaStream_t st, void *dst, const void *src, size_t n, int dtype) {
    if (g_world == 1) {
        if (dst != src && n) MYNN_CUDA_OK(cudaMemcpyAsync(dst, src, n * dtype_size(dtype), cudaMemcpyDeviceToDevice, st));
        return MYNN_OK;
    }
    if (!g_comm) return fail(MYNN_E_STATE, "all_reduce: communicator not initialised");
    ncclDataType_t dt;
    int rc = nccl_dtype(dtype, &dt);
    if (rc) return rc;
    NCCL_OK(g_nccl.AllReduce(src, dst, n, dt, ncclSum, g_comm, st));
    return MYNN_OK;
}

int comm_all_gather(cudaStream_t st, void *dst, const void *src, size_t bytes_per_rank) {
    if (g_world == 1) {
        if (dst != src && bytes_per_rank) MYNN_CUDA_OK(cudaMemcpyAsync(dst, src, bytes_per_rank, cudaMemcpyDeviceToDevice, st));
        return MYNN_OK;
    }
    if (!g_comm) return fail(MYNN_E_STATE, "all_gather: communicator not initialised");
    NCCL_OK(g_nccl.AllGather(src, dst, bytes_per_rank, ncclInt8, g_comm, st));
    return MYNN_OK;
}

}  // namespace mynn

using namespace mynn;

extern "C" int mynn_b200_comm_unique_id(void *id_out) {
    if (!id_out) return fail(MYNN_E_ARG, "comm_unique_id: null pointer");
    int rc = load_nccl();
    if (rc) return rc;
    static_assert(sizeof(ncclUniqueId) == 128, "unique id is 128 bytes");
    NCCL_OK(g_nccl.GetUniqueId(reinterpret_cast<ncclUniqueId *>(id_out)));
    return MYNN_OK;
}

extern "C" int mynn_b200_comm_init(const void *unique_id, int rank, int world_size) {
    if (world_size < 1 || rank < 0 || rank >= world_size)
        return fail(MYNN_E_ARG, "comm_init: rank %d is not inside a world of %d", rank, world_size);
    if (g_comm) return fail(MYNN_E_STATE, "comm_init: communicator already initialised");
    g_rank = rank;
    g_world = world_size;
    if (world_size == 1) return MYNN_OK;  // identity communicator, no NCCL needed
    if (!unique_id) return fail(MYNN_E_ARG, "comm_init: null unique id");
    int rc = load_nccl();
    if (rc) return rc;
    ncclUniqueId id;
    memcpy(&id, unique_id, sizeof id);
    NCCL_OK(g_nccl.CommInitRank(&g_comm, world_size, id, rank));
    MYNN_CUDA_OK(cudaMalloc(&g_barrier_buf, sizeof(float)));
    MYNN_CUDA_OK(cudaMemset(g_barrier_buf, 0, sizeof(float)));
    return MYNN_OK;
}

extern "C" int mynn_b200_comm_rank(void) { return g_rank; }
extern "C" int mynn_b200_comm_world_size(void) { return g_world; }

extern "C" int mynn_b200_all_reduce(void *stream, void *dst, const void *src, int64_t num_elements, int dtype) {
    if (num_elements < 0) return fail(MYNN_E_ARG, "all_reduce: negative element count");
    if (!dtype_ok(dtype)) return fail(MYNN_E_ARG, "all_reduce: bad dtype %d", dtype);
    if (num_elements == 0) return MYNN_OK;
    if (!dst || !src) return fail(MYNN_E_ARG, "all_reduce: null pointer");
    return comm_all_reduce((cudaStream_t)stream, dst, src, (size_t)num_elements, dtype);
}

extern "C" int mynn_b200_comm_barrier(void *stream) {
    if (g_world == 1) return MYNN_OK;
    if (!g_comm) return fail(MYNN_E_STATE, "barrier: communicator not initialised");
    int rc = comm_all_reduce((cudaStream_t)stream, g_barrier_buf, g_barrier_buf, 1, MYNN_F32);
    if (rc) return rc;
    MYNN_CUDA_OK(cudaStreamSynchronize((cudaStream_t)stream));
    return MYNN_OK;
}

extern "C" int mynn_b200_comm_destroy(void) {
    if (g_comm) {
        g_nccl.CommDestroy(g_comm);
        g_comm = nullptr;
    }
    if (g_barrier_buf) {
        cudaFree(g_barrier_buf);
        g_barrier_buf = nullptr;
    }
    g_rank = 0;
    g_world = 1;
    return MYNN_OK;
}
