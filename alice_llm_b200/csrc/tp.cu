// Tensor-parallel plumbing of the C ABI: one process per GPU, output rows of every projection
// sharded over the ranks, the full vector rebuilt on every rank by an all-gather
// (the row split is where the reference parallelises a matvec, src/gguf.rs:3664).
//
// NCCL is bound at run time (dlopen of libnccl.so.2, reusing the copy the host process already
// loaded if there is one) so single-GPU users of the library need no NCCL at all. All collectives
// are queued on the engine's stream and are capturable in a CUDA graph.
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>

#include "abi_internal.cuh"
#include "tp.cuh"

namespace {

struct NcclApi {
    void* lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

NcclApi g_nccl;

int load_nccl() {
    if (g_nccl.lib) return ALICE_OK;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);   // the copy the process already uses, if any
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return alice_fail(ALICE_E_UNSUPPORTED, "tensor parallel: cannot load libnccl.so.2 (%s)", dlerror());
    NcclApi a;
    a.lib = h;
    a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
    a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
    a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
    a.AllGather = reinterpret_cast<decltype(a.AllGather)>(dlsym(h, "ncclAllGather"));
    a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
    if (!a.GetUniqueId || !a.CommInitRank || !a.CommDestroy || !a.AllGather || !a.GetErrorString)
        return alice_fail(ALICE_E_UNSUPPORTED, "tensor parallel: libnccl.so.2 lacks a required symbol");
    g_nccl = a;
    return ALICE_OK;
}

int nccl_fail(ncclResult_t r, const char* what) {
    return alice_fail(ALICE_E_CUDA, "%s: NCCL error %d (%s)", what, (int)r, g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "?");
}

}  // namespace

namespace alice {

int tp_all_gather(alice_engine* e, void* base, size_t bytes_per_rank) {
    if (e->tp_world <= 1) return ALICE_OK;
    // in place: rank r's contribution already sits at base + r * bytes_per_rank
    const char* send = static_cast<const char*>(base) + (size_t)e->tp_rank * bytes_per_rank;
    const ncclResult_t r = g_nccl.AllGather(send, base, bytes_per_rank, ncclInt8, static_cast<ncclComm_t>(e->tp_comm), e->stream);
    if (r != ncclSuccess) return nccl_fail(r, "ncclAllGather");
    return ALICE_OK;
}

void tp_release(alice_engine* e) {
    if (e->tp_comm && g_nccl.CommDestroy) g_nccl.CommDestroy(static_cast<ncclComm_t>(e->tp_comm));
    e->tp_comm = nullptr;
    e->tp_world = 1;
    e->tp_rank = 0;
}

}  // namespace alice

extern "C" {

int32_t alice_tp_unique_id(void* out, size_t nbytes) {
    if (!out || nbytes < sizeof(ncclUniqueId))
        return alice_fail(ALICE_E_INVALID, "alice_tp_unique_id: need a buffer of %zu bytes", sizeof(ncclUniqueId));
    int rc = load_nccl();
    if (rc) return rc;
    ncclUniqueId id;
    const ncclResult_t r = g_nccl.GetUniqueId(&id);
    if (r != ncclSuccess) return nccl_fail(r, "ncclGetUniqueId");
    std::memset(out, 0, nbytes);
    std::memcpy(out, &id, sizeof(id));
    return ALICE_OK;
}

int32_t alice_engine_tp_init(alice_engine* e, uint32_t rank, uint32_t world, const void* unique_id, size_t nbytes) {
    if (!e || !unique_id) return alice_fail(ALICE_E_INVALID, "alice_engine_tp_init: null argument");
    if (world == 0 || world > 8 || rank >= world) return alice_fail(ALICE_E_INVALID, "alice_engine_tp_init: rank %u of %u", rank, world);
    if (nbytes < sizeof(ncclUniqueId)) return alice_fail(ALICE_E_INVALID, "alice_engine_tp_init: unique id of %zu bytes, need %zu", nbytes, sizeof(ncclUniqueId));
    if (e->tp_comm) return alice_fail(ALICE_E_INVALID, "alice_engine_tp_init: engine already belongs to a group");
    if (world == 1) { e->tp_rank = 0; e->tp_world = 1; return ALICE_OK; }
    int rc = load_nccl();
    if (rc) return rc;
    cudaError_t err = cudaSetDevice(e->device);
    if (err != cudaSuccess) return alice_cuda_fail(err, "cudaSetDevice");
    ncclUniqueId id;
    std::memcpy(&id, unique_id, sizeof(id));
    ncclComm_t comm = nullptr;
    const ncclResult_t r = g_nccl.CommInitRank(&comm, (int)world, id, (int)rank);
    if (r != ncclSuccess) return nccl_fail(r, "ncclCommInitRank");
    e->tp_comm = comm;
    e->tp_rank = rank;
    e->tp_world = world;
    return ALICE_OK;
}

int32_t alice_engine_tp_info(const alice_engine* e, uint32_t* rank, uint32_t* world) {
    if (!e) return alice_fail(ALICE_E_INVALID, "alice_engine_tp_info: null engine");
    if (rank) *rank = e->tp_rank;
    if (world) *world = e->tp_world;
    return ALICE_OK;
}

}  // extern "C"
