// Library all-reduce as the comparison arm of the tensor-parallel sums.
//
// The product path adds the ranks' partial products of o_proj / down_proj by pushing them from the GEMV's epilogue
// into every rank's memory (tp.cuh). This file provides the conventional alternative — the partial product to scratch,
// ncclAllReduce on the engine's stream (captured into the step graph like any other node), one add into the residual
// stream — so the two can be timed side by side on the same engine. NCCL is not linked: the library is opened at run
// time from a path the caller names (the copy its process already uses), and only when this arm is switched on.
#include <dlfcn.h>

#include <cstring>
#include <mutex>
#include <string>

#include "engine.h"

namespace sp {

namespace {
struct UniqueId { char internal[128]; };  // ncclUniqueId
typedef void* Comm;                       // ncclComm_t
typedef int (*GetUniqueIdFn)(UniqueId*);
typedef int (*CommInitRankFn)(Comm*, int, UniqueId, int);
typedef int (*AllReduceFn)(const void*, void*, size_t, int, int, Comm, cudaStream_t);
typedef int (*CommDestroyFn)(Comm);
typedef const char* (*GetErrorStringFn)(int);
constexpr int NCCL_FLOAT32 = 7, NCCL_SUM = 0;

struct Api {
    void* lib = nullptr;
    GetUniqueIdFn get_unique_id = nullptr;
    CommInitRankFn comm_init_rank = nullptr;
    AllReduceFn all_reduce = nullptr;
    CommDestroyFn comm_destroy = nullptr;
    GetErrorStringFn error_string = nullptr;
};
Api g_api;
std::mutex g_api_mu;

int load_api(const char* path) {
    std::lock_guard<std::mutex> lk(g_api_mu);
    if (g_api.lib) return SP_OK;
    void* lib = dlopen(path && *path ? path : "libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) { set_error(std::string("cannot open the NCCL library: ") + dlerror()); return SP_ERR_STATE; }
    Api a;
    a.lib = lib;
    a.get_unique_id = (GetUniqueIdFn)dlsym(lib, "ncclGetUniqueId");
    a.comm_init_rank = (CommInitRankFn)dlsym(lib, "ncclCommInitRank");
    a.all_reduce = (AllReduceFn)dlsym(lib, "ncclAllReduce");
    a.comm_destroy = (CommDestroyFn)dlsym(lib, "ncclCommDestroy");
    a.error_string = (GetErrorStringFn)dlsym(lib, "ncclGetErrorString");
    if (!a.get_unique_id || !a.comm_init_rank || !a.all_reduce || !a.comm_destroy || !a.error_string) {
        set_error("the NCCL library lacks an expected symbol");
        return SP_ERR_STATE;
    }
    g_api = a;
    return SP_OK;
}

int fail(const char* what, int rc) {
    set_error(std::string(what) + ": " + (g_api.error_string ? g_api.error_string(rc) : "NCCL error"));
    return SP_ERR_COMM;
}
}  // namespace

int nccl_unique_id(const char* libpath, void* out, size_t cap) {
    if (!out || cap < sizeof(UniqueId)) { set_error("nccl_unique_id: buffer smaller than 128 bytes"); return SP_ERR_ARG; }
    const int st = load_api(libpath);
    if (st != SP_OK) return st;
    UniqueId id;
    const int rc = g_api.get_unique_id(&id);
    if (rc != 0) return fail("ncclGetUniqueId", rc);
    std::memcpy(out, &id, sizeof(id));
    return SP_OK;
}

// Collective over the ranks of the group: every rank calls it with the id rank 0 generated.
int Engine::tp_nccl_init(const char* libpath, const void* unique_id) {
    if (d.tp_size <= 1) { set_error("tp_nccl_init: not a tensor-parallel engine"); return SP_ERR_STATE; }
    if (!unique_id) { set_error("tp_nccl_init: null id"); return SP_ERR_ARG; }
    if (nccl_comm_) return SP_OK;
    const int st = load_api(libpath);
    if (st != SP_OK) return st;
    SP_CUDA_TRY(cudaSetDevice(d.device));
    UniqueId id;
    std::memcpy(&id, unique_id, sizeof(id));
    Comm comm = nullptr;
    const int rc = g_api.comm_init_rank(&comm, d.tp_size, id, d.tp_rank);
    if (rc != 0) return fail("ncclCommInitRank", rc);
    nccl_comm_ = comm;
    return SP_OK;
}

void Engine::tp_nccl_release() {
    if (nccl_comm_ && g_api.comm_destroy) g_api.comm_destroy((Comm)nccl_comm_);
    nccl_comm_ = nullptr;
}

int Engine::tp_set_allreduce(int mode) {
    if (mode != 0 && !nccl_comm_) { set_error("tp_set_allreduce: call tp_nccl_init first"); return SP_ERR_STATE; }
    if ((mode != 0) != tp_use_nccl_) drop_graphs();
    tp_use_nccl_ = mode != 0;
    return SP_OK;
}

// In-place sum of buf[count] floats over the ranks, on the engine's stream.
int Engine::nccl_all_reduce(float* buf, size_t count) {
    const int rc = g_api.all_reduce(buf, buf, count, NCCL_FLOAT32, NCCL_SUM, (Comm)nccl_comm_, stream);
    if (rc != 0) return fail("ncclAllReduce", rc);
    return SP_OK;
}

}  // namespace sp
