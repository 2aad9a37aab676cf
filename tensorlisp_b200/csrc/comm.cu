// Tensor-parallel plumbing: one NCCL communicator per device handle, used by the ALLREDUCE
// pseudo-op after each row-parallel MUL_MAT. The reference has no multi-GPU path of its own
// (crates/tensorlisp/src/model.rs:415-422 takes the first GPU); the only collective in its tree is
// vendored ggml-cuda's ncclAllReduce per activation tensor (vendor/ggml/src/ggml-cuda/ggml-cuda.cu:997-1069),
// which tensorlisp never builds.
//
// NCCL is resolved at run time (dlopen of libnccl.so.2, which is the copy the host process already
// loaded when it uses torch.distributed), so the library loads on machines without NCCL.
#include <dlfcn.h>

#include <mutex>

#include "tlb_internal.h"

namespace tlb {

typedef struct ncclComm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
enum { ncclSuccess = 0 };
enum { ncclFloat32 = 7 };
enum { ncclSum = 0 };

struct NcclApi {
    int (*GetUniqueId)(ncclUniqueId *) = nullptr;
    int (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    int (*CommDestroy)(ncclComm_t) = nullptr;
    int (*AllReduce)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
    bool ok = false;
    std::string why;
};

static NcclApi &nccl() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) {
            api.why = std::string("NCCL is not available: ") + dlerror();
            return;
        }
        api.GetUniqueId = (decltype(api.GetUniqueId))dlsym(h, "ncclGetUniqueId");
        api.CommInitRank = (decltype(api.CommInitRank))dlsym(h, "ncclCommInitRank");
        api.CommDestroy = (decltype(api.CommDestroy))dlsym(h, "ncclCommDestroy");
        api.AllReduce = (decltype(api.AllReduce))dlsym(h, "ncclAllReduce");
        api.GetErrorString = (decltype(api.GetErrorString))dlsym(h, "ncclGetErrorString");
        api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllReduce && api.GetErrorString;
        if (!api.ok) api.why = "NCCL is missing entry points";
    });
    return api;
}

struct Comm {
    ncclComm_t comm = nullptr;
    int n_ranks = 1, rank = 0;
};

cudaError_t comm_allreduce_f32(tlb_device *dev, float *buf, size_t n, cudaStream_t st) {
    if (!dev->comm || dev->comm->n_ranks == 1) return cudaSuccess;
    const int r = nccl().AllReduce(buf, buf, n, ncclFloat32, ncclSum, dev->comm->comm, st);
    return r == ncclSuccess ? cudaSuccess : cudaErrorUnknown;
}
int comm_ranks(tlb_device *dev) { return dev->comm ? dev->comm->n_ranks : 1; }

}  // namespace tlb

using namespace tlb;

extern "C" {

tlb_status tlb_comm_unique_id(void *out128) {
    if (!out128) return fail(TLB_INVALID, "null id buffer");
    NcclApi &api = nccl();
    if (!api.ok) return fail(TLB_PIPELINE, api.why);
    ncclUniqueId id;
    const int r = api.GetUniqueId(&id);
    if (r != ncclSuccess) return fail(TLB_EXECUTION, std::string("ncclGetUniqueId: ") + api.GetErrorString(r));
    std::memcpy(out128, &id, 128);
    return TLB_OK;
}

tlb_status tlb_comm_init(tlb_device *dev, int n_ranks, int rank, const void *id128) {
    if (!dev || n_ranks < 1 || rank < 0 || rank >= n_ranks) return fail(TLB_INVALID, "tlb_comm_init: bad arguments");
    if (dev->comm) return fail(TLB_INVALID, "the device already has a communicator");
    Comm *c = new Comm;
    c->n_ranks = n_ranks;
    c->rank = rank;
    if (n_ranks > 1) {
        if (!id128) {
            delete c;
            return fail(TLB_INVALID, "null communicator id");
        }
        NcclApi &api = nccl();
        if (!api.ok) {
            delete c;
            return fail(TLB_PIPELINE, api.why);
        }
        ncclUniqueId id;
        std::memcpy(&id, id128, 128);
        cudaSetDevice(dev->ordinal);
        const int r = api.CommInitRank(&c->comm, n_ranks, id, rank);
        if (r != ncclSuccess) {
            delete c;
            return fail(TLB_EXECUTION, std::string("ncclCommInitRank: ") + api.GetErrorString(r));
        }
    }
    dev->comm = c;
    return TLB_OK;
}

tlb_status tlb_comm_destroy(tlb_device *dev) {
    if (!dev || !dev->comm) return TLB_OK;
    if (dev->comm->comm) nccl().CommDestroy(dev->comm->comm);
    delete dev->comm;
    dev->comm = nullptr;
    return TLB_OK;
}

}  // extern "C"
