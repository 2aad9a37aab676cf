// Tensor-parallel plumbing: one NCCL communicator per device handle, used by the ALLREDUCE
// pseudo-op after each row-parallel MUL_MAT. The reference has no multi-GPU path of its own
// (crates/tensorlisp/src/model.rs:415-422 takes the first GPU); the only collective in its tree is
// vendored ggml-cuda's ncclAllReduce per activation tensor (vendor/ggml/src/ggml-cuda/ggml-cuda.cu:997-1069),
// which tensorlisp never builds.
//
// NCCL is resolved at run time (dlopen of libnccl.so.2, which is the copy the host process already
// loaded when it uses torch.distributed), so the library loads on machines without NCCL.
#include <dlfcn.h>

#include <algorithm>
#include <mutex>
#include <vector>

#include "kernels.h"
#include "tlb_internal.h"
#include "exchange.cuh"

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

// ---------------------------------------------------------------- one-shot all-reduce over peer memory
// For the 512 KB activations of a decode step NCCL's ring costs 20+ us per call, 64 calls per step. Here
// every rank PUSHES its data into a slot of every peer's exchange buffer with plain stores over NVLink
// (so remote data always lands in local memory first), raises a per-CTA flag there, waits for the
// flags of all ranks in its own buffer (bounded), and adds the slots up in rank order - the same order
// on every rank, so all ranks end with bit-identical sums. CTA c of every rank owns chunk c of the
// data, so no grid-wide barrier is needed. Sequence numbers only grow; slots alternate by parity
// (a rank can be one call ahead of a peer, never two: finishing call s needs every peer's flags of call s).
__device__ __forceinline__ void ar_body(const ArRank &a, int n, int n_ranks, int c, int n_ctas) {
    __shared__ int s_fail;
    const int tid = threadIdx.x;
    if (a.skip_push) return;   // self tests: a rank that never shows up
    char *local = a.peer[a.rank];
    uint32_t *seqs = reinterpret_cast<uint32_t *>(local + AR_SEQ_OFF);
    const uint32_t seq = seqs[c] + 1;
    const uint32_t par = seq & 1;
    const int per = ((n / 4 + n_ctas - 1) / n_ctas);          // float4 per CTA
    const int v0 = c * per, v1 = min(n / 4, v0 + per);
    if (tid == 0) s_fail = 0;
    // ---- push my chunk (first summed over the K split, in split order) into slot [par][my rank] of every rank
    const float4 *src = reinterpret_cast<const float4 *>(a.n_split > 0 ? a.partial : a.data);
    const size_t slot_off = AR_DATA_OFF + ((size_t)par * AR_MAX_RANKS + a.rank) * AR_SLOT_BYTES;
    for (int i = v0 + tid; i < v1; i += AR_THREADS) {
        float4 v = src[i];
        for (int s0 = 1; s0 < a.n_split; s0 += 4) {
            // four loads in flight before the adds that need them
            float4 t[4];
#pragma unroll
            for (int k = 0; k < 4; k++) t[k] = s0 + k < a.n_split ? src[(size_t)(s0 + k) * (n / 4) + i] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int k = 0; k < 4; k++)
                if (s0 + k < a.n_split) { v.x += t[k].x; v.y += t[k].y; v.z += t[k].z; v.w += t[k].w; }
        }
        for (int p = 0; p < n_ranks; p++) reinterpret_cast<float4 *>(a.peer[p] + slot_off)[i] = v;
    }
    __threadfence_system();
    __syncthreads();
    if (tid < n_ranks) {
        uint32_t *flag = reinterpret_cast<uint32_t *>(a.peer[tid] + AR_FLAG_OFF) + ((size_t)par * AR_MAX_RANKS + a.rank) * AR_CTAS + c;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(seq) : "memory");
        // ---- wait (bounded) for chunk c of rank `tid` to have landed here
        const uint32_t *mine = reinterpret_cast<const uint32_t *>(local + AR_FLAG_OFF) + ((size_t)par * AR_MAX_RANKS + tid) * AR_CTAS + c;
        bool ok = false;
        for (uint32_t it = 0; it < a.spin_limit; it++) {
            uint32_t f;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(f) : "l"(mine) : "memory");
            if ((int32_t)(f - seq) >= 0) { ok = true; break; }
        }
        if (!ok) s_fail = 1;
    }
    __syncthreads();
    if (s_fail) {
        if (tid == 0) {
            atomicExch(a.err, 3);
            seqs[c] = seq;
        }
        return;
    }
    // ---- add the slots in rank order (L2 loads: L1 may still hold this slot's lines of two calls ago)
    const char *slots = local + AR_DATA_OFF + (size_t)par * AR_MAX_RANKS * AR_SLOT_BYTES;
    float4 *out = reinterpret_cast<float4 *>(a.data);
    for (int i = v0 + tid; i < v1; i += AR_THREADS) {
        float4 acc = __ldcg(reinterpret_cast<const float4 *>(slots) + i);
        for (int p = 1; p < n_ranks; p++) {
            const float4 x = __ldcg(reinterpret_cast<const float4 *>(slots + (size_t)p * AR_SLOT_BYTES) + i);
            acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
        }
        out[i] = acc;
    }
    if (tid == 0) seqs[c] = seq;
}

__global__ void __launch_bounds__(AR_THREADS) k_allreduce_oneshot(ArRank a, int n, int n_ranks) {
    ar_body(a, n, n_ranks, blockIdx.x, gridDim.x);
}
// All ranks in ONE cooperative launch on one GPU (blockIdx.y = rank): the single-GPU test of the protocol.
// Ranks that wait on one another must not be separate launches on one device.
struct ArAll { ArRank r[AR_MAX_RANKS]; };
__global__ void __launch_bounds__(AR_THREADS) k_allreduce_emulated(ArAll all, int n, int n_ranks) {
    ar_body(all.r[blockIdx.y], n, n_ranks, blockIdx.x, gridDim.x);
}

static int ar_grid(size_t n) { return (int)std::max<size_t>(1, std::min<size_t>(AR_CTAS, (n / 4 + 511) / 512)); }

struct Comm {
    ncclComm_t comm = nullptr;
    int n_ranks = 1, rank = 0;
    char *xbuf = nullptr;                    // this rank's exchange buffer (cudaMalloc)
    char *peer[AR_MAX_RANKS] = {nullptr};    // all ranks' buffers as mapped here; peer[rank] == xbuf
    bool p2p = false;
};

bool comm_p2p_takes(tlb_device *dev, size_t n) {
    return dev->comm && dev->comm->n_ranks > 1 && dev->comm->p2p && n % 4 == 0 && n * 4 <= AR_SLOT_BYTES;
}

cudaError_t comm_allreduce_f32(tlb_device *dev, float *buf, size_t n, cudaStream_t st, int *err, const float *partial, int n_split) {
    if (!dev->comm || dev->comm->n_ranks == 1) return n_split > 0 ? cudaErrorInvalidValue : cudaSuccess;
    Comm *c = dev->comm;
    if (comm_p2p_takes(dev, n) && ((uintptr_t)buf & 15) == 0 && ((uintptr_t)partial & 15) == 0 && err) {
        ArRank a{};
        a.data = buf;
        a.partial = partial;
        a.n_split = partial ? n_split : 0;
        a.rank = c->rank;
        a.err = err;
        a.spin_limit = ar_spin_limit();
        for (int p = 0; p < c->n_ranks; p++) a.peer[p] = c->peer[p];
        k_allreduce_oneshot<<<ar_grid(n), AR_THREADS, 0, st>>>(a, (int)n, c->n_ranks);
        return cudaGetLastError();
    }
    if (n_split > 0) return cudaErrorInvalidValue;   // the caller asks comm_p2p_takes first
    const int r = nccl().AllReduce(buf, buf, n, ncclFloat32, ncclSum, c->comm, st);
    return r == ncclSuccess ? cudaSuccess : cudaErrorUnknown;
}
int comm_ranks(tlb_device *dev) { return dev->comm ? dev->comm->n_ranks : 1; }

// the exchange fused with residual add + RMS norm + quantizer (k_fused.cu); the caller asked comm_p2p_takes and
// exchange_row_quant_supported first
cudaError_t comm_exchange_row_quant(tlb_device *dev, float *data, const float *partial, int n_split, const RowQuantArgs &p, cudaStream_t st,
                                    int *err) {
    Comm *c = dev->comm;
    if (!c || !c->p2p || !err) return cudaErrorInvalidValue;
    ArRank a{};
    a.data = data;
    a.partial = partial;
    a.n_split = partial ? n_split : 0;
    a.rank = c->rank;
    a.err = err;
    a.spin_limit = ar_spin_limit();
    a.flagged_words = xr_flagged_words(c->n_ranks);
    for (int r = 0; r < c->n_ranks; r++) a.peer[r] = c->peer[r];
    return launch_exchange_row_quant(a, p, c->n_ranks, st);
}

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
    dev->comm_generation++;
    return TLB_OK;
}

tlb_status tlb_comm_p2p_export(tlb_device *dev, void *handle64) {
    if (!dev || !dev->comm || !handle64) return fail(TLB_INVALID, "tlb_comm_p2p_export: needs a device with a communicator");
    Comm *c = dev->comm;
    if (c->n_ranks > AR_MAX_RANKS) return fail(TLB_INVALID, "the peer-memory all-reduce takes at most 8 ranks");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    cudaSetDevice(dev->ordinal);
    if (!c->xbuf) {
        if (cudaMalloc(&c->xbuf, AR_BUF_BYTES) != cudaSuccess) {
            cudaGetLastError();
            return fail(TLB_ALLOC, "exchange buffer allocation failed");
        }
        cudaMemset(c->xbuf, 0, AR_BUF_BYTES);
        cudaDeviceSynchronize();
    }
    cudaIpcMemHandle_t h;
    const cudaError_t e = cudaIpcGetMemHandle(&h, c->xbuf);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(TLB_EXECUTION, std::string("cudaIpcGetMemHandle: ") + cudaGetErrorString(e));
    }
    std::memcpy(handle64, &h, 64);
    return TLB_OK;
}

tlb_status tlb_comm_p2p_import(tlb_device *dev, const void *handles) {
    if (!dev || !dev->comm || !handles) return fail(TLB_INVALID, "tlb_comm_p2p_import: needs a device with a communicator");
    Comm *c = dev->comm;
    if (!c->xbuf) return fail(TLB_INVALID, "call tlb_comm_p2p_export first");
    cudaSetDevice(dev->ordinal);
    for (int p = 0; p < c->n_ranks; p++) {
        if (p == c->rank) {
            c->peer[p] = c->xbuf;
            continue;
        }
        cudaIpcMemHandle_t h;
        std::memcpy(&h, (const char *)handles + (size_t)p * 64, 64);
        void *ptr = nullptr;
        const cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return fail(TLB_EXECUTION, "cudaIpcOpenMemHandle (rank " + std::to_string(p) + "): " + cudaGetErrorString(e));
        }
        c->peer[p] = (char *)ptr;
    }
    // Measured on B200 (batch-32 decode, 512 KB messages, the exchange fused with the row quantizer): peer memory
    // is 6% faster per step than NCCL with 2 ranks and 13% with 8. TLB_NO_P2P_ALLREDUCE=1 keeps NCCL for everything.
    const char *off = getenv("TLB_NO_P2P_ALLREDUCE");
    c->p2p = !(off && off[0] == '1');
    dev->comm_generation++;
    return TLB_OK;
}

// Single-GPU check of the all-reduce protocol: `n_ranks` emulated ranks (their buffers all on this
// device) run as ONE cooperative launch; in[r] / out[r] are n floats per rank on the host.
static tlb_status p2p_selftest(tlb_device *dev, int n_ranks, int n, int calls, int n_split, const float *in, float *out, int absent_rank,
                               uint32_t spin_limit);
tlb_status tlb_comm_p2p_selftest(tlb_device *dev, int n_ranks, int n, int calls, int n_split, const float *in, float *out) {
    return p2p_selftest(dev, n_ranks, n, calls, n_split, in, out, -1, ar_spin_limit());
}
// The same launch with one emulated rank that never pushes: the waits of the others run out after `spin_limit`
// probes, the kernel returns, and the call reports TLB_EXECUTION ("gave up waiting") instead of hanging.
tlb_status tlb_comm_p2p_selftest_absent(tlb_device *dev, int n_ranks, int n, int absent_rank, uint32_t spin_limit, const float *in, float *out) {
    if (absent_rank < 0 || absent_rank >= n_ranks || spin_limit == 0) return fail(TLB_INVALID, "tlb_comm_p2p_selftest_absent: bad arguments");
    return p2p_selftest(dev, n_ranks, n, 1, 0, in, out, absent_rank, spin_limit);
}
static tlb_status p2p_selftest(tlb_device *dev, int n_ranks, int n, int calls, int n_split, const float *in, float *out, int absent_rank,
                               uint32_t spin_limit) {
    if (!dev || n_ranks < 1 || n_ranks > AR_MAX_RANKS || n < 4 || n % 4 || (size_t)n * 4 > AR_SLOT_BYTES || calls < 1 || n_split < 0 ||
        n_split > 16 || !in || !out)
        return fail(TLB_INVALID, "tlb_comm_p2p_selftest: bad arguments");
    const int parts = n_split > 0 ? n_split : 1;   // floats per rank in `in`: parts x n
    cudaSetDevice(dev->ordinal);
    ArAll all{};
    char *bufs[AR_MAX_RANKS] = {nullptr};
    float *data[AR_MAX_RANKS] = {nullptr}, *part[AR_MAX_RANKS] = {nullptr};
    int *err = nullptr;
    cudaError_t e = cudaMalloc(&err, 256);
    if (e == cudaSuccess) e = cudaMemset(err, 0, 256);
    for (int r = 0; r < n_ranks && e == cudaSuccess; r++) {
        e = cudaMalloc(&bufs[r], AR_BUF_BYTES);
        if (e == cudaSuccess) e = cudaMemset(bufs[r], 0, AR_BUF_BYTES);
        if (e == cudaSuccess) e = cudaMalloc(&data[r], (size_t)n * 4);
        if (e == cudaSuccess) e = cudaMemset(data[r], 0, (size_t)n * 4);
        if (e == cudaSuccess && n_split > 0) e = cudaMalloc(&part[r], (size_t)parts * n * 4);
    }
    for (int r = 0; r < n_ranks && e == cudaSuccess; r++) {
        all.r[r].data = data[r];
        all.r[r].partial = part[r];
        all.r[r].n_split = n_split;
        all.r[r].rank = r;
        all.r[r].err = err;
        all.r[r].spin_limit = spin_limit;
        all.r[r].skip_push = r == absent_rank;
        for (int p = 0; p < n_ranks; p++) all.r[r].peer[p] = bufs[p];
    }
    int flag = 0;
    std::vector<float> h((size_t)n_ranks * parts * n);
    for (int call = 0; call < calls && e == cudaSuccess; call++) {
        // every call reduces fresh inputs scaled by (call + 1), so a stale slot would show. The copies go
        // through the launching stream: a plain cudaMemcpy from pageable memory may return before its DMA
        // has landed, and the stream of this device does not wait for the default stream.
        for (size_t i = 0; i < h.size(); i++) h[i] = in[i] * (float)(call + 1);
        for (int r = 0; r < n_ranks && e == cudaSuccess; r++)
            e = cudaMemcpyAsync(n_split > 0 ? part[r] : data[r], h.data() + (size_t)r * parts * n, (size_t)parts * n * 4, cudaMemcpyHostToDevice,
                                dev->stream);
        if (e != cudaSuccess) break;
        void *args[] = {&all, &n, &n_ranks};
        e = cudaLaunchCooperativeKernel((void *)k_allreduce_emulated, dim3(ar_grid((size_t)n), n_ranks), dim3(AR_THREADS), args, 0, dev->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(dev->stream);
    }
    if (e == cudaSuccess) e = cudaMemcpy(&flag, err, 4, cudaMemcpyDeviceToHost);
    for (int r = 0; r < n_ranks && e == cudaSuccess; r++) e = cudaMemcpy(out + (size_t)r * n, data[r], (size_t)n * 4, cudaMemcpyDeviceToHost);
    for (int r = 0; r < n_ranks; r++) {
        if (bufs[r]) cudaFree(bufs[r]);
        if (data[r]) cudaFree(data[r]);
        if (part[r]) cudaFree(part[r]);
    }
    if (err) cudaFree(err);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(TLB_EXECUTION, std::string("all-reduce self test: ") + cudaGetErrorString(e));
    }
    if (flag) return fail(TLB_EXECUTION, "all-reduce self test: a rank gave up waiting for its peers");
    return TLB_OK;
}

// Single-GPU check of the fused exchange + residual add + RMS norm + Q8_K kernel: n_ranks <= 4 emulated ranks in one
// cooperative launch. in: n_ranks x n_split x rows x K partial results (n_split >= 1), resid: rows x K, w: K.
// out_sum: n_ranks x rows x K (the new residual stream of every rank), out_q: n_ranks x act_bytes (the Q8_K block).
static tlb_status p2p_selftest_rows(tlb_device *dev, int n_ranks, int rows, int K, int n_split, int calls, const float *in, const float *resid,
                                    const float *w, float eps, float *out_sum, void *out_q, uint64_t act_bytes, int absent_rank, uint32_t spin_limit);
tlb_status tlb_comm_p2p_selftest_rows(tlb_device *dev, int n_ranks, int rows, int K, int n_split, int calls, const float *in,
                                      const float *resid, const float *w, float eps, float *out_sum, void *out_q, uint64_t act_bytes) {
    return p2p_selftest_rows(dev, n_ranks, rows, K, n_split, calls, in, resid, w, eps, out_sum, out_q, act_bytes, -1, ar_spin_limit());
}
// One emulated rank never pushes its rows: the others give up after `spin_limit` probes and the call fails.
tlb_status tlb_comm_p2p_selftest_rows_absent(tlb_device *dev, int n_ranks, int rows, int K, int absent_rank, uint32_t spin_limit, const float *in,
                                             const float *resid, const float *w, float eps, float *out_sum, void *out_q, uint64_t act_bytes) {
    if (absent_rank < 0 || absent_rank >= n_ranks || spin_limit == 0) return fail(TLB_INVALID, "tlb_comm_p2p_selftest_rows_absent: bad arguments");
    return p2p_selftest_rows(dev, n_ranks, rows, K, 1, 1, in, resid, w, eps, out_sum, out_q, act_bytes, absent_rank, spin_limit);
}
static tlb_status p2p_selftest_rows(tlb_device *dev, int n_ranks, int rows, int K, int n_split, int calls, const float *in, const float *resid,
                                    const float *w, float eps, float *out_sum, void *out_q, uint64_t act_bytes, int absent_rank, uint32_t spin_limit) {
    if (!dev || n_ranks < 1 || n_ranks > 4 || n_split < 1 || n_split > 16 || calls < 1 || !in || !resid || !w || !out_sum || !out_q ||
        !exchange_row_quant_supported(K, rows))
        return fail(TLB_INVALID, "tlb_comm_p2p_selftest_rows: bad arguments");
    const ActLayout al = act_layout(ACT_Q8_K, K, rows);
    if (act_bytes != al.bytes) return fail(TLB_INVALID, "tlb_comm_p2p_selftest_rows: out_q must hold " + std::to_string(al.bytes) + " bytes per rank");
    cudaSetDevice(dev->ordinal);
    const size_t n = (size_t)rows * K;
    char *bufs[4] = {nullptr};
    float *part[4] = {nullptr}, *sum[4] = {nullptr}, *d_res = nullptr, *d_w = nullptr;
    char *q[4] = {nullptr};
    int *err = nullptr;
    cudaError_t e = cudaMalloc(&err, 256);
    if (e == cudaSuccess) e = cudaMemset(err, 0, 256);
    if (e == cudaSuccess) e = cudaMalloc(&d_res, n * 4);
    if (e == cudaSuccess) e = cudaMalloc(&d_w, (size_t)K * 4);
    for (int r = 0; r < n_ranks && e == cudaSuccess; r++) {
        e = cudaMalloc(&bufs[r], AR_BUF_BYTES);
        if (e == cudaSuccess) e = cudaMemset(bufs[r], 0, AR_BUF_BYTES);
        if (e == cudaSuccess) e = cudaMalloc(&part[r], (size_t)n_split * n * 4);
        if (e == cudaSuccess) e = cudaMalloc(&sum[r], n * 4);
        if (e == cudaSuccess) e = cudaMalloc(&q[r], al.bytes);
    }
    ArRank a[4];
    RowQuantArgs p[4];
    for (int r = 0; r < n_ranks && e == cudaSuccess; r++) {
        a[r] = ArRank{};
        a[r].data = nullptr;
        a[r].partial = part[r];
        a[r].n_split = n_split;
        a[r].rank = r;
        a[r].err = err;
        a[r].spin_limit = spin_limit;
        a[r].flagged_words = xr_flagged_words(n_ranks);
        a[r].skip_push = r == absent_rank;
        for (int k = 0; k < n_ranks; k++) a[r].peer[k] = bufs[k];
        p[r] = RowQuantArgs{};
        p[r].mode = RQ_NORM;
        p[r].K = K;
        p[r].N = rows;
        p[r].a = d_res;
        p[r].lda = K;
        p[r].sum_out = sum[r];
        p[r].ld_sum = K;
        p[r].w = d_w;
        p[r].wn = K;
        p[r].eps = eps;
        p[r].out = q[r];
        p[r].qs_off = al.qs_off;
        p[r].d_off = al.d_off;
        p[r].bsum_off = al.bsum_off;
    }
    std::vector<float> h((size_t)n_ranks * n_split * n);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_res, resid, n * 4, cudaMemcpyHostToDevice, dev->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_w, w, (size_t)K * 4, cudaMemcpyHostToDevice, dev->stream);
    for (int call = 0; call < calls && e == cudaSuccess; call++) {
        for (size_t i = 0; i < h.size(); i++) h[i] = in[i] * (float)(call + 1);
        for (int r = 0; r < n_ranks && e == cudaSuccess; r++)
            e = cudaMemcpyAsync(part[r], h.data() + (size_t)r * n_split * n, (size_t)n_split * n * 4, cudaMemcpyHostToDevice, dev->stream);
        if (e == cudaSuccess) e = launch_exchange_row_quant_emulated(a, p, n_ranks, dev->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(dev->stream);
    }
    int flag = 0;
    if (e == cudaSuccess) e = cudaMemcpy(&flag, err, 4, cudaMemcpyDeviceToHost);
    for (int r = 0; r < n_ranks && e == cudaSuccess; r++) {
        e = cudaMemcpy(out_sum + (size_t)r * n, sum[r], n * 4, cudaMemcpyDeviceToHost);
        if (e == cudaSuccess) e = cudaMemcpy((char *)out_q + (size_t)r * al.bytes, q[r], al.bytes, cudaMemcpyDeviceToHost);
    }
    for (int r = 0; r < n_ranks; r++) {
        if (bufs[r]) cudaFree(bufs[r]);
        if (part[r]) cudaFree(part[r]);
        if (sum[r]) cudaFree(sum[r]);
        if (q[r]) cudaFree(q[r]);
    }
    if (d_res) cudaFree(d_res);
    if (d_w) cudaFree(d_w);
    if (err) cudaFree(err);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(TLB_EXECUTION, std::string("fused exchange self test: ") + cudaGetErrorString(e));
    }
    if (flag) return fail(TLB_EXECUTION, "fused exchange self test: a rank gave up waiting for its peers");
    return TLB_OK;
}

tlb_status tlb_comm_destroy(tlb_device *dev) {
    if (!dev || !dev->comm) return TLB_OK;
    cudaSetDevice(dev->ordinal);
    for (int p = 0; p < dev->comm->n_ranks && p < AR_MAX_RANKS; p++)
        if (dev->comm->peer[p] && p != dev->comm->rank) cudaIpcCloseMemHandle(dev->comm->peer[p]);
    if (dev->comm->xbuf) cudaFree(dev->comm->xbuf);
    if (dev->comm->comm) nccl().CommDestroy(dev->comm->comm);
    delete dev->comm;
    dev->comm = nullptr;
    dev->comm_generation++;   // captured graphs that hold the closed peer mappings are never replayed
    return TLB_OK;
}

}  // extern "C"
