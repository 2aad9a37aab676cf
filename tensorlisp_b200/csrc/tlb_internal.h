// Internal types of the executor: IR, planner output, device objects and the launch helpers the
// kernel files export. Host-side counterpart of the reference's crates/kernels/src/{graph,plan}.rs
// and cuda/{mod,exec,lower}.rs, redone in C++ behind the C ABI of include/tlb200.h.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>
#include <functional>
#include <map>
#include <string>
#include <vector>

#include "../../include/tlb200.h"

namespace tlb {

// ---------------------------------------------------------------------------- errors
void set_error(const std::string &msg);
tlb_status fail(tlb_status st, const std::string &msg);
std::string cuda_msg(cudaError_t e);

struct Unsupported {  // crates/kernels/src/lib.rs Error::Unsupported
    std::string op, node, why;
};

// ---------------------------------------------------------------------------- IR
struct TypeTraits {
    const char *name;
    int64_t blck;
    uint64_t size;
};
const TypeTraits *type_traits(uint32_t ty);  // nullptr when unknown

enum Storage : uint32_t { WEIGHT = 0, STATE = 1, INPUT = 2, TEMP = 3 };

struct Tensor {
    uint32_t ty = 0;
    int64_t ne[4] = {1, 1, 1, 1};
    uint64_t nb[4] = {0, 0, 0, 0};
    std::string op = "NONE";
    int32_t op_params[16] = {0};
    int32_t src[10] = {-1, -1, -1, -1, -1, -1, -1, -1, -1, -1};
    int32_t view_src = -1;
    uint64_t view_offs = 0;
    uint32_t storage_kind = TEMP;
    uint32_t storage_index = 0;
    std::string name;
    // executor-internal: byte size override for opaque scratch tensors (quantized activations)
    uint64_t opaque_bytes = 0;

    int64_t nelements() const { return ne[0] * ne[1] * ne[2] * ne[3]; }
    int64_t nrows() const { return ne[1] * ne[2] * ne[3]; }
    uint64_t nbytes() const;
    uint64_t row_size() const;
    bool is_contiguous() const { return is_contiguous_n(0); }
    bool is_contiguous_n(int n) const;
    bool is_contiguous_rows() const;
    bool is_view_op() const {
        return op == "NONE" || op == "RESHAPE" || op == "VIEW" || op == "TRANSPOSE" || op == "PERMUTE";
    }
    float param_f32(int i) const {
        float f;
        std::memcpy(&f, &op_params[i], 4);
        return f;
    }
};

struct Graph {
    std::vector<Tensor> tensors;
    std::vector<int32_t> nodes;
    std::vector<int32_t> keep;
    int32_t root(int32_t id, uint64_t *offs = nullptr) const {
        const Tensor &t = tensors[id];
        if (t.view_src >= 0) {
            if (offs) *offs = t.view_offs;
            return t.view_src;
        }
        if (offs) *offs = 0;
        return id;
    }
};

// ---------------------------------------------------------------------------- plan
constexpr uint64_t ALIGN = 256;
inline uint64_t align_up(uint64_t n) { return (n + ALIGN - 1) / ALIGN * ALIGN; }

enum BufKind : uint8_t { BUF_WEIGHTS = 0, BUF_STATE = 1, BUF_IO = 2, BUF_ARENA = 3 };
struct Place {
    BufKind buf = BUF_ARENA;
    uint32_t index = 0;  // weights buffer index
    uint64_t off = 0;
};

struct Layout {
    std::vector<Place> place;                          // per tensor, views included
    uint64_t arena_size = 0, io_size = 0;
    std::vector<std::pair<uint64_t, uint64_t>> inputs;  // per input: offset, bytes in the io buffer
    std::vector<int64_t> scratch;                       // per node position: arena offset or -1
};

struct Leaves {
    std::vector<std::pair<uint32_t, uint64_t>> weights;
    std::vector<uint64_t> states;
};

Layout plan(const Graph &g, const Leaves &leaves, const std::function<uint64_t(int32_t)> &scratch_bytes);

// ---------------------------------------------------------------------------- device objects
struct Comm;  // NCCL communicator wrapper (comm.cpp)

}  // namespace tlb

struct tlb_device {
    int ordinal = 0;
    cudaStream_t stream = nullptr;
    cudaDeviceProp prop{};
    std::string name;
    tlb::Comm *comm = nullptr;
    // Bumped whenever the communicator changes (tlb_comm_init, tlb_comm_p2p_import, tlb_comm_destroy). The launches of
    // a captured CUDA graph have the communicator's state baked in (which all-reduce path, the peers' mapped
    // pointers), so the generation is part of the key a captured graph is replayed under.
    uint64_t comm_generation = 0;
};

struct tlb_buffer {
    tlb_device *dev = nullptr;
    int ordinal = 0;  // kept so a buffer can still be freed after its device handle was closed
    void *ptr = nullptr;
    uint64_t size = 0;
};

namespace tlb {

// What a launch sees at run time: base pointers of the four buffer kinds.
struct RunCtx {
    std::vector<char *> weights;
    char *state = nullptr;
    char *io = nullptr;
    char *arena = nullptr;
    cudaStream_t stream = nullptr;
    tlb_device *dev = nullptr;
    int *err = nullptr;  // device error word written by kernels whose bounded waits gave up
    char *at(const Place &p) const {
        switch (p.buf) {
            case BUF_WEIGHTS: return weights[p.index] + p.off;
            case BUF_STATE: return state + p.off;
            case BUF_IO: return io + p.off;
            default: return arena + p.off;
        }
    }
};

struct Dispatch {
    std::string label;
    std::function<cudaError_t(const RunCtx &)> fn;
};

// lower.cpp: one node -> launches; throws Unsupported
struct LowerCtx {
    tlb_device *dev;
    const Graph *g;
    const Layout *layout;
};
void lower_node(const LowerCtx &c, int32_t id, int pos, std::vector<Dispatch> &out);
uint64_t node_scratch_bytes(const Graph &g, int32_t id, int sm_count);
// comm.cu: sum over the ranks of the device's communicator, in place (no-op without one)
// (err: the device error word of bounded waits; the peer-memory path needs it, NCCL is used without it)
// partial / n_split: the input is the sum of n_split partial results (n floats each) instead of buf; only the
// peer-memory path takes that form (ask comm_p2p_takes first)
cudaError_t comm_allreduce_f32(tlb_device *dev, float *buf, size_t n, cudaStream_t st, int *err, const float *partial = nullptr, int n_split = 0);
bool comm_p2p_takes(tlb_device *dev, size_t n);
struct RowQuantArgs;
cudaError_t comm_exchange_row_quant(tlb_device *dev, float *data, const float *partial, int n_split, const RowQuantArgs &p, cudaStream_t st,
                                    int *err);
int comm_ranks(tlb_device *dev);
// IR rewrites before planning (fusion, shared activation quantization); fuse.cpp
void rewrite_graph(Graph &g);

}  // namespace tlb

struct tlb_program {
    tlb_device *dev = nullptr;
    int ordinal = 0;
    tlb::Graph graph;
    tlb::Layout layout;
    std::vector<tlb::Dispatch> dispatches;
    void *arena = nullptr;
    void *io = nullptr;
    uint32_t n_user_tensors = 0;
    // one captured CUDA graph per (weights, state) pointer set
    struct Captured {
        std::vector<void *> key;
        cudaGraphExec_t exec = nullptr;
    };
    std::vector<Captured> captured;
    uint32_t kernel_nodes = 0;   // kernel launches in the most recently captured graph
    bool use_graph = true;
};
