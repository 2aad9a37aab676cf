// C ABI of include/tlb200.h: device, buffers, graph IR, arena planner and program replay.
// Reference counterparts: crates/kernels/src/cuda/mod.rs (Device/Buffer), graph.rs (IR),
// plan.rs (planner), cuda/exec.rs (Executor::compile, Program::run/read).
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "kernels.h"
#include "tlb_internal.h"

namespace tlb {

static thread_local std::string g_last_error;
void set_error(const std::string &msg) { g_last_error = msg; }
tlb_status fail(tlb_status st, const std::string &msg) {
    g_last_error = msg;
    return st;
}
std::string cuda_msg(cudaError_t e) { return std::string(cudaGetErrorName(e)) + ": " + cudaGetErrorString(e); }

// ---------------------------------------------------------------------------- type table
// crates/kernels/src/graph.rs:30-50
const TypeTraits *type_traits(uint32_t ty) {
    static const TypeTraits f32{"f32", 1, 4}, f16{"f16", 1, 2}, q4_0{"q4_0", 32, 18}, q4_1{"q4_1", 32, 20},
        q5_0{"q5_0", 32, 22}, q5_1{"q5_1", 32, 24}, q8_0{"q8_0", 32, 34}, q2_K{"q2_K", 256, 84}, q3_K{"q3_K", 256, 110},
        q4_K{"q4_K", 256, 144}, q5_K{"q5_K", 256, 176}, q6_K{"q6_K", 256, 210}, i8{"i8", 1, 1}, i16{"i16", 1, 2},
        i32{"i32", 1, 4}, i64{"i64", 1, 8}, bf16{"bf16", 1, 2};
    switch (ty) {
        case 0: return &f32;
        case 1: return &f16;
        case 2: return &q4_0;
        case 3: return &q4_1;
        case 6: return &q5_0;
        case 7: return &q5_1;
        case 8: return &q8_0;
        case 10: return &q2_K;
        case 11: return &q3_K;
        case 12: return &q4_K;
        case 13: return &q5_K;
        case 14: return &q6_K;
        case 24: return &i8;
        case 25: return &i16;
        case 26: return &i32;
        case 27: return &i64;
        case 30: return &bf16;
        default: return nullptr;
    }
}

// ggml_nbytes (graph.rs:112-129)
uint64_t Tensor::nbytes() const {
    if (opaque_bytes) return opaque_bytes;
    for (int i = 0; i < 4; i++)
        if (ne[i] == 0) return 0;
    const TypeTraits *tr = type_traits(ty);
    if (!tr) return 0;
    uint64_t n;
    if (tr->blck == 1) {
        n = tr->size + (uint64_t)(ne[0] - 1) * nb[0];
    } else {
        n = (uint64_t)ne[0] * nb[0] / (uint64_t)tr->blck;
    }
    for (int i = 1; i < 4; i++) n += (uint64_t)(ne[i] - 1) * nb[i];
    return n;
}
uint64_t Tensor::row_size() const {
    const TypeTraits *tr = type_traits(ty);
    return tr ? tr->size * (uint64_t)ne[0] / (uint64_t)tr->blck : 0;
}
bool Tensor::is_contiguous_rows() const {
    const TypeTraits *tr = type_traits(ty);
    return tr && nb[0] == tr->size;
}
// ggml_is_contiguous_n (graph.rs:147-171)
bool Tensor::is_contiguous_n(int n) const {
    for (int i = 0; i < 4; i++)
        if (ne[i] == 0) return true;
    const TypeTraits *tr = type_traits(ty);
    if (!tr) return false;
    if (ne[0] != tr->blck && nb[0] != tr->size) return false;
    uint64_t next = tr->size * (uint64_t)ne[0] / (uint64_t)tr->blck;
    for (int i = 1; i < 4; i++) {
        if (ne[i] != 1) {
            if (i > n) {
                if (nb[i] != next) return false;
                next *= (uint64_t)ne[i];
            } else {
                next = (uint64_t)ne[i] * nb[i];
            }
        }
    }
    return true;
}

// ---------------------------------------------------------------------------- planner
// crates/kernels/src/plan.rs:56-189: liveness of arena roots in node positions, first-fit by start
// time over the lowest free offset, one short-lived scratch block per node that asks for one,
// inputs in their own io buffer, views resolved through their root.
Layout plan(const Graph &g, const Leaves &leaves, const std::function<uint64_t(int32_t)> &scratch_bytes) {
    const size_t n = g.nodes.size(), nt = g.tensors.size();
    std::vector<size_t> first(nt, SIZE_MAX), last(nt, 0);
    auto touch = [&](int32_t root, size_t pos) {
        first[root] = std::min(first[root], pos);
        last[root] = std::max(last[root], pos);
    };
    for (size_t pos = 0; pos < n; pos++) {
        const Tensor &t = g.tensors[g.nodes[pos]];
        touch(g.root(g.nodes[pos]), pos);
        for (int s : t.src)
            if (s >= 0) touch(g.root(s), pos);
    }
    for (int32_t id : g.keep) last[g.root(id)] = n;

    struct Block {
        int32_t id;
        size_t first, last;
        uint64_t size;
        bool scratch;
        size_t pos;
    };
    std::vector<Block> blocks;
    for (size_t id = 0; id < nt; id++) {
        const Tensor &t = g.tensors[id];
        if (t.view_src < 0 && t.storage_kind == TEMP && first[id] != SIZE_MAX)
            blocks.push_back({(int32_t)id, first[id], last[id], align_up(std::max<uint64_t>(t.nbytes(), 1)), false, 0});
    }
    for (size_t pos = 0; pos < n; pos++) {
        const uint64_t bytes = scratch_bytes(g.nodes[pos]);
        // a scratch block outlives its node by two positions: the exchange that follows a K-split mul_mat,
        // or the row quantizer that took the exchange in, reads the partial sums itself
        if (bytes > 0) blocks.push_back({g.nodes[pos], pos, std::min(pos + 2, n - 1), align_up(bytes), true, pos});
    }
    std::stable_sort(blocks.begin(), blocks.end(), [](const Block &a, const Block &b) {
        if (a.first != b.first) return a.first < b.first;
        return a.scratch < b.scratch;
    });

    struct Live {
        uint64_t off, size;
        size_t last;
    };
    std::vector<Live> live;
    Layout L;
    std::vector<uint64_t> offsets(nt, 0);
    L.scratch.assign(n, -1);
    for (const Block &b : blocks) {
        live.erase(std::remove_if(live.begin(), live.end(), [&](const Live &l) { return l.last < b.first; }), live.end());
        std::sort(live.begin(), live.end(), [](const Live &x, const Live &y) { return x.off < y.off; });
        uint64_t off = 0;
        for (const Live &l : live) {
            if (l.off >= off + b.size) break;
            off = std::max(off, l.off + l.size);
        }
        live.push_back({off, b.size, b.last});
        L.arena_size = std::max(L.arena_size, off + b.size);
        if (b.scratch) L.scratch[b.pos] = (int64_t)off;
        else offsets[b.id] = off;
    }

    for (const Tensor &t : g.tensors) {
        if (t.view_src < 0 && t.storage_kind == INPUT) {
            if (L.inputs.size() <= t.storage_index) L.inputs.resize(t.storage_index + 1, {0, 0});
        }
    }
    // io offsets in input-index order so set_input(i) is independent of tensor order
    std::vector<uint64_t> in_bytes(L.inputs.size(), 0);
    for (const Tensor &t : g.tensors)
        if (t.view_src < 0 && t.storage_kind == INPUT) in_bytes[t.storage_index] = t.nbytes();
    for (size_t i = 0; i < L.inputs.size(); i++) {
        L.inputs[i] = {L.io_size, in_bytes[i]};
        L.io_size += align_up(std::max<uint64_t>(in_bytes[i], 1));
    }

    L.place.resize(nt);
    for (size_t id = 0; id < nt; id++) {
        uint64_t extra = 0;
        const int32_t root = g.root((int32_t)id, &extra);
        const Tensor &t = g.tensors[root];
        Place p;
        switch (t.storage_kind) {
            case WEIGHT:
                p.buf = BUF_WEIGHTS;
                p.index = leaves.weights[t.storage_index].first;
                p.off = leaves.weights[t.storage_index].second;
                break;
            case STATE:
                p.buf = BUF_STATE;
                p.off = leaves.states[t.storage_index];
                break;
            case INPUT:
                p.buf = BUF_IO;
                p.off = L.inputs[t.storage_index].first;
                break;
            default:
                p.buf = BUF_ARENA;
                p.off = offsets[root];
        }
        p.off += extra;
        L.place[id] = p;
    }
    return L;
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) applies to the device that is current when it is called, so the
// kernels are configured once per ordinal, with that ordinal current.
static std::mutex g_configure_mutex;
static uint64_t g_configured_ordinals = 0;   // bit per ordinal (a box has at most 64 GPUs)
static void configure_kernels_once(int ordinal) {
    std::lock_guard<std::mutex> lock(g_configure_mutex);
    const uint64_t bit = 1ull << (ordinal & 63);
    if (g_configured_ordinals & bit) return;
    gemv_configure();
    attn_configure();
    mmq_tc_configure();
    mmq_tc8_configure();
    flash_tc_configure();
    g_configured_ordinals |= bit;
}

}  // namespace tlb

using namespace tlb;

#define TLB_TRY_CUDA(expr, st)                                          \
    do {                                                                \
        cudaError_t e__ = (expr);                                       \
        if (e__ != cudaSuccess) return fail(st, std::string(#expr) + " failed: " + cuda_msg(e__)); \
    } while (0)

extern "C" {

const char *tlb_last_error(void) { return g_last_error.c_str(); }

uint64_t tlb_row_size(uint32_t type, int64_t ne0) {
    const TypeTraits *tr = type_traits(type);
    if (!tr || ne0 < 0 || ne0 % tr->blck != 0) return 0;
    return tr->size * (uint64_t)ne0 / (uint64_t)tr->blck;
}

// ------------------------------------------------------------------ device
tlb_status tlb_device_open(int ordinal, tlb_device **dev) {
    if (!dev) return fail(TLB_INVALID, "tlb_device_open: null output");
    *dev = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        cudaGetLastError();
        return fail(TLB_NO_DEVICE, "no GPU device available");
    }
    if (ordinal < 0 || ordinal >= count) return fail(TLB_NO_DEVICE, "no GPU device with ordinal " + std::to_string(ordinal));
    TLB_TRY_CUDA(cudaSetDevice(ordinal), TLB_NO_DEVICE);
    tlb_device *d = new tlb_device;
    d->ordinal = ordinal;
    e = cudaGetDeviceProperties(&d->prop, ordinal);
    if (e != cudaSuccess) {
        delete d;
        return fail(TLB_NO_DEVICE, "cudaGetDeviceProperties: " + cuda_msg(e));
    }
    if (d->prop.major != 10) {
        const std::string m = "this library is built for sm_100a only; device " + std::string(d->prop.name) + " is sm_" +
                              std::to_string(d->prop.major) + std::to_string(d->prop.minor);
        delete d;
        return fail(TLB_NO_DEVICE, m);
    }
    e = cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
        delete d;
        return fail(TLB_NO_DEVICE, "cudaStreamCreate: " + cuda_msg(e));
    }
    d->name = std::string("native ") + d->prop.name;
    configure_kernels_once(ordinal);   // cudaSetDevice(ordinal) above made it current
    *dev = d;
    return TLB_OK;
}

void tlb_device_close(tlb_device *dev) {
    if (!dev) return;
    tlb_comm_destroy(dev);
    cudaSetDevice(dev->ordinal);
    if (dev->stream) cudaStreamDestroy(dev->stream);
    delete dev;
}

tlb_status tlb_device_name(tlb_device *dev, char *out, size_t n) {
    if (!dev || !out || n == 0) return fail(TLB_INVALID, "tlb_device_name: bad arguments");
    snprintf(out, n, "%s", dev->name.c_str());
    return TLB_OK;
}

tlb_status tlb_device_sync(tlb_device *dev) {
    if (!dev) return fail(TLB_INVALID, "null device");
    cudaSetDevice(dev->ordinal);
    TLB_TRY_CUDA(cudaStreamSynchronize(dev->stream), TLB_EXECUTION);
    return TLB_OK;
}

void *tlb_device_stream(tlb_device *dev) { return dev ? (void *)dev->stream : nullptr; }
int tlb_device_sm_count(tlb_device *dev) { return dev ? dev->prop.multiProcessorCount : 0; }

// ------------------------------------------------------------------ buffers
static tlb_status buffer_create(tlb_device *dev, uint64_t bytes, bool zero, tlb_buffer **out) {
    if (!dev || !out) return fail(TLB_INVALID, "buffer create: bad arguments");
    *out = nullptr;
    cudaSetDevice(dev->ordinal);
    void *p = nullptr;
    const uint64_t n = std::max<uint64_t>(bytes, 1);
    cudaError_t e = cudaMalloc(&p, n);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(TLB_ALLOC, "buffer allocation of " + std::to_string(n) + " bytes failed");
    }
    if (zero) {
        e = cudaMemsetAsync(p, 0, n, dev->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(dev->stream);
        if (e != cudaSuccess) {
            cudaFree(p);
            return fail(TLB_EXECUTION, "zeroing a buffer failed: " + cuda_msg(e));
        }
    }
    tlb_buffer *b = new tlb_buffer;
    b->dev = dev;
    b->ordinal = dev->ordinal;
    b->ptr = p;
    b->size = n;
    *out = b;
    return TLB_OK;
}

tlb_status tlb_weights_create(tlb_device *dev, uint64_t total_bytes, tlb_buffer **w) { return buffer_create(dev, total_bytes, false, w); }
tlb_status tlb_state_create(tlb_device *dev, uint64_t bytes, tlb_buffer **s) { return buffer_create(dev, bytes, true, s); }

tlb_status tlb_state_zero(tlb_buffer *s) {
    if (!s) return fail(TLB_INVALID, "null buffer");
    cudaSetDevice(s->dev->ordinal);
    TLB_TRY_CUDA(cudaMemsetAsync(s->ptr, 0, s->size, s->dev->stream), TLB_EXECUTION);
    TLB_TRY_CUDA(cudaStreamSynchronize(s->dev->stream), TLB_EXECUTION);
    return TLB_OK;
}

tlb_status tlb_state_fork(tlb_buffer *src, tlb_buffer **copy) {
    if (!src || !copy) return fail(TLB_INVALID, "tlb_state_fork: bad arguments");
    tlb_status st = buffer_create(src->dev, src->size, false, copy);
    if (st != TLB_OK) return st;
    cudaError_t e = cudaMemcpyAsync((*copy)->ptr, src->ptr, src->size, cudaMemcpyDeviceToDevice, src->dev->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(src->dev->stream);
    if (e != cudaSuccess) {
        tlb_buffer_free(*copy);
        *copy = nullptr;
        return fail(TLB_EXECUTION, "copying a state block failed: " + cuda_msg(e));
    }
    return TLB_OK;
}

// copy_blocks of the reference (crates/kernels/src/cuda/paged_attn.rs:423-448): pages copied inside the K and V pools of
// one state block.
tlb_status tlb_state_copy_blocks(tlb_buffer *state, uint64_t k_pool_offset, uint64_t v_pool_offset, uint64_t pool_blocks, uint64_t bytes_per_block,
                                 const int64_t *pairs, uint32_t n_pairs) {
    if (!state || (!pairs && n_pairs)) return fail(TLB_INVALID, "tlb_state_copy_blocks: bad arguments");
    if (bytes_per_block == 0 || bytes_per_block % 16 || k_pool_offset % 16 || v_pool_offset % 16)
        return fail(TLB_INVALID, "tlb_state_copy_blocks: pools and pages must be multiples of 16 bytes");
    const uint64_t pool_bytes = pool_blocks * bytes_per_block;
    if (k_pool_offset > state->size || pool_bytes > state->size - k_pool_offset || v_pool_offset > state->size || pool_bytes > state->size - v_pool_offset)
        return fail(TLB_INVALID, "tlb_state_copy_blocks: a pool of " + std::to_string(pool_bytes) + " bytes does not fit the state block of " + std::to_string(state->size));
    for (uint32_t i = 0; i < 2 * n_pairs; i++)
        if (pairs[i] < 0 || (uint64_t)pairs[i] >= pool_blocks) return fail(TLB_INVALID, "tlb_state_copy_blocks: block " + std::to_string(pairs[i]) + " is outside a pool of " + std::to_string(pool_blocks) + " blocks");
    for (uint32_t i = 0; i < n_pairs; i++)
        for (uint32_t j = 0; j < n_pairs; j++)
            if (pairs[2 * i + 1] == pairs[2 * j] || (i != j && pairs[2 * i + 1] == pairs[2 * j + 1]))
                return fail(TLB_INVALID, "tlb_state_copy_blocks: block " + std::to_string(pairs[2 * i + 1]) + " is written and also read or written by another pair");
    if (n_pairs == 0) return TLB_OK;
    cudaSetDevice(state->dev->ordinal);
    int64_t *map = nullptr;
    if (cudaMalloc(&map, (size_t)n_pairs * 16) != cudaSuccess) {
        cudaGetLastError();
        return fail(TLB_ALLOC, "buffer allocation of " + std::to_string((size_t)n_pairs * 16) + " bytes failed");
    }
    cudaError_t e = cudaMemcpyAsync(map, pairs, (size_t)n_pairs * 16, cudaMemcpyHostToDevice, state->dev->stream);
    if (e == cudaSuccess)
        e = launch_copy_blocks((char *)state->ptr + k_pool_offset, (char *)state->ptr + v_pool_offset, map, (int)n_pairs, (int64_t)bytes_per_block, state->dev->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(state->dev->stream);
    cudaFree(map);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(TLB_EXECUTION, "copying cache pages failed: " + cuda_msg(e));
    }
    return TLB_OK;
}

// gather_kv_cache of the reference (crates/kernels/src/cuda/paged_attn.rs:450-509): the cached keys and values of some
// sequences, read page by page through their block tables, as dense f16 rows in host memory.
tlb_status tlb_state_gather_kv(tlb_buffer *state, uint64_t k_pool_offset, uint64_t v_pool_offset, uint64_t pool_blocks, uint32_t kv_heads,
                               uint32_t head_size, uint32_t block_size, const int32_t *tables, uint32_t max_blocks, const int32_t *lens,
                               uint32_t seqs, void *k_out, void *v_out) {
    if (!state || ((!tables || !lens) && seqs)) return fail(TLB_INVALID, "tlb_state_gather_kv: bad arguments");
    if (kv_heads == 0 || head_size == 0 || head_size % 8 || block_size == 0 || k_pool_offset % 16 || v_pool_offset % 16)
        return fail(TLB_INVALID, "tlb_state_gather_kv: the head size must be a multiple of 8, the block size at least 1, the pools 16-byte aligned");
    const uint64_t token_bytes = (uint64_t)kv_heads * head_size * 2, pool_bytes = pool_blocks * block_size * token_bytes;
    if (k_pool_offset > state->size || pool_bytes > state->size - k_pool_offset || v_pool_offset > state->size || pool_bytes > state->size - v_pool_offset)
        return fail(TLB_INVALID, "tlb_state_gather_kv: a pool of " + std::to_string(pool_bytes) + " bytes does not fit the state block of " + std::to_string(state->size));
    std::vector<int64_t> first(seqs + 1, 0);   // first output row of each sequence
    int64_t longest = 0;
    for (uint32_t s = 0; s < seqs; s++) {
        const int64_t n = lens[s];
        if (n < 0 || (uint64_t)n > (uint64_t)max_blocks * block_size)
            return fail(TLB_INVALID, "tlb_state_gather_kv: sequence " + std::to_string(s) + " has length " + std::to_string(n) + ", its table covers " +
                                         std::to_string((uint64_t)max_blocks * block_size));
        for (int64_t b = 0; b < (n + block_size - 1) / block_size; b++) {
            const int64_t blk = tables[(size_t)s * max_blocks + b];
            if (blk < 0 || (uint64_t)blk >= pool_blocks)
                return fail(TLB_INVALID, "tlb_state_gather_kv: block " + std::to_string(blk) + " of sequence " + std::to_string(s) + " is outside a pool of " +
                                             std::to_string(pool_blocks) + " blocks");
        }
        first[s + 1] = first[s] + n;
        longest = std::max(longest, n);
    }
    const uint64_t out_bytes = (uint64_t)first[seqs] * token_bytes;
    if (out_bytes == 0) return TLB_OK;
    if (!k_out || !v_out) return fail(TLB_INVALID, "tlb_state_gather_kv: null output");
    cudaSetDevice(state->dev->ordinal);
    cudaStream_t st = state->dev->stream;
    const size_t tab_bytes = (size_t)seqs * max_blocks * 4, len_bytes = (size_t)seqs * 4, first_bytes = (size_t)(seqs + 1) * 8;
    char *dev_mem = nullptr;   // tables | lens | first rows | keys | values, each 256-byte aligned
    auto up = [](size_t n) { return (n + 255) / 256 * 256; };
    const size_t o_len = up(tab_bytes), o_first = o_len + up(len_bytes), o_k = o_first + up(first_bytes), o_v = o_k + up(out_bytes), total = o_v + up(out_bytes);
    if (cudaMalloc(&dev_mem, total) != cudaSuccess) {
        cudaGetLastError();
        return fail(TLB_ALLOC, "buffer allocation of " + std::to_string(total) + " bytes failed");
    }
    cudaError_t e = cudaMemcpyAsync(dev_mem, tables, tab_bytes, cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dev_mem + o_len, lens, len_bytes, cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dev_mem + o_first, first.data(), first_bytes, cudaMemcpyHostToDevice, st);
    for (int which = 0; which < 2 && e == cudaSuccess; which++)
        e = launch_paged_gather((int)seqs, (int)kv_heads, (int)head_size, (int)block_size, (int)max_blocks,
                                (char *)state->ptr + (which ? v_pool_offset : k_pool_offset), (const int32_t *)dev_mem, (const int32_t *)(dev_mem + o_len),
                                (const int64_t *)(dev_mem + o_first), dev_mem + (which ? o_v : o_k), (int)longest, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(k_out, dev_mem + o_k, out_bytes, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(v_out, dev_mem + o_v, out_bytes, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    cudaFree(dev_mem);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(TLB_EXECUTION, "gathering cached keys and values failed: " + cuda_msg(e));
    }
    return TLB_OK;
}

tlb_status tlb_buffer_write(tlb_buffer *b, uint64_t offset, const void *host, uint64_t n) {
    if (!b || (!host && n)) return fail(TLB_INVALID, "tlb_buffer_write: bad arguments");
    if (offset > b->size || n > b->size - offset)
        return fail(TLB_INVALID, "write of " + std::to_string(n) + " bytes at " + std::to_string(offset) + " past a buffer of " + std::to_string(b->size));
    if (n == 0) return TLB_OK;
    cudaSetDevice(b->dev->ordinal);
    TLB_TRY_CUDA(cudaMemcpyAsync((char *)b->ptr + offset, host, n, cudaMemcpyHostToDevice, b->dev->stream), TLB_EXECUTION);
    TLB_TRY_CUDA(cudaStreamSynchronize(b->dev->stream), TLB_EXECUTION);
    return TLB_OK;
}

tlb_status tlb_buffer_read(tlb_buffer *b, uint64_t offset, void *host, uint64_t n) {
    if (!b || (!host && n)) return fail(TLB_INVALID, "tlb_buffer_read: bad arguments");
    if (offset > b->size || n > b->size - offset)
        return fail(TLB_INVALID, "read of " + std::to_string(n) + " bytes at " + std::to_string(offset) + " past a buffer of " + std::to_string(b->size));
    if (n == 0) return TLB_OK;
    cudaSetDevice(b->dev->ordinal);
    TLB_TRY_CUDA(cudaMemcpyAsync(host, (char *)b->ptr + offset, n, cudaMemcpyDeviceToHost, b->dev->stream), TLB_EXECUTION);
    TLB_TRY_CUDA(cudaStreamSynchronize(b->dev->stream), TLB_EXECUTION);
    return TLB_OK;
}

tlb_status tlb_buffer_copy_device(tlb_buffer *b, uint64_t offset, const void *device_src, uint64_t n) {
    if (!b || (!device_src && n)) return fail(TLB_INVALID, "tlb_buffer_copy_device: bad arguments");
    if (offset > b->size || n > b->size - offset)
        return fail(TLB_INVALID, "write of " + std::to_string(n) + " bytes at " + std::to_string(offset) + " past a buffer of " + std::to_string(b->size));
    if (n == 0) return TLB_OK;
    cudaSetDevice(b->dev->ordinal);
    TLB_TRY_CUDA(cudaMemcpyAsync((char *)b->ptr + offset, device_src, n, cudaMemcpyDeviceToDevice, b->dev->stream), TLB_EXECUTION);
    TLB_TRY_CUDA(cudaStreamSynchronize(b->dev->stream), TLB_EXECUTION);
    return TLB_OK;
}

uint64_t tlb_buffer_size(tlb_buffer *b) { return b ? b->size : 0; }
void *tlb_buffer_device_ptr(tlb_buffer *b) { return b ? b->ptr : nullptr; }
void tlb_buffer_free(tlb_buffer *b) {
    if (!b) return;
    cudaSetDevice(b->ordinal);
    cudaFree(b->ptr);
    delete b;
}

// Copies and validates the IR of a caller (tensor ids in range, views of roots only, known types, leaves present).
// Returns an empty string, or what is wrong.
static std::string import_graph(const tlb_graph *graph, const tlb_leaves *leaves, Graph &g, Leaves &lv) {
    g.tensors.resize(graph->n_tensors);
    const int32_t nt = (int32_t)graph->n_tensors;
    for (int32_t i = 0; i < nt; i++) {
        const tlb_tensor &s = graph->tensors[i];
        Tensor &t = g.tensors[i];
        t.ty = s.ty;
        for (int k = 0; k < 4; k++) {
            t.ne[k] = s.ne[k];
            t.nb[k] = s.nb[k];
            if (s.ne[k] < 0) return "tensor " + std::to_string(i) + " has a negative dimension";
        }
        t.op.assign(s.op, strnlen(s.op, sizeof(s.op)));
        std::memcpy(t.op_params, s.op_params, sizeof(t.op_params));
        for (int k = 0; k < 10; k++) {
            t.src[k] = s.src[k];
            if (s.src[k] >= nt || s.src[k] < -1) return "tensor " + std::to_string(i) + " has a source out of range";
        }
        t.view_src = s.view_src;
        if (s.view_src >= nt || s.view_src < -1) return "tensor " + std::to_string(i) + " has a view source out of range";
        t.view_offs = s.view_offs;
        t.storage_kind = s.storage_kind;
        t.storage_index = s.storage_index;
        t.name.assign(s.name, strnlen(s.name, sizeof(s.name)));
        if (!type_traits(t.ty)) return "tensor `" + t.name + "` has unknown ggml type " + std::to_string(t.ty);
        if (t.storage_kind > TEMP) return "tensor `" + t.name + "` has an unknown storage kind";
    }
    for (int32_t i = 0; i < nt; i++) {
        const Tensor &t = g.tensors[i];
        if (t.view_src >= 0 && g.tensors[t.view_src].view_src >= 0) return "tensor `" + t.name + "`: view_src must be a root";
        if (t.view_src < 0) {
            if (t.storage_kind == WEIGHT && (!leaves || t.storage_index >= leaves->n_weights))
                return "tensor `" + t.name + "` names weight " + std::to_string(t.storage_index) + ", which the leaves do not have";
            if (t.storage_kind == STATE && (!leaves || t.storage_index >= leaves->n_states))
                return "tensor `" + t.name + "` names state " + std::to_string(t.storage_index) + ", which the leaves do not have";
        }
    }
    for (uint32_t i = 0; i < graph->n_nodes; i++) {
        if (graph->nodes[i] < 0 || graph->nodes[i] >= nt) return "node id out of range";
        g.nodes.push_back(graph->nodes[i]);
    }
    for (uint32_t i = 0; i < graph->n_keep; i++) {
        if (graph->keep[i] < 0 || graph->keep[i] >= nt) return "kept tensor id out of range";
        g.keep.push_back(graph->keep[i]);
    }
    if (leaves) {
        for (uint32_t i = 0; i < leaves->n_weights; i++) lv.weights.push_back({leaves->weight_buffer[i], leaves->weight_offset[i]});
        for (uint32_t i = 0; i < leaves->n_states; i++) lv.states.push_back(leaves->state_offset[i]);
    }
    return "";
}

// ------------------------------------------------------------------ programs
static void copy_err(const std::string &m, char *err, size_t errlen) {
    if (err && errlen) snprintf(err, errlen, "%s", m.c_str());
}

tlb_status tlb_program_compile(tlb_device *dev, const tlb_graph *graph, const tlb_leaves *leaves, tlb_program **prog,
                               char *err, size_t errlen) {
    if (err && errlen) err[0] = 0;
    auto bad = [&](tlb_status st, const std::string &m) {
        copy_err(m, err, errlen);
        return fail(st, m);
    };
    if (!dev || !graph || !prog) return bad(TLB_INVALID, "tlb_program_compile: bad arguments");
    *prog = nullptr;
    Graph g;
    Leaves lv;
    {
        const std::string why = import_graph(graph, leaves, g, lv);
        if (!why.empty()) return bad(TLB_INVALID, why);
    }

    tlb_program *p = new tlb_program;
    p->dev = dev;
    p->ordinal = dev->ordinal;
    p->n_user_tensors = graph->n_tensors;
    p->graph = std::move(g);
    rewrite_graph(p->graph);   // TL_NATIVE_NOFUSE turns the fusions off inside; the shared activation quantizers always go in
    const int sm = dev->prop.multiProcessorCount;
    const Graph &G = p->graph;
    p->layout = plan(G, lv, [&](int32_t id) { return node_scratch_bytes(G, id, sm); });

    // ---- lower every node before failing, so one compile reports every missing op (exec.rs:39-58)
    struct Missing {
        std::string op;
        int count;
        std::string detail;
    };
    std::vector<Missing> missing;
    LowerCtx lc{dev, &p->graph, &p->layout};
    for (size_t pos = 0; pos < G.nodes.size(); pos++) {
        try {
            lower_node(lc, G.nodes[pos], (int)pos, p->dispatches);
        } catch (const Unsupported &u) {
            bool found = false;
            for (Missing &m : missing)
                if (m.op == u.op) {
                    m.count++;
                    found = true;
                }
            if (!found) missing.push_back({u.op, 1, u.node + ": " + u.why});
        } catch (const std::string &m) {
            delete p;
            return bad(TLB_INVALID, m);
        }
    }
    if (!missing.empty()) {
        std::string m = "native CUDA: not implemented: ";
        for (size_t i = 0; i < missing.size(); i++) {
            if (i) m += "; ";
            m += missing[i].op + " x" + std::to_string(missing[i].count) + " (e.g. " + missing[i].detail + ")";
        }
        delete p;
        return bad(TLB_UNSUPPORTED, m);
    }
    cudaSetDevice(dev->ordinal);
    cudaError_t e = cudaMalloc(&p->arena, std::max<uint64_t>(p->layout.arena_size, 1) + 256);
    if (e == cudaSuccess) e = cudaMalloc(&p->io, std::max<uint64_t>(p->layout.io_size, 1));
    if (e != cudaSuccess) {
        cudaGetLastError();
        const uint64_t want = p->layout.arena_size + p->layout.io_size;
        tlb_program_free(p);
        return bad(TLB_ALLOC, "buffer allocation of " + std::to_string(want) + " bytes failed");
    }
    // the last 256 bytes of the arena allocation hold the device error word of bounded waits
    cudaMemsetAsync((char *)p->arena + std::max<uint64_t>(p->layout.arena_size, 1), 0, 256, dev->stream);
    cudaStreamSynchronize(dev->stream);
    const char *ng = getenv("TLB_NO_CUDA_GRAPH");
    p->use_graph = !(ng && ng[0] == '1');
    *prog = p;
    return TLB_OK;
}

// The planner alone, for tests that check its invariants on graphs no kernel could run: no device, no lowering, no
// rewrites. node_scratch[i] (may be NULL) is the scratch node i asks for. Per tensor: the buffer kind it resolves to
// (0 weights, 1 state, 2 io, 3 arena) and its byte offset there; per node: the offset of its scratch block or -1.
tlb_status tlb_plan_only(const tlb_graph *graph, const tlb_leaves *leaves, const uint64_t *node_scratch, uint64_t *arena_size, uint64_t *io_size,
                         uint8_t *tensor_buffer, uint64_t *tensor_offset, int64_t *scratch_offset) {
    if (!graph || !arena_size || !io_size || !tensor_buffer || !tensor_offset || !scratch_offset) return fail(TLB_INVALID, "tlb_plan_only: bad arguments");
    Graph g;
    Leaves lv;
    const std::string why = import_graph(graph, leaves, g, lv);
    if (!why.empty()) return fail(TLB_INVALID, why);
    std::vector<uint64_t> want(g.tensors.size(), 0);
    if (node_scratch)
        for (size_t pos = 0; pos < g.nodes.size(); pos++) want[g.nodes[pos]] = node_scratch[pos];
    const Layout L = plan(g, lv, [&](int32_t id) { return want[id]; });
    *arena_size = L.arena_size;
    *io_size = L.io_size;
    for (size_t i = 0; i < g.tensors.size(); i++) {
        tensor_buffer[i] = (uint8_t)L.place[i].buf;
        tensor_offset[i] = L.place[i].off;
    }
    for (size_t pos = 0; pos < g.nodes.size(); pos++) scratch_offset[pos] = L.scratch[pos];
    return TLB_OK;
}

void tlb_program_free(tlb_program *prog) {
    if (!prog) return;
    cudaSetDevice(prog->ordinal);
    for (auto &c : prog->captured)
        if (c.exec) cudaGraphExecDestroy(c.exec);
    if (prog->arena) cudaFree(prog->arena);
    if (prog->io) cudaFree(prog->io);
    delete prog;
}

tlb_status tlb_program_set_input(tlb_program *prog, uint32_t i, const void *bytes, uint64_t n) {
    if (!prog) return fail(TLB_INVALID, "null program");
    if (i >= prog->layout.inputs.size()) return fail(TLB_INVALID, "no graph input " + std::to_string(i));
    const auto in = prog->layout.inputs[i];
    if (n != in.second) return fail(TLB_INVALID, "input " + std::to_string(i) + " takes " + std::to_string(in.second) + " bytes, got " + std::to_string(n));
    if (n == 0) return TLB_OK;
    if (!bytes) return fail(TLB_INVALID, "null input data");
    cudaSetDevice(prog->dev->ordinal);
    TLB_TRY_CUDA(cudaMemcpyAsync((char *)prog->io + in.first, bytes, n, cudaMemcpyHostToDevice, prog->dev->stream), TLB_EXECUTION);
    TLB_TRY_CUDA(cudaStreamSynchronize(prog->dev->stream), TLB_EXECUTION);
    return TLB_OK;
}

// Device-side feedback: the bytes of a kept arena tensor become the next run's input, without the host (a decode loop
// feeds the ARGMAX of one step to the GET_ROWS of the next). Enqueued on the device stream, not waited for.
tlb_status tlb_program_feed_input(tlb_program *prog, uint32_t input, uint32_t tensor_id) {
    if (!prog) return fail(TLB_INVALID, "null program");
    if (input >= prog->layout.inputs.size()) return fail(TLB_INVALID, "no graph input " + std::to_string(input));
    if (tensor_id >= prog->n_user_tensors) return fail(TLB_INVALID, "no tensor " + std::to_string(tensor_id));
    const Place pl = prog->layout.place[tensor_id];
    const auto in = prog->layout.inputs[input];
    const uint64_t n = prog->graph.tensors[tensor_id].nbytes();
    if (pl.buf != BUF_ARENA) return fail(TLB_INVALID, "tensor " + std::to_string(tensor_id) + " does not live in the arena");
    if (n != in.second) return fail(TLB_INVALID, "input " + std::to_string(input) + " takes " + std::to_string(in.second) + " bytes, got " + std::to_string(n));
    bool kept = false;
    for (int32_t k : prog->graph.keep) kept = kept || (uint32_t)k == tensor_id;
    if (!kept) return fail(TLB_INVALID, "tensor " + std::to_string(tensor_id) + " is not kept: its bytes may be reused before the run ends");
    if (n == 0) return TLB_OK;
    cudaSetDevice(prog->dev->ordinal);
    TLB_TRY_CUDA(cudaMemcpyAsync((char *)prog->io + in.first, (char *)prog->arena + pl.off, n, cudaMemcpyDeviceToDevice, prog->dev->stream), TLB_EXECUTION);
    return TLB_OK;
}

static tlb_status make_ctx(tlb_program *prog, tlb_buffer *const *weights, uint32_t n_weights, tlb_buffer *state, RunCtx &rc) {
    uint32_t need_w = 0;
    bool need_state = false;
    for (const Place &pl : prog->layout.place) {
        if (pl.buf == BUF_WEIGHTS) need_w = std::max(need_w, pl.index + 1);
        if (pl.buf == BUF_STATE) need_state = true;
    }
    if (need_w > n_weights) return fail(TLB_INVALID, "the program reads weight buffer " + std::to_string(need_w - 1) + " but only " + std::to_string(n_weights) + " were given");
    if (need_state && !state) return fail(TLB_INVALID, "the program reads state tensors but no state block was given");
    for (uint32_t i = 0; i < n_weights; i++) {
        if (!weights[i]) return fail(TLB_INVALID, "null weight buffer");
        rc.weights.push_back((char *)weights[i]->ptr);
    }
    rc.state = state ? (char *)state->ptr : nullptr;
    rc.io = (char *)prog->io;
    rc.arena = (char *)prog->arena;
    rc.stream = prog->dev->stream;
    rc.dev = prog->dev;
    rc.err = (int *)((char *)prog->arena + std::max<uint64_t>(prog->layout.arena_size, 1));
    return TLB_OK;
}

static tlb_status launch_all(tlb_program *prog, const RunCtx &rc, bool profile) {
    for (const Dispatch &d : prog->dispatches) {
        cudaError_t e = d.fn(rc);
        if (e == cudaSuccess && profile) e = cudaStreamSynchronize(rc.stream);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return fail(TLB_EXECUTION, "launching `" + d.label + "`: " + cuda_msg(e));
        }
    }
    return TLB_OK;
}

tlb_status tlb_program_enqueue(tlb_program *prog, tlb_buffer *const *weights, uint32_t n_weights, tlb_buffer *state) {
    if (!prog) return fail(TLB_INVALID, "null program");
    cudaSetDevice(prog->dev->ordinal);
    cudaGetLastError();  // a stale error of an unrelated earlier call must not be blamed on a launch
    RunCtx rc;
    tlb_status st = make_ctx(prog, weights, n_weights, state, rc);
    if (st != TLB_OK) return st;
    const bool profile = getenv("TL_NATIVE_PROFILE") != nullptr;
    if (!prog->use_graph || profile || prog->dispatches.size() < 2) return launch_all(prog, rc, profile);
    // replay a captured CUDA graph, one per set of buffer addresses (sessions switch state blocks)
    std::vector<void *> key;
    for (char *w : rc.weights) key.push_back(w);
    key.push_back(rc.state);
    key.push_back((void *)(uintptr_t)prog->dev->comm_generation);   // the launches bake the communicator's state in
    for (auto &c : prog->captured)
        if (c.key == key) {
            TLB_TRY_CUDA(cudaGraphLaunch(c.exec, rc.stream), TLB_EXECUTION);
            return TLB_OK;
        }
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamBeginCapture(rc.stream, cudaStreamCaptureModeThreadLocal);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return launch_all(prog, rc, false);
    }
    st = launch_all(prog, rc, false);
    e = cudaStreamEndCapture(rc.stream, &graph);
    if (st != TLB_OK || e != cudaSuccess || !graph) {
        cudaGetLastError();
        if (graph) cudaGraphDestroy(graph);
        if (st != TLB_OK) return st;
        prog->use_graph = false;
        return launch_all(prog, rc, false);
    }
    {   // how many kernels one run of the program launches (tlb_program_kernel_count)
        size_t n_nodes = 0;
        prog->kernel_nodes = 0;
        if (cudaGraphGetNodes(graph, nullptr, &n_nodes) == cudaSuccess && n_nodes > 0) {
            std::vector<cudaGraphNode_t> nodes(n_nodes);
            if (cudaGraphGetNodes(graph, nodes.data(), &n_nodes) == cudaSuccess)
                for (size_t i = 0; i < n_nodes; i++) {
                    cudaGraphNodeType ty;
                    if (cudaGraphNodeGetType(nodes[i], &ty) == cudaSuccess && ty == cudaGraphNodeTypeKernel) prog->kernel_nodes++;
                }
        }
        cudaGetLastError();
    }
    cudaGraphExec_t exec = nullptr;
    e = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) {
        cudaGetLastError();
        prog->use_graph = false;
        return launch_all(prog, rc, false);
    }
    if (prog->captured.size() >= 8) {
        cudaGraphExecDestroy(prog->captured.front().exec);
        prog->captured.erase(prog->captured.begin());
    }
    prog->captured.push_back({key, exec});
    TLB_TRY_CUDA(cudaGraphLaunch(exec, rc.stream), TLB_EXECUTION);
    return TLB_OK;
}

tlb_status tlb_program_profile(tlb_program *prog, tlb_buffer *const *weights, uint32_t n_weights, tlb_buffer *state,
                               float *ms, uint32_t n) {
    if (!prog || (!ms && n)) return fail(TLB_INVALID, "tlb_program_profile: bad arguments");
    if (n != prog->dispatches.size()) return fail(TLB_INVALID, "the program has " + std::to_string(prog->dispatches.size()) + " launches, room for " + std::to_string(n));
    cudaSetDevice(prog->dev->ordinal);
    cudaGetLastError();
    RunCtx rc;
    tlb_status st = make_ctx(prog, weights, n_weights, state, rc);
    if (st != TLB_OK) return st;
    std::vector<cudaEvent_t> ev(n + 1);
    for (auto &e : ev) TLB_TRY_CUDA(cudaEventCreate(&e), TLB_EXECUTION);
    cudaError_t e = cudaEventRecord(ev[0], rc.stream);
    std::string where;
    for (uint32_t i = 0; i < n && e == cudaSuccess; i++) {
        e = prog->dispatches[i].fn(rc);
        if (e == cudaSuccess) e = cudaEventRecord(ev[i + 1], rc.stream);
        else where = prog->dispatches[i].label;
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(rc.stream);
    for (uint32_t i = 0; i < n && e == cudaSuccess; i++) e = cudaEventElapsedTime(&ms[i], ev[i], ev[i + 1]);
    for (auto &x : ev) cudaEventDestroy(x);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(TLB_EXECUTION, (where.empty() ? std::string("profiling: ") : "launching `" + where + "`: ") + cuda_msg(e));
    }
    return TLB_OK;
}

tlb_status tlb_program_run(tlb_program *prog, tlb_buffer *const *weights, uint32_t n_weights, tlb_buffer *state) {
    tlb_status st = tlb_program_enqueue(prog, weights, n_weights, state);
    if (st != TLB_OK) return st;
    cudaError_t e = cudaStreamSynchronize(prog->dev->stream);
    if (e != cudaSuccess)
        return fail(TLB_EXECUTION, cuda_msg(e) + " (graph of " + std::to_string(prog->dispatches.size()) + " dispatches)");
    // bounded waits inside kernels report through the error word behind the arena
    int flag = 0;
    e = cudaMemcpy(&flag, (char *)prog->arena + std::max<uint64_t>(prog->layout.arena_size, 1), 4, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fail(TLB_EXECUTION, cuda_msg(e));
    if (flag != 0) {
        cudaMemset((char *)prog->arena + std::max<uint64_t>(prog->layout.arena_size, 1), 0, 4);
        if (flag == TLB_ERR_INDEX)
            return fail(TLB_EXECUTION, "a context length, block id or cache slot from the caller was out of range (skipped on the device; device error word 4)");
        return fail(TLB_EXECUTION, "a kernel gave up waiting for its own copies (device error word " + std::to_string(flag) + ")");
    }
    return TLB_OK;
}

tlb_status tlb_program_read(tlb_program *prog, uint32_t tensor_id, uint64_t bytes, void *out) {
    if (!prog || (!out && bytes)) return fail(TLB_INVALID, "tlb_program_read: bad arguments");
    if (tensor_id >= prog->n_user_tensors) return fail(TLB_INVALID, "no tensor " + std::to_string(tensor_id));
    const Place pl = prog->layout.place[tensor_id];
    char *base;
    uint64_t size;
    if (pl.buf == BUF_ARENA) {
        base = (char *)prog->arena;
        size = prog->layout.arena_size;
    } else if (pl.buf == BUF_IO) {
        base = (char *)prog->io;
        size = prog->layout.io_size;
    } else {
        return fail(TLB_INVALID, "tensor " + std::to_string(tensor_id) + " lives in " + (pl.buf == BUF_STATE ? "State" : "Weights") + ", which Program cannot read");
    }
    if (pl.off + bytes > size) return fail(TLB_INVALID, "tensor " + std::to_string(tensor_id) + " reads past its buffer");
    if (bytes == 0) return TLB_OK;
    cudaSetDevice(prog->dev->ordinal);
    TLB_TRY_CUDA(cudaMemcpyAsync(out, base + pl.off, bytes, cudaMemcpyDeviceToHost, prog->dev->stream), TLB_EXECUTION);
    TLB_TRY_CUDA(cudaStreamSynchronize(prog->dev->stream), TLB_EXECUTION);
    return TLB_OK;
}

uint32_t tlb_program_graph_count(tlb_program *prog) { return prog ? (uint32_t)prog->captured.size() : 0; }
uint32_t tlb_program_kernel_count(tlb_program *prog) { return prog ? prog->kernel_nodes : 0; }
uint64_t tlb_device_comm_generation(tlb_device *dev) { return dev ? dev->comm_generation : 0; }
uint32_t tlb_program_dispatch_count(tlb_program *prog) { return prog ? (uint32_t)prog->dispatches.size() : 0; }
const char *tlb_program_label(tlb_program *prog, uint32_t i) {
    return prog && i < prog->dispatches.size() ? prog->dispatches[i].label.c_str() : "";
}
uint64_t tlb_program_arena_bytes(tlb_program *prog) { return prog ? prog->layout.arena_size : 0; }

void *tlb_program_tensor_ptr(tlb_program *prog, uint32_t tensor_id, uint64_t *bytes) {
    if (!prog || tensor_id >= prog->n_user_tensors) return nullptr;
    const Place pl = prog->layout.place[tensor_id];
    if (bytes) *bytes = prog->graph.tensors[tensor_id].nbytes();
    if (pl.buf == BUF_ARENA) return (char *)prog->arena + pl.off;
    if (pl.buf == BUF_IO) return (char *)prog->io + pl.off;
    return nullptr;
}

// ------------------------------------------------------------------ test hook: a bounded wait that runs out
tlb_status tlb_selftest_wait_runs_out(tlb_device *dev, uint32_t limit, uint32_t nap_ns, double *waited_us) {
    if (!dev || limit == 0) return fail(TLB_INVALID, "tlb_selftest_wait_runs_out: bad arguments");
    cudaSetDevice(dev->ordinal);
    char *buf = nullptr;
    if (cudaMalloc(&buf, 512) != cudaSuccess) {
        cudaGetLastError();
        return fail(TLB_ALLOC, "buffer allocation of 512 bytes failed");
    }
    cudaError_t e = cudaMemsetAsync(buf, 0, 512, dev->stream);
    if (e == cudaSuccess) e = launch_wait_runs_out(limit, nap_ns, (int *)buf, (unsigned long long *)(buf + 256), dev->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(dev->stream);
    int flag = 0;
    unsigned long long ns = 0;
    if (e == cudaSuccess) e = cudaMemcpy(&flag, buf, 4, cudaMemcpyDeviceToHost);
    if (e == cudaSuccess) e = cudaMemcpy(&ns, buf + 256, 8, cudaMemcpyDeviceToHost);
    cudaFree(buf);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(TLB_EXECUTION, "wait self test: " + cuda_msg(e));
    }
    if (waited_us) *waited_us = (double)ns / 1e3;
    if (flag != 0) return fail(TLB_EXECUTION, "a kernel gave up waiting for its own copies (device error word " + std::to_string(flag) + ")");
    return TLB_OK;
}

// ------------------------------------------------------------------ quantizers
tlb_status tlb_quantize_rows_device(tlb_device *dev, uint32_t type, const void *src, int64_t rows, int64_t n_per_row, void *out) {
    if (!dev) return fail(TLB_INVALID, "null device");
    const TypeTraits *tr = type_traits(type);
    const bool have = type == TLB_TYPE_Q8_0 || type == TLB_TYPE_Q4_0 || type == TLB_TYPE_Q4_K || type == TLB_TYPE_F16 || type == TLB_TYPE_BF16 ||
                      type == TLB_TYPE_Q4_1 || type == TLB_TYPE_Q5_0 || type == TLB_TYPE_Q5_1 || type == TLB_TYPE_Q2_K || type == TLB_TYPE_Q3_K ||
                      type == TLB_TYPE_Q5_K || type == TLB_TYPE_Q6_K;
    if (!tr || !have)
        return fail(TLB_UNSUPPORTED, std::string("quantizing to ggml type ") + (tr ? tr->name : "?") + " is not implemented");
    if (rows < 0 || n_per_row < 0 || n_per_row % tr->blck != 0)
        return fail(TLB_INVALID, "row length " + std::to_string(n_per_row) + " is not a multiple of the block size " + std::to_string(tr->blck));
    cudaSetDevice(dev->ordinal);
    TLB_TRY_CUDA(launch_quantize_rows(type, (const float *)src, rows, n_per_row, out, dev->stream), TLB_EXECUTION);
    return TLB_OK;
}

tlb_status tlb_quantize_rows(tlb_device *dev, uint32_t type, const float *src, int64_t rows, int64_t n_per_row, void *out) {
    if (!dev || (!src && rows * n_per_row) || (!out && rows * n_per_row)) return fail(TLB_INVALID, "tlb_quantize_rows: bad arguments");
    const uint64_t rs = tlb_row_size(type, n_per_row);
    if (rows * n_per_row == 0) return tlb_quantize_rows_device(dev, type, nullptr, rows, n_per_row, nullptr);
    if (rs == 0) return tlb_quantize_rows_device(dev, type, nullptr, rows, n_per_row, nullptr);  // reports the reason
    cudaSetDevice(dev->ordinal);
    const uint64_t in_bytes = (uint64_t)rows * n_per_row * 4, out_bytes = (uint64_t)rows * rs;
    void *din = nullptr, *dout = nullptr;
    if (cudaMalloc(&din, in_bytes) != cudaSuccess || cudaMalloc(&dout, out_bytes) != cudaSuccess) {
        cudaGetLastError();
        if (din) cudaFree(din);
        return fail(TLB_ALLOC, "buffer allocation of " + std::to_string(in_bytes + out_bytes) + " bytes failed");
    }
    tlb_status st = TLB_OK;
    cudaError_t e = cudaMemcpyAsync(din, src, in_bytes, cudaMemcpyHostToDevice, dev->stream);
    if (e == cudaSuccess) {
        st = tlb_quantize_rows_device(dev, type, din, rows, n_per_row, dout);
        if (st == TLB_OK) e = cudaMemcpyAsync(out, dout, out_bytes, cudaMemcpyDeviceToHost, dev->stream);
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(dev->stream);
    cudaFree(din);
    cudaFree(dout);
    if (st != TLB_OK) return st;
    if (e != cudaSuccess) return fail(TLB_EXECUTION, "tlb_quantize_rows: " + cuda_msg(e));
    return TLB_OK;
}

}  // extern "C"
