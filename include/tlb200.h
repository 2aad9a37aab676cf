/* tlb200 -- C ABI of the B200-native executor for tensorlisp's Device::Native path.
 *
 * The reference reaches its native CUDA executor through Rust types
 * (crates/tensorlisp/src/native_cuda.rs:28-168 over crates/kernels/src/cuda/exec.rs:20-240); there
 * is no C ABI at that seam. This header is the seam restated as plain C so a Rust shim with the
 * same eleven methods as native_cuda.rs can bind it through `extern "C"` declarations of the
 * functions below. Every entry point names the reference item it replaces.
 *
 * Conventions
 *  - every function returns a tlb_status; TLB_OK is 0. No entry point aborts, throws or exits.
 *  - tlb_last_error() returns the message of the last failing call on the calling thread.
 *  - handles may be used from any thread; callers run one program at a time per device, as the
 *    reference does under its per-model mutex (crates/tensorlisp/src/model.rs:96,802).
 *  - the library never computes on the CPU: without a usable GPU, tlb_device_open fails with
 *    TLB_NO_DEVICE and nothing else can be called.
 */
#ifndef TLB200_H
#define TLB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* crates/kernels/src/lib.rs:43-60 (enum Error) */
typedef enum tlb_status {
    TLB_OK = 0,
    TLB_NO_DEVICE = 1,   /* Error::NoDevice     */
    TLB_COMPILE = 2,     /* Error::Compile      */
    TLB_PIPELINE = 3,    /* Error::Pipeline     */
    TLB_ALLOC = 4,       /* Error::Alloc        */
    TLB_EXECUTION = 5,   /* Error::Execution    */
    TLB_INVALID = 6,     /* Error::Invalid      */
    TLB_UNSUPPORTED = 7  /* Error::Unsupported  */
} tlb_status;

typedef struct tlb_device tlb_device;
typedef struct tlb_buffer tlb_buffer;
typedef struct tlb_program tlb_program;

/* ggml's enum ggml_type numbering (crates/kernels/src/graph.rs:12-27) */
enum {
    TLB_TYPE_F32 = 0, TLB_TYPE_F16 = 1, TLB_TYPE_Q4_0 = 2, TLB_TYPE_Q4_1 = 3, TLB_TYPE_Q5_0 = 6,
    TLB_TYPE_Q5_1 = 7, TLB_TYPE_Q8_0 = 8, TLB_TYPE_Q2_K = 10, TLB_TYPE_Q3_K = 11, TLB_TYPE_Q4_K = 12,
    TLB_TYPE_Q5_K = 13, TLB_TYPE_Q6_K = 14, TLB_TYPE_I8 = 24, TLB_TYPE_I16 = 25, TLB_TYPE_I32 = 26,
    TLB_TYPE_I64 = 27, TLB_TYPE_BF16 = 30
};

/* crates/kernels/src/graph.rs:70-81 (enum Storage) */
enum { TLB_STORAGE_WEIGHT = 0, TLB_STORAGE_STATE = 1, TLB_STORAGE_INPUT = 2, TLB_STORAGE_TEMP = 3 };

/* crates/kernels/src/graph.rs:83-101 (struct Tensor); filled the way
 * crates/tensorlisp/src/native_ir.rs:66-95 fills it from a ggml_tensor. */
typedef struct tlb_tensor {
    uint32_t ty;            /* ggml type id                                              */
    int64_t  ne[4];         /* elements per dimension, innermost first                   */
    uint64_t nb[4];         /* byte strides                                              */
    char     op[32];        /* ggml op name ("MUL_MAT", "NONE" for leaves, ...)          */
    int32_t  op_params[16]; /* copied verbatim from ggml                                 */
    int32_t  src[10];       /* tensor ids, -1 = absent                                   */
    int32_t  view_src;      /* root tensor this one aliases, -1 = none                   */
    uint64_t view_offs;     /* byte offset into view_src                                 */
    uint32_t storage_kind;  /* TLB_STORAGE_*; meaningful for roots                       */
    uint32_t storage_index; /* weight / state / input index                              */
    char     name[64];
} tlb_tensor;

/* crates/kernels/src/graph.rs:204-209 (struct Graph: tensors, nodes, keep) */
typedef struct tlb_graph {
    const tlb_tensor *tensors;
    uint32_t          n_tensors;
    const int32_t    *nodes;    /* execution order; view ops included (they launch nothing) */
    uint32_t          n_nodes;
    const int32_t    *keep;     /* outputs and taps: valid after the last node              */
    uint32_t          n_keep;
} tlb_graph;

/* crates/kernels/src/plan.rs:42-47 (struct Leaves) */
typedef struct tlb_leaves {
    const uint32_t *weight_buffer; /* per weight: index into the buffers given to tlb_program_run */
    const uint64_t *weight_offset; /* per weight: byte offset in that buffer (256-byte aligned)    */
    uint32_t        n_weights;
    const uint64_t *state_offset;  /* per state tensor: byte offset in the state block             */
    uint32_t        n_states;
} tlb_leaves;

/* ------------------------------------------------------------------ device
 * Device::system_default (crates/kernels/src/cuda/mod.rs:244-277): primary context of one GPU and
 * one non-blocking stream. Fails with TLB_NO_DEVICE instead of aborting when there is no GPU. */
tlb_status tlb_device_open(int ordinal, tlb_device **dev);
void       tlb_device_close(tlb_device *dev);
/* "native <gpu name>" -- Native::device_name (crates/tensorlisp/src/native_cuda.rs:124-126) */
tlb_status tlb_device_name(tlb_device *dev, char *out, size_t n);
/* Device::sync (cuda/mod.rs): waits for everything enqueued on the device's stream. */
tlb_status tlb_device_sync(tlb_device *dev);
/* The cudaStream_t every launch of this device goes to, so callers can record events on it
 * (the reference keeps its stream private; cuda/mod.rs:258). */
void      *tlb_device_stream(tlb_device *dev);
int        tlb_device_sm_count(tlb_device *dev);
const char *tlb_last_error(void);

/* ------------------------------------------------------------------ buffers
 * Weights: Native::load puts every tensor of the file into one allocation at 256-byte aligned
 * offsets and copies each from host memory (native_cuda.rs:48-70). */
tlb_status tlb_weights_create(tlb_device *dev, uint64_t total_bytes, tlb_buffer **w);
/* State blocks: alloc_states / new_state_block (zeroed), fork_block, reset_block
 * (native_cuda.rs:85-122). One block per session. */
tlb_status tlb_state_create(tlb_device *dev, uint64_t bytes, tlb_buffer **s);
tlb_status tlb_state_zero(tlb_buffer *s);
tlb_status tlb_state_fork(tlb_buffer *src, tlb_buffer **copy);
/* copy_blocks (crates/kernels/src/cuda/paged_attn.rs:423-448, shaders/copy_blocks.cu:9-27): for every pair (src, dst)
 * of `pairs` (n_pairs x 2 block numbers, host memory) page src is copied to page dst in the K pool and in the V pool
 * of a state block -- the copy a forked sequence needs for the partly filled page it cannot share. The pools start at
 * the given byte offsets of the block and hold `pool_blocks` pages of `bytes_per_block` bytes (all of one block's
 * KV heads). Bounds-checked; a page that is written may not be read or written by another pair. Waits. */
tlb_status tlb_state_copy_blocks(tlb_buffer *state, uint64_t k_pool_offset, uint64_t v_pool_offset, uint64_t pool_blocks,
                                 uint64_t bytes_per_block, const int64_t *pairs, uint32_t n_pairs);
/* gather_kv_cache (crates/kernels/src/cuda/paged_attn.rs:450-509, shaders/gather_kv_cache_kernel.cu): the cached keys and
 * values of `seqs` sequences, read page by page through their block tables (`tables`: seqs x max_blocks block numbers,
 * `lens`: tokens per sequence; host memory), as dense f16 rows [token][kv_head][head_size] in host memory, one sequence
 * after another -- what exporting or inspecting a session's cache needs. The pools start at the given byte offsets of the
 * state block and hold `pool_blocks` pages of `block_size` tokens. Lengths and block numbers are checked on the host
 * before anything is launched. Waits. */
tlb_status tlb_state_gather_kv(tlb_buffer *state, uint64_t k_pool_offset, uint64_t v_pool_offset, uint64_t pool_blocks,
                               uint32_t kv_heads, uint32_t head_size, uint32_t block_size, const int32_t *tables,
                               uint32_t max_blocks, const int32_t *lens, uint32_t seqs, void *k_out, void *v_out);
/* Buffer::write_at / read_range (cuda/mod.rs:79-120): bounds-checked blocking copies. */
tlb_status tlb_buffer_write(tlb_buffer *b, uint64_t offset, const void *host, uint64_t n);
tlb_status tlb_buffer_read(tlb_buffer *b, uint64_t offset, void *host, uint64_t n);
uint64_t   tlb_buffer_size(tlb_buffer *b);
void      *tlb_buffer_device_ptr(tlb_buffer *b);
/* Device-to-device copy into a buffer, enqueued on the device stream and waited for (no counterpart:
 * the reference only writes buffers from host memory). For callers whose data is already in HBM. */
tlb_status tlb_buffer_copy_device(tlb_buffer *b, uint64_t offset, const void *device_src, uint64_t n);
void       tlb_buffer_free(tlb_buffer *b);

/* ------------------------------------------------------------------ programs
 * Executor::compile (crates/kernels/src/cuda/exec.rs:27-62): plans every tensor into one arena
 * (crates/kernels/src/plan.rs:56-189), lowers every node by ggml op name
 * (crates/kernels/src/cuda/lower.rs:177-213) and records the launches. Every node is lowered before
 * failing; the error then reads
 *   "native CUDA: not implemented: OP xN (e.g. node: why); ..."        (exec.rs:48-58)
 * View ops and tensors without elements launch nothing (lower.rs:179-181).
 * `err` (may be NULL) receives the message as well. */
tlb_status tlb_program_compile(tlb_device *dev, const tlb_graph *graph, const tlb_leaves *leaves,
                               tlb_program **prog, char *err, size_t errlen);
void       tlb_program_free(tlb_program *prog);
/* plan::plan alone (crates/kernels/src/plan.rs:56-189), without a device and without lowering, for tests of its
 * invariants (live tensors never share bytes, a node never writes over a source it still reads, views keep their
 * root alive; the reference's own checks are plan.rs:191-315). node_scratch (n_nodes entries, may be NULL) is the
 * scratch each node asks for. Outputs: arena and io sizes; per tensor the buffer it resolves to (0 weights, 1 state,
 * 2 io, 3 arena) and its byte offset there; per node the arena offset of its scratch block, -1 for none. */
tlb_status tlb_plan_only(const tlb_graph *graph, const tlb_leaves *leaves, const uint64_t *node_scratch, uint64_t *arena_size,
                         uint64_t *io_size, uint8_t *tensor_buffer, uint64_t *tensor_offset, int64_t *scratch_offset);
/* Program::set_input (exec.rs:91-98): n must equal the input tensor's byte size, else
 * "input i takes N bytes, got M". Blocking host-to-device copy into the program's io buffer. */
tlb_status tlb_program_set_input(tlb_program *prog, uint32_t i, const void *bytes, uint64_t n);
/* Device-side feedback for loops: copies the bytes of a KEPT tensor of the arena into graph input `input` (same byte
 * size), on the device stream, without waiting -- the next run sees them. A decode loop feeds the ARGMAX of a step
 * to the token-id input of the next one this way, so the ids never visit the host (the reference's graph-updatable
 * inputs, crates/kernels/src/cuda/backend.rs:57-260, serve the same loop). */
tlb_status tlb_program_feed_input(tlb_program *prog, uint32_t input, uint32_t tensor_id);
/* Program::run (exec.rs:186-225): enqueues every launch and waits. `weights` are the buffers the
 * leaves' weight_buffer indices refer to; `state` may be NULL when the graph has no state. */
tlb_status tlb_program_run(tlb_program *prog, tlb_buffer *const *weights, uint32_t n_weights, tlb_buffer *state);
/* Program::run_n (exec.rs:176-183) without the final wait: enqueue only, for timing with events on
 * tlb_device_stream. */
tlb_status tlb_program_enqueue(tlb_program *prog, tlb_buffer *const *weights, uint32_t n_weights, tlb_buffer *state);
/* Program::read (exec.rs:228-239): bytes of a tensor that lives in the arena or the io buffer. */
tlb_status tlb_program_read(tlb_program *prog, uint32_t tensor_id, uint64_t bytes, void *out);
/* Program::dispatch_count / labels (exec.rs:81-88) */
uint32_t   tlb_program_dispatch_count(tlb_program *prog);
const char *tlb_program_label(tlb_program *prog, uint32_t i);
/* How many CUDA graphs the program holds: one is captured per set of (weight buffers, state block, communicator
 * generation) it has been run with, and replayed on later runs with the same set (no counterpart: the reference
 * relaunches every kernel, exec.rs:186-225). */
uint32_t   tlb_program_graph_count(tlb_program *prog);
/* Kernel launches in the CUDA graph captured last, i.e. per run of the program (0 before the first run or when
 * runs are not captured). A dispatch may launch more than one kernel (a K-split mul_mat and the launch that adds its
 * partial sums) or none (a view), so this is the count to quote next to a timing (no counterpart in the reference). */
uint32_t   tlb_program_kernel_count(tlb_program *prog);
/* Device address and size of an input / kept tensor, so a caller that already has data in HBM can
 * write inputs and read results without the host (no counterpart: the reference only has the
 * blocking host copies). Returns NULL for tensors outside the io buffer and the arena. */
void      *tlb_program_tensor_ptr(tlb_program *prog, uint32_t tensor_id, uint64_t *bytes);
/* Layout figures of the plan (plan.rs Layout: arena_size, io_size). */
uint64_t   tlb_program_arena_bytes(tlb_program *prog);
/* TL_NATIVE_PROFILE of the reference (exec.rs:187-223) as a call: runs the program once, launch by
 * launch (no CUDA graph), with a CUDA event between launches on the device stream, and writes the
 * device time of each launch in milliseconds to ms[0..n) (n = tlb_program_dispatch_count). */
tlb_status tlb_program_profile(tlb_program *prog, tlb_buffer *const *weights, uint32_t n_weights, tlb_buffer *state,
                               float *ms, uint32_t n);

/* ------------------------------------------------------------------ quantizers
 * DType::from_f32 (crates/tensorlisp/src/dtype.rs:98-124) -> ggml_quantize_chunk: f32 rows to
 * Q4_0 / Q4_1 / Q5_0 / Q5_1 / Q8_0 / Q2_K / Q3_K / Q4_K / Q5_K / Q6_K blocks (also F16 and BF16),
 * bit-exact with the reference's build (the quantize targets of dtype.rs:28-33 that need no
 * importance matrix, except IQ4_NL, IQ4_XS, TQ1_0, TQ2_0 and MXFP4: TLB_UNSUPPORTED by name).
 * Host pointers; the rows are quantized on the GPU. n_per_row must be a multiple of the block
 * size (32 / 256). */
tlb_status tlb_quantize_rows(tlb_device *dev, uint32_t type, const float *src, int64_t rows, int64_t n_per_row, void *out);
/* Same on device-resident data (src and out are device pointers), enqueued on the device stream. */
tlb_status tlb_quantize_rows_device(tlb_device *dev, uint32_t type, const void *src, int64_t rows, int64_t n_per_row, void *out);
/* Type table of crates/kernels/src/graph.rs:30-50: bytes of a row of ne0 elements, 0 if unknown. */
uint64_t   tlb_row_size(uint32_t type, int64_t ne0);

/* ------------------------------------------------------------------ paged attention with no allocation
 * No counterpart in the reference (its paged attention allocates its scratch when the node is lowered,
 * crates/kernels/src/cuda/paged_attn.rs). For callers that may not allocate device memory -- a decode
 * loop that keeps the allocator off its latency path, a host confined to a fixed reservation, code
 * that runs while another component owns the allocator -- this is paged-attention decode (the CUSTOM
 * kind-1 node, same kernels and same results as through a program) whose only scratch, the
 * split-context partial sums, lives in an 8 MiB array inside the library image. Every GPU that
 * loads the library holds those 8 MiB until the process exits.
 *   q, out          f16 [seqs][heads][head_size]          (device pointers, caller-owned)
 *   k_pool, v_pool  f16 [block][kv_heads][block_size][head_size], as the cache-write node fills them
 *   block_tables    i32 [seqs][max_blocks], context_lens i32 [seqs]
 * Calls no cudaMalloc/cudaFree and no allocating library routine; enqueues on the device's stream and
 * waits. Shapes whose partial sums exceed 8 MiB are refused with TLB_INVALID (the message gives both
 * sizes); run those through a compiled program instead. The first call on a device looks up the
 * array's device address (cudaGetSymbolAddress): make that first call before any stream capture.
 * All calls share the one array and leave their partial sums in it; nothing in it needs clearing
 * between calls, but two calls that overlap on the same GPU race on it (each GPU has its own copy of
 * the array): issue them one after another. */
tlb_status tlb_paged_attention_static(tlb_device *dev, const void *q, const void *k_pool, const void *v_pool,
                                      const int32_t *block_tables, const int32_t *context_lens, void *out, int seqs,
                                      int heads, int kv_heads, int head_size, int block_size, int max_blocks,
                                      int max_context, float scale);

/* ------------------------------------------------------------------ tensor parallelism
 * No counterpart in the reference (single device: model.rs:415-422). A communicator joins the
 * ranks of one box; programs compiled on a device with a communicator may contain the pseudo-op
 * "ALLREDUCE" (sum over ranks of an f32 tensor, in place of its source), which the sharding pass
 * inserts after each row-parallel MUL_MAT. */
tlb_status tlb_comm_unique_id(void *out128);
tlb_status tlb_comm_init(tlb_device *dev, int n_ranks, int rank, const void *id128);
tlb_status tlb_comm_destroy(tlb_device *dev);
/* One-shot all-reduce over NVLink peer memory for messages up to 1 MiB (the activations of a decode
 * step), used by "ALLREDUCE" in place of NCCL once set up: every rank calls export (allocates its
 * exchange buffer, returns a 64-byte CUDA IPC handle), the host gathers the handles of all ranks in
 * rank order (n_ranks x 64 bytes) and every rank calls import. Up to 8 ranks of one box. The kernel's
 * waits are bounded; a rank that never arrives makes tlb_program_run fail instead of hanging.
 * Used by default with more than 2 ranks (measured faster there); TLB_P2P_ALLREDUCE=1 turns it on for 2
 * ranks, TLB_NO_P2P_ALLREDUCE=1 keeps NCCL everywhere. */
/* A counter that grows with every change of the device's communicator (init, import, destroy). A captured CUDA graph
 * has the communicator's state baked into its launches (the all-reduce path, the peers' mapped addresses), so a
 * program run after such a change captures a new graph instead of replaying an old one. */
uint64_t   tlb_device_comm_generation(tlb_device *dev);
tlb_status tlb_comm_p2p_export(tlb_device *dev, void *handle64);
tlb_status tlb_comm_p2p_import(tlb_device *dev, const void *handles);
/* The same protocol with n_ranks emulated ranks on ONE device in one cooperative launch (test hook):
 * out is n_ranks x n floats on the host; `calls` all-reduces in a row, call k on inputs x (k+1). With
 * n_split > 0 every rank's input is the sum of n_split partial results (in: n_ranks x n_split x n floats),
 * the form the exchange takes behind a K-split mul_mat; otherwise in is n_ranks x n floats. */
tlb_status tlb_comm_p2p_selftest(tlb_device *dev, int n_ranks, int n, int calls, int n_split, const float *in, float *out);
/* The exchange fused with what follows it in a decoder layer (residual add + RMS norm * w + Q8_K quantization of
 * the next mul_mat's input), checked the same way with up to 4 emulated ranks: in is n_ranks x n_split x rows x K
 * partial results, resid rows x K, w K floats; out_sum gets n_ranks x rows x K (the new residual stream as every
 * rank sees it), out_q n_ranks x act_bytes (the Q8_K activation block: int8 codes, f32 d per 256, int16 sums
 * per 16, each section 256-byte aligned; act_bytes must be the size the library computes for (K, rows)). */
tlb_status tlb_comm_p2p_selftest_rows(tlb_device *dev, int n_ranks, int rows, int K, int n_split, int calls, const float *in,
                                      const float *resid, const float *w, float eps, float *out_sum, void *out_q,
                                      uint64_t act_bytes);

/* The two self tests with one emulated rank (`absent_rank`) that never pushes: the other ranks' waits run out after
 * `spin_limit` probes of its flag, the launch ends, and the call returns TLB_EXECUTION ("gave up waiting") -- what
 * tlb_program_run reports when a real rank never arrives. TLB_AR_SPIN_LIMIT sets the limit of the real kernels
 * (default 2^22 probes). */
tlb_status tlb_comm_p2p_selftest_absent(tlb_device *dev, int n_ranks, int n, int absent_rank, uint32_t spin_limit, const float *in,
                                        float *out);
tlb_status tlb_comm_p2p_selftest_rows_absent(tlb_device *dev, int n_ranks, int rows, int K, int absent_rank, uint32_t spin_limit,
                                             const float *in, const float *resid, const float *w, float eps, float *out_sum,
                                             void *out_q, uint64_t act_bytes);
/* Test hook for the bounded mbarrier waits of the TMA / tcgen05 kernels: one CTA waits on a barrier nothing arrives
 * on, gives up after `limit` probes (`nap_ns` nanoseconds apart, 0 = back to back) and sets the device error word
 * the way the mul_mat kernels do; the call then fails with TLB_EXECUTION like tlb_program_run would, and
 * *waited_us says how long the wait lasted. No counterpart in the reference (its kernels have no waits). */
tlb_status tlb_selftest_wait_runs_out(tlb_device *dev, uint32_t limit, uint32_t nap_ns, double *waited_us);

#ifdef __cplusplus
}
#endif
#endif /* TLB200_H */
