// Layout of a rank's exchange buffer and the per-rank arguments of the peer-memory all-reduce kernels
// (comm.cu: plain all-reduce; k_fused.cu: all-reduce fused with residual add, RMS norm and quantization).
// The buffer holds two independent sets (flags, per-CTA sequence counters, data slots): kernels that cut the
// data into different chunks must not share a set, because the parity argument that protects a slot from
// being overwritten while a peer still reads it needs CTA c to own the same bytes in every call.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cstdlib>

namespace tlb {

constexpr int AR_MAX_RANKS = 8;
constexpr int AR_CTAS = 64;
constexpr int AR_THREADS = 256;
constexpr size_t AR_SLOT_BYTES = 1u << 20;                     // largest message
constexpr size_t AR_FLAG_OFF = 0;                              // u32 [2][AR_MAX_RANKS][AR_CTAS]
constexpr size_t AR_SEQ_OFF = 4096;                            // u32 [AR_CTAS], local only: calls seen by CTA c
constexpr size_t AR_DATA_OFF = 8192;                           // [2][AR_MAX_RANKS][AR_SLOT_BYTES]
constexpr size_t AR_SET_BYTES = AR_DATA_OFF + 2 * AR_MAX_RANKS * AR_SLOT_BYTES;
constexpr int AR_SETS = 2;                                    // 0: plain all-reduce, 1: the fused row kernel
constexpr size_t AR_BUF_BYTES = AR_SETS * AR_SET_BYTES;
constexpr uint32_t AR_SPIN_LIMIT = 1u << 22;   // default number of probes of a local flag, a few seconds (TLB_AR_SPIN_LIMIT overrides)

struct ArRank {
    float *data;                 // n floats, reduced in place
    const float *partial;        // n_split > 0: this rank's input is the sum of n_split partial results of n floats each
    int n_split;                 // (the K split of the row-parallel mul_mat in front of the exchange), `data` is only written
    char *peer[AR_MAX_RANKS];    // exchange buffers of all ranks as mapped into this rank (own one included)
    int rank;
    int *err;
    uint32_t spin_limit;         // probes of a peer's flag before the wait gives up and the error word is set
    int skip_push;               // self tests only: this rank neither pushes nor raises its flags, so its peers' waits run out
    int flagged_words;           // fused row exchange: 1 = every value carries the sequence number (lowest latency, twice the
                                 // bytes), 0 = plain values, a system fence and one flag per (rank, row)
};
// Which of the two the fused row exchange uses: flagged words at 2 ranks, fence and flag above. Measured on B200, batch-32
// decode step: 2 ranks 3.56 ms with flagged words against 3.95 with fence and flag; 4 ranks 3.96 against 3.59; 8 ranks 5.40
// against 3.76 (every rank pushes to every peer, so the doubled bytes (7.3 MB per exchange and GPU at 8 ranks) and sixteen
// thousand polling threads per GPU cost more than the round trip they save). TLB_XR_FLAGGED=0/1 overrides.
inline int xr_flagged_words(int n_ranks) {
    const char *v = getenv("TLB_XR_FLAGGED");
    if (v && (v[0] == '0' || v[0] == '1')) return v[0] == '1';
    return n_ranks <= 2;
}
// the limit the host passes to the kernels
inline uint32_t ar_spin_limit() {
    const char *v = getenv("TLB_AR_SPIN_LIMIT");
    const long n = v ? atol(v) : 0;
    return n > 0 ? (uint32_t)n : AR_SPIN_LIMIT;
}


}  // namespace tlb
