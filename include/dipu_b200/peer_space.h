/*
 * Peer space: the memory a tensor-parallel group shares for collectives that are fused into compute kernels.
 *
 * No counterpart in the reference, whose row-parallel linear is a matrix product followed by ProcessGroupDICL::allreduce
 * (dipu/torch_dipu/csrc_dipu/runtime/distributed/ProcessGroupDICL.cpp:539-567 -> devapis::diclAllReduce ->
 * ncclAllReduce, vendor/cuda/communiatorimpl.cpp:84-92). Here the product's epilogue pushes every output tile to the rank
 * that owns its rows while the remaining tiles are still being computed, and one kernel per rank then sums the arrived
 * partial tiles, adds the residual and pushes the finished rows to everybody (b200_dicl_peer_reduce_gather).
 *
 * Every rank allocates the same three blocks and maps the peers' blocks (CUDA IPC over NVLink):
 *
 *   stage  [slots][slot_bytes]   partial sums on their way to this rank. In a slot, source rank s writes the rows this
 *                                rank owns at element offset s * (rows / nranks) * cols, dense, row pitch = cols.
 *   gout   [slots][slot_bytes]   results: the full [rows, cols] tensor, written by the owners of its row ranges.
 *   flags  uint32, all zero at creation, only ever growing (a call's number, "epoch", is written):
 *            ready [slots][nranks][max_units]  piece `unit` of source rank s has arrived in stage
 *            gdone [slots][nranks][ctas]       CTA c of rank s has pushed all its result rows into gout
 *            sfree [slots][nranks]             rank s has finished reading its own stage slot (it may be overwritten)
 *
 * A piece is what one epilogue warp of the product owns: 32 rows x 256 columns. Its unit number inside the owner's rows is
 * (local_row / 32) * (cols / 256) + column_block.
 *
 * The struct is plain C and is passed by value to kernels; pointers are this process's mappings of every rank's blocks.
 */
#ifndef DIPU_B200_PEER_SPACE_H_
#define DIPU_B200_PEER_SPACE_H_

#include <stddef.h>
#include <stdint.h>

#define B200_PEER_MAX_RANKS 8
#define B200_PEER_PIECE_ROWS 32
#define B200_PEER_PIECE_COLS 256

#ifdef __cplusplus
extern "C" {
#endif

typedef struct b200PeerSpace {
    int32_t rank, nranks;
    int32_t slots;
    uint32_t max_units;  /* pieces per source rank a slot can announce */
    uint32_t ctas;       /* grid of the reduce kernel: the same on every rank, in every call */
    uint32_t pad_;
    uint64_t slot_bytes;
    void* stage[B200_PEER_MAX_RANKS];
    void* gout[B200_PEER_MAX_RANKS];
    uint32_t* flags[B200_PEER_MAX_RANKS];
} b200PeerSpace;

#ifdef __cplusplus
}
#endif

#if defined(__CUDACC__)
#define B200_PEER_HD __host__ __device__ static inline
#else
#define B200_PEER_HD static inline
#endif

/* Offsets (in uint32 words) into a rank's flag block. */
B200_PEER_HD size_t b200_peer_ready_off(const b200PeerSpace* s, int slot, int src, uint32_t unit) {
    return ((size_t)slot * (size_t)s->nranks + (size_t)src) * s->max_units + unit;
}
B200_PEER_HD size_t b200_peer_gdone_off(const b200PeerSpace* s, int slot, int src, uint32_t cta) {
    const size_t ready_words = (size_t)s->slots * (size_t)s->nranks * s->max_units;
    return ready_words + ((size_t)slot * (size_t)s->nranks + (size_t)src) * s->ctas + cta;
}
B200_PEER_HD size_t b200_peer_sfree_off(const b200PeerSpace* s, int slot, int src) {
    const size_t ready_words = (size_t)s->slots * (size_t)s->nranks * s->max_units;
    const size_t gdone_words = (size_t)s->slots * (size_t)s->nranks * s->ctas;
    return ready_words + gdone_words + (size_t)slot * (size_t)s->nranks + (size_t)src;
}
B200_PEER_HD size_t b200_peer_flag_words(const b200PeerSpace* s) {
    return b200_peer_sfree_off(s, s->slots, 0);
}

#endif /* DIPU_B200_PEER_SPACE_H_ */
