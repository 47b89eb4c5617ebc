// Attention over the paged cache for callers that must not allocate device memory.
//
// This entry point has no counterpart in mcelrath/braidinfer; it is this library's own.
//
// Who it is for.  Some programs cannot call cudaMalloc once they are running: a server
// that handed every byte of the device to an arena of its own at start-up, a plug-in
// living inside a host process whose memory policy it does not control, a control loop
// with a hard deadline where an allocation (which may synchronise the device) is not
// allowed after initialisation.  braid_attn_mma(), the ordinary entry point of this
// library, slices the context of a few-token step over many CTAs and needs a scratch
// buffer for the slices' partial results, which its caller allocates.  Here the scratch
// is a fixed array inside the library instead.
//
// What the caller gives up.
//   * Size.  The array holds BRAID_ATTN_NOALLOC_MAX_FLOATS floats (8 MiB), and every GPU
//     that loads this library holds that much until the process exits.  A call needs
//     rows * nqh * n_splits * (head_dim + 2) floats; more than the array holds is refused
//     with BRAID_REFUSED and a message in braid_last_error(), never truncated.
//   * Sharing.  All calls on a device use the same array.  It keeps the last call's
//     contents; nothing in it has to start at zero, because every slot that the merge
//     kernel reads is written by the attention kernel of the same call first.  Two calls
//     whose kernels overlap on the GPU (different streams, no ordering between them)
//     race on it: order them, or use braid_attn_mma() with buffers of your own.
//   * First call.  The first call on each device looks the array's device address up
//     (cudaGetSymbolAddress, with that device current).  That lookup is set-up work:
//     make the first call on a device before any stream capture begins.
//
//   * Consistent arguments.  "Every slot that is read was written first" holds only when the
//     host scalars describe the device tables: max_q_len must be at least the largest
//     q_len[s], rows the number of rows the tables speak of, n_seqs their sequences.  With a
//     max_q_len that is too small the attention grid leaves the slots of the rows beyond
//     it unwritten and the merge reads what an earlier call left there (with a buffer of
//     the caller's own the same mistake would read the caller's own stale data).  The
//     entry point cannot see the device tables, so it cannot check this.
//
// It calls no cudaMalloc, cudaFree or other allocating routine.  Arguments are those of
// braid_attn_mma() without `partial` (see attn_mma.cu for their meaning); `error_flag` is
// one int of device memory that the caller owns, set to 1 if a page-table entry of a
// visible key lies outside [0, num_pages).
#pragma once

#define BRAID_ATTN_NOALLOC_MAX_FLOATS (2 * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

int braid_attn_mma_noalloc(const void* q, void* out, const void* cache, const int* page_table,
                           const int* q_start, const int* q_len, const int* kv_before, const int* token_seq,
                           int q_row_stride, int out_row_stride, int rows, int n_seqs, int max_q_len,
                           int nqh, int nkh, int hd, int table_cols, int num_pages, int window, int n_splits,
                           int kind, float scale, int* error_flag, void* stream);

// The capacity of the built-in scratch, in floats (for callers that size their steps by it).
long long braid_attn_noalloc_capacity_floats(void);

#ifdef __cplusplus
}
#endif
