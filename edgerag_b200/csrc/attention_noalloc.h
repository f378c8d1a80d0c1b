// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference project: it exists for hosts that embed
// this library somewhere cudaMalloc is off limits.  Examples: a serving loop that has already
// handed every free byte of the GPU to its own pool and would fail (or stall the whole device)
// on one more allocation; a plug-in that runs inside another program's CUDA context and is only
// allowed to launch work on a stream it was given.  Such a caller still owns its inputs and
// outputs, but has nowhere to put the partial results that split-KV attention needs between its
// two kernels.
//
// `erb_attention_decode_static` is `erb_attention_decode` with that scratch taken from a
// fixed array inside the library instead of from the caller:
//
//   * The array is `ERB_STATIC_SCRATCH_FLOATS` floats (4 MiB).  Every GPU on which the library's
//     device code is loaded holds that much until the process exits.  The CUDA runtime may load
//     that code lazily, at the first call into the library on a device, and this load is the one
//     moment at which the array's 4 MiB are taken: on a GPU that is already full it fails with an
//     out-of-memory error.  So make one call on each device at start-up, before the memory is
//     given away.
//   * A call needs n_seqs * nq * max_splits * (head_dim + 2) floats.  A call that needs more is
//     refused with ERB_ERR_UNSUPPORTED and a message; nothing is launched.  `max_splits` must be
//     at least the number of splits of the longest sequence; with a smaller value only the first
//     `max_splits` splits of a sequence are computed and merged (the result is then wrong, but no
//     kernel reads or writes outside the part of the array that the call was sized for).
//   * The first call on each device looks up the array's device address (cudaGetSymbolAddress,
//     with that device current) and remembers it.  Make that first call outside of any stream
//     capture.  Later calls only launch kernels.
//   * The function never calls cudaMalloc, cudaFree or any routine that allocates.
//   * All calls on a device share the one array, and it keeps whatever the previous call left in
//     it.  That is harmless here: every scratch entry that the combine step reads was written by
//     the split step of the same call, so nothing has to start at zero.  But two calls whose
//     kernels can overlap on the GPU (different streams, no ordering between them) race on the
//     array and corrupt each other's results; order them on one stream or with events.
//
// Arguments are those of `erb_attention_decode` without `part_acc` and `part_ml`; results are
// identical to it bit for bit, since the same kernels run on the same split boundaries.
#pragma once

#define ERB_STATIC_SCRATCH_FLOATS (1 << 20)

#ifdef __cplusplus
extern "C" {
#endif

int erb_attention_decode_static(const void* q, int q_row_stride, const void* k_pages, const void* v_pages,
                                const int* block_tables, int max_pages, const int* token_of_seq,
                                const int* positions, void* out, int out_row_stride, int max_splits,
                                int n_seqs, int nq, int nkv, int head_dim, int page_size, int window,
                                int split_keys, float scale, void* stream);

// Floats of the static array a call with these sizes would use (for callers that want to check first).
long long erb_attention_decode_static_floats(int n_seqs, int nq, int head_dim, int max_splits);

#ifdef __cplusplus
}
#endif
