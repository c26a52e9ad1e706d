/*
 * thrust_b200 -- C ABI of the B200 (sm_100a) backend for Thrust's core parallel algorithms.
 *
 * This is the boundary a binding generator (cgo, JNI, ctypes, a C++ header overlay) links
 * against.  Conventions, the same for every entry point:
 *
 *   - All data pointers are DEVICE pointers on the current device unless a parameter name starts
 *     with h_.  The caller owns every buffer; nothing here allocates or frees device memory.
 *   - Scratch memory is passed in as (d_ws, ws_bytes).  Calling with d_ws == NULL performs no
 *     work and stores the required size in *ws_bytes -- the two-phase convention of the
 *     reference's doit_step (thrust/system/cuda/detail/copy_if.h:602-691).  With d_ws != NULL,
 *     *ws_bytes must be at least that size, else cudaErrorInvalidValue (1) is returned.
 *   - Work is enqueued on `stream` and the call returns without synchronising.  Counts (number
 *     of selected items, number of runs) are written to device words the caller names and, as a
 *     copy, into the workspace header; read them after synchronising the stream.
 *   - The return value is a cudaError_t (0 = success).  Unsupported type combinations return
 *     cudaErrorNotSupported (801).  Kernels bound every inter-CTA wait; a wait that ran out is
 *     reported by tb200_workspace_status(), never by a hang.
 *   - Element types are named by tb200_dtype codes, operators by tb200_op, predicates by
 *     tb200_pred with two integer operands.
 */
#ifndef THRUST_B200_H
#define THRUST_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* tb200_stream_t; /* == cudaStream_t */

enum tb200_dtype {
  TB200_I8 = 0, TB200_U8 = 1, TB200_I16 = 2, TB200_U16 = 3, TB200_I32 = 4,
  TB200_U32 = 5, TB200_I64 = 6, TB200_U64 = 7, TB200_F32 = 8, TB200_F64 = 9
};
enum tb200_op { TB200_PLUS = 0, TB200_MIN = 1, TB200_MAX = 2 };
/* MOD_EQ: x % a == b    LT: x < a    GE: x >= a    NE: x != a */
enum tb200_pred { TB200_PRED_MOD_EQ = 0, TB200_PRED_LT = 1, TB200_PRED_GE = 2, TB200_PRED_NE = 3 };

/* Library version (major * 10000 + minor * 100 + patch) and the SM architecture it was built for. */
int tb200_version(void);
int tb200_sm_arch(void);

/* Reads the status word of a workspace after the work that used it has completed: synchronises
 * `stream`, copies 4 bytes back.  *h_status: 0 = ok, 1 = a look-back wait ran out (results of
 * that call are invalid).  Stands in for the reference's post-launch error check,
 * cuda_cub::throw_on_error (thrust/system/cuda/detail/util.h:180-243). */
int tb200_workspace_status(const void* d_ws, tb200_stream_t stream, unsigned* h_status);

/* thrust::reduce(first, last, init, op) -- thrust/system/cuda/detail/reduce.h:1015-1067
 * (cuda_cub::reduce_n).  Accumulates in acc_t, the type of *h_init; each input element is
 * converted to acc_t first.  Result: one acc_t at d_out.  n == 0 stores init.
 * (in_t, acc_t): equal 4/8-byte types, or widening within a family: I8/I16/I32 -> I32/I64,
 * U8/U16/U32 -> U32/U64, F32 -> F64. */
int tb200_reduce(const void* d_in, size_t n, int in_t, int acc_t, int op, const void* h_init,
                 void* d_out, void* d_ws, size_t* ws_bytes, tb200_stream_t stream);

/* thrust::inclusive_scan / thrust::exclusive_scan -- thrust/system/cuda/detail/scan.h:215-361
 * (cuda_cub::inclusive_scan_n, exclusive_scan_n).  Element type t (I32 U32 I64 U64 F32 F64) for
 * input, output and accumulator.  d_in == d_out is allowed.  h_init of the inclusive scan may be
 * NULL (the classic form); when given, it is combined in front of the first element, which is how
 * a shard of a multi-GPU scan receives the carry of the shards before it. */
int tb200_inclusive_scan(const void* d_in, void* d_out, size_t n, int t, int op, const void* h_init,
                         void* d_ws, size_t* ws_bytes, tb200_stream_t stream);
int tb200_exclusive_scan(const void* d_in, void* d_out, size_t n, int t, int op,
                         const void* h_init, void* d_ws, size_t* ws_bytes, tb200_stream_t stream);

/* The same two scans with the initial value in DEVICE memory (d_init: one element of type t, read
 * when the kernels run, not when the call is made), so that a value produced by earlier work on the
 * stream -- the carry of a multi-GPU scan -- never visits the host.  No counterpart in the
 * reference.  tb200_inclusive_scan_dinit with d_init == NULL is tb200_inclusive_scan without init. */
int tb200_inclusive_scan_dinit(const void* d_in, void* d_out, size_t n, int t, int op,
                               const void* d_init, void* d_ws, size_t* ws_bytes, tb200_stream_t stream);
int tb200_exclusive_scan_dinit(const void* d_in, void* d_out, size_t n, int t, int op,
                               const void* d_init, void* d_ws, size_t* ws_bytes, tb200_stream_t stream);


/* thrust::sort / stable_sort / sort_by_key / stable_sort_by_key with thrust::less (descending=0)
 * or thrust::greater (descending=1) on arithmetic keys -- thrust/system/cuda/detail/sort.h:
 * 1621-1754, radix path :1438-1508.  Stable.  Sorts d_keys (and d_vals) in place; d_keys_alt /
 * d_vals_alt are caller-provided buffers of the same size that play the part of the reference's
 * double buffer (sort.h:1465-1484).  key_t: any of the ten dtypes.  val_bytes: 0 (keys only),
 * 4 or 8.  Only key bits [begin_bit, end_bit) are compared (multiples of 8; pass 0 and
 * 8*sizeof(key) for a full sort).  n < 2^31, as in the reference (sort.h:1346). */
int tb200_sort_by_key(void* d_keys, void* d_keys_alt, void* d_vals, void* d_vals_alt, size_t n,
                      int key_t, int val_bytes, int descending, int begin_bit, int end_bit,
                      void* d_ws, size_t* ws_bytes, tb200_stream_t stream);

/* thrust::copy_if(first, last, [stencil,] result, pred) -- thrust/system/cuda/detail/copy_if.h:
 * 780-853.  Stable.  Without a stencil (d_stencil == NULL) the predicate tests the element; with
 * one it tests stencil[i] (stencil_t: U8 or I32) and copies in[i].  The number of elements
 * written goes to *d_count (device, may be NULL) and to the workspace header.  d_out == d_in is
 * allowed (the remove_if use of thrust/system/cuda/detail/remove.h:38-65). */
int tb200_copy_if(const void* d_in, const void* d_stencil, void* d_out, size_t n, int t,
                  int stencil_t, int pred, long long a, long long b, unsigned long long* d_count,
                  void* d_ws, size_t* ws_bytes, tb200_stream_t stream);

/* thrust::stable_partition_copy / partition_copy(first, last, [stencil,] out_true, out_false,
 * pred) -- thrust/system/cuda/detail/partition.h:909-1075.  Both outputs keep input order.
 * *d_count = number of elements written to d_out_true. */
int tb200_partition_copy(const void* d_in, const void* d_stencil, void* d_out_true,
                         void* d_out_false, size_t n, int t, int stencil_t, int pred, long long a,
                         long long b, unsigned long long* d_count, void* d_ws, size_t* ws_bytes,
                         tb200_stream_t stream);

/* thrust::partition / thrust::stable_partition(first, last, pred), in place --
 * thrust/system/cuda/detail/partition.h:833-907 and :1077-1132.  Always stable (which satisfies
 * both).  The workspace includes room for a copy of the data, like the reference's temporary
 * (partition.h:808-810).  *d_count = number of elements satisfying pred (the split point). */
int tb200_partition(void* d_data, size_t n, int t, int pred, long long a, long long b,
                    unsigned long long* d_count, void* d_ws, size_t* ws_bytes,
                    tb200_stream_t stream);

/* thrust::unique_copy(first, last, result) with equal_to; d_out == d_in is thrust::unique --
 * thrust/system/cuda/detail/unique.h:710-795.  *d_count = number of elements kept. */
int tb200_unique_copy(const void* d_in, void* d_out, size_t n, int t, unsigned long long* d_count,
                      void* d_ws, size_t* ws_bytes, tb200_stream_t stream);

/* thrust::reduce_by_key(keys, keys + n, vals, keys_out, vals_out, equal_to, op) --
 * thrust/system/cuda/detail/reduce_by_key.h:1063-1161.  key_t: any dtype; val_t: I32 U32 I64 U64
 * F32 F64; values of a run are combined left to right.  *d_count = number of runs.  n < 2^31,
 * as in the reference (reduce_by_key.h:983). */
int tb200_reduce_by_key(const void* d_keys, const void* d_vals, void* d_keys_out, void* d_vals_out,
                        size_t n, int key_t, int val_t, int op, unsigned long long* d_count,
                        void* d_ws, size_t* ws_bytes, tb200_stream_t stream);

/* thrust::inclusive_scan_by_key / exclusive_scan_by_key(keys, keys + n, vals, out, [init,] equal_to,
 * op) -- thrust/system/cuda/detail/scan_by_key.h:172-588 (not one of the eight hot-path headers:
 * the first of the "next" components).  The scan restarts at every run of equal keys; the
 * exclusive form writes init at each run head.  key_t: any dtype; val_t: I32 U32 I64 U64 F32 F64.
 * d_out may be d_vals.  n < 2^31. */
int tb200_scan_by_key(const void* d_keys, const void* d_vals, void* d_out, size_t n, int key_t,
                      int val_t, int op, int exclusive, const void* h_init, void* d_ws,
                      size_t* ws_bytes, tb200_stream_t stream);

/* thrust::unique_by_key_copy(keys, keys + n, vals, keys_out, vals_out) with equal_to --
 * thrust/system/cuda/detail/unique_by_key.h:189-616: the first (key, value) of every run.
 * val_bytes: 4 or 8.  *d_count = number of runs.  Outputs may alias the inputs (unique_by_key). */
int tb200_unique_by_key_copy(const void* d_keys, const void* d_vals, void* d_keys_out,
                             void* d_vals_out, size_t n, int key_t, int val_bytes,
                             unsigned long long* d_count, void* d_ws, size_t* ws_bytes,
                             tb200_stream_t stream);

/* thrust::min_element / max_element / minmax_element(first, last) with thrust::less --
 * thrust/system/cuda/detail/extrema.h:376-569 (the second of the "next" components).  The POSITION
 * of the first smallest / first largest element is written to device memory: d_index[0] for
 * min_element and max_element; d_index[0] = minimum and d_index[1] = maximum for minmax_element.
 * n == 0 writes 0 (first == last).  t: any dtype.  NaNs compare false both ways, as with less. */
int tb200_min_element(const void* d_in, size_t n, int t, unsigned long long* d_index, void* d_ws,
                      size_t* ws_bytes, tb200_stream_t stream);
int tb200_max_element(const void* d_in, size_t n, int t, unsigned long long* d_index, void* d_ws,
                      size_t* ws_bytes, tb200_stream_t stream);
int tb200_minmax_element(const void* d_in, size_t n, int t, unsigned long long* d_index,
                         void* d_ws, size_t* ws_bytes, tb200_stream_t stream);

/* thrust::merge / thrust::merge_by_key(A, B, [payload A, payload B,] out, [payload out,] comp)
 * with thrust::less (descending=0) or thrust::greater (descending=1) --
 * thrust/system/cuda/detail/merge.h:862-1013.  Both inputs must already be sorted by comp.
 * Stable: on equal keys the element of A comes first (merge.h:70-84).  key_t: I32 U32 I64 U64 F32
 * F64; val_bytes: 0 (keys only), 4 or 8.  Outputs must not overlap the inputs. */
int tb200_merge_by_key(const void* d_keys_a, const void* d_vals_a, size_t na, const void* d_keys_b,
                       const void* d_vals_b, size_t nb, void* d_keys_out, void* d_vals_out,
                       int key_t, int val_bytes, int descending, void* d_ws, size_t* ws_bytes,
                       tb200_stream_t stream);

/* The comparison-sort route of thrust::stable_sort / stable_sort_by_key --
 * thrust/system/cuda/detail/sort.h:1278-1321 (__merge_sort::merge_sort), the path the reference
 * takes for user comparators and non-arithmetic keys.  Here the comparator is less / greater on
 * the key; payloads move with their keys, which is exactly
 * stable_sort(zip(keys, vals), [](a, b){ return get<0>(a) < get<0>(b); }).  In place; d_keys_alt /
 * d_vals_alt are same-sized scratch (sort.h:1200-1205).  Types as tb200_merge_by_key. */
int tb200_merge_sort_by_key(void* d_keys, void* d_keys_alt, void* d_vals, void* d_vals_alt, size_t n,
                            int key_t, int val_bytes, int descending, void* d_ws, size_t* ws_bytes,
                            tb200_stream_t stream);

/* Batched lower bound: d_out[j] = number of elements of the sorted range d_sorted[0, n) that
 * order strictly before d_needles[j] (thrust::lower_bound with less / greater).  Used by the
 * multi-GPU sort to cut each GPU's sorted shard at the splitters.  key_t: I32 U32 I64 U64 F32 F64.
 * Has no counterpart among the reference files on the hot path (the reference's vectorised
 * binary search is thrust/system/cuda/detail/binary_search.h). */
int tb200_lower_bound(const void* d_sorted, size_t n, const void* d_needles, size_t m,
                      unsigned long long* d_out, int key_t, int descending, tb200_stream_t stream);

/* Per-kernel device timing, off by default.  tb200_kernel_timing(1) makes every launcher bracket
 * its dominant kernel with CUDA events on the launching stream (and clears earlier records);
 * tb200_kernel_timing_read waits for the recorded launches and returns up to `capacity` pairs
 * (kernel id, milliseconds), then clears the records.  Kernel ids: 1 reduce, 2 scan, 3 onesweep
 * pass, 4 radix histogram, 5 compaction, 6 reduce_by_key, 7 merge, 8 block sort.  This is the
 * library's counterpart of the reference's THRUST_DEBUG_SYNC launch log
 * (thrust/system/cuda/detail/core/agent_launcher.h:518-590).  At most 256 launches are kept. */
int tb200_kernel_timing(int enable);
int tb200_kernel_timing_read(int capacity, int* h_kernel_ids, float* h_ms, int* h_count);

/* Inclusive scan for callers that cannot allocate device memory.  (No counterpart in the
 * reference, whose every algorithm obtains temporary storage through the policy's allocator.)
 *
 * Who needs it: a caller that may not call cudaMalloc at the point where it needs a scan -- inside
 * a stream-ordered pool's callback, in a latency-critical loop where cudaMalloc's device-wide
 * synchronisation is not acceptable, in a plug-in that receives buffers but no allocator, or when
 * its own data has already claimed all device memory.  The other entry points make such a caller
 * bring the scratch; this one brings its own: a 512 KiB array in the library's device data
 * segment, which every GPU that loads the library holds until the process exits.
 *
 * Same arguments and result as tb200_inclusive_scan minus the workspace pair.  Limit: the
 * descriptors must fit the array, i.e. n <= 536,600,576 elements (just under 2^29) for
 * I32/U32/F32 and n <= 134,148,096 (just under 2^27) for I64/U64/F64 with the present tile sizes;
 * tb200_inclusive_scan_static_limit(t, &max_n) reports the exact figure of the loaded library.
 * Beyond it the call does nothing and returns TB200_ERR_EXCEEDS_STATIC_SCRATCH.  It calls no
 * cudaMalloc, cudaFree or other allocating routine.
 *
 * A wait inside the kernels that runs out (see tb200_workspace_status) is recorded in the array's
 * first word, which the caller cannot address: tb200_inclusive_scan_static_status(stream,
 * &status) synchronises `stream` and reads it back (0 = ok, 1 = the last call's result is invalid).
 *
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 * that device current) and remembers it; make that first call before starting any stream capture.
 * All calls on a device share the one array.  Each call clears what it needs before use, so calls
 * issued one after another on a stream are independent, but two calls whose kernels can overlap on
 * the GPU (different streams, different host threads) race on it: serialise them. */
#define TB200_ERR_EXCEEDS_STATIC_SCRATCH 100001
int tb200_inclusive_scan_static(const void* d_in, void* d_out, size_t n, int t, int op,
                                const void* h_init, tb200_stream_t stream);
int tb200_inclusive_scan_static_limit(int t, size_t* h_max_n);
int tb200_inclusive_scan_static_status(tb200_stream_t stream, unsigned* h_status);

/* Stable merge of num_runs (<= 64) sorted runs, given as host arrays of device pointers and
 * lengths, into d_keys_out / d_vals_out (sum of the lengths); ties keep the earlier run first.  A
 * pairwise tree of merge-path merges ping-pongs between the output and the same-sized d_*_tmp
 * buffers; everything is enqueued by this one call.  Run pointers may lie in a peer GPU's memory
 * (tb200_ipc_open): this is the last stage of the multi-GPU sort, where the merges read the pieces
 * they need straight out of the other GPUs' sorted shards.  Generalises
 * thrust::merge_by_key (thrust/system/cuda/detail/merge.h:940-982) to many inputs; types as
 * tb200_merge_by_key. */
int tb200_merge_runs(const void* const* h_run_keys, const void* const* h_run_vals,
                     const size_t* h_counts, int num_runs, void* d_keys_out, void* d_vals_out,
                     void* d_keys_tmp, void* d_vals_tmp, int key_t, int val_bytes, int descending,
                     void* d_ws, size_t* ws_bytes, tb200_stream_t stream);

/* The exchange step of the multi-GPU sort_by_key, fused with the collective: one kernel that
 * splits a GPU's (key, value) pairs by key range and stores every pair straight into the receive
 * buffer of the GPU that owns its range (ordinary stores over NVLink into buffers opened with
 * tb200_ipc_open; a local pointer for the rank itself).  No counterpart in the reference.
 *   d_splitters   num_buckets - 1 keys in ascending (descending=1: descending) order, on the device;
 *                 bucket b holds the keys k with exactly b splitters <= k (in that order), so equal
 *                 keys always share a bucket;
 *   tb200_bucket_count   adds the bucket histogram of d_keys to d_counts[0, num_buckets) (zero it first);
 *   tb200_bucket_scatter writes bucket b's pairs, in input order (stable), to
 *                 h_dst_keys[b][h_dst_offsets[b] ...] and h_dst_vals[b][h_dst_offsets[b] ...].
 * num_buckets <= 16, n < 2^30, key_t / val_bytes as tb200_sort_by_key.  The receivers must not touch
 * their buffers until every sender's scatter has completed (order with a collective). */
int tb200_bucket_count(const void* d_keys, size_t n, int key_t, int descending,
                       const void* d_splitters, int num_buckets, unsigned long long* d_counts,
                       tb200_stream_t stream);
int tb200_bucket_scatter(const void* d_keys, const void* d_vals, size_t n, int key_t, int val_bytes,
                         int descending, const void* d_splitters, int num_buckets,
                         void* const* h_dst_keys, void* const* h_dst_vals,
                         const unsigned long long* h_dst_offsets, void* d_ws, size_t* ws_bytes,
                         tb200_stream_t stream);

/* thrust::set_union / set_intersection / set_difference / set_symmetric_difference and their
 * _by_key forms on sorted ranges -- thrust/system/cuda/detail/set_operations.h:1260-1760.
 * op: 0 union, 1 intersection, 2 difference, 3 symmetric difference; multiset semantics as in the
 * reference (an element occurring m times in A and n times in B: max(m, n), min(m, n), max(m - n, 0),
 * |m - n| copies; where both sides contribute, A's copies come first).  Keys of type key_t (I32 U32
 * I64 U64 F32 F64) sorted ascending (descending=1: descending); val_bytes 0, 4 or 8: values that
 * travel with the kept keys (d_vals_b may be NULL for the intersection and the difference, which
 * only keep A's).  The outputs must hold na + nb items (union, symmetric difference), na
 * (difference) or min(na, nb) (intersection); the count goes to *d_count (device, may be NULL) and
 * the workspace header.  na, nb < 2^32 - 1. */
int tb200_set_operation(int op, const void* d_keys_a, size_t na, const void* d_keys_b, size_t nb,
                        const void* d_vals_a, const void* d_vals_b, void* d_keys_out, void* d_vals_out,
                        int key_t, int val_bytes, int descending, unsigned long long* d_count,
                        void* d_ws, size_t* ws_bytes, tb200_stream_t stream);

/* The same exchange with splitters taken from a digit histogram instead of a sorted sample: no
 * second pass over the keys, one collective, no sampling error.  No counterpart in the reference.
 *   tb200_exchange_sizes   words of one rank's histogram row, bytes of a plan, and bytes of the plan's
 *                          head (what a host needs to read back: field, ranks, send_offset[16],
 *                          recv_total[16], tag[16], 8 bytes each after two 4-byte words);
 *   tb200_exchange_hist    d_row = histograms of the 12-bit fields of the keys' order-preserving
 *                          codes (I32/U32/F32: the top field; 64-bit keys: the four top fields),
 *                          followed by `tag` and n; all-gather the rows of all ranks (rank order);
 *   tb200_exchange_plan    from the gathered rows, identically on every rank: the highest field in
 *                          which the keys differ partitions them, contiguous bin ranges go to the
 *                          ranks in order, balanced to one bin's size; this rank's offsets into every
 *                          receive buffer (source-rank-major) and every rank's receive total;
 *   tb200_exchange_scatter one kernel: every pair stored straight into the receive buffer of the
 *                          rank that owns its bin (h_dst_keys[r] / h_dst_vals[r], local or opened
 *                          with tb200_ipc_open), in input order inside a source (stable).
 * ranks <= 16, n < 2^30 per rank.  Receivers must not touch their buffers until every sender's
 * scatter has completed (order with a collective); a stable local sort of what arrived finishes. */
int tb200_exchange_sizes(int key_t, size_t* h_row_words, size_t* h_plan_bytes, size_t* h_plan_head_bytes);
int tb200_exchange_hist(const void* d_keys, size_t n, int key_t, int descending, unsigned long long tag,
                        unsigned* d_row, tb200_stream_t stream);
int tb200_exchange_plan(const unsigned* d_rows, int ranks, int rank, int key_t, void* d_plan,
                        tb200_stream_t stream);
int tb200_exchange_scatter(const void* d_keys, const void* d_vals, size_t n, int key_t, int val_bytes,
                           int descending, const void* d_plan, int ranks, void* const* h_dst_keys,
                           void* const* h_dst_vals, void* d_ws, size_t* ws_bytes, tb200_stream_t stream);

/* Helpers of a sort_by_key whose keys and values start and end in host memory: the keys are sorted
 * together with their positions (tb200_sequence_u32: d_out[i] = i, the job of thrust::sequence,
 * thrust/system/cuda/detail/sequence.h / tabulate.h) while the values are still being copied to the
 * device, and the values are then permuted by the sorted positions (tb200_gather:
 * d_out[i] = d_src[d_index_u32[i]], the job of thrust::gather, thrust/system/cuda/detail/gather.h:
 * 41-59), which lets the device-to-host copy of the sorted keys overlap the host-to-device copy of
 * the values.  The result equals tb200_sort_by_key's (the sort is stable).  n <= 2^32 - 1;
 * val_bytes 4 or 8; d_out of tb200_sequence_u32 16-byte aligned. */
int tb200_sequence_u32(void* d_out, size_t n, tb200_stream_t stream);
int tb200_gather(const void* d_src, const void* d_index_u32, void* d_out, size_t n, int val_bytes,
                 tb200_stream_t stream);

/* Sharing device buffers between the ranks of a one-process-per-GPU job, so that a kernel on one
 * GPU reads another GPU's buffer directly over NVLink with ordinary loads (the multi-GPU sort
 * merges the runs it needs straight out of its peers' memory instead of copying them first).
 * No counterpart in the reference, which has no multi-GPU path.
 *   tb200_ipc_export   fills a 64-byte handle and the offset of d_ptr inside its allocation
 *                      (cudaIpcGetMemHandle); send both to the peer process by any means;
 *   tb200_ipc_open     maps the peer's allocation into this process (once per handle; later calls
 *                      reuse the mapping) and returns the device pointer of the same bytes;
 *   tb200_ipc_close    unmaps the allocation of one handle (every pointer tb200_ipc_open returned
 *                      for it dies; a handle that is not open is not an error): call it when the
 *                      peer is about to free or replace the buffer, after the work that used it;
 *   tb200_ipc_close_all unmaps everything opened so far.
 * The exporting process must keep the buffer allocated while peers use it, and the two sides
 * order their accesses themselves (a collective or a stream wait between writer and reader). */
int tb200_ipc_export(const void* d_ptr, void* h_handle64, size_t* h_offset);
int tb200_ipc_open(const void* h_handle64, size_t offset, void** d_ptr_out);
int tb200_ipc_close(const void* h_handle64);
int tb200_ipc_close_all(void);

#ifdef __cplusplus
}
#endif
#endif
