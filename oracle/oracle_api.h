/*
 * CPU oracle for the parallel-algorithm hot path -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * Two shared objects export exactly this interface:
 *   _ref/liboracle_ref.so   the reference Thrust 1.14.0 itself (OpenMP device system),
 *                           compiled from the reference's own headers by oracle/Makefile;
 *   _build/liboracle_port.so  a plain-C restatement of the same algorithms (oracle/port.c).
 * Only the tests, the smoke check and the CPU-baseline legs of the benchmark may load them.
 * Nothing in the product library links, imports or executes anything in this directory.
 *
 * All pointers are HOST pointers.  Element types are named by the ora_dtype codes below, which
 * are deliberately the same numbers as the product's tb200_dtype so a test can pass one code to
 * both sides.  Every function returns a count (or 0) and never allocates on behalf of the caller.
 */
#ifndef ORACLE_API_H
#define ORACLE_API_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum ora_dtype {
  ORA_I8 = 0, ORA_U8 = 1, ORA_I16 = 2, ORA_U16 = 3, ORA_I32 = 4,
  ORA_U32 = 5, ORA_I64 = 6, ORA_U64 = 7, ORA_F32 = 8, ORA_F64 = 9
};

enum ora_op { ORA_PLUS = 0, ORA_MIN = 1, ORA_MAX = 2 };

/* predicate on an integer or float element x, with two integer operands a and b:
 *   MOD_EQ: x % a == b     LT: x < a     GE: x >= a     NE: x != a                     */
enum ora_pred { ORA_PRED_MOD_EQ = 0, ORA_PRED_LT = 1, ORA_PRED_GE = 2, ORA_PRED_NE = 3 };

/* which library am I?  "reference" (Thrust OMP) or "port" (C restatement) */
const char* ora_kind(void);
/* number of OpenMP threads the library will use (1 for the port) */
int ora_threads(void);

/* thrust::reduce(first, last, init, op): accumulates in acc_t, the type of init.
 * Supported (in_t, acc_t): equal types, or a widening within the same family
 * (I8/I16/I32 -> I32/I64, U8/U16/U32 -> U32/U64, F32 -> F64).  Returns 0, or -1 if unsupported. */
int ora_reduce(const void* in, size_t n, int in_t, int acc_t, int op, const void* init, void* out);

/* thrust::inclusive_scan / exclusive_scan, element type t for input, output and accumulator;
 * in == out (in place) is allowed.  Types: I32 U32 I64 U64 F32 F64. */
int ora_inclusive_scan(const void* in, void* out, size_t n, int t, int op);
int ora_exclusive_scan(const void* in, void* out, size_t n, int t, int op, const void* init);
/* fp64-accumulated restatement of an fp32 plus-scan (running sum kept in double, rounded once
 * per output).  This, not the fp32 sequential scan, is the yardstick for fp32 parity. */
int ora_scan_f32_via_f64(const float* in, float* out, size_t n, int exclusive, float init);

/* thrust::sort / thrust::stable_sort_by_key with thrust::less (descending=0) or thrust::greater
 * (descending=1).  Keys: all ten dtypes.  val_bytes in {0, 1, 2, 4, 8} (0 = keys only). */
int ora_sort_by_key(void* keys, void* vals, size_t n, int key_t, int val_bytes, int descending);

/* thrust::stable_sort(zip(keys, vals), comp) where comp orders on the u32 key alone
 * (get<0>(a) < get<0>(b)); vals are 4-byte payloads moved bit for bit. */
int ora_stable_sort_zip_u32_by_first(uint32_t* keys, uint32_t* vals, size_t n);

/* thrust::copy_if(first, last, [stencil,] result, pred) -> number of elements written.
 * Without a stencil the predicate sees the element; with one it sees the stencil entry. */
int64_t ora_copy_if(const void* in, const void* stencil, void* out, size_t n, int t, int stencil_t,
                    int pred, int64_t a, int64_t b);

/* thrust::partition (order of the rejected half as the reference's CPU backend leaves it),
 * thrust::stable_partition (in place), thrust::stable_partition_copy.  Return: #selected. */
int64_t ora_partition(void* data, size_t n, int t, int pred, int64_t a, int64_t b);
int64_t ora_stable_partition(void* data, size_t n, int t, int pred, int64_t a, int64_t b);
int64_t ora_partition_copy(const void* in, void* out_true, void* out_false, size_t n, int t,
                           int pred, int64_t a, int64_t b);

/* thrust::unique_copy with equal_to (in == out allowed: that is thrust::unique). -> #kept */
int64_t ora_unique_copy(const void* in, void* out, size_t n, int t);

/* thrust::reduce_by_key(keys, vals, keys_out, vals_out, equal_to, op) -> number of runs */
int64_t ora_reduce_by_key(const void* keys, const void* vals, void* keys_out, void* vals_out,
                          size_t n, int key_t, int val_t, int op);
/* fp64-accumulated restatement for fp32 values (per-run sum in double, rounded once) */
int64_t ora_reduce_by_key_f32_via_f64(const void* keys, const float* vals, void* keys_out,
                                      float* vals_out, size_t n, int key_t);

/* thrust::inclusive_scan_by_key / exclusive_scan_by_key(keys, vals, out, [init,] equal_to, op): the
 * scan restarts at every run of equal keys.  val_t: I32 U32 I64 U64 F32 F64; out may be vals. */
int ora_scan_by_key(const void* keys, const void* vals, void* out, size_t n, int key_t, int val_t,
                    int op, int exclusive, const void* init);

/* thrust::unique_by_key_copy(keys, vals, keys_out, vals_out) with equal_to: first (key, value) of
 * every run.  val_bytes in {4, 8}. -> number of runs */
int64_t ora_unique_by_key_copy(const void* keys, const void* vals, void* keys_out, void* vals_out,
                               size_t n, int key_t, int val_bytes);

/* thrust::minmax_element(first, last) with less: idx[0] = position of the first smallest element,
 * idx[1] = position of the first largest (thrust::min_element / max_element return the same two).
 * n == 0 gives 0 and 0.  All ten dtypes. */
int ora_minmax_element(const void* in, size_t n, int t, uint64_t* idx);

/* thrust::merge / thrust::merge_by_key with less (or greater when descending=1); ties take
 * from range A first.  val_bytes in {0, 4, 8}. */
int ora_merge_by_key(const void* ka, const void* va, size_t na, const void* kb, const void* vb,
                     size_t nb, void* ko, void* vo, int key_t, int val_bytes, int descending);

#ifdef __cplusplus
}
#endif
#endif
