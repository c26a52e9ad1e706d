/*
 * CPU oracle, kind "port" -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A plain-C, single-threaded restatement of what the reference Thrust 1.14.0 computes on its
 * CPU backends for the algorithms on the hot path.  Each function cites the reference file it
 * follows (paths are relative to the reference checkout).  The restatement is pinned two ways by
 * the CPU test-suite: against the known-answer cases of the reference's own unit tests, and,
 * where oracle/_ref/liboracle_ref.so has been built, against the reference itself on random
 * inputs of every supported type.
 *
 * Floating-point note: integer results are order-independent; fp32/fp64 sums here are strict
 * left-to-right, which is what the reference's sequential scan and reduce_by_key do, but not
 * what its OpenMP reduce does (that one splits the range by core count), so tests compare
 * floating-point reductions with a tolerance and everything else bit for bit.
 */
#include <stdlib.h>
#include <string.h>

#include "oracle_api.h"

#define ORA_EXPORT __attribute__((visibility("default")))

ORA_EXPORT const char* ora_kind(void) { return "port"; }
ORA_EXPORT int ora_threads(void) { return 1; }

static size_t dtype_size(int t) {
  switch (t) {
    case ORA_I8: case ORA_U8: return 1;
    case ORA_I16: case ORA_U16: return 2;
    case ORA_I32: case ORA_U32: case ORA_F32: return 4;
    case ORA_I64: case ORA_U64: case ORA_F64: return 8;
  }
  return 0;
}

/* X(code, ctype, suffix) */
#define FOR_ALL_TYPES(X) \
  X(ORA_I8, int8_t, i8) X(ORA_U8, uint8_t, u8) X(ORA_I16, int16_t, i16) X(ORA_U16, uint16_t, u16) \
  X(ORA_I32, int32_t, i32) X(ORA_U32, uint32_t, u32) X(ORA_I64, int64_t, i64) \
  X(ORA_U64, uint64_t, u64) X(ORA_F32, float, f32) X(ORA_F64, double, f64)
#define FOR_WIDE_TYPES(X) \
  X(ORA_I32, int32_t, i32) X(ORA_U32, uint32_t, u32) X(ORA_I64, int64_t, i64) \
  X(ORA_U64, uint64_t, u64) X(ORA_F32, float, f32) X(ORA_F64, double, f64)

/* ---------------------------------------------------------------- reduce
 * thrust/system/omp/detail/reduce.inl:48-62 computes init (+) x0 (+) ... (+) x(n-1) in the type
 * of init, each input converted to that type first (thrust/system/cuda/detail/reduce.h:1031-1043
 * has the same contract).  Order differs per backend; for integers it does not matter. */
#define REDUCE_BODY(IN, ACC)                                                           \
  {                                                                                    \
    const IN* p = (const IN*)in; ACC acc; memcpy(&acc, init, sizeof(ACC));             \
    for (size_t i = 0; i < n; ++i) {                                                   \
      ACC x = (ACC)p[i];                                                               \
      if (op == ORA_PLUS) acc = (ACC)(acc + x);                                        \
      else if (op == ORA_MIN) acc = x < acc ? x : acc;                                 \
      else acc = acc < x ? x : acc;                                                    \
    }                                                                                  \
    memcpy(out, &acc, sizeof(ACC)); return 0;                                          \
  }

ORA_EXPORT int ora_reduce(const void* in, size_t n, int in_t, int acc_t, int op, const void* init,
                          void* out) {
#define RCASE(ti, IN, ta, ACC) if (in_t == ti && acc_t == ta) REDUCE_BODY(IN, ACC)
  RCASE(ORA_I8, int8_t, ORA_I32, int32_t) RCASE(ORA_I8, int8_t, ORA_I64, int64_t)
  RCASE(ORA_I16, int16_t, ORA_I32, int32_t) RCASE(ORA_I16, int16_t, ORA_I64, int64_t)
  RCASE(ORA_I32, int32_t, ORA_I32, int32_t) RCASE(ORA_I32, int32_t, ORA_I64, int64_t)
  RCASE(ORA_U8, uint8_t, ORA_U32, uint32_t) RCASE(ORA_U8, uint8_t, ORA_U64, uint64_t)
  RCASE(ORA_U16, uint16_t, ORA_U32, uint32_t) RCASE(ORA_U16, uint16_t, ORA_U64, uint64_t)
  RCASE(ORA_U32, uint32_t, ORA_U32, uint32_t) RCASE(ORA_U32, uint32_t, ORA_U64, uint64_t)
  RCASE(ORA_I64, int64_t, ORA_I64, int64_t) RCASE(ORA_U64, uint64_t, ORA_U64, uint64_t)
  RCASE(ORA_F32, float, ORA_F32, float) RCASE(ORA_F32, float, ORA_F64, double)
  RCASE(ORA_F64, double, ORA_F64, double)
#undef RCASE
  return -1;
}

/* ---------------------------------------------------------------- scan
 * thrust/system/omp/detail/scan.h:22 forwards to thrust/system/detail/sequential/scan.h:
 * inclusive (:48-76) keeps `sum` in the input value type; exclusive (:87-118) reads the input
 * element into a temporary before writing, so that in == out works. */
#define SCAN_CASE(code, T, sfx)                                                        \
  if (t == code) {                                                                     \
    const T* p = (const T*)in; T* o = (T*)out;                                         \
    if (n == 0) return 0;                                                              \
    T sum = p[0]; o[0] = sum;                                                          \
    for (size_t i = 1; i < n; ++i) {                                                   \
      T x = p[i];                                                                      \
      if (op == ORA_PLUS) sum = (T)(sum + x);                                          \
      else if (op == ORA_MIN) sum = x < sum ? x : sum;                                 \
      else sum = sum < x ? x : sum;                                                    \
      o[i] = sum;                                                                      \
    }                                                                                  \
    return 0;                                                                          \
  }
ORA_EXPORT int ora_inclusive_scan(const void* in, void* out, size_t n, int t, int op) {
  FOR_WIDE_TYPES(SCAN_CASE)
  return -1;
}

#define XSCAN_CASE(code, T, sfx)                                                       \
  if (t == code) {                                                                     \
    const T* p = (const T*)in; T* o = (T*)out; T sum; memcpy(&sum, init, sizeof(T));   \
    for (size_t i = 0; i < n; ++i) {                                                   \
      T x = p[i]; o[i] = sum;                                                          \
      if (op == ORA_PLUS) sum = (T)(sum + x);                                          \
      else if (op == ORA_MIN) sum = x < sum ? x : sum;                                 \
      else sum = sum < x ? x : sum;                                                    \
    }                                                                                  \
    return 0;                                                                          \
  }
ORA_EXPORT int ora_exclusive_scan(const void* in, void* out, size_t n, int t, int op,
                                  const void* init) {
  FOR_WIDE_TYPES(XSCAN_CASE)
  return -1;
}

ORA_EXPORT int ora_scan_f32_via_f64(const float* in, float* out, size_t n, int exclusive,
                                    float init) {
  /* same loop shape as sequential/scan.h:67-72 and :104-113 with the running sum in double */
  double sum = exclusive ? (double)init : 0.0;
  for (size_t i = 0; i < n; ++i) {
    float x = in[i];
    if (exclusive) { out[i] = (float)sum; sum += (double)x; }
    else { sum += (double)x; out[i] = (float)sum; }
  }
  return 0;
}

/* ---------------------------------------------------------------- sort
 * Keys are mapped to unsigned integers whose natural order is the key order, exactly as the
 * RadixEncoder specialisations do (thrust/system/detail/sequential/stable_radix_sort.inl:54-138:
 * unsigned unchanged, signed with the sign bit flipped, floating point with all bits flipped if
 * negative else only the sign bit).  The sort itself is a stable LSD radix sort on 8-bit digits
 * that skips a pass whose histogram puts every key in one bucket (same file, :243-324).  Any
 * stable sort yields the same output, which is why the result also equals the reference's
 * per-thread radix + stable merge tree (thrust/system/omp/detail/sort.inl:181-254). */
static uint64_t encode_key(const void* p, int t) {
  switch (t) {
    case ORA_U8: return *(const uint8_t*)p;
    case ORA_U16: return *(const uint16_t*)p;
    case ORA_U32: return *(const uint32_t*)p;
    case ORA_U64: return *(const uint64_t*)p;
    case ORA_I8: return (uint8_t)(*(const uint8_t*)p ^ 0x80u);
    case ORA_I16: return (uint16_t)(*(const uint16_t*)p ^ 0x8000u);
    case ORA_I32: return *(const uint32_t*)p ^ 0x80000000u;
    case ORA_I64: return *(const uint64_t*)p ^ 0x8000000000000000ull;
    case ORA_F32: {
      uint32_t u = *(const uint32_t*)p;
      uint32_t mask = (uint32_t)(-(int32_t)(u >> 31)) | 0x80000000u;
      return u ^ mask;
    }
    case ORA_F64: {
      uint64_t u = *(const uint64_t*)p;
      uint64_t mask = (uint64_t)(-(int64_t)(u >> 63)) | 0x8000000000000000ull;
      return u ^ mask;
    }
  }
  return 0;
}

/* sorts the permutation `idx` (initially identity) by the encoded keys `enc`, stably */
static void radix_argsort(const uint64_t* enc, size_t n, int key_bytes, uint32_t* idx,
                          uint32_t* tmp) {
  for (int pass = 0; pass < key_bytes; ++pass) {
    size_t hist[256] = {0};
    int shift = 8 * pass;
    for (size_t i = 0; i < n; ++i) hist[(enc[i] >> shift) & 255]++;
    int skip = 0;
    for (int d = 0; d < 256; ++d) if (hist[d] == n) skip = 1;
    if (skip) continue;
    size_t sum = 0;
    for (int d = 0; d < 256; ++d) { size_t c = hist[d]; hist[d] = sum; sum += c; }
    for (size_t i = 0; i < n; ++i) tmp[hist[(enc[idx[i]] >> shift) & 255]++] = idx[i];
    memcpy(idx, tmp, n * sizeof(uint32_t));
  }
}

static void apply_perm(void* data, size_t n, size_t elem, const uint32_t* idx) {
  if (!data || !elem || !n) return;
  char* copy = (char*)malloc(n * elem);
  memcpy(copy, data, n * elem);
  for (size_t i = 0; i < n; ++i) memcpy((char*)data + i * elem, copy + (size_t)idx[i] * elem, elem);
  free(copy);
}

ORA_EXPORT int ora_sort_by_key(void* keys, void* vals, size_t n, int key_t, int val_bytes,
                               int descending) {
  size_t ks = dtype_size(key_t);
  if (!ks || n > 0xffffffffu) return -1;
  if (n == 0) return 0;
  uint64_t* enc = (uint64_t*)malloc(n * sizeof(uint64_t));
  uint32_t* idx = (uint32_t*)malloc(n * sizeof(uint32_t));
  uint32_t* tmp = (uint32_t*)malloc(n * sizeof(uint32_t));
  uint64_t flip = descending ? (ks == 8 ? ~0ull : ((1ull << (8 * ks)) - 1)) : 0;
  for (size_t i = 0; i < n; ++i) {
    /* thrust::greater on the same stable sort == ascending order of the complemented code */
    enc[i] = encode_key((const char*)keys + i * ks, key_t) ^ flip;
    idx[i] = (uint32_t)i;
  }
  radix_argsort(enc, n, (int)ks, idx, tmp);
  apply_perm(keys, n, ks, idx);
  apply_perm(vals, n, (size_t)val_bytes, idx);
  free(enc); free(idx); free(tmp);
  return 0;
}

/* thrust::stable_sort on zip(keys, vals) with a comparator that looks at get<0> only takes the
 * comparison-sort route (thrust/system/omp/detail/sort.inl:100-170: per-thread stable merge sort
 * + stable merges).  A stable sort by the u32 key moves each (key, val) pair as a unit, so the
 * stable radix sort above produces the identical sequence. */
ORA_EXPORT int ora_stable_sort_zip_u32_by_first(uint32_t* keys, uint32_t* vals, size_t n) {
  return ora_sort_by_key(keys, vals, n, ORA_U32, 4, 0);
}

/* ---------------------------------------------------------------- predicates */
#define PRED_FN(code, T, sfx)                                                          \
  static int pred_##sfx(const void* p, int kind, int64_t a, int64_t b) {               \
    T x = *(const T*)p;                                                                \
    switch (kind) {                                                                    \
      case ORA_PRED_MOD_EQ: return (int64_t)x % a == b;                                \
      case ORA_PRED_LT: return x < (T)a;                                               \
      case ORA_PRED_GE: return x >= (T)a;                                              \
      default: return x != (T)a;                                                       \
    }                                                                                  \
  }
FOR_ALL_TYPES(PRED_FN)

typedef int (*pred_fn)(const void*, int, int64_t, int64_t);
static pred_fn pred_for(int t) {
#define PRED_PICK(code, T, sfx) if (t == code) return pred_##sfx;
  FOR_ALL_TYPES(PRED_PICK)
  return 0;
}

/* ---------------------------------------------------------------- copy_if
 * Stable compaction; the stencil form tests the stencil entry and copies the item
 * (thrust/system/detail/generic/copy_if.inl:54-94, thrust/system/cuda/detail/copy_if.h:388-415). */
ORA_EXPORT int64_t ora_copy_if(const void* in, const void* stencil, void* out, size_t n, int t,
                               int stencil_t, int pred, int64_t a, int64_t b) {
  size_t es = dtype_size(t);
  const char* tested = stencil ? (const char*)stencil : (const char*)in;
  int tt = stencil ? stencil_t : t;
  size_t ts = dtype_size(tt);
  pred_fn f = pred_for(tt);
  if (!es || !f) return -1;
  int64_t cnt = 0;
  for (size_t i = 0; i < n; ++i)
    if (f(tested + i * ts, pred, a, b)) {
      memmove((char*)out + (size_t)cnt * es, (const char*)in + i * es, es);
      ++cnt;
    }
  return cnt;
}

/* ---------------------------------------------------------------- partition
 * thrust::partition on the CPU backends is the forward swap loop of
 * thrust/system/detail/sequential/partition.h:72-101 (OMP does not override it): skip the
 * leading selected elements, then swap each later selected element into the first rejected
 * slot.  Selected elements keep their order; rejected ones do not. */
ORA_EXPORT int64_t ora_partition(void* data, size_t n, int t, int pred, int64_t a, int64_t b) {
  size_t es = dtype_size(t); pred_fn f = pred_for(t);
  if (!es || !f) return -1;
  char* d = (char*)data; char tmp[8];
  size_t first = 0;
  if (n == 0) return 0;
  while (f(d + first * es, pred, a, b)) if (++first == n) return (int64_t)first;
  for (size_t next = first + 1; next < n; ++next)
    if (f(d + next * es, pred, a, b)) {
      memcpy(tmp, d + first * es, es);
      memcpy(d + first * es, d + next * es, es);
      memcpy(d + next * es, tmp, es);
      ++first;
    }
  return (int64_t)first;
}

/* stable_partition_copy: selected to out_true, rejected to out_false, both in input order
 * (thrust/system/detail/sequential/partition.h:265-305; CUDA: partition.h:265-272). */
ORA_EXPORT int64_t ora_partition_copy(const void* in, void* out_true, void* out_false, size_t n,
                                      int t, int pred, int64_t a, int64_t b) {
  size_t es = dtype_size(t); pred_fn f = pred_for(t);
  if (!es || !f) return -1;
  size_t nt = 0, nf = 0;
  for (size_t i = 0; i < n; ++i) {
    const char* p = (const char*)in + i * es;
    if (f(p, pred, a, b)) memcpy((char*)out_true + (nt++) * es, p, es);
    else memcpy((char*)out_false + (nf++) * es, p, es);
  }
  return (int64_t)nt;
}

/* stable_partition in place: copy out, then stable_partition_copy back with the rejected
 * elements following the selected ones (thrust/system/detail/sequential/partition.h:180-262). */
ORA_EXPORT int64_t ora_stable_partition(void* data, size_t n, int t, int pred, int64_t a,
                                        int64_t b) {
  size_t es = dtype_size(t); pred_fn f = pred_for(t);
  if (!es || !f) return -1;
  if (n == 0) return 0;
  char* copy = (char*)malloc(n * es);
  memcpy(copy, data, n * es);
  size_t nt = 0;
  for (size_t i = 0; i < n; ++i) nt += (size_t)(f(copy + i * es, pred, a, b) != 0);
  int64_t r = ora_partition_copy(copy, data, (char*)data + nt * es, n, t, pred, a, b);
  free(copy);
  return r;
}

/* ---------------------------------------------------------------- unique
 * Keeps the first element of every run of equal neighbours; element i is compared with element
 * i-1 of the INPUT (thrust/system/cuda/detail/unique.h:344-354), which for equal_to gives the
 * same survivors as the sequential loop (thrust/system/detail/sequential/unique.h:41-76). */
#define UNIQUE_CASE(code, T, sfx)                                                      \
  if (t == code) {                                                                     \
    const T* p = (const T*)in; T* o = (T*)out; int64_t cnt = 0;                        \
    T prev = 0;                                                                        \
    for (size_t i = 0; i < n; ++i) {                                                   \
      T x = p[i];                                                                      \
      if (i == 0 || !(prev == x)) o[cnt++] = x;                                        \
      prev = x;                                                                        \
    }                                                                                  \
    return cnt;                                                                        \
  }
ORA_EXPORT int64_t ora_unique_copy(const void* in, void* out, size_t n, int t) {
  FOR_ALL_TYPES(UNIQUE_CASE)
  return -1;
}

/* ---------------------------------------------------------------- reduce_by_key
 * A run starts where key[i] != key[i-1]; its key is the first key of the run and its value the
 * left-to-right reduction of the run's values in the value type
 * (thrust/system/detail/generic/reduce_by_key.inl:81-135, scanned sequentially on the CPU
 * backends; CUDA: thrust/system/cuda/detail/reduce_by_key.h:584-620). */
#define RBK_VAL_CASE(code, V, sfx)                                                     \
  if (val_t == code) {                                                                 \
    const V* v = (const V*)vals; V* vo = (V*)vals_out; V acc = 0;                      \
    for (size_t i = 0; i < n; ++i) {                                                   \
      const char* kp = (const char*)keys + i * ks;                                     \
      int head = i == 0 || !key_eq(kp, kp - ks, key_t);                                \
      if (head) {                                                                      \
        if (i) vo[runs - 1] = acc;                                                     \
        memcpy((char*)keys_out + (size_t)runs * ks, kp, ks); ++runs; acc = v[i];       \
      } else if (op == ORA_PLUS) acc = (V)(acc + v[i]);                                \
      else if (op == ORA_MIN) acc = v[i] < acc ? v[i] : acc;                           \
      else acc = acc < v[i] ? v[i] : acc;                                              \
    }                                                                                  \
    if (n) vo[runs - 1] = acc;                                                         \
    return runs;                                                                       \
  }

static int key_eq(const void* x, const void* y, int t) {
  if (t == ORA_F32) return *(const float*)x == *(const float*)y;
  if (t == ORA_F64) return *(const double*)x == *(const double*)y;
  return memcmp(x, y, dtype_size(t)) == 0;
}

ORA_EXPORT int64_t ora_reduce_by_key(const void* keys, const void* vals, void* keys_out,
                                     void* vals_out, size_t n, int key_t, int val_t, int op) {
  size_t ks = dtype_size(key_t); int64_t runs = 0;
  if (!ks) return -1;
  FOR_WIDE_TYPES(RBK_VAL_CASE)
  return -1;
}

ORA_EXPORT int64_t ora_reduce_by_key_f32_via_f64(const void* keys, const float* vals,
                                                 void* keys_out, float* vals_out, size_t n,
                                                 int key_t) {
  size_t ks = dtype_size(key_t); int64_t runs = 0; double acc = 0.0;
  if (!ks) return -1;
  for (size_t i = 0; i < n; ++i) {
    const char* kp = (const char*)keys + i * ks;
    if (i == 0 || !key_eq(kp, kp - ks, key_t)) {
      if (i) vals_out[runs - 1] = (float)acc;
      memcpy((char*)keys_out + (size_t)runs * ks, kp, ks); ++runs; acc = 0.0;
    }
    acc += (double)vals[i];
  }
  if (n) vals_out[runs - 1] = (float)acc;
  return runs;
}

/* ---------------------------------------------------------------- scan_by_key, unique_by_key
 * The scan restarts wherever key[i] != key[i-1] (thrust/system/detail/generic/scan_by_key.inl:
 * 103-131 builds head flags this way and scans (value, flag) pairs with segmented_scan_functor,
 * :43-61; the exclusive form, :198-234, seeds every run with init).  Left to right in the value
 * type. */
#define SBK_VAL_CASE(code, V, sfx)                                                     \
  if (val_t == code) {                                                                 \
    const V* v = (const V*)vals; V* o = (V*)out; V i0 = 0; V acc = 0;                  \
    if (exclusive) memcpy(&i0, init, sizeof(V));                                       \
    for (size_t i = 0; i < n; ++i) {                                                   \
      const char* kp = (const char*)keys + i * ks;                                     \
      int head = i == 0 || !key_eq(kp, kp - ks, key_t);                                \
      V x = v[i];                                                                      \
      if (exclusive) {                                                                 \
        if (head) acc = i0;                                                            \
        o[i] = acc;                                                                    \
        if (op == ORA_PLUS) acc = (V)(acc + x);                                        \
        else if (op == ORA_MIN) acc = x < acc ? x : acc;                               \
        else acc = acc < x ? x : acc;                                                  \
      } else {                                                                         \
        if (head) acc = x;                                                             \
        else if (op == ORA_PLUS) acc = (V)(acc + x);                                   \
        else if (op == ORA_MIN) acc = x < acc ? x : acc;                               \
        else acc = acc < x ? x : acc;                                                  \
        o[i] = acc;                                                                    \
      }                                                                                \
    }                                                                                  \
    return 0;                                                                          \
  }
ORA_EXPORT int ora_scan_by_key(const void* keys, const void* vals, void* out, size_t n, int key_t,
                               int val_t, int op, int exclusive, const void* init) {
  size_t ks = dtype_size(key_t);
  if (!ks) return -1;
  FOR_WIDE_TYPES(SBK_VAL_CASE)
  return -1;
}

/* unique_by_key_copy keeps the first (key, value) of every run
 * (thrust/system/detail/generic/unique_by_key.inl: unique_by_key_copy with equal_to). */
ORA_EXPORT int64_t ora_unique_by_key_copy(const void* keys, const void* vals, void* keys_out,
                                          void* vals_out, size_t n, int key_t, int val_bytes) {
  size_t ks = dtype_size(key_t), vs = (size_t)val_bytes;
  int64_t cnt = 0;
  if (!ks || !vs) return -1;
  for (size_t i = 0; i < n; ++i) {
    const char* kp = (const char*)keys + i * ks;
    if (i == 0 || !key_eq(kp, kp - ks, key_t)) {
      memmove((char*)keys_out + (size_t)cnt * ks, kp, ks);
      memmove((char*)vals_out + (size_t)cnt * vs, (const char*)vals + i * vs, vs);
      ++cnt;
    }
  }
  return cnt;
}

/* ---------------------------------------------------------------- extrema
 * One sequential walk with strict comparisons, so the first smallest and the first largest element
 * win (thrust/system/detail/sequential/extrema.h:36-118: "if comp(*first, *min) min = first" and
 * "if comp(*max, *first) max = first"). */
#define MINMAX_CASE(T, CODE)                                                           \
  if (t == CODE) {                                                                     \
    const T* p = (const T*)in; size_t lo = 0, hi = 0;                                  \
    for (size_t i = 1; i < n; ++i) { if (p[i] < p[lo]) lo = i; if (p[hi] < p[i]) hi = i; } \
    idx[0] = lo; idx[1] = hi; return 0;                                                \
  }
ORA_EXPORT int ora_minmax_element(const void* in, size_t n, int t, uint64_t* idx) {
  MINMAX_CASE(int8_t, ORA_I8) MINMAX_CASE(uint8_t, ORA_U8) MINMAX_CASE(int16_t, ORA_I16) MINMAX_CASE(uint16_t, ORA_U16)
  MINMAX_CASE(int32_t, ORA_I32) MINMAX_CASE(uint32_t, ORA_U32) MINMAX_CASE(int64_t, ORA_I64) MINMAX_CASE(uint64_t, ORA_U64)
  MINMAX_CASE(float, ORA_F32) MINMAX_CASE(double, ORA_F64)
  return -1;
}

/* ---------------------------------------------------------------- merge
 * Sequential two-finger merge; on equal keys the element of range A is emitted first
 * (thrust/system/detail/sequential/merge.inl:36-76 and :85-140: "if comp(*first2, *first1) take
 * from 2 else take from 1").  thrust::greater is the same walk on complemented key codes. */
ORA_EXPORT int ora_merge_by_key(const void* ka, const void* va, size_t na, const void* kb,
                                const void* vb, size_t nb, void* ko, void* vo, int key_t,
                                int val_bytes, int descending) {
  size_t ks = dtype_size(key_t), vs = (size_t)val_bytes;
  if (!ks) return -1;
  size_t i = 0, j = 0, o = 0;
  while (i < na || j < nb) {
    int take_b;
    if (i == na) take_b = 1;
    else if (j == nb) take_b = 0;
    else {
      uint64_t ea = encode_key((const char*)ka + i * ks, key_t);
      uint64_t eb = encode_key((const char*)kb + j * ks, key_t);
      take_b = descending ? (eb > ea) : (eb < ea);
    }
    if (take_b) {
      memcpy((char*)ko + o * ks, (const char*)kb + j * ks, ks);
      if (vs) memcpy((char*)vo + o * vs, (const char*)vb + j * vs, vs);
      ++j;
    } else {
      memcpy((char*)ko + o * ks, (const char*)ka + i * ks, ks);
      if (vs) memcpy((char*)vo + o * vs, (const char*)va + i * vs, vs);
      ++i;
    }
    ++o;
  }
  return 0;
}
