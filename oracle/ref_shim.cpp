// CPU oracle, kind "reference" -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// Thin extern "C" wrappers around the reference Thrust (1.14.0) compiled with its OpenMP device
// system: every function below is one call of the reference's public algorithm under
// thrust::device, which with THRUST_DEVICE_SYSTEM=THRUST_DEVICE_SYSTEM_OMP resolves to
// thrust/system/omp/detail/*.  The reference headers are taken from the include path given by
// oracle/Makefile (the read-only reference checkout); no reference source is copied here.
// The resulting shared object is written to oracle/_ref/ and is never committed.
#include <thrust/execution_policy.h>
#include <thrust/reduce.h>
#include <thrust/scan.h>
#include <thrust/sort.h>
#include <thrust/copy.h>
#include <thrust/partition.h>
#include <thrust/unique.h>
#include <thrust/merge.h>
#include <thrust/extrema.h>
#include <thrust/scan.h>
#include <thrust/functional.h>
#include <thrust/iterator/zip_iterator.h>
#include <thrust/tuple.h>
#include <omp.h>
#include <cstring>
#include <vector>

#include "oracle_api.h"

#define ORA_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

template <typename T> struct min_op { T operator()(T a, T b) const { return b < a ? b : a; } };
template <typename T> struct max_op { T operator()(T a, T b) const { return a < b ? b : a; } };

struct pred_t {
  int kind; int64_t a, b;
  template <typename T> bool operator()(T x) const {
    switch (kind) {
      case ORA_PRED_MOD_EQ: return (int64_t)x % a == b;
      case ORA_PRED_LT: return x < (T)a;
      case ORA_PRED_GE: return x >= (T)a;
      default: return x != (T)a;
    }
  }
};

template <typename F> int by_dtype(int t, F f) {
  switch (t) {
    case ORA_I8: f((int8_t)0); return 0;
    case ORA_U8: f((uint8_t)0); return 0;
    case ORA_I16: f((int16_t)0); return 0;
    case ORA_U16: f((uint16_t)0); return 0;
    case ORA_I32: f((int32_t)0); return 0;
    case ORA_U32: f((uint32_t)0); return 0;
    case ORA_I64: f((int64_t)0); return 0;
    case ORA_U64: f((uint64_t)0); return 0;
    case ORA_F32: f((float)0); return 0;
    case ORA_F64: f((double)0); return 0;
  }
  return -1;
}
template <typename F> int by_wide_dtype(int t, F f) {  // 4- and 8-byte arithmetic types only
  switch (t) {
    case ORA_I32: f((int32_t)0); return 0;
    case ORA_U32: f((uint32_t)0); return 0;
    case ORA_I64: f((int64_t)0); return 0;
    case ORA_U64: f((uint64_t)0); return 0;
    case ORA_F32: f((float)0); return 0;
    case ORA_F64: f((double)0); return 0;
  }
  return -1;
}
template <typename F> int by_bytes(int nbytes, F f) {
  switch (nbytes) {
    case 1: f((uint8_t)0); return 0;
    case 2: f((uint16_t)0); return 0;
    case 4: f((uint32_t)0); return 0;
    case 8: f((uint64_t)0); return 0;
  }
  return -1;
}

template <typename In, typename Acc>
void reduce_typed(const void* in, size_t n, int op, const void* init, void* out) {
  const In* p = static_cast<const In*>(in);
  Acc i0; std::memcpy(&i0, init, sizeof(Acc));
  Acc r;
  if (op == ORA_PLUS) r = thrust::reduce(thrust::device, p, p + n, i0, thrust::plus<Acc>());
  else if (op == ORA_MIN) r = thrust::reduce(thrust::device, p, p + n, i0, min_op<Acc>());
  else r = thrust::reduce(thrust::device, p, p + n, i0, max_op<Acc>());
  std::memcpy(out, &r, sizeof(Acc));
}

bool widens(int in_t, int acc_t) {
  if (in_t == acc_t) return true;
  bool sin = in_t == ORA_I8 || in_t == ORA_I16 || in_t == ORA_I32;
  bool uin = in_t == ORA_U8 || in_t == ORA_U16 || in_t == ORA_U32;
  if (sin && (acc_t == ORA_I32 || acc_t == ORA_I64)) return true;
  if (uin && (acc_t == ORA_U32 || acc_t == ORA_U64)) return true;
  if (in_t == ORA_F32 && acc_t == ORA_F64) return true;
  return false;
}

}  // namespace

ORA_EXPORT const char* ora_kind(void) { return "reference"; }
ORA_EXPORT int ora_threads(void) { return omp_get_max_threads(); }

ORA_EXPORT int ora_reduce(const void* in, size_t n, int in_t, int acc_t, int op, const void* init,
                          void* out) {
  if (!widens(in_t, acc_t)) return -1;
  return by_dtype(in_t, [&](auto iv) {
    by_dtype(acc_t, [&](auto av) {
      using In = decltype(iv); using Acc = decltype(av);
      // only instantiate the widening combinations: anything else was rejected above
      if constexpr (sizeof(Acc) >= sizeof(In) && sizeof(Acc) >= 4 &&
                    std::is_floating_point<In>::value == std::is_floating_point<Acc>::value &&
                    std::is_signed<In>::value == std::is_signed<Acc>::value)
        reduce_typed<In, Acc>(in, n, op, init, out);
    });
  });
}

ORA_EXPORT int ora_inclusive_scan(const void* in, void* out, size_t n, int t, int op) {
  return by_wide_dtype(t, [&](auto v) {
    using T = decltype(v);
    const T* p = static_cast<const T*>(in); T* o = static_cast<T*>(out);
    if (op == ORA_PLUS) thrust::inclusive_scan(thrust::device, p, p + n, o, thrust::plus<T>());
    else if (op == ORA_MIN) thrust::inclusive_scan(thrust::device, p, p + n, o, min_op<T>());
    else thrust::inclusive_scan(thrust::device, p, p + n, o, max_op<T>());
  });
}

ORA_EXPORT int ora_exclusive_scan(const void* in, void* out, size_t n, int t, int op,
                                  const void* init) {
  return by_wide_dtype(t, [&](auto v) {
    using T = decltype(v);
    const T* p = static_cast<const T*>(in); T* o = static_cast<T*>(out);
    T i0; std::memcpy(&i0, init, sizeof(T));
    if (op == ORA_PLUS) thrust::exclusive_scan(thrust::device, p, p + n, o, i0, thrust::plus<T>());
    else if (op == ORA_MIN) thrust::exclusive_scan(thrust::device, p, p + n, o, i0, min_op<T>());
    else thrust::exclusive_scan(thrust::device, p, p + n, o, i0, max_op<T>());
  });
}

ORA_EXPORT int ora_scan_f32_via_f64(const float* in, float* out, size_t n, int exclusive,
                                    float init) {
  // Not a reference call: the fp64-accumulated yardstick, restating the loop shape of
  // thrust/system/detail/sequential/scan.h:67-72 (inclusive) and :104-113 (exclusive).
  double sum = exclusive ? (double)init : 0.0;
  for (size_t i = 0; i < n; ++i) {
    float x = in[i];
    if (exclusive) { out[i] = (float)sum; sum += (double)x; }
    else { sum += (double)x; out[i] = (float)sum; }
  }
  return 0;
}

ORA_EXPORT int ora_sort_by_key(void* keys, void* vals, size_t n, int key_t, int val_bytes,
                               int descending) {
  int rc = by_dtype(key_t, [&](auto kv) {
    using K = decltype(kv);
    K* k = static_cast<K*>(keys);
    if (val_bytes == 0) {
      if (descending) thrust::stable_sort(thrust::device, k, k + n, thrust::greater<K>());
      else thrust::stable_sort(thrust::device, k, k + n, thrust::less<K>());
    } else {
      by_bytes(val_bytes, [&](auto vv) {
        using V = decltype(vv);
        V* v = static_cast<V*>(vals);
        if (descending)
          thrust::stable_sort_by_key(thrust::device, k, k + n, v, thrust::greater<K>());
        else
          thrust::stable_sort_by_key(thrust::device, k, k + n, v, thrust::less<K>());
      });
    }
  });
  return rc;
}

namespace {
struct first_less {
  template <typename A, typename B> bool operator()(const A& a, const B& b) const {
    return thrust::get<0>(a) < thrust::get<0>(b);
  }
};
}  // namespace

ORA_EXPORT int ora_stable_sort_zip_u32_by_first(uint32_t* keys, uint32_t* vals, size_t n) {
  auto z = thrust::make_zip_iterator(thrust::make_tuple(keys, vals));
  thrust::stable_sort(thrust::device, z, z + n, first_less());
  return 0;
}

ORA_EXPORT int64_t ora_copy_if(const void* in, const void* stencil, void* out, size_t n, int t,
                               int stencil_t, int pred, int64_t a, int64_t b) {
  int64_t cnt = -1;
  pred_t p{pred, a, b};
  by_dtype(t, [&](auto v) {
    using T = decltype(v);
    const T* i = static_cast<const T*>(in); T* o = static_cast<T*>(out);
    if (!stencil) { cnt = thrust::copy_if(thrust::device, i, i + n, o, p) - o; return; }
    by_dtype(stencil_t, [&](auto sv) {
      using S = decltype(sv);
      const S* s = static_cast<const S*>(stencil);
      cnt = thrust::copy_if(thrust::device, i, i + n, s, o, p) - o;
    });
  });
  return cnt;
}

ORA_EXPORT int64_t ora_partition(void* data, size_t n, int t, int pred, int64_t a, int64_t b) {
  int64_t cnt = -1; pred_t p{pred, a, b};
  by_dtype(t, [&](auto v) {
    using T = decltype(v); T* d = static_cast<T*>(data);
    cnt = thrust::partition(thrust::device, d, d + n, p) - d;
  });
  return cnt;
}

ORA_EXPORT int64_t ora_stable_partition(void* data, size_t n, int t, int pred, int64_t a,
                                        int64_t b) {
  int64_t cnt = -1; pred_t p{pred, a, b};
  by_dtype(t, [&](auto v) {
    using T = decltype(v); T* d = static_cast<T*>(data);
    cnt = thrust::stable_partition(thrust::device, d, d + n, p) - d;
  });
  return cnt;
}

ORA_EXPORT int64_t ora_partition_copy(const void* in, void* out_true, void* out_false, size_t n,
                                      int t, int pred, int64_t a, int64_t b) {
  int64_t cnt = -1; pred_t p{pred, a, b};
  by_dtype(t, [&](auto v) {
    using T = decltype(v);
    const T* i = static_cast<const T*>(in);
    T* ot = static_cast<T*>(out_true); T* of = static_cast<T*>(out_false);
    cnt = thrust::stable_partition_copy(thrust::device, i, i + n, ot, of, p).first - ot;
  });
  return cnt;
}

ORA_EXPORT int64_t ora_unique_copy(const void* in, void* out, size_t n, int t) {
  int64_t cnt = -1;
  by_dtype(t, [&](auto v) {
    using T = decltype(v);
    const T* i = static_cast<const T*>(in); T* o = static_cast<T*>(out);
    if (in == out) cnt = thrust::unique(thrust::device, o, o + n) - o;
    else cnt = thrust::unique_copy(thrust::device, i, i + n, o) - o;
  });
  return cnt;
}

ORA_EXPORT int64_t ora_reduce_by_key(const void* keys, const void* vals, void* keys_out,
                                     void* vals_out, size_t n, int key_t, int val_t, int op) {
  int64_t cnt = -1;
  by_dtype(key_t, [&](auto kv) {
    using K = decltype(kv);
    const K* k = static_cast<const K*>(keys); K* ko = static_cast<K*>(keys_out);
    by_wide_dtype(val_t, [&](auto vv) {
      using V = decltype(vv);
      const V* v = static_cast<const V*>(vals); V* vo = static_cast<V*>(vals_out);
      if (op == ORA_PLUS)
        cnt = thrust::reduce_by_key(thrust::device, k, k + n, v, ko, vo, thrust::equal_to<K>(),
                                    thrust::plus<V>()).first - ko;
      else if (op == ORA_MIN)
        cnt = thrust::reduce_by_key(thrust::device, k, k + n, v, ko, vo, thrust::equal_to<K>(),
                                    min_op<V>()).first - ko;
      else
        cnt = thrust::reduce_by_key(thrust::device, k, k + n, v, ko, vo, thrust::equal_to<K>(),
                                    max_op<V>()).first - ko;
    });
  });
  return cnt;
}

ORA_EXPORT int64_t ora_reduce_by_key_f32_via_f64(const void* keys, const float* vals,
                                                 void* keys_out, float* vals_out, size_t n,
                                                 int key_t) {
  // Not a reference call: fp64 yardstick with the run semantics of
  // thrust/system/detail/generic/reduce_by_key.inl:98-133 (a run starts where key[i] != key[i-1];
  // its output key is the first key of the run).
  int64_t runs = 0;
  by_dtype(key_t, [&](auto kv) {
    using K = decltype(kv);
    const K* k = static_cast<const K*>(keys); K* ko = static_cast<K*>(keys_out);
    double acc = 0.0;
    for (size_t i = 0; i < n; ++i) {
      if (i == 0 || !(k[i] == k[i - 1])) {
        if (i) vals_out[runs - 1] = (float)acc;
        ko[runs++] = k[i]; acc = 0.0;
      }
      acc += (double)vals[i];
    }
    if (n) vals_out[runs - 1] = (float)acc;
  });
  return runs;
}

ORA_EXPORT int ora_scan_by_key(const void* keys, const void* vals, void* out, size_t n, int key_t, int val_t, int op,
                               int exclusive, const void* init) {
  int rc = -1;
  by_dtype(key_t, [&](auto kv) {
    using K = decltype(kv);
    const K* k = static_cast<const K*>(keys);
    rc = by_wide_dtype(val_t, [&](auto vv) {
      using V = decltype(vv);
      const V* v = static_cast<const V*>(vals); V* o = static_cast<V*>(out);
      V i0 = V(); if (exclusive) std::memcpy(&i0, init, sizeof(V));
      auto run = [&](auto f) {
        if (exclusive) thrust::exclusive_scan_by_key(thrust::device, k, k + n, v, o, i0, thrust::equal_to<K>(), f);
        else thrust::inclusive_scan_by_key(thrust::device, k, k + n, v, o, thrust::equal_to<K>(), f);
      };
      if (op == ORA_PLUS) run(thrust::plus<V>()); else if (op == ORA_MIN) run(min_op<V>()); else run(max_op<V>());
    });
  });
  return rc;
}

ORA_EXPORT int64_t ora_unique_by_key_copy(const void* keys, const void* vals, void* keys_out, void* vals_out, size_t n,
                                          int key_t, int val_bytes) {
  int64_t cnt = -1;
  by_dtype(key_t, [&](auto kv) {
    using K = decltype(kv);
    const K* k = static_cast<const K*>(keys); K* ko = static_cast<K*>(keys_out);
    by_bytes(val_bytes, [&](auto vv) {
      using V = decltype(vv);
      const V* v = static_cast<const V*>(vals); V* vo = static_cast<V*>(vals_out);
      cnt = thrust::unique_by_key_copy(thrust::device, k, k + n, v, ko, vo).first - ko;
    });
  });
  return cnt;
}

ORA_EXPORT int ora_minmax_element(const void* in, size_t n, int t, uint64_t* idx) {
  return by_dtype(t, [&](auto tv) {
    using T = decltype(tv);
    const T* p = static_cast<const T*>(in);
    // the three entry points are called separately: they must agree
    auto both = thrust::minmax_element(thrust::device, p, p + n);
    const T* lo = thrust::min_element(thrust::device, p, p + n);
    const T* hi = thrust::max_element(thrust::device, p, p + n);
    idx[0] = (uint64_t)(lo - p);
    idx[1] = (uint64_t)(hi - p);
    if (both.first != lo || both.second != hi) { idx[0] = ~(uint64_t)0; idx[1] = ~(uint64_t)0; }
  });
}

ORA_EXPORT int ora_merge_by_key(const void* ka, const void* va, size_t na, const void* kb,
                                const void* vb, size_t nb, void* ko, void* vo, int key_t,
                                int val_bytes, int descending) {
  return by_dtype(key_t, [&](auto kv) {
    using K = decltype(kv);
    const K* a = static_cast<const K*>(ka); const K* b = static_cast<const K*>(kb);
    K* o = static_cast<K*>(ko);
    if (val_bytes == 0) {
      if (descending) thrust::merge(thrust::device, a, a + na, b, b + nb, o, thrust::greater<K>());
      else thrust::merge(thrust::device, a, a + na, b, b + nb, o, thrust::less<K>());
      return;
    }
    by_bytes(val_bytes, [&](auto vv) {
      using V = decltype(vv);
      const V* pa = static_cast<const V*>(va); const V* pb = static_cast<const V*>(vb);
      V* po = static_cast<V*>(vo);
      if (descending)
        thrust::merge_by_key(thrust::device, a, a + na, b, b + nb, pa, pb, o, po,
                             thrust::greater<K>());
      else
        thrust::merge_by_key(thrust::device, a, a + na, b, b + nb, pa, pb, o, po,
                             thrust::less<K>());
    });
  });
}
