// Helpers shared by the C-ABI translation units: dtype dispatch and workspace checks.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "thrust_b200.h"
#include "thrust_b200/common.cuh"

#define TB200_API extern "C" __attribute__((visibility("default")))

namespace tb200_abi {

constexpr int ERR_INVALID = 1;         // cudaErrorInvalidValue
constexpr int ERR_UNSUPPORTED = 801;   // cudaErrorNotSupported

inline size_t dtype_size(int t) {
  switch (t) {
    case TB200_I8: case TB200_U8: return 1;
    case TB200_I16: case TB200_U16: return 2;
    case TB200_I32: case TB200_U32: case TB200_F32: return 4;
    case TB200_I64: case TB200_U64: case TB200_F64: return 8;
  }
  return 0;
}

// Size query / size check shared by every entry point.  Returns true when the caller only asked
// for the size (or passed too little) and `rc` holds the value to return.
inline bool workspace_gate(void* d_ws, size_t* ws_bytes, size_t need, int& rc) {
  if (!ws_bytes) { rc = ERR_INVALID; return true; }
  if (!d_ws) { *ws_bytes = need; rc = 0; return true; }
  if (*ws_bytes < need) { rc = ERR_INVALID; return true; }
  return false;
}

template <class F> int by_wide_dtype(int t, F f) {
  switch (t) {
    case TB200_I32: return f((int32_t)0);
    case TB200_U32: return f((uint32_t)0);
    case TB200_I64: return f((long long)0);
    case TB200_U64: return f((unsigned long long)0);
    case TB200_F32: return f((float)0);
    case TB200_F64: return f((double)0);
  }
  return ERR_UNSUPPORTED;
}

template <class F> int by_dtype(int t, F f) {
  switch (t) {
    case TB200_I8: return f((int8_t)0);
    case TB200_U8: return f((uint8_t)0);
    case TB200_I16: return f((int16_t)0);
    case TB200_U16: return f((uint16_t)0);
    default: return by_wide_dtype(t, f);
  }
}

template <class F> int by_op(int op, F f) {
  switch (op) {
    case TB200_PLUS: return f(tb200::plus_op());
    case TB200_MIN: return f(tb200::min_op());
    case TB200_MAX: return f(tb200::max_op());
  }
  return ERR_UNSUPPORTED;
}

}  // namespace tb200_abi
