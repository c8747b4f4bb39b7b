// common.h — shared host-side helpers of the library: error reporting, layout access, launch checks.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdarg>
#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <cstring>

#include "../../include/ops_b200.h"

#define OPS_API extern "C" __attribute__((visibility("default")))

typedef ptrdiff_t isz;
typedef size_t usz;

namespace ops {

// Calling thread's last error message / workspace need (ops_last_error, ops_last_workspace_need).
char *error_buf();
usz &workspace_need();
int fail(int kind, const char *fmt, ...) __attribute__((format(printf, 2, 3)));
int need_workspace(usz bytes);

inline usz dt_size(uint32_t dt) { return ops_dtype_nbytes(dt); }
inline bool is_float_dt(uint32_t dt) { return dt == OPS_DT_F16 || dt == OPS_DT_BF16 || dt == OPS_DT_F32 || dt == OPS_DT_F64; }
inline bool is_unsigned_dt(uint32_t dt) { return dt == OPS_DT_U8 || dt == OPS_DT_U16 || dt == OPS_DT_U32 || dt == OPS_DT_U64; }

inline bool dyn(usz v) { return v == OPS_DYN_SIZE; }
inline bool dyn(isz v) { return v == OPS_DYN_STRIDE; }
inline bool dyn(float v) { return std::isinf(v) && v > 0; }

// MaybeDyn::merge (operators/src/common/maybe_dyn.rs:80-94) through utils::dim_distinct
// (operators/src/common/mod.rs:56-61): equal-or-dynamic dims merge, anything else is ShapeMismatch.
inline bool merge_dims(const usz *vals, int n, usz *out) {
  usz acc = vals[0];
  for (int i = 1; i < n; ++i) {
    if (dyn(vals[i])) continue;
    if (dyn(acc)) acc = vals[i];
    else if (acc != vals[i]) return false;
  }
  *out = acc;
  return true;
}

// Every op handle starts with this.
struct OpBase {
  int device;
  int sm_count;
};
int init_base(OpBase *b, int device);

// Kernel launch epilogue: turns a launch-time CUDA error into ExecutionFailed.
inline int check_launch(const char *what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(OPS_EXECUTION_FAILED, "%s: %s", what, cudaGetErrorString(e));
  return OPS_OK;
}

inline bool aligned(const void *p, usz a) { return ((uintptr_t)p % a) == 0; }

}  // namespace ops

#define OPS_TRY(expr)            \
  do {                           \
    int _rc = (expr);            \
    if (_rc != OPS_OK) return _rc; \
  } while (0)

// Boilerplate shared by the operators whose handle holds nothing but the device.
#define OPS_DEFINE_SIMPLE_HANDLE(NAME)                                              \
  struct ops_##NAME {                                                               \
    ops::OpBase base;                                                               \
  };                                                                                \
  OPS_API int ops_##NAME##_create(int device, ops_##NAME **out) {                   \
    if (!out) return ops::fail(OPS_ARGS_NOT_SUPPORT, "null out pointer");           \
    ops_##NAME *h = new ops_##NAME();                                               \
    int rc = ops::init_base(&h->base, device);                                      \
    if (rc != OPS_OK) {                                                             \
      delete h;                                                                     \
      return rc;                                                                    \
    }                                                                               \
    *out = h;                                                                       \
    return OPS_OK;                                                                  \
  }                                                                                 \
  OPS_API void ops_##NAME##_destroy(ops_##NAME *op) { delete op; }
