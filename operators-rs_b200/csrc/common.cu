// common.cu — error state, dtype table and device probing shared by every operator.
#include "common.h"

namespace ops {

static thread_local char g_err[512];
static thread_local usz g_ws_need = 0;

char *error_buf() { return g_err; }
usz &workspace_need() { return g_ws_need; }

int fail(int kind, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return kind;
}

int need_workspace(usz bytes) {
  g_ws_need = bytes;
  snprintf(g_err, sizeof(g_err), "workspace too small: %zu bytes needed", bytes);
  return OPS_WORKSPACE_TOO_SMALL;
}

int init_base(OpBase *b, int device) {
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0) {
    cudaGetLastError();
    return fail(OPS_EXECUTION_FAILED, "no CUDA device: this library has no CPU path (%s)",
                e == cudaSuccess ? "device count 0" : cudaGetErrorString(e));
  }
  if (device < 0 || device >= count) return fail(OPS_ARGS_NOT_SUPPORT, "device %d out of range (count %d)", device, count);
  cudaDeviceProp prop;
  e = cudaGetDeviceProperties(&prop, device);
  if (e != cudaSuccess) return fail(OPS_EXECUTION_FAILED, "cudaGetDeviceProperties: %s", cudaGetErrorString(e));
  if (prop.major != 10) return fail(OPS_EXECUTION_FAILED, "device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);
  b->device = device;
  b->sm_count = prop.multiProcessorCount;
  return OPS_OK;
}

}  // namespace ops

OPS_API const char *ops_last_error(void) { return ops::error_buf(); }
OPS_API size_t ops_last_workspace_need(void) { return ops::workspace_need(); }

OPS_API size_t ops_dtype_nbytes(uint32_t dt) {
  switch (dt) {
    case OPS_DT_U8: case OPS_DT_I8: return 1;
    case OPS_DT_F16: case OPS_DT_BF16: case OPS_DT_U16: case OPS_DT_I16: return 2;
    case OPS_DT_F32: case OPS_DT_U32: case OPS_DT_I32: return 4;
    case OPS_DT_F64: case OPS_DT_U64: case OPS_DT_I64: case OPS_DT_KVPAIR: return 8;
    default: return 0;
  }
}

OPS_API int ops_device_count(void) {
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return count;
}

OPS_API const char *ops_build_info(void) { return "ops_b200: sm_100a, CUDA " __DATE__; }
