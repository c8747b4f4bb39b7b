// swiglu.cu — gate <- gate * sigmoid(gate) * up, in place.
//
// Replaces swiglu::common_cpu::Operator (operators/src/swiglu/common_cpu/mod.rs:27-81, arithmetic
// :109-137); argument checks follow Args::meta (operators/src/swiglu/args.rs:27-50).
//
// HBM-bound: 3*n*d*2 bytes.  Each thread handles 8 halves per 128-bit access (one gate and one up load in
// flight); one CTA per (row, 2048-column chunk), so no index division and enough CTAs to cover HBM latency.
#include "common.h"
#include "device_utils.cuh"

namespace ops {

__device__ __forceinline__ float swiglu_f32(float a, float b) {
  // a * (1 / (1 + exp(-a))) * b.  The exponential and the reciprocal come from the special-function unit (ex2 / rcp
  // approximations, relative error ~2^-22): with libm-grade expf and an IEEE division the kernel is bound by instruction
  // issue, not by HBM, and the difference is far below the 16-bit rounding of the result.
  const float e = __expf(-a);
  const float sig = __fdividef(1.f, 1.f + e);
  return __fmul_rn(__fmul_rn(a, sig), b);
}

// Fast path: f16, unit inner strides, d % 8 == 0, 16-byte aligned rows.  blockIdx.x = row, blockIdx.y = 2048-column
// chunk (blockIdx.x = row * chunks + chunk): no per-element index division, one 128-bit gate load and one up load in flight per thread, thousands of CTAs.
template <class E>
__global__ void __launch_bounds__(256) swiglu_vec_kernel(E *__restrict__ gate, long long sgn, const E *__restrict__ up,
                                                         long long sun, int vec_per_row, int chunks) {
  const unsigned row = blockIdx.x / (unsigned)chunks, chunk = blockIdx.x - row * (unsigned)chunks;  // one division per CTA
  const int v = (int)chunk * (int)blockDim.x + (int)threadIdx.x;
  if (v >= vec_per_row) return;
  E *g = byte_off(gate, (long long)row * sgn) + v * 8;
  const E *u = byte_off(up, (long long)row * sun) + v * 8;
  Vec8<E> gv, uv, out;
  gv.u = ld_global_16(g);
  uv.u = ld_stream_16(u);
#pragma unroll
  for (int e = 0; e < 8; ++e) out.h[e] = from_f32<E>(swiglu_f32(to_f32(gv.h[e]), to_f32(uv.h[e])));
  st_global_16(g, out.u);
}

template <class T>
__global__ void __launch_bounds__(256) swiglu_generic_kernel(T *gate, long long sgn, long long sgd, const T *up, long long sun,
                                                             long long sud, long long d, long long total) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / d, col = i - row * d;
    T *g = byte_off(gate, row * sgn + col * sgd);
    const T *u = byte_off(up, row * sun + col * sud);
    *g = from_f32<T>(swiglu_f32(to_f32(*g), to_f32(*u)));
  }
}

struct SwigluMeta {
  uint32_t dt;
  usz n, d;
};

static int swiglu_meta(const ops_swiglu_args *a, SwigluMeta *m) {
  if (a->gate_layout.ndim != 2) return fail(OPS_RANK_NOT_SUPPORT, "gate.ndim = %u, 2 expected", a->gate_layout.ndim);
  if (a->up_layout.ndim != 2) return fail(OPS_RANK_NOT_SUPPORT, "up.ndim = %u, 2 expected", a->up_layout.ndim);
  if (a->gate_layout.dt != a->up_layout.dt) return fail(OPS_TYPE_MISMATCH, "gate and up element types differ");
  m->dt = a->gate_layout.dt;
  const usz ns[2] = {a->gate_layout.shape[0], a->up_layout.shape[0]};
  const usz ds[2] = {a->gate_layout.shape[1], a->up_layout.shape[1]};
  if (!merge_dims(ns, 2, &m->n)) return fail(OPS_SHAPE_MISMATCH, "n of gate and up differ");
  if (!merge_dims(ds, 2, &m->d)) return fail(OPS_SHAPE_MISMATCH, "d of gate and up differ");
  return OPS_OK;
}

}  // namespace ops

using namespace ops;

OPS_DEFINE_SIMPLE_HANDLE(swiglu)

OPS_API int ops_swiglu_scheme(ops_swiglu *op, const ops_swiglu_args *args, size_t max_ws, size_t *ws_out) {
  (void)op;
  (void)max_ws;
  SwigluMeta m;
  OPS_TRY(swiglu_meta(args, &m));
  if (ws_out) *ws_out = 0;
  return OPS_OK;
}

OPS_API int ops_swiglu_launch(const ops_swiglu *op, const ops_swiglu_args *a, void *ws, size_t ws_len, void *stream) {
  (void)ws;
  (void)ws_len;
  SwigluMeta m;
  OPS_TRY(swiglu_meta(a, &m));
  const isz sgn = a->gate_layout.strides[0], sgd = a->gate_layout.strides[1];
  const isz sun = a->up_layout.strides[0], sud = a->up_layout.strides[1];
  if (dyn(m.n) || dyn(m.d) || dyn(sgn) || dyn(sgd) || dyn(sun) || dyn(sud))
    return fail(OPS_DYNAMIC_NOT_SUPPORT, "swiglu: every shape and stride must be static at launch");
  if (m.dt != OPS_DT_F16 && m.dt != OPS_DT_BF16 && m.dt != OPS_DT_F32) return fail(OPS_TYPE_NOT_SUPPORT, "swiglu: f16, bf16 or f32 expected");
  if (m.n == 0 || m.d == 0) return OPS_OK;
  if (!a->gate_base || !a->up_base) return fail(OPS_DYNAMIC_NOT_SUPPORT, "swiglu: null base pointer at launch");
  cudaStream_t s = (cudaStream_t)stream;
  cudaSetDevice(op->base.device);
  const int max_blocks = op->base.sm_count * 8;

  const bool fast = (m.dt == OPS_DT_F16 || m.dt == OPS_DT_BF16) && sgd == 2 && sud == 2 && m.d % 8 == 0 && sgn % 16 == 0 && sun % 16 == 0 &&
                    aligned(a->gate_base, 16) && aligned(a->up_base, 16) && m.n * ((m.d / 8 + 255) / 256) <= 0x7fffffffu;
  if (fast) {
    const int vpr = (int)(m.d / 8);
    const int chunks = (vpr + 255) / 256;
    if (m.dt == OPS_DT_F16)
      swiglu_vec_kernel<__half><<<(unsigned)(m.n * (usz)chunks), 256, 0, s>>>((__half *)a->gate_base, sgn, (const __half *)a->up_base, sun, vpr, chunks);
    else
      swiglu_vec_kernel<__nv_bfloat16><<<(unsigned)(m.n * (usz)chunks), 256, 0, s>>>((__nv_bfloat16 *)a->gate_base, sgn, (const __nv_bfloat16 *)a->up_base, sun, vpr, chunks);
  } else {
    const long long total = (long long)m.n * (long long)m.d;
    const long long blocks = (total + 255) / 256;
    const unsigned grid = (unsigned)(blocks < max_blocks ? blocks : max_blocks);
    if (m.dt == OPS_DT_F16)
      swiglu_generic_kernel<__half><<<grid, 256, 0, s>>>((__half *)a->gate_base, sgn, sgd, (const __half *)a->up_base, sun, sud, (long long)m.d, total);
    else if (m.dt == OPS_DT_BF16)
      swiglu_generic_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((__nv_bfloat16 *)a->gate_base, sgn, sgd, (const __nv_bfloat16 *)a->up_base, sun, sud, (long long)m.d, total);
    else
      swiglu_generic_kernel<float><<<grid, 256, 0, s>>>((float *)a->gate_base, sgn, sgd, (const float *)a->up_base, sun, sud, (long long)m.d, total);
  }
  return check_launch("swiglu");
}
