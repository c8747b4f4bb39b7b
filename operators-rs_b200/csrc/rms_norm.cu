// rms_norm.cu — y[i,:] = x[i,:] * w / sqrt(mean(x[i,:]^2) + eps)
//
// Replaces rms_norm::common_cpu::Operator (operators/src/rms_norm/common_cpu/mod.rs:28-93, arithmetic
// :128-137 and :195-208); argument checks follow Args::meta (operators/src/rms_norm/args.rs:25-49).
//
// HBM-bound: 2*n*d*2 bytes (+ w once).  One CTA per row; the row lives in registers between the
// sum-of-squares pass and the scaling pass, so x is read from HBM exactly once.  128-bit accesses,
// warp-shuffle + one shared-memory hop for the block reduction.
#include "common.h"
#include "device_utils.cuh"

namespace ops {

__device__ __forceinline__ float rms_scale(float sum, float d, float eps) {
  // (sum / d + eps).sqrt().recip(): three IEEE-rounded steps, no fast-math
  return __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(sum, d), eps)));
}

// Fast path: f16 activations, unit inner strides, 16-byte aligned rows, d % 8 == 0.
// Each thread owns VPT vectors of 8 halves: vector index v = threadIdx.x + i * blockDim.x.
// ADD: the residual form.  x <- x + r first (one rounding to the element type, as the crate's add operator rounds,
// operators/src/add/common_cpu/mod.rs:29-75), written back in place, and the norm is taken of that sum.
template <int VPT, class A, class W, bool ADD>
__global__ void __launch_bounds__(1024) rms_norm_rows_kernel(A *__restrict__ y, long long nsy, A *__restrict__ x,
                                                             long long nsx, const W *__restrict__ w, int d, float eps,
                                                             const A *__restrict__ r, long long nsr) {
  __shared__ float scratch[33];
  const int nvec = d >> 3;
  A *xr = byte_off(x, (long long)blockIdx.x * nsx);
  A *yr = byte_off(y, (long long)blockIdx.x * nsy);
  const A *rr = ADD ? byte_off(r, (long long)blockIdx.x * nsr) : nullptr;

  Vec8<A> xv[VPT];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
      xv[i].u = ld_global_16(xr + v * 8);
      if constexpr (ADD) {
        Vec8<A> rv;
        rv.u = ld_global_16(rr + v * 8);
#pragma unroll
        for (int e = 0; e < 8; ++e) xv[i].h[e] = from_f32<A>(__fadd_rn(to_f32(xv[i].h[e]), to_f32(rv.h[e])));
        st_global_16(xr + v * 8, xv[i].u);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float f = to_f32(xv[i].h[e]);
        sum = fmaf(f, f, sum);
      }
    }
  }
  sum = block_sum(sum, scratch);
  const float k = rms_scale(sum, (float)d, eps);

#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
      float wf[8];
      if constexpr (sizeof(W) == 2) {
        Vec8<W> wv;
        wv.u = __ldg(reinterpret_cast<const uint4 *>(w) + v);
#pragma unroll
        for (int e = 0; e < 8; ++e) wf[e] = to_f32(wv.h[e]);
      } else {
        const float4 a = __ldg(reinterpret_cast<const float4 *>(w) + 2 * v);
        const float4 b = __ldg(reinterpret_cast<const float4 *>(w) + 2 * v + 1);
        wf[0] = a.x; wf[1] = a.y; wf[2] = a.z; wf[3] = a.w;
        wf[4] = b.x; wf[5] = b.y; wf[6] = b.z; wf[7] = b.w;
      }
      Vec8<A> out;
#pragma unroll
      for (int e = 0; e < 8; ++e) out.h[e] = from_f32<A>(__fmul_rn(__fmul_rn(k, wf[e]), to_f32(xv[i].h[e])));
      st_global_16(yr + v * 8, out.u);
    }
  }
}

// Generic path: any strides, f16 or f32 activations, f16 or f32 weights.  Two passes over the row.
template <class A, class W>
__global__ void __launch_bounds__(256) rms_norm_generic_kernel(A *y, long long nsy, long long dsy, const A *x, long long nsx,
                                                               long long dsx, const W *w, long long dsw, long long d, float eps) {
  __shared__ float scratch[33];
  const A *xr = byte_off(x, (long long)blockIdx.x * nsx);
  A *yr = byte_off(y, (long long)blockIdx.x * nsy);
  float sum = 0.f;
  for (long long j = threadIdx.x; j < d; j += blockDim.x) {
    float f = to_f32(*byte_off(xr, j * dsx));
    sum = fmaf(f, f, sum);
  }
  sum = block_sum(sum, scratch);
  const float k = rms_scale(sum, (float)d, eps);
  for (long long j = threadIdx.x; j < d; j += blockDim.x) {
    float f = to_f32(*byte_off(xr, j * dsx));
    float wv = to_f32(*byte_off(w, j * dsw));
    *byte_off(yr, j * dsy) = from_f32<A>(__fmul_rn(__fmul_rn(k, wv), f));
  }
}

struct RmsMeta {
  uint32_t dt_a, dt_w;
  usz n, d;
};

static int rms_meta(const ops_rms_norm_args *a, RmsMeta *m) {
  if (a->y_layout.ndim != 2) return fail(OPS_RANK_NOT_SUPPORT, "y.ndim = %u, 2 expected", a->y_layout.ndim);
  if (a->x_layout.ndim != 2) return fail(OPS_RANK_NOT_SUPPORT, "x.ndim = %u, 2 expected", a->x_layout.ndim);
  if (a->w_layout.ndim != 1) return fail(OPS_RANK_NOT_SUPPORT, "w.ndim = %u, 1 expected", a->w_layout.ndim);
  if (a->y_layout.dt != a->x_layout.dt) return fail(OPS_TYPE_MISMATCH, "y and x element types differ");
  m->dt_a = a->x_layout.dt;
  m->dt_w = a->w_layout.dt;
  const usz ns[2] = {a->y_layout.shape[0], a->x_layout.shape[0]};
  const usz ds[3] = {a->y_layout.shape[1], a->x_layout.shape[1], a->w_layout.shape[0]};
  if (!merge_dims(ns, 2, &m->n)) return fail(OPS_SHAPE_MISMATCH, "n of y and x differ");
  if (!merge_dims(ds, 3, &m->d)) return fail(OPS_SHAPE_MISMATCH, "d of y, x and w differ");
  return OPS_OK;
}

template <class A, class W, bool ADD = false>
static void launch_rows(const ops_rms_norm_args *a, const RmsMeta &m, cudaStream_t s, const void *r_base = nullptr, long long nsr = 0) {
  const int nvec = (int)(m.d / 8);
  int vpt = 1;
  while (vpt < 4 && (nvec + vpt - 1) / vpt > 256) vpt *= 2;  // prefer <= 256 threads per row
  while ((nvec + vpt - 1) / vpt > 1024) vpt *= 2;            // vpt <= 4 guaranteed by the caller
  int threads = ((nvec + vpt - 1) / vpt + 31) / 32 * 32;
  A *y = (A *)a->y_base;
  A *x = (A *)a->x_base;
  const W *w = (const W *)a->w_base;
  const A *r = (const A *)r_base;
  const long long nsy = a->y_layout.strides[0], nsx = a->x_layout.strides[0];
  dim3 grid((unsigned)m.n);
  switch (vpt) {
    case 1: rms_norm_rows_kernel<1, A, W, ADD><<<grid, threads, 0, s>>>(y, nsy, x, nsx, w, (int)m.d, a->epsilon, r, nsr); break;
    case 2: rms_norm_rows_kernel<2, A, W, ADD><<<grid, threads, 0, s>>>(y, nsy, x, nsx, w, (int)m.d, a->epsilon, r, nsr); break;
    default: rms_norm_rows_kernel<4, A, W, ADD><<<grid, threads, 0, s>>>(y, nsy, x, nsx, w, (int)m.d, a->epsilon, r, nsr); break;
  }
}

template <class A, class W>
static void launch_generic(const ops_rms_norm_args *a, const RmsMeta &m, cudaStream_t s) {
  rms_norm_generic_kernel<A, W><<<(unsigned)m.n, 256, 0, s>>>(
      (A *)a->y_base, a->y_layout.strides[0], a->y_layout.strides[1], (const A *)a->x_base, a->x_layout.strides[0],
      a->x_layout.strides[1], (const W *)a->w_base, a->w_layout.strides[0], (long long)m.d, a->epsilon);
}

}  // namespace ops

using namespace ops;

OPS_DEFINE_SIMPLE_HANDLE(rms_norm)

OPS_API int ops_rms_norm_scheme(ops_rms_norm *op, const ops_rms_norm_args *args, size_t max_ws, size_t *ws_out) {
  (void)op;
  (void)max_ws;
  RmsMeta m;
  OPS_TRY(rms_meta(args, &m));
  if (ws_out) *ws_out = 0;
  return OPS_OK;
}

OPS_API int ops_rms_norm_launch(const ops_rms_norm *op, const ops_rms_norm_args *a, void *ws, size_t ws_len, void *stream) {
  (void)ws;
  (void)ws_len;
  RmsMeta m;
  OPS_TRY(rms_meta(a, &m));
  const isz nsy = a->y_layout.strides[0], dsy = a->y_layout.strides[1];
  const isz nsx = a->x_layout.strides[0], dsx = a->x_layout.strides[1];
  const isz dsw = a->w_layout.strides[0];
  if (dyn(m.n) || dyn(m.d) || dyn(nsy) || dyn(dsy) || dyn(nsx) || dyn(dsx) || dyn(dsw) || dyn(a->epsilon))
    return fail(OPS_DYNAMIC_NOT_SUPPORT, "rms_norm: every shape, stride and epsilon must be static at launch");
  const bool a16 = m.dt_a == OPS_DT_F16, abf = m.dt_a == OPS_DT_BF16, a32 = m.dt_a == OPS_DT_F32;
  const bool w16 = m.dt_w == OPS_DT_F16, wbf = m.dt_w == OPS_DT_BF16, w32 = m.dt_w == OPS_DT_F32;
  if (!((a16 && (w16 || w32)) || (abf && (wbf || w32)) || (a32 && w32)))
    return fail(OPS_TYPE_NOT_SUPPORT, "rms_norm: (w, a) must be (f16,f16), (f32,f16), (bf16,bf16), (f32,bf16) or (f32,f32)");
  if (m.n == 0 || m.d == 0) return OPS_OK;
  if (m.n > 0x7fffffffu) return fail(OPS_SHAPE_NOT_SUPPORT, "rms_norm: n too large");
  if (!a->y_base || !a->x_base || !a->w_base) return fail(OPS_DYNAMIC_NOT_SUPPORT, "rms_norm: null base pointer at launch");
  cudaStream_t s = (cudaStream_t)stream;
  cudaSetDevice(op->base.device);

  const bool fast = (a16 || abf) && dsx == 2 && dsy == 2 && dsw == (isz)dt_size(m.dt_w) && m.d % 8 == 0 && m.d <= 8 * 4 * 1024 &&
                    nsx % 16 == 0 && nsy % 16 == 0 && aligned(a->x_base, 16) && aligned(a->y_base, 16) && aligned(a->w_base, 16);
  if (fast) {
    if (a16 && w16) launch_rows<__half, __half>(a, m, s);
    else if (a16) launch_rows<__half, float>(a, m, s);
    else if (wbf) launch_rows<__nv_bfloat16, __nv_bfloat16>(a, m, s);
    else launch_rows<__nv_bfloat16, float>(a, m, s);
  } else if (a16 && w16) launch_generic<__half, __half>(a, m, s);
  else if (a16) launch_generic<__half, float>(a, m, s);
  else if (abf && wbf) launch_generic<__nv_bfloat16, __nv_bfloat16>(a, m, s);
  else if (abf) launch_generic<__nv_bfloat16, float>(a, m, s);
  else launch_generic<float, float>(a, m, s);
  return check_launch("rms_norm");
}

// rms_norm with the residual add in front of it folded in: x <- x + r (in place), y <- rms_norm(x).  No counterpart in the
// crate, which chains add and rms_norm as two operators; one pass over the row instead of two.  Takes the layouts the
// vectorised kernel takes (f16 or bf16 rows with unit inner stride, 16-byte aligned, d a multiple of 8 up to 32768) and
// answers OPS_ARGS_NOT_SUPPORT otherwise: chain ops_add_launch and ops_rms_norm_launch then.
OPS_API int ops_rms_norm_add_launch(const ops_rms_norm *op, const ops_rms_norm_add_args *aa, void *stream) {
  const ops_rms_norm_args *a = &aa->norm;
  RmsMeta m;
  OPS_TRY(rms_meta(a, &m));
  if (aa->r_layout.ndim != 2) return fail(OPS_RANK_NOT_SUPPORT, "r.ndim = %u, 2 expected", aa->r_layout.ndim);
  if (aa->r_layout.dt != m.dt_a) return fail(OPS_TYPE_MISMATCH, "r and x element types differ");
  const isz nsy = a->y_layout.strides[0], dsy = a->y_layout.strides[1];
  const isz nsx = a->x_layout.strides[0], dsx = a->x_layout.strides[1];
  const isz nsr = aa->r_layout.strides[0], dsr = aa->r_layout.strides[1];
  const isz dsw = a->w_layout.strides[0];
  if (dyn(m.n) || dyn(m.d) || dyn(nsy) || dyn(dsy) || dyn(nsx) || dyn(dsx) || dyn(nsr) || dyn(dsr) || dyn(dsw) || dyn(a->epsilon) ||
      dyn(aa->r_layout.shape[0]) || dyn(aa->r_layout.shape[1]))
    return fail(OPS_DYNAMIC_NOT_SUPPORT, "rms_norm_add: every shape, stride and epsilon must be static at launch");
  if (aa->r_layout.shape[0] != m.n || aa->r_layout.shape[1] != m.d) return fail(OPS_SHAPE_MISMATCH, "shape of r differs from x");
  const bool a16 = m.dt_a == OPS_DT_F16, abf = m.dt_a == OPS_DT_BF16;
  const bool w16 = m.dt_w == OPS_DT_F16, wbf = m.dt_w == OPS_DT_BF16, w32 = m.dt_w == OPS_DT_F32;
  if (!((a16 && (w16 || w32)) || (abf && (wbf || w32)))) return fail(OPS_TYPE_NOT_SUPPORT, "rms_norm_add: (w, a) must be (f16,f16), (f32,f16), (bf16,bf16) or (f32,bf16)");
  if (m.n == 0 || m.d == 0) return OPS_OK;
  if (m.n > 0x7fffffffu) return fail(OPS_SHAPE_NOT_SUPPORT, "rms_norm_add: n too large");
  if (!a->y_base || !a->x_base || !a->w_base || !aa->r_base) return fail(OPS_DYNAMIC_NOT_SUPPORT, "rms_norm_add: null base pointer at launch");
  const bool fast = dsx == 2 && dsy == 2 && dsr == 2 && dsw == (isz)dt_size(m.dt_w) && m.d % 8 == 0 && m.d <= 8 * 4 * 1024 && nsx % 16 == 0 &&
                    nsy % 16 == 0 && nsr % 16 == 0 && aligned(a->x_base, 16) && aligned(a->y_base, 16) && aligned(a->w_base, 16) && aligned(aa->r_base, 16);
  if (!fast) return fail(OPS_ARGS_NOT_SUPPORT, "rms_norm_add: needs contiguous, 16-byte aligned rows with d a multiple of 8 (<= 32768); chain add and rms_norm instead");
  cudaStream_t s = (cudaStream_t)stream;
  cudaSetDevice(op->base.device);
  if (a16 && w16) launch_rows<__half, __half, true>(a, m, s, aa->r_base, nsr);
  else if (a16) launch_rows<__half, float, true>(a, m, s, aa->r_base, nsr);
  else if (wbf) launch_rows<__nv_bfloat16, __nv_bfloat16, true>(a, m, s, aa->r_base, nsr);
  else launch_rows<__nv_bfloat16, float, true>(a, m, s, aa->r_base, nsr);
  return check_launch("rms_norm_add");
}
