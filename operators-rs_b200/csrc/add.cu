// add.cu — the two small elementwise operators on either side of the decoder layer:
//   add       c = a + b over N-d strided tensors       (residual connections written as an operator)
//   add_rows  dst[b, m, :] += src[idx[b, m], :]        (embedding / position rows added to the stream)
//
// Replace add::common_cpu::Operator (operators/src/add/common_cpu/mod.rs:29-75, planning add/args.rs:42-167) and
// add_rows::common_cpu::Operator (operators/src/add_rows/common_cpu/mod.rs:35-148, checks add_rows/args.rs:46-81).
// Both HBM-bound (3 resp. 3 element streams); rows with a contiguous last dim move as 128-bit vectors.
#include <algorithm>
#include <type_traits>
#include <vector>

#include "common.h"
#include "device_utils.cuh"

namespace ops {

constexpr int ADD_MAX_DIMS = 6;

struct AddParams {
  char *c;
  const char *a, *b;
  int ndim;                 // outer dims (the innermost, vectorised dim is separate)
  unsigned int len[ADD_MAX_DIMS];
  long long sc[ADD_MAX_DIMS], sa[ADD_MAX_DIMS], sb[ADD_MAX_DIMS];
  unsigned int inner;       // elements (generic) or 8-element vectors (vector kernel) of the innermost dim
  long long ic, ia, ib;     // byte strides of the innermost dim (generic kernel)
  unsigned long long total; // outer count * inner
};

__device__ __forceinline__ void add_locate(const AddParams &p, unsigned long long i, long long &oc, long long &oa, long long &ob, unsigned int &in) {
  unsigned long long outer = i / p.inner;
  in = (unsigned int)(i - outer * p.inner);
  oc = oa = ob = 0;
  for (int d = p.ndim - 1; d >= 0; --d) {
    const unsigned long long q = outer / p.len[d];
    const unsigned int k = (unsigned int)(outer - q * p.len[d]);
    outer = q;
    oc += (long long)k * p.sc[d];
    oa += (long long)k * p.sa[d];
    ob += (long long)k * p.sb[d];
  }
}

template <class E>
__global__ void __launch_bounds__(256) add_vec_kernel(const __grid_constant__ AddParams p) {
  const unsigned long long i = blockIdx.x * 256ull + threadIdx.x;
  if (i >= p.total) return;
  long long oc, oa, ob;
  unsigned int in;
  add_locate(p, i, oc, oa, ob, in);
  Vec8<E> x, y, z;
  x.u = ld_global_16(p.a + oa + 16ll * in);
  y.u = ld_global_16(p.b + ob + 16ll * in);
#pragma unroll
  for (int e = 0; e < 8; ++e) z.h[e] = from_f32<E>(__fadd_rn(to_f32(x.h[e]), to_f32(y.h[e])));
  st_global_16(p.c + oc + 16ll * in, z.u);
}

template <class T>
__global__ void __launch_bounds__(256) add_generic_kernel(const __grid_constant__ AddParams p) {
  const unsigned long long i = blockIdx.x * 256ull + threadIdx.x;
  if (i >= p.total) return;
  long long oc, oa, ob;
  unsigned int in;
  add_locate(p, i, oc, oa, ob, in);
  const T x = *reinterpret_cast<const T *>(p.a + oa + p.ia * in), y = *reinterpret_cast<const T *>(p.b + ob + p.ib * in);
  *reinterpret_cast<T *>(p.c + oc + p.ic * in) = from_f32<T>(__fadd_rn(to_f32(x), to_f32(y)));
}

template <class T, class I>
__global__ void __launch_bounds__(256) add_rows_kernel(T *dst, long long bsd, long long msd, long long nsd, const T *src, long long kss, long long nss,
                                                       const I *idx, long long bsi, long long msi, unsigned int m, unsigned int n, unsigned long long k,
                                                       int vec, int *status) {
  const unsigned int row = blockIdx.x;
  const unsigned int bi = row / m, mi = row - bi * m;
  const unsigned long long id = (unsigned long long)*byte_off(idx, bi * bsi + mi * msi);
  if (id >= k) {  // the CPU operator asserts here; record it and leave the row untouched
    if (threadIdx.x == 0) atomicCAS(status, 0, 1);
    return;
  }
  T *d = byte_off(dst, bi * bsd + mi * msd);
  const T *s = byte_off(src, (long long)id * kss);
  if (vec) {
    for (unsigned int v = blockIdx.y * 256u + threadIdx.x; v < n / 8; v += gridDim.y * 256u) {
      typedef typename std::conditional<sizeof(T) == 2, T, __half>::type E;  // the vector path is only taken by 16-bit types
      Vec8<E> x, y;
      x.u = ld_global_16(reinterpret_cast<const E *>(d) + v * 8);
      y.u = ld_global_16(reinterpret_cast<const E *>(s) + v * 8);
#pragma unroll
      for (int e = 0; e < 8; ++e) x.h[e] = from_f32<E>(__fadd_rn(to_f32(x.h[e]), to_f32(y.h[e])));
      st_global_16(reinterpret_cast<E *>(d) + v * 8, x.u);
    }
  } else {
    for (unsigned int j = blockIdx.y * 256u + threadIdx.x; j < n; j += gridDim.y * 256u) {
      T *dp = byte_off(d, (long long)j * nsd);
      *dp = from_f32<T>(__fadd_rn(to_f32(*dp), to_f32(*byte_off(s, (long long)j * nss))));
    }
  }
}

}  // namespace ops

using namespace ops;

OPS_DEFINE_SIMPLE_HANDLE(add)

static int add_check(const ops_add_args *a) {
  if (a->c_layout.dt != a->a_layout.dt || a->c_layout.dt != a->b_layout.dt) return fail(OPS_TYPE_MISMATCH, "c, a, b element types differ");
  if (a->a_layout.ndim != a->c_layout.ndim || a->b_layout.ndim != a->c_layout.ndim)
    return fail(OPS_RANK_MISMATCH, "c.ndim = %u, a.ndim = %u, b.ndim = %u", a->c_layout.ndim, a->a_layout.ndim, a->b_layout.ndim);
  return OPS_OK;
}

OPS_API int ops_add_scheme(ops_add *op, const ops_add_args *args, size_t max_ws, size_t *ws_out) {
  (void)op;
  (void)max_ws;
  if (ws_out) *ws_out = 0;
  return add_check(args);
}

OPS_API int ops_add_launch(const ops_add *op, const ops_add_args *a, void *ws, size_t ws_len, void *stream) {
  (void)ws;
  (void)ws_len;
  OPS_TRY(add_check(a));
  const uint32_t dt = a->c_layout.dt;
  if (dt != OPS_DT_F16 && dt != OPS_DT_BF16 && dt != OPS_DT_F32) return fail(OPS_TYPE_NOT_SUPPORT, "add: f16, bf16 or f32 expected");
  const isz es = (isz)dt_size(dt);
  struct Dim {
    usz d;
    isz c, a, b;
  };
  std::vector<Dim> dims;
  for (uint32_t i = 0; i < a->c_layout.ndim; ++i) {
    const usz d = a->c_layout.shape[i], da = a->a_layout.shape[i], db = a->b_layout.shape[i];
    const isz sc = a->c_layout.strides[i], sa = a->a_layout.strides[i], sb = a->b_layout.strides[i];
    if (dyn(d) || dyn(da) || dyn(db) || dyn(sc) || dyn(sa) || dyn(sb)) return fail(OPS_DYNAMIC_NOT_SUPPORT, "add: dynamic shape or stride at launch");
    if (da != d || db != d) return fail(OPS_SHAPE_MISMATCH, "add: shapes of c, a, b differ in dim %u", i);
    if (d == 0) return OPS_OK;
    if (d != 1) {
      if (sc == 0) return fail(OPS_SHAPE_NOT_SUPPORT, "Reducing is not allowed for add");
      dims.push_back(Dim{d, sc, sa, sb});
    }
  }
  if (!a->c_base || !a->a_base || !a->b_base) return fail(OPS_DYNAMIC_NOT_SUPPORT, "add: null base pointer at launch");
  // merge neighbouring dims that continue each other in all three tensors (the layout stays in the caller's order)
  for (size_t i = dims.size(); i-- > 1;) {
    Dim &f = dims[i - 1], &b = dims[i];
    if (b.c * (isz)b.d == f.c && b.a * (isz)b.d == f.a && b.b * (isz)b.d == f.b) {
      f = Dim{f.d * b.d, b.c, b.a, b.b};
      dims.erase(dims.begin() + i);
    }
  }
  if (dims.empty()) dims.push_back(Dim{1, es, es, es});
  if (dims.size() > (size_t)ADD_MAX_DIMS + 1) return fail(OPS_RANK_NOT_SUPPORT, "add: more than %d merged dims", ADD_MAX_DIMS + 1);
  AddParams p;
  p.c = (char *)a->c_base;
  p.a = (const char *)a->a_base;
  p.b = (const char *)a->b_base;
  const Dim in = dims.back();
  dims.pop_back();
  p.ndim = (int)dims.size();
  unsigned long long outer = 1;
  bool vec = (dt == OPS_DT_F16 || dt == OPS_DT_BF16) && in.c == es && in.a == es && in.b == es && in.d % 8 == 0 && aligned(p.c, 16) && aligned(p.a, 16) && aligned(p.b, 16);
  for (int i = 0; i < p.ndim; ++i) {
    if (dims[i].d > 0xffffffffu) return fail(OPS_SHAPE_NOT_SUPPORT, "add: dim too long");
    p.len[i] = (unsigned int)dims[i].d;
    p.sc[i] = dims[i].c;
    p.sa[i] = dims[i].a;
    p.sb[i] = dims[i].b;
    outer *= dims[i].d;
    vec = vec && dims[i].c % 16 == 0 && dims[i].a % 16 == 0 && dims[i].b % 16 == 0;
  }
  if (in.d > 0xffffffffu) return fail(OPS_SHAPE_NOT_SUPPORT, "add: dim too long");
  p.inner = (unsigned int)(vec ? in.d / 8 : in.d);
  p.ic = in.c;
  p.ia = in.a;
  p.ib = in.b;
  p.total = outer * p.inner;
  const unsigned long long blocks = (p.total + 255) / 256;
  if (blocks > 0x7fffffffull) return fail(OPS_SHAPE_NOT_SUPPORT, "add: tensor too large");
  cudaStream_t s = (cudaStream_t)stream;
  cudaSetDevice(op->base.device);
  if (vec && dt == OPS_DT_F16) add_vec_kernel<__half><<<(unsigned)blocks, 256, 0, s>>>(p);
  else if (vec) add_vec_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, s>>>(p);
  else if (dt == OPS_DT_F16) add_generic_kernel<__half><<<(unsigned)blocks, 256, 0, s>>>(p);
  else if (dt == OPS_DT_BF16) add_generic_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, s>>>(p);
  else add_generic_kernel<float><<<(unsigned)blocks, 256, 0, s>>>(p);
  return check_launch("add");
}

// ------------------------------------------------------------------------------------------------ add_rows
struct ops_add_rows {
  ops::OpBase base;
  int *status_dev;
};

struct AddRowsMeta {
  uint32_t dt, dt_idx;
  usz batch, m, n, k;
};

static int add_rows_meta(const ops_add_rows_args *a, AddRowsMeta *mt) {
  if (a->dst_layout.dt != a->src_layout.dt) return fail(OPS_TYPE_MISMATCH, "dst and src element types differ");
  mt->dt = a->dst_layout.dt;
  mt->dt_idx = a->idx_layout.dt;
  if (!is_unsigned_dt(mt->dt_idx)) return fail(OPS_TYPE_NOT_SUPPORT, "data type of idx is not supported, must be unsigned integers");
  if (a->dst_layout.ndim != 3) return fail(OPS_RANK_NOT_SUPPORT, "dst.ndim = %u, 3 expected", a->dst_layout.ndim);
  if (a->src_layout.ndim != 2) return fail(OPS_RANK_NOT_SUPPORT, "src.ndim = %u, 2 expected", a->src_layout.ndim);
  if (a->idx_layout.ndim != 2) return fail(OPS_RANK_NOT_SUPPORT, "idx.ndim = %u, 2 expected", a->idx_layout.ndim);
  const usz bs[2] = {a->dst_layout.shape[0], a->idx_layout.shape[0]}, ms[2] = {a->dst_layout.shape[1], a->idx_layout.shape[1]};
  const usz ns[2] = {a->dst_layout.shape[2], a->src_layout.shape[1]};
  if (!merge_dims(bs, 2, &mt->batch)) return fail(OPS_SHAPE_MISMATCH, "batch of dst and idx differ");
  if (!merge_dims(ms, 2, &mt->m)) return fail(OPS_SHAPE_MISMATCH, "m of dst and idx differ");
  if (!merge_dims(ns, 2, &mt->n)) return fail(OPS_SHAPE_MISMATCH, "n of dst and src differ");
  mt->k = a->src_layout.shape[0];
  return OPS_OK;
}

OPS_API int ops_add_rows_create(int device, ops_add_rows **out) {
  if (!out) return fail(OPS_ARGS_NOT_SUPPORT, "null out pointer");
  ops_add_rows *h = new ops_add_rows();
  h->status_dev = nullptr;
  int rc = init_base(&h->base, device);
  if (rc == OPS_OK) {
    cudaSetDevice(device);
    if (cudaMalloc(&h->status_dev, sizeof(int)) != cudaSuccess || cudaMemset(h->status_dev, 0, sizeof(int)) != cudaSuccess)
      rc = fail(OPS_EXECUTION_FAILED, "add_rows: cannot allocate the status word");
  }
  if (rc != OPS_OK) {
    delete h;
    return rc;
  }
  *out = h;
  return OPS_OK;
}

OPS_API void ops_add_rows_destroy(ops_add_rows *op) {
  if (!op) return;
  if (op->status_dev) cudaFree(op->status_dev);
  delete op;
}

OPS_API int ops_add_rows_status(const ops_add_rows *op) {
  int v = -1;
  cudaSetDevice(op->base.device);
  if (cudaMemcpy(&v, op->status_dev, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  return v;
}

OPS_API int ops_add_rows_scheme(ops_add_rows *op, const ops_add_rows_args *args, size_t max_ws, size_t *ws_out) {
  (void)op;
  (void)max_ws;
  AddRowsMeta mt;
  OPS_TRY(add_rows_meta(args, &mt));
  if (ws_out) *ws_out = 0;
  return OPS_OK;
}

OPS_API int ops_add_rows_launch(const ops_add_rows *op, const ops_add_rows_args *a, void *ws, size_t ws_len, void *stream) {
  (void)ws;
  (void)ws_len;
  AddRowsMeta mt;
  OPS_TRY(add_rows_meta(a, &mt));
  const isz *sd = a->dst_layout.strides, *ss = a->src_layout.strides, *si = a->idx_layout.strides;
  if (dyn(mt.batch) || dyn(mt.m) || dyn(mt.n) || dyn(mt.k) || dyn(sd[0]) || dyn(sd[1]) || dyn(sd[2]) || dyn(ss[0]) || dyn(ss[1]) || dyn(si[0]) || dyn(si[1]))
    return fail(OPS_DYNAMIC_NOT_SUPPORT, "add_rows: every shape and stride must be static at launch");
  if (mt.dt != OPS_DT_F16 && mt.dt != OPS_DT_BF16 && mt.dt != OPS_DT_F32) return fail(OPS_TYPE_NOT_SUPPORT, "add_rows: f16, bf16 or f32 expected");
  if (mt.dt_idx != OPS_DT_U32 && mt.dt_idx != OPS_DT_U64) return fail(OPS_TYPE_NOT_SUPPORT, "add_rows: idx must be u32 or u64");
  if (mt.batch == 0 || mt.m == 0 || mt.n == 0) return OPS_OK;
  if (mt.batch * mt.m > 0x7fffffffu || mt.n > 0xffffffffu) return fail(OPS_SHAPE_NOT_SUPPORT, "add_rows: shape too large");
  if (!a->dst_base || !a->src_base || !a->idx_base) return fail(OPS_DYNAMIC_NOT_SUPPORT, "add_rows: null base pointer at launch");
  cudaStream_t s = (cudaStream_t)stream;
  cudaSetDevice(op->base.device);
  const int vec = (mt.dt == OPS_DT_F16 || mt.dt == OPS_DT_BF16) && sd[2] == 2 && ss[1] == 2 && mt.n % 8 == 0 && sd[0] % 16 == 0 && sd[1] % 16 == 0 && ss[0] % 16 == 0 &&
                  aligned(a->dst_base, 16) && aligned(a->src_base, 16);
  const unsigned per_row = (unsigned)std::min<usz>(8, ((vec ? mt.n / 8 : mt.n) + 255) / 256);
  dim3 grid((unsigned)(mt.batch * mt.m), per_row);
#define ADD_ROWS(T, I)                                                                                                                        \
  add_rows_kernel<T, I><<<grid, 256, 0, s>>>((T *)a->dst_base, sd[0], sd[1], sd[2], (const T *)a->src_base, ss[0], ss[1], (const I *)a->idx_base, si[0], \
                                              si[1], (unsigned)mt.m, (unsigned)mt.n, (unsigned long long)mt.k, vec, op->status_dev)
  if (mt.dt == OPS_DT_F16 && mt.dt_idx == OPS_DT_U32) ADD_ROWS(__half, uint32_t);
  else if (mt.dt == OPS_DT_F16) ADD_ROWS(__half, unsigned long long);
  else if (mt.dt == OPS_DT_BF16 && mt.dt_idx == OPS_DT_U32) ADD_ROWS(__nv_bfloat16, uint32_t);
  else if (mt.dt == OPS_DT_BF16) ADD_ROWS(__nv_bfloat16, unsigned long long);
  else if (mt.dt_idx == OPS_DT_U32) ADD_ROWS(float, uint32_t);
  else ADD_ROWS(float, unsigned long long);
#undef ADD_ROWS
  return check_launch("add_rows");
}
