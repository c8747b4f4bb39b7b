// rearrange.cu — byte-exact strided N-d copy.
//
// Replaces rearrange::common_cpu::Operator (operators/src/rearrange/common_cpu/mod.rs:26-59).  The
// host-side planning restates rearrange::Scheme::new (operators/src/rearrange/args.rs:34-153): drop
// length-1 dims, refuse a zero dst stride, order dims by |dst| desc, |src| desc, len asc, fold the
// trailing contiguous dims into one `unit` of bytes, merge adjacent dims that continue each other.
//
// HBM-bound: 2 * bytes moved.  A unit is cut into the widest accesses (16/8/4/2/1 bytes) that the
// unit length, both base addresses and every stride allow; each thread moves four such pieces per
// CTA trip (all loads issued before the stores); index arithmetic in 32 bits with shifts wherever the sizes allow.
#include <algorithm>
#include <vector>

#include "common.h"
#include "device_utils.cuh"

namespace ops {

constexpr int REARRANGE_MAX_DIMS = 8;

struct RearrangeParams {
  char *dst;
  const char *src;
  long long total_vec;      // count * vec_per_unit
  long long vec_per_unit;   // unit / VEC
  int vec_shift;            // log2(vec_per_unit) when that is a power of two, else -1
  int ndim;
  long long idx[REARRANGE_MAX_DIMS];  // units per step of dim i
  long long ds[REARRANGE_MAX_DIMS];
  long long ss[REARRANGE_MAX_DIMS];
};

template <int VEC> struct VecType;
template <> struct VecType<16> { typedef uint4 type; };
template <> struct VecType<8> { typedef uint2 type; };
template <> struct VecType<4> { typedef uint32_t type; };
template <> struct VecType<2> { typedef uint16_t type; };
template <> struct VecType<1> { typedef uint8_t type; };

// Vector index -> byte offsets in dst and src.  Idx = uint32_t whenever every count fits (the usual case: 32-bit
// division is an order of magnitude cheaper than 64-bit), long long otherwise.
template <class Idx>
__device__ __forceinline__ void locate(const RearrangeParams &p, Idx v, long long &d, long long &s, int vec) {
  Idx u, o;
  if (p.vec_shift >= 0) {  // pieces per unit is a power of two
    u = v >> p.vec_shift;
    o = v & (Idx)((1ll << p.vec_shift) - 1);
  } else {
    u = v / (Idx)p.vec_per_unit;
    o = v - u * (Idx)p.vec_per_unit;
  }
  d = (long long)o * vec;
  s = d;
  for (int i = 0; i < p.ndim; ++i) {
    const Idx k = u / (Idx)p.idx[i];
    u -= k * (Idx)p.idx[i];
    d += (long long)k * p.ds[i];
    s += (long long)k * p.ss[i];
  }
}

// One CTA moves 4 * blockDim.x consecutive pieces: all four loads of a thread are issued before its stores.
template <int VEC, class Idx>
__global__ void __launch_bounds__(256) rearrange_kernel(const __grid_constant__ RearrangeParams p) {
  typedef typename VecType<VEC>::type V;
  const long long base = (long long)blockIdx.x * (4 * 256) + threadIdx.x;
  long long d[4], s[4];
  V val[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long v = base + i * 256;
    if (v < p.total_vec) {
      locate<Idx>(p, (Idx)v, d[i], s[i], VEC);
      val[i] = *reinterpret_cast<const V *>(p.src + s[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
    if (base + i * 256 < p.total_vec) *reinterpret_cast<V *>(p.dst + d[i]) = val[i];
}

struct Dim {
  usz len;
  isz dst, src;
};
static inline isz iabs(isz v) { return v < 0 ? -v : v; }

// layout = [unit, idx_strides (ndim + 1 entries, first = count, last = 1), dst_strides, src_strides]
int rearrange_plan(const ops_rearrange_args *a, std::vector<isz> &layout) {
  const ops_layout &D = a->dst_layout, &S = a->src_layout;
  if (D.dt != S.dt) return fail(OPS_TYPE_MISMATCH, "dst and src element types differ");
  if (D.ndim != S.ndim) return fail(OPS_RANK_MISMATCH, "dst.ndim = %u, src.ndim = %u", D.ndim, S.ndim);
  const usz esize = dt_size(D.dt);
  if (esize == 0) return fail(OPS_TYPE_NOT_SUPPORT, "unknown element type %u", D.dt);
  std::vector<Dim> dims;
  dims.reserve(D.ndim);
  for (uint32_t i = 0; i < D.ndim; ++i) {
    if (dyn(D.shape[i]) || dyn(S.shape[i])) return fail(OPS_DYNAMIC_NOT_SUPPORT, "rearrange: dynamic shape");
    if (D.shape[i] != S.shape[i]) return fail(OPS_SHAPE_MISMATCH, "dst[%u] = %zu, src[%u] = %zu", i, D.shape[i], i, S.shape[i]);
    if (dyn(D.strides[i]) || dyn(S.strides[i])) return fail(OPS_DYNAMIC_NOT_SUPPORT, "rearrange: dynamic stride");
    Dim dim{D.shape[i], D.strides[i], S.strides[i]};
    if (dim.len != 1) {
      if (dim.dst == 0) return fail(OPS_SHAPE_NOT_SUPPORT, "Reducing is not allowed for rearrangement.");
      dims.push_back(dim);
    }
  }
  std::sort(dims.begin(), dims.end(), [](const Dim &x, const Dim &y) {
    if (iabs(x.dst) != iabs(y.dst)) return iabs(x.dst) > iabs(y.dst);
    if (iabs(x.src) != iabs(y.src)) return iabs(x.src) > iabs(y.src);
    return x.len < y.len;
  });
  isz unit = (isz)esize;
  usz ndim = dims.size();
  while (ndim > 0 && dims[ndim - 1].dst == unit && dims[ndim - 1].src == unit) {
    unit *= (isz)dims[ndim - 1].len;
    --ndim;
  }
  dims.resize(ndim);
  for (usz i = dims.size(); i-- > 1;) {
    Dim &front = dims[i - 1], &back = dims[i];
    const isz len = (isz)back.len;
    if (back.dst * len == front.dst && back.src * len == front.src) {
      front = Dim{back.len * front.len, back.dst, back.src};
      back = Dim{1, 0, 0};
      --ndim;
    }
  }
  layout.assign(2 + 3 * ndim, 0);
  layout[0] = unit;
  layout[ndim + 1] = 1;
  usz w = 0;
  for (const Dim &dm : dims) {
    if (dm.len == 1) continue;
    layout[1 + w] = (isz)dm.len;
    layout[2 + ndim + w] = dm.dst;
    layout[2 + 2 * ndim + w] = dm.src;
    ++w;
  }
  for (usz r = ndim; r >= 1; --r) layout[r] *= layout[r + 1];
  return OPS_OK;
}

static usz pow2_divisor(usz v, usz cap) {  // largest power of two <= cap dividing v (v == 0 -> cap)
  usz r = 1;
  while (r < cap && v % (r * 2) == 0) r *= 2;
  return r;
}

// Enqueue the copy described by `a` on `s`.  Shared with attention and the KV-cache operator.
int rearrange_enqueue(const OpBase &base, const ops_rearrange_args *a, cudaStream_t s) {
  std::vector<isz> L;
  OPS_TRY(rearrange_plan(a, L));
  const usz ndim = (L.size() - 2) / 3;
  const usz unit = (usz)L[0];
  const usz count = (usz)L[1];
  if (unit == 0 || count == 0) return OPS_OK;
  if (ndim > (usz)REARRANGE_MAX_DIMS) return fail(OPS_RANK_NOT_SUPPORT, "rearrange: more than %d merged dims", REARRANGE_MAX_DIMS);
  if (!a->dst_base || !a->src_base) return fail(OPS_DYNAMIC_NOT_SUPPORT, "rearrange: null base pointer at launch");

  usz vec = pow2_divisor(unit, 16);
  vec = std::min(vec, pow2_divisor((usz)(uintptr_t)a->dst_base, 16));
  vec = std::min(vec, pow2_divisor((usz)(uintptr_t)a->src_base, 16));
  RearrangeParams p;
  p.dst = (char *)a->dst_base;
  p.src = (const char *)a->src_base;
  p.ndim = (int)ndim;
  for (usz i = 0; i < ndim; ++i) {
    p.idx[i] = L[2 + i];
    p.ds[i] = L[2 + ndim + i];
    p.ss[i] = L[2 + 2 * ndim + i];
    vec = std::min(vec, pow2_divisor((usz)iabs(p.ds[i]), 16));
    vec = std::min(vec, pow2_divisor((usz)iabs(p.ss[i]), 16));
  }
  p.vec_per_unit = (long long)(unit / vec);
  p.total_vec = (long long)count * p.vec_per_unit;

  p.vec_shift = -1;
  if ((p.vec_per_unit & (p.vec_per_unit - 1)) == 0) {
    p.vec_shift = 0;
    while ((1ll << p.vec_shift) < p.vec_per_unit) ++p.vec_shift;
  }
  cudaSetDevice(base.device);
  const long long blocks = (p.total_vec + 1023) / 1024;
  if (blocks > 0x7fffffffll) return fail(OPS_SHAPE_NOT_SUPPORT, "rearrange: tensor too large");
  const unsigned grid = (unsigned)blocks;
  const bool small = p.total_vec < 0x7fffffffll;  // every index (vector, unit, per-dim count) fits 32 bits
#define REARRANGE_LAUNCH(VEC)                                              \
  do {                                                                     \
    if (small) rearrange_kernel<VEC, unsigned int><<<grid, 256, 0, s>>>(p); \
    else rearrange_kernel<VEC, long long><<<grid, 256, 0, s>>>(p);          \
  } while (0)
  switch (vec) {
    case 16: REARRANGE_LAUNCH(16); break;
    case 8: REARRANGE_LAUNCH(8); break;
    case 4: REARRANGE_LAUNCH(4); break;
    case 2: REARRANGE_LAUNCH(2); break;
    default: REARRANGE_LAUNCH(1); break;
  }
#undef REARRANGE_LAUNCH
  return check_launch("rearrange");
}

}  // namespace ops

using namespace ops;

OPS_DEFINE_SIMPLE_HANDLE(rearrange)

OPS_API int ops_rearrange_plan(const ops_rearrange_args *args, ptrdiff_t *out, size_t cap, size_t *ndim_out) {
  std::vector<isz> L;
  OPS_TRY(rearrange_plan(args, L));
  if (L.size() > cap) return fail(OPS_ARGS_NOT_SUPPORT, "plan needs %zu words, %zu given", L.size(), cap);
  std::copy(L.begin(), L.end(), out);
  if (ndim_out) *ndim_out = (L.size() - 2) / 3;
  return OPS_OK;
}

// The crate's CPU rearrange does no work in scheme() (operators/src/rearrange/common_cpu/mod.rs:18-24);
// here static arguments are planned once so that bad layouts surface early, dynamic ones pass.
OPS_API int ops_rearrange_scheme(ops_rearrange *op, const ops_rearrange_args *args, size_t max_ws, size_t *ws_out) {
  (void)op;
  (void)max_ws;
  if (ws_out) *ws_out = 0;
  if (args->dst_layout.dt != args->src_layout.dt) return fail(OPS_TYPE_MISMATCH, "dst and src element types differ");
  if (args->dst_layout.ndim != args->src_layout.ndim) return fail(OPS_RANK_MISMATCH, "dst.ndim = %u, src.ndim = %u", args->dst_layout.ndim, args->src_layout.ndim);
  return OPS_OK;
}

OPS_API int ops_rearrange_launch(const ops_rearrange *op, const ops_rearrange_args *args, void *ws, size_t ws_len, void *stream) {
  (void)ws;
  (void)ws_len;
  return rearrange_enqueue(op->base, args, (cudaStream_t)stream);
}
