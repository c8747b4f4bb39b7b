// fused_softmax.cu — in-place masked softmax over the last dim of att [nh, seq, att_len].
//
// Replaces fuesd_softmax::common_cpu::Operator (operators/src/fuesd_softmax/common_cpu/mod.rs:32-82;
// row rule :99-114, f16 arithmetic :117-145); argument checks follow Args::meta
// (operators/src/fuesd_softmax/args.rs:31-37).
//
// HBM-bound: every element is written (masked ones as zero) but only the unmasked prefix of a causal
// row is read.  A row lives in registers between the max, exp/sum and scale steps, so the prefix is
// read from HBM once.  Rows up to 4096 columns: one warp per row; longer rows: one CTA per row.  The f16 rounding
// sequence of the CPU path is kept: exp is rounded to f16, the sum uses the unrounded f32 exps, the
// rounded value is re-widened, scaled by 1/sum and rounded again.
#include "common.h"
#include "device_utils.cuh"
#include "internal.h"

namespace ops {

struct SoftmaxParams {
  void *base;
  long long sh, ss, sa;
  int nh, seq, att_len;
  int causal;
};

__device__ __forceinline__ int row_limit(const SoftmaxParams &p, int k) { return p.causal ? p.att_len - p.seq + k + 1 : p.att_len; }

// Register-resident row.  GROUP threads cooperate on one row (32 = a warp, else the whole CTA);
// each owns VPT vectors of 8 halves, vector v = lane + i * GROUP.
template <class E, int VPT, bool WARP>
__global__ void __launch_bounds__(256) softmax_f16_reg_kernel(const __grid_constant__ SoftmaxParams p) {
  __shared__ float scratch[33];
  const int group = WARP ? 32 : blockDim.x;
  const int lane = WARP ? (threadIdx.x & 31) : threadIdx.x;
  const long long rows = (long long)p.nh * p.seq;
  const long long row = WARP ? (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5) : (long long)blockIdx.x;
  if (row >= rows) return;  // warp-uniform in WARP mode, CTA-uniform otherwise
  const int j = (int)(row / p.seq), k = (int)(row - (long long)j * p.seq);
  E *att = byte_off((E *)p.base, j * p.sh + k * p.ss);
  const int limit = row_limit(p, k);

  Vec8<E> xv[VPT];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c0 = (lane + i * group) * 8;
    if (c0 < limit) {
      xv[i].u = ld_global_16(att + c0);
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if (c0 + e < limit) mx = fmaxf(mx, to_f32(xv[i].h[e]));
    }
  }
  mx = WARP ? warp_max(mx) : block_max(mx, scratch);

  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c0 = (lane + i * group) * 8;
    if (c0 < limit) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if (c0 + e < limit) {
          // special-function-unit exponential (relative error ~2^-22, far below the 16-bit rounding that follows): with
          // libm-grade expf the register kernel is bound by instruction issue, not by HBM
          const float ex = __expf(__fsub_rn(to_f32(xv[i].h[e]), mx));
          xv[i].h[e] = from_f32<E>(ex);
          sum += ex;
        }
      }
    }
  }
  sum = WARP ? warp_sum(sum) : block_sum(sum, scratch);
  const float div = __frcp_rn(sum);

#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c0 = (lane + i * group) * 8;
    if (c0 < p.att_len) {
      Vec8<E> out;
#pragma unroll
      for (int e = 0; e < 8; ++e)
        out.h[e] = (c0 + e < limit) ? from_f32<E>(__fmul_rn(to_f32(xv[i].h[e]), div)) : from_f32<E>(0.f);
      st_global_16(att + c0, out.u);
    }
  }
}

// Generic path: any strides and length, f16 or f32; three passes over the row from global memory.
template <class T>
__global__ void __launch_bounds__(256) softmax_generic_kernel(const __grid_constant__ SoftmaxParams p) {
  __shared__ float scratch[33];
  const long long row = blockIdx.x;
  const int j = (int)(row / p.seq), k = (int)(row - (long long)j * p.seq);
  T *att = byte_off((T *)p.base, j * p.sh + k * p.ss);
  const int limit = row_limit(p, k);
  float mx = -INFINITY;
  for (int c = threadIdx.x; c < limit; c += blockDim.x) mx = fmaxf(mx, to_f32(*byte_off(att, c * p.sa)));
  mx = block_max(mx, scratch);
  float sum = 0.f;
  for (int c = threadIdx.x; c < limit; c += blockDim.x) {
    T *x = byte_off(att, c * p.sa);
    const float ex = expf(__fsub_rn(to_f32(*x), mx));
    *x = from_f32<T>(ex);
    sum += ex;
  }
  sum = block_sum(sum, scratch);
  const float div = __frcp_rn(sum);
  for (int c = threadIdx.x; c < p.att_len; c += blockDim.x) {
    T *x = byte_off(att, c * p.sa);
    *x = c < limit ? from_f32<T>(__fmul_rn(to_f32(*x), div)) : from_f32<T>(0.f);
  }
}

static int softmax_meta(const ops_fused_softmax_args *a) {
  if (a->att_layout.ndim != 3) return fail(OPS_RANK_NOT_SUPPORT, "att.ndim = %u, 3 expected", a->att_layout.ndim);
  return OPS_OK;
}

}  // namespace ops

using namespace ops;

OPS_DEFINE_SIMPLE_HANDLE(fused_softmax)

OPS_API int ops_fused_softmax_scheme(ops_fused_softmax *op, const ops_fused_softmax_args *args, size_t max_ws, size_t *ws_out) {
  (void)op;
  (void)max_ws;
  OPS_TRY(softmax_meta(args));
  if (ws_out) *ws_out = 0;
  return OPS_OK;
}

int ops::fused_softmax_enqueue(const OpBase &base, const ops_fused_softmax_args *a, cudaStream_t s) {
  OPS_TRY(softmax_meta(a));
  const uint32_t dt = a->att_layout.dt;
  const usz nh = a->att_layout.shape[0], seq = a->att_layout.shape[1], att_len = a->att_layout.shape[2];
  const isz sh = a->att_layout.strides[0], ss = a->att_layout.strides[1], sa = a->att_layout.strides[2];
  if (dyn(nh) || dyn(seq) || dyn(att_len) || dyn(sh) || dyn(ss) || dyn(sa))
    return fail(OPS_DYNAMIC_NOT_SUPPORT, "fused_softmax: every shape and stride must be static at launch");
  if (dt != OPS_DT_F16 && dt != OPS_DT_BF16 && dt != OPS_DT_F32) return fail(OPS_TYPE_NOT_SUPPORT, "fused_softmax: f16, bf16 or f32 expected");
  if (a->att_mask != OPS_MASK_NONE && a->att_mask != OPS_MASK_CAUSAL) return fail(OPS_ARGS_NOT_SUPPORT, "fused_softmax: unknown mask %u", a->att_mask);
  if (nh == 0 || seq == 0 || att_len == 0) return OPS_OK;
  if (a->att_mask == OPS_MASK_CAUSAL && att_len < seq) return fail(OPS_SHAPE_NOT_SUPPORT, "fused_softmax: causal mask needs att_len >= seq_len");
  if (att_len > 0x7fffffffu || seq > 0x7fffffffu || nh > 0x7fffffffu || nh * seq > 0x7fffffffu)
    return fail(OPS_SHAPE_NOT_SUPPORT, "fused_softmax: shape too large");
  if (!a->att_base) return fail(OPS_DYNAMIC_NOT_SUPPORT, "fused_softmax: null base pointer at launch");
  cudaSetDevice(base.device);

  SoftmaxParams p{a->att_base, sh, ss, sa, (int)nh, (int)seq, (int)att_len, a->att_mask == OPS_MASK_CAUSAL};
  const long long rows = (long long)nh * (long long)seq;
  const bool vec = (dt == OPS_DT_F16 || dt == OPS_DT_BF16) && sa == 2 && att_len % 8 == 0 && sh % 16 == 0 && ss % 16 == 0 && aligned(a->att_base, 16);
  const int nvec = (int)(att_len / 8);
#define OPS_SOFTMAX_REG(E)                                                                                     \
  do {                                                                                                         \
    if (nvec <= 32 * 16) {                                                                                     \
      /* one warp per row (rows up to 4096 columns live in 64 registers per lane): no block-level synchronisation, */ \
      /* 8 rows per CTA keep enough bytes in flight even when a causal mask leaves most lanes of a row idle */ \
      const unsigned grid = (unsigned)((rows + 7) / 8);                                                        \
      if (nvec <= 32) softmax_f16_reg_kernel<E, 1, true><<<grid, 256, 0, s>>>(p);                              \
      else if (nvec <= 64) softmax_f16_reg_kernel<E, 2, true><<<grid, 256, 0, s>>>(p);                         \
      else if (nvec <= 128) softmax_f16_reg_kernel<E, 4, true><<<grid, 256, 0, s>>>(p);                        \
      else if (nvec <= 256) softmax_f16_reg_kernel<E, 8, true><<<grid, 256, 0, s>>>(p);                        \
      else softmax_f16_reg_kernel<E, 16, true><<<grid, 256, 0, s>>>(p);                                        \
    } else {                                                                                                   \
      /* one CTA per row; every thread owns at most 8 vectors */                                               \
      softmax_f16_reg_kernel<E, 8, false><<<(unsigned)rows, 256, 0, s>>>(p);                                   \
    }                                                                                                          \
  } while (0)
  if (vec && nvec <= 256 * 8) {
    if (dt == OPS_DT_F16) OPS_SOFTMAX_REG(__half);
    else OPS_SOFTMAX_REG(__nv_bfloat16);
  } else if (dt == OPS_DT_F16) {
    softmax_generic_kernel<__half><<<(unsigned)rows, 256, 0, s>>>(p);
  } else if (dt == OPS_DT_BF16) {
    softmax_generic_kernel<__nv_bfloat16><<<(unsigned)rows, 256, 0, s>>>(p);
  } else {
    softmax_generic_kernel<float><<<(unsigned)rows, 256, 0, s>>>(p);
  }
#undef OPS_SOFTMAX_REG
  return check_launch("fused_softmax");
}

OPS_API int ops_fused_softmax_launch(const ops_fused_softmax *op, const ops_fused_softmax_args *a, void *ws, size_t ws_len, void *stream) {
  (void)ws;
  (void)ws_len;
  return fused_softmax_enqueue(op->base, a, (cudaStream_t)stream);
}
