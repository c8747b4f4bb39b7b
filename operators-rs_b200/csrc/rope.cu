// rope.cu — in-place rotary position embedding on t [nt, nh, dh], adjacent pairs (2k, 2k+1).
//
// Replaces rope::common_cpu::Operator (operators/src/rope/common_cpu/mod.rs:65-130; arithmetic
// :164-202, loop :212-240); argument checks follow Args::meta (operators/src/rope/args.rs:28-72).
//
// HBM-bound: 2*nt*nh*dh*2 bytes.  One CTA per token: sin/cos of the dh/2 angles are computed ONCE
// per token into shared memory (the CPU path recomputes them for every head), then every thread
// rotates 4 pairs per 128-bit access across all heads.
//
// The dh/2 divisors theta^(k/(dh/2)) are evaluated on the host with libm powf — the function the
// crate's CPU path lowers to — and travel as a kernel parameter, so the angle pos/divisor is formed
// from bit-identical divisors; the division is IEEE and sincosf is the full-range (non fast-math) one.
#include "common.h"
#include "device_utils.cuh"

namespace ops {

constexpr int ROPE_MAX_HALF = 256;  // divisors passed by value: dh <= 512

struct RopeDivisors {
  float v[ROPE_MAX_HALF];
};

// `toks` tokens per CTA: the sin/cos pairs of all of them are computed first, one per thread (one token per CTA left three
// quarters of a 256-thread CTA idle through the sincosf latency, which then bounded the launch, not HBM), then the CTA
// streams the tokens' rows (few registers on purpose: eight CTAs per SM hide the latency of each other's phases).
template <class E, class P>
__global__ void __launch_bounds__(256) rope_f16_kernel(E *__restrict__ t, long long st, long long sh, const P *__restrict__ pos,
                                                       long long sp, int nt, int toks, int nh, int half_dh,
                                                       const __grid_constant__ RopeDivisors div) {
  extern __shared__ float2 sincos_tab[];  // [toks][half_dh] (sin, cos)
  const long long tok0 = (long long)blockIdx.x * toks;
  const int here = (int)min((long long)toks, (long long)nt - tok0);
  for (int i = threadIdx.x; i < here * half_dh; i += blockDim.x) {
    const int tk = i / half_dh, k = i - tk * half_dh;
    const float p = (float)*byte_off(pos, (tok0 + tk) * sp);
    float s, c;
    sincosf(__fdiv_rn(p, div.v[k]), &s, &c);
    sincos_tab[i] = make_float2(s, c);
  }
  __syncthreads();
  const int vec_per_head = half_dh >> 2;  // 4 pairs = 8 halves per vector
  const int per_tok = nh * vec_per_head;
  const int total = here * per_tok;
  for (int v = threadIdx.x; v < total; v += blockDim.x) {
    const int tk = v / per_tok, r = v - tk * per_tok;
    const int head = r / vec_per_head, kv = r - head * vec_per_head;
    E *ptr = byte_off(byte_off(t, (tok0 + tk) * st), (long long)head * sh) + kv * 8;
    const float2 *tab = sincos_tab + tk * half_dh + kv * 4;
    Vec8<E> in, out;
    in.u = ld_global_16(ptr);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 sc = tab[e];
      const float a = to_f32(in.h[2 * e]), b = to_f32(in.h[2 * e + 1]);
      out.h[2 * e] = from_f32<E>(__fsub_rn(__fmul_rn(a, sc.y), __fmul_rn(b, sc.x)));
      out.h[2 * e + 1] = from_f32<E>(__fadd_rn(__fmul_rn(a, sc.x), __fmul_rn(b, sc.y)));
    }
    st_global_16(ptr, out.u);
  }
}

// Generic path: f16 or f32 data, any dh (even), no alignment demands; divisors by device powf when
// the table does not fit.
template <class T, class P>
__global__ void __launch_bounds__(256) rope_generic_kernel(T *t, long long st, long long sh, const P *pos, long long sp, int nh,
                                                           int half_dh, float theta, const __grid_constant__ RopeDivisors div,
                                                           int use_table) {
  const long long tok = blockIdx.x;
  const float p = (float)*byte_off(pos, tok * sp);
  T *row = byte_off(t, tok * st);
  const long long total = (long long)nh * half_dh;
  for (long long i = threadIdx.x; i < total; i += blockDim.x) {
    const int head = (int)(i / half_dh), k = (int)(i - (long long)head * half_dh);
    const float dv = use_table ? div.v[k] : powf(theta, __fdiv_rn((float)k, (float)half_dh));
    float s, c;
    sincosf(__fdiv_rn(p, dv), &s, &c);
    T *ptr = byte_off(row, (long long)head * sh) + 2 * k;
    const float a = to_f32(ptr[0]), b = to_f32(ptr[1]);
    ptr[0] = from_f32<T>(__fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s)));
    ptr[1] = from_f32<T>(__fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c)));
  }
}

struct RopeMeta {
  uint32_t dt_t, dt_p;
  usz nt, dh;
};

static int rope_meta(const ops_rope_args *a, RopeMeta *m) {
  if (a->t_layout.ndim != 3) return fail(OPS_RANK_NOT_SUPPORT, "t.ndim = %u, 3 expected", a->t_layout.ndim);
  if (a->p_layout.ndim != 1) return fail(OPS_RANK_NOT_SUPPORT, "p.ndim = %u, 1 expected", a->p_layout.ndim);
  if (a->sin_layout.ndim != 2) return fail(OPS_RANK_NOT_SUPPORT, "sin.ndim = %u, 2 expected", a->sin_layout.ndim);
  if (a->cos_layout.ndim != 2) return fail(OPS_RANK_NOT_SUPPORT, "cos.ndim = %u, 2 expected", a->cos_layout.ndim);
  m->dt_t = a->t_layout.dt;
  m->dt_p = a->p_layout.dt;
  if (!is_float_dt(m->dt_t)) return fail(OPS_TYPE_NOT_SUPPORT, "data type of t is not supported, must be floating-point numbers");
  if (!is_unsigned_dt(m->dt_p)) return fail(OPS_TYPE_NOT_SUPPORT, "data type of p is not supported, must be unsigned integers");
  const usz nts[2] = {a->t_layout.shape[0], a->p_layout.shape[0]};
  const usz dhs[3] = {a->t_layout.shape[2], a->sin_layout.shape[1], a->cos_layout.shape[1]};
  if (!merge_dims(nts, 2, &m->nt)) return fail(OPS_SHAPE_MISMATCH, "nt of t and p differ");
  if (!merge_dims(dhs, 3, &m->dh)) return fail(OPS_SHAPE_MISMATCH, "dh of t, sin and cos differ");
  return OPS_OK;
}

}  // namespace ops

using namespace ops;

OPS_DEFINE_SIMPLE_HANDLE(rope)

OPS_API int ops_rope_scheme(ops_rope *op, const ops_rope_args *args, size_t max_ws, size_t *ws_out) {
  (void)op;
  (void)max_ws;
  RopeMeta m;
  OPS_TRY(rope_meta(args, &m));
  if (ws_out) *ws_out = 0;
  return OPS_OK;
}

OPS_API int ops_rope_launch(const ops_rope *op, const ops_rope_args *a, void *ws, size_t ws_len, void *stream) {
  (void)ws;
  (void)ws_len;
  RopeMeta m;
  OPS_TRY(rope_meta(a, &m));
  const usz nh = a->t_layout.shape[1], dh = a->t_layout.shape[2];
  const isz st = a->t_layout.strides[0], sh = a->t_layout.strides[1], sd = a->t_layout.strides[2];
  const isz sp = a->p_layout.strides[0];
  if (dyn(m.nt) || dyn(nh) || dyn(dh) || dyn(st) || dyn(sh) || dyn(sd) || dyn(sp) || dyn(a->theta))
    return fail(OPS_DYNAMIC_NOT_SUPPORT, "rope: every shape, stride and theta must be static at launch");
  if (sd != (isz)dt_size(m.dt_t)) return fail(OPS_STRIDES_NOT_SUPPORT, "rope: last dim of t must be contiguous");
  if (m.dt_t != OPS_DT_F16 && m.dt_t != OPS_DT_BF16 && m.dt_t != OPS_DT_F32) return fail(OPS_TYPE_NOT_SUPPORT, "rope: t must be f16, bf16 or f32");
  if (m.dt_p != OPS_DT_U32 && m.dt_p != OPS_DT_U64) return fail(OPS_TYPE_NOT_SUPPORT, "rope: p must be u32 or u64");
  if (dh % 2) return fail(OPS_SHAPE_NOT_SUPPORT, "rope: dh must be even");
  if (m.nt == 0 || nh == 0 || dh == 0) return OPS_OK;
  if (m.nt > 0x7fffffffu || nh > 0x7fffffu || dh > 0x7fffffu) return fail(OPS_SHAPE_NOT_SUPPORT, "rope: shape too large");
  if (!a->t_base || !a->p_base) return fail(OPS_DYNAMIC_NOT_SUPPORT, "rope: null base pointer at launch");
  cudaStream_t s = (cudaStream_t)stream;
  cudaSetDevice(op->base.device);

  const int half_dh = (int)(dh / 2);
  RopeDivisors div;
  const int use_table = half_dh <= ROPE_MAX_HALF;
  if (use_table)
    for (int k = 0; k < half_dh; ++k) div.v[k] = powf(a->theta, (float)k / (float)half_dh);
  const bool t16 = m.dt_t == OPS_DT_F16 || m.dt_t == OPS_DT_BF16;
  const bool fast = t16 && use_table && dh % 8 == 0 && st % 16 == 0 && sh % 16 == 0 && aligned(a->t_base, 16);
  const dim3 grid((unsigned)m.nt);
  if (fast) {
    // tokens per CTA: one when a token's heads alone give every thread a 128-bit vector (a whole layer: measured faster
    // with many small CTAs); with few heads per token (a tensor-parallel shard) as many as fill the CTA's threads, at
    // most one sin/cos pair per thread (256 / half_dh); fewer when there are too few tokens to fill the machine otherwise
    const int vec_per_tok = (int)nh * (half_dh >> 2);
    int toks = std::max(1, std::min(256 / half_dh, 256 / std::max(1, vec_per_tok)));
    while (toks > 1 && (m.nt + toks - 1) / toks < 2 * (usz)op->base.sm_count) toks >>= 1;
    const dim3 fgrid((unsigned)((m.nt + toks - 1) / toks));
    const usz smem = (usz)toks * half_dh * sizeof(float2);
#define ROPE_FAST(E, P) \
  rope_f16_kernel<E, P><<<fgrid, 256, smem, s>>>((E *)a->t_base, st, sh, (const P *)a->p_base, sp, (int)m.nt, toks, (int)nh, half_dh, div)
    if (m.dt_t == OPS_DT_F16 && m.dt_p == OPS_DT_U32) ROPE_FAST(__half, uint32_t);
    else if (m.dt_t == OPS_DT_F16) ROPE_FAST(__half, unsigned long long);
    else if (m.dt_p == OPS_DT_U32) ROPE_FAST(__nv_bfloat16, uint32_t);
    else ROPE_FAST(__nv_bfloat16, unsigned long long);
#undef ROPE_FAST
  } else {
#define ROPE_GENERIC(T, P) rope_generic_kernel<T, P><<<grid, 256, 0, s>>>((T *)a->t_base, st, sh, (const P *)a->p_base, sp, (int)nh, half_dh, a->theta, div, use_table)
    if (m.dt_t == OPS_DT_F16 && m.dt_p == OPS_DT_U32) ROPE_GENERIC(__half, uint32_t);
    else if (m.dt_t == OPS_DT_F16) ROPE_GENERIC(__half, unsigned long long);
    else if (m.dt_t == OPS_DT_BF16 && m.dt_p == OPS_DT_U32) ROPE_GENERIC(__nv_bfloat16, uint32_t);
    else if (m.dt_t == OPS_DT_BF16) ROPE_GENERIC(__nv_bfloat16, unsigned long long);
    else if (m.dt_p == OPS_DT_U32) ROPE_GENERIC(float, uint32_t);
    else ROPE_GENERIC(float, unsigned long long);
#undef ROPE_GENERIC
  }
  return check_launch("rope");
}

// Rope::build_pos / fill_pos (operators/src/rope/mod.rs:44-58): positions of each (pos, len) run.
OPS_API int ops_rope_build_pos(uint32_t dt, size_t nt, const size_t *seq_pos, const size_t *seq_len, size_t nseq, void *host_out) {
  if (dt != OPS_DT_U32 && dt != OPS_DT_U64) return fail(OPS_TYPE_NOT_SUPPORT, "build_pos: u32 or u64 expected");
  size_t i = 0;
  for (size_t s = 0; s < nseq && i < nt; ++s)
    for (size_t p = seq_pos[s]; p < seq_pos[s] + seq_len[s] && i < nt; ++p, ++i) {
      if (dt == OPS_DT_U32) ((uint32_t *)host_out)[i] = (uint32_t)p;
      else ((uint64_t *)host_out)[i] = (uint64_t)p;
    }
  return OPS_OK;
}
