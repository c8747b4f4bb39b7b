// attention_decode.cu — attention for a handful of query tokens over a long KV range (decode steps of
// attention_kv_cached: seq = 1..2 new tokens against a cache of hundreds or thousands of keys).
//
// Same function as attention::Operator (operators/src/attention/operator.rs:136-277) for shapes where the
// tensor cores have nothing to chew on: group * seq <= 8 query rows per kv head.  The work is reading K and
// V once — E * 2 * nkvh * att * dh bytes, HBM-bound — so the key range of every kv head is split over many
// CTAs ("flash decoding"): each CTA streams its slice of K and V with 128-bit loads (half a warp per key
// row), keeps a running max / sum / output per query row in registers, and parks (m, l, o) in a scratch
// buffer owned by the operator handle; the last CTA of a kv head to finish merges the slices and writes o.
// The q rows of one GQA group share every K/V load.
#include "common.h"
#include "device_utils.cuh"
#include "internal.h"

namespace ops {

constexpr int DEC_THREADS = 256;
constexpr int DEC_WARPS = DEC_THREADS / 32;
constexpr int DEC_MAX_ROWS = 8;
constexpr int DEC_MAX_SPLITS = 64;
constexpr int DEC_MAX_KV_HEADS = 1024;  // arrival counters in the handle's scratch

struct DecodeArgs {
  const unsigned short *q, *k, *v;
  unsigned short *o;
  long long q_sh, q_ss, k_sh, k_ss, v_sh, v_ss, o_sh, o_ss;  // element strides: head, row (dh contiguous)
  int group, seq, att, rows;  // rows = group * seq
  int causal;
  int bf16;                   // elements are bf16 (else f16)
  int splits, keys_per_split;
  float scale_log2;
  float *partial;          // [nkvh][splits][rows][DH + 2]
  unsigned int *tickets;   // [nkvh], self-resetting
};

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float dec_to_f32(unsigned short b, int bf) {
  return bf ? __uint_as_float((uint32_t)b << 16) : __half2float(__ushort_as_half(b));
}
__device__ __forceinline__ unsigned short dec_from_f32(float v, int bf) {
  return bf ? __bfloat16_as_ushort(__float2bfloat16_rn(v)) : __half_as_ushort(__float2half_rn(v));
}

// DH = 64 or 128.  A key row is DH/8 lanes wide (8 elements per lane); LPK = lanes per key.
template <int DH, int ROWS>
__global__ void __launch_bounds__(DEC_THREADS) attention_decode_kernel(const __grid_constant__ DecodeArgs a) {
  constexpr int LPK = DH / 8;              // 16 or 8 lanes per key row
  constexpr int KPW = 32 / LPK;            // keys per warp per step
  constexpr int GROUPS = DEC_THREADS / LPK;  // key rows in flight per CTA step
  __shared__ float q_s[ROWS][DH];
  __shared__ float red_m[DEC_WARPS][ROWS], red_l[DEC_WARPS][ROWS];
  __shared__ float red_o[DEC_WARPS][ROWS][DH];  // 32 KB at most
  __shared__ unsigned int s_last;
  const int kvh = blockIdx.x, split = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane / LPK, li = lane % LPK;  // which key of the warp step, which 8-column slice of dh
  const int off = a.att - a.seq;
  const int bf = a.bf16;

  // q rows of this kv head, pre-scaled into the exp2 domain
  for (int i = threadIdx.x; i < ROWS * DH; i += DEC_THREADS) {
    const int r = i / DH, c = i - r * DH;
    float val = 0.f;
    if (r < a.rows) {
      const int gi = r / a.seq, si = r - gi * a.seq;
      val = dec_to_f32(a.q[(long long)(kvh * a.group + gi) * a.q_sh + (long long)si * a.q_ss + c], bf) * a.scale_log2;
    }
    q_s[r][c] = val;
  }
  __syncthreads();
  float qr[ROWS][8];
#pragma unroll
  for (int r = 0; r < ROWS; ++r)
#pragma unroll
    for (int e = 0; e < 8; ++e) qr[r][e] = q_s[r][li * 8 + e];
  int lim[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int si = r % a.seq;
    lim[r] = r < a.rows ? (a.causal ? min(a.att - 1, off + si) : a.att - 1) : -1;
  }

  float m[ROWS], l[ROWS], o[ROWS][8];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    m[r] = -INFINITY;
    l[r] = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) o[r][e] = 0.f;
  }
  const int k_begin = split * a.keys_per_split, k_end = min(a.att, k_begin + a.keys_per_split);
  const unsigned short *kbase = a.k + (long long)kvh * a.k_sh + li * 8;
  const unsigned short *vbase = a.v + (long long)kvh * a.v_sh + li * 8;
  // Keys are taken eight steps at a time: the sixteen 128-bit loads of a batch (K and V of eight key rows per lane) are
  // all issued before the first is used, so a CTA pays the DRAM latency once per 128 keys, not once per 16.
  constexpr int UN = 8;
  for (int kb0 = k_begin + warp * KPW; kb0 < k_end; kb0 += GROUPS * UN) {  // warp-uniform trip count: the shuffles need every lane
    uint4 kq[UN], vq[UN];
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int key = kb0 + u * GROUPS + sub;
      const int kload = key < k_end ? key : k_end - 1;
      kq[u] = __ldcs(reinterpret_cast<const uint4 *>(kbase + (long long)kload * a.k_ss));
      vq[u] = __ldcs(reinterpret_cast<const uint4 *>(vbase + (long long)kload * a.v_ss));
    }
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int key = kb0 + u * GROUPS + sub;
      const bool valid = key < k_end;
      Vec8<unsigned short> kk, vv;
      kk.u = kq[u];
      vv.u = vq[u];
      float kf[8], vf[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        kf[e] = dec_to_f32(kk.h[e], bf);
        vf[e] = dec_to_f32(vv.h[e], bf);
      }
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        float s = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) s = fmaf(qr[r][e], kf[e], s);
#pragma unroll
        for (int d = LPK / 2; d > 0; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);  // stays inside the LPK-lane group
        if (valid && key <= lim[r]) {
          const float m_new = fmaxf(m[r], s);
          const float alpha = ex2f(m[r] - m_new), p = ex2f(s - m_new);
          l[r] = fmaf(l[r], alpha, p);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[r][e] = fmaf(o[r][e], alpha, p * vf[e]);
          m[r] = m_new;
        }
      }
    }
  }

  // merge the key groups of one warp with shuffles (common max, rescaled sums), then the warps through shared memory
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    float mm = m[r];
#pragma unroll
    for (int d = LPK; d < 32; d <<= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, d));
    const float sc = (m[r] == -INFINITY) ? 0.f : ex2f(m[r] - mm);
    float lr = l[r] * sc;
#pragma unroll
    for (int d = LPK; d < 32; d <<= 1) lr += __shfl_xor_sync(0xffffffffu, lr, d);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float ov = o[r][e] * sc;
#pragma unroll
      for (int d = LPK; d < 32; d <<= 1) ov += __shfl_xor_sync(0xffffffffu, ov, d);
      o[r][e] = ov;
    }
    m[r] = mm;
    l[r] = lr;
    if (lane == 0) red_m[warp][r] = mm;
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) mm = fmaxf(mm, red_m[w][r]);
    const float sc = (m[r] == -INFINITY) ? 0.f : ex2f(m[r] - mm);
    if (lane == 0) red_l[warp][r] = l[r] * sc;
    if (sub == 0) {
#pragma unroll
      for (int e = 0; e < 8; ++e) red_o[warp][r][li * 8 + e] = o[r][e] * sc;
    }
  }
  __syncthreads();
  // park (m, l, o) of this split
  float *part = a.partial + (((long long)kvh * a.splits + split) * ROWS) * (DH + 2);
  for (int i = threadIdx.x; i < ROWS * DH; i += DEC_THREADS) {
    const int r = i / DH, c = i - r * DH;
    float acc = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) acc += red_o[w][r][c];
    part[r * (DH + 2) + 2 + c] = acc;
  }
  if (threadIdx.x < ROWS) {
    const int r = threadIdx.x;
    float ls = 0.f, mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      ls += red_l[w][r];
      mm = fmaxf(mm, red_m[w][r]);
    }
    part[r * (DH + 2)] = mm;
    part[r * (DH + 2) + 1] = ls;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(&a.tickets[kvh], 1u) == (unsigned)(a.splits - 1) ? 1u : 0u;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (threadIdx.x == 0) a.tickets[kvh] = 0;  // ready for the next launch
  // last CTA of this kv head: merge the splits in split order.  First the per-split weights 2^(m_s - m) and the
  // denominators (one thread per (row, split) then per row), then every output element as an independent dot product
  // over the splits whose loads are all in flight together (one round trip to L2 for up to 16 splits).
  __shared__ float w_s[ROWS][DEC_MAX_SPLITS], l_s[ROWS][DEC_MAX_SPLITS];
  __shared__ float den_s[ROWS];
  const float *pall = a.partial + ((long long)kvh * a.splits) * ROWS * (DH + 2);
  for (int i = threadIdx.x; i < ROWS * a.splits; i += DEC_THREADS) {
    const int r = i / a.splits, sp = i - r * a.splits;
    const float *pr = pall + ((long long)sp * ROWS + r) * (DH + 2);
    w_s[r][sp] = __ldcg(pr);  // m of this split, turned into a weight below
    l_s[r][sp] = __ldcg(pr + 1);
  }
  __syncthreads();
  if (threadIdx.x < ROWS) {
    const int r = threadIdx.x;
    float mm = -INFINITY;
    for (int sp = 0; sp < a.splits; ++sp) mm = fmaxf(mm, w_s[r][sp]);
    float den = 0.f;
    for (int sp = 0; sp < a.splits; ++sp) {
      const float ms = w_s[r][sp];
      const float w = ms == -INFINITY ? 0.f : ex2f(ms - mm);
      w_s[r][sp] = w;
      den = fmaf(l_s[r][sp], w, den);
    }
    den_s[r] = den;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < a.rows * DH; i += DEC_THREADS) {
    const int r = i / DH, c = i - r * DH;
    const float *col = pall + (long long)r * (DH + 2) + 2 + c;
    float num = 0.f;
    int sp = 0;
    for (; sp + 16 <= a.splits; sp += 16) {  // sixteen loads in flight
      float v[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) v[u] = __ldcg(col + (long long)(sp + u) * ROWS * (DH + 2));
#pragma unroll
      for (int u = 0; u < 16; ++u) num = fmaf(v[u], w_s[r][sp + u], num);
    }
    for (; sp + 4 <= a.splits; sp += 4) {
      float v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = __ldcg(col + (long long)(sp + u) * ROWS * (DH + 2));
#pragma unroll
      for (int u = 0; u < 4; ++u) num = fmaf(v[u], w_s[r][sp + u], num);
    }
    for (; sp < a.splits; ++sp) num = fmaf(__ldcg(col + (long long)sp * ROWS * (DH + 2)), w_s[r][sp], num);
    const int gi = r / a.seq, si = r - gi * a.seq;
    a.o[(long long)(kvh * a.group + gi) * a.o_sh + (long long)si * a.o_ss + c] = dec_from_f32(num / den_s[r], bf);
  }
}

static bool rows_ok(const void *p, const isz *st, usz dh, bool need16) {
  if (st[2] != 2 || st[0] % 2 || st[1] % 2) return false;
  if (need16 && (!aligned(p, 16) || st[0] % 16 || st[1] % 16)) return false;
  (void)dh;
  return true;
}

bool attention_decode_supported(const ops_attention_args *a, usz nh, usz nkvh, usz seq, usz att, usz dh) {
  if ((a->q_layout.dt != OPS_DT_F16 && a->q_layout.dt != OPS_DT_BF16) || (dh != 64 && dh != 128)) return false;
  const usz rows = nh / nkvh * seq;
  if (rows == 0 || rows > (usz)DEC_MAX_ROWS || att < 256 || nkvh > (usz)DEC_MAX_KV_HEADS || att > 0x3fffffffu) return false;
  const isz *sv = a->v_layout.strides, *so = a->o_layout.strides;
  if (dyn(sv[0]) || dyn(sv[1]) || dyn(sv[2]) || dyn(so[0]) || dyn(so[1]) || dyn(so[2])) return false;
  return rows_ok(a->q_base, a->q_layout.strides, dh, false) && rows_ok(a->k_base, a->k_layout.strides, dh, true) &&
         rows_ok(a->v_base, sv, dh, true) && rows_ok(a->o_base, so, dh, false);
}

usz attention_decode_scratch_bytes() { return (usz)4 << 20; }
usz attention_decode_ticket_bytes() { return (usz)DEC_MAX_KV_HEADS * sizeof(unsigned int); }

int attention_decode_enqueue(const OpBase &base, const ops_attention_args *a, usz nh, usz nkvh, usz seq, usz att, usz dh, float *scratch,
                             unsigned int *tickets, cudaStream_t s) {
  DecodeArgs g;
  const isz *sq = a->q_layout.strides, *sk = a->k_layout.strides, *sv = a->v_layout.strides, *so = a->o_layout.strides;
  g.q = (const unsigned short *)a->q_base;
  g.k = (const unsigned short *)a->k_base;
  g.v = (const unsigned short *)a->v_base;
  g.o = (unsigned short *)a->o_base;
  g.bf16 = a->q_layout.dt == OPS_DT_BF16;
  g.q_sh = sq[0] / 2; g.q_ss = sq[1] / 2;
  g.k_sh = sk[0] / 2; g.k_ss = sk[1] / 2;
  g.v_sh = sv[0] / 2; g.v_ss = sv[1] / 2;
  g.o_sh = so[0] / 2; g.o_ss = so[1] / 2;
  g.group = (int)(nh / nkvh);
  g.seq = (int)seq;
  g.att = (int)att;
  g.rows = g.group * g.seq;
  g.causal = a->mask == OPS_MASK_CAUSAL;
  const int row_slots = g.rows <= 4 ? 4 : 8;
  // about one 256-thread CTA per SM, at least 256 keys each (16 steps of 16 key rows), and partials that fit the scratch
  // buffer; few splits keep the merge by the last CTA of a kv head short
  usz splits = ((usz)base.sm_count + nkvh - 1) / nkvh;
  splits = std::min<usz>(splits, (att + 255) / 256);
  splits = std::min<usz>(splits, DEC_MAX_SPLITS);
  const usz per_split = nkvh * (usz)row_slots * (dh + 2) * sizeof(float);
  splits = std::min<usz>(splits, attention_decode_scratch_bytes() / per_split);
  if (splits < 1) return fail(OPS_SHAPE_NOT_SUPPORT, "attention: too many kv heads for the decode scratch buffer");
  g.splits = (int)splits;
  g.keys_per_split = (int)((att + splits - 1) / splits);
  g.splits = (int)((att + g.keys_per_split - 1) / g.keys_per_split);
  const float inv_sqrt = 1.f / sqrtf((float)dh);
  const float alpha = g.bf16 ? __bfloat162float(__float2bfloat16_rn(inv_sqrt)) : __half2float(__float2half_rn(inv_sqrt));
  g.scale_log2 = alpha * 1.4426950408889634f;
  g.partial = scratch;
  g.tickets = tickets;
  cudaSetDevice(base.device);
  dim3 grid((unsigned)nkvh, (unsigned)g.splits);
  if (dh == 128) {
    if (row_slots == 4) attention_decode_kernel<128, 4><<<grid, DEC_THREADS, 0, s>>>(g);
    else attention_decode_kernel<128, 8><<<grid, DEC_THREADS, 0, s>>>(g);
  } else {
    if (row_slots == 4) attention_decode_kernel<64, 4><<<grid, DEC_THREADS, 0, s>>>(g);
    else attention_decode_kernel<64, 8><<<grid, DEC_THREADS, 0, s>>>(g);
  }
  return check_launch("attention(decode)");
}

}  // namespace ops
