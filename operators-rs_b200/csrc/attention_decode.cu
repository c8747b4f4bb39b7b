// attention_decode.cu — attention for a handful of query tokens over a long KV range (decode steps of
// attention_kv_cached: seq = 1..2 new tokens against a cache of hundreds or thousands of keys).
//
// Same function as attention::Operator (operators/src/attention/operator.rs:136-277) for shapes where a 128-row
// tcgen05 tile has nothing to chew on: group * seq <= 8 query rows per kv head.  The work is reading K and V once —
// E * 2 * nkvh * att * dh bytes, HBM-bound — so the key range of every kv head is split over many CTAs ("flash
// decoding"): a CTA takes 128 keys at a time, 16 per warp, every warp issuing all of its K and V loads (sixteen
// 128-bit loads per lane, 64 KB in flight per CTA) before touching the first.  The arithmetic rides on warp-level
// m16n8k16 MMAs so that the instruction stream stays far below the load stream:
//   S[16 x 8 keys]   = Q[16 rows (8 used) x 16 dh] . K^T      A = q rows (registers), B = K straight from global
//   O^T[16 dh x 8]   = V^T[16 dh x 16 keys] . P^T[16 keys x 8] B = the S fragments of two key tiles, exponentiated
// Both contractions are invariant under a permutation of the contracted index, so a lane's 128-bit load of a K row
// (8 consecutive dh) serves as the B fragments of two k-steps without any shuffle, and the V^T fragments are byte
// permutes of four 128-bit loads of V rows.  Running max / sum per query row stay in registers; the 8 warps meet in
// shared memory, the CTA parks (m, l, o) in a scratch buffer owned by the operator handle, and the last CTA of a kv
// head to finish merges the splits and writes o.  The q rows of one GQA group share every K/V load.
// When there are enough kv heads to fill the machine with 8 CTAs each, the 8 splits of a head form one thread-block
// cluster (16 warps per CTA) and meet in distributed shared memory instead: no partials in global memory, no fence, no
// arrival counter — a decode step over 4096 keys is short enough for those round trips to show.
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.h"
#include "device_utils.cuh"
#include "internal.h"

namespace ops {

constexpr int DEC_WARPS = 8;              // split kernel; the cluster kernel runs DEC_CLUSTER_WARPS
constexpr int DEC_CLUSTER_WARPS = 16;
constexpr int DEC_CLUSTER = 8;            // CTAs (key-range splits) per kv head in the cluster kernel
constexpr int DEC_CLUSTER_MAX = 8;        // bound of the merge loops
constexpr int DEC_MAX_ROWS = 8;           // the n extent of the MMA
constexpr int DEC_MAX_SPLITS = 64;
constexpr int DEC_MAX_KV_HEADS = 1024;  // arrival counters in the handle's scratch

struct DecodeArgs {
  const unsigned short *q, *k, *v;
  unsigned short *o;
  long long q_sh, q_ss, k_sh, k_ss, v_sh, v_ss, o_sh, o_ss;  // element strides: head, row (dh contiguous)
  int group, seq, att, rows;  // rows = group * seq
  int causal;
  int splits, keys_per_split;
  int q_vec;                  // q rows are 16-byte aligned: fragments are loaded straight from global memory
  float scale_log2;
  float *partial;          // [nkvh][splits][8][DH + 2]
  unsigned int *tickets;   // [nkvh], self-resetting
};

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
template <bool BF>
__device__ __forceinline__ unsigned short dec_from_f32(float v) {
  return BF ? __bfloat16_as_ushort(__float2bfloat16_rn(v)) : __half_as_ushort(__float2half_rn(v));
}
template <bool BF>
__device__ __forceinline__ uint32_t dec_pack(float lo, float hi) {
  if (BF) {
    __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&t);
  }
  __half2 t = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&t);
}
// d += a . b, one warp, m16n8k16, f32 accumulate
template <bool BF>
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  if (BF)
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  else
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t word_of(const uint4 &v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

// DH = 64 or 128.  Lane = (g, c) = (lane / 4, lane % 4), the row / column-pair coordinates of the MMA fragments.
//   QK^T:  A[m = q row][k]: a0 = Q[g][slots 2c,2c+1], a2 = Q[g][slots 2c+8,2c+9]; rows 8..15 (a1, a3) are zero.
//          B[k][n = key g of the tile]: b0, b1 = the same slots of K[key g].  Slot s of k-step t is column
//          32*(t/2) + 8c + 4*(t%2) + {0,1 | 2,3}: the four words of ONE 128-bit load of K[key g][32*(t/2) + 8c ..] are
//          (b0, b1) of k-step t = even and (b0, b1) of k-step t + 1.
//          C: c0, c1 = S[row g][keys 2c, 2c+1 of the tile].
//   PV:    B[k = key][n = row g] = P[g][keys 2c,2c+1 | 2c+8,2c+9] = the exponentiated c0, c1 of key tiles 0 and 1.
//          A[m][k = key]: m-tile i of half hh, m = g -> dh 64hh + 8g + 2i, m = g + 8 -> dh 64hh + 8g + 2i + 1: word i
//          of the 128-bit loads V[key][64hh + 8g ..] of keys 2c, 2c+1 (a0 = low halves, a1 = high halves) and of keys
//          2c+8, 2c+9 (a2, a3).
//          C: c0, c1 = O[rows 2c, 2c+1][dh of m = g], c2, c3 = the same rows at dh + 1.
template <int DH, bool BF, int WARPS, bool CLUSTER>
__global__ void __launch_bounds__(WARPS * 32, CLUSTER ? 1 : 2) attention_decode_kernel(const __grid_constant__ DecodeArgs a) {
  constexpr int ROWS = DEC_MAX_ROWS;
  constexpr int CH = DH / 32;   // 128-bit loads per K row per lane
  constexpr int HH = DH / 64;   // 64-wide halves of a V row
  constexpr int DEC_THREADS = WARPS * 32, DEC_WARPS = WARPS, DEC_KEYS_PER_STEP = WARPS * 16;
  __shared__ __align__(16) unsigned short q_s[ROWS][DH];
  __shared__ float red_m[DEC_WARPS][ROWS], red_l[DEC_WARPS][ROWS];
  extern __shared__ __align__(16) float red_o_raw[];  // [WARPS][ROWS][DH]: 32 or 64 KB
  float (*red_o)[ROWS][DH] = reinterpret_cast<float (*)[ROWS][DH]>(red_o_raw);
  __shared__ unsigned int s_last;
  const int kvh = blockIdx.x, split = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int off = a.att - a.seq;

  const int k_begin = split * a.keys_per_split, k_end = min(a.att, k_begin + a.keys_per_split);
  const unsigned short *kbase = a.k + (long long)kvh * a.k_sh + c * 8;
  const unsigned short *vbase = a.v + (long long)kvh * a.v_sh + g * 8;

  uint4 kq[2][CH], vq[HH][4];
  // keys kb .. kb+15 of this warp; rows past k_end re-read the last row and are masked
  auto issue_k = [&](int kb) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int key = min(kb + j * 8 + g, k_end - 1);
      const unsigned short *kr = kbase + (long long)key * a.k_ss;
#pragma unroll
      for (int ch = 0; ch < CH; ++ch) kq[j][ch] = __ldcs(reinterpret_cast<const uint4 *>(kr + ch * 32));
    }
  };
  auto issue_v = [&](int kb) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int key = min(kb + 2 * c + (j & 1) + (j >> 1) * 8, k_end - 1);
      const unsigned short *vr = vbase + (long long)key * a.v_ss;
#pragma unroll
      for (int hh = 0; hh < HH; ++hh) vq[hh][j] = __ldcs(reinterpret_cast<const uint4 *>(vr + hh * 64));
    }
  };
  int kb = k_begin + warp * 16;
  if (kb < k_end) {  // in flight while q is staged
    issue_k(kb);
    issue_v(kb);
  }

  if (a.q_vec) {
    // one warp fetches q with 128-bit loads (lane (g, c): row g, columns 32 ch + 8 c ..): four loads per lane instead of
    // a scalar loop over the rows
    if (warp == 0) {
      uint4 qv[CH];
#pragma unroll
      for (int ch = 0; ch < CH; ++ch) {
        qv[ch] = make_uint4(0, 0, 0, 0);
        if (g < a.rows) {
          const int gi = g / a.seq, si = g - gi * a.seq;
          qv[ch] = *reinterpret_cast<const uint4 *>(a.q + (long long)(kvh * a.group + gi) * a.q_sh + (long long)si * a.q_ss + ch * 32 + c * 8);
        }
      }
#pragma unroll
      for (int ch = 0; ch < CH; ++ch) *reinterpret_cast<uint4 *>(&q_s[g][ch * 32 + c * 8]) = qv[ch];
    }
  } else {
    for (int i = threadIdx.x; i < ROWS * DH; i += DEC_THREADS) {
      const int r = i / DH, col = i - r * DH;
      unsigned short val = 0;
      if (r < a.rows) {
        const int gi = r / a.seq, si = r - gi * a.seq;
        val = a.q[(long long)(kvh * a.group + gi) * a.q_sh + (long long)si * a.q_ss + col];
      }
      q_s[r][col] = val;
    }
  }
  __syncthreads();
  // q fragments are re-read from shared memory at every use (volatile: hoisting them would cost 16 registers that the
  // loads in flight need)
  const volatile uint4 *q_frag = reinterpret_cast<const volatile uint4 *>(&q_s[g][c * 8]);
  const int lim = g < a.rows ? (a.causal ? min(a.att - 1, off + g % a.seq) : a.att - 1) : -1;  // last visible key of row g

  float m = -INFINITY, l = 0.f;   // row g: m is common to the four lanes of a row, l is this lane's share
  float o[HH][4][4];
#pragma unroll
  for (int hh = 0; hh < HH; ++hh)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[hh][i][e] = 0.f;

  for (; kb < k_end; kb += DEC_KEYS_PER_STEP) {  // warp-uniform
    float s[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
#pragma unroll
      for (int ch = 0; ch < CH; ++ch) {
        const uint32_t q0 = q_frag[ch * 4].x, q1 = q_frag[ch * 4].y, q2 = q_frag[ch * 4].z, q3 = q_frag[ch * 4].w;
        mma16816<BF>(s[j], q0, 0u, q1, 0u, kq[j][ch].x, kq[j][ch].y);
        mma16816<BF>(s[j], q2, 0u, q3, 0u, kq[j][ch].z, kq[j][ch].w);
      }
    }
    const bool more = kb + DEC_KEYS_PER_STEP < k_end;
    if (more) issue_k(kb + DEC_KEYS_PER_STEP);  // the K registers are free again
    // scores of row g at keys kb + 8j + 2c + {0,1}
    float sv[4];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int key = kb + j * 8 + 2 * c + e;
        const float x = (key < k_end && key <= lim) ? s[j][e] * a.scale_log2 : -INFINITY;
        sv[j * 2 + e] = x;
        mx = fmaxf(mx, x);
      }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m, mx);
    const float m_use = m_new == -INFINITY ? 0.f : m_new;
    const float alpha = ex2f(m - m_use);
    float p[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) p[e] = ex2f(sv[e] - m_use);
    l = fmaf(l, alpha, (p[0] + p[1]) + (p[2] + p[3]));
    m = m_new;
    const uint32_t pb0 = dec_pack<BF>(p[0], p[1]), pb1 = dec_pack<BF>(p[2], p[3]);
    // the accumulators of this lane belong to rows 2c and 2c + 1
    const float al0 = __shfl_sync(0xffffffffu, alpha, (2 * c) << 2), al1 = __shfl_sync(0xffffffffu, alpha, (2 * c + 1) << 2);
#pragma unroll
    for (int hh = 0; hh < HH; ++hh)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        o[hh][i][0] *= al0;
        o[hh][i][1] *= al1;
        o[hh][i][2] *= al0;
        o[hh][i][3] *= al1;
        const uint32_t w0 = word_of(vq[hh][0], i), w1 = word_of(vq[hh][1], i), w2 = word_of(vq[hh][2], i), w3 = word_of(vq[hh][3], i);
        mma16816<BF>(o[hh][i], __byte_perm(w0, w1, 0x5410), __byte_perm(w0, w1, 0x7632), __byte_perm(w2, w3, 0x5410),
                     __byte_perm(w2, w3, 0x7632), pb0, pb1);
      }
    if (more) issue_v(kb + DEC_KEYS_PER_STEP);
  }

  // the 8 warps meet in shared memory: common max per row, rescaled sums
  l += __shfl_xor_sync(0xffffffffu, l, 1);
  l += __shfl_xor_sync(0xffffffffu, l, 2);
  if (c == 0) red_m[warp][g] = m;
  __syncthreads();
  {
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) mm = fmaxf(mm, red_m[w][g]);
    if (c == 0) red_l[warp][g] = m == -INFINITY ? 0.f : l * ex2f(m - mm);
    float sc[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int r = 2 * c + e;
      float mr = -INFINITY;
#pragma unroll
      for (int w = 0; w < DEC_WARPS; ++w) mr = fmaxf(mr, red_m[w][r]);
      const float mw = red_m[warp][r];
      sc[e] = mw == -INFINITY ? 0.f : ex2f(mw - mr);
    }
#pragma unroll
    for (int hh = 0; hh < HH; ++hh)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int col = hh * 64 + g * 8 + 2 * i;
        *reinterpret_cast<float2 *>(&red_o[warp][2 * c][col]) = make_float2(o[hh][i][0] * sc[0], o[hh][i][2] * sc[0]);
        *reinterpret_cast<float2 *>(&red_o[warp][2 * c + 1][col]) = make_float2(o[hh][i][1] * sc[1], o[hh][i][3] * sc[1]);
      }
  }
  __syncthreads();
  if constexpr (CLUSTER) {
    // the CTA's own (m, l, o) into the first warp's slots, then the 8 CTAs of the kv head meet in distributed shared memory:
    // CTA k of the cluster finishes output elements [k, k+1) * rows * DH / 8
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    for (int i = threadIdx.x; i < a.rows * DH; i += DEC_THREADS) {
      const int r = i / DH, col = i - r * DH;
      float acc = 0.f;
#pragma unroll
      for (int w = 0; w < DEC_WARPS; ++w) acc += red_o[w][r][col];
      red_o[0][r][col] = acc;  // slot (0, r, col) is read by this thread only
    }
    float ls = 0.f, mm = -INFINITY;
    if (threadIdx.x < ROWS) {
#pragma unroll
      for (int w = 0; w < DEC_WARPS; ++w) {
        ls += red_l[w][threadIdx.x];
        mm = fmaxf(mm, red_m[w][threadIdx.x]);
      }
    }
    __syncthreads();
    if (threadIdx.x < ROWS) {
      red_m[0][threadIdx.x] = mm;
      red_l[0][threadIdx.x] = ls;
    }
    cluster.sync();
    const int nclus = a.splits;  // 8 or 16 CTAs per kv head
    const int share = (a.rows * DH + nclus - 1) / nclus;
    const int first = (int)cluster.block_rank() * share;
    for (int i = first + threadIdx.x; i < min(first + share, a.rows * DH); i += DEC_THREADS) {
      const int r = i / DH, col = i - r * DH;
      float ms[DEC_CLUSTER_MAX], lsum[DEC_CLUSTER_MAX], ov[DEC_CLUSTER_MAX];
#pragma unroll
      for (int q = 0; q < DEC_CLUSTER_MAX; ++q) {  // all remote loads in flight together
        ms[q] = -INFINITY;
        lsum[q] = 0.f;
        ov[q] = 0.f;
        if (q < nclus) {
          ms[q] = *cluster.map_shared_rank(&red_m[0][r], q);
          lsum[q] = *cluster.map_shared_rank(&red_l[0][r], q);
          ov[q] = *cluster.map_shared_rank(&red_o[0][r][col], q);
        }
      }
      float top = -INFINITY;
#pragma unroll
      for (int q = 0; q < DEC_CLUSTER_MAX; ++q) top = fmaxf(top, ms[q]);
      float den = 0.f, num = 0.f;
#pragma unroll
      for (int q = 0; q < DEC_CLUSTER_MAX; ++q) {  // split order
        const float w = ms[q] == -INFINITY ? 0.f : ex2f(ms[q] - top);
        den = fmaf(lsum[q], w, den);
        num = fmaf(ov[q], w, num);
      }
      const int gi = r / a.seq, si = r - gi * a.seq;
      a.o[(long long)(kvh * a.group + gi) * a.o_sh + (long long)si * a.o_ss + col] = dec_from_f32<BF>(num / den);
    }
    cluster.sync();  // nobody leaves while its shared memory may still be read
    return;
  }
  // park (m, l, o) of this split
  float *part = a.partial + (((long long)kvh * a.splits + split) * ROWS) * (DH + 2);
  for (int i = threadIdx.x; i < a.rows * DH; i += DEC_THREADS) {
    const int r = i / DH, col = i - r * DH;
    float acc = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) acc += red_o[w][r][col];
    part[r * (DH + 2) + 2 + col] = acc;
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
    const int r = i / DH, col = i - r * DH;
    const float *colp = pall + (long long)r * (DH + 2) + 2 + col;
    float num = 0.f;
    int sp = 0;
    for (; sp + 16 <= a.splits; sp += 16) {  // sixteen loads in flight
      float v[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) v[u] = __ldcg(colp + (long long)(sp + u) * ROWS * (DH + 2));
#pragma unroll
      for (int u = 0; u < 16; ++u) num = fmaf(v[u], w_s[r][sp + u], num);
    }
    for (; sp + 4 <= a.splits; sp += 4) {
      float v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = __ldcg(colp + (long long)(sp + u) * ROWS * (DH + 2));
#pragma unroll
      for (int u = 0; u < 4; ++u) num = fmaf(v[u], w_s[r][sp + u], num);
    }
    for (; sp < a.splits; ++sp) num = fmaf(__ldcg(colp + (long long)sp * ROWS * (DH + 2)), w_s[r][sp], num);
    const int gi = r / a.seq, si = r - gi * a.seq;
    a.o[(long long)(kvh * a.group + gi) * a.o_sh + (long long)si * a.o_ss + col] = dec_from_f32<BF>(num / den_s[r]);
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
  const bool bf16 = a->q_layout.dt == OPS_DT_BF16;
  g.q_sh = sq[0] / 2; g.q_ss = sq[1] / 2;
  g.k_sh = sk[0] / 2; g.k_ss = sk[1] / 2;
  g.v_sh = sv[0] / 2; g.v_ss = sv[1] / 2;
  g.o_sh = so[0] / 2; g.o_ss = so[1] / 2;
  g.group = (int)(nh / nkvh);
  g.seq = (int)seq;
  g.att = (int)att;
  g.rows = g.group * g.seq;
  g.causal = a->mask == OPS_MASK_CAUSAL;
  g.q_vec = aligned(a->q_base, 16) && sq[0] % 16 == 0 && sq[1] % 16 == 0;
  const float inv_sqrt = 1.f / sqrtf((float)dh);
  const float alpha = bf16 ? __bfloat162float(__float2bfloat16_rn(inv_sqrt)) : __half2float(__float2half_rn(inv_sqrt));
  g.scale_log2 = alpha * 1.4426950408889634f;
  g.partial = scratch;
  g.tickets = tickets;
  cudaSetDevice(base.device);
  // Enough kv heads to put 8 CTAs each on a third of the machine or more, and a key range a CTA walks in a few steps:
  // the splits of a head meet in cluster shared memory.
  const usz cluster_step = (usz)DEC_CLUSTER_WARPS * 16;
  if (nkvh * DEC_CLUSTER * 3 >= (usz)base.sm_count && nkvh <= 4096 && att <= (usz)DEC_CLUSTER * cluster_step * 16) {
    const usz steps = (att + cluster_step - 1) / cluster_step;
    void (*kern)(const DecodeArgs) = dh == 128 ? (bf16 ? attention_decode_kernel<128, true, DEC_CLUSTER_WARPS, true> : attention_decode_kernel<128, false, DEC_CLUSTER_WARPS, true>)
                                               : (bf16 ? attention_decode_kernel<64, true, DEC_CLUSTER_WARPS, true> : attention_decode_kernel<64, false, DEC_CLUSTER_WARPS, true>);
    const size_t smem = (size_t)DEC_CLUSTER_WARPS * DEC_MAX_ROWS * dh * sizeof(float);
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(OPS_EXECUTION_FAILED, "attention(decode): cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    // (16 CTAs per kv head, a non-portable cluster size, was measured: 19.0 us against 14.3 for 4096 keys — few GPCs can
    // hold a cluster of sixteen 512-thread CTAs, so the clusters queue)
    g.keys_per_split = (int)(((steps + DEC_CLUSTER - 1) / DEC_CLUSTER) * cluster_step);
    g.splits = DEC_CLUSTER;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)nkvh, DEC_CLUSTER);
    cfg.blockDim = dim3(DEC_CLUSTER_WARPS * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 1;
    attr.val.clusterDim.y = DEC_CLUSTER;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, kern, g);
    if (e != cudaSuccess) return fail(OPS_EXECUTION_FAILED, "attention(decode): cluster launch failed: %s", cudaGetErrorString(e));
    return check_launch("attention(decode, cluster)");
  }
  // about two 256-thread CTAs per SM (both resident: every load of the launch is in flight at once), whole 128-key
  // steps per CTA, and partials that fit the scratch buffer; few splits keep the merge by the last CTA of a kv head short
  constexpr usz split_step = (usz)DEC_WARPS * 16;
  usz splits = (2 * (usz)base.sm_count + nkvh - 1) / nkvh;
  splits = std::min<usz>(splits, (att + split_step - 1) / split_step);
  splits = std::min<usz>(splits, DEC_MAX_SPLITS);
  const usz per_split = nkvh * (usz)DEC_MAX_ROWS * (dh + 2) * sizeof(float);
  splits = std::min<usz>(splits, attention_decode_scratch_bytes() / per_split);
  if (splits < 1) return fail(OPS_SHAPE_NOT_SUPPORT, "attention: too many kv heads for the decode scratch buffer");
  const usz steps = (att + split_step - 1) / split_step;
  g.keys_per_split = (int)((steps + splits - 1) / splits) * (int)split_step;
  g.splits = (int)((att + g.keys_per_split - 1) / g.keys_per_split);
  dim3 grid((unsigned)nkvh, (unsigned)g.splits);
  const size_t smem = (size_t)DEC_WARPS * DEC_MAX_ROWS * dh * sizeof(float);
  if (dh == 128) {
    if (bf16) attention_decode_kernel<128, true, DEC_WARPS, false><<<grid, DEC_WARPS * 32, smem, s>>>(g);
    else attention_decode_kernel<128, false, DEC_WARPS, false><<<grid, DEC_WARPS * 32, smem, s>>>(g);
  } else {
    if (bf16) attention_decode_kernel<64, true, DEC_WARPS, false><<<grid, DEC_WARPS * 32, smem, s>>>(g);
    else attention_decode_kernel<64, false, DEC_WARPS, false><<<grid, DEC_WARPS * 32, smem, s>>>(g);
  }
  return check_launch("attention(decode)");
}

}  // namespace ops
