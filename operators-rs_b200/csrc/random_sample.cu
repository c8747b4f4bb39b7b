// random_sample.cu — one row of logits -> one KVPair {idx, val-bits}: argmax or seeded top-k/top-p sampling.
//
// Replaces random_sample::common_cpu::Operator (operators/src/random_sample/common_cpu/mod.rs:41-99;
// argmax :102-109, random :111-144; ordering operators/src/random_sample/kv_pair.rs:62-84); argument
// checks follow Args::meta (operators/src/random_sample/args.rs:92-120).
//
// Both modes are bit-exact restatements of serial CPU loops:
//   argmax  — the LAST index among equal maxima (Iterator::max_by keeps the later element on Equal, and
//             an unordered compare counts as Equal).  A 64-bit (ordered value, index) atomicMax gives
//             exactly that; rows holding NaN take a serial finish that replays the CPU loop.
//   random  — all n logits are ordered by (value desc, index asc); c0 = 1, c_i = fl32(c_{i-1} +
//             exp((x_i - x_0)/t)) serially; the answer is the first i with c_i >= seed*min(c_{k-1},
//             c_{n-1}*top_p) and val = the logit type's rounding of c_i.  Terms below 2^-25 can never
//             change a sum that is >= 1, so only the prefix with (x - max)/t >= -16.7 is ordered (stable
//             4-bit LSD radix sort inside one CTA).  The serial f32 sum is reproduced exactly in
//             parallel: while the sum stays inside one binade its ulp u is constant, so each add is the
//             integer update S += round_half_even(e/u); a tie's outcome depends only on the parity of
//             S, so every element is a pair (delta if S even, delta if S odd) and pairs compose
//             associatively -> block-wide scan.  The add that crosses into the next binade is done by
//             one hardware f32 add, then the scan restarts with the doubled ulp.
//             exp is evaluated in double and rounded to f32 (= the correctly rounded f32 exp).
//
// HBM-bound on paper (rows * n * sizeof(T) bytes read); argmax splits a row over several CTAs.
#include <cooperative_groups.h>

#include <mutex>

#include "common.h"
#include "device_utils.cuh"

namespace ops {

struct KVPair {
  uint32_t idx;
  uint32_t val;
};

// Monotone map float -> u32 with -0 folded onto +0 (they compare Equal in the CPU loop).
__device__ __forceinline__ uint32_t ordered_key(float v) {
  uint32_t u = __float_as_uint(v + 0.f);  // -0 + 0 = +0
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_to_float(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

template <class T> __device__ __forceinline__ uint32_t raw_bits(T v);
template <> __device__ __forceinline__ uint32_t raw_bits<__half>(__half v) { return (uint32_t)__half_as_ushort(v); }
template <> __device__ __forceinline__ uint32_t raw_bits<float>(float v) { return __float_as_uint(v); }
template <> __device__ __forceinline__ uint32_t raw_bits<__nv_bfloat16>(__nv_bfloat16 v) { return (uint32_t)__bfloat16_as_ushort(v); }

// ------------------------------------------------------------------------------------------------
// argmax
// ------------------------------------------------------------------------------------------------
struct ArgmaxScratch {          // per row; all zero between launches (the CTA that finishes a row puts it back)
  unsigned long long best;      // (ordered value << 32) | index, over non-NaN elements
  unsigned int last_nan;        // 1 + index of the last NaN, 0 if none
  unsigned int tickets;         // CTAs of this row that have finished
};

// Scans elements [begin, end) of row x with the whole CTA.  Thread 0 returns the CTA's best (ordered value << 32 | index
// over non-NaN elements, 0 if none) and 1 + the index of its last NaN (0 if none).
template <class T>
__device__ __forceinline__ void argmax_scan(const T *x, int begin, int end, unsigned long long *s_best, unsigned int *s_nan,
                                            unsigned long long &best_out, unsigned int &nan_out) {
  // per thread: running (value, index) with ">=" so that the later of equal values wins (+0 and -0 compare equal);
  // NaNs are skipped here and only remembered (their last index), see argmax_finish
  float best_v = -INFINITY;
  int best_i = -1;
  unsigned int last_nan = 0;
  auto visit = [&](float v, int i) {
    if (v >= best_v) {
      best_v = v;
      best_i = i;
    } else if (v != v) {
      last_nan = (unsigned)i + 1u;  // indices only grow within a thread
    }
  };
  const bool vec_ok = (((uintptr_t)x) & 15) == 0;
  constexpr int PER = 16 / (int)sizeof(T);
  constexpr int UN = 8;
  if (vec_ok) {
    const int vend = begin + ((end - begin) / PER) * PER;
    const int step = blockDim.x * PER;
    // batches of eight independent 128-bit loads per thread, every load of a batch issued before the first value is used
    // (a CTA's share of a row is a few vectors per thread: one trip to DRAM instead of one per vector)
    for (int i0 = begin + threadIdx.x * PER; i0 < vend; i0 += UN * step) {
      uint4 raw[UN];
#pragma unroll
      for (int u = 0; u < UN; ++u)
        if (i0 + u * step < vend) raw[u] = ld_stream_16(x + i0 + u * step);
#pragma unroll
      for (int u = 0; u < UN; ++u) {
        if (i0 + u * step < vend) {
          const T *e = reinterpret_cast<const T *>(&raw[u]);
#pragma unroll
          for (int j = 0; j < PER; ++j) visit(to_f32(e[j]), i0 + u * step + j);
        }
      }
    }
    for (int k = vend + threadIdx.x; k < end; k += blockDim.x) visit(to_f32(x[k]), k);
  } else {
    for (int k = begin + threadIdx.x; k < end; k += blockDim.x) visit(to_f32(x[k]), k);
  }
  unsigned long long best = best_i < 0 ? 0ull : (((unsigned long long)ordered_key(best_v) << 32) | (unsigned)best_i);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
    last_nan = max(last_nan, __shfl_xor_sync(0xffffffffu, last_nan, o));
  }
  if ((threadIdx.x & 31) == 0) {
    s_best[threadIdx.x >> 5] = best;
    s_nan[threadIdx.x >> 5] = last_nan;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) {
      best = max(best, s_best[w]);
      last_nan = max(last_nan, s_nan[w]);
    }
  }
  best_out = best;
  nan_out = last_nan;
}

// One thread: the row's answer from its best non-NaN element and its last NaN.
template <class T>
__device__ __forceinline__ void argmax_finish(const T *x, int n, unsigned long long gbest, unsigned int gnan, KVPair *out) {
  unsigned int idx;
  if (gnan == 0) {
    idx = (unsigned int)(gbest & 0xffffffffull);
  } else {
    // replay of the CPU loop from the last NaN on: the NaN is taken, then replaced by whatever follows
    idx = gnan - 1;
    for (unsigned int i = gnan; i < (unsigned)n; ++i)
      if (!(to_f32(x[idx]) > to_f32(x[i]))) idx = i;
  }
  out->idx = idx;
  out->val = raw_bits(x[idx]);
}

__device__ __forceinline__ void argmax_chunk(int n, int split, int part, int &begin, int &end) {
  int chunk = (n + split - 1) / split;
  chunk = (chunk + 7) & ~7;
  begin = min(n, part * chunk);
  end = min(n, begin + chunk);
}

// A row split over `split` CTAs that meet in global memory (any split, any number of rows).
template <class T>
__global__ void __launch_bounds__(256) argmax_kernel(const T *__restrict__ logits, long long row_stride, int n, int split,
                                                     ArgmaxScratch *scratch, KVPair *out) {
  __shared__ unsigned long long s_best[8];
  __shared__ unsigned int s_nan[8];
  const int row = blockIdx.x / split, part = blockIdx.x - row * split;
  const T *x = byte_off(logits, (long long)row * row_stride);
  int begin, end;
  argmax_chunk(n, split, part, begin, end);
  unsigned long long best;
  unsigned int last_nan;
  argmax_scan(x, begin, end, s_best, s_nan, best, last_nan);
  if (threadIdx.x != 0) return;
  ArgmaxScratch *sc = scratch + row;
  if (best) atomicMax(&sc->best, best);
  if (last_nan) atomicMax(&sc->last_nan, last_nan);
  __threadfence();
  if (atomicAdd(&sc->tickets, 1u) != (unsigned)(split - 1)) return;
  // last CTA of the row: finish
  __threadfence();
  const unsigned long long gbest = atomicExch(&sc->best, 0ull);  // read and leave zero for the next launch
  const unsigned int gnan = atomicExch(&sc->last_nan, 0u);
  sc->tickets = 0;
  argmax_finish(x, n, gbest, gnan, out + row);
}

// A row split over the eight CTAs of one thread-block cluster that meet in distributed shared memory: no scratch, no
// atomics, no fences — the launch of a decode step's single row costs one pass over the row plus a cluster barrier.
constexpr int ARGMAX_CLUSTER = 8;
template <class T>
__global__ void __cluster_dims__(ARGMAX_CLUSTER, 1, 1) __launch_bounds__(256)
    argmax_cluster_kernel(const T *__restrict__ logits, long long row_stride, int n, KVPair *out) {
  namespace cg = cooperative_groups;
  __shared__ unsigned long long s_best[8];
  __shared__ unsigned int s_nan[8];
  __shared__ unsigned long long c_best;  // this CTA's result, read by the cluster's first CTA
  __shared__ unsigned int c_nan;
  cg::cluster_group cluster = cg::this_cluster();
  const int row = blockIdx.x / ARGMAX_CLUSTER, part = (int)cluster.block_rank();
  const T *x = byte_off(logits, (long long)row * row_stride);
  int begin, end;
  argmax_chunk(n, ARGMAX_CLUSTER, part, begin, end);
  unsigned long long best;
  unsigned int last_nan;
  argmax_scan(x, begin, end, s_best, s_nan, best, last_nan);
  if (threadIdx.x == 0) {
    c_best = best;
    c_nan = last_nan;
  }
  cluster.sync();
  if (part == 0 && threadIdx.x < 32) {
    unsigned long long b = 0;
    unsigned int nn = 0;
    if (threadIdx.x < ARGMAX_CLUSTER) {
      b = *cluster.map_shared_rank(&c_best, threadIdx.x);
      nn = *cluster.map_shared_rank(&c_nan, threadIdx.x);
    }
#pragma unroll
    for (int o = ARGMAX_CLUSTER / 2; o > 0; o >>= 1) {
      b = max(b, __shfl_xor_sync(0xffffffffu, b, o));
      nn = max(nn, __shfl_xor_sync(0xffffffffu, nn, o));
    }
    if (threadIdx.x == 0) argmax_finish(x, n, b, nn, out + row);
  }
  cluster.sync();  // nobody leaves while its shared memory may still be read
}

// ------------------------------------------------------------------------------------------------
// seeded sampling: one CTA of 1024 threads per row
// ------------------------------------------------------------------------------------------------
constexpr int SAMPLE_THREADS = 1024;
constexpr int SCAN_ITEMS = 4;
constexpr float KEEP_ARG = -16.7f;  // exp(-16.7) < 2^-24: anything below can never move a sum >= 1

struct Pair64 {  // increment of the integer sum if it is even (d0) / odd (d1) before this span
  long long d0, d1;
};
__device__ __forceinline__ Pair64 compose(Pair64 f, Pair64 g) {  // f first, then g
  Pair64 h;
  h.d0 = f.d0 + ((f.d0 & 1) ? g.d1 : g.d0);
  h.d1 = f.d1 + (((1 + f.d1) & 1) ? g.d1 : g.d0);
  return h;
}
__device__ __forceinline__ Pair64 shfl_up_pair(Pair64 p, int o) {
  Pair64 r;
  r.d0 = __shfl_up_sync(0xffffffffu, p.d0, o);
  r.d1 = __shfl_up_sync(0xffffffffu, p.d1, o);
  return r;
}

struct SampleShared {
  int warp_cnt[16][32];
  int warp_off[16][32];
  int digit_base[16];
  int tile_cnt[16];
  int hist[16];
  int scan_i[33];
  float red_f[33];
  Pair64 scan_p[33];
  int kept;
  int i0;
  int cross;
  int tail_flag;
  float s;
};

// exclusive block scan of one int per thread; returns the exclusive prefix, *total = block total
__device__ __forceinline__ int block_excl_scan(int v, int *scratch, int *total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  __syncthreads();
  if (lane == 31) scratch[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int w = scratch[lane];
    int winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int t = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += t;
    }
    scratch[lane] = winc - w;
    if (lane == 31) scratch[32] = winc;
  }
  __syncthreads();
  *total = scratch[32];
  return scratch[warp] + inc - v;
}

template <class T> struct KeyBits;
template <> struct KeyBits<__half> { static constexpr int bits = 16; };
template <> struct KeyBits<float> { static constexpr int bits = 32; };
template <> struct KeyBits<__nv_bfloat16> { static constexpr int bits = 16; };

// sort key: ascending key = descending value.  f16 rows get 16-bit keys (4 radix passes), f32 rows 32-bit.
template <class T> __device__ __forceinline__ uint32_t sort_key(T v);
template <> __device__ __forceinline__ uint32_t sort_key<float>(float v) { return ~ordered_key(v); }
template <> __device__ __forceinline__ uint32_t sort_key<__half>(__half v) {
  uint32_t h = __half_as_ushort(v);
  if ((h & 0x7fffu) == 0) h = 0;  // -0 -> +0
  const uint32_t k = (h & 0x8000u) ? (~h & 0xffffu) : (h | 0x8000u);
  return (~k) & 0xffffu;
}
template <> __device__ __forceinline__ uint32_t sort_key<__nv_bfloat16>(__nv_bfloat16 v) {  // same sign-magnitude layout as f16
  uint32_t h = __bfloat16_as_ushort(v);
  if ((h & 0x7fffu) == 0) h = 0;  // -0 -> +0
  const uint32_t k = (h & 0x8000u) ? (~h & 0xffffu) : (h | 0x8000u);
  return (~k) & 0xffffu;
}
template <class T> __device__ __forceinline__ float key_value(uint32_t key);
template <> __device__ __forceinline__ float key_value<__nv_bfloat16>(uint32_t key) {
  const uint32_t k = (~key) & 0xffffu;
  const uint32_t h = (k & 0x8000u) ? (k & 0x7fffu) : (~k & 0xffffu);
  return __uint_as_float(h << 16);
}
template <> __device__ __forceinline__ float key_value<float>(uint32_t key) { return key_to_float(~key); }
template <> __device__ __forceinline__ float key_value<__half>(uint32_t key) {
  const uint32_t k = (~key) & 0xffffu;
  const uint32_t h = (k & 0x8000u) ? (k & 0x7fffu) : (~k & 0xffffu);
  return __half2float(__ushort_as_half((unsigned short)h));
}

// maximum of a row over the whole CTA (NaNs ignored), 128-bit loads when the row is 16-byte aligned
template <class T>
__device__ __forceinline__ float sample_row_max(const T *__restrict__ x, int n, float *red) {
  const int tid = threadIdx.x;
  float mx = -INFINITY;
  {
    constexpr int PER = 16 / (int)sizeof(T);
    if ((((uintptr_t)x) & 15) == 0) {
      const int nv = n / PER;
      int v = tid;
      for (; v + 3 * SAMPLE_THREADS < nv; v += 4 * SAMPLE_THREADS) {  // four 128-bit loads in flight per thread
        uint4 raw[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) raw[u] = ld_global_16(reinterpret_cast<const uint4 *>(x) + v + u * SAMPLE_THREADS);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const T *e = reinterpret_cast<const T *>(&raw[u]);
#pragma unroll
          for (int j = 0; j < PER; ++j) mx = fmaxf(mx, to_f32(e[j]));
        }
      }
      for (; v < nv; v += SAMPLE_THREADS) {
        const uint4 raw = ld_global_16(reinterpret_cast<const uint4 *>(x) + v);
        const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
        for (int j = 0; j < PER; ++j) mx = fmaxf(mx, to_f32(e[j]));
      }
      for (int i = nv * PER + tid; i < n; i += SAMPLE_THREADS) mx = fmaxf(mx, to_f32(x[i]));
    } else {
      for (int i = tid; i < n; i += SAMPLE_THREADS) mx = fmaxf(mx, to_f32(x[i]));
    }
  }
  return block_max(mx, red);
}

// The sampling path for any element type and row length: order the kept prefix with a stable radix sort in the row's
// workspace, then the exact prefix sums.  One CTA of SAMPLE_THREADS threads per row.
template <class T>
__device__ void sample_sort_body(SampleShared &sh, const T *__restrict__ x, int n, float temperature, float top_p, unsigned long long top_k,
                                 float seed, char *__restrict__ ws_row, KVPair *out_row) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint2 *buf_a = reinterpret_cast<uint2 *>(ws_row);
  uint2 *buf_b = buf_a + n;

  // ---- S1: row maximum --------------------------------------------------------------------------
  const float mx = sample_row_max(x, n, sh.red_f);

  // ---- S2: keep (in index order) every element that can still move the sum ----------------------
  if (tid == 0) sh.kept = 0;
  __syncthreads();
  for (int base = 0; base < n; base += SAMPLE_THREADS * 8) {
    const int i0 = base + tid * 8;
    uint32_t keys[8];
    int cnt = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int i = i0 + j;
      bool keep = false;
      if (i < n) {
        const T v = x[i];
        const float arg = __fdiv_rn(__fsub_rn(to_f32(v), mx), temperature);
        keep = arg >= KEEP_ARG;
        keys[j] = sort_key(v);
      }
      if (!keep) keys[j] = 0xffffffffu;  // marker; real keys of kept f32 elements are never all-ones (that is -NaN)
      cnt += keep;
    }
    int total;
    int off = block_excl_scan(cnt, sh.scan_i, &total) + sh.kept;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (keys[j] != 0xffffffffu) buf_a[off++] = make_uint2(keys[j], (uint32_t)(i0 + j));
    __syncthreads();
    if (tid == 0) sh.kept += total;
    __syncthreads();
  }
  const int M = sh.kept;
  if (M == 0) {
    // Nothing can be ordered: every logit is -inf, or one is +inf or NaN poisons x - max.  The CPU loop panics or
    // produces garbage on such rows; here the row gets a defined answer without touching the scratch: the argmax rule
    // (last index of the maximum) with the cumulative mass 1 as value.
    if (tid == 0) {
      int best = 0;
      for (int i = 1; i < n; ++i)
        if (!(to_f32(x[best]) > to_f32(x[i]))) best = i;
      out_row->idx = (unsigned)best;
      out_row->val = raw_bits(from_f32<T>(1.f));
    }
    return;
  }

  // ---- S3: stable LSD radix sort of the kept prefix, 4 bits per pass ----------------------------
  uint2 *src = buf_a, *dst = buf_b;
  for (int shift = 0; shift < KeyBits<T>::bits; shift += 4) {
    if (tid < 16) sh.hist[tid] = 0;
    __syncthreads();
    for (int base = 0; base < M; base += SAMPLE_THREADS) {
      const int i = base + tid;
      const int d = i < M ? (int)((src[i].x >> shift) & 15u) : 16;
      const unsigned m = __match_any_sync(0xffffffffu, d);
      if (d < 16 && (m & ((1u << lane) - 1u)) == 0) atomicAdd(&sh.hist[d], __popc(m));
    }
    __syncthreads();
    if (tid == 0) {
      int acc = 0;
      for (int d = 0; d < 16; ++d) {
        sh.digit_base[d] = acc;
        acc += sh.hist[d];
      }
    }
    __syncthreads();
    for (int base = 0; base < M; base += SAMPLE_THREADS) {
      const int i = base + tid;
      uint2 el = make_uint2(0, 0);
      int d = 16;
      if (i < M) {
        el = src[i];
        d = (int)((el.x >> shift) & 15u);
      }
      const unsigned m = __match_any_sync(0xffffffffu, d);
      const int rank = __popc(m & ((1u << lane) - 1u));
      if (tid < 512) (&sh.warp_cnt[0][0])[tid] = 0;
      __syncthreads();
      if (d < 16 && rank == 0) sh.warp_cnt[d][warp] = __popc(m);
      __syncthreads();
      if (warp < 16) {  // warp d scans the 32 per-warp counts of digit d
        const int v = sh.warp_cnt[warp][lane];
        int inc = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          int t = __shfl_up_sync(0xffffffffu, inc, o);
          if (lane >= o) inc += t;
        }
        sh.warp_off[warp][lane] = inc - v;
        if (lane == 31) sh.tile_cnt[warp] = inc;
      }
      __syncthreads();
      if (d < 16) dst[sh.digit_base[d] + sh.warp_off[d][warp] + rank] = el;
      __syncthreads();
      if (tid < 16) sh.digit_base[tid] += sh.tile_cnt[tid];
      __syncthreads();
    }
    uint2 *t = src;
    src = dst;
    dst = t;
  }
  // sorted (key, idx) pairs are in `src`; `dst` is free: first M floats = e_i, next M floats = c_i
  float *E = reinterpret_cast<float *>(dst);
  float *C = E + n;

  // ---- S4: e_i, then the exact serial prefix sums -----------------------------------------------
  const float x0 = key_value<T>(src[0].x);
  for (int i = tid; i < M; i += SAMPLE_THREADS) {
    const float arg = __fdiv_rn(__fsub_rn(key_value<T>(src[i].x), x0), temperature);
    E[i] = (float)exp((double)arg);
  }
  if (tid == 0) {
    C[0] = 1.f;
    sh.i0 = 1;
    sh.s = 1.f;
  }
  __syncthreads();

  while (true) {
    const int i0 = sh.i0;
    if (i0 >= M) break;
    const float s = sh.s;
    const int ex = (int)((__float_as_uint(s) >> 23) & 0xffu) - 127;   // s in [2^ex, 2^(ex+1))
    const float u = __uint_as_float((uint32_t)(ex - 23 + 127) << 23);  // ulp of s
    const float u_inv = __uint_as_float((uint32_t)(23 - ex + 127) << 23);
    long long S = (long long)(s * u_inv);  // exact integer in [2^23, 2^24)
    bool restarted = false;
    for (int base = i0; base < M; base += SAMPLE_THREADS * SCAN_ITEMS) {
      __syncthreads();
      if (tid == 0) {
        sh.cross = 0x7fffffff;
        sh.tail_flag = (E[base] * u_inv < 0.5f) ? 1 : 0;  // sorted descending: nothing later can contribute
      }
      __syncthreads();
      if (sh.tail_flag) {
        const float cs = (float)S * u;
        for (int i = base + tid; i < M; i += SAMPLE_THREADS) C[i] = cs;
        __syncthreads();
        if (tid == 0) {
          sh.i0 = M;
          sh.s = cs;
        }
        restarted = true;
        break;
      }
      // per-thread span of SCAN_ITEMS consecutive elements
      long long q[SCAN_ITEMS];
      bool tie[SCAN_ITEMS];
      Pair64 mine{0, 0};
      const int first = base + tid * SCAN_ITEMS;
#pragma unroll
      for (int j = 0; j < SCAN_ITEMS; ++j) {
        const int i = first + j;
        q[j] = 0;
        tie[j] = false;
        if (i < M) {
          const float a = E[i] * u_inv;  // exact power-of-two scaling, a < 2^24
          const float fl = floorf(a);
          const float r = a - fl;        // exact
          q[j] = (long long)fl + (r > 0.5f ? 1 : 0);
          tie[j] = r == 0.5f;
        }
        Pair64 el;
        if (tie[j]) {
          el.d0 = q[j] + (q[j] & 1);
          el.d1 = q[j] + ((q[j] & 1) ^ 1);
        } else {
          el.d0 = el.d1 = q[j];
        }
        mine = compose(mine, el);
      }
      // inclusive scan of `mine` across the block (compose is associative, not commutative)
      Pair64 inc = mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        Pair64 t = shfl_up_pair(inc, o);
        if (lane >= o) inc = compose(t, inc);
      }
      if (lane == 31) sh.scan_p[warp] = inc;
      __syncthreads();
      if (warp == 0) {
        Pair64 w = sh.scan_p[lane];
        Pair64 winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          Pair64 t = shfl_up_pair(winc, o);
          if (lane >= o) winc = compose(t, winc);
        }
        // exclusive prefix of warps: shift down by one
        Pair64 wex = shfl_up_pair(winc, 1);
        if (lane == 0) wex = Pair64{0, 0};
        sh.scan_p[lane] = wex;
        if (lane == 31) sh.scan_p[32] = winc;
      }
      __syncthreads();
      Pair64 lane_ex = shfl_up_pair(inc, 1);  // exclusive within the warp
      if (lane == 0) lane_ex = Pair64{0, 0};
      const Pair64 before = compose(sh.scan_p[warp], lane_ex);
      long long St = S + ((S & 1) ? before.d1 : before.d0);
#pragma unroll
      for (int j = 0; j < SCAN_ITEMS; ++j) {
        const int i = first + j;
        if (i < M) {
          St += q[j] + ((tie[j] && ((St + q[j]) & 1)) ? 1 : 0);
          if (St >= (1ll << 24)) atomicMin(&sh.cross, i);
          else C[i] = (float)St * u;
        }
      }
      __syncthreads();
      if (sh.cross != 0x7fffffff) {
        if (tid == 0) {
          const int ic = sh.cross;
          const float c_new = __fadd_rn(C[ic - 1], E[ic]);  // the one add that changes binade: hardware f32
          C[ic] = c_new;
          sh.s = c_new;
          sh.i0 = ic + 1;
        }
        restarted = true;
        break;
      }
      const Pair64 tot = sh.scan_p[32];
      S += (S & 1) ? tot.d1 : tot.d0;
    }
    __syncthreads();
    if (!restarted) {
      if (tid == 0) {
        sh.i0 = M;
        sh.s = (float)S * u;
      }
      __syncthreads();
    }
  }
  __syncthreads();

  // ---- S5: threshold and pick -------------------------------------------------------------------
  const unsigned long long kk = (top_k < (unsigned long long)n ? top_k : (unsigned long long)n) - 1ull;
  const float pk = C[kk < (unsigned long long)M ? (int)kk : M - 1];
  const float pp = __fmul_rn(C[M - 1], top_p);
  const float plimit = __fmul_rn(seed, fminf(pk, pp));
  int below = 0;
  for (int i = tid; i < M; i += SAMPLE_THREADS) below += (C[i] < plimit) ? 1 : 0;
  int total;
  block_excl_scan(below, sh.scan_i, &total);
  if (tid == 0) {
    const int j = total < M ? total : M - 1;
    out_row->idx = src[j].y;
    out_row->val = raw_bits(from_f32<T>(C[j]));
  }
}

template <class T>
__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(const T *__restrict__ logits, long long row_stride, int n,
                                                                float temperature, float top_p, unsigned long long top_k,
                                                                const float *__restrict__ seeds, float seed_scalar,
                                                                char *__restrict__ ws, long long ws_row_bytes, KVPair *out) {
  __shared__ SampleShared sh;
  const int row = blockIdx.x;
  sample_sort_body<T>(sh, byte_off(logits, (long long)row * row_stride), n, temperature, top_p, top_k, seeds ? seeds[row] : seed_scalar,
                      ws + (long long)row * ws_row_bytes, out + row);
}

// ------------------------------------------------------------------------------------------------
// seeded sampling of 16-bit logits: counting sort by value
//
// The cumulative sums of the CPU loop depend on the sorted VALUES only, and a 16-bit type has at most 65536 of them.  So
// instead of ordering tens of thousands of (value, index) pairs, the kept prefix is counted into a histogram over the value
// keys (shared memory, one bin per representable value below the row maximum), and the serial f32 prefix sum is
// reproduced over RUNS of equal terms: inside one binade of the running sum every add of the term e is the integer update
// S += round_half_even(e / ulp), so m adds of the same e have a closed form (the first add may depend on the parity of S,
// after a tie the sum is even and the increment is constant), runs compose associatively as (delta if S even, delta if S
// odd) pairs, and one block-wide scan gives the sum after every bin.  A run that reaches the next binade is finished by
// its owner thread (one hardware add per binade it crosses), then the scan restarts behind it with the doubled ulp.
// The index of the chosen element — the r-th of its value in index order — is found by one more pass over the row.
// Rows whose kept values span more bins than fit fall back to the sort above.
// ------------------------------------------------------------------------------------------------
constexpr int HIST_BPT = 49;  // bins per thread: odd, so that the threads' walks over their bins hit 32 different shared-memory banks
constexpr int HIST_BINS = HIST_BPT * SAMPLE_THREADS;  // 50176 value bins: 196 KB of counters
constexpr long long BINADE = 1ll << 24;

struct HistState {
  int thr;        // last kept bin (-1: nothing can be ordered)
  int overflow;   // a kept element lies beyond the histogram
  int i0;         // first bin whose sums are not final yet
  long long rem0; // adds of bin i0 still to do
  float s;        // running sum in front of bin i0
  int cross;      // first bin in which the running sum leaves its binade
  int q_bin;      // answers of the position / threshold queries
  long long q_off;
  float q_val;
};

__device__ __forceinline__ void split_term(float e, float u_inv, long long &q, bool &tie) {
  const float a = e * u_inv;  // exact power-of-two scaling, a < 2^24
  const float fl = floorf(a);
  const float r = a - fl;     // exact
  q = (long long)fl + (r > 0.5f ? 1 : 0);
  tie = r == 0.5f;
}
// m >= 1 adds of the same term inside one binade, as (increment if the integer sum is even, increment if it is odd)
__device__ __forceinline__ Pair64 run_pair(long long q, bool tie, long long m) {
  const long long d2 = q + ((tie && (q & 1)) ? 1 : 0);  // after a tie add the sum is even: from then on the increment is constant
  Pair64 p;
  p.d0 = q + ((tie && (q & 1)) ? 1 : 0) + (m - 1) * d2;
  p.d1 = q + ((tie && !(q & 1)) ? 1 : 0) + (m - 1) * d2;
  return p;
}
// c after m serial f32 adds of e (c >= 1, 0 < e <= 1): closed form inside a binade, one hardware add at each crossing
__device__ float advance_sum(float c, float e, long long m) {
  while (m > 0) {
    const int ex = (int)((__float_as_uint(c) >> 23) & 0xffu) - 127;
    const float u = __uint_as_float((uint32_t)(ex - 23 + 127) << 23);
    const float u_inv = __uint_as_float((uint32_t)(23 - ex + 127) << 23);
    long long S = (long long)(c * u_inv);
    long long q;
    bool tie;
    split_term(e, u_inv, q, tie);
    const long long d1 = q + ((tie && ((S + q) & 1)) ? 1 : 0);
    if (S + d1 >= BINADE) {  // this very add reaches the next binade
      c = __fadd_rn(c, e);
      --m;
      continue;
    }
    S += d1;
    --m;
    if (m > 0) {
      const long long d2 = q + ((tie && (q & 1)) ? 1 : 0);
      if (d2 == 0) {
        m = 0;  // nothing moves the sum any more
      } else {
        const long long room = (BINADE - 1 - S) / d2;  // further adds that stay inside the binade
        const long long k = m < room ? m : room;
        S += k * d2;
        m -= k;
      }
    }
    c = (float)S * u;
    if (m > 0) {
      c = __fadd_rn(c, e);
      --m;
    }
  }
  return c;
}

template <class T>
__global__ void __launch_bounds__(SAMPLE_THREADS) sample_hist_kernel(const T *__restrict__ logits, long long row_stride, int n,
                                                                     float temperature, float top_p, unsigned long long top_k,
                                                                     const float *__restrict__ seeds, float seed_scalar,
                                                                     char *__restrict__ ws, long long ws_row_bytes, KVPair *out) {
  extern __shared__ __align__(16) unsigned int hist[];  // HIST_BINS counters
  __shared__ SampleShared sh;
  __shared__ HistState hs;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int row = blockIdx.x;
  const T *x = byte_off(logits, (long long)row * row_stride);
  char *ws_row = ws + (long long)row * ws_row_bytes;
  float *E = reinterpret_cast<float *>(ws_row);  // term of every non-empty bin
  float *C = E + HIST_BINS;                      // running sum behind every bin
  const float seed = seeds ? seeds[row] : seed_scalar;
  KVPair *out_row = out + row;
  constexpr int PER = 16 / (int)sizeof(T);
  const bool vec_ok = (((uintptr_t)x) & 15) == 0;

  // ---- S1: row maximum, kept range in key space ------------------------------------------------------
  const float mx = sample_row_max(x, n, sh.red_f);
  for (int i = tid; i < HIST_BINS / 4; i += SAMPLE_THREADS) reinterpret_cast<uint4 *>(hist)[i] = make_uint4(0, 0, 0, 0);
  const uint32_t key0 = sort_key<T>(from_f32<T>(mx));
  if (tid == 0) {
    // keep(v) = (v - max) / t >= KEEP_ARG is monotone in v, so the kept values are the keys key0 .. key0 + thr
    auto keep = [&](uint32_t key) { return __fdiv_rn(__fsub_rn(key_value<T>(key), mx), temperature) >= KEEP_ARG; };
    int thr = -1;
    if (keep(key0)) {
      const uint32_t kinf = sort_key<T>(from_f32<T>(-INFINITY));
      int lo = 0, hi = (int)(kinf - key0) + 1;  // keep(lo) holds, keep(hi) does not (-inf is never kept)
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (keep(key0 + (uint32_t)mid)) lo = mid;
        else hi = mid;
      }
      thr = lo;
    }
    hs.thr = thr;
    hs.overflow = 0;
  }
  __syncthreads();
  const int thr = hs.thr;
  if (thr < 0) {
    // Nothing can be ordered (every logit -inf, or a +inf makes x - max NaN): the argmax rule with the mass 1 as value,
    // as in the sort path.
    if (tid == 0) {
      int best = 0;
      for (int i = 1; i < n; ++i)
        if (!(to_f32(x[best]) > to_f32(x[i]))) best = i;
      out_row->idx = (unsigned)best;
      out_row->val = raw_bits(from_f32<T>(1.f));
    }
    return;
  }
  const int nbins = thr + 1 < HIST_BINS ? thr + 1 : HIST_BINS;

  // ---- S2: histogram of the kept values -----------------------------------------------------------------
  {
    auto count = [&](T v) {
      const uint32_t b = sort_key<T>(v) - key0;  // wraps for values above the maximum (NaN patterns): never kept
      if (b <= (uint32_t)thr) {
        if (b < (uint32_t)HIST_BINS) atomicAdd(&hist[b], 1u);
        else hs.overflow = 1;
      }
    };
    if (vec_ok) {
      const int nv = n / PER;
      for (int v0 = tid; v0 < nv; v0 += 4 * SAMPLE_THREADS) {
        uint4 raw[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (v0 + u * SAMPLE_THREADS < nv) raw[u] = ld_global_16(reinterpret_cast<const uint4 *>(x) + v0 + u * SAMPLE_THREADS);
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (v0 + u * SAMPLE_THREADS < nv) {
            const T *e = reinterpret_cast<const T *>(&raw[u]);
#pragma unroll
            for (int j = 0; j < PER; ++j) count(e[j]);
          }
      }
      for (int i = nv * PER + tid; i < n; i += SAMPLE_THREADS) count(x[i]);
    } else {
      for (int i = tid; i < n; i += SAMPLE_THREADS) count(x[i]);
    }
  }
  __syncthreads();
  if (hs.overflow) {  // kept values beyond the histogram: order them the long way
    __syncthreads();
    sample_sort_body<T>(sh, x, n, temperature, top_p, top_k, seed, ws_row, out_row);
    return;
  }

  // ---- S3: the term of every non-empty bin; adds per thread ------------------------------------------
  const float x0 = key_value<T>(key0);
  for (int b = tid; b < nbins; b += SAMPLE_THREADS)
    if (hist[b]) E[b] = (float)exp((double)__fdiv_rn(__fsub_rn(key_value<T>(key0 + (uint32_t)b), x0), temperature));
  const int b_lo = tid * HIST_BPT, b_hi = min(nbins, b_lo + HIST_BPT);
  // the maximum itself is position 0 with sum 1; every other kept element is one add
  auto adds_of = [&](int b) -> long long { return (long long)hist[b] - (b == 0 ? 1 : 0); };
  int own = 0;
  for (int b = b_lo; b < b_hi; ++b) own += (int)adds_of(b);
  int total_adds;
  const int pre = block_excl_scan(own, sh.scan_i, &total_adds);  // (also makes E visible to the whole CTA)
  const long long M = (long long)total_adds + 1;                 // kept elements

  // ---- S4: the running sum behind every bin ----------------------------------------------------------
  if (tid == 0) {
    hs.i0 = 0;
    hs.rem0 = adds_of(0);
    hs.s = 1.f;
  }
  __syncthreads();
  // Passes over a WINDOW of bins behind i0, k bins per thread (thread t: bins i0 + k t ..): the sum doubles from binade to
  // binade, so the first binades end after a handful of bins — a pass that walked all 50176 bins to find a crossing a
  // few bins ahead cost 17 us, and there are 5-12 of them per row.  The window starts at one bin per thread and grows
  // (odd k: the threads' reads of `hist` stay on different banks) each time a window ends without leaving the binade.
  int k = 1;
  while (true) {
    const int i0 = hs.i0;
    if (i0 >= nbins) break;
    const long long rem0 = hs.rem0;
    const float s = hs.s;
    const int ex = (int)((__float_as_uint(s) >> 23) & 0xffu) - 127;   // s in [2^ex, 2^(ex+1))
    const float u = __uint_as_float((uint32_t)(ex - 23 + 127) << 23);  // ulp of s
    const float u_inv = __uint_as_float((uint32_t)(23 - ex + 127) << 23);
    const long long S = (long long)(s * u_inv);  // exact integer in [2^23, 2^24)
    if (tid == 0) hs.cross = 0x7fffffff;
    const int win_end = (int)min((long long)nbins, (long long)i0 + (long long)SAMPLE_THREADS * k);
    const int w_lo = (int)min((long long)win_end, (long long)i0 + (long long)tid * k), w_hi = min(win_end, w_lo + k);
    // this thread's bins as one composed pair
    Pair64 mine{0, 0};
    for (int b = w_lo; b < w_hi; ++b) {
      const long long m = b == i0 ? rem0 : (long long)hist[b];
      if (m > 0) {
        long long q;
        bool tie;
        split_term(E[b], u_inv, q, tie);
        mine = compose(mine, run_pair(q, tie, m));
      }
    }
    // exclusive scan of the threads' pairs (compose is associative, not commutative)
    Pair64 inc = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      Pair64 t = shfl_up_pair(inc, o);
      if (lane >= o) inc = compose(t, inc);
    }
    __syncthreads();  // scan_p may still be read from the previous pass; hs.cross is reset
    if (lane == 31) sh.scan_p[warp] = inc;
    __syncthreads();
    if (warp == 0) {
      Pair64 w = sh.scan_p[lane];
      Pair64 winc = w;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        Pair64 t = shfl_up_pair(winc, o);
        if (lane >= o) winc = compose(t, winc);
      }
      Pair64 wex = shfl_up_pair(winc, 1);
      if (lane == 0) wex = Pair64{0, 0};
      sh.scan_p[lane] = wex;
    }
    __syncthreads();
    Pair64 lane_ex = shfl_up_pair(inc, 1);
    if (lane == 0) lane_ex = Pair64{0, 0};
    const Pair64 before = compose(sh.scan_p[warp], lane_ex);
    long long St = S + ((S & 1) ? before.d1 : before.d0);
    // second walk: the sum behind every bin, until a run leaves the binade
    long long cross_S = 0;
    for (int b = w_lo; b < w_hi; ++b) {
      const long long m = b == i0 ? rem0 : (long long)hist[b];
      if (m > 0) {
        long long q;
        bool tie;
        split_term(E[b], u_inv, q, tie);
        const Pair64 p = run_pair(q, tie, m);
        const long long S2 = St + ((St & 1) ? p.d1 : p.d0);
        if (S2 >= BINADE) {
          atomicMin(&hs.cross, b);
          cross_S = St;
          break;  // everything behind is recomputed with the next ulp
        }
        St = S2;
      }
      C[b] = (float)St * u;
    }
    __syncthreads();
    const int cross = hs.cross;
    if (cross == 0x7fffffff) {
      // the whole window lies inside this binade: go on behind it with the same ulp and a wider window
      if (win_end >= nbins) break;
      if (w_hi == win_end && w_lo < w_hi) {  // the thread that owns the window's last bin knows the sum behind it
        hs.s = (float)St * u;
        hs.i0 = win_end;
        hs.rem0 = (long long)hist[win_end];
      }
      k = k >= HIST_BPT ? HIST_BPT : min(HIST_BPT, 2 * k + 1);
      __syncthreads();
      continue;
    }
    if (cross >= w_lo && cross < w_hi) {
      // the owner finishes the crossing run through as many binades as it takes (its own walk stopped exactly there,
      // and no earlier bin crossed, so cross_S is the true sum in front of the run)
      const long long m = cross == i0 ? rem0 : (long long)hist[cross];
      const float c = advance_sum((float)cross_S * u, E[cross], m);
      C[cross] = c;
      hs.s = c;
      hs.i0 = cross + 1;
      hs.rem0 = cross + 1 < nbins ? (long long)hist[cross + 1] : 0;
    }
    __syncthreads();
  }
  __syncthreads();

  // ---- S5: thresholds, the chosen position, its value and index ---------------------------------------
  const float total = C[nbins - 1];
  // sum at sorted position `pos` (block-wide): 1 at position 0, else the (pos)-th add
  auto locate = [&](long long pos) {
    if (pos == 0) {
      if (tid == 0) {
        hs.q_bin = 0;
        hs.q_off = -1;  // the maximum itself: rank 0 of bin 0
        hs.q_val = 1.f;
      }
    } else {
      const long long t = pos - 1;
      if (t >= pre && t < (long long)pre + own) {
        long long running = pre;
        for (int b = b_lo; b < b_hi; ++b) {
          const long long m = adds_of(b);
          if (t < running + m) {
            const long long a = t - running;
            hs.q_bin = b;
            hs.q_off = a;
            hs.q_val = advance_sum(b == 0 ? 1.f : C[b - 1], E[b], a + 1);
            break;
          }
          running += m;
        }
      }
    }
    __syncthreads();
  };
  const unsigned long long kk = (top_k < (unsigned long long)n ? top_k : (unsigned long long)n) - 1ull;
  float pk = total;
  if (kk < (unsigned long long)M) {
    locate((long long)kk);
    pk = hs.q_val;
  }
  __syncthreads();
  const float pp = __fmul_rn(total, top_p);
  const float plimit = __fmul_rn(seed, fminf(pk, pp));
  if (1.f >= plimit) {
    locate(0);
  } else {
    int below = 0;
    for (int b = b_lo; b < b_hi; ++b) below += (C[b] < plimit) ? 1 : 0;
    int bstar;
    block_excl_scan(below, sh.scan_i, &bstar);  // sums behind the bins never decrease: the count is the first bin that reaches plimit
    if (bstar >= nbins) {
      locate(M - 1);  // (cannot happen for seed < 1: the last sum is the largest)
    } else {
      if (bstar >= b_lo && bstar < b_hi) {
        const long long m = adds_of(bstar);
        const float c_before = bstar == 0 ? 1.f : C[bstar - 1], e = E[bstar];
        long long lo = -1, hi = m - 1;  // sum after add hi reaches plimit, after add lo it does not
        while (hi - lo > 1) {
          const long long mid = (lo + hi) >> 1;
          if (advance_sum(c_before, e, mid + 1) >= plimit) hi = mid;
          else lo = mid;
        }
        hs.q_bin = bstar;
        hs.q_off = hi;
        hs.q_val = advance_sum(c_before, e, hi + 1);
      }
      __syncthreads();
    }
  }
  const int q_bin = hs.q_bin;
  const long long rank = hs.q_off + (q_bin == 0 ? 1 : 0);  // among the elements of that value, in index order
  const float cj = hs.q_val;
  const uint32_t want = key0 + (uint32_t)q_bin;
  // the rank-th element with that value: every thread counts a contiguous piece of the row, then the piece holding it is walked
  int piece = (n + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
  piece = (piece + 7) & ~7;
  const long long p_lo = (long long)tid * piece;
  const int i_lo = p_lo < n ? (int)p_lo : n, i_hi = p_lo + piece < n ? (int)(p_lo + piece) : n;
  int hits = 0;
  if (vec_ok) {
    int i = i_lo;
    for (; i + PER <= i_hi; i += PER) {
      const uint4 raw = ld_global_16(x + i);
      const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
      for (int j = 0; j < PER; ++j) hits += sort_key<T>(e[j]) == want ? 1 : 0;
    }
    for (; i < i_hi; ++i) hits += sort_key<T>(x[i]) == want ? 1 : 0;
  } else {
    for (int i = i_lo; i < i_hi; ++i) hits += sort_key<T>(x[i]) == want ? 1 : 0;
  }
  int all_hits;
  const int before_me = block_excl_scan(hits, sh.scan_i, &all_hits);
  if (rank >= before_me && rank < (long long)before_me + hits) {
    long long left = rank - before_me;
    for (int i = i_lo; i < i_hi; ++i)
      if (sort_key<T>(x[i]) == want && left-- == 0) {
        out_row->idx = (unsigned)i;
        out_row->val = raw_bits(from_f32<T>(cj));
        break;
      }
  }
}

struct SampleMeta {
  uint32_t dt;
  usz n;
};

static int sample_meta(const ops_random_sample_args *a, SampleMeta *m) {
  if (a->kv_pair.dt != OPS_DT_KVPAIR) return fail(OPS_TYPE_NOT_SUPPORT, "output must be KVpair");
  m->dt = a->logits.dt;
  if (dt_size(m->dt) > 4 || dt_size(m->dt) == 0) return fail(OPS_TYPE_NOT_SUPPORT, "element too large");
  if (a->indices.dt != OPS_DT_U32) return fail(OPS_TYPE_NOT_SUPPORT, "indices must be u32");
  if (a->logits.ndim != 1) return fail(OPS_RANK_NOT_SUPPORT, "logits.ndim = %u, 1 expected", a->logits.ndim);
  if (a->indices.ndim != 1) return fail(OPS_RANK_NOT_SUPPORT, "indices.ndim = %u, 1 expected", a->indices.ndim);
  m->n = a->logits.shape[0];
  return OPS_OK;
}

static inline bool is_argmax(const ops_sample_args &c) { return c.temperature == 0.f || c.top_k == 1; }

static usz argmax_ws(usz rows) { return rows * sizeof(ArgmaxScratch); }
static usz sample_ws_row(usz n) { return (n * 16 + 255) / 256 * 256; }

// `arg_scratch`: `arg_rows` zeroed, self-resetting ArgmaxScratch records that belong to the caller's handle (or to the
// built-in array of the allocation-free entry); rows beyond that take theirs from the workspace, cleared on the stream.
static int launch_rows(const OpBase &base, uint32_t dt, usz rows, usz n, const void *logits, isz row_stride, void *kv_out,
                       const ops_sample_args &cfg, const float *seeds_dev, float seed_scalar, void *ws, usz ws_len,
                       ArgmaxScratch *arg_scratch, usz arg_rows, cudaStream_t s) {
  if (dt != OPS_DT_F16 && dt != OPS_DT_BF16 && dt != OPS_DT_F32) return fail(OPS_TYPE_NOT_SUPPORT, "random_sample: f16, bf16 or f32 logits expected");
  if (rows == 0) return OPS_OK;
  if (n == 0) return fail(OPS_SHAPE_NOT_SUPPORT, "random_sample: empty logits");
  if (n > 0x7fffffffu / 16 || rows > 0x7fffffu) return fail(OPS_SHAPE_NOT_SUPPORT, "random_sample: shape too large");
  if (!logits || !kv_out) return fail(OPS_DYNAMIC_NOT_SUPPORT, "random_sample: null base pointer at launch");
  cudaSetDevice(base.device);
  if (is_argmax(cfg)) {
    const usz row_bytes = n * dt_size(dt);
    // Few rows of ordinary length (a decode step: one row of a 128k vocabulary): one cluster of eight CTAs per row
    if (rows * ARGMAX_CLUSTER <= 4 * (usz)base.sm_count && row_bytes >= ((usz)32 << 10) && row_bytes <= ((usz)4 << 20)) {
      const unsigned grid = (unsigned)(rows * ARGMAX_CLUSTER);
      if (dt == OPS_DT_F16)
        argmax_cluster_kernel<__half><<<grid, 256, 0, s>>>((const __half *)logits, row_stride, (int)n, (KVPair *)kv_out);
      else if (dt == OPS_DT_BF16)
        argmax_cluster_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16 *)logits, row_stride, (int)n, (KVPair *)kv_out);
      else
        argmax_cluster_kernel<float><<<grid, 256, 0, s>>>((const float *)logits, row_stride, (int)n, (KVPair *)kv_out);
      return check_launch("random_sample(argmax, cluster)");
    }
    ArgmaxScratch *scratch = arg_scratch;
    if (!scratch || rows > arg_rows) {
      const usz need = argmax_ws(rows);
      if (ws_len < need || !ws) return need_workspace(need);
      cudaMemsetAsync(ws, 0, need, s);
      scratch = (ArgmaxScratch *)ws;
    }
    // split a row over several CTAs when there are few rows; keep >= 8 KiB per CTA
    usz split = (8 * (usz)base.sm_count + rows - 1) / rows;  // ~8 CTAs per SM keep enough loads in flight
    const usz max_split = (row_bytes + 8191) / 8192;
    if (split > max_split) split = max_split;
    if (split < 1) split = 1;
    const unsigned grid = (unsigned)(rows * split);
    if (dt == OPS_DT_F16)
      argmax_kernel<__half><<<grid, 256, 0, s>>>((const __half *)logits, row_stride, (int)n, (int)split, scratch, (KVPair *)kv_out);
    else if (dt == OPS_DT_BF16)
      argmax_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16 *)logits, row_stride, (int)n, (int)split, scratch, (KVPair *)kv_out);
    else
      argmax_kernel<float><<<grid, 256, 0, s>>>((const float *)logits, row_stride, (int)n, (int)split, scratch, (KVPair *)kv_out);
    return check_launch("random_sample(argmax)");
  }
  if (!(cfg.temperature > 0.f)) return fail(OPS_ARGS_NOT_SUPPORT, "random_sample: temperature must be >= 0");
  if (cfg.top_k == 0 || !(cfg.top_p > 0.f)) return fail(OPS_ARGS_NOT_SUPPORT, "random_sample: top_k and top_p must be positive");
  const usz per_row = sample_ws_row(n);
  const usz need = per_row * rows;
  if (ws_len < need || !ws) return need_workspace(need);
  if (!aligned(ws, 16)) return fail(OPS_ARGS_NOT_SUPPORT, "random_sample: workspace must be 16-byte aligned");
  const float top_p = cfg.top_p > 1.f ? 1.f : cfg.top_p;
  // 16-bit logits in rows long enough for their workspace to hold the per-bin arrays take the counting-sort kernel
  const bool hist_path = dt != OPS_DT_F32 && per_row >= (usz)HIST_BINS * 2 * sizeof(float);
  if (hist_path) {
    constexpr int smem = HIST_BINS * (int)sizeof(unsigned int);
    static bool attr_set[2][64];  // [type][device]: the opt-in to 196 KB of dynamic shared memory, once per device
    const int ti = dt == OPS_DT_F16 ? 0 : 1, di = base.device & 63;
    if (!attr_set[ti][di]) {
      cudaError_t e = ti == 0 ? cudaFuncSetAttribute(sample_hist_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)
                              : cudaFuncSetAttribute(sample_hist_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return fail(OPS_EXECUTION_FAILED, "random_sample: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
      attr_set[ti][di] = true;
    }
    if (dt == OPS_DT_F16)
      sample_hist_kernel<__half><<<(unsigned)rows, SAMPLE_THREADS, smem, s>>>((const __half *)logits, row_stride, (int)n, cfg.temperature, top_p,
                                                                              (unsigned long long)cfg.top_k, seeds_dev, seed_scalar, (char *)ws,
                                                                              (long long)per_row, (KVPair *)kv_out);
    else
      sample_hist_kernel<__nv_bfloat16><<<(unsigned)rows, SAMPLE_THREADS, smem, s>>>((const __nv_bfloat16 *)logits, row_stride, (int)n, cfg.temperature,
                                                                                     top_p, (unsigned long long)cfg.top_k, seeds_dev, seed_scalar,
                                                                                     (char *)ws, (long long)per_row, (KVPair *)kv_out);
    return check_launch("random_sample(sample, counting sort)");
  }
#define OPS_SAMPLE_SORT(T)                                                                                                                   \
  sample_kernel<T><<<(unsigned)rows, SAMPLE_THREADS, 0, s>>>((const T *)logits, row_stride, (int)n, cfg.temperature, top_p, (unsigned long long)cfg.top_k, \
                                                            seeds_dev, seed_scalar, (char *)ws, (long long)per_row, (KVPair *)kv_out)
  if (dt == OPS_DT_F16) OPS_SAMPLE_SORT(__half);
  else if (dt == OPS_DT_BF16) OPS_SAMPLE_SORT(__nv_bfloat16);
  else OPS_SAMPLE_SORT(float);
#undef OPS_SAMPLE_SORT
  return check_launch("random_sample(sample)");
}

}  // namespace ops

using namespace ops;

// The handle owns the few bytes per row the argmax kernel meets in (zeroed once, left at zero by every launch), so the
// argmax path needs neither a workspace nor a clearing launch.  One stream at a time per handle.
constexpr usz ARGMAX_OWN_ROWS = 4096;
struct ops_random_sample {
  ops::OpBase base;
  ops::ArgmaxScratch *arg_scratch;
};

namespace ops {
static int noalloc_scratch(int device, void **out);
}

OPS_API int ops_random_sample_create(int device, ops_random_sample **out) {
  if (!out) return fail(OPS_ARGS_NOT_SUPPORT, "null out pointer");
  ops_random_sample *h = new ops_random_sample();
  h->arg_scratch = nullptr;
  int rc = init_base(&h->base, device);
  if (rc != OPS_OK) {
    delete h;
    return rc;
  }
  cudaSetDevice(device);
  if (cudaMalloc(&h->arg_scratch, ARGMAX_OWN_ROWS * sizeof(ArgmaxScratch)) != cudaSuccess ||
      cudaMemset(h->arg_scratch, 0, ARGMAX_OWN_ROWS * sizeof(ArgmaxScratch)) != cudaSuccess) {
    cudaGetLastError();  // without it the argmax path takes its records from the caller's workspace
    if (h->arg_scratch) cudaFree(h->arg_scratch);
    h->arg_scratch = nullptr;
  }
  // Look up the built-in scratch array of the allocation-free entry point now, so that its launches — the first one
  // included — do no driver work.  A failure here is not fatal: that entry point tries again when it is first used.
  void *unused = nullptr;
  if (noalloc_scratch(device, &unused) != OPS_OK) cudaGetLastError();
  *out = h;
  return OPS_OK;
}

OPS_API void ops_random_sample_destroy(ops_random_sample *op) {
  if (!op) return;
  if (op->arg_scratch) {
    cudaSetDevice(op->base.device);
    cudaFree(op->arg_scratch);
  }
  delete op;
}

OPS_API int ops_sample_args_new(float temperature, float top_p, size_t top_k, ops_sample_args *out) {
  if (temperature < 0.f) return 1;
  if (top_k == 0 || top_p <= 0.f) return 2;
  out->temperature = temperature;
  out->top_p = top_p < 1.f ? top_p : 1.f;
  out->top_k = top_k;
  return 0;
}

OPS_API size_t ops_random_sample_batched_workspace(uint32_t dt, size_t rows, size_t n, const ops_sample_args *config) {
  (void)dt;
  return is_argmax(*config) ? argmax_ws(rows) : sample_ws_row(n) * rows;
}

// Like the crate's GPU operator (operators/src/random_sample/cuda/mod.rs:58-81) the reported size
// covers both modes when it fits, else the smaller one, else 0.
OPS_API int ops_random_sample_scheme(ops_random_sample *op, const ops_random_sample_args *args, size_t max_ws, size_t *ws_out) {
  (void)op;
  SampleMeta m{};
  OPS_TRY(sample_meta(args, &m));
  if (ws_out) {
    *ws_out = 0;
    if (!dyn(m.n)) {
      const usz big = sample_ws_row(m.n), small = argmax_ws(1);
      *ws_out = big <= max_ws ? big : (small <= max_ws ? small : 0);
    }
  }
  return OPS_OK;
}

OPS_API int ops_random_sample_launch(const ops_random_sample *op, const ops_random_sample_args *a, void *ws, size_t ws_len, void *stream) {
  SampleMeta m{};
  OPS_TRY(sample_meta(a, &m));
  const isz st = a->logits.strides[0];
  if (dyn(st) || st != (isz)dt_size(m.dt)) return fail(OPS_STRIDES_NOT_SUPPORT, "random_sample: logits must be contiguous");
  if (dyn(m.n)) return fail(OPS_DYNAMIC_NOT_SUPPORT, "random_sample: n must be static at launch");
  return launch_rows(op->base, m.dt, 1, m.n, a->logits_base, 0, a->kv_pair_base, a->config, nullptr, a->seed, ws, ws_len, op->arg_scratch, ARGMAX_OWN_ROWS,
                     (cudaStream_t)stream);
}

OPS_API int ops_random_sample_launch_batched(const ops_random_sample *op, uint32_t dt, size_t rows, size_t n, const void *logits_base,
                                             ptrdiff_t row_stride, void *kv_pairs_base, const ops_sample_args *config,
                                             const float *seeds_dev, void *ws, size_t ws_len, void *stream) {
  if (!is_argmax(*config) && !seeds_dev) return fail(OPS_ARGS_NOT_SUPPORT, "random_sample: batched sampling needs one seed per row");
  return launch_rows(op->base, dt, rows, n, logits_base, row_stride, kv_pairs_base, *config, seeds_dev, 0.f, ws, ws_len, op->arg_scratch, ARGMAX_OWN_ROWS,
                     (cudaStream_t)stream);
}

OPS_API int ops_random_sample_build_indices(size_t n, uint32_t *host_out) {
  for (size_t i = 0; i < n; ++i) host_out[i] = (uint32_t)i;
  return OPS_OK;
}

// ------------------------------------------------------------------------------------------------
// Allocation-free variant.
//
// Some callers cannot allocate device memory at the point where they sample: code that runs inside a
// latency-critical decode loop with the allocator locked down, plugins that are handed a stream but
// no allocator, processes whose memory budget is fixed at start-up.  For them the scratch that
// ops_random_sample_launch takes from the caller's workspace lives here instead, in one fixed array
// inside the library's device image.  Every GPU that loads the library carries the array until the
// process exits.
//
// The array is shared by every call on a device and keeps whatever the previous call left in it.  The
// argmax path meets in a record behind the sampling area that starts at zero when the library is loaded
// and that the kernel itself puts back to zero before it ends; the sampling path overwrites everything
// it later reads.  Two calls that overlap on the GPU (different
// streams, or graphs replayed concurrently) would race on the array: serialise them.
// ------------------------------------------------------------------------------------------------
namespace ops {

constexpr usz NOALLOC_MAX_LOGITS = 131072;                       // one row of up to 128 Ki logits
constexpr usz NOALLOC_SCRATCH_BYTES = NOALLOC_MAX_LOGITS * 16;   // 2 MiB: what the sampling kernel needs for such a row

constexpr usz NOALLOC_ARGMAX_BYTES = 256;                        // behind it: the argmax record (zero at load, left at zero by every call)

static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES + NOALLOC_ARGMAX_BYTES];

constexpr int NOALLOC_MAX_DEVICES = 64;
static void *g_noalloc_ptr[NOALLOC_MAX_DEVICES];  // device address of the array on each device: looked up when a handle is created there
static std::mutex g_noalloc_mutex;

// In host code `g_noalloc_scratch` is only a handle for the runtime, not an address a kernel can use:
// the device address has to be asked for, once per device, with that device current.
static int noalloc_scratch(int device, void **out) {
  if (device < 0 || device >= NOALLOC_MAX_DEVICES) return fail(OPS_ARGS_NOT_SUPPORT, "random_sample: device %d out of range", device);
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (!g_noalloc_ptr[device]) {
    cudaError_t e = cudaSetDevice(device);
    void *p = nullptr;
    if (e == cudaSuccess) e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || !p) {
      cudaGetLastError();
      return fail(OPS_EXECUTION_FAILED, "random_sample: cannot resolve the built-in scratch array on device %d: %s", device, cudaGetErrorString(e));
    }
    g_noalloc_ptr[device] = p;
  }
  *out = g_noalloc_ptr[device];
  return OPS_OK;
}

}  // namespace ops

OPS_API size_t ops_random_sample_noalloc_max_logits(void) { return NOALLOC_MAX_LOGITS; }

OPS_API int ops_random_sample_launch_noalloc(const ops_random_sample *op, const ops_random_sample_args *a, void *stream) {
  SampleMeta m{};
  OPS_TRY(sample_meta(a, &m));
  const isz st = a->logits.strides[0];
  if (dyn(st) || st != (isz)dt_size(m.dt)) return fail(OPS_STRIDES_NOT_SUPPORT, "random_sample: logits must be contiguous");
  if (dyn(m.n)) return fail(OPS_DYNAMIC_NOT_SUPPORT, "random_sample: n must be static at launch");
  if (m.n > NOALLOC_MAX_LOGITS)
    return fail(OPS_SHAPE_NOT_SUPPORT, "random_sample: %zu logits exceed the %zu the built-in scratch array is sized for; use ops_random_sample_launch with a workspace",
                m.n, NOALLOC_MAX_LOGITS);
  void *scratch = nullptr;
  OPS_TRY(noalloc_scratch(op->base.device, &scratch));
  return launch_rows(op->base, m.dt, 1, m.n, a->logits_base, 0, a->kv_pair_base, a->config, nullptr, a->seed, scratch, NOALLOC_SCRATCH_BYTES,
                     (ArgmaxScratch *)((unsigned char *)scratch + NOALLOC_SCRATCH_BYTES), 1, (cudaStream_t)stream);
}
