// attention_fused.cu — one-kernel causal attention on tcgen05 tensor cores (no score matrix in HBM).
//
// The fast path behind attention::Args (operators/src/attention/args.rs:10-24).  The crate composes
// attention from mat_mul, fused_softmax and rearrange with the [nh, seq, att] score matrix in workspace
// (operators/src/attention/operator.rs:199-275); this kernel computes the same function with online
// softmax, so HBM sees q, k, v and o once: E*(2*nh*seq*dh + 2*nkvh*att*dh) bytes for
// 4*nh*dh*sum_k(att-seq+k+1) useful flops — tensor-bound.
//
// One CTA per (head, 128-row q block), 6 warps:
//   warp 0   TMA producer: Q once, then K and V blocks of 128 keys through two-stage rings;
//   warp 1   tcgen05.mma issuer: S_j = Q K_j^T into tensor memory (two S buffers), then
//            PV_j = P_j V_j into a second pair of tensor-memory buffers — never accumulating across
//            blocks, so no rescaling ever touches tensor memory;
//   warps 2-9  softmax: two threads per q row (two warps per scheduler hide each other's latencies).
//            Both tcgen05.ld the whole S_j row for its maximum; each then turns HALF of the keys into
//            P_j (exp2 domain, f16, written to shared memory in the swizzled K-major layout the MMA
//            reads) and keeps HALF of the dh columns of O = O * alpha + PV_{j-1} in REGISTERS;
//            partial row sums meet once at the end, then 1/l and the store.
// The issue order QK_j, PV_{j-1}, QK_{j+1}, ... lets the tensor pipe work on the next block while
// the softmax warps are busy with the current one.  Every mbarrier wait is bounded.
#include <cuda.h>

#include "common.h"
#include "device_utils.cuh"
#include "internal.h"
#include "sm100_ptx.cuh"

namespace ops {

using namespace sm100;

constexpr int FA_BM = 128;       // q rows per CTA
constexpr int FA_BN = 128;       // keys per block
constexpr int FA_THREADS = 320;   // TMA warp, MMA warp, 8 softmax warps (two per scheduler)

struct FusedAttnArgs {
  unsigned short *o;     // f16 or bf16 bit patterns
  long long o_sh, o_ss;  // element strides of o: head, row (dh contiguous)
  int nh, group, seq, att;
  int causal;
  int q_blocks;
  float scale_log2;      // alpha * log2(e)
  int vec_store;
  int bf16;              // q, k, v, o are bf16 (else f16); the probabilities fed to the second MMA take the same type
  int *status;
};

template <int DH> struct FaCfg {
  static constexpr int HALVES = DH / 64;                 // 64-element (128-byte) column groups of a dh row
  static constexpr int Q_BYTES = FA_BM * DH * 2;
  static constexpr int K_BYTES = FA_BN * DH * 2;
  static constexpr int V_BYTES = FA_BN * DH * 2;
  static constexpr int P_BYTES = FA_BM * FA_BN * 2;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + Q_BYTES;          // 2 stages
  static constexpr int OFF_V = OFF_K + 2 * K_BYTES;      // 2 stages
  static constexpr int OFF_P = OFF_V + 2 * V_BYTES;      // 2 buffers
  static constexpr int OFF_BAR = OFF_P + 2 * P_BYTES;
  static constexpr int NUM_BARS = 1 + 8 + 12 + 4;        // q_full; k/v full+empty x2; s/p/pv full+empty x2; row-sum exchange x4
  static constexpr int OFF_LSUM = OFF_BAR + NUM_BARS * 8 + 16;  // [2 halves][128 rows] f32 partial row sums
  static constexpr int SMEM_BYTES = OFF_LSUM + 2 * FA_BM * 4 + 1024;
  static constexpr int TMEM_COLS = 512;                  // S0 S1 (128 each) | PV0 PV1 (128 each, DH used)
};

__device__ __forceinline__ float max3(float a, float b, float c) {  // three-input maximum (sm_100)
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
// two f32 -> one packed pair of f16 or bf16 (first value in the low half)
__device__ __forceinline__ uint32_t pack_pair(float lo, float hi, int bf) {
  if (bf) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
  }
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int DH>
__global__ void __launch_bounds__(FA_THREADS, 1)
    attention_fused_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                           const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ FusedAttnArgs g) {
  typedef FaCfg<DH> Cfg;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bar0 = base + Cfg::OFF_BAR;
  // barrier indices
  const uint32_t q_full = bar0;
  auto k_full = [&](int s) { return bar0 + 8u * (1 + s); };
  auto k_empty = [&](int s) { return bar0 + 8u * (3 + s); };
  auto v_full = [&](int s) { return bar0 + 8u * (5 + s); };
  auto v_empty = [&](int s) { return bar0 + 8u * (7 + s); };
  auto s_full = [&](int b) { return bar0 + 8u * (9 + b); };
  auto s_empty = [&](int b) { return bar0 + 8u * (11 + b); };
  auto p_full = [&](int b) { return bar0 + 8u * (13 + b); };
  auto p_empty = [&](int b) { return bar0 + 8u * (15 + b); };
  auto pv_full = [&](int b) { return bar0 + 8u * (17 + b); };
  auto pv_empty = [&](int b) { return bar0 + 8u * (19 + b); };
  auto l_bar = [&](int q) { return bar0 + 8u * (21 + q); };
  const uint32_t tmem_slot = bar0 + 8u * Cfg::NUM_BARS;
  uint32_t *tmem_slot_ptr = reinterpret_cast<uint32_t *>(base_ptr + Cfg::OFF_BAR + 8 * Cfg::NUM_BARS);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heavy (late, long) q blocks first: they set the tail of the launch
  const int qb = g.q_blocks - 1 - (int)(blockIdx.x % g.q_blocks);
  const int head = (int)(blockIdx.x / g.q_blocks);
  const int kv_head = head / g.group;
  const int q0 = qb * FA_BM;
  const int off = g.att - g.seq;  // causal row r sees keys <= off + r
  int k_end = g.att;              // exclusive bound of keys this q block can see
  if (g.causal) k_end = min(g.att, off + q0 + FA_BM);
  const int nblk = (k_end + FA_BN - 1) / FA_BN;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(k_full(s), 1);
      mbar_init(k_empty(s), 1);
      mbar_init(v_full(s), 1);
      mbar_init(v_empty(s), 1);
      mbar_init(s_full(s), 1);
      mbar_init(s_empty(s), 8);
      mbar_init(p_full(s), 8);
      mbar_init(p_empty(s), 1);
      mbar_init(pv_full(s), 1);
      mbar_init(pv_empty(s), 8);
    }
    for (int q = 0; q < 4; ++q) mbar_init(l_bar(q), 2);
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, Cfg::Q_BYTES);
#pragma unroll
      for (int h = 0; h < Cfg::HALVES; ++h) tma_load_3d(base + Cfg::OFF_Q + h * (FA_BM * 128), &tmap_q, q_full, h * 64, q0, head);
      bool ok = true;
      for (int j = 0; j < nblk && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (uint32_t)((j >> 1) & 1);
        if (!(ok = mbar_wait(k_empty(s), ph ^ 1u, g.status, 11))) break;
        mbar_arrive_expect_tx(k_full(s), Cfg::K_BYTES);
#pragma unroll
        for (int h = 0; h < Cfg::HALVES; ++h)
          tma_load_3d(base + Cfg::OFF_K + s * Cfg::K_BYTES + h * (FA_BN * 128), &tmap_k, k_full(s), h * 64, j * FA_BN, kv_head);
        if (!(ok = mbar_wait(v_empty(s), ph ^ 1u, g.status, 12))) break;
        mbar_arrive_expect_tx(v_full(s), Cfg::V_BYTES);
#pragma unroll
        for (int kg = 0; kg < FA_BN / 64; ++kg)
#pragma unroll
          for (int c = 0; c < Cfg::HALVES; ++c)
            tma_load_3d(base + Cfg::OFF_V + s * Cfg::V_BYTES + (kg * Cfg::HALVES + c) * 8192, &tmap_v, v_full(s), c * 64, j * FA_BN + kg * 64,
                        kv_head);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_qk = make_idesc_f16(FA_BM, FA_BN, 0, 0, g.bf16);
      const uint32_t idesc_pv = make_idesc_f16(FA_BM, DH, 0, 1, g.bf16);
      bool ok = mbar_wait(q_full, 0, g.status, 21);
      auto issue_pv = [&](int i) -> bool {
        const int b = i & 1;
        const uint32_t ph = (uint32_t)((i >> 1) & 1);
        if (!mbar_wait(v_full(b), ph, g.status, 22)) return false;
        if (!mbar_wait(p_full(b), ph, g.status, 23)) return false;
        if (!mbar_wait(pv_empty(b), ph ^ 1u, g.status, 24)) return false;
        tc_fence_after();
        const uint32_t pa = base + Cfg::OFF_P + b * Cfg::P_BYTES, va = base + Cfg::OFF_V + b * Cfg::V_BYTES;
        const uint32_t d = tmem_base + 256u + (uint32_t)(b * 128);
#pragma unroll
        for (int ks = 0; ks < FA_BN / 16; ++ks) {
          const uint64_t da = make_smem_desc_sw128(pa + (ks >> 2) * (FA_BM * 128) + (ks & 3) * 32, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(va + (ks >> 2) * (Cfg::HALVES * 8192) + (ks & 3) * 2048, 8192, 1024);
          umma_f16_ss(d, da, db, idesc_pv, ks != 0 ? 1u : 0u);
        }
        umma_commit(v_empty(b));
        umma_commit(p_empty(b));
        umma_commit(pv_full(b));
        return true;
      };
      for (int j = 0; j < nblk && ok; ++j) {
        const int b = j & 1;
        const uint32_t ph = (uint32_t)((j >> 1) & 1);
        if (!(ok = mbar_wait(k_full(b), ph, g.status, 25))) break;
        if (!(ok = mbar_wait(s_empty(b), ph ^ 1u, g.status, 26))) break;
        tc_fence_after();
        const uint32_t qa = base + Cfg::OFF_Q, ka = base + Cfg::OFF_K + b * Cfg::K_BYTES;
        const uint32_t d = tmem_base + (uint32_t)(b * 128);
#pragma unroll
        for (int ks = 0; ks < DH / 16; ++ks) {
          const uint64_t da = make_smem_desc_sw128(qa + (ks >> 2) * (FA_BM * 128) + (ks & 3) * 32, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(ka + (ks >> 2) * (FA_BN * 128) + (ks & 3) * 32, 16, 1024);
          umma_f16_ss(d, da, db, idesc_qk, ks != 0 ? 1u : 0u);
        }
        umma_commit(k_empty(b));
        umma_commit(s_full(b));
        if (j > 0) ok = issue_pv(j - 1);
      }
      if (ok && nblk > 0) issue_pv(nblk - 1);
    }
  } else {
    // ------------------------------------------------------------------ softmax + output (warps 2..9)
    // Two warps share each 32-row quarter of tensor memory (a warp may touch lanes 32*(warp%4)..+31 only): both scan the
    // whole S row for its maximum (so they agree on it without talking), then each takes HALF of the key columns for
    // exp/P and HALF of the dh columns of O.  Their partial row sums meet once, after the last block.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    constexpr int DHH = DH / 2;
    const int row_in_tile = quarter * 32 + lane;
    const int q_row = q0 + row_in_tile;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const int limit = g.causal ? min(g.att - 1, off + q_row) : g.att - 1;  // last key this row may see
    float o[DHH];
#pragma unroll
    for (int i = 0; i < DHH; ++i) o[i] = 0.f;
    float m = -INFINITY, l = 0.f, alpha_prev = 0.f;
    bool ok = true;

    // Tensor-memory loads are issued one ahead of the arithmetic that consumes them (tcgen05.wait::ld waits for every
    // load in flight, so the pattern is: wait, issue the next load, work on the previous one).
    auto accumulate_pv = [&](int i, float a) -> bool {
      const int b = i & 1;
      if (!mbar_wait(pv_full(b), (uint32_t)((i >> 1) & 1), g.status, 31)) return false;
      tc_fence_after();
      const uint32_t t = tmem_base + lane_addr + 256u + (uint32_t)(b * 128 + half * DHH);
      uint32_t va[32], vb[32];
      tmem_ld_32x32(t, va);
      tmem_wait_ld();
      if constexpr (DHH > 32) tmem_ld_32x32(t + 32u, vb);
#pragma unroll
      for (int e = 0; e < 32; ++e) o[e] = fmaf(o[e], a, __uint_as_float(va[e]));
      if constexpr (DHH > 32) {
        tmem_wait_ld();
#pragma unroll
        for (int e = 0; e < 32; ++e) o[32 + e] = fmaf(o[32 + e], a, __uint_as_float(vb[e]));
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(pv_empty(b));
      return true;
    };
    // maximum over 32 columns starting at key index k0 (masked beyond `limit` when the block touches the diagonal / tail)
    auto chunk_max = [&](const uint32_t (&v)[32], int k0, bool need_mask, float mx) -> float {
      if (need_mask) {
#pragma unroll
        for (int e = 0; e < 32; ++e)
          if (k0 + e <= limit) mx = fmaxf(mx, __uint_as_float(v[e]));
        return mx;
      }
      float m0 = mx, m1 = -INFINITY;
#pragma unroll
      for (int e = 0; e < 32; e += 4) {
        m0 = max3(m0, __uint_as_float(v[e]), __uint_as_float(v[e + 1]));
        m1 = max3(m1, __uint_as_float(v[e + 2]), __uint_as_float(v[e + 3]));
      }
      return fmaxf(m0, m1);
    };

    for (int j = 0; j < nblk && ok; ++j) {
      const int b = j & 1;
      const uint32_t ph = (uint32_t)((j >> 1) & 1);
      const int kv0 = j * FA_BN;
      if (!(ok = mbar_wait(s_full(b), ph, g.status, 32))) break;
      tc_fence_after();
      const uint32_t t = tmem_base + lane_addr + (uint32_t)(b * 128);
      const bool need_mask = kv0 + FA_BN - 1 > limit;
      // The whole S row is read once: the other warp's half only for the maximum, this warp's half (64 keys) stays in
      // registers for the exponentials.
      const int own = half * 64, oth = own ^ 64;
      uint32_t k0[32], k1[32], x0[32], x1[32];
      float mx = -INFINITY;
      tmem_ld_32x32(t + (uint32_t)oth, x0);
      tmem_wait_ld();
      tmem_ld_32x32(t + (uint32_t)oth + 32u, x1);
      mx = chunk_max(x0, kv0 + oth, need_mask, mx);
      tmem_wait_ld();
      tmem_ld_32x32(t + (uint32_t)own, k0);
      mx = chunk_max(x1, kv0 + oth + 32, need_mask, mx);
      tmem_wait_ld();
      tmem_ld_32x32(t + (uint32_t)own + 32u, k1);
      mx = chunk_max(k0, kv0 + own, need_mask, mx);
      tmem_wait_ld();
      mx = chunk_max(k1, kv0 + own + 32, need_mask, mx);
      // S is in registers: hand the buffer back to the tensor pipe before the exponentials
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_empty(b));
      const float m_raw = fmaxf(m, mx * g.scale_log2);
      const float m_new = m_raw == -INFINITY ? 0.f : m_raw;  // a row with nothing visible yet: keep the arithmetic finite
      const float alpha = ex2_approx(m - m_new);             // 0 on the first block (m = -inf)
      // probabilities -> shared memory (K-major, 128-byte swizzle), row sum
      if (!(ok = mbar_wait(p_empty(b), ph ^ 1u, g.status, 33))) break;
      uint8_t *p_row = base_ptr + Cfg::OFF_P + b * Cfg::P_BYTES + (row_in_tile >> 3) * 1024 + (row_in_tile & 7) * 128;
      float rowsum = 0.f;
      auto emit = [&](const uint32_t (&v)[32], int c) {  // c = first key column (0..127) of these 32 values
        uint32_t packed[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float p0 = ex2_approx(fmaf(__uint_as_float(v[e]), g.scale_log2, -m_new));
          float p1 = ex2_approx(fmaf(__uint_as_float(v[e + 1]), g.scale_log2, -m_new));
          if (need_mask) {
            if (kv0 + c + e > limit) p0 = 0.f;
            if (kv0 + c + e + 1 > limit) p1 = 0.f;
          }
          rowsum += p0 + p1;
          packed[e >> 1] = pack_pair(p0, p1, g.bf16);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int unit = (c >> 3) + u;  // 16-byte unit index along the 128 keys
          uint8_t *dst = p_row + (unit >> 3) * (FA_BM * 128) + (((unit & 7) ^ (row_in_tile & 7)) << 4);
          *reinterpret_cast<uint4 *>(dst) = make_uint4(packed[4 * u], packed[4 * u + 1], packed[4 * u + 2], packed[4 * u + 3]);
        }
      };
      emit(k0, own);
      emit(k1, own + 32);
      fence_proxy_async();  // the MMA reads these shared-memory writes through the async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full(b));
      l = fmaf(l, alpha, rowsum);
      if (j > 0) ok = accumulate_pv(j - 1, alpha_prev);
      alpha_prev = alpha;
      m = m_new;
    }
    if (ok && nblk > 0) ok = accumulate_pv(nblk - 1, alpha_prev);
    // the two warps of a quarter add up their partial row sums
    float *lsum = reinterpret_cast<float *>(base_ptr + Cfg::OFF_LSUM);
    lsum[half * FA_BM + row_in_tile] = l;
    __syncwarp();
    if (lane == 0) mbar_arrive(l_bar(quarter));
    if (ok) ok = mbar_wait(l_bar(quarter), 0, g.status, 34);
    if (ok && q_row < g.seq) {
      const float inv = __frcp_rn(l + lsum[(half ^ 1) * FA_BM + row_in_tile]);
      unsigned short *orow = g.o + (long long)head * g.o_sh + (long long)q_row * g.o_ss + half * DHH;
      if (g.vec_store) {
#pragma unroll
        for (int c = 0; c < DHH; c += 8) {
          uint4 out;
          out.x = pack_pair(o[c] * inv, o[c + 1] * inv, g.bf16);
          out.y = pack_pair(o[c + 2] * inv, o[c + 3] * inv, g.bf16);
          out.z = pack_pair(o[c + 4] * inv, o[c + 5] * inv, g.bf16);
          out.w = pack_pair(o[c + 6] * inv, o[c + 7] * inv, g.bf16);
          st_global_16(orow + c, out);
        }
      } else {
#pragma unroll
        for (int c = 0; c < DHH; c += 2) {
          const uint32_t pr = pack_pair(o[c] * inv, o[c + 1] * inv, g.bf16);
          orow[c] = (unsigned short)(pr & 0xffffu);
          orow[c + 1] = (unsigned short)(pr >> 16);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (*reinterpret_cast<volatile int *>(g.status) != 0) __nanosleep(1000000);
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------------
// The kernel for dh = 128: two 128-row q tiles per CTA played against each other.
//
// The fast path behind attention::Args (operators/src/attention/args.rs:10-24) for dh = 128: the same function as the
// crate's composition (operators/src/attention/operator.rs:199-275) computed with online softmax, so HBM sees q, k, v and o
// once.  What bounds a one-tile kernel on this machine is not the tensor pipe but the chain of hand-offs around the softmax
// of each 128-key block; here one CTA owns TWO q tiles (256 rows of one head) and the tensor pipe always has the other
// tile's products to run while one tile's exponentials are in flight:
//
//   warp 0        TMA producer: both q tiles once, then K and V blocks of 128 keys through two-stage rings;
//   warp 1        tcgen05.mma issuer, in the order  PV(t0,j)  QK(t0,j+1)  PV(t1,j)  QK(t1,j+1)  ...  so that the two tiles
//                 fall half a period apart;
//   warps 4-11    softmax of tile 0, warps 12-19 of tile 1: TWO threads per q row, one per half of the block's 128 keys
//                 (a measured block period was the softmax of one tile plus that tile's two products; the softmax of a
//                 single warp per scheduler runs at a third of an instruction per clock, so a second warp on the same
//                 scheduler nearly halves it).  A thread reads its 64 S values from tensor memory, the two threads of a
//                 row meet through shared memory and a 64-thread named barrier for the row maximum, and each writes its
//                 probabilities back INTO tensor memory as packed 16-bit pairs over the first half of the columns its S
//                 values occupied — the second product takes them from there (A operand in tensor memory).
// O lives in tensor memory and accumulates across blocks.  Rescaling is lazy (see below), so it is rare; when a row maximum
// of a warp has moved, that warp rescales its half of the O columns itself before it publishes the probabilities.  At the
// end the same threads divide by the row sums and store o.
// Registers are redistributed after start-up (setmaxnreg).  Every mbarrier wait is bounded; a wait that runs out records
// its code and every role unwinds to the common teardown.
//
// Few heads (a tensor-parallel shard): heads x tile pairs CTAs would leave most SMs idle behind the longest causal pair, so
// the key blocks of every pair are cut into `chunks` runs, one CTA each; a CTA then parks its unnormalised O (f32), its
// reference point m and row sum l in the caller's workspace and `attention_combine_kernel` merges the runs of a row.
constexpr int FP_BM = 128;        // rows per q tile
constexpr int FP_BN = 128;        // keys per block
constexpr int FP_DH = 128;
constexpr int FP_THREADS = 640;   // 5 warpgroups: {TMA, MMA, 2 idle}, softmax tile 0 (two), softmax tile 1 (two)
constexpr int FP_TILE_BYTES = FP_BM * FP_DH * 2;  // one q tile, one K block or one V block: 32 KB

struct PairAttnArgs {
  unsigned short *o;     // f16 or bf16 bit patterns
  long long o_sh, o_ss;  // element strides of o: head, row (dh contiguous)
  int nh, group, seq, att;
  int causal;
  int pairs;             // q-tile pairs per head
  float scale_log2;      // alpha * log2(e)
  int vec_store;
  int *status;
  int chunks;            // runs of key blocks per tile pair (1: the CTA finishes its rows itself)
  float *partial;        // chunks > 1: [head][q row][chunk][FP_PART_LD] = O (128 f32, unnormalised), m, l
};
constexpr int FP_PART_LD = FP_DH + 4;  // 16-byte aligned records

// Key blocks of the two q tiles of pair `pair`, the number of runs the pair is cut into (longer pairs into more runs, so
// that every run is about as long as a run of the longest pair: short pairs stay whole and write o themselves), and the
// run [jb0, jb0 + len) that `chunk` takes (empty when chunk >= runs).
struct FpRange {
  int nblk[2];  // blocks of each tile inside the run
  int jb0;
  int runs;
};
__host__ __device__ __forceinline__ FpRange fp_range(int pair, int chunk, int chunks, int seq, int att, int causal) {
  const int off = att - seq;
  int total[2];
  for (int t = 0; t < 2; ++t) {
    const int r0 = (pair * 2 + t) * FP_BM;
    int k_end = att;
    if (causal) k_end = min(att, off + r0 + FP_BM);
    total[t] = r0 < seq ? (k_end + FP_BN - 1) / FP_BN : 0;
  }
  const int nmax = max(total[0], total[1]);
  const int longest = (att + FP_BN - 1) / FP_BN;            // the last pair's (or, unmasked, every pair's) block count
  const int target = max(1, (longest + chunks - 1) / chunks);  // blocks per run of the longest pair
  FpRange r;
  r.runs = min(chunks, max(1, (nmax + target / 2) / target));
  const int len = (nmax + r.runs - 1) / r.runs;
  r.jb0 = chunk * len;
  for (int t = 0; t < 2; ++t) r.nblk[t] = chunk < r.runs ? max(0, min(total[t], r.jb0 + len) - r.jb0) : 0;
  return r;
}

struct FpSmem {
  static constexpr int OFF_Q = 0;                          // 2 tiles
  static constexpr int OFF_K = OFF_Q + 2 * FP_TILE_BYTES;  // 2 stages
  static constexpr int OFF_V = OFF_K + 2 * FP_TILE_BYTES;  // 2 stages
  static constexpr int OFF_BAR = OFF_V + 2 * FP_TILE_BYTES;
  static constexpr int NUM_BARS = 16;
  static constexpr int OFF_TMEM_SLOT = OFF_BAR + NUM_BARS * 8;
  static constexpr int OFF_MAX = OFF_TMEM_SLOT + 16;              // [2 tiles][2 halves][128 rows] f32: block maxima of a half row
  static constexpr int OFF_L = OFF_MAX + 4 * FP_BM * 4;           // [2 tiles][2 halves][128 rows] f32: row sums of a half row
  static constexpr int BYTES = OFF_L + 4 * FP_BM * 4 + 1024 /* alignment slack */;
};

__device__ __forceinline__ float fp_max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ float fp_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
template <bool BF>
__device__ __forceinline__ uint32_t fp_pack(float lo, float hi) {
  if (BF) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
  }
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&h);
}

template <bool BF>
__global__ void __launch_bounds__(FP_THREADS, 1)
    attention_pair_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                          const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ PairAttnArgs g) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bar0 = base + FpSmem::OFF_BAR;
  auto q_full = [&](int t) { return bar0 + 8u * (0 + t); };
  auto k_full = [&](int s) { return bar0 + 8u * (2 + s); };
  auto k_empty = [&](int s) { return bar0 + 8u * (4 + s); };
  auto v_full = [&](int s) { return bar0 + 8u * (6 + s); };
  auto v_empty = [&](int s) { return bar0 + 8u * (8 + s); };
  auto s_full = [&](int t) { return bar0 + 8u * (10 + t); };      // S of tile t complete (tensor pipe -> softmax)
  auto p_full = [&](int t) { return bar0 + 8u * (12 + t); };      // P of tile t written, O rescaled if needed (softmax -> issuer)
  auto o_final = [&](int t) { return bar0 + 8u * (14 + t); };     // last PV of tile t complete (tensor pipe -> softmax)
  const uint32_t tmem_slot = base + FpSmem::OFF_TMEM_SLOT;
  uint32_t *tmem_slot_ptr = reinterpret_cast<uint32_t *>(base_ptr + FpSmem::OFF_TMEM_SLOT);
  float *max_s = reinterpret_cast<float *>(base_ptr + FpSmem::OFF_MAX);
  float *l_s = reinterpret_cast<float *>(base_ptr + FpSmem::OFF_L);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heaviest pairs first, the heads of one (pair, run) next to each other (a GQA group shares its K/V blocks through L2)
  const int item = (int)(blockIdx.x / g.nh);
  const int pair = g.pairs - 1 - item / g.chunks, chunk = item % g.chunks;
  const int head = (int)(blockIdx.x % g.nh);
  const int kv_head = head / g.group;
  const int q0 = pair * 2 * FP_BM;
  const int off = g.att - g.seq;  // causal row r sees keys <= off + r
  // this CTA's run of key blocks: local block j is block jb0 + j of the pair; nblk[t] local blocks concern tile t
  const FpRange range = fp_range(pair, chunk, g.chunks, g.seq, g.att, g.causal);
  const int nblk[2] = {range.nblk[0], range.nblk[1]};
  const int jb0 = range.jb0;
  const int nmax = max(nblk[0], nblk[1]);
  if (nmax == 0) return;  // a run beyond those this pair is cut into (CTA-uniform, before anything is set up)

  if (threadIdx.x == 0) {
    for (int t = 0; t < 2; ++t) {
      mbar_init(q_full(t), 1);
      mbar_init(k_full(t), 1);
      mbar_init(k_empty(t), 1);
      mbar_init(v_full(t), 1);
      mbar_init(v_empty(t), 1);
      mbar_init(s_full(t), 1);
      mbar_init(p_full(t), 8);
      mbar_init(o_final(t), 1);
    }
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  // tensor memory columns: S0 | S1 | O0 | O1, 128 each; the P of keys [64h, 64h+64) of a tile overwrites columns
  // [64h, 64h+32) of its S (the first half of what the thread that wrote it had read)
  auto s_col = [&](int t) { return (uint32_t)(t * 128); };
  auto o_col = [&](int t) { return (uint32_t)(256 + t * 128); };

  if (warp < 4) {
    setmaxnreg_dec<56>();
    if (warp == 0 && lane == 0) {
      // ------------------------------------------------------------------ TMA producer
      for (int t = 0; t < 2; ++t) {
        if (nblk[t] == 0) continue;
        mbar_arrive_expect_tx(q_full(t), FP_TILE_BYTES);
#pragma unroll
        for (int h = 0; h < 2; ++h)
          tma_load_3d(base + FpSmem::OFF_Q + t * FP_TILE_BYTES + h * (FP_BM * 128), &tmap_q, q_full(t), h * 64, q0 + t * FP_BM, head);
      }
      bool ok = true;
      for (int j = 0; j < nmax && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (uint32_t)((j >> 1) & 1);
        if (!(ok = mbar_wait(k_empty(s), ph ^ 1u, g.status, 111))) break;
        mbar_arrive_expect_tx(k_full(s), FP_TILE_BYTES);
#pragma unroll
        for (int h = 0; h < 2; ++h)
          tma_load_3d(base + FpSmem::OFF_K + s * FP_TILE_BYTES + h * (FP_BN * 128), &tmap_k, k_full(s), h * 64, (jb0 + j) * FP_BN, kv_head);
        if (!(ok = mbar_wait(v_empty(s), ph ^ 1u, g.status, 112))) break;
        mbar_arrive_expect_tx(v_full(s), FP_TILE_BYTES);
#pragma unroll
        for (int kg = 0; kg < 2; ++kg)
#pragma unroll
          for (int c = 0; c < 2; ++c)
            tma_load_3d(base + FpSmem::OFF_V + s * FP_TILE_BYTES + (kg * 2 + c) * 8192, &tmap_v, v_full(s), c * 64, (jb0 + j) * FP_BN + kg * 64, kv_head);
      }
    } else if (warp == 1 && lane == 0) {
      // ------------------------------------------------------------------ MMA issuer
      const uint32_t idesc_qk = make_idesc_f16(FP_BM, FP_BN, 0, 0, BF ? 1 : 0);
      const uint32_t idesc_pv = make_idesc_f16(FP_BM, FP_DH, 0, 1, BF ? 1 : 0);
      bool ok = true;
      // S(t) = Q(t) K_b^T
      auto issue_qk = [&](int t, int b) -> bool {
        const int s = b & 1;
        if (!mbar_wait(k_full(s), (uint32_t)((b >> 1) & 1), g.status, 121)) return false;
        tc_fence_after();
        const uint32_t qa = base + FpSmem::OFF_Q + t * FP_TILE_BYTES, ka = base + FpSmem::OFF_K + s * FP_TILE_BYTES;
        const uint32_t d = tmem_base + s_col(t);
#pragma unroll
        for (int ks = 0; ks < FP_DH / 16; ++ks) {
          const uint64_t da = make_smem_desc_sw128(qa + (ks >> 2) * (FP_BM * 128) + (ks & 3) * 32, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(ka + (ks >> 2) * (FP_BN * 128) + (ks & 3) * 32, 16, 1024);
          umma_f16_ss(d, da, db, idesc_qk, ks != 0 ? 1u : 0u);
        }
        umma_commit(s_full(t));
        const bool last_user = t == 1 || b >= nblk[1];
        if (last_user) umma_commit(k_empty(s));
        return true;
      };
      // O(t) (+)= P(t) V_b, P from tensor memory
      auto issue_pv = [&](int t, int b) -> bool {
        const int s = b & 1;
        if (!mbar_wait(v_full(s), (uint32_t)((b >> 1) & 1), g.status, 122)) return false;
        if (!mbar_wait(p_full(t), (uint32_t)(b & 1), g.status, 123)) return false;
        tc_fence_after();
        const uint32_t va = base + FpSmem::OFF_V + s * FP_TILE_BYTES;
        const uint32_t d = tmem_base + o_col(t);
        const uint32_t p = tmem_base + s_col(t);
#pragma unroll
        for (int ks = 0; ks < FP_BN / 16; ++ks) {
          const uint64_t db = make_smem_desc_sw128(va + (ks >> 2) * (2 * 8192) + (ks & 3) * 2048, 8192, 1024);
          // 16 keys = 8 packed columns; keys 64.. sit behind the second half row's S columns
          umma_f16_ts(d, p + (uint32_t)((ks >> 2) * 64 + (ks & 3) * 8), db, idesc_pv, (b != 0 || ks != 0) ? 1u : 0u);
        }
        if (b == nblk[t] - 1) umma_commit(o_final(t));
        const bool last_user = t == 1 || b >= nblk[1];
        if (last_user) umma_commit(v_empty(s));
        return true;
      };
      for (int t = 0; t < 2 && ok; ++t) {
        if (nblk[t] == 0) continue;
        if (!(ok = mbar_wait(q_full(t), 0, g.status, 120))) break;
        ok = issue_qk(t, 0);
      }
      for (int j = 0; j < nmax && ok; ++j) {
        for (int t = 0; t < 2 && ok; ++t) {
          if (j >= nblk[t]) continue;
          ok = issue_pv(t, j);
          if (ok && j + 1 < nblk[t]) ok = issue_qk(t, j + 1);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax, rescaling, output: two threads per q row
    setmaxnreg_inc<104>();
    const int idx = warp - 4;
    const int t = idx >> 3;          // q tile
    const int h = (idx >> 2) & 1;    // which 64 keys of a block, and which 64 columns of O
    const int quarter = idx & 3;     // = warp & 3: tensor-memory lanes [32 * quarter, +32)
    const int row_in_tile = quarter * 32 + lane;
    const int q_row = q0 + t * FP_BM + row_in_tile;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const int limit = g.causal ? min(g.att - 1, off + q_row) : g.att - 1;  // last key this row may see
    const int pair_bar = 1 + t * 4 + quarter;  // named barrier of the two warps that share these 32 rows
    float *max_mine = max_s + (t * 2 + h) * FP_BM + row_in_tile, *max_other = max_s + (t * 2 + (h ^ 1)) * FP_BM + row_in_tile;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nblk[t]; ++j) {
      const int kv0 = (jb0 + j) * FP_BN + h * 64;
      // After a wait has run out this thread only keeps its appointments at the named barrier (its partner may be in it)
      if (ok) ok = mbar_wait(s_full(t), (uint32_t)(j & 1), g.status, 131);
      if (!ok) {
        named_bar_sync(pair_bar, 64);
        continue;
      }
      tc_fence_after();
      const uint32_t ta = tmem_base + lane_addr + s_col(t) + (uint32_t)(h * 64);
      uint32_t s0[32], s1[32];
      tmem_ld_32x32(ta, s0);
      tmem_ld_32x32(ta + 32u, s1);
      tmem_wait_ld();
      const bool need_mask = kv0 + 63 > limit;
      auto chunk_max = [&](const uint32_t (&v)[32], int k0, float mx) -> float {
        if (need_mask) {
#pragma unroll
          for (int e = 0; e < 32; ++e)
            if (k0 + e <= limit) mx = fmaxf(mx, __uint_as_float(v[e]));
          return mx;
        }
        float m0 = mx, m1 = -INFINITY;
#pragma unroll
        for (int e = 0; e < 32; e += 4) {
          m0 = fp_max3(m0, __uint_as_float(v[e]), __uint_as_float(v[e + 1]));
          m1 = fp_max3(m1, __uint_as_float(v[e + 2]), __uint_as_float(v[e + 3]));
        }
        return fmaxf(m0, m1);
      };
      float mx = fmaxf(chunk_max(s0, kv0, -INFINITY), chunk_max(s1, kv0 + 32, -INFINITY));
      // the other half of the row: its maximum over its 64 keys.  A slot is rewritten one block later, after the partner has
      // published the probabilities of this block, i.e. after it has read the slot.
      *max_mine = mx;
      named_bar_sync(pair_bar, 64);
      mx = fmaxf(mx, *max_other);
      // Lazy rescaling: the reference point m of the exponentials only follows the row maximum when that has moved by more
      // than 2^8 — until then the probabilities are taken relative to the older, smaller m (they stay below 256, exact in
      // the 16-bit operand; the f32 row sum and O carry the same factor, which cancels in o = O / l).  Rescaling O costs
      // a round trip through tensor memory on the critical path of a block; this way it happens a few times per row.
      const float m_raw = fmaxf(m, mx * g.scale_log2);
      const bool move = m_raw > m + 8.f;                     // also true on the first block (m = -inf)
      const float m_next = move ? m_raw : m;
      const float m_new = m_next == -INFINITY ? 0.f : m_next;  // a row with nothing visible yet: keep the arithmetic finite
      const float alpha = move ? fp_ex2(m - m_new) : 1.f;    // 0 on the first block
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
        // some row maximum of these 32 rows moved: rescale this thread's 64 columns of O.  S of block j being complete says
        // that PV of block j-1 has completed too (the tensor pipe retires in order), so O is stable.
        const uint32_t to = tmem_base + lane_addr + o_col(t) + (uint32_t)(h * 64);
#pragma unroll 1
        for (int c = 0; c < 64; c += 16) {
          uint32_t v[16];
          tmem_ld_32x16(to + (uint32_t)c, v);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 16; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * alpha);
          tmem_st_32x16(to + (uint32_t)c, v);
        }
      }
      // probabilities -> tensor memory, packed pairs over the first 32 of this thread's 64 S columns; row sum
      float rs0 = 0.f, rs1 = 0.f;
      auto emit = [&](const uint32_t (&v)[32], int c) {  // c = first key (0 or 32) of these 32 values within the half row
        uint32_t packed[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float p0 = fp_ex2(fmaf(__uint_as_float(v[e]), g.scale_log2, -m_new));
          float p1 = fp_ex2(fmaf(__uint_as_float(v[e + 1]), g.scale_log2, -m_new));
          if (need_mask) {
            if (kv0 + c + e > limit) p0 = 0.f;
            if (kv0 + c + e + 1 > limit) p1 = 0.f;
          }
          rs0 += p0;
          rs1 += p1;
          packed[e >> 1] = fp_pack<BF>(p0, p1);
        }
        tmem_st_32x16(ta + (uint32_t)(c >> 1), packed);
      };
      emit(s0, 0);
      emit(s1, 32);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full(t));
      l = fmaf(l, alpha, rs0 + rs1);
      m = m_next;
    }
    // whole-row sum: both halves carry the same reference point
    l_s[(t * 2 + h) * FP_BM + row_in_tile] = l;
    named_bar_sync(pair_bar, 64);
    l += l_s[(t * 2 + (h ^ 1)) * FP_BM + row_in_tile];
    if (ok && nblk[t] > 0 && range.runs > 1 && (ok = mbar_wait(o_final(t), 0, g.status, 142))) {
      // one run of several: park the unnormalised O with its reference point and row sum
      tc_fence_after();
      const uint32_t to = tmem_base + lane_addr + o_col(t) + (uint32_t)(h * 64);
      float *prow = g.partial + (((long long)head * g.seq + q_row) * g.chunks + chunk) * FP_PART_LD;
      if (q_row < g.seq && h == 0) {
        prow[FP_DH] = m;
        prow[FP_DH + 1] = l;
      }
#pragma unroll 1
      for (int c = 0; c < 64; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(to + (uint32_t)c, v);
        tmem_wait_ld();
        if (q_row < g.seq) {
#pragma unroll
          for (int q4 = 0; q4 < 8; ++q4)
            *reinterpret_cast<uint4 *>(prow + h * 64 + c + q4 * 4) = make_uint4(v[q4 * 4], v[q4 * 4 + 1], v[q4 * 4 + 2], v[q4 * 4 + 3]);
        }
      }
    } else if (ok && nblk[t] > 0 && (ok = mbar_wait(o_final(t), 0, g.status, 142))) {
      tc_fence_after();
      const float inv = __frcp_rn(l);
      const uint32_t to = tmem_base + lane_addr + o_col(t) + (uint32_t)(h * 64);
      unsigned short *orow = g.o + (long long)head * g.o_sh + (long long)q_row * g.o_ss + h * 64;
      auto store32 = [&](const uint32_t (&v)[32], int c) {
        if (q_row >= g.seq) return;
        if (g.vec_store) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 out;
            out.x = fp_pack<BF>(__uint_as_float(v[q4 * 8 + 0]) * inv, __uint_as_float(v[q4 * 8 + 1]) * inv);
            out.y = fp_pack<BF>(__uint_as_float(v[q4 * 8 + 2]) * inv, __uint_as_float(v[q4 * 8 + 3]) * inv);
            out.z = fp_pack<BF>(__uint_as_float(v[q4 * 8 + 4]) * inv, __uint_as_float(v[q4 * 8 + 5]) * inv);
            out.w = fp_pack<BF>(__uint_as_float(v[q4 * 8 + 6]) * inv, __uint_as_float(v[q4 * 8 + 7]) * inv);
            st_global_16(orow + c + q4 * 8, out);
          }
        } else {
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            const uint32_t pr = fp_pack<BF>(__uint_as_float(v[e]) * inv, __uint_as_float(v[e + 1]) * inv);
            orow[c + e] = (unsigned short)(pr & 0xffffu);
            orow[c + e + 1] = (unsigned short)(pr >> 16);
          }
        }
      };
#pragma unroll 1
      for (int c = 0; c < 64; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(to + (uint32_t)c, v);
        tmem_wait_ld();
        store32(v, c);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (*reinterpret_cast<volatile int *>(g.status) != 0) __nanosleep(1000000);  // let stray copies land before the CTA goes away
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}


// Merges the runs of a q row left by attention_pair_kernel (chunks > 1): one warp per (head, row), a lane per 4 columns.
//   o = sum_c 2^(m_c - M) O_c / sum_c 2^(m_c - M) l_c,  M = max_c m_c, runs taken in order.
template <bool BF>
__global__ void __launch_bounds__(256) attention_combine_kernel(const __grid_constant__ PairAttnArgs g) {
  const long long row_id = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row_id >= (long long)g.nh * g.seq) return;
  const int head = (int)(row_id / g.seq), q_row = (int)(row_id - (long long)head * g.seq);
  const int pair = q_row / (2 * FP_BM), t = (q_row / FP_BM) & 1;
  const int runs = fp_range(pair, 0, g.chunks, g.seq, g.att, g.causal).runs;
  if (runs == 1) return;  // a pair that was not cut: its CTA has written o itself
  const float *prow = g.partial + row_id * g.chunks * FP_PART_LD;
  float ms[8];
  float top = -INFINITY;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    ms[c] = -INFINITY;
    if (c < runs && fp_range(pair, c, g.chunks, g.seq, g.att, g.causal).nblk[t] > 0) ms[c] = prow[c * FP_PART_LD + FP_DH];
    top = fmaxf(top, ms[c]);
  }
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float den = 0.f;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    if (c < runs && ms[c] != -INFINITY) {
      const float w = fp_ex2(ms[c] - top);
      const float4 v = *reinterpret_cast<const float4 *>(prow + c * FP_PART_LD + lane * 4);
      den = fmaf(prow[c * FP_PART_LD + FP_DH + 1], w, den);
      acc.x = fmaf(v.x, w, acc.x);
      acc.y = fmaf(v.y, w, acc.y);
      acc.z = fmaf(v.z, w, acc.z);
      acc.w = fmaf(v.w, w, acc.w);
    }
  }
  const float inv = den > 0.f ? __frcp_rn(den) : 0.f;
  const uint32_t lo = fp_pack<BF>(acc.x * inv, acc.y * inv), hi = fp_pack<BF>(acc.z * inv, acc.w * inv);
  unsigned short *orow = g.o + (long long)head * g.o_sh + (long long)q_row * g.o_ss + lane * 4;
  if (g.vec_store) {
    *reinterpret_cast<uint2 *>(orow) = make_uint2(lo, hi);
  } else {
    orow[0] = (unsigned short)(lo & 0xffffu);
    orow[1] = (unsigned short)(lo >> 16);
    orow[2] = (unsigned short)(hi & 0xffffu);
    orow[3] = (unsigned short)(hi >> 16);
  }
}

constexpr int FP_MAX_CHUNKS = OPS_ATTENTION_MAX_RUNS;
static_assert(FP_PART_LD * sizeof(float) == OPS_ATTENTION_RUN_RECORD_BYTES, "record size published in the header");

// cuTensorMapEncodeTiled through the runtime's driver entry point (shared with mat_mul.cu's approach)
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn fa_encode_fn() {
  static EncodeTiledFn fn = [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
    return (EncodeTiledFn)p;
  }();
  return fn;
}

// [heads, rows, dh] f16 tensor with dh contiguous as a rank-3 map (dh, rows, heads)
static bool encode_hrd(CUtensorMap *map, bool bf16, const void *ptr, usz dh, usz rows, usz heads, isz row_stride_b, isz head_stride_b, uint32_t box_rows) {
  EncodeTiledFn fn = fa_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {dh, rows, heads};
  cuuint64_t rs = rows > 1 ? (cuuint64_t)row_stride_b : (cuuint64_t)(dh * 2);
  cuuint64_t hs = heads > 1 ? (cuuint64_t)head_stride_b : rs * rows;
  cuuint64_t strides[2] = {rs, hs};
  cuuint32_t box[3] = {64, box_rows, 1};
  cuuint32_t es[3] = {1, 1, 1};
  return fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void *>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static bool hrd_ok(const void *p, const isz *st, usz heads, usz rows) {
  if (!aligned(p, 16) || st[2] != 2) return false;
  if (rows > 1 && (st[1] <= 0 || st[1] % 16)) return false;
  if (heads > 1 && (st[0] <= 0 || st[0] % 16)) return false;
  return true;
}

bool attention_fused_supported(const ops_attention_args *a, usz nh, usz nkvh, usz seq, usz att, usz dh) {
  if ((a->q_layout.dt != OPS_DT_F16 && a->q_layout.dt != OPS_DT_BF16) || (dh != 64 && dh != 128)) return false;
  if (nh > 65535 || seq > 0x3fffffffu || att > 0x3fffffffu) return false;
  const isz *sv = a->v_layout.strides, *so = a->o_layout.strides;
  if (dyn(sv[0]) || dyn(sv[1]) || dyn(sv[2]) || dyn(so[0]) || dyn(so[1]) || dyn(so[2])) return false;
  if (!hrd_ok(a->q_base, a->q_layout.strides, nh, seq) || !hrd_ok(a->k_base, a->k_layout.strides, nkvh, att) ||
      !hrd_ok(a->v_base, sv, nkvh, att))
    return false;
  if (so[2] != 2 || so[0] % 2 || so[1] % 2) return false;
  return fa_encode_fn() != nullptr;
}

template <int DH>
static int launch_fused(const OpBase &base, const ops_attention_args *a, usz nh, usz nkvh, usz seq, usz att, int *status, bool *attr_set,
                        cudaStream_t s) {
  typedef FaCfg<DH> Cfg;
  CUtensorMap tq, tk, tv;
  const isz *sq = a->q_layout.strides, *sk = a->k_layout.strides, *sv = a->v_layout.strides, *so = a->o_layout.strides;
  const bool bf = a->q_layout.dt == OPS_DT_BF16;
  if (!encode_hrd(&tq, bf, a->q_base, DH, seq, nh, sq[1], sq[0], FA_BM) || !encode_hrd(&tk, bf, a->k_base, DH, att, nkvh, sk[1], sk[0], FA_BN) ||
      !encode_hrd(&tv, bf, a->v_base, DH, att, nkvh, sv[1], sv[0], 64))
    return fail(OPS_EXECUTION_FAILED, "attention: cuTensorMapEncodeTiled failed");
  FusedAttnArgs g;
  g.o = (unsigned short *)a->o_base;
  g.bf16 = bf ? 1 : 0;
  g.o_sh = so[0] / 2;
  g.o_ss = so[1] / 2;
  g.nh = (int)nh;
  g.group = (int)(nh / nkvh);
  g.seq = (int)seq;
  g.att = (int)att;
  g.causal = a->mask == OPS_MASK_CAUSAL;
  g.q_blocks = (int)((seq + FA_BM - 1) / FA_BM);
  // the CPU path rounds alpha = 1/sqrt(dh) to f16 before the product (mat_mul/common_cpu/mod.rs:101)
  const float inv_sqrt = 1.f / sqrtf((float)DH);
  const float alpha = bf ? __bfloat162float(__float2bfloat16_rn(inv_sqrt)) : __half2float(__float2half_rn(inv_sqrt));
  g.scale_log2 = alpha * 1.4426950408889634f;
  g.vec_store = aligned(a->o_base, 16) && so[0] % 16 == 0 && so[1] % 16 == 0;
  g.status = status;
  cudaSetDevice(base.device);
  if (!*attr_set) {
    cudaError_t e = cudaFuncSetAttribute(attention_fused_kernel<DH>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return fail(OPS_EXECUTION_FAILED, "attention: cannot reserve %d bytes of shared memory: %s", Cfg::SMEM_BYTES, cudaGetErrorString(e));
    *attr_set = true;
  }
  const unsigned grid = (unsigned)(nh * (usz)g.q_blocks);
  attention_fused_kernel<DH><<<grid, FA_THREADS, Cfg::SMEM_BYTES, s>>>(tq, tk, tv, g);
  return check_launch("attention(fused)");
}

static int launch_pair(const OpBase &base, const ops_attention_args *a, usz nh, usz nkvh, usz seq, usz att, int *status, bool *attr_set,
                       void *ws, usz ws_len, cudaStream_t s) {
  CUtensorMap tq, tk, tv;
  const isz *sq = a->q_layout.strides, *sk = a->k_layout.strides, *sv = a->v_layout.strides, *so = a->o_layout.strides;
  const bool bf = a->q_layout.dt == OPS_DT_BF16;
  if (!encode_hrd(&tq, bf, a->q_base, FP_DH, seq, nh, sq[1], sq[0], FP_BM) || !encode_hrd(&tk, bf, a->k_base, FP_DH, att, nkvh, sk[1], sk[0], FP_BN) ||
      !encode_hrd(&tv, bf, a->v_base, FP_DH, att, nkvh, sv[1], sv[0], 64))
    return fail(OPS_EXECUTION_FAILED, "attention: cuTensorMapEncodeTiled failed");
  PairAttnArgs g;
  g.o = (unsigned short *)a->o_base;
  g.o_sh = so[0] / 2;
  g.o_ss = so[1] / 2;
  g.nh = (int)nh;
  g.group = (int)(nh / nkvh);
  g.seq = (int)seq;
  g.att = (int)att;
  g.causal = a->mask == OPS_MASK_CAUSAL;
  g.pairs = (int)((seq + 2 * FP_BM - 1) / (2 * FP_BM));
  // the CPU path rounds alpha = 1/sqrt(dh) to the element type before the product (mat_mul/common_cpu/mod.rs:101)
  const float inv_sqrt = 1.f / sqrtf((float)FP_DH);
  const float alpha = bf ? __bfloat162float(__float2bfloat16_rn(inv_sqrt)) : __half2float(__float2half_rn(inv_sqrt));
  g.scale_log2 = alpha * 1.4426950408889634f;
  g.vec_store = aligned(a->o_base, 16) && so[0] % 16 == 0 && so[1] % 16 == 0;
  g.status = status;
  cudaSetDevice(base.device);
  if (!*attr_set) {
    cudaError_t e = cudaFuncSetAttribute(attention_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, FpSmem::BYTES);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attention_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, FpSmem::BYTES);
    if (e != cudaSuccess) return fail(OPS_EXECUTION_FAILED, "attention: cannot reserve %d bytes of shared memory: %s", FpSmem::BYTES, cudaGetErrorString(e));
    *attr_set = true;
  }
  // Runs per pair, if the caller's workspace holds the partial results (the chain's own workspace request, which
  // ops_attention_scheme reports, is far larger).  The longest pairs are cut into `chunks` runs, shorter ones into fewer (fp_range).  Most runs that still fit one wave
  // of CTAs (up to 1.15 x the SM count) win: measured with 4096 tokens, 4 heads 43.9 us at four runs (148 CTAs) against
  // 79.7 whole; 8 heads 69.5 at two runs (168 CTAs), 81.4 at four (296 CTAs, a second wave), 80.7 whole.
  usz chunks = 1;
  for (usz c = 2; c <= (usz)FP_MAX_CHUNKS; ++c) {
    usz ctas = 0;
    for (int pr = 0; pr < g.pairs; ++pr) ctas += (usz)fp_range(pr, 0, (int)c, g.seq, g.att, g.causal).runs;
    if (ctas * nh * 100 <= (usz)base.sm_count * 115) chunks = c;
  }
  const usz longest = (att + FP_BN - 1) / FP_BN;
  chunks = std::max<usz>(1, std::min(chunks, longest / 4));  // at least four key blocks per run
  while (chunks > 1 && (!ws || !aligned(ws, 16) || ws_len < nh * seq * chunks * FP_PART_LD * sizeof(float))) --chunks;
  g.chunks = (int)chunks;
  g.partial = (float *)ws;
  const unsigned grid = (unsigned)(nh * (usz)g.pairs * chunks);
  if (bf) attention_pair_kernel<true><<<grid, FP_THREADS, FpSmem::BYTES, s>>>(tq, tk, tv, g);
  else attention_pair_kernel<false><<<grid, FP_THREADS, FpSmem::BYTES, s>>>(tq, tk, tv, g);
  OPS_TRY(check_launch("attention(fused, tile pair)"));
  if (chunks > 1) {
    const unsigned cgrid = (unsigned)((nh * seq + 7) / 8);
    if (bf) attention_combine_kernel<true><<<cgrid, 256, 0, s>>>(g);
    else attention_combine_kernel<false><<<cgrid, 256, 0, s>>>(g);
    return check_launch("attention(fused, combine)");
  }
  return OPS_OK;
}

int attention_fused_enqueue(const OpBase &base, const ops_attention_args *a, usz nh, usz nkvh, usz seq, usz att, usz dh, int *status,
                            bool *attr_set, void *ws, usz ws_len, cudaStream_t s, bool single_tile) {
  // dh = 128 with more than one q tile: the two-tile kernel; everything else (and on request) one tile per CTA
  if (dh == 128 && seq > (usz)FP_BM && !single_tile) return launch_pair(base, a, nh, nkvh, seq, att, status, &attr_set[2], ws, ws_len, s);
  if (dh == 128) return launch_fused<128>(base, a, nh, nkvh, seq, att, status, &attr_set[0], s);
  return launch_fused<64>(base, a, nh, nkvh, seq, att, status, &attr_set[1], s);
}

}  // namespace ops
