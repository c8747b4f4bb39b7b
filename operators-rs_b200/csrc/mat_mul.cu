// mat_mul.cu — C <- beta*C + alpha*A*B (rank 2 or 3, one broadcastable batch dim).
//
// Replaces mat_mul::common_cpu::Operator (operators/src/mat_mul/common_cpu/mod.rs:26-107); the layout
// checks restate Args::layout and Matrix::try_from (operators/src/mat_mul/args.rs:64-192).
//
// f16 runs on the 5th-generation tensor cores:
//   * one persistent CTA per SM, 6 warps: warp 0 = TMA producer, warp 1 = tcgen05.mma issuer (one
//     elected lane each), warps 2-5 = epilogue (one per 32-lane quarter of tensor memory);
//   * operands are staged in shared memory by tiled TMA loads with the 128-byte swizzle the
//     tcgen05 shared-memory descriptors expect; an mbarrier ring (full/empty per stage) couples
//     producer and issuer, tcgen05.commit releases a stage when its MMAs have retired;
//   * the 128 x BN f32 accumulator lives in tensor memory, double buffered (2 x BN columns), so the
//     epilogue of tile i overlaps the main loop of tile i+1; epilogue = tcgen05.ld -> alpha/beta in
//     f32 -> f16 -> 128-bit global stores;
//   * both operand majors are handled by descriptors (K-major or MN-major), so no operand is ever
//     transposed in memory; a column-major C is computed as C^T = B^T A^T.
//   * wave quantisation: the tiles of a last, partial wave are cut along K over the idle CTAs; f32 partials meet in
//     a scratch buffer owned by the handle and the last slice to arrive adds them in slice order (deterministic);
// Layouts TMA cannot describe (unaligned bases or strides) and f32 take a plain tiled SIMT kernel.
// Tensor-bound when 2mnk / bytes exceeds the ridge, HBM-bound otherwise (k = 128 attention products).
#include <cuda.h>

#include <mutex>
#include <type_traits>
#include <unordered_map>
#include <vector>

#include "comm.h"
#include "common.h"
#include "device_utils.cuh"
#include "internal.h"
#include "sm100_ptx.cuh"

namespace ops {

using namespace sm100;

// ------------------------------------------------------------------------------------------------
// device side: tcgen05 kernel
// ------------------------------------------------------------------------------------------------
constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;                       // 64 f16 = one 128-byte swizzle row
constexpr int GEMM_UMMA_K = 16;
constexpr int GEMM_EPI_WARPS = 8;       // plain kernel: two epilogue warps per 32-row quarter, each half of the tile's columns
constexpr int GEMM_THREADS = 64 + 32 * GEMM_EPI_WARPS;
constexpr int GEMM_FUSED_THREADS = 448;  // + 8 warps that reduce finished tiles across ranks while the GEMM goes on
constexpr int GEMM_A_BYTES = GEMM_BM * GEMM_BK * 2;
constexpr int GEMM_CHUNK_BYTES = 64 * GEMM_BK * 2;  // one 64 (MN) x 64 (K) MN-major box
constexpr int GEMM_SPLIT_MAX_UNITS = 160;          // CTAs that may hold a K-slice partial (>= SM count)
constexpr int GEMM_SPLIT_MAX_SLICES = 8;
constexpr int GEMM_SPLIT_COST_KB = 16;             // what cutting a remainder tile along K costs, in k-blocks of tile time
constexpr int GEMM_EPI_LD = 36;                    // padded row length (words) of the epilogue's shared-memory pad: conflict-free both ways

struct GemmKernelArgs {
  unsigned short *d;     // row-major output (f16 or bf16 bit patterns)
  long long ldd, d_bs;   // elements
  int m, n, k, batch;
  int tiles_m, tiles_n;
  int a_mn_major, b_mn_major;
  int a_batched, b_batched;  // 0: operand is shared by all batches (coordinate 0)
  float alpha, beta;
  int read_c;
  int vec_store;         // rows of D are 16-byte aligned
  int bf16;              // elements are bf16 (else f16)
  int group_m;           // tile raster: m-tiles walked in groups of this many (>= tiles_m: plain m-fastest order)
  int *status;
  // Remainder wave: the tiles beyond the last full wave are cut along K into `split_g` slices, one (tile, slice) unit
  // per CTA; partial sums meet in `split_ws` (f32); once all slices of a tile are there, slice s finishes the 32-column
  // chunks j with j mod split_g == s (a reduce-scatter: every slice reads one tile's worth of partials, none reads G).
  long long normal_tiles;  // tiles computed whole (a multiple of the grid when split_g > 1)
  int normal_iters;        // normal_tiles / grid
  int split_r, split_g;    // remainder tiles, slices per tile (1 = no split)
  int kb_per_slice;
  float *split_ws;         // [grid][4 quarters][BN/32 chunks][8][32 lanes] float4: a lane's 128-bit stores of one step are contiguous
  unsigned int *split_tickets;  // [split_r][4 quarters][2 column halves][2] arrivals and departures, self-resetting
};

// GEMM whose output is summed over the ranks of a tensor-parallel group inside the same kernel (row-parallel
// projections).  Every rank writes its partial tile into its peer-mapped "in" region and flags it at the tile's owner
// (rank = tile mod p); extra warps in every CTA sum the owner's tiles from all ranks with ordinary NVLink loads as soon as
// they are flagged (eight extra warps, 16 tile rows each), push the result into every rank's "out" region and flag that; finally each CTA moves its share of
// finished tiles from "out" to the caller's C.  The NVLink traffic of a two-shot all_reduce, hidden behind the MMAs.
struct FusedArArgs {
  char *peers[MAX_RANKS];
  unsigned long long region_bytes;
  int rank, size;
  int *status;
};

// 16-bit float <-> f32 for either element type (warp-uniform selector)
__device__ __forceinline__ float h16_to_f32(unsigned short b, int bf) {
  return bf ? __uint_as_float((uint32_t)b << 16) : __half2float(__ushort_as_half(b));
}
__device__ __forceinline__ unsigned short f32_to_h16(float v, int bf) {
  return bf ? __bfloat16_as_ushort(__float2bfloat16_rn(v)) : __half_as_ushort(__float2half_rn(v));
}

// Tile number r of a batch -> (m-tile, n-tile).  Plain order walks m fastest, so a wave of CTAs shares a few B panels and
// streams all of A (right when A fits in L2).  When A is too large for that, m-tiles are walked in groups of `group_m`, a
// wave then covers a near-square block of tiles and re-reads less of both operands.
__device__ __forceinline__ void tile_coords(int tiles_m, int tiles_n, int group_m, long long r, int &tm, int &tn) {
  if (group_m >= tiles_m) {
    tn = (int)(r / tiles_m);
    tm = (int)(r - (long long)tn * tiles_m);
    return;
  }
  const long long per_group = (long long)group_m * tiles_n;
  const int grp = (int)(r / per_group);
  const int first = grp * group_m;
  const int gm = min(group_m, tiles_m - first);
  const long long within = r - (long long)grp * per_group;
  tn = (int)(within / gm);
  tm = first + (int)(within - (long long)tn * gm);
}

struct GemmWork {
  long long t;
  int kb0, kb1;
  int slice;  // -1: whole tile
};

// Work unit number `it` of this CTA: whole tiles strided by the grid, then at most one K-slice of a remainder tile.
__device__ __forceinline__ bool gemm_work(const GemmKernelArgs &g, int it, int num_kb, GemmWork &w) {
  const long long t = blockIdx.x + (long long)it * gridDim.x;
  if (t < g.normal_tiles) {
    w.t = t;
    w.kb0 = 0;
    w.kb1 = num_kb;
    w.slice = -1;
    return true;
  }
  if (g.split_g > 1 && it == g.normal_iters && (int)blockIdx.x < g.split_r * g.split_g) {
    w.t = g.normal_tiles + (int)blockIdx.x / g.split_g;
    w.slice = (int)blockIdx.x % g.split_g;
    w.kb0 = w.slice * g.kb_per_slice;
    w.kb1 = min(num_kb, w.kb0 + g.kb_per_slice);
    return true;
  }
  return false;
}

template <int BN> struct GemmCfg {
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = GEMM_A_BYTES + B_BYTES;
  static constexpr int STAGES = BN == 256 ? 4 : 6;
  static constexpr int TMEM_COLS = BN == 128 ? 256 : 512;  // two accumulators of BN columns, rounded up to a power of two
  static constexpr int EPI_OFF = STAGES * STAGE_BYTES + 256;            // after the barriers
  static constexpr int EPI_BYTES = GEMM_EPI_WARPS * 16 * GEMM_EPI_LD * 4;  // one 16 x 32 f32 transposition pad per epilogue warp
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/ + EPI_BYTES;
};

template <int BN, bool FUSED>
__global__ void __launch_bounds__(FUSED ? GEMM_FUSED_THREADS : GEMM_THREADS, 1)
    gemm_f16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                            const __grid_constant__ GemmKernelArgs g, const __grid_constant__ FusedArArgs fa) {
  typedef GemmCfg<BN> Cfg;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + Cfg::STAGES * Cfg::STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (Cfg::STAGES + s); };
  auto tmem_full_bar = [&](int b) { return bar_base + 8u * (2 * Cfg::STAGES + b); };
  auto tmem_empty_bar = [&](int b) { return bar_base + 8u * (2 * Cfg::STAGES + 2 + b); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * Cfg::STAGES + 4);
  uint32_t *tmem_slot_ptr = reinterpret_cast<uint32_t *>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (g.k + GEMM_BK - 1) / GEMM_BK;
  const int bf = g.bf16;
  unsigned int fa_epoch = 0;  // epoch of this launch of the fused all_reduce (read from device memory: replay-safe)
  if constexpr (FUSED) fa_epoch = p2p_epoch(fa.peers[fa.rank]);
  const long long tiles_per_batch = (long long)g.tiles_m * g.tiles_n;
  const long long num_tiles = tiles_per_batch * g.batch;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tmem_full_bar(b), 1);
      mbar_init(tmem_empty_bar(b), FUSED ? 4 : GEMM_EPI_WARPS);
    }
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
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
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      GemmWork w;
      for (int it = 0; ok && gemm_work(g, it, num_kb, w); ++it) {
        const long long t = w.t;
        const int b = (int)(t / tiles_per_batch);
        const long long r = t - (long long)b * tiles_per_batch;
        int tn, tm;
        tile_coords(g.tiles_m, g.tiles_n, g.group_m, r, tm, tn);
        const int m0 = tm * GEMM_BM, n0 = tn * BN;
        const int ba = g.a_batched ? b : 0, bb = g.b_batched ? b : 0;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!(ok = mbar_wait(empty_bar(stage), phase ^ 1u, g.status, 1))) break;
          mbar_arrive_expect_tx(full_bar(stage), Cfg::STAGE_BYTES);
          const uint32_t sa = smem_base + stage * Cfg::STAGE_BYTES, sb = sa + GEMM_A_BYTES;
          const int k0 = kb * GEMM_BK;
          if (g.a_mn_major) {
#pragma unroll
            for (int c = 0; c < GEMM_BM / 64; ++c) tma_load_3d(sa + c * GEMM_CHUNK_BYTES, &tmap_a, full_bar(stage), m0 + 64 * c, k0, ba);
          } else {
            tma_load_3d(sa, &tmap_a, full_bar(stage), k0, m0, ba);
          }
          if (g.b_mn_major) {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tma_load_3d(sb + c * GEMM_CHUNK_BYTES, &tmap_b, full_bar(stage), n0 + 64 * c, k0, bb);
          } else {
            tma_load_3d(sb, &tmap_b, full_bar(stage), k0, n0, bb);
          }
          if (++stage == Cfg::STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(GEMM_BM, BN, g.a_mn_major, g.b_mn_major, g.bf16);
      const uint32_t a_lbo = g.a_mn_major ? GEMM_CHUNK_BYTES : 16, b_lbo = g.b_mn_major ? GEMM_CHUNK_BYTES : 16;
      const uint32_t a_kstep = g.a_mn_major ? GEMM_UMMA_K * 128 : GEMM_UMMA_K * 2;  // bytes per UMMA_K
      const uint32_t b_kstep = g.b_mn_major ? GEMM_UMMA_K * 128 : GEMM_UMMA_K * 2;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      GemmWork w;
      for (int it = 0; ok && gemm_work(g, it, num_kb, w); ++it) {
        if (!(ok = mbar_wait(tmem_empty_bar(acc), acc_phase ^ 1u, g.status, 2))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!(ok = mbar_wait(full_bar(stage), phase, g.status, 3))) break;
          tc_fence_after();
          const uint32_t sa = smem_base + stage * Cfg::STAGE_BYTES, sb = sa + GEMM_A_BYTES;
#pragma unroll
          for (int ks = 0; ks < GEMM_BK / GEMM_UMMA_K; ++ks) {
            const uint64_t da = make_smem_desc_sw128(sa + ks * a_kstep, a_lbo, 1024);
            const uint64_t db = make_smem_desc_sw128(sb + ks * b_kstep, b_lbo, 1024);
            umma_f16_ss(d_tmem, da, db, idesc, (kb != w.kb0 || ks != 0) ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));  // stage reusable once these MMAs have read it
          if (++stage == Cfg::STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(tmem_full_bar(acc));  // accumulator complete
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
  } else if (warp < 2 + (FUSED ? 4 : GEMM_EPI_WARPS)) {
    // ------------------------------------------------------------------ epilogue (warps 2..5, plain kernel 2..9)
    // Plain kernel: eight warps, two per 32-row quarter, warp 2 + 4h + i taking column half h of the tile — with short K
    // (k = 128 attention products, 8-way row-parallel shards) the epilogue of four warps took longer than the mainloop.
    const int quarter = warp & 3;  // tensor-memory lanes [32*quarter, +32) belong to this warp
    const int col_half = FUSED ? 0 : (warp - 2) >> 2;
    const int c_begin = FUSED ? 0 : col_half * (BN / 2), c_end = FUSED ? BN : c_begin + BN / 2;
    const int qh = quarter * 2 + col_half;  // arrival counters of the K split: one per (quarter, column half)
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    GemmWork w;
    for (int it = 0; ok && gemm_work(g, it, num_kb, w); ++it) {
      const long long t = w.t;
      const int b = (int)(t / tiles_per_batch);
      const long long r = t - (long long)b * tiles_per_batch;
      int tn, tm;
      tile_coords(g.tiles_m, g.tiles_n, g.group_m, r, tm, tn);
      const int row = tm * GEMM_BM + quarter * 32 + lane;
      const int n0 = tn * BN;
      if (!(ok = mbar_wait(tmem_full_bar(acc), acc_phase, g.status, 4))) break;
      tc_fence_after();
      unsigned short *drow = g.d + (long long)b * g.d_bs + (long long)row * g.ldd;
      // fused all_reduce: the partial goes to this rank's peer-visible "in" region (dense rows of n), C is only read
      unsigned short *wrow = drow;
      if constexpr (FUSED) wrow = reinterpret_cast<unsigned short *>(region_in(fa.peers[fa.rank], fa.region_bytes, fa_epoch & 1u)) + (long long)row * g.n;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN);
      // K-slice of a remainder tile: park the f32 partial, wait (bounded) until every slice of the tile has parked its
      // own, then finish this slice's share of the column chunks from the sum of all of them, taken in slice order
      // whoever does the adding.  Every CTA of the grid is resident (cooperative launch), so the wait cannot starve.
      bool finish = true;
      const float4 *part_q = nullptr;  // this quarter's partial of slice 0 of the tile
      unsigned int *ticket = nullptr;
      if (!FUSED && w.slice >= 0) {
        const int tile_r = (int)(t - g.normal_tiles);
        constexpr int QUARTER_F4 = (BN / 32) * 8 * 32;
        float4 *mine = reinterpret_cast<float4 *>(g.split_ws) + ((long long)blockIdx.x * 4 + quarter) * QUARTER_F4 + lane;
#pragma unroll 1
        for (int c = c_begin; c < c_end; c += 32) {
          uint32_t v[32];
          tmem_ld_32x32(taddr + (uint32_t)c, v);
          tmem_wait_ld();
          if (row < g.m) {  // rows outside C are never read back
#pragma unroll
            for (int q = 0; q < 8; ++q)
              mine[((c >> 5) * 8 + q) * 32] = make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]), __uint_as_float(v[4 * q + 2]),
                                                           __uint_as_float(v[4 * q + 3]));
          }
        }
        __threadfence();
        __syncwarp();
        ticket = g.split_tickets + (tile_r * 8 + qh) * 2;
        int there = 1;
        if (lane == 0) {
          atomicAdd(ticket, 1u);
          const unsigned long long t0 = globaltimer_ns();
          while (ld_acquire_gpu(ticket) < (unsigned)g.split_g) {
            if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
              atomicCAS(g.status, 0, 6);
              there = 0;
              break;
            }
          }
        }
        there = __shfl_sync(0xffffffffu, there, 0);
        finish = ok = there != 0;
        part_q = reinterpret_cast<const float4 *>(g.split_ws) + (((long long)tile_r * g.split_g) * 4 + quarter) * QUARTER_F4 + lane;
      }
#pragma unroll 1
      for (int c = c_begin; c < c_end && finish; c += 32) {
        if (!FUSED && w.slice >= 0 && (c >> 5) % g.split_g != w.slice) continue;  // another slice's chunk (warp-uniform)
        uint32_t v[32];
        // interior fast path: the chunk's 32 columns are all inside C and rows are 16-byte aligned.  The old values of C
        // (beta != 0) are requested before the tensor-memory load is waited for, four 128-bit loads in flight per lane.
        // (warp-uniform) — it goes through a shared-memory pad that turns "one lane = one row" into "eight rows x 64
        // contiguous bytes per instruction", so that C is read and written in full 32-byte sectors.
        const bool fast = g.vec_store && n0 + c + 32 <= g.n;
        const int rsub = lane >> 2, unit = lane & 3;
        const int tile_row0 = row - lane;
        Vec8<unsigned short> oldc[4];
        if (FUSED || w.slice < 0) {
          tmem_ld_32x32(taddr + (uint32_t)c, v);
          if (fast && g.read_c) {
#pragma unroll
            for (int it = 0; it < 4; ++it) {
              const int grow = tile_row0 + it * 8 + rsub;
              if (grow < g.m) oldc[it].u = ld_global_16(g.d + (long long)b * g.d_bs + (long long)grow * g.ldd + n0 + c + unit * 8);
            }
          }
          tmem_wait_ld();
        } else {
          float sum[32];
#pragma unroll
          for (int e = 0; e < 32; ++e) sum[e] = 0.f;
          if (row < g.m) {
            constexpr long long UNIT_F4 = 4LL * (BN / 32) * 8 * 32;  // one slice further
            const float4 *src = part_q + (c >> 5) * 8 * 32;
            // two slices at a time: sixteen 128-bit loads in flight, added in slice order
            for (int sl = 0; sl < g.split_g; sl += 2) {
              const bool two = sl + 1 < g.split_g;
              float4 f0[8], f1[8];
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                f0[q] = __ldcg(src + sl * UNIT_F4 + q * 32);
                if (two) f1[q] = __ldcg(src + (sl + 1) * UNIT_F4 + q * 32);
              }
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                sum[4 * q] += f0[q].x;
                sum[4 * q + 1] += f0[q].y;
                sum[4 * q + 2] += f0[q].z;
                sum[4 * q + 3] += f0[q].w;
              }
              if (two) {
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                  sum[4 * q] += f1[q].x;
                  sum[4 * q + 1] += f1[q].y;
                  sum[4 * q + 2] += f1[q].z;
                  sum[4 * q + 3] += f1[q].w;
                }
              }
            }
          }
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(sum[e]);
        }
        if (fast) {
          if (!(FUSED || w.slice < 0) && g.read_c) {
#pragma unroll
            for (int it = 0; it < 4; ++it) {
              const int grow = tile_row0 + it * 8 + rsub;
              if (grow < g.m) oldc[it].u = ld_global_16(g.d + (long long)b * g.d_bs + (long long)grow * g.ldd + n0 + c + unit * 8);
            }
          }
          // the pad holds 16 rows: lanes 0-15 go first, then lanes 16-31 (half the shared memory per warp, which is what
          // lets eight epilogue warps fit beside the four pipeline stages)
          float *pad = reinterpret_cast<float *>(smem_raw + (smem_base - smem_u32(smem_raw)) + Cfg::EPI_OFF) + (warp - 2) * 16 * GEMM_EPI_LD;
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            if ((lane >> 4) == hh) {
#pragma unroll
              for (int q = 0; q < 8; ++q)
                *reinterpret_cast<uint4 *>(pad + (lane & 15) * GEMM_EPI_LD + 4 * q) = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            }
            __syncwarp();
#pragma unroll
            for (int i2 = 0; i2 < 2; ++i2) {
              const int it = hh * 2 + i2;
              const int rr = i2 * 8 + rsub, grow = tile_row0 + it * 8 + rsub;
              const float4 f0 = *reinterpret_cast<const float4 *>(pad + rr * GEMM_EPI_LD + unit * 8);
              const float4 f1 = *reinterpret_cast<const float4 *>(pad + rr * GEMM_EPI_LD + unit * 8 + 4);
              const float acc8[8] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w};
              Vec8<unsigned short> out;
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                float val = __fmul_rn(g.alpha, acc8[e]);
                if (g.read_c) val = __fadd_rn(__fmul_rn(g.beta, h16_to_f32(oldc[it].h[e], bf)), val);
                out.h[e] = f32_to_h16(val, bf);
              }
              if (grow < g.m) {
                unsigned short *wp;
                if constexpr (FUSED) wp = reinterpret_cast<unsigned short *>(region_in(fa.peers[fa.rank], fa.region_bytes, fa_epoch & 1u)) + (long long)grow * g.n;
                else wp = g.d + (long long)b * g.d_bs + (long long)grow * g.ldd;
                st_global_16(wp + n0 + c + unit * 8, out.u);
              }
            }
            __syncwarp();  // the pad is rewritten by the other half / the next chunk
          }
        } else if (row < g.m) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int col = n0 + c + q * 8;
            if (col >= g.n) break;
            unsigned short *dp = drow + col;
            if (g.vec_store && col + 8 <= g.n) {
              Vec8<unsigned short> out, old;
              if (g.read_c) old.u = ld_global_16(dp);
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                float val = __fmul_rn(g.alpha, __uint_as_float(v[q * 8 + e]));
                if (g.read_c) val = __fadd_rn(__fmul_rn(g.beta, h16_to_f32(old.h[e], bf)), val);
                out.h[e] = f32_to_h16(val, bf);
              }
              st_global_16(wrow + col, out.u);
            } else {
              for (int e = 0; e < 8 && col + e < g.n; ++e) {
                float val = __fmul_rn(g.alpha, __uint_as_float(v[q * 8 + e]));
                if (g.read_c) val = __fadd_rn(__fmul_rn(g.beta, h16_to_f32(dp[e], bf)), val);
                dp[e] = f32_to_h16(val, bf);
              }
            }
          }
        }
      }
      if (!FUSED && ticket != nullptr && finish && lane == 0) {
        // the last slice to leave puts both counters back to zero for the next launch (every slice has seen the arrivals)
        if (atomicAdd(ticket + 1, 1u) == (unsigned)(g.split_g - 1)) {
          ticket[0] = 0;
          ticket[1] = 0;
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty_bar(acc));
      if constexpr (FUSED) {  // tell the tile's owner that this rank's quarter of the partial is in place
        __threadfence_system();
        __syncwarp();
        if (lane == 0) {
          P2PFlags *owner = reinterpret_cast<P2PFlags *>(fa.peers[(int)(t % fa.size)]);
          st_release_sys(&owner->tile_ready[fa.rank][t * 4 + quarter], fa_epoch);
        }
      }
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
  } else if constexpr (FUSED) {
    // ------------------------------------------------------------------ cross-rank reduction (warps 6..13)
    // Eight warps; warp c works on rows [16c, 16c+16) of a tile, i.e. half of the 32-row quarter c/2 whose flag it watches.
    const int cw = warp - 6;
    const int cq = cw >> 1;  // quarter whose flags gate these rows
    const unsigned int parity = fa_epoch & 1u;
    P2PFlags *mine = reinterpret_cast<P2PFlags *>(fa.peers[fa.rank]);
    constexpr int VPR = BN / 8;       // 16-byte vectors per tile row
    constexpr int RPP = 32 / VPR;     // tile rows per warp pass
    const int sub = lane / VPR, vec = lane % VPR;
    bool ok = true;
    auto wait_flag = [&](const unsigned int *flag, int code) -> bool {
      const unsigned long long t0 = p2p_now();
      while ((int)(ld_acquire_sys(flag) - fa_epoch) < 0) {
        if (p2p_now() - t0 > P2P_WAIT_LIMIT_NS) {
          atomicCAS(fa.status, 0, code);
          return false;
        }
      }
      return true;
    };
    // rows row0, row0 + RPP, ... (NR of them) of one tile column block: all ranks' copies requested before the first is used
    auto reduce_rows = [&](auto nr_tag, auto np_tag, int row0, int col) {
      constexpr int NR = decltype(nr_tag)::value, NP = decltype(np_tag)::value;
      uint4 raw[NR][NP];
      long long off[NR];
      bool live[NR];
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        const int row = row0 + r * RPP;
        live[r] = row < g.m && col < g.n;
        off[r] = ((long long)row * g.n + col) * 2;
#pragma unroll
        for (int q = 0; q < NP; ++q)
          if (live[r] && q < fa.size) raw[r][q] = ld_peer_16(region_in(fa.peers[q], fa.region_bytes, parity) + off[r]);
      }
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        if (!live[r]) continue;
        float accv[8] = {};
#pragma unroll
        for (int q = 0; q < NP; ++q)
          if (q < fa.size) {
            const __half *h = reinterpret_cast<const __half *>(&raw[r][q]);
#pragma unroll
            for (int e = 0; e < 8; ++e) accv[e] += __half2float(h[e]);
          }
        Pack8 out;
#pragma unroll
        for (int e = 0; e < 8; ++e) out.h[e] = __float2half_rn(accv[e]);
#pragma unroll
        for (int q = 0; q < NP; ++q)
          if (q < fa.size) *reinterpret_cast<uint4 *>(region_out(fa.peers[q], fa.region_bytes, parity) + off[r]) = out.u;
      }
    };
    // phase A: the tiles this rank owns (t = rank + p * j), spread over the CTAs in the order the GEMM produces them
    const long long owned = num_tiles > fa.rank ? (num_tiles - fa.rank + fa.size - 1) / fa.size : 0;
    for (long long j = blockIdx.x; j < owned && ok; j += gridDim.x) {
      const long long t = fa.rank + (long long)fa.size * j;
      const int f = (int)(t * 4 + cq);
      bool mine_ok = true;
      if (lane < fa.size) mine_ok = wait_flag(&mine->tile_ready[lane][f], 40 + lane);
      ok = __all_sync(0xffffffffu, mine_ok);
      if (!ok) break;
      int tn, tm;
      tile_coords(g.tiles_m, g.tiles_n, g.group_m, t, tm, tn);
      const int col = tn * BN + vec * 8;
      const int rbase = tm * GEMM_BM + cw * 16 + sub;
      if (fa.size <= 4) {
        for (int i = 0; i < 16; i += 4 * RPP) reduce_rows(std::integral_constant<int, 4>{}, std::integral_constant<int, 4>{}, rbase + i, col);
      } else {
        for (int i = 0; i < 16; i += 2 * RPP) reduce_rows(std::integral_constant<int, 2>{}, std::integral_constant<int, 8>{}, rbase + i, col);
      }
      __threadfence_system();
      __syncwarp();
      // these 16 rows of the tile are final on every rank: flag them (per tile and warp, so that the warp that moves the
      // same rows to C in phase B depends on nothing else)
      if (lane < fa.size) st_release_sys(&reinterpret_cast<P2PFlags *>(fa.peers[lane])->tile_done[t * 8 + cw], fa_epoch);
    }
    // phase B: every rank needs every tile: move this CTA's share from the "out" region to C
    for (long long t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      bool mine_ok = true;
      if (lane == 0) mine_ok = wait_flag(&mine->tile_done[t * 8 + cw], 60);
      ok = __all_sync(0xffffffffu, mine_ok);
      if (!ok) break;
      int tn, tm;
      tile_coords(g.tiles_m, g.tiles_n, g.group_m, t, tm, tn);
      const int col = tn * BN + vec * 8;
      const char *outp = region_out(fa.peers[fa.rank], fa.region_bytes, parity);
      const int rbase = tm * GEMM_BM + cw * 16 + sub;
      uint4 buf[16 / RPP];
#pragma unroll
      for (int i = 0; i < 16 / RPP; ++i) {
        const int row = rbase + i * RPP;
        if (row < g.m && col < g.n) buf[i] = ld_peer_16(outp + ((long long)row * g.n + col) * 2);
      }
#pragma unroll
      for (int i = 0; i < 16 / RPP; ++i) {
        const int row = rbase + i * RPP;
        if (row < g.m && col < g.n) st_global_16(g.d + (long long)row * g.ldd + col, buf[i]);
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (*reinterpret_cast<volatile int *>(g.status) != 0) __nanosleep(1000000);  // let stray copies land before the CTA goes away
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
  if constexpr (FUSED) {
    if (threadIdx.x == 0) p2p_launch_done(fa.peers[fa.rank]);
  }
}

// ------------------------------------------------------------------------------------------------
// device side: generic SIMT kernel (any strides, f16 or f32), 64x64 tile, 256 threads, 4x4 per thread
// ------------------------------------------------------------------------------------------------
struct SimtArgs {
  void *c;
  const void *a, *b;
  long long c_rs, c_cs, c_bs, a_rs, a_cs, a_bs, b_rs, b_cs, b_bs;  // elements
  int m, n, k, batch;
  float alpha, beta;
  int read_c;
};

template <class T>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const __grid_constant__ SimtArgs g) {
  __shared__ float As[16][64 + 1];
  __shared__ float Bs[16][64 + 1];
  const int b = blockIdx.z;
  const T *A = (const T *)g.a + (long long)b * g.a_bs;
  const T *B = (const T *)g.b + (long long)b * g.b_bs;
  T *C = (T *)g.c + (long long)b * g.c_bs;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < g.k; k0 += 16) {
    for (int i = threadIdx.x; i < 16 * 64; i += 256) {
      const int kk = i & 15, mm = i >> 4;
      const int gm = m0 + mm, gk = k0 + kk;
      As[kk][mm] = (gm < g.m && gk < g.k) ? to_f32(A[(long long)gm * g.a_rs + (long long)gk * g.a_cs]) : 0.f;
      const int nn = i & 63, kb = i >> 6;
      const int gn = n0 + nn, gk2 = k0 + kb;
      Bs[kb][nn] = (gn < g.n && gk2 < g.k) ? to_f32(B[(long long)gk2 * g.b_rs + (long long)gn * g.b_cs]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gm = m0 + ty * 4 + i, gn = n0 + tx * 4 + j;
      if (gm < g.m && gn < g.n) {
        T *cp = C + (long long)gm * g.c_rs + (long long)gn * g.c_cs;
        float val = __fmul_rn(g.alpha, acc[i][j]);
        if (g.read_c) val = __fadd_rn(__fmul_rn(g.beta, to_f32(*cp)), val);
        *cp = from_f32<T>(val);
      }
    }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
struct Mat {  // element strides (operators/src/mat_mul/args.rs:124-131)
  usz batch;
  isz stride;
  usz r, c;
  isz rs, cs;
};

static int to_matrix(const ops_layout &L, const char *name, Mat *mt) {
  for (uint32_t i = 0; i < L.ndim; ++i)
    if (dyn(L.shape[i]) || dyn(L.strides[i])) return fail(OPS_DYNAMIC_NOT_SUPPORT, "mat_mul: %s has dynamic shape or strides", name);
  if (L.ndim < 2) return fail(OPS_RANK_NOT_SUPPORT, "Matrix must have rank 2 or more");
  if (L.ndim > 3) return fail(OPS_SHAPE_NOT_SUPPORT, "Higher-rank tensors not supported");
  const isz unit = (isz)dt_size(L.dt);
  if (unit == 0) return fail(OPS_TYPE_NOT_SUPPORT, "mat_mul: unknown element type %u", L.dt);
  mt->batch = 1;
  mt->stride = 0;
  if (L.ndim == 3 && L.shape[0] != 1) {
    mt->batch = L.shape[0];
    mt->stride = L.strides[0] / unit;
  }
  mt->r = L.shape[L.ndim - 2];
  mt->c = L.shape[L.ndim - 1];
  mt->rs = L.strides[L.ndim - 2] / unit;
  mt->cs = L.strides[L.ndim - 1] / unit;
  return OPS_OK;
}

static inline void transpose(Mat &m) {
  std::swap(m.r, m.c);
  std::swap(m.rs, m.cs);
}

struct GemmProblem {  // D (row-major, unit column stride) = alpha * A * B + beta * D
  uint32_t dt;
  usz batch, m, n, k;
  Mat a, b, d;
  const void *a_ptr, *b_ptr;
  void *d_ptr;
};

static int solve_layout(const ops_mat_mul_args *args, GemmProblem *p) {
  Mat c, a, b;
  OPS_TRY(to_matrix(args->c_layout, "c", &c));
  OPS_TRY(to_matrix(args->a_layout, "a", &a));
  OPS_TRY(to_matrix(args->b_layout, "b", &b));
  if (c.r != a.r || c.c != b.c || a.c != b.r) return fail(OPS_SHAPE_MISMATCH, "Inconsistent matrix shapes");
  const usz batch = c.batch;
  if (!(a.batch == 1 || a.batch == batch) || !(b.batch == 1 || b.batch == batch)) return fail(OPS_SHAPE_MISMATCH, "Inconsistent batch sizes");
  if (!(c.rs == 1 || c.cs == 1) || !(a.rs == 1 || a.cs == 1) || !(b.rs == 1 || b.cs == 1))
    return fail(OPS_STRIDES_NOT_SUPPORT, "Matrix is not contiguous");
  if (args->c_layout.dt != args->a_layout.dt || args->c_layout.dt != args->b_layout.dt) return fail(OPS_TYPE_MISMATCH, "mat_mul: element types differ");
  p->dt = args->c_layout.dt;
  p->a_ptr = args->a_base;
  p->b_ptr = args->b_base;
  p->d_ptr = args->c_base;
  if (c.cs != 1) {  // column-major C: compute C^T = B^T A^T, which is row-major
    transpose(c);
    transpose(a);
    transpose(b);
    std::swap(a, b);
    std::swap(p->a_ptr, p->b_ptr);
  }
  p->batch = batch;
  p->m = c.r;
  p->n = c.c;
  p->k = a.c;
  p->a = a;
  p->b = b;
  p->d = c;
  return OPS_OK;
}

// cuTensorMapEncodeTiled, fetched from the driver at run time (no link-time dependency on libcuda)
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
    return (EncodeTiledFn)p;
  }();
  return fn;
}

// One operand as a rank-3 f16 tensor map: dims (inner, outer, batch), 128-byte swizzle.
static bool encode_operand(CUtensorMap *map, bool bf16, const void *ptr, usz inner, usz outer, usz batch, isz outer_stride_el, isz batch_stride_el,
                           uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {inner, outer, batch};
  // strides of size-1 dims are never used for addressing; give them a valid dummy
  cuuint64_t os = outer > 1 ? (cuuint64_t)outer_stride_el * 2 : (cuuint64_t)((inner * 2 + 15) / 16 * 16);
  cuuint64_t bs = batch > 1 ? (cuuint64_t)batch_stride_el * 2 : os * (outer ? outer : 1);
  cuuint64_t strides[2] = {os, bs};
  cuuint32_t box[3] = {box_inner, box_outer, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static bool tma_ok(const void *ptr, usz outer, usz batch, isz outer_stride_el, isz batch_stride_el) {
  if (!aligned(ptr, 16)) return false;
  if (outer > 1 && (outer_stride_el <= 0 || (outer_stride_el * 2) % 16 != 0)) return false;
  if (batch > 1 && (batch_stride_el <= 0 || (batch_stride_el * 2) % 16 != 0)) return false;
  return true;
}

struct GemmState {
  int *status_dev = nullptr;
  bool attr_set[4] = {false, false, false, false};
  // scratch of the remainder-wave K split, owned by the handle (launch never allocates): one 128 x 256 f32 partial per
  // CTA and the arrival counters, which every launch leaves at zero again.  One stream at a time per handle.
  float *split_ws = nullptr;
  unsigned int *split_tickets = nullptr;
};

}  // namespace ops

using namespace ops;

struct ops_mat_mul {
  ops::OpBase base;
  ops::GemmState st;
};

namespace ops {

template <int BN>
static int launch_tcgen05(const ops_mat_mul *op, const GemmProblem &p, bool a_mn, bool b_mn, usz eff_batch_a, usz eff_batch_b, float alpha,
                          float beta, cudaStream_t s, ops_comm *comm = nullptr) {
  typedef GemmCfg<BN> Cfg;
  CUtensorMap ta, tb;
  bool ok;
  const bool bf = p.dt == OPS_DT_BF16;
  if (a_mn) ok = encode_operand(&ta, bf, p.a_ptr, p.m, p.k, eff_batch_a, p.a.cs, p.a.stride, 64, GEMM_BK);
  else ok = encode_operand(&ta, bf, p.a_ptr, p.k, p.m, eff_batch_a, p.a.rs, p.a.stride, GEMM_BK, GEMM_BM);
  if (!ok) return fail(OPS_EXECUTION_FAILED, "mat_mul: cuTensorMapEncodeTiled failed for A");
  if (b_mn) ok = encode_operand(&tb, bf, p.b_ptr, p.n, p.k, eff_batch_b, p.b.rs, p.b.stride, 64, GEMM_BK);
  else ok = encode_operand(&tb, bf, p.b_ptr, p.k, p.n, eff_batch_b, p.b.cs, p.b.stride, GEMM_BK, BN);
  if (!ok) return fail(OPS_EXECUTION_FAILED, "mat_mul: cuTensorMapEncodeTiled failed for B");

  GemmKernelArgs g;
  g.d = (unsigned short *)p.d_ptr;
  g.ldd = p.d.rs;
  g.d_bs = p.d.stride;
  g.m = (int)p.m;
  g.n = (int)p.n;
  g.k = (int)p.k;
  g.batch = (int)p.batch;
  g.tiles_m = (int)((p.m + GEMM_BM - 1) / GEMM_BM);
  g.tiles_n = (int)((p.n + BN - 1) / BN);
  g.a_mn_major = a_mn;
  g.b_mn_major = b_mn;
  g.a_batched = eff_batch_a > 1;
  g.b_batched = eff_batch_b > 1;
  g.alpha = alpha;
  g.beta = beta;
  g.read_c = beta != 0.f;
  g.vec_store = aligned(p.d_ptr, 16) && (p.m == 1 || p.d.rs % 8 == 0) && (p.batch == 1 || p.d.stride % 8 == 0);
  g.bf16 = bf ? 1 : 0;
  // A panel set too large to stay in L2 next to the streamed B panels: walk m-tiles in groups so that a wave re-reads less
  g.group_m = (p.m * p.k * 2 > ((usz)48 << 20) && g.tiles_m > 16) ? 16 : g.tiles_m;
  g.status = op->st.status_dev;
  const long long tiles = (long long)g.tiles_m * g.tiles_n * g.batch;
  const unsigned grid = (unsigned)std::min<long long>(tiles, op->base.sm_count);
  // Wave quantisation: with R = tiles mod grid tiles left for a last, partial wave, cut each of them along K into
  // G = grid / R slices so that the whole grid works on that wave too (the partial sums meet in split_ws).
  g.normal_tiles = tiles;
  g.normal_iters = 0;
  g.split_r = 0;
  g.split_g = 1;
  g.kb_per_slice = 0;
  g.split_ws = op->st.split_ws;
  g.split_tickets = op->st.split_tickets;
  {
    const long long sms = op->base.sm_count;
    const long long rem = tiles % sms;
    const int num_kb = (int)((p.k + GEMM_BK - 1) / GEMM_BK);
    if (rem > 0 && op->st.split_ws && sms <= GEMM_SPLIT_MAX_UNITS) {
      int G = (int)std::min<long long>(sms / rem, GEMM_SPLIT_MAX_SLICES);
      G = std::min(G, num_kb / 4);  // at least four k-blocks per slice
      // Splitting costs a few microseconds (one tile of f32 partials out to L2 and one back per CTA, a second pipeline
      // fill), priced at GEMM_SPLIT_COST_KB k-blocks of tile time; it pays when the tile time it removes from the tail,
      // (1 - 1/G) * num_kb k-blocks, is larger.
      // A machine that is less than half full (skinny decode-time products: a few tiles, each streaming a whole weight
      // panel) is a different case: there the split is what puts every SM on the HBM stream, and the partials are small
      // (rows beyond m are neither written nor read).
      const bool underfilled = tiles * 2 <= sms && p.m <= 64;
      if (G >= 2 && !underfilled && (long long)(G - 1) * num_kb < (long long)GEMM_SPLIT_COST_KB * G) G = 1;
      if (G >= 2) {
        const int per = (num_kb + G - 1) / G;
        G = (num_kb + per - 1) / per;  // drop empty slices
        if (G >= 2) {
          g.normal_tiles = tiles - rem;
          g.normal_iters = (int)(g.normal_tiles / sms);
          g.split_r = (int)rem;
          g.split_g = G;
          g.kb_per_slice = per;
        }
      }
    }
  }
  ops_mat_mul *mop = const_cast<ops_mat_mul *>(op);
  FusedArArgs fa;
  memset(&fa, 0, sizeof(fa));
  if (comm) {
    // fused all_reduce: whole tiles only (no K split), every CTA resident, flags for every (tile, quarter)
    g.normal_tiles = tiles;
    g.split_g = 1;
    g.split_r = 0;
    for (int q = 0; q < MAX_RANKS; ++q) fa.peers[q] = q < comm->size ? comm->peers[q] : nullptr;
    fa.region_bytes = comm->region_bytes;
    fa.rank = comm->rank;
    fa.size = comm->size;
    fa.status = comm->status_dev;
    const int slot = BN == 256 ? 2 : 3;
    if (!mop->st.attr_set[slot]) {
      cudaError_t e = cudaFuncSetAttribute(gemm_f16_tcgen05_kernel<BN, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
      if (e != cudaSuccess) return fail(OPS_EXECUTION_FAILED, "mat_mul: cannot reserve %d bytes of shared memory: %s", Cfg::SMEM_BYTES, cudaGetErrorString(e));
      mop->st.attr_set[slot] = true;
    }
    gemm_f16_tcgen05_kernel<BN, true><<<grid, GEMM_FUSED_THREADS, Cfg::SMEM_BYTES, s>>>(ta, tb, g, fa);
    return check_launch("mat_mul+all_reduce(tcgen05)");
  }
  const unsigned launch_grid = g.split_g > 1 ? (unsigned)op->base.sm_count : grid;
  const int slot = BN == 256 ? 0 : 1;
  if (!mop->st.attr_set[slot]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_f16_tcgen05_kernel<BN, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return fail(OPS_EXECUTION_FAILED, "mat_mul: cannot reserve %d bytes of shared memory: %s", Cfg::SMEM_BYTES, cudaGetErrorString(e));
    mop->st.attr_set[slot] = true;
  }
  if (g.split_g > 1) {
    // the slices of a tile wait for one another: a cooperative launch makes the whole grid resident before any CTA runs
    void *params[] = {(void *)&ta, (void *)&tb, (void *)&g, (void *)&fa};
    cudaError_t e = cudaLaunchCooperativeKernel((const void *)gemm_f16_tcgen05_kernel<BN, false>, dim3(launch_grid), dim3(GEMM_THREADS), params,
                                                (size_t)Cfg::SMEM_BYTES, s);
    if (e != cudaSuccess) return fail(OPS_EXECUTION_FAILED, "mat_mul: cooperative launch failed: %s", cudaGetErrorString(e));
    return check_launch("mat_mul(tcgen05, K-split remainder)");
  }
  gemm_f16_tcgen05_kernel<BN, false><<<launch_grid, GEMM_THREADS, Cfg::SMEM_BYTES, s>>>(ta, tb, g, fa);
  return check_launch("mat_mul(tcgen05)");
}

int mat_mul_enqueue_impl(const ops_mat_mul *op, const ops_mat_mul_args *args, cudaStream_t s, ops_comm *comm);

int mat_mul_enqueue(const ops_mat_mul *op, const ops_mat_mul_args *args, cudaStream_t s) { return mat_mul_enqueue_impl(op, args, s, nullptr); }

int mat_mul_enqueue_impl(const ops_mat_mul *op, const ops_mat_mul_args *args, cudaStream_t s, ops_comm *comm) {
  GemmProblem p;
  OPS_TRY(solve_layout(args, &p));
  if (dyn(args->alpha) || dyn(args->beta)) return fail(OPS_DYNAMIC_NOT_SUPPORT, "mat_mul: alpha and beta must be static at launch");
  if (p.dt != OPS_DT_F16 && p.dt != OPS_DT_BF16 && p.dt != OPS_DT_F32) return fail(OPS_TYPE_NOT_SUPPORT, "Unsupported element type %u", p.dt);
  if (p.m == 0 || p.n == 0 || p.batch == 0) return OPS_OK;
  if (p.m > 0x7fffffffu || p.n > 0x7fffffffu || p.k > 0x7fffffffu || p.batch > 65535u) return fail(OPS_SHAPE_NOT_SUPPORT, "mat_mul: shape too large");
  if (!p.a_ptr || !p.b_ptr || !p.d_ptr) return fail(OPS_DYNAMIC_NOT_SUPPORT, "mat_mul: null base pointer at launch");
  cudaSetDevice(op->base.device);
  float alpha = args->alpha, beta = args->beta;
  if (p.dt == OPS_DT_F16) {  // the CPU path rounds both scalars to the element type first (mat_mul/common_cpu/mod.rs:101)
    alpha = __half2float(__float2half_rn(alpha));
    beta = __half2float(__float2half_rn(beta));
  } else if (p.dt == OPS_DT_BF16) {  // the same rule for the second 16-bit type
    alpha = __bfloat162float(__float2bfloat16_rn(alpha));
    beta = __bfloat162float(__float2bfloat16_rn(beta));
  }

  if ((p.dt == OPS_DT_F16 || p.dt == OPS_DT_BF16) && p.k > 0) {
    // operand majors: A is [m,k] (K-major when its column stride is 1), B is [k,n] (K-major when its row stride is 1)
    const bool a_mn = !(p.a.cs == 1 || p.k == 1) ;
    const bool b_mn = !(p.b.rs == 1 || p.k == 1);
    const usz ea = (p.a.batch > 1 && p.a.stride != 0) ? p.batch : 1;
    const usz eb = (p.b.batch > 1 && p.b.stride != 0) ? p.batch : 1;
    const bool a_ok = a_mn ? (p.a.rs == 1 && tma_ok(p.a_ptr, p.k, ea, p.a.cs, p.a.stride)) : tma_ok(p.a_ptr, p.m, ea, p.a.rs, p.a.stride);
    const bool b_ok = b_mn ? (p.b.cs == 1 && tma_ok(p.b_ptr, p.k, eb, p.b.rs, p.b.stride)) : tma_ok(p.b_ptr, p.n, eb, p.b.cs, p.b.stride);
    const bool d_ok = p.d.rs >= 0 && p.d.stride >= 0;
    if (comm) {
      // what the fused kernel needs on top of the tensor-core path: one matrix, dense 16-byte rows, a staging region that
      // holds the whole partial, a flag per (tile, quarter), one CTA per SM resident
      const long long tiles = (long long)((p.m + GEMM_BM - 1) / GEMM_BM) * (long long)((p.n + (p.n > 128 ? 256 : 128) - 1) / (p.n > 128 ? 256 : 128));
      const bool fused_ok = p.dt == OPS_DT_F16 && a_ok && b_ok && d_ok && encode_tiled_fn() && p.batch == 1 && p.n % 8 == 0 && p.d.rs % 8 == 0 && aligned(p.d_ptr, 16) &&
                            comm->p2p_ready && p.m * p.n * 2 <= comm->region_bytes && tiles * 8 <= P2P_MAX_TILE_FLAGS && comm->device == op->base.device;
      if (!fused_ok) return fail(OPS_ARGS_NOT_SUPPORT, "mat_mul_all_reduce: needs f16 TMA-describable operands, one dense matrix whose partial fits the attached staging region");
      if (p.n > 128) return launch_tcgen05<256>(op, p, a_mn, b_mn, ea, eb, alpha, beta, s, comm);
      return launch_tcgen05<128>(op, p, a_mn, b_mn, ea, eb, alpha, beta, s, comm);
    }
    if (a_ok && b_ok && d_ok && encode_tiled_fn()) {
      // 128 x 256 tiles unless the product is skinny and would leave three quarters of the SMs without a tile: then
      // narrower tiles (and the K split above them) spread the weight stream over the machine
      const long long tiles256 = (long long)((p.m + GEMM_BM - 1) / GEMM_BM) * (long long)((p.n + 255) / 256) * (long long)p.batch;
      const bool narrow = p.n <= 128 || (p.m <= 64 && tiles256 * 4 <= op->base.sm_count);
      if (narrow) return launch_tcgen05<128>(op, p, a_mn, b_mn, ea, eb, alpha, beta, s);
      return launch_tcgen05<256>(op, p, a_mn, b_mn, ea, eb, alpha, beta, s);
    }
  }
  if (comm) return fail(OPS_ARGS_NOT_SUPPORT, "mat_mul_all_reduce: f16 operands with k > 0 expected");
  SimtArgs g;
  g.c = p.d_ptr;
  g.a = p.a_ptr;
  g.b = p.b_ptr;
  g.c_rs = p.d.rs; g.c_cs = p.d.cs; g.c_bs = p.d.stride;
  g.a_rs = p.a.rs; g.a_cs = p.a.cs; g.a_bs = p.a.stride;
  g.b_rs = p.b.rs; g.b_cs = p.b.cs; g.b_bs = p.b.stride;
  g.m = (int)p.m; g.n = (int)p.n; g.k = (int)p.k; g.batch = (int)p.batch;
  g.alpha = alpha; g.beta = beta; g.read_c = beta != 0.f;
  dim3 grid((unsigned)((p.n + 63) / 64), (unsigned)((p.m + 63) / 64), (unsigned)p.batch);
  if (grid.y > 65535u) return fail(OPS_SHAPE_NOT_SUPPORT, "mat_mul: m too large for the generic kernel");
  if (p.dt == OPS_DT_F16) gemm_simt_kernel<__half><<<grid, 256, 0, s>>>(g);
  else if (p.dt == OPS_DT_BF16) gemm_simt_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(g);
  else gemm_simt_kernel<float><<<grid, 256, 0, s>>>(g);
  return check_launch("mat_mul(simt)");
}

}  // namespace ops

OPS_API int ops_mat_mul_create(int device, ops_mat_mul **out) {
  if (!out) return fail(OPS_ARGS_NOT_SUPPORT, "null out pointer");
  ops_mat_mul *h = new ops_mat_mul();
  int rc = init_base(&h->base, device);
  if (rc != OPS_OK) {
    delete h;
    return rc;
  }
  cudaSetDevice(device);
  if (cudaMalloc(&h->st.status_dev, sizeof(int)) != cudaSuccess || cudaMemset(h->st.status_dev, 0, sizeof(int)) != cudaSuccess) {
    delete h;
    return fail(OPS_EXECUTION_FAILED, "mat_mul: cannot allocate the status word");
  }
  const size_t ws_bytes = (size_t)GEMM_SPLIT_MAX_UNITS * GEMM_BM * 256 * sizeof(float), tk_bytes = (size_t)GEMM_SPLIT_MAX_UNITS * 16 * sizeof(unsigned int);
  if (cudaMalloc(&h->st.split_ws, ws_bytes) != cudaSuccess || cudaMalloc(&h->st.split_tickets, tk_bytes) != cudaSuccess ||
      cudaMemset(h->st.split_tickets, 0, tk_bytes) != cudaSuccess) {
    cudaGetLastError();  // without the scratch the kernel simply runs its last wave unsplit
    if (h->st.split_ws) cudaFree(h->st.split_ws);
    if (h->st.split_tickets) cudaFree(h->st.split_tickets);
    h->st.split_ws = nullptr;
    h->st.split_tickets = nullptr;
  }
  *out = h;
  return OPS_OK;
}

OPS_API void ops_mat_mul_destroy(ops_mat_mul *op) {
  if (!op) return;
  if (op->st.status_dev) cudaFree(op->st.status_dev);
  if (op->st.split_ws) cudaFree(op->st.split_ws);
  if (op->st.split_tickets) cudaFree(op->st.split_tickets);
  delete op;
}

// Non-zero when a bounded wait inside the tensor-core kernel ran out (1 producer, 2/3 issuer, 4 epilogue).
// Synchronises the device; meant for tests and post-mortems, not for the hot path.
OPS_API int ops_mat_mul_status(const ops_mat_mul *op) {
  int v = -1;
  cudaSetDevice(op->base.device);
  if (cudaMemcpy(&v, op->st.status_dev, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  return v;
}

// After a bounded wait has run out the status word sticks and the arrival counters of the K split may be left non-zero:
// this puts the handle back (synchronises the device first).  The output of the launch that timed out is undefined.
OPS_API int ops_mat_mul_status_reset(ops_mat_mul *op) {
  if (!op) return fail(OPS_ARGS_NOT_SUPPORT, "null handle");
  cudaSetDevice(op->base.device);
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemset(op->st.status_dev, 0, sizeof(int));
  if (e == cudaSuccess && op->st.split_tickets) e = cudaMemset(op->st.split_tickets, 0, (size_t)GEMM_SPLIT_MAX_UNITS * 16 * sizeof(unsigned int));
  if (e != cudaSuccess) return fail(OPS_EXECUTION_FAILED, "mat_mul status reset: %s", cudaGetErrorString(e));
  return OPS_OK;
}

OPS_API int ops_mat_mul_scheme(ops_mat_mul *op, const ops_mat_mul_args *args, size_t max_ws, size_t *ws_out) {
  (void)op;
  (void)max_ws;
  (void)args;  // like the crate's CPU operator, scheme() plans nothing (mat_mul/common_cpu/mod.rs:18-24)
  if (ws_out) *ws_out = 0;
  return OPS_OK;
}

OPS_API int ops_mat_mul_launch(const ops_mat_mul *op, const ops_mat_mul_args *args, void *ws, size_t ws_len, void *stream) {
  (void)ws;
  (void)ws_len;
  return mat_mul_enqueue(op, args, (cudaStream_t)stream);
}

// mat_mul immediately followed by all_reduce(sum) of its result over the group of `node`, as ONE kernel: the transfer of
// finished tiles overlaps the tensor-core work on the remaining ones.  On return of the kernel C holds the reduced
// result on every rank.  beta applies to this rank's partial only (fold a residual in on exactly one rank).
OPS_API int ops_mat_mul_all_reduce_launch(const ops_mat_mul *op, ops_comm *node, const ops_mat_mul_args *args, void *stream) {
  if (!node) return fail(OPS_ARGS_NOT_SUPPORT, "mat_mul_all_reduce: null communicator");
  if (node->size == 1) return mat_mul_enqueue(op, args, (cudaStream_t)stream);
  return mat_mul_enqueue_impl(op, args, (cudaStream_t)stream, node);
}
