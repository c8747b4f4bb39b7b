// all_reduce.cu — tensor-parallel all_reduce over the GPUs of one NVLink/NVSwitch box.
//
// Replaces all_reduce::common_cpu::Operator over InprocNode (operators/src/all_reduce/common_cpu.rs:43-104)
// and the crate's NCCL operator (operators/src/all_reduce/nccl.rs:36-62); argument checks follow
// Args::meta (operators/src/all_reduce/args.rs:26-75).  The topology node (rank, group size,
// communicator) is `ops_comm`, one per process and GPU.
//
// Two data paths:
//   * NCCL: one ncclAllReduce on the caller's stream (any dtype NCCL knows, every ReduceOp).  NCCL is
//     opened at run time (the copy PyTorch ships, already loaded in a torch process).
//   * peer-to-peer kernels for f16/f32 sums.  Every rank owns a staging buffer that all peers map
//     through CUDA IPC.  ONE kernel per call does copy-in, signalling, waiting and reduction with
//     ordinary loads from peer memory:
//       one-shot (small messages): every rank sums all p staged copies in rank order in f32 -> all
//         ranks produce bit-identical results after one NVLink read of (p-1) messages;
//       two-shot (large messages): rank r reduces the r-th 1/p of the message from all peers
//         (reduce-scatter), publishes it in its staging buffer, then gathers the other reduced parts
//         from the peers straight into dst -> 2 (p-1)/p message bytes over NVLink per rank.
//     CTA b of every rank works on slice b, so synchronisation is pairwise between same-index CTAs
//     through per-CTA epoch flags in peer memory; no grid-wide barrier.  Staging is double buffered by
//     epoch parity, which makes one signalling round per phase sufficient.  Every spin is bounded: after
//     WAIT_LIMIT_NS the kernel records the phase in the communicator's status word and returns.
//
// NVLink-bound: bus bytes per rank 2 (p-1)/p S (two-shot) or (p-1) S read (one-shot).
#include <dlfcn.h>
#include <nccl.h>

#include <string>

#include "comm.h"
#include "common.h"
#include "device_utils.cuh"
#include "internal.h"

namespace ops {

// ------------------------------------------------------------------------------------------------
// NCCL, bound at run time
// ------------------------------------------------------------------------------------------------
struct NcclApi {
  void *lib = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Broadcast)(const void *, void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  const char *(*GetErrorString)(ncclResult_t) = nullptr;
  std::string error;
};

static NcclApi &nccl_api() {
  static NcclApi api = [] {
    NcclApi a;
    const char *names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char *n : names) {
      a.lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (a.lib) break;
    }
    if (!a.lib) {
      a.error = std::string("cannot open libnccl.so.2: ") + (dlerror() ? dlerror() : "?");
      return a;
    }
    a.GetUniqueId = (decltype(a.GetUniqueId))dlsym(a.lib, "ncclGetUniqueId");
    a.CommInitRank = (decltype(a.CommInitRank))dlsym(a.lib, "ncclCommInitRank");
    a.CommDestroy = (decltype(a.CommDestroy))dlsym(a.lib, "ncclCommDestroy");
    a.AllReduce = (decltype(a.AllReduce))dlsym(a.lib, "ncclAllReduce");
    a.Broadcast = (decltype(a.Broadcast))dlsym(a.lib, "ncclBroadcast");
    a.GetErrorString = (decltype(a.GetErrorString))dlsym(a.lib, "ncclGetErrorString");
    if (!a.GetUniqueId || !a.CommInitRank || !a.CommDestroy || !a.AllReduce || !a.Broadcast || !a.GetErrorString) a.error = "libnccl lacks a required symbol";
    return a;
  }();
  return api;
}


// Thread q < size waits until flags[q] has reached `epoch`; returns false for the whole CTA on time-out.
__device__ __forceinline__ bool wait_flags(const unsigned int *flags_row0, int size, unsigned int epoch, int *status, int code) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  if ((int)threadIdx.x < size) {
    const unsigned int *f = flags_row0 + (size_t)threadIdx.x * P2P_MAX_CTAS;
    const unsigned long long t0 = p2p_now();
    while ((int)(ld_acquire_sys(f) - epoch) < 0) {
      if (p2p_now() - t0 > P2P_WAIT_LIMIT_NS) {
        atomicCAS(status, 0, code + 16 * ((int)threadIdx.x + 1));
        s_fail = 1;
        break;
      }
    }
  }
  __syncthreads();
  return s_fail == 0;
}

template <class T> struct Acc8;  // 16 bytes of T widened to f32 and back
template <> struct Acc8<__half> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void add(float *acc, uint4 raw) {
    const __half *h = reinterpret_cast<const __half *>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] += __half2float(h[i]);
  }
  static __device__ __forceinline__ uint4 pack(const float *acc) {
    Pack8 o;
#pragma unroll
    for (int i = 0; i < 8; ++i) o.h[i] = __float2half_rn(acc[i]);
    return o.u;
  }
};
template <> struct Acc8<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void add(float *acc, uint4 raw) {
    const __nv_bfloat16 *h = reinterpret_cast<const __nv_bfloat16 *>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] += __bfloat162float(h[i]);
  }
  static __device__ __forceinline__ uint4 pack(const float *acc) {
    union {
      uint4 u;
      __nv_bfloat16 h[8];
    } o;
#pragma unroll
    for (int i = 0; i < 8; ++i) o.h[i] = __float2bfloat16_rn(acc[i]);
    return o.u;
  }
};
template <> struct Acc8<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void add(float *acc, uint4 raw) {
    const float *f = reinterpret_cast<const float *>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] += f[i];
  }
  static __device__ __forceinline__ uint4 pack(const float *acc) {
    uint4 o;
    o.x = __float_as_uint(acc[0]); o.y = __float_as_uint(acc[1]); o.z = __float_as_uint(acc[2]); o.w = __float_as_uint(acc[3]);
    return o;
  }
};

// One-shot: stage own input, tell the peers, wait for theirs, sum everything in rank order.
// `vecs` = number of 16-byte vectors; CTA b owns vectors [b*per, (b+1)*per).
// P = compile-time bound on the group size (2, 4 or 8).  A thread keeps 8 peer loads in flight whatever the group size:
// U = 8 / P vectors per trip, each requested from every rank before the first is consumed — with one peer a single
// 16-byte load per thread and trip would leave an NVLink round trip (~2.5 us) mostly idle.
template <class T, int P>
__device__ __forceinline__ void one_shot_body(const P2PKernelArgs &a, unsigned int epoch, const uint4 *__restrict__ src, uint4 *__restrict__ dst,
                                              long long vecs) {
  constexpr int U = 8 / P;
  const unsigned int parity = epoch & 1u;
  const long long per = (vecs + gridDim.x - 1) / gridDim.x;
  const long long lo = (long long)blockIdx.x * per, hi = min(vecs, lo + per);
  uint4 *mine = reinterpret_cast<uint4 *>(region_in(a.peers[a.rank], a.region_bytes, parity));
  for (long long v = lo + threadIdx.x; v < hi; v += blockDim.x) mine[v] = src[v];
  __threadfence_system();
  __syncthreads();
  if ((int)threadIdx.x < a.size) {
    P2PFlags *pf = reinterpret_cast<P2PFlags *>(a.peers[threadIdx.x]);
    st_release_sys(&pf->ready[a.rank][blockIdx.x], epoch);
  }
  const P2PFlags *own = reinterpret_cast<const P2PFlags *>(a.peers[a.rank]);
  if (!wait_flags(&own->ready[0][blockIdx.x], a.size, epoch, a.status, 1)) return;
  const uint4 *pin[P];
#pragma unroll
  for (int q = 0; q < P; ++q) pin[q] = reinterpret_cast<const uint4 *>(region_in(a.peers[q < a.size ? q : 0], a.region_bytes, parity));
  for (long long v0 = lo + threadIdx.x; v0 < hi; v0 += (long long)U * blockDim.x) {
    uint4 raw[U][P];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long v = v0 + (long long)u * blockDim.x;
#pragma unroll
      for (int q = 0; q < P; ++q)
        if (v < hi && q < a.size) raw[u][q] = ld_peer_16(pin[q] + v);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long v = v0 + (long long)u * blockDim.x;
      if (v < hi) {
        float acc[Acc8<T>::N] = {};
#pragma unroll
        for (int q = 0; q < P; ++q)
          if (q < a.size) Acc8<T>::add(acc, raw[u][q]);
        dst[v] = Acc8<T>::pack(acc);
      }
    }
  }
}

template <class T, int P>
__global__ void __launch_bounds__(512) all_reduce_one_shot_kernel(const __grid_constant__ P2PKernelArgs a, const uint4 *__restrict__ src,
                                                                  uint4 *__restrict__ dst, long long vecs) {
  const unsigned int epoch = p2p_epoch(a.peers[a.rank]);
  one_shot_body<T, P>(a, epoch, src, dst, vecs);
  __syncthreads();
  if (threadIdx.x == 0) p2p_launch_done(a.peers[a.rank]);
}

// Two-shot: the message is cut into `size` parts of `part_vecs` vectors; CTA b owns slice b of every part.
//   DIRECT: `src` already lies in this rank's "direct" region at byte offset `direct_off` (the same on every rank), so
//           nothing is staged; peers are read at that offset of their direct regions.
//   ADD:    dst <- dst + sum over ranks of src: the old value of dst (identical on every rank, e.g. a replicated residual
//           stream) enters the f32 sum of the part this rank reduces, first, before rank 0's partial.
//   P:      as for the one-shot kernel: 8 / P vectors per thread and trip, 8 peer loads in flight.
// 256 threads per CTA so that one of its CTAs fits on an SM beside a CTA of the persistent tensor-core GEMM (192 threads,
// ~35 K registers, nearly all the shared memory): an exchange on one stream can overlap a projection on another.
constexpr int P2P_TWO_SHOT_THREADS = 256;

template <bool DIRECT>
__device__ __forceinline__ const uint4 *two_shot_in(const P2PKernelArgs &a, int q, unsigned int parity, unsigned long long direct_off) {
  char *pb = a.peers[q];
  return reinterpret_cast<const uint4 *>(DIRECT ? region_direct(pb, a.region_bytes) + direct_off : region_in(pb, a.region_bytes, parity));
}

// Second half of the two-shot exchange: slice b of every other rank's reduced part, from that rank's "out" region to dst;
// U vectors from every peer in flight per thread and trip.
template <int P>
__device__ __forceinline__ void two_shot_gather(const P2PKernelArgs &a, unsigned int parity, uint4 *__restrict__ dst, long long vecs, long long part_vecs,
                                                long long s_lo, long long s_hi) {
  constexpr int U = 8 / P;
  for (long long v0 = s_lo + threadIdx.x; v0 < s_hi; v0 += (long long)U * blockDim.x) {
    uint4 raw[U][P - 1];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long v = v0 + (long long)u * blockDim.x;
#pragma unroll
      for (int i = 0; i < P - 1; ++i)
        if (i < a.size - 1 && v < s_hi) {
          int q = a.rank + 1 + i;  // rank r starts at peer r+1: spreads the load over the links
          if (q >= a.size) q -= a.size;
          if ((long long)q * part_vecs + v < vecs) raw[u][i] = ld_peer_16(reinterpret_cast<const uint4 *>(region_out(a.peers[q], a.region_bytes, parity)) + v);
        }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long v = v0 + (long long)u * blockDim.x;
#pragma unroll
      for (int i = 0; i < P - 1; ++i)
        if (i < a.size - 1 && v < s_hi) {
          int q = a.rank + 1 + i;
          if (q >= a.size) q -= a.size;
          if ((long long)q * part_vecs + v < vecs) dst[(long long)q * part_vecs + v] = raw[u][i];
        }
    }
  }
}

template <class T, bool DIRECT, bool ADD, int P>
__device__ __forceinline__ void two_shot_body(const P2PKernelArgs &a, unsigned int epoch, const uint4 *__restrict__ src, uint4 *__restrict__ dst,
                                              long long vecs, long long part_vecs, unsigned long long direct_off) {
  constexpr int U = 8 / P;
  const unsigned int parity = epoch & 1u;
  const long long per = (part_vecs + gridDim.x - 1) / gridDim.x;
  const long long s_lo = (long long)blockIdx.x * per, s_hi = min(part_vecs, s_lo + per);
  uint4 *mine_out = reinterpret_cast<uint4 *>(region_out(a.peers[a.rank], a.region_bytes, parity));
  if constexpr (!DIRECT) {
    uint4 *mine_in = reinterpret_cast<uint4 *>(region_in(a.peers[a.rank], a.region_bytes, parity));
    // stage slice b of every part (four vectors in flight per thread)
    for (int part = 0; part < a.size; ++part) {
      const long long base = (long long)part * part_vecs;
      const long long stop = min(s_hi, vecs - base);
      long long v = s_lo + threadIdx.x;
      for (; v + 3 * blockDim.x < stop; v += 4 * blockDim.x) {
        uint4 r[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) r[u] = src[base + v + u * blockDim.x];
#pragma unroll
        for (int u = 0; u < 4; ++u) mine_in[base + v + u * blockDim.x] = r[u];
      }
      for (; v < stop; v += blockDim.x) mine_in[base + v] = src[base + v];
    }
    __threadfence_system();
  }
  __syncthreads();
  if ((int)threadIdx.x < a.size) {
    P2PFlags *pf = reinterpret_cast<P2PFlags *>(a.peers[threadIdx.x]);
    st_release_sys(&pf->ready[a.rank][blockIdx.x], epoch);
  }
  const P2PFlags *own = reinterpret_cast<const P2PFlags *>(a.peers[a.rank]);
  if (!wait_flags(&own->ready[0][blockIdx.x], a.size, epoch, a.status, 2)) return;
  // reduce my part, slice b: every peer's copy of U vectors is requested before the first is consumed
  {
    const long long base = (long long)a.rank * part_vecs;
    const long long stop = min(s_hi, vecs - base);
    const uint4 *pin[P];
#pragma unroll
    for (int q = 0; q < P; ++q) pin[q] = two_shot_in<DIRECT>(a, q < a.size ? q : 0, parity, direct_off) + base;
    for (long long v0 = s_lo + threadIdx.x; v0 < stop; v0 += (long long)U * blockDim.x) {
      uint4 raw[U][P], old[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long v = v0 + (long long)u * blockDim.x;
#pragma unroll
        for (int q = 0; q < P; ++q)
          if (v < stop && q < a.size) raw[u][q] = ld_peer_16(pin[q] + v);
        if constexpr (ADD) {
          if (v < stop) old[u] = dst[base + v];
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long v = v0 + (long long)u * blockDim.x;
        if (v < stop) {
          float acc[Acc8<T>::N] = {};
          if constexpr (ADD) Acc8<T>::add(acc, old[u]);
#pragma unroll
          for (int q = 0; q < P; ++q)
            if (q < a.size) Acc8<T>::add(acc, raw[u][q]);
          const uint4 r = Acc8<T>::pack(acc);
          mine_out[v] = r;
          dst[base + v] = r;
        }
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  if ((int)threadIdx.x < a.size) {
    P2PFlags *pf = reinterpret_cast<P2PFlags *>(a.peers[threadIdx.x]);
    st_release_sys(&pf->reduced[a.rank][blockIdx.x], epoch);
  }
  if (!wait_flags(&own->reduced[0][blockIdx.x], a.size, epoch, a.status, 3)) return;
  two_shot_gather<P>(a, parity, dst, vecs, part_vecs, s_lo, s_hi);
}

template <class T, bool DIRECT, bool ADD, int P>
__global__ void __maxnreg__(104) all_reduce_two_shot_kernel(const __grid_constant__ P2PKernelArgs a, const uint4 *__restrict__ src,
                                                                                      uint4 *__restrict__ dst, long long vecs, long long part_vecs,
                                                                                      unsigned long long direct_off) {
  const unsigned int epoch = p2p_epoch(a.peers[a.rank]);
  two_shot_body<T, DIRECT, ADD, P>(a, epoch, src, dst, vecs, part_vecs, direct_off);
  __syncthreads();
  if (threadIdx.x == 0) p2p_launch_done(a.peers[a.rank]);
}

// ------------------------------------------------------------------------------------------------
// In-switch reduction (NVLS).  The partial of every rank lies in the first half of a buffer bound to an NVLink multicast
// object, at the same offset.  Rank r owns the r-th 1/p of the message: one `multimem.ld_reduce` per 16 bytes returns the
// sum over ALL ranks, added up inside the NVSwitch (f32 accumulation), so the reduce-scatter half brings S/p bytes into a
// rank instead of (p-1)/p S; the result (plus the replicated residual, ADD) goes to dst and to the rank's peer-mapped "out"
// region, and the all-gather half is the two-shot kernel's: ordinary peer loads.  (A first form delivered the result with
// `multimem.st` to every rank and copied it out locally: 147-150 us per 32 MiB at 2 and 4 ranks, 85-100 us of it in the
// loop where 16-byte multicast stores and reducing loads queue behind each other, 20 us in the fence behind the stores.)
// Flags and epochs are those of the peer-to-peer staging buffer (same-index CTAs meet pairwise, every wait bounded).
// ------------------------------------------------------------------------------------------------
template <class T> struct Multimem;
template <> struct Multimem<__half> {
  static __device__ __forceinline__ uint4 ld_reduce(const void *mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
  }
};
template <> struct Multimem<__nv_bfloat16> {
  static __device__ __forceinline__ uint4 ld_reduce(const void *mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
  }
};
template <> struct Multimem<float> {
  static __device__ __forceinline__ uint4 ld_reduce(const void *mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
  }
};

template <class T, bool ADD, int P>
__global__ void __maxnreg__(104) all_reduce_nvls_kernel(const __grid_constant__ P2PKernelArgs a, const char *__restrict__ mc_in, uint4 *__restrict__ dst,
                                                        long long vecs, long long part_vecs) {
  constexpr int U = 8;
  const unsigned int epoch = p2p_epoch(a.peers[a.rank]);
  const unsigned int parity = epoch & 1u;
  const long long per = (part_vecs + gridDim.x - 1) / gridDim.x;
  const long long s_lo = (long long)blockIdx.x * per, s_hi = min(part_vecs, s_lo + per);
  const P2PFlags *own = reinterpret_cast<const P2PFlags *>(a.peers[a.rank]);
  uint4 *mine_out = reinterpret_cast<uint4 *>(region_out(a.peers[a.rank], a.region_bytes, parity));
  // every rank's partial is in place (written by the kernel before this one on the same stream)
  __threadfence_system();
  __syncthreads();
  if ((int)threadIdx.x < a.size) {
    P2PFlags *pf = reinterpret_cast<P2PFlags *>(a.peers[threadIdx.x]);
    st_release_sys(&pf->ready[a.rank][blockIdx.x], epoch);
  }
  bool ok = wait_flags(&own->ready[0][blockIdx.x], a.size, epoch, a.status, 4);
  if (ok) {
    // reduce-scatter half inside the switch: this rank's part, slice b
    const long long base = (long long)a.rank * part_vecs;
    const long long stop = min(s_hi, vecs - base);
    const uint4 *in = reinterpret_cast<const uint4 *>(mc_in) + base;
    for (long long v0 = s_lo + threadIdx.x; v0 < stop; v0 += (long long)U * blockDim.x) {
      uint4 sum[U], old[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long v = v0 + (long long)u * blockDim.x;
        if (v < stop) {
          sum[u] = Multimem<T>::ld_reduce(in + v);
          if constexpr (ADD) old[u] = dst[base + v];
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long v = v0 + (long long)u * blockDim.x;
        if (v < stop) {
          uint4 r = sum[u];
          if constexpr (ADD) {
            float acc[Acc8<T>::N] = {};
            Acc8<T>::add(acc, old[u]);
            Acc8<T>::add(acc, sum[u]);
            r = Acc8<T>::pack(acc);
          }
          mine_out[v] = r;
          dst[base + v] = r;
        }
      }
    }
    __threadfence_system();
    __syncthreads();
    if ((int)threadIdx.x < a.size) {
      P2PFlags *pf = reinterpret_cast<P2PFlags *>(a.peers[threadIdx.x]);
      st_release_sys(&pf->reduced[a.rank][blockIdx.x], epoch);
    }
    ok = wait_flags(&own->reduced[0][blockIdx.x], a.size, epoch, a.status, 5);
  }
  // all-gather half: ordinary peer loads from the other ranks' "out" regions, as in the two-shot kernel
  if (ok) two_shot_gather<P>(a, parity, dst, vecs, part_vecs, s_lo, s_hi);
  __syncthreads();
  if (threadIdx.x == 0) p2p_launch_done(a.peers[a.rank]);
}

struct AllReduceMeta {
  uint32_t dt;
  usz len;  // elements
};

// One contiguous run?  (ArrayLayout::merge_be over all dims, operators/src/all_reduce/args.rs:46-68)
static int contiguous_len(const ops_layout &L, const char *name, usz *len) {
  const usz es = dt_size(L.dt);
  for (uint32_t i = 0; i < L.ndim; ++i)
    if (dyn(L.shape[i]) || dyn(L.strides[i])) return fail(OPS_DYNAMIC_NOT_SUPPORT, "all_reduce: %s has dynamic shape or strides", name);
  usz total = 1;
  isz expect = (isz)es;
  for (uint32_t i = L.ndim; i-- > 0;) {
    if (L.shape[i] != 1 && L.strides[i] != expect) return fail(OPS_STRIDES_NOT_SUPPORT, "all_reduce: %s is not one contiguous run", name);
    expect *= (isz)L.shape[i];
    total *= L.shape[i];
  }
  *len = total;
  return OPS_OK;
}

static int all_reduce_meta(const ops_all_reduce_args *a, AllReduceMeta *m) {
  if (a->pair.dst_layout.dt != a->pair.src_layout.dt) return fail(OPS_TYPE_MISMATCH, "dst and src element types differ");
  m->dt = a->pair.dst_layout.dt;
  if (dt_size(m->dt) == 0) return fail(OPS_TYPE_NOT_SUPPORT, "all_reduce: unknown element type %u", m->dt);
  usz d, s;
  OPS_TRY(contiguous_len(a->pair.dst_layout, "dst", &d));
  OPS_TRY(contiguous_len(a->pair.src_layout, "src", &s));
  if (d != s) return fail(OPS_SHAPE_MISMATCH, "all_reduce: dst has %zu elements, src %zu", d, s);
  m->len = d;
  return OPS_OK;
}

static bool nccl_types(uint32_t dt, uint8_t op, ncclDataType_t *t, ncclRedOp_t *o) {
  switch (dt) {
    case OPS_DT_F16: *t = ncclHalf; break;
    case OPS_DT_BF16: *t = ncclBfloat16; break;
    case OPS_DT_F32: *t = ncclFloat; break;
    case OPS_DT_F64: *t = ncclDouble; break;
    case OPS_DT_U8: *t = ncclUint8; break;
    case OPS_DT_I8: *t = ncclInt8; break;
    case OPS_DT_U32: *t = ncclUint32; break;
    case OPS_DT_I32: *t = ncclInt32; break;
    case OPS_DT_U64: *t = ncclUint64; break;
    case OPS_DT_I64: *t = ncclInt64; break;
    default: return false;
  }
  switch (op) {  // operators/src/all_reduce/nccl.rs:66-76
    case OPS_REDUCE_SUM: *o = ncclSum; break;
    case OPS_REDUCE_PROD: *o = ncclProd; break;
    case OPS_REDUCE_MIN: *o = ncclMin; break;
    case OPS_REDUCE_MAX: *o = ncclMax; break;
    case OPS_REDUCE_MEAN: *o = ncclAvg; break;
    default: return false;
  }
  return true;
}

}  // namespace ops

using namespace ops;

struct ops_all_reduce {
  ops_comm *comm;
  int algo;
};

// ------------------------------------------------------------------------------------------------
// communicator
// ------------------------------------------------------------------------------------------------
OPS_API int ops_comm_unique_id(uint8_t id_out[OPS_COMM_ID_BYTES]) {
  NcclApi &n = nccl_api();
  if (!n.error.empty()) return fail(OPS_EXECUTION_FAILED, "%s", n.error.c_str());
  static_assert(sizeof(ncclUniqueId) == OPS_COMM_ID_BYTES, "ncclUniqueId size");
  ncclUniqueId id;
  ncclResult_t r = n.GetUniqueId(&id);
  if (r != ncclSuccess) return fail(OPS_EXECUTION_FAILED, "ncclGetUniqueId: %s", n.GetErrorString(r));
  memcpy(id_out, &id, sizeof(id));
  return OPS_OK;
}

OPS_API int ops_comm_init_rank(int device, int rank, int group_size, const uint8_t id[OPS_COMM_ID_BYTES], ops_comm **out) {
  if (!out) return fail(OPS_ARGS_NOT_SUPPORT, "null out pointer");
  if (group_size < 1 || group_size > MAX_RANKS || rank < 0 || rank >= group_size)
    return fail(OPS_ARGS_NOT_SUPPORT, "rank %d of %d: group size must be 1..%d", rank, group_size, MAX_RANKS);
  OpBase base;
  OPS_TRY(init_base(&base, device));
  ops_comm *c = new ops_comm();
  memset(c, 0, sizeof(*c));
  c->device = device;
  c->rank = rank;
  c->size = group_size;
  c->sm_count = base.sm_count;
  cudaSetDevice(device);
  if (group_size > 1) {
    if (!id) {
      delete c;
      return fail(OPS_ARGS_NOT_SUPPORT, "group size %d needs a unique id", group_size);
    }
    NcclApi &n = nccl_api();
    if (!n.error.empty()) {
      delete c;
      return fail(OPS_EXECUTION_FAILED, "%s", n.error.c_str());
    }
    ncclUniqueId uid;
    memcpy(&uid, id, sizeof(uid));
    ncclResult_t r = n.CommInitRank(&c->nccl, group_size, uid, rank);
    if (r != ncclSuccess) {
      delete c;
      return fail(OPS_EXECUTION_FAILED, "ncclCommInitRank: %s", n.GetErrorString(r));
    }
    c->has_nccl = true;
  }
  if (cudaMalloc(&c->status_dev, sizeof(int)) != cudaSuccess || cudaMemset(c->status_dev, 0, sizeof(int)) != cudaSuccess) {
    delete c;
    return fail(OPS_EXECUTION_FAILED, "all_reduce: cannot allocate the status word");
  }
  *out = c;
  return OPS_OK;
}

// A communicator whose `group_size` ranks all map THIS rank's staging buffer: no NCCL, no second process.  The other
// "ranks" never run, so a peer-to-peer all_reduce on it can only end through its bounded waits — which is the point: it
// lets one GPU exercise the time-out path (status word set, kernel returns, context intact) without a hung peer.
OPS_API int ops_comm_create_loopback(int device, int group_size, size_t staging_bytes, ops_comm **out) {
  if (!out || group_size < 2 || group_size > MAX_RANKS) return fail(OPS_ARGS_NOT_SUPPORT, "loopback communicator: group size 2..%d", MAX_RANKS);
  ops_comm *c = nullptr;
  OPS_TRY(ops_comm_init_rank(device, 0, 1, nullptr, &c));
  c->size = group_size;
  uint8_t handle[OPS_COMM_P2P_HANDLE_BYTES];
  int rc = ops_comm_p2p_export(c, staging_bytes, handle);
  if (rc != OPS_OK) {
    ops_comm_destroy(c);
    return rc;
  }
  for (int q = 0; q < group_size; ++q) c->peers[q] = c->staging;
  c->p2p_ready = false;  // nothing to close at destroy: every entry is the own buffer
  c->loopback = true;
  *out = c;
  return OPS_OK;
}

OPS_API int ops_comm_rank(const ops_comm *c) { return c->rank; }
OPS_API int ops_comm_group_size(const ops_comm *c) { return c->size; }

OPS_API void ops_comm_destroy(ops_comm *c) {
  if (!c) return;
  cudaSetDevice(c->device);
  if (c->p2p_ready)
    for (int q = 0; q < c->size; ++q)
      if (q != c->rank && c->peers[q]) cudaIpcCloseMemHandle(c->peers[q]);
  if (c->staging) cudaFree(c->staging);
  if (c->status_dev) cudaFree(c->status_dev);
  if (c->has_nccl) nccl_api().CommDestroy(c->nccl);
  delete c;
}

OPS_API int ops_comm_p2p_export(ops_comm *c, size_t staging_bytes, uint8_t handle_out[OPS_COMM_P2P_HANDLE_BYTES]) {
  memset(handle_out, 0, OPS_COMM_P2P_HANDLE_BYTES);
  if (c->staging) return fail(OPS_ARGS_NOT_SUPPORT, "p2p staging already exported");
  cudaSetDevice(c->device);
  const size_t region = (staging_bytes + 255) / 256 * 256;
  const size_t total = sizeof(P2PFlags) + (size_t)P2P_REGIONS * region;
  if (cudaMalloc(&c->staging, total) != cudaSuccess) {
    cudaGetLastError();
    c->staging = nullptr;
    return fail(OPS_EXECUTION_FAILED, "p2p: cannot allocate %zu staging bytes", total);
  }
  cudaMemset(c->staging, 0, sizeof(P2PFlags));
  cudaDeviceSynchronize();
  c->staging_bytes = total;
  c->region_bytes = region;
  P2PHandleBlob blob;
  memset(&blob, 0, sizeof(blob));
  cudaError_t e = cudaIpcGetMemHandle(&blob.mem, c->staging);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(OPS_EXECUTION_FAILED, "cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
  }
  blob.region_bytes = region;
  blob.rank = c->rank;
  blob.valid = 1;
  memcpy(handle_out, &blob, sizeof(blob));
  return OPS_OK;
}

OPS_API int ops_comm_p2p_attach(ops_comm *c, const uint8_t *all_handles) {
  if (!c->staging) return fail(OPS_ARGS_NOT_SUPPORT, "p2p: export before attach");
  cudaSetDevice(c->device);
  for (int q = 0; q < c->size; ++q) {
    P2PHandleBlob blob;
    memcpy(&blob, all_handles + (size_t)q * OPS_COMM_P2P_HANDLE_BYTES, sizeof(blob));
    if (!blob.valid || blob.rank != q || blob.region_bytes != c->region_bytes)
      return fail(OPS_ARGS_NOT_SUPPORT, "p2p: handle %d is invalid or sized differently", q);
    if (q == c->rank) {
      c->peers[q] = c->staging;
      continue;
    }
    void *p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, blob.mem, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail(OPS_EXECUTION_FAILED, "cudaIpcOpenMemHandle(rank %d): %s", q, cudaGetErrorString(e));
    }
    c->peers[q] = (char *)p;
  }
  c->p2p_ready = true;
  return OPS_OK;
}

OPS_API int ops_comm_p2p_status(ops_comm *c) {
  int v = -1;
  cudaSetDevice(c->device);
  if (cudaMemcpy(&v, c->status_dev, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  return v;
}

// ------------------------------------------------------------------------------------------------
// operator
// ------------------------------------------------------------------------------------------------
OPS_API int ops_all_reduce_create(ops_comm *node, ops_all_reduce **out) {
  if (!node || !out) return fail(OPS_ARGS_NOT_SUPPORT, "null communicator or out pointer");
  ops_all_reduce *h = new ops_all_reduce();
  h->comm = node;
  h->algo = OPS_ALL_REDUCE_AUTO;
  *out = h;
  return OPS_OK;
}

OPS_API void ops_all_reduce_destroy(ops_all_reduce *op) { delete op; }

OPS_API int ops_all_reduce_set_algo(ops_all_reduce *op, int algo) {
  if (algo < OPS_ALL_REDUCE_AUTO || algo > OPS_ALL_REDUCE_P2P_TWO_SHOT) return fail(OPS_ARGS_NOT_SUPPORT, "all_reduce: unknown algorithm %d", algo);
  if (algo >= OPS_ALL_REDUCE_P2P_ONE_SHOT && !op->comm->p2p_ready && !op->comm->loopback && op->comm->size > 1)
    return fail(OPS_ARGS_NOT_SUPPORT, "all_reduce: peer-to-peer staging is not attached");
  op->algo = algo;
  return OPS_OK;
}

OPS_API int ops_all_reduce_scheme(ops_all_reduce *op, const ops_all_reduce_args *args, size_t max_ws, size_t *ws_out) {
  (void)op;
  (void)max_ws;
  (void)args;  // the crate's operators plan nothing here (all_reduce/common_cpu.rs:35-41, nccl.rs:28-34)
  if (ws_out) *ws_out = 0;
  return OPS_OK;
}

// Which path AUTO takes for a message of `bytes` over `p` ranks once the staging buffers are attached.  Measured on B200s
// behind NVSwitch (max over ranks, back-to-back calls): the one-shot kernel wins while the message is latency-bound, NCCL
// in the middle, and from a few MiB the two-shot kernel, whose NVLink traffic (2 (p-1)/p S per rank) matches NCCL's with
// fewer synchronisation rounds.
// Measured on this machine (f16 sums; microseconds for 8 KiB / 512 KiB / 4 MiB / 32 MiB):
//   2 ranks: NCCL 13.7 / 12.6 / 38.8 / 81.5, one-shot 14.4 / 22.6 / 42.8 / -, two-shot (staged) 22.1 / 37.5 / 42.1 / 100
//   8 ranks: NCCL 27.2 / 30.6 / 54.7 / 158,  one-shot 15.3 / 28.4 / 69.8 / -, two-shot (staged) 24.0 / 47.3 / 56.3 / 140
// (the zero-copy two-shot with the residual folded in, which a caller reaches through ops_all_reduce_add_launch, runs
// 32 MiB in 82 us on 2 ranks and 123 us on 8).
static int choose_algo(int p, usz bytes) {
  if (p <= 2) return bytes <= (usz)(16 << 10) ? OPS_ALL_REDUCE_P2P_ONE_SHOT : OPS_ALL_REDUCE_NCCL;
  if (bytes <= (usz)(p >= 8 ? (1 << 20) : (256 << 10))) return OPS_ALL_REDUCE_P2P_ONE_SHOT;
  if (bytes >= (usz)(p >= 8 ? (8 << 20) : (16 << 20))) return OPS_ALL_REDUCE_P2P_TWO_SHOT;
  return OPS_ALL_REDUCE_NCCL;
}

template <class T>
static int launch_p2p(ops_comm *c, int algo, const void *src, void *dst, usz bytes, bool add, cudaStream_t s) {
  P2PKernelArgs a;
  for (int q = 0; q < MAX_RANKS; ++q) a.peers[q] = q < c->size ? c->peers[q] : nullptr;
  a.region_bytes = c->region_bytes;
  a.rank = c->rank;
  a.size = c->size;
  a.status = c->status_dev;
  const long long vecs = (long long)(bytes / 16);
  if (algo == OPS_ALL_REDUCE_P2P_ONE_SHOT) {
    long long ctas = (vecs + 511) / 512;  // 8 KiB per CTA
    if (ctas > 2 * c->sm_count) ctas = 2 * c->sm_count;
    if (ctas > P2P_MAX_CTAS) ctas = P2P_MAX_CTAS;
    if (ctas < 1) ctas = 1;
    if (c->size <= 2) all_reduce_one_shot_kernel<T, 2><<<(unsigned)ctas, 512, 0, s>>>(a, (const uint4 *)src, (uint4 *)dst, vecs);
    else if (c->size <= 4) all_reduce_one_shot_kernel<T, 4><<<(unsigned)ctas, 512, 0, s>>>(a, (const uint4 *)src, (uint4 *)dst, vecs);
    else all_reduce_one_shot_kernel<T, 8><<<(unsigned)ctas, 512, 0, s>>>(a, (const uint4 *)src, (uint4 *)dst, vecs);
  } else {
    const long long part = (vecs + c->size - 1) / c->size;
    long long ctas = (part + 4 * P2P_TWO_SHOT_THREADS - 1) / (4 * P2P_TWO_SHOT_THREADS);
    if (ctas > c->sm_count) ctas = c->sm_count;  // every CTA must be resident: same-index CTAs of different ranks wait for each other
    if (ctas > P2P_MAX_CTAS) ctas = P2P_MAX_CTAS;
    if (ctas < 1) ctas = 1;
    // in-switch reduction: the partial lies in the "in" half of the attached multicast buffer
    if (c->nvls_mc && (const char *)src >= c->nvls_local && (const char *)src + bytes <= c->nvls_local + c->nvls_region) {
      const char *mc_in = c->nvls_mc + (size_t)((const char *)src - c->nvls_local);
#define OPS_NVLS(ADD, P) all_reduce_nvls_kernel<T, ADD, P><<<(unsigned)ctas, P2P_TWO_SHOT_THREADS, 0, s>>>(a, mc_in, (uint4 *)dst, vecs, part)
      if (add) {
        if (c->size <= 2) OPS_NVLS(true, 2);
        else if (c->size <= 4) OPS_NVLS(true, 4);
        else OPS_NVLS(true, 8);
      } else {
        if (c->size <= 2) OPS_NVLS(false, 2);
        else if (c->size <= 4) OPS_NVLS(false, 4);
        else OPS_NVLS(false, 8);
      }
#undef OPS_NVLS
      return check_launch("all_reduce(nvls)");
    }
    // zero-copy: the partial already lies in this rank's direct region (the producing kernel wrote it there)
    const char *direct = region_direct(c->peers[c->rank], c->region_bytes);
    const bool in_direct = (const char *)src >= direct && (const char *)src + bytes <= direct + c->region_bytes;
    const unsigned long long off = in_direct ? (unsigned long long)((const char *)src - direct) : 0ull;
#define OPS_TWO_SHOT_P(DIRECT, ADD, P) \
  all_reduce_two_shot_kernel<T, DIRECT, ADD, P><<<(unsigned)ctas, P2P_TWO_SHOT_THREADS, 0, s>>>(a, (const uint4 *)src, (uint4 *)dst, vecs, part, off)
#define OPS_TWO_SHOT(DIRECT, ADD)                          \
  do {                                                     \
    if (c->size <= 2) OPS_TWO_SHOT_P(DIRECT, ADD, 2);      \
    else if (c->size <= 4) OPS_TWO_SHOT_P(DIRECT, ADD, 4); \
    else OPS_TWO_SHOT_P(DIRECT, ADD, 8);                   \
  } while (0)
    if (in_direct && add) OPS_TWO_SHOT(true, true);
    else if (in_direct) OPS_TWO_SHOT(true, false);
    else if (add) OPS_TWO_SHOT(false, true);
    else OPS_TWO_SHOT(false, false);
#undef OPS_TWO_SHOT
#undef OPS_TWO_SHOT_P
  }
  return check_launch("all_reduce(p2p)");
}

static int all_reduce_impl(const ops_all_reduce *op, const ops_all_reduce_args *args, bool add, cudaStream_t s) {
  ops_comm *c = op->comm;
  AllReduceMeta m;
  OPS_TRY(all_reduce_meta(args, &m));
  const usz bytes = m.len * dt_size(m.dt);
  if (bytes == 0) return OPS_OK;
  void *dst = args->pair.dst_base;
  const void *src = args->pair.src_base;
  if (!dst || !src) return fail(OPS_DYNAMIC_NOT_SUPPORT, "all_reduce: null base pointer at launch");
  if (add && dst == src) return fail(OPS_ARGS_NOT_SUPPORT, "all_reduce_add: dst and src must be different buffers");
  cudaSetDevice(c->device);
  if (c->size == 1 && !add) {
    // single rank: NonAllReduce, a plain copy unless in place (operators/src/lib.rs:199-224)
    if (dst != src) {
      OpBase base{c->device, c->sm_count};
      return rearrange_enqueue(base, &args->pair, s);
    }
    return OPS_OK;
  }
  int algo = op->algo;
  const bool p2p_dt = m.dt == OPS_DT_F16 || m.dt == OPS_DT_BF16 || m.dt == OPS_DT_F32;
  const bool p2p_able = (c->p2p_ready || c->loopback) && args->op == OPS_REDUCE_SUM && p2p_dt && bytes % 16 == 0 && aligned(dst, 16) && aligned(src, 16) &&
                        bytes <= c->region_bytes;
  if (add) {
    // the residual enters the sum inside the two-shot kernel; there is no NCCL form of it
    if (!p2p_able || c->size < 2)
      return fail(OPS_ARGS_NOT_SUPPORT, "all_reduce_add: needs >= 2 ranks, an attached staging buffer of >= %zu bytes, f16/bf16/f32 Sum, 16-byte aligned data", bytes);
    algo = OPS_ALL_REDUCE_P2P_TWO_SHOT;
  }
  // a partial that already lies in the attached multicast buffer is reduced inside the switch whatever its size
  const bool in_nvls = c->nvls_mc && (const char *)src >= c->nvls_local && (const char *)src + bytes <= c->nvls_local + c->nvls_region;
  if (algo == OPS_ALL_REDUCE_AUTO && in_nvls && p2p_able) algo = OPS_ALL_REDUCE_P2P_TWO_SHOT;
  if (algo == OPS_ALL_REDUCE_AUTO) algo = p2p_able ? choose_algo(c->size, bytes) : OPS_ALL_REDUCE_NCCL;
  if (algo == OPS_ALL_REDUCE_NCCL) {
    if (!c->has_nccl) return fail(OPS_EXECUTION_FAILED, "all_reduce: communicator has no NCCL handle");
    ncclDataType_t t;
    ncclRedOp_t o;
    if (!nccl_types(m.dt, args->op, &t, &o)) return fail(OPS_TYPE_NOT_SUPPORT, "all_reduce: dtype %u / op %u not supported by NCCL", m.dt, args->op);
    NcclApi &n = nccl_api();
    ncclResult_t r = n.AllReduce(src, dst, m.len, t, o, c->nccl, s);
    if (r != ncclSuccess) return fail(OPS_EXECUTION_FAILED, "ncclAllReduce: %s", n.GetErrorString(r));
    return OPS_OK;
  }
  if (!p2p_able) return fail(OPS_ARGS_NOT_SUPPORT, "all_reduce: the peer-to-peer path needs an attached staging buffer of >= %zu bytes, f16/bf16/f32 Sum, 16-byte aligned data", bytes);
  if (m.dt == OPS_DT_F16) return launch_p2p<__half>(c, algo, src, dst, bytes, add, s);
  if (m.dt == OPS_DT_BF16) return launch_p2p<__nv_bfloat16>(c, algo, src, dst, bytes, add, s);
  return launch_p2p<float>(c, algo, src, dst, bytes, add, s);
}

OPS_API int ops_all_reduce_launch(const ops_all_reduce *op, const ops_all_reduce_args *args, void *ws, size_t ws_len, void *stream) {
  (void)ws;
  (void)ws_len;
  return all_reduce_impl(op, args, false, (cudaStream_t)stream);
}

// dst <- dst + sum over ranks of src, one kernel: the all_reduce of a row-parallel projection with the residual add that
// follows it folded in (the crate chains all_reduce and add, operators/src/add/common_cpu/mod.rs:29-75).
OPS_API int ops_all_reduce_add_launch(const ops_all_reduce *op, const ops_all_reduce_args *args, void *stream) {
  return all_reduce_impl(op, args, true, (cudaStream_t)stream);
}

// The zero-copy input region of this rank: a kernel that writes its partial here (same offset on every rank) lets
// ops_all_reduce_launch / ops_all_reduce_add_launch skip their copy-in when they are given that pointer as src.
OPS_API int ops_comm_p2p_direct(ops_comm *c, void **ptr_out, size_t *bytes_out) {
  if (!c || !c->staging) return fail(OPS_ARGS_NOT_SUPPORT, "p2p: no staging buffer exported");
  if (ptr_out) *ptr_out = region_direct(c->staging, c->region_bytes);
  if (bytes_out) *bytes_out = c->region_bytes;
  return OPS_OK;
}

// In-switch reduction: `local` is this rank's address of a buffer of `bytes` bytes that the caller has bound to an NVLink
// multicast object together with the same-sized buffers of all ranks (same order of ranks as this communicator), `multicast`
// its multicast address.  The first half is the zero-copy input region (what ops_comm_p2p_direct is to the peer-to-peer
// kernels): an all_reduce whose src lies there is reduced inside the switch.  The second half is reserved.  Needs the
// peer-to-peer staging buffer attached as well (its flags synchronise the ranks).  Pass nulls to detach.
OPS_API int ops_comm_nvls_attach(ops_comm *c, void *multicast, void *local, size_t bytes) {
  if (!c) return fail(OPS_ARGS_NOT_SUPPORT, "null communicator");
  if (!multicast || !local || bytes == 0) {
    c->nvls_mc = c->nvls_local = nullptr;
    c->nvls_region = 0;
    return OPS_OK;
  }
  if (!c->p2p_ready) return fail(OPS_ARGS_NOT_SUPPORT, "nvls: attach the peer-to-peer staging buffer first");
  if (!aligned(multicast, 16) || !aligned(local, 16) || bytes % 512) return fail(OPS_ARGS_NOT_SUPPORT, "nvls: 16-byte aligned addresses and a multiple of 512 bytes expected");
  c->nvls_mc = (char *)multicast;
  c->nvls_local = (char *)local;
  c->nvls_region = bytes / 2;
  return OPS_OK;
}

// After a bounded wait has run out (ops_comm_p2p_status != 0) the ranks' epochs and flags no longer agree.  Once every
// rank's streams are idle and the ranks have met at a host-side barrier, each rank calls this to start over: status word,
// launch counter and every flag go back to zero.  Outputs of the launch that timed out are undefined.
OPS_API int ops_comm_p2p_reset(ops_comm *c) {
  if (!c) return fail(OPS_ARGS_NOT_SUPPORT, "null communicator");
  cudaSetDevice(c->device);
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess && c->staging) e = cudaMemset(c->staging, 0, sizeof(P2PFlags));
  if (e == cudaSuccess) e = cudaMemset(c->status_dev, 0, sizeof(int));
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return fail(OPS_EXECUTION_FAILED, "p2p reset: %s", cudaGetErrorString(e));
  return OPS_OK;
}

// ------------------------------------------------------------------------------------------------
// broadcast — broadcast::Args (operators/src/broadcast/args.rs:7-75): root's src bytes land in every rank's dst.
// One ncclBroadcast on the caller's stream (operators/src/broadcast/nccl/mod.rs:53-58); a single rank copies.
// ------------------------------------------------------------------------------------------------
struct ops_broadcast {
  ops_comm *comm;
};

OPS_API int ops_broadcast_create(ops_comm *node, ops_broadcast **out) {
  if (!node || !out) return fail(OPS_ARGS_NOT_SUPPORT, "null communicator or out pointer");
  ops_broadcast *h = new ops_broadcast();
  h->comm = node;
  *out = h;
  return OPS_OK;
}

OPS_API void ops_broadcast_destroy(ops_broadcast *op) { delete op; }

OPS_API int ops_broadcast_scheme(ops_broadcast *op, const ops_broadcast_args *args, size_t max_ws, size_t *ws_out) {
  (void)op;
  (void)max_ws;
  (void)args;
  if (ws_out) *ws_out = 0;
  return OPS_OK;
}

OPS_API int ops_broadcast_launch(const ops_broadcast *op, const ops_broadcast_args *args, void *ws, size_t ws_len, void *stream) {
  (void)ws;
  (void)ws_len;
  ops_comm *c = op->comm;
  cudaStream_t s = (cudaStream_t)stream;
  ops_all_reduce_args as_pair{args->pair, OPS_REDUCE_SUM};
  AllReduceMeta m;
  OPS_TRY(all_reduce_meta(&as_pair, &m));  // same layout rules: both sides one contiguous run of equal length
  const usz bytes = m.len * dt_size(m.dt);
  if (args->root >= (size_t)c->size) return fail(OPS_ARGS_NOT_SUPPORT, "broadcast: root %zu outside a group of %d", args->root, c->size);
  if (bytes == 0) return OPS_OK;
  void *dst = args->pair.dst_base;
  const void *src = args->pair.src_base;
  if (!dst || ((int)args->root == c->rank && !src)) return fail(OPS_DYNAMIC_NOT_SUPPORT, "broadcast: null base pointer at launch");
  cudaSetDevice(c->device);
  if (c->size == 1) {
    if (dst != src) {
      OpBase base{c->device, c->sm_count};
      return rearrange_enqueue(base, &args->pair, s);
    }
    return OPS_OK;
  }
  if (!c->has_nccl) return fail(OPS_EXECUTION_FAILED, "broadcast: communicator has no NCCL handle");
  NcclApi &n = nccl_api();
  ncclResult_t r = n.Broadcast(src ? src : dst, dst, bytes, ncclUint8, (int)args->root, c->nccl, s);
  if (r != ncclSuccess) return fail(OPS_EXECUTION_FAILED, "ncclBroadcast: %s", n.GetErrorString(r));
  return OPS_OK;
}
