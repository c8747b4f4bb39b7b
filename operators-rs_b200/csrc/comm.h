// comm.h — the topology node (`ops_comm`) and the layout of the peer-mapped staging buffer, shared by the
// all_reduce / broadcast operators and the GEMM that reduces its own output across ranks.
#pragma once
#include <nccl.h>

#include "common.h"
#include "device_utils.cuh"

namespace ops {

constexpr int MAX_RANKS = 8;
constexpr int P2P_MAX_CTAS = 256;
constexpr int P2P_MAX_TILE_FLAGS = 16384;  // (tile, 32-row quarter) flags of the GEMM + all_reduce kernel: up to 4096 tiles
constexpr unsigned long long P2P_WAIT_LIMIT_NS = 1000000000ull;  // 1 s

// ------------------------------------------------------------------------------------------------
// peer-to-peer state
// ------------------------------------------------------------------------------------------------
// Staging buffer of one rank: [flags | in(parity 0) | in(parity 1) | out(parity 0) | out(parity 1) | direct]
// "direct" is the zero-copy input region: a caller that lets the producing kernel write its partial there (same offset on
// every rank) spares the all_reduce its copy-in.
struct alignas(256) P2PFlags {  // the data regions start right behind it: keep them 256-byte aligned
  unsigned int ready[MAX_RANKS][P2P_MAX_CTAS];   // ready[q][b]: epoch up to which rank q's CTA b has staged its input
  unsigned int reduced[MAX_RANKS][P2P_MAX_CTAS]; // reduced[q][b]: epoch up to which rank q's CTA b has published its reduced slice
  // GEMM + all_reduce kernel: tile_ready[q][f] = epoch at which rank q stored its partial of (tile, quarter) f in its "in"
  // region (written into the OWNER's copy of this struct); tile_done[8 * tile + w] = epoch at which the owner has pushed rows
  // [16w, 16w+16) of the reduced tile into this rank's "out" region
  unsigned int tile_ready[MAX_RANKS][P2P_MAX_TILE_FLAGS];
  unsigned int tile_done[P2P_MAX_TILE_FLAGS];
  // Launch counter of this rank's peer-to-peer kernels.  It lives on the device and is advanced by the kernels themselves
  // (the last CTA of a launch to finish), never by the host: a launch that is replayed from a CUDA graph therefore sees a
  // fresh epoch every time.  Only the own copy is used; `done` counts the CTAs of the running launch that have finished.
  unsigned int epoch;
  unsigned int done;
};

static_assert(sizeof(P2PFlags) % 256 == 0, "the staging regions behind the flags must stay aligned");

constexpr int P2P_REGIONS = 5;  // in x2, out x2, direct

struct P2PHandleBlob {  // what ops_comm_p2p_export ships (<= OPS_COMM_P2P_HANDLE_BYTES)
  cudaIpcMemHandle_t mem;
  unsigned long long region_bytes;
  int rank;
  int valid;
};
static_assert(sizeof(P2PHandleBlob) <= OPS_COMM_P2P_HANDLE_BYTES, "handle blob too large");

struct P2PKernelArgs {
  char *peers[MAX_RANKS];  // peers[q]: base of rank q's staging buffer as mapped here (own buffer for q == rank)
  unsigned long long region_bytes;
  int rank, size;
  int *status;
};

}  // namespace ops

struct ops_comm {
  int device;
  int rank, size;
  ncclComm_t nccl;
  bool has_nccl;
  // p2p
  char *staging;               // own buffer (cudaMalloc)
  size_t staging_bytes;        // total allocation
  size_t region_bytes;         // bytes of each of the four data regions
  char *peers[ops::MAX_RANKS];
  bool p2p_ready;
  bool loopback;               // every peer entry is the own buffer (time-out tests on one GPU)
  int *status_dev;
  int sm_count;
  // NVLS: a buffer of 2 * nvls_region bytes ([in | out]) that the caller has bound to an NVLink multicast object — the
  // same offsets on every rank; nvls_mc is its multicast address (multimem instructions), nvls_local this rank's own copy
  char *nvls_mc, *nvls_local;
  size_t nvls_region;
};

namespace ops {

__device__ __forceinline__ void st_release_sys(unsigned int *p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int *p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_peer_16(const void *p) {  // system-scope relaxed load: never served from a stale L1 line
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long p2p_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ char *region_in(char *base, unsigned long long region, unsigned int parity) {
  return base + sizeof(P2PFlags) + (unsigned long long)parity * region;
}
__device__ __forceinline__ char *region_out(char *base, unsigned long long region, unsigned int parity) {
  return base + sizeof(P2PFlags) + (2ull + parity) * region;
}
__host__ __device__ __forceinline__ char *region_direct(char *base, unsigned long long region) { return base + sizeof(P2PFlags) + 4ull * region; }

// Epoch of the running launch: one more than the number of peer-to-peer launches this rank has completed.  Every thread
// that needs it reads it at kernel start; it only changes after the last CTA of the launch has passed p2p_launch_done().
__device__ __forceinline__ unsigned int p2p_epoch(const char *own_base) {
  return *reinterpret_cast<const volatile unsigned int *>(&reinterpret_cast<const P2PFlags *>(own_base)->epoch) + 1u;
}
// Called by ONE thread per CTA after the CTA's last use of the epoch (on every exit path, time-outs included).
__device__ __forceinline__ void p2p_launch_done(char *own_base) {
  P2PFlags *f = reinterpret_cast<P2PFlags *>(own_base);
  __threadfence();
  if (atomicAdd(&f->done, 1u) == gridDim.x * gridDim.y * gridDim.z - 1u) {
    f->done = 0;
    __threadfence();
    atomicAdd(&f->epoch, 1u);
  }
}

}  // namespace ops
