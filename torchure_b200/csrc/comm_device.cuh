// Device-side cross-rank handshake shared by the collective kernels and the fused GEMM+collective kernels.
#pragma once
#include "comm_api.h"
#include "common.cuh"

namespace tb {

__device__ __forceinline__ uint32_t* flag_ptr(uint64_t base, int phase, int block, int rank) {
  return reinterpret_cast<uint32_t*>(base) + (phase * kCommMaxBlocks + block) * kCommMaxRanks + rank;
}

__device__ __forceinline__ uint32_t cas_sys(uint32_t* addr, uint32_t cmp, uint32_t val) {
  uint32_t old;
  asm volatile("atom.acq_rel.sys.global.cas.b32 %0, [%1], %2, %3;" : "=r"(old) : "l"(addr), "r"(cmp), "r"(val) : "memory");
  return old;
}

// One thread's half of a barrier: raise my flag at `peer`, then consume the flag `peer` raised here.  Bounded; returns
// false (and records kErrPeerFlagWait) when the limit expires or an error is already recorded.
__device__ __forceinline__ bool peer_handshake(const CommCtx& c, int phase, int peer) {
  const uint64_t t0 = globaltimer_ns();
  bool ok = true;
  // raise my flag in the peer's memory (only if a peer exists; pretend-world barriers have no peer memory)
  if (peer < c.world) {
    uint32_t* theirs = flag_ptr(c.peer_bufs[peer], phase, blockIdx.x, c.rank);
    while (cas_sys(theirs, 0u, 1u) != 0u) {
      if (globaltimer_ns() - t0 > c.wait_limit_ns || *reinterpret_cast<volatile int*>(c.err) != 0) { ok = false; break; }
    }
  }
  if (ok) {
    uint32_t* mine = flag_ptr(c.peer_bufs[c.rank], phase, blockIdx.x, peer);
    while (cas_sys(mine, 1u, 0u) != 1u) {
      if (globaltimer_ns() - t0 > c.wait_limit_ns || *reinterpret_cast<volatile int*>(c.err) != 0) { ok = false; break; }
    }
  }
  if (!ok) atomicCAS(c.err, 0, kErrPeerFlagWait);
  return ok;
}

// Block-level barrier with the same block of every peer.  Returns false if a wait expired.
__device__ __forceinline__ bool block_barrier(const CommCtx& c, int phase, int world) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  __threadfence_system();
  if (threadIdx.x < world && threadIdx.x != c.rank) {
    if (!peer_handshake(c, phase, threadIdx.x)) s_fail = 1;
  }
  __syncthreads();
  return s_fail == 0;
}

}  // namespace tb
