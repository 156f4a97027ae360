// Host-callable launchers of the NVLink collective kernels (comm.cu).
//
// Every rank maps the same symmetric allocation: peer_bufs[p] is rank p's copy as seen from this GPU,
// mc_buf (may be null) is the NVSwitch multicast address of the allocation.  The first kFlagBytes of the
// allocation are cross-rank flags (zero before first use); data offsets passed to the launchers are
// relative to the allocation base and must be 16-byte aligned.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tb {

constexpr int kCommMaxRanks = 8;
constexpr int kCommMaxBlocks = 64;
constexpr int kFlagBytes = 64 * 1024;   // [2 barriers][kCommMaxBlocks][kCommMaxRanks] uint32 + spare
constexpr int kPartialBytes = 512 * 1024;  // sum-of-squares partials [256 slots][ranks][blocks] fp32

struct CommCtx {
  uint64_t peer_bufs[kCommMaxRanks];  // device-visible base address of every rank's allocation
  uint64_t mc_buf;                    // multicast base or 0
  int rank;
  int world;
  int* err;               // device error word
  uint64_t wait_limit_ns;  // bound of every flag wait
  uint32_t* grid_counter;  // local (not symmetric) monotonically increasing grid-barrier counter
};

enum CommOp : int { kOpSum = 0, kOpAvg = 1, kOpMax = 2, kOpMin = 3 };
enum CommDtype : int { kF32 = 0, kBF16 = 1 };

// In-place all-reduce of `n` elements at byte offset `off` of the symmetric allocation (two-shot: every rank
// reduces its 1/world slice and broadcasts it).  use_mc selects multimem.ld_reduce/multimem.st (sum/avg only).
// sq_slot >= 0: the sum of squares of this rank's reduced fp32 slice is stored into every rank's partial table
// at [sq_slot][rank].  `generation` must increase by one per launch on a communicator.
void comm_all_reduce(const CommCtx& c, uint64_t off, int64_t n, int dtype, int op, bool use_mc, int sq_slot,
                     uint32_t generation, int blocks, cudaStream_t stream);
// One-shot all-reduce for small messages: every rank reads all peers and writes `out` (local, may be outside
// the symmetric allocation).
void comm_all_reduce_oneshot(const CommCtx& c, uint64_t off, void* out, int64_t n, int dtype, int op,
                             uint32_t generation, int blocks, cudaStream_t stream);
// all_gather: my `n` elements at `src_off` are written to offset dst_off + rank*n*elt of every rank.
void comm_all_gather(const CommCtx& c, uint64_t src_off, uint64_t dst_off, int64_t n, int dtype, bool use_mc,
                     uint32_t generation, int blocks, cudaStream_t stream);
// reduce_scatter: input of world*n elements at `off` on every rank; rank r writes reduce(slice r) to `out` (local).
void comm_reduce_scatter(const CommCtx& c, uint64_t off, void* out, int64_t n, int dtype, int op, bool use_mc,
                         uint32_t generation, int blocks, cudaStream_t stream);
// all_to_all: chunk j (n elements) of my input at src_off goes to rank j's dst_off + rank*n*elt.
void comm_all_to_all(const CommCtx& c, uint64_t src_off, uint64_t dst_off, int64_t n, int dtype,
                     uint32_t generation, int blocks, cudaStream_t stream);
// broadcast: rank `src` writes its n elements at `off` to the same offset of every rank.
void comm_broadcast(const CommCtx& c, uint64_t off, int64_t n, int dtype, int src, bool use_mc, uint32_t generation,
                    int blocks, cudaStream_t stream);
// cross-rank barrier only (also the bounded-wait self test: with world == 1 and expect_peers > 1 nothing ever
// arrives and the kernel records kErrPeerFlagWait).
void comm_barrier(const CommCtx& c, uint32_t generation, int pretend_world, cudaStream_t stream);

}  // namespace tb
