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
constexpr int kCommMaxBlocks = 128;
constexpr int kFlagBytes = 64 * 1024;   // [2 barriers][kCommMaxBlocks][kCommMaxRanks] uint32 + spare
constexpr int kPartialBytes = 1024 * 1024;  // sum-of-squares partials [256 slots][ranks][blocks] fp32

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
// at [sq_slot][rank][block].
void comm_all_reduce(const CommCtx& c, uint64_t off, int64_t n, int dtype, int op, bool use_mc, int sq_slot,
                     uint32_t generation, int blocks, cudaStream_t stream);
// The launchers below work on ordinary LOCAL tensors (`in`, `out`, `buf`: 16-byte aligned, byte size a multiple of 16)
// and use the symmetric staging area at `off` / `dst_off` as the exchange medium, all inside one kernel launch.
void comm_all_reduce_fused(const CommCtx& c, uint64_t off, const void* in, void* out, int64_t n, int dtype, int op,
                           bool use_mc, bool oneshot, int blocks, cudaStream_t stream);
// all_gather: out[r * n + i] = rank r's in[i]; staging needs world * n elements.
void comm_all_gather(const CommCtx& c, uint64_t dst_off, const void* in, void* out, int64_t n, int dtype, bool use_mc,
                     int blocks, cudaStream_t stream);
// reduce_scatter: in holds world * n elements, out receives reduce over ranks of slice [rank]; staging world * n.
void comm_reduce_scatter(const CommCtx& c, uint64_t off, const void* in, void* out, int64_t n, int dtype, int op,
                         bool use_mc, int blocks, cudaStream_t stream);
// all_to_all: in/out hold world chunks of n elements; staging world * n.
void comm_all_to_all(const CommCtx& c, uint64_t dst_off, const void* in, void* out, int64_t n, int dtype, int blocks,
                     cudaStream_t stream);
// broadcast (in place on buf) from rank `src`; staging n elements.
void comm_broadcast(const CommCtx& c, uint64_t off, void* buf, int64_t n, int dtype, int src, bool use_mc, int blocks,
                    cudaStream_t stream);
// Segments of the symmetric allocation for the sharded-training collectives: segment s holds `world` equal chunks
// of nvec[s] 16-byte vectors at byte offset off[s] (chunk r = rank r's shard); out[s] is a local fp32 destination.
constexpr int kCommMaxSegments = 8;
struct CommSegments {
  int n;
  uint64_t off[kCommMaxSegments];
  int64_t nvec[kCommMaxSegments];
  void* out[kCommMaxSegments];
};
// In place: every rank's own chunk of every segment is replicated into all peers' copies (no staging, no copy-out).
void comm_all_gather_inplace(const CommCtx& c, const CommSegments& segs, bool use_mc, int blocks, cudaStream_t stream);
// fp32: out[s] = op over ranks of chunk `rank` of segment s, read straight from the peers' copies; with sq_slot >= 0
// the sum of squares of this rank's results goes to every rank's partial table at [sq_slot][rank][block].
void comm_reduce_scatter_symm(const CommCtx& c, const CommSegments& segs, int op, bool use_mc, int sq_slot, int blocks,
                              cudaStream_t stream);

// cross-rank barrier only (also the bounded-wait self test: with world == 1 and pretend_world > 1 nothing ever
// arrives and the kernel records kErrPeerFlagWait).
// `phase` picks the flag row: 0 and 1 belong to the collectives above, 4 and 6 to the fused GEMMs, so a barrier that
// may run on another stream at the same time as those (the embedding-row exchange of DDP) uses 2 and 3.
void comm_barrier(const CommCtx& c, int phase, int pretend_world, cudaStream_t stream);

// Fused compute + collective tcgen05 GEMMs (gemm_sm100.cu).
// ag_gemm: C[M, N] = concat_ranks(A_r)[M, K] * B[N, K]^T.  A_r ([M/world, K] bf16) sits at byte offset a_off of every
// rank's symmetric allocation; the assembled A ([M, K] bf16) is written at byte offset g_off of every rank's
// allocation (each rank pushes its shard to all); `epoch` is the 1-based count of ag_gemm calls made on this
// communicator (the arrival words compare against it).
int ag_gemm_bf16(const CommCtx& c, uint64_t a_off, uint64_t g_off, uint32_t epoch, const void* B, void* C, int M, int N,
                 int K, int64_t ldb, int64_t ldc, bool b_mn, int num_sms, cudaStream_t stream);
int gemm_rs_bf16(const CommCtx& c, const void* A, const void* B, uint64_t c_off, int M, int N, int K, int64_t lda,
                 int64_t ldb, bool b_mn, int num_sms, cudaStream_t stream);
// b_mn: B is stored [K, N] (MN-major) instead of [N, K].

}  // namespace tb
