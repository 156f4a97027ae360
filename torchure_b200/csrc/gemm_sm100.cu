// Persistent warp-specialised bf16 GEMM for sm_100a: TMA -> shared-memory ring -> tcgen05.mma into
// TMEM -> tcgen05.ld epilogue -> TMA store.
//
//   CTA tile 128 x 256 x 64, 4 pipeline stages (48 KB each), 192 threads:
//     warp 0      TMA producer (one elected lane)
//     warp 1      TMEM allocator + MMA issuer (one elected lane issues tcgen05.mma / tcgen05.commit)
//     warps 2..5  epilogue: each owns the 32 TMEM lanes its warp id maps to (warp_id % 4), converts
//                 64-column slabs to bf16 (or 32-column slabs to fp32), stages them in shared memory in
//                 the 128-byte swizzle and writes them with its own TMA store (or TMA reduce-add)
//   Two 256-column accumulators fill the 512 TMEM columns, so the epilogue of tile i overlaps the
//   main loop of tile i+1.  One CTA per SM, tiles assigned round-robin, M fastest so that concurrently
//   running CTAs share the same weight tile in L2.
//
// Operands may be K-major or MN-major (transposed in memory); that covers forward (x W^T), dgrad
// (dy W) and wgrad (dy^T x) without any transpose kernel.  Edges are handled by TMA (zero fill on
// loads, clipping on stores); every coordinate passed to TMA is a multiple of 32 elements.
#include "api.h"
#include "comm_device.cuh"
#include "common.cuh"

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>

namespace tb {

namespace {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;            // 16 KB
constexpr int B_BYTES = BN * BK * 2;            // 32 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;  // 48 KB
constexpr int EPI_BUF = 4096;                   // 32 rows x 128 B
constexpr int EPI_BYTES = 4 * 2 * EPI_BUF;
constexpr int BAR_BYTES = 256;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + BAR_BYTES + 1024;
constexpr int NUM_THREADS = 192;
constexpr uint32_t TMEM_COLS = 512;

// Fused GEMM + collective: per-rank tensor maps over the same symmetric buffer on every peer.
//   COMM == 1  all-gather -> GEMM: A row-block r lives on rank r.  Every remote row crosses NVLink once: the
//              kernel runs four extra copy warps per CTA that push this rank's shard into the gathered copy of every
//              rank (multimem.st through the switch, or one posted store per peer; 32-row segments round-robin over
//              CTAs) and then set the segment's arrival word on every peer; tiles are ordered local rows first, so
//              the tensor cores start at once, and the TMA producer of a tile on remote rows waits (bounded) for the
//              owner's arrival words.
//              The gathered copy is an output too (the backward pass needs it for the weight gradient).
//   COMM == 2  GEMM -> reduce-scatter: C row-block r belongs to rank r; every CTA adds its partial tiles into the
//              owner's fp32 buffer with TMA reduce-add over NVLink.
struct GemmComm {
  CUtensorMap maps[kCommMaxRanks];
  CommCtx c;
  int rows_per_rank;
  // COMM == 1 only
  uint64_t a_off;       // byte offset of the A shard inside every rank's symmetric allocation
  uint64_t g_off;       // byte offset of the gathered [M, K] bf16 copy inside every rank's symmetric allocation
  uint32_t* ready;      // [row block][segment]: epoch of the last call whose copy of that segment is complete
  uint32_t epoch;       // this call's epoch (1-based, monotonic per communicator)
};

constexpr int kAgMaxRowBlocks = 2048;      // arrival words live at [32 KiB, 64 KiB) of the flag area
constexpr uint64_t kAgReadyOffset = 32768;
constexpr int kAgSeg = 4;                  // copy segments per 128-row block
constexpr int kAgSegRows = BM / kAgSeg;    // 32 rows
static_assert(kAgSeg == 4, "the consumer polls a block's arrival words with one 16-byte load");
constexpr int kAgUnroll = 16;              // 16-byte loads in flight per thread
constexpr int kAgThreads = NUM_THREADS + 128;  // the all-gather kernel adds four copy warps (6..9)

struct V4u { uint32_t x, y, z, w; };
__device__ __forceinline__ V4u local_ld16(const void* p) {
  V4u v;
  asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void peer_st16(void* p, const V4u& v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void mc_st16(void* p, const V4u& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Gather phase of the all-gather -> GEMM kernel, run by the four copy warps (128 threads) of every CTA: PUSH this
// rank's own shard into the gathered copy of every rank (posted stores need no round trip, unlike peer loads).
// With a multicast mapping one multimem.st reaches all ranks through the switch; otherwise one store per peer.
// Items = (row block of my shard, 32-row segment), round-robin over CTAs, in the order the peers consume them.
// After a segment is written everywhere, its arrival word on every peer is set to this call's epoch.
__device__ __forceinline__ void ag_copy_phase(const GemmComm* gc, int K, int tid) {
  const CommCtx& c = gc->c;
  const int bpr = gc->rows_per_rank / BM;  // row blocks per rank
  const int items = bpr * kAgSeg;
  const int64_t row_bytes = static_cast<int64_t>(K) * 2;
  const int64_t seg_bytes = row_bytes * kAgSegRows;
  // a multicast store also comes back to the sender, which at two ranks doubles the inbound traffic for nothing
  const bool use_mc = c.mc_buf != 0 && c.world > 2;
  for (int it = blockIdx.x; it < items; it += gridDim.x) {
    const int j = it / kAgSeg, seg = it % kAgSeg;
    const int mb = c.rank * bpr + j;  // global row block
    const uint8_t* src = reinterpret_cast<const uint8_t*>(c.peer_bufs[c.rank] + gc->a_off) +
                         (static_cast<int64_t>(j) * BM + seg * kAgSegRows) * row_bytes;
    const uint64_t dst_off = gc->g_off + (static_cast<int64_t>(mb) * BM + seg * kAgSegRows) * row_bytes;
    for (int64_t off = static_cast<int64_t>(tid) * 16; off < seg_bytes; off += 128 * 16 * kAgUnroll) {
      V4u v[kAgUnroll];
#pragma unroll
      for (int u = 0; u < kAgUnroll; ++u) {
        const int64_t o = off + static_cast<int64_t>(u) * 128 * 16;
        if (o < seg_bytes) v[u] = local_ld16(src + o);
      }
      if (use_mc) {
#pragma unroll
        for (int u = 0; u < kAgUnroll; ++u) {
          const int64_t o = off + static_cast<int64_t>(u) * 128 * 16;
          if (o < seg_bytes) mc_st16(reinterpret_cast<void*>(c.mc_buf + dst_off + o), v[u]);
        }
      } else {
        for (int p = 0; p < c.world; ++p) {
          uint8_t* dst = reinterpret_cast<uint8_t*>(c.peer_bufs[p] + dst_off);
#pragma unroll
          for (int u = 0; u < kAgUnroll; ++u) {
            const int64_t o = off + static_cast<int64_t>(u) * 128 * 16;
            if (o < seg_bytes) peer_st16(dst + o, v[u]);
          }
        }
      }
    }
    fence_proxy_async_all();  // the consumers read these bytes through TMA
    __threadfence_system();
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (tid < c.world && tid != c.rank) {
      uint32_t* flag = reinterpret_cast<uint32_t*>(c.peer_bufs[tid] + kAgReadyOffset) + mb * kAgSeg + seg;
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(gc->epoch) : "memory");
    }
  }
}

template <bool A_MN, bool B_MN, int OUT, int COMM>
__device__ __forceinline__ void gemm_body(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, int M,
                                          int N, int K, int splits, int* err, const GemmComm* gc) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi = smem + STAGES * STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi + EPI_BYTES);
  uint64_t* full = bars;                  // [STAGES]
  uint64_t* empty = bars + STAGES;        // [STAGES]
  uint64_t* tfull = bars + 2 * STAGES;    // [2]
  uint64_t* tempty = bars + 2 * STAGES + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (M + BM - 1) / BM;
  const int num_n = (N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (K + BK - 1) / BK;
  // split-K: work unit u = (tile u % num_tiles, K slice u / num_tiles); slices add into C with TMA reduce-add
  const int num_units = num_tiles * splits;
  const int kb_per = (num_kb + splits - 1) / splits;
  // tile -> (m0, n0).  Default: M fastest, so that concurrently running CTAs share a weight tile in L2.
  // COMM == 1: grouped by owning rank, this rank's rows first, then the peers' in ring order (all N columns of a
  // group before the next group), so that no tile on remote rows is visited before every local tile was handed out.
  const int bpr = (COMM == 1) ? gc->rows_per_rank / BM : 1;
  auto tile_coords = [&](int tile, int& m0, int& n0) {
    if (COMM == 1) {
      const int per_group = bpr * num_n;
      const int g = tile / per_group, rem = tile - g * per_group;
      int owner = g + gc->c.rank;
      if (owner >= gc->c.world) owner -= gc->c.world;
      n0 = (rem / bpr) * BN;
      m0 = (owner * bpr + rem % bpr) * BM;
    } else {
      m0 = (tile % num_m) * BM;
      n0 = (tile / num_m) * BN;
    }
  };

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 128);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  bool peers_ok = true;
  if (COMM != 0) peers_ok = block_barrier(gc->c, 4, gc->c.world);  // every peer's operand / zeroed output is in place

  if (!peers_ok) {
    // a peer never showed up: skip the work, fall through to the teardown
  } else if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x) {
        const int tile = unit % num_tiles;
        const int kb0 = (unit / num_tiles) * kb_per;
        const int kb1 = min(num_kb, kb0 + kb_per);
        int m0, n0;
        tile_coords(tile, m0, n0);
        int owner = 0;
        if (COMM == 1) {
          owner = m0 / gc->rows_per_rank;
          if (owner != gc->c.rank) {
            // the gathered copy of this row block must be complete (bounded wait)
            // one 16-byte relaxed load covers the block's four arrival words (peers write them into this GPU's
            // memory, so the poll is an L2 hit); a single acquire fence follows once all four carry this epoch
            const uint32_t* flag = gc->ready + (m0 / BM) * kAgSeg;
            const uint64_t t0 = globaltimer_ns();
            for (;;) {
              uint32_t f0, f1, f2, f3;
              asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                           : "=r"(f0), "=r"(f1), "=r"(f2), "=r"(f3) : "l"(flag) : "memory");
              const uint32_t e = gc->epoch;
              if (static_cast<int32_t>(f0 - e) >= 0 && static_cast<int32_t>(f1 - e) >= 0 &&
                  static_cast<int32_t>(f2 - e) >= 0 && static_cast<int32_t>(f3 - e) >= 0) break;
              if (*reinterpret_cast<volatile int*>(err) != 0) { ok = false; break; }
              if (globaltimer_ns() - t0 > gc->c.wait_limit_ns) { atomicCAS(err, 0, kErrPeerFlagWait); ok = false; break; }
              __nanosleep(100);
            }
            if (!ok) break;
            asm volatile("fence.acq_rel.sys;" ::: "memory");
            fence_proxy_async_all();
          }
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, err, kErrProducerEmptyWait)) { ok = false; break; }
          uint8_t* sA = smem + stage * STAGE_BYTES;
          uint8_t* sB = sA + A_BYTES;
          mbar_expect_tx(&full[stage], STAGE_BYTES);
          const int k0 = kb * BK;
          if (COMM == 1 && owner == gc->c.rank) {
            tma_load_2d(sA, &gc->maps[owner], &full[stage], k0, m0 - owner * gc->rows_per_rank);  // my own shard
          } else if (!A_MN) {
            tma_load_2d(sA, &tmA, &full[stage], k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(sA + j * 8192, &tmA, &full[stage], m0 + j * 64, k0);
          }
          if (!B_MN) {
            tma_load_2d(sB, &tmB, &full[stage], k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(sB + j * 8192, &tmB, &full[stage], n0 + j * 64, k0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      constexpr uint32_t a_lbo = A_MN ? 8192u : 16u, b_lbo = B_MN ? 8192u : 16u;
      constexpr uint32_t a_step = A_MN ? (2048u >> 4) : (32u >> 4);  // descriptor advance per k=16
      constexpr uint32_t b_step = B_MN ? (2048u >> 4) : (32u >> 4);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x) {
        const int kb0 = (unit / num_tiles) * kb_per;
        const int kb1 = min(num_kb, kb0 + kb_per);
        if (kb0 >= kb1) continue;  // empty K slice: every role skips it
        const int acc = it & 1;
        if (!mbar_wait(&tempty[acc], ((it >> 1) & 1) ^ 1, err, kErrMmaTmemEmptyWait)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full[stage], phase, err, kErrMmaFullWait)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * STAGE_BYTES);
          const uint64_t da = make_desc_sw128(a_addr, a_lbo, 1024);
          const uint64_t db = make_desc_sw128(a_addr + A_BYTES, b_lbo, 1024);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            umma_f16_ss(d_tmem, da + static_cast<uint64_t>(k * a_step), db + static_cast<uint64_t>(k * b_step), idesc,
                        (kb != kb0 || k != 0) ? 1u : 0u);
          }
          umma_commit(&empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tfull[acc]);
        ++it;
      }
    }
  } else if (warp >= 6) {
    // ------------------------------ copy warps (COMM == 1 only) ---------------
    if (COMM == 1) ag_copy_phase(gc, K, threadIdx.x - NUM_THREADS);
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    uint8_t* buf0 = epi + q * 2 * EPI_BUF;
    constexpr int COLS = (OUT == 0) ? 64 : 32;  // columns per staged slab (128 B per row)
    int it = 0;
    int slab = 0;
    bool ok = true;
    for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x) {
      const int tile = unit % num_tiles;
      if ((unit / num_tiles) * kb_per >= num_kb) continue;  // empty K slice
      int m0, n0;
      tile_coords(tile, m0, n0);
      const int acc = it & 1;
      if (!mbar_wait(&tfull[acc], (it >> 1) & 1, err, kErrEpilogueTmemFullWait)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      const bool rows_live = (m0 + q * 32) < M;
#pragma unroll 1
      for (int c = 0; c < BN / COLS; ++c) {
        uint32_t v[64];
        if (OUT == 0) {
          tmem_ld_32x32b_x32(t_row + c * 64, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
          tmem_ld_32x32b_x32(t_row + c * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
        } else {
          tmem_ld_32x32b_x32(t_row + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
        }
        tmem_ld_wait();
        if (c == BN / COLS - 1) {
          // the accumulator is in registers: hand it back to the MMA warp
          tc_fence_before();
          mbar_arrive(&tempty[acc]);
        }
        const bool live = rows_live && (n0 + c * COLS) < N;
        if (live) {
          uint8_t* buf = buf0 + (slab & 1) * EPI_BUF;
          ++slab;
          if (lane == 0) tma_wait_group_read<1>();  // the store that last used this buffer has read it
          __syncwarp();
          uint8_t* row = buf + lane * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4 pk;
            if (OUT == 0) {
              pk.x = pack_bf16x2(__uint_as_float(v[8 * j + 0]), __uint_as_float(v[8 * j + 1]));
              pk.y = pack_bf16x2(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
              pk.z = pack_bf16x2(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
              pk.w = pack_bf16x2(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
            } else {
              pk.x = v[4 * j + 0]; pk.y = v[4 * j + 1]; pk.z = v[4 * j + 2]; pk.w = v[4 * j + 3];
            }
            *reinterpret_cast<uint4*>(row + ((j ^ (lane & 7)) << 4)) = pk;
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (COMM == 2) {
              const int owner = m0 / gc->rows_per_rank;
              tma_reduce_add_2d(&gc->maps[owner], buf, n0 + c * COLS, m0 - owner * gc->rows_per_rank + q * 32);
            } else if (OUT == 2) {
              tma_reduce_add_2d(&tmC, buf, n0 + c * COLS, m0 + q * 32);
            } else {
              tma_store_2d(&tmC, buf, n0 + c * COLS, m0 + q * 32);
            }
            tma_commit_group();
          }
        }
      }
      ++it;
    }
    if (lane == 0) tma_wait_group<0>();
  }

  // ------------------------------ teardown ------------------------------------
  if (*reinterpret_cast<volatile int*>(err) != 0) {
    // a wait expired somewhere: give copies and MMAs in flight time to land before TMEM is released
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  if (COMM == 2 && peers_ok) block_barrier(gc->c, 6, gc->c.world);  // every peer's adds have landed
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <bool A_MN, bool B_MN, int OUT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, int M, int N, int K, int splits, int* err) {
  pdl_wait();
  pdl_launch_dependents();
  gemm_body<A_MN, B_MN, OUT, 0>(tmA, tmB, tmC, M, N, K, splits, err, nullptr);
}

template <int COMM, bool B_MN>
__global__ void __launch_bounds__(COMM == 1 ? kAgThreads : NUM_THREADS, 1)
gemm_comm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const __grid_constant__ GemmComm gc, int M, int N, int K,
                 int* err) {
  // COMM 1: bf16 store of C; COMM 2: fp32 reduce-add of C into the owners
  gemm_body<false, B_MN, COMM == 1 ? 0 : 2, COMM>(tmA, tmB, tmC, M, N, K, 1, err, &gc);
}

// ---- host side --------------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(p);
  });
  return fn;
}

}  // namespace

// 2-D row-major tensor [rows, cols] with row stride `ld` elements, box [box_rows, box_cols], 128B swizzle.
// Encoding a tensor map costs several microseconds on the host; activations and weights come back at the same
// addresses step after step, so encoded maps are cached by their full description.
namespace {
struct TmapKey {
  const void* base; uint64_t rows, cols, ld; uint32_t box_rows, box_cols; int elem_bytes;
  bool operator==(const TmapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows &&
           box_cols == o.box_cols && elem_bytes == o.elem_bytes;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    uint64_t h = reinterpret_cast<uint64_t>(k.base) * 0x9E3779B97F4A7C15ull;
    h ^= (k.rows + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
    h ^= (k.cols * 31 + k.ld * 131 + k.box_rows * 7 + k.box_cols * 3 + k.elem_bytes + (h << 6) + (h >> 2));
    return static_cast<size_t>(h);
  }
};
}  // namespace

int make_tmap_2d(CUtensorMap* map, const void* base, int elem_bytes, uint64_t rows, uint64_t cols, uint64_t ld,
                 uint32_t box_rows, uint32_t box_cols) {
  static thread_local std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  const TmapKey key{base, rows, cols, ld, box_rows, box_cols, elem_bytes};
  auto hit = cache.find(key);
  if (hit != cache.end()) {
    std::memcpy(map, &hit->second, sizeof(CUtensorMap));
    return 0;
  }
  EncodeFn fn = encode_fn();
  if (!fn) return -10;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return -11;
  if ((ld * elem_bytes) % 16 != 0) return -12;
  if (box_cols * elem_bytes != 128) return -13;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -14;
  if (cache.size() > 16384) cache.clear();
  cache.emplace(key, *map);
  return 0;
}

template <bool A_MN, bool B_MN, int OUT>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb_, const CUtensorMap& tc, int M, int N, int K, int splits,
                  int* err, int grid, cudaStream_t stream) {
  auto kern = gemm_bf16_kernel<A_MN, B_MN, OUT>;
  if (!ensure_dynamic_smem(reinterpret_cast<const void*>(kern), SMEM_BYTES)) return -20;
  return launch_pdl(kern, dim3(grid), dim3(NUM_THREADS), SMEM_BYTES, stream, ta, tb_, tc, M, N, K, splits, err) ==
                 cudaSuccess
             ? 0
             : -21;
}

// Problems with more than 128 rows run on CTA pairs (gemm2_sm100.cu) unless TORCHURE_B200_GEMM_PAIR=0.
static bool pair_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("TORCHURE_B200_GEMM_PAIR");
    return !(e && e[0] == '0');
  }();
  return on;
}

int gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
              bool a_mn, bool b_mn, int out_mode, int* err, int num_sms, cudaStream_t stream, int force_splits) {
  if (M <= 0 || N <= 0 || K <= 0) return -1;
  const bool pair = pair_enabled() && M > BM && num_sms >= 2;
  CUtensorMap ta, tb_, tc;
  int r;
  if (!pair) {
  // K-major operand [R, K]: box 64 (k) x tile rows.  MN-major operand stored [K, R]: box 64 (r) x 64 (k rows).
  r = a_mn ? make_tmap_2d(&ta, A, 2, K, M, lda, 64, 64) : make_tmap_2d(&ta, A, 2, M, K, lda, BM, 64);
  if (r) return r;
  r = b_mn ? make_tmap_2d(&tb_, B, 2, K, N, ldb, 64, 64) : make_tmap_2d(&tb_, B, 2, N, K, ldb, BN, 64);
  if (r) return r - 100;
  r = out_mode == 0 ? make_tmap_2d(&tc, C, 2, M, N, ldc, 32, 64) : make_tmap_2d(&tc, C, 4, M, N, ldc, 32, 32);
  if (r) return r - 200;
  }
  // work units and workers: 128 x 256 tiles on SMs, or 256 x 256 tiles on SM pairs
  const int tiles = ((M + (pair ? 2 : 1) * BM - 1) / ((pair ? 2 : 1) * BM)) * ((N + BN - 1) / BN);
  const int workers = pair ? (gemm_pair_capacity() > 0 ? gemm_pair_capacity() : num_sms / 2) : num_sms;
  // split-K for fp32 outputs (wgrad: few output tiles, long K): pick the slice count with the least wave time
  int splits = 1;
  const int num_kb = (K + BK - 1) / BK;
  if (force_splits > 0) {
    splits = force_splits;
  } else if (out_mode != 0 && num_kb >= 32 && tiles < 2 * workers) {
    float best = 1e30f;
    for (int s = 1; s <= 8 && s * 8 <= num_kb; ++s) {
      const int waves = (tiles * s + workers - 1) / workers;
      const float cost = static_cast<float>(waves) / s + 0.02f * (s - 1);
      if (cost < best - 1e-6f) { best = cost; splits = s; }
    }
  }
  if (splits > 1 && out_mode == 1) {
    // the slices all add into C: clear it first
    if (cudaMemset2DAsync(C, static_cast<size_t>(ldc) * 4, 0, static_cast<size_t>(N) * 4, M, stream) != cudaSuccess) return -22;
    out_mode = 2;
  }
  if (pair)
    return gemm2_bf16(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, out_mode, splits, err, num_sms, stream);
  const int units = tiles * splits;
  const int grid = units < num_sms ? units : num_sms;
#define TB_GEMM_CASE(AM, BMN, O) \
  if (a_mn == AM && b_mn == BMN && out_mode == O) return launch<AM, BMN, O>(ta, tb_, tc, M, N, K, splits, err, grid, stream);
  TB_GEMM_CASE(false, false, 0)
  TB_GEMM_CASE(false, false, 1)
  TB_GEMM_CASE(false, false, 2)
  TB_GEMM_CASE(false, true, 0)
  TB_GEMM_CASE(false, true, 1)
  TB_GEMM_CASE(true, true, 0)
  TB_GEMM_CASE(true, true, 1)
  TB_GEMM_CASE(true, true, 2)
  TB_GEMM_CASE(true, false, 0)
#undef TB_GEMM_CASE
  return -2;
}

// A_r [M/world, K] bf16 sits at byte offset a_off of every rank's symmetric allocation; B [N, K] and C [M, N] (bf16)
// are local.  C = concat_r(A_r) * B^T.
int ag_gemm_bf16(const CommCtx& c, uint64_t a_off, uint64_t g_off, uint32_t epoch, const void* B, void* C, int M, int N,
                 int K, int64_t ldb, int64_t ldc, bool b_mn, int num_sms, cudaStream_t stream) {
  if (M % (c.world * BM) != 0 || K % 8 != 0 || M / BM > kAgMaxRowBlocks) return -3;
  GemmComm gc{};
  gc.c = c;
  gc.rows_per_rank = M / c.world;
  gc.a_off = a_off;
  gc.g_off = g_off;
  gc.ready = reinterpret_cast<uint32_t*>(c.peer_bufs[c.rank] + kAgReadyOffset);
  gc.epoch = epoch;
  // only the map of this rank's own shard is used (local tiles); remote rows are read from the gathered copy
  int rc = make_tmap_2d(&gc.maps[c.rank], reinterpret_cast<const void*>(c.peer_bufs[c.rank] + a_off), 2,
                        gc.rows_per_rank, K, K, BM, 64);
  if (rc) return rc;
  CUtensorMap ta, tb_, tc;
  rc = make_tmap_2d(&ta, reinterpret_cast<const void*>(c.peer_bufs[c.rank] + g_off), 2, M, K, K, BM, 64);
  if (rc) return rc - 300;
  rc = b_mn ? make_tmap_2d(&tb_, B, 2, K, N, ldb, 64, 64) : make_tmap_2d(&tb_, B, 2, N, K, ldb, BN, 64);
  if (rc) return rc - 100;
  rc = make_tmap_2d(&tc, C, 2, M, N, ldc, 32, 64);
  if (rc) return rc - 200;
  auto kern = b_mn ? gemm_comm_kernel<1, true> : gemm_comm_kernel<1, false>;
  if (!ensure_dynamic_smem(reinterpret_cast<const void*>(kern), SMEM_BYTES)) return -20;
  const int tiles = (M / BM) * ((N + BN - 1) / BN);
  const int cap = num_sms < kCommMaxBlocks ? num_sms : kCommMaxBlocks;  // the handshake has one flag row per CTA
  const int grid = tiles < cap ? tiles : cap;
  kern<<<grid, kAgThreads, SMEM_BYTES, stream>>>(ta, tb_, tc, gc, M, N, K, c.err);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

// A [M, K_local], B [N, K_local] bf16 local; the fp32 output shard [M/world, N] sits at byte offset c_off of every
// rank's symmetric allocation and must be zero on entry.  out_r = sum over ranks of (A B^T)[rows of r].
int gemm_rs_bf16(const CommCtx& c, const void* A, const void* B, uint64_t c_off, int M, int N, int K, int64_t lda,
                 int64_t ldb, bool b_mn, int num_sms, cudaStream_t stream) {
  if (M % (c.world * BM) != 0) return -3;
  GemmComm gc{};
  gc.c = c;
  gc.rows_per_rank = M / c.world;
  for (int r = 0; r < c.world; ++r) {
    int rc = make_tmap_2d(&gc.maps[r], reinterpret_cast<const void*>(c.peer_bufs[r] + c_off), 4, gc.rows_per_rank, N, N,
                          32, 32);
    if (rc) return rc;
  }
  CUtensorMap ta, tb_;
  int rc = make_tmap_2d(&ta, A, 2, M, K, lda, BM, 64);
  if (rc) return rc - 100;
  rc = b_mn ? make_tmap_2d(&tb_, B, 2, K, N, ldb, 64, 64) : make_tmap_2d(&tb_, B, 2, N, K, ldb, BN, 64);
  if (rc) return rc - 200;
  auto kern = b_mn ? gemm_comm_kernel<2, true> : gemm_comm_kernel<2, false>;
  if (!ensure_dynamic_smem(reinterpret_cast<const void*>(kern), SMEM_BYTES)) return -20;
  const int tiles = (M / BM) * ((N + BN - 1) / BN);
  const int cap = num_sms < kCommMaxBlocks ? num_sms : kCommMaxBlocks;
  const int grid = tiles < cap ? tiles : cap;
  kern<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb_, gc.maps[c.rank], gc, M, N, K, c.err);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

}  // namespace tb
