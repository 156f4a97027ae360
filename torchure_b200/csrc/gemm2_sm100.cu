// bf16 GEMM on CTA PAIRS (tcgen05.mma.cta_group::2): two CTAs of a cluster, on two SMs, compute one 256 x 256 output
// tile.  Each CTA brings its own 128 rows of A and HALF of the 256 rows of B into its shared memory; one
// instruction, issued by the leader CTA, runs both tensor cores on 256 x 256 x 16, each reading the other half of B
// from its partner.  A single CTA with a 128 x 256 tile fetches 12 KB of operands per k-step of 16 and measures 160
// cycles for it on B200 (128 would be the arithmetic); the pair fetches 8 KB per CTA and measures 128.
//
//   per CTA: 6 pipeline stages of 32 KB (A 128 x 64, B 128 x 64), 192 threads:
//     warp 0      TMA producer: its A rows and its half of B, completing on the LEADER's "full" barrier (which the
//                 leader's producer arms with the byte count of both CTAs)
//     warp 1      TMEM allocator; in the leader also the MMA issuer.  tcgen05.commit with a cluster mask releases the
//                 stage in both CTAs ("empty") and hands the accumulator to both epilogues ("tfull")
//     warps 2..5  epilogue of this CTA's 128 rows (TMEM lanes), as in the single-CTA kernel; both CTAs' epilogue
//                 threads arrive on the leader's "tempty" barrier
//   Two 256-column accumulators per CTA: the epilogue of tile i overlaps the main loop of tile i + 1.
//
// Operand layouts, output modes (bf16 store, fp32 store, fp32 reduce-add) and split-K are those of the single-CTA
// kernel in gemm_sm100.cu, which remains the path of the fused GEMM + collective kernels and of small problems.
// Every wait is bounded; the two CTAs meet at a cluster barrier before anyone touches a partner's barrier and again
// before either releases its tensor memory.
#include "api.h"
#include "common.cuh"

namespace tb {

int make_tmap_2d(CUtensorMap* map, const void* base, int elem_bytes, uint64_t rows, uint64_t cols, uint64_t ld,
                 uint32_t box_rows, uint32_t box_cols);

namespace {

constexpr int BM = 128;            // rows of A (and of the output) per CTA
constexpr int BN = 256;            // output columns of the pair's tile
constexpr int BNH = BN / 2;        // rows of B held by one CTA
constexpr int BK = 64, STAGES = 6;
constexpr int A_BYTES = BM * BK * 2;             // 16 KB
constexpr int B_BYTES = BNH * BK * 2;            // 16 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;   // 32 KB
constexpr int EPI_BUF = 4096;                    // 32 rows x 128 B
constexpr int EPI_BYTES = 4 * 2 * EPI_BUF;
constexpr int BAR_BYTES = 256;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + BAR_BYTES + 1024;
constexpr int NUM_THREADS = 192;
constexpr uint32_t TMEM_COLS = 512;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the address, in the cluster's shared window, of `local` in the CTA of rank `rank`
__device__ __forceinline__ uint32_t map_to_cta(const void* local, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_u32(local)), "r"(rank));
  return out;
}
__device__ __forceinline__ void remote_arrive(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// tiled TMA load whose completion is counted on a barrier that may live in the partner CTA (no multicast)
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t cluster_bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(cluster_bar), "r"(c0), "r"(c1)
      : "memory");
}
// D[tmem, both CTAs] (+)= A * B over the pair
__device__ __forceinline__ void umma2_f16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t accumulate) {
  const uint32_t zero = 0;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(zero)
      : "memory");
}
// the barrier at this shared-memory offset, in both CTAs, gets one arrival when every MMA issued so far has completed
__device__ __forceinline__ void umma2_commit_both(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                   smem_u32(bar)),
               "h"(mask)
               : "memory");
}

template <bool A_MN, bool B_MN, int OUT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmC, int M, int N, int K, int splits, int* err) {
  pdl_wait();
  pdl_launch_dependents();
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023);
  uint8_t* epi = smem + STAGES * STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi + EPI_BYTES);
  uint64_t* full = bars;                     // [STAGES]  used in the leader
  uint64_t* empty = bars + STAGES;           // [STAGES]  one per CTA
  uint64_t* tfull = bars + 2 * STAGES;       // [2]       one per CTA
  uint64_t* tempty = bars + 2 * STAGES + 2;  // [2]       used in the leader
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();           // 0: leader
  const int cluster = static_cast<int>(blockIdx.x) >> 1;
  const int num_clusters = static_cast<int>(gridDim.x) >> 1;
  const int num_m = (M + 2 * BM - 1) / (2 * BM);
  const int num_n = (N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (K + BK - 1) / BK;
  // split-K: work unit u = (tile u % num_tiles, K slice u / num_tiles); slices add into C with TMA reduce-add
  const int num_units = num_tiles * splits;
  const int kb_per = (num_kb + splits - 1) / splits;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);      // the leader's producer arrives, announcing the bytes of both CTAs
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 256);  // the epilogue threads of both CTAs
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    tc_fence_before();
  }
  __syncthreads();
  cluster_sync_all();   // the partner's barriers exist before anything is signalled on them
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      uint32_t lead_full_addr[STAGES];
#pragma unroll
      for (int s = 0; s < STAGES; ++s) lead_full_addr[s] = map_to_cta(&full[s], 0);
      for (int unit = cluster; unit < num_units && ok; unit += num_clusters) {
        const int tile = unit % num_tiles;
        const int kb0 = (unit / num_tiles) * kb_per;
        const int kb1 = min(num_kb, kb0 + kb_per);
        const int m0 = (tile % num_m) * 2 * BM + static_cast<int>(rank) * BM;
        const int n0 = (tile / num_m) * BN + static_cast<int>(rank) * BNH;   // the leader holds the first 128 B rows
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, err, kErrProducerEmptyWait)) { ok = false; break; }
          uint8_t* sA = smem + stage * STAGE_BYTES;
          uint8_t* sB = sA + A_BYTES;
          // Only the leader arms its barrier, with the byte count of both CTAs: the partner's copies may well land
          // first (the pending count then dips below zero until the leader's announcement arrives), and a remote
          // arrival per stage would put a cluster-scope release on the producer's critical path.
          const uint32_t lead_full = lead_full_addr[stage];
          if (rank == 0) mbar_expect_tx(&full[stage], 2 * STAGE_BYTES);
          const int k0 = kb * BK;
          if (!A_MN) {
            tma_load_2d_pair(sA, &tmA, lead_full, k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(sA + j * 8192, &tmA, lead_full, m0 + j * 64, k0);
          }
          if (!B_MN) {
            tma_load_2d_pair(sB, &tmB, lead_full, k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BNH / 64; ++j) tma_load_2d_pair(sB + j * 8192, &tmB, lead_full, n0 + j * 64, k0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader only) ------------------
    if (rank == 0 && elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN, A_MN, B_MN);
      constexpr uint32_t a_lbo = A_MN ? 8192u : 16u, b_lbo = B_MN ? 8192u : 16u;
      constexpr uint32_t a_step = A_MN ? (2048u >> 4) : (32u >> 4);  // descriptor advance per k=16
      constexpr uint32_t b_step = B_MN ? (2048u >> 4) : (32u >> 4);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int unit = cluster; unit < num_units && ok; unit += num_clusters) {
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
            umma2_f16_ss(d_tmem, da + static_cast<uint64_t>(k * a_step), db + static_cast<uint64_t>(k * b_step), idesc,
                         (kb != kb0 || k != 0) ? 1u : 0u);
          }
          umma2_commit_both(&empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma2_commit_both(&tfull[acc]);
        ++it;
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs) ----------------------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    uint8_t* buf0 = epi + q * 2 * EPI_BUF;
    constexpr int COLS = (OUT == 0) ? 64 : 32;  // columns per staged slab (128 B per row)
    int it = 0;
    int slab = 0;
    bool ok = true;
    for (int unit = cluster; unit < num_units && ok; unit += num_clusters) {
      const int tile = unit % num_tiles;
      if ((unit / num_tiles) * kb_per >= num_kb) continue;  // empty K slice
      const int m0 = (tile % num_m) * 2 * BM + static_cast<int>(rank) * BM;
      const int n0 = (tile / num_m) * BN;
      const int acc = it & 1;
      if (!mbar_wait(&tfull[acc], (it >> 1) & 1, err, kErrEpilogueTmemFullWait)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      const bool rows_live = (m0 + q * 32) < M;
      const uint32_t lead_tempty = map_to_cta(&tempty[acc], 0);
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
          // the accumulator is in registers: hand it back to the leader's MMA warp
          tc_fence_before();
          remote_arrive(lead_tempty);
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
            if (OUT == 2) tma_reduce_add_2d(&tmC, buf, n0 + c * COLS, m0 + q * 32);
            else tma_store_2d(&tmC, buf, n0 + c * COLS, m0 + q * 32);
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
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // neither CTA retires while its partner may still signal its barriers or read its operands
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// How many CTA pairs the device can hold at once.  The two CTAs of a pair sit on the two SMs of one TPC; a part with
// TPCs of which one SM is fused off holds fewer pairs than SMs / 2.  The persistent schedule hands work to exactly this
// many pairs: a pair that had to wait for a free TPC would start a whole problem late.
int g_pair_capacity = 0;

template <bool A_MN, bool B_MN, int OUT>
int launch2(const CUtensorMap& ta, const CUtensorMap& tb_, const CUtensorMap& tc, int M, int N, int K, int splits,
            int* err, int units, int num_sms, cudaStream_t stream) {
  auto kern = gemm2_bf16_kernel<A_MN, B_MN, OUT>;
  if (!ensure_dynamic_smem(reinterpret_cast<const void*>(kern), SMEM_BYTES)) return -20;
  cudaLaunchConfig_t cfg{};
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  if (g_pair_capacity == 0) {
    cudaLaunchAttribute cattr[1];
    cattr[0].id = cudaLaunchAttributeClusterDimension;
    cattr[0].val.clusterDim.x = 2;
    cattr[0].val.clusterDim.y = 1;
    cattr[0].val.clusterDim.z = 1;
    cfg.gridDim = dim3(2 * (num_sms / 2));
    cfg.attrs = cattr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) return -23;
    g_pair_capacity = n < num_sms / 2 ? n : num_sms / 2;
  }
  const int clusters = units < g_pair_capacity ? units : g_pair_capacity;
  cfg.gridDim = dim3(2 * clusters);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, kern, ta, tb_, tc, M, N, K, splits, err) == cudaSuccess ? 0 : -21;
}

}  // namespace

int gemm_pair_capacity() { return g_pair_capacity; }

// Same contract as gemm_bf16 (gemm_sm100.cu), which calls this for problems with more than 128 rows.
int gemm2_bf16(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
               bool a_mn, bool b_mn, int out_mode, int splits, int* err, int num_sms, cudaStream_t stream) {
  CUtensorMap ta, tb_, tc;
  int r;
  // K-major operand [R, K]: box 64 (k) x tile rows.  MN-major operand stored [K, R]: box 64 (r) x 64 (k rows).
  r = a_mn ? make_tmap_2d(&ta, A, 2, K, M, lda, 64, 64) : make_tmap_2d(&ta, A, 2, M, K, lda, BM, 64);
  if (r) return r;
  r = b_mn ? make_tmap_2d(&tb_, B, 2, K, N, ldb, 64, 64) : make_tmap_2d(&tb_, B, 2, N, K, ldb, BNH, 64);
  if (r) return r - 100;
  r = out_mode == 0 ? make_tmap_2d(&tc, C, 2, M, N, ldc, 32, 64) : make_tmap_2d(&tc, C, 4, M, N, ldc, 32, 32);
  if (r) return r - 200;
  const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
  const int units = tiles * splits;
#define TB_GEMM2_CASE(AM, BMN, O) \
  if (a_mn == AM && b_mn == BMN && out_mode == O) \
    return launch2<AM, BMN, O>(ta, tb_, tc, M, N, K, splits, err, units, num_sms, stream);
  TB_GEMM2_CASE(false, false, 0)
  TB_GEMM2_CASE(false, false, 1)
  TB_GEMM2_CASE(false, false, 2)
  TB_GEMM2_CASE(false, true, 0)
  TB_GEMM2_CASE(false, true, 1)
  TB_GEMM2_CASE(true, true, 0)
  TB_GEMM2_CASE(true, true, 1)
  TB_GEMM2_CASE(true, true, 2)
  TB_GEMM2_CASE(true, false, 0)
#undef TB_GEMM2_CASE
  return -2;
}

}  // namespace tb
