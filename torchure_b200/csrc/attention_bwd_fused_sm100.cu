// Flash-attention backward in ONE pass: dQ, dK and dV from five tile products per (query block, key block) pair.
//
// One CTA owns 128 keys of one KV head and visits every (query head of the GQA group, visible query block) pair, so
// dK and dV are reduced over query heads and query blocks in TMEM.  Scores are computed TRANSPOSED (keys on TMEM
// lanes, queries on columns); probabilities and score gradients then already have the layout the tensor core wants
// for the A operand of the dV and dK products and never leave TMEM.  The score gradient is additionally written to
// shared memory as the B operand of the third product, dQ^T = K^T dS^T, whose fp32 tile is added to a global fp32
// dQ accumulator (the only quantity that crosses CTAs); a light kernel converts that accumulator to bf16.
//
// A query block is processed as two halves of 64 queries that ping-pong between two TMEM buffers of 128 columns:
//     S^T_h  = K Q_h^T          (SS, 128x64x128)   columns [0, 64)
//     dP^T_h = V dO_h^T         (SS, 128x64x128)   columns [64, 128)
//     P^T_h  = exp2(S^T_h c - lse2[q]);  dS^T_h = P^T_h o (dP^T_h - delta[q]) / sqrt(d)
//                               bf16 P^T_h / dS^T_h -> 8 + 8 columns in place of every 16 S^T columns; dS^T_h also
//                               goes to shared memory
//     dV    += P^T_h  dO_h      (TS, 128x128x64)   columns 256..383
//     dK    += dS^T_h Q_h       (TS, 128x128x64)   columns 384..511
//     dQ^T_h = K^T dS^T_h       (SS, 128x64x128, both operands MN-major)   columns [64, 128) of the half's buffer
// 576 threads: TMA warp, MMA warp and two groups of 8 compute warps, one group per half (two warps per TMEM lane
// quarter, 32 query columns each).  The tensor core alternates between the halves, dQ^T first, and so do the groups:
// while one waits for its products, moves tiles between TMEM and registers or issues its burst of reductions, the
// other runs its exp2 / multiply pass.  A group takes its dQ^T tile out of TMEM as soon as the product has completed
// (which releases the columns for the next block's dP^T) and adds it to the global accumulator with 32 fp32
// reductions per thread.  The element-wise part runs on packed fp32 pairs (fma.rn.f32x2), 16 columns at a time, with
// every constant folded into the row statistics (-lse*log2e and -delta/sqrt(d), written by the statistics kernel
// below, which also clears the dQ accumulator).  The accumulator is head-major ([B, Hq, Sq, 128] fp32) so that the
// 32 reductions of a thread differ by compile-time offsets.
//
// `causal`: query block qb sees key blocks <= qb (Sq == Skv); otherwise every query sees every key (the off-diagonal
// steps of ring attention).  Because partial dQ tiles are added in whatever order CTAs finish, dQ is not bitwise
// reproducible from run to run; the two-kernel backward (attention_bwd_dq/dkv) is.
#include "attn_api.h"
#include "common.cuh"

namespace tb {

int make_tmap_2d(CUtensorMap* map, const void* base, int elem_bytes, uint64_t rows, uint64_t cols, uint64_t ld,
                 uint32_t box_rows, uint32_t box_cols);

namespace {

constexpr int HD = 128;
constexpr int TILE_BYTES = 128 * HD * 2;  // 32 KB
constexpr int HALF_BYTES = 16384;
constexpr int Q_STAGES = 2;
constexpr int STAT_BYTES = 1024;          // -lse2[128] | -delta*scale[128]
constexpr int STAGE_BYTES = 2 * TILE_BYTES + STAT_BYTES;
constexpr int DS_BYTES = 128 * 64 * 2;    // dS^T of one half: 128 key rows x 64 queries, bf16
constexpr int BAR_BYTES = 256;
constexpr int SMEM_USED = 2 * TILE_BYTES + Q_STAGES * STAGE_BYTES + 2 * DS_BYTES + BAR_BYTES;
constexpr int SMEM_BYTES = 232448;        // the whole 227 KB: SMEM_USED plus alignment slack
static_assert(SMEM_USED <= SMEM_BYTES, "shared-memory plan exceeds the per-CTA limit");
constexpr int COMPUTE_WARPS = 8;           // per half of a query block
constexpr int NUM_THREADS = (2 + 2 * COMPUTE_WARPS) * 32;

struct Bars {
  uint64_t kv_full;
  uint64_t q_full[Q_STAGES];
  uint64_t q_empty[Q_STAGES];
  uint64_t st_full[2];      // S^T_h and dP^T_h are in TMEM
  uint64_t pds_ready[2];    // P^T_h, dS^T_h written (one arrival per compute warp)
  uint64_t dq_full[2];      // dV/dK/dQ^T products of half h have completed
  uint64_t dq_drained[2];   // dQ^T_h has been read out of TMEM (one arrival per compute warp)
  uint64_t acc_done;
  uint32_t tmem_slot;
};
static_assert(sizeof(Bars) <= BAR_BYTES, "barrier block");

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// A reduction nobody in this kernel reads back: no "memory" clobber, so that the compiler may keep scheduling
// shared-memory loads and arithmetic of later loop iterations across it.
__device__ __forceinline__ void red_add_unordered(float* p, float x) {
  asm volatile("red.relaxed.gpu.global.add.f32 [%0], %1;" ::"l"(p), "f"(x));
}

struct FusedArgs {
  float* dq_acc;     // [B, Hq, Sq, 128] fp32
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  int64_t ld_dkv;
  const float* nds;    // [B, Hq, Sq]  -delta / sqrt(d)
  const float* nlse2;  // [B, Hq, Sq]  -lse * log2(e)
  int B, Sq, Skv, Hq, Hkv;
  int q_col0, k_col0, v_col0;
  // rows of batch b: q / dO at b * q_bstride + q_row0, k / v at b * kv_bstride + kv_row0; the statistics and the dQ
  // accumulator are [B, Hq, stat_stride(, 128)] with this call's queries starting at stat_row0
  int q_bstride, q_row0, kv_bstride, kv_row0, stat_stride, stat_row0;
  int causal;
  float scale, scale_log2;
};

__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_bwd_fused_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                      const __grid_constant__ FusedArgs a, int* err) {
  pdl_wait();
  pdl_launch_dependents();
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  {
    uint32_t dyn;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn));
    if (static_cast<uint32_t>(smem - smem_raw) + SMEM_USED > dyn) {   // uniform over the CTA: nothing is set up yet
      if (threadIdx.x == 0) atomicCAS(err, 0, kErrAttnWait);
      return;
    }
  }
  uint8_t* sK = smem;
  uint8_t* sV = smem + TILE_BYTES;
  uint8_t* sStage = smem + 2 * TILE_BYTES;                 // [stage][Q 32 KB | dO 32 KB | stats 1 KB]
  uint8_t* sDS = sStage + Q_STAGES * STAGE_BYTES;          // [half][128 key rows x 128 B]
  Bars* bars = reinterpret_cast<Bars*>(sDS + 2 * DS_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqb = a.Sq / 128;
  const int ratio = a.Hq / a.Hkv;
  const int groups = a.B * a.Hkv;
  const int kblk = static_cast<int>(blockIdx.x) / groups;   // causal: block 0 sees the most query blocks, it goes first
  const int g = static_cast<int>(blockIdx.x) % groups;
  const int kvh = g % a.Hkv, b = g / a.Hkv;
  const int krow0 = b * a.Skv + kblk * 128;                          // in the dK / dV outputs
  const int krow_in = b * a.kv_bstride + a.kv_row0 + kblk * 128;     // in the k / v tensors
  const int qb0 = a.causal ? kblk : 0;       // first visible query block
  const int n_qb = nqb - qb0;
  const int n_iter = n_qb * ratio;           // iteration = (query head of the group, query block)

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmDO);
    mbar_init(&bars->kv_full, 1);
    for (int s = 0; s < Q_STAGES; ++s) {
      mbar_init(&bars->q_full[s], 1);
      mbar_init(&bars->q_empty[s], 1);
    }
    for (int hh = 0; hh < 2; ++hh) {
      mbar_init(&bars->st_full[hh], 1);
      mbar_init(&bars->pds_ready[hh], COMPUTE_WARPS);
      mbar_init(&bars->dq_full[hh], 1);
      mbar_init(&bars->dq_drained[hh], COMPUTE_WARPS);
    }
    mbar_init(&bars->acc_done, 1);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_slot, 512);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_slot);

  if (warp == 0) {
    // ------------------------------------------------ TMA producer
    if (elect_one()) {
      const int kcol = a.k_col0 + kvh * HD, vcol = a.v_col0 + kvh * HD;
      mbar_expect_tx(&bars->kv_full, 2 * TILE_BYTES);
      tma_load_2d(sK, &tmK, &bars->kv_full, kcol, krow_in);
      tma_load_2d(sK + HALF_BYTES, &tmK, &bars->kv_full, kcol + 64, krow_in);
      tma_load_2d(sV, &tmV, &bars->kv_full, vcol, krow_in);
      tma_load_2d(sV + HALF_BYTES, &tmV, &bars->kv_full, vcol + 64, krow_in);
      for (int it = 0; it < n_iter; ++it) {
        const int s = it % Q_STAGES;
        const uint32_t ph = (it / Q_STAGES) & 1;
        if (!mbar_wait(&bars->q_empty[s], ph ^ 1, err, kErrAttnWait)) break;
        const int h = kvh * ratio + it / n_qb;
        const int qb = qb0 + it % n_qb;
        const int qrow = b * a.q_bstride + a.q_row0 + qb * 128;
        uint8_t* sQ = sStage + s * STAGE_BYTES;
        uint8_t* sDO = sQ + TILE_BYTES;
        float* sStat = reinterpret_cast<float*>(sDO + TILE_BYTES);
        mbar_expect_tx(&bars->q_full[s], 2 * TILE_BYTES + STAT_BYTES);
        tma_load_2d(sQ, &tmQ, &bars->q_full[s], a.q_col0 + h * HD, qrow);
        tma_load_2d(sQ + HALF_BYTES, &tmQ, &bars->q_full[s], a.q_col0 + h * HD + 64, qrow);
        tma_load_2d(sDO, &tmDO, &bars->q_full[s], h * HD, qrow);
        tma_load_2d(sDO + HALF_BYTES, &tmDO, &bars->q_full[s], h * HD + 64, qrow);
        const int64_t stat = (static_cast<int64_t>(b) * a.Hq + h) * a.stat_stride + a.stat_row0 + qb * 128;
        bulk_load_1d(sStat, a.nlse2 + stat, 512, &bars->q_full[s]);
        bulk_load_1d(sStat + 128, a.nds + stat, 512, &bars->q_full[s]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc_st = make_idesc_bf16(128, 64, false, false);   // S^T / dP^T halves: N = 64 queries
      constexpr uint32_t idesc_acc = make_idesc_bf16(128, 128, false, true);  // A in TMEM, B MN-major, N = 128 (hd)
      constexpr uint32_t idesc_dq = make_idesc_bf16(128, 64, true, true);     // K^T (MN-major) x dS^T (MN-major)
      // Descriptors are built once per operand; a K step only adds a constant to the 14-bit address field (16-byte
      // units; every operand lies below 256 KB, so the sum never carries into the next field).
      const uint64_t dK_k = make_desc_sw128(smem_u32(sK), 16, 1024);                  // K, K-major (S^T)
      const uint64_t dV_k = make_desc_sw128(smem_u32(sV), 16, 1024);                  // V, K-major (dP^T)
      const uint64_t dK_mn = make_desc_sw128(smem_u32(sK), HALF_BYTES, 1024);         // K^T, MN-major (dQ^T)
      uint64_t dQ_k[Q_STAGES], dO_k[Q_STAGES], dQ_mn[Q_STAGES], dO_mn[Q_STAGES], dDS[2];
#pragma unroll
      for (int st = 0; st < Q_STAGES; ++st) {
        const uint32_t qa = smem_u32(sStage + st * STAGE_BYTES), oa = qa + TILE_BYTES;
        dQ_k[st] = make_desc_sw128(qa, 16, 1024);
        dO_k[st] = make_desc_sw128(oa, 16, 1024);
        dQ_mn[st] = make_desc_sw128(qa, HALF_BYTES, 1024);
        dO_mn[st] = make_desc_sw128(oa, HALF_BYTES, 1024);
      }
      dDS[0] = make_desc_sw128(smem_u32(sDS), HALF_BYTES, 1024);
      dDS[1] = make_desc_sw128(smem_u32(sDS + DS_BYTES), HALF_BYTES, 1024);
      constexpr uint64_t kHalfRows = 8192 >> 4;     // 64 query rows of a K-major / MN-major tile
      auto issue_s = [&](int hh, int st) {
        const uint64_t qd = dQ_k[st] + hh * kHalfRows;                   // query rows 64h.. of the Q tile
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t o = ((ks >> 2) * HALF_BYTES + (ks & 3) * 32) >> 4;
          umma_f16_ss(tmem_base + hh * 128, dK_k + o, qd + o, idesc_st, ks != 0 ? 1u : 0u);
        }
      };
      auto issue_dp = [&](int hh, int st) {
        const uint64_t od = dO_k[st] + hh * kHalfRows;                   // same rows of dO
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t o = ((ks >> 2) * HALF_BYTES + (ks & 3) * 32) >> 4;
          umma_f16_ss(tmem_base + hh * 128 + 64, dV_k + o, od + o, idesc_st, ks != 0 ? 1u : 0u);
        }
        umma_commit(&bars->st_full[hh]);
      };
      // dQ^T_h = K^T dS^T_h goes first and is committed on its own: the compute warps take it out of TMEM in the
      // middle of the other half's element-wise pass, so the columns are free again before dP^T of the next block
      // wants them.  Then dV += P^T_h dO_h and dK += dS^T_h Q_h.
      auto issue_acc = [&](int hh, int st, bool first) {
        const uint64_t qd = dQ_mn[st] + hh * kHalfRows, od = dO_mn[st] + hh * kHalfRows;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)   // 16 keys per step: 16 rows of K (both 64-wide d halves) and of dS^T
          umma_f16_ss(tmem_base + hh * 128 + 64, dK_mn + ks * (2048 >> 4), dDS[hh] + ks * (2048 >> 4), idesc_dq,
                      ks != 0 ? 1u : 0u);
        umma_commit(&bars->dq_full[hh]);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          // queries [16 ks, 16 ks + 16) of the half: their P^T sits in columns [16 ks, 16 ks + 8), their dS^T in
          // [16 ks + 8, 16 ks + 16) (each group of 16 S^T columns is replaced by its own two products)
          umma_f16_ts(tmem_base + 256, tmem_base + hh * 128 + ks * 16, od + ks * (2048 >> 4), idesc_acc,
                      (first && ks == 0) ? 0u : 1u);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_f16_ts(tmem_base + 384, tmem_base + hh * 128 + ks * 16 + 8, qd + ks * (2048 >> 4), idesc_acc,
                      (first && ks == 0) ? 0u : 1u);
      };
      bool ok = mbar_wait(&bars->kv_full, 0, err, kErrAttnWait) && mbar_wait(&bars->q_full[0], 0, err, kErrAttnWait);
      if (ok) {
        tc_fence_after();
        issue_s(0, 0);
        issue_dp(0, 0);
        issue_s(1, 0);
        issue_dp(1, 0);
      }
      for (int it = 0; it < n_iter && ok; ++it) {
        const int s = it % Q_STAGES, sn = (it + 1) % Q_STAGES;
        const uint32_t phn = ((it + 1) / Q_STAGES) & 1;
        const bool more = it + 1 < n_iter;
        for (int hh = 0; hh < 2 && ok; ++hh) {
          if (!mbar_wait(&bars->pds_ready[hh], it & 1, err, kErrAttnWait)) { ok = false; break; }
          tc_fence_after();
          issue_acc(hh, s, it == 0 && hh == 0);
          if (hh == 1) umma_commit(&bars->q_empty[s]);
          if (more) {
            if (hh == 0 && !mbar_wait(&bars->q_full[sn], phn, err, kErrAttnWait)) { ok = false; break; }
            tc_fence_after();
            issue_s(hh, sn);         // overwrites P^T_h / dS^T_h: ordered behind the products that read them
            // the dP^T columns still hold dQ^T_h until the compute warps have read it
            if (!mbar_wait(&bars->dq_drained[hh], it & 1, err, kErrAttnWait)) { ok = false; break; }
            tc_fence_after();
            issue_dp(hh, sn);
          }
        }
      }
      if (ok) umma_commit(&bars->acc_done);
    }
  } else {
    // ------------------------------------------------ compute warps
    // Two groups of eight warps: group g owns half g of every query block (two warps per TMEM lane quarter, 32 of
    // the half's 64 query columns each).  The groups run out of phase, like the tensor core's work on the two halves,
    // so the waits, TMEM round trips and reduction bursts of one group are covered by the arithmetic of the other.
    const int grp = (warp - 2) >> 3;
    const int quarter = warp & 3;             // TMEM lane quarter this warp may touch
    const int cg = ((warp - 2) >> 2) & 1;     // which 32 of the half's 64 query columns
    const int row = quarter * 32 + lane;      // key inside the block (S^T, dP^T) / head-dim index (dQ^T)
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    const float2 c2 = make_float2(a.scale_log2, a.scale_log2), sc2 = make_float2(a.scale, a.scale);
    // byte offsets of this thread's four 16-byte chunks inside its 128-byte dS^T row (128-byte swizzle)
    uint32_t ds_off[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) ds_off[j] = row * 128 + (((4 * cg + j) ^ (row & 7)) << 4);
    const uint32_t tH = tmem_base + lane_sel + grp * 128 + cg * 32;
    uint8_t* dsb = sDS + grp * DS_BYTES;      // dS^T row of this key: queries q0..q0+31 are four swizzled 16-byte chunks
    bool ok = true;
    // P^T and dS^T of this warp's 32 query columns (one key per lane), 16 columns at a time.  Each group of 16 S^T
    // columns is overwritten by its own P^T (8 columns of bf16 pairs) and dS^T (8 columns), so the warps need no
    // barrier among them and the second group's scores are still intact when the first group's results are stored.
    auto softmax_half = [&](const float* sStat, bool diag) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t sv[16], dv[16];
        tmem_ld_32x32b_x16(tH + c * 16, sv);
        tmem_ld_32x32b_x16(tH + 64 + c * 16, dv);
        tmem_ld_wait();
        uint32_t pp[8], pd[8];
        const int q0 = grp * 64 + cg * 32 + c * 16;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float2 nl = *reinterpret_cast<const float2*>(sStat + q0 + 2 * i);          // -lse2 of the two queries
          const float2 nd = *reinterpret_cast<const float2*>(sStat + 128 + q0 + 2 * i);    // -delta * scale
          const float2 t = fma2(make_float2(__uint_as_float(sv[2 * i]), __uint_as_float(sv[2 * i + 1])), c2, nl);
          float2 p = make_float2(ex2(t.x), ex2(t.y));
          if (diag) {
            if (q0 + 2 * i < row) p.x = 0.f;       // query before key: masked
            if (q0 + 2 * i + 1 < row) p.y = 0.f;
          }
          const float2 u = fma2(make_float2(__uint_as_float(dv[2 * i]), __uint_as_float(dv[2 * i + 1])), sc2, nd);
          const float2 ds = mul2(p, u);
          pp[i] = pack_bf16x2(p.x, p.y);
          pd[i] = pack_bf16x2(ds.x, ds.y);
        }
        tmem_st_32x32b_x8(tH + c * 16, pp);
        tmem_st_32x32b_x8(tH + c * 16 + 8, pd);
#pragma unroll
        for (int j = 0; j < 2; ++j)
          *reinterpret_cast<uint4*>(dsb + ds_off[2 * c + j]) =
              make_uint4(pd[4 * j], pd[4 * j + 1], pd[4 * j + 2], pd[4 * j + 3]);
      }
      tmem_st_wait();
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->pds_ready[grp]);
    };
    for (int it = 0; it < n_iter && ok; ++it) {
      const int s = it % Q_STAGES;
      const bool diag = a.causal && (it % n_qb) == 0;     // query block == key block
      const float* sStat = reinterpret_cast<const float*>(sStage + s * STAGE_BYTES + 2 * TILE_BYTES);
      if (!mbar_wait(&bars->st_full[grp], it & 1, err, kErrAttnWait)) { ok = false; break; }
      tc_fence_after();
      if (diag) softmax_half(sStat, true);
      else softmax_half(sStat, false);
      // dQ^T of this half (the first product the tensor core runs on it): 32 query columns of this warp, one head-dim
      // index per lane.  The tile leaves TMEM first, which releases its columns for the next block's dP^T; the 32
      // fp32 reductions follow.  The accumulator is head-major, so they differ by compile-time offsets.
      if (!mbar_wait(&bars->dq_full[grp], it & 1, err, kErrAttnWait)) { ok = false; break; }
      tc_fence_after();
      uint32_t v[32];
      tmem_ld_32x32b_x32(tH + 64, v);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->dq_drained[grp]);
      const int h = kvh * ratio + it / n_qb;
      const int qb = qb0 + it % n_qb;
      float* dst = a.dq_acc +
                   ((static_cast<int64_t>(b) * a.Hq + h) * a.stat_stride + a.stat_row0 + qb * 128 + grp * 64 + cg * 32) * HD + row;
#pragma unroll
      for (int j = 0; j < 32; ++j) red_add_unordered(dst + j * HD, __uint_as_float(v[j]));
    }
    if (ok && mbar_wait(&bars->acc_done, 0, err, kErrAttnWait)) {
      tc_fence_after();
      // group 0 writes dV, group 1 dK: this warp's 64 of the 128 head-dim columns, one key row per lane, straight to
      // global memory
      {
        const int which = grp;
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          const int col = cg * 64 + c * 32;
          uint32_t v[32];
          tmem_ld_32x32b_x32(tmem_base + lane_sel + 256 + which * 128 + col, v);
          tmem_ld_wait();
          __nv_bfloat16* dst = (which == 0 ? a.dv : a.dk) + static_cast<int64_t>(krow0 + row) * a.ld_dkv + kvh * HD + col;
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            uint4 pk;
            pk.x = pack_bf16x2(__uint_as_float(v[8 * jj + 0]), __uint_as_float(v[8 * jj + 1]));
            pk.y = pack_bf16x2(__uint_as_float(v[8 * jj + 2]), __uint_as_float(v[8 * jj + 3]));
            pk.z = pack_bf16x2(__uint_as_float(v[8 * jj + 4]), __uint_as_float(v[8 * jj + 5]));
            pk.w = pack_bf16x2(__uint_as_float(v[8 * jj + 6]), __uint_as_float(v[8 * jj + 7]));
            *reinterpret_cast<uint4*>(dst + 8 * jj) = pk;
          }
        }
      }
    }
  }

  if (*reinterpret_cast<volatile int*>(err) != 0) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// Row statistics for the single-pass backward, one warp per token row (16 lanes per head, two heads at a time):
//   nds[b,h,s]   = -rowsum(dO * O) / sqrt(d)        nlse2[b,h,s] = -lse * log2(e)
// and the token's rows of the head-major dQ accumulator are cleared.
__global__ void __launch_bounds__(256)
attn_bwd_stats_kernel(const __nv_bfloat16* __restrict__ d_o, const __nv_bfloat16* __restrict__ o,
                      const float* __restrict__ lse, float* __restrict__ nds, float* __restrict__ nlse2,
                      float* __restrict__ dq_acc, int B, int S, int Hq, float scale) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= static_cast<int64_t>(B) * S) return;
  const int sub = lane & 15, hsel = lane >> 4;
  const int b = static_cast<int>(row / S), pos = static_cast<int>(row % S);
  const __nv_bfloat16* pa = d_o + row * Hq * HD + sub * 8;
  const __nv_bfloat16* pc = o + row * Hq * HD + sub * 8;
  const int pairs = (Hq + 1) >> 1;
  constexpr int U = 4;
  for (int hp = 0; hp < pairs; hp += U) {
    uint4 x[U], y[U];
#pragma unroll
    for (int k = 0; k < U; ++k) {
      const int h = 2 * (hp + k) + hsel;
      x[k] = y[k] = make_uint4(0u, 0u, 0u, 0u);
      if (hp + k < pairs && h < Hq) {
        x[k] = *reinterpret_cast<const uint4*>(pa + h * HD);
        y[k] = *reinterpret_cast<const uint4*>(pc + h * HD);
      }
    }
#pragma unroll
    for (int k = 0; k < U; ++k) {
      const int h = 2 * (hp + k) + hsel;
      const __nv_bfloat162* xa = reinterpret_cast<const __nv_bfloat162*>(&x[k]);
      const __nv_bfloat162* xc = reinterpret_cast<const __nv_bfloat162*>(&y[k]);
      float acc = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 u = __bfloat1622float2(xa[e]), w = __bfloat1622float2(xc[e]);
        acc += u.x * w.x + u.y * w.y;
      }
#pragma unroll
      for (int s2 = 8; s2 > 0; s2 >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s2);
      if (sub == 0 && hp + k < pairs && h < Hq) {
        const int64_t idx = (static_cast<int64_t>(b) * Hq + h) * S + pos;
        nds[idx] = -acc * scale;
        nlse2[idx] = -lse[idx] * 1.4426950408889634f;
      }
    }
  }
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int h = 0; h < Hq; ++h)
    reinterpret_cast<float4*>(dq_acc + ((static_cast<int64_t>(b) * Hq + h) * S + pos) * HD)[lane] = zero;
}

// dst[(b S + s), h 128 + d] (bf16, row stride ld_dst) = acc[b, h, s, d] (fp32): one thread per 8 values
__global__ void __launch_bounds__(256)
dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dst, int64_t ld_dst, int B, int S, int Hq) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t total = static_cast<int64_t>(B) * S * Hq * (HD / 8);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % (HD / 8)) * 8;
    int64_t r = i / (HD / 8);              // (b, s, h) with h fastest: consecutive threads write one token row
    const int h = static_cast<int>(r % Hq);
    r /= Hq;
    const int s = static_cast<int>(r % S), b = static_cast<int>(r / S);
    const float* src = acc + ((static_cast<int64_t>(b) * Hq + h) * S + s) * HD + c;
    const float4 x = *reinterpret_cast<const float4*>(src);
    const float4 y = *reinterpret_cast<const float4*>(src + 4);
    uint4 pk;
    pk.x = pack_bf16x2(x.x, x.y);
    pk.y = pack_bf16x2(x.z, x.w);
    pk.z = pack_bf16x2(y.x, y.y);
    pk.w = pack_bf16x2(y.z, y.w);
    *reinterpret_cast<uint4*>(dst + (static_cast<int64_t>(b) * S + s) * ld_dst + h * HD + c) = pk;
  }
}

}  // namespace

int attn_bwd_stats(const void* d_o, const void* o, const float* lse, float* nds, float* nlse2, float* dq_acc, int B,
                   int S, int Hq, cudaStream_t stream) {
  const int64_t warps = static_cast<int64_t>(B) * S;  // one warp per token row
  return launch_pdl(attn_bwd_stats_kernel, dim3(static_cast<int>((warps + 7) / 8)), dim3(256), 0, stream,
                    reinterpret_cast<const __nv_bfloat16*>(d_o), reinterpret_cast<const __nv_bfloat16*>(o), lse, nds,
                    nlse2, dq_acc, B, S, Hq, 1.f / sqrtf(static_cast<float>(HD))) == cudaSuccess
             ? 0
             : -21;
}

int attn_bwd_fused(const AttnOperand& q, const AttnOperand& k, const AttnOperand& v, const void* d_o, float* dq_acc,
                   void* dk, void* dv, int64_t ld_dkv, const float* nds, const float* nlse2, int B, int Sq, int Skv,
                   int Hq, int Hkv, bool causal, int* err, cudaStream_t stream, const AttnPairLayout* lay) {
  if (Sq % 128 != 0 || Skv % 128 != 0 || Hq % Hkv != 0 || B <= 0 || Sq <= 0 || Skv <= 0) return -1;
  AttnPairLayout whole{static_cast<int64_t>(B) * Sq, Sq, 0, static_cast<int64_t>(B) * Skv, Skv, 0, Sq, 0};
  if (lay == nullptr) lay = &whole;
  if (causal && Sq != Skv) return -2;
  if (ld_dkv % 8 != 0 || (reinterpret_cast<uintptr_t>(dk) & 15) || (reinterpret_cast<uintptr_t>(dv) & 15) ||
      (reinterpret_cast<uintptr_t>(dq_acc) & 15))
    return -3;
  const uint64_t Mq = static_cast<uint64_t>(lay->q_rows), Mk = static_cast<uint64_t>(lay->kv_rows);
  CUtensorMap tq, tk, tv, tdo;
  int r = make_tmap_2d(&tq, q.ptr, 2, Mq, q.ld, q.ld, 128, 64);
  if (r) return r;
  r = make_tmap_2d(&tk, k.ptr, 2, Mk, k.ld, k.ld, 128, 64);
  if (r) return r - 100;
  r = make_tmap_2d(&tv, v.ptr, 2, Mk, v.ld, v.ld, 128, 64);
  if (r) return r - 200;
  r = make_tmap_2d(&tdo, d_o, 2, Mq, static_cast<uint64_t>(Hq) * HD, static_cast<uint64_t>(Hq) * HD, 128, 64);
  if (r) return r - 300;
  if (!ensure_dynamic_smem(reinterpret_cast<const void*>(attn_bwd_fused_kernel), SMEM_BYTES)) return -20;
  FusedArgs a{};
  a.dq_acc = dq_acc;
  a.dk = reinterpret_cast<__nv_bfloat16*>(dk);
  a.dv = reinterpret_cast<__nv_bfloat16*>(dv);
  a.ld_dkv = ld_dkv;
  a.nds = nds;
  a.nlse2 = nlse2;
  a.B = B; a.Sq = Sq; a.Skv = Skv; a.Hq = Hq; a.Hkv = Hkv;
  a.q_col0 = static_cast<int>(q.col0);
  a.k_col0 = static_cast<int>(k.col0);
  a.v_col0 = static_cast<int>(v.col0);
  a.causal = causal ? 1 : 0;
  a.q_bstride = lay->q_bstride; a.q_row0 = lay->q_row0; a.kv_bstride = lay->kv_bstride; a.kv_row0 = lay->kv_row0;
  a.stat_stride = lay->stat_stride; a.stat_row0 = lay->stat_row0;
  a.scale = 1.f / sqrtf(static_cast<float>(HD));
  a.scale_log2 = a.scale * 1.4426950408889634f;
  const int grid = (Skv / 128) * B * Hkv;
  if (launch_pdl(attn_bwd_fused_kernel, dim3(grid), dim3(NUM_THREADS), SMEM_BYTES, stream, tq, tk, tv, tdo, a, err) !=
      cudaSuccess)
    return -21;
  return 0;
}

int attn_dq_convert(const float* dq_acc, void* dst, int64_t ld_dst, int B, int S, int Hq, cudaStream_t stream) {
  if (ld_dst % 8 != 0 || (reinterpret_cast<uintptr_t>(dst) & 15)) return -1;
  const int64_t total = static_cast<int64_t>(B) * S * Hq * (HD / 8);
  const int grid = static_cast<int>(total / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  return launch_pdl(dq_convert_kernel, dim3(grid > 0 ? grid : 1), dim3(256), 0, stream, dq_acc,
                    reinterpret_cast<__nv_bfloat16*>(dst), ld_dst, B, S, Hq) == cudaSuccess
             ? 0
             : -21;
}

}  // namespace tb
