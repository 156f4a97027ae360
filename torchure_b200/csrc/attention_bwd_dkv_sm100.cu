// Flash-attention backward, part 2 of 2: dK and dV.
//
// One CTA owns 128 keys of one KV head and visits every (query head of the GQA group, causal query block) pair, so the
// GQA reduction over query heads happens in the TMEM accumulators.  Scores are computed TRANSPOSED (keys on TMEM lanes,
// queries on columns): the probability and score-gradient tiles then already have the layout the tensor core wants
// for the A operand of the two accumulating products, and never leave TMEM.
//
// A query block is processed as two halves of 64 queries that ping-pong between two TMEM buffers:
//     S^T_h  = K Q_h^T       (SS, 128x64x128)   \  buffer h: columns [128h, 128h+64) and [128h+64, 128h+128)
//     dP^T_h = V dO_h^T      (SS, 128x64x128)   /
//     P^T_h  = exp2(S^T_h * c - lse2[q]) ; dS^T_h = P^T_h o (dP^T_h - delta[q]) / sqrt(d)      one thread per key
//     dV += P^T_h  dO_h      (TS, 128x128x64, dO read MN-major)       accumulators: columns 256..383
//     dK += dS^T_h Q_h       (TS, 128x128x64, Q  read MN-major)                     columns 384..511
// While the 128 compute threads work on one half, the tensor core runs the other half's products.
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
constexpr int STAT_BYTES = 1024;          // lse2[128] | delta[128]
constexpr int STAGE_BYTES = 2 * TILE_BYTES + STAT_BYTES;
constexpr int SMEM_BYTES = 2 * TILE_BYTES + Q_STAGES * STAGE_BYTES + 256 + 1024;
constexpr int NUM_THREADS = 320;  // TMA warp, MMA warp, 8 compute warps (two per TMEM lane quarter)

struct Bars {
  uint64_t kv_full;
  uint64_t q_full[Q_STAGES];
  uint64_t q_empty[Q_STAGES];
  uint64_t st_full[2];    // S^T_h and dP^T_h are in TMEM
  uint64_t pds_ready[2];  // P^T_h and dS^T_h written (128 arrivals)
  uint64_t acc_done;
  uint32_t tmem_slot;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}


__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQK, const __grid_constant__ CUtensorMap tmV,
                    const __grid_constant__ CUtensorMap tmDO, const __grid_constant__ CUtensorMap tmDQKV,
                    const float* __restrict__ delta, const float* __restrict__ lse2, int B, int S, int Hq, int Hkv,
                    float scale, float scale_log2, int* err) {
  pdl_wait();
  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + TILE_BYTES;
  uint8_t* sStage = smem + 2 * TILE_BYTES;   // [stage][Q 32 KB | dO 32 KB | stats 1 KB]
  Bars* bars = reinterpret_cast<Bars*>(sStage + Q_STAGES * STAGE_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nblk = S / 128;
  const int ratio = Hq / Hkv;
  const int groups = B * Hkv;
  const int kblk = static_cast<int>(blockIdx.x) / groups;   // block 0 has the most query blocks: it goes first
  const int g = static_cast<int>(blockIdx.x) % groups;
  const int kvh = g % Hkv, b = g / Hkv;
  const int krow0 = b * S + kblk * 128;
  const int n_qb = nblk - kblk;             // query blocks kblk .. nblk-1
  const int n_iter = n_qb * ratio;          // iteration = (query head of the group, query block)

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmDO);
    tma_prefetch_desc(&tmDQKV);
    mbar_init(&bars->kv_full, 1);
    for (int s = 0; s < Q_STAGES; ++s) {
      mbar_init(&bars->q_full[s], 1);
      mbar_init(&bars->q_empty[s], 1);
    }
    for (int hh = 0; hh < 2; ++hh) {
      mbar_init(&bars->st_full[hh], 1);
      mbar_init(&bars->pds_ready[hh], 256);
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
    if (elect_one()) {
      const int kcol = (Hq + kvh) * HD, vcol = (Hq + Hkv + kvh) * HD;
      mbar_expect_tx(&bars->kv_full, 2 * TILE_BYTES);
      tma_load_2d(sK, &tmQK, &bars->kv_full, kcol, krow0);
      tma_load_2d(sK + HALF_BYTES, &tmQK, &bars->kv_full, kcol + 64, krow0);
      tma_load_2d(sV, &tmV, &bars->kv_full, vcol, krow0);
      tma_load_2d(sV + HALF_BYTES, &tmV, &bars->kv_full, vcol + 64, krow0);
      for (int it = 0; it < n_iter; ++it) {
        const int s = it % Q_STAGES;
        const uint32_t ph = (it / Q_STAGES) & 1;
        if (!mbar_wait(&bars->q_empty[s], ph ^ 1, err, kErrAttnWait)) break;
        const int h = kvh * ratio + it / n_qb;
        const int qb = kblk + it % n_qb;
        const int qrow = b * S + qb * 128;
        uint8_t* sQ = sStage + s * STAGE_BYTES;
        uint8_t* sDO = sQ + TILE_BYTES;
        float* sStat = reinterpret_cast<float*>(sDO + TILE_BYTES);
        mbar_expect_tx(&bars->q_full[s], 2 * TILE_BYTES + STAT_BYTES);
        tma_load_2d(sQ, &tmQK, &bars->q_full[s], h * HD, qrow);
        tma_load_2d(sQ + HALF_BYTES, &tmQK, &bars->q_full[s], h * HD + 64, qrow);
        tma_load_2d(sDO, &tmDO, &bars->q_full[s], h * HD, qrow);
        tma_load_2d(sDO + HALF_BYTES, &tmDO, &bars->q_full[s], h * HD + 64, qrow);
        const int64_t stat = (static_cast<int64_t>(b) * Hq + h) * S + qb * 128;
        bulk_load_1d(sStat, lse2 + stat, 512, &bars->q_full[s]);
        bulk_load_1d(sStat + 128, delta + stat, 512, &bars->q_full[s]);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc_st = make_idesc_bf16(128, 64, false, false);   // S^T / dP^T halves: N = 64 queries
      constexpr uint32_t idesc_acc = make_idesc_bf16(128, 128, false, true);  // A in TMEM, B MN-major, N = 128 (hd)
      // S^T_h / dP^T_h of the iteration whose tiles live at `stage`
      auto issue_st = [&](int hh, const uint8_t* stage) {
        const uint32_t ka = smem_u32(sK), va = smem_u32(sV);
        const uint32_t qa = smem_u32(stage) + hh * 8192;                 // query rows 64h.. of the Q tile
        const uint32_t da = smem_u32(stage + TILE_BYTES) + hh * 8192;    // same rows of dO
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t o = (ks >> 2) * HALF_BYTES + (ks & 3) * 32;
          umma_f16_ss(tmem_base + hh * 128, make_desc_sw128(ka + o, 16, 1024), make_desc_sw128(qa + o, 16, 1024),
                      idesc_st, ks != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t o = (ks >> 2) * HALF_BYTES + (ks & 3) * 32;
          umma_f16_ss(tmem_base + hh * 128 + 64, make_desc_sw128(va + o, 16, 1024), make_desc_sw128(da + o, 16, 1024),
                      idesc_st, ks != 0 ? 1u : 0u);
        }
        umma_commit(&bars->st_full[hh]);
      };
      // dV += P^T_h dO_h ; dK += dS^T_h Q_h
      auto issue_acc = [&](int hh, const uint8_t* stage, bool first) {
        const uint32_t qa = smem_u32(stage) + hh * 8192;
        const uint32_t da = smem_u32(stage + TILE_BYTES) + hh * 8192;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_f16_ts(tmem_base + 256, tmem_base + hh * 128 + (ks >> 1) * 32 + (ks & 1) * 8,
                      make_desc_sw128(da + ks * 2048, HALF_BYTES, 1024),
                      idesc_acc, (first && ks == 0) ? 0u : 1u);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_f16_ts(tmem_base + 384, tmem_base + hh * 128 + 64 + (ks >> 1) * 32 + (ks & 1) * 8,
                      make_desc_sw128(qa + ks * 2048, HALF_BYTES, 1024), idesc_acc, (first && ks == 0) ? 0u : 1u);
      };
      bool ok = mbar_wait(&bars->kv_full, 0, err, kErrAttnWait) && mbar_wait(&bars->q_full[0], 0, err, kErrAttnWait);
      if (ok) {
        tc_fence_after();
        issue_st(0, sStage);
        issue_st(1, sStage);
      }
      for (int it = 0; it < n_iter && ok; ++it) {
        const int s = it % Q_STAGES, sn = (it + 1) % Q_STAGES;
        const uint32_t phn = ((it + 1) / Q_STAGES) & 1;
        const bool more = it + 1 < n_iter;
        const uint8_t* stage = sStage + s * STAGE_BYTES;
        const uint8_t* next = sStage + sn * STAGE_BYTES;
        for (int hh = 0; hh < 2 && ok; ++hh) {
          if (!mbar_wait(&bars->pds_ready[hh], it & 1, err, kErrAttnWait)) { ok = false; break; }
          tc_fence_after();
          issue_acc(hh, stage, it == 0 && hh == 0);
          if (hh == 1) umma_commit(&bars->q_empty[s]);
          if (more) {
            if (hh == 0 && !mbar_wait(&bars->q_full[sn], phn, err, kErrAttnWait)) { ok = false; break; }
            tc_fence_after();
            issue_st(hh, next);
          }
        }
      }
      if (ok) umma_commit(&bars->acc_done);
    }
  } else {
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;      // key inside the block
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    bool ok = true;
    for (int it = 0; it < n_iter && ok; ++it) {
      const int s = it % Q_STAGES;
      const bool diag = (it % n_qb) == 0;     // query block == key block
      const float* sStat = reinterpret_cast<const float*>(sStage + s * STAGE_BYTES + 2 * TILE_BYTES);
      for (int hh = 0; hh < 2; ++hh) {
        if (!mbar_wait(&bars->st_full[hh], it & 1, err, kErrAttnWait)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tS = tmem_base + lane_sel + hh * 128;
        const uint32_t tP = tS + 64;
        {
          const int c = (warp - 2) >> 2;   // this warp's 32 of the half's 64 query columns
          uint32_t sv[32], dv[32];
          tmem_ld_32x32b_x32(tS + c * 32, sv);
          tmem_ld_32x32b_x32(tP + c * 32, dv);
          tmem_ld_wait();
          {
            uint32_t pp[16], pd[16];
            const int q0 = hh * 64 + c * 32;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float2 l2 = *reinterpret_cast<const float2*>(sStat + q0 + 2 * i);
              const float2 dl = *reinterpret_cast<const float2*>(sStat + 128 + q0 + 2 * i);
              float p0 = ex2(fmaf(__uint_as_float(sv[2 * i]), scale_log2, -l2.x));
              float p1 = ex2(fmaf(__uint_as_float(sv[2 * i + 1]), scale_log2, -l2.y));
              if (diag) {
                if (q0 + 2 * i < row) p0 = 0.f;       // query before key: masked
                if (q0 + 2 * i + 1 < row) p1 = 0.f;
              }
              pp[i] = pack_bf16x2(p0, p1);
              pd[i] = pack_bf16x2(p0 * (__uint_as_float(dv[2 * i]) - dl.x) * scale,
                                  p1 * (__uint_as_float(dv[2 * i + 1]) - dl.y) * scale);
            }
            tmem_st_32x32b_x16(tS + c * 32, pp);   // inside the columns this warp itself consumed
            tmem_st_32x32b_x16(tP + c * 32, pd);
          }
        }
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(&bars->pds_ready[hh]);
      }
    }
    if (ok && warp < 6 && mbar_wait(&bars->acc_done, 0, err, kErrAttnWait)) {
      tc_fence_after();
      // stage 0's Q/dO tiles are dead: 4 warps x 8 KB of staging
      uint8_t* stage = sStage + quarter * 8192;
      uint32_t v[32];
      for (int which = 0; which < 2; ++which) {   // 0: dV, 1: dK
        const uint32_t tA = tmem_base + lane_sel + 256 + which * 128;
        if (which == 1) {
          if (lane == 0) tma_wait_group_read<0>();
          __syncwarp();
        }
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          tmem_ld_32x32b_x32(tA + c * 32, v);
          tmem_ld_wait();
          uint8_t* rowp = stage + (c >> 1) * 4096 + lane * 128;
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            uint4 pk;
            pk.x = pack_bf16x2(__uint_as_float(v[8 * jj + 0]), __uint_as_float(v[8 * jj + 1]));
            pk.y = pack_bf16x2(__uint_as_float(v[8 * jj + 2]), __uint_as_float(v[8 * jj + 3]));
            pk.z = pack_bf16x2(__uint_as_float(v[8 * jj + 4]), __uint_as_float(v[8 * jj + 5]));
            pk.w = pack_bf16x2(__uint_as_float(v[8 * jj + 6]), __uint_as_float(v[8 * jj + 7]));
            const int chunk = (c & 1) * 4 + jj;
            *reinterpret_cast<uint4*>(rowp + ((chunk ^ (lane & 7)) << 4)) = pk;
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          const int col = which == 0 ? (Hq + Hkv + kvh) * HD : (Hq + kvh) * HD;
          tma_store_2d(&tmDQKV, stage, col, krow0 + quarter * 32);
          tma_store_2d(&tmDQKV, stage + 4096, col + 64, krow0 + quarter * 32);
          tma_commit_group();
        }
      }
      if (lane == 0) tma_wait_group<0>();
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

}  // namespace

int attn_bwd_dkv(const void* qk, const void* qkv, const void* d_o, void* dqkv, const float* delta, const float* lse2,
                 int B, int S, int Hq, int Hkv, int* err, cudaStream_t stream) {
  if (S % 128 != 0 || Hq % Hkv != 0) return -1;
  const uint64_t M = static_cast<uint64_t>(B) * S;
  const uint64_t wqk = static_cast<uint64_t>(Hq + Hkv) * HD, wqkv = static_cast<uint64_t>(Hq + 2 * Hkv) * HD;
  CUtensorMap tq, tv, tdo, tdq;
  int r = make_tmap_2d(&tq, qk, 2, M, wqk, wqk, 128, 64);
  if (r) return r;
  r = make_tmap_2d(&tv, qkv, 2, M, wqkv, wqkv, 128, 64);
  if (r) return r - 100;
  r = make_tmap_2d(&tdo, d_o, 2, M, static_cast<uint64_t>(Hq) * HD, static_cast<uint64_t>(Hq) * HD, 128, 64);
  if (r) return r - 200;
  r = make_tmap_2d(&tdq, dqkv, 2, M, wqkv, wqkv, 32, 64);
  if (r) return r - 300;
  if (!ensure_dynamic_smem(reinterpret_cast<const void*>(attn_bwd_dkv_kernel), SMEM_BYTES)) return -20;
  const int grid = (S / 128) * B * Hkv;
  const float scale = 1.f / sqrtf(static_cast<float>(HD));
  launch_pdl(attn_bwd_dkv_kernel, dim3(grid), dim3(NUM_THREADS), SMEM_BYTES, stream, tq, tv, tdo, tdq, delta, lse2, B, S, Hq, Hkv, scale,
                                                                  scale * 1.4426950408889634f, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

}  // namespace tb
