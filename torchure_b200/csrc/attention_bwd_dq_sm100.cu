// Flash-attention backward, part 1 of 2: dQ (and the row statistics both parts need).
//
//   attn_bwd_prep_kernel   delta[b,h,s] = sum_d dO*O  and  lse2 = lse * log2(e)   (scratch rows for both kernels)
//   attn_bwd_dq_kernel     one CTA per (128 query rows, query head): loops over the causal KV blocks
//                            S  = Q K_j^T            (SS)      -> TMEM S[j&1]
//                            dP = dO V_j^T           (SS)      -> TMEM dP
//                            dS = P o (dP - delta) / sqrt(d)   two threads per row (64 keys each); bf16 dS overwrites S
//                            dQ += dS K_j            (TS: dS read from TMEM, K_j read MN-major)
//                          The next S tile is issued while the current dS is being computed (S is double buffered).
// dQ is accumulated in TMEM over all KV blocks, so there are no atomics and no fp32 dQ buffer in global memory; the
// result is written as bf16 straight into the q columns of the fused dqkv gradient.
#include "attn_api.h"
#include "common.cuh"

namespace tb {

int make_tmap_2d(CUtensorMap* map, const void* base, int elem_bytes, uint64_t rows, uint64_t cols, uint64_t ld,
                 uint32_t box_rows, uint32_t box_cols);

namespace {

constexpr int HD = 128;
constexpr int TILE_BYTES = 128 * HD * 2;  // 32 KB
constexpr int HALF_BYTES = 16384;
constexpr int KV_STAGES = 2;
constexpr int SMEM_BYTES = 2 * TILE_BYTES + KV_STAGES * 2 * TILE_BYTES + 256 + 1024;
constexpr int NUM_THREADS = 320;  // TMA warp, MMA warp, 8 compute warps (two per TMEM lane quarter)

struct Bars {
  uint64_t q_full;
  uint64_t kv_full[KV_STAGES];
  uint64_t kv_empty[KV_STAGES];
  uint64_t sd_full;    // S_j and dP_j are in TMEM
  uint64_t ds_ready;   // dS_j written (128 arrivals)
  uint64_t dq_done;
  uint32_t tmem_slot;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// delta = rowsum(dO * O) and lse in base 2, per (batch, head, position).  One warp per token row; 16 lanes per head
// (one 16-byte load per lane and tensor), four head pairs in flight.
__global__ void __launch_bounds__(256)
attn_bwd_prep_kernel(const __nv_bfloat16* __restrict__ d_o, const __nv_bfloat16* __restrict__ o,
                     const float* __restrict__ lse, float* __restrict__ delta, float* __restrict__ lse2, int B, int S,
                     int Hq) {
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
    uint4 a[U], c[U];
#pragma unroll
    for (int k = 0; k < U; ++k) {
      const int h = 2 * (hp + k) + hsel;
      a[k] = c[k] = make_uint4(0u, 0u, 0u, 0u);
      if (h < Hq) {
        a[k] = *reinterpret_cast<const uint4*>(pa + h * HD);
        c[k] = *reinterpret_cast<const uint4*>(pc + h * HD);
      }
    }
#pragma unroll
    for (int k = 0; k < U; ++k) {
      const int h = 2 * (hp + k) + hsel;
      const __nv_bfloat162* xa = reinterpret_cast<const __nv_bfloat162*>(&a[k]);
      const __nv_bfloat162* xc = reinterpret_cast<const __nv_bfloat162*>(&c[k]);
      float acc = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 x = __bfloat1622float2(xa[e]), y = __bfloat1622float2(xc[e]);
        acc += x.x * y.x + x.y * y.y;
      }
#pragma unroll
      for (int s2 = 8; s2 > 0; s2 >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s2);
      if (sub == 0 && h < Hq) {
        const int64_t idx = (static_cast<int64_t>(b) * Hq + h) * S + pos;
        delta[idx] = acc;
        lse2[idx] = lse[idx] * 1.4426950408889634f;
      }
    }
  }
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQK, const __grid_constant__ CUtensorMap tmV,
                   const __grid_constant__ CUtensorMap tmDO, const __grid_constant__ CUtensorMap tmDQKV,
                   const float* __restrict__ delta, const float* __restrict__ lse2, int B, int S, int Hq, int Hkv,
                   float scale, float scale_log2, int* err) {
  pdl_wait();
  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sDO = smem + TILE_BYTES;
  uint8_t* sKV = smem + 2 * TILE_BYTES;
  Bars* bars = reinterpret_cast<Bars*>(sKV + KV_STAGES * 2 * TILE_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nblk = S / 128;
  const int groups = B * Hq;
  const int qblk = nblk - 1 - static_cast<int>(blockIdx.x) / groups;
  const int g = static_cast<int>(blockIdx.x) % groups;
  const int h = g % Hq, b = g / Hq;
  const int kvh = h / (Hq / Hkv);
  const int row0 = b * S + qblk * 128;
  const int n_kv = qblk + 1;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmDO);
    tma_prefetch_desc(&tmDQKV);
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&bars->kv_full[s], 1);
      mbar_init(&bars->kv_empty[s], 1);
    }
    mbar_init(&bars->sd_full, 1);
    mbar_init(&bars->ds_ready, 256);
    mbar_init(&bars->dq_done, 1);
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
  // TMEM columns: S[0] 0..127, S[1] 128..255, dP 256..383, dQ 384..511

  if (warp == 0) {
    if (elect_one()) {
      mbar_expect_tx(&bars->q_full, 2 * TILE_BYTES);
      for (int hf = 0; hf < 2; ++hf) {
        tma_load_2d(sQ + hf * HALF_BYTES, &tmQK, &bars->q_full, h * HD + hf * 64, row0);
        tma_load_2d(sDO + hf * HALF_BYTES, &tmDO, &bars->q_full, h * HD + hf * 64, row0);
      }
      const int kcol = (Hq + kvh) * HD, vcol = (Hq + Hkv + kvh) * HD;
      for (int j = 0; j < n_kv; ++j) {
        const int s = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        if (!mbar_wait(&bars->kv_empty[s], ph ^ 1, err, kErrAttnWait)) break;
        uint8_t* sK = sKV + s * 2 * TILE_BYTES;
        uint8_t* sV = sK + TILE_BYTES;
        const int krow = b * S + j * 128;
        mbar_expect_tx(&bars->kv_full[s], 2 * TILE_BYTES);
        tma_load_2d(sK, &tmQK, &bars->kv_full[s], kcol, krow);
        tma_load_2d(sK + HALF_BYTES, &tmQK, &bars->kv_full[s], kcol + 64, krow);
        tma_load_2d(sV, &tmV, &bars->kv_full[s], vcol, krow);
        tma_load_2d(sV + HALF_BYTES, &tmV, &bars->kv_full[s], vcol + 64, krow);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc_kk = make_idesc_bf16(128, 128, false, false);  // both operands K-major
      constexpr uint32_t idesc_ts = make_idesc_bf16(128, 128, false, true);   // A in TMEM, B MN-major
      auto issue_ss = [&](uint32_t d_col, const uint8_t* a_tile, const uint8_t* b_tile) {
        const uint32_t aa = smem_u32(a_tile), ba = smem_u32(b_tile);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t o = (ks >> 2) * HALF_BYTES + (ks & 3) * 32;
          umma_f16_ss(tmem_base + d_col, make_desc_sw128(aa + o, 16, 1024), make_desc_sw128(ba + o, 16, 1024), idesc_kk,
                      ks != 0 ? 1u : 0u);
        }
      };
      bool ok = mbar_wait(&bars->q_full, 0, err, kErrAttnWait) && mbar_wait(&bars->kv_full[0], 0, err, kErrAttnWait);
      if (ok) {
        tc_fence_after();
        issue_ss(0, sQ, sKV);                       // S_0
        issue_ss(256, sDO, sKV + TILE_BYTES);       // dP_0
        umma_commit(&bars->sd_full);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j % KV_STAGES, sn = (j + 1) % KV_STAGES;
        const uint32_t phn = ((j + 1) / KV_STAGES) & 1;
        const bool more = j + 1 < n_kv;
        if (more) {
          if (!mbar_wait(&bars->kv_full[sn], phn, err, kErrAttnWait)) { ok = false; break; }
          tc_fence_after();
          issue_ss(((j + 1) & 1) * 128, sQ, sKV + sn * 2 * TILE_BYTES);   // S_{j+1} while dS_j is computed
        }
        if (!mbar_wait(&bars->ds_ready, j & 1, err, kErrAttnWait)) { ok = false; break; }
        tc_fence_after();
        const uint32_t ka = smem_u32(sKV + s * 2 * TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          // dS keys 0..63 sit at columns 0..31 of the S tile, keys 64..127 at columns 64..95
          umma_f16_ts(tmem_base + 384, tmem_base + (j & 1) * 128 + (ks >> 2) * 64 + (ks & 3) * 8,
                      make_desc_sw128(ka + ks * 2048, HALF_BYTES, 1024), idesc_ts, (j == 0 && ks == 0) ? 0u : 1u);
        }
        umma_commit(&bars->kv_empty[s]);
        if (more) {
          issue_ss(256, sDO, sKV + sn * 2 * TILE_BYTES + TILE_BYTES);    // dP_{j+1}
          umma_commit(&bars->sd_full);
        }
      }
      if (ok) umma_commit(&bars->dq_done);
    }
  } else {
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    const int64_t stat = (static_cast<int64_t>(b) * Hq + h) * S + qblk * 128 + row;
    const float my_lse2 = lse2[stat], my_delta = delta[stat];
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      if (!mbar_wait(&bars->sd_full, j & 1, err, kErrAttnWait)) { ok = false; break; }
      tc_fence_after();
      const bool diag = j == n_kv - 1;
      const uint32_t tS = tmem_base + lane_sel + (j & 1) * 128;
      const uint32_t tP = tmem_base + lane_sel + 256;
      {   // this warp's 64 of the 128 key columns: four TMEM loads in flight, one wait
        const int hc = (warp - 2) >> 2;
        uint32_t sv[64], dv[64];
        tmem_ld_32x32b_x32(tS + hc * 64, *reinterpret_cast<uint32_t(*)[32]>(&sv[0]));
        tmem_ld_32x32b_x32(tS + hc * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[32]));
        tmem_ld_32x32b_x32(tP + hc * 64, *reinterpret_cast<uint32_t(*)[32]>(&dv[0]));
        tmem_ld_32x32b_x32(tP + hc * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&dv[32]));
        tmem_ld_wait();
#pragma unroll
        for (int c2 = 0; c2 < 2; ++c2) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int k0 = c2 * 32 + 2 * i;
            float p0 = ex2(fmaf(__uint_as_float(sv[k0]), scale_log2, -my_lse2));
            float p1 = ex2(fmaf(__uint_as_float(sv[k0 + 1]), scale_log2, -my_lse2));
            if (diag) {
              if (hc * 64 + k0 > row) p0 = 0.f;
              if (hc * 64 + k0 + 1 > row) p1 = 0.f;
            }
            const float d0 = p0 * (__uint_as_float(dv[k0]) - my_delta) * scale;
            const float d1 = p1 * (__uint_as_float(dv[k0 + 1]) - my_delta) * scale;
            pk[i] = pack_bf16x2(d0, d1);
          }
          tmem_st_32x32b_x16(tS + hc * 64 + c2 * 16, pk);   // inside the columns this warp itself consumed
        }
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars->ds_ready);
    }
    if (ok && warp < 6 && mbar_wait(&bars->dq_done, 0, err, kErrAttnWait)) {
      tc_fence_after();
      uint8_t* stage = sQ + quarter * 8192;   // Q is dead once the last S tile has been produced
      const uint32_t tD = tmem_base + lane_sel + 384;
      uint32_t v[32];
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        tmem_ld_32x32b_x32(tD + c * 32, v);
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
        tma_store_2d(&tmDQKV, stage, h * HD, row0 + quarter * 32);
        tma_store_2d(&tmDQKV, stage + 4096, h * HD + 64, row0 + quarter * 32);
        tma_commit_group();
        tma_wait_group<0>();
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

}  // namespace

int attn_bwd_prep(const void* d_o, const void* o, const float* lse, float* delta, float* lse2, int B, int S, int Hq,
                  cudaStream_t stream) {
  const int64_t warps = static_cast<int64_t>(B) * S;  // one warp per token row
  return launch_pdl(attn_bwd_prep_kernel, dim3(static_cast<int>((warps + 7) / 8)), dim3(256), 0, stream, 
      reinterpret_cast<const __nv_bfloat16*>(d_o), reinterpret_cast<const __nv_bfloat16*>(o), lse, delta, lse2, B, S, Hq) == cudaSuccess ? 0 : -21;
}

int attn_bwd_dq(const void* qk, const void* qkv, const void* d_o, void* dqkv, const float* delta, const float* lse2,
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
  if (!ensure_dynamic_smem(reinterpret_cast<const void*>(attn_bwd_dq_kernel), SMEM_BYTES)) return -20;
  const int grid = (S / 128) * B * Hq;
  const float scale = 1.f / sqrtf(static_cast<float>(HD));
  launch_pdl(attn_bwd_dq_kernel, dim3(grid), dim3(NUM_THREADS), SMEM_BYTES, stream, tq, tv, tdo, tdq, delta, lse2, B, S, Hq, Hkv, scale,
                                                                 scale * 1.4426950408889634f, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

}  // namespace tb
