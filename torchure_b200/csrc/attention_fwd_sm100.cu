// Causal GQA flash-attention forward for sm_100a (head_dim 128), tcgen05 + TMEM + TMA.
//
// One CTA owns 128 query positions of TWO query heads that share a KV head (GQA), so every K/V tile brought
// into shared memory feeds four MMAs and both heads do identical causal work.  320 threads:
//   warp 0      TMA producer: Q of both heads once, then a 2-stage ring of K_j / V_j tiles (128 keys each)
//   warp 1      MMA issuer:   S_t = Q_t K_j^T (SS, 128x128x128)  and  O_t += P_t V_j (TS: P read from TMEM)
//   warps 2-5   softmax of head 0, one thread per query row     } while one group runs exp2 on its S tile the
//   warps 6-9   softmax of head 1                               } tensor core works on the other head's tiles
// TMEM (512 columns): S0 | S1 | O0 | O1, 128 fp32 columns each.  P (bf16) overwrites the first 64 columns of its
// S tile and is consumed from there as the A operand of the second MMA, so probabilities never touch shared memory.
// The running maximum is only refreshed when it grew by more than 2^8 (exact after the final 1/l normalisation),
// which makes rescaling the TMEM accumulator a rare event.  LSE (natural log) is written for backward.
#include "attn_api.h"
#include "common.cuh"

namespace tb {

namespace {

constexpr int BQ = 128, BKV = 128, HD = 128;
constexpr int TILE_BYTES = BQ * HD * 2;   // 32 KB: two 64-column halves of 16 KB
constexpr int HALF_BYTES = 16384;
constexpr int KV_STAGES = 2;
constexpr int SMEM_BYTES = 2 * TILE_BYTES + KV_STAGES * 2 * TILE_BYTES + 256 + 1024;
constexpr int NUM_THREADS = 320;
constexpr float RESCALE_THRESHOLD = 8.f;

struct Bars {
  uint64_t q_full;
  uint64_t k_full[KV_STAGES];
  uint64_t v_full[KV_STAGES];
  uint64_t kv_empty[KV_STAGES];
  uint64_t s_full[2];
  uint64_t p_ready[2];
  uint64_t o_done[2];
  uint32_t tmem_slot;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Shapes and strides of one call.  Query / output rows of batch b start at b * q_bstride + q_row0 in the q tensor and at
// b * Sq in o and lse; key / value rows at b * kv_bstride + kv_row0.  causal: query block qb sees key blocks <= qb and
// the last one is masked along its diagonal (Sq == Skv); otherwise every query sees all Skv keys (an off-diagonal
// block pair of ring attention).
struct FwdArgs {
  float* lse;
  int B, Sq, Skv, Hq, Hkv;
  int q_col0, k_col0, v_col0;
  int q_bstride, q_row0, kv_bstride, kv_row0;
  int causal;
  float scale_log2;
};

__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                const __grid_constant__ FwdArgs a, int* err) {
  float* __restrict__ lse = a.lse;
  const int B = a.B, S = a.Sq, Hq = a.Hq, Hkv = a.Hkv;
  const float scale_log2 = a.scale_log2;
  pdl_wait();
  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                        // [2][32 KB]
  uint8_t* sKV = smem + 2 * TILE_BYTES;      // [stage][K 32 KB | V 32 KB]
  Bars* bars = reinterpret_cast<Bars*>(sKV + KV_STAGES * 2 * TILE_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nblk = S / BQ;
  const int ratio = Hq / Hkv;
  const int pairs = ratio / 2;
  const int groups = B * Hkv * pairs;
  const int qblk = nblk - 1 - static_cast<int>(blockIdx.x) / groups;   // heaviest tiles first
  int g = static_cast<int>(blockIdx.x) % groups;
  const int pair = g % pairs; g /= pairs;
  const int kvh = g % Hkv;
  const int b = g / Hkv;
  const int h0 = kvh * ratio + pair * 2;    // the two query heads of this CTA: h0, h0 + 1
  const int row0 = b * a.q_bstride + a.q_row0 + qblk * BQ;   // first token row of the query tile in the q tensor
  const int orow0 = b * S + qblk * BQ;                       // ... and in the output
  const int n_kv = a.causal ? qblk + 1 : a.Skv / BKV;        // causal: KV blocks 0..qblk

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmO);
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&bars->k_full[s], 1);
      mbar_init(&bars->v_full[s], 1);
      mbar_init(&bars->kv_empty[s], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&bars->s_full[t], 1);
      mbar_init(&bars->p_ready[t], 128);
      mbar_init(&bars->o_done[t], 1);
    }
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
      mbar_expect_tx(&bars->q_full, 2 * TILE_BYTES);
      for (int t = 0; t < 2; ++t)
        for (int hf = 0; hf < 2; ++hf)
          tma_load_2d(sQ + t * TILE_BYTES + hf * HALF_BYTES, &tmQ, &bars->q_full, a.q_col0 + (h0 + t) * HD + hf * 64, row0);
      const int kcol = a.k_col0 + kvh * HD, vcol = a.v_col0 + kvh * HD;
      for (int j = 0; j < n_kv; ++j) {
        const int s = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        if (!mbar_wait(&bars->kv_empty[s], ph ^ 1, err, kErrAttnWait)) break;
        uint8_t* sK = sKV + s * 2 * TILE_BYTES;
        uint8_t* sV = sK + TILE_BYTES;
        const int krow = b * a.kv_bstride + a.kv_row0 + j * BKV;
        mbar_expect_tx(&bars->k_full[s], TILE_BYTES);
        tma_load_2d(sK, &tmK, &bars->k_full[s], kcol, krow);
        tma_load_2d(sK + HALF_BYTES, &tmK, &bars->k_full[s], kcol + 64, krow);
        mbar_expect_tx(&bars->v_full[s], TILE_BYTES);
        tma_load_2d(sV, &tmV, &bars->v_full[s], vcol, krow);
        tma_load_2d(sV + HALF_BYTES, &tmV, &bars->v_full[s], vcol + 64, krow);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(128, 128, false, true);
      // Descriptors are built once per operand; a K step only adds a constant to the 14-bit address field (16-byte
      // units; every operand lies below 256 KB, so the sum never carries into the next field).
      uint64_t dQ[2], dK[KV_STAGES], dV[KV_STAGES];
#pragma unroll
      for (int t = 0; t < 2; ++t) dQ[t] = make_desc_sw128(smem_u32(sQ + t * TILE_BYTES), 16, 1024);
#pragma unroll
      for (int st = 0; st < KV_STAGES; ++st) {
        dK[st] = make_desc_sw128(smem_u32(sKV + st * 2 * TILE_BYTES), 16, 1024);
        dV[st] = make_desc_sw128(smem_u32(sKV + st * 2 * TILE_BYTES + TILE_BYTES), HALF_BYTES, 1024);
      }
      auto issue_s = [&](int t, int stage) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t o = ((ks >> 2) * HALF_BYTES + (ks & 3) * 32) >> 4;
          umma_f16_ss(tmem_base + t * 128, dQ[t] + o, dK[stage] + o, idesc_s, ks != 0 ? 1u : 0u);
        }
        umma_commit(&bars->s_full[t]);
      };
      auto issue_pv = [&](int t, int stage, bool first) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          umma_f16_ts(tmem_base + 256 + t * 128, tmem_base + t * 128 + ks * 8, dV[stage] + ks * (2048 >> 4), idesc_pv,
                      (first && ks == 0) ? 0u : 1u);
        }
        umma_commit(&bars->o_done[t]);
      };
      bool ok = mbar_wait(&bars->q_full, 0, err, kErrAttnWait);
      ok = ok && mbar_wait(&bars->k_full[0], 0, err, kErrAttnWait);
      if (ok) {
        tc_fence_after();
        issue_s(0, 0);
        issue_s(1, 0);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        const int sn = (j + 1) % KV_STAGES;
        const uint32_t phn = ((j + 1) / KV_STAGES) & 1;
        const bool more = j + 1 < n_kv;
        if (!mbar_wait(&bars->v_full[s], ph, err, kErrAttnWait)) { ok = false; break; }
        for (int t = 0; t < 2 && ok; ++t) {
          if (!mbar_wait(&bars->p_ready[t], j & 1, err, kErrAttnWait)) { ok = false; break; }
          tc_fence_after();
          issue_pv(t, s, j == 0);
          if (t == 1) umma_commit(&bars->kv_empty[s]);
          if (more) {
            if (t == 0 && !mbar_wait(&bars->k_full[sn], phn, err, kErrAttnWait)) { ok = false; break; }
            tc_fence_after();
            issue_s(t, sn);
          }
        }
      }
    }
  } else {
    // ------------------------------------------------ softmax + epilogue
    const int t = (warp - 2) >> 2;          // which head of the pair
    const int quarter = warp & 3;           // TMEM lane quarter of this warp
    const int row = quarter * 32 + lane;    // query row inside the tile
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t tS = tmem_base + lane_sel + t * 128;
    const uint32_t tO = tmem_base + lane_sel + 256 + t * 128;
    float m_used = -1e30f, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      if (!mbar_wait(&bars->s_full[t], j & 1, err, kErrAttnWait)) { ok = false; break; }
      tc_fence_after();
      const bool diag = a.causal && j == n_kv - 1;
      // the whole score row (128 fp32) comes out of TMEM once: four loads in flight, one wait
      uint32_t sv[128];
      tmem_ld_32x32b_x32(tS, *reinterpret_cast<uint32_t(*)[32]>(&sv[0]));
      tmem_ld_32x32b_x32(tS + 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[32]));
      tmem_ld_32x32b_x32(tS + 64, *reinterpret_cast<uint32_t(*)[32]>(&sv[64]));
      tmem_ld_32x32b_x32(tS + 96, *reinterpret_cast<uint32_t(*)[32]>(&sv[96]));
      tmem_ld_wait();
      if (diag) {
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (i > row) sv[i] = 0xff800000u;  // -inf: exp2 gives exactly 0
      }
      float mx0 = -1e30f, mx1 = -1e30f, mx2 = -1e30f, mx3 = -1e30f;
#pragma unroll
      for (int i = 0; i < 128; i += 4) {
        mx0 = fmaxf(mx0, __uint_as_float(sv[i]));
        mx1 = fmaxf(mx1, __uint_as_float(sv[i + 1]));
        mx2 = fmaxf(mx2, __uint_as_float(sv[i + 2]));
        mx3 = fmaxf(mx3, __uint_as_float(sv[i + 3]));
      }
      const float m_new = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * scale_log2;
      if (j == 0) {
        m_used = m_new;
      } else {
        const bool need = m_new > m_used + RESCALE_THRESHOLD;
        if (__any_sync(0xffffffffu, need)) {
          if (!mbar_wait(&bars->o_done[t], (j - 1) & 1, err, kErrAttnWait)) { ok = false; break; }
          tc_fence_after();
          const float alpha = need ? fast_exp2(m_used - m_new) : 1.f;
          uint32_t v[32];
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            tmem_ld_32x32b_x32(tO + c * 32, v);
            tmem_ld_wait();
            uint32_t lo[16], hi[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              lo[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
              hi[i] = __float_as_uint(__uint_as_float(v[16 + i]) * alpha);
            }
            tmem_st_32x32b_x16(tO + c * 32, lo);
            tmem_st_32x32b_x16(tO + c * 32 + 16, hi);
          }
          tmem_st_wait();
          l *= alpha;
          if (need) m_used = m_new;
        }
      }
      float l0 = 0.f, l1 = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(sv[c * 32 + 2 * i]), scale_log2, -m_used));
          const float p1 = fast_exp2(fmaf(__uint_as_float(sv[c * 32 + 2 * i + 1]), scale_log2, -m_used));
          l0 += p0;
          l1 += p1;
          pk[i] = pack_bf16x2(p0, p1);
        }
        tmem_st_32x32b_x16(tS + c * 16, pk);   // P overwrites the first 64 columns of its own S tile
      }
      l += l0 + l1;
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars->p_ready[t]);
    }
    if (ok && mbar_wait(&bars->o_done[t], (n_kv - 1) & 1, err, kErrAttnWait)) {
      tc_fence_after();
      const float inv_l = 1.f / l;
      lse[(static_cast<int64_t>(b) * Hq + h0 + t) * S + qblk * BQ + row] = (m_used + log2f(l)) * 0.6931471805599453f;
      uint8_t* stage = sQ + t * TILE_BYTES + quarter * 8192;   // this head's Q tile is dead: reuse it for staging
      uint32_t v[32];
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        tmem_ld_32x32b_x32(tO + c * 32, v);
        tmem_ld_wait();
        uint8_t* rowp = stage + (c >> 1) * 4096 + lane * 128;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          uint4 pk;
          pk.x = pack_bf16x2(__uint_as_float(v[8 * jj + 0]) * inv_l, __uint_as_float(v[8 * jj + 1]) * inv_l);
          pk.y = pack_bf16x2(__uint_as_float(v[8 * jj + 2]) * inv_l, __uint_as_float(v[8 * jj + 3]) * inv_l);
          pk.z = pack_bf16x2(__uint_as_float(v[8 * jj + 4]) * inv_l, __uint_as_float(v[8 * jj + 5]) * inv_l);
          pk.w = pack_bf16x2(__uint_as_float(v[8 * jj + 6]) * inv_l, __uint_as_float(v[8 * jj + 7]) * inv_l);
          const int chunk = (c & 1) * 4 + jj;   // 16-byte chunk inside the 128-byte row
          *reinterpret_cast<uint4*>(rowp + ((chunk ^ (lane & 7)) << 4)) = pk;
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        tma_store_2d(&tmO, stage, (h0 + t) * HD, orow0 + quarter * 32);
        tma_store_2d(&tmO, stage + 4096, (h0 + t) * HD + 64, orow0 + quarter * 32);
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

int make_tmap_2d(CUtensorMap* map, const void* base, int elem_bytes, uint64_t rows, uint64_t cols, uint64_t ld,
                 uint32_t box_rows, uint32_t box_cols);

namespace {
// Online-softmax merge of a block pair's partial result into the running one, one warp per (token, head) row:
//   new = logaddexp(lse_acc, lse_p);  out = out * exp(lse_acc - new) + o_p * exp(lse_p - new);  lse_acc = new
// out_acc fp32 [B * acc_stride, Hq*128] and lse_acc [B, Hq, acc_stride] cover the whole local sequence, the pair's
// queries start at acc_row0; o_p bf16 [B*Sq, Hq*128], lse_p [B, Hq, Sq] are compact.
__global__ void __launch_bounds__(256)
attn_merge_kernel(float* __restrict__ out_acc, float* __restrict__ lse_acc, const __nv_bfloat16* __restrict__ o_p,
                  const float* __restrict__ lse_p, int B, int Sq, int Hq, int acc_stride, int acc_row0) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t item = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= static_cast<int64_t>(B) * Sq * Hq) return;
  const int h = static_cast<int>(item % Hq);
  const int64_t tok = item / Hq;
  const int s = static_cast<int>(tok % Sq), b = static_cast<int>(tok / Sq);
  const int64_t li = (static_cast<int64_t>(b) * Hq + h) * acc_stride + acc_row0 + s;
  const float l1 = lse_acc[li], l2 = lse_p[(static_cast<int64_t>(b) * Hq + h) * Sq + s];
  const float mx = fmaxf(l1, l2);
  const float e1 = (l1 == -INFINITY) ? 0.f : __expf(l1 - mx), e2 = (l2 == -INFINITY) ? 0.f : __expf(l2 - mx);
  const float inv = 1.f / (e1 + e2);
  const float w1 = e1 * inv, w2 = e2 * inv;
  float* orow = out_acc + (static_cast<int64_t>(b) * acc_stride + acc_row0 + s) * Hq * HD + h * HD + lane * 4;
  const __nv_bfloat16* prow = o_p + tok * Hq * HD + h * HD + lane * 4;
  float4 x = *reinterpret_cast<const float4*>(orow);
  const uint2 u = *reinterpret_cast<const uint2*>(prow);
  const float2 p0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
  const float2 p1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
  x.x = x.x * w1 + p0.x * w2;
  x.y = x.y * w1 + p0.y * w2;
  x.z = x.z * w1 + p1.x * w2;
  x.w = x.w * w1 + p1.y * w2;
  *reinterpret_cast<float4*>(orow) = x;
  if (lane == 0) lse_acc[li] = mx + __logf(e1 + e2);
}
}  // namespace

int attn_merge(float* out_acc, float* lse_acc, const void* o_p, const float* lse_p, int B, int Sq, int Hq, int acc_stride,
               int acc_row0, cudaStream_t stream) {
  const int64_t items = static_cast<int64_t>(B) * Sq * Hq;
  return launch_pdl(attn_merge_kernel, dim3(static_cast<int>((items + 7) / 8)), dim3(256), 0, stream, out_acc, lse_acc,
                    reinterpret_cast<const __nv_bfloat16*>(o_p), lse_p, B, Sq, Hq, acc_stride, acc_row0) == cudaSuccess
             ? 0
             : -21;
}

int attn_fwd_pair(const AttnOperand& q, const AttnOperand& k, const AttnOperand& v, void* o, float* lse, int B, int Sq,
                  int Skv, int Hq, int Hkv, int64_t q_rows, int q_bstride, int q_row0, int64_t kv_rows, int kv_bstride,
                  int kv_row0, bool causal, int* err, cudaStream_t stream) {
  if (Sq % 128 != 0 || Skv % 128 != 0 || Hq % Hkv != 0 || (Hq / Hkv) % 2 != 0 || B <= 0) return -1;
  if (causal && Sq != Skv) return -2;
  CUtensorMap tq, tk, tv, to;
  int r = make_tmap_2d(&tq, q.ptr, 2, static_cast<uint64_t>(q_rows), q.ld, q.ld, 128, 64);
  if (r) return r;
  r = make_tmap_2d(&tk, k.ptr, 2, static_cast<uint64_t>(kv_rows), k.ld, k.ld, 128, 64);
  if (r) return r - 100;
  r = make_tmap_2d(&tv, v.ptr, 2, static_cast<uint64_t>(kv_rows), v.ld, v.ld, 128, 64);
  if (r) return r - 150;
  r = make_tmap_2d(&to, o, 2, static_cast<uint64_t>(B) * Sq, static_cast<uint64_t>(Hq) * HD, static_cast<uint64_t>(Hq) * HD,
                   32, 64);
  if (r) return r - 200;
  if (!ensure_dynamic_smem(reinterpret_cast<const void*>(attn_fwd_kernel), SMEM_BYTES)) return -20;
  FwdArgs a{};
  a.lse = lse;
  a.B = B; a.Sq = Sq; a.Skv = Skv; a.Hq = Hq; a.Hkv = Hkv;
  a.q_col0 = static_cast<int>(q.col0);
  a.k_col0 = static_cast<int>(k.col0);
  a.v_col0 = static_cast<int>(v.col0);
  a.q_bstride = q_bstride; a.q_row0 = q_row0; a.kv_bstride = kv_bstride; a.kv_row0 = kv_row0;
  a.causal = causal ? 1 : 0;
  a.scale_log2 = 1.4426950408889634f / sqrtf(static_cast<float>(HD));
  const int grid = (Sq / 128) * B * Hkv * ((Hq / Hkv) / 2);
  return launch_pdl(attn_fwd_kernel, dim3(grid), dim3(NUM_THREADS), SMEM_BYTES, stream, tq, tk, tv, to, a, err) ==
                 cudaSuccess
             ? 0
             : -21;
}

int attn_fwd(const void* qk, const void* qkv, void* o, float* lse, int B, int S, int Hq, int Hkv, int* err,
             cudaStream_t stream) {
  const int64_t wqk = static_cast<int64_t>(Hq + Hkv) * HD, wqkv = static_cast<int64_t>(Hq + 2 * Hkv) * HD;
  const int64_t M = static_cast<int64_t>(B) * S;
  return attn_fwd_pair({qk, wqk, 0}, {qk, wqk, static_cast<int64_t>(Hq) * HD},
                       {qkv, wqkv, static_cast<int64_t>(Hq + Hkv) * HD}, o, lse, B, S, S, Hq, Hkv, M, S, 0, M, S, 0, true, err,
                       stream);
}

}  // namespace tb
