// Memory-bound kernels of the transformer block: fused residual-add + RMSNorm (forward and backward),
// fused per-head QK-norm + RoPE (forward and backward), SwiGLU, embedding scatter-add, the fused
// softmax / loss / dlogits step of linear+cross-entropy, casts and conditional scaling.
//
// All of them stream each byte from HBM once with 16-byte accesses where the layout allows; statistics
// are fp32.  A row is handled by one warp (norms, RoPE) or one CTA (vocabulary rows).
#include "api.h"
#include "common.cuh"

#include <cuda_bf16.h>
#include <stdint.h>

#include <algorithm>
#include <type_traits>

namespace tb {

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float2 bf2_to_f2(uint32_t u) {
  __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(b);
}
__device__ __forceinline__ uint32_t f2_to_bf2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// ---------------------------------------------------------------------------------------------
// add + rmsnorm forward: one warp per row, D % 128 == 0 (lane handles float4 groups strided by 32)
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
add_rmsnorm_fwd_kernel(const float* __restrict__ x, const __nv_bfloat16* __restrict__ y,
                       const int64_t* __restrict__ ids, const float* __restrict__ table,
                       const __nv_bfloat16* __restrict__ table_bf16, const float* __restrict__ w,
                       float* __restrict__ x_out, __nv_bfloat16* __restrict__ h, float* __restrict__ rstd, int M,
                       int D, float eps) {
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= M) return;
  // the gathered row comes from the fp32 table, or from its bf16 copy when only that exists whole (sharded masters)
  const __nv_bfloat16* tr = (ids && table_bf16) ? table_bf16 + ids[row] * static_cast<int64_t>(D) : nullptr;
  const float* xr = tr ? nullptr : (ids ? table + ids[row] * static_cast<int64_t>(D) : x + static_cast<int64_t>(row) * D);
  const __nv_bfloat16* yr = y ? y + static_cast<int64_t>(row) * D : nullptr;
  float* xo = x_out ? x_out + static_cast<int64_t>(row) * D : nullptr;
  __nv_bfloat16* hr = h + static_cast<int64_t>(row) * D;
  const int nvec = D >> 2;
  float ss = 0.f;
  for (int i = lane; i < nvec; i += 32) {
    float4 v;
    if (tr) {
      uint2 u = reinterpret_cast<const uint2*>(tr)[i];
      float2 a = bf2_to_f2(u.x), b = bf2_to_f2(u.y);
      v = make_float4(a.x, a.y, b.x, b.y);
    } else {
      v = reinterpret_cast<const float4*>(xr)[i];
    }
    if (yr) {
      uint2 u = reinterpret_cast<const uint2*>(yr)[i];
      float2 a = bf2_to_f2(u.x), b = bf2_to_f2(u.y);
      v.x += a.x; v.y += a.y; v.z += b.x; v.w += b.y;
    }
    if (xo) reinterpret_cast<float4*>(xo)[i] = v;
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / D + eps);
  if (lane == 0) rstd[row] = r;
  // second pass: the row was just touched by this warp (its own writes when x_out is given)
  const float* src = xo ? xo : xr;
  const bool readd = (xo == nullptr) && (yr != nullptr);
  __syncwarp();
  for (int i = lane; i < nvec; i += 32) {
    float4 v = reinterpret_cast<const float4*>(src)[i];
    if (readd) {
      uint2 u = reinterpret_cast<const uint2*>(yr)[i];
      float2 a = bf2_to_f2(u.x), b = bf2_to_f2(u.y);
      v.x += a.x; v.y += a.y; v.z += b.x; v.w += b.y;
    }
    float4 g = reinterpret_cast<const float4*>(w)[i];
    uint2 o;
    o.x = f2_to_bf2(v.x * r * g.x, v.y * r * g.y);
    o.y = f2_to_bf2(v.z * r * g.z, v.w * r * g.w);
    reinterpret_cast<uint2*>(hr)[i] = o;
  }
}

// ---------------------------------------------------------------------------------------------
// rmsnorm backward (+ residual grad add): persistent warps, dw accumulated per CTA then atomics
// ---------------------------------------------------------------------------------------------
template <int MAX_VEC>  // float4 groups per lane kept in registers for the dw partial (D <= 128*MAX_VEC)
__global__ void __launch_bounds__(256)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dh, const float* __restrict__ x, const float* __restrict__ w,
                   const float* __restrict__ rstd, const float* __restrict__ dx_in, float* __restrict__ dx,
                   __nv_bfloat16* __restrict__ dx_bf16, float* __restrict__ dw, int M, int D) {
  const int lane = threadIdx.x & 31;
  const int wid = threadIdx.x >> 5;
  const int warps_total = gridDim.x * 8;
  const int nvec = D >> 2;
  float4 dw_acc[MAX_VEC];
#pragma unroll
  for (int j = 0; j < MAX_VEC; ++j) dw_acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int row = blockIdx.x * 8 + wid; row < M; row += warps_total) {
    const int64_t off = static_cast<int64_t>(row) * D;
    const float r = rstd[row];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < MAX_VEC; ++j) {
      const int i = lane + j * 32;
      if (i < nvec) {
        float4 xv = reinterpret_cast<const float4*>(x + off)[i];
        float4 g = reinterpret_cast<const float4*>(w)[i];
        uint2 u = reinterpret_cast<const uint2*>(dh + off)[i];
        float2 a = bf2_to_f2(u.x), b = bf2_to_f2(u.y);
        dot += (a.x * g.x) * (xv.x * r) + (a.y * g.y) * (xv.y * r) + (b.x * g.z) * (xv.z * r) + (b.y * g.w) * (xv.w * r);
      }
    }
    dot = warp_sum(dot) / D;
#pragma unroll
    for (int j = 0; j < MAX_VEC; ++j) {
      const int i = lane + j * 32;
      if (i < nvec) {
        float4 xv = reinterpret_cast<const float4*>(x + off)[i];
        float4 g = reinterpret_cast<const float4*>(w)[i];
        uint2 u = reinterpret_cast<const uint2*>(dh + off)[i];
        float2 a = bf2_to_f2(u.x), b = bf2_to_f2(u.y);
        float4 xh = make_float4(xv.x * r, xv.y * r, xv.z * r, xv.w * r);
        float4 o;
        o.x = r * (a.x * g.x - xh.x * dot);
        o.y = r * (a.y * g.y - xh.y * dot);
        o.z = r * (b.x * g.z - xh.z * dot);
        o.w = r * (b.y * g.w - xh.w * dot);
        if (dx_in) {
          float4 p = reinterpret_cast<const float4*>(dx_in + off)[i];
          o.x += p.x; o.y += p.y; o.z += p.z; o.w += p.w;
        }
        reinterpret_cast<float4*>(dx + off)[i] = o;
        if (dx_bf16) {
          uint2 ob;
          ob.x = f2_to_bf2(o.x, o.y);
          ob.y = f2_to_bf2(o.z, o.w);
          reinterpret_cast<uint2*>(dx_bf16 + off)[i] = ob;
        }
        dw_acc[j].x += a.x * xh.x; dw_acc[j].y += a.y * xh.y; dw_acc[j].z += b.x * xh.z; dw_acc[j].w += b.y * xh.w;
      }
    }
  }
  // reduce the 8 warps of the CTA through shared memory, then one atomic per element per CTA
  extern __shared__ float red[];  // [D]
  for (int i = threadIdx.x; i < D; i += blockDim.x) red[i] = 0.f;
  __syncthreads();
#pragma unroll
  for (int j = 0; j < MAX_VEC; ++j) {
    const int i = lane + j * 32;
    if (i < nvec) {
      atomicAdd(&red[4 * i + 0], dw_acc[j].x);
      atomicAdd(&red[4 * i + 1], dw_acc[j].y);
      atomicAdd(&red[4 * i + 2], dw_acc[j].z);
      atomicAdd(&red[4 * i + 3], dw_acc[j].w);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < D; i += blockDim.x) atomicAdd(&dw[i], red[i]);
}

// ---------------------------------------------------------------------------------------------
// rmsnorm backward for D <= 1024: four 4-warp CTAs per SM, each owning a contiguous range of rows; a warp keeps its
// row's x and dh in registers between the dot-product pass and the output pass (each byte is read once), and the
// weight gradient leaves the CTA as 16-byte vector reductions (one per four columns per CTA).  The CTAs are small
// (16 K registers, 16 KB shared memory) so that they also fit on an SM that hosts a CTA of a gradient all-reduce
// kernel; one 64 K-register CTA per SM had to wait for those SMs and ran in two waves during DDP steps.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void red_add_v4(float* p, const float4& v) {
  asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

template <int MAX_VEC, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, 16 / WARPS)
rmsnorm_bwd_rows_kernel(const __nv_bfloat16* __restrict__ dh, const float* __restrict__ x, const float* __restrict__ w,
                        const float* __restrict__ rstd, const float* __restrict__ dx_in, float* __restrict__ dx,
                        __nv_bfloat16* __restrict__ dx_bf16, float* __restrict__ dw, int M, int D) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int wid = threadIdx.x >> 5;
  const int nvec = D >> 2;
  const int lo = static_cast<int>(static_cast<int64_t>(M) * blockIdx.x / gridDim.x);
  const int hi = static_cast<int>(static_cast<int64_t>(M) * (blockIdx.x + 1) / gridDim.x);
  float4 dw_acc[MAX_VEC];
#pragma unroll
  for (int j = 0; j < MAX_VEC; ++j) dw_acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int row = lo + wid; row < hi; row += WARPS) {
    const int64_t off = static_cast<int64_t>(row) * D;
    float4 xv[MAX_VEC];
    uint2 dv[MAX_VEC];
#pragma unroll
    for (int j = 0; j < MAX_VEC; ++j) {
      const int i = lane + j * 32;
      if (i < nvec) {
        xv[j] = reinterpret_cast<const float4*>(x + off)[i];
        dv[j] = reinterpret_cast<const uint2*>(dh + off)[i];
      }
    }
    const float r = rstd[row];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < MAX_VEC; ++j) {
      const int i = lane + j * 32;
      if (i < nvec) {
        const float4 g = reinterpret_cast<const float4*>(w)[i];
        const float2 a = bf2_to_f2(dv[j].x), b = bf2_to_f2(dv[j].y);
        xv[j].x *= r; xv[j].y *= r; xv[j].z *= r; xv[j].w *= r;  // normalised row from here on
        dot += (a.x * g.x) * xv[j].x + (a.y * g.y) * xv[j].y + (b.x * g.z) * xv[j].z + (b.y * g.w) * xv[j].w;
      }
    }
    dot = warp_sum(dot) / D;
#pragma unroll
    for (int j = 0; j < MAX_VEC; ++j) {
      const int i = lane + j * 32;
      if (i < nvec) {
        const float4 g = reinterpret_cast<const float4*>(w)[i];
        const float2 a = bf2_to_f2(dv[j].x), b = bf2_to_f2(dv[j].y);
        float4 o;
        o.x = r * (a.x * g.x - xv[j].x * dot);
        o.y = r * (a.y * g.y - xv[j].y * dot);
        o.z = r * (b.x * g.z - xv[j].z * dot);
        o.w = r * (b.y * g.w - xv[j].w * dot);
        if (dx_in) {   // requested here on purpose: hoisting these loads above the reduction costs 30 registers and
                       // measured 20 % slower
          const float4 p = reinterpret_cast<const float4*>(dx_in + off)[i];
          o.x += p.x; o.y += p.y; o.z += p.z; o.w += p.w;
        }
        reinterpret_cast<float4*>(dx + off)[i] = o;
        if (dx_bf16) {
          uint2 ob;
          ob.x = f2_to_bf2(o.x, o.y);
          ob.y = f2_to_bf2(o.z, o.w);
          reinterpret_cast<uint2*>(dx_bf16 + off)[i] = ob;
        }
        dw_acc[j].x += a.x * xv[j].x; dw_acc[j].y += a.y * xv[j].y;
        dw_acc[j].z += b.x * xv[j].z; dw_acc[j].w += b.y * xv[j].w;
      }
    }
  }
  // WARPS warps -> one partial per column in shared memory -> one vector reduction per four columns
  extern __shared__ float red[];  // [WARPS][D]
#pragma unroll
  for (int j = 0; j < MAX_VEC; ++j) {
    const int i = lane + j * 32;
    if (i < nvec) reinterpret_cast<float4*>(red + wid * D)[i] = dw_acc[j];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int k = 0; k < WARPS; ++k) {
      const float4 v = reinterpret_cast<const float4*>(red + k * D)[i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    red_add_v4(dw + 4 * i, acc);
  }
}

// ---------------------------------------------------------------------------------------------
// rmsnorm backward for D <= 1024, rows staged through shared memory by bulk copies (the scheme of the QK-norm / RoPE
// backward further down): every warp of one persistent CTA per SM owns one or two row buffers [x fp32 | dh bf16 |
// dx_in fp32]; while it works on a row the next one is in flight, at no register cost, and the second pass (outputs
// and gain gradient) re-reads the row from shared memory instead of holding it in registers.  Eight warps of at most
// 128 registers: the CTA fits beside a 512-thread CTA of a gradient all-reduce kernel.
// ---------------------------------------------------------------------------------------------
constexpr int RNB_MAX_WARPS = 8;

__global__ void __launch_bounds__(RNB_MAX_WARPS * 32, 2)
rmsnorm_bwd_staged_kernel(const __nv_bfloat16* __restrict__ dh, const float* __restrict__ x, const float* __restrict__ w,
                          const float* __restrict__ rstd, const float* __restrict__ dx_in, float* __restrict__ dx,
                          __nv_bfloat16* __restrict__ dx_bf16, float* __restrict__ dw, int M, int D, int stage_bytes,
                          int stages, int* err) {
  pdl_wait();
  pdl_launch_dependents();
  constexpr int MAX_VEC = 8;
  extern __shared__ __align__(128) uint8_t rn_smem[];
  __shared__ uint64_t bars[RNB_MAX_WARPS][2];
  const int lane = threadIdx.x & 31;
  const int wid = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int nvec = D >> 2;
  uint8_t* buf = rn_smem + static_cast<size_t>(wid) * stages * stage_bytes;
  const int off_dh = D * 4, off_in = D * 6;
  if (lane == 0) {
    mbar_init(&bars[wid][0], 1);
    mbar_init(&bars[wid][1], 1);
    fence_barrier_init();
  }
  __syncthreads();
  float4 wv[MAX_VEC], dw_acc[MAX_VEC];
#pragma unroll
  for (int j = 0; j < MAX_VEC; ++j) {
    const int i = lane + j * 32;
    wv[j] = i < nvec ? reinterpret_cast<const float4*>(w)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    dw_acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const uint32_t tx_bytes = static_cast<uint32_t>(D * (dx_in ? 10 : 6));
  auto issue = [&](int row, int stage) {
    uint8_t* dst = buf + stage * stage_bytes;
    uint64_t* bar = &bars[wid][stage];
    if (lane == 0) mbar_expect_tx(bar, tx_bytes);
    __syncwarp();
    const int64_t off = static_cast<int64_t>(row) * D;
    if (lane == 0) bulk_load_1d(dst, x + off, static_cast<uint32_t>(D * 4), bar);
    else if (lane == 1) bulk_load_1d(dst + off_dh, dh + off, static_cast<uint32_t>(D * 2), bar);
    else if (lane == 2 && dx_in) bulk_load_1d(dst + off_in, dx_in + off, static_cast<uint32_t>(D * 4), bar);
  };
  const int row0 = blockIdx.x * warps + wid, row_step = gridDim.x * warps;
  const bool two = stages == 2;
  bool ok = true;
  if (two && row0 < M) issue(row0, 0);
  float r_next = row0 < M ? rstd[row0] : 0.f;
  int k = 0;
  for (int row = row0; row < M; row += row_step, ++k) {
    const int stage = two ? (k & 1) : 0;
    if (!two) issue(row, 0);
    else if (row + row_step < M) issue(row + row_step, stage ^ 1);
    const float r = r_next;
    if (row + row_step < M) r_next = rstd[row + row_step];
    if (!mbar_wait(&bars[wid][stage], (two ? (k >> 1) : k) & 1, err, kErrStagedRowWait)) { ok = false; break; }
    const uint8_t* st = buf + stage * stage_bytes;
    const float2 r2 = make_float2(r, r);
    // pass 1: dot = mean(dh w xhat)
    float2 dot2 = make_float2(0.f, 0.f);
#pragma unroll
    for (int j = 0; j < MAX_VEC; ++j) {
      const int i = lane + j * 32;
      if (i < nvec) {
        const float4 xv = reinterpret_cast<const float4*>(st)[i];
        const uint2 dv = reinterpret_cast<const uint2*>(st + off_dh)[i];
        const float2 a = bf2_to_f2(dv.x), b = bf2_to_f2(dv.y);
        dot2 = fma2(mul2(a, make_float2(wv[j].x, wv[j].y)), make_float2(xv.x, xv.y), dot2);
        dot2 = fma2(mul2(b, make_float2(wv[j].z, wv[j].w)), make_float2(xv.z, xv.w), dot2);
      }
    }
    const float dot = warp_sum(dot2.x + dot2.y) * r / D;
    const float2 nd2 = make_float2(-dot, -dot);
    // pass 2: dx = r (dh w - xhat dot) (+ dx_in), dw += dh xhat
    const int64_t off = static_cast<int64_t>(row) * D;
#pragma unroll
    for (int j = 0; j < MAX_VEC; ++j) {
      const int i = lane + j * 32;
      if (i < nvec) {
        const float4 xv = reinterpret_cast<const float4*>(st)[i];
        const uint2 dv = reinterpret_cast<const uint2*>(st + off_dh)[i];
        const float2 a = bf2_to_f2(dv.x), b = bf2_to_f2(dv.y);
        const float2 xh0 = mul2(make_float2(xv.x, xv.y), r2), xh1 = mul2(make_float2(xv.z, xv.w), r2);
        float2 o0 = mul2(fma2(xh0, nd2, mul2(a, make_float2(wv[j].x, wv[j].y))), r2);
        float2 o1 = mul2(fma2(xh1, nd2, mul2(b, make_float2(wv[j].z, wv[j].w))), r2);
        if (dx_in) {
          const float4 p = reinterpret_cast<const float4*>(st + off_in)[i];
          o0.x += p.x; o0.y += p.y; o1.x += p.z; o1.y += p.w;
        }
        reinterpret_cast<float4*>(dx + off)[i] = make_float4(o0.x, o0.y, o1.x, o1.y);
        if (dx_bf16) reinterpret_cast<uint2*>(dx_bf16 + off)[i] = make_uint2(f2_to_bf2(o0.x, o0.y), f2_to_bf2(o1.x, o1.y));
        const float2 d0 = fma2(a, xh0, make_float2(dw_acc[j].x, dw_acc[j].y));
        const float2 d1 = fma2(b, xh1, make_float2(dw_acc[j].z, dw_acc[j].w));
        dw_acc[j] = make_float4(d0.x, d0.y, d1.x, d1.y);
      }
    }
    __syncwarp();   // every lane is done with this buffer before the next iteration's copies overwrite it
  }
  if (!ok) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  // warps -> one partial per column in shared memory (the row buffers are free now) -> one vector reduction per four
  // columns per CTA
  __syncthreads();
  float* red = reinterpret_cast<float*>(rn_smem);
#pragma unroll
  for (int j = 0; j < MAX_VEC; ++j) {
    const int i = lane + j * 32;
    if (i < nvec) reinterpret_cast<float4*>(red + wid * D)[i] = dw_acc[j];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int kk = 0; kk < warps; ++kk) {
      const float4 v = reinterpret_cast<const float4*>(red + kk * D)[i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    red_add_v4(dw + 4 * i, acc);
  }
}

// ---------------------------------------------------------------------------------------------
// QK-norm + RoPE, hd == 128.  One warp per token row; 16 lanes per head, so a warp instruction covers two heads.
// Lane sub = lane & 15 holds elements 4*sub .. 4*sub+3 AND 64+4*sub .. 64+4*sub+3 of its head (two 8-byte accesses):
// the rotation pairs element i with i + 64, so both partners sit in the same lane and need no shuffle.  cos/sin of
// the row and both gain vectors are loaded once per row and reused by all heads.
// ---------------------------------------------------------------------------------------------
constexpr int QK_UNROLL = 4;      // forward: head pairs in flight per warp
constexpr int QKB_U = 2;         // backward: head pairs whose reductions are interleaved
constexpr int QKB_MAX_WARPS = 8;  // backward: warps of the one persistent CTA per SM (see the kernel)

__device__ __forceinline__ void unpack4(const uint2& u, float (&f)[4]) {
  float2 a = bf2_to_f2(u.x), b = bf2_to_f2(u.y);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
__device__ __forceinline__ uint2 pack4(const float (&f)[4]) {
  uint2 u;
  u.x = f2_to_bf2(f[0], f[1]); u.y = f2_to_bf2(f[2], f[3]);
  return u;
}
__device__ __forceinline__ float group16_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ void load4f(const float* p, float (&f)[4]) {
  float4 a = *reinterpret_cast<const float4*>(p);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
}

__global__ void __launch_bounds__(256)
qknorm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ qw,
                       const float* __restrict__ kw, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                       __nv_bfloat16* __restrict__ out, int M, int S, int Hq, int Hkv, float eps, int use_norm) {
  pdl_wait();
  pdl_launch_dependents();
  const int heads = Hq + Hkv;
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= M) return;
  const int sub = lane & 15, hsel = lane >> 4;
  const int in_ld = (Hq + 2 * Hkv) * 128, out_ld = heads * 128;
  const __nv_bfloat16* src = qkv + static_cast<int64_t>(row) * in_ld + sub * 4;
  __nv_bfloat16* dst = out + static_cast<int64_t>(row) * out_ld + sub * 4;
  const int pos = row % S;
  float c[4], sn[4], gq_lo[4], gq_hi[4], gk_lo[4], gk_hi[4];
  load4f(cos_t + static_cast<int64_t>(pos) * 128 + sub * 4, c);  // cos[i] == cos[i + 64]
  load4f(sin_t + static_cast<int64_t>(pos) * 128 + sub * 4, sn);
  if (use_norm) {
    load4f(qw + sub * 4, gq_lo); load4f(qw + 64 + sub * 4, gq_hi);
    load4f(kw + sub * 4, gk_lo); load4f(kw + 64 + sub * 4, gk_hi);
  }
  const int pairs = (heads + 1) >> 1;
  for (int hp = 0; hp < pairs; hp += QK_UNROLL) {
    uint2 ulo[QK_UNROLL], uhi[QK_UNROLL];
#pragma unroll
    for (int k = 0; k < QK_UNROLL; ++k) {
      const int h = 2 * (hp + k) + hsel;
      ulo[k] = uhi[k] = make_uint2(0u, 0u);
      if (h < heads) {
        ulo[k] = *reinterpret_cast<const uint2*>(src + h * 128);
        uhi[k] = *reinterpret_cast<const uint2*>(src + h * 128 + 64);
      }
    }
#pragma unroll
    for (int k = 0; k < QK_UNROLL; ++k) {
      const int h = 2 * (hp + k) + hsel;
      float lo[4], hi[4];
      unpack4(ulo[k], lo);
      unpack4(uhi[k], hi);
      if (use_norm) {
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) ss += lo[e] * lo[e] + hi[e] * hi[e];
        ss = group16_sum(ss);
        const float r = rsqrtf(ss * (1.f / 128.f) + eps);
        const bool is_q = h < Hq;
        // the reference normalises in bf16 precision before RoPE (its q_norm returns bf16)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          lo[e] = lo[e] * r * (is_q ? gq_lo[e] : gk_lo[e]);
          hi[e] = hi[e] * r * (is_q ? gq_hi[e] : gk_hi[e]);
        }
        const uint2 rl = pack4(lo), rh = pack4(hi);
        unpack4(rl, lo);
        unpack4(rh, hi);
      }
      float olo[4], ohi[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        olo[e] = lo[e] * c[e] - hi[e] * sn[e];
        ohi[e] = hi[e] * c[e] + lo[e] * sn[e];
      }
      if (h < heads) {
        *reinterpret_cast<uint2*>(dst + h * 128) = pack4(olo);
        *reinterpret_cast<uint2*>(dst + h * 128 + 64) = pack4(ohi);
      }
    }
  }
}

// Backward of QK-norm + RoPE, one warp per token row, rows staged through shared memory by the TMA unit.
//
// A row needs dq (from the q columns of dqkv, or, ACC, from the head-major fp32 accumulator [B, Hq, S, 128] of the
// single-pass attention backward, which is rounded to bf16 here on the way in instead of by a conversion pass of its
// own), dk, the forward inputs x of the same heads and 64 cos / sin values: 16 KB for 16 + 8 heads.  Loaded straight
// into registers, the bytes a warp keeps in flight are bounded by its register budget and the kernel ran at about a
// third of the copy bandwidth.  Here every warp owns two row buffers; while it works on one row, up to 32 bulk
// copies (one per lane: a head of the accumulator, the dk columns, the x columns, cos, sin) fill the other and
// signal an mbarrier, so that a persistent CTA of eight warps keeps 100 KB and more in flight at no register cost.
// Results are written to dqkv with 8-byte stores (16 lanes cover the 128 contiguous bytes of half a head).
// Eight warps of 128 registers use half of the SM's register file: the CTA also fits on an SM that hosts a 512-thread
// CTA of a gradient all-reduce kernel, so a launch during a data-parallel backward pass does not wait for those SMs.
// Measured on B200, 8192 rows of 16 + 8 heads: 39 us with bf16 dq (two buffers per warp), 52 us with the fp32
// accumulator (16.9 KB rows: one buffer per warp); twelve warps would gain 3 us but fill the register file.
struct QkBwdPlan {
  int dq_bytes;      // Hq * 512 (ACC) or Hq * 256
  int off_dk, off_x, off_cs, stage_bytes;
  int stages;        // row buffers per warp: 2 (the next row loads during this one's arithmetic) or 1
};

template <bool ACC>
__global__ void __launch_bounds__(QKB_MAX_WARPS * 32, 2)   // <= 128 registers
qknorm_rope_bwd_kernel(__nv_bfloat16* __restrict__ dqkv, const __nv_bfloat16* __restrict__ qkv,
                       const float* __restrict__ qw, const float* __restrict__ kw, const float* __restrict__ cos_t,
                       const float* __restrict__ sin_t, float* __restrict__ dqw, float* __restrict__ dkw,
                       const float* __restrict__ dq_acc, int M, int S, int Hq, int Hkv, float eps, int use_norm,
                       QkBwdPlan plan, int* err) {
  pdl_wait();
  pdl_launch_dependents();
  extern __shared__ __align__(128) uint8_t qk_smem[];
  __shared__ uint64_t bars[QKB_MAX_WARPS][2];
  __shared__ __align__(16) float red[2][128];
  const int heads = Hq + Hkv;
  const int lane = threadIdx.x & 31;
  const int wid = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int sub = lane & 15, hsel = lane >> 4;
  const int ld = (Hq + 2 * Hkv) * 128;
  const int pairs = (heads + 1) >> 1;
  uint8_t* buf = qk_smem + static_cast<size_t>(wid) * plan.stages * plan.stage_bytes;
  if (lane == 0) {
    mbar_init(&bars[wid][0], 1);
    mbar_init(&bars[wid][1], 1);
    fence_barrier_init();
  }
  for (int i = threadIdx.x; i < 256; i += blockDim.x) (&red[0][0])[i] = 0.f;
  __syncthreads();
  // gains and this lane's gain-gradient partials as fp32 pairs: [0], [1] elements 4*sub.., [2], [3] elements 64+4*sub..
  float2 gq[4], gk[4], aq[4], ak[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    gq[e] = gk[e] = make_float2(1.f, 1.f);
    aq[e] = ak[e] = make_float2(0.f, 0.f);
  }
  if (use_norm) {
    const float4 q0 = *reinterpret_cast<const float4*>(qw + sub * 4), q1 = *reinterpret_cast<const float4*>(qw + 64 + sub * 4);
    const float4 k0 = *reinterpret_cast<const float4*>(kw + sub * 4), k1 = *reinterpret_cast<const float4*>(kw + 64 + sub * 4);
    gq[0] = make_float2(q0.x, q0.y); gq[1] = make_float2(q0.z, q0.w); gq[2] = make_float2(q1.x, q1.y); gq[3] = make_float2(q1.z, q1.w);
    gk[0] = make_float2(k0.x, k0.y); gk[1] = make_float2(k0.z, k0.w); gk[2] = make_float2(k1.x, k1.y); gk[3] = make_float2(k1.z, k1.w);
  }
  const uint32_t tx_bytes = static_cast<uint32_t>(plan.dq_bytes + Hkv * 256 + (use_norm ? heads * 256 : 0) + 512);
  // every lane issues the copies whose index it owns: [0, n_dq) accumulator heads (or one copy of the q columns),
  // then dk, x, cos, sin
  auto issue = [&](int row, int stage) {
    uint8_t* dst = buf + stage * plan.stage_bytes;
    uint64_t* bar = &bars[wid][stage];
    if (lane == 0) mbar_expect_tx(bar, tx_bytes);
    __syncwarp();
    const int pos = row % S;
    const __nv_bfloat16* drow = dqkv + static_cast<int64_t>(row) * ld;
    const int n_dq = ACC ? Hq : 1;
    for (int i = lane; i < n_dq + 4; i += 32) {
      if (i < n_dq) {
        if (ACC)
          bulk_load_1d(dst + i * 512, dq_acc + ((static_cast<int64_t>(row / S) * Hq + i) * S + pos) * 128, 512, bar);
        else
          bulk_load_1d(dst, drow, static_cast<uint32_t>(Hq * 256), bar);
      } else if (i == n_dq) {
        bulk_load_1d(dst + plan.off_dk, drow + Hq * 128, static_cast<uint32_t>(Hkv * 256), bar);
      } else if (i == n_dq + 1) {
        if (use_norm)
          bulk_load_1d(dst + plan.off_x, qkv + static_cast<int64_t>(row) * ld, static_cast<uint32_t>(heads * 256), bar);
      } else if (i == n_dq + 2) {
        bulk_load_1d(dst + plan.off_cs, cos_t + static_cast<int64_t>(pos) * 128, 256, bar);   // cos[i] == cos[i + 64]
      } else {
        bulk_load_1d(dst + plan.off_cs + 256, sin_t + static_cast<int64_t>(pos) * 128, 256, bar);
      }
    }
  };
  const int row0 = blockIdx.x * warps + wid, row_step = gridDim.x * warps;
  bool ok = true;
  const bool two = plan.stages == 2;
  if (two && row0 < M) issue(row0, 0);
  int k = 0;
  for (int row = row0; row < M; row += row_step, ++k) {
    const int stage = two ? (k & 1) : 0;
    if (!two) issue(row, 0);
    else if (row + row_step < M) issue(row + row_step, stage ^ 1);
    if (!mbar_wait(&bars[wid][stage], (two ? (k >> 1) : k) & 1, err, kErrStagedRowWait)) { ok = false; break; }
    const uint8_t* st = buf + stage * plan.stage_bytes;
    float2 c[2], sn[2], nsn[2];
    {
      const float4 cv = *reinterpret_cast<const float4*>(st + plan.off_cs + sub * 16);
      const float4 sv = *reinterpret_cast<const float4*>(st + plan.off_cs + 256 + sub * 16);
      c[0] = make_float2(cv.x, cv.y); c[1] = make_float2(cv.z, cv.w);
      sn[0] = make_float2(sv.x, sv.y); sn[1] = make_float2(sv.z, sv.w);
      nsn[0] = make_float2(-sv.x, -sv.y); nsn[1] = make_float2(-sv.z, -sv.w);
    }
    __nv_bfloat16* dptr = dqkv + static_cast<int64_t>(row) * ld + sub * 4;
    // One call handles the head pairs [first, first + count) of one kind (q or k, so the gains are not selected per
    // element), QKB_U pairs at a time with every step written across the group: their shuffle chains, the only long
    // dependency of a pass, then overlap.  All arithmetic is on fp32 pairs.  With xh = x r the normalised input,
    // t = n g and d = mean(t xh):  dx = r (t - xh d) = r (g n - (r d) x),  dgain += n xh = (n x) r.
    auto run = [&](auto is_q_tag, int first, int count, const float2 (&g)[4], float2 (&acc)[4]) {
      constexpr bool IS_Q = decltype(is_q_tag)::value;
      for (int p0 = 0; p0 < count; p0 += QKB_U) {
        float2 n[QKB_U][4], x[QKB_U][4], ssd[QKB_U][2];   // ssd: partial sums of x^2 and of g n x
        bool live[QKB_U];
        int hh[QKB_U];
#pragma unroll
        for (int u = 0; u < QKB_U; ++u) {
          const int h = first + 2 * (p0 + u) + hsel;
          live[u] = p0 + u < count && h < (IS_Q ? Hq : heads);   // an idle pass still takes part in the shuffles
          hh[u] = h;
          const int hs = live[u] ? h : first;
          float2 d[4];
          if (ACC && IS_Q) {
            const float4 lo = *reinterpret_cast<const float4*>(st + hs * 512 + sub * 16);
            const float4 hi = *reinterpret_cast<const float4*>(st + hs * 512 + 256 + sub * 16);
            d[0] = make_float2(lo.x, lo.y); d[1] = make_float2(lo.z, lo.w);
            d[2] = make_float2(hi.x, hi.y); d[3] = make_float2(hi.z, hi.w);
          } else {
            const uint8_t* src = IS_Q ? st + hs * 256 : st + plan.off_dk + (hs - Hq) * 256;
            const uint2 lo = *reinterpret_cast<const uint2*>(src + sub * 8), hi = *reinterpret_cast<const uint2*>(src + 128 + sub * 8);
            d[0] = bf2_to_f2(lo.x); d[1] = bf2_to_f2(lo.y); d[2] = bf2_to_f2(hi.x); d[3] = bf2_to_f2(hi.y);
          }
          // transpose of the rotation: n_lo = d_lo c + d_hi s, n_hi = d_hi c - d_lo s
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            n[u][e] = fma2(d[2 + e], sn[e], mul2(d[e], c[e]));
            n[u][2 + e] = fma2(d[e], nsn[e], mul2(d[2 + e], c[e]));
          }
          if (use_norm) {
            const uint8_t* xs = st + plan.off_x + hs * 256;
            const uint2 lo = *reinterpret_cast<const uint2*>(xs + sub * 8), hi = *reinterpret_cast<const uint2*>(xs + 128 + sub * 8);
            x[u][0] = bf2_to_f2(lo.x); x[u][1] = bf2_to_f2(lo.y); x[u][2] = bf2_to_f2(hi.x); x[u][3] = bf2_to_f2(hi.y);
            ssd[u][0] = ssd[u][1] = make_float2(0.f, 0.f);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              ssd[u][0] = fma2(x[u][e], x[u][e], ssd[u][0]);
              ssd[u][1] = fma2(mul2(n[u][e], x[u][e]), g[e], ssd[u][1]);
            }
          }
        }
        if (use_norm) {
          float ss[QKB_U], dot[QKB_U];
#pragma unroll
          for (int u = 0; u < QKB_U; ++u) {
            ss[u] = ssd[u][0].x + ssd[u][0].y;
            dot[u] = ssd[u][1].x + ssd[u][1].y;
          }
#pragma unroll
          for (int o = 8; o > 0; o >>= 1) {
#pragma unroll
            for (int u = 0; u < QKB_U; ++u) {
              ss[u] += __shfl_xor_sync(0xffffffffu, ss[u], o);
              dot[u] += __shfl_xor_sync(0xffffffffu, dot[u], o);
            }
          }
#pragma unroll
          for (int u = 0; u < QKB_U; ++u) {
            const float r = rsqrtf(ss[u] * (1.f / 128.f) + eps);
            const float nrd = -r * r * dot[u] * (1.f / 128.f);      // -(r d)
            const float2 r2 = make_float2(r, r), nrd2 = make_float2(nrd, nrd);
            const float2 ra = live[u] ? r2 : make_float2(0.f, 0.f);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              acc[e] = fma2(mul2(n[u][e], x[u][e]), ra, acc[e]);
              n[u][e] = mul2(fma2(x[u][e], nrd2, mul2(n[u][e], g[e])), r2);
            }
          }
        }
#pragma unroll
        for (int u = 0; u < QKB_U; ++u) {
          if (live[u]) {
            *reinterpret_cast<uint2*>(dptr + hh[u] * 128) =
                make_uint2(f2_to_bf2(n[u][0].x, n[u][0].y), f2_to_bf2(n[u][1].x, n[u][1].y));
            *reinterpret_cast<uint2*>(dptr + hh[u] * 128 + 64) =
                make_uint2(f2_to_bf2(n[u][2].x, n[u][2].y), f2_to_bf2(n[u][3].x, n[u][3].y));
          }
        }
      }
    };
    run(std::true_type{}, 0, (Hq + 1) >> 1, gq, aq);
    run(std::false_type{}, Hq, (Hkv + 1) >> 1, gk, ak);
    __syncwarp();   // every lane is done with this buffer before the next iteration's copies overwrite it
  }
  if (!ok) {
    // a copy may still be landing in this CTA's shared memory: give it time before the CTA retires
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  if (use_norm) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      atomicAdd(&red[0][sub * 4 + 2 * e], aq[e].x);
      atomicAdd(&red[0][sub * 4 + 2 * e + 1], aq[e].y);
      atomicAdd(&red[0][64 + sub * 4 + 2 * e], aq[2 + e].x);
      atomicAdd(&red[0][64 + sub * 4 + 2 * e + 1], aq[2 + e].y);
      atomicAdd(&red[1][sub * 4 + 2 * e], ak[e].x);
      atomicAdd(&red[1][sub * 4 + 2 * e + 1], ak[e].y);
      atomicAdd(&red[1][64 + sub * 4 + 2 * e], ak[2 + e].x);
      atomicAdd(&red[1][64 + sub * 4 + 2 * e + 1], ak[2 + e].y);
    }
    __syncthreads();
    // one 16-byte reduction per four columns per CTA
    if (threadIdx.x < 64) {
      const int which = threadIdx.x >> 5, i = threadIdx.x & 31;
      const float4 v = *reinterpret_cast<const float4*>(&red[which][4 * i]);
      red_add_v4((which ? dkw : dqw) + 4 * i, v);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// SwiGLU: gu [M, 2F] = [gate | up]; act = silu(gate) * up
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ act, int64_t total_vec, int Fv) {
  pdl_wait();
  pdl_launch_dependents();
  // two 16-byte vectors of gate and of up per thread and round: four loads in flight; the quotient is the
  // approximate division (the result is rounded to bf16 anyway)
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < total_vec; i0 += 2 * stride) {
    uint4 g[2], u[2];
#pragma unroll
    for (int v = 0; v < 2; ++v) {
      const int64_t i = i0 + v * stride;
      if (i < total_vec) {
        const int64_t row = i / Fv, col = i % Fv;
        g[v] = reinterpret_cast<const uint4*>(gu)[row * 2 * Fv + col];
        u[v] = reinterpret_cast<const uint4*>(gu)[row * 2 * Fv + Fv + col];
      }
    }
#pragma unroll
    for (int v = 0; v < 2; ++v) {
      const int64_t i = i0 + v * stride;
      if (i >= total_vec) break;
      const uint32_t gs[4] = {g[v].x, g[v].y, g[v].z, g[v].w}, us[4] = {u[v].x, u[v].y, u[v].z, u[v].w};
      uint32_t o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 a = bf2_to_f2(gs[k]), b = bf2_to_f2(us[k]);
        o[k] = f2_to_bf2(__fdividef(a.x, 1.f + __expf(-a.x)) * b.x, __fdividef(a.y, 1.f + __expf(-a.y)) * b.y);
      }
      reinterpret_cast<uint4*>(act)[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dact, const __nv_bfloat16* __restrict__ gu,
                  __nv_bfloat16* __restrict__ dgu, int64_t total_vec, int Fv) {
  pdl_wait();
  pdl_launch_dependents();
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total_vec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = i / Fv, col = i % Fv;
    const uint4 g = reinterpret_cast<const uint4*>(gu)[row * 2 * Fv + col];
    const uint4 u = reinterpret_cast<const uint4*>(gu)[row * 2 * Fv + Fv + col];
    const uint4 d = reinterpret_cast<const uint4*>(dact)[i];
    const uint32_t gs[4] = {g.x, g.y, g.z, g.w}, us[4] = {u.x, u.y, u.z, u.w}, ds[4] = {d.x, d.y, d.z, d.w};
    uint32_t og[4], ou[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 a = bf2_to_f2(gs[k]), b = bf2_to_f2(us[k]), e = bf2_to_f2(ds[k]);
      const float s0 = 1.f / (1.f + __expf(-a.x)), s1 = 1.f / (1.f + __expf(-a.y));
      // d silu(g)/dg = s (1 + g (1 - s))
      og[k] = f2_to_bf2(e.x * b.x * s0 * (1.f + a.x * (1.f - s0)), e.y * b.y * s1 * (1.f + a.y * (1.f - s1)));
      ou[k] = f2_to_bf2(e.x * a.x * s0, e.y * a.y * s1);
    }
    reinterpret_cast<uint4*>(dgu)[row * 2 * Fv + col] = make_uint4(og[0], og[1], og[2], og[3]);
    reinterpret_cast<uint4*>(dgu)[row * 2 * Fv + Fv + col] = make_uint4(ou[0], ou[1], ou[2], ou[3]);
  }
}

// ---------------------------------------------------------------------------------------------
// embedding backward: dtable[ids[r]] += dx[r]  (fp32 atomics; rows of one token id collide rarely)
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
embedding_bwd_kernel(const float* __restrict__ dx, const int64_t* __restrict__ ids, float* __restrict__ dtable,
                     int M, int D) {
  const int row = blockIdx.x;
  if (row >= M) return;
  float* dst = dtable + ids[row] * static_cast<int64_t>(D);
  const float* src = dx + static_cast<int64_t>(row) * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) atomicAdd(&dst[i], src[i]);
}

// Deterministic scatter-add of embedding-row gradients from up to 8 sources (this GPU's rows and, over NVLink, the
// rows every other data-parallel rank left in its symmetric buffer):
//     dtable[id] += scale * sum over sources p = 0..n-1 and rows r = 0..M-1 with ids_p[r] == id of rows_p[r]
// Each destination row belongs to exactly one warp of one CTA (CTA = id mod grid, warp = (id / grid) mod 8), which
// applies its rows with plain loads and stores in (p, r) order: no atomics, so the result has the same bits on every
// rank and in every run.  A CTA scans all ids once, 256 at a time, appending its own matches to a list in shared
// memory by an ordered compaction; the list is applied whenever it fills up.  When sq_delta is given, CTA b stores
// sum(new^2 - old^2) over everything it touched into sq_delta[b] (the sums telescope over repeated rows), which
// turns a sum of squares taken before the scatter into the one after it.
constexpr int EB_THREADS = 256, EB_WARPS = 8, EB_SCAN = 4, EB_LIST = 4096;
struct EmbedSources {
  int n;
  const int64_t* ids[8];
  const float* rows[8];
};

__device__ __forceinline__ float4 ld_sys_f4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int64_t ld_sys_i64(const int64_t* p) {
  int64_t v;
  asm volatile("ld.relaxed.sys.global.s64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// ids of every source -> one local array [n, M]: the scatter kernel below makes every CTA scan all ids, which must
// not be remote reads (at eight ranks that would be 300 MB over NVLink for 512 KB of ids)
__global__ void __launch_bounds__(256)
embedding_gather_ids_kernel(EmbedSources src, int64_t* __restrict__ out, int M) {
  const int total = src.n * M;
  constexpr int U = 4;
  for (int base = (blockIdx.x * 256 + threadIdx.x) * U; base < total; base += gridDim.x * 256 * U) {
    int64_t v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = base + u;
      if (i < total) v[u] = ld_sys_i64(src.ids[i / M] + i % M);
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (base + u < total) out[base + u] = v[u];
  }
}

__global__ void __launch_bounds__(EB_THREADS)
embedding_scatter_kernel(EmbedSources src, float* __restrict__ dtable, int M, int D, float scale,
                         float* __restrict__ sq_delta) {
  __shared__ uint32_t list[EB_LIST];        // (source << 27) | row, in application order
  __shared__ int list_id[EB_LIST];          // the row's token id
  __shared__ int warp_count[EB_SCAN][EB_WARPS];
  __shared__ float warp_delta[EB_WARPS];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nb = gridDim.x;
  int count = 0;
  float delta = 0.f;
  auto apply = [&]() {
    __syncthreads();
    for (int e = 0; e < count; ++e) {
      const int id = list_id[e];
      if ((id / nb) % EB_WARPS != warp) continue;   // another warp of this CTA owns that row
      const uint32_t ent = list[e];
      const int p = ent >> 27, r = ent & ((1u << 27) - 1);
      const float* s = src.rows[p] + static_cast<int64_t>(r) * D;
      float* d = dtable + id * static_cast<int64_t>(D);
      for (int i = lane * 4; i < D; i += 128) {
        const float4 a = ld_sys_f4(s + i);
        float4 b = *reinterpret_cast<float4*>(d + i);
        const float4 o = b;
        b.x = fmaf(scale, a.x, b.x); b.y = fmaf(scale, a.y, b.y); b.z = fmaf(scale, a.z, b.z); b.w = fmaf(scale, a.w, b.w);
        *reinterpret_cast<float4*>(d + i) = b;
        delta += (b.x * b.x - o.x * o.x) + (b.y * b.y - o.y * o.y) + (b.z * b.z - o.z * o.z) + (b.w * b.w - o.w * o.w);
      }
      __syncwarp();   // the next entry of this warp may hit the same row
    }
    __syncthreads();
    count = 0;
  };
  // scan: EB_SCAN ids per thread and round, all loads issued before the first is used; entries are appended in
  // (source, round, slot, warp, lane) order, the same on every rank
  for (int p = 0; p < src.n; ++p) {
    for (int base = 0; base < M; base += EB_THREADS * EB_SCAN) {
      int64_t id[EB_SCAN];
      uint32_t ballot[EB_SCAN];
#pragma unroll
      for (int u = 0; u < EB_SCAN; ++u) {
        const int r = base + u * EB_THREADS + tid;
        id[u] = r < M ? ld_sys_i64(src.ids[p] + r) : -1;
      }
#pragma unroll
      for (int u = 0; u < EB_SCAN; ++u) {
        const bool mine = id[u] >= 0 && static_cast<int>(id[u]) % nb == static_cast<int>(blockIdx.x);
        ballot[u] = __ballot_sync(0xffffffffu, mine);
        if (lane == 0) warp_count[u][warp] = __popc(ballot[u]);
      }
      __syncthreads();
      int at = count, total = 0;
#pragma unroll
      for (int u = 0; u < EB_SCAN; ++u) {
        int before = 0, slot_total = 0;
#pragma unroll
        for (int w = 0; w < EB_WARPS; ++w) {
          const int c = warp_count[u][w];
          if (w < warp) before += c;
          slot_total += c;
        }
        if (ballot[u] & (1u << lane)) {
          const int pos = at + before + __popc(ballot[u] & ((1u << lane) - 1));
          list[pos] = (static_cast<uint32_t>(p) << 27) | static_cast<uint32_t>(base + u * EB_THREADS + tid);
          list_id[pos] = static_cast<int>(id[u]);
        }
        at += slot_total;
        total += slot_total;
      }
      count += total;
      __syncthreads();   // warp_count is rewritten by the next round
      if (count > EB_LIST - EB_THREADS * EB_SCAN) apply();
    }
  }
  apply();
  if (sq_delta != nullptr) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) delta += __shfl_xor_sync(0xffffffffu, delta, o);
    if (lane == 0) warp_delta[warp] = delta;
    __syncthreads();
    if (tid == 0) {
      float t = 0.f;
      for (int w = 0; w < EB_WARPS; ++w) t += warp_delta[w];   // fixed order
      sq_delta[blockIdx.x] = t;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// cross-entropy on one vocabulary row per CTA: online max/sum, target gather, loss, in-place dlogits
// ---------------------------------------------------------------------------------------------
// 1024 threads per row: at most two rows per SM are in flight (296 rows = 90 MB of bf16 logits), so the second pass
// over a row has a chance to find it in the 126 MB L2.  Measured 537 us per 4096 x 151936 chunk (2.5 GB read + written
// once = 4.6 TB/s; three passes' worth of traffic would be the copy bandwidth, so part of the second pass still comes
// from HBM).  A variant that kept the row on chip (a cluster of two 512-thread CTAs, half a row each in shared memory,
// partials exchanged through distributed shared memory) measured 804 us: 74 rows in flight are too few.
constexpr int CE_THREADS = 1024;

//
// Three forms of one kernel.  CE_FUSED: the whole vocabulary is in the row (statistics, loss and gradient in one
// launch).  The other two split it for a vocabulary sharded over ranks, where a row's log-sum-exp needs every rank's
// columns: CE_STATS reads the rank's columns [vocab_lo, vocab_lo + V) once and writes the row's maximum, the sum of
// exponentials relative to it and the target's logit (0 when another rank holds the target) to stats[0 / 1 / 2][row];
// after the ranks have combined these, CE_GRAD overwrites the columns with (exp(logit - lse[row]) - [target]) *
// *inv_n_valid.
enum { CE_FUSED = 0, CE_STATS = 1, CE_GRAD = 2 };

template <int MODE>
__global__ void __launch_bounds__(CE_THREADS)
ce_softmax_grad_kernel(__nv_bfloat16* __restrict__ logits, int64_t ldl, const int64_t* __restrict__ labels,
                       float* __restrict__ row_loss, const float* __restrict__ inv_n_valid, int V,
                       int ignore_index, int64_t vocab_lo, float* __restrict__ stats,
                       const float* __restrict__ lse) {
  const int row = blockIdx.x;
  __nv_bfloat16* lr = logits + static_cast<int64_t>(row) * ldl;
  const int64_t global_label = labels[row];
  const bool valid = global_label != ignore_index;
  // the target's column among this rank's, -1 when it is ignored or lies in another rank's shard
  const int64_t label = (valid && global_label >= vocab_lo && global_label < vocab_lo + V) ? global_label - vocab_lo : -1;
  const int nvec = V >> 3;  // 8 bf16 per 16 B
  __shared__ float s_m[CE_THREADS / 32], s_s[CE_THREADS / 32];
  __shared__ float s_stats[2];
  if (MODE != CE_STATS && !valid) {  // ignored rows contribute neither loss nor gradient
    for (int i = threadIdx.x; i < nvec; i += CE_THREADS) reinterpret_cast<uint4*>(lr)[i] = make_uint4(0, 0, 0, 0);
    for (int i = (nvec << 3) + threadIdx.x; i < V; i += CE_THREADS) lr[i] = __float2bfloat16(0.f);
    if (MODE == CE_FUSED && threadIdx.x == 0) row_loss[row] = 0.f;
    return;
  }
  if constexpr (MODE != CE_GRAD) {
    float m = -INFINITY, s = 0.f;
    auto push = [&](float v) {
      if (v > m) { s = s * __expf(m - v) + 1.f; m = v; }
      else s += __expf(v - m);
    };
#pragma unroll 4
    for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
      uint4 u = reinterpret_cast<const uint4*>(lr)[i];
      const uint32_t us[4] = {u.x, u.y, u.z, u.w};
      float vals[8];
      float lm = -INFINITY;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float2 f = bf2_to_f2(us[k]);
        vals[2 * k] = f.x; vals[2 * k + 1] = f.y;
        lm = fmaxf(lm, fmaxf(f.x, f.y));
      }
      if (lm > m) { s *= __expf(m - lm); m = lm; }
#pragma unroll
      for (int k = 0; k < 8; ++k) s += __expf(vals[k] - m);
    }
    for (int i = (nvec << 3) + threadIdx.x; i < V; i += CE_THREADS) push(__bfloat162float(lr[i]));
    // combine (m, s) across the CTA
    float wm = warp_max(m);
    s = warp_sum(m == -INFINITY ? 0.f : s * __expf(m - wm));
    if ((threadIdx.x & 31) == 0) { s_m[threadIdx.x >> 5] = wm; s_s[threadIdx.x >> 5] = s; }
    __syncthreads();
    if (threadIdx.x < 32) {
      float mm = threadIdx.x < CE_THREADS / 32 ? s_m[threadIdx.x] : -INFINITY;
      float sv = threadIdx.x < CE_THREADS / 32 ? s_s[threadIdx.x] : 0.f;
      float gm = warp_max(mm);
      float gs = warp_sum(mm == -INFINITY ? 0.f : sv * __expf(mm - gm));
      if (threadIdx.x == 0) {
        s_stats[0] = gm;
        s_stats[1] = gs;
        if constexpr (MODE == CE_FUSED) {
          row_loss[row] = gm + __logf(gs) - (label >= 0 ? __bfloat162float(lr[label]) : 0.f);
        } else {
          const int64_t n_rows = gridDim.x;
          stats[row] = gm;
          stats[n_rows + row] = gs;
          stats[2 * n_rows + row] = label >= 0 ? __bfloat162float(lr[label]) : 0.f;
        }
      }
    }
    if constexpr (MODE == CE_STATS) return;
    __syncthreads();
  }
  const float gm = MODE == CE_GRAD ? lse[row] : s_stats[0];
  const float scale = *inv_n_valid;
  const float inv_s = MODE == CE_GRAD ? 1.f : 1.f / s_stats[1];
  const int lvec = label >= 0 ? static_cast<int>(label >> 3) : -1, lsub = static_cast<int>(label & 7);
#pragma unroll 4
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    uint4 u = reinterpret_cast<const uint4*>(lr)[i];
    const uint32_t us[4] = {u.x, u.y, u.z, u.w};
    float vals[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 f = bf2_to_f2(us[k]);
      vals[2 * k] = __expf(f.x - gm) * inv_s;
      vals[2 * k + 1] = __expf(f.y - gm) * inv_s;
    }
    if (i == lvec) vals[lsub] -= 1.f;
    uint4 o;
    o.x = f2_to_bf2(vals[0] * scale, vals[1] * scale);
    o.y = f2_to_bf2(vals[2] * scale, vals[3] * scale);
    o.z = f2_to_bf2(vals[4] * scale, vals[5] * scale);
    o.w = f2_to_bf2(vals[6] * scale, vals[7] * scale);
    reinterpret_cast<uint4*>(lr)[i] = o;
  }
  for (int i = (nvec << 3) + threadIdx.x; i < V; i += CE_THREADS) {
    float p = __expf(__bfloat162float(lr[i]) - gm) * inv_s;
    if (i == label) p -= 1.f;
    lr[i] = __float2bfloat16(p * scale);
  }
}

__global__ void __launch_bounds__(256)
cast_f32_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int64_t n) {
  const int64_t nvec = n >> 2;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float4 v = reinterpret_cast<const float4*>(src)[i];
    uint2 o;
    o.x = f2_to_bf2(v.x, v.y);
    o.y = f2_to_bf2(v.z, v.w);
    reinterpret_cast<uint2*>(dst)[i] = o;
  }
  if (blockIdx.x == 0)
    for (int64_t i = (nvec << 2) + threadIdx.x; i < n; i += blockDim.x) dst[i] = __float2bfloat16(src[i]);
}

__global__ void __launch_bounds__(256)
scale_f32_kernel(float* __restrict__ x, const float* __restrict__ scale, int64_t n) {
  const float s = *scale;
  if (s == 1.f) return;
  const int64_t nvec = n >> 2;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float4 v = reinterpret_cast<float4*>(x)[i];
    v.x *= s; v.y *= s; v.z *= s; v.w *= s;
    reinterpret_cast<float4*>(x)[i] = v;
  }
  if (blockIdx.x == 0)
    for (int64_t i = (nvec << 2) + threadIdx.x; i < n; i += blockDim.x) x[i] *= s;
}

__global__ void __launch_bounds__(256)
scale_bf16_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ scale, int64_t n) {
  const float s = *scale;
  if (s == 1.f) return;
  const int64_t nvec = n >> 3;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    uint4 u = reinterpret_cast<uint4*>(x)[i];
    uint32_t us[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 f = bf2_to_f2(us[k]);
      us[k] = f2_to_bf2(f.x * s, f.y * s);
    }
    reinterpret_cast<uint4*>(x)[i] = make_uint4(us[0], us[1], us[2], us[3]);
  }
  if (blockIdx.x == 0)
    for (int64_t i = (nvec << 3) + threadIdx.x; i < n; i += blockDim.x)
      x[i] = __float2bfloat16(__bfloat162float(x[i]) * s);
}

inline int grid_for(int64_t work_items, int threads, int cap) {
  int64_t g = (work_items + threads - 1) / threads;
  if (g < 1) g = 1;
  return static_cast<int>(g < cap ? g : cap);
}

}  // namespace

void add_rmsnorm_fwd(const float* x, const __nv_bfloat16* y, const int64_t* ids, const float* table,
                     const __nv_bfloat16* table_bf16, const float* w, float* x_out, __nv_bfloat16* h, float* rstd, int M,
                     int D, float eps, cudaStream_t stream) {
  launch_pdl(add_rmsnorm_fwd_kernel, dim3((M + 7) / 8), dim3(256), 0, stream, x, y, ids, table, table_bf16, w, x_out, h,
             rstd, M, D, eps);
}

void rmsnorm_bwd(const __nv_bfloat16* dh, const float* x, const float* w, const float* rstd, const float* dx_in,
                 float* dx, __nv_bfloat16* dx_bf16, float* dw, int M, int D, int num_sms, int* err, cudaStream_t stream,
                 int variant) {
  const bool aligned = D % 8 == 0 && ((reinterpret_cast<uintptr_t>(dh) | reinterpret_cast<uintptr_t>(x) |
                                       reinterpret_cast<uintptr_t>(dx_in)) & 15) == 0;
  if (variant != 1 && D <= 128 * 8 && M >= 4 * num_sms && aligned && err != nullptr) {
    const int stage_bytes = D * (dx_in ? 10 : 6);
    const int budget = 200 * 1024;
    const int stages = 2 * stage_bytes * RNB_MAX_WARPS <= budget ? 2 : 1;
    const int warps = std::min(RNB_MAX_WARPS, budget / (stages * stage_bytes));
    const int smem = std::max(warps * stages * stage_bytes, warps * D * 4);
    if (warps >= 1 && ensure_dynamic_smem(reinterpret_cast<const void*>(rmsnorm_bwd_staged_kernel), smem)) {
      const int grid = std::max(1, std::min((M + warps - 1) / warps, num_sms));
      launch_pdl(rmsnorm_bwd_staged_kernel, dim3(grid), dim3(warps * 32), smem, stream, dh, x, w, rstd, dx_in, dx,
                 dx_bf16, dw, M, D, stage_bytes, stages, err);
      return;
    }
  }
  // two rows per warp keeps every warp equally loaded and the per-CTA atomics on dw few
  if (D <= 128 * 8 && M >= 4 * num_sms) {
    constexpr int W = 4;
    const size_t smem_w = static_cast<size_t>(W) * D * sizeof(float);
    launch_pdl(rmsnorm_bwd_rows_kernel<8, W>, dim3(num_sms * (16 / W)), dim3(W * 32), smem_w, stream, dh, x, w, rstd,
               dx_in, dx, dx_bf16, dw, M, D);
    return;
  }
  const int grid = std::max(1, (M + 15) / 16);
  const size_t smem = static_cast<size_t>(D) * sizeof(float);
  if (D <= 128 * 8) rmsnorm_bwd_kernel<8><<<grid, 256, smem, stream>>>(dh, x, w, rstd, dx_in, dx, dx_bf16, dw, M, D);
  else if (D <= 128 * 20) rmsnorm_bwd_kernel<20><<<grid, 256, smem, stream>>>(dh, x, w, rstd, dx_in, dx, dx_bf16, dw, M, D);
  else rmsnorm_bwd_kernel<64><<<grid, 256, smem, stream>>>(dh, x, w, rstd, dx_in, dx, dx_bf16, dw, M, D);
}

void qknorm_rope_fwd(const __nv_bfloat16* qkv, const float* qw, const float* kw, const float* cos, const float* sin,
                     __nv_bfloat16* out, int M, int S, int Hq, int Hkv, int hd, float eps, int use_norm,
                     cudaStream_t stream) {
  (void)hd;  // 128 only (checked by the caller)
  launch_pdl(qknorm_rope_fwd_kernel, dim3((M + 7) / 8), dim3(256), 0, stream, qkv, qw, kw, cos, sin, out, M, S, Hq, Hkv, eps, use_norm);
}

int qknorm_rope_bwd(__nv_bfloat16* dqkv, const __nv_bfloat16* qkv, const float* qw, const float* kw, const float* cos,
                    const float* sin, float* dqw, float* dkw, const float* dq_acc, int M, int S, int Hq, int Hkv, int hd,
                    float eps, int use_norm, int num_sms, int* err, cudaStream_t stream, int force_stages, int force_warps) {
  (void)hd;
  const bool acc = dq_acc != nullptr;
  QkBwdPlan plan;
  plan.dq_bytes = Hq * (acc ? 512 : 256);
  plan.off_dk = plan.dq_bytes;
  plan.off_x = plan.off_dk + Hkv * 256;
  plan.off_cs = plan.off_x + (Hq + Hkv) * 256;
  plan.stage_bytes = plan.off_cs + 512;
  // as many warps (two row buffers each) as fit into the shared memory of one persistent CTA per SM
  const int budget = 220 * 1024;
  // two buffers per warp when all warps can have them, else one (more warps beat deeper buffers)
  plan.stages = force_stages > 0 ? force_stages : (2 * plan.stage_bytes * QKB_MAX_WARPS <= budget ? 2 : 1);
  int warps = std::min(force_warps > 0 ? std::min(force_warps, QKB_MAX_WARPS) : QKB_MAX_WARPS,
                       budget / (plan.stages * plan.stage_bytes));
  if (warps < 1) return -1;
  const int smem = warps * plan.stages * plan.stage_bytes;
  const void* fn = acc ? reinterpret_cast<const void*>(qknorm_rope_bwd_kernel<true>)
                       : reinterpret_cast<const void*>(qknorm_rope_bwd_kernel<false>);
  if (!ensure_dynamic_smem(fn, smem)) return -2;
  const int grid = std::max(1, std::min((M + warps - 1) / warps, num_sms));
  const cudaError_t rc =
      acc ? launch_pdl(qknorm_rope_bwd_kernel<true>, dim3(grid), dim3(warps * 32), smem, stream, dqkv, qkv, qw, kw, cos,
                       sin, dqw, dkw, dq_acc, M, S, Hq, Hkv, eps, use_norm, plan, err)
          : launch_pdl(qknorm_rope_bwd_kernel<false>, dim3(grid), dim3(warps * 32), smem, stream, dqkv, qkv, qw, kw, cos,
                       sin, dqw, dkw, dq_acc, M, S, Hq, Hkv, eps, use_norm, plan, err);
  return rc == cudaSuccess ? 0 : -3;
}

void swiglu_fwd(const __nv_bfloat16* gu, __nv_bfloat16* act, int M, int F, cudaStream_t stream) {
  const int Fv = F / 8;
  const int64_t total = static_cast<int64_t>(M) * Fv;
  launch_pdl(swiglu_fwd_kernel, dim3(grid_for(total, 256, 148 * 16)), dim3(256), 0, stream, gu, act, total, Fv);
}

void swiglu_bwd(const __nv_bfloat16* dact, const __nv_bfloat16* gu, __nv_bfloat16* dgu, int M, int F,
                cudaStream_t stream) {
  const int Fv = F / 8;
  const int64_t total = static_cast<int64_t>(M) * Fv;
  launch_pdl(swiglu_bwd_kernel, dim3(grid_for(total, 256, 148 * 16)), dim3(256), 0, stream, dact, gu, dgu, total, Fv);
}

void embedding_bwd(const float* dx, const int64_t* ids, float* dtable, int M, int D, cudaStream_t stream) {
  embedding_bwd_kernel<<<M, 256, 0, stream>>>(dx, ids, dtable, M, D);
}

int embedding_scatter(int n_sources, const int64_t* const* ids, const float* const* rows, float* dtable, int M, int D,
                      float scale, float* sq_delta, int blocks, cudaStream_t stream, int64_t* ids_scratch) {
  if (n_sources < 1 || n_sources > 8 || D % 4 != 0 || M <= 0 || M >= (1 << 27) || blocks < 1) return -1;
  EmbedSources src{};
  src.n = n_sources;
  for (int p = 0; p < n_sources; ++p) {
    src.ids[p] = ids[p];
    src.rows[p] = rows[p];
  }
  if (ids_scratch != nullptr) {
    // sources may live on peer GPUs: bring the ids here once, then scan the local copy
    const int total = n_sources * M;
    embedding_gather_ids_kernel<<<std::max(1, std::min(148, (total + 1023) / 1024)), 256, 0, stream>>>(src, ids_scratch, M);
    for (int p = 0; p < n_sources; ++p) src.ids[p] = ids_scratch + static_cast<int64_t>(p) * M;
  }
  embedding_scatter_kernel<<<blocks, EB_THREADS, 0, stream>>>(src, dtable, M, D, scale, sq_delta);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

void ce_softmax_grad(__nv_bfloat16* logits, int64_t ldl, const int64_t* labels, float* row_loss,
                     const float* inv_n_valid, int C, int V, int ignore_index, cudaStream_t stream) {
  ce_softmax_grad_kernel<CE_FUSED><<<C, CE_THREADS, 0, stream>>>(logits, ldl, labels, row_loss, inv_n_valid, V,
                                                                 ignore_index, 0, nullptr, nullptr);
}

void ce_row_stats(const __nv_bfloat16* logits, int64_t ldl, const int64_t* labels, float* stats, int C, int V,
                  int64_t vocab_lo, int ignore_index, cudaStream_t stream) {
  ce_softmax_grad_kernel<CE_STATS><<<C, CE_THREADS, 0, stream>>>(const_cast<__nv_bfloat16*>(logits), ldl, labels, nullptr,
                                                                 nullptr, V, ignore_index, vocab_lo, stats, nullptr);
}

void ce_grad_from_lse(__nv_bfloat16* logits, int64_t ldl, const int64_t* labels, const float* lse,
                      const float* inv_n_valid, int C, int V, int64_t vocab_lo, int ignore_index, cudaStream_t stream) {
  ce_softmax_grad_kernel<CE_GRAD><<<C, CE_THREADS, 0, stream>>>(logits, ldl, labels, nullptr, inv_n_valid, V, ignore_index,
                                                                vocab_lo, nullptr, lse);
}

void cast_f32_to_bf16(const float* src, __nv_bfloat16* dst, int64_t n, cudaStream_t stream) {
  cast_f32_to_bf16_kernel<<<grid_for(n / 4, 256, 148 * 16), 256, 0, stream>>>(src, dst, n);
}

void scale_inplace_f32(float* x, const float* scale, int64_t n, cudaStream_t stream) {
  scale_f32_kernel<<<grid_for(n / 4, 256, 148 * 16), 256, 0, stream>>>(x, scale, n);
}

void scale_inplace_bf16(__nv_bfloat16* x, const float* scale, int64_t n, cudaStream_t stream) {
  scale_bf16_kernel<<<grid_for(n / 8, 256, 148 * 16), 256, 0, stream>>>(x, scale, n);
}

}  // namespace tb
