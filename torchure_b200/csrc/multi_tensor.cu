// Multi-tensor kernels: one launch covers every tensor of a parameter set through a device-resident
// table (pointers, sizes, per-block (tensor, chunk) assignment) that is built once and reused, so a
// step costs no host-to-device table traffic and no per-tensor launches.
//
//   adamw_multi        fp32 master / m / v update from fp32 or bf16 grads, optional device-resident
//                      clip coefficient, optional bf16 shadow write
//   sqnorm_multi       sum of squares over all tensors (grad norm)
//   scale_multi        x *= *scale (skipped when the scale is 1)
//   zero_multi         x = 0 for a list of fp32 tensors
//   bucket_pack_multi  DDP bucket fill: bucket (= | +=) fp32(grad), optional post-scale, optional sum
//                      of squares of the result
#include "api.h"

#include <cuda_bf16.h>

namespace tb {

namespace {

constexpr int MT_THREADS = 512;

__device__ __forceinline__ float block_sum(float v) {
  __shared__ float part[MT_THREADS / 32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = threadIdx.x < MT_THREADS / 32 ? part[threadIdx.x] : 0.f;
  if (threadIdx.x < 32) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  }
  return t;  // valid in thread 0
}

__device__ __forceinline__ float load_grad(const void* g, bool is_bf16, int64_t i) {
  return is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(g)[i])
                 : reinterpret_cast<const float*>(g)[i];
}

__global__ void __launch_bounds__(MT_THREADS)
adamw_kernel(TensorList t, float lr, float beta1, float beta2, float eps, float wd, float bias1, float bias2,
             const float* __restrict__ grad_scale, int maximize, const float* __restrict__ hyper) {
  if (hyper) {  // step-dependent scalars read from device memory: the launch can be replayed from a CUDA graph
    lr = hyper[0];
    bias1 = hyper[1];
    bias2 = hyper[2];
  }
  const int ti = t.block_tensor[blockIdx.x];
  const int64_t n = t.numel[ti];
  const int64_t lo = static_cast<int64_t>(t.block_chunk[blockIdx.x]) * kChunkElems;
  const int64_t hi = lo + kChunkElems < n ? lo + kChunkElems : n;
  float* p = reinterpret_cast<float*>(t.ptrs_a[ti]);
  const void* g = reinterpret_cast<const void*>(t.ptrs_b[ti]);
  float* m = reinterpret_cast<float*>(t.ptrs_c[ti]);
  float* v = reinterpret_cast<float*>(t.ptrs_d[ti]);
  __nv_bfloat16* sh = reinterpret_cast<__nv_bfloat16*>(t.ptrs_e[ti]);
  const bool g_bf16 = (t.flags[ti] & 1) != 0;
  float gs = grad_scale ? *grad_scale : 1.f;
  if (maximize) gs = -gs;
  const float step_size = lr / bias1;
  const float inv_sqrt_bias2 = rsqrtf(bias2);
  const float decay = 1.f - lr * wd;
  const bool vec = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(m) |
                     reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(sh)) & 15) == 0 &&
                   ((hi - lo) & 3) == 0 && !g_bf16;
  if (vec) {
    for (int64_t i = lo + threadIdx.x * 4; i < hi; i += MT_THREADS * 4) {
      float4 pv = *reinterpret_cast<float4*>(p + i);
      float4 gv = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(g) + i);
      float4 mv = *reinterpret_cast<float4*>(m + i);
      float4 vv = *reinterpret_cast<float4*>(v + i);
      float* pp = &pv.x; float* gg = &gv.x; float* mm = &mv.x; float* vq = &vv.x;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float gk = gg[k] * gs;
        mm[k] = beta1 * mm[k] + (1.f - beta1) * gk;
        vq[k] = beta2 * vq[k] + (1.f - beta2) * gk * gk;
        const float denom = sqrtf(vq[k]) * inv_sqrt_bias2 + eps;
        pp[k] = pp[k] * decay - step_size * (mm[k] / denom);
      }
      *reinterpret_cast<float4*>(p + i) = pv;
      *reinterpret_cast<float4*>(m + i) = mv;
      *reinterpret_cast<float4*>(v + i) = vv;
      if (sh) {
        __nv_bfloat162 a = __floats2bfloat162_rn(pv.x, pv.y), b = __floats2bfloat162_rn(pv.z, pv.w);
        uint2 o;
        o.x = *reinterpret_cast<uint32_t*>(&a);
        o.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(sh + i) = o;
      }
    }
  } else {
    for (int64_t i = lo + threadIdx.x; i < hi; i += MT_THREADS) {
      const float gk = load_grad(g, g_bf16, i) * gs;
      const float mk = beta1 * m[i] + (1.f - beta1) * gk;
      const float vk = beta2 * v[i] + (1.f - beta2) * gk * gk;
      const float denom = sqrtf(vk) * inv_sqrt_bias2 + eps;
      const float pk = p[i] * decay - step_size * (mk / denom);
      m[i] = mk; v[i] = vk; p[i] = pk;
      if (sh) sh[i] = __float2bfloat16(pk);
    }
  }
}

__global__ void __launch_bounds__(MT_THREADS)
sqnorm_kernel(TensorList t, float* __restrict__ out) {
  const int ti = t.block_tensor[blockIdx.x];
  const int64_t n = t.numel[ti];
  const int64_t lo = static_cast<int64_t>(t.block_chunk[blockIdx.x]) * kChunkElems;
  const int64_t hi = lo + kChunkElems < n ? lo + kChunkElems : n;
  const void* x = reinterpret_cast<const void*>(t.ptrs_a[ti]);
  const bool is_bf16 = (t.flags[ti] & 1) != 0;
  float acc = 0.f;
  for (int64_t i = lo + threadIdx.x; i < hi; i += MT_THREADS) {
    const float v = load_grad(x, is_bf16, i);
    acc += v * v;
  }
  acc = block_sum(acc);
  if (threadIdx.x == 0) atomicAdd(out, acc);
}

__global__ void __launch_bounds__(MT_THREADS)
scale_kernel(TensorList t, const float* __restrict__ scale) {
  const float s = *scale;
  if (s == 1.f) return;
  const int ti = t.block_tensor[blockIdx.x];
  const int64_t n = t.numel[ti];
  const int64_t lo = static_cast<int64_t>(t.block_chunk[blockIdx.x]) * kChunkElems;
  const int64_t hi = lo + kChunkElems < n ? lo + kChunkElems : n;
  if (t.flags[ti] & 1) {
    __nv_bfloat16* x = reinterpret_cast<__nv_bfloat16*>(t.ptrs_a[ti]);
    for (int64_t i = lo + threadIdx.x; i < hi; i += MT_THREADS) x[i] = __float2bfloat16(__bfloat162float(x[i]) * s);
  } else {
    float* x = reinterpret_cast<float*>(t.ptrs_a[ti]);
    for (int64_t i = lo + threadIdx.x; i < hi; i += MT_THREADS) x[i] *= s;
  }
}

// fp32 tensors := 0 (the many small gain-gradient slices of a step, in one launch)
__global__ void __launch_bounds__(MT_THREADS)
zero_kernel(TensorList t) {
  const int ti = t.block_tensor[blockIdx.x];
  const int64_t n = t.numel[ti];
  const int64_t lo = static_cast<int64_t>(t.block_chunk[blockIdx.x]) * kChunkElems;
  const int64_t hi = lo + kChunkElems < n ? lo + kChunkElems : n;
  float* x = reinterpret_cast<float*>(t.ptrs_a[ti]);
  for (int64_t i = lo + threadIdx.x; i < hi; i += MT_THREADS) x[i] = 0.f;
}

// ptrs_a: source grad (bf16 or fp32), ptrs_b: destination slice inside the fp32 bucket
__global__ void __launch_bounds__(MT_THREADS)
bucket_pack_kernel(TensorList t, int accumulate, float post_scale, float* __restrict__ sq) {
  const int ti = t.block_tensor[blockIdx.x];
  const int64_t n = t.numel[ti];
  const int64_t lo = static_cast<int64_t>(t.block_chunk[blockIdx.x]) * kChunkElems;
  const int64_t hi = lo + kChunkElems < n ? lo + kChunkElems : n;
  const void* g = reinterpret_cast<const void*>(t.ptrs_a[ti]);
  float* dst = reinterpret_cast<float*>(t.ptrs_b[ti]);
  const bool is_bf16 = (t.flags[ti] & 1) != 0;
  float acc = 0.f;
  for (int64_t i = lo + threadIdx.x; i < hi; i += MT_THREADS) {
    float v = load_grad(g, is_bf16, i);
    if (accumulate) v += dst[i];
    v *= post_scale;
    dst[i] = v;
    acc += v * v;
  }
  if (sq) {
    acc = block_sum(acc);
    if (threadIdx.x == 0) atomicAdd(sq, acc);
  }
}

}  // namespace

void adamw_multi(const TensorList& t, float lr, float beta1, float beta2, float eps, float weight_decay, float bias1,
                 float bias2, const float* grad_scale, int maximize, const float* hyper, cudaStream_t stream) {
  if (t.n_blocks <= 0) return;
  adamw_kernel<<<t.n_blocks, MT_THREADS, 0, stream>>>(t, lr, beta1, beta2, eps, weight_decay, bias1, bias2,
                                                      grad_scale, maximize, hyper);
}

// Gradient-norm finalisation in one launch: out[0] = sqrt(sum of `n` partial sums of squares), out[1] = the clip
// coefficient min(1, max_norm / (norm + eps)) (1 when max_norm <= 0).  The sum runs in a fixed order (strided per
// thread, then a shared-memory tree), so ranks holding the same partials derive the same bits.
__global__ void __launch_bounds__(256)
finalize_norm_kernel(const float* __restrict__ partials, int n, float max_norm, float eps, float* __restrict__ out) {
  __shared__ float s[256];
  float a = 0.f;
  for (int i = threadIdx.x; i < n; i += 256) a += partials[i];
  s[threadIdx.x] = a;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) s[threadIdx.x] += s[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const float norm = sqrtf(s[0]);
    out[0] = norm;
    out[1] = max_norm > 0.f ? fminf(1.f, max_norm / (norm + eps)) : 1.f;
  }
}

void finalize_norm(const float* partials, int n, float max_norm, float eps, float* out, cudaStream_t stream) {
  finalize_norm_kernel<<<1, 256, 0, stream>>>(partials, n, max_norm, eps, out);
}

void sqnorm_multi(const TensorList& t, float* out, cudaStream_t stream) {
  if (t.n_blocks <= 0) return;
  sqnorm_kernel<<<t.n_blocks, MT_THREADS, 0, stream>>>(t, out);
}

void scale_multi(const TensorList& t, const float* scale, cudaStream_t stream) {
  if (t.n_blocks <= 0) return;
  scale_kernel<<<t.n_blocks, MT_THREADS, 0, stream>>>(t, scale);
}

void zero_multi(const TensorList& t, cudaStream_t stream) {
  if (t.n_blocks <= 0) return;
  zero_kernel<<<t.n_blocks, MT_THREADS, 0, stream>>>(t);
}

void bucket_pack_multi(const TensorList& t, int accumulate, float post_scale, float* sq, cudaStream_t stream) {
  if (t.n_blocks <= 0) return;
  bucket_pack_kernel<<<t.n_blocks, MT_THREADS, 0, stream>>>(t, accumulate, post_scale, sq);
}

}  // namespace tb
