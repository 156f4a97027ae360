// NVLink / NVSwitch collectives written as plain kernels over a symmetric allocation.
//
// Transport per kernel: either `multimem` instructions on the multicast mapping (the switch reduces or
// replicates: NVLS) or plain 16-byte loads/stores on peer pointers.  No TMA and no library call is involved,
// so nothing here ever issues a multicast TMA load from peer memory.
//
// Cross-rank synchronisation is a per-block flag exchange: block b of every rank handshakes with block b of
// every peer (same grid everywhere).  A flag is raised with CAS 0->1 in the peer's memory and consumed with CAS
// 1->0 locally, so flags reset themselves.  Every spin is bounded by CommCtx::wait_limit_ns; on expiry the block
// records kErrPeerFlagWait and the kernel finishes without touching peer memory again.
#include "comm_api.h"
#include "comm_device.cuh"
#include "common.cuh"

namespace tb {

namespace {

constexpr int CT = 512;  // threads per block

// ---- 16-byte vector helpers ---------------------------------------------------------------------------
struct V4 { uint32_t x, y, z, w; };

__device__ __forceinline__ V4 ld16(const void* p) {
  V4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st16(void* p, const V4& v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ V4 mc_ld_reduce_f32(const void* p) {
  V4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ V4 mc_ld_reduce_bf16(const void* p) {
  V4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void mc_st(void* p, const V4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__device__ __forceinline__ float combine(float a, float b, int op) {
  return op == kOpMax ? fmaxf(a, b) : (op == kOpMin ? fminf(a, b) : a + b);
}

// 4 fp32 accumulators per 16 B of fp32; 8 per 16 B of bf16
template <int DT>
struct Acc {
  static constexpr int N = DT == kF32 ? 4 : 8;
  float f[N];
  __device__ __forceinline__ void load(const V4& v) {
    if (DT == kF32) {
      f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
    } else {
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        f[2 * k] = __uint_as_float(u[k] << 16);
        f[2 * k + 1] = __uint_as_float(u[k] & 0xffff0000u);
      }
    }
  }
  __device__ __forceinline__ V4 store() const {
    V4 v;
    if (DT == kF32) {
      v.x = __float_as_uint(f[0]); v.y = __float_as_uint(f[1]); v.z = __float_as_uint(f[2]); v.w = __float_as_uint(f[3]);
    } else {
      v.x = pack_bf16x2(f[0], f[1]); v.y = pack_bf16x2(f[2], f[3]); v.z = pack_bf16x2(f[4], f[5]); v.w = pack_bf16x2(f[6], f[7]);
    }
    return v;
  }
};

// reduce one 16-byte vector at byte offset `o` over all ranks
template <int DT>
__device__ __forceinline__ Acc<DT> reduce_vec(const CommCtx& c, uint64_t o, int op, bool use_mc) {
  Acc<DT> a;
  if (use_mc) {
    a.load(DT == kF32 ? mc_ld_reduce_f32(reinterpret_cast<void*>(c.mc_buf + o))
                      : mc_ld_reduce_bf16(reinterpret_cast<void*>(c.mc_buf + o)));
  } else {
    a.load(ld16(reinterpret_cast<void*>(c.peer_bufs[0] + o)));
    for (int p = 1; p < c.world; ++p) {
      Acc<DT> b;
      b.load(ld16(reinterpret_cast<void*>(c.peer_bufs[p] + o)));
#pragma unroll
      for (int k = 0; k < Acc<DT>::N; ++k) a.f[k] = combine(a.f[k], b.f[k], op);
    }
  }
  if (op == kOpAvg) {
    const float s = 1.f / c.world;
#pragma unroll
    for (int k = 0; k < Acc<DT>::N; ++k) a.f[k] *= s;
  }
  return a;
}

__device__ __forceinline__ void write_all(const CommCtx& c, uint64_t o, const V4& v, bool use_mc) {
  if (use_mc) {
    mc_st(reinterpret_cast<void*>(c.mc_buf + o), v);
  } else {
    for (int p = 0; p < c.world; ++p) st16(reinterpret_cast<void*>(c.peer_bufs[(c.rank + p) % c.world] + o), v);
  }
}

__device__ __forceinline__ float block_reduce_sum(float v) {
  __shared__ float part[CT / 32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = threadIdx.x < CT / 32 ? part[threadIdx.x] : 0.f;
  if (threadIdx.x < 32) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  }
  return t;
}

// ---- kernels ------------------------------------------------------------------------------------------
constexpr int UNROLL = 4;  // independent 16-byte transactions in flight per thread

// reduce UNROLL vectors starting at i (stride `step`), bounds-checked against hi
template <int DT>
__device__ __forceinline__ void reduce_batch(const CommCtx& c, uint64_t off, int64_t i, int64_t step, int64_t hi, int op,
                                             bool use_mc, Acc<DT> (&acc)[UNROLL]) {
  if (use_mc) {
    V4 raw[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int64_t k = i + u * step;
      if (k < hi) raw[u] = DT == kF32 ? mc_ld_reduce_f32(reinterpret_cast<void*>(c.mc_buf + off + k * 16))
                                      : mc_ld_reduce_bf16(reinterpret_cast<void*>(c.mc_buf + off + k * 16));
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) acc[u].load(raw[u]);
  } else {
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int64_t k = i + u * step;
      if (k < hi) {
        V4 raw[kCommMaxRanks];
        for (int p = 0; p < c.world; ++p) raw[p] = ld16(reinterpret_cast<void*>(c.peer_bufs[p] + off + k * 16));
        acc[u].load(raw[0]);
        for (int p = 1; p < c.world; ++p) {
          Acc<DT> b;
          b.load(raw[p]);
#pragma unroll
          for (int e = 0; e < Acc<DT>::N; ++e) acc[u].f[e] = combine(acc[u].f[e], b.f[e], op);
        }
      }
    }
  }
  if (op == kOpAvg) {
    const float sc = 1.f / c.world;
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
#pragma unroll
      for (int e = 0; e < Acc<DT>::N; ++e) acc[u].f[e] *= sc;
  }
}

// In-place two-shot all-reduce of data that already lives in the symmetric allocation (DDP buckets).
template <int DT>
__global__ void __launch_bounds__(CT)
all_reduce_kernel(CommCtx c, uint64_t off, int64_t nvec, int op, int use_mc, int sq_slot) {
  if (!block_barrier(c, 0, c.world)) return;
  const int64_t per = nvec / c.world, rem = nvec % c.world;
  // slice of this rank (the remainder goes to the last rank)
  const int64_t lo = per * c.rank, hi = lo + per + (c.rank == c.world - 1 ? rem : 0);
  const int64_t step = static_cast<int64_t>(gridDim.x) * CT;
  float sq = 0.f;
  for (int64_t i = lo + static_cast<int64_t>(blockIdx.x) * CT + threadIdx.x; i < hi; i += step * UNROLL) {
    Acc<DT> acc[UNROLL];
    reduce_batch<DT>(c, off, i, step, hi, op, use_mc != 0, acc);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int64_t k = i + u * step;
      if (k < hi) {
#pragma unroll
        for (int e = 0; e < Acc<DT>::N; ++e) sq += acc[u].f[e] * acc[u].f[e];
        write_all(c, off + k * 16, acc[u].store(), use_mc != 0);
      }
    }
  }
  if (sq_slot >= 0) {
    sq = block_reduce_sum(sq);
    if (threadIdx.x < c.world) {
      // publish this block's partial to every rank: table[slot][rank][block]
      float* table = reinterpret_cast<float*>(c.peer_bufs[threadIdx.x] + kFlagBytes);
      table[(static_cast<int64_t>(sq_slot) * kCommMaxRanks + c.rank) * kCommMaxBlocks + blockIdx.x] = sq;
    }
  }
  block_barrier(c, 1, c.world);
}

// All-reduce of an ordinary local tensor, one launch: copy into my staging area, handshake, reduce, write `out`.
//   oneshot: every rank reduces the whole message from all staging areas (latency bound sizes)
//   two-shot: every rank reduces its slice, broadcasts it into all staging areas, handshake, copy out
// Element i is always handled by block (i / CT) % gridDim on every rank (slices are multiples of gridDim * CT), which is
// what makes the per-block handshake sufficient.
template <int DT>
__global__ void __launch_bounds__(CT)
all_reduce_fused_kernel(CommCtx c, uint64_t off, const void* in, void* out, int64_t nvec, int op, int use_mc, int oneshot) {
  const int64_t step = static_cast<int64_t>(gridDim.x) * CT;
  const int64_t first = static_cast<int64_t>(blockIdx.x) * CT + threadIdx.x;
  uint8_t* mine = reinterpret_cast<uint8_t*>(c.peer_bufs[c.rank] + off);
  for (int64_t i = first; i < nvec; i += step) st16(mine + i * 16, ld16(reinterpret_cast<const uint8_t*>(in) + i * 16));
  if (!block_barrier(c, 0, c.world)) return;
  if (oneshot) {
    for (int64_t i = first; i < nvec; i += step * UNROLL) {
      Acc<DT> acc[UNROLL];
      reduce_batch<DT>(c, off, i, step, nvec, op, false, acc);
#pragma unroll
      for (int u = 0; u < UNROLL; ++u)
        if (i + u * step < nvec) st16(reinterpret_cast<uint8_t*>(out) + (i + u * step) * 16, acc[u].store());
    }
    block_barrier(c, 1, c.world);  // my staging area may be rewritten only after every peer has read it
    return;
  }
  const int64_t per = ((nvec + c.world - 1) / c.world + step - 1) / step * step;
  const int64_t lo = per * c.rank;
  const int64_t hi = lo + per < nvec ? lo + per : nvec;
  for (int64_t i = lo + first; i < hi; i += step * UNROLL) {
    Acc<DT> acc[UNROLL];
    reduce_batch<DT>(c, off, i, step, hi, op, use_mc != 0, acc);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
      if (i + u * step < hi) write_all(c, off + (i + u * step) * 16, acc[u].store(), use_mc != 0);
  }
  if (!block_barrier(c, 1, c.world)) return;
  for (int64_t i = first; i < nvec; i += step) st16(reinterpret_cast<uint8_t*>(out) + i * 16, ld16(mine + i * 16));
}

// all_gather of local `in` (nvec vectors) into local `out` (world * nvec): my chunk goes straight from `in` into every
// rank's staging area, handshake, copy out.
__global__ void __launch_bounds__(CT)
all_gather_kernel(CommCtx c, uint64_t dst_off, const void* in, void* out, int64_t nvec, int use_mc) {
  const int64_t step = static_cast<int64_t>(gridDim.x) * CT;
  const int64_t first = static_cast<int64_t>(blockIdx.x) * CT + threadIdx.x;
  if (!block_barrier(c, 0, c.world)) return;  // every rank's staging area is free (its previous copy-out is done)
  const uint64_t my_dst = dst_off + static_cast<uint64_t>(c.rank) * nvec * 16;
  for (int64_t i = first; i < nvec; i += step)
    write_all(c, my_dst + i * 16, ld16(reinterpret_cast<const uint8_t*>(in) + i * 16), use_mc != 0);
  if (!block_barrier(c, 1, c.world)) return;
  const uint8_t* mine = reinterpret_cast<const uint8_t*>(c.peer_bufs[c.rank] + dst_off);
  // chunk r element i was written by block (i / CT) % gridDim of rank r: keep that mapping per chunk
  for (int r = 0; r < c.world; ++r)
    for (int64_t i = first; i < nvec; i += step)
      st16(reinterpret_cast<uint8_t*>(out) + (r * nvec + i) * 16, ld16(mine + (r * nvec + i) * 16));
}

// reduce_scatter of local `in` (world * nvec) into local `out` (nvec)
template <int DT>
__global__ void __launch_bounds__(CT)
reduce_scatter_kernel(CommCtx c, uint64_t off, const void* in, void* out, int64_t nvec, int op, int use_mc) {
  const int64_t step = static_cast<int64_t>(gridDim.x) * CT;
  const int64_t first = static_cast<int64_t>(blockIdx.x) * CT + threadIdx.x;
  uint8_t* mine = reinterpret_cast<uint8_t*>(c.peer_bufs[c.rank] + off);
  for (int r = 0; r < c.world; ++r)
    for (int64_t i = first; i < nvec; i += step)
      st16(mine + (r * nvec + i) * 16, ld16(reinterpret_cast<const uint8_t*>(in) + (r * nvec + i) * 16));
  if (!block_barrier(c, 0, c.world)) return;
  const uint64_t base = off + static_cast<uint64_t>(c.rank) * nvec * 16;
  for (int64_t i = first; i < nvec; i += step * UNROLL) {
    Acc<DT> acc[UNROLL];
    reduce_batch<DT>(c, base, i, step, nvec, op, use_mc != 0, acc);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
      if (i + u * step < nvec) st16(reinterpret_cast<uint8_t*>(out) + (i + u * step) * 16, acc[u].store());
  }
  block_barrier(c, 1, c.world);
}

// all_to_all: chunk j of local `in` goes into rank j's staging slot [my rank], handshake, copy out
__global__ void __launch_bounds__(CT)
all_to_all_kernel(CommCtx c, uint64_t dst_off, const void* in, void* out, int64_t nvec) {
  const int64_t step = static_cast<int64_t>(gridDim.x) * CT;
  const int64_t first = static_cast<int64_t>(blockIdx.x) * CT + threadIdx.x;
  if (!block_barrier(c, 0, c.world)) return;
  for (int j = 0; j < c.world; ++j) {
    const int peer = (c.rank + j) % c.world;  // stagger peers so links are used evenly
    const uint8_t* src = reinterpret_cast<const uint8_t*>(in) + static_cast<uint64_t>(peer) * nvec * 16;
    uint8_t* dst = reinterpret_cast<uint8_t*>(c.peer_bufs[peer] + dst_off + static_cast<uint64_t>(c.rank) * nvec * 16);
    for (int64_t i = first; i < nvec; i += step) st16(dst + i * 16, ld16(src + i * 16));
  }
  if (!block_barrier(c, 1, c.world)) return;
  const uint8_t* mine = reinterpret_cast<const uint8_t*>(c.peer_bufs[c.rank] + dst_off);
  for (int r = 0; r < c.world; ++r)
    for (int64_t i = first; i < nvec; i += step)
      st16(reinterpret_cast<uint8_t*>(out) + (r * nvec + i) * 16, ld16(mine + (r * nvec + i) * 16));
}

// broadcast of local `buf` (in place): the source writes every staging area, handshake, the others copy out
__global__ void __launch_bounds__(CT)
broadcast_kernel(CommCtx c, uint64_t off, void* buf, int64_t nvec, int src, int use_mc) {
  const int64_t step = static_cast<int64_t>(gridDim.x) * CT;
  const int64_t first = static_cast<int64_t>(blockIdx.x) * CT + threadIdx.x;
  if (!block_barrier(c, 0, c.world)) return;
  if (c.rank == src) {
    for (int64_t i = first; i < nvec; i += step) {
      V4 v = ld16(reinterpret_cast<const uint8_t*>(buf) + i * 16);
      if (use_mc) mc_st(reinterpret_cast<void*>(c.mc_buf + off + i * 16), v);
      else
        for (int p = 0; p < c.world; ++p)
          if (p != src) st16(reinterpret_cast<void*>(c.peer_bufs[p] + off + i * 16), v);
    }
  }
  if (!block_barrier(c, 1, c.world)) return;
  if (c.rank != src) {
    const uint8_t* mine = reinterpret_cast<const uint8_t*>(c.peer_bufs[c.rank] + off);
    for (int64_t i = first; i < nvec; i += step) st16(reinterpret_cast<uint8_t*>(buf) + i * 16, ld16(mine + i * 16));
  }
}

// ---- sharded-training collectives on tensors that LIVE in the symmetric allocation (no staging copies) ----------
// A segment is a matrix of `world` equal row chunks at byte offset off of every rank's allocation (nvec 16-byte
// vectors per chunk); chunk r is the shard that rank r owns.

// In-place all-gather: every rank pushes its own chunk of every segment into every peer's copy (one multimem.st
// through the switch above two ranks, posted peer stores at two).  The first handshake says "my consumers of the old
// contents are done", the second "every chunk has landed".
__global__ void __launch_bounds__(CT)
all_gather_inplace_kernel(CommCtx c, CommSegments segs, int use_mc) {
  if (!block_barrier(c, 0, c.world)) return;
  const int64_t step = static_cast<int64_t>(gridDim.x) * CT;
  const int64_t first = static_cast<int64_t>(blockIdx.x) * CT + threadIdx.x;
  for (int sgm = 0; sgm < segs.n; ++sgm) {
    const int64_t nvec = segs.nvec[sgm];
    const uint64_t base = segs.off[sgm] + static_cast<uint64_t>(c.rank) * nvec * 16;
    const uint8_t* mine = reinterpret_cast<const uint8_t*>(c.peer_bufs[c.rank] + base);
    for (int64_t i = first; i < nvec; i += step * UNROLL) {
      V4 v[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u)
        if (i + u * step < nvec) v[u] = ld16(mine + (i + u * step) * 16);
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int64_t k = i + u * step;
        if (k >= nvec) continue;
        if (use_mc) {
          mc_st(reinterpret_cast<void*>(c.mc_buf + base + k * 16), v[u]);
        } else {
          for (int p = 1; p < c.world; ++p)
            st16(reinterpret_cast<void*>(c.peer_bufs[(c.rank + p) % c.world] + base + k * 16), v[u]);
        }
      }
    }
  }
  block_barrier(c, 1, c.world);
}

// Reduce-scatter out of symmetric memory: out[s] (local fp32) = op over ranks of chunk `rank` of segment s.  The sum
// of squares of everything this rank wrote is published to every rank's partial table like all_reduce_kernel does.
// The first handshake says "my contribution is complete", the second "I no longer read your buffer".
__global__ void __launch_bounds__(CT)
reduce_scatter_symm_kernel(CommCtx c, CommSegments segs, int op, int use_mc, int sq_slot) {
  if (!block_barrier(c, 0, c.world)) return;
  const int64_t step = static_cast<int64_t>(gridDim.x) * CT;
  const int64_t first = static_cast<int64_t>(blockIdx.x) * CT + threadIdx.x;
  float sq = 0.f;
  for (int sgm = 0; sgm < segs.n; ++sgm) {
    const int64_t nvec = segs.nvec[sgm];
    const uint64_t base = segs.off[sgm] + static_cast<uint64_t>(c.rank) * nvec * 16;
    uint8_t* out = reinterpret_cast<uint8_t*>(segs.out[sgm]);
    for (int64_t i = first; i < nvec; i += step * UNROLL) {
      Acc<kF32> acc[UNROLL];
      reduce_batch<kF32>(c, base, i, step, nvec, op, use_mc != 0, acc);
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int64_t k = i + u * step;
        if (k < nvec) {
#pragma unroll
          for (int e = 0; e < 4; ++e) sq += acc[u].f[e] * acc[u].f[e];
          st16(out + k * 16, acc[u].store());
        }
      }
    }
  }
  if (sq_slot >= 0) {
    sq = block_reduce_sum(sq);
    if (threadIdx.x < c.world) {
      float* table = reinterpret_cast<float*>(c.peer_bufs[threadIdx.x] + kFlagBytes);
      table[(static_cast<int64_t>(sq_slot) * kCommMaxRanks + c.rank) * kCommMaxBlocks + blockIdx.x] = sq;
    }
  }
  block_barrier(c, 1, c.world);
}

__global__ void __launch_bounds__(CT) barrier_kernel(CommCtx c, int pretend_world, int phase) {
  block_barrier(c, phase, pretend_world);
}

}  // namespace

#define TB_DT_DISPATCH(dtype, CALL_F32, CALL_BF16) \
  do { if ((dtype) == kF32) { CALL_F32; } else { CALL_BF16; } } while (0)

static int64_t vecs(int64_t n, int dtype) { return n * (dtype == kF32 ? 4 : 2) / 16; }

void comm_all_reduce(const CommCtx& c, uint64_t off, int64_t n, int dtype, int op, bool use_mc, int sq_slot,
                     uint32_t, int blocks, cudaStream_t stream) {
  const int64_t nvec = vecs(n, dtype);
  TB_DT_DISPATCH(dtype, (all_reduce_kernel<kF32><<<blocks, CT, 0, stream>>>(c, off, nvec, op, use_mc, sq_slot)),
                 (all_reduce_kernel<kBF16><<<blocks, CT, 0, stream>>>(c, off, nvec, op, use_mc, sq_slot)));
}

void comm_all_reduce_fused(const CommCtx& c, uint64_t off, const void* in, void* out, int64_t n, int dtype, int op,
                           bool use_mc, bool oneshot, int blocks, cudaStream_t stream) {
  const int64_t nvec = vecs(n, dtype);
  TB_DT_DISPATCH(dtype,
                 (all_reduce_fused_kernel<kF32><<<blocks, CT, 0, stream>>>(c, off, in, out, nvec, op, use_mc, oneshot)),
                 (all_reduce_fused_kernel<kBF16><<<blocks, CT, 0, stream>>>(c, off, in, out, nvec, op, use_mc, oneshot)));
}

void comm_all_gather(const CommCtx& c, uint64_t dst_off, const void* in, void* out, int64_t n, int dtype, bool use_mc,
                     int blocks, cudaStream_t stream) {
  all_gather_kernel<<<blocks, CT, 0, stream>>>(c, dst_off, in, out, vecs(n, dtype), use_mc);
}

void comm_reduce_scatter(const CommCtx& c, uint64_t off, const void* in, void* out, int64_t n, int dtype, int op,
                         bool use_mc, int blocks, cudaStream_t stream) {
  const int64_t nvec = vecs(n, dtype);
  TB_DT_DISPATCH(dtype, (reduce_scatter_kernel<kF32><<<blocks, CT, 0, stream>>>(c, off, in, out, nvec, op, use_mc)),
                 (reduce_scatter_kernel<kBF16><<<blocks, CT, 0, stream>>>(c, off, in, out, nvec, op, use_mc)));
}

void comm_all_to_all(const CommCtx& c, uint64_t dst_off, const void* in, void* out, int64_t n, int dtype, int blocks,
                     cudaStream_t stream) {
  all_to_all_kernel<<<blocks, CT, 0, stream>>>(c, dst_off, in, out, vecs(n, dtype));
}

void comm_broadcast(const CommCtx& c, uint64_t off, void* buf, int64_t n, int dtype, int src, bool use_mc, int blocks,
                    cudaStream_t stream) {
  broadcast_kernel<<<blocks, CT, 0, stream>>>(c, off, buf, vecs(n, dtype), src, use_mc);
}

void comm_all_gather_inplace(const CommCtx& c, const CommSegments& segs, bool use_mc, int blocks, cudaStream_t stream) {
  all_gather_inplace_kernel<<<blocks, CT, 0, stream>>>(c, segs, use_mc);
}

void comm_reduce_scatter_symm(const CommCtx& c, const CommSegments& segs, int op, bool use_mc, int sq_slot, int blocks,
                              cudaStream_t stream) {
  reduce_scatter_symm_kernel<<<blocks, CT, 0, stream>>>(c, segs, op, use_mc, sq_slot);
}

void comm_barrier(const CommCtx& c, int phase, int pretend_world, cudaStream_t stream) {
  barrier_kernel<<<1, CT, 0, stream>>>(c, pretend_world, phase);
}

}  // namespace tb
