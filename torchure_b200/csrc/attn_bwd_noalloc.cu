// Allocation-free variant of the attention backward (see no_alloc_api.h for who needs it and why).
#include "no_alloc_api.h"

#include <mutex>

#include "attn_api.h"

namespace {

// Row statistics of one call: delta[rows] followed by lse2[rows].  File scope, lives in the library image on every
// device that loads it.  In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) float g_rows_scratch[2 * TB_ATTN_BWD_NOALLOC_MAX_ROWS];

// Never launched: naming the array in device code keeps the compiler from discarding an otherwise unreferenced symbol.
__global__ void tb_noalloc_scratch_anchor(float* out) { out[0] = g_rows_scratch[0]; }

constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {};
std::mutex g_setup_mutex;

// Resolve the scratch array's device address once per device (with that device current).
float* scratch_for_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_rows_scratch) != cudaSuccess) return nullptr;
    g_scratch_ptr[dev] = p;
  }
  return g_scratch_ptr[dev];
}

}  // namespace

extern "C" int tb_attn_bwd_noalloc(const void* d_o, const void* qk, const void* qkv, const void* o, const float* lse,
                                   void* dqkv, int B, int S, int Hq, int Hkv, int* status, cudaStream_t stream) {
  if (!d_o || !qk || !qkv || !o || !lse || !dqkv || !status) return -1;
  // the same shapes the forward pass accepts: whole 128-token blocks and an even number of query heads per KV head
  if (B <= 0 || S <= 0 || Hq <= 0 || Hkv <= 0 || S % 128 != 0 || Hq % Hkv != 0 || (Hq / Hkv) % 2 != 0) return -2;
  const long long rows = static_cast<long long>(B) * Hq * S;
  if (rows > TB_ATTN_BWD_NOALLOC_MAX_ROWS) return -30;  // larger problems need the allocating entry point
  float* scratch = scratch_for_current_device();
  if (scratch == nullptr) return -31;
  float* delta = scratch;
  float* lse2 = scratch + TB_ATTN_BWD_NOALLOC_MAX_ROWS;
  int rc = tb::attn_bwd_prep(d_o, o, lse, delta, lse2, B, S, Hq, stream);
  if (rc != 0) return rc;
  rc = tb::attn_bwd_dq(qk, qkv, d_o, dqkv, delta, lse2, B, S, Hq, Hkv, status, stream);
  if (rc != 0) return rc;
  return tb::attn_bwd_dkv(qk, qkv, d_o, dqkv, delta, lse2, B, S, Hq, Hkv, status, stream);
}
