// Cost of one tcgen05.mma instruction on B200, by shape and operand source: a chain of 1024 instructions (eight k-steps
// per accumulator pass, as in a GEMM main loop) issued by one thread per CTA on all 148 SMs at once, operands resident
// in shared memory (zeros), timed with clock64 from the first issue to the completion of the commit.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -I torchure_b200/csrc \
//        -o /tmp/mma_issue_bench benchmarks/mma_issue_bench.cu && /tmp/mma_issue_bench
//
// mode 0: both operands from shared memory, K-major; mode 1: A from tensor memory; mode 2: both operands MN-major;
// "pair": cta_group::2, M = 256 over the two CTAs of a cluster, each holding 128 rows of A and half of B.
// Every wait is bounded (mbar_wait); nothing here spins on another kernel.
#include "common.cuh"
#include <cstdio>
using namespace tb;

struct Cfg { int n; int mode; int accs; int total; };  // mode 0: SS K-major, 1: TS, 2: SS both MN-major

__global__ void __launch_bounds__(128, 1) bench(Cfg c, long long* out, int* err) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023);
  __shared__ uint64_t bar;
  __shared__ uint32_t slot;
  const int warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < 160 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (threadIdx.x == 0) { mbar_init(&bar, 1); fence_barrier_init(); }
  if (warp == 0) { tmem_alloc(&slot, 512); tmem_relinquish(); tc_fence_before(); }
  fence_proxy_async_smem();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&slot);
  if (warp == 0 && elect_one()) {
    const uint32_t a_addr = smem_u32(smem), b_addr = smem_u32(smem + 32768);
    const uint64_t da = c.mode == 2 ? make_desc_sw128(a_addr, 16384, 1024) : make_desc_sw128(a_addr, 16, 1024);
    const uint64_t db = c.mode == 2 ? make_desc_sw128(b_addr, 16384, 1024) : make_desc_sw128(b_addr, 16, 1024);
    uint32_t idesc;
    if (c.n == 64) idesc = c.mode == 2 ? make_idesc_bf16(128, 64, true, true) : make_idesc_bf16(128, 64, false, false);
    else if (c.n == 128) idesc = c.mode == 2 ? make_idesc_bf16(128, 128, true, true) : make_idesc_bf16(128, 128, false, false);
    else idesc = make_idesc_bf16(128, 256, false, false);
    const long long t0 = clock64();
    for (int i = 0; i < c.total; ++i) {
      const int ks = i & 7;
      const uint32_t d = tmem + ((i >> 3) % c.accs) * c.n % 512;
      const uint64_t o = c.mode == 2 ? ks * (2048 >> 4) : (((ks >> 2) * 16384 + (ks & 3) * 32) >> 4);
      if (c.mode == 1) umma_f16_ts(d, tmem + 448 + ks * 8, db + o, idesc, ks != 0);
      else umma_f16_ss(d, da + o, db + o, idesc, ks != 0);
    }
    const long long t1 = clock64();
    umma_commit(&bar);
    mbar_wait(&bar, 0, err, 1);
    const long long t2 = clock64();
    if (blockIdx.x == 0) { out[0] = t1 - t0; out[1] = t2 - t0; }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

__global__ void __launch_bounds__(128, 1) bench2(int n, int total, long long* out, int* err) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023);
  __shared__ uint64_t bar;
  __shared__ uint32_t slot;
  const int warp = threadIdx.x >> 5;
  const uint32_t rank = cluster_rank();
  for (int i = threadIdx.x; i < 160 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (threadIdx.x == 0) { mbar_init(&bar, 1); fence_barrier_init(); }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    tc_fence_before();
  }
  fence_proxy_async_smem();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&slot);
  if (rank == 0 && warp == 0 && elect_one()) {
    const uint32_t a_addr = smem_u32(smem), b_addr = smem_u32(smem + 32768);
    const uint64_t da = make_desc_sw128(a_addr, 16, 1024);
    const uint64_t db = make_desc_sw128(b_addr, 16, 1024);
    const uint32_t idesc = make_idesc_bf16(256, n, false, false);
    const long long t0 = clock64();
    for (int i = 0; i < total; ++i) {
      const int ks = i & 7;
      const uint32_t d = tmem + ((i >> 3) & 1) * (n % 512 == 0 ? 0 : n);
      const uint64_t o = (((ks >> 2) * 16384 + (ks & 3) * 32) >> 4);
      const uint32_t acc = ks != 0, z = 0;
      asm volatile(
          "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
          "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
          ::"r"(d), "l"(da + o), "l"(db + o), "r"(idesc), "r"(acc), "r"(z)
          : "memory");
    }
    const long long t1 = clock64();
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bar)) : "memory");
    mbar_wait(&bar, 0, err, 1);
    const long long t2 = clock64();
    if (blockIdx.x == 0) { out[0] = t1 - t0; out[1] = t2 - t0; }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
  }
}

static int run_single() {
  long long* out; int* err;
  cudaMalloc(&out, 16); cudaMalloc(&err, 4); cudaMemset(err, 0, 4);
  cudaFuncSetAttribute(bench, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  const Cfg cfgs[] = {{64, 0, 1, 1024}, {64, 0, 2, 1024}, {64, 0, 4, 1024}, {128, 0, 1, 1024}, {128, 0, 2, 1024},
                      {256, 0, 1, 1024}, {256, 0, 2, 1024}, {64, 1, 1, 1024}, {64, 1, 2, 1024}, {128, 1, 1, 1024},
                      {128, 1, 2, 1024}, {64, 2, 1, 1024}, {64, 2, 2, 1024}, {128, 2, 1, 1024}};
  for (const Cfg& c : cfgs) {
    for (int rep = 0; rep < 2; ++rep) bench<<<148, 128, 200 * 1024>>>(c, out, err);
    cudaError_t e = cudaDeviceSynchronize();
    long long h[2]; int herr;
    cudaMemcpy(h, out, 16, cudaMemcpyDeviceToHost); cudaMemcpy(&herr, err, 4, cudaMemcpyDeviceToHost);
    const double ideal = 2.0 * 128 * c.n * 16 / 8192.0;
    printf("N=%3d mode=%d accs=%d: issue %.1f cyc/mma, complete %.1f cyc/mma (ideal %.0f) err=%d cuda=%d\n", c.n, c.mode,
           c.accs, double(h[0]) / c.total, double(h[1]) / c.total, ideal, herr, int(e));
    if (e != cudaSuccess || herr) return 1;
  }
  return 0;
}

static int run_pair() {
  long long* out; int* err;
  cudaMalloc(&out, 16); cudaMalloc(&err, 4); cudaMemset(err, 0, 4);
  cudaFuncSetAttribute(bench2, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  const int ns[] = {256, 128, 64};
  for (int n : ns) {
    for (int rep = 0; rep < 2; ++rep) {
      cudaLaunchConfig_t cfg{};
      cfg.gridDim = dim3(148); cfg.blockDim = dim3(128); cfg.dynamicSmemBytes = 200 * 1024;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr; cfg.numAttrs = 1;
      cudaError_t le = cudaLaunchKernelEx(&cfg, bench2, n, 1024, out, err);
      if (le != cudaSuccess) { printf("launch error %d\n", int(le)); return 1; }
    }
    cudaError_t e = cudaDeviceSynchronize();
    long long h[2]; int herr;
    cudaMemcpy(h, out, 16, cudaMemcpyDeviceToHost); cudaMemcpy(&herr, err, 4, cudaMemcpyDeviceToHost);
    const double ideal = 2.0 * 128 * n * 16 / 8192.0;   // per SM
    printf("2-CTA M=256 N=%3d: issue %.1f cyc/mma, complete %.1f cyc/mma (ideal per SM %.0f) err=%d cuda=%d\n", n,
           double(h[0]) / 1024, double(h[1]) / 1024, ideal, herr, int(e));
    if (e != cudaSuccess || herr) return 1;
  }
  return 0;
}

int main() {
  const int a = run_single();
  if (a) return a;
  return run_pair();
}
