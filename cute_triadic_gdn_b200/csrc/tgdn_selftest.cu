// Self-test kernels for the tcgen05 / TMA building blocks: one 128 x N x K product with operands staged in any of the
// shared-memory layouts the production kernels use, and a tensor-map tile load whose shared-memory image is returned
// verbatim.  They exist so that a descriptor or layout mistake shows up in a ten-line test instead of inside a recurrence.
#include "tgdn_common.cuh"
#include "tgdn_host.h"

namespace tgdn {

// layout codes: 0 SW128 K-major, 1 SW128 MN-major, 2 plain K-major, 3 plain MN-major
__device__ __forceinline__ uint32_t st_operand_off(int layout, int mn, int k, int MN, int K) {
  switch (layout) {
    case 0: return (k >> 6) * (MN * 128) + sw128_off(mn, k & 63);
    case 1: return (mn >> 6) * (K * 128) + sw128_off(k, mn & 63);
    case 2: return img_off(mn, k, 128, MN * 16);
    default: return img_off(k, mn, 128, K * 16);
  }
}
__device__ __forceinline__ uint64_t st_operand_desc(int layout, uint32_t base, int MN, int K) {
  switch (layout) {
    case 0: return make_desc(base, 16, 1024, LAYOUT_SW128);
    case 1: return make_desc(base, K * 128, 1024, LAYOUT_SW128);
    case 2: return make_desc(base, MN * 16, 128, LAYOUT_PLAIN);
    default: return make_desc(base, 128, K * 16, LAYOUT_PLAIN);
  }
}
__device__ __forceinline__ uint32_t st_operand_kstep(int layout, int kk, int MN, int K) {
  switch (layout) {
    case 0: return (kk >> 2) * (MN * 128) + (kk & 3) * 32;
    case 1: return kk * 2048;
    case 2: return kk * 2 * (MN * 16);
    default: return kk * 256;
  }
}

__global__ void __launch_bounds__(128) selftest_mma_kernel(const __nv_bfloat16* __restrict__ A,   // [M][K]
                                                           const __nv_bfloat16* __restrict__ B,   // [K][N]
                                                           float* __restrict__ D,                 // [128][N]
                                                           int M, int N, int K, int la, int lb, int* status) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int MA = 128;                       // operand A always holds 128 rows; rows >= M are zero
  uint8_t* sA = smem;
  uint8_t* sB = smem + ((MA * K * 2 + 1023) & ~1023);
  if (tid == 0) { mbar_init(&bar, 1); mbar_fence_init(); abort_s = 0; }
  if (warp == 0) { tmem_alloc(&tmem_base_s, 256); tmem_relinquish(); }
  for (int idx = tid; idx < MA * K; idx += 128) {
    int m = idx / K, k = idx % K;
    __nv_bfloat16 val = (m < M) ? A[m * K + k] : __float2bfloat16(0.f);
    *reinterpret_cast<__nv_bfloat16*>(sA + st_operand_off(la, m, k, MA, K)) = val;
  }
  for (int idx = tid; idx < K * N; idx += 128) {
    int k = idx / N, n = idx % N;
    *reinterpret_cast<__nv_bfloat16*>(sB + st_operand_off(lb, n, k, N, K)) = B[k * N + n];
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  WaitCtl ctl{&abort_s, status};
  if (tid == 0) {
    // M = 64 probe: first the full 128-row product (rows >= M of A are zero), then the 64-row product accumulated on
    // top of it, so that the lanes the 64-row form writes show up as "twice the row" in the returned matrix.
    const uint32_t id128 = make_idesc(128, N, la & 1, lb & 1);
    const uint32_t idesc = make_idesc(M, N, la & 1, lb & 1);
    const uint64_t da = st_operand_desc(la, smem_u32(sA), MA, K), db = st_operand_desc(lb, smem_u32(sB), N, K);
    if (M != 128) {
      for (int kk = 0; kk < K / 16; ++kk)
        umma_bf16(tmem, desc_advance(da, st_operand_kstep(la, kk, MA, K)),
                  desc_advance(db, st_operand_kstep(lb, kk, N, K)), id128, kk > 0);
    }
    for (int kk = 0; kk < K / 16; ++kk)
      umma_bf16(tmem, desc_advance(da, st_operand_kstep(la, kk, MA, K)),
                desc_advance(db, st_operand_kstep(lb, kk, N, K)), idesc, (M != 128 || kk > 0) ? 1u : 0u);
    umma_commit(&bar);
  }
  mbar_wait_spin(&bar, 0, ctl, DEV_TIMEOUT_MMA);
  tc_fence_after();
  const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
  for (int c0 = 0; c0 < N; c0 += 8) {
    float v[8];
    tmem_ld8(tmem + lane_base + c0, v);
    tmem_wait_ld();
    for (int j = 0; j < 8; ++j) D[tid * N + c0 + j] = v[j];
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

// Loads one [64 tokens][64 columns] SW128 box of a (B,T,H,128) bf16 tensor and returns the 8 KB shared-memory image,
// then a 1-D bulk copy of `bulk_bytes` from `bulk_src` returned behind it.
__global__ void __launch_bounds__(128) selftest_tma_kernel(const __grid_constant__ CUtensorMap map, int col0, int head,
                                                           int tok0, int batch, const uint8_t* bulk_src, int bulk_bytes,
                                                           uint8_t* out, int* status) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar;
  __shared__ int abort_s;
  const int tid = threadIdx.x;
  if (tid == 0) { mbar_init(&bar, 1); mbar_fence_init(); abort_s = 0; }
  __syncthreads();
  WaitCtl ctl{&abort_s, status};
  if (tid == 0) {
    mbar_expect_tx(&bar, 8192 + bulk_bytes);
    tma_load_4d(smem, &map, &bar, col0, head, tok0, batch);
    if (bulk_bytes > 0) bulk_load(smem + 8192, bulk_src, bulk_bytes, &bar);
  }
  mbar_wait(&bar, 0, ctl, DEV_TIMEOUT_LOAD);
  for (int i = tid; i < 8192 + bulk_bytes; i += 128) out[i] = smem[i];
}

// A CTA of two warps waits, with a short limit, for a barrier that nothing will ever arrive at: both warps must give up,
// the status word must read DEV_TIMEOUT_LOAD, the second warp (which starts waiting later) must see the abort flag of
// the first, and the kernel must end normally.  This is the path every production kernel takes when a pipeline stalls.
__global__ void __launch_bounds__(64) selftest_wait_kernel(long long limit_cycles, int* status, int* out) {
  __shared__ uint64_t bar;
  __shared__ int abort_s;
  if (threadIdx.x == 0) { mbar_init(&bar, 1); mbar_fence_init(); abort_s = 0; }
  __syncthreads();
  WaitCtl ctl{&abort_s, status};
  const long long t0 = clock64();
  const bool ok = mbar_wait(&bar, 0, ctl, DEV_TIMEOUT_LOAD, limit_cycles);
  const long long waited = clock64() - t0;
  __syncthreads();
  if (threadIdx.x == 0) {
    out[0] = ok ? 1 : 0;                 // 0: the wait gave up
    out[1] = abort_s;                    // 1: the CTA's abort flag is up
    out[2] = waited > 0x7fffffffLL ? 0x7fffffff : static_cast<int>(waited);
  }
}

}  // namespace tgdn

using namespace tgdn;

extern "C" int tgdn_selftest_wait(long long limit_cycles, int* out3, void* stream) {
  if (!out3) return TGDN_ERR_NULL;
  if (limit_cycles < 1 || limit_cycles > (1ll << 28)) return TGDN_ERR_SHAPE;      // a test must not hold a GPU: at most ~0.15 s
  if (!tgdn_check_device()) return TGDN_ERR_DEVICE;
  selftest_wait_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(limit_cycles, tgdn_status_word(), out3);
  return tgdn_cuda_error(cudaGetLastError());
}


extern "C" int tgdn_selftest_mma(const void* A, const void* B, void* D, int M, int N, int K, int layout_a, int layout_b,
                                 void* stream) {
  if ((M != 128 && M != 64) || N % 16 || N < 16 || N > 128 || K % 64 || K < 64 || K > 256) return TGDN_ERR_SHAPE;
  if (layout_a < 0 || layout_a > 3 || layout_b < 0 || layout_b > 3) return TGDN_ERR_SHAPE;
  const int smem = 1024 + ((128 * K * 2 + 1023) & ~1023) + (N < 64 ? 64 : N) * K * 2 + 1024;   // swizzled rows are 64 wide
  cudaError_t e = cudaFuncSetAttribute(selftest_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return tgdn_cuda_error(e);
  selftest_mma_kernel<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(A), static_cast<const __nv_bfloat16*>(B), static_cast<float*>(D), M, N, K,
      layout_a, layout_b, tgdn_status_word());
  return tgdn_cuda_error(cudaGetLastError());
}

extern "C" int tgdn_selftest_tma(const void* x, int B, int T, int H, int col0, int head, int tok0, int batch,
                                 const void* bulk_src, int bulk_bytes, void* out, void* stream) {
  if (bulk_bytes % 16 || bulk_bytes < 0 || bulk_bytes > 65536) return TGDN_ERR_SHAPE;
  CUtensorMap map;
  int rc = tgdn_make_token_map(&map, x, B, T, H, 64, 64, /*swizzle128=*/1);
  if (rc) return rc;
  const int smem = 1024 + 8192 + bulk_bytes;
  cudaError_t e = cudaFuncSetAttribute(selftest_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return tgdn_cuda_error(e);
  selftest_tma_kernel<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(
      map, col0, head, tok0, batch, static_cast<const uint8_t*>(bulk_src), bulk_bytes, static_cast<uint8_t*>(out),
      tgdn_status_word());
  return tgdn_cuda_error(cudaGetLastError());
}
