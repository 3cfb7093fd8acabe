// Per-chunk masks of the Triadic GDN: cumulative log decay, the UT transform A and the intra-chunk output operator.
//
// For every (batch, chunk, head) one CTA computes, with K, Q the 64x128 key/query tiles of the chunk:
//   gc[t,e]  = inclusive cumulative sum of the log gate over the chunk (rows past the end of a document add 0)
//   M[t,s]   = sum_e k2[t,e] k2[s,e] exp(gc[t,e]-gc[s,e]) (s <  t),  Mp[t,s] = sum_e q2[t,e] k2[s,e] exp(.) (s <= t)
//   A        = (I + strict_lower(beta_t (K K^T)[t,s] M[t,s]))^-1
//   Pm       = scale * lower(Q K^T * Mp),   PA = Pm A
// and stores gc (f32), the stacked operand image [A; PA] (bf16, 128x64) that the forward recurrence multiplies with
// beta*W, and the Pm image (bf16, 64x64) that the reverse recurrence needs.
//
// Replaces cute_triadic_gdn/kernels/sm90_joint_scan.py:21-80 (scan_kernel, forward direction) and
// cute_triadic_gdn/kernels/sm100_joint_masks.py:34-267 (masks_kernel); math as in
// cute_triadic_gdn/ops/gdn_joint.py:36-39, :45-60.  The Gram product [K;Q] K^T is one tcgen05 MMA group (M=128, N=64,
// K=128) on TMA-staged 128B-swizzled tiles; the mask sums, the blocked triangular inverse (16 -> 32 -> 64) and Pm A run
// on the CUDA cores in f32 and are rounded to bf16 once, when stored.
#include "tgdn_common.cuh"
#include "tgdn_host.h"
#include "tgdn_kernels.h"

namespace tgdn {

constexpr int MASK_THREADS = 128;

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 64x64 f32 matrix in shared memory, column index XOR-swizzled with the row so that both "lanes along a row" and
// "lanes along a column" accesses are conflict-free.
__device__ __forceinline__ int mat_idx(int i, int j) { return i * 64 + (j ^ (i & 31)); }

struct MaskSmem {
  // KQ tile (two 64-column blocks of 128 rows x 128 B) while the Gram product runs; L and X afterwards
  union {
    uint8_t kq[32768];
    struct { float L[4096]; float X[4096]; } m;
  } u;
  float Pm[4096];
  float T[1024];
  float gc2[64 * 17];      // log2-domain cumulative gate, row stride E+1
  float k2[64 * 17];
  float q2[64 * 17];
  float beta[64];
  uint64_t bar_load, bar_mma;
  uint32_t tmem_base;
  int abort;
};

// X21 = -X22 (L21 X11) for `nm` diagonal blocks of size 2n, all 128 threads.
__device__ __forceinline__ void tri_merge(float* L, float* X, float* T, int n, int nm, int tid) {
  const int total = nm * n * n;
  for (int idx = tid; idx < total; idx += MASK_THREADS) {
    const int m = idx / (n * n), rem = idx % (n * n), i = rem / n, j = rem % n, r = m * 2 * n;
    float acc = 0.f;
    for (int k = j; k < n; ++k) acc = fmaf(L[mat_idx(r + n + i, r + k)], X[mat_idx(r + k, r + j)], acc);
    T[idx] = acc;
  }
  __syncthreads();
  for (int idx = tid; idx < total; idx += MASK_THREADS) {
    const int m = idx / (n * n), rem = idx % (n * n), i = rem / n, j = rem % n, r = m * 2 * n;
    float acc = 0.f;
    for (int k = 0; k <= i; ++k) acc = fmaf(X[mat_idx(r + n + i, r + n + k)], T[m * n * n + k * n + j], acc);
    X[mat_idx(r + n + i, r + j)] = -acc;
  }
  __syncthreads();
}

template <int E>
__global__ void __launch_bounds__(MASK_THREADS)
masks_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_q, MaskParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  MaskSmem& sm = *reinterpret_cast<MaskSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.x % p.H, n = (blockIdx.x / p.H) % p.NC, b = blockIdx.x / (p.H * p.NC);
  constexpr int ES = E + 1;
  constexpr float LOG2E = 1.4426950408889634f;

  int t0 = n * CHUNK, rows = CHUNK;
  if (p.cmap != nullptr) {
    t0 = p.cmap[n];
    rows = p.cmap[p.NC + n];
    if (rows <= 0) return;                                  // unused tail of the chunk map
    if (t0 < 0 || rows > CHUNK || t0 + rows > p.T) {        // never follow a bad map entry
      if (tid == 0) atomicCAS(p.status, DEV_OK, DEV_BAD_CHUNK_MAP);
      return;
    }
  }
  if (tid == 0) {
    mbar_init(&sm.bar_load, 1);
    mbar_init(&sm.bar_mma, 1);
    mbar_fence_init();
    sm.abort = 0;
  }
  if (warp == 0) { tmem_alloc(&sm.tmem_base, 64); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  WaitCtl ctl{&sm.abort, p.status};

  if (tid == 0) {
    mbar_expect_tx(&sm.bar_load, 32768);
    tma_load_4d(sm.u.kq, &map_k, &sm.bar_load, 0, h, t0, b);
    tma_load_4d(sm.u.kq + 8192, &map_q, &sm.bar_load, 0, h, t0, b);
    tma_load_4d(sm.u.kq + 16384, &map_k, &sm.bar_load, 64, h, t0, b);
    tma_load_4d(sm.u.kq + 24576, &map_q, &sm.bar_load, 64, h, t0, b);
  }

  // gates of the chunk: rows past the document end count as g = 0, k2 = q2 = beta = 0
  const int64_t tok = static_cast<int64_t>(b) * p.T + t0;
  for (int idx = tid; idx < 64 * E; idx += MASK_THREADS) {
    const int r = idx / E, e = idx % E;
    const bool ok = r < rows;
    const int64_t g_off = ((tok + r) * p.H + h) * E + e;
    sm.gc2[r * ES + e] = ok ? p.g[g_off] : 0.f;
    sm.k2[r * ES + e] = ok ? p.k2[g_off] : 0.f;
    sm.q2[r * ES + e] = ok ? p.q2[g_off] : 0.f;
  }
  if (tid < 64) sm.beta[tid] = (tid < rows) ? p.beta[(tok + tid) * p.H + h] : 0.f;
  __syncthreads();
  // inclusive scan over the 64 rows, one warp per gate column
  float* gc_out = p.gc + ((static_cast<int64_t>(b) * p.NC + n) * p.H + h) * (64 * E);
  for (int e = warp; e < E; e += MASK_THREADS / 32) {
    float v0 = sm.gc2[lane * ES + e], v1 = sm.gc2[(lane + 32) * ES + e];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float a0 = __shfl_up_sync(0xffffffffu, v0, o), a1 = __shfl_up_sync(0xffffffffu, v1, o);
      if (lane >= o) { v0 += a0; v1 += a1; }
    }
    v1 += __shfl_sync(0xffffffffu, v0, 31);
    gc_out[lane * E + e] = v0;
    gc_out[(lane + 32) * E + e] = v1;
    sm.gc2[lane * ES + e] = v0 * LOG2E;
    sm.gc2[(lane + 32) * ES + e] = v1 * LOG2E;
  }
  __syncthreads();

  // Gram product [K;Q] K^T
  mbar_wait(&sm.bar_load, 0, ctl, DEV_TIMEOUT_LOAD);
  const uint32_t tmem = sm.tmem_base;
  if (tid == 0) {
    tc_fence_after();
    const uint64_t desc = make_desc(smem_u32(sm.u.kq), 16, 1024, LAYOUT_SW128);
    constexpr uint32_t idesc = make_idesc(128, 64, 0, 0);
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
      umma_bf16(tmem, desc_advance(desc, off), desc_advance(desc, off), idesc, kk > 0);
    }
    umma_commit(&sm.bar_mma);
  }
  mbar_wait(&sm.bar_mma, 0, ctl, DEV_TIMEOUT_MMA);
  tc_fence_after();
  float pr[64];                                             // row `tid` of [K K^T ; Q K^T]
  tmem_ld<64>(tmem + (static_cast<uint32_t>(warp * 32) << 16), pr);
  tmem_wait_ld();
  tc_fence_before();
  __syncthreads();                                          // the KQ tile is dead from here: L and X take its place

  // mask sums: threads 0..63 rows of M (strictly lower) -> L, threads 64..127 rows of Mp (lower) -> Pm
  {
    const int t = tid & 63;
    const bool isq = tid >= 64;
    float my2[E], mygc[E];
#pragma unroll
    for (int e = 0; e < E; ++e) {
      my2[e] = isq ? sm.q2[t * ES + e] : sm.k2[t * ES + e];
      mygc[e] = sm.gc2[t * ES + e];
    }
    const float rowscale = isq ? p.scale : sm.beta[t];
    float* dst = isq ? sm.Pm : sm.u.m.L;
    const int smax = ((warp & 1) ? 63 : 31);              // largest row of this warp
#pragma unroll
    for (int s = 0; s < 64; ++s) {
      float val = 0.f;
      if (s <= smax) {
        const bool use = isq ? (s <= t) : (s < t);
        if (use) {
          float acc = 0.f;
#pragma unroll
          for (int e = 0; e < E; ++e)
            acc = fmaf(my2[e] * sm.k2[s * ES + e], fast_exp2(mygc[e] - sm.gc2[s * ES + e]), acc);
          val = rowscale * pr[s] * acc;
        }
      }
      dst[mat_idx(t, s)] = val;
    }
  }
  __syncthreads();

  // triangular inverse X = (I + L)^-1: 16x16 diagonal blocks by forward substitution, then two merge levels
  float* L = sm.u.m.L;
  float* X = sm.u.m.X;
  if (tid < 64) {
    const int r0 = (tid >> 4) * 16, j = tid & 15;
    float x[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float acc = 0.f;
#pragma unroll
      for (int k = 0; k < i; ++k) acc = fmaf(L[mat_idx(r0 + i, r0 + k)], x[k], acc);
      x[i] = (i == j) ? 1.f : (i < j ? 0.f : -acc);
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) X[mat_idx(r0 + i, r0 + j)] = x[i];
  } else {
    // zero everything outside the diagonal 16x16 blocks that the merges do not write (the upper triangle)
    for (int idx = tid - 64; idx < 4096; idx += 64) {
      const int i = idx >> 6, j = idx & 63;
      if ((j >> 4) > (i >> 4)) X[mat_idx(i, j)] = 0.f;
    }
  }
  __syncthreads();
  tri_merge(L, X, sm.T, 16, 2, tid);
  tri_merge(L, X, sm.T, 32, 1, tid);

  // PA = Pm X (both lower triangular); L is dead, PA takes its place
  float* PA = sm.u.m.L;
  for (int idx = tid; idx < 4096; idx += MASK_THREADS) {
    const int t = idx >> 6, j = idx & 63;
    float acc = 0.f;
    for (int k = j; k <= t; ++k) acc = fmaf(sm.Pm[mat_idx(t, k)], X[mat_idx(k, j)], acc);
    PA[mat_idx(t, j)] = acc;
  }
  __syncthreads();

  // stores: operand images, one 16-byte piece (8 columns of one row) per thread and step, linear in global memory
  const int64_t item = (static_cast<int64_t>(b) * p.NC + n) * p.H + h;
  uint4* ap_out = reinterpret_cast<uint4*>(p.AP + item * (128 * 64));
  uint4* pm_out = reinterpret_cast<uint4*>(p.Pm + item * (64 * 64));
#pragma unroll
  for (int jb = 0; jb < 8; ++jb) {
    const float* src = (tid < 64) ? X : PA;
    const int i = tid & 63;
    float v[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) v[c] = src[mat_idx(i, jb * 8 + c)];
    uint4 u;
    u.x = pack_bf16(v[0], v[1]); u.y = pack_bf16(v[2], v[3]); u.z = pack_bf16(v[4], v[5]); u.w = pack_bf16(v[6], v[7]);
    ap_out[jb * 128 + tid] = u;                              // image (i = row 0..127, j = column), SI = 128, SJ = 2048
  }
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int piece = it * MASK_THREADS + tid, i = piece & 63, jb = piece >> 6;
    float v[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) v[c] = sm.Pm[mat_idx(i, jb * 8 + c)];
    uint4 u;
    u.x = pack_bf16(v[0], v[1]); u.y = pack_bf16(v[2], v[3]); u.z = pack_bf16(v[4], v[5]); u.w = pack_bf16(v[6], v[7]);
    pm_out[piece] = u;                                       // image (i = t, j = s), SI = 128, SJ = 1024
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 64);
}

}  // namespace tgdn

using namespace tgdn;

template <int E>
static int launch_masks(const CUtensorMap& mk, const CUtensorMap& mq, const MaskParams& p, cudaStream_t s) {
  const int smem = static_cast<int>(sizeof(MaskSmem)) + 1024;
  cudaError_t e = cudaFuncSetAttribute(masks_kernel<E>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return tgdn_cuda_error(e);
  masks_kernel<E><<<p.B * p.NC * p.H, MASK_THREADS, smem, s>>>(mk, mq, p);
  return tgdn_cuda_error(cudaGetLastError());
}

extern "C" int tgdn_masks(const void* q, const void* k, const float* k2, const float* q2, const float* g,
                          const float* beta, float scale, const int32_t* chunk_map, int B, int T, int H, int E, int NC,
                          float* gc, void* AP, void* Pm, void* stream) {
  if (!q || !k || !k2 || !q2 || !g || !beta || !gc || !AP || !Pm) return TGDN_ERR_NULL;
  int rc = tgdn_check_core_shape(B, T, H, E, NC, chunk_map != nullptr);
  if (rc) return rc;
  if ((reinterpret_cast<uintptr_t>(AP) | reinterpret_cast<uintptr_t>(Pm)) & 15) return TGDN_ERR_ALIGN;
  CUtensorMap mk, mq;
  if ((rc = tgdn_make_token_map(&mk, k, B, T, H, 64, 64, 1))) return rc;
  if ((rc = tgdn_make_token_map(&mq, q, B, T, H, 64, 64, 1))) return rc;
  MaskParams p{k2, q2, g, beta, gc, static_cast<__nv_bfloat16*>(AP), static_cast<__nv_bfloat16*>(Pm), chunk_map,
               B, T, H, NC, scale, tgdn_status_word()};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (E) {
    case 1: return launch_masks<1>(mk, mq, p, s);
    case 2: return launch_masks<2>(mk, mq, p, s);
    case 4: return launch_masks<4>(mk, mq, p, s);
    case 8: return launch_masks<8>(mk, mq, p, s);
    case 12: return launch_masks<12>(mk, mq, p, s);
    case 16: return launch_masks<16>(mk, mq, p, s);
    default: return TGDN_ERR_SHAPE;
  }
}
