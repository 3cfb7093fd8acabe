// Per-chunk matrix gradients of the Triadic GDN backward, the mask gradients and the final assembly of dq, dk, dk2,
// dq2, dg, dbeta.
//
// One CTA of 128 threads per (batch, chunk, head); thread r < 64 owns key row t = r, thread 64 + t owns query row t.
//   G1  P    = [K;Q] K^T                     (Pkk rows 0..63, Pqk rows 64..127)
//   G2  [dU;dO] [W;U]^T                      (rows 0..63, cols 0..63: dA' = dU W^T;  rows 64..127, cols 64..127: dPm' = dO U^T)
//       X    = scale*lower(Mp*dPm'),  dmp = scale*lower(Pqk*dPm'),  dA = dA' diag(beta),  dbeta_col = colsum(dA'*A)
//   G3  Y    = A^T dA          G4  dp = Y A^T,   dL = -strict_lower(dp)
//       dbeta_row = rowsum(dL*Pkk*M),  dPkk = beta_t dL*M,  dm = beta_t dL*Pkk
//   G5  [dK;dQ] = [[dPkk+dPkk^T, X^T],[X, 0]] [K;Q]  + state part (from the state-gradient kernel)
//   mask gradients r1, c1 (from dmp) and r2, c2 (from dm) with the decay factors recomputed, gate-table gradients
//   folded in, reverse cumulative sum of dgc inside the chunk -> dg.
//
// Replaces cute_triadic_gdn/kernels/sm100_joint_bwd_parallel.py:80-405 (matrix_kernel),
// cute_triadic_gdn/kernels/sm90_joint_bwd_parallel.py:278-372 (mask_grad_kernel) and the reverse pass of
// cute_triadic_gdn/kernels/sm90_joint_scan.py:21-80; math as listed in cute_triadic_gdn/ops/gdn_joint.py:45-90 differentiated.
#include "tgdn_common.cuh"
#include "tgdn_host.h"
#include "tgdn_kernels.h"

namespace tgdn {

constexpr int MAT_THREADS = 128;

__device__ __forceinline__ float mexp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ int midx(int i, int j) { return i * 64 + (j ^ (i & 31)); }
__device__ __forceinline__ void st_shared_b16(uint32_t saddr, float v) {
  const unsigned short b = __bfloat16_as_ushort(__float2bfloat16_rn(v));
  asm volatile("st.shared.b16 [%0], %1;" ::"r"(saddr), "h"(b) : "memory");
}

struct MatSmem {
  uint8_t kq[32768];                 // [K;Q] tile
  union {
    uint8_t dudo[32768];             // [dU;dO] tile (until G2), then the 128x128 operand of G5:
    uint8_t a5[32768];               //   image (i = row, j = col), SI = 128, SJ = 2048
  } u1;
  union {
    uint8_t wu[32768];               // [W;U] tile (until G2), then two f32 64x64 matrices
    struct { float dmp[4096]; float dm[4096]; } f;
  } u2;
  uint8_t ap[16384];                 // [A;PmA] image, rows 0..63 = A
  uint8_t da[8192];                  // dA image (i = t, j = s), SI = 128, SJ = 1024
  uint8_t y[8192];                   // Y image (i = s', j = t'), SI = 128, SJ = 1024 (read as 128 rows: daa follows)
  float daa[4096];                   // dA' * A, for the column sums
  float gc2[64 * 17], k2[64 * 17], q2[64 * 17];
  float r1[64 * 17], c1[64 * 17], dgc[64 * 17];
  float beta[64];
  uint64_t bar_load, bar_mma;
  uint32_t tmem_base;
  int abort;
};

template <int E>
__global__ void __launch_bounds__(MAT_THREADS, 1)
mat_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_q,
           const __grid_constant__ CUtensorMap map_do, const __grid_constant__ CUtensorMap map_du,
           const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_u, MatParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  MatSmem& sm = *reinterpret_cast<MatSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int ES = 17;
  constexpr float LOG2E = 1.4426950408889634f;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool krow = tid < 64;
  const int t = tid & 63;
  const int h = blockIdx.x % p.H, n = (blockIdx.x / p.H) % p.NC, b = blockIdx.x / (p.H * p.NC);
  const int64_t item = blockIdx.x;

  int t0 = n * CHUNK, rows = CHUNK;
  if (p.cmap != nullptr) {
    t0 = p.cmap[n];
    rows = p.cmap[p.NC + n];
    if (rows <= 0) return;
    if (t0 < 0 || rows > CHUNK || t0 + rows > p.T) {
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
  if (warp == 0) { tmem_alloc(&sm.tmem_base, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  const uint32_t tmem_row = tmem + (static_cast<uint32_t>(warp * 32) << 16);
  WaitCtl ctl{&sm.abort, p.status};
  const int crow = static_cast<int>(item) * 64;           // first row of this item in the chunk-layout tensors

  if (tid == 0) {
    mbar_expect_tx(&sm.bar_load, 3 * 32768 + 16384);
    for (int half = 0; half < 2; ++half) {
      const int col = half * 64;
      tma_load_4d(sm.kq + half * 16384, &map_k, &sm.bar_load, col, h, t0, b);
      tma_load_4d(sm.kq + half * 16384 + 8192, &map_q, &sm.bar_load, col, h, t0, b);
      tma_load_4d(sm.u1.dudo + half * 16384, &map_du, &sm.bar_load, col, 0, crow, 0);
      tma_load_4d(sm.u1.dudo + half * 16384 + 8192, &map_do, &sm.bar_load, col, h, t0, b);
      tma_load_4d(sm.u2.wu + half * 16384, &map_w, &sm.bar_load, col, 0, crow, 0);
      tma_load_4d(sm.u2.wu + half * 16384 + 8192, &map_u, &sm.bar_load, col, 0, crow, 0);
    }
    bulk_load(sm.ap, p.AP + item * (128 * 64), 16384, &sm.bar_load);
  }
  // gates (log2 domain), rows past the document end: k2 = q2 = beta = 0
  const int64_t tok = static_cast<int64_t>(b) * p.T + t0;
  for (int idx = tid; idx < 64 * E; idx += MAT_THREADS) {
    const int r = idx / E, e = idx % E;
    const bool ok = r < rows;
    const int64_t off = ((tok + r) * p.H + h) * E + e;
    sm.gc2[r * ES + e] = p.gc[item * (64 * E) + idx] * LOG2E;
    sm.k2[r * ES + e] = ok ? p.k2[off] : 0.f;
    sm.q2[r * ES + e] = ok ? p.q2[off] : 0.f;
  }
  if (tid < 64) sm.beta[tid] = (tid < rows) ? p.beta[(tok + tid) * p.H + h] : 0.f;
  __syncthreads();

  // ---- G1, G2 ----------------------------------------------------------------------------------------------------
  mbar_wait(&sm.bar_load, 0, ctl, DEV_TIMEOUT_LOAD);
  if (tid == 0) {
    tc_fence_after();
    const uint64_t dkq = make_desc(smem_u32(sm.kq), 16, 1024, LAYOUT_SW128);
    const uint64_t dd = make_desc(smem_u32(sm.u1.dudo), 16, 1024, LAYOUT_SW128);
    const uint64_t dw = make_desc(smem_u32(sm.u2.wu), 16, 1024, LAYOUT_SW128);
    constexpr uint32_t id1 = make_idesc(128, 64, 0, 0), id2 = make_idesc(128, 128, 0, 0);
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
      umma_bf16(tmem, desc_advance(dkq, off), desc_advance(dkq, off), id1, kk > 0);
    }
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
      umma_bf16(tmem + 64, desc_advance(dd, off), desc_advance(dw, off), id2, kk > 0);
    }
    umma_commit(&sm.bar_mma);
  }
  uint32_t mma_phase = 0;
  mbar_wait(&sm.bar_mma, mma_phase & 1, ctl, DEV_TIMEOUT_MMA);
  ++mma_phase;
  tc_fence_after();
  float pr[64];                                            // Pkk row (key rows) / Pqk row (query rows)
  float gr[64];                                            // dA' row (key rows) / dPm' row (query rows)
  tmem_ld<64>(tmem_row, pr);
  tmem_ld<64>(tmem_row + 64 + (krow ? 0 : 64), gr);
  tmem_wait_ld();
  tc_fence_before();
  __syncthreads();                                         // dudo and wu are dead: a5, dmp, dm take their place

  float my2[E], mygc[E];
#pragma unroll
  for (int e = 0; e < E; ++e) {
    my2[e] = krow ? sm.k2[t * ES + e] : sm.q2[t * ES + e];
    mygc[e] = sm.gc2[t * ES + e];
  }
  const uint32_t a5 = smem_u32(sm.u1.a5);
  float r1v[E];                                            // query rows: r1;  key rows (later): r2
#pragma unroll
  for (int e = 0; e < E; ++e) r1v[e] = 0.f;
  float dbeta = 0.f;

  if (!krow) {
    // query row t: X row -> a5 (row 64+t and, transposed, column 64+t), dmp row, r1
    const float live = (t < rows) ? 1.f : 0.f;
    float xrow[64];
#pragma unroll
    for (int s = 0; s < 64; ++s) {
      float x = 0.f, dmpv = 0.f;
      if (s <= ((warp & 1) ? 63 : 31) && s <= t) {
        float dec[E];
        float mp = 0.f;
#pragma unroll
        for (int e = 0; e < E; ++e) {
          dec[e] = mexp2(mygc[e] - sm.gc2[s * ES + e]) * sm.k2[s * ES + e];
          mp = fmaf(my2[e], dec[e], mp);
        }
        x = p.scale * mp * gr[s];
        dmpv = live * p.scale * pr[s] * gr[s];
#pragma unroll
        for (int e = 0; e < E; ++e) r1v[e] = fmaf(dmpv, dec[e], r1v[e]);
      }
      xrow[s] = x;
      sm.u2.f.dmp[midx(t, s)] = dmpv;
      st_shared_b16(a5 + (s >> 3) * 128 + ((64 + t) >> 3) * 2048 + (s & 7) * 16 + (t & 7) * 2, x);   // a5[s][64+t]
    }
    const uint32_t rowbase = a5 + ((64 + t) >> 3) * 128 + (t & 7) * 16;
#pragma unroll
    for (int jb = 0; jb < 8; ++jb) {
      st_shared_v4(rowbase + jb * 2048, pack_bf16(xrow[jb * 8], xrow[jb * 8 + 1]), pack_bf16(xrow[jb * 8 + 2], xrow[jb * 8 + 3]),
                   pack_bf16(xrow[jb * 8 + 4], xrow[jb * 8 + 5]), pack_bf16(xrow[jb * 8 + 6], xrow[jb * 8 + 7]));
      st_shared_v4(rowbase + (8 + jb) * 2048, 0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int e = 0; e < E; ++e) sm.r1[t * ES + e] = r1v[e];
  } else {
    // key row t: dA = dA' diag(beta) -> operand image; dA' * A -> column sums
    const uint32_t apr = smem_u32(sm.ap) + (t >> 3) * 128 + (t & 7) * 16;
    const uint32_t dar = smem_u32(sm.da) + (t >> 3) * 128 + (t & 7) * 16;
#pragma unroll
    for (int jb = 0; jb < 8; ++jb) {
      uint32_t aw[4];
      asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(aw[0]), "=r"(aw[1]), "=r"(aw[2]), "=r"(aw[3]) : "r"(apr + jb * 2048));
      float dav[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const int s = jb * 8 + c;
        const float a_ts = (c & 1) ? bf16_hi(aw[c >> 1]) : bf16_lo(aw[c >> 1]);
        sm.daa[midx(t, s)] = gr[s] * a_ts;
        dav[c] = gr[s] * sm.beta[s];
      }
      st_shared_v4(dar + jb * 1024, pack_bf16(dav[0], dav[1]), pack_bf16(dav[2], dav[3]), pack_bf16(dav[4], dav[5]),
                   pack_bf16(dav[6], dav[7]));
    }
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();

  // ---- G3: Y = A^T dA ----------------------------------------------------------------------------------------------
  if (tid == 0) {
    tc_fence_after();
    const uint64_t da = make_desc(smem_u32(sm.ap), 128, 2048, LAYOUT_PLAIN);     // A^T, MN-major
    const uint64_t db = make_desc(smem_u32(sm.da), 128, 1024, LAYOUT_PLAIN);     // dA (K = t, N = s), MN-major
    constexpr uint32_t idesc = make_idesc(128, 64, 1, 1);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) umma_bf16(tmem + 192, desc_advance(da, kk * 256), desc_advance(db, kk * 256), idesc, kk > 0);
    umma_commit(&sm.bar_mma);
  }
  if (krow) {                                              // meanwhile: dbeta_col[s = t] = sum_t' dA'[t',s] A[t',s]
    float acc = 0.f;
    for (int tt = 0; tt < 64; ++tt) acc += sm.daa[midx(tt, t)];
    dbeta = acc;
  }
  mbar_wait(&sm.bar_mma, mma_phase & 1, ctl, DEV_TIMEOUT_MMA);
  ++mma_phase;
  tc_fence_after();
  if (krow) {
    float yr[64];
    tmem_ld<64>(tmem_row + 192, yr);
    tmem_wait_ld();
    const uint32_t yb = smem_u32(sm.y) + (t >> 3) * 128 + (t & 7) * 16;
#pragma unroll
    for (int jb = 0; jb < 8; ++jb)
      st_shared_v4(yb + jb * 1024, pack_bf16(yr[jb * 8], yr[jb * 8 + 1]), pack_bf16(yr[jb * 8 + 2], yr[jb * 8 + 3]),
                   pack_bf16(yr[jb * 8 + 4], yr[jb * 8 + 5]), pack_bf16(yr[jb * 8 + 6], yr[jb * 8 + 7]));
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();

  // ---- G4: dp = Y A^T ----------------------------------------------------------------------------------------------
  if (tid == 0) {
    tc_fence_after();
    const uint64_t da = make_desc(smem_u32(sm.y), 1024, 128, LAYOUT_PLAIN);      // Y, K-major
    const uint64_t db = make_desc(smem_u32(sm.ap), 2048, 128, LAYOUT_PLAIN);     // B[k][j] = A[j][k]: A rows as N, K-major
    constexpr uint32_t idesc = make_idesc(128, 64, 0, 0);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) umma_bf16(tmem + 256, desc_advance(da, kk * 2048), desc_advance(db, kk * 4096), idesc, kk > 0);
    umma_commit(&sm.bar_mma);
  }
  mbar_wait(&sm.bar_mma, mma_phase & 1, ctl, DEV_TIMEOUT_MMA);
  ++mma_phase;
  tc_fence_after();
  if (krow) {
    // key row t: dL row, dbeta_row, dm row, r2, and dPkk + dPkk^T into a5[0..63][0..63]
    float dpr[64];
    tmem_ld<64>(tmem_row + 256, dpr);
    tmem_wait_ld();
    const float bt = sm.beta[t];
    float brow = 0.f;
#pragma unroll
    for (int s = 0; s < 64; ++s) {
      float dmv = 0.f;
      if (s <= ((warp & 1) ? 63 : 31) && s < t) {
        float dec[E];
        float m = 0.f;
#pragma unroll
        for (int e = 0; e < E; ++e) {
          dec[e] = mexp2(mygc[e] - sm.gc2[s * ES + e]) * sm.k2[s * ES + e];
          m = fmaf(my2[e], dec[e], m);
        }
        const float dl = -dpr[s];
        brow = fmaf(dl * pr[s], m, brow);
        dmv = bt * dl * pr[s];
        const float dpk = bt * dl * m;
#pragma unroll
        for (int e = 0; e < E; ++e) r1v[e] = fmaf(dmv, dec[e], r1v[e]);
        st_shared_b16(a5 + (t >> 3) * 128 + (s >> 3) * 2048 + (t & 7) * 16 + (s & 7) * 2, dpk);     // a5[t][s]
        st_shared_b16(a5 + (s >> 3) * 128 + (t >> 3) * 2048 + (s & 7) * 16 + (t & 7) * 2, dpk);     // a5[s][t]
      }
      sm.u2.f.dm[midx(t, s)] = dmv;
    }
    st_shared_b16(a5 + (t >> 3) * 128 + (t >> 3) * 2048 + (t & 7) * 16 + (t & 7) * 2, 0.f);         // diagonal
    dbeta += brow;
  } else {
    // query thread 64+s: c1[s,e] = sum_{t'>=s} dmp[t',s] exp(gc[t']-gc[s]) q2[t',e]
    const int s = t;
    float c1v[E];
#pragma unroll
    for (int e = 0; e < E; ++e) c1v[e] = 0.f;
    for (int tt = s; tt < 64; ++tt) {
      const float dv = sm.u2.f.dmp[midx(tt, s)];
#pragma unroll
      for (int e = 0; e < E; ++e)
        c1v[e] = fmaf(dv * sm.q2[tt * ES + e], mexp2(sm.gc2[tt * ES + e] - mygc[e]), c1v[e]);
    }
#pragma unroll
    for (int e = 0; e < E; ++e) sm.c1[s * ES + e] = c1v[e];
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();

  // ---- G5: [dK;dQ] = a5 [K;Q] --------------------------------------------------------------------------------------
  if (tid == 0) {
    tc_fence_after();
    const uint64_t da = make_desc(a5, 2048, 128, LAYOUT_PLAIN);
    const uint64_t db = make_desc(smem_u32(sm.kq), 16384, 1024, LAYOUT_SW128);   // (K = token rows, N = d), MN-major
    constexpr uint32_t idesc = make_idesc(128, 128, 0, 1);
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) umma_bf16(tmem, desc_advance(da, kk * 4096), desc_advance(db, kk * 2048), idesc, kk > 0);
    umma_commit(&sm.bar_mma);
  }
  // meanwhile the gate gradients of key row t
  if (krow) {
    float c2v[E];
#pragma unroll
    for (int e = 0; e < E; ++e) c2v[e] = 0.f;
    for (int tt = t + 1; tt < 64; ++tt) {
      const float dv = sm.u2.f.dm[midx(tt, t)];
#pragma unroll
      for (int e = 0; e < E; ++e)
        c2v[e] = fmaf(dv * sm.k2[tt * ES + e], mexp2(sm.gc2[tt * ES + e] - mygc[e]), c2v[e]);
    }
    const bool live = t < rows;
    const float* dap = p.da + (item * 64 + t) * E;
    const float* dcp = p.dc + (item * 64 + t) * E;
    float* dk2p = p.dk2 + ((tok + t) * p.H + h) * E;
    float* dq2p = p.dq2 + ((tok + t) * p.H + h) * E;
#pragma unroll
    for (int e = 0; e < E; ++e) {
      float drv = 0.f;
      for (int v = 0; v < p.NV; ++v) drv += p.dr[((item * p.NV + v) * 64 + t) * E + e];
      const float gl = sm.gc2[63 * ES + e];
      const float eg = mexp2(mygc[e]), egr = mexp2(gl - mygc[e]);
      const float k2v = my2[e], q2v = sm.q2[t * ES + e];
      const float dav = dap[e], dcv = dcp[e];
      const float r1e = sm.r1[t * ES + e], c1e = sm.c1[t * ES + e], r2e = r1v[e], c2e = c2v[e];
      if (live) {
        dk2p[e] = dav * eg + drv * egr + c1e + r2e + c2e;
        dq2p[e] = dcv * p.scale * eg + r1e;
      }
      // dgc[t,e]; the chunk-end terms are added to row 63 below
      sm.dgc[t * ES + e] = dav * (k2v * eg) + dcv * (p.scale * q2v * eg) - drv * (k2v * egr) + q2v * r1e + k2v * (r2e - c1e - c2e);
      sm.r1[t * ES + e] = drv * (k2v * egr);                // reuse: dr*r, summed over the rows below
    }
    if (live) p.dbeta[(tok + t) * p.H + h] = dbeta;
  }
  __syncthreads();
  if (tid < E) {                                            // chunk-end terms: sum_t dr*r + dd*exp(gL)
    float acc = 0.f;
    for (int tt = 0; tt < 64; ++tt) acc += sm.r1[tt * ES + tid];
    acc += p.dd[item * E + tid] * mexp2(sm.gc2[63 * ES + tid]);
    sm.dgc[63 * ES + tid] += acc;
  }
  __syncthreads();
  // dg = reverse inclusive cumulative sum of dgc over the chunk, one warp per gate column
  for (int e = warp; e < E; e += MAT_THREADS / 32) {
    float v1 = sm.dgc[(63 - lane) * ES + e], v0 = sm.dgc[(31 - lane) * ES + e];      // lane l: rows 63-l and 31-l
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float a1 = __shfl_up_sync(0xffffffffu, v1, o), a0 = __shfl_up_sync(0xffffffffu, v0, o);
      if (lane >= o) { v1 += a1; v0 += a0; }
    }
    v0 += __shfl_sync(0xffffffffu, v1, 31);
    const int ra = 63 - lane, rb = 31 - lane;
    if (ra < rows) p.dg[((tok + ra) * p.H + h) * E + e] = v1;
    if (rb < rows) p.dg[((tok + rb) * p.H + h) * E + e] = v0;
  }

  // ---- dk, dq ------------------------------------------------------------------------------------------------------
  mbar_wait(&sm.bar_mma, mma_phase & 1, ctl, DEV_TIMEOUT_MMA);
  ++mma_phase;
  tc_fence_after();
  {
    const float* sp = p.dkq + (item * 128 + tid) * HEAD;
    __nv_bfloat16* outp = (krow ? p.dk : p.dq) + ((tok + t) * p.H + h) * HEAD;
    const bool live = t < rows;
#pragma unroll
    for (int c0 = 0; c0 < 128; c0 += 16) {
      float a[16];
      tmem_ld<16>(tmem_row + c0, a);
      tmem_wait_ld();
      if (live) {
#pragma unroll
        for (int j = 0; j < 16; j += 8) {
          const float4 s0 = *reinterpret_cast<const float4*>(sp + c0 + j), s1 = *reinterpret_cast<const float4*>(sp + c0 + j + 4);
          uint4 u;
          u.x = pack_bf16(a[j] + s0.x, a[j + 1] + s0.y);
          u.y = pack_bf16(a[j + 2] + s0.z, a[j + 3] + s0.w);
          u.z = pack_bf16(a[j + 4] + s1.x, a[j + 5] + s1.y);
          u.w = pack_bf16(a[j + 6] + s1.z, a[j + 7] + s1.w);
          *reinterpret_cast<uint4*>(outp + c0 + j) = u;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

}  // namespace tgdn

using namespace tgdn;

template <int E>
static int launch_mat(const CUtensorMap* maps, const MatParams& p, cudaStream_t s) {
  const int smem = static_cast<int>(sizeof(MatSmem)) + 1024;
  cudaError_t e = cudaFuncSetAttribute(mat_kernel<E>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return tgdn_cuda_error(e);
  mat_kernel<E><<<p.B * p.NC * p.H, MAT_THREADS, smem, s>>>(maps[0], maps[1], maps[2], maps[3], maps[4], maps[5], p);
  return tgdn_cuda_error(cudaGetLastError());
}

extern "C" int tgdn_bwd_matrix(const void* q, const void* k, const void* dO, const void* dU, const void* W, const void* U,
                               const void* AP, const float* k2, const float* q2, const float* beta, const float* gc,
                               const float* dkq, const float* da, const float* dc, const float* dd, const float* dr,
                               float scale, const int32_t* chunk_map, int B, int T, int H, int E, int NC, void* dq,
                               void* dk, float* dk2, float* dq2, float* dg, float* dbeta, void* stream) {
  if (!q || !k || !dO || !dU || !W || !U || !AP || !k2 || !q2 || !beta || !gc || !dkq || !da || !dc || !dd || !dr ||
      !dq || !dk || !dk2 || !dq2 || !dg || !dbeta)
    return TGDN_ERR_NULL;
  int rc = tgdn_check_core_shape(B, T, H, E, NC, chunk_map != nullptr);
  if (rc) return rc;
  if ((reinterpret_cast<uintptr_t>(AP) | reinterpret_cast<uintptr_t>(dkq) | reinterpret_cast<uintptr_t>(dq) |
       reinterpret_cast<uintptr_t>(dk)) & 15)
    return TGDN_ERR_ALIGN;
  const long long crows = static_cast<long long>(B) * NC * H * 64;
  if (crows > 0x7fffffffLL) return TGDN_ERR_SHAPE;
  CUtensorMap maps[6];
  if ((rc = tgdn_make_token_map(&maps[0], k, B, T, H, 64, 64, 1))) return rc;
  if ((rc = tgdn_make_token_map(&maps[1], q, B, T, H, 64, 64, 1))) return rc;
  if ((rc = tgdn_make_token_map(&maps[2], dO, B, T, H, 64, 64, 1))) return rc;
  // chunk-layout tensors are plain (rows, 128) matrices: one batch row, one head
  if ((rc = tgdn_make_token_map(&maps[3], dU, 1, static_cast<int>(crows), 1, 64, 64, 1))) return rc;
  if ((rc = tgdn_make_token_map(&maps[4], W, 1, static_cast<int>(crows), 1, 64, 64, 1))) return rc;
  if ((rc = tgdn_make_token_map(&maps[5], U, 1, static_cast<int>(crows), 1, 64, 64, 1))) return rc;
  MatParams p{k2, q2, beta, gc, static_cast<const __nv_bfloat16*>(AP), dkq, da, dc, dd, dr,
              static_cast<__nv_bfloat16*>(dq), static_cast<__nv_bfloat16*>(dk), dk2, dq2, dg, dbeta, chunk_map,
              B, T, H, NC, 128 / tgdn_value_block(E), scale, tgdn_status_word()};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (E) {
    case 1: return launch_mat<1>(maps, p, s);
    case 2: return launch_mat<2>(maps, p, s);
    case 4: return launch_mat<4>(maps, p, s);
    case 8: return launch_mat<8>(maps, p, s);
    case 12: return launch_mat<12>(maps, p, s);
    case 16: return launch_mat<16>(maps, p, s);
    default: return TGDN_ERR_SHAPE;
  }
}
