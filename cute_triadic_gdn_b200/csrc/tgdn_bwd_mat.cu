// Per-chunk matrix gradients of the Triadic GDN backward, the mask gradients and the final assembly of dq, dk, dk2,
// dq2, dg, dbeta.
//
// One CTA of 512 threads per (batch, chunk, head).  Thread (r, cq): r = tensor-memory lane = matrix row (r < 64: key row
// t = r, r >= 64: query row t = r - 64), cq = which 16 of the 64 columns s it works on.
//   G1  P    = [K;Q] K^T                     (Pkk rows 0..63, Pqk rows 64..127)
//   G2  [dU;dO] [W;U]^T                      (rows 0..63, cols 0..63: dA' = dU W^T;  rows 64..127, cols 64..127: dPm' = dO U^T)
//       X    = scale*lower(Mp*dPm'),  dmp = scale*lower(Pqk*dPm'),  dA = dA' diag(beta),  dbeta_col = colsum(dA'*A)
//   G3  Y    = A^T dA          G4  dp = Y A^T,   dL = -strict_lower(dp)
//       dbeta_row = rowsum(dL*Pkk*M),  dPkk = beta_t dL*M,  dm = beta_t dL*Pkk
//   G5  [dK;dQ] = [[dPkk+dPkk^T, X^T],[X, 0]] [K;Q]  + state part (from the state-gradient kernel); the operand is P + P^T
//       with P = [[dPkk, 0],[X, 0]] written by rows: two MMA groups on one image, read K-major and MN-major
//   mask gradients r1, c1 (from dmp) and r2, c2 (from dm) with the decay factors recomputed, gate-table gradients
//   folded in, reverse cumulative sum of dgc inside the chunk -> dg.
// Row and column sums that span the four column quarters go through four-copy partial tables in shared memory and are
// added in a fixed order (no atomics: results are bitwise reproducible).
//
// Replaces cute_triadic_gdn/kernels/sm100_joint_bwd_parallel.py:80-405 (matrix_kernel),
// cute_triadic_gdn/kernels/sm90_joint_bwd_parallel.py:278-372 (mask_grad_kernel) and the reverse pass of
// cute_triadic_gdn/kernels/sm90_joint_scan.py:21-80; math as listed in cute_triadic_gdn/ops/gdn_joint.py:45-90 differentiated.
#include "tgdn_common.cuh"
#include "tgdn_host.h"
#include "tgdn_kernels.h"

namespace tgdn {

constexpr int MAT_THREADS = 512;

__device__ __forceinline__ float mexp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ int midx(int i, int j) { return i * 64 + (j ^ (i & 31)); }

template <int E>
struct MatSmem {
  static constexpr int ES = E | 1;
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
  // decay tables whose rows are read by whole warps at once (dense rows, 16-byte loads):
  alignas(16) float hkv[64 * E];     // until the two chains join: exp2(gc[r0(s)] - gc[s]) * k2[s], r0(s) the first row of
                                     // s's 16-row block; afterwards: k2[t] * exp2(gc[t] - gc[r0(t)])
  alignas(16) float qxv[64 * E];     // q2[t] * exp2(gc[t] - gc[r0(t)])
  float gc2[64 * ES], k2[64 * ES], q2[64 * ES];
  float r1[64 * ES], c1[64 * ES], r2[64 * ES], dgc[64 * ES], drr[64 * ES];
  float part[2][4][64 * ES];         // per column quarter partial sums
  float browp[4][64];
  float beta[64], brow[64], bcol[64];
  uint64_t bar_load, bar_mma;
  uint32_t tmem_base;
  int abort;
  int steep;                         // set when a 16-row block decays by more than 2^-100: the direct decay path is taken
};

template <int E>
__global__ void __launch_bounds__(MAT_THREADS, 1)
mat_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_q,
           const __grid_constant__ CUtensorMap map_do, const __grid_constant__ CUtensorMap map_du,
           const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_u,
           const __grid_constant__ CUtensorMap map_dk, const __grid_constant__ CUtensorMap map_dq, MatParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  using SM = MatSmem<E>;
  SM& sm = *reinterpret_cast<SM*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int ES = SM::ES;
  constexpr float LOG2E = 1.4426950408889634f;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cq = warp >> 2;                                // column quarter
  const int r = (warp & 3) * 32 + lane;                    // tensor-memory lane = matrix row
  const bool krow = r < 64;
  const int t = r & 63;
  const int s0 = cq * 16;
  // The CTA is persistent (one per SM): it walks the items blockIdx.x, blockIdx.x + gridDim.x, ... and keeps its barriers
  // and its tensor memory.  Both barriers complete an even number of phases per item (two loads, four MMA groups), so
  // every item starts at parity zero.
  const int64_t n_items = static_cast<int64_t>(p.B) * p.NC * p.H;
  const int warp_u = __shfl_sync(0xffffffffu, warp, 0);   // warp index as a warp-uniform value
  if (warp_u == 1 && elect_one()) {
    mbar_init(&sm.bar_load, 1);
    mbar_init(&sm.bar_mma, 1);
    mbar_fence_init();
    sm.abort = 0;
  }
  __syncwarp();
  if (warp_u == 0) { tmem_alloc(&sm.tmem_base, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = __shfl_sync(0xffffffffu, sm.tmem_base, 0);
  const uint32_t tmem_row = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
  WaitCtl ctl{&sm.abort, p.status};

  for (int64_t item = blockIdx.x; item < n_items; item += gridDim.x) {
  // (items fit in 32 bits, the entry point checks that: 64-bit divisions are a few hundred cycles each on this machine)
  const int item32 = static_cast<int>(item);
  const int h = item32 % p.H, n = (item32 / p.H) % p.NC;
  const int b = item32 / (p.H * p.NC);
  int t0 = n * CHUNK, rows = CHUNK;
  if (p.cmap != nullptr) {
    t0 = p.cmap[n];
    rows = p.cmap[p.NC + n];
    if (rows <= 0) continue;                               // unused tail of the chunk map (the same for every thread)
    if (t0 < 0 || rows > CHUNK || t0 + rows > p.T) {
      if (tid == 0) atomicCAS(p.status, DEV_OK, DEV_BAD_CHUNK_MAP);
      continue;
    }
  }
  // One thread of the second warp sends the tile loads off at once; everybody else is already requesting its global
  // inputs.  (The previous item's stores from these buffers were waited for by the same thread.)
  const int crow = static_cast<int>(item) * 64;           // first row of this item in the chunk-layout tensors
  if (warp_u == 1 && elect_one()) {
    sm.steep = 0;
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
  __syncwarp();
  // Every global value this thread needs later is requested here, in one batch, from clamped (always valid) addresses,
  // and masked when it is used: a load that waits until its consumer is reached costs a full memory round trip, which
  // under the streaming load of the other blocks is microseconds.
  const int64_t tok = static_cast<int64_t>(b) * p.T + t0;
  constexpr int GATE_ITERS = (64 * E + MAT_THREADS - 1) / MAT_THREADS;
  constexpr int NV_MAX = 8;                                // value blocks of the reverse recurrence (4 or 8)
  float da_in[GATE_ITERS], dc_in[GATE_ITERS];              // row-sum gradients of the state-gradient kernel, used at the end
  const float dd_in = __ldg(p.dd + item * E + min(warp, E - 1));   // warp e adds the chunk-end term of gate column e
  const float beta_in = __ldg(p.beta + (tok + min(tid & 63, rows - 1)) * p.H + h);
  {
    float gc_in[GATE_ITERS], k2_in[GATE_ITERS], q2_in[GATE_ITERS], dr_in[GATE_ITERS][NV_MAX];
#pragma unroll
    for (int it = 0; it < GATE_ITERS; ++it) {
      const int idx = min(tid + it * MAT_THREADS, 64 * E - 1);
      const int rr = idx / E, e = idx % E;
      const int64_t off = ((tok + min(rr, rows - 1)) * p.H + h) * E + e;
      gc_in[it] = __ldg(p.gc + item * gate_item_floats(E) + idx);
      k2_in[it] = __ldg(p.k2 + off);
      q2_in[it] = __ldg(p.q2 + off);
      da_in[it] = __ldg(p.da + item * (64 * E) + idx);
      dc_in[it] = __ldg(p.dc + item * (64 * E) + idx);
      const float* drp = p.dr + (item * p.NV * 64 + rr) * E + e;   // value block v is 64 * E floats further on
#pragma unroll
      for (int v = 0; v < 4; ++v) dr_in[it][v] = __ldg(drp + v * (64 * E));
      if (p.NV > 4) {                                      // four or eight value blocks: the same for every thread
#pragma unroll
        for (int v = 4; v < NV_MAX; ++v) dr_in[it][v] = __ldg(drp + v * (64 * E));
      } else {
#pragma unroll
        for (int v = 4; v < NV_MAX; ++v) dr_in[it][v] = 0.f;
      }
    }
#pragma unroll
    for (int it = 0; it < GATE_ITERS; ++it) {
      const int idx = tid + it * MAT_THREADS;
      if (idx < 64 * E) {
        const int rr = idx / E, e = idx % E;
        const bool ok = rr < rows;
        sm.gc2[rr * ES + e] = gc_in[it] * LOG2E;
        sm.k2[rr * ES + e] = ok ? k2_in[it] : 0.f;
        sm.q2[rr * ES + e] = ok ? q2_in[it] : 0.f;
        float drv = 0.f;                                   // summed over the value blocks in index order
#pragma unroll
        for (int v = 0; v < NV_MAX; ++v) drv += (v < p.NV) ? dr_in[it][v] : 0.f;
        sm.drr[rr * ES + e] = drv;
      }
    }
  }
  if (tid < 64) sm.beta[tid] = (tid < rows) ? beta_in : 0.f;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  // ---- G1, G2 ----------------------------------------------------------------------------------------------------
  mbar_wait(&sm.bar_load, 0, ctl, DEV_TIMEOUT_LOAD);
  if (warp_u == 0 && elect_one()) {
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
  __syncwarp();                                           // the other lanes must not run ahead into a spin wait
  // Decay tables, built while G1 and G2 run.  With r0(s) the first row of s's 16-row block,
  //   exp2(gc[t] - gc[s]) = exp2(gc[t] - gc[r0(s)]) * exp2(gc[r0(s)] - gc[s])        for every t >= s:
  // a factor that depends on t and on the column block only (E exponentials per thread and block) and a factor that
  // depends on s only (a table).  The second exponent is positive but bounded by the decay inside one block; when a
  // block decays by more than 2^-100 (a flush of the first factor could then hide a product of order one) the whole
  // CTA takes the direct path with one exponential per (t, s, e) instead.
  //   Hd[s][e] = exp2(gc[r0(s)][e] - gc[s][e]) * k2[s][e]          Xd[t][e] = exp2(gc[t][e] - gc[r0(t)][e])
  for (int idx = tid; idx < 64 * E; idx += MAT_THREADS) {
    const int rr = idx / E, e = idx % E, o = rr * ES + e;
    const float up = sm.gc2[(rr & ~15) * ES + e] - sm.gc2[o];    // >= 0 when gc does not increase
    // too steep, NaN, or not monotone (a log gate above zero makes gc rise from one row to the next: the factorised form,
    // which clamps its first factor at one, would then be wrong for rows of later blocks)
    if (!(up <= 100.f) || up < 0.f || (rr > 0 && sm.gc2[o] > sm.gc2[o - ES])) sm.steep = 1;
    sm.hkv[idx] = mexp2(up) * sm.k2[o];
    sm.qxv[idx] = sm.q2[o] * mexp2(-up);
  }
  uint32_t mma_phase = 0;
  mbar_wait_spin(&sm.bar_mma, mma_phase & 1, ctl, DEV_TIMEOUT_MMA);
  ++mma_phase;
  tc_fence_after();
  float pr[16];                                            // Pkk (key rows) / Pqk (query rows), this thread's 16 columns
  float gr[16];                                            // dA' (key rows) / dPm' (query rows)
  tmem_ld<16>(tmem_row + s0, pr);
  tmem_ld<16>(tmem_row + 64 + (krow ? 0 : 64) + s0, gr);
  tmem_wait_ld();
  tc_fence_before();
  __syncthreads();                                         // dudo and wu are dead: a5, dmp, dm take their place

  float my2[E], mygc[E];
#pragma unroll
  for (int e = 0; e < E; ++e) {
    my2[e] = krow ? sm.k2[t * ES + e] : sm.q2[t * ES + e];
    mygc[e] = sm.gc2[t * ES + e];
  }
  const bool fast = sm.steep == 0;                         // block-uniform
  auto table_row = [&](const float* tab, int row, float* out) {   // E floats of a dense table row (the same row for the whole warp)
    if constexpr (E % 4 == 0) {
#pragma unroll
      for (int e = 0; e < E; e += 4) {
        const float4 x = *reinterpret_cast<const float4*>(tab + row * E + e);
        out[e] = x.x; out[e + 1] = x.y; out[e + 2] = x.z; out[e + 3] = x.w;
      }
    } else {
#pragma unroll
      for (int e = 0; e < E; ++e) out[e] = tab[row * E + e];
    }
  };
  const int warp_tmin = (warp & 1) ? 32 : 0;               // smallest row index t in this warp
  const uint32_t a5 = smem_u32(sm.u1.a5);
  const int warp_tmax = (warp & 1) ? 63 : 31;              // largest row index t in this warp
  // From here to the barrier before G5 the two halves of the CTA run independent chains and synchronise among
  // themselves only (named barriers of 256 threads): the key-row warps carry dA -> G3 -> Y -> G4 -> dL, the query-row
  // warps the Mp-side mask gradients.  Neither waits for the other's long loops.
  auto half_sync = [&]() {
    if (krow) asm volatile("bar.sync 1, 256;" ::: "memory"); else asm volatile("bar.sync 2, 256;" ::: "memory");
  };

  if (!krow) {
    // ================================ query-row chain ================================
    // query row t, columns s0..s0+15: X -> a5 (row 64+t and, transposed, column 64+t), dmp, partial r1
    const float live = (t < rows) ? 1.f : 0.f;
    float r1v[E];
#pragma unroll
    for (int e = 0; e < E; ++e) r1v[e] = 0.f;
    float xrow[16];
    if (fast) {
      float F[E], G[E], accr[E];
#pragma unroll
      for (int e = 0; e < E; ++e) {
        F[e] = mexp2(fminf(mygc[e] - sm.gc2[s0 * ES + e], 0.f));   // rows above the block (masked below) would give > 0
        G[e] = my2[e] * F[e];
        accr[e] = 0.f;
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int s = s0 + j;
        float x = 0.f, dmpv = 0.f;
        if (s0 <= warp_tmax) {
          float hk[E];
          table_row(sm.hkv, s, hk);
          float mp = 0.f;
#pragma unroll
          for (int e = 0; e < E; ++e) mp = fmaf(G[e], hk[e], mp);
          const float in = (s <= t) ? p.scale * gr[j] : 0.f;
          x = in * mp;
          dmpv = live * in * pr[j];
#pragma unroll
          for (int e = 0; e < E; ++e) accr[e] = fmaf(dmpv, hk[e], accr[e]);
        }
        xrow[j] = x;
        sm.u2.f.dmp[midx(t, s)] = dmpv;
      }
#pragma unroll
      for (int e = 0; e < E; ++e) r1v[e] = F[e] * accr[e];
    } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int s = s0 + j;
      float x = 0.f, dmpv = 0.f;
      if (s0 <= warp_tmax && s <= t) {
        float dec[E];
        float mp = 0.f;
#pragma unroll
        for (int e = 0; e < E; ++e) {
          dec[e] = mexp2(mygc[e] - sm.gc2[s * ES + e]) * sm.k2[s * ES + e];
          mp = fmaf(my2[e], dec[e], mp);
        }
        x = p.scale * mp * gr[j];
        dmpv = live * p.scale * pr[j] * gr[j];
#pragma unroll
        for (int e = 0; e < E; ++e) r1v[e] = fmaf(dmpv, dec[e], r1v[e]);
      }
      xrow[j] = x;
      sm.u2.f.dmp[midx(t, s)] = dmpv;
    }
    }
    const uint32_t rowbase = a5 + ((64 + t) >> 3) * 128 + (t & 7) * 16;
#pragma unroll
    for (int jb = 0; jb < 2; ++jb) {
      st_shared_v4(rowbase + (2 * cq + jb) * 2048, pack_bf16(xrow[jb * 8], xrow[jb * 8 + 1]), pack_bf16(xrow[jb * 8 + 2], xrow[jb * 8 + 3]),
                   pack_bf16(xrow[jb * 8 + 4], xrow[jb * 8 + 5]), pack_bf16(xrow[jb * 8 + 6], xrow[jb * 8 + 7]));
      st_shared_v4(rowbase + (8 + 2 * cq + jb) * 2048, 0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int e = 0; e < E; ++e) sm.part[1][cq][t * ES + e] = r1v[e];
    half_sync();
    // r1 = sum of the four partials (256 query-row threads over the 64*E entries)
    for (int idx = cq * 64 + t; idx < 64 * E; idx += 256) {
      const int o = (idx / E) * ES + idx % E;
      sm.r1[o] = (sm.part[1][0][o] + sm.part[1][1][o]) + (sm.part[1][2][o] + sm.part[1][3][o]);
    }
    half_sync();                                           // part[1] is free again, dmp complete
    // query thread (64+s, cq): partial c1[s,e] over t' in quarter cq: dmp[t',s] exp(gc[t']-gc[s]) q2[t',e]
    {
      const int s = t;
      float c1v[E];
#pragma unroll
      for (int e = 0; e < E; ++e) c1v[e] = 0.f;
      if (fast) {
        // the same sixteen rows t' for every lane (dmp is zero above the diagonal); nothing to do where the whole warp
        // lies below the quarter
        if (s0 + 15 >= warp_tmin) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int tt = s0 + j;
            const float dv = sm.u2.f.dmp[midx(tt, s)];
            float qx[E];
            table_row(sm.qxv, tt, qx);
#pragma unroll
            for (int e = 0; e < E; ++e) c1v[e] = fmaf(dv, qx[e], c1v[e]);
          }
        }
        if (s0 + 15 >= s) {
#pragma unroll
          for (int e = 0; e < E; ++e) c1v[e] *= mexp2(sm.gc2[s0 * ES + e] - mygc[e]);
        }
      } else {
        for (int tt = max(s, s0); tt < s0 + 16; ++tt) {
          const float dv = sm.u2.f.dmp[midx(tt, s)];
  #pragma unroll
          for (int e = 0; e < E; ++e)
            c1v[e] = fmaf(dv * sm.q2[tt * ES + e], mexp2(sm.gc2[tt * ES + e] - mygc[e]), c1v[e]);
        }
      }
#pragma unroll
      for (int e = 0; e < E; ++e) sm.part[1][cq][s * ES + e] = c1v[e];
    }
    mma_phase += 2;                                        // G3 and G4 complete without the query rows watching
  } else {
    // ================================ key-row chain ================================
    // key row t, columns s0..s0+15: dA = dA' diag(beta) -> operand image; dA' * A -> column sums
    {
      const uint32_t apr = smem_u32(sm.ap) + (t >> 3) * 128 + (t & 7) * 16;
      const uint32_t dar = smem_u32(sm.da) + (t >> 3) * 128 + (t & 7) * 16;
#pragma unroll
      for (int jb = 0; jb < 2; ++jb) {
        uint32_t aw[4];
        asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(aw[0]), "=r"(aw[1]), "=r"(aw[2]), "=r"(aw[3]) : "r"(apr + (2 * cq + jb) * 2048));
        float dav[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const int j = jb * 8 + c, s = s0 + j;
          const float a_ts = (c & 1) ? bf16_hi(aw[c >> 1]) : bf16_lo(aw[c >> 1]);
          sm.daa[midx(t, s)] = gr[j] * a_ts;
          dav[c] = gr[j] * sm.beta[s];
        }
        st_shared_v4(dar + (2 * cq + jb) * 1024, pack_bf16(dav[0], dav[1]), pack_bf16(dav[2], dav[3]), pack_bf16(dav[4], dav[5]),
                     pack_bf16(dav[6], dav[7]));
      }
    }
    fence_async_smem();
    tc_fence_before();
    half_sync();

    // ---- G3: Y = A^T dA ----
    if (warp_u == 0 && elect_one()) {
      tc_fence_after();
      const uint64_t da = make_desc(smem_u32(sm.ap), 128, 2048, LAYOUT_PLAIN);     // A^T, MN-major
      const uint64_t db = make_desc(smem_u32(sm.da), 128, 1024, LAYOUT_PLAIN);     // dA (K = t, N = s), MN-major
      constexpr uint32_t idesc = make_idesc(128, 64, 1, 1);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) umma_bf16(tmem + 192, desc_advance(da, kk * 256), desc_advance(db, kk * 256), idesc, kk > 0);
      umma_commit(&sm.bar_mma);
    }
    __syncwarp();                                          // the other lanes must not run ahead into a spin wait
    // meanwhile: dbeta_col[s] = sum_t dA'[t,s] A[t,s] (the 64 key-row threads of the last column quarter)
    if (cq == 3) {
      const int s = t;
      float acc = 0.f;
      for (int tt = 0; tt < 64; ++tt) acc += sm.daa[midx(tt, s)];
      sm.bcol[s] = acc;
    }
    mbar_wait_spin(&sm.bar_mma, mma_phase & 1, ctl, DEV_TIMEOUT_MMA);
    ++mma_phase;
    tc_fence_after();
    {
      float yr[16];
      tmem_ld<16>(tmem_row + 192 + s0, yr);
      tmem_wait_ld();
      const uint32_t yb = smem_u32(sm.y) + (t >> 3) * 128 + (t & 7) * 16;
#pragma unroll
      for (int jb = 0; jb < 2; ++jb)
        st_shared_v4(yb + (2 * cq + jb) * 1024, pack_bf16(yr[jb * 8], yr[jb * 8 + 1]), pack_bf16(yr[jb * 8 + 2], yr[jb * 8 + 3]),
                     pack_bf16(yr[jb * 8 + 4], yr[jb * 8 + 5]), pack_bf16(yr[jb * 8 + 6], yr[jb * 8 + 7]));
    }
    fence_async_smem();
    tc_fence_before();
    half_sync();

    // ---- G4: dp = Y A^T ----
    if (warp_u == 0 && elect_one()) {
      tc_fence_after();
      const uint64_t da = make_desc(smem_u32(sm.y), 1024, 128, LAYOUT_PLAIN);      // Y, K-major
      const uint64_t db = make_desc(smem_u32(sm.ap), 2048, 128, LAYOUT_PLAIN);     // B[k][j] = A[j][k]: A rows as N, K-major
      constexpr uint32_t idesc = make_idesc(128, 64, 0, 0);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) umma_bf16(tmem + 256, desc_advance(da, kk * 2048), desc_advance(db, kk * 4096), idesc, kk > 0);
      umma_commit(&sm.bar_mma);
    }
    __syncwarp();                                          // the other lanes must not run ahead into a spin wait
    mbar_wait_spin(&sm.bar_mma, mma_phase & 1, ctl, DEV_TIMEOUT_MMA);
    ++mma_phase;
    tc_fence_after();
    // ap, da, y and daa (48 KB in a row) are dead from here on: the state part of dK, dQ (32 KB bf16 image written by
    // the state-gradient kernel) is fetched into their place now, so that its HBM round trip runs under the remaining
    // phases.  (The column sums over daa were finished before the barrier that preceded G4.)
    if (warp_u == 0 && elect_one()) {
      mbar_expect_tx(&sm.bar_load, 32768);
      bulk_load(sm.ap, reinterpret_cast<const uint8_t*>(p.dkq) + item * 32768, 32768, &sm.bar_load);
    }
    __syncwarp();
    // Pull the inputs of this CTA's next item into L2: its prologue, which nothing on this SM overlaps, then waits for L2
    // instead of for HBM.
    if (warp_u == 1) {
      const int64_t item2 = item + gridDim.x;              // this CTA's next item
      if (item2 < n_items) {
        const int i2 = static_cast<int>(item2);
        const int h2 = i2 % p.H, n2 = (i2 / p.H) % p.NC;
        const int b2 = i2 / (p.H * p.NC);
        int t2 = n2 * CHUNK, rows2 = CHUNK;
        if (p.cmap != nullptr) { t2 = p.cmap[n2]; rows2 = p.cmap[p.NC + n2]; }
        if (rows2 > 0 && rows2 <= CHUNK && t2 >= 0 && t2 + rows2 <= p.T) {
          if (lane == 0) {
            const int crow2 = static_cast<int>(item2) * 64;
            for (int col = 0; col < 128; col += 64) {
              tma_prefetch_4d(&map_k, col, h2, t2, b2);
              tma_prefetch_4d(&map_q, col, h2, t2, b2);
              tma_prefetch_4d(&map_do, col, h2, t2, b2);
              tma_prefetch_4d(&map_du, col, 0, crow2, 0);
              tma_prefetch_4d(&map_w, col, 0, crow2, 0);
              tma_prefetch_4d(&map_u, col, 0, crow2, 0);
            }
            bulk_prefetch(p.AP + item2 * (128 * 64), 16384);
            bulk_prefetch(reinterpret_cast<const uint8_t*>(p.dkq) + item2 * 32768, 32768);
            bulk_prefetch(p.gc + item2 * gate_item_floats(E), 64 * E * 4);
            bulk_prefetch(p.da + item2 * (64 * E), 64 * E * 4);
            bulk_prefetch(p.dc + item2 * (64 * E), 64 * E * 4);
            bulk_prefetch(p.dr + item2 * p.NV * (64 * E), static_cast<uint32_t>(p.NV) * 64 * E * 4);
          }
          const int64_t tok2 = static_cast<int64_t>(b2) * p.T + t2;
          for (int rr = lane; rr < rows2; rr += 32) {
            const int64_t ro = (tok2 + rr) * p.H + h2;
            prefetch_l2(p.k2 + ro * E);
            prefetch_l2(p.q2 + ro * E);
            if (E > 8) { prefetch_l2(p.k2 + ro * E + 8); prefetch_l2(p.q2 + ro * E + 8); }
          }
        }
      }
    }
    {
      // key row t, columns s0..s0+15: dL, partial dbeta_row, dm, partial r2, and dPkk + dPkk^T into a5[0..63][0..63]
      float dpr[16];
      tmem_ld<16>(tmem_row + 256 + s0, dpr);
      tmem_wait_ld();
      const float bt = sm.beta[t];
      float brow = 0.f;
      float r2v[E];
#pragma unroll
      for (int e = 0; e < E; ++e) r2v[e] = 0.f;
      float dpk[16];                                       // dPkk, this thread's 16 columns of row t
#pragma unroll
      for (int j = 0; j < 16; ++j) dpk[j] = 0.f;
      if (fast) {
        float F[E], G[E], accr[E];
#pragma unroll
        for (int e = 0; e < E; ++e) {
          F[e] = mexp2(fminf(mygc[e] - sm.gc2[s0 * ES + e], 0.f));
          G[e] = my2[e] * F[e];
          accr[e] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int s = s0 + j;
          float dmv = 0.f;
          if (s0 <= warp_tmax) {
            float hk[E];
            table_row(sm.hkv, s, hk);
            float m = 0.f;
#pragma unroll
            for (int e = 0; e < E; ++e) m = fmaf(G[e], hk[e], m);
            const float dl = (s < t) ? -dpr[j] : 0.f;
            brow = fmaf(dl * pr[j], m, brow);
            dmv = bt * dl * pr[j];
            dpk[j] = bt * dl * m;                          // zero on and above the diagonal
#pragma unroll
            for (int e = 0; e < E; ++e) accr[e] = fmaf(dmv, hk[e], accr[e]);
          }
          sm.u2.f.dm[midx(t, s)] = dmv;
        }
#pragma unroll
        for (int e = 0; e < E; ++e) r2v[e] = F[e] * accr[e];
      } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int s = s0 + j;
        float dmv = 0.f;
        if (s0 <= warp_tmax && s < t) {
          float dec[E];
          float m = 0.f;
#pragma unroll
          for (int e = 0; e < E; ++e) {
            dec[e] = mexp2(mygc[e] - sm.gc2[s * ES + e]) * sm.k2[s * ES + e];
            m = fmaf(my2[e], dec[e], m);
          }
          const float dl = -dpr[j];
          brow = fmaf(dl * pr[j], m, brow);
          dmv = bt * dl * pr[j];
          dpk[j] = bt * dl * m;
#pragma unroll
          for (int e = 0; e < E; ++e) r2v[e] = fmaf(dmv, dec[e], r2v[e]);
        }
        sm.u2.f.dm[midx(t, s)] = dmv;
      }
      }
      const uint32_t rowbase = a5 + (t >> 3) * 128 + (t & 7) * 16;
#pragma unroll
      for (int jb = 0; jb < 2; ++jb) {
        st_shared_v4(rowbase + (2 * cq + jb) * 2048, pack_bf16(dpk[jb * 8], dpk[jb * 8 + 1]), pack_bf16(dpk[jb * 8 + 2], dpk[jb * 8 + 3]),
                     pack_bf16(dpk[jb * 8 + 4], dpk[jb * 8 + 5]), pack_bf16(dpk[jb * 8 + 6], dpk[jb * 8 + 7]));
        st_shared_v4(rowbase + (8 + 2 * cq + jb) * 2048, 0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int e = 0; e < E; ++e) sm.part[0][cq][t * ES + e] = r2v[e];
      sm.browp[cq][t] = brow;
    }
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();

  // ---- G5: [dK;dQ] = (P + P^T) [K;Q] with P = [[dPkk, 0], [X, 0]] ------------------------------------------------------
  // The image of P is written by rows only; its transpose is the same image read MN-major.
  if (warp_u == 0 && elect_one()) {
    tc_fence_after();
    const uint64_t da = make_desc(a5, 2048, 128, LAYOUT_PLAIN);                  // P, K-major: only columns 0..63 are not zero
    const uint64_t dat = make_desc(a5, 128, 2048, LAYOUT_PLAIN);                 // P^T, MN-major
    const uint64_t db = make_desc(smem_u32(sm.kq), 16384, 1024, LAYOUT_SW128);   // (K = token rows, N = d), MN-major
    constexpr uint32_t idesc = make_idesc(128, 128, 0, 1), idesc_t = make_idesc(128, 128, 1, 1);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) umma_bf16(tmem, desc_advance(da, kk * 4096), desc_advance(db, kk * 2048), idesc, kk > 0);
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) umma_bf16(tmem, desc_advance(dat, kk * 256), desc_advance(db, kk * 2048), idesc_t, true);
    umma_commit(&sm.bar_mma);
  }
  __syncwarp();                                           // the other lanes must not run ahead into a spin wait
  // sums of the partials written before the barrier: r2 (key-row chain) and c1 (query-row chain)
  for (int idx = tid; idx < 64 * E; idx += MAT_THREADS) {
    const int o = (idx / E) * ES + idx % E;
    sm.r2[o] = (sm.part[0][0][o] + sm.part[0][1][o]) + (sm.part[0][2][o] + sm.part[0][3][o]);
    sm.c1[o] = (sm.part[1][0][o] + sm.part[1][1][o]) + (sm.part[1][2][o] + sm.part[1][3][o]);
    // the first decay table has been read for the last time: the column sums below want k2[t] exp2(gc[t] - gc[r0(t)])
    sm.hkv[idx] = sm.k2[o] * mexp2(sm.gc2[o] - sm.gc2[((idx / E) & ~15) * ES + idx % E]);
  }
  if (tid < 64) sm.brow[tid] = (sm.browp[0][tid] + sm.browp[1][tid]) + (sm.browp[2][tid] + sm.browp[3][tid]);
  __syncthreads();
  {
    // thread (s = t, cq): partial c2[s,e] = sum over t' > s of dm[t',s] exp(gc[t']-gc[s]) k2[t',e]; the key-row thread takes
    // the first eight t' of quarter cq, the query-row thread of the same (t, cq) the other eight
    float c2v[E];
#pragma unroll
    for (int e = 0; e < E; ++e) c2v[e] = 0.f;
    const int lo = s0 + (krow ? 0 : 8);
    if (fast) {
      if (lo + 7 > warp_tmin) {                            // dm is zero on and above the diagonal
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int tt = lo + j;
          const float dv = sm.u2.f.dm[midx(tt, t)];
          float kx[E];
          table_row(sm.hkv, tt, kx);
#pragma unroll
          for (int e = 0; e < E; ++e) c2v[e] = fmaf(dv, kx[e], c2v[e]);
        }
      }
      if (s0 + 15 > t) {
#pragma unroll
        for (int e = 0; e < E; ++e) c2v[e] *= mexp2(sm.gc2[s0 * ES + e] - mygc[e]);
      }
    } else {
      for (int tt = max(t + 1, lo); tt < lo + 8; ++tt) {
        const float dv = sm.u2.f.dm[midx(tt, t)];
  #pragma unroll
        for (int e = 0; e < E; ++e)
          c2v[e] = fmaf(dv * sm.k2[tt * ES + e], mexp2(sm.gc2[tt * ES + e] - mygc[e]), c2v[e]);
      }
    }
#pragma unroll
    for (int e = 0; e < E; ++e) sm.part[krow ? 0 : 1][cq][t * ES + e] = c2v[e];
  }
  __syncthreads();
  // gate gradients: one thread per (row, gate column)
#pragma unroll
  for (int it = 0; it < GATE_ITERS; ++it) {
    const int idx = tid + it * MAT_THREADS;
    if (idx < 64 * E) {
      const int rr = idx / E, e = idx % E, o = rr * ES + e;
      const float c2e = ((sm.part[0][0][o] + sm.part[1][0][o]) + (sm.part[0][1][o] + sm.part[1][1][o])) +
                        ((sm.part[0][2][o] + sm.part[1][2][o]) + (sm.part[0][3][o] + sm.part[1][3][o]));
      const float gcv = sm.gc2[o], gl = sm.gc2[63 * ES + e];
      const float eg = mexp2(gcv), egr = mexp2(gl - gcv);
      const float k2v = sm.k2[o], q2v = sm.q2[o];
      const float dav = da_in[it], dcv = dc_in[it];
      const float drv = sm.drr[o], r1e = sm.r1[o], c1e = sm.c1[o], r2e = sm.r2[o];
      if (rr < rows) {
        const int64_t off = ((tok + rr) * p.H + h) * E + e;
        p.dk2[off] = dav * eg + drv * egr + c1e + r2e + c2e;
        p.dq2[off] = dcv * p.scale * eg + r1e;
      }
      sm.dgc[o] = dav * (k2v * eg) + dcv * (p.scale * q2v * eg) - drv * (k2v * egr) + q2v * r1e + k2v * (r2e - c1e - c2e);
      sm.drr[o] = drv * (k2v * egr);                        // dr*r, summed over the rows below
    }
  }
  if (tid < 64 && tid < rows) p.dbeta[(tok + tid) * p.H + h] = sm.bcol[tid] + sm.brow[tid];
  __syncthreads();
  // dg = reverse inclusive cumulative sum of dgc over the chunk, one warp per gate column; the last row first takes the
  // chunk-end terms sum_t dr*r + dd*exp(gL)
  static_assert(E <= MAT_THREADS / 32, "one warp per gate column");
  for (int e = warp; e < E; e += MAT_THREADS / 32) {
    float tot = sm.drr[lane * ES + e] + sm.drr[(lane + 32) * ES + e];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
    float v1 = sm.dgc[(63 - lane) * ES + e], v0 = sm.dgc[(31 - lane) * ES + e];      // lane l: rows 63-l and 31-l
    if (lane == 0) v1 += tot + dd_in * mexp2(sm.gc2[63 * ES + e]);
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

  // ---- dk, dq: this thread's row, 32 of the 128 columns ------------------------------------------------------------
  mbar_wait_spin(&sm.bar_mma, mma_phase & 1, ctl, DEV_TIMEOUT_MMA);
  ++mma_phase;
  tc_fence_after();
  {
    float a[32];
    tmem_ld<32>(tmem_row + cq * 32, a);
    tmem_wait_ld();
    mbar_wait(&sm.bar_load, 1, ctl, DEV_TIMEOUT_LOAD);     // state part: image [column / 8][row][column % 8]
    // Sum with the state part, round once, and stage the 128x128 bf16 result in the [K;Q] buffer (dead since G5) so
    // that it can leave as whole 256-byte rows: a thread owns one row and 32 columns, and storing those directly would
    // scatter every warp store over 32 rows.  16-byte chunks are XOR-swizzled with the row so that neither the staging
    // stores (fixed chunk, 32 rows) nor the row reads (one row, 32 lanes) meet a bank twice.
    // A whole chunk leaves by TMA instead: four 64 x 64 tiles (dk | dq, column half) staged in the 128-byte swizzle of the
    // tensor maps.  (A chunk cut short by a document end may not: the rows behind it belong to the next document.)
    const uint32_t xb = smem_u32(sm.ap) + (cq * 4) * 2048 + r * 16;
    const bool whole = rows == CHUNK;
    const uint32_t stage = whole ? smem_u32(sm.kq) + ((r >> 6) * 2 + (cq >> 1)) * 8192 + t * 128 : smem_u32(sm.kq) + r * 256;
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      uint32_t x[4];
      asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(x[0]), "=r"(x[1]), "=r"(x[2]), "=r"(x[3]) : "r"(xb + (j >> 3) * 2048));
      st_shared_v4(stage + (whole ? ((((cq & 1) * 4 + (j >> 3)) ^ (t & 7)) << 4) : (((cq * 4 + (j >> 3)) ^ (r & 15)) << 4)),
                   pack_bf16(a[j] + bf16_lo(x[0]), a[j + 1] + bf16_hi(x[0])), pack_bf16(a[j + 2] + bf16_lo(x[1]), a[j + 3] + bf16_hi(x[1])),
                   pack_bf16(a[j + 4] + bf16_lo(x[2]), a[j + 5] + bf16_hi(x[2])), pack_bf16(a[j + 6] + bf16_lo(x[3]), a[j + 7] + bf16_hi(x[3])));
    }
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  if (rows == CHUNK) {
    if (warp_u == 1 && elect_one()) {
      tma_store_4d(&map_dk, sm.kq, 0, h, t0, b);
      tma_store_4d(&map_dk, sm.kq + 8192, 64, h, t0, b);
      tma_store_4d(&map_dq, sm.kq + 16384, 0, h, t0, b);
      tma_store_4d(&map_dq, sm.kq + 24576, 64, h, t0, b);
      bulk_commit_group();
      bulk_wait_group_read();                              // the staging buffer must outlive the copies: the next item loads into it
    }
    __syncwarp();
  } else {
    // rows 0..63 -> dk, rows 64..127 -> dq; warp w stores rows w, w + 16, ...: one coalesced 256-byte row per instruction
    for (int rr = warp; rr < 128; rr += MAT_THREADS / 32) {
      const int tt = rr & 63;
      if (tt < rows) {
        const uint32_t src = smem_u32(sm.kq) + rr * 256 + ((((lane >> 1) ^ (rr & 15)) << 4) | ((lane & 1) << 3));
        uint2 v;
        asm volatile("ld.shared.v2.b32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(src));
        __nv_bfloat16* dst = (rr < 64 ? p.dk : p.dq) + ((tok + tt) * p.H + h) * HEAD + lane * 4;
        *reinterpret_cast<uint2*>(dst) = v;
      }
    }
    __syncthreads();                                       // the staging buffer is read: the next item may load into it
  }
  }   // items
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

}  // namespace tgdn

using namespace tgdn;

template <int E>
static int launch_mat(const CUtensorMap* maps, const MatParams& p, cudaStream_t s) {
  const int smem = static_cast<int>(sizeof(MatSmem<E>)) + 1024;
  static_assert(sizeof(MatSmem<E>) + 1024 <= 232448, "shared memory budget of one CTA exceeded");
  cudaError_t e = cudaFuncSetAttribute(mat_kernel<E>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return tgdn_cuda_error(e);
  const long long items = static_cast<long long>(p.B) * p.NC * p.H;
  mat_kernel<E><<<static_cast<int>(items < p.ahead ? items : p.ahead), MAT_THREADS, smem, s>>>(maps[0], maps[1], maps[2], maps[3], maps[4], maps[5], maps[6], maps[7], p);
  return tgdn_cuda_error(cudaGetLastError());
}

extern "C" int tgdn_bwd_matrix(const void* q, const void* k, const void* dO, const void* dU, const void* W, const void* U,
                               const void* AP, const float* k2, const float* q2, const float* beta, const float* gc,
                               const void* dkq, const float* da, const float* dc, const float* dd, const float* dr,
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
  CUtensorMap maps[8];
  if ((rc = tgdn_make_token_map(&maps[0], k, B, T, H, 64, 64, 1))) return rc;
  if ((rc = tgdn_make_token_map(&maps[1], q, B, T, H, 64, 64, 1))) return rc;
  if ((rc = tgdn_make_token_map(&maps[2], dO, B, T, H, 64, 64, 1))) return rc;
  // chunk-layout tensors are plain (rows, 128) matrices: one batch row, one head
  if ((rc = tgdn_make_token_map(&maps[3], dU, 1, static_cast<int>(crows), 1, 64, 64, 1))) return rc;
  if ((rc = tgdn_make_token_map(&maps[4], W, 1, static_cast<int>(crows), 1, 64, 64, 1))) return rc;
  if ((rc = tgdn_make_token_map(&maps[5], U, 1, static_cast<int>(crows), 1, 64, 64, 1))) return rc;
  if ((rc = tgdn_make_token_map(&maps[6], dk, B, T, H, 64, 64, 1))) return rc;
  if ((rc = tgdn_make_token_map(&maps[7], dq, B, T, H, 64, 64, 1))) return rc;
  MatParams p{k2, q2, beta, gc, static_cast<const __nv_bfloat16*>(AP), static_cast<const __nv_bfloat16*>(dkq), da, dc, dd, dr,
              static_cast<__nv_bfloat16*>(dq), static_cast<__nv_bfloat16*>(dk), dk2, dq2, dg, dbeta, chunk_map,
              B, T, H, NC, 128 / tgdn_value_block(E), scale, tgdn_status_word(), tgdn_sm_count()};
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
