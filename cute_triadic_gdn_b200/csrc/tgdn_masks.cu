// Per-chunk masks of the Triadic GDN: cumulative log decay, the UT transform A and the intra-chunk output operator.
//
// For every (batch, chunk, head) one CTA of 256 threads computes, with K, Q the 64x128 key/query tiles of the chunk:
//   gc[t,e]  = inclusive cumulative sum of the log gate over the chunk (rows past the end of a document add 0)
//   M[t,s]   = sum_e k2[t,e] k2[s,e] exp(gc[t,e]-gc[s,e]) (s <  t),  Mp[t,s] = sum_e q2[t,e] k2[s,e] exp(.) (s <= t)
//   A        = (I + strict_lower(beta_t (K K^T)[t,s] M[t,s]))^-1
//   Pm       = scale * lower(Q K^T * Mp),   PA = Pm A
// and stores gc (f32) followed by the gate factors a = k2 exp(gc), r = k2 exp(gL - gc), c = scale q2 exp(gc), d = exp(gL)
// that the recurrences multiply their rows with (layout in tgdn_kernels.h), the stacked operand image [A; PA] (bf16,
// 128x64) that the forward recurrence multiplies with beta*W, and the Pm image (bf16, 64x64) that the reverse recurrence
// needs.
//
// Replaces cute_triadic_gdn/kernels/sm90_joint_scan.py:21-80 (scan_kernel, forward direction) and
// cute_triadic_gdn/kernels/sm100_joint_masks.py:34-267 (masks_kernel); math as in
// cute_triadic_gdn/ops/gdn_joint.py:36-39, :45-60.
//   * Gram product [K;Q] K^T: one tcgen05 MMA group (M=128, N=64, K=128) on TMA-staged 128B-swizzled tiles.
//   * Mask sums: thread (row, column half) with the half's 8-column blocks interleaved so that the triangle is balanced.
//   * Triangular inverse in f32: four 16x16 diagonal blocks by forward substitution, then the 16->32 and 32->64
//     merges X21 = -X22 (L21 X11) as warp-level mma.sync m16n8k8 products with a 3-term TF32 split (f32-grade accuracy).
//   * PA = Pm A: a second tcgen05 MMA group on the bf16 images of Pm and A that are about to be stored anyway.
#include "tgdn_common.cuh"
#include "tgdn_host.h"
#include "tgdn_kernels.h"

namespace tgdn {

constexpr int MASK_THREADS = 256;

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 64x64 f32 matrix in shared memory, column index XOR-swizzled with the row so that both "lanes along a row" and
// "lanes along a column" accesses are conflict-free.
__device__ __forceinline__ int mat_idx(int i, int j) { return i * 64 + (j ^ (i & 31)); }
__device__ __forceinline__ int t_idx(int k, int j) { return k * 32 + ((j ^ k) & 31); }
__device__ __forceinline__ void st_shared_b16(uint32_t saddr, float v) {      // v is a bf16 value held as f32
  const unsigned short b = __bfloat16_as_ushort(__float2bfloat16_rn(v));
  asm volatile("st.shared.b16 [%0], %1;" ::"r"(saddr), "h"(b) : "memory");
}

// ---- warp-level TF32 products with a 3-term split --------------------------------------------------------------------
__device__ __forceinline__ void tf32_split(float x, uint32_t& hi, uint32_t& lo) {
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hi) : "f"(x));
  const float rest = x - __uint_as_float(hi);
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lo) : "f"(rest));
}
__device__ __forceinline__ void mma_tf32(float* c, const uint32_t* a, const uint32_t* b) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
// c (16x8 tile, standard fragment) += A(16x8) B(8x8) with A(i,k), B(k,j) given as element functors
template <typename FA, typename FB>
__device__ __forceinline__ void mma_step_3x(float* c, FA a_at, FB b_at, int lane) {
  const int gid = lane >> 2, tig = lane & 3;
  uint32_t ah[4], al[4], bh[2], bl[2];
  tf32_split(a_at(gid, tig), ah[0], al[0]);
  tf32_split(a_at(gid + 8, tig), ah[1], al[1]);
  tf32_split(a_at(gid, tig + 4), ah[2], al[2]);
  tf32_split(a_at(gid + 8, tig + 4), ah[3], al[3]);
  tf32_split(b_at(tig, gid), bh[0], bl[0]);
  tf32_split(b_at(tig + 4, gid), bh[1], bl[1]);
  mma_tf32(c, al, bh);
  mma_tf32(c, ah, bl);
  mma_tf32(c, ah, bh);
}

template <int E>
struct MaskSmem {
  // KQ tile (two 64-column blocks of 128 rows x 128 B) while the Gram product runs; L and X afterwards
  union {
    uint8_t kq[32768];
    struct { float L[4096]; float X[4096]; } m;
  } u;
  float Pm[4096];
  float T[1024];
  uint8_t img_ap[16384];   // [A; PA] image (i = row 0..127, j = column), SI = 128, SJ = 2048
  uint8_t img_pm[8192];    // Pm image (i = t, j = s), SI = 128, SJ = 1024; read as 128 rows by the PA product: keep >= 8 KB behind it
  float gc2[64 * E];       // log2-domain cumulative gate
  float k2[64 * E];
  float q2[64 * E];
  float pad[(3 * 64 * E * 4 >= 8192) ? 1 : (8192 - 3 * 64 * E * 4) / 4];
  float beta[64];
  uint64_t bar_load, bar_mma;
  uint32_t tmem_base;
  int abort;
  int steep;               // a 16-row block decays by more than 2^-100 (or gc is not monotone): direct decay path
  // Operands of the mask-sum products (see the kernel), in buffers that are written only after those products are done:
  //   G images: four blocks of (128 rows x KP) bf16, image (i = row, j = k), SI = 128, SJ = 2048, over Pm, T, img_ap
  //   H images: two of (64 rows x KP) bf16, image (i = s, j = k), SI = 128, SJ = 1024, over img_pm
  static constexpr int KP = 2 * E <= 16 ? 16 : 32;         // [hi | lo] halves of the E factors, padded to the MMA's K = 16
  static constexpr int G_BYTES = KP / 8 * 2048, H_BYTES = KP / 8 * 1024;
  __device__ uint8_t* img_g() { return reinterpret_cast<uint8_t*>(Pm); }
  __device__ uint8_t* img_h() { return img_pm; }
  static_assert(4 * G_BYTES <= 16384 + 4096 + 16384 && 2 * H_BYTES <= 8192, "operand images fit the buffers they borrow");
};

// X21 = -X22 (L21 X11) for the diagonal blocks of size 2n (n = 16: two blocks, n = 32: one), one 16x8 tile per warp.
template <int N>
__device__ __forceinline__ void tri_merge_mma(const float* L, float* X, float* T, int warp, int lane) {
  constexpr int NT = N / 8, MT = N / 16, TASKS = (64 / (2 * N)) * MT * NT;      // 4 tasks (N=16) or 8 (N=32)
  const int gid = lane >> 2, tig = lane & 3;
  const int m = warp / (MT * NT), mt = (warp / NT) % MT, nt = warp % NT, r = m * 2 * N;
  if (warp < TASKS) {
    float c[4] = {0.f, 0.f, 0.f, 0.f};
    for (int kb = nt; kb < NT; ++kb)                           // X11 is lower triangular: rows k < column block are zero
      mma_step_3x(c,
                  [&](int i, int k) { return L[mat_idx(r + N + 16 * mt + i, r + 8 * kb + k)]; },
                  [&](int k, int j) { return X[mat_idx(r + 8 * kb + k, r + 8 * nt + j)]; }, lane);
    float* Tm = T + m * 512;
    Tm[t_idx(16 * mt + gid, 8 * nt + 2 * tig)] = c[0];
    Tm[t_idx(16 * mt + gid, 8 * nt + 2 * tig + 1)] = c[1];
    Tm[t_idx(16 * mt + gid + 8, 8 * nt + 2 * tig)] = c[2];
    Tm[t_idx(16 * mt + gid + 8, 8 * nt + 2 * tig + 1)] = c[3];
  }
  __syncthreads();
  if (warp < TASKS) {
    float c[4] = {0.f, 0.f, 0.f, 0.f};
    const float* Tm = T + m * 512;
    for (int kb = 0; kb <= 2 * mt + 1; ++kb)                   // X22 is lower triangular: columns k > row block are zero
      mma_step_3x(c,
                  [&](int i, int k) { return X[mat_idx(r + N + 16 * mt + i, r + N + 8 * kb + k)]; },
                  [&](int k, int j) { return Tm[t_idx(8 * kb + k, 8 * nt + j)]; }, lane);
    X[mat_idx(r + N + 16 * mt + gid, r + 8 * nt + 2 * tig)] = -c[0];
    X[mat_idx(r + N + 16 * mt + gid, r + 8 * nt + 2 * tig + 1)] = -c[1];
    X[mat_idx(r + N + 16 * mt + gid + 8, r + 8 * nt + 2 * tig)] = -c[2];
    X[mat_idx(r + N + 16 * mt + gid + 8, r + 8 * nt + 2 * tig + 1)] = -c[3];
  }
  __syncthreads();
}

template <int E>
__global__ void __launch_bounds__(MASK_THREADS, 2)
masks_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_q, MaskParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  using SM = MaskSmem<E>;
  SM& sm = *reinterpret_cast<SM*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int ch = warp >> 2;                                 // column half (interleaved 8-column blocks)
  const int r = (warp & 3) * 32 + lane;                     // tensor-memory lane = row of [K K^T ; Q K^T]
  const int h = blockIdx.x % p.H, n = (blockIdx.x / p.H) % p.NC, b = blockIdx.x / (p.H * p.NC);
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
  // One thread of the second warp sets the barriers up and sends the tile load off at once; the first warp allocates
  // tensor memory meanwhile; everybody else is already requesting the gate inputs.  The barrier after the gate stores ends
  // all three.
  WaitCtl ctl{&sm.abort, p.status};
  const int warp_u = __shfl_sync(0xffffffffu, warp, 0);   // warp index as a warp-uniform value
  if (warp_u == 1 && elect_one()) {
    mbar_init(&sm.bar_load, 1);
    mbar_init(&sm.bar_mma, 1);
    mbar_fence_init();
    sm.abort = 0;
    sm.steep = 0;
    mbar_expect_tx(&sm.bar_load, 32768);
    tma_load_4d(sm.u.kq, &map_k, &sm.bar_load, 0, h, t0, b);
    tma_load_4d(sm.u.kq + 8192, &map_q, &sm.bar_load, 0, h, t0, b);
    tma_load_4d(sm.u.kq + 16384, &map_k, &sm.bar_load, 64, h, t0, b);
    tma_load_4d(sm.u.kq + 24576, &map_q, &sm.bar_load, 64, h, t0, b);
  }
  __syncwarp();
  if (warp_u == 0) { tmem_alloc(&sm.tmem_base, 128); tmem_relinquish(); }
  for (int i = tid; i < 2 * SM::H_BYTES / 16; i += MASK_THREADS) reinterpret_cast<uint4*>(sm.img_h())[i] = make_uint4(0, 0, 0, 0);

  // gates of the chunk: rows past the document end count as g = 0, k2 = q2 = beta = 0.  All loads are requested first, from
  // clamped (always valid) addresses, and masked when stored: the block pays one memory round trip, not one per iteration.
  const int64_t tok = static_cast<int64_t>(b) * p.T + t0;
  {
    constexpr int GATE_ITERS = (64 * E + MASK_THREADS - 1) / MASK_THREADS;
    float g_in[GATE_ITERS], k2_in[GATE_ITERS], q2_in[GATE_ITERS];
    const float beta_in = __ldg(p.beta + (tok + min(tid & 63, rows - 1)) * p.H + h);
#pragma unroll
    for (int it = 0; it < GATE_ITERS; ++it) {
      const int idx = min(tid + it * MASK_THREADS, 64 * E - 1);
      const int64_t g_off = ((tok + min(idx / E, rows - 1)) * p.H + h) * E + (idx % E);
      g_in[it] = __ldg(p.g + g_off);
      k2_in[it] = __ldg(p.k2 + g_off);
      q2_in[it] = __ldg(p.q2 + g_off);
    }
#pragma unroll
    for (int it = 0; it < GATE_ITERS; ++it) {
      const int idx = tid + it * MASK_THREADS;
      if (idx < 64 * E) {
        const bool ok = idx / E < rows;
        sm.gc2[idx] = ok ? g_in[it] : 0.f;
        sm.k2[idx] = ok ? k2_in[it] : 0.f;
        sm.q2[idx] = ok ? q2_in[it] : 0.f;
      }
    }
    if (tid < 64) sm.beta[tid] = (tid < rows) ? beta_in : 0.f;
  }
  tc_fence_before();
  __syncthreads();                                          // gate values, barriers and the tensor-memory address are visible
  tc_fence_after();
  // inclusive scan over the 64 rows, one warp per gate column
  float* gc_out = p.gc + ((static_cast<int64_t>(b) * p.NC + n) * p.H + h) * gate_item_floats(E);
  for (int e = warp; e < E; e += MASK_THREADS / 32) {
    float v0 = sm.gc2[lane * E + e], v1 = sm.gc2[(lane + 32) * E + e];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float a0 = __shfl_up_sync(0xffffffffu, v0, o), a1 = __shfl_up_sync(0xffffffffu, v1, o);
      if (lane >= o) { v0 += a0; v1 += a1; }
    }
    v1 += __shfl_sync(0xffffffffu, v0, 31);
    gc_out[lane * E + e] = v0;
    gc_out[(lane + 32) * E + e] = v1;
    sm.gc2[lane * E + e] = v0 * LOG2E;
    sm.gc2[(lane + 32) * E + e] = v1 * LOG2E;
  }
  __syncthreads();
  // Mask sums on the tensor core.  With r0(s) the first row of s's 16-row block,
  //   exp2(gc[t] - gc[s]) = exp2(gc[t] - gc[r0(s)]) * exp2(gc[r0(s)] - gc[s])        for every t >= s,
  // so that for the 16 columns of block i
  //   M[t, s] = sum_e G_i[t, e] H[s, e],   G_i[t, e] = x2[t, e] exp2(min(gc[t, e] - gc[16 i, e], 0)),
  //                                         H[s, e]  = k2[s, e] exp2(gc[r0(s), e] - gc[s, e])
  // (x2 = k2 for key rows, q2 for query rows): four products of (128 x E)(E x 16).  Both factors go in as a bf16 pair
  // hi + lo; with K laid out as [hi | lo] two MMAs per block give hi*hi + lo*hi + hi*lo, an error of 2^-16 per term.
  // The exponent of H is positive but bounded by the decay inside one block; when a block decays by more than 2^-100 (a
  // flush of the first factor could then hide a product of order one) the CTA takes one exponential per (t, s, e) instead.
  constexpr int KP = SM::KP;
  {
    const uint32_t hb = smem_u32(sm.img_h());
    for (int idx = tid; idx < 64 * E; idx += MASK_THREADS) {
      const int rr = idx / E, e = idx % E;
      const float up = sm.gc2[(rr & ~15) * E + e] - sm.gc2[idx];   // >= 0 when gc does not increase
      // too steep, NaN, or not monotone: a log gate above zero anywhere in the chunk makes gc rise from one row to the
      // next, and the factorised form (which clamps its first factor at one) would then be wrong for rows of later blocks
      if (!(up <= 100.f) || up < 0.f || (rr > 0 && sm.gc2[idx] > sm.gc2[idx - E])) sm.steep = 1;
      // the gate factors of the recurrences, formed here once instead of by every value block of every recurrence
      {
        const float eg = fast_exp2(sm.gc2[idx]), k2v = sm.k2[idx];
        gc_out[64 * E + idx] = k2v * eg;
        gc_out[128 * E + idx] = k2v * fast_exp2(sm.gc2[63 * E + e] - sm.gc2[idx]);
        gc_out[192 * E + idx] = p.scale * sm.q2[idx] * eg;
        if (idx < 16) gc_out[256 * E + idx] = idx < E ? fast_exp2(sm.gc2[63 * E + idx]) : 0.f;
      }
      const float hv = fast_exp2(up) * sm.k2[idx];
      const float hi = round_bf16(hv), lo = hv - hi;
      const uint32_t row = hb + (rr >> 3) * 128 + (rr & 7) * 16;
      st_shared_b16(row + (e >> 3) * 1024 + (e & 7) * 2, hi);                                    // first image:  [hi | hi]
      st_shared_b16(row + ((E + e) >> 3) * 1024 + ((E + e) & 7) * 2, hi);
      st_shared_b16(row + SM::H_BYTES + (e >> 3) * 1024 + (e & 7) * 2, lo);                      // second image: [lo | 0]
    }
  }
  const int t = r & 63;
  const bool isq = r >= 64;
  {
    float my2[E], mygc[E];
#pragma unroll
    for (int e = 0; e < E; ++e) {
      my2[e] = isq ? sm.q2[t * E + e] : sm.k2[t * E + e];
      mygc[e] = sm.gc2[t * E + e];
    }
#pragma unroll
    for (int ii = 0; ii < 2; ++ii) {
      const int i = 2 * ch + ii;                              // the two column halves of a row share the four blocks
      float vals[KP];
#pragma unroll
      for (int k = 0; k < KP; ++k) vals[k] = 0.f;
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const float g = my2[e] * fast_exp2(fminf(mygc[e] - sm.gc2[(16 * i) * E + e], 0.f));   // rows above the block are masked later
        vals[e] = round_bf16(g);
        vals[E + e] = g - vals[e];
      }
      const uint32_t row = smem_u32(sm.img_g()) + i * SM::G_BYTES + (r >> 3) * 128 + (r & 7) * 16;
#pragma unroll
      for (int kb = 0; kb < KP / 8; ++kb)
        st_shared_v4(row + kb * 2048, pack_bf16(vals[8 * kb], vals[8 * kb + 1]), pack_bf16(vals[8 * kb + 2], vals[8 * kb + 3]),
                     pack_bf16(vals[8 * kb + 4], vals[8 * kb + 5]), pack_bf16(vals[8 * kb + 6], vals[8 * kb + 7]));
    }
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  // Gram product [K;Q] K^T, then the four mask-sum products
  mbar_wait(&sm.bar_load, 0, ctl, DEV_TIMEOUT_LOAD);
  const uint32_t tmem = __shfl_sync(0xffffffffu, sm.tmem_base, 0);
  const uint32_t tmem_row = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
  if (warp_u == 0 && elect_one()) {
    tc_fence_after();
    const uint64_t desc = make_desc(smem_u32(sm.u.kq), 16, 1024, LAYOUT_SW128);
    constexpr uint32_t idesc = make_idesc(128, 64, 0, 0);
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
      umma_bf16(tmem, desc_advance(desc, off), desc_advance(desc, off), idesc, kk > 0);
    }
    constexpr uint32_t idm = make_idesc(128, 16, 0, 0);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint64_t da = make_desc(smem_u32(sm.img_g()) + i * SM::G_BYTES, 2048, 128, LAYOUT_PLAIN);
      const uint64_t db = make_desc(smem_u32(sm.img_h()) + i * 256, 1024, 128, LAYOUT_PLAIN);
#pragma unroll
      for (int kk = 0; kk < KP / 16; ++kk)
        umma_bf16(tmem + 64 + 16 * i, desc_advance(da, kk * 4096), desc_advance(db, kk * 2048), idm, kk > 0);
#pragma unroll
      for (int kk = 0; kk < KP / 16; ++kk)
        umma_bf16(tmem + 64 + 16 * i, desc_advance(da, kk * 4096), desc_advance(db, SM::H_BYTES + kk * 2048), idm, 1);
    }
    umma_commit(&sm.bar_mma);
  }
  __syncwarp();                                           // the other lanes must not run ahead into a spin wait
  mbar_wait_spin(&sm.bar_mma, 0, ctl, DEV_TIMEOUT_MMA);
  tc_fence_after();
  // The KQ tile and the operand images are dead from here (every thread has seen the products complete): L, X, Pm take
  // their places.  Rows 0..63 -> M (strictly lower) -> L, rows 64..127 -> Mp (lower) -> Pm.
  {
    const float rowscale = isq ? p.scale : sm.beta[t];
    float* dst = isq ? sm.Pm : sm.u.m.L;
    const int tmax = (warp & 1) ? 63 : 31;                  // largest row of this warp
    if (sm.steep == 0) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int sb = 16 * i + 8 * ch;
        float pr8[8], m8[8];
        if (sb <= tmax) {                                   // warp-uniform: blocks above the warp's rows are all zero
          tmem_ld8(tmem_row + sb, pr8);
          tmem_ld8(tmem_row + 64 + sb, m8);
          tmem_wait_ld();
        }
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const int s = sb + c;
          const bool in = sb <= tmax && (isq ? (s <= t) : (s < t));
          dst[mat_idx(t, s)] = in ? rowscale * pr8[c] * m8[c] : 0.f;
          if (!isq) sm.u.m.X[mat_idx(t, s)] = 0.f;        // the inverse fills in the blocks on and below the diagonal
        }
      }
    } else {
      float my2[E], mygc[E];
#pragma unroll
      for (int e = 0; e < E; ++e) {
        my2[e] = isq ? sm.q2[t * E + e] : sm.k2[t * E + e];
        mygc[e] = sm.gc2[t * E + e];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int sb = 16 * i + 8 * ch;
        float pr8[8];
        tmem_ld8(tmem_row + sb, pr8);
        tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const int s = sb + c;
          float val = 0.f;
          if (sb <= tmax && (isq ? (s <= t) : (s < t))) {
            float acc = 0.f;
#pragma unroll
            for (int e = 0; e < E; ++e)
              acc = fmaf(my2[e] * sm.k2[s * E + e], fast_exp2(mygc[e] - sm.gc2[s * E + e]), acc);
            val = rowscale * pr8[c] * acc;
          }
          dst[mat_idx(t, s)] = val;
          if (!isq) sm.u.m.X[mat_idx(t, s)] = 0.f;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();

  // triangular inverse X = (I + L)^-1: 16x16 diagonal blocks by forward substitution, then two merge levels
  float* L = sm.u.m.L;
  float* X = sm.u.m.X;
  // 8x8 diagonal blocks by forward substitution (one column per thread)
  if (tid < 64) {
    const int r0 = (tid >> 3) * 8, j = tid & 7;
    float x[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float acc = 0.f;
#pragma unroll
      for (int k = 0; k < i; ++k) acc = fmaf(L[mat_idx(r0 + i, r0 + k)], x[k], acc);
      x[i] = (i == j) ? 1.f : (i < j ? 0.f : -acc);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) X[mat_idx(r0 + i, r0 + j)] = x[i];
  }
  __syncthreads();
  // 8 -> 16: X21 = -X22 (L21 X11), one element per thread and step
  {
    const int r0 = (tid >> 6) * 16, i = (tid >> 3) & 7, j = tid & 7;
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) acc = fmaf(L[mat_idx(r0 + 8 + i, r0 + k)], X[mat_idx(r0 + k, r0 + j)], acc);
    sm.T[tid] = acc;
    __syncthreads();
    float acc2 = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) acc2 = fmaf(X[mat_idx(r0 + 8 + i, r0 + 8 + k)], sm.T[(tid & ~63) + k * 8 + j], acc2);
    X[mat_idx(r0 + 8 + i, r0 + j)] = -acc2;
  }
  __syncthreads();
  tri_merge_mma<16>(L, X, sm.T, warp, lane);
  tri_merge_mma<32>(L, X, sm.T, warp, lane);

  // bf16 images of A (rows 0..63 of the [A;PA] image) and Pm: one 16-byte piece per thread and step
#pragma unroll
  for (int it = 0; it < 2; ++it) {
    const int piece = it * MASK_THREADS + tid, i = piece & 63, jb = piece >> 6;
    float va[8], vp[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      va[c] = X[mat_idx(i, jb * 8 + c)];
      vp[c] = sm.Pm[mat_idx(i, jb * 8 + c)];
    }
    st_shared_v4(smem_u32(sm.img_ap) + (i >> 3) * 128 + (i & 7) * 16 + jb * 2048, pack_bf16(va[0], va[1]),
                 pack_bf16(va[2], va[3]), pack_bf16(va[4], va[5]), pack_bf16(va[6], va[7]));
    st_shared_v4(smem_u32(sm.img_pm) + (i >> 3) * 128 + (i & 7) * 16 + jb * 1024, pack_bf16(vp[0], vp[1]),
                 pack_bf16(vp[2], vp[3]), pack_bf16(vp[4], vp[5]), pack_bf16(vp[6], vp[7]));
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();

  // PA = Pm A on the tensor core, from the bf16 images
  if (warp_u == 0 && elect_one()) {
    tc_fence_after();
    const uint64_t da = make_desc(smem_u32(sm.img_pm), 1024, 128, LAYOUT_PLAIN);   // Pm, K-major (rows past 63: don't care)
    const uint64_t db = make_desc(smem_u32(sm.img_ap), 128, 2048, LAYOUT_PLAIN);   // A as (K = s, N = j), MN-major
    constexpr uint32_t idesc = make_idesc(128, 64, 0, 1);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) umma_bf16(tmem + 64, desc_advance(da, kk * 2048), desc_advance(db, kk * 256), idesc, kk > 0);
    umma_commit(&sm.bar_mma);
  }
  __syncwarp();                                           // the other lanes must not run ahead into a spin wait
  mbar_wait_spin(&sm.bar_mma, 1, ctl, DEV_TIMEOUT_MMA);
  tc_fence_after();
  if (r < 64) {                                             // PA row r, columns 32*ch .. +32 -> rows 64.. of the image
    float pa[32];
    tmem_ld<32>(tmem_row + 64 + 32 * ch, pa);
    tmem_wait_ld();
    const uint32_t base = smem_u32(sm.img_ap) + ((64 + r) >> 3) * 128 + (r & 7) * 16;
#pragma unroll
    for (int jb = 0; jb < 4; ++jb)
      st_shared_v4(base + (4 * ch + jb) * 2048, pack_bf16(pa[jb * 8], pa[jb * 8 + 1]), pack_bf16(pa[jb * 8 + 2], pa[jb * 8 + 3]),
                   pack_bf16(pa[jb * 8 + 4], pa[jb * 8 + 5]), pack_bf16(pa[jb * 8 + 6], pa[jb * 8 + 7]));
  }
  tc_fence_before();
  __syncthreads();

  // images -> global, linear 16-byte copies
  const int64_t item = (static_cast<int64_t>(b) * p.NC + n) * p.H + h;
  uint4* ap_out = reinterpret_cast<uint4*>(p.AP + item * (128 * 64));
  uint4* pm_out = reinterpret_cast<uint4*>(p.Pm + item * (64 * 64));
  const uint4* ap_src = reinterpret_cast<const uint4*>(sm.img_ap);
  const uint4* pm_src = reinterpret_cast<const uint4*>(sm.img_pm);
#pragma unroll
  for (int it = 0; it < 4; ++it) ap_out[it * MASK_THREADS + tid] = ap_src[it * MASK_THREADS + tid];
#pragma unroll
  for (int it = 0; it < 2; ++it) pm_out[it * MASK_THREADS + tid] = pm_src[it * MASK_THREADS + tid];
  if (warp == 0) tmem_dealloc(tmem, 128);
}

}  // namespace tgdn

using namespace tgdn;

template <int E>
static int launch_masks(const CUtensorMap& mk, const CUtensorMap& mq, const MaskParams& p, cudaStream_t s) {
  const int smem = static_cast<int>(sizeof(MaskSmem<E>)) + 1024;
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
