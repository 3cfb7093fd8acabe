// Reverse chunk recurrence of the Triadic GDN backward.
//
// One CTA of 512 threads owns one (sequence, head, value block) and walks the chunks from last to first with
// G_e = dL/dS_e[:, value block] (f32) in registers.  Per chunk, with dO, U the chunk's rows of the value block:
//   (a) KG = [K;Q] G                tcgen05 M=128, N=E*VC, K=128   (rows 0..63 are used)
//       Y  = Pm^T dO                tcgen05 M=128 (64 used), N=VC, K=64
//       dU = sum_e r_e*KG_e + Y ;   dr_e = sum_v U*KG_e  (per value block, summed later)
//   (c) Z  = A^T dU                 tcgen05 M=128 (64 used), N=VC, K=64
//       dW = beta*Z = dV ;  X = [-a_e*dW ; c_e*dO]
//   (d) dG = [K^T | Q^T] X          tcgen05 M=128, N=E*VC, K=128
//       G_e <- d_e G_e + dG_e ; bf16 copy -> operand of the next (a) and saved ds
//
// Replaces cute_triadic_gdn/kernels/sm100_joint_bwd_recurrent.py:59-533 (rec_kernel).  Same thread/column organisation
// as the forward recurrence (tgdn_fwd.cu); the operand X and the bf16 image of G share one buffer because they are never
// live at the same time.
#include "tgdn_common.cuh"
#include "tgdn_host.h"
#include "tgdn_kernels.h"

namespace tgdn {


__device__ __forceinline__ float rexp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// NWG warpgroups split the VC value columns; STAGES = 2 prefetches the next chunk's tiles (one CTA per SM), STAGES = 1 is
// sized so that two CTAs share an SM and hide each other's dependent-MMA latency.
template <int E, int VC, int NWG, int STAGES>
struct RecCfg {
  static constexpr int THREADS = NWG * 128;
  static constexpr int NCOLS = E * VC;
  static constexpr int CW = VC / NWG;
  static constexpr int TPC = E * CW;
  static constexpr int ES = E | 1;
  static constexpr int TMEM_NEED = NCOLS + 2 * VC;
  static constexpr int TMEM_COLS = TMEM_NEED <= 64 ? 64 : TMEM_NEED <= 128 ? 128 : TMEM_NEED <= 256 ? 256 : 512;
  static constexpr int KQ_BYTES = 32768;
  static constexpr int AP_BYTES = 16384;
  static constexpr int PM_BYTES = 8192;
  static constexpr int GX_BYTES = NCOLS * 256;    // image (i = row 0..127, j = n'), SI = 128, SJ = 2048
  static constexpr int DO_BYTES = VC * 128;       // image (i = t, j = v), SI = 128, SJ = 1024
  static constexpr int OFF_KQ = 0;
  static constexpr int OFF_GX = OFF_KQ + STAGES * KQ_BYTES;
  static constexpr int OFF_AP = OFF_GX + GX_BYTES;
  static constexpr int OFF_PM = OFF_AP + STAGES * AP_BYTES;
  // the 128-row descriptors over the 64-row Pm image read up to 8 KB past it: keep 8 KB of owned memory behind it
  static constexpr int OFF_DO = OFF_PM + STAGES * PM_BYTES;
  static constexpr int OFF_DU = OFF_DO + ((DO_BYTES + 1023) & ~1023);
  static constexpr int OFF_GATES = OFF_DU + ((DO_BYTES + 1023) & ~1023);
  static constexpr int GATE_FLOATS = 3 * 64 * ES + 64 + 16;
  static constexpr int OFF_DRP = OFF_GATES + 2 * GATE_FLOATS * 4;   // two table buffers: next chunk's are built ahead
  static constexpr int DRP_FLOATS = NWG * 64 * ES;
  static constexpr int OFF_PAD = OFF_DRP + DRP_FLOATS * 4;
  static constexpr int PAD = (OFF_PAD - OFF_DO) >= 8192 ? 0 : 8192 - (OFF_PAD - OFF_DO);
  static constexpr int OFF_CTRL = OFF_PAD + PAD;
  static constexpr int SMEM_BYTES = OFF_CTRL + 64 + 1024;
};

struct RecCtrl {
  uint64_t bar_load[2];
  uint64_t bar_mma;
  uint32_t tmem_base;
  int abort;
};

template <int E, int VC, int NWG, int STAGES>
__global__ void __launch_bounds__(NWG * 128, STAGES == 1 ? 2 : 1)
rec_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_q, RecParams p) {
  using C = RecCfg<E, VC, NWG, STAGES>;
  constexpr int REC_THREADS = C::THREADS;
  constexpr int NCOLS = C::NCOLS, CW = C::CW, TPC = C::TPC, ES = C::ES;
  constexpr int NV = HEAD / VC;
  constexpr float LOG2E = 1.4426950408889634f;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* gate_buf = reinterpret_cast<float*>(smem + C::OFF_GATES);
  float* drp = reinterpret_cast<float*>(smem + C::OFF_DRP);
  RecCtrl& ctrl = *reinterpret_cast<RecCtrl*>(smem + C::OFF_CTRL);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wg = warp >> 2;
  const int row = (warp & 3) * 32 + lane;
  const bool krow = row < 64;
  const int t = row & 63;

  const int vb = blockIdx.x % NV, h = (blockIdx.x / NV) % p.H, seq_rank = blockIdx.x / (NV * p.H);
  int b = seq_rank, first = 0, count = p.NC;
  if (p.cmap != nullptr) {
    const int doc = p.cmap[2 * p.NC + seq_rank];
    if (doc < 0 || doc >= p.n_seq) return;
    b = 0;
    first = p.offsets[doc];
    count = p.offsets[doc + 1] - first;
    if (first < 0 || count <= 0 || first + count > p.NC) return;
  }

  if (tid == 0) {
    mbar_init(&ctrl.bar_load[0], 1);
    mbar_init(&ctrl.bar_load[1], 1);
    mbar_init(&ctrl.bar_mma, 1);
    mbar_fence_init();
    ctrl.abort = 0;
  }
  if (warp == 0) { tmem_alloc(&ctrl.tmem_base, C::TMEM_COLS); tmem_relinquish(); }
  float G[TPC];
#pragma unroll
  for (int j = 0; j < TPC; ++j) G[j] = 0.f;
  for (int i = tid; i < C::GX_BYTES / 16; i += REC_THREADS) reinterpret_cast<uint4*>(smem + C::OFF_GX)[i] = make_uint4(0, 0, 0, 0);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = __shfl_sync(0xffffffffu, ctrl.tmem_base, 0);
  const int warp_u = __shfl_sync(0xffffffffu, warp, 0);   // warp index as a warp-uniform value
  const uint32_t tmem_row = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
  WaitCtl ctl{&ctrl.abort, p.status};

  auto chunk_info = [&](int i, int& t0, int& rows) {
    const int n = first + i;
    if (p.cmap != nullptr) { t0 = p.cmap[n]; rows = p.cmap[p.NC + n]; } else { t0 = n * CHUNK; rows = CHUNK; }
    if (t0 < 0 || rows < 0 || rows > CHUNK || t0 + rows > p.T) {
      atomicCAS(p.status, DEV_OK, DEV_BAD_CHUNK_MAP);
      t0 = 0; rows = 0;
    }
  };
  auto issue_loads = [&](int i, int st) {           // thread 0: K/Q tiles, [A;PmA] image and Pm image of local chunk i
    int t0, rows;
    chunk_info(i, t0, rows);
    uint8_t* kq = smem + C::OFF_KQ + st * C::KQ_BYTES;
    const int64_t item = (static_cast<int64_t>(b) * p.NC + first + i) * p.H + h;
    mbar_expect_tx(&ctrl.bar_load[st], C::KQ_BYTES + C::AP_BYTES + C::PM_BYTES);
    tma_load_4d(kq, &map_k, &ctrl.bar_load[st], 0, h, t0, b);
    tma_load_4d(kq + 8192, &map_q, &ctrl.bar_load[st], 0, h, t0, b);
    tma_load_4d(kq + 16384, &map_k, &ctrl.bar_load[st], 64, h, t0, b);
    tma_load_4d(kq + 24576, &map_q, &ctrl.bar_load[st], 64, h, t0, b);
    bulk_load(smem + C::OFF_AP + st * C::AP_BYTES, p.AP + item * (128 * 64), C::AP_BYTES, &ctrl.bar_load[st]);
    bulk_load(smem + C::OFF_PM + st * C::PM_BYTES, p.Pm + item * (64 * 64), C::PM_BYTES, &ctrl.bar_load[st]);
  };
  auto store_state = [&](int64_t item, const uint32_t* packed) {
    uint8_t* base = reinterpret_cast<uint8_t*>(p.ds) + item * (static_cast<int64_t>(E) * 32768);
#pragma unroll
    for (int e = 0; e < E; ++e) {
      const int v0 = vb * VC + wg * CW;
      uint8_t* dst = base + e * 32768 + (v0 >> 3) * 2048 + row * 16 + (v0 & 7) * 2;
      if constexpr (CW == 8) {
        *reinterpret_cast<uint4*>(dst) = make_uint4(packed[e * 4], packed[e * 4 + 1], packed[e * 4 + 2], packed[e * 4 + 3]);
      } else {
        *reinterpret_cast<uint2*>(dst) = make_uint2(packed[e * 2], packed[e * 2 + 1]);
      }
    }
  };
  // Prefetched inputs of a chunk, one chunk ahead.  Every thread: its row piece (K-row threads: U, Q-row threads: dO) as
  // raw bf16.  Q-row threads only: the raw gate inputs of their table entries; they turn them into the next chunk's gate
  // tables while the K-row threads run the epilogue of (a), in which Q rows have nothing else to do.  Loads are
  // unconditional from clamped addresses and masked at use.
  constexpr int QTHREADS = REC_THREADS / 2;
  constexpr int GQ = (64 * E + QTHREADS - 1) / QTHREADS;     // table entries per Q-row thread
  const int qid = wg * 64 + t;                               // Q-row threads: 0 .. QTHREADS-1
  struct GateRaw { float gcv[GQ], gl[GQ], k2v[GQ], q2v[GQ], beta; int rows; };
  auto load_row = [&](int i) {
    int t0, rows;
    chunk_info(i, t0, rows);
    const int last = max(rows, 1) - 1;
    const int64_t item = (static_cast<int64_t>(b) * p.NC + first + i) * p.H + h;
    const int64_t tok = static_cast<int64_t>(b) * p.T + t0;
    const __nv_bfloat16* rp = krow ? p.U + (item * 64 + t) * HEAD + vb * VC + wg * CW
                                   : p.dO + ((tok + min(t, last)) * p.H + h) * HEAD + vb * VC + wg * CW;
    if constexpr (CW == 8) {
      return __ldg(reinterpret_cast<const uint4*>(rp));
    } else {
      const uint2 w = __ldg(reinterpret_cast<const uint2*>(rp));
      return make_uint4(w.x, w.y, 0u, 0u);
    }
  };
  auto load_gates = [&](int i) {                             // Q-row threads
    GateRaw g;
    int t0, rows;
    chunk_info(i, t0, rows);
    g.rows = rows;
    const int last = max(rows, 1) - 1;
    const int64_t item = (static_cast<int64_t>(b) * p.NC + first + i) * p.H + h;
    const int64_t tok = static_cast<int64_t>(b) * p.T + t0;
    const float* gcp = p.gc + item * (64 * E);
#pragma unroll
    for (int it = 0; it < GQ; ++it) {
      const int idx = min(qid + it * QTHREADS, 64 * E - 1);
      const int r = idx / E, e = idx % E;
      const int64_t off = ((tok + min(r, last)) * p.H + h) * E + e;
      g.gcv[it] = __ldg(gcp + idx);
      g.gl[it] = __ldg(gcp + 63 * E + e);
      g.k2v[it] = __ldg(p.k2 + off);
      g.q2v[it] = __ldg(p.q2 + off);
    }
    g.beta = __ldg(p.beta + (tok + min(qid & 63, last)) * p.H + h);
    return g;
  };
  auto write_gates = [&](const GateRaw& g, int buf) {        // Q-row threads
    float* ga = gate_buf + buf * C::GATE_FLOATS;
    float* gr = ga + 64 * ES;
    float* gc_ = gr + 64 * ES;
    float* gb = gc_ + 64 * ES;
    float* gd = gb + 64;
#pragma unroll
    for (int it = 0; it < GQ; ++it) {
      const int idx = qid + it * QTHREADS;
      if (idx < 64 * E) {
        const int r = idx / E, e = idx % E;
        const bool ok = r < g.rows;
        const float k2v = ok ? g.k2v[it] : 0.f, q2v = ok ? g.q2v[it] : 0.f;
        const float gcv = g.gcv[it] * LOG2E, gl = g.gl[it] * LOG2E;
        const float eg = rexp2(gcv);
        ga[r * ES + e] = k2v * eg;
        gr[r * ES + e] = k2v * rexp2(gl - gcv);
        gc_[r * ES + e] = p.scale * q2v * eg;
        if (r == 0) gd[e] = rexp2(gl);
      }
    }
    if (qid < 64) gb[qid] = (qid < g.rows) ? g.beta : 0.f;
  };
  auto prefetch_loads = [&](int i) {                         // one lane: next chunk's tiles into L2 (single-stage configuration)
    int t0, rows;
    chunk_info(i, t0, rows);
    const int64_t item = (static_cast<int64_t>(b) * p.NC + first + i) * p.H + h;
    tma_prefetch_4d(&map_k, 0, h, t0, b);
    tma_prefetch_4d(&map_q, 0, h, t0, b);
    tma_prefetch_4d(&map_k, 64, h, t0, b);
    tma_prefetch_4d(&map_q, 64, h, t0, b);
    bulk_prefetch(p.AP + item * (128 * 64), C::AP_BYTES);
    bulk_prefetch(p.Pm + item * (64 * 64), C::PM_BYTES);
  };
  auto prefetch_gates = [&](int i) {                         // Q-row threads: one request per distinct 128-byte line
    int t0, rows;
    chunk_info(i, t0, rows);
    const int last = max(rows, 1) - 1;
    const int64_t item = (static_cast<int64_t>(b) * p.NC + first + i) * p.H + h;
    const int64_t tok = static_cast<int64_t>(b) * p.T + t0;
    if (qid < 64) {
      const int64_t ro = (tok + min(qid, last)) * p.H + h;
      prefetch_l2(p.k2 + ro * E);
      prefetch_l2(p.q2 + ro * E);
      prefetch_l2(p.beta + ro);
    }
    if (qid * 32 < 64 * E) prefetch_l2(p.gc + item * (64 * E) + qid * 32);
  };
  // Where registers allow (small E) the raw gate inputs are held in registers one chunk ahead; otherwise they are only
  // pulled into L2 a chunk ahead and loaded where they are used, by threads that have slack there.
  constexpr bool HOLD_RAW = E <= 4;
  auto store_row_global = [&](__nv_bfloat16* ptr, const float* src) {
    if constexpr (CW == 8)
      *reinterpret_cast<uint4*>(ptr) = make_uint4(pack_bf16(src[0], src[1]), pack_bf16(src[2], src[3]),
                                                  pack_bf16(src[4], src[5]), pack_bf16(src[6], src[7]));
    else
      *reinterpret_cast<uint2*>(ptr) = make_uint2(pack_bf16(src[0], src[1]), pack_bf16(src[2], src[3]));
  };
  auto store_row_image = [&](uint32_t dst, const float* src, float f) {
    if constexpr (CW == 8)
      st_shared_v4(dst, pack_bf16(f * src[0], f * src[1]), pack_bf16(f * src[2], f * src[3]),
                   pack_bf16(f * src[4], f * src[5]), pack_bf16(f * src[6], f * src[7]));
    else
      st_shared_v2(dst, pack_bf16(f * src[0], f * src[1]), pack_bf16(f * src[2], f * src[3]));
  };

  if (tid == 0) issue_loads(count - 1, 0);
  uint4 row_cur = load_row(count - 1);
  GateRaw raw_next;
  if (!krow) {
    raw_next = load_gates(count - 1);
    write_gates(raw_next, 0);
    if (count > 1) {
      if constexpr (HOLD_RAW) raw_next = load_gates(count - 2); else prefetch_gates(count - 2);
    }
  }
  uint32_t mma_phase = 0;
  {
    uint32_t zeros[TPC / 2];
#pragma unroll
    for (int j = 0; j < TPC / 2; ++j) zeros[j] = 0u;
    store_state((static_cast<int64_t>(b) * p.NC + first + count - 1) * p.H + h, zeros);
  }

  for (int kstep = 0; kstep < count; ++kstep) {
    const int i = count - 1 - kstep;
    const int st = (STAGES == 2) ? (kstep & 1) : 0;
    int t0, rows;
    chunk_info(i, t0, rows);
    const int64_t item = (static_cast<int64_t>(b) * p.NC + first + i) * p.H + h;
    const int64_t tok = static_cast<int64_t>(b) * p.T + t0;
    uint8_t* kq = smem + C::OFF_KQ + st * C::KQ_BYTES;
    uint8_t* ap = smem + C::OFF_AP + st * C::AP_BYTES;
    uint8_t* pm = smem + C::OFF_PM + st * C::PM_BYTES;
    const int v0 = wg * CW;                          // first value column of this thread inside the block

    // this chunk's row piece was loaded while the previous one was processed (K-row threads: U, Q-row threads: dO, which
    // also goes into the dO operand image); its gate tables were built during the previous chunk's (a) epilogue
    float* g_a = gate_buf + (kstep & 1) * C::GATE_FLOATS;
    float* g_r = g_a + 64 * ES;
    float* g_c = g_r + 64 * ES;
    float* g_beta = g_c + 64 * ES;
    float* g_d = g_beta + 64;
    float rowv[CW];
    {
      const uint32_t rw[4] = {row_cur.x, row_cur.y, row_cur.z, row_cur.w};
      const bool live = krow || t < rows;
#pragma unroll
      for (int c = 0; c < CW; ++c) rowv[c] = live ? ((c & 1) ? bf16_hi(rw[c >> 1]) : bf16_lo(rw[c >> 1])) : 0.f;
    }
    if (!krow)
      store_row_image(smem_u32(smem + C::OFF_DO) + (t >> 3) * 128 + (v0 >> 3) * 1024 + (t & 7) * 16 + (v0 & 7) * 2, rowv, 1.f);
    if (kstep + 1 < count) row_cur = load_row(i - 1);        // consumed at the top of the next iteration
    fence_async_smem();
    tc_fence_before();
    __syncthreads();

    // ---- (a) KG = [K;Q] G and Y = Pm^T dO -----------------------------------------------------------------------
    mbar_wait(&ctrl.bar_load[st], (STAGES == 2 ? (kstep >> 1) : kstep) & 1, ctl, DEV_TIMEOUT_LOAD);
    if (warp_u == 0 && elect_one()) {
      tc_fence_after();
      {
        const uint64_t da = make_desc(smem_u32(kq), 16, 1024, LAYOUT_SW128);
        const uint64_t db = make_desc(smem_u32(smem + C::OFF_GX), 128, 2048, LAYOUT_PLAIN);
        constexpr uint32_t idesc = make_idesc(128, NCOLS, 0, 1);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_bf16(tmem, desc_advance(da, (kk >> 2) * 16384 + (kk & 3) * 32), desc_advance(db, kk * 256), idesc, kk > 0);
      }
      {
        const uint64_t da = make_desc(smem_u32(pm), 128, 1024, LAYOUT_PLAIN);       // Pm^T: MN-major over (i = t, j = s)
        const uint64_t db = make_desc(smem_u32(smem + C::OFF_DO), 128, 1024, LAYOUT_PLAIN);
        constexpr uint32_t idesc = make_idesc(128, VC, 1, 1);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_bf16(tmem + NCOLS, desc_advance(da, kk * 256), desc_advance(db, kk * 256), idesc, kk > 0);
      }
      umma_commit(&ctrl.bar_mma);
    }
    __syncwarp();                                    // the other lanes must not run ahead into a spin wait
    if (warp_u == 1 && kstep + 1 < count && elect_one()) {
      if (STAGES == 2) issue_loads(i - 1, st ^ 1); else prefetch_loads(i - 1);
    }
    mbar_wait_spin(&ctrl.bar_mma, mma_phase & 1, ctl, DEV_TIMEOUT_MMA);
    ++mma_phase;
    tc_fence_after();
    if (krow) {
      float du[CW];
      tmem_ld<CW>(tmem_row + NCOLS + v0, du);
      tmem_wait_ld();
#pragma unroll
      for (int e0 = 0; e0 < E; e0 += (16 / CW)) {
        constexpr int EP = (16 / CW) < E ? (16 / CW) : E;
        float kg[EP * CW];
        tmem_ld<EP * CW>(tmem_row + wg * TPC + e0 * CW, kg);
        tmem_wait_ld();
#pragma unroll
        for (int ee = 0; ee < EP; ++ee) {
          const float re = g_r[t * ES + e0 + ee];
          float dot = 0.f;
#pragma unroll
          for (int c = 0; c < CW; ++c) {
            du[c] = fmaf(re, kg[ee * CW + c], du[c]);
            dot = fmaf(rowv[c], kg[ee * CW + c], dot);
          }
          drp[(wg * 64 + t) * ES + e0 + ee] = dot;
        }
      }
      store_row_global(p.dU + (item * 64 + t) * HEAD + vb * VC + v0, du);
      store_row_image(smem_u32(smem + C::OFF_DU) + (t >> 3) * 128 + (v0 >> 3) * 1024 + (t & 7) * 16 + (v0 & 7) * 2, du, 1.f);
    } else if (kstep + 1 < count) {
      if constexpr (!HOLD_RAW) raw_next = load_gates(i - 1);
      write_gates(raw_next, (kstep + 1) & 1);                // tables of the chunk processed next
      if (kstep + 2 < count) {
        if constexpr (HOLD_RAW) raw_next = load_gates(i - 2); else prefetch_gates(i - 2);
      }
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();

    // ---- (c) Z = A^T dU -----------------------------------------------------------------------------------------
    if (warp_u == 0 && elect_one()) {
      tc_fence_after();
      const uint64_t da = make_desc(smem_u32(ap), 128, 2048, LAYOUT_PLAIN);         // A^T: MN-major over (i = t, j = s)
      const uint64_t db = make_desc(smem_u32(smem + C::OFF_DU), 128, 1024, LAYOUT_PLAIN);
      constexpr uint32_t idesc = make_idesc(128, VC, 1, 1);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        umma_bf16(tmem + NCOLS + VC, desc_advance(da, kk * 256), desc_advance(db, kk * 256), idesc, kk > 0);
      umma_commit(&ctrl.bar_mma);
    }
    __syncwarp();                                    // the other lanes must not run ahead into a spin wait
    // meanwhile: the value-block partial of dr, summed over the four warpgroups in a fixed order
    for (int idx = tid; idx < 64 * E; idx += REC_THREADS) {
      const int r = idx / E, e = idx % E;
      float s4 = 0.f;
#pragma unroll
      for (int w = 0; w < NWG; ++w) s4 += drp[(w * 64 + r) * ES + e];
      p.dr[((item * NV + vb) * 64 + r) * E + e] = s4;
    }
    mbar_wait_spin(&ctrl.bar_mma, mma_phase & 1, ctl, DEV_TIMEOUT_MMA);
    ++mma_phase;
    tc_fence_after();
    {
      float xr[CW];                                  // K rows: dW; Q rows: dO
      if (krow) {
        float z[CW];
        tmem_ld<CW>(tmem_row + NCOLS + VC + v0, z);
        tmem_wait_ld();
        const float bt = g_beta[t];
#pragma unroll
        for (int c = 0; c < CW; ++c) xr[c] = bt * z[c];
        if (t < rows) store_row_global(p.dV + ((tok + t) * p.H + h) * HEAD + vb * VC + v0, xr);
      } else {
#pragma unroll
        for (int c = 0; c < CW; ++c) xr[c] = rowv[c];
      }
      // X image (i = row, j = n'): rows 0..63 -a_e*dW, rows 64..127 c_e*dO
      const float* tab = krow ? g_a : g_c;
      const uint32_t base = smem_u32(smem + C::OFF_GX) + (row >> 3) * 128 + (row & 7) * 16;
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const float f = krow ? -tab[t * ES + e] : tab[t * ES + e];
        const int n0 = wg * TPC + e * CW;
        store_row_image(base + (n0 >> 3) * 2048 + (n0 & 7) * 2, xr, f);
      }
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();

    // ---- (d) dG = [K^T | Q^T] X, G <- d G + dG ------------------------------------------------------------------
    if (warp_u == 0 && elect_one()) {
      tc_fence_after();
      const uint64_t da = make_desc(smem_u32(kq), 16384, 1024, LAYOUT_SW128);
      const uint64_t db = make_desc(smem_u32(smem + C::OFF_GX), 128, 2048, LAYOUT_PLAIN);
      constexpr uint32_t idesc = make_idesc(128, NCOLS, 1, 1);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)
        umma_bf16(tmem, desc_advance(da, kk * 2048), desc_advance(db, kk * 256), idesc, kk > 0);
      umma_commit(&ctrl.bar_mma);
    }
    __syncwarp();                                    // the other lanes must not run ahead into a spin wait
    mbar_wait_spin(&ctrl.bar_mma, mma_phase & 1, ctl, DEV_TIMEOUT_MMA);
    ++mma_phase;
    tc_fence_after();
    if (STAGES == 1 && warp_u == 1 && kstep + 1 < count && elect_one()) issue_loads(i - 1, 0);   // the only stage is free once (d) has completed
    {
      uint32_t packed[TPC / 2];
#pragma unroll
      for (int j0 = 0; j0 < TPC; j0 += 16) {
        constexpr int PIECE = TPC < 16 ? TPC : 16;
        float dg[PIECE];
        tmem_ld<PIECE>(tmem_row + wg * TPC + j0, dg);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < PIECE; ++j) {
          const float de = g_d[(j0 + j) / CW];
          G[j0 + j] = fmaf(de, G[j0 + j], dg[j]);
        }
#pragma unroll
        for (int j = 0; j < PIECE; j += 2) packed[(j0 + j) / 2] = pack_bf16(G[j0 + j], G[j0 + j + 1]);
      }
      const uint32_t base = smem_u32(smem + C::OFF_GX) + (row >> 3) * 128 + (row & 7) * 16;
#pragma unroll
      for (int j0 = 0; j0 < TPC; j0 += 8) {
        const int n0 = wg * TPC + j0;
        st_shared_v4(base + (n0 >> 3) * 2048, packed[j0 / 2], packed[j0 / 2 + 1], packed[j0 / 2 + 2], packed[j0 / 2 + 3]);
      }
      if (i > 0) store_state(item - p.H, packed);
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
  }
  if (warp == 0) tmem_dealloc(tmem, C::TMEM_COLS);
}

}  // namespace tgdn

using namespace tgdn;

template <int E, int VC, int NWG, int STAGES>
static int launch_rec(const CUtensorMap& mk, const CUtensorMap& mq, const RecParams& p, cudaStream_t s) {
  using C = RecCfg<E, VC, NWG, STAGES>;
  static_assert(STAGES == 2 || C::SMEM_BYTES <= 115712, "two CTAs per SM need at most 113 KB each");
  static_assert(C::SMEM_BYTES <= 232448, "shared memory budget of one CTA exceeded");
  cudaError_t e = cudaFuncSetAttribute(rec_kernel<E, VC, NWG, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
  if (e != cudaSuccess) return tgdn_cuda_error(e);
  const int grid = p.n_seq * p.H * (HEAD / VC);
  rec_kernel<E, VC, NWG, STAGES><<<grid, C::THREADS, C::SMEM_BYTES, s>>>(mk, mq, p);
  return tgdn_cuda_error(cudaGetLastError());
}

extern "C" int tgdn_bwd_recurrent(const void* q, const void* k, const void* dO, const float* k2, const float* q2,
                                  const float* beta, const float* gc, const void* AP, const void* Pm, const void* U,
                                  float scale, const int32_t* doc_offsets, const int32_t* chunk_map, int n_docs, int B,
                                  int T, int H, int E, int NC, void* dV, void* dU, void* ds, float* dr, void* stream) {
  if (!q || !k || !dO || !k2 || !q2 || !beta || !gc || !AP || !Pm || !U || !dV || !dU || !ds || !dr) return TGDN_ERR_NULL;
  const bool packed = chunk_map != nullptr;
  if (packed && (!doc_offsets || n_docs < 1)) return TGDN_ERR_NULL;
  int rc = tgdn_check_core_shape(B, T, H, E, NC, packed);
  if (rc) return rc;
  if ((reinterpret_cast<uintptr_t>(dO) | reinterpret_cast<uintptr_t>(AP) | reinterpret_cast<uintptr_t>(Pm) |
       reinterpret_cast<uintptr_t>(U) | reinterpret_cast<uintptr_t>(dV) | reinterpret_cast<uintptr_t>(dU) |
       reinterpret_cast<uintptr_t>(ds)) & 15)
    return TGDN_ERR_ALIGN;
  CUtensorMap mk, mq;
  if ((rc = tgdn_make_token_map(&mk, k, B, T, H, 64, 64, 1))) return rc;
  if ((rc = tgdn_make_token_map(&mq, q, B, T, H, 64, 64, 1))) return rc;
  RecParams p{static_cast<const __nv_bfloat16*>(dO), k2, q2, beta, gc, static_cast<const __nv_bfloat16*>(AP),
              static_cast<const __nv_bfloat16*>(Pm), static_cast<const __nv_bfloat16*>(U),
              static_cast<__nv_bfloat16*>(dV), static_cast<__nv_bfloat16*>(dU), static_cast<__nv_bfloat16*>(ds), dr,
              doc_offsets, chunk_map, B, T, H, NC, packed ? n_docs : B, scale, tgdn_status_word()};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (E) {
    case 1: return launch_rec<1, 32, 4, 2>(mk, mq, p, s);
    case 2: return launch_rec<2, 32, 4, 2>(mk, mq, p, s);
    case 4: return launch_rec<4, 32, 4, 2>(mk, mq, p, s);
    case 8: return launch_rec<8, 16, 2, 1>(mk, mq, p, s);
    case 12: return launch_rec<12, 16, 4, 2>(mk, mq, p, s);
    case 16: return launch_rec<16, 16, 4, 2>(mk, mq, p, s);
    default: return TGDN_ERR_SHAPE;
  }
}
