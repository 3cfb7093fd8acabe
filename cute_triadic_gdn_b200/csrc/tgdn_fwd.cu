// Forward chunk recurrence of the Triadic GDN.
//
// One CTA of 512 threads owns one (sequence, head, value block of VC columns) and walks the sequence's 64-token
// chunks in order, with the E state slices S_e[:, value block] (128 x VC each, f32) in registers.  Per chunk:
//   (1) R  = [K;Q] S          tcgen05, M=128, N=E*VC, K=128   rows 0..63: K S_e, rows 64..127: Q S_e
//       W  = V - sum_e a_e*R_e (K rows);   Oq = sum_e c_e*R_e (Q rows)
//   (2) [U;Oi] = [A;PmA] (beta*W)   tcgen05, M=128, N=VC, K=64
//       o  = Oq + Oi  ->  bf16;   Vn_e = r_e*U
//   (3) dS = K^T Vn           tcgen05, M=128, N=E*VC, K=64
//       S_e <- d_e S_e + dS_e  (registers), bf16 copy -> shared memory operand of the next (1) and saved state h
// with a = k2 exp(gc), r = k2 exp(gL-gc), c = scale q2 exp(gc), d = exp(gL).
//
// Replaces cute_triadic_gdn/kernels/sm100_joint_fwd.py:66-527 (fwd_kernel); math as cute_triadic_gdn/ops/gdn_joint.py:63-90.
// K/Q tiles arrive by TMA (128B swizzle) one chunk ahead, the [A;PmA] operand image by a bulk copy; every wait is bounded.
//
// Column order inside the CTA: thread (warpgroup w, row i) owns, for every slice e, the CW = VC/4 value columns
// w*CW..w*CW+CW-1; its E*CW columns are contiguous in tensor memory and in the operand images:
// n' = w*(E*CW) + e*CW + c  <->  (slice e, value column w*CW + c of the block).
#include "tgdn_common.cuh"
#include "tgdn_host.h"
#include "tgdn_kernels.h"

namespace tgdn {


__device__ __forceinline__ float fexp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// NWG warpgroups (128 threads each) split the VC value columns; STAGES = 2 prefetches the next chunk's tiles and runs
// one CTA per SM, STAGES = 1 is sized so that two CTAs share an SM and hide each other's dependent-MMA latency.
template <int E, int VC, int NWG, int STAGES>
struct FwdCfg {
  static constexpr int THREADS = NWG * 128;
  static constexpr int NCOLS = E * VC;            // columns of R and dS
  static constexpr int CW = VC / NWG;             // value columns per thread and slice
  static constexpr int TPC = E * CW;              // state columns per thread
  static constexpr int ES = E | 1;                // row stride of the gate tables (odd: conflict-free)
  static constexpr int TMEM_COLS = (NCOLS + VC) <= 64 ? 64 : (NCOLS + VC) <= 128 ? 128 : (NCOLS + VC) <= 256 ? 256 : 512;
  // shared memory carve-up (bytes); every operand base is 1024-byte aligned
  static constexpr int KQ_BYTES = 32768;
  static constexpr int AP_BYTES = 16384;
  static constexpr int S_BYTES = NCOLS * 256;     // image (i = d, j = n'), SI = 128, SJ = 2048
  static constexpr int VN_BYTES = NCOLS * 128;    // image (i = t, j = n'), SI = 128, SJ = 1024
  static constexpr int BW_BYTES = VC * 128;       // image (i = s, j = v),  SI = 128, SJ = 1024
  static constexpr int OFF_KQ = 0;
  static constexpr int OFF_AP = OFF_KQ + STAGES * KQ_BYTES;
  static constexpr int OFF_S = OFF_AP + STAGES * AP_BYTES;
  static constexpr int OFF_VN = OFF_S + S_BYTES;
  static constexpr int OFF_BW = OFF_VN + VN_BYTES;
  static constexpr int OFF_GATES = OFF_BW + ((BW_BYTES + 1023) & ~1023);
  static constexpr int GATE_FLOATS = 3 * 64 * ES + 64 + 32;     // a, r, c tables, beta, two copies of d
  static constexpr int OFF_CTRL = OFF_GATES + GATE_FLOATS * 4;
  static constexpr int SMEM_BYTES = OFF_CTRL + 64 + 1024;       // + control block + alignment slack
};

struct FwdCtrl {
  uint64_t bar_load[2];
  uint64_t bar_mma;
  uint32_t tmem_base;
  int abort;
};

template <int E, int VC, int NWG, int STAGES>
__global__ void __launch_bounds__(NWG * 128, STAGES == 1 ? 2 : 1)
fwd_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_q, FwdParams p) {
  using C = FwdCfg<E, VC, NWG, STAGES>;
  constexpr int FWD_THREADS = C::THREADS;
  constexpr int NCOLS = C::NCOLS, CW = C::CW, TPC = C::TPC, ES = C::ES;
  constexpr float LOG2E = 1.4426950408889634f;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* gate_base = reinterpret_cast<float*>(smem + C::OFF_GATES);
  FwdCtrl& ctrl = *reinterpret_cast<FwdCtrl*>(smem + C::OFF_CTRL);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wg = warp >> 2;                         // warpgroup: which CW columns of every slice
  const int row = (warp & 3) * 32 + lane;           // tensor-memory lane = operand row
  const bool krow = row < 64;                       // rows 0..63 work on K rows (W, U, Vn), 64..127 on Q rows (o)
  const int t = row & 63;

  // work item
  constexpr int NV = HEAD / VC;
  const int vb = blockIdx.x % NV, h = (blockIdx.x / NV) % p.H, seq_rank = blockIdx.x / (NV * p.H);
  int b = seq_rank, first = 0, count = p.NC;
  if (p.cmap != nullptr) {
    const int doc = p.cmap[2 * p.NC + seq_rank];    // longest documents first
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
  // zero state: registers and operand image
  float S[TPC];
#pragma unroll
  for (int j = 0; j < TPC; ++j) S[j] = 0.f;
  for (int i = tid; i < C::S_BYTES / 16; i += FWD_THREADS) reinterpret_cast<uint4*>(smem + C::OFF_S)[i] = make_uint4(0, 0, 0, 0);
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
  auto issue_loads = [&](int i) {                   // thread 0: K/Q tiles and the [A;PmA] image of local chunk i
    int t0, rows;
    chunk_info(i, t0, rows);
    const int st = (STAGES == 2) ? (i & 1) : 0;
    uint8_t* kq = smem + C::OFF_KQ + st * C::KQ_BYTES;
    const int64_t item = (static_cast<int64_t>(b) * p.NC + first + i) * p.H + h;
    mbar_expect_tx(&ctrl.bar_load[st], C::KQ_BYTES + C::AP_BYTES);
    tma_load_4d(kq, &map_k, &ctrl.bar_load[st], 0, h, t0, b);
    tma_load_4d(kq + 8192, &map_q, &ctrl.bar_load[st], 0, h, t0, b);
    tma_load_4d(kq + 16384, &map_k, &ctrl.bar_load[st], 64, h, t0, b);
    tma_load_4d(kq + 24576, &map_q, &ctrl.bar_load[st], 64, h, t0, b);
    bulk_load(smem + C::OFF_AP + st * C::AP_BYTES, p.AP + item * (128 * 64), C::AP_BYTES, &ctrl.bar_load[st]);
  };
  auto prefetch_loads = [&](int i) {                // thread 0: pull the next chunk's tiles into L2 while this chunk is worked on
    int t0, rows;
    chunk_info(i, t0, rows);
    const int64_t item = (static_cast<int64_t>(b) * p.NC + first + i) * p.H + h;
    tma_prefetch_4d(&map_k, 0, h, t0, b);
    tma_prefetch_4d(&map_q, 0, h, t0, b);
    tma_prefetch_4d(&map_k, 64, h, t0, b);
    tma_prefetch_4d(&map_q, 64, h, t0, b);
    bulk_prefetch(p.AP + item * (128 * 64), C::AP_BYTES);
  };
  // saved state of chunk item: this thread's pieces of slice e live at [e][(vb*VC + wg*CW)/8][row][...]
  auto store_state = [&](int64_t item, const uint32_t* packed /* TPC/2 words */) {
    if (p.h == nullptr) return;
    uint8_t* base = reinterpret_cast<uint8_t*>(p.h) + item * (static_cast<int64_t>(E) * 32768);
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

  // Gate tables.  The Q-row threads own them.  During the epilogue of (2), where Q rows have little else to do, they load
  // the next chunk's raw inputs (pulled into L2 one chunk earlier, so the loads are short and nothing is held in
  // registers across a chunk), turn them into table values and store a, c and beta, which nobody reads after the
  // epilogue of (1); r, which the K rows still read in (2), and d, which (3) itself uses (two copies), follow at the start
  // of the epilogue of (3).  Loads are unconditional from clamped (always valid) addresses and masked at use.
  constexpr int QTHREADS = FWD_THREADS / 2;
  constexpr int GQ = (64 * E + QTHREADS - 1) / QTHREADS;     // table entries per Q-row thread
  const int qid = wg * 64 + t;                               // Q-row threads: 0 .. QTHREADS-1
  struct GateRaw { float gcv[GQ], gl[GQ], k2v[GQ], q2v[GQ], beta; int rows; };
  struct GateVal { float a[GQ], r[GQ], c[GQ], d[GQ], beta; };
  float* g_a = gate_base;
  float* g_r = g_a + 64 * ES;
  float* g_c = g_r + 64 * ES;
  float* g_beta = g_c + 64 * ES;
  float* g_dd = g_beta + 64;                                 // [2][16]
  auto load_gates = [&](int i) {
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
  auto gate_values = [&](const GateRaw& g) {
    GateVal v;
#pragma unroll
    for (int it = 0; it < GQ; ++it) {
      const int idx = min(qid + it * QTHREADS, 64 * E - 1);
      const bool ok = idx / E < g.rows;
      const float k2v = ok ? g.k2v[it] : 0.f, q2v = ok ? g.q2v[it] : 0.f;
      const float gcv = g.gcv[it] * LOG2E, gl = g.gl[it] * LOG2E;
      const float eg = fexp2(gcv);
      v.a[it] = k2v * eg;
      v.r[it] = k2v * fexp2(gl - gcv);
      v.c[it] = p.scale * q2v * eg;
      v.d[it] = fexp2(gl);
    }
    v.beta = ((qid & 63) < g.rows) ? g.beta : 0.f;
    return v;
  };
  auto store_gates_early = [&](const GateVal& v) {            // a, c, beta
#pragma unroll
    for (int it = 0; it < GQ; ++it) {
      const int idx = qid + it * QTHREADS;
      if (idx < 64 * E) {
        const int r = idx / E, e = idx % E;
        g_a[r * ES + e] = v.a[it];
        g_c[r * ES + e] = v.c[it];
      }
    }
    if (qid < 64) g_beta[qid] = v.beta;
  };
  auto store_gates_late = [&](const float* vr, float vd, int dbuf) {   // r, d
#pragma unroll
    for (int it = 0; it < GQ; ++it) {
      const int idx = qid + it * QTHREADS;
      if (idx < 64 * E) g_r[(idx / E) * ES + idx % E] = vr[it];
    }
    if (qid < E) g_dd[dbuf * 16 + qid] = vd;                  // entry (row 0, e = qid) is this thread's first
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
  auto load_vrow = [&](int i) {                      // this thread's CW value columns of row t (clamped), raw bf16
    int t0, rows;
    chunk_info(i, t0, rows);
    const int64_t tok = static_cast<int64_t>(b) * p.T + t0;
    const __nv_bfloat16* vp = p.v + ((tok + min(t, max(rows, 1) - 1)) * p.H + h) * HEAD + vb * VC + wg * CW;
    uint4 u;
    if constexpr (CW == 8) {
      u = __ldg(reinterpret_cast<const uint4*>(vp));
    } else {
      const uint2 w = __ldg(reinterpret_cast<const uint2*>(vp));
      u = make_uint4(w.x, w.y, 0u, 0u);
    }
    return u;
  };

  if (tid == 0) issue_loads(0);
  uint4 vnext = load_vrow(0);
  // Where registers allow (small E), the raw inputs are held in registers one chunk ahead instead of only sitting in L2.
  constexpr bool HOLD_RAW = E <= 4;
  GateRaw raw_next;
  float r_next[GQ], d_next = 0.f;                      // Q-row threads: table values that wait for the epilogue of (3)
  if (!krow) {
    const GateVal v = gate_values(load_gates(0));
    store_gates_early(v);
    store_gates_late(v.r, v.d[0], 0);
    if (count > 1) {
      if constexpr (HOLD_RAW) raw_next = load_gates(1); else prefetch_gates(1);
    }
  }
  uint32_t mma_phase = 0;
  {
    uint32_t zeros[TPC / 2];
#pragma unroll
    for (int j = 0; j < TPC / 2; ++j) zeros[j] = 0u;
    store_state((static_cast<int64_t>(b) * p.NC + first) * p.H + h, zeros);
  }
  __syncthreads();                                   // first chunk's gate tables visible

  for (int i = 0; i < count; ++i) {
    const int st = (STAGES == 2) ? (i & 1) : 0;
    int t0, rows;
    chunk_info(i, t0, rows);
    const int64_t item = (static_cast<int64_t>(b) * p.NC + first + i) * p.H + h;
    const int64_t tok = static_cast<int64_t>(b) * p.T + t0;
    uint8_t* kq = smem + C::OFF_KQ + st * C::KQ_BYTES;
    uint8_t* ap = smem + C::OFF_AP + st * C::AP_BYTES;

    // ---- (1) R = [K;Q] S --------------------------------------------------------------------------------------
    mbar_wait(&ctrl.bar_load[st], (STAGES == 2 ? (i >> 1) : i) & 1, ctl, DEV_TIMEOUT_LOAD);
    if (warp_u == 0 && elect_one()) {
      tc_fence_after();
      const uint64_t da = make_desc(smem_u32(kq), 16, 1024, LAYOUT_SW128);
      const uint64_t db = make_desc(smem_u32(smem + C::OFF_S), 128, 2048, LAYOUT_PLAIN);
      constexpr uint32_t idesc = make_idesc(128, NCOLS, 0, 1);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)
        umma_bf16(tmem, desc_advance(da, (kk >> 2) * 16384 + (kk & 3) * 32), desc_advance(db, kk * 256), idesc, kk > 0);
      umma_commit(&ctrl.bar_mma);
    }
    __syncwarp();                                    // the other lanes must not run ahead into a spin wait
    if (warp_u == 1 && i + 1 < count && elect_one()) {
      if (STAGES == 2) issue_loads(i + 1);             // the other stage was released by the previous chunk's (3)
      if (STAGES == 1) prefetch_loads(i + 1);
    }
    // the load of the next chunk's value row goes out now; it is consumed one iteration later
    const float* g_d = g_dd + (i & 1) * 16;
    const uint4 vraw = vnext;
    if (i + 1 < count) vnext = load_vrow(i + 1);
    mbar_wait_spin(&ctrl.bar_mma, mma_phase & 1, ctl, DEV_TIMEOUT_MMA);
    ++mma_phase;
    tc_fence_after();

    float acc[CW];                                   // K rows: W (starts from V); Q rows: Oq
    {
      const uint32_t vw[4] = {vraw.x, vraw.y, vraw.z, vraw.w};
#pragma unroll
      for (int c = 0; c < CW; ++c)
        acc[c] = (krow && t < rows) ? ((c & 1) ? bf16_hi(vw[c >> 1]) : bf16_lo(vw[c >> 1])) : 0.f;
    }
    {
      const float* tab = krow ? g_a : g_c;
      constexpr int EP = (TPC % 32 == 0) ? 32 / CW : ((TPC % 16 == 0) ? 16 / CW : E);   // slices per tensor-memory round trip
#pragma unroll
      for (int e0 = 0; e0 < E; e0 += EP) {
        float rr[EP * CW];
        tmem_ld<EP * CW>(tmem_row + wg * TPC + e0 * CW, rr);
        tmem_wait_ld();
#pragma unroll
        for (int ee = 0; ee < EP; ++ee) {
          const float gsc = tab[t * ES + e0 + ee];
          const float sg = krow ? -gsc : gsc;
#pragma unroll
          for (int c = 0; c < CW; ++c) acc[c] = fmaf(sg, rr[ee * CW + c], acc[c]);
        }
      }
    }
    if (krow) {
      // W -> saved (bf16), beta*W -> operand image (i = s, j = v)
      const float bt = g_beta[t];
      uint32_t wsave[CW / 2], wop[CW / 2];
#pragma unroll
      for (int c = 0; c < CW; c += 2) {
        wsave[c / 2] = pack_bf16(acc[c], acc[c + 1]);
        wop[c / 2] = pack_bf16(bt * acc[c], bt * acc[c + 1]);
      }
      const int v0 = wg * CW;
      const uint32_t dst = smem_u32(smem + C::OFF_BW) + (t >> 3) * 128 + (v0 >> 3) * 1024 + (t & 7) * 16 + (v0 & 7) * 2;
      if constexpr (CW == 8) st_shared_v4(dst, wop[0], wop[1], wop[2], wop[3]); else st_shared_v2(dst, wop[0], wop[1]);
      if (p.W != nullptr) {
        __nv_bfloat16* wp = p.W + (item * 64 + t) * HEAD + vb * VC + v0;
        if constexpr (CW == 8) *reinterpret_cast<uint4*>(wp) = make_uint4(wsave[0], wsave[1], wsave[2], wsave[3]);
        else *reinterpret_cast<uint2*>(wp) = make_uint2(wsave[0], wsave[1]);
      }
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();

    // ---- (2) [U;Oi] = [A;PmA] (beta W) ------------------------------------------------------------------------
    if (warp_u == 0 && elect_one()) {
      tc_fence_after();
      const uint64_t da = make_desc(smem_u32(ap), 2048, 128, LAYOUT_PLAIN);
      const uint64_t db = make_desc(smem_u32(smem + C::OFF_BW), 128, 1024, LAYOUT_PLAIN);
      constexpr uint32_t idesc = make_idesc(128, VC, 0, 1);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        umma_bf16(tmem + NCOLS, desc_advance(da, kk * 4096), desc_advance(db, kk * 256), idesc, kk > 0);
      umma_commit(&ctrl.bar_mma);
    }
    __syncwarp();                                    // the other lanes must not run ahead into a spin wait
    mbar_wait_spin(&ctrl.bar_mma, mma_phase & 1, ctl, DEV_TIMEOUT_MMA);
    ++mma_phase;
    tc_fence_after();
    {
      float u[CW];
      tmem_ld<CW>(tmem_row + NCOLS + wg * CW, u);
      tmem_wait_ld();
      if (krow) {
        if (p.U != nullptr) {
          __nv_bfloat16* up = p.U + (item * 64 + t) * HEAD + vb * VC + wg * CW;
          if constexpr (CW == 8)
            *reinterpret_cast<uint4*>(up) = make_uint4(pack_bf16(u[0], u[1]), pack_bf16(u[2], u[3]), pack_bf16(u[4], u[5]), pack_bf16(u[6], u[7]));
          else
            *reinterpret_cast<uint2*>(up) = make_uint2(pack_bf16(u[0], u[1]), pack_bf16(u[2], u[3]));
        }
        // Vn_e = r_e * U -> operand image (i = t, j = n')
        const uint32_t base = smem_u32(smem + C::OFF_VN) + (t >> 3) * 128 + (t & 7) * 16;
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const float re = g_r[t * ES + e];
          const int n0 = wg * TPC + e * CW;
          const uint32_t dst = base + (n0 >> 3) * 1024 + (n0 & 7) * 2;
          if constexpr (CW == 8)
            st_shared_v4(dst, pack_bf16(re * u[0], re * u[1]), pack_bf16(re * u[2], re * u[3]),
                         pack_bf16(re * u[4], re * u[5]), pack_bf16(re * u[6], re * u[7]));
          else
            st_shared_v2(dst, pack_bf16(re * u[0], re * u[1]), pack_bf16(re * u[2], re * u[3]));
        }
      } else if (t < rows) {
        __nv_bfloat16* op = p.o + ((tok + t) * p.H + h) * HEAD + vb * VC + wg * CW;
        if constexpr (CW == 8)
          *reinterpret_cast<uint4*>(op) = make_uint4(pack_bf16(acc[0] + u[0], acc[1] + u[1]), pack_bf16(acc[2] + u[2], acc[3] + u[3]),
                                                     pack_bf16(acc[4] + u[4], acc[5] + u[5]), pack_bf16(acc[6] + u[6], acc[7] + u[7]));
        else
          *reinterpret_cast<uint2*>(op) = make_uint2(pack_bf16(acc[0] + u[0], acc[1] + u[1]), pack_bf16(acc[2] + u[2], acc[3] + u[3]));
      }
      if (!krow && i + 1 < count) {                    // next chunk's tables
        if constexpr (!HOLD_RAW) raw_next = load_gates(i + 1);
        const GateVal v = gate_values(raw_next);
        store_gates_early(v);
#pragma unroll
        for (int it = 0; it < GQ; ++it) r_next[it] = v.r[it];
        d_next = v.d[0];
        if (i + 2 < count) {
          if constexpr (HOLD_RAW) raw_next = load_gates(i + 2); else prefetch_gates(i + 2);
        }
      }
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();

    // ---- (3) dS = K^T Vn, S <- d S + dS -----------------------------------------------------------------------
    if (warp_u == 0 && elect_one()) {
      tc_fence_after();
      const uint64_t da = make_desc(smem_u32(kq), 16384, 1024, LAYOUT_SW128);
      const uint64_t db = make_desc(smem_u32(smem + C::OFF_VN), 128, 1024, LAYOUT_PLAIN);
      constexpr uint32_t idesc = make_idesc(128, NCOLS, 1, 1);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        umma_bf16(tmem, desc_advance(da, kk * 2048), desc_advance(db, kk * 256), idesc, kk > 0);
      umma_commit(&ctrl.bar_mma);
    }
    __syncwarp();                                    // the other lanes must not run ahead into a spin wait
    mbar_wait_spin(&ctrl.bar_mma, mma_phase & 1, ctl, DEV_TIMEOUT_MMA);
    ++mma_phase;
    tc_fence_after();
    if (STAGES == 1 && warp_u == 1 && i + 1 < count && elect_one()) issue_loads(i + 1);   // the only stage is free once (3) has completed
    if (!krow && i + 1 < count) store_gates_late(r_next, d_next, (i + 1) & 1);   // this chunk's r table is dead by now
    {
      constexpr int PIECE = (TPC % 32 == 0) ? 32 : ((TPC % 16 == 0) ? 16 : TPC);
      const uint32_t base = smem_u32(smem + C::OFF_S) + (row >> 3) * 128 + (row & 7) * 16;
      uint8_t* hbase = (p.h != nullptr && i + 1 < count)
                           ? reinterpret_cast<uint8_t*>(p.h) + (item + p.H) * (static_cast<int64_t>(E) * 32768) : nullptr;
      const int v0 = vb * VC + wg * CW;
#pragma unroll
      for (int j0 = 0; j0 < TPC; j0 += PIECE) {
        float ds[PIECE];
        tmem_ld<PIECE>(tmem_row + wg * TPC + j0, ds);
        tmem_wait_ld();
        uint32_t packed[PIECE / 2];
#pragma unroll
        for (int j = 0; j < PIECE; j += 2) {
          S[j0 + j] = fmaf(g_d[(j0 + j) / CW], S[j0 + j], ds[j]);
          S[j0 + j + 1] = fmaf(g_d[(j0 + j + 1) / CW], S[j0 + j + 1], ds[j + 1]);
          packed[j / 2] = pack_bf16(S[j0 + j], S[j0 + j + 1]);
        }
        // operand image (i = d, j = n') for the next chunk's (1)
#pragma unroll
        for (int j = 0; j < PIECE; j += 8) {
          const int n0 = wg * TPC + j0 + j;
          st_shared_v4(base + (n0 >> 3) * 2048, packed[j / 2], packed[j / 2 + 1], packed[j / 2 + 2], packed[j / 2 + 3]);
        }
        // saved state of the next chunk: slice e as [v/8][d][v%8]
        if (hbase != nullptr) {
#pragma unroll
          for (int j = 0; j < PIECE; j += CW) {
            const int e = (j0 + j) / CW;
            uint8_t* dst = hbase + e * 32768 + (v0 >> 3) * 2048 + row * 16 + (v0 & 7) * 2;
            if constexpr (CW == 8)
              *reinterpret_cast<uint4*>(dst) = make_uint4(packed[j / 2], packed[j / 2 + 1], packed[j / 2 + 2], packed[j / 2 + 3]);
            else
              *reinterpret_cast<uint2*>(dst) = make_uint2(packed[j / 2], packed[j / 2 + 1]);
          }
        }
      }
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
static int launch_fwd(const CUtensorMap& mk, const CUtensorMap& mq, const FwdParams& p, cudaStream_t s) {
  using C = FwdCfg<E, VC, NWG, STAGES>;
  static_assert(STAGES == 2 || C::SMEM_BYTES <= 115712, "two CTAs per SM need at most 113 KB each");
  static_assert(C::SMEM_BYTES <= 232448, "shared memory budget of one CTA exceeded");
  cudaError_t e = cudaFuncSetAttribute(fwd_kernel<E, VC, NWG, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
  if (e != cudaSuccess) return tgdn_cuda_error(e);
  const int grid = p.n_seq * p.H * (HEAD / VC);
  fwd_kernel<E, VC, NWG, STAGES><<<grid, C::THREADS, C::SMEM_BYTES, s>>>(mk, mq, p);
  return tgdn_cuda_error(cudaGetLastError());
}

extern "C" int tgdn_fwd(const void* q, const void* k, const void* v, const float* k2, const float* q2, const float* beta,
                        const float* gc, const void* AP, float scale, const int32_t* doc_offsets,
                        const int32_t* chunk_map, int n_docs, int B, int T, int H, int E, int NC, void* o, void* W,
                        void* U, void* h, void* stream) {
  if (!q || !k || !v || !k2 || !q2 || !beta || !gc || !AP || !o) return TGDN_ERR_NULL;
  const bool packed = chunk_map != nullptr;
  if (packed && (!doc_offsets || n_docs < 1)) return TGDN_ERR_NULL;
  int rc = tgdn_check_core_shape(B, T, H, E, NC, packed);
  if (rc) return rc;
  if ((reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(AP) |
       reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(U) | reinterpret_cast<uintptr_t>(h)) & 15)
    return TGDN_ERR_ALIGN;
  CUtensorMap mk, mq;
  if ((rc = tgdn_make_token_map(&mk, k, B, T, H, 64, 64, 1))) return rc;
  if ((rc = tgdn_make_token_map(&mq, q, B, T, H, 64, 64, 1))) return rc;
  FwdParams p{static_cast<const __nv_bfloat16*>(v), k2, q2, beta, gc, static_cast<const __nv_bfloat16*>(AP),
              static_cast<__nv_bfloat16*>(o), static_cast<__nv_bfloat16*>(W), static_cast<__nv_bfloat16*>(U),
              static_cast<__nv_bfloat16*>(h), doc_offsets, chunk_map, B, T, H, NC, packed ? n_docs : B, scale,
              tgdn_status_word()};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (E) {
    case 1: return launch_fwd<1, 32, 4, 2>(mk, mq, p, s);
    case 2: return launch_fwd<2, 32, 4, 2>(mk, mq, p, s);
    case 4: return launch_fwd<4, 32, 4, 2>(mk, mq, p, s);
    case 8: return launch_fwd<8, 16, 2, 1>(mk, mq, p, s);
    case 12: return launch_fwd<12, 16, 4, 2>(mk, mq, p, s);
    case 16: return launch_fwd<16, 16, 4, 2>(mk, mq, p, s);
    default: return TGDN_ERR_SHAPE;
  }
}
