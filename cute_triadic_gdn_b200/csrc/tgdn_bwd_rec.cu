// Reverse chunk recurrence of the Triadic GDN backward.
//
// One CTA owns one (sequence, head, block of VC value columns) and walks the chunks from last to first with
// G_e = dL/dS_e[:, value block] (f32) in registers.  Per chunk, with dO, U the chunk's rows of the value block:
//   (a) KG = [K;Q] G                tcgen05 M=128, N=E*VC, K=128   (rows 0..63 are used)
//       Y  = Pm^T dO                tcgen05 M=128 (64 used), N=VC, K=64
//       dU = sum_e r_e*KG_e + Y ;   dr_e = sum_v U*KG_e  (per value block, summed later)
//   (c) Z  = A^T dU                 tcgen05 M=128 (64 used), N=VC, K=64
//       dW = beta*Z = dV ;  X = [-a_e*dW ; c_e*dO]
//   (p) P  = G Xu^T                 tcgen05 M=128 (key rows d), N=64 (tokens), K=E*VC     Xu_e = r_e*U
//       the value block's share of  sum_e (r_e*U) G_e^T, the part of dK that contracts the gradient state over the
//       value axis; it leaves as a bf16 operand image (16 KB) and the state-gradient kernel adds the blocks up
//   (d) dG = [K^T | Q^T] X          tcgen05 M=128, N=E*VC, K=128
//       G_e <- d_e G_e + dG_e ; bf16 copy -> operand of the next (a)
//
// Because (p) runs here, where G lives, the gradient state itself never has to travel: the reference writes it to HBM at
// every chunk (32 KB x E per chunk and head) and reads it back in its state-gradient kernel.  The one other consumer of
// G_e outside this kernel is dd_e = <h_e, G_e>, the gradient of the chunk decay d_e = exp(gL_e), which enters the result
// only as d_e*dd_e: slices whose chunk decay is below 2^-24 contribute less than one part in 10^7 of <h_e, G_e> and are
// skipped there (dd_e = 0); G_e is stored (ds) only for the slices of chunks whose decay is above that threshold.
//
// (p) is off the dependent chain of the chunk: it is issued behind (a) as soon as its operand Xu is built, runs while the
// epilogue of (a) occupies the threads, and is read out of tensor memory while (d) runs.
//
// The gate factors (a, r, c per row and slice, d per slice) were formed by the masks kernel and arrive with one bulk copy
// per chunk; every thread reads those of its own row from shared memory.  The gradient state can be handed in (dL/dS after the last token) and out (before the first), so
// that sequences can be processed in segments (tgdn_bwd_recurrent_state).
//
// Replaces cute_triadic_gdn/kernels/sm100_joint_bwd_recurrent.py:59-533 (rec_kernel) and the (r*U) G^T product of
// cute_triadic_gdn/kernels/sm100_joint_state_grads.py:373-378.  Same thread/column organisation as the forward
// recurrence before it was split into chains: NWG warpgroups split the VC value columns (and, with NSG = 2, the slices) and
// move in lockstep; the operand X and the bf16 image of G share one buffer because they are never live at the same time.
// Two query-row warps of the first warpgroup issue the MMAs and the copies; the key-row warps, which build the operand
// of (p) under the first MMA group, carry no extra role.
#include "tgdn_common.cuh"
#include "tgdn_host.h"
#include "tgdn_kernels.h"

namespace tgdn {

// N floats of a gate row in shared memory; 16-byte loads where N allows (the offsets used are then 16-byte aligned too),
// 8-byte loads otherwise (N even)
template <int N>
__device__ __forceinline__ void rec_lds_part(const float* p, float* out) {
  if constexpr (N == 1) {
    out[0] = p[0];
  } else if constexpr (N % 4 == 0) {
#pragma unroll
    for (int j = 0; j < N / 4; ++j) {
      const float4 x = *(reinterpret_cast<const float4*>(p) + j);
      out[4 * j] = x.x; out[4 * j + 1] = x.y; out[4 * j + 2] = x.z; out[4 * j + 3] = x.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < N / 2; ++j) {
      const float2 x = *(reinterpret_cast<const float2*>(p) + j);
      out[2 * j] = x.x; out[2 * j + 1] = x.y;
    }
  }
}

// STAGES = 2 prefetches the next chunk's tiles (one CTA per SM), STAGES = 1 is sized so that two CTAs share an SM and
// hide each other's dependent-MMA latency.
// NSG > 1 splits the SLICES of a column group over NSG warpgroups (warpgroup w = slice group * NCG + column group): at
// twelve and sixteen slices a thread then holds eight value columns of half the slices instead of four columns of all of
// them, which restores the 16-byte accesses of the E = 8 kernel; the one sum over all slices (dU) is completed through
// shared memory.
template <int E, int VC, int NWG, int STAGES, int NSG = 1>
struct RecCfg {
  static constexpr int THREADS = NWG * 128;
  static constexpr int NCOLS = E * VC;
  static constexpr int NCG = NWG / NSG;           // column groups
  static constexpr int CW = VC / NCG;             // value columns per thread
  static constexpr int EL = E / NSG;              // slices per thread
  static constexpr int TPC = EL * CW;             // state columns per thread
  // The two wide products, (a) and (d), go out in PARTS column parts with a commit each: a warpgroup starts its epilogue
  // when the part that holds its own columns has completed, while the tensor core is still working on the later parts.
  static constexpr int PN = (NWG * TPC >= 192 && NWG % 2 == 0) ? NWG * TPC / 2 : NWG * TPC;   // columns per part
  static constexpr int PARTS = NWG * TPC / PN;
  static_assert((NWG * TPC) % PN == 0 && PN % TPC == 0 && PN % 16 == 0 && PARTS <= 4, "column parts of the wide products");
  static constexpr int ES = E | 1;
  static_assert(NWG % NSG == 0 && E % NSG == 0 && (NSG == 1 || EL % 2 == 0), "slice groups split the slices evenly");
  static constexpr int TMEM_NEED = NCOLS + 2 * VC + 64;       // KG/dG, Y, Z, P
  static constexpr int TMEM_COLS = TMEM_NEED <= 64 ? 64 : TMEM_NEED <= 128 ? 128 : TMEM_NEED <= 256 ? 256 : 512;
  static constexpr int KQ_BYTES = 32768;
  static constexpr int A_BYTES = 8192;            // image (i = t, j = s), SI = 128, SJ = 1024: the A half of [A; Pm A]
  static constexpr int PM_BYTES = 8192;
  static constexpr int GX_BYTES = NCOLS * 256;    // image (i = row 0..127, j = n'), SI = 128, SJ = 2048
  static constexpr int XU_BYTES = NCOLS * 128;    // image (i = t, j = n'), SI = 128, SJ = 1024
  static constexpr int DO_BYTES = VC * 128;       // image (i = t, j = v), SI = 128, SJ = 1024
  static constexpr int DOB = (DO_BYTES + 1023) & ~1023;
  static constexpr int DRP_FLOATS = NCG * 64 * ES + (NSG > 1 ? 64 * VC : 0);   // dr partials per column group; partial dU of the other slice group
  // the gate factors of a chunk as the masks kernel stored them: a, r, c as 64 dense rows of E floats each, then d
  static constexpr int GT_BYTES = gate_factor_bytes(E);
  static constexpr int GT_STRIDE = (GT_BYTES + 127) & ~127;
  static constexpr int GF_R = 64 * E, GF_C = 128 * E, GF_D = 192 * E;   // float offsets of r, c, d behind a
  static constexpr int LIMIT = STAGES == 1 ? 115712 : 232448;
  // Shared memory of a layout with `nb` copies of Pm, A and the gate factors
  static constexpr int layout_bytes(int nb) {
    const int xu = XU_BYTES < 8192 ? 8192 : XU_BYTES;
    const int upto_dt = STAGES * KQ_BYTES + GX_BYTES + nb * (PM_BYTES + A_BYTES) + xu + 2 * STAGES * DOB + DRP_FLOATS * 4;
    const int off_gt = (upto_dt + 128 + 127) & ~127;
    return off_gt + nb * GT_STRIDE + 128 + 1024;
  }
  // With two stages, Pm, A and the gate factors get a second copy too where that fits.  Where it does not (sixteen slices),
  // they stay single and are requested LATE: each is dead by the end of the epilogue of (c), and the next chunk's copies,
  // requested right then on a barrier of their own, have the whole of (d) to arrive; only the K/Q tiles and the dO / U
  // rows, which (d) and its epilogue still read, live in the stage.  Measured: the late scheme costs 12% at E = 4, where
  // both fit, and gains 7% at E = 16, where it makes room for the gate factors in shared memory.
  static constexpr bool LATE = STAGES == 2 && !(layout_bytes(2) <= LIMIT);
  static constexpr int NB = (STAGES == 2 && !LATE) ? 2 : 1;              // copies of Pm, A and the gate factors
  static_assert(layout_bytes(NB) <= LIMIT, "shared memory budget of one CTA exceeded");
  static constexpr int OFF_KQ = 0;
  static constexpr int OFF_GX = OFF_KQ + STAGES * KQ_BYTES;
  // the 128-row descriptors over the 64-row Pm and A images read up to 8 KB past them: Pm is followed by A, A by Xu
  static constexpr int OFF_PM = OFF_GX + GX_BYTES;
  static constexpr int OFF_A = OFF_PM + NB * PM_BYTES;
  static constexpr int OFF_XU = OFF_A + NB * A_BYTES;
  // per stage: the dO rows of the value block, which TMA writes straight into the operand image of Y, and the U rows,
  // which TMA writes into the place where the operand image of dU is built later (every thread reads its piece of U
  // before it overwrites that very piece with dU)
  static constexpr int OFF_DO = OFF_XU + (XU_BYTES < 8192 ? 8192 : XU_BYTES);
  static constexpr int OFF_DU = OFF_DO + STAGES * DOB;
  static constexpr int OFF_DRP = OFF_DU + STAGES * DOB;
  static constexpr int OFF_DT = OFF_DRP + DRP_FLOATS * 4;     // exp(gL) of this chunk and the store flags of the next: 2 x 16 words
  static constexpr int OFF_GT = (OFF_DT + 128 + 127) & ~127;
  static constexpr int OFF_CTRL = OFF_GT + NB * GT_STRIDE;
  static constexpr int SMEM_BYTES = OFF_CTRL + 128 + 1024;
};

struct RecCtrl {
  uint64_t bar_load[2];      // K/Q tiles, dO and U rows of a stage (STAGES == 1: everything)
  uint64_t bar_late;         // late scheme only: Pm and the gate factors of the chunk
  uint64_t bar_a;            // late scheme only: A of the chunk
  uint64_t bar_mma;          // (c)
  uint64_t bar_part[4];      // (a) and (d): one per column part
  uint64_t bar_p;
  uint64_t bar_xu;           // the key-row warps have written the operand Xu of (p): one arrival per warp
  uint32_t tmem_base;
  int abort;
};

template <int E, int VC, int NWG, int STAGES, int NSG>
__global__ void __launch_bounds__(NWG * 128, STAGES == 1 ? 2 : 1)
rec_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_q,
           const __grid_constant__ CUtensorMap map_do, const __grid_constant__ CUtensorMap map_u,
           const __grid_constant__ CUtensorMap map_du, RecParams p) {
  using C = RecCfg<E, VC, NWG, STAGES, NSG>;
  constexpr int REC_THREADS = C::THREADS;
  constexpr int NCOLS = C::NCOLS, CW = C::CW, TPC = C::TPC, ES = C::ES, NCG = C::NCG, EL = C::EL;
  constexpr int NV = HEAD / VC;
  constexpr float LOG2E = 1.4426950408889634f;   // the decay threshold below is in the log2 domain
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* drp = reinterpret_cast<float*>(smem + C::OFF_DRP);
  float* dured = drp + NCG * 64 * ES;                                 // NSG > 1: [64 rows][VC] partial dU
  float* dtab = reinterpret_cast<float*>(smem + C::OFF_DT);           // [16] exp(gL_e)
  int* ftab = reinterpret_cast<int*>(smem + C::OFF_DT) + 16;          // [16] store G_e of the next chunk?
  RecCtrl& ctrl = *reinterpret_cast<RecCtrl*>(smem + C::OFF_CTRL);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wg = warp >> 2;
  const int cgp = NSG == 1 ? wg : wg % NCG;         // column group: value columns cgp*CW .. of the block
  const int sgp = NSG == 1 ? 0 : wg / NCG;          // slice group: slices sgp*EL ..
  const int e0 = sgp * EL;
  const int row = (warp & 3) * 32 + lane;
  const bool krow = row < 64;
  const int t = row & 63;

  const int vb = blockIdx.x % NV, h = (blockIdx.x / NV) % p.H, seq_rank = blockIdx.x / (NV * p.H);
  int b = seq_rank, first = 0, count = p.NC, seq = seq_rank;
  if (p.cmap != nullptr) {
    const int doc = p.cmap[2 * p.NC + seq_rank];
    if (doc < 0 || doc >= p.n_seq) return;
    b = 0;
    seq = doc;
    first = p.offsets[doc];
    count = p.offsets[doc + 1] - first;
    if (first < 0 || count <= 0 || first + count > p.NC) return;
  }

  if (tid == 0) {
    mbar_init(&ctrl.bar_load[0], 1);
    mbar_init(&ctrl.bar_load[1], 1);
    mbar_init(&ctrl.bar_late, 1);
    mbar_init(&ctrl.bar_a, 1);
    mbar_init(&ctrl.bar_mma, 1);
    for (int c = 0; c < 4; ++c) mbar_init(&ctrl.bar_part[c], 1);
    mbar_init(&ctrl.bar_p, 1);
    mbar_init(&ctrl.bar_xu, NWG * 2);
    mbar_fence_init();
    ctrl.abort = 0;
  }
  // Roles: the key-row warps (0, 1 of a warpgroup) build the operand of (p) under the first MMA
  // group, so two query-row warps of the first warpgroup take the extra work: warp 2 issues the MMAs, warp 3 every load and
  // store of the CTA.
  constexpr int ISSUE_WARP = 2, COPY_WARP = 3;
  if (warp == 0) { tmem_alloc(&ctrl.tmem_base, C::TMEM_COLS); tmem_relinquish(); }
  // The gradient state after the last token: zero, or what a later segment of the same sequence handed over
  // (f32 [sequence][H][E][128 d][128 v]); its bf16 image is the operand of the first chunk's products.
  float G[TPC];
  if (p.g_in != nullptr) {
    static_assert(CW % 4 == 0 && TPC % 8 == 0, "state hand-off: whole 16-byte pieces per thread");
    const float* src = p.g_in + ((static_cast<int64_t>(seq) * p.H + h) * E + e0) * (HEAD * HEAD) + row * HEAD + vb * VC + cgp * CW;
#pragma unroll
    for (int e = 0; e < EL; ++e)
#pragma unroll
      for (int c = 0; c < CW; c += 4) {
        const float4 x = __ldg(reinterpret_cast<const float4*>(src + e * (HEAD * HEAD) + c));
        G[e * CW + c] = x.x; G[e * CW + c + 1] = x.y; G[e * CW + c + 2] = x.z; G[e * CW + c + 3] = x.w;
      }
    const uint32_t base = smem_u32(smem + C::OFF_GX) + (row >> 3) * 128 + (row & 7) * 16;
#pragma unroll
    for (int j = 0; j < TPC; j += 8)
      st_shared_v4(base + ((wg * TPC + j) >> 3) * 2048, pack_bf16(G[j], G[j + 1]), pack_bf16(G[j + 2], G[j + 3]),
                   pack_bf16(G[j + 4], G[j + 5]), pack_bf16(G[j + 6], G[j + 7]));
  } else {
#pragma unroll
    for (int j = 0; j < TPC; ++j) G[j] = 0.f;
    for (int i = tid; i < C::GX_BYTES / 16; i += REC_THREADS) reinterpret_cast<uint4*>(smem + C::OFF_GX)[i] = make_uint4(0, 0, 0, 0);
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = __shfl_sync(0xffffffffu, ctrl.tmem_base, 0);
  const int warp_u = __shfl_sync(0xffffffffu, warp, 0);   // warp index as a warp-uniform value
  const uint32_t tmem_row = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
  constexpr uint32_t TM_Y = NCOLS, TM_Z = NCOLS + VC, TM_P = NCOLS + 2 * VC;
  WaitCtl ctl{&ctrl.abort, p.status};

  auto chunk_info = [&](int i, int& t0, int& rows) {
    const int n = first + i;
    if (p.cmap != nullptr) { t0 = p.cmap[n]; rows = p.cmap[p.NC + n]; } else { t0 = n * CHUNK; rows = CHUNK; }
    if (t0 < 0 || rows < 0 || rows > CHUNK || t0 + rows > p.T) {
      atomicCAS(p.status, DEV_OK, DEV_BAD_CHUNK_MAP);
      t0 = 0; rows = 0;
    }
  };
  auto issue_gates_pm = [&](int i, int nb, uint64_t* bar) {   // one thread: the Pm image and the gate factors of local chunk i -> copy nb
    const int64_t item = (static_cast<int64_t>(b) * p.NC + first + i) * p.H + h;
    bulk_load(smem + C::OFF_GT + nb * C::GT_STRIDE, p.gc + item * gate_item_floats(E) + 64 * E, C::GT_BYTES, bar);
    bulk_load(smem + C::OFF_PM + nb * C::PM_BYTES, p.Pm + item * (64 * 64), C::PM_BYTES, bar);
  };
  auto issue_a = [&](int i, int nb, uint64_t* bar) {          // one thread: the A half of [A;PmA] of local chunk i -> copy nb
    const int64_t item = (static_cast<int64_t>(b) * p.NC + first + i) * p.H + h;
    // [A; Pm A] is an image of 128 rows: per 8-column block (2 KB) the first 1 KB holds the rows of A
    const __nv_bfloat16* ap = p.AP + item * (128 * 64);
#pragma unroll
    for (int jb = 0; jb < 8; ++jb) bulk_load(smem + C::OFF_A + nb * C::A_BYTES + jb * 1024, ap + jb * 1024, 1024, bar);
  };
  constexpr uint32_t GATES_PM_TX = C::PM_BYTES + C::GT_BYTES;
  constexpr uint32_t LATE_TX = C::A_BYTES + GATES_PM_TX;
  auto issue_loads = [&](int i, int st) {           // one thread: K/Q tiles and the dO / U rows of local chunk i (STAGES == 1: the rest too)
    int t0, rows;
    chunk_info(i, t0, rows);
    uint8_t* kq = smem + C::OFF_KQ + st * C::KQ_BYTES;
    const int64_t item = (static_cast<int64_t>(b) * p.NC + first + i) * p.H + h;
    // the stage's U / dU buffer may still be the source of a store of dU issued by this thread
    bulk_wait_group_read();
    mbar_expect_tx(&ctrl.bar_load[st], C::KQ_BYTES + 2 * C::DO_BYTES + (C::LATE ? 0u : LATE_TX));
#pragma unroll
    for (int jb = 0; jb < VC / 8; ++jb) {            // eight value columns x 64 rows = one 1 KB column block of the image
      tma_load_4d(smem + C::OFF_DO + st * C::DOB + jb * 1024, &map_do, &ctrl.bar_load[st], vb * VC + jb * 8, h, t0, b);
      tma_load_4d(smem + C::OFF_DU + st * C::DOB + jb * 1024, &map_u, &ctrl.bar_load[st], vb * VC + jb * 8, 0,
                  static_cast<int>(item * 64), 0);
    }
    tma_load_4d(kq, &map_k, &ctrl.bar_load[st], 0, h, t0, b);
    tma_load_4d(kq + 8192, &map_q, &ctrl.bar_load[st], 0, h, t0, b);
    tma_load_4d(kq + 16384, &map_k, &ctrl.bar_load[st], 64, h, t0, b);
    tma_load_4d(kq + 24576, &map_q, &ctrl.bar_load[st], 64, h, t0, b);
    if constexpr (!C::LATE) {
      issue_gates_pm(i, C::NB == 2 ? st : 0, &ctrl.bar_load[st]);
      issue_a(i, C::NB == 2 ? st : 0, &ctrl.bar_load[st]);
    }
  };
  auto prefetch_loads = [&](int i) {                         // one lane: next chunk's tiles into L2 (single-stage configuration)
    int t0, rows;
    chunk_info(i, t0, rows);
    const int64_t item = (static_cast<int64_t>(b) * p.NC + first + i) * p.H + h;
    tma_prefetch_4d(&map_k, 0, h, t0, b);
    tma_prefetch_4d(&map_q, 0, h, t0, b);
    tma_prefetch_4d(&map_k, 64, h, t0, b);
    tma_prefetch_4d(&map_q, 64, h, t0, b);
    bulk_prefetch(p.AP + item * (128 * 64), 16384);
    bulk_prefetch(p.Pm + item * (64 * 64), C::PM_BYTES);
    bulk_prefetch(p.gc + item * gate_item_floats(E) + 64 * E, C::GT_BYTES);
#pragma unroll
    for (int jb = 0; jb < VC / 8; ++jb) {
      tma_prefetch_4d(&map_do, vb * VC + jb * 8, h, t0, b);
      tma_prefetch_4d(&map_u, vb * VC + jb * 8, 0, static_cast<int>(item * 64), 0);
    }
  };
  auto prefetch_rows = [&](int i) {                          // the first warpgroup: what threads load themselves, for a later chunk -> L2
    if (wg != 0) return;
    int t0, rows;
    chunk_info(i, t0, rows);
    const int last = max(rows, 1) - 1;
    const int64_t ro = (static_cast<int64_t>(b) * p.T + t0 + min(t, last)) * p.H + h;
    if (krow) prefetch_l2(p.beta + ro);
  };
  // This thread's piece of a row of an operand image (i = t, j = v) that TMA filled: CW value columns as raw bf16
  auto image_piece = [&](const uint8_t* img) {
    const int v0 = cgp * CW;
    const uint8_t* src = img + (t >> 3) * 128 + (t & 7) * 16 + (v0 >> 3) * 1024 + (v0 & 7) * 2;
    if constexpr (CW == 8) {
      return *reinterpret_cast<const uint4*>(src);
    } else {
      const uint2 w = *reinterpret_cast<const uint2*>(src);
      return make_uint4(w.x, w.y, 0u, 0u);
    }
  };
  auto unpack_piece = [&](const uint4& w, bool use, float* out) {
    const uint32_t rw[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int c = 0; c < CW; ++c) out[c] = use ? ((c & 1) ? bf16_hi(rw[c >> 1]) : bf16_lo(rw[c >> 1])) : 0.f;
  };
  auto store_row_image = [&](uint32_t dst, const float* src, float f) {
    if constexpr (CW == 8)
      st_shared_v4(dst, pack_bf16(f * src[0], f * src[1]), pack_bf16(f * src[2], f * src[3]),
                   pack_bf16(f * src[4], f * src[5]), pack_bf16(f * src[6], f * src[7]));
    else
      st_shared_v2(dst, pack_bf16(f * src[0], f * src[1]), pack_bf16(f * src[2], f * src[3]));
  };
  // The same from a row that is already packed bf16 (CW/2 words), scaled by a factor in both halves of a packed pair: the
  // operand is bf16 either way, and the product of two bf16 values rounded once costs a fifth of the f32 route.
  auto store_row_image_scaled = [&](uint32_t dst, const uint32_t* w, float f) {
    const uint32_t ff = pack_bf16(f, f);
    if constexpr (CW == 8)
      st_shared_v4(dst, mul_bf16x2(w[0], ff), mul_bf16x2(w[1], ff), mul_bf16x2(w[2], ff), mul_bf16x2(w[3], ff));
    else
      st_shared_v2(dst, mul_bf16x2(w[0], ff), mul_bf16x2(w[1], ff));
  };
  // G_e of one chunk boundary, for the slices the state-gradient kernel will ask for: slice e as [v/8][d][v%8]
  auto store_state = [&](int64_t item, const uint32_t* packed) {
    uint8_t* base = reinterpret_cast<uint8_t*>(p.ds) + item * (static_cast<int64_t>(E) * 32768);
#pragma unroll
    for (int e = 0; e < EL; ++e) {
      if (!ftab[e0 + e]) continue;
      const int v0 = vb * VC + cgp * CW;
      uint8_t* dst = base + (e0 + e) * 32768 + (v0 >> 3) * 2048 + row * 16 + (v0 & 7) * 2;
      if constexpr (CW == 8) {
        *reinterpret_cast<uint4*>(dst) = make_uint4(packed[e * 4], packed[e * 4 + 1], packed[e * 4 + 2], packed[e * 4 + 3]);
      } else {
        *reinterpret_cast<uint2*>(dst) = make_uint2(packed[e * 2], packed[e * 2 + 1]);
      }
    }
  };
  auto decay_flag = [&](int64_t item, int e) {      // does d_e*dd_e of this chunk matter?  (same expression in the state-gradient kernel)
    return __ldg(p.gc + item * gate_item_floats(E) + 63 * E + e) * LOG2E >= DD_MIN_LOG2_DECAY ? 1 : 0;
  };

  if (warp_u == COPY_WARP && elect_one()) {                 // the lane that issues every load and every store of this CTA
    issue_loads(count - 1, 0);
    if constexpr (C::LATE) {
      mbar_expect_tx(&ctrl.bar_late, GATES_PM_TX);
      issue_gates_pm(count - 1, 0, &ctrl.bar_late);
      mbar_expect_tx(&ctrl.bar_a, C::A_BYTES);
      issue_a(count - 1, 0, &ctrl.bar_a);
    }
  }
  __syncwarp();
  if (count > 1) prefetch_rows(count - 2);
  uint32_t part_phase = 0;                            // completions of this thread's column part so far: two per chunk
  const int part = wg * TPC / C::PN;
  {
    // the gradient state at the end of the last chunk (zero unless handed in)
    if (tid < E) ftab[tid] = decay_flag((static_cast<int64_t>(b) * p.NC + first + count - 1) * p.H + h, tid);
    __syncthreads();
    uint32_t packed0[TPC / 2];
#pragma unroll
    for (int j = 0; j < TPC / 2; ++j) packed0[j] = pack_bf16(G[2 * j], G[2 * j + 1]);
    store_state((static_cast<int64_t>(b) * p.NC + first + count - 1) * p.H + h, packed0);
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
  }

  // The chunk decays of the chunk below decide whether its gradient state is stored; they are read a whole chunk before they
  // are looked at (the warp that reads them must not arrive late at the chunk's first barrier).
  // (A query-row warp without any other role reads them: the key-row warps are the critical path of the chunk's first phase.)
  constexpr int FLAG_WARP = 7;
  static_assert(NWG >= 2, "the flag warp is the last warp of the second warpgroup");
  const bool flag_lane = warp_u == FLAG_WARP && lane < E;
  auto decay_of = [&](int i) {                       // local chunk i, slice `lane` (lane < E)
    return __ldg(p.gc + ((static_cast<int64_t>(b) * p.NC + first + i) * p.H + h) * gate_item_floats(E) + 63 * E + lane);
  };
  float gl_below = (flag_lane && count > 1) ? decay_of(count - 2) : 0.f;
  for (int kstep = 0; kstep < count; ++kstep) {
    const int i = count - 1 - kstep;
    const float gl_use = gl_below;
    if (flag_lane && i > 1) gl_below = decay_of(i - 2);
    const int st = (STAGES == 2) ? (kstep & 1) : 0;
    int t0, rows;
    chunk_info(i, t0, rows);
    const int64_t item = (static_cast<int64_t>(b) * p.NC + first + i) * p.H + h;
    const int64_t tok = static_cast<int64_t>(b) * p.T + t0;
    const bool live = t < rows;
    uint8_t* kq = smem + C::OFF_KQ + st * C::KQ_BYTES;
    const int nbi = C::NB == 2 ? st : 0;             // which copy of Pm, A and the gate factors this chunk uses
    uint8_t* am = smem + C::OFF_A + nbi * C::A_BYTES;
    uint8_t* pm = smem + C::OFF_PM + nbi * C::PM_BYTES;
    const int v0 = cgp * CW;                         // first value column of this thread inside the block

    uint8_t* doimg = smem + C::OFF_DO + st * C::DOB;     // dO rows of the value block: operand image of Y, by TMA
    uint8_t* duimg = smem + C::OFF_DU + st * C::DOB;     // U rows by TMA, later the operand image of dU

    // ---- (a) KG = [K;Q] G and Y = Pm^T dO -----------------------------------------------------------------------
    mbar_wait(&ctrl.bar_load[st], (STAGES == 2 ? (kstep >> 1) : kstep) & 1, ctl, DEV_TIMEOUT_LOAD);
    if constexpr (C::LATE) mbar_wait(&ctrl.bar_late, kstep & 1, ctl, DEV_TIMEOUT_LOAD);
    if (warp_u == ISSUE_WARP && elect_one()) {
      tc_fence_after();
      {
        const uint64_t da = make_desc(smem_u32(pm), 128, 1024, LAYOUT_PLAIN);       // Pm^T: MN-major over (i = t, j = s)
        const uint64_t db = make_desc(smem_u32(doimg), 128, 1024, LAYOUT_PLAIN);
        constexpr uint32_t idesc = make_idesc(128, VC, 1, 1);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_bf16(tmem + TM_Y, desc_advance(da, kk * 256), desc_advance(db, kk * 256), idesc, kk > 0);
      }
      {
        const uint64_t da = make_desc(smem_u32(kq), 16, 1024, LAYOUT_SW128);
        const uint64_t db = make_desc(smem_u32(smem + C::OFF_GX), 128, 2048, LAYOUT_PLAIN);
        constexpr uint32_t idesc = make_idesc(128, C::PN, 0, 1);
#pragma unroll
        for (int pt = 0; pt < C::PARTS; ++pt) {       // Y and part 0 first; every commit covers all that was issued before it
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_bf16(tmem + pt * C::PN, desc_advance(da, (kk >> 2) * 16384 + (kk & 3) * 32),
                      desc_advance(db, pt * (C::PN / 8) * 2048 + kk * 256), idesc, kk > 0);
          umma_commit(&ctrl.bar_part[pt]);
        }
      }
    }
    __syncwarp();                                    // the other lanes must not run ahead into a spin wait
    if (warp_u == ISSUE_WARP) {
      // (p) P = G Xu^T goes out as soon as the key-row warps have built Xu (they do that first thing in this phase): it runs
      // behind (a), under the epilogue of (a), where the tensor core would otherwise idle, and nobody waits for it later.
      mbar_wait(&ctrl.bar_xu, kstep & 1, ctl, DEV_TIMEOUT_MMA);
      if (elect_one()) {
        tc_fence_after();
        const uint64_t da = make_desc(smem_u32(smem + C::OFF_GX), 2048, 128, LAYOUT_PLAIN);   // G: K-major over (i = d, j = n')
        const uint64_t db = make_desc(smem_u32(smem + C::OFF_XU), 1024, 128, LAYOUT_PLAIN);   // Xu: K-major over (i = t, j = n')
        constexpr uint32_t idesc = make_idesc(128, 64, 0, 0);
#pragma unroll
        for (int kk = 0; kk < NCOLS / 16; ++kk)
          umma_bf16(tmem + TM_P, desc_advance(da, kk * 4096), desc_advance(db, kk * 2048), idesc, kk > 0);
        umma_commit(&ctrl.bar_p);
      }
      __syncwarp();
    }
    if (warp_u == COPY_WARP && kstep + 1 < count && elect_one()) {
      if (STAGES == 2) issue_loads(i - 1, st ^ 1); else prefetch_loads(i - 1);
    }
    __syncwarp();
    // Under the MMA: this row's gate factors, and (K-row threads, which would otherwise only wait for the MMA) the operand
    // Xu of (p).
    float ga[EL];                                    // this thread's slices.  K rows: a_e = k2 exp(gc); Q rows: c_e = scale q2 exp(gc)
    float gr[EL];                                    // K rows: r_e = k2 exp(gL - gc)
    float bt = 0.f;
    {
      const float* gf = reinterpret_cast<const float*>(smem + C::OFF_GT + nbi * C::GT_STRIDE);
      rec_lds_part<EL>(gf + (krow ? 0 : C::GF_C) + t * E + e0, ga);
      if (krow) {
        rec_lds_part<EL>(gf + C::GF_R + t * E + e0, gr);
        bt = __ldg(p.beta + (tok + min(t, max(rows, 1) - 1)) * p.H + h);   // masked where it is used, after (c): nothing here waits for it
        const uint4 up = image_piece(duimg);
        const uint32_t uw[4] = {up.x, up.y, up.z, up.w};
        // Xu_e = r_e * U -> operand image (i = t, j = n') of (p)
        const uint32_t base = smem_u32(smem + C::OFF_XU) + (t >> 3) * 128 + (t & 7) * 16;
#pragma unroll
        for (int e = 0; e < EL; ++e) {
          const int n0 = wg * TPC + e * CW;
          store_row_image_scaled(base + (n0 >> 3) * 1024 + (n0 & 7) * 2, uw, gr[e]);
        }
        fence_async_smem();                            // Xu is read by the tensor core: say so, one arrival per key-row warp
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctrl.bar_xu);
      } else {
#pragma unroll
        for (int e = 0; e < EL; ++e) gr[e] = 0.f;
      }
      if (tid < E) dtab[tid] = gf[C::GF_D + tid];
      if (flag_lane && i > 0) {
        float glv = gl_use;
        asm volatile("" : "+f"(glv));                // the comparison stays here: nothing waits for the load before this point
        ftab[lane] = glv * LOG2E >= DD_MIN_LOG2_DECAY ? 1 : 0;   // read after the chunk's last barrier but one
      }
      if (kstep + 2 < count) prefetch_rows(i - 2);
    }
    mbar_wait_spin(&ctrl.bar_part[part], part_phase & 1, ctl, DEV_TIMEOUT_MMA);
    ++part_phase;
    tc_fence_after();
    float du[CW];                                    // K rows: dU of this thread's columns (NSG > 1: its slice group's part)
    if (krow) {
      float uv[CW];
      unpack_piece(image_piece(duimg), true, uv);
      constexpr int EP = (8 / CW) < 1 ? 1 : (8 / CW) < EL ? (8 / CW) : EL;   // slices per piece of eight columns
      constexpr int NP = EL / EP;
      float kg[2][EP * CW];
      if (sgp == 0) {
        tmem_ld<CW>(tmem_row + TM_Y + v0, du);
      } else {
#pragma unroll
        for (int c = 0; c < CW; ++c) du[c] = 0.f;
      }
      tmem_ld<EP * CW>(tmem_row + wg * TPC, kg[0]);
#pragma unroll
      for (int pc = 0; pc < NP; ++pc) {                       // the next piece travels while this one is used
        tmem_wait_ld();
        if (pc + 1 < NP) tmem_ld<EP * CW>(tmem_row + wg * TPC + (pc + 1) * EP * CW, kg[(pc + 1) & 1]);
        const float* kp = kg[pc & 1];
#pragma unroll
        for (int ee = 0; ee < EP; ++ee) {
          const float re = gr[pc * EP + ee];
          float dot = 0.f;
#pragma unroll
          for (int c = 0; c < CW; ++c) {
            du[c] = fmaf(re, kp[ee * CW + c], du[c]);
            dot = fmaf(uv[c], kp[ee * CW + c], dot);
          }
          drp[(cgp * 64 + t) * ES + e0 + pc * EP + ee] = dot;
        }
      }
      if constexpr (NSG > 1) {
        static_assert(NSG <= 2 && (NSG == 1 || CW % 4 == 0), "the exchange below is written for two slice groups");
        if (sgp != 0) {
#pragma unroll
          for (int c = 0; c < CW; c += 4)
            *reinterpret_cast<float4*>(dured + t * VC + v0 + c) = make_float4(du[c], du[c + 1], du[c + 2], du[c + 3]);
        }
      }
    }
    if constexpr (NSG > 1) __syncthreads();          // the other slice group's part of dU; every reader of the U piece is done
    if (krow && sgp == 0) {
      if constexpr (NSG > 1) {
#pragma unroll
        for (int c = 0; c < CW; c += 4) {
          const float4 x = *reinterpret_cast<const float4*>(dured + t * VC + v0 + c);
          du[c] += x.x; du[c + 1] += x.y; du[c + 2] += x.z; du[c + 3] += x.w;
        }
      }
      // dU replaces this thread's piece of U in the image; the image then leaves for global memory by a TMA store
      store_row_image(smem_u32(duimg) + (t >> 3) * 128 + (v0 >> 3) * 1024 + (t & 7) * 16 + (v0 & 7) * 2, du, 1.f);
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();

    // ---- (c) Z = A^T dU -----------------------------------------------------------------------------------------
    if constexpr (C::LATE) {
      // Pm was last read by the MMAs of (a) and the gate factors by every thread before the barrier above: the next chunk's
      // copies are asked for now and have the rest of the chunk to arrive.  A, which (c) is about to read, has its own
      // barrier and was asked for when the previous chunk's (c) had completed.
      if (warp_u == COPY_WARP && kstep + 1 < count && elect_one()) {
        mbar_expect_tx(&ctrl.bar_late, GATES_PM_TX);
        issue_gates_pm(i - 1, 0, &ctrl.bar_late);
      }
      __syncwarp();
      if (warp_u == ISSUE_WARP) mbar_wait(&ctrl.bar_a, kstep & 1, ctl, DEV_TIMEOUT_LOAD);
    }
    if (warp_u == ISSUE_WARP && elect_one()) {
      tc_fence_after();
      {
        const uint64_t da = make_desc(smem_u32(am), 128, 1024, LAYOUT_PLAIN);         // A^T: MN-major over (i = t, j = s)
        const uint64_t db = make_desc(smem_u32(duimg), 128, 1024, LAYOUT_PLAIN);
        constexpr uint32_t idesc = make_idesc(128, VC, 1, 1);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_bf16(tmem + TM_Z, desc_advance(da, kk * 256), desc_advance(db, kk * 256), idesc, kk > 0);
        umma_commit(&ctrl.bar_mma);
      }
    }
    __syncwarp();                                    // the other lanes must not run ahead into a spin wait
    if (warp_u == COPY_WARP && elect_one()) {                // dU (chunk layout) straight from its operand image
#pragma unroll
      for (int jb = 0; jb < VC / 8; ++jb)
        tma_store_4d(&map_du, duimg + jb * 1024, vb * VC + jb * 8, 0, static_cast<int>(item * 64), 0);
      bulk_commit_group();
    }
    __syncwarp();
    // meanwhile: the value-block partial of dr, summed over the warpgroups in a fixed order
    for (int idx = tid; idx < 64 * E; idx += REC_THREADS) {
      const int r = idx / E, e = idx % E;
      float s4 = 0.f;
#pragma unroll
      for (int w = 0; w < NCG; ++w) s4 += drp[(w * 64 + r) * ES + e];
      p.dr[((item * NV + vb) * 64 + r) * E + e] = s4;
    }
    mbar_wait_spin(&ctrl.bar_mma, kstep & 1, ctl, DEV_TIMEOUT_MMA);
    tc_fence_after();
    if constexpr (C::LATE) {                         // (c) has read A: the next chunk's copy may land
      if (warp_u == COPY_WARP && kstep + 1 < count && elect_one()) {
        mbar_expect_tx(&ctrl.bar_a, C::A_BYTES);
        issue_a(i - 1, 0, &ctrl.bar_a);
      }
      __syncwarp();
    }
    {
      uint32_t xw[4] = {0u, 0u, 0u, 0u};             // K rows: dW; Q rows: dO; packed bf16, the form both leave in
      if (krow) {
        float z[CW];
        tmem_ld<CW>(tmem_row + TM_Z + v0, z);
        tmem_wait_ld();
        asm volatile("" : "+f"(bt));                   // first use of the beta load of phase (a)
        if (!live) bt = 0.f;
#pragma unroll
        for (int c = 0; c < CW; c += 2) xw[c >> 1] = pack_bf16(bt * z[c], bt * z[c + 1]);
        if (live && sgp == 0) {
          __nv_bfloat16* dst = p.dV + ((tok + t) * p.H + h) * HEAD + vb * VC + v0;
          if constexpr (CW == 8) *reinterpret_cast<uint4*>(dst) = make_uint4(xw[0], xw[1], xw[2], xw[3]);
          else *reinterpret_cast<uint2*>(dst) = make_uint2(xw[0], xw[1]);
        }
      } else if (live) {
        const uint4 w = image_piece(doimg);
        xw[0] = w.x; xw[1] = w.y; xw[2] = w.z; xw[3] = w.w;
      }
      // (p) reads the image of G that X is about to replace
      mbar_wait_spin(&ctrl.bar_p, kstep & 1, ctl, DEV_TIMEOUT_MMA);
      // X image (i = row, j = n'): rows 0..63 -a_e*dW, rows 64..127 c_e*dO
      const uint32_t base = smem_u32(smem + C::OFF_GX) + (row >> 3) * 128 + (row & 7) * 16;
#pragma unroll
      for (int e = 0; e < EL; ++e) {
        const float f = krow ? -ga[e] : ga[e];
        const int n0 = wg * TPC + e * CW;
        store_row_image_scaled(base + (n0 >> 3) * 2048 + (n0 & 7) * 2, xw, f);
      }
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();

    // ---- (d) dG = [K^T | Q^T] X, G <- d G + dG ------------------------------------------------------------------
    if (warp_u == ISSUE_WARP && elect_one()) {
      tc_fence_after();
      const uint64_t da = make_desc(smem_u32(kq), 16384, 1024, LAYOUT_SW128);
      const uint64_t db = make_desc(smem_u32(smem + C::OFF_GX), 128, 2048, LAYOUT_PLAIN);
      constexpr uint32_t idesc = make_idesc(128, C::PN, 1, 1);
#pragma unroll
      for (int pt = 0; pt < C::PARTS; ++pt) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_bf16(tmem + pt * C::PN, desc_advance(da, kk * 2048), desc_advance(db, pt * (C::PN / 8) * 2048 + kk * 256), idesc, kk > 0);
        umma_commit(&ctrl.bar_part[pt]);
      }
    }
    __syncwarp();                                    // the other lanes must not run ahead into a spin wait
    // meanwhile: P (128 key rows x 64 tokens, f32) -> bf16 operand image (i = d, j = t), SI = 128, SJ = 2048, of this
    // value block: a warp's 16-byte stores cover 512 contiguous bytes
    {
      tc_fence_after();
      constexpr int PW = 64 / NWG;                   // token columns per warpgroup
      uint8_t* dst = reinterpret_cast<uint8_t*>(p.dkg) + (item * NV + vb) * 16384 + row * 16;
#pragma unroll
      for (int c0 = 0; c0 < PW; c0 += 16) {
        float pv[16];
        tmem_ld<16>(tmem_row + TM_P + wg * PW + c0, pv);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; j += 8)
          *reinterpret_cast<uint4*>(dst + ((wg * PW + c0 + j) >> 3) * 2048) =
              make_uint4(pack_bf16(pv[j], pv[j + 1]), pack_bf16(pv[j + 2], pv[j + 3]), pack_bf16(pv[j + 4], pv[j + 5]),
                         pack_bf16(pv[j + 6], pv[j + 7]));
      }
    }
    mbar_wait_spin(&ctrl.bar_part[part], part_phase & 1, ctl, DEV_TIMEOUT_MMA);
    ++part_phase;
    tc_fence_after();
    if constexpr (STAGES == 1) {                     // the only stage is free once every part of (d) has completed
      if (warp_u == COPY_WARP) mbar_wait_spin(&ctrl.bar_part[C::PARTS - 1], (part_phase - 1) & 1, ctl, DEV_TIMEOUT_MMA);
      if (warp_u == COPY_WARP && kstep + 1 < count && elect_one()) issue_loads(i - 1, 0);
    }
    __syncwarp();
    {
      constexpr int PIECE = TPC < 16 ? TPC : 16;
      const uint32_t base = smem_u32(smem + C::OFF_GX) + (row >> 3) * 128 + (row & 7) * 16;
      uint8_t* sbase = i > 0 ? reinterpret_cast<uint8_t*>(p.ds) + (item - p.H) * (static_cast<int64_t>(E) * 32768) : nullptr;
      const int vg = vb * VC + cgp * CW;
      float dg[2][PIECE];
      tmem_ld<PIECE>(tmem_row + wg * TPC, dg[0]);
#pragma unroll
      for (int j0 = 0; j0 < TPC; j0 += PIECE) {               // the next piece travels while this one is used
        tmem_wait_ld();
        if (j0 + PIECE < TPC) tmem_ld<PIECE>(tmem_row + wg * TPC + j0 + PIECE, dg[((j0 / PIECE) + 1) & 1]);
        const float* dp = dg[(j0 / PIECE) & 1];
        uint32_t packed[PIECE / 2];
#pragma unroll
        for (int j = 0; j < PIECE; j += 2) {
          G[j0 + j] = fmaf(dtab[e0 + (j0 + j) / CW], G[j0 + j], dp[j]);
          G[j0 + j + 1] = fmaf(dtab[e0 + (j0 + j + 1) / CW], G[j0 + j + 1], dp[j + 1]);
          packed[j / 2] = pack_bf16(G[j0 + j], G[j0 + j + 1]);
        }
        // operand image (i = d, j = n') of the next (a)
#pragma unroll
        for (int j = 0; j < PIECE; j += 8) {
          const int n0 = wg * TPC + j0 + j;
          st_shared_v4(base + (n0 >> 3) * 2048, packed[j / 2], packed[j / 2 + 1], packed[j / 2 + 2], packed[j / 2 + 3]);
        }
        // G_e at the end of the previous chunk, for the slices the state-gradient kernel will ask for: [v/8][d][v%8]
        if (sbase != nullptr) {
#pragma unroll
          for (int j = 0; j < PIECE; j += CW) {
            const int e = e0 + (j0 + j) / CW;
            if (!ftab[e]) continue;
            uint8_t* dst = sbase + e * 32768 + (vg >> 3) * 2048 + row * 16 + (vg & 7) * 2;
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
  // dL/dS before the first token, for an earlier segment of the same sequence
  if (p.g_out != nullptr) {
    float* dst = p.g_out + ((static_cast<int64_t>(seq) * p.H + h) * E + e0) * (HEAD * HEAD) + row * HEAD + vb * VC + cgp * CW;
#pragma unroll
    for (int e = 0; e < EL; ++e)
#pragma unroll
      for (int c = 0; c < CW; c += 4)
        *reinterpret_cast<float4*>(dst + e * (HEAD * HEAD) + c) = make_float4(G[e * CW + c], G[e * CW + c + 1], G[e * CW + c + 2], G[e * CW + c + 3]);
  }
  if (warp_u == COPY_WARP && elect_one()) bulk_wait_group();   // the last store of dU reads shared memory of this CTA
  __syncwarp();
  if (warp == 0) tmem_dealloc(tmem, C::TMEM_COLS);
}

}  // namespace tgdn

using namespace tgdn;

template <int E, int VC, int NWG, int STAGES, int NSG = 1>
static int launch_rec(const CUtensorMap& mk, const CUtensorMap& mq,
                      const CUtensorMap& mdo, const CUtensorMap& mu, const CUtensorMap& mdu, const RecParams& p, cudaStream_t s) {
  using C = RecCfg<E, VC, NWG, STAGES, NSG>;
  static_assert(STAGES == 2 || C::SMEM_BYTES <= 115712, "two CTAs per SM need at most 113 KB each");
  static_assert(C::SMEM_BYTES <= 232448, "shared memory budget of one CTA exceeded");
  static_assert((STAGES == 1 ? 2 : 1) * C::TMEM_COLS <= 512, "tensor memory budget of one SM exceeded");
  static_assert(64 % NWG == 0 && (64 / NWG) % 16 == 0, "the readout of P splits 64 token columns over the warpgroups in pieces of 16");
  static bool configured[64] = {};                  // per device: the attribute is sticky, set it once
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(rec_kernel<E, VC, NWG, STAGES, NSG>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return tgdn_cuda_error(e);
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  const int grid = p.n_seq * p.H * (HEAD / VC);
  rec_kernel<E, VC, NWG, STAGES, NSG><<<grid, C::THREADS, C::SMEM_BYTES, s>>>(mk, mq, mdo, mu, mdu, p);
  return tgdn_cuda_error(cudaGetLastError());
}

extern "C" int tgdn_bwd_recurrent_state(const void* q, const void* k, const void* dO, const float* k2, const float* q2,
                                        const float* beta, const float* gc, const void* AP, const void* Pm, const void* U,
                                        float scale, const int32_t* doc_offsets, const int32_t* chunk_map, int n_docs, int B,
                                        int T, int H, int E, int NC, void* dV, void* dU, void* ds, void* dkg, float* dr,
                                        const float* grad_state_in, float* grad_state_out, void* stream) {
  if ((reinterpret_cast<uintptr_t>(grad_state_in) | reinterpret_cast<uintptr_t>(grad_state_out)) & 15) return TGDN_ERR_ALIGN;
  if (!q || !k || !dO || !k2 || !q2 || !beta || !gc || !AP || !Pm || !U || !dV || !dU || !ds || !dkg || !dr) return TGDN_ERR_NULL;
  const bool packed = chunk_map != nullptr;
  if (packed && (!doc_offsets || n_docs < 1)) return TGDN_ERR_NULL;
  int rc = tgdn_check_core_shape(B, T, H, E, NC, packed);
  if (rc) return rc;
  if ((reinterpret_cast<uintptr_t>(dO) | reinterpret_cast<uintptr_t>(AP) | reinterpret_cast<uintptr_t>(Pm) |
       reinterpret_cast<uintptr_t>(U) | reinterpret_cast<uintptr_t>(dV) | reinterpret_cast<uintptr_t>(dU) |
       reinterpret_cast<uintptr_t>(ds) | reinterpret_cast<uintptr_t>(dkg) | reinterpret_cast<uintptr_t>(k2) |
       reinterpret_cast<uintptr_t>(q2) | reinterpret_cast<uintptr_t>(gc)) & 15)
    return TGDN_ERR_ALIGN;
  CUtensorMap mk, mq;
  if ((rc = tgdn_make_token_map(&mk, k, B, T, H, 64, 64, 1))) return rc;
  if ((rc = tgdn_make_token_map(&mq, q, B, T, H, 64, 64, 1))) return rc;
  // dO (token layout) and U, dU (chunk layout: item * 64 + t rows of 128 columns) in boxes of 8 columns x 64 rows
  const int64_t crows = static_cast<int64_t>(B) * NC * H * 64;
  if (crows > 0x7fffffffLL) return TGDN_ERR_SHAPE;
  CUtensorMap mdo, mu, mdu;
  if ((rc = tgdn_make_token_map(&mdo, dO, B, T, H, 8, 64, 0))) return rc;
  if ((rc = tgdn_make_token_map(&mu, U, 1, static_cast<int>(crows), 1, 8, 64, 0))) return rc;
  if ((rc = tgdn_make_token_map(&mdu, dU, 1, static_cast<int>(crows), 1, 8, 64, 0))) return rc;
  RecParams p{static_cast<const __nv_bfloat16*>(dO), k2, q2, beta, gc, static_cast<const __nv_bfloat16*>(AP),
              static_cast<const __nv_bfloat16*>(Pm), static_cast<const __nv_bfloat16*>(U),
              static_cast<__nv_bfloat16*>(dV), static_cast<__nv_bfloat16*>(dU), static_cast<__nv_bfloat16*>(ds),
              static_cast<__nv_bfloat16*>(dkg), dr, doc_offsets, chunk_map, B, T, H, NC, packed ? n_docs : B, scale,
              tgdn_status_word(), grad_state_in, grad_state_out};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (E) {
    case 1: return launch_rec<1, 32, 4, 2>(mk, mq, mdo, mu, mdu, p, s);
    case 2: return launch_rec<2, 32, 4, 2>(mk, mq, mdo, mu, mdu, p, s);
    case 4: return launch_rec<4, 32, 4, 2>(mk, mq, mdo, mu, mdu, p, s);
    // E = 8: four warpgroups on 32 value columns with a two-stage ring, one CTA per SM, measured 9% faster than two CTAs
    // per SM of two warpgroups on 16 columns each (5.26 -> 4.77 ms at B=8, T=8192, H=32), and the state-gradient kernel
    // then adds four value-block images per item instead of eight.
    case 8: return launch_rec<8, 32, 4, 2>(mk, mq, mdo, mu, mdu, p, s);
    case 12: return launch_rec<12, 16, 4, 2, 2>(mk, mq, mdo, mu, mdu, p, s);
    case 16: return launch_rec<16, 16, 4, 2, 2>(mk, mq, mdo, mu, mdu, p, s);
    default: return TGDN_ERR_SHAPE;
  }
}

extern "C" int tgdn_bwd_recurrent(const void* q, const void* k, const void* dO, const float* k2, const float* q2,
                                  const float* beta, const float* gc, const void* AP, const void* Pm, const void* U,
                                  float scale, const int32_t* doc_offsets, const int32_t* chunk_map, int n_docs, int B,
                                  int T, int H, int E, int NC, void* dV, void* dU, void* ds, void* dkg, float* dr,
                                  void* stream) {
  return tgdn_bwd_recurrent_state(q, k, dO, k2, q2, beta, gc, AP, Pm, U, scale, doc_offsets, chunk_map, n_docs, B, T, H, E, NC,
                                  dV, dU, ds, dkg, dr, nullptr, nullptr, stream);
}
