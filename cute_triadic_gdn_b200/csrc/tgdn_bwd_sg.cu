// State gradients of the Triadic GDN backward: everything that contracts over the value axis with the saved forward states.
//
// Persistent CTAs (one per SM), each walking (batch, chunk, head) items: 256 worker threads, one warp that only issues the MMAs and one
// that only issues the bulk loads, so that instruction issue to the tensor core never sits on the workers' path, and the loads of the
// next item's first ring round travel while the workers finish one item and open the next.  With h_e the forward state at the start of the chunk
// (128x128 bf16, streamed from HBM in 16 KB half-slices by bulk copies):
//   dK_state = sum_e (-a_e*dW) h_e^T + sum_blocks P_block^T     (64 x 128)
//   dQ_state = sum_e ( c_e*dO) h_e^T                            (64 x 128)
//   da_e[t]  = -sum_v dW[t,v] (K h_e)[t,v]     dc_e[t] = sum_v dO[t,v] (Q h_e)[t,v]     dd_e = <h_e, G_e>
// P_block = sum_e G_e (r_e*U)^T over one block of value columns is formed by the reverse recurrence, where G lives, and
// arrives as 128/VC bf16 operand images of 16 KB; they are added up, transposed, by the tensor core itself: one product
// [I;0] P_block^T per image accumulates into the dK tile in tensor memory (exact: every term is a bf16 value times one).
// The tensor core forms, per slice, P_e = [dW ; dO] h_e^T (128 x 128, f32 in tensor memory, contraction over the value
// axis in two half-slice steps) from the raw [dW ; dO] tile, which TMA loads once: the workers then take both the row
// sums (da_e[t] = -<K[t], P_e[t]>, dc_e[t] = <Q[t], P_e[t]>: the same numbers as the sums over v above, with the
// contractions exchanged) and the gate-weighted accumulation over the slices (f32, in registers) from one read of P_e.
// dd_e enters the result only as exp(gL_e)*dd_e; it is the trace of one more product, h_e G_e^T, formed only for the
// slices whose chunk decay exp(gL_e) is at least 2^-24: only for those does the reverse recurrence store G_e, and only
// those half-slices of G are loaded here (for the others dd_e = 0, an error below 2^-24 of <h_e, G_e>).
//
// Replaces cute_triadic_gdn/kernels/sm100_joint_state_grads.py:53-449 (sg_kernel).
#include <type_traits>

#include "tgdn_common.cuh"
#include "tgdn_host.h"
#include "tgdn_kernels.h"

namespace tgdn {

constexpr int SG_THREADS = 256;      // eight worker warps ...
constexpr int SG_BLOCK = SG_THREADS + 64;   // ... plus one warp that only issues MMAs and one that only issues bulk loads
constexpr int PF_AHEAD = 8;          // half-slices of h pulled into L2 ahead of the ring's own loads

// Four ring stages: about two half-slice pairs (64 KB) travel while two more wait for their MMAs.  Measured at E = 8:
// three stages are 3% slower, five were slower too.
template <int E>
struct SgSmem {
  static constexpr int ES = E | 1;   // row stride of the gate tables and partials (odd: conflict-free)
  static constexpr int NSTAGE = 4;
  uint8_t xt[32768];            // [dW ; dO] tile, 128B swizzle: two column halves of 128 rows x 64 columns
  uint8_t hp[NSTAGE][16384];    // half-slices of h: image (i = d, j = v), SI = 128, SJ = 2048
  uint8_t gp[NSTAGE][16384];    // first the value-block images of sum_e G_e (r_e U)^T, then half-slices of G (slices with a trace only)
  uint8_t ident[16384];         // [I;0], image (i = row 0..127, j = k 0..63), SI = 128, SJ = 2048
  float ga[64 * ES], gcq[64 * ES];
  float part[2 * 128 * ES];     // row sums per half of the key axis
  float red[E * 4];             // per slice and 32-row block: partial trace of h_e G_e^T
  int flag[16];                 // per slice: is exp(gL_e) large enough for dd_e to matter?
  uint64_t bar_kq, bar_load[NSTAGE], bar_g[NSTAGE], bar_pt[NSTAGE], bar_pfree[NSTAGE], bar_mma[2], bar_pread[2], bar_read[NSTAGE], bar_diag;
  uint32_t tmem_base;
  int abort;
};

template <int E>
__global__ void __launch_bounds__(SG_BLOCK, 1)
sg_kernel(const __grid_constant__ CUtensorMap map_dv, const __grid_constant__ CUtensorMap map_do, SgParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  using SM = SgSmem<E>;
  SM& sm = *reinterpret_cast<SM*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int ES = SM::ES, NS = SM::NSTAGE;
  constexpr float LOG2E = 1.4426950408889634f;
  constexpr int STEPS = 2 * E;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool worker = warp < SG_THREADS / 32;
  const bool issuer = tid == SG_THREADS;             // first lane of the first extra warp
  const int warp_u = __shfl_sync(0xffffffffu, warp, 0);   // warp index as a warp-uniform value
  const int wg = (warp >> 2) & 1;                    // half of the key axis (P_e, outputs) and of a step's 64 value columns (U)
  const int row = (warp & 3) * 32 + lane;
  const bool krow = row < 64;
  const int t = row & 63;
  const int NVB = p.NV;
  const int64_t n_items = static_cast<int64_t>(p.B) * p.NC * p.H;

  // The CTA is persistent: it walks the items blockIdx.x, blockIdx.x + gridDim.x, ... and keeps its barriers, its tensor
  // memory and the [I;0] operand.  While the workers finish one item (epilogue) and start the next (prologue), the loads of
  // the next item's first ring round are already in flight.
  auto item_rows = [&](int64_t item, int& t0, int& rows) {       // false: nothing to do for this item
    const int n = (static_cast<int>(item) / p.H) % p.NC;   // items fit in 32 bits (checked at the entry point); 64-bit divisions are slow
    t0 = n * CHUNK;
    rows = CHUNK;
    if (p.cmap != nullptr) {
      t0 = p.cmap[n];
      rows = p.cmap[p.NC + n];
      if (rows <= 0) return false;                       // unused tail of the chunk map
      if (t0 < 0 || rows > CHUNK || t0 + rows > p.T) {   // never follow a bad map entry
        atomicCAS(p.status, DEV_OK, DEV_BAD_CHUNK_MAP);
        return false;
      }
    }
    return true;
  };
  auto next_item = [&](int64_t from, int& t0, int& rows) {       // first item >= from (in steps of the grid) with work
    int64_t it = from;
    while (it < n_items && !item_rows(it, t0, rows)) it += gridDim.x;
    return it;
  };
  WaitCtl ctl{&sm.abort, p.status};
  auto issue_h = [&](int64_t item, int s) {            // one lane: half-slice s of h
    const int st = s % NS;
    mbar_expect_tx(&sm.bar_load[st], 16384);
    bulk_load(sm.hp[st], reinterpret_cast<const uint8_t*>(p.h) + item * (static_cast<int64_t>(E) * 32768) + s * 16384, 16384,
              &sm.bar_load[st]);
  };
  auto issue_g = [&](int64_t item, int s) {            // one lane: half-slice s of G (slices with a trace only)
    const int st = s % NS;
    mbar_expect_tx(&sm.bar_g[st], 16384);
    bulk_load(sm.gp[st], reinterpret_cast<const uint8_t*>(p.ds) + item * (static_cast<int64_t>(E) * 32768) + s * 16384, 16384,
              &sm.bar_g[st]);
  };
  auto issue_block = [&](int64_t item, int u) {        // one lane: value-block image u of the G part of dK
    const int st = u % NS;
    mbar_expect_tx(&sm.bar_pt[st], 16384);
    bulk_load(sm.gp[st], reinterpret_cast<const uint8_t*>(p.dkg) + item * (static_cast<int64_t>(NVB) * 16384) + u * 16384, 16384,
              &sm.bar_pt[st]);
  };
  auto issue_first_round = [&](int64_t item, int t0) { // one lane: the [dW ; dO] tile and the first ring round of an item
    const int h = static_cast<int>(item) % p.H, b = static_cast<int>(item) / (p.H * p.NC);
    mbar_expect_tx(&sm.bar_kq, 32768);
    tma_load_4d(sm.xt, &map_dv, &sm.bar_kq, 0, h, t0, b);
    tma_load_4d(sm.xt + 8192, &map_do, &sm.bar_kq, 0, h, t0, b);
    tma_load_4d(sm.xt + 16384, &map_dv, &sm.bar_kq, 64, h, t0, b);
    tma_load_4d(sm.xt + 24576, &map_do, &sm.bar_kq, 64, h, t0, b);
    for (int u = 0; u < NS && u < NVB; ++u) issue_block(item, u);
    for (int s = 0; s < NS && s < STEPS; ++s) issue_h(item, s);
  };

  int t0 = 0, rows = 0;
  int64_t item = next_item(blockIdx.x, t0, rows);
  if (item >= n_items) return;
  if (issuer) {
    mbar_init(&sm.bar_kq, 1);
    for (int i = 0; i < NS; ++i) {
      mbar_init(&sm.bar_load[i], 1);
      mbar_init(&sm.bar_g[i], 1);
      mbar_init(&sm.bar_pt[i], 1);
      mbar_init(&sm.bar_pfree[i], 1);
    }
    mbar_init(&sm.bar_mma[0], 1);
    mbar_init(&sm.bar_mma[1], 1);
    mbar_init(&sm.bar_pread[0], SG_THREADS / 32);
    mbar_init(&sm.bar_pread[1], SG_THREADS / 32);
    for (int i = 0; i < NS; ++i) mbar_init(&sm.bar_read[i], SG_THREADS / 32);
    mbar_init(&sm.bar_diag, 4);
    mbar_fence_init();
    sm.abort = 0;
    issue_first_round(item, t0);                       // every stage is free at the start
  }
  if (warp_u == 0) { tmem_alloc(&sm.tmem_base, 512); tmem_relinquish(); }
  // [I;0]: the operand that adds the value-block images, transposed, into the dK tile
  if (worker) {
    for (int i = tid; i < 16384 / 16; i += SG_THREADS) reinterpret_cast<uint4*>(sm.ident)[i] = make_uint4(0, 0, 0, 0);
  }
  __syncthreads();                                     // the zeroed operand before its diagonal
  if (tid < 64) *reinterpret_cast<uint16_t*>(sm.ident + img_off(tid, tid, 128, 2048)) = 0x3F80;   // bf16 1.0
  fence_async_smem();
  tc_fence_before();
  __syncthreads();                                     // barriers, operand and the tensor-memory address are visible
  tc_fence_after();
  const uint32_t tmem = __shfl_sync(0xffffffffu, sm.tmem_base, 0);
  const uint32_t tmem_row = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);

  // Barrier phases run on from item to item.  Every wait below is written with the phase parity it would have in the
  // CTA's first item; `ph` holds, per barrier, the parity of the completions of all earlier items.
  //   completions per item: bar_kq 1; bar_load / bar_read stage st: the steps s = st (mod NS); bar_pt / bar_pfree stage st:
  //   the images u = st (mod NS); bar_mma[0], bar_mma[1], bar_diag: E; bar_pread[b]: the slices e = b (mod 2);
  //   bar_g: counted as they happen (g_uses).
  constexpr uint32_t ODD_STEP = []() { uint32_t m = 0; for (int st = 0; st < NS; ++st) { int c = 0; for (int s = st; s < STEPS; s += NS) ++c; m |= (c & 1u) << st; } return m; }();
  uint32_t odd_img = 0;
  for (int st = 0; st < NS; ++st) { int c = 0; for (int u = st; u < NVB; u += NS) ++c; odd_img |= (c & 1u) << st; }
  constexpr uint32_t ODD_PREAD = (((E + 1) / 2) & 1u) | (((E / 2) & 1u) << 1);
  uint32_t ph_kq = 0, ph_step = 0, ph_img = 0, ph_e = 0, ph_pread = 0;
  uint32_t g_uses[NS];                                 // completed loads per stage of the G ring (slices with a trace only)
#pragma unroll
  for (int i = 0; i < NS; ++i) g_uses[i] = 0;

  // chunk decays of an item, one lane per slice of the two extra warps: they decide per slice whether a trace is taken
  auto load_gl = [&](int64_t it) {
    return (!worker && lane < E && it < n_items) ? __ldg(p.gc + it * gate_item_floats(E) + 63 * E + lane) : 0.f;
  };
  float my_gl = load_gl(item);

  while (item < n_items) {
    int t0n = 0, rowsn = 0;
    const int64_t nxt = next_item(item + gridDim.x, t0n, rowsn);
    const float next_gl = load_gl(nxt);                // asked for a whole item ahead
    const int h = static_cast<int>(item) % p.H, b = static_cast<int>(item) / (p.H * p.NC);
    const uint32_t fmask = __ballot_sync(0xffffffffu, !worker && lane < E && my_gl * LOG2E >= DD_MIN_LOG2_DECAY);

    // ---- workers: prologue.  All global loads go out together, from clamped (always valid) addresses, and are masked when
    // they are used; the tensor core is meanwhile adding the value-block images and forming the first P tiles, which need
    // no gate.
    const int64_t tok = static_cast<int64_t>(b) * p.T + t0;
    uint32_t kw[32];                                   // this thread's K row (Q row) over the key columns wg*64 .. +64, packed bf16 pairs
    if (worker) {
      const int tl = min(t, rows - 1);
      const __nv_bfloat16* ksrc = (krow ? p.k : p.q) + ((tok + tl) * p.H + h) * HEAD + wg * 64;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint4 x = __ldg(reinterpret_cast<const uint4*>(ksrc) + j);
        kw[4 * j] = x.x; kw[4 * j + 1] = x.y; kw[4 * j + 2] = x.z; kw[4 * j + 3] = x.w;
      }
      // the gate factors a = k2 exp(gc) and c = scale q2 exp(gc) of the chunk, as the masks kernel stored them (zero in rows
      // past a document end)
      constexpr int GATE_ITERS = (64 * E + SG_THREADS - 1) / SG_THREADS;
      float raw_a[GATE_ITERS], raw_c[GATE_ITERS];
      float raw_gl = 0.f;
      const float* gcp = p.gc + item * gate_item_floats(E);
#pragma unroll
      for (int it = 0; it < GATE_ITERS; ++it) {
        const int idx = min(tid + it * SG_THREADS, 64 * E - 1);
        raw_a[it] = __ldg(gcp + 64 * E + idx);
        raw_c[it] = __ldg(gcp + 192 * E + idx);
      }
      if (tid < E) raw_gl = __ldg(gcp + 63 * E + tid);
#pragma unroll
      for (int it = 0; it < GATE_ITERS; ++it) {
        const int idx = tid + it * SG_THREADS;
        if (idx < 64 * E) {
          const int r = idx / E, e = idx % E;
          sm.ga[r * ES + e] = raw_a[it];
          sm.gcq[r * ES + e] = raw_c[it];
        }
      }
      if (tid < E) sm.flag[tid] = raw_gl * LOG2E >= DD_MIN_LOG2_DECAY ? 1 : 0;
      if (tid < E * 4) sm.red[tid] = 0.f;
      if (t >= rows) {                                   // token rows past the end of a ragged chunk contribute nothing
#pragma unroll
        for (int j = 0; j < 32; ++j) kw[j] = 0u;
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");     // the workers only
    }

    // Pipeline.  First the value-block images: as each lands in a stage of the G ring the MMA warp adds it into the dK tile
    // (tensor-memory columns 256..383) and hands the stage back.  Then the 2E half-slice steps s = 2e + vh: the MMAs of
    // step s go out as soon as its half-slice of h (and of G, for a slice with a trace) is there; after the second step of a
    // slice four warps take the diagonal of the trace tile and every worker reads its part of the (double-buffered) P_e
    // tile.  The workers never read the half-slices themselves: shared memory is read by the tensor core only.
    auto issue_block_mma = [&](int u) {                    // one lane of the issuing warp: dK += [I;0] P_u^T
      const uint64_t did = make_desc(smem_u32(sm.ident), 2048, 128, LAYOUT_PLAIN);          // K = k
      const uint64_t dpk = make_desc(smem_u32(sm.gp[u % NS]), 2048, 128, LAYOUT_PLAIN);     // (i = d, j = t): K = t
      constexpr uint32_t id_acc = make_idesc(128, 128, 0, 0);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        umma_bf16(tmem + 256, desc_advance(did, kk * 4096), desc_advance(dpk, kk * 4096), id_acc, (u > 0 || kk > 0) ? 1u : 0u);
      umma_commit(&sm.bar_pfree[u % NS]);
    };
    auto issue_mma = [&](int s, int vh) {                  // one lane of the issuing warp
      const int st = s % NS;
      const uint64_t dhk = make_desc(smem_u32(sm.hp[st]), 2048, 128, LAYOUT_PLAIN);   // K = v
      const uint64_t dxt = make_desc(smem_u32(sm.xt), 16, 1024, LAYOUT_SW128);
      constexpr uint32_t id_acc = make_idesc(128, 128, 0, 0);
      const uint32_t tmem_p = tmem + ((s >> 1) & 1) * 128;       // P tile of this slice
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)                            // P_e (+)= [dW ; dO][:, 64 value columns] h_e[:, those columns]^T
        umma_bf16(tmem_p, desc_advance(dxt, vh * 16384 + kk * 32), desc_advance(dhk, kk * 4096), id_acc, (vh > 0 || kk > 0) ? 1u : 0u);
    };
    auto issue_trace = [&](int s, int vh) {                // h_e G_e^T over the step's value columns; its diagonal sums to <h_e, G_e>
      const int st = s % NS;
      const uint64_t dhk = make_desc(smem_u32(sm.hp[st]), 2048, 128, LAYOUT_PLAIN);
      const uint64_t dgk = make_desc(smem_u32(sm.gp[st]), 2048, 128, LAYOUT_PLAIN);
      constexpr uint32_t id_acc = make_idesc(128, 128, 0, 0);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        umma_bf16(tmem + 384, desc_advance(dhk, kk * 4096), desc_advance(dgk, kk * 4096), id_acc, (vh > 0 || kk > 0) ? 1u : 0u);
    };
    float acc[64];                                         // this row's gate-weighted sum over the slices, key columns wg*64 .. +64
#pragma unroll
    for (int j = 0; j < 64; ++j) acc[j] = 0.f;
    auto take_slice = [&](int e) {                         // P_e complete: row sum against the K (Q) row, and acc += gate * P_e
      const float gate = krow ? -sm.ga[t * ES + e] : sm.gcq[t * ES + e];
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;          // independent chains
      // sixteen columns at a time, the next piece travelling while this one is used
      const uint32_t src = tmem_row + (e & 1) * 128 + wg * 64;
      float pv[2][16];
      tmem_ld<16>(src, pv[0]);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        tmem_wait_ld();
        if (c + 1 < 4) tmem_ld<16>(src + (c + 1) * 16, pv[(c + 1) & 1]);
        const float* pc = pv[c & 1];
#pragma unroll
        for (int j = 0; j < 16; j += 4) {
          const uint32_t w0 = kw[(c * 16 + j) >> 1], w1 = kw[((c * 16 + j) >> 1) + 1];
          a0 = fmaf(bf16_lo(w0), pc[j], a0);
          a1 = fmaf(bf16_hi(w0), pc[j + 1], a1);
          a2 = fmaf(bf16_lo(w1), pc[j + 2], a2);
          a3 = fmaf(bf16_hi(w1), pc[j + 3], a3);
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[c * 16 + j + i] = fmaf(gate, pc[j + i], acc[c * 16 + j + i]);
        }
      }
      const float rowsum = (a0 + a1) + (a2 + a3);
      sm.part[(wg * 128 + row) * ES + e] = krow ? -rowsum : rowsum;
    };
    auto take_diag = [&](int e) {                          // <h_e, G_e> = trace(h_e G_e^T): this warp's 32 diagonal elements
      float dv[32];
      tmem_ld<32>(tmem_row + 384 + (warp & 3) * 32, dv);
      tmem_wait_ld();
      float d = 0.f;
#pragma unroll
      for (int j = 0; j < 32; ++j) d = (lane == j) ? dv[j] : d;
      for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
      if (lane == 0) sm.red[e * 4 + (warp & 3)] = d;
    };
    auto step_bit = [&](int s) { return (ph_step >> (s % NS)) & 1u; };
    auto img_bit = [&](int st) { return (ph_img >> st) & 1u; };

    // The issuing warp, the loading warp and the workers run decoupled, coupled only by mbarriers:
    //   bar_kq         TMA -> issuer       the [dW ; dO] tile of the item landed
    //   bar_pt[st]     TMA -> issuer       a value-block image landed in stage st of the G ring
    //   bar_pfree[st]  tensor core -> loads  its product is complete: the stage may be refilled
    //   bar_load[st]   TMA -> issuer       the half-slice of h of a step landed in stage st
    //   bar_g[st]      TMA -> issuer       the half-slice of G of a step landed (slices with a trace only)
    //   bar_mma[vh]    tensor core -> workers  MMAs of a step complete; after vh = 1 the P tile (and the trace tile) is ready
    //   bar_read[st]   workers -> loads    MMAs of a step seen complete: stage st of both rings may be refilled
    //   bar_pread[b]   workers -> issuer   P tile b has been read: the slice after next may overwrite it
    //   bar_diag       workers -> issuer   diagonal of the trace tile read (or not needed): the next slice may overwrite it
    if (worker) {
#pragma unroll 1
      for (int e = 0; e < E; ++e) {
        // ---- step s = 2e (vh = 0) ----
        {
          const int s = 2 * e;
          mbar_wait(&sm.bar_mma[0], ((s >> 1) & 1) ^ ph_e, ctl, DEV_TIMEOUT_MMA);
          __syncwarp();
          if (lane == 0) mbar_arrive(&sm.bar_read[s % NS]);   // the tensor core, the only reader of the stage, is done with it
        }
        // ---- step s = 2e + 1 (vh = 1) ----
        {
          const int s = 2 * e + 1;
          mbar_wait(&sm.bar_mma[1], ((s >> 1) & 1) ^ ph_e, ctl, DEV_TIMEOUT_MMA);
          tc_fence_after();
          __syncwarp();
          if (lane == 0) mbar_arrive(&sm.bar_read[s % NS]);
          if (wg == 0) {                                       // the trace tile is single: read it first and hand it back
            if (sm.flag[e]) take_diag(e);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.bar_diag);
          }
          take_slice(e);
          tc_fence_before();                                   // orders the reads of P_e before the MMAs that will overwrite it
          __syncwarp();
          if (lane == 0) mbar_arrive(&sm.bar_pread[e & 1]);
        }
      }
    } else if (warp_u == SG_THREADS / 32) {                // MMA issue
#pragma unroll 1
      for (int u = 0; u < NVB; ++u) {
        mbar_wait(&sm.bar_pt[u % NS], ((u / NS) & 1) ^ img_bit(u % NS), ctl, DEV_TIMEOUT_LOAD);
        tc_fence_after();
        if (elect_one()) issue_block_mma(u);
        __syncwarp();
      }
      mbar_wait(&sm.bar_kq, ph_kq, ctl, DEV_TIMEOUT_LOAD);   // the P products read the [dW ; dO] tile
#pragma unroll 1
      for (int s = 0; s < STEPS; ++s) {
        const int vh = s & 1, e = s >> 1;
        const bool tr = (fmask >> e) & 1u;
        if (vh == 0 && e >= 2) {                             // P tile (e & 1) was last used by slice e - 2
          mbar_wait(&sm.bar_pread[e & 1], (((e >> 1) - 1) & 1) ^ ((ph_pread >> (e & 1)) & 1u), ctl, DEV_TIMEOUT_MMA);
        }
        mbar_wait(&sm.bar_load[s % NS], ((s / NS) & 1) ^ step_bit(s), ctl, DEV_TIMEOUT_LOAD);
        tc_fence_after();
        if (elect_one()) issue_mma(s, vh);
        __syncwarp();
        // the trace tile of the previous slice must have been read before the first step of this one overwrites it
        if (vh == 0 && s > 0) {
          mbar_wait(&sm.bar_diag, (((s >> 1) - 1) & 1) ^ ph_e, ctl, DEV_TIMEOUT_MMA);
          tc_fence_after();
        }
        if (tr) {
#pragma unroll
          for (int i = 0; i < NS; ++i)
            if (i == s % NS) { mbar_wait(&sm.bar_g[i], g_uses[i] & 1, ctl, DEV_TIMEOUT_LOAD); ++g_uses[i]; }
          tc_fence_after();
          if (elect_one()) issue_trace(s, vh);
          __syncwarp();
        }
        if (elect_one()) umma_commit(&sm.bar_mma[vh]);
        __syncwarp();
      }
    } else {                                               // bulk loads
      // (the tile and the first ring round of this item went out before the item began)
      // value-block images beyond the first ring round: stage u % NS is free once the product of image u - NS is complete
#pragma unroll 1
      for (int u = NS; u < NVB; ++u) {
        mbar_wait(&sm.bar_pfree[u % NS], (((u / NS) - 1) & 1) ^ img_bit(u % NS), ctl, DEV_TIMEOUT_LOAD);
        if (elect_one()) issue_block(item, u);
        __syncwarp();
      }
      // half-slices of G for the first ring round of steps: their stage held a value-block image last
#pragma unroll 1
      for (int s = 0; s < NS && s < STEPS; ++s) {
        if (!((fmask >> (s >> 1)) & 1u)) continue;
        const int uses = (NVB - 1 - s % NS) / NS + 1;        // images that went through stage s % NS (0 if none)
        if (s % NS < NVB) mbar_wait(&sm.bar_pfree[s % NS], ((uses - 1) & 1) ^ img_bit(s % NS), ctl, DEV_TIMEOUT_LOAD);
        if (elect_one()) issue_g(item, s);
        __syncwarp();
      }
      // A worker warp releases a stage only after it has seen the MMAs of that step complete, so bar_read alone says that
      // both readers of the stage are done; this warp never waits on bar_mma, whose phases it could fall behind.
#pragma unroll 1
      for (int s = 0; s < STEPS; ++s) {
        // The ring holds NS half-slices (64 KB), less than what keeps this SM's share of HBM busy at HBM latency: the
        // half-slice PF_AHEAD steps further on (of this item or of the CTA's next one) is pulled into L2 now, so that the
        // ring's own load of it later finds it there.
        // (Up to eight slices: at twelve and sixteen the pulled lines were evicted again before the ring asked for them, 22%
        // more DRAM traffic for no gain.)
        if (E <= 8 && elect_one()) {
          const int q = s + NS + PF_AHEAD;
          const int64_t it2 = q < STEPS ? item : nxt;
          const int q2 = q < STEPS ? q : q - STEPS;
          if (it2 < n_items && q2 < STEPS)
            bulk_prefetch(reinterpret_cast<const uint8_t*>(p.h) + it2 * (static_cast<int64_t>(E) * 32768) + q2 * 16384, 16384);
          if (s == 0 && nxt < n_items) {                 // and the next item's value-block images and [dW ; dO] tile
            const int h2 = static_cast<int>(nxt) % p.H, b2 = static_cast<int>(nxt) / (p.H * p.NC);
            bulk_prefetch(reinterpret_cast<const uint8_t*>(p.dkg) + nxt * (static_cast<int64_t>(NVB) * 16384), static_cast<uint32_t>(NVB) * 16384);
            tma_prefetch_4d(&map_dv, 0, h2, t0n, b2);
            tma_prefetch_4d(&map_do, 0, h2, t0n, b2);
            tma_prefetch_4d(&map_dv, 64, h2, t0n, b2);
            tma_prefetch_4d(&map_do, 64, h2, t0n, b2);
          }
        }
        __syncwarp();
        mbar_wait(&sm.bar_read[s % NS], ((s / NS) & 1) ^ step_bit(s), ctl, DEV_TIMEOUT_LOAD);
        if (s + NS < STEPS && elect_one()) {
          issue_h(item, s + NS);
          if ((fmask >> ((s + NS) >> 1)) & 1u) issue_g(item, s + NS);
        }
        __syncwarp();
      }
      // Every step's MMAs are complete: the tile and both rings are free.  Stages of the G ring that no step used still
      // have to see their last value-block product complete.  Then the next item's first round goes out, to land while the
      // workers finish this item and open the next.
      if (nxt < n_items) {
#pragma unroll 1
        for (int st = 0; st < NS && st < NVB; ++st) {
          const int uses = (NVB - 1 - st) / NS + 1;
          mbar_wait(&sm.bar_pfree[st], ((uses - 1) & 1) ^ img_bit(st), ctl, DEV_TIMEOUT_LOAD);
        }
        if (elect_one()) issue_first_round(nxt, t0n);
        __syncwarp();
      }
    }
    __syncthreads();
    if (tid < E)                                         // <h_e, G_e>: the four row blocks' partial traces in a fixed order
      p.dd[item * E + tid] = (sm.red[tid * 4] + sm.red[tid * 4 + 1]) + (sm.red[tid * 4 + 2] + sm.red[tid * 4 + 3]);
    // row sums: add the two column halves
    for (int idx = tid; idx < 128 * E && worker; idx += SG_THREADS) {
      const int r = idx / E, e = idx % E;
      const float v = sm.part[r * ES + e] + sm.part[(128 + r) * ES + e];
      if (r < 64) p.da[(item * 64 + r) * E + e] = v; else p.dc[(item * 64 + r - 64) * E + e] = v;
    }
    // dkq, bf16 image [column / 8][row][column % 8]: rows 0..63 = the K rows' sum + (r*U) G^T from tensor memory (dK), rows
    // 64..127 = the Q rows' sum (dQ).  This thread: its row, 64 columns; a warp's 16-byte store covers 32 consecutive rows =
    // 512 contiguous bytes.
    tc_fence_after();
    if (worker) {
      uint8_t* outp = reinterpret_cast<uint8_t*>(p.dkq) + item * 32768 + row * 16;
      const bool live_row = t < rows;
#pragma unroll
      for (int c0 = 0; c0 < 64; c0 += 16) {
        float a2[16];
        tmem_ld<16>(tmem_row + 256 + wg * 64 + c0, a2);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; j += 8) {
          float v[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = live_row ? acc[c0 + j + i] + (krow ? a2[j + i] : 0.f) : 0.f;
          uint4 u;
          u.x = pack_bf16(v[0], v[1]);
          u.y = pack_bf16(v[2], v[3]);
          u.z = pack_bf16(v[4], v[5]);
          u.w = pack_bf16(v[6], v[7]);
          *reinterpret_cast<uint4*>(outp + ((wg * 64 + c0 + j) >> 3) * 2048) = u;
        }
      }
    }
    tc_fence_before();
    __syncthreads();                                     // the tiles in tensor memory and the tables are free for the next item
    tc_fence_after();
    // completions of this item, for the phase parities of the next
    ph_kq ^= 1u;
    ph_step ^= ODD_STEP;
    ph_img ^= odd_img;
    ph_e ^= (E & 1u);
    ph_pread ^= ODD_PREAD;
    item = nxt;
    t0 = t0n;
    rows = rowsn;
    my_gl = next_gl;
  }
  if (warp == 0) tmem_dealloc(tmem, 512);
}

}  // namespace tgdn

using namespace tgdn;

template <int E>
static int launch_sg(const CUtensorMap& mdv, const CUtensorMap& mdo, const SgParams& p, cudaStream_t s) {
  const int smem = static_cast<int>(sizeof(SgSmem<E>)) + 1024;
  static_assert(sizeof(SgSmem<E>) + 1024 <= 232448, "shared memory budget of one CTA exceeded");
  cudaError_t e = cudaFuncSetAttribute(sg_kernel<E>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return tgdn_cuda_error(e);
  const long long items = static_cast<long long>(p.B) * p.NC * p.H;
  const int grid = static_cast<int>(items < p.ahead ? items : p.ahead);      // persistent: one CTA per SM
  sg_kernel<E><<<grid, SG_BLOCK, smem, s>>>(mdv, mdo, p);
  return tgdn_cuda_error(cudaGetLastError());
}

extern "C" int tgdn_bwd_state_grads(const void* q, const void* k, const void* dO, const void* dV,
                                    const void* h, const void* ds, const void* dkg, const float* k2, const float* q2,
                                    const float* gc, float scale, const int32_t* chunk_map, int B, int T, int H, int E, int NC, void* dkq,
                                    float* da, float* dc, float* dd, void* stream) {
  if (!q || !k || !dO || !dV || !h || !ds || !dkg || !k2 || !q2 || !gc || !dkq || !da || !dc || !dd) return TGDN_ERR_NULL;
  int rc = tgdn_check_core_shape(B, T, H, E, NC, chunk_map != nullptr);
  if (rc) return rc;
  if (static_cast<long long>(B) * NC * H * 64 > 0x7fffffffLL) return TGDN_ERR_SHAPE;   // item indices are 32-bit in the kernel
  if ((reinterpret_cast<uintptr_t>(dO) | reinterpret_cast<uintptr_t>(dV) |
       reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(ds) | reinterpret_cast<uintptr_t>(dkg) |
       reinterpret_cast<uintptr_t>(dkq)) & 15)
    return TGDN_ERR_ALIGN;
  if ((reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(q)) & 15) return TGDN_ERR_ALIGN;
  CUtensorMap mdv, mdo;
  if ((rc = tgdn_make_token_map(&mdv, dV, B, T, H, 64, 64, 1))) return rc;
  if ((rc = tgdn_make_token_map(&mdo, dO, B, T, H, 64, 64, 1))) return rc;
  SgParams p{static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(dO), static_cast<const __nv_bfloat16*>(dV),
             static_cast<const __nv_bfloat16*>(h),
             static_cast<const __nv_bfloat16*>(ds), static_cast<const __nv_bfloat16*>(dkg), k2, q2, gc,
             static_cast<__nv_bfloat16*>(dkq), da, dc, dd, chunk_map, B, T, H, NC, HEAD / tgdn_value_block(E), scale,
             tgdn_status_word(), tgdn_sm_count()};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (E) {
    case 1: return launch_sg<1>(mdv, mdo, p, s);
    case 2: return launch_sg<2>(mdv, mdo, p, s);
    case 4: return launch_sg<4>(mdv, mdo, p, s);
    case 8: return launch_sg<8>(mdv, mdo, p, s);
    case 12: return launch_sg<12>(mdv, mdo, p, s);
    case 16: return launch_sg<16>(mdv, mdo, p, s);
    default: return TGDN_ERR_SHAPE;
  }
}
