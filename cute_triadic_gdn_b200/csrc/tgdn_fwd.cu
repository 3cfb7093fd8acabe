// Forward chunk recurrence of the Triadic GDN.
//
// One CTA owns one (sequence, head, block of VC value columns) and walks the sequence's 64-token chunks in order.  The
// block is split over NCH independent CHAINS of WPC warpgroups (a warpgroup = 128 threads = the 128 rows of [K;Q]); chain c
// owns CW value columns of every slice: its E state slices S_e[:, columns] (128 x CW each, f32) live in the registers of its
// threads (WPC = 2, at twelve and sixteen slices: each of the chain's two warpgroups holds half of the slices).
// Per chunk a chain runs three dependent MMA groups of its own, with its own accumulators in tensor memory:
//   (1) R  = [K;Q] S          tcgen05, M=128, N=E*CW, K=128   rows 0..63: K S_e, rows 64..127: Q S_e
//       W  = V - sum_e a_e*R_e (K rows);   Oq = sum_e c_e*R_e (Q rows)
//   (2) [U;Oi] = [A;PmA] (beta*W)   tcgen05, M=128, N=16 (CW used), K=64
//       o  = Oq + Oi  ->  bf16;   Vn_e = r_e*U
//   (3) dS = K^T Vn           tcgen05, M=128, N=E*CW, K=64
//       S_e <- d_e S_e + dS_e  (registers), bf16 copy -> shared memory operand of the next (1) and saved state h
// with a = k2 exp(gc), r = k2 exp(gL-gc), c = scale q2 exp(gc), d = exp(gL).
//
// The chains of a CTA share only the chunk's tiles (K/Q, the [A;PmA] image, the gate factors, the value rows of the block
// and the beta rows), which arrive by TMA in a ring of STAGES stages; a stage is refilled by whichever chain is the last to
// hand it back, so no chain ever waits for another one except through that ring.  Everything else is private to a chain
// (its columns are independent of all other columns of the problem): its barrier is a named barrier of its own threads,
// its MMAs are issued by one of its own lanes and complete on its own mbarrier.  While one chain waits for its MMA or its tensor-memory load, the tensor core and the
// issue slots work for the others: the dependent chain of a chunk (three MMA -> load -> epilogue round trips) is what
// bounds this kernel, and the number of independent chains per SM is what hides it.
//
// The gate factors of a chunk (a, r, c per row and slice, d per slice) were formed by the masks kernel and arrive in the
// stage with one bulk copy; every thread reads those of its own row (K rows: a, r, beta; Q rows: c) right after its
// chain's MMA (1) went out.  Nothing couples the chains but the tile ring.  The key-row warps have the longer phases (two
// gate factors per slice, the operand images of beta*W and r_e*U), so the chain's extra roles sit on its query-row
// warps: one issues the MMAs and polls their barrier, one hands stages back and issues the loads.
//
// Replaces cute_triadic_gdn/kernels/sm100_joint_fwd.py:66-527 (fwd_kernel); math as cute_triadic_gdn/ops/gdn_joint.py:63-90.
// Column order inside a chain: n' = e*CW + c  <->  (slice e, value column c of the chain).
#include "tgdn_common.cuh"
#include "tgdn_host.h"
#include "tgdn_kernels.h"

namespace tgdn {

template <int THREADS>
__device__ __forceinline__ void chain_sync(int chain) {     // the threads of one chain
  asm volatile("bar.sync %0, %1;" ::"r"(chain + 1), "n"(THREADS) : "memory");
}

// N floats from shared memory; 16-byte loads where N and the address allow, else 8-byte loads (N even) or one float
template <int N>
__device__ __forceinline__ void lds_part(const float* p, float* out) {
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

// WPC warpgroups share one chain and split its SLICES (warpgroup w of a chain owns slices w*E/WPC ..): the chain's MMAs
// then have N = E*CW columns with CW = 8 columns per thread even at twelve and sixteen slices, where a warpgroup alone
// could hold only four columns of every slice in its registers; the sums over the slices (W, and the state part of o) are
// completed through shared memory.
template <int E, int CW, int NCH, int WPC, int STAGES>
struct FwdCfg {
  static constexpr int CHAIN_THREADS = WPC * 128;
  static constexpr int THREADS = NCH * CHAIN_THREADS;
  static constexpr int VC = CW * NCH;             // value columns of the CTA
  static constexpr int TPC = E * CW;              // state columns per chain
  static constexpr int ET = E / WPC;              // slices per thread
  static constexpr int TPT = ET * CW;             // state columns per thread
  static constexpr int UW = 16;                   // columns of the (2) accumulator (the smallest N of an M=128 MMA)
  static constexpr int TW = TPC + UW;             // tensor-memory columns per chain
  static constexpr int TMEM_NEED = NCH * TW;
  static constexpr int TMEM_COLS = TMEM_NEED <= 32 ? 32 : TMEM_NEED <= 64 ? 64 : TMEM_NEED <= 128 ? 128 : TMEM_NEED <= 256 ? 256 : 512;
  // shared memory carve-up (bytes); the swizzled tiles are 1024-byte aligned
  static constexpr int KQ_BYTES = 32768;
  static constexpr int AP_BYTES = 16384;
  static constexpr int S_BYTES = TPC * 256;       // per chain: image (i = d, j = n'), SI = 128, SJ = 2048
  static constexpr int VN_BYTES = TPC * 128;      // per chain: image (i = t, j = n'), SI = 128, SJ = 1024
  static constexpr int BW_BYTES = 2048;           // per chain: image (i = s, j = v), 16 columns, SI = 128, SJ = 1024
  static constexpr int OFF_KQ = 0;
  static constexpr int OFF_AP = OFF_KQ + STAGES * KQ_BYTES;
  static constexpr int OFF_S = OFF_AP + STAGES * AP_BYTES;
  static constexpr int OFF_VN = OFF_S + NCH * S_BYTES;
  static constexpr int OFF_BW = OFF_VN + NCH * VN_BYTES;
  // per stage: the gate factors of the chunk as the masks kernel stored them, a, r, c as 64 dense rows of E floats each,
  // then d (one bulk copy)
  static constexpr int GT_BYTES = gate_factor_bytes(E);
  static constexpr int GT_STRIDE = (GT_BYTES + 127) & ~127;
  static constexpr int GF_R = 64 * E, GF_C = 128 * E, GF_D = 192 * E;   // float offsets of r, c, d behind a
  static constexpr int OFF_GT = (OFF_BW + NCH * BW_BYTES + 127) & ~127;
  // per stage: the value rows of the CTA's columns, one box of 64 rows x CW columns per chain (TMA; a row of a box is at
  // least 16 bytes), and the beta rows of the chunk for the four heads h & ~3 .. (TMA when H is a multiple of 4)
  static constexpr bool TMA_V = CW >= 8;
  static constexpr int VBOX_BYTES = 64 * CW * 2;
  static constexpr int VT_BYTES = TMA_V ? NCH * VBOX_BYTES : 0;
  static constexpr int OFF_VT = OFF_GT + STAGES * GT_STRIDE;
  static constexpr int OFF_BT = OFF_VT + STAGES * VT_BYTES;
  static constexpr bool TMA_BETA = OFF_BT + STAGES * 1024 + 128 + 1024 <= 232448;   // where the beta rows still fit
  static constexpr int BT_BYTES = TMA_BETA ? 1024 : 0;
  static constexpr int OFF_CTRL = OFF_BT + STAGES * BT_BYTES;
  static constexpr int SMEM_BYTES = OFF_CTRL + 128 + 1024;    // + control block + alignment slack
  static_assert(CW == 4 || CW == 8 || CW == 16, "a chain owns 4, 8 or 16 value columns");
  static_assert(E % WPC == 0 && (WPC == 1 || ET % 2 == 0), "the slices split evenly over the chain's warpgroups");
  static_assert(TPC % 16 == 0 && TPC <= 256, "columns per chain: a multiple of 16 (MMA N)");
  static_assert(TPT % 16 == 0 && TPT <= 64, "columns per thread: a multiple of 16 (tensor-memory loads), at most 64 registers of state");
  static_assert(WPC == 1 || VN_BYTES >= 2 * 64 * CW * 4, "the exchange of partial sums borrows the chain's Vn image");
};

struct FwdCtrl {
  uint64_t bar_load[2];
  uint64_t bar_mma[4];
  uint32_t released[2];      // chains that have finished with the stage (counts up forever; a multiple of NCH = all)
  uint32_t tmem_base;
  int abort;
};

template <int E, int CW, int NCH, int WPC, int STAGES, int MINB>
__global__ void __launch_bounds__(NCH * WPC * 128, MINB)
fwd_kernel(const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_beta,
           const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_q, FwdParams p) {
  using C = FwdCfg<E, CW, NCH, WPC, STAGES>;
  constexpr int TPC = C::TPC, VC = C::VC, ET = C::ET, TPT = C::TPT, CT = C::CHAIN_THREADS;
  // Roles inside a chain: its key-row warps (0, 1) have the longer epilogues (gate factors r_e, the operand images of W
  // and of r_e U), so the query-row warps take the extra work: warp 2 issues the MMAs and polls their barrier, warp 3
  // hands stages back and issues the loads.
  constexpr int ISSUE_WARP = 2, REFILL_WARP = 3;
  const bool beta_tma = C::TMA_BETA && p.beta_tma;
  constexpr bool LATE_R = E >= 12;                   // read r_e after the epilogue of (1) (register pressure at many slices)
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  FwdCtrl& ctrl = *reinterpret_cast<FwdCtrl*>(smem + C::OFF_CTRL);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int chain = WPC == 1 ? (warp >> 2) : (warp >> 2) / WPC;   // WPC warpgroups form a chain
  const int sw = WPC == 1 ? 0 : (warp >> 2) % WPC;  // which share of the chain's slices this warpgroup owns
  const int e0 = sw * ET;                           // first slice of this thread
  const int col0 = sw * TPT;                        // its first column among the chain's E*CW
  const int row = (warp & 3) * 32 + lane;           // tensor-memory lane = operand row
  const bool krow = row < 64;                       // rows 0..63 work on K rows (W, U, Vn), 64..127 on Q rows (o)
  const int t = row & 63;
  uint8_t* s_img = smem + C::OFF_S + chain * C::S_BYTES;
  uint8_t* vn_img = smem + C::OFF_VN + chain * C::VN_BYTES;
  uint8_t* bw_img = smem + C::OFF_BW + chain * C::BW_BYTES;

  // work item
  constexpr int NV = HEAD / VC;
  const int vb = blockIdx.x % NV, h = (blockIdx.x / NV) % p.H, seq_rank = blockIdx.x / (NV * p.H);
  int b = seq_rank, first = 0, count = p.NC, seq = seq_rank;
  if (p.cmap != nullptr) {
    const int doc = p.cmap[2 * p.NC + seq_rank];    // longest documents first
    if (doc < 0 || doc >= p.n_seq) return;
    b = 0;
    seq = doc;
    first = p.offsets[doc];
    count = p.offsets[doc + 1] - first;
    if (first < 0 || count <= 0 || first + count > p.NC) return;
  }
  const int v0g = vb * VC + chain * CW;             // first value column of this chain in the head

  if (tid == 0) {
    mbar_init(&ctrl.bar_load[0], 1);
    mbar_init(&ctrl.bar_load[1], 1);
    for (int c = 0; c < 4; ++c) mbar_init(&ctrl.bar_mma[c], 1);
    mbar_fence_init();
    ctrl.released[0] = ctrl.released[1] = 0;
    ctrl.abort = 0;
  }
  if (warp == 0) { tmem_alloc(&ctrl.tmem_base, C::TMEM_COLS); tmem_relinquish(); }
  // state: zero, or the caller's initial state (f32 [seq][H][E][128 d][128 v])
  float S[TPT];
  if (p.s_in != nullptr) {
    const float* src = p.s_in + ((static_cast<int64_t>(seq) * p.H + h) * E + e0) * (HEAD * HEAD) + row * HEAD + v0g;
#pragma unroll
    for (int e = 0; e < ET; ++e)
#pragma unroll
      for (int c = 0; c < CW; ++c) S[e * CW + c] = __ldg(src + e * (HEAD * HEAD) + c);
  } else {
#pragma unroll
    for (int j = 0; j < TPT; ++j) S[j] = 0.f;
  }
  // the second 8-column block of the (2) operand is never written: keep it zero (its products land in unused columns)
  for (int i = (tid & (CT - 1)); i < C::BW_BYTES / 16; i += CT) reinterpret_cast<uint4*>(bw_img)[i] = make_uint4(0, 0, 0, 0);

  // saved state / operand image of this thread's S: pieces of 8 columns (one 16-byte store each into the image)
  auto state_item_ptr = [&](int64_t item) {
    return reinterpret_cast<uint8_t*>(p.h) + item * (static_cast<int64_t>(E) * 32768);
  };
  auto store_state_slices = [&](uint8_t* hbase, int j0, const uint32_t* packed /* 8 words = 16 columns from j0 */) {
#pragma unroll
    for (int j = 0; j < 16; j += CW) {
      const int e = e0 + (j0 + j) / CW;
      uint8_t* dst = hbase + e * 32768 + (v0g >> 3) * 2048 + row * 16 + (v0g & 7) * 2;
      if constexpr (CW == 16) {
        *reinterpret_cast<uint4*>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        *reinterpret_cast<uint4*>(dst + 2048) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
      } else if constexpr (CW == 8) {
        *reinterpret_cast<uint4*>(dst) = make_uint4(packed[j / 2], packed[j / 2 + 1], packed[j / 2 + 2], packed[j / 2 + 3]);
      } else {
        *reinterpret_cast<uint2*>(dst) = make_uint2(packed[j / 2], packed[j / 2 + 1]);
      }
    }
  };
  {
    const uint32_t base = smem_u32(s_img) + (row >> 3) * 128 + (row & 7) * 16;
    uint8_t* hbase = p.h != nullptr ? state_item_ptr((static_cast<int64_t>(b) * p.NC + first) * p.H + h) : nullptr;
#pragma unroll
    for (int j0 = 0; j0 < TPT; j0 += 16) {
      uint32_t packed[8];
#pragma unroll
      for (int j = 0; j < 16; j += 2) packed[j / 2] = pack_bf16(S[j0 + j], S[j0 + j + 1]);
      st_shared_v4(base + ((col0 + j0) >> 3) * 2048, packed[0], packed[1], packed[2], packed[3]);
      st_shared_v4(base + ((col0 + j0 + 8) >> 3) * 2048, packed[4], packed[5], packed[6], packed[7]);
      if (hbase != nullptr) store_state_slices(hbase, j0, packed);
    }
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = __shfl_sync(0xffffffffu, ctrl.tmem_base, 0);
  const int cwarp_u = __shfl_sync(0xffffffffu, warp & (CT / 32 - 1), 0);   // warp index inside the chain as a warp-uniform value
  const uint32_t tmem_c = tmem + chain * C::TW;                  // this chain's columns: [0, TPC) R / dS, [TPC, TPC+16) U / Oi
  const uint32_t tmem_row = tmem_c + (static_cast<uint32_t>((warp & 3) * 32) << 16);
  WaitCtl ctl{&ctrl.abort, p.status};

  auto chunk_info = [&](int i, int& t0, int& rows) {
    const int n = first + i;
    if (p.cmap != nullptr) { t0 = p.cmap[n]; rows = p.cmap[p.NC + n]; } else { t0 = n * CHUNK; rows = CHUNK; }
    if (t0 < 0 || rows < 0 || rows > CHUNK || t0 + rows > p.T) {
      atomicCAS(p.status, DEV_OK, DEV_BAD_CHUNK_MAP);
      t0 = 0; rows = 0;
    }
  };
  auto issue_loads = [&](int i) {                   // one thread: K/Q tiles and the [A;PmA] image of local chunk i
    int t0, rows;
    chunk_info(i, t0, rows);
    const int st = i % STAGES;
    uint8_t* kq = smem + C::OFF_KQ + st * C::KQ_BYTES;
    const int64_t item = (static_cast<int64_t>(b) * p.NC + first + i) * p.H + h;
    mbar_expect_tx(&ctrl.bar_load[st], C::KQ_BYTES + C::AP_BYTES + C::GT_BYTES + C::VT_BYTES + (beta_tma ? C::BT_BYTES : 0));
    if constexpr (C::TMA_V) {
#pragma unroll
      for (int c = 0; c < NCH; ++c)
        tma_load_4d(smem + C::OFF_VT + st * C::VT_BYTES + c * C::VBOX_BYTES, &map_v, &ctrl.bar_load[st], vb * VC + c * CW, h, t0, b);
    }
    if (beta_tma) tma_load_4d(smem + C::OFF_BT + st * C::BT_BYTES, &map_beta, &ctrl.bar_load[st], 0, h >> 2, t0, b);
    bulk_load(smem + C::OFF_GT + st * C::GT_STRIDE, p.gc + item * gate_item_floats(E) + 64 * E, C::GT_BYTES, &ctrl.bar_load[st]);
    tma_load_4d(kq, &map_k, &ctrl.bar_load[st], 0, h, t0, b);
    tma_load_4d(kq + 8192, &map_q, &ctrl.bar_load[st], 0, h, t0, b);
    tma_load_4d(kq + 16384, &map_k, &ctrl.bar_load[st], 64, h, t0, b);
    tma_load_4d(kq + 24576, &map_q, &ctrl.bar_load[st], 64, h, t0, b);
    bulk_load(smem + C::OFF_AP + st * C::AP_BYTES, p.AP + item * (128 * 64), C::AP_BYTES, &ctrl.bar_load[st]);
  };
  auto prefetch_tiles = [&](int i) {                // one thread: pull a later chunk's tiles into L2
    int t0, rows;
    chunk_info(i, t0, rows);
    const int64_t item = (static_cast<int64_t>(b) * p.NC + first + i) * p.H + h;
    tma_prefetch_4d(&map_k, 0, h, t0, b);
    tma_prefetch_4d(&map_q, 0, h, t0, b);
    tma_prefetch_4d(&map_k, 64, h, t0, b);
    tma_prefetch_4d(&map_q, 64, h, t0, b);
    bulk_prefetch(p.AP + item * (128 * 64), C::AP_BYTES);
    bulk_prefetch(p.gc + item * gate_item_floats(E) + 64 * E, C::GT_BYTES);
  };
  auto prefetch_rows = [&](int i) {                 // what threads still load themselves, for a later chunk -> L2
    if (sw != 0 || chain != 0 || !krow) return;      // the value columns of all chains of the CTA share their 128-byte lines
    int t0, rows;
    chunk_info(i, t0, rows);
    const int last = max(rows, 1) - 1;
    const int64_t ro = (static_cast<int64_t>(b) * p.T + t0 + min(t, last)) * p.H + h;
    if (!beta_tma) prefetch_l2(p.beta + ro);
    if (!C::TMA_V) prefetch_l2(p.v + ro * HEAD + v0g);
  };
  auto load_vrow = [&](int t0, int rows, uint32_t* out /* CW/2 words */) {   // CW value columns of row t (clamped), raw bf16
    const int64_t tok = static_cast<int64_t>(b) * p.T + t0;
    const __nv_bfloat16* vp = p.v + ((tok + min(t, max(rows, 1) - 1)) * p.H + h) * HEAD + v0g;
    if constexpr (CW == 16) {
      const uint4 u0 = __ldg(reinterpret_cast<const uint4*>(vp)), u1 = __ldg(reinterpret_cast<const uint4*>(vp) + 1);
      out[0] = u0.x; out[1] = u0.y; out[2] = u0.z; out[3] = u0.w; out[4] = u1.x; out[5] = u1.y; out[6] = u1.z; out[7] = u1.w;
    } else if constexpr (CW == 8) {
      const uint4 u0 = __ldg(reinterpret_cast<const uint4*>(vp));
      out[0] = u0.x; out[1] = u0.y; out[2] = u0.z; out[3] = u0.w;
    } else {
      const uint2 u0 = __ldg(reinterpret_cast<const uint2*>(vp));
      out[0] = u0.x; out[1] = u0.y;
    }
  };
  auto store_row_global = [&](__nv_bfloat16* ptr, const float* src) {         // CW consecutive bf16
#pragma unroll
    for (int c = 0; c < CW; c += 8) {
      if constexpr (CW >= 8)
        *reinterpret_cast<uint4*>(ptr + c) = make_uint4(pack_bf16(src[c], src[c + 1]), pack_bf16(src[c + 2], src[c + 3]),
                                                        pack_bf16(src[c + 4], src[c + 5]), pack_bf16(src[c + 6], src[c + 7]));
      else
        *reinterpret_cast<uint2*>(ptr) = make_uint2(pack_bf16(src[0], src[1]), pack_bf16(src[2], src[3]));
    }
  };
  // CW consecutive columns n0.. of row r of an image whose 8-column blocks are SJ bytes apart
  auto store_row_image = [&](uint32_t row_base, int n0, uint32_t SJ, const float* src, float f) {
    if constexpr (CW >= 8) {
#pragma unroll
      for (int c = 0; c < CW; c += 8)
        st_shared_v4(row_base + ((n0 + c) >> 3) * SJ, pack_bf16(f * src[c], f * src[c + 1]), pack_bf16(f * src[c + 2], f * src[c + 3]),
                     pack_bf16(f * src[c + 4], f * src[c + 5]), pack_bf16(f * src[c + 6], f * src[c + 7]));
    } else {
      st_shared_v2(row_base + (n0 >> 3) * SJ + (n0 & 7) * 2, pack_bf16(f * src[0], f * src[1]), pack_bf16(f * src[2], f * src[3]));
    }
  };

  if (tid == 0) {
    issue_loads(0);
    if (STAGES == 2 && count > 1) issue_loads(1);
  }
  if (count > 1) prefetch_rows(1);
  uint32_t mma_phase = 0;

  for (int i = 0; i < count; ++i) {
    const int st = i % STAGES;
    int t0, rows;
    chunk_info(i, t0, rows);
    const int64_t item = (static_cast<int64_t>(b) * p.NC + first + i) * p.H + h;
    const int64_t tok = static_cast<int64_t>(b) * p.T + t0;
    const bool live = t < rows;
    uint8_t* kq = smem + C::OFF_KQ + st * C::KQ_BYTES;
    uint8_t* ap = smem + C::OFF_AP + st * C::AP_BYTES;

    // ---- (1) R = [K;Q] S --------------------------------------------------------------------------------------
    // Every thread reads rows of the stage (gates, value row, beta) under the MMA, so every warp waits for the loads itself.
    // (The MMA completions below are polled by the chain's first warp only: the other three sleep in the chain's hardware
    // barrier, where they take no issue slots from the chains that are in an epilogue at that moment.)
    mbar_wait(&ctrl.bar_load[st], (i / STAGES) & 1, ctl, DEV_TIMEOUT_LOAD);
    if (cwarp_u == ISSUE_WARP && elect_one()) {
      tc_fence_after();
      const uint64_t da = make_desc(smem_u32(kq), 16, 1024, LAYOUT_SW128);
      const uint64_t db = make_desc(smem_u32(s_img), 128, 2048, LAYOUT_PLAIN);
      constexpr uint32_t idesc = make_idesc(128, TPC, 0, 1);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)
        umma_bf16(tmem_c, desc_advance(da, (kk >> 2) * 16384 + (kk & 3) * 32), desc_advance(db, kk * 256), idesc, kk > 0);
      umma_commit(&ctrl.bar_mma[chain]);
    }
    __syncwarp();                                    // the other lanes must not run ahead into a spin wait
    // The chain finished with the previous chunk's tiles when its third MMA group completed.  It says so now, under this
    // MMA, where its warps have time to spare; the last chain to say so refills that stage with the chunk STAGES ahead.
    if (i > 0 && cwarp_u == REFILL_WARP && elect_one()) {
      const uint32_t done = atomicAdd(&ctrl.released[(i - 1) % STAGES], 1u) + 1u;
      if (done % NCH == 0) {
        if (i - 1 + STAGES < count) issue_loads(i - 1 + STAGES);
        if (i + STAGES < count) prefetch_tiles(i + STAGES);
      }
    }
    __syncwarp();
    // Under the MMA: this row's gate factors, value row and beta from the stage.
    const float* gf = reinterpret_cast<const float*>(smem + C::OFF_GT + st * C::GT_STRIDE);
    float ga[ET];                                    // this thread's slices.  K rows: a_e = k2 exp(gc); Q rows: c_e = scale q2 exp(gc)
    float gr[ET];                                    // K rows: r_e = k2 exp(gL - gc)
    float bt = 0.f;
    uint32_t vraw[CW / 2];
    if constexpr (WPC > 1) {
#pragma unroll
      for (int c = 0; c < CW / 2; ++c) vraw[c] = 0u;
    }
    {
      lds_part<ET>(gf + (krow ? 0 : C::GF_C) + t * E + e0, ga);
      if (krow) {
        if constexpr (!LATE_R) lds_part<ET>(gf + C::GF_R + t * E + e0, gr);
        if (sw == 0) {                               // the warpgroup that completes W: beta and the value row
          if (beta_tma) {
            bt = reinterpret_cast<const float*>(smem + C::OFF_BT + st * C::BT_BYTES)[t * 4 + (h & 3)];
          } else {
            bt = __ldg(p.beta + (tok + min(t, max(rows, 1) - 1)) * p.H + h);
          }
          if constexpr (C::TMA_V) {
            const uint32_t va = smem_u32(smem + C::OFF_VT + st * C::VT_BYTES + chain * C::VBOX_BYTES) + t * (CW * 2);
#pragma unroll
            for (int c = 0; c < CW / 2; c += 4)
              asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(vraw[c]), "=r"(vraw[c + 1]), "=r"(vraw[c + 2]), "=r"(vraw[c + 3]) : "r"(va + c * 4));
          } else {
            load_vrow(t0, rows, vraw);
          }
        }
        if (!live) bt = 0.f;
      } else {
#pragma unroll
        for (int e = 0; e < ET; ++e) gr[e] = 0.f;
      }
      if (i + 2 < count) prefetch_rows(i + 2);
    }
    if (cwarp_u == ISSUE_WARP) mbar_wait(&ctrl.bar_mma[chain], mma_phase & 1, ctl, DEV_TIMEOUT_MMA);
    chain_sync<CT>(chain);
    ++mma_phase;
    tc_fence_after();

    float acc[CW];                                   // K rows: W (starts from V); Q rows: Oq
#pragma unroll
    for (int c = 0; c < CW; ++c) acc[c] = (krow && live && sw == 0) ? ((c & 1) ? bf16_hi(vraw[c >> 1]) : bf16_lo(vraw[c >> 1])) : 0.f;
    {
      // sixteen columns at a time, the next piece travelling while this one is used
      float rr[2][16];
      tmem_ld<16>(tmem_row + col0, rr[0]);
#pragma unroll
      for (int pc = 0; pc < TPT / 16; ++pc) {
        tmem_wait_ld();
        if (pc + 1 < TPT / 16) tmem_ld<16>(tmem_row + col0 + (pc + 1) * 16, rr[(pc + 1) & 1]);
        const float* rp = rr[pc & 1];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int e = (pc * 16 + j) / CW, c = (pc * 16 + j) % CW;
          acc[c] = fmaf(krow ? -ga[e] : ga[e], rp[j], acc[c]);
        }
      }
    }
    if constexpr (WPC > 1) {
      // The sums over the slices are split over the chain's warpgroups: the first one completes W (K rows), the last one
      // the state part of o (Q rows); the others hand their partial sums over through shared memory (the chain's Vn image
      // is free between the last MMA of the previous chunk and the epilogue of (2)).
      static_assert(WPC == 2, "the exchange below is written for two warpgroups per chain");
      float* red = reinterpret_cast<float*>(vn_img) + (krow ? 0 : 64 * CW) + t * CW;
      const bool owner = krow ? (sw == 0) : (sw == WPC - 1);
      if (!owner) {
#pragma unroll
        for (int c = 0; c < CW; c += 4) *reinterpret_cast<float4*>(red + c) = make_float4(acc[c], acc[c + 1], acc[c + 2], acc[c + 3]);
      }
      chain_sync<CT>(chain);
      if (owner) {
#pragma unroll
        for (int c = 0; c < CW; c += 4) {
          const float4 x = *reinterpret_cast<const float4*>(red + c);
          acc[c] += x.x; acc[c + 1] += x.y; acc[c + 2] += x.z; acc[c + 3] += x.w;
        }
      }
    }
    if (krow && sw == 0) {
      // W -> saved (bf16), beta*W -> operand image (i = s, j = v)
      store_row_image(smem_u32(bw_img) + (t >> 3) * 128 + (t & 7) * 16, 0, 1024, acc, bt);
      if (p.W != nullptr) store_row_global(p.W + (item * 64 + t) * HEAD + v0g, acc);
    }
    fence_async_smem();
    tc_fence_before();
    chain_sync<CT>(chain);

    // ---- (2) [U;Oi] = [A;PmA] (beta W) ------------------------------------------------------------------------
    if (cwarp_u == ISSUE_WARP && elect_one()) {
      tc_fence_after();
      const uint64_t da = make_desc(smem_u32(ap), 2048, 128, LAYOUT_PLAIN);
      const uint64_t db = make_desc(smem_u32(bw_img), 128, 1024, LAYOUT_PLAIN);
      constexpr uint32_t idesc = make_idesc(128, C::UW, 0, 1);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        umma_bf16(tmem_c + TPC, desc_advance(da, kk * 4096), desc_advance(db, kk * 256), idesc, kk > 0);
      umma_commit(&ctrl.bar_mma[chain]);
    }
    __syncwarp();
    if constexpr (LATE_R) {                          // r_e only now, from the stage: sixteen registers fewer are live
      if (krow) lds_part<ET>(gf + C::GF_R + t * E + e0, gr);   // through the epilogue of (1)
    }
    if (cwarp_u == ISSUE_WARP) mbar_wait(&ctrl.bar_mma[chain], mma_phase & 1, ctl, DEV_TIMEOUT_MMA);
    chain_sync<CT>(chain);
    ++mma_phase;
    tc_fence_after();
    {
      float u[CW];
      tmem_ld<CW>(tmem_row + TPC, u);
      tmem_wait_ld();
      if (krow) {
        // U leaves as bf16 (the backward reads it back in that form); Vn_e = r_e * U is formed from the same packed row,
        // two products per instruction, and goes into the operand image (i = t, j = n'), this thread's slices
        uint32_t uw[CW / 2];
#pragma unroll
        for (int c = 0; c < CW; c += 2) uw[c >> 1] = pack_bf16(u[c], u[c + 1]);
        if (p.U != nullptr && sw == 0) {
          __nv_bfloat16* dst = p.U + (item * 64 + t) * HEAD + v0g;
          if constexpr (CW >= 8) {
#pragma unroll
            for (int c = 0; c < CW / 2; c += 4) *reinterpret_cast<uint4*>(dst + 2 * c) = make_uint4(uw[c], uw[c + 1], uw[c + 2], uw[c + 3]);
          } else {
            *reinterpret_cast<uint2*>(dst) = make_uint2(uw[0], uw[1]);
          }
        }
        const uint32_t base = smem_u32(vn_img) + (t >> 3) * 128 + (t & 7) * 16;
#pragma unroll
        for (int e = 0; e < ET; ++e) {
          const uint32_t rr = pack_bf16(gr[e], gr[e]);
          const int n0 = (e0 + e) * CW;
          if constexpr (CW >= 8) {
#pragma unroll
            for (int c = 0; c < CW / 2; c += 4)
              st_shared_v4(base + ((n0 + 2 * c) >> 3) * 1024, mul_bf16x2(uw[c], rr), mul_bf16x2(uw[c + 1], rr), mul_bf16x2(uw[c + 2], rr),
                           mul_bf16x2(uw[c + 3], rr));
          } else {
            st_shared_v2(base + (n0 >> 3) * 1024 + (n0 & 7) * 2, mul_bf16x2(uw[0], rr), mul_bf16x2(uw[1], rr));
          }
        }
      } else if (live && sw == WPC - 1) {
        float ov[CW];
#pragma unroll
        for (int c = 0; c < CW; ++c) ov[c] = acc[c] + u[c];
        store_row_global(p.o + ((tok + t) * p.H + h) * HEAD + v0g, ov);
      }
    }
    fence_async_smem();
    tc_fence_before();
    chain_sync<CT>(chain);

    // ---- (3) dS = K^T Vn, S <- d S + dS -----------------------------------------------------------------------
    if (cwarp_u == ISSUE_WARP && elect_one()) {
      tc_fence_after();
      const uint64_t da = make_desc(smem_u32(kq), 16384, 1024, LAYOUT_SW128);
      const uint64_t db = make_desc(smem_u32(vn_img), 128, 1024, LAYOUT_PLAIN);
      constexpr uint32_t idesc = make_idesc(128, TPC, 1, 1);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        umma_bf16(tmem_c, desc_advance(da, kk * 2048), desc_advance(db, kk * 256), idesc, kk > 0);
      umma_commit(&ctrl.bar_mma[chain]);
    }
    __syncwarp();
    if (cwarp_u == ISSUE_WARP) mbar_wait(&ctrl.bar_mma[chain], mma_phase & 1, ctl, DEV_TIMEOUT_MMA);
    chain_sync<CT>(chain);
    ++mma_phase;
    tc_fence_after();
    {
      float dch[ET];                                 // exp(gL) of this thread's slices
      lds_part<ET>(gf + C::GF_D + e0, dch);
      const uint32_t base = smem_u32(s_img) + (row >> 3) * 128 + (row & 7) * 16;
      uint8_t* hbase = (p.h != nullptr && i + 1 < count) ? state_item_ptr(item + p.H) : nullptr;
      float ds[2][16];
      tmem_ld<16>(tmem_row + col0, ds[0]);
#pragma unroll
      for (int pc = 0; pc < TPT / 16; ++pc) {
        const int j0 = pc * 16;
        tmem_wait_ld();
        if (pc + 1 < TPT / 16) tmem_ld<16>(tmem_row + col0 + j0 + 16, ds[(pc + 1) & 1]);
        const float* dp = ds[pc & 1];
        uint32_t packed[8];
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
          S[j0 + j] = fmaf(dch[(j0 + j) / CW], S[j0 + j], dp[j]);
          S[j0 + j + 1] = fmaf(dch[(j0 + j + 1) / CW], S[j0 + j + 1], dp[j + 1]);
          packed[j / 2] = pack_bf16(S[j0 + j], S[j0 + j + 1]);
        }
        // operand image (i = d, j = n') for the next chunk's (1)
        st_shared_v4(base + ((col0 + j0) >> 3) * 2048, packed[0], packed[1], packed[2], packed[3]);
        st_shared_v4(base + ((col0 + j0 + 8) >> 3) * 2048, packed[4], packed[5], packed[6], packed[7]);
        // saved state of the next chunk: slice e as [v/8][d][v%8]
        if (hbase != nullptr) store_state_slices(hbase, j0, packed);
      }
    }
    fence_async_smem();
    tc_fence_before();
    chain_sync<CT>(chain);
  }
  // final state for the caller (f32, same form as the initial state)
  if (p.s_out != nullptr) {
    float* dst = p.s_out + ((static_cast<int64_t>(seq) * p.H + h) * E + e0) * (HEAD * HEAD) + row * HEAD + v0g;
#pragma unroll
    for (int e = 0; e < ET; ++e)
#pragma unroll
      for (int c = 0; c < CW; ++c) dst[e * (HEAD * HEAD) + c] = S[e * CW + c];
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, C::TMEM_COLS);
}

}  // namespace tgdn

using namespace tgdn;

template <int E, int CW, int NCH, int WPC, int STAGES, int MINB>
static int launch_fwd(const CUtensorMap& mk, const CUtensorMap& mq, const void* v, const FwdParams& p, cudaStream_t s) {
  using C = FwdCfg<E, CW, NCH, WPC, STAGES>;
  static_assert(MINB == 1 || C::SMEM_BYTES <= 115712, "two CTAs per SM need at most 113 KB each");
  static_assert(C::SMEM_BYTES <= 232448, "shared memory budget of one CTA exceeded");
  static_assert(MINB * C::TMEM_COLS <= 512, "tensor memory budget of one SM exceeded");
  static bool configured[64] = {};                  // per device: the attribute is sticky, set it once
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(fwd_kernel<E, CW, NCH, WPC, STAGES, MINB>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return tgdn_cuda_error(e);
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  CUtensorMap mv = mk, mb = mk;                     // placeholders where the rows are not loaded by TMA
  if (C::TMA_V) {
    const int rc = tgdn_make_token_map(&mv, v, p.B, p.T, p.H, CW, 64, 0);
    if (rc) return rc;
  }
  if (C::TMA_BETA && p.beta_tma) {
    const int rc = tgdn_make_gate_map(&mb, p.beta, p.B, p.T, p.H / 4, 4);    // (B, T, H) read as (B, T, H/4, 4)
    if (rc) return rc;
  }
  const int grid = p.n_seq * p.H * (HEAD / C::VC);
  fwd_kernel<E, CW, NCH, WPC, STAGES, MINB><<<grid, C::THREADS, C::SMEM_BYTES, s>>>(mv, mb, mk, mq, p);
  return tgdn_cuda_error(cudaGetLastError());
}


extern "C" int tgdn_fwd_state(const void* q, const void* k, const void* v, const float* k2, const float* q2,
                              const float* beta, const float* gc, const void* AP, float scale, const int32_t* doc_offsets,
                              const int32_t* chunk_map, int n_docs, int B, int T, int H, int E, int NC, void* o, void* W,
                              void* U, void* h, const float* state_in, float* state_out, void* stream) {
  if (!q || !k || !v || !k2 || !q2 || !beta || !gc || !AP || !o) return TGDN_ERR_NULL;
  const bool packed = chunk_map != nullptr;
  if (packed && (!doc_offsets || n_docs < 1)) return TGDN_ERR_NULL;
  int rc = tgdn_check_core_shape(B, T, H, E, NC, packed);
  if (rc) return rc;
  if ((reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(AP) |
       reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(U) | reinterpret_cast<uintptr_t>(h) |
       reinterpret_cast<uintptr_t>(k2) | reinterpret_cast<uintptr_t>(q2) | reinterpret_cast<uintptr_t>(gc) |
       reinterpret_cast<uintptr_t>(state_in) | reinterpret_cast<uintptr_t>(state_out)) & 15)
    return TGDN_ERR_ALIGN;
  CUtensorMap mk, mq;
  if ((rc = tgdn_make_token_map(&mk, k, B, T, H, 64, 64, 1))) return rc;
  if ((rc = tgdn_make_token_map(&mq, q, B, T, H, 64, 64, 1))) return rc;
  FwdParams p{static_cast<const __nv_bfloat16*>(v), k2, q2, beta, gc, static_cast<const __nv_bfloat16*>(AP),
              static_cast<__nv_bfloat16*>(o), static_cast<__nv_bfloat16*>(W), static_cast<__nv_bfloat16*>(U),
              static_cast<__nv_bfloat16*>(h), state_in, state_out, doc_offsets, chunk_map, B, T, H, NC,
              packed ? n_docs : B, scale, tgdn_status_word(),
              (H % 4 == 0 && (reinterpret_cast<uintptr_t>(beta) & 15) == 0) ? 1 : 0};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (E) {
    case 1: return launch_fwd<1, 16, 2, 1, 2, 1>(mk, mq, v, p, s);
    case 2: return launch_fwd<2, 8, 4, 1, 2, 1>(mk, mq, v, p, s);
    case 4: {
      // One CTA per SM: the grid runs in whole waves.  Where a block of 32 value columns needs a second, partly filled wave
      // and a block of 64 does not, the wider block wins although its chunks take a little longer (B=4, H=16: 256 CTAs on
      // 148 SMs are two waves, 128 CTAs are one).
      const long long sms = tgdn_sm_count(), seqs = static_cast<long long>(p.n_seq) * p.H;
      const long long waves32 = (seqs * 4 + sms - 1) / sms, waves64 = (seqs * 2 + sms - 1) / sms;
      if (waves64 * 5 < waves32 * 4) return launch_fwd<4, 16, 4, 1, 2, 1>(mk, mq, v, p, s);
      return launch_fwd<4, 8, 4, 1, 2, 1>(mk, mq, v, p, s);
    }
    // (two warpgroups per chain at E = 8, sixteen columns per thread, measured 17% slower than four one-warpgroup chains)
    case 8: return launch_fwd<8, 8, 4, 1, 2, 1>(mk, mq, v, p, s);
    case 12: return launch_fwd<12, 8, 2, 2, 2, 1>(mk, mq, v, p, s);
    case 16: return launch_fwd<16, 8, 2, 2, 2, 1>(mk, mq, v, p, s);
    default: return TGDN_ERR_SHAPE;
  }
}

extern "C" int tgdn_fwd(const void* q, const void* k, const void* v, const float* k2, const float* q2, const float* beta,
                        const float* gc, const void* AP, float scale, const int32_t* doc_offsets,
                        const int32_t* chunk_map, int n_docs, int B, int T, int H, int E, int NC, void* o, void* W,
                        void* U, void* h, void* stream) {
  return tgdn_fwd_state(q, k, v, k2, q2, beta, gc, AP, scale, doc_offsets, chunk_map, n_docs, B, T, H, E, NC, o, W, U, h,
                        nullptr, nullptr, stream);
}
