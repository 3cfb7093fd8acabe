// Width-4 causal depthwise convolution with SiLU on the leading channels: forward and backward.
//
// Replaces the reference's Triton kernels cute_triadic_gdn/ops/conv_split_act.py:20-55 (_fwd_kernel) and :58-107
// (_bwd_kernel).  HBM-bound, so the kernels are built around bytes in flight: a CTA owns a tile of 256 channels and
// walks a run of 32-token tiles; the [tokens + halo][256 channels] input tiles arrive by TMA (cp.async.bulk.tensor, no
// swizzle) into a multi-stage shared-memory ring, several tiles ahead of the arithmetic, and rows before the start of a
// batch row come back as zeros from the tensor map's out-of-range fill.  Each warp computes 8 of the 32 output rows
// for the tile's 256 channels (8 channels = one 16-byte vector per lane) and stores them with coalesced 512-byte rows.
// The backward recomputes the bf16-rounded pre-activation from the same x window (the reference launches a second
// forward for it), so x and dy are read once and dx written once; the weight gradient is accumulated in registers
// over all tiles of the CTA, reduced across its warps in shared memory and written as one f32 partial per CTA; a
// second small kernel sums the partials in a fixed order.
#include <algorithm>
#include <mutex>

#include "tgdn_common.cuh"
#include "tgdn_host.h"
#include "tgdn_kernels.h"

namespace tgdn {

constexpr int CONV_W = 4;
constexpr int CONV_THREADS = 256;      // 8 warps = 4 row groups x 2 channel halves
constexpr int CONV_CH = 256;           // channels per CTA tile (2 halves x 32 lanes x 4)
constexpr int CONV_VEC = 4;            // channels per thread (one 8-byte vector)
constexpr int CONV_TOK = 32;           // output tokens per tile (4 row groups x 8 rows)
constexpr int CONV_FWD_ROWS = CONV_TOK + 3;       // x rows t0-3 .. t0+31
constexpr int CONV_BWD_XROWS = CONV_TOK + 6;      // x rows t0-3 .. t0+34
constexpr int CONV_BWD_GROWS = CONV_TOK + 3;      // dy rows t0 .. t0+34
constexpr int CONV_FWD_STAGES = 3;     // 54 KB per CTA: four CTAs per SM
constexpr int CONV_BWD_STAGES = 3;     // 112 KB per CTA: two CTAs per SM
constexpr int CONV_BWD_NP = 2;         // channel pairs per thread of the backward (512 threads per CTA)

// Four channels of a thread as two packed pairs: the arithmetic runs on the two-wide f32 instructions (one instruction per
// pair, each lane an ordinary IEEE fma), which halves the instruction count of the kernels' inner loops.
struct Vec4 {
  float2 p[2];                  // channels (0,1) and (2,3)
};

__device__ __forceinline__ Vec4 unpack4(uint2 u) {
  Vec4 r;
  r.p[0] = make_float2(bf16_lo(u.x), bf16_hi(u.x));
  r.p[1] = make_float2(bf16_lo(u.y), bf16_hi(u.y));
  return r;
}
__device__ __forceinline__ Vec4 zero4() {
  Vec4 r;
  r.p[0] = r.p[1] = make_float2(0.f, 0.f);
  return r;
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const Vec4& a) {
  *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16(a.p[0].x, a.p[0].y), pack_bf16(a.p[1].x, a.p[1].y));
}
// sigmoid with the fast exponential and the fast reciprocal: relative error of a few f32 ulps
__device__ __forceinline__ float fast_sigmoid(float y) { return __fdividef(1.f, 1.f + __expf(-y)); }
__device__ __forceinline__ float silu(float y) { return y * fast_sigmoid(y); }
// Derivative of SiLU for the backward, where the result is rounded to bf16 after further products: the sigmoid comes
// from one tanh.approx (absolute error about 2^-11) instead of an exponential and a reciprocal.
__device__ __forceinline__ float silu_grad(float y) {
  float th;
  asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(0.5f * y));
  const float s = fmaf(0.5f, th, 0.5f);
  return s * fmaf(y, 1.f - s, 1.f);
}

// Walks document boundaries as the token index grows: one binary search per tile, then a compare per token.
struct DocCursor {
  const int32_t* cu;
  int n_docs, d, start, next;
  __device__ __forceinline__ void init(const int32_t* cu_, int n_docs_, int t, int T) {
    cu = cu_; n_docs = n_docs_; d = 0; start = 0; next = 0x7fffffff;
    if (cu == nullptr) return;
    int lo = 0, hi = n_docs - 1;
    while (lo < hi) {
      int mid = (lo + hi + 1) >> 1;
      if (__ldg(cu + mid) <= t) lo = mid; else hi = mid - 1;
    }
    d = lo;
    start = __ldg(cu + d);
    next = (d + 1 < n_docs) ? __ldg(cu + d + 1) : 0x7fffffff;
  }
  // true when token t is the first token of a document that starts after the one the cursor was on
  __device__ __forceinline__ bool advance(int t) {
    if (t < next) return false;
    do {
      ++d; start = next;
      next = (d + 1 < n_docs) ? __ldg(cu + d + 1) : 0x7fffffff;
    } while (t >= next);
    return true;
  }
};

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

struct ConvArgs {
  const __nv_bfloat16* weight;
  __nv_bfloat16* out;            // y (forward) or dx (backward), contiguous (B, T, C)
  float* dw_partial;             // backward: [B * groups][C][4]
  const int32_t* cu;
  int n_docs, T, C, act_channels, tiles_per_group;
  int* status;
};

// w2[p][j]: tap j of the channel pair p (channels c0 + 2p, c0 + 2p + 1)
__device__ __forceinline__ void load_weights(const __nv_bfloat16* weight, int c0, int C, float2 (*w2)[CONV_W]) {
  float w[CONV_VEC][CONV_W];
#pragma unroll
  for (int c = 0; c < CONV_VEC; ++c)
#pragma unroll
    for (int j = 0; j < CONV_W; ++j) w[c][j] = 0.f;
  if (c0 < C) {                                 // C % 8 == 0 and c0 % 4 == 0: the four channels are all inside
    const uint4* wp = reinterpret_cast<const uint4*>(weight + static_cast<int64_t>(c0) * CONV_W);
#pragma unroll
    for (int i = 0; i < 2; ++i) {               // 4 channels x 4 taps = 16 bf16 = 2 vectors
      uint4 u = __ldg(wp + i);
      const uint32_t ws[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        int e = i * 8 + j * 2;
        w[e / 4][e % 4] = bf16_lo(ws[j]);
        w[(e + 1) / 4][(e + 1) % 4] = bf16_hi(ws[j]);
      }
    }
  }
#pragma unroll
  for (int p = 0; p < 2; ++p)
#pragma unroll
    for (int j = 0; j < CONV_W; ++j) w2[p][j] = make_float2(w[2 * p][j], w[2 * p + 1][j]);
}

__global__ void __launch_bounds__(CONV_THREADS, 4)
conv_fwd_kernel(const __grid_constant__ CUtensorMap map_x, ConvArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  constexpr int STAGE_BYTES = CONV_FWD_ROWS * CONV_CH * 2;
  __shared__ uint64_t full[CONV_FWD_STAGES];
  __shared__ int abort_s;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int half = warp & 1, rg = warp >> 1;
  const int cbase = blockIdx.x * CONV_CH, c0 = cbase + half * 128 + lane * CONV_VEC, b = blockIdx.z;
  const int n_tiles = (a.T + CONV_TOK - 1) / CONV_TOK;
  const int tile_lo = blockIdx.y * a.tiles_per_group, tile_hi = min(n_tiles, tile_lo + a.tiles_per_group);
  if (tile_lo >= tile_hi) return;
  if (tid == 0) {
    for (int s = 0; s < CONV_FWD_STAGES; ++s) mbar_init(&full[s], 1);
    mbar_fence_init();
    abort_s = 0;
  }
  __syncthreads();
  WaitCtl ctl{&abort_s, a.status};
  auto issue = [&](int tile) {                         // thread 0
    const int s = (tile - tile_lo) % CONV_FWD_STAGES;
    mbar_expect_tx(&full[s], STAGE_BYTES);
    tma_load_3d(smem + s * STAGE_BYTES, &map_x, &full[s], cbase, tile * CONV_TOK - 3, b);
  };
  if (tid == 0)
    for (int i = 0; i < CONV_FWD_STAGES && tile_lo + i < tile_hi; ++i) issue(tile_lo + i);

  float2 w2[2][CONV_W];
  load_weights(a.weight, c0, a.C, w2);
  __nv_bfloat16* yb = a.out + (static_cast<int64_t>(b) * a.T) * a.C + c0;
  const int col_off = half * 256 + lane * 8;             // byte offset of this thread's channels inside a tile row
  const bool live = c0 < a.C;
  bool act[CONV_VEC];
#pragma unroll
  for (int c = 0; c < CONV_VEC; ++c) act[c] = c0 + c < a.act_channels;

  for (int tile = tile_lo; tile < tile_hi; ++tile) {
    const int k = tile - tile_lo, s = k % CONV_FWD_STAGES;
    mbar_wait(&full[s], (k / CONV_FWD_STAGES) & 1, ctl, DEV_TIMEOUT_LOAD);
    const uint8_t* st = smem + s * STAGE_BYTES + col_off;
    const int t_first = tile * CONV_TOK + rg * 8;         // this warp's first output token; its smem row is rg*8 + 3
    DocCursor doc;
    doc.init(a.cu, a.n_docs, min(t_first, a.T - 1), a.T);
    __nv_bfloat16* yrow = yb + static_cast<int64_t>(t_first) * a.C;
    // Interior of a document and of the sequence: no start of a document among the warp's eight rows or their three halo
    // rows (rows before the sequence come back as zeros from the tensor map, which is what a start at token 0 means),
    // all eight rows exist.  Then the rows need no cursor, no bounds and no window resets; almost every tile is like this.
    const bool interior = t_first + 8 <= a.T && doc.next >= t_first + 8 && doc.start <= max(t_first - 3, 0);
    if (interior && live && (act[0] == act[3])) {
      const bool on = act[0];
      Vec4 xm[3];
#pragma unroll
      for (int j = 0; j < 3; ++j) xm[j] = unpack4(*reinterpret_cast<const uint2*>(st + (rg * 8 + 2 - j) * (CONV_CH * 2)));
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const Vec4 x0 = unpack4(*reinterpret_cast<const uint2*>(st + (rg * 8 + 3 + i) * (CONV_CH * 2)));
        Vec4 out;
#pragma unroll
        for (int p = 0; p < 2; ++p) {
          float2 acc = __fmul2_rn(xm[2].p[p], w2[p][0]);
          acc = __ffma2_rn(xm[1].p[p], w2[p][1], acc);
          acc = __ffma2_rn(xm[0].p[p], w2[p][2], acc);
          acc = __ffma2_rn(x0.p[p], w2[p][3], acc);
          out.p[p] = on ? make_float2(silu(acc.x), silu(acc.y)) : acc;
        }
        store4(yrow + static_cast<int64_t>(i) * a.C, out);
        xm[2] = xm[1]; xm[1] = xm[0]; xm[0] = x0;
      }
    } else {
      Vec4 xm[3];                                           // x[t-1], x[t-2], x[t-3]
#pragma unroll
      for (int j = 0; j < 3; ++j) {
        const int tj = t_first - 1 - j;
        xm[j] = (tj >= doc.start) ? unpack4(*reinterpret_cast<const uint2*>(st + (rg * 8 + 2 - j) * (CONV_CH * 2))) : zero4();
      }
      const int n_rows = min(8, a.T - t_first);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (i >= n_rows) break;
        if (i > 0 && doc.advance(t_first + i)) { xm[0] = zero4(); xm[1] = zero4(); xm[2] = zero4(); }   // a document starts here
        const Vec4 x0 = unpack4(*reinterpret_cast<const uint2*>(st + (rg * 8 + 3 + i) * (CONV_CH * 2)));
        Vec4 out;
#pragma unroll
        for (int p = 0; p < 2; ++p) {
          float2 acc = __fmul2_rn(xm[2].p[p], w2[p][0]);
          acc = __ffma2_rn(xm[1].p[p], w2[p][1], acc);
          acc = __ffma2_rn(xm[0].p[p], w2[p][2], acc);
          acc = __ffma2_rn(x0.p[p], w2[p][3], acc);
          out.p[p] = make_float2(act[2 * p] ? silu(acc.x) : acc.x, act[2 * p + 1] ? silu(acc.y) : acc.y);
        }
        if (live) store4(yrow, out);
        yrow += a.C;
        xm[2] = xm[1]; xm[1] = xm[0]; xm[0] = x0;
      }
    }
    __syncthreads();                                      // every warp is done with this stage
    if (tid == 0 && tile + CONV_FWD_STAGES < tile_hi) issue(tile + CONV_FWD_STAGES);
  }
}

// NP channel pairs of a thread (the forward's Vec4 is the NP = 2 case with its own helpers).
template <int NP>
struct VecP {
  float2 p[NP];
};
template <int NP>
__device__ __forceinline__ VecP<NP> load_pairs(const uint8_t* s) {
  VecP<NP> r;
  if constexpr (NP == 2) {
    const uint2 u = *reinterpret_cast<const uint2*>(s);
    r.p[0] = make_float2(bf16_lo(u.x), bf16_hi(u.x));
    r.p[1] = make_float2(bf16_lo(u.y), bf16_hi(u.y));
  } else {
    const uint32_t u = *reinterpret_cast<const uint32_t*>(s);
    r.p[0] = make_float2(bf16_lo(u), bf16_hi(u));
  }
  return r;
}
template <int NP>
__device__ __forceinline__ VecP<NP> zero_pairs() {
  VecP<NP> r;
#pragma unroll
  for (int p = 0; p < NP; ++p) r.p[p] = make_float2(0.f, 0.f);
  return r;
}
template <int NP>
__device__ __forceinline__ void store_pairs(__nv_bfloat16* dst, const VecP<NP>& a) {
  if constexpr (NP == 2)
    *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(a.p[0].x, a.p[0].y), pack_bf16(a.p[1].x, a.p[1].y));
  else
    *reinterpret_cast<uint32_t*>(dst) = pack_bf16(a.p[0].x, a.p[0].y);
}
// SiLU' of the bf16-rounded pre-activations of a channel pair: one packed conversion rounds both, the polynomial part runs
// on the two-wide f32 instructions (each lane the same bits as silu_grad).
__device__ __forceinline__ float2 silu_grad_pair(float2 pre) {
  const uint32_t r = pack_bf16(pre.x, pre.y);
  const float2 y = make_float2(bf16_lo(r), bf16_hi(r));
  const float2 h = __fmul2_rn(y, make_float2(0.5f, 0.5f));
  float2 th;
  asm("tanh.approx.f32 %0, %1;" : "=f"(th.x) : "f"(h.x));
  asm("tanh.approx.f32 %0, %1;" : "=f"(th.y) : "f"(h.y));
  const float2 half2 = make_float2(0.5f, 0.5f), one2 = make_float2(1.f, 1.f);
  const float2 s = __ffma2_rn(half2, th, half2);
  const float2 om = __ffma2_rn(s, make_float2(-1.f, -1.f), one2);
  return __fmul2_rn(s, __ffma2_rn(y, om, one2));
}

// Backward.  NP = 1: 512 threads = 4 row groups x 4 channel slices of 64, one channel pair per thread, so that the kernel
// fits 64 registers and two CTAs put 32 warps on an SM: the per-row chain (4 fma, rounding, tanh, 4 more fma) is all
// fixed-latency dependency, which only more warps per scheduler hide.
template <int NP>
__global__ void __launch_bounds__(CONV_THREADS * 2 / NP, 2)
conv_bwd_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_dy, ConvArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  constexpr int X_BYTES = CONV_BWD_XROWS * CONV_CH * 2, G_BYTES = CONV_BWD_GROWS * CONV_CH * 2;
  constexpr int STAGE_BYTES = X_BYTES + G_BYTES;
  constexpr int SLICES = 4 / NP, NCH = 2 * NP;                         // channel slices per tile, channels per thread
  constexpr int ROW = CONV_CH * 2;                                     // bytes of a tile row
  __shared__ uint64_t full[CONV_BWD_STAGES];
  __shared__ int abort_s;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int slice = warp % SLICES, rg = warp / SLICES;
  const int cin = slice * (32 * NCH) + lane * NCH;                     // first channel of the thread inside the tile
  const int cbase = blockIdx.x * CONV_CH, c0 = cbase + cin, b = blockIdx.z;
  const int n_tiles = (a.T + CONV_TOK - 1) / CONV_TOK;
  const int tile_lo = blockIdx.y * a.tiles_per_group, tile_hi = min(n_tiles, tile_lo + a.tiles_per_group);
  if (tid == 0) {
    for (int s = 0; s < CONV_BWD_STAGES; ++s) mbar_init(&full[s], 1);
    mbar_fence_init();
    abort_s = 0;
  }
  __syncthreads();
  WaitCtl ctl{&abort_s, a.status};
  auto issue = [&](int tile) {                         // thread 0
    const int s = (tile - tile_lo) % CONV_BWD_STAGES;
    mbar_expect_tx(&full[s], STAGE_BYTES);
    tma_load_3d(smem + s * STAGE_BYTES, &map_x, &full[s], cbase, tile * CONV_TOK - 3, b);
    tma_load_3d(smem + s * STAGE_BYTES + X_BYTES, &map_dy, &full[s], cbase, tile * CONV_TOK, b);
  };
  if (tid == 0)
    for (int i = 0; i < CONV_BWD_STAGES && tile_lo + i < tile_hi; ++i) issue(tile_lo + i);

  const bool live = c0 < a.C;                          // C % 8 == 0 and c0 % NCH == 0: the thread's channels are all inside
  float2 w2[NP][CONV_W];
  {
    float w[NCH][CONV_W];
#pragma unroll
    for (int c = 0; c < NCH; ++c)
#pragma unroll
      for (int j = 0; j < CONV_W; ++j) w[c][j] = 0.f;
    if (live) {
      const uint4* wp = reinterpret_cast<const uint4*>(a.weight + static_cast<int64_t>(c0) * CONV_W);
#pragma unroll
      for (int i = 0; i < NP; ++i) {                   // two channels x four taps per 16-byte vector
        const uint4 u = __ldg(wp + i);
        w[2 * i][0] = bf16_lo(u.x); w[2 * i][1] = bf16_hi(u.x); w[2 * i][2] = bf16_lo(u.y); w[2 * i][3] = bf16_hi(u.y);
        w[2 * i + 1][0] = bf16_lo(u.z); w[2 * i + 1][1] = bf16_hi(u.z);
        w[2 * i + 1][2] = bf16_lo(u.w); w[2 * i + 1][3] = bf16_hi(u.w);
      }
    }
#pragma unroll
    for (int p = 0; p < NP; ++p)
#pragma unroll
      for (int j = 0; j < CONV_W; ++j) w2[p][j] = make_float2(w[2 * p][j], w[2 * p + 1][j]);
  }
  float2 dwa[NP][CONV_W];                                              // weight gradient of the channel pairs
#pragma unroll
  for (int p = 0; p < NP; ++p)
#pragma unroll
    for (int j = 0; j < CONV_W; ++j) dwa[p][j] = make_float2(0.f, 0.f);
  __nv_bfloat16* dxb = a.out + (static_cast<int64_t>(b) * a.T) * a.C + c0;
  const int col_off = cin * 2;
  bool act[NCH];
#pragma unroll
  for (int c = 0; c < NCH; ++c) act[c] = c0 + c < a.act_channels;
  using V = VecP<NP>;

  for (int tile = tile_lo; tile < tile_hi; ++tile) {
    const int k = tile - tile_lo, s = k % CONV_BWD_STAGES;
    mbar_wait(&full[s], (k / CONV_BWD_STAGES) & 1, ctl, DEV_TIMEOUT_LOAD);
    const uint8_t* sx = smem + s * STAGE_BYTES + col_off;              // row r holds x[t0 - 3 + r]
    const uint8_t* sg = sx + X_BYTES;                                  // row r holds dy[t0 + r]
    const int t0 = tile * CONV_TOK, u_first = t0 + rg * 8;             // this warp's output tokens u_first .. +7
    // dx[u] = sum_j dy'[u+j] w[3-j] over tokens of the same document; dy'[t] needs x[t-3..t].  Walk t = u_first .. u_first+10
    // (three tokens past the warp's rows) with the x window and the last three dy' in registers.
    DocCursor doc;
    doc.init(a.cu, a.n_docs, min(u_first, a.T - 1), a.T);
    // Interior of a document and of the sequence: no start of a document among the eleven tokens the warp walks or their
    // three halo rows, and all of them exist.  Then no cursor, no bounds and no masks are needed; almost every tile is
    // like this.
    const bool interior = u_first + 11 <= a.T && doc.next >= u_first + 11 && doc.start <= max(u_first - 3, 0);
    if (interior && live && (act[0] == act[NCH - 1])) {
      const bool on = act[0];
      V xw[3];
#pragma unroll
      for (int j = 0; j < 3; ++j) xw[j] = load_pairs<NP>(sx + (rg * 8 + 2 - j) * ROW);
      V gw[3] = {zero_pairs<NP>(), zero_pairs<NP>(), zero_pairs<NP>()};
      __nv_bfloat16* dxr = dxb + static_cast<int64_t>(u_first) * a.C;
#pragma unroll
      for (int i = 0; i < 11; ++i) {
        const V x0 = load_pairs<NP>(sx + (rg * 8 + 3 + i) * ROW);
        V gy = load_pairs<NP>(sg + (rg * 8 + i) * ROW);
        if (on) {
#pragma unroll
          for (int p = 0; p < NP; ++p) {
            float2 pre = __fmul2_rn(xw[2].p[p], w2[p][0]);
            pre = __ffma2_rn(xw[1].p[p], w2[p][1], pre);
            pre = __ffma2_rn(xw[0].p[p], w2[p][2], pre);
            pre = __ffma2_rn(x0.p[p], w2[p][3], pre);
            gy.p[p] = __fmul2_rn(gy.p[p], silu_grad_pair(pre));
          }
        }
        if (i < 8) {
#pragma unroll
          for (int p = 0; p < NP; ++p) {
            dwa[p][0] = __ffma2_rn(gy.p[p], xw[2].p[p], dwa[p][0]);
            dwa[p][1] = __ffma2_rn(gy.p[p], xw[1].p[p], dwa[p][1]);
            dwa[p][2] = __ffma2_rn(gy.p[p], xw[0].p[p], dwa[p][2]);
            dwa[p][3] = __ffma2_rn(gy.p[p], x0.p[p], dwa[p][3]);
          }
        }
        if (i >= 3) {
          V out;
#pragma unroll
          for (int p = 0; p < NP; ++p) {
            float2 acc = __fmul2_rn(gw[2].p[p], w2[p][3]);
            acc = __ffma2_rn(gw[1].p[p], w2[p][2], acc);
            acc = __ffma2_rn(gw[0].p[p], w2[p][1], acc);
            acc = __ffma2_rn(gy.p[p], w2[p][0], acc);
            out.p[p] = acc;
          }
          store_pairs<NP>(dxr, out);
          dxr += a.C;
        }
        gw[2] = gw[1]; gw[1] = gw[0]; gw[0] = gy;
        xw[2] = xw[1]; xw[1] = xw[0]; xw[0] = x0;
      }
    } else {
      V xw[3];                                                           // x[t-1], x[t-2], x[t-3]
#pragma unroll
      for (int j = 0; j < 3; ++j) {
        const int tj = u_first - 1 - j;
        xw[j] = (tj >= doc.start) ? load_pairs<NP>(sx + (rg * 8 + 2 - j) * ROW) : zero_pairs<NP>();
      }
      V gw[3] = {zero_pairs<NP>(), zero_pairs<NP>(), zero_pairs<NP>()};  // dy'[t-1], dy'[t-2], dy'[t-3]
      int ds1 = 0x7fffffff, ds2 = 0x7fffffff;                            // document starts of tokens t-1, t-2
#pragma unroll
      for (int i = 0; i < 11; ++i) {
        const int t = u_first + i;
        V gy = zero_pairs<NP>(), x0 = zero_pairs<NP>();
        int ds0 = 0x7fffffff;
        if (t < a.T) {
          if (i > 0 && doc.advance(t)) { xw[0] = zero_pairs<NP>(); xw[1] = zero_pairs<NP>(); xw[2] = zero_pairs<NP>(); }
          ds0 = doc.start;
          x0 = load_pairs<NP>(sx + (rg * 8 + 3 + i) * ROW);
          const V g = load_pairs<NP>(sg + (rg * 8 + i) * ROW);
#pragma unroll
          for (int p = 0; p < NP; ++p) {                                 // dy'[t] = dy[t] * silu'(bf16(pre-activation[t]))
            float2 pre = __fmul2_rn(xw[2].p[p], w2[p][0]);
            pre = __ffma2_rn(xw[1].p[p], w2[p][1], pre);
            pre = __ffma2_rn(xw[0].p[p], w2[p][2], pre);
            pre = __ffma2_rn(x0.p[p], w2[p][3], pre);
            const float2 sgp = silu_grad_pair(pre);
            gy.p[p] = __fmul2_rn(g.p[p], make_float2(act[2 * p] ? sgp.x : 1.f, act[2 * p + 1] ? sgp.y : 1.f));
          }
          if (i < 8) {                                                   // the weight gradient of token t belongs to this warp
#pragma unroll
            for (int p = 0; p < NP; ++p) {
              dwa[p][0] = __ffma2_rn(gy.p[p], xw[2].p[p], dwa[p][0]);
              dwa[p][1] = __ffma2_rn(gy.p[p], xw[1].p[p], dwa[p][1]);
              dwa[p][2] = __ffma2_rn(gy.p[p], xw[0].p[p], dwa[p][2]);
              dwa[p][3] = __ffma2_rn(gy.p[p], x0.p[p], dwa[p][3]);
            }
          }
        }
        if (i >= 3) {
          const int u = t - 3;
          if (u < a.T && live) {
            const float m2 = (ds2 <= u) ? 1.f : 0.f, m1 = (ds1 <= u) ? 1.f : 0.f, m0 = (ds0 <= u) ? 1.f : 0.f;
            const float2 m22 = make_float2(m2, m2), m12 = make_float2(m1, m1), m02 = make_float2(m0, m0);
            V out;
#pragma unroll
            for (int p = 0; p < NP; ++p) {
              float2 acc = __fmul2_rn(gw[2].p[p], w2[p][3]);
              acc = __ffma2_rn(__fmul2_rn(m22, gw[1].p[p]), w2[p][2], acc);
              acc = __ffma2_rn(__fmul2_rn(m12, gw[0].p[p]), w2[p][1], acc);
              acc = __ffma2_rn(__fmul2_rn(m02, gy.p[p]), w2[p][0], acc);
              out.p[p] = acc;
            }
            store_pairs<NP>(dxb + static_cast<int64_t>(u) * a.C, out);
          }
        }
        gw[2] = gw[1]; gw[1] = gw[0]; gw[0] = gy;
        ds2 = ds1; ds1 = ds0;
        xw[2] = xw[1]; xw[1] = xw[0]; xw[0] = x0;
      }
    }
    __syncthreads();
    if (tid == 0 && tile + CONV_BWD_STAGES < tile_hi) issue(tile + CONV_BWD_STAGES);
  }
  // weight-gradient partial of this CTA: sum over its four row groups in a fixed order through shared memory
  float* red = reinterpret_cast<float*>(smem);                         // [4 row groups][256 channels][4 taps]
  __syncthreads();
#pragma unroll
  for (int p = 0; p < NP; ++p) {
    float* dst = red + (rg * CONV_CH + cin + 2 * p) * CONV_W;
    *reinterpret_cast<float4*>(dst) = make_float4(dwa[p][0].x, dwa[p][1].x, dwa[p][2].x, dwa[p][3].x);
    *reinterpret_cast<float4*>(dst + CONV_W) = make_float4(dwa[p][0].y, dwa[p][1].y, dwa[p][2].y, dwa[p][3].y);
  }
  __syncthreads();
  float* out = a.dw_partial + (static_cast<int64_t>(b) * gridDim.y + blockIdx.y) * (static_cast<int64_t>(a.C) * CONV_W);
  for (int e = tid; e < CONV_CH * CONV_W; e += blockDim.x) {
    const int ch = cbase + e / CONV_W;
    if (ch < a.C)
      out[static_cast<int64_t>(ch) * CONV_W + e % CONV_W] =
          (red[e] + red[CONV_CH * CONV_W + e]) + (red[2 * CONV_CH * CONV_W + e] + red[3 * CONV_CH * CONV_W + e]);
  }
}

__global__ void conv_dw_reduce_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ dw, int n_partial,
                                      int n_elem) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_elem) return;
  float acc = 0.f;
  for (int p = 0; p < n_partial; ++p) acc += partial[static_cast<int64_t>(p) * n_elem + i];
  dw[i] = __float2bfloat16_rn(acc);
}

}  // namespace tgdn

using namespace tgdn;

static int conv_check(const void* x, const void* weight, const void* y, const int32_t* cu, int n_docs, int B, int T,
                      int C, int64_t stride_b, int64_t stride_t) {
  if (!x || !weight || !y) return TGDN_ERR_NULL;
  if (B <= 0 || T <= 0 || C <= 0 || C % 8) return TGDN_ERR_SHAPE;
  if (cu && (B != 1 || n_docs < 1)) return TGDN_ERR_SHAPE;
  if (B > 65535) return TGDN_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(y)) & 15)
    return TGDN_ERR_ALIGN;
  if ((stride_b % 8) || (stride_t % 8) || stride_t < C) return TGDN_ERR_ALIGN;
  return 0;
}

// Token tiles per CTA and number of CTAs along the token axis.  A CTA walks a run of tokens with its ring of tiles in flight,
// and each CTA of the backward leaves a weight-gradient partial, so runs should be long; but the grid must not end in a
// nearly empty wave (306 CTAs on 296 resident slots take as long as 592), and the SMs do not finish in step, so several
// short waves balance better than one long one.  Measured at (1, 32768, 13056): the time falls until about four waves
// (backward) or six (forward) and is flat beyond, until the partials of the backward start to cost.  So: as many token
// groups as fill `waves` waves of resident CTAs without spilling into the next, with runs of at least eight tiles.
static void conv_groups(int B, int T, int C, int ctas_per_sm, int waves, int* groups, int* tiles_per_group) {
  const int n_tiles = (T + CONV_TOK - 1) / CONV_TOK;
  const int64_t columns = static_cast<int64_t>((C + CONV_CH - 1) / CONV_CH) * B;      // CTAs per token group
  int64_t g = static_cast<int64_t>(waves) * ctas_per_sm * tgdn_sm_count() / columns;   // 148 on a B200 (and without a device)
  if (g > n_tiles / 8) g = n_tiles / 8;
  if (g < 1) g = 1;
  *tiles_per_group = static_cast<int>((n_tiles + g - 1) / g);
  *groups = (n_tiles + *tiles_per_group - 1) / *tiles_per_group;
}
constexpr int CONV_FWD_WAVES = 6, CONV_BWD_WAVES = 4;

extern "C" int tgdn_conv_fwd(const void* x, const void* weight, void* y, const int32_t* cu_seqlens, int n_docs, int B,
                             int T, int C, int64_t stride_b, int64_t stride_t, int act_channels, void* stream) {
  int rc = conv_check(x, weight, y, cu_seqlens, n_docs, B, T, C, stride_b, stride_t);
  if (rc) return rc;
  // the device query also binds the CUDA context to the calling thread, which the tensor-map encoder needs
  if (!tgdn_check_device()) return TGDN_ERR_DEVICE;
  CUtensorMap mx;
  if ((rc = tgdn_make_rows_map(&mx, x, C, T, B, stride_t, stride_b, CONV_CH, CONV_FWD_ROWS))) return rc;
  int groups, tpg;
  conv_groups(B, T, C, 4, CONV_FWD_WAVES, &groups, &tpg);
  ConvArgs a{static_cast<const __nv_bfloat16*>(weight), static_cast<__nv_bfloat16*>(y), nullptr, cu_seqlens, n_docs, T, C,
             act_channels, tpg, tgdn_status_word()};
  const int smem = CONV_FWD_STAGES * CONV_FWD_ROWS * CONV_CH * 2 + 128;
  cudaError_t e = cudaFuncSetAttribute(conv_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return tgdn_cuda_error(e);
  dim3 grid((C + CONV_CH - 1) / CONV_CH, groups, B);
  conv_fwd_kernel<<<grid, CONV_THREADS, smem, static_cast<cudaStream_t>(stream)>>>(mx, a);
  return tgdn_cuda_error(cudaGetLastError());
}

extern "C" int64_t tgdn_conv_bwd_scratch_bytes(int B, int T, int C) {
  if (B <= 0 || T <= 0 || C <= 0) return 0;
  int groups, tpg;
  conv_groups(B, T, C, 2, CONV_BWD_WAVES, &groups, &tpg);
  return static_cast<int64_t>(B) * groups * C * CONV_W * static_cast<int64_t>(sizeof(float));
}

// Shared by tgdn_conv_bwd and tgdn_conv_bwd_static: both kernels of the backward with the partials in `scratch`.
static int conv_bwd_launch(const void* x, const void* weight, const void* dy, void* dx, void* dw, const int32_t* cu_seqlens,
                           int n_docs, int B, int T, int C, int64_t stride_b, int64_t stride_t, int64_t dy_stride_b,
                           int64_t dy_stride_t, int act_channels, float* scratch, cudaStream_t s) {
  // the device query also binds the CUDA context to the calling thread (autograd runs the backward on a worker thread
  // that may not have made a runtime call yet), which the tensor-map encoder needs
  if (!tgdn_check_device()) return TGDN_ERR_DEVICE;
  CUtensorMap mx, mg;
  int rc;
  if ((rc = tgdn_make_rows_map(&mx, x, C, T, B, stride_t, stride_b, CONV_CH, CONV_BWD_XROWS))) return rc;
  if ((rc = tgdn_make_rows_map(&mg, dy, C, T, B, dy_stride_t, dy_stride_b, CONV_CH, CONV_BWD_GROWS))) return rc;
  int groups, tpg;
  conv_groups(B, T, C, 2, CONV_BWD_WAVES, &groups, &tpg);
  ConvArgs a{static_cast<const __nv_bfloat16*>(weight), static_cast<__nv_bfloat16*>(dx), scratch, cu_seqlens, n_docs, T, C,
             act_channels, tpg, tgdn_status_word()};
  const int smem = CONV_BWD_STAGES * (CONV_BWD_XROWS + CONV_BWD_GROWS) * CONV_CH * 2 + 128;
  cudaError_t e = cudaFuncSetAttribute(conv_bwd_kernel<CONV_BWD_NP>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return tgdn_cuda_error(e);
  dim3 grid((C + CONV_CH - 1) / CONV_CH, groups, B);
  conv_bwd_kernel<CONV_BWD_NP><<<grid, CONV_THREADS * 2 / CONV_BWD_NP, smem, s>>>(mx, mg, a);
  rc = tgdn_cuda_error(cudaGetLastError());
  if (rc) return rc;
  const int n_elem = C * CONV_W;
  conv_dw_reduce_kernel<<<(n_elem + 255) / 256, 256, 0, s>>>(scratch, static_cast<__nv_bfloat16*>(dw), B * groups, n_elem);
  return tgdn_cuda_error(cudaGetLastError());
}

extern "C" int tgdn_conv_bwd(const void* x, const void* weight, const void* dy, void* dx, void* dw,
                             const int32_t* cu_seqlens, int n_docs, int B, int T, int C, int64_t stride_b,
                             int64_t stride_t, int64_t dy_stride_b, int64_t dy_stride_t, int act_channels, void* scratch,
                             int64_t scratch_bytes, void* stream) {
  int rc = conv_check(x, weight, dx, cu_seqlens, n_docs, B, T, C, stride_b, stride_t);
  if (rc) return rc;
  if (!dy || !dw) return TGDN_ERR_NULL;
  if ((reinterpret_cast<uintptr_t>(dy) & 15) || (dy_stride_b % 8) || (dy_stride_t % 8) || dy_stride_t < C) return TGDN_ERR_ALIGN;
  if (!scratch || scratch_bytes < tgdn_conv_bwd_scratch_bytes(B, T, C) || (reinterpret_cast<uintptr_t>(scratch) & 15))
    return TGDN_ERR_SCRATCH;
  return conv_bwd_launch(x, weight, dy, dx, dw, cu_seqlens, n_docs, B, T, C, stride_b, stride_t, dy_stride_b, dy_stride_t,
                         act_channels, static_cast<float*>(scratch), static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------------------------------------------------------------
// tgdn_conv_bwd_static: the same backward, for hosts that may not allocate device memory.
//
// Some embedders load this library into a process whose device memory is owned by someone else: an inference server
// with a fixed arena, a plugin inside a framework that forbids cudaMalloc on its worker threads, a latency-critical loop
// in which an allocation (which can synchronise the whole device, or fail once memory is fragmented) is not acceptable.
// They can hand over inputs and outputs but have no pool to take the weight-gradient partials from.  For them the
// partials live in a fixed array that is part of the library image itself.
//
// The array costs TGDN_CONV_STATIC_SCRATCH_BYTES on every GPU that loads the library, until the process exits.
// Its device address is looked up once per device (cudaGetSymbolAddress, with that device current) on the first call
// made on that device; make that first call outside any stream capture.  The array is shared by every call on the
// device and keeps whatever the previous call left in it: this kernel overwrites every partial it later reads, so
// nothing has to be cleared, but two calls that overlap on the GPU (different streams) would corrupt each other.
// ---------------------------------------------------------------------------------------------------------------------
static __device__ __align__(256) float g_conv_static_scratch[TGDN_CONV_STATIC_SCRATCH_BYTES / sizeof(float)];

namespace {
constexpr int kMaxDevices = 64;
float* g_static_ptr[kMaxDevices] = {nullptr};
std::mutex g_static_mutex;

// Device address of the static scratch array on the current device (looked up once per device).
int conv_static_scratch(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return tgdn_cuda_error(e);
  if (dev < 0 || dev >= kMaxDevices) return TGDN_ERR_DEVICE;
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_ptr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_conv_static_scratch);
    if (e != cudaSuccess) return tgdn_cuda_error(e);
    g_static_ptr[dev] = p;
  }
  *out = g_static_ptr[dev];
  return 0;
}
}  // namespace

extern "C" int tgdn_conv_bwd_static(const void* x, const void* weight, const void* dy, void* dx, void* dw,
                                    const int32_t* cu_seqlens, int n_docs, int B, int T, int C, int64_t stride_b,
                                    int64_t stride_t, int64_t dy_stride_b, int64_t dy_stride_t, int act_channels,
                                    void* stream) {
  int rc = conv_check(x, weight, dx, cu_seqlens, n_docs, B, T, C, stride_b, stride_t);
  if (rc) return rc;
  if (!dy || !dw) return TGDN_ERR_NULL;
  if ((reinterpret_cast<uintptr_t>(dy) & 15) || (dy_stride_b % 8) || (dy_stride_t % 8) || dy_stride_t < C) return TGDN_ERR_ALIGN;
  if (tgdn_conv_bwd_scratch_bytes(B, T, C) > static_cast<int64_t>(TGDN_CONV_STATIC_SCRATCH_BYTES)) return TGDN_ERR_STATIC_LIMIT;
  float* scratch = nullptr;
  if ((rc = conv_static_scratch(&scratch))) return rc;
  return conv_bwd_launch(x, weight, dy, dx, dw, cu_seqlens, n_docs, B, T, C, stride_b, stride_t, dy_stride_b, dy_stride_t,
                         act_channels, scratch, static_cast<cudaStream_t>(stream));
}

// ----------------------------------------------------------------------------------------------------------------------
// The layer glue around the convolution, fused: x (B, T, C) with C = H (3*128 + 2E) channels laid out as
// [q: H x 128 | k: H x 128 | v: H x 128 | k2: H x E | q2: H x E] goes straight to the tensors the core takes:
//   q, k  = l2norm(SiLU(conv))   bf16 (B, T, H, 128)         v = SiLU(conv)   bf16 (B, T, H, 128)
//   k2, q2 = l2norm(softplus(conv))   f32 (B, T, H, E)        l2norm(s) = s * rsqrt(sum s^2 + eps)
// which the reference only describes (cute_triadic_gdn/ops/conv_split_act.py:3-5: "q, k, v (SiLU) and its second key and
// query (no activation, softplus afterwards)"); its callers run the split, the activations and the norms as separate
// elementwise passes over (T, C).  Here nothing of the convolution's output is written in between.
//
// Main kernel (both directions): the forward's tiling, a warp owning one head's 128 channels of 8 token rows, so that a
// head's norm is a sum over the 32 lanes.  Forward: writes q, k, v.  Backward: recomputes s = SiLU(conv) from the same x
// window, takes the gradients of q, k, v and writes the gradient of s, which is what the convolution's own backward takes:
//   ds = r dy - r^3 <s, dy> s,   r = rsqrt(sum s^2 + eps)              (v: ds = dv)
// Gate kernel (both directions): one thread per (token, head, k2 | q2), E channels each, straight from global memory (the
// gate channels are 2E of 384 + 2E per head).  Backward writes dc = du * sigmoid(c) with du as above for u = softplus(c).
// ----------------------------------------------------------------------------------------------------------------------
namespace tgdn {

struct GlueArgs {
  const __nv_bfloat16* weight;
  const int32_t* cu;
  int n_docs, T, C, H, E, tiles_per_group;
  float eps;
  // forward: outputs; backward: the gradients of the same tensors
  __nv_bfloat16 *q, *k, *v;      // (B, T, H, 128) each
  float *k2, *q2;                // (B, T, H, E) each
  __nv_bfloat16* dy;             // backward: (B, T, C) gradient for the convolution's backward
  const __nv_bfloat16* x;        // gate kernel: the input itself (element strides below)
  int64_t stride_b, stride_t;
  int* status;
};

template <bool BWD>
__global__ void __launch_bounds__(CONV_THREADS, BWD ? 3 : 4)
glue_main_kernel(const __grid_constant__ CUtensorMap map_x, GlueArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  constexpr int STAGE_BYTES = CONV_FWD_ROWS * CONV_CH * 2;
  __shared__ uint64_t full[CONV_FWD_STAGES];
  __shared__ int abort_s;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int half = warp & 1, rg = warp >> 1;
  const int cbase = blockIdx.x * CONV_CH, c0 = cbase + half * 128 + lane * CONV_VEC, b = blockIdx.z;
  const int n_tiles = (a.T + CONV_TOK - 1) / CONV_TOK;
  const int tile_lo = blockIdx.y * a.tiles_per_group, tile_hi = min(n_tiles, tile_lo + a.tiles_per_group);
  if (tile_lo >= tile_hi) return;
  if (tid == 0) {
    for (int s = 0; s < CONV_FWD_STAGES; ++s) mbar_init(&full[s], 1);
    mbar_fence_init();
    abort_s = 0;
  }
  __syncthreads();
  WaitCtl ctl{&abort_s, a.status};
  auto issue = [&](int tile) {                         // thread 0
    const int s = (tile - tile_lo) % CONV_FWD_STAGES;
    mbar_expect_tx(&full[s], STAGE_BYTES);
    tma_load_3d(smem + s * STAGE_BYTES, &map_x, &full[s], cbase, tile * CONV_TOK - 3, b);
  };
  if (tid == 0)
    for (int i = 0; i < CONV_FWD_STAGES && tile_lo + i < tile_hi; ++i) issue(tile_lo + i);

  // this warp's head: unit = which 128-channel block of [q heads | k heads | v heads]
  const int unit = (cbase + half * 128) >> 7;
  const bool live = unit < 3 * a.H;                    // a last, half-filled channel tile
  const int region = live ? unit / a.H : 0, head = live ? unit % a.H : 0;
  const bool normed = region < 2;
  float2 w2[2][CONV_W];
  load_weights(a.weight, c0, live ? a.C : 0, w2);
  __nv_bfloat16* tb = (region == 0 ? a.q : region == 1 ? a.k : a.v) + ((static_cast<int64_t>(b) * a.T) * a.H + head) * HEAD + lane * CONV_VEC;
  __nv_bfloat16* dyb = BWD ? a.dy + (static_cast<int64_t>(b) * a.T) * a.C + c0 : nullptr;
  const int col_off = half * 256 + lane * 8;
  const int64_t trow = static_cast<int64_t>(a.H) * HEAD;    // elements between token rows of q, k, v

  for (int tile = tile_lo; tile < tile_hi; ++tile) {
    const int k = tile - tile_lo, s = k % CONV_FWD_STAGES;
    mbar_wait(&full[s], (k / CONV_FWD_STAGES) & 1, ctl, DEV_TIMEOUT_LOAD);
    const uint8_t* st = smem + s * STAGE_BYTES + col_off;
    const int t_first = tile * CONV_TOK + rg * 8;
    DocCursor doc;
    doc.init(a.cu, a.n_docs, min(t_first, a.T - 1), a.T);
    Vec4 xm[3];                                           // x[t-1], x[t-2], x[t-3]
#pragma unroll
    for (int j = 0; j < 3; ++j) {
      const int tj = t_first - 1 - j;
      xm[j] = (tj >= doc.start) ? unpack4(*reinterpret_cast<const uint2*>(st + (rg * 8 + 2 - j) * (CONV_CH * 2))) : zero4();
    }
    const int n_rows = live ? min(8, a.T - t_first) : 0;
    // Interior of a document and of the sequence (almost every tile): no document starts among the warp's eight rows or
    // their three halo rows and all eight rows exist, so the rows need no cursor and no bounds.
    const bool interior = live && t_first + 8 <= a.T && doc.next >= t_first + 8 && doc.start <= max(t_first - 3, 0);
    // the gradient rows of this warp's eight tokens are asked for before the arithmetic needs them
    uint2 gin[8];
    if constexpr (BWD) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        gin[i] = (i < n_rows) ? __ldg(reinterpret_cast<const uint2*>(tb + (t_first + i) * trow)) : make_uint2(0u, 0u);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (!interior) {                                     // warp-uniform
        if (i >= n_rows) break;
        if (i > 0 && doc.advance(t_first + i)) { xm[0] = zero4(); xm[1] = zero4(); xm[2] = zero4(); }   // a document starts here
      }
      const Vec4 x0 = unpack4(*reinterpret_cast<const uint2*>(st + (rg * 8 + 3 + i) * (CONV_CH * 2)));
      Vec4 sv;
      float ss = 0.f;
#pragma unroll
      for (int p = 0; p < 2; ++p) {
        float2 acc = __fmul2_rn(xm[2].p[p], w2[p][0]);
        acc = __ffma2_rn(xm[1].p[p], w2[p][1], acc);
        acc = __ffma2_rn(xm[0].p[p], w2[p][2], acc);
        acc = __ffma2_rn(x0.p[p], w2[p][3], acc);
        sv.p[p] = make_float2(silu(acc.x), silu(acc.y));
        ss = fmaf(sv.p[p].x, sv.p[p].x, fmaf(sv.p[p].y, sv.p[p].y, ss));
      }
      if constexpr (!BWD) {
        float r = 1.f;
        if (normed) {
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
          r = rsqrtf(ss + a.eps);
        }
        Vec4 out;
        out.p[0] = make_float2(sv.p[0].x * r, sv.p[0].y * r);
        out.p[1] = make_float2(sv.p[1].x * r, sv.p[1].y * r);
        store4(tb + (t_first + i) * trow, out);
      } else {
        Vec4 g = unpack4(gin[i]);
        if (normed) {
          float dot = fmaf(sv.p[0].x, g.p[0].x, fmaf(sv.p[0].y, g.p[0].y, fmaf(sv.p[1].x, g.p[1].x, sv.p[1].y * g.p[1].y)));
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            ss += __shfl_xor_sync(0xffffffffu, ss, o);
            dot += __shfl_xor_sync(0xffffffffu, dot, o);
          }
          const float r = rsqrtf(ss + a.eps), f = r * r * r * dot;
#pragma unroll
          for (int p = 0; p < 2; ++p) g.p[p] = make_float2(fmaf(r, g.p[p].x, -f * sv.p[p].x), fmaf(r, g.p[p].y, -f * sv.p[p].y));
        }
        store4(dyb + static_cast<int64_t>(t_first + i) * a.C, g);
      }
      xm[2] = xm[1]; xm[1] = xm[0]; xm[0] = x0;
    }
    __syncthreads();                                      // every warp is done with this stage
    if (tid == 0 && tile + CONV_FWD_STAGES < tile_hi) issue(tile + CONV_FWD_STAGES);
  }
}

template <int E, bool BWD>
__global__ void __launch_bounds__(256)
glue_gate_kernel(GlueArgs a, int B) {
  const int64_t n = static_cast<int64_t>(B) * a.T * 2 * a.H;
  const int gbase = 3 * a.H * HEAD;                    // first gate channel
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < n;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    int u, t, b;                                        // u = which * H + head: consecutive threads, consecutive channel groups
    if (n <= 0x7fffffffLL) {                            // 64-bit divisions cost a few hundred cycles each: avoid them where 32 bits do
      const int i32 = static_cast<int>(idx), bt = i32 / (2 * a.H);
      u = i32 - bt * (2 * a.H);
      b = bt / a.T;
      t = bt - b * a.T;
    } else {
      u = static_cast<int>(idx % (2 * a.H));
      const int64_t bt = idx / (2 * a.H);
      t = static_cast<int>(bt % a.T);
      b = static_cast<int>(bt / a.T);
    }
    const int which = u / a.H, head = u % a.H;
    const int c0 = gbase + u * E;
    int start = 0;                                      // first token of t's document
    if (a.cu != nullptr) {
      int lo = 0, hi = a.n_docs - 1;
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (__ldg(a.cu + mid) <= t) lo = mid; else hi = mid - 1;
      }
      start = __ldg(a.cu + lo);
    }
    float c[E];
#pragma unroll
    for (int e = 0; e < E; ++e) c[e] = 0.f;
    const __nv_bfloat16* xb = a.x + b * a.stride_b + c0;
    // taps of the E channels: four bf16 = one 8-byte load per channel (c0 * 4 taps * 2 bytes is a multiple of 8)
    float w[E][CONV_W];
#pragma unroll
    for (int e = 0; e < E; ++e) {
      const uint2 u2 = __ldg(reinterpret_cast<const uint2*>(a.weight + static_cast<int64_t>(c0 + e) * CONV_W));
      w[e][0] = bf16_lo(u2.x); w[e][1] = bf16_hi(u2.x); w[e][2] = bf16_lo(u2.y); w[e][3] = bf16_hi(u2.y);
    }
#pragma unroll
    for (int j = 0; j < CONV_W; ++j) {
      const int tj = t - 3 + j;
      if (tj < start) continue;
      const __nv_bfloat16* xr = xb + tj * a.stride_t;
      if constexpr (E % 4 == 0) {                       // rows and c0 are multiples of 4 channels: 8-byte loads
#pragma unroll
        for (int e = 0; e < E; e += 4) {
          const uint2 u2 = __ldg(reinterpret_cast<const uint2*>(xr + e));
          c[e] = fmaf(bf16_lo(u2.x), w[e][j], c[e]);
          c[e + 1] = fmaf(bf16_hi(u2.x), w[e + 1][j], c[e + 1]);
          c[e + 2] = fmaf(bf16_lo(u2.y), w[e + 2][j], c[e + 2]);
          c[e + 3] = fmaf(bf16_hi(u2.y), w[e + 3][j], c[e + 3]);
        }
      } else {
#pragma unroll
        for (int e = 0; e < E; ++e) c[e] = fmaf(__bfloat162float(xr[e]), w[e][j], c[e]);
      }
    }
    float uu[E], ss = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) {
      uu[e] = c[e] > 15.f ? c[e] : __logf(1.f + __expf(c[e]));     // softplus; absolute error below 1e-7 at either end
      ss = fmaf(uu[e], uu[e], ss);
    }
    const float r = rsqrtf(ss + a.eps);
    float* gp = (which == 0 ? a.k2 : a.q2) + ((static_cast<int64_t>(b) * a.T + t) * a.H + head) * E;
    if constexpr (!BWD) {
#pragma unroll
      for (int e = 0; e < E; ++e) gp[e] = uu[e] * r;
    } else {
      float g[E], dot = 0.f;
#pragma unroll
      for (int e = 0; e < E; ++e) {
        g[e] = gp[e];
        dot = fmaf(uu[e], g[e], dot);
      }
      const float f = r * r * r * dot;
      __nv_bfloat16* dyr = a.dy + (static_cast<int64_t>(b) * a.T + t) * a.C + c0;
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const float du = fmaf(r, g[e], -f * uu[e]);
        dyr[e] = __float2bfloat16_rn(du * fast_sigmoid(c[e]));      // d softplus = sigmoid
      }
    }
  }
}

}  // namespace tgdn

using namespace tgdn;

template <bool BWD>
static int glue_launch(const void* x, const void* weight, const int32_t* cu, int n_docs, int B, int T, int C, int64_t stride_b,
                       int64_t stride_t, int H, int E, float eps, void* q, void* k, void* v, float* k2, float* q2, void* dy,
                       cudaStream_t s) {
  if (!q || !k || !v || !k2 || !q2 || (BWD && !dy)) return TGDN_ERR_NULL;
  int rc = conv_check(x, weight, q, cu, n_docs, B, T, C, stride_b, stride_t);
  if (rc) return rc;
  if (H <= 0 || C != H * (3 * HEAD + 2 * E)) return TGDN_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(dy)) & 15) return TGDN_ERR_ALIGN;
  if (!tgdn_check_device()) return TGDN_ERR_DEVICE;
  CUtensorMap mx;
  if ((rc = tgdn_make_rows_map(&mx, x, C, T, B, stride_t, stride_b, CONV_CH, CONV_FWD_ROWS))) return rc;
  const int main_channels = 3 * H * HEAD;
  int groups, tpg;
  conv_groups(B, T, main_channels, 4, CONV_FWD_WAVES, &groups, &tpg);
  GlueArgs a{static_cast<const __nv_bfloat16*>(weight), cu, n_docs, T, C, H, E, tpg, eps,
             static_cast<__nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(k), static_cast<__nv_bfloat16*>(v), k2, q2,
             static_cast<__nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x), stride_b, stride_t, tgdn_status_word()};
  const int smem = CONV_FWD_STAGES * CONV_FWD_ROWS * CONV_CH * 2 + 128;
  cudaError_t e = cudaFuncSetAttribute(glue_main_kernel<BWD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return tgdn_cuda_error(e);
  dim3 grid((main_channels + CONV_CH - 1) / CONV_CH, groups, B);
  glue_main_kernel<BWD><<<grid, CONV_THREADS, smem, s>>>(mx, a);
  if ((e = cudaGetLastError()) != cudaSuccess) return tgdn_cuda_error(e);
  const int64_t n = static_cast<int64_t>(B) * T * 2 * H;
  const int blocks = static_cast<int>(std::min<int64_t>((n + 255) / 256, static_cast<int64_t>(tgdn_sm_count()) * 16));
  switch (E) {
    case 1: glue_gate_kernel<1, BWD><<<blocks, 256, 0, s>>>(a, B); break;
    case 2: glue_gate_kernel<2, BWD><<<blocks, 256, 0, s>>>(a, B); break;
    case 4: glue_gate_kernel<4, BWD><<<blocks, 256, 0, s>>>(a, B); break;
    case 8: glue_gate_kernel<8, BWD><<<blocks, 256, 0, s>>>(a, B); break;
    case 12: glue_gate_kernel<12, BWD><<<blocks, 256, 0, s>>>(a, B); break;
    case 16: glue_gate_kernel<16, BWD><<<blocks, 256, 0, s>>>(a, B); break;
    default: return TGDN_ERR_SHAPE;
  }
  return tgdn_cuda_error(cudaGetLastError());
}

extern "C" int tgdn_glue_fwd(const void* x, const void* weight, const int32_t* cu_seqlens, int n_docs, int B, int T, int C,
                             int64_t stride_b, int64_t stride_t, int H, int E, float eps, void* q, void* k, void* v, float* k2,
                             float* q2, void* stream) {
  return glue_launch<false>(x, weight, cu_seqlens, n_docs, B, T, C, stride_b, stride_t, H, E, eps, q, k, v, k2, q2, nullptr,
                            static_cast<cudaStream_t>(stream));
}

extern "C" int tgdn_glue_bwd_norm(const void* x, const void* weight, const int32_t* cu_seqlens, int n_docs, int B, int T, int C,
                                  int64_t stride_b, int64_t stride_t, int H, int E, float eps, const void* dq, const void* dk,
                                  const void* dv, const float* dk2, const float* dq2, void* dy, void* stream) {
  return glue_launch<true>(x, weight, cu_seqlens, n_docs, B, T, C, stride_b, stride_t, H, E, eps, const_cast<void*>(dq),
                           const_cast<void*>(dk), const_cast<void*>(dv), const_cast<float*>(dk2), const_cast<float*>(dq2), dy,
                           static_cast<cudaStream_t>(stream));
}
