// Width-4 causal depthwise convolution with SiLU on the leading channels: forward and backward.
//
// Replaces the reference's Triton kernels cute_triadic_gdn/ops/conv_split_act.py:20-55 (_fwd_kernel) and :58-107
// (_bwd_kernel).  HBM-bound: every thread owns 8 adjacent channels (one 16-byte vector) and walks a run of
// consecutive tokens with the 4-tap window held in registers, so x is read once, y written once.  The backward
// recomputes the bf16-rounded pre-activation from the same window (the reference launches a second forward for it),
// reads x and dy once, writes dx once, and leaves one f32 weight-gradient partial per token tile in scratch memory; a
// second small kernel sums the partials in a fixed order.
#include <mutex>

#include "tgdn_common.cuh"
#include "tgdn_host.h"

namespace tgdn {

constexpr int CONV_W = 4;
constexpr int CONV_THREADS = 128;
constexpr int CONV_FWD_TOKENS = 32;    // tokens per thread in the forward
constexpr int CONV_BWD_TOKENS = 256;   // tokens per thread (= per weight-gradient partial) in the backward

struct Vec8 {
  float v[8];
};

__device__ __forceinline__ Vec8 load8(const __nv_bfloat16* p) {
  uint4 u = __ldg(reinterpret_cast<const uint4*>(p));
  Vec8 r;
  r.v[0] = bf16_lo(u.x); r.v[1] = bf16_hi(u.x); r.v[2] = bf16_lo(u.y); r.v[3] = bf16_hi(u.y);
  r.v[4] = bf16_lo(u.z); r.v[5] = bf16_hi(u.z); r.v[6] = bf16_lo(u.w); r.v[7] = bf16_hi(u.w);
  return r;
}
__device__ __forceinline__ Vec8 zero8() {
  Vec8 r;
#pragma unroll
  for (int i = 0; i < 8; ++i) r.v[i] = 0.f;
  return r;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const Vec8& a) {
  uint4 u;
  u.x = pack_bf16(a.v[0], a.v[1]); u.y = pack_bf16(a.v[2], a.v[3]);
  u.z = pack_bf16(a.v[4], a.v[5]); u.w = pack_bf16(a.v[6], a.v[7]);
  *reinterpret_cast<uint4*>(p) = u;
}
__device__ __forceinline__ float silu(float y) { return y / (1.f + __expf(-y)); }
__device__ __forceinline__ float silu_grad(float y) {
  float s = 1.f / (1.f + __expf(-y));
  return s * (1.f + y * (1.f - s));
}

// Index of the document that holds token t: largest d with cu[d] <= t.
__device__ __forceinline__ int find_doc(const int32_t* cu, int n_docs, int t) {
  int lo = 0, hi = n_docs - 1;
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (__ldg(cu + mid) <= t) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// Walks document boundaries as the token index grows.
struct DocCursor {
  const int32_t* cu;
  int n_docs, d, start, next;
  __device__ __forceinline__ void init(const int32_t* cu_, int n_docs_, int t, int T) {
    cu = cu_; n_docs = n_docs_;
    if (cu == nullptr) { d = 0; start = 0; next = T; return; }
    d = find_doc(cu, n_docs, t);
    start = __ldg(cu + d);
    next = __ldg(cu + d + 1);
  }
  __device__ __forceinline__ void advance(int t) {      // call with increasing t
    while (cu != nullptr && t >= next && d + 1 < n_docs) {
      ++d; start = next; next = __ldg(cu + d + 1);
    }
  }
};

__global__ void __launch_bounds__(CONV_THREADS)
conv_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ weight,
                __nv_bfloat16* __restrict__ y, const int32_t* __restrict__ cu, int n_docs, int T, int C,
                int64_t stride_b, int64_t stride_t, int act_channels) {
  const int c0 = (blockIdx.x * CONV_THREADS + threadIdx.x) * 8;
  if (c0 >= C) return;
  const int t0 = blockIdx.y * CONV_FWD_TOKENS;
  const int t1 = min(T, t0 + CONV_FWD_TOKENS);
  const __nv_bfloat16* xb = x + static_cast<int64_t>(blockIdx.z) * stride_b + c0;
  __nv_bfloat16* yb = y + (static_cast<int64_t>(blockIdx.z) * T) * C + c0;

  float w[8][CONV_W];
  {
    const uint4* wp = reinterpret_cast<const uint4*>(weight + static_cast<int64_t>(c0) * CONV_W);
#pragma unroll
    for (int i = 0; i < 4; ++i) {              // 8 channels x 4 taps = 32 bf16 = 4 vectors
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
  DocCursor doc;
  doc.init(cu, n_docs, t0, T);
  Vec8 xm1 = zero8(), xm2 = zero8(), xm3 = zero8();
  if (t0 - 1 >= doc.start) xm1 = load8(xb + static_cast<int64_t>(t0 - 1) * stride_t);
  if (t0 - 2 >= doc.start) xm2 = load8(xb + static_cast<int64_t>(t0 - 2) * stride_t);
  if (t0 - 3 >= doc.start) xm3 = load8(xb + static_cast<int64_t>(t0 - 3) * stride_t);

  for (int tb = t0; tb < t1; tb += 8) {
    Vec8 xs[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      xs[i] = (tb + i < t1) ? load8(xb + static_cast<int64_t>(tb + i) * stride_t) : zero8();
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int t = tb + i;
      if (t >= t1) break;
      doc.advance(t);
      if (t == doc.start) { xm1 = zero8(); xm2 = zero8(); xm3 = zero8(); }
      Vec8 out;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        float acc = xm3.v[c] * w[c][0];
        acc = fmaf(xm2.v[c], w[c][1], acc);
        acc = fmaf(xm1.v[c], w[c][2], acc);
        acc = fmaf(xs[i].v[c], w[c][3], acc);
        out.v[c] = (c0 + c < act_channels) ? silu(acc) : acc;
      }
      store8(yb + static_cast<int64_t>(t) * C, out);
      xm3 = xm2; xm2 = xm1; xm1 = xs[i];
    }
  }
}

__global__ void __launch_bounds__(CONV_THREADS)
conv_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ weight,
                const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_partial,
                const int32_t* __restrict__ cu, int n_docs, int T, int C, int64_t stride_b, int64_t stride_t,
                int64_t dy_stride_b, int64_t dy_stride_t, int act_channels) {
  const int c0 = (blockIdx.x * CONV_THREADS + threadIdx.x) * 8;
  if (c0 >= C) return;
  const int t0 = blockIdx.y * CONV_BWD_TOKENS;
  const int t1 = min(T, t0 + CONV_BWD_TOKENS);
  const __nv_bfloat16* xb = x + static_cast<int64_t>(blockIdx.z) * stride_b + c0;
  const __nv_bfloat16* dyb = dy + static_cast<int64_t>(blockIdx.z) * dy_stride_b + c0;
  __nv_bfloat16* dxb = dx + (static_cast<int64_t>(blockIdx.z) * T) * C + c0;

  float w[8][CONV_W];
  {
    const uint4* wp = reinterpret_cast<const uint4*>(weight + static_cast<int64_t>(c0) * CONV_W);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
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
  float dwa[8][CONV_W];
#pragma unroll
  for (int c = 0; c < 8; ++c)
#pragma unroll
    for (int j = 0; j < CONV_W; ++j) dwa[c][j] = 0.f;

  DocCursor doc;
  doc.init(cu, n_docs, t0, T);
  // x window: xw[j] = x[t - j] while token t is processed (xw[0] is loaded in the loop)
  Vec8 xw1 = zero8(), xw2 = zero8(), xw3 = zero8();
  if (t0 - 1 >= doc.start) xw1 = load8(xb + static_cast<int64_t>(t0 - 1) * stride_t);
  if (t0 - 2 >= doc.start) xw2 = load8(xb + static_cast<int64_t>(t0 - 2) * stride_t);
  if (t0 - 3 >= doc.start) xw3 = load8(xb + static_cast<int64_t>(t0 - 3) * stride_t);
  // dy' of the last four tokens (gw0 = token t ... gw3 = token t-3) and the document start of each
  Vec8 gw1 = zero8(), gw2 = zero8(), gw3 = zero8();
  int ds1 = 0x7fffffff, ds2 = 0x7fffffff;

  // dx[u] = sum_j dy'[u+j] * w[3-j] over tokens u+j of the same document: token u is complete once t = u+3 is seen,
  // so the loop runs three tokens past the tile (dy' = 0 past the end of the row).
  for (int t = t0; t < t1 + CONV_W - 1; ++t) {
    Vec8 gy = zero8();
    Vec8 x0 = zero8();
    int ds0 = 0x7fffffff;
    if (t < T) {
      doc.advance(t);
      ds0 = doc.start;
      if (t == doc.start) { xw1 = zero8(); xw2 = zero8(); xw3 = zero8(); }
      x0 = load8(xb + static_cast<int64_t>(t) * stride_t);
      const Vec8 g = load8(dyb + static_cast<int64_t>(t) * dy_stride_t);
#pragma unroll
      for (int c = 0; c < 8; ++c) {                // dy'[t] = dy[t] * silu'(bf16(pre-activation[t]))
        float gv = g.v[c];
        if (c0 + c < act_channels) {
          float pre = xw3.v[c] * w[c][0];
          pre = fmaf(xw2.v[c], w[c][1], pre);
          pre = fmaf(xw1.v[c], w[c][2], pre);
          pre = fmaf(x0.v[c], w[c][3], pre);
          gv *= silu_grad(round_bf16(pre));
        }
        gy.v[c] = gv;
      }
      if (t < t1) {                                // the weight gradient of token t belongs to this tile
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          dwa[c][0] = fmaf(gy.v[c], xw3.v[c], dwa[c][0]);
          dwa[c][1] = fmaf(gy.v[c], xw2.v[c], dwa[c][1]);
          dwa[c][2] = fmaf(gy.v[c], xw1.v[c], dwa[c][2]);
          dwa[c][3] = fmaf(gy.v[c], x0.v[c], dwa[c][3]);
        }
      }
    }
    const int u = t - 3;
    if (u >= t0) {
      const float m2 = (ds2 <= u) ? 1.f : 0.f, m1 = (ds1 <= u) ? 1.f : 0.f, m0 = (ds0 <= u) ? 1.f : 0.f;
      Vec8 out;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        float acc = gw3.v[c] * w[c][3];
        acc = fmaf(m2 * gw2.v[c], w[c][2], acc);
        acc = fmaf(m1 * gw1.v[c], w[c][1], acc);
        acc = fmaf(m0 * gy.v[c], w[c][0], acc);
        out.v[c] = acc;
      }
      store8(dxb + static_cast<int64_t>(u) * C, out);
    }
    gw3 = gw2; gw2 = gw1; gw1 = gy;
    ds2 = ds1; ds1 = ds0;
    xw3 = xw2; xw2 = xw1; xw1 = x0;
  }
  float* out = dw_partial + (static_cast<int64_t>(blockIdx.z) * gridDim.y + blockIdx.y) * (static_cast<int64_t>(C) * CONV_W) +
               static_cast<int64_t>(c0) * CONV_W;
#pragma unroll
  for (int c = 0; c < 8; ++c)
    *reinterpret_cast<float4*>(out + c * CONV_W) = make_float4(dwa[c][0], dwa[c][1], dwa[c][2], dwa[c][3]);
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
  if ((stride_b % 8) || (stride_t % 8)) return TGDN_ERR_ALIGN;
  return 0;
}

extern "C" int tgdn_conv_fwd(const void* x, const void* weight, void* y, const int32_t* cu_seqlens, int n_docs, int B,
                             int T, int C, int64_t stride_b, int64_t stride_t, int act_channels, void* stream) {
  int rc = conv_check(x, weight, y, cu_seqlens, n_docs, B, T, C, stride_b, stride_t);
  if (rc) return rc;
  dim3 grid((C / 8 + CONV_THREADS - 1) / CONV_THREADS, (T + CONV_FWD_TOKENS - 1) / CONV_FWD_TOKENS, B);
  conv_fwd_kernel<<<grid, CONV_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(weight), static_cast<__nv_bfloat16*>(y),
      cu_seqlens, n_docs, T, C, stride_b, stride_t, act_channels);
  return tgdn_cuda_error(cudaGetLastError());
}

extern "C" int64_t tgdn_conv_bwd_scratch_bytes(int B, int T, int C) {
  if (B <= 0 || T <= 0 || C <= 0) return 0;
  const int64_t tiles = (T + CONV_BWD_TOKENS - 1) / CONV_BWD_TOKENS;
  return static_cast<int64_t>(B) * tiles * C * CONV_W * static_cast<int64_t>(sizeof(float));
}

extern "C" int tgdn_conv_bwd(const void* x, const void* weight, const void* dy, void* dx, void* dw,
                             const int32_t* cu_seqlens, int n_docs, int B, int T, int C, int64_t stride_b,
                             int64_t stride_t, int64_t dy_stride_b, int64_t dy_stride_t, int act_channels, void* scratch,
                             int64_t scratch_bytes, void* stream) {
  int rc = conv_check(x, weight, dx, cu_seqlens, n_docs, B, T, C, stride_b, stride_t);
  if (rc) return rc;
  if (!dy || !dw) return TGDN_ERR_NULL;
  if ((reinterpret_cast<uintptr_t>(dy) & 15) || (dy_stride_b % 8) || (dy_stride_t % 8)) return TGDN_ERR_ALIGN;
  if (!scratch || scratch_bytes < tgdn_conv_bwd_scratch_bytes(B, T, C) || (reinterpret_cast<uintptr_t>(scratch) & 15))
    return TGDN_ERR_SCRATCH;
  const int tiles = (T + CONV_BWD_TOKENS - 1) / CONV_BWD_TOKENS;
  dim3 grid((C / 8 + CONV_THREADS - 1) / CONV_THREADS, tiles, B);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  conv_bwd_kernel<<<grid, CONV_THREADS, 0, s>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(weight),
      static_cast<const __nv_bfloat16*>(dy), static_cast<__nv_bfloat16*>(dx), static_cast<float*>(scratch), cu_seqlens,
      n_docs, T, C, stride_b, stride_t, dy_stride_b, dy_stride_t, act_channels);
  rc = tgdn_cuda_error(cudaGetLastError());
  if (rc) return rc;
  const int n_elem = C * CONV_W;
  conv_dw_reduce_kernel<<<(n_elem + 255) / 256, 256, 0, s>>>(static_cast<const float*>(scratch),
                                                             static_cast<__nv_bfloat16*>(dw), B * tiles, n_elem);
  return tgdn_cuda_error(cudaGetLastError());
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
  if ((reinterpret_cast<uintptr_t>(dy) & 15) || (dy_stride_b % 8) || (dy_stride_t % 8)) return TGDN_ERR_ALIGN;
  if (tgdn_conv_bwd_scratch_bytes(B, T, C) > static_cast<int64_t>(TGDN_CONV_STATIC_SCRATCH_BYTES)) return TGDN_ERR_STATIC_LIMIT;
  float* scratch = nullptr;
  if ((rc = conv_static_scratch(&scratch))) return rc;
  const int tiles = (T + CONV_BWD_TOKENS - 1) / CONV_BWD_TOKENS;
  dim3 grid((C / 8 + CONV_THREADS - 1) / CONV_THREADS, tiles, B);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  conv_bwd_kernel<<<grid, CONV_THREADS, 0, s>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(weight),
      static_cast<const __nv_bfloat16*>(dy), static_cast<__nv_bfloat16*>(dx), scratch, cu_seqlens, n_docs, T, C, stride_b,
      stride_t, dy_stride_b, dy_stride_t, act_channels);
  rc = tgdn_cuda_error(cudaGetLastError());
  if (rc) return rc;
  const int n_elem = C * CONV_W;
  conv_dw_reduce_kernel<<<(n_elem + 255) / 256, 256, 0, s>>>(scratch, static_cast<__nv_bfloat16*>(dw), B * tiles, n_elem);
  return tgdn_cuda_error(cudaGetLastError());
}
