// One-token step of the Triadic GDN recurrence on a resident state: the decode path of inference.
//
// Per (batch row b, head h), with S_e the E state slices (128 key rows x 128 value columns, f32) and the token's
// q, k, v (bf16), k2, q2, g (f32, E each), beta:
//   S_e  <- exp(g_e) S_e
//   pred  = sum_e k2_e (k^T S_e)                                  (128 value columns)
//   S_e  <- S_e + beta k2_e k (v - pred)^T
//   o     = scale sum_e q2_e (q^T S_e)
// which is the token-by-token definition the chunk kernels reproduce (cute_triadic_gdn/ops/gdn_joint.py:45-90 with a chunk
// of one token: A = 1, Pm = scale <q,k> sum_e q2_e k2_e).  The reference has no decode entry; this one continues from
// the state that tgdn_fwd_state hands out.
//
// The step is a stream over the state: 2 x E x 64 KB per (b, h), everything else is noise.  One CTA of 256 threads owns
// a block of VB value columns of one (b, h): it reads its E x 128 x VB state values once into registers (16-byte loads,
// whole 32-byte sectors), forms the two contractions over the key axis from them (warp shuffles, then a fixed-order sum
// over the warps in shared memory), and writes the updated values back from the same registers.
#include "tgdn_common.cuh"
#include "tgdn_host.h"
#include "tgdn_kernels.h"

namespace tgdn {

constexpr int DEC_THREADS = 256;

template <int E>
struct DecCfg {
  static constexpr int VB = E <= 8 ? 16 : 8;                   // value columns per CTA
  static constexpr int TPR = VB / 4;                           // threads per key row (a thread holds 4 columns)
  static constexpr int ROWS = DEC_THREADS / TPR;               // key rows per pass
  static constexpr int PASSES = 128 / ROWS;
  static constexpr int NV = HEAD / VB;
  static_assert(E * PASSES * 4 <= 64, "state values per thread");
};

struct DecParams {
  const __nv_bfloat16* q;     // (B, H, 128)
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  const float* k2;            // (B, H, E)
  const float* q2;
  const float* g;
  const float* beta;          // (B, H)
  float* state;               // (B, H, E, 128, 128), updated in place
  __nv_bfloat16* o;           // (B, H, 128)
  int B, H;
  float scale;
};

template <int E>
__global__ void __launch_bounds__(DEC_THREADS)
decode_kernel(DecParams p) {
  using C = DecCfg<E>;
  constexpr int VB = C::VB, TPR = C::TPR, ROWS = C::ROWS, PASSES = C::PASSES;
  __shared__ float red[2][DEC_THREADS / 32][VB];               // per warp: partial pred and partial readout
  __shared__ __align__(16) float delta[VB];
  __shared__ float kq[2][HEAD];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int vb = blockIdx.x % C::NV;
  const int64_t bh = blockIdx.x / C::NV;
  const int c4 = (tid % TPR) * 4;                              // this thread's 4 columns inside the block
  const int r0 = tid / TPR;                                    // its key row in pass 0
  float* sbase = p.state + bh * (static_cast<int64_t>(E) * HEAD * HEAD) + vb * VB + c4;

  // the state first: these loads are the kernel
  float4 S[E][PASSES];
#pragma unroll
  for (int e = 0; e < E; ++e)
#pragma unroll
    for (int ps = 0; ps < PASSES; ++ps)
      S[e][ps] = *reinterpret_cast<const float4*>(sbase + (static_cast<int64_t>(e) * HEAD + ps * ROWS + r0) * HEAD);
  if (tid < HEAD) {
    kq[0][tid] = __bfloat162float(p.k[bh * HEAD + tid]);
    kq[1][tid] = __bfloat162float(p.q[bh * HEAD + tid]);
  }
  float dec[E], k2v[E], q2v[E];
  float mix = 0.f;                                             // sum_e q2_e k2_e
#pragma unroll
  for (int e = 0; e < E; ++e) {
    dec[e] = __expf(__ldg(p.g + bh * E + e));
    k2v[e] = __ldg(p.k2 + bh * E + e);
    q2v[e] = __ldg(p.q2 + bh * E + e);
    mix = fmaf(q2v[e], k2v[e], mix);
  }
  const float beta = __ldg(p.beta + bh);
  __syncthreads();

  // contractions over the key axis on the decayed state: pk = sum_e k2_e d_e k^T S_e, pq = sum_e q2_e d_e q^T S_e
  float pk[4] = {0.f, 0.f, 0.f, 0.f}, pq[4] = {0.f, 0.f, 0.f, 0.f};
  float qk_part = 0.f;
#pragma unroll
  for (int ps = 0; ps < PASSES; ++ps) {
    const float kd = kq[0][ps * ROWS + r0], qd = kq[1][ps * ROWS + r0];
    if (tid % TPR == 0) qk_part = fmaf(kd, qd, qk_part);
#pragma unroll
    for (int e = 0; e < E; ++e) {
      const float wk = k2v[e] * dec[e] * kd, wq = q2v[e] * dec[e] * qd;
      pk[0] = fmaf(wk, S[e][ps].x, pk[0]); pk[1] = fmaf(wk, S[e][ps].y, pk[1]);
      pk[2] = fmaf(wk, S[e][ps].z, pk[2]); pk[3] = fmaf(wk, S[e][ps].w, pk[3]);
      pq[0] = fmaf(wq, S[e][ps].x, pq[0]); pq[1] = fmaf(wq, S[e][ps].y, pq[1]);
      pq[2] = fmaf(wq, S[e][ps].z, pq[2]); pq[3] = fmaf(wq, S[e][ps].w, pq[3]);
    }
  }
  // over the rows of a warp (lanes with the same column group), then over the warps in index order
#pragma unroll
  for (int o = TPR; o < 32; o <<= 1) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      pk[c] += __shfl_xor_sync(0xffffffffu, pk[c], o);
      pq[c] += __shfl_xor_sync(0xffffffffu, pq[c], o);
    }
    qk_part += __shfl_xor_sync(0xffffffffu, qk_part, o);
  }
  __shared__ float qk_w[DEC_THREADS / 32];
  if (lane < TPR) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      red[0][warp][lane * 4 + c] = pk[c];
      red[1][warp][lane * 4 + c] = pq[c];
    }
  }
  if (lane == 0) qk_w[warp] = qk_part;
  __syncthreads();
  if (tid < VB) {
    float pred = 0.f, read = 0.f, qk = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_THREADS / 32; ++w) {
      pred += red[0][w][tid];
      read += red[1][w][tid];
      qk += qk_w[w];
    }
    const float vv = __bfloat162float(p.v[bh * HEAD + vb * VB + tid]);
    const float d = beta * (vv - pred);
    delta[tid] = d;
    // o from the updated state: the decayed part plus the rank-one update seen through q
    p.o[bh * HEAD + vb * VB + tid] = __float2bfloat16_rn(p.scale * (read + mix * qk * d));
  }
  __syncthreads();
  const float4 dl = *reinterpret_cast<const float4*>(&delta[c4]);
#pragma unroll
  for (int e = 0; e < E; ++e)
#pragma unroll
    for (int ps = 0; ps < PASSES; ++ps) {
      const float w = k2v[e] * kq[0][ps * ROWS + r0];
      float4 s = S[e][ps];
      s.x = fmaf(dec[e], s.x, w * dl.x); s.y = fmaf(dec[e], s.y, w * dl.y);
      s.z = fmaf(dec[e], s.z, w * dl.z); s.w = fmaf(dec[e], s.w, w * dl.w);
      *reinterpret_cast<float4*>(sbase + (static_cast<int64_t>(e) * HEAD + ps * ROWS + r0) * HEAD) = s;
    }
}

}  // namespace tgdn

using namespace tgdn;

template <int E>
static int launch_decode(const DecParams& p, cudaStream_t s) {
  decode_kernel<E><<<p.B * p.H * DecCfg<E>::NV, DEC_THREADS, 0, s>>>(p);
  return tgdn_cuda_error(cudaGetLastError());
}

extern "C" int tgdn_decode_step(const void* q, const void* k, const void* v, const float* k2, const float* q2, const float* g,
                                const float* beta, float scale, int B, int H, int E, float* state, void* o, void* stream) {
  if (!q || !k || !v || !k2 || !q2 || !g || !beta || !state || !o) return TGDN_ERR_NULL;
  if (B <= 0 || H <= 0 || static_cast<long long>(B) * H * 16 > 0x7fffffffLL) return TGDN_ERR_SHAPE;
  if (reinterpret_cast<uintptr_t>(state) & 15) return TGDN_ERR_ALIGN;
  if (!tgdn_check_device()) return TGDN_ERR_DEVICE;
  DecParams p{static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v),
              k2, q2, g, beta, state, static_cast<__nv_bfloat16*>(o), B, H, scale};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (E) {
    case 1: return launch_decode<1>(p, s);
    case 2: return launch_decode<2>(p, s);
    case 4: return launch_decode<4>(p, s);
    case 8: return launch_decode<8>(p, s);
    case 12: return launch_decode<12>(p, s);
    case 16: return launch_decode<16>(p, s);
    default: return TGDN_ERR_SHAPE;
  }
}
