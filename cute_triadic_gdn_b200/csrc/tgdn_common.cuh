// Device-side building blocks shared by the Triadic GDN kernels (sm_100a only):
// mbarrier / TMA / tcgen05 wrappers in inline PTX, shared-memory operand layouts and their matrix descriptors.
//
// Reference counterpart: cute_triadic_gdn/kernels/sm100_tc.py:1-166 (the reference emits the same PTX
// instructions from its Python DSL); this file is an independent CUDA C++ formulation.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tgdn {

constexpr int CHUNK = 64;     // tokens per chunk
constexpr int HEAD = 128;     // key and value head dimension

// Device status word values (first failure wins).  A kernel that gives up on a wait records one of these and
// runs to its end without waiting again, so the launch always terminates and the context stays usable.
enum DeviceStatus : int {
  DEV_OK = 0,
  DEV_TIMEOUT_LOAD = 1,    // a TMA / bulk-copy transaction barrier did not complete in time
  DEV_TIMEOUT_MMA = 2,     // a tcgen05.commit barrier did not complete in time
  DEV_BAD_CHUNK_MAP = 3,   // a chunk-map entry pointed outside the token range
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ------------------------------------------------------------------------------------------------
// mbarrier
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.b32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Non-blocking probe: unlike try_wait it never parks the warp, so a spinning waiter sees the flip within a few cycles.
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.b32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Shared per-CTA control block of a kernel with bounded waits.
struct WaitCtl {
  volatile int* abort;   // shared-memory flag: once set, every wait of the CTA returns at once
  int* status;           // global status word
};

constexpr long long WAIT_LIMIT_CYCLES = 1ll << 31;   // about a second of SM clocks

// Wait for `parity` of `bar`; gives up after WAIT_LIMIT_CYCLES, records `code` and raises the CTA's abort flag.
// Spins on the non-parking probe: the parking form (try_wait) was measured to wake a waiter up to a microsecond after
// the barrier flipped, which is as long as a whole pipeline phase here.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const WaitCtl& ctl, int code,
                                          long long limit_cycles = WAIT_LIMIT_CYCLES) {
#pragma unroll 1
  for (int it = 0; it < 2048; ++it)
    if (mbar_test_wait(bar, parity)) return true;
  const long long start = clock64();
  for (uint32_t it = 1;; ++it) {
    if (mbar_test_wait(bar, parity)) return true;
    if ((it & 63u) == 0u) {
      if (*ctl.abort) return false;
      if (clock64() - start > limit_cycles) {
        *ctl.abort = 1;
        atomicCAS(ctl.status, DEV_OK, code);
        return false;
      }
    }
  }
}
__device__ __forceinline__ bool mbar_wait_spin(uint64_t* bar, uint32_t parity, const WaitCtl& ctl, int code) {
  return mbar_wait(bar, parity, ctl, code);
}

// ------------------------------------------------------------------------------------------------
// TMA (tensor-map tiles and plain bulk copies), completion on an mbarrier.  No multicast anywhere.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2,
                                            int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// Tile store shared -> global (bulk async-group completion).  The issuing thread commits the group and, before the
// shared-memory source may be overwritten, waits until the group's reads of shared memory are done.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, const void* src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               ::"l"(map), "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_group_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_group() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void tma_prefetch_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
// 1-D bulk copy global -> shared; both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// Hints that pull a tile / a byte range into L2 ahead of the real load (no shared memory, no completion to wait for).
__device__ __forceinline__ void tma_prefetch_4d(const CUtensorMap* map, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];"
               ::"l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void bulk_prefetch(const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
// Generic-proxy writes to shared memory -> visible to the async proxy (tcgen05.mma operands, bulk stores).
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ------------------------------------------------------------------------------------------------
// tcgen05: tensor memory, MMA, commit, loads
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {   // one whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {     // one whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc]; bf16 operands, f32 accumulator; issued by ONE thread.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive once on `bar` when every tcgen05.mma issued so far by this thread has completed.
// One lane of a fully active warp.  Tensor-core and TMA instructions are issued as "warp-uniform branch, then elected
// lane": their operands then stay warp-uniform values, which a branch on the thread index would not allow.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n.reg .pred p;\nelect.sync _|p, 0xffffffff;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// tcgen05.ld 32x32b: lane L of the warp reads row (lane base + L); N consecutive f32 columns.  The lane base in
// `taddr` must be 32 * (warp index % 4).
__device__ __forceinline__ void tmem_ld4(uint32_t taddr, float* v) {
  uint32_t r[4];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr) : "memory");
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float* v) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr) : "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
// N columns (multiple of 4) starting at taddr, in the widest pieces available; the caller waits with tmem_wait_ld().
template <int N>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, float* v) {
  static_assert(N % 4 == 0, "column count must be a multiple of 4");
  int done = 0;
#pragma unroll
  for (; done + 16 <= N; done += 16) tmem_ld16(taddr + done, v + done);
  if (N - done >= 8) { tmem_ld8(taddr + done, v + done); done += 8; }
  if (N - done >= 4) { tmem_ld4(taddr + done, v + done); }
}

// ------------------------------------------------------------------------------------------------
// Shared-memory operand layouts (bf16) and descriptors
//
// (1) SW128 tile: rows of 64 elements (128 bytes), 16-byte pieces XOR-swizzled with (row % 8); what a TMA tile load with
//     128-byte swizzle writes.  The tile base must be 1024-byte aligned.  Wider matrices are several such 64-column
//     blocks.  Read as K-major when the 64-element rows run along K, as MN-major when they run along M or N.
// (2) Plain image: 8x8 core matrices of 128 contiguous bytes; element (i, j) with j the direction that is contiguous
//     inside a 16-byte piece:  off = (i/8)*SI + (j/8)*SJ + (i%8)*16 + (j%8)*2.
//     K-major use (j = K):  SBO = SI, LBO = SJ.   MN-major use (j = M or N, i = K):  SBO = SJ, LBO = SI.
// ------------------------------------------------------------------------------------------------
__host__ __device__ __forceinline__ uint32_t sw128_off(uint32_t row, uint32_t col /* 0..63 */) {
  return row * 128u + ((((col >> 3) ^ row) & 7u) << 4) + ((col & 7u) << 1);
}
__host__ __device__ __forceinline__ uint32_t img_off(uint32_t i, uint32_t j, uint32_t SI, uint32_t SJ) {
  return (i >> 3) * SI + (j >> 3) * SJ + ((i & 7u) << 4) + ((j & 7u) << 1);
}

constexpr uint32_t LAYOUT_PLAIN = 0;
constexpr uint32_t LAYOUT_SW128 = 2;

__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
  uint64_t d = static_cast<uint64_t>((saddr >> 4) & 0x3FFFu);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;                                   // descriptor version of this architecture
  d |= static_cast<uint64_t>(layout) << 61;
  return d;
}
__device__ __forceinline__ uint64_t desc_advance(uint64_t d, uint32_t bytes) { return d + (bytes >> 4); }

// kind::f16 instruction descriptor: bf16 A and B, f32 D.  major: 0 = K-major, 1 = MN-major.
__host__ __device__ constexpr uint32_t make_idesc(int M, int N, int a_major, int b_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(a_major) << 15) |
         (static_cast<uint32_t>(b_major) << 16) | (static_cast<uint32_t>(N >> 3) << 17) |
         (static_cast<uint32_t>(M >> 4) << 24);
}

// Issue `ksteps` MMAs of K=16 each; operand descriptors advance by a_step / b_step bytes per step.
__device__ __forceinline__ void umma_ksteps(uint32_t d_tmem, uint64_t adesc, uint32_t a_step, uint64_t bdesc,
                                            uint32_t b_step, uint32_t idesc, int ksteps, bool accumulate) {
  for (int k = 0; k < ksteps; ++k)
    umma_bf16(d_tmem, desc_advance(adesc, k * a_step), desc_advance(bdesc, k * b_step), idesc,
              (accumulate || k > 0) ? 1u : 0u);
}

// ------------------------------------------------------------------------------------------------
// small helpers
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);    // .x (low half, lower address) = lo
  return *reinterpret_cast<uint32_t*>(&p);
}
// Two bf16 products at once, each rounded to nearest: scaling a packed row by a packed factor costs one instruction per
// pair where unpacking, two f32 multiplies and a repack cost five.
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ void st_shared_v4(uint32_t saddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(saddr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void st_shared_v2(uint32_t saddr, uint32_t a, uint32_t b) {
  asm volatile("st.shared.v2.b32 [%0], {%1,%2};" ::"r"(saddr), "r"(a), "r"(b) : "memory");
}

// Global loads that stay where they are written.  A plain read-only load may be sunk by the compiler to its first use,
// which turns a prefetch issued one loop iteration ahead back into an exposed memory round trip; volatile asm keeps its
// program order relative to the barrier and tensor-core instructions around it.
__device__ __forceinline__ float ldg_pinned_f32(const float* p) {
  float v;
  asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ldg_pinned_v2(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.v2.b32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ldg_pinned_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

}  // namespace tgdn
