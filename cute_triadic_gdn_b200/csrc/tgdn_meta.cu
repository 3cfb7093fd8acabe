// Packed-document metadata: chunk offsets per document, the chunk map and the longest-first document order.
//
// Replaces cute_triadic_gdn/kernels/sm90_joint_packed.py:64-129 (metadata_kernel, joint_metadata) and
// cute_triadic_gdn/ops/joint_packing.py:16-20 (chunk_capacity).  Same outputs; the prefix sums are block reductions
// instead of a per-document serial loop, and the unused tail of the chunk map is filled (start = T, rows = 0) so
// that a kernel that walks the whole capacity sees empty chunks instead of uninitialised memory.
#include "tgdn_common.cuh"
#include "tgdn_host.h"

namespace tgdn {

constexpr int META_THREADS = 256;

__device__ __forceinline__ long long cu_at(const void* cu, int is64, int i) {
  return is64 ? static_cast<const long long*>(cu)[i] : static_cast<long long>(static_cast<const int*>(cu)[i]);
}
__device__ __forceinline__ bool pair_ok(const void* cu, int is64, int i, int T) {
  const long long a = cu_at(cu, is64, i), b = cu_at(cu, is64, i + 1);
  return a >= 0 && b <= T && b > a;
}
__device__ __forceinline__ int chunks_of(const void* cu, int is64, int i) {
  return static_cast<int>((cu_at(cu, is64, i + 1) - cu_at(cu, is64, i) + 63) / 64);
}

template <typename T>
__device__ __forceinline__ T block_sum(T v, T* scratch) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  T total = 0;
  for (int w = 0; w < META_THREADS / 32; ++w) total += scratch[w];
  return total;
}

// One block per document.
__global__ void __launch_bounds__(META_THREADS)
metadata_kernel(const void* __restrict__ cu, int is64, int n_docs, int T, int32_t* __restrict__ offsets,
                int32_t* __restrict__ mapping, int capacity, uint8_t* __restrict__ valid) {
  __shared__ long long s_first[META_THREADS / 32];
  __shared__ int s_bad[META_THREADS / 32];
  __shared__ int s_rank[META_THREADS / 32];
  const int doc = blockIdx.x, tid = threadIdx.x;

  // first chunk of this document and validity of every pair up to and including it
  long long part = 0;
  int bad = 0;
  for (int i = tid; i < doc; i += META_THREADS) {
    if (!pair_ok(cu, is64, i, T)) bad = 1; else part += chunks_of(cu, is64, i);
  }
  const long long first = block_sum<long long>(part, s_first);
  bad = block_sum<int>(bad, s_bad);
  const bool own_ok = pair_ok(cu, is64, doc, T);
  const int count = own_ok ? chunks_of(cu, is64, doc) : 0;
  const bool safe = own_ok && bad == 0 && first + count <= capacity;

  // rank among the documents, longest first, ties in document order
  int rank = 0;
  for (int i = tid; i < n_docs; i += META_THREADS) {
    const int other = pair_ok(cu, is64, i, T) ? chunks_of(cu, is64, i) : 0;
    if (other > count || (other == count && i < doc)) ++rank;
  }
  rank = block_sum<int>(rank, s_rank);

  if (tid == 0) {
    offsets[doc] = safe ? static_cast<int32_t>(first) : 0;
    if (doc == n_docs - 1) offsets[n_docs] = safe ? static_cast<int32_t>(first + count) : 0;
    mapping[2 * capacity + rank] = doc;         // rank is a permutation of 0..n_docs-1 whatever the offsets are
  }
  if (safe) {
    const int start = static_cast<int>(cu_at(cu, is64, doc)), end = static_cast<int>(cu_at(cu, is64, doc + 1));
    for (int s = tid; s < count; s += META_THREADS) {
      mapping[first + s] = start + s * 64;
      mapping[capacity + first + s] = min(64, end - start - s * 64);
    }
    if (doc == n_docs - 1) {                    // empty tail of the map
      for (int s = static_cast<int>(first) + count + tid; s < capacity; s += META_THREADS) {
        mapping[s] = T;
        mapping[capacity + s] = 0;
      }
    }
  }
  if (doc == n_docs - 1) {
    // the last block has looked at every pair: it owns the verdict
    const bool ends_ok = cu_at(cu, is64, 0) == 0 && cu_at(cu, is64, n_docs) == T;
    if (tid == 0) valid[0] = (safe && ends_ok) ? 1 : 0;
    for (int s = n_docs + tid; s < capacity; s += META_THREADS) mapping[2 * capacity + s] = -1;
  }
}

}  // namespace tgdn

using namespace tgdn;

extern "C" int tgdn_chunk_capacity(int T, int n_docs) {
  if (T <= 0 || n_docs <= 0) return 0;
  const long long exact = (static_cast<long long>(T) + 63) / 64 + n_docs - 1;
  return static_cast<int>((exact + 15) / 16 * 16);
}

extern "C" int tgdn_metadata(const void* cu_seqlens, int cu_is_int64, int n_docs, int T, int32_t* offsets,
                             int32_t* mapping, int capacity, uint8_t* valid, void* stream) {
  if (!cu_seqlens || !offsets || !mapping || !valid) return TGDN_ERR_NULL;
  if (n_docs < 1 || T < 1 || capacity < tgdn_chunk_capacity(T, n_docs)) return TGDN_ERR_SHAPE;
  metadata_kernel<<<n_docs, META_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(cu_seqlens, cu_is_int64, n_docs, T,
                                                                                 offsets, mapping, capacity, valid);
  return tgdn_cuda_error(cudaGetLastError());
}
