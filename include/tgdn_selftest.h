/* Self-test entry points of libtgdn_b200: small kernels that exercise one building block each (a tcgen05 product in a
 * given operand layout, a TMA tile load, a wait that runs out).  They are exported by the library for its own test-suite
 * and are not part of the interface an embedder binds; none of them has a counterpart in the reference.
 */
#ifndef TGDN_SELFTEST_H_
#define TGDN_SELFTEST_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* D (128, N) f32 = A (M, K) * B (K, N) with bf16 operands staged in shared memory in the given layouts
 * (0 = 128B-swizzled K-major, 1 = 128B-swizzled MN-major, 2 = plain K-major, 3 = plain MN-major).
 * No counterpart in the reference. */
int tgdn_selftest_mma(const void* A, const void* B, void* D, int M, int N, int K, int layout_a, int layout_b, void* stream);
/* Returns the shared-memory image (8192 bytes) of one 64x64 128B-swizzled tile load of a (B,T,H,128) bf16 tensor at
 * (batch, tok0, head, col0), followed by bulk_bytes copied by a 1-D bulk copy.  No counterpart in the reference. */
int tgdn_selftest_tma(const void* x, int B, int T, int H, int col0, int head, int tok0, int batch, const void* bulk_src,
                      int bulk_bytes, void* out, void* stream);

/* Launches one CTA that waits, for at most limit_cycles SM clocks (1 .. 2^28), on a barrier nothing arrives at.  out3
 * (device, 3 ints) receives: [0] 1 if the wait was satisfied (never), 0 if it gave up; [1] the CTA's abort flag;
 * [2] the clocks the wait took.  The device status word then reads 1 (a load barrier timed out) until it is read.
 * No counterpart in the reference (its waits are unbounded: cute_triadic_gdn/kernels/sm100_tc.py:116-119). */
int tgdn_selftest_wait(long long limit_cycles, int* out3, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TGDN_SELFTEST_H_ */
