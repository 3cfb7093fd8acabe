// Parameter blocks of the Triadic GDN kernels and the layouts of the tensors that travel between them.
//
// Chunk-layout tensors are indexed by item = (b * NC + n) * H + h (b batch row, n chunk, h head):
//   gc   f32  [item][GATE_ITEM_FLOATS(E)]  the gates of the chunk, five blocks (rows past a document end: a = r = c = 0):
//          [0, 64E)        gc[t][e]  cumulative log gate
//          [64E, 128E)     a[t][e] = k2 exp(gc)                [128E, 192E)   r[t][e] = k2 exp(gL - gc),  gL = gc[63]
//          [192E, 256E)    c[t][e] = scale q2 exp(gc)          [256E, 256E+16)  d[e] = exp(gL), padded to 16 floats
//        The masks kernel forms the factors once; the recurrences fetch [64E, 256E+16) with one bulk copy per chunk.
//   AP   bf16 [item][16 KB image]        [A; Pm A] stacked, image (i = row 0..127, j = column 0..63), SI = 128, SJ = 2048
//   Pm   bf16 [item][ 8 KB image]        image (i = t, j = s), SI = 128, SJ = 1024
//   W, U, dU  bf16 [item][64][128]       row-major token rows of the chunk (rows past a document end are zero)
//   h, ds     bf16 [item][E][16][128][8] state slice e as [value column / 8][key row d][value column % 8]: a plain
//                                        operand image (i = d, j = v) with SI = 16 bytes * 8 = 128, SJ = 2048
// "image" = 8x8 core matrices of 128 contiguous bytes, see tgdn_common.cuh.
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

namespace tgdn {

// dd_e = <h_e, G_e>, the gradient of the chunk decay d_e = exp(gL_e), enters the result only as d_e * dd_e.  Where
// log2(d_e) is below this bound the product is under 2^-24 of <h_e, G_e> and is taken as zero: the reverse recurrence
// then does not store G_e of that chunk and the state-gradient kernel does not read it.  Both kernels evaluate
// gc[63][e] * log2(e) >= DD_MIN_LOG2_DECAY on the same f32 value.
constexpr float DD_MIN_LOG2_DECAY = -24.f;

// Floats per item of the gate tensor, and where its blocks start.
__host__ __device__ constexpr int gate_item_floats(int E) { return 256 * E + 16; }
__host__ __device__ constexpr int gate_factor_bytes(int E) { return (192 * E + 16) * 4; }   // a, r, c, d: one bulk copy

struct MaskParams {
  const float* k2;
  const float* q2;
  const float* g;
  const float* beta;
  float* gc;
  __nv_bfloat16* AP;
  __nv_bfloat16* Pm;
  const int32_t* cmap;      // (3, NC) chunk map of a packed row, or nullptr
  int B, T, H, NC;
  float scale;
  int* status;
};

struct FwdParams {
  const __nv_bfloat16* v;   // token layout
  const float* k2;
  const float* q2;
  const float* beta;
  const float* gc;
  const __nv_bfloat16* AP;
  __nv_bfloat16* o;         // token layout
  __nv_bfloat16* W;         // chunk layout; may be nullptr (inference: nothing saved)
  __nv_bfloat16* U;
  __nv_bfloat16* h;
  const float* s_in;        // f32 [sequence][H][E][128 d][128 v] initial state, or nullptr (zero)
  float* s_out;             // same form: the state after the last token, or nullptr
  const int32_t* offsets;   // packed: first chunk of every document (n_seq + 1 entries), else nullptr
  const int32_t* cmap;
  int B, T, H, NC, n_seq;   // n_seq = documents (packed) or batch rows (dense)
  float scale;
  int* status;
  int beta_tma;             // beta rows of a chunk arrive by TMA (H a multiple of 4, base 16-byte aligned), else by global loads
};

struct RecParams {
  const __nv_bfloat16* dO;  // token layout
  const float* k2;
  const float* q2;
  const float* beta;
  const float* gc;
  const __nv_bfloat16* AP;
  const __nv_bfloat16* Pm;
  const __nv_bfloat16* U;   // chunk layout
  __nv_bfloat16* dV;        // token layout (out): the gradient of v, and the dW the later stages use
  __nv_bfloat16* dU;        // chunk layout (out)
  __nv_bfloat16* ds;        // chunk layout (out), same form as h: dL/dS at the END of a chunk; only slices above DD_MIN_LOG2_DECAY
  __nv_bfloat16* dkg;       // bf16 image [item][128/VC][t/8][128 d][t%8] (out): per value block, sum_e G_e (r_e U)^T
  float* dr;                // f32 [item][128/VC][64][E] (out): sum_v U*(K G_e) per value block
  const int32_t* offsets;
  const int32_t* cmap;
  int B, T, H, NC, n_seq;
  float scale;
  int* status;
  const float* g_in;        // f32 [sequence][H][E][128 d][128 v]: dL/dS after the last token (a later segment's hand-off), or nullptr (zero)
  float* g_out;             // same form: dL/dS before the first token, or nullptr
};

struct SgParams {
  const __nv_bfloat16* k;   // token layout
  const __nv_bfloat16* q;   // token layout
  const __nv_bfloat16* dO;  // token layout
  const __nv_bfloat16* dV;  // token layout
  const __nv_bfloat16* h;
  const __nv_bfloat16* ds;  // read only for slices above DD_MIN_LOG2_DECAY
  const __nv_bfloat16* dkg; // [item][NV][16 KB image] from the reverse recurrence
  const float* k2;
  const float* q2;
  const float* gc;
  __nv_bfloat16* dkq;       // bf16 image [item][col/8][128 rows][col%8] (out): rows 0..63 state part of dK, 64..127 of dQ
  float* da;                // f32 [item][64][E] (out)
  float* dc;                // f32 [item][64][E] (out)
  float* dd;                // f32 [item][E] (out)
  const int32_t* cmap;
  int B, T, H, NC, NV;
  float scale;
  int* status;
  int ahead;                // CTAs to launch (the SM count): the kernel is persistent, CTA c takes items c, c + ahead, ...
};

struct MatParams {
  const float* k2;
  const float* q2;
  const float* beta;
  const float* gc;
  const __nv_bfloat16* AP;
  const __nv_bfloat16* dkq; // bf16 image [item][col/8][128 rows][col%8] from the state-gradient kernel
  const float* da;
  const float* dc;
  const float* dd;
  const float* dr;          // [item][NV][64][E]
  __nv_bfloat16* dq;        // token layout (out)
  __nv_bfloat16* dk;
  float* dk2;               // token layout (out)
  float* dq2;
  float* dg;
  float* dbeta;
  const int32_t* cmap;
  int B, T, H, NC, NV;
  float scale;
  int* status;
  int ahead;                // CTAs to launch (the SM count): the kernel is persistent, CTA c takes items c, c + ahead, ...
};

}  // namespace tgdn

// E in {1,2,4,8,12,16}; dense rows need T % 64 == 0 and NC == T/64; packed rows need B == 1.
int tgdn_check_core_shape(int B, int T, int H, int E, int NC, int packed);
// Width of the value-axis block one CTA of the recurrences owns, by E.
int tgdn_value_block(int E);
int tgdn_sm_count();
