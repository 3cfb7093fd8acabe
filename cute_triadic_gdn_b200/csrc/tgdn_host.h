// Host-side helpers shared by the translation units of libtgdn_b200 (not part of the public ABI).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/tgdn.h"
#include "../../include/tgdn_selftest.h"

// -(1000 + e) for a CUDA runtime error, 0 for cudaSuccess.
int tgdn_cuda_error(cudaError_t e);

// Device pointer of the status word of the current device (a __device__ int of this library).
int* tgdn_status_word();

// Tensor map over a (B, T, H, 128) bf16 tensor in token layout: box = [box_cols columns][1 head][box_rows tokens][1 row].
// swizzle128 = 1 asks for the 128-byte swizzle (box_cols must then be 64).
int tgdn_make_token_map(CUtensorMap* map, const void* base, int B, int T, int H, int box_cols, int box_rows, int swizzle128);

// Tensor map over a (B, T, H, E) f32 gate tensor (k2, q2) in token layout, E a multiple of 4: box = [E][1 head][64 tokens][1 row],
// which lands in shared memory as 64 dense rows of E floats.
int tgdn_make_gate_map(CUtensorMap* map, const float* base, int B, int T, int H, int E);

// Tensor map over a (B, T, C) bf16 tensor with element strides (stride_b, stride_t, 1): box = [box_cols][box_rows][1], no swizzle.
int tgdn_make_rows_map(CUtensorMap* map, const void* base, int C, int T, int B, int64_t stride_t, int64_t stride_b, int box_cols,
                       int box_rows);

// True when the current device is compute capability 10.x; also binds the device's primary context to the calling thread.
int tgdn_check_device();
