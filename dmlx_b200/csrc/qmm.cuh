// Shared definitions of the quantised-matmul kernels (see qmm.cu for the weight layout).
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

#include "dmlx_b200.h"

struct b200_qweight {
  int mode = 0, n_experts = 1, n = 0, k = 0, nt = 0, kc = 0, block_bytes = 0;
  unsigned char* d_blocks = nullptr;  // [expert][n tile][k chunk][block_bytes]
};

struct QmmArgs {
  const unsigned char* blocks;  // first block of the weight (expert) this launch/tile uses
  const __nv_bfloat16* x;       // [rows, k]
  __nv_bfloat16* y;             // [rows, n] (or [rows, n/2] with the SwiGLU epilogue)
  const __nv_bfloat16* residual;
  const float* row_scales;      // optional per-row multiplier applied in the epilogue
  float* ws;                    // split-K scratch: [tile][split][tn][128] f32
  int* err;                     // device error word
  int rows, n, k, nt, kc;
  int chunks_per_split, tn, stages;
  int epilogue;
  int x_row0;                   // first row of this launch within the tensor map
  float swiglu_limit;

  __device__ __forceinline__ int row_base_out(int token) const { return token; }
  __device__ __forceinline__ float row_scale(int token) const { return row_scales ? row_scales[token] : 1.0f; }
};
