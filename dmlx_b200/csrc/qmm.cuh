// Shared definitions of the quantised-matmul kernels (see qmm.cu for the weight layout).
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

#include "dmlx_b200.h"

struct b200_qweight {
  int mode = 0, n_experts = 1, n = 0, k = 0, nt = 0, kc = 0, block_bytes = 0;
  unsigned char* d_blocks = nullptr;  // [expert][n tile][k chunk][block_bytes]
  // MXFP4 only, built on first use of the block-scaled tensor-core path: the codes as a plain row-major
  // matrix [expert * nt * 128, k / 2] (two codes per byte, even column in the low nibble) read by TMA,
  // and the E8M0 scales in 512-byte atoms [expert][n tile][k / 128]: byte (row % 32) * 16 + (row / 32) * 4 + block.
  unsigned char* d_mx_codes = nullptr;
  unsigned char* d_mx_sf = nullptr;
  alignas(64) unsigned char mx_map[128] = {};  // CUtensorMap over d_mx_codes
};

struct QmmArgs {
  const unsigned char* blocks;  // first block of the weight (expert) this launch/tile uses
  const __nv_bfloat16* x;       // [rows, k]
  __nv_bfloat16* y;             // [rows, n] (or [rows, n/2] with the SwiGLU epilogue)
  const __nv_bfloat16* residual;
  const float* row_scales;      // optional per-row multiplier applied in the epilogue
  float* ws;                    // split-K scratch: [split][row][nt*128] f32
  const int4* items;            // grouped mode: {expert, first row, rows, -} per work item (device)
  const int* n_items;           // grouped mode: number of valid items (device)
  size_t expert_stride;         // grouped mode: bytes between consecutive experts' blocks
  int max_items;
  int* err;                     // device error word
  int rows, n, k, nt, kc;
  int chunks_per_split, tn, stages;
  int a_slots;                  // tensor-memory-operand kernel: slots of dequantised weights in tensor memory
  int x_slots;                  // tensor-memory-operand kernel: ring slots of activation tiles (the raw weight blocks have their own ring of `stages` slots); tile-pair kernel: ring slots of raw block pairs
  int direct_large;             // one K split and many token tiles: write the output from the kernel, no scratch
  int splits;                   // small-batch kernel: number of K splits (the grid is persistent)
  int epilogue;
  int x_slab;                   // small-batch kernel: activations staged in shared memory
  int x_row0;                   // first row of this launch within the tensor map
  float swiglu_limit;
  // split-K finish fused with the RMSNorm that reads the result next (residual epilogue only)
  const __nv_bfloat16* norm_w;  // non-null: the finish pass also writes norm_out = rmsnorm(y) * norm_w
  __nv_bfloat16* norm_out;
  float norm_eps;
  // block-scaled MXFP4 path
  const unsigned char* mx_sf;   // scale atoms of the weight
  const float* act_unscale;     // per activation row: factor that undoes the row's power-of-two scaling
  const int* x_gather;          // optional: activation row p is x[x_gather[p] / x_gather_div] (expert-sorted rows
  int x_gather_div;             //   taken straight from the token matrix while they are split; no sorted copy)
  const int* rows_valid;        // optional (device): only the first *rows_valid rows exist; the rest of `rows` is capacity
  int mx_expert_rows;           // rows of the code matrix per expert (nt * 128)
  int kc128;                    // K / 128
  int did_norm;                 // host only: the finish pass also wrote norm_out
  b200_qmm_partials* defer = nullptr;  // when set, a dense launch with epilogue NONE leaves its finish pass to the caller

  __device__ __forceinline__ int row_base_out(int token) const { return token; }
  __device__ __forceinline__ float row_scale(int token) const { return row_scales ? row_scales[token] : 1.0f; }
};

b200_status b200_qmm_grouped(const b200_qweight* w, const void* d_x, int32_t rows, void* d_y, int32_t epilogue,
                             const float* d_row_scales, float swiglu_limit, const int4* d_items, const int* d_n_items,
                             int32_t max_items, int32_t tile_rows, void* stream);
// 1 if b200_qmm_grouped_from_tokens can serve this weight and tile size (block-scaled MXFP4 path).
int b200_qmm_grouped_takes_tokens(const b200_qweight* w, int32_t tile_rows);
// The same matmul with the expert-sorted activation rows read from the unsorted token matrix:
// row p = d_tokens[d_order[p] / top_k].
// d_rows_valid (optional, device): the number of rows that exist; `rows` is then only the capacity of the buffers.
b200_status b200_qmm_grouped_from_tokens(const b200_qweight* w, const void* d_tokens, const int* d_order, int32_t top_k,
                                         int32_t rows, void* d_y, int32_t epilogue, const float* d_row_scales,
                                         float swiglu_limit, const int4* d_items, const int* d_n_items, int32_t max_items,
                                         int32_t tile_rows, void* stream, const int* d_rows_valid = nullptr);
// Queues copies of the matmul error words into pinned host memory on `stream` (no synchronisation,
// nothing cleared): h_out[0] = the word of b200_qmm and the grouped launches, h_out[1] = the word of
// b200_qmm_static_scratch on the current device.
b200_status b200_qmm_error_words_async(int32_t* h_out, void* stream);
