// Shared definitions of the device page pool (see kv_pool.cu for the layout).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "dmlx_b200.h"

enum { ST_FREE_TOP = 0, ST_ERR = 1, ST_N_TOUCH = 2, ST_N_COW = 3, ST_ATTN_ERR = 4 };

// Plain-old-data view of the pool, passed to kernels by value.
struct KvDev {
  void* k_pool = nullptr;
  void* v_pool = nullptr;
  float* k_scale = nullptr;
  float* v_scale = nullptr;
  int* free_stack = nullptr;
  int* ref_count = nullptr;
  int* tokens_used = nullptr;
  int* block_table = nullptr;
  int* seq_pages = nullptr;
  int* seq_len = nullptr;
  int* state = nullptr;
  int4* touch_list = nullptr;  // {page, first packed row, rows, first slot in page}
  int2* cow_list = nullptr;    // {source page, private copy}
  int n_layers = 0, n_kv_heads = 0, head_dim = 0, page_size = 0, n_pages = 0, max_seqs = 0, max_pages_per_seq = 0;
  int elem_bytes = 2;
  int max_touch = 0;
};

struct b200_kv {
  b200_kv_config cfg;
  KvDev dev;
  int* d_admin_in = nullptr;
  int* d_admin_out = nullptr;
  int admin_cap = 0;
  // split-K attention scratch
  int* d_chunk_start = nullptr;  // [max_rows + 2]
  float* d_part_o = nullptr;     // [max_chunks][n_q_heads][head_dim]
  float* d_part_ml = nullptr;    // [max_chunks][n_q_heads][2]  (running max in log2 units, sum)
  int max_chunks = 0;
  // row-group plan of the prefill attention path: [3][max_rows + 2] = group_first | part_base | row_group
  int* d_groups = nullptr;
  // 3-D tensor maps over the bf16 pools: [layer][page*kv_head*32 rows][head_dim], box 64 x 32 x 1
  CUtensorMap kmap, vmap;
};

// Internal variants with explicit row strides (elements), used when q/k/v live inside a fused
// projection output.  reuse_plan = 1 skips the split-K planning kernel: the caller guarantees that the
// previous attention call on this pool used the same row arrays (the layers of one model step).
b200_status b200_kv_append_strided(b200_kv* kv, int32_t layer, const void* d_k_rows, const void* d_v_rows,
                                   int32_t k_stride, int32_t v_stride, int32_t total_rows, void* stream);
b200_status b200_kv_rope_append_strided(b200_kv* kv, int32_t layer, void* d_q, const void* d_k_rows, const void* d_v_rows,
                                        int32_t q_stride, int32_t k_stride, int32_t v_stride, const int32_t* d_positions,
                                        const int32_t* d_row_seq, int32_t total_rows, int32_t n_q_heads, float theta, void* stream);
b200_status b200_paged_attn_decode_strided(b200_kv* kv, int32_t layer, const void* d_q, int32_t q_stride,
                                           const int32_t* d_row_seq, const int32_t* d_row_ctx, int32_t total_rows,
                                           void* d_out, void* stream, int32_t reuse_plan);
b200_status b200_paged_attn_prefill_strided(b200_kv* kv, int32_t layer, const void* d_q, int32_t q_stride,
                                            const int32_t* d_row_seq, const int32_t* d_row_ctx, int32_t total_rows,
                                            void* d_out, void* stream, int32_t reuse_plan);
