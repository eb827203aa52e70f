// Ragged batch packing on the GPU: cu_seqlens, position ids, flat token list and the per-row
// descriptors the attention kernel consumes.  Replaces the host loops and the T x T mask of
// src/batch_builder.zig:122-205 — the mask is implied by (row_seq, row_ctx).
#include "common.h"

namespace {

constexpr int kScanThreads = 1024;
constexpr int kScanItems = 4;

__global__ void __launch_bounds__(kScanThreads) pack_scan_kernel(const b200_pack_desc* __restrict__ desc, int n_req,
                                                                 int* __restrict__ cu_seqlens, int* __restrict__ last_row) {
  __shared__ int warp_sums[32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int c[kScanItems], sum = 0;
#pragma unroll
  for (int k = 0; k < kScanItems; ++k) {
    int i = tid * kScanItems + k;
    c[k] = i < n_req ? max(desc[i].count, 0) : 0;
    sum += c[k];
  }
  int inc = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == 31) warp_sums[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int w = warp_sums[lane], winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int t = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += t;
    }
    warp_sums[lane] = winc - w;
  }
  __syncthreads();
  int off = warp_sums[warp] + inc - sum;
  if (tid == 0) cu_seqlens[0] = 0;
#pragma unroll
  for (int k = 0; k < kScanItems; ++k) {
    int i = tid * kScanItems + k;
    off += c[k];
    if (i < n_req) {
      cu_seqlens[i + 1] = off;
      last_row[i] = off - 1;  // -1 for an empty request that opens the batch
    }
  }
}

__global__ void pack_fill_kernel(const b200_pack_desc* __restrict__ desc, int n_req, const int* __restrict__ cu_seqlens,
                                 const uint32_t* __restrict__ prefill_tokens, const uint32_t* __restrict__ last_token,
                                 uint32_t* __restrict__ token_ids, int* __restrict__ position_ids,
                                 int* __restrict__ row_to_req, int* __restrict__ row_seq, int* __restrict__ row_ctx,
                                 int total_rows) {
  int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= total_rows) return;
  // last request r with cu[r] <= row
  int lo = 0, hi = n_req - 1;
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (cu_seqlens[mid] <= row) lo = mid; else hi = mid - 1;
  }
  b200_pack_desc d = desc[lo];
  int j = row - cu_seqlens[lo];
  int pos = d.base_pos + j;
  token_ids[row] = d.src_offset >= 0 ? prefill_tokens[d.src_offset + j] : last_token[d.seq_slot];
  position_ids[row] = pos;
  row_to_req[row] = lo;
  row_seq[row] = d.seq_slot;
  row_ctx[row] = pos + 1;
}

}  // namespace

extern "C" b200_status b200_pack_batch(const b200_pack_desc* d_desc, int32_t n_req, const uint32_t* d_prefill_tokens,
                                       const uint32_t* d_last_token, int32_t* d_cu_seqlens, uint32_t* d_token_ids,
                                       int32_t* d_position_ids, int32_t* d_row_to_req, int32_t* d_row_seq,
                                       int32_t* d_row_ctx, int32_t* d_last_row, int32_t total_rows, void* stream) {
  b200_status st = b200_require_device();
  if (st != B200_OK) return st;
  if (n_req < 0 || n_req > kScanThreads * kScanItems) {
    b200_set_error("pack: %d requests in one step (limit %d)", n_req, kScanThreads * kScanItems);
    return B200_ERR_INVALID_ARGUMENT;
  }
  cudaStream_t s = (cudaStream_t)stream;
  pack_scan_kernel<<<1, kScanThreads, 0, s>>>(d_desc, n_req, d_cu_seqlens, d_last_row);
  B200_LAUNCH_CHECK();
  if (total_rows > 0 && n_req > 0) {
    pack_fill_kernel<<<(total_rows + 255) / 256, 256, 0, s>>>(d_desc, n_req, d_cu_seqlens, d_prefill_tokens, d_last_token,
                                                            d_token_ids, d_position_ids, d_row_to_req, d_row_seq,
                                                            d_row_ctx, total_rows);
    B200_LAUNCH_CHECK();
  }
  return B200_OK;
}
