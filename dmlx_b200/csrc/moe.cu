// Mixture-of-experts routing and the ragged grouped matmul around it.
//
//   route   : per token, f32 scoring of the router logits (softmax / sigmoid / sqrt-softplus),
//             + selection bias, top-k with the tie rule of an ascending stable argsort's last k
//             (src/moe_router.zig:59-96, src/models/deepseek_v4.zig:383-396,555-681): among equal
//             scores the larger expert index wins, output in ascending (score, index) order;
//             weights come from the unbiased scores.  One warp per token, no sort.
//   group   : stable counting sort of the N*k assignments by expert
//             (the two argsorts of src/models/deepseek_v4.zig:747-784): expert_offsets[E+1],
//             order[N*k], inv_order[N*k], and the work items of the grouped matmul.
//   gather  : x_sorted[p] = x[order[p] / k], row_scales[p] = weights[order[p]].
//   grouped matmul : b200_qmm_grouped (tcgen05, one work item per expert token tile).
//   combine : out[t] = sum_j y_sorted[inv_order[t*k + j]] (+ shared expert)
//             (src/models/deepseek_v4.zig:809-819,1051).
#include <cuda_bf16.h>

#include <vector>

#include "common.h"
#include "qmm.cuh"

b200_status b200_gather_rows(const void* d_src, const int32_t* d_idx, void* d_dst, int32_t rows, int32_t hidden, void* stream);

namespace {

constexpr int kMaxExperts = 1024;
constexpr int kMaxTopK = 16;

__device__ __forceinline__ bool beats(float va, int ia, float vb, int ib) { return va > vb || (va == vb && ia > ib); }

// One warp per token.  E <= 1024 (32 experts per lane).
template <typename LogitT>
__global__ void route_kernel(const LogitT* __restrict__ logits, const float* __restrict__ bias, int n_tokens, int n_experts,
                             int k, int scoring, float route_scale, uint32_t* __restrict__ out_idx,
                             float* __restrict__ out_w, int* __restrict__ counts) {
  const int token = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (token >= n_tokens) return;
  constexpr int PER = kMaxExperts / 32;
  float sc[PER];      // unbiased scores
  float ch[PER];      // scores used for the choice
  const int per = (n_experts + 31) / 32;
  float mx = -INFINITY;
  for (int i = 0; i < per; ++i) {
    const int e = i * 32 + lane;
    float v = -INFINITY;
    if (e < n_experts) v = (float)logits[(size_t)token * n_experts + e];
    sc[i] = v;
    mx = fmaxf(mx, v);
  }
  if (scoring == 0) {  // softmax in f32 (deepseek_v4.zig:562-564)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (int i = 0; i < per; ++i) {
      const float e = (i * 32 + lane < n_experts) ? expf(sc[i] - mx) : 0.f;
      sc[i] = e;
      sum += e;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    for (int i = 0; i < per; ++i) sc[i] = sc[i] / sum;
  } else if (scoring == 1) {  // sigmoid
    for (int i = 0; i < per; ++i) sc[i] = 1.0f / (1.0f + expf(-sc[i]));
  } else {  // sqrt(softplus)
    for (int i = 0; i < per; ++i) sc[i] = sqrtf(log1pf(expf(sc[i])));
  }
  for (int i = 0; i < per; ++i) {
    const int e = i * 32 + lane;
    ch[i] = e < n_experts ? sc[i] + (bias ? bias[e] : 0.f) : -INFINITY;
  }
  // k rounds of warp arg-max under (score, index) order; results come out descending.
  float sel_w[kMaxTopK];
  int sel_e[kMaxTopK];
  for (int r = 0; r < k; ++r) {
    float bv = -INFINITY;
    int be = -1, bi = -1;
    for (int i = 0; i < per; ++i) {
      const int e = i * 32 + lane;
      if (e < n_experts && beats(ch[i], e, bv, be)) { bv = ch[i]; be = e; bi = i; }
    }
    float wv = bv;
    int we = be;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, wv, o);
      const int oe = __shfl_xor_sync(0xffffffffu, we, o);
      if (beats(ov, oe, wv, we)) { wv = ov; we = oe; }
    }
    // the owning lane retires the winner and publishes its unbiased score
    float w_unbiased = 0.f;
    if (we == be && bi >= 0) { w_unbiased = sc[bi]; ch[bi] = -INFINITY; }
    w_unbiased = __shfl_sync(0xffffffffu, w_unbiased, we & 31);
    sel_w[r] = w_unbiased;
    sel_e[r] = we;
  }
  if (lane == 0) {
    float denom = 1.0f;
    if (scoring != 0) {  // non-softmax scores are renormalised over the selection (deepseek_v4.zig:663-672)
      float s = 0.f;
      for (int r = k - 1; r >= 0; --r) s += sel_w[r];  // ascending order, as the reference sums
      denom = s + 1e-20f;
    }
    for (int r = 0; r < k; ++r) {
      const int src = k - 1 - r;  // ascending (score, index)
      out_idx[(size_t)token * k + r] = (uint32_t)sel_e[src];
      out_w[(size_t)token * k + r] = (scoring != 0 ? sel_w[src] / denom : sel_w[src]) * route_scale;
      if (counts) atomicAdd(&counts[sel_e[src]], 1);
    }
  }
}

// offsets = exclusive scan of counts; work items {expert, first row, rows} for tiles of `tile_rows`.
__global__ void offsets_items_kernel(const int* __restrict__ counts, int n_experts, int tile_rows, int* __restrict__ offsets,
                                     int4* __restrict__ items, int* __restrict__ n_items) {
  __shared__ int s_off[kMaxExperts + 1], s_item[kMaxExperts + 1];
  if (threadIdx.x == 0) {
    int o = 0, it = 0;
    for (int e = 0; e < n_experts; ++e) {
      s_off[e] = o;
      s_item[e] = it;
      o += counts[e];
      it += (counts[e] + tile_rows - 1) / tile_rows;
    }
    s_off[n_experts] = o;
    s_item[n_experts] = it;
    *n_items = it;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= n_experts; e += blockDim.x) offsets[e] = s_off[e];
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
    const int cnt = s_off[e + 1] - s_off[e];
    for (int t = 0, i = s_item[e]; t < cnt; t += tile_rows, ++i) items[i] = make_int4(e, s_off[e] + t, min(tile_rows, cnt - t), 0);
  }
}

// One CTA per expert: collects, in flat order, the assignments routed to it (stable).  A thread looks
// at 8 consecutive assignments per pass (two 16-byte loads), so a pass of the CTA covers 8192 of them
// with one block scan.
__global__ void __launch_bounds__(1024) place_kernel(const uint32_t* __restrict__ indices, int n_assign,
                                                     const int* __restrict__ offsets, int* __restrict__ order,
                                                     int* __restrict__ inv_order) {
  __shared__ int warp_sums[32];
  __shared__ int s_base;
  const int e = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) s_base = offsets[e];
  __syncthreads();
  const bool vec = (reinterpret_cast<uintptr_t>(indices) & 15) == 0;
  for (int start = 0; start < n_assign; start += blockDim.x * 8) {
    const int a0 = start + tid * 8;
    uint32_t idx[8];
    if (vec && a0 + 8 <= n_assign) {
      const uint4 q0 = *reinterpret_cast<const uint4*>(indices + a0), q1 = *reinterpret_cast<const uint4*>(indices + a0 + 4);
      idx[0] = q0.x; idx[1] = q0.y; idx[2] = q0.z; idx[3] = q0.w; idx[4] = q1.x; idx[5] = q1.y; idx[6] = q1.z; idx[7] = q1.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) idx[j] = a0 + j < n_assign ? indices[a0 + j] : 0xFFFFFFFFu;
    }
    unsigned mask = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) mask |= ((int)idx[j] == e ? 1u : 0u) << j;
    const int mine = __popc(mask);
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    int before = 0, total = 0;
    {
      const int v = warp_sums[lane];  // 32 warps
      int sc = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, sc, o);
        if (lane >= o) sc += t;
      }
      total = __shfl_sync(0xffffffffu, sc, 31);
      before = __shfl_sync(0xffffffffu, sc - v, warp);
    }
    int pos = s_base + before + incl - mine;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (mask & (1u << j)) {
        order[pos] = a0 + j;
        inv_order[a0 + j] = pos;
        ++pos;
      }
    }
    __syncthreads();
    if (tid == 0) s_base += total;
    __syncthreads();
  }
}

// row_scales[p] = weights[order[p]] alone (the rows themselves are read in place by the matmul).
// n_valid (optional, device): rows that exist when n is only the capacity.
__global__ void row_scales_kernel(const int* __restrict__ order, const float* __restrict__ weights, int n, float* __restrict__ out,
                                  const int* __restrict__ n_valid) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p < n && (!n_valid || p < *n_valid)) out[p] = weights[order[p]];
}

// Expert parallelism: global expert ids -> ids among this rank's experts, everything else marked as
// "not mine" (a value no expert matches, so the counting sort leaves those assignments out).
__global__ void localize_kernel(const uint32_t* __restrict__ idx, int n_assign, int first_expert, int n_local,
                                uint32_t* __restrict__ local_idx) {
  const int a = blockIdx.x * blockDim.x + threadIdx.x;
  if (a >= n_assign) return;
  const int e = (int)idx[a] - first_expert;
  local_idx[a] = (e >= 0 && e < n_local) ? (uint32_t)e : 0xFFFFFFFFu;
}

// Expert parallelism: this rank's share of every token's sum over k (f32; zero where none of the
// token's experts lives here).  inv_order[a] < 0 marks an assignment served by another rank.
__global__ void combine_partial_kernel(const __nv_bfloat16* __restrict__ y_sorted, const int* __restrict__ inv_order, int k,
                                       int hidden, float* __restrict__ out) {
  const int t = blockIdx.x;
  int rows[kMaxTopK];
  for (int j = 0; j < k; ++j) rows[j] = inv_order[t * k + j];
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < k; ++j) {
      if (rows[j] < 0) continue;
      const uint4 q = reinterpret_cast<const uint4*>(y_sorted + (size_t)rows[j] * hidden)[i];
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        acc[2 * e] += __uint_as_float(w[e] << 16);
        acc[2 * e + 1] += __uint_as_float(w[e] & 0xFFFF0000u);
      }
    }
    float4* dst = reinterpret_cast<float4*>(out + (size_t)t * hidden) + 2 * i;
    dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
}

// Expert parallelism: out = bf16(routed sum (f32, reduced over the ranks) + shared expert).
__global__ void add_shared_kernel(const float* __restrict__ routed, const __nv_bfloat16* __restrict__ shared_out, size_t n8,
                                  __nv_bfloat16* __restrict__ out) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  const float4 a = reinterpret_cast<const float4*>(routed)[2 * i], b = reinterpret_cast<const float4*>(routed)[2 * i + 1];
  float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
  if (shared_out) {
    const uint4 q = reinterpret_cast<const uint4*>(shared_out)[i];
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) { v[2 * e] += __uint_as_float(w[e] << 16); v[2 * e + 1] += __uint_as_float(w[e] & 0xFFFF0000u); }
  }
  uint4 o;
  __nv_bfloat162 p0 = __floats2bfloat162_rn(v[0], v[1]), p1 = __floats2bfloat162_rn(v[2], v[3]);
  __nv_bfloat162 p2 = __floats2bfloat162_rn(v[4], v[5]), p3 = __floats2bfloat162_rn(v[6], v[7]);
  o.x = *reinterpret_cast<uint32_t*>(&p0); o.y = *reinterpret_cast<uint32_t*>(&p1);
  o.z = *reinterpret_cast<uint32_t*>(&p2); o.w = *reinterpret_cast<uint32_t*>(&p3);
  reinterpret_cast<uint4*>(out)[i] = o;
}

__global__ void gather_sorted_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ order,
                                     const float* __restrict__ weights, int k, int hidden,
                                     __nv_bfloat16* __restrict__ x_sorted, float* __restrict__ row_scales,
                                     const int* __restrict__ n_valid) {
  const int p = blockIdx.x;
  if (n_valid && p >= *n_valid) return;
  const int a = order[p];
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(a / k) * hidden);
  uint4* dst = reinterpret_cast<uint4*>(x_sorted + (size_t)p * hidden);
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) dst[i] = src[i];
  if (threadIdx.x == 0 && row_scales) row_scales[p] = weights[a];
}

__global__ void combine_kernel(const __nv_bfloat16* __restrict__ y_sorted, const int* __restrict__ inv_order, int k, int hidden,
                               const __nv_bfloat16* __restrict__ shared_out, __nv_bfloat16* __restrict__ out) {
  const int t = blockIdx.x;
  if (hidden % 8 == 0 && k <= 16) {  // 16-byte loads, the row indices read once
    int rows[16];
    for (int j = 0; j < k; ++j) rows[j] = inv_order[t * k + j];
    for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = 0; j <= k; ++j) {
        if (j == k && !shared_out) break;
        const __nv_bfloat16* src = j < k ? y_sorted + (size_t)rows[j] * hidden : shared_out + (size_t)t * hidden;
        const uint4 q = reinterpret_cast<const uint4*>(src)[i];
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          acc[2 * e] += __uint_as_float(w[e] << 16);
          acc[2 * e + 1] += __uint_as_float(w[e] & 0xFFFF0000u);
        }
      }
      uint4 o;
      __nv_bfloat162 p0 = __floats2bfloat162_rn(acc[0], acc[1]), p1 = __floats2bfloat162_rn(acc[2], acc[3]);
      __nv_bfloat162 p2 = __floats2bfloat162_rn(acc[4], acc[5]), p3 = __floats2bfloat162_rn(acc[6], acc[7]);
      o.x = *reinterpret_cast<uint32_t*>(&p0); o.y = *reinterpret_cast<uint32_t*>(&p1);
      o.z = *reinterpret_cast<uint32_t*>(&p2); o.w = *reinterpret_cast<uint32_t*>(&p3);
      reinterpret_cast<uint4*>(out + (size_t)t * hidden)[i] = o;
    }
    return;
  }
  for (int i = threadIdx.x; i < hidden / 2; i += blockDim.x) {
    float2 acc = make_float2(0.f, 0.f);
    for (int j = 0; j < k; ++j) {
      const float2 v = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(y_sorted + (size_t)inv_order[t * k + j] * hidden)[i]);
      acc.x += v.x; acc.y += v.y;
    }
    if (shared_out) {
      const float2 v = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(shared_out + (size_t)t * hidden)[i]);
      acc.x += v.x; acc.y += v.y;
    }
    reinterpret_cast<__nv_bfloat162*>(out + (size_t)t * hidden)[i] = __floats2bfloat162_rn(acc.x, acc.y);
  }
}

}  // namespace

extern "C" {

b200_status b200_moe_route(const void* d_logits, int32_t logits_are_f32, const float* d_bias, int32_t n_tokens,
                           int32_t n_experts, int32_t k, int32_t scoring, float route_scale, uint32_t* d_indices,
                           float* d_weights, int32_t* d_counts, void* stream) {
  b200_status st = b200_require_device();
  if (st != B200_OK) return st;
  if (n_experts <= 0 || n_experts > kMaxExperts || k <= 0 || k > kMaxTopK || k > n_experts || scoring < 0 || scoring > 2) {
    b200_set_error("route: need 1 <= k <= min(%d, E), E <= %d, scoring in {0,1,2}", kMaxTopK, kMaxExperts);
    return B200_ERR_INVALID_ARGUMENT;
  }
  if (n_tokens <= 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  if (d_counts) B200_CUDA_TRY(cudaMemsetAsync(d_counts, 0, sizeof(int) * n_experts, s));
  const int blocks = (n_tokens * 32 + 255) / 256;
  if (logits_are_f32)
    route_kernel<float><<<blocks, 256, 0, s>>>((const float*)d_logits, d_bias, n_tokens, n_experts, k, scoring, route_scale,
                                               d_indices, d_weights, d_counts);
  else
    route_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((const __nv_bfloat16*)d_logits, d_bias, n_tokens, n_experts, k, scoring,
                                                       route_scale, d_indices, d_weights, d_counts);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

b200_status b200_moe_group(const uint32_t* d_indices, const int32_t* d_counts, int32_t n_tokens, int32_t k,
                           int32_t n_experts, int32_t tile_rows, int32_t* d_offsets, int32_t* d_order,
                           int32_t* d_inv_order, void* d_items, int32_t* d_n_items, void* stream) {
  b200_status st = b200_require_device();
  if (st != B200_OK) return st;
  if (n_experts <= 0 || n_experts > kMaxExperts || tile_rows <= 0) { b200_set_error("group: bad expert count or tile"); return B200_ERR_INVALID_ARGUMENT; }
  if (n_tokens <= 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  offsets_items_kernel<<<1, 256, 0, s>>>(d_counts, n_experts, tile_rows, d_offsets, (int4*)d_items, d_n_items);
  B200_LAUNCH_CHECK();
  place_kernel<<<n_experts, 1024, 0, s>>>(d_indices, n_tokens * k, d_offsets, d_order, d_inv_order);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

b200_status b200_moe_gather(const void* d_x, const int32_t* d_order, const float* d_weights, int32_t n_assign, int32_t k,
                            int32_t hidden, void* d_x_sorted, float* d_row_scales, void* stream) {
  b200_status st = b200_require_device();
  if (st != B200_OK) return st;
  if (hidden % 8) { b200_set_error("gather: hidden must be a multiple of 8"); return B200_ERR_INVALID_ARGUMENT; }
  if (n_assign <= 0) return B200_OK;
  gather_sorted_kernel<<<n_assign, 128, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)d_x, d_order, d_weights, k, hidden,
                                                                  (__nv_bfloat16*)d_x_sorted, d_row_scales, nullptr);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

b200_status b200_moe_grouped_qmm(const b200_qweight* w, const void* d_x_sorted, int32_t rows, void* d_y_sorted,
                                 int32_t epilogue, const float* d_row_scales, float swiglu_limit, const void* d_items,
                                 const int32_t* d_n_items, int32_t max_items, int32_t tile_rows, void* stream) {
  if (tile_rows % 16 != 0 || tile_rows < 16 || tile_rows > 256) { b200_set_error("grouped qmm: tile_rows must be a multiple of 16 in 16..256"); return B200_ERR_INVALID_ARGUMENT; }
  return b200_qmm_grouped(w, d_x_sorted, rows, d_y_sorted, epilogue, d_row_scales, swiglu_limit, (const int4*)d_items,
                          d_n_items, max_items, tile_rows, stream);
}

b200_status b200_moe_gather_rows(const void* d_src, const int32_t* d_idx, void* d_dst, int32_t rows, int32_t hidden,
                                 void* stream) {
  b200_status st = b200_require_device();
  if (st != B200_OK) return st;
  if (hidden % 8) { b200_set_error("gather_rows: hidden must be a multiple of 8"); return B200_ERR_INVALID_ARGUMENT; }
  return b200_gather_rows(d_src, d_idx, d_dst, rows, hidden, stream);
}

b200_status b200_moe_combine(const void* d_y_sorted, const int32_t* d_inv_order, int32_t n_tokens, int32_t k,
                             int32_t hidden, const void* d_shared_out, void* d_out, void* stream) {
  b200_status st = b200_require_device();
  if (st != B200_OK) return st;
  if (hidden % 2) { b200_set_error("combine: hidden must be even"); return B200_ERR_INVALID_ARGUMENT; }
  if (n_tokens <= 0) return B200_OK;
  combine_kernel<<<n_tokens, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)d_y_sorted, d_inv_order, k, hidden,
                                                             (const __nv_bfloat16*)d_shared_out, (__nv_bfloat16*)d_out);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

// Expert parallelism, the plan of one rank (the grouping of src/models/deepseek_v4.zig:747-784 restricted
// to the experts that live on `rank`): of the N*k assignments of all ranks' tokens, those whose expert is
// one of this rank's n_experts / world are grouped by local expert (stable); offsets [E_local + 1],
// order [<= N*k] (row p of the grouped matmul is assignment order[p]), inv_order [N*k] (-1 where the
// assignment is served elsewhere), work items, and the local ids as scratch.  d_counts is the histogram
// over the global experts that b200_moe_route produced.
b200_status b200_ep_plan(const uint32_t* d_indices, const int32_t* d_counts, int32_t n_tokens, int32_t k, int32_t n_experts,
                         int32_t rank, int32_t world, int32_t tile_rows, uint32_t* d_local_idx, int32_t* d_offsets,
                         int32_t* d_order, int32_t* d_inv_order, void* d_items, int32_t* d_n_items, void* stream) {
  b200_status st = b200_require_device();
  if (st != B200_OK) return st;
  if (world <= 0 || n_experts % world != 0 || rank < 0 || rank >= world || tile_rows <= 0 || n_experts / world > kMaxExperts) {
    b200_set_error("ep plan: %d experts over %d ranks (rank %d)", n_experts, world, rank);
    return B200_ERR_INVALID_ARGUMENT;
  }
  if (n_tokens <= 0) return B200_OK;
  const int n_local = n_experts / world, A = n_tokens * k;
  cudaStream_t s = (cudaStream_t)stream;
  localize_kernel<<<(A + 255) / 256, 256, 0, s>>>(d_indices, A, rank * n_local, n_local, d_local_idx);
  B200_LAUNCH_CHECK();
  B200_CUDA_TRY(cudaMemsetAsync(d_inv_order, 0xFF, sizeof(int) * (size_t)A, s));
  offsets_items_kernel<<<1, 256, 0, s>>>(d_counts + rank * n_local, n_local, tile_rows, d_offsets, (int4*)d_items, d_n_items);
  B200_LAUNCH_CHECK();
  place_kernel<<<n_local, 1024, 0, s>>>(d_local_idx, A, d_offsets, d_order, d_inv_order);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// One MoE layer: DSV4MoE.forward (src/models/deepseek_v4.zig:1010-1056) =
// shared expert + gate (route) + SwitchGLU over the routed experts (:721-848) + sum.
// ---------------------------------------------------------------------------------------------
struct b200_moe {
  b200_moe_config cfg{};
  const b200_qweight *gate = nullptr, *exp_gu = nullptr, *exp_down = nullptr, *sh_gu = nullptr, *sh_down = nullptr;
  float* d_bias = nullptr;
  __nv_bfloat16 *logits = nullptr, *x_sorted = nullptr, *act_sorted = nullptr, *y_sorted = nullptr, *sh_act = nullptr,
                *sh_out = nullptr;
  uint32_t* indices = nullptr;
  float *weights = nullptr, *row_scales = nullptr;
  int *counts = nullptr, *offsets = nullptr, *order = nullptr, *inv_order = nullptr, *n_items = nullptr;
  int4* items = nullptr;
  int max_items = 0;
  // expert parallelism (cfg.ep_world > 1): the weights hold this rank's n_experts / ep_world experts; the
  // buffers above are sized for the tokens of all ranks
  int n_local = 0, first_expert = 0;
  __nv_bfloat16* x_all = nullptr;   // [world * max_tokens, hidden]: every rank's tokens (all-gather)
  uint32_t* local_idx = nullptr;    // [world * max_tokens * k]
  float *partial = nullptr;         // [world * max_tokens, hidden] f32: this rank's share of every token's sum
  float *reduced = nullptr;         // [max_tokens, hidden] f32: the sums of this rank's tokens (reduce-scatter)
};

extern "C" {

void b200_moe_destroy(b200_moe* m) {
  if (!m) return;
  void* ptrs[] = {m->d_bias, m->logits, m->x_sorted, m->act_sorted, m->y_sorted, m->sh_act, m->sh_out, m->indices, m->weights,
                  m->row_scales, m->counts, m->offsets, m->order, m->inv_order, m->n_items, m->items, m->x_all, m->local_idx,
                  m->partial, m->reduced};
  for (void* p : ptrs) if (p) cudaFree(p);
  delete m;
}

b200_status b200_moe_create(const b200_moe_config* c, const b200_qweight* gate, const float* h_bias,
                            const b200_qweight* experts_gate_up, const b200_qweight* experts_down,
                            const b200_qweight* shared_gate_up, const b200_qweight* shared_down, b200_moe** out) {
  *out = nullptr;
  b200_status st = b200_require_device();
  if (st != B200_OK) return st;
  const bool ep_mode = c->ep_world >= 1;  // a group of one rank runs the same path (tests on one GPU)
  const int world = ep_mode ? c->ep_world : 1;
  if (ep_mode && (c->n_experts % world != 0 || c->ep_rank < 0 || c->ep_rank >= world || c->hidden % 8 != 0)) {
    b200_set_error("moe: %d experts do not divide over %d ranks (rank %d)", c->n_experts, world, c->ep_rank);
    return B200_ERR_INVALID_ARGUMENT;
  }
  const int n_local = c->n_experts / world;
  if (!gate || !experts_gate_up || !experts_down || gate->n != c->n_experts || gate->k != c->hidden ||
      experts_gate_up->n_experts != n_local || experts_gate_up->n != 2 * c->inter || experts_gate_up->k != c->hidden ||
      experts_down->n_experts != n_local || experts_down->n != c->hidden || experts_down->k != c->inter ||
      c->tile_rows % 16 != 0 || c->tile_rows < 16 || c->tile_rows > 256 || c->max_tokens <= 0) {
    b200_set_error("moe: weight shapes do not match the configuration");
    return B200_ERR_INVALID_ARGUMENT;
  }
  auto* m = new b200_moe();
  m->cfg = *c;
  m->gate = gate; m->exp_gu = experts_gate_up; m->exp_down = experts_down; m->sh_gu = shared_gate_up; m->sh_down = shared_down;
  m->n_local = n_local;
  m->first_expert = ep_mode ? c->ep_rank * n_local : 0;
  // with expert parallelism every rank routes the tokens of all ranks; a rank's matmul rows are the
  // assignments that fall on its experts, at most all of them
  const size_t N = (size_t)c->max_tokens * world, A = N * c->top_k;
  m->max_items = n_local + (int)((A + c->tile_rows - 1) / c->tile_rows);
#define M_ALLOC(ptr, bytes)                                                                  \
  do {                                                                                       \
    if (cudaMalloc((void**)&(ptr), (bytes)) != cudaSuccess) {                                \
      b200_set_error("moe: cudaMalloc(%zu) failed", (size_t)(bytes));                        \
      cudaGetLastError();                                                                    \
      b200_moe_destroy(m);                                                                   \
      return B200_ERR_CUDA;                                                                  \
    }                                                                                        \
  } while (0)
  M_ALLOC(m->logits, N * c->n_experts * 2);
  M_ALLOC(m->indices, A * 4);
  M_ALLOC(m->weights, A * 4);
  M_ALLOC(m->row_scales, A * 4);
  M_ALLOC(m->counts, sizeof(int) * c->n_experts);
  M_ALLOC(m->offsets, sizeof(int) * (c->n_experts + 1));
  M_ALLOC(m->order, A * 4);
  M_ALLOC(m->inv_order, A * 4);
  M_ALLOC(m->n_items, sizeof(int));
  M_ALLOC(m->items, sizeof(int4) * m->max_items);
  M_ALLOC(m->x_sorted, A * c->hidden * 2);
  M_ALLOC(m->act_sorted, A * c->inter * 2);
  M_ALLOC(m->y_sorted, A * c->hidden * 2);
  if (shared_gate_up && shared_down) {
    M_ALLOC(m->sh_act, N * (shared_gate_up->n / 2) * 2);
    M_ALLOC(m->sh_out, N * c->hidden * 2);
  }
  if (ep_mode) {
    M_ALLOC(m->x_all, N * c->hidden * 2);
    M_ALLOC(m->local_idx, A * 4);
    M_ALLOC(m->partial, N * c->hidden * 4);
    M_ALLOC(m->reduced, (size_t)c->max_tokens * c->hidden * 4);
  }
  if (h_bias) {
    M_ALLOC(m->d_bias, sizeof(float) * c->n_experts);
    cudaMemcpy(m->d_bias, h_bias, sizeof(float) * c->n_experts, cudaMemcpyHostToDevice);
  }
#undef M_ALLOC
  *out = m;
  return B200_OK;
}

b200_status b200_moe_forward(b200_moe* m, const void* d_x, int32_t n_tokens, void* d_out, void* stream) {
  const b200_moe_config& c = m->cfg;
  if (c.ep_world >= 1) { b200_set_error("moe: a layer built for expert parallelism runs through b200_moe_forward_ep"); return B200_ERR_INVALID_ARGUMENT; }
  if (n_tokens > c.max_tokens) { b200_set_error("moe: %d tokens > max_tokens %d", n_tokens, c.max_tokens); return B200_ERR_CAPACITY; }
  if (n_tokens <= 0) return B200_OK;
  const int A = n_tokens * c.top_k;
  b200_status st;
#define STEP(call) do { if ((st = (call)) != B200_OK) return st; } while (0)
  if (m->sh_gu) {  // shared expert on every token (deepseek_v4.zig:1017-1022, 489-517)
    STEP(b200_qmm(m->sh_gu, d_x, n_tokens, m->sh_act, B200_EPI_SWIGLU, nullptr, c.shared_swiglu_limit, B200_QMM_AUTO, stream));
    STEP(b200_qmm(m->sh_down, m->sh_act, n_tokens, m->sh_out, B200_EPI_NONE, nullptr, 0.f, B200_QMM_AUTO, stream));
  }
  STEP(b200_qmm(m->gate, d_x, n_tokens, m->logits, B200_EPI_NONE, nullptr, 0.f, B200_QMM_AUTO, stream));
  STEP(b200_moe_route(m->logits, 0, m->d_bias, n_tokens, c.n_experts, c.top_k, c.scoring, c.route_scale, m->indices,
                      m->weights, m->counts, stream));
  STEP(b200_moe_group(m->indices, m->counts, n_tokens, c.top_k, c.n_experts, c.tile_rows, m->offsets, m->order,
                      m->inv_order, m->items, m->n_items, stream));
  // gate/up with clipped SwiGLU and the routing score folded in before the down projection (:787-805)
  if (b200_qmm_grouped_takes_tokens(m->exp_gu, c.tile_rows)) {
    // the block-scaled path re-encodes every activation row anyway: it reads the rows from the token
    // matrix through `order`, and no expert-sorted bf16 copy is made
    row_scales_kernel<<<(A + 255) / 256, 256, 0, (cudaStream_t)stream>>>(m->order, m->weights, A, m->row_scales, nullptr);
    B200_LAUNCH_CHECK();
    STEP(b200_qmm_grouped_from_tokens(m->exp_gu, d_x, m->order, c.top_k, A, m->act_sorted, B200_EPI_SWIGLU, m->row_scales,
                                      c.swiglu_limit, m->items, m->n_items, m->max_items, c.tile_rows, stream));
  } else {
    STEP(b200_moe_gather(d_x, m->order, m->weights, A, c.top_k, c.hidden, m->x_sorted, m->row_scales, stream));
    STEP(b200_qmm_grouped(m->exp_gu, m->x_sorted, A, m->act_sorted, B200_EPI_SWIGLU, m->row_scales, c.swiglu_limit, m->items,
                          m->n_items, m->max_items, c.tile_rows, stream));
  }
  STEP(b200_qmm_grouped(m->exp_down, m->act_sorted, A, m->y_sorted, B200_EPI_NONE, nullptr, 0.f, m->items, m->n_items,
                        m->max_items, c.tile_rows, stream));
  STEP(b200_moe_combine(m->y_sorted, m->inv_order, n_tokens, c.top_k, c.hidden, m->sh_out, d_out, stream));
#undef STEP
  return B200_OK;
}

// The same layer with the routed experts sharded over the ranks of `ep` (no reference counterpart: the
// reference keeps every expert on one device and streams them from SSD, src/models/expert_stream.zig).
// DSV4SwitchGLU is cut where its two argsorts sit (src/models/deepseek_v4.zig:747-784 sort by expert,
// :809-819 unsort and sum over k):
//   dispatch  all-gather of the token rows, so that every rank holds the tokens of all ranks; every rank
//             routes all of them (the router is replicated and deterministic, so all ranks agree) and
//             keeps the assignments that fall on its own experts.  With top-6 of 8 ranks a token is
//             needed by most ranks anyway: the all-gather moves (W-1)/W of the rows, a selective
//             exchange 1-(1-1/W)^k of them, and nothing has to be counted on the host first.
//   experts   stable grouping by local expert, grouped gate/up (clipped SwiGLU x routing weight) and
//             down matmuls on the rows that exist (the count stays on the device).
//   combine   each rank sums, per token, the outputs of its own experts in f32; a reduce-scatter adds
//             the ranks' shares and leaves every rank with the sums of its own tokens; the shared expert
//             (computed on the rank's own tokens) is added last.
// Two collectives per layer, no host synchronisation, every rank passes the same n_tokens.
b200_status b200_moe_forward_ep(b200_moe* m, b200_ep* ep, const void* d_x, int32_t n_tokens, void* d_out, void* stream) {
  const b200_moe_config& c = m->cfg;
  const int world = c.ep_world;
  if (world < 1 || !ep || b200_ep_world(ep) != world || b200_ep_rank(ep) != c.ep_rank) {
    b200_set_error("moe: this layer was not built for expert parallelism on this communicator");
    return B200_ERR_INVALID_ARGUMENT;
  }
  if (n_tokens > c.max_tokens) { b200_set_error("moe: %d tokens > max_tokens %d", n_tokens, c.max_tokens); return B200_ERR_CAPACITY; }
  if (n_tokens <= 0) return B200_OK;
  const int N = n_tokens * world, A = N * c.top_k;
  cudaStream_t s = (cudaStream_t)stream;
  b200_status st;
#define STEP(call) do { if ((st = (call)) != B200_OK) return st; } while (0)
  STEP(b200_ep_dispatch(ep, d_x, m->x_all, n_tokens, c.hidden, stream));
  if (m->sh_gu) {  // shared expert on the rank's own tokens
    STEP(b200_qmm(m->sh_gu, d_x, n_tokens, m->sh_act, B200_EPI_SWIGLU, nullptr, c.shared_swiglu_limit, B200_QMM_AUTO, stream));
    STEP(b200_qmm(m->sh_down, m->sh_act, n_tokens, m->sh_out, B200_EPI_NONE, nullptr, 0.f, B200_QMM_AUTO, stream));
  }
  STEP(b200_qmm(m->gate, m->x_all, N, m->logits, B200_EPI_NONE, nullptr, 0.f, B200_QMM_AUTO, stream));
  STEP(b200_moe_route(m->logits, 0, m->d_bias, N, c.n_experts, c.top_k, c.scoring, c.route_scale, m->indices, m->weights,
                      m->counts, stream));
  STEP(b200_ep_plan(m->indices, m->counts, N, c.top_k, c.n_experts, c.ep_rank, world, c.tile_rows, m->local_idx, m->offsets,
                    m->order, m->inv_order, m->items, m->n_items, stream));
  const int* rows_valid = m->offsets + m->n_local;  // assignments served here
  row_scales_kernel<<<(A + 255) / 256, 256, 0, s>>>(m->order, m->weights, A, m->row_scales, rows_valid);
  B200_LAUNCH_CHECK();
  if (b200_qmm_grouped_takes_tokens(m->exp_gu, c.tile_rows)) {
    STEP(b200_qmm_grouped_from_tokens(m->exp_gu, m->x_all, m->order, c.top_k, A, m->act_sorted, B200_EPI_SWIGLU, m->row_scales,
                                      c.swiglu_limit, m->items, m->n_items, m->max_items, c.tile_rows, stream, rows_valid));
  } else {
    gather_sorted_kernel<<<A, 128, 0, s>>>(m->x_all, m->order, m->weights, c.top_k, c.hidden, m->x_sorted, nullptr, rows_valid);
    B200_LAUNCH_CHECK();
    STEP(b200_qmm_grouped(m->exp_gu, m->x_sorted, A, m->act_sorted, B200_EPI_SWIGLU, m->row_scales, c.swiglu_limit, m->items,
                          m->n_items, m->max_items, c.tile_rows, stream));
  }
  STEP(b200_qmm_grouped(m->exp_down, m->act_sorted, A, m->y_sorted, B200_EPI_NONE, nullptr, 0.f, m->items, m->n_items,
                        m->max_items, c.tile_rows, stream));
  combine_partial_kernel<<<N, 256, 0, s>>>(m->y_sorted, m->inv_order, c.top_k, c.hidden, m->partial);
  B200_LAUNCH_CHECK();
  STEP(b200_ep_combine(ep, m->partial, m->reduced, n_tokens, c.hidden, stream));
  const size_t n8 = (size_t)n_tokens * c.hidden / 8;
  add_shared_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, s>>>(m->reduced, m->sh_out, n8, (__nv_bfloat16*)d_out);
  B200_LAUNCH_CHECK();
#undef STEP
  return B200_OK;
}

// Routing results of the last forward (tests): indices [N,k] u32, weights [N,k] f32, offsets [E+1].
b200_status b200_moe_last_routing(b200_moe* m, int32_t n_tokens, uint32_t* h_indices, float* h_weights, int32_t* h_offsets) {
  const size_t A = (size_t)n_tokens * m->cfg.top_k;
  B200_CUDA_TRY(cudaMemcpy(h_indices, m->indices, A * 4, cudaMemcpyDeviceToHost));
  B200_CUDA_TRY(cudaMemcpy(h_weights, m->weights, A * 4, cudaMemcpyDeviceToHost));
  const int n_off = (m->cfg.ep_world >= 1 ? m->n_local : m->cfg.n_experts) + 1;  // expert parallel: this rank's experts
  B200_CUDA_TRY(cudaMemcpy(h_offsets, m->offsets, sizeof(int) * n_off, cudaMemcpyDeviceToHost));
  return B200_OK;
}

}  // extern "C"
