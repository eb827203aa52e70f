// Device page pool for the Paged KV strategy.
//
// Layout in HBM (per pool):
//   k_pool, v_pool : [layer][page][kv_head][32 tokens][head_dim]   bf16 or E4M3 bytes
//                    -> one (page, kv_head) tile is 32*head_dim contiguous elements (8 KiB for
//                       bf16 at head_dim 128), the unit the attention kernel stages with one bulk
//                       copy.
//   k_scale,v_scale: [layer][page][kv_head] f32 (FP8 pools only)
//   free_stack     : [n_pages] i32, entries [0, free_top) are free; free_stack[free_top-1] pops next
//   ref_count, tokens_used : [n_pages] i32
//   block_table    : [max_seqs][max_pages_per_seq] i32 ; seq_pages, seq_len : [max_seqs] i32
//   state          : {free_top, error word, n_touch, n_cow}
// The allocator reproduces the sequential semantics of the reference's LIFO block manager
// (src/kvcache/paged.zig:61-73,116-118,156): within one step, requests take pages in batch order,
// which a single CTA realises with a prefix sum over "pages needed" instead of a loop of pops.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include <vector>

#include "common.h"
#include "kv_pool.cuh"
#include "tma.cuh"

static int g_device_state = -1;  // -1 unknown, 0 none, 1 ok
static int g_bound_device = -1;  // the device this process first used the library on

b200_status b200_require_any_device() {
  if (g_device_state < 0) {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    g_device_state = (e == cudaSuccess && n > 0) ? 1 : 0;
    if (e != cudaSuccess) cudaGetLastError();
  }
  if (g_device_state == 0) {
    b200_set_error("no CUDA device is visible; this library has no CPU fallback");
    return B200_ERR_NO_DEVICE;
  }
  return B200_OK;
}

// The library keeps per-process caches (scratch buffers, shared-memory opt-ins, SM count) that belong
// to one device: the first device a compute entry point runs on is the process's device from then on,
// and a call made with another device current is refused instead of running with the wrong pointers.
b200_status b200_require_device() {
  b200_status st = b200_require_any_device();
  if (st != B200_OK) return st;
  int dev = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  if (g_bound_device < 0) g_bound_device = dev;
  if (dev != g_bound_device) {
    b200_set_error("this process uses the library on device %d, the current device is %d (one device per process)",
                   g_bound_device, dev);
    return B200_ERR_UNSUPPORTED;
  }
  return B200_OK;
}

extern "C" int32_t b200_device_available(void) { return b200_require_any_device() == B200_OK; }

// ---------------------------------------------------------------------------------------------
// kernels
// ---------------------------------------------------------------------------------------------
namespace {

constexpr int kReserveThreads = 1024;
constexpr int kReserveItems = 4;  // requests per thread -> 4096 requests per step

__global__ void init_pool_kernel(KvDev d) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < d.n_pages) {
    d.free_stack[i] = d.n_pages - 1 - i;
    d.ref_count[i] = 0;
    d.tokens_used[i] = 0;
  }
  if (i < d.max_seqs) {
    d.seq_pages[i] = 0;
    d.seq_len[i] = 0;
  }
  if (i == 0) {
    d.state[ST_FREE_TOP] = d.n_pages;
    d.state[ST_ERR] = 0;
    d.state[ST_N_TOUCH] = 0;
    d.state[ST_N_COW] = 0;
    d.state[ST_ATTN_ERR] = 0;
  }
}

// Block-wide exclusive scan of one int per thread (1024 threads); returns the exclusive prefix and
// writes the block total to *total.
__device__ int block_exscan(int v, int* total, int* warp_sums) {
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == 31) warp_sums[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int w = warp_sums[lane];
    int winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int t = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += t;
    }
    warp_sums[lane] = winc - w;  // exclusive
    if (lane == 31) *total = winc;
  }
  __syncthreads();
  int res = warp_sums[warp] + inc - v;
  __syncthreads();
  return res;
}

// One CTA.  See b200_kv_reserve in the header for the contract.
__global__ void __launch_bounds__(kReserveThreads) reserve_kernel(KvDev d, const b200_pack_desc* desc, int n_req) {
  __shared__ int warp_sums[32];
  __shared__ int s_total_need, s_total_touch, s_total_cow, s_total_rows, s_any_cow;
  const int tid = threadIdx.x;
  const int ps = d.page_size;

  int seq[kReserveItems], cnt[kReserveItems], len[kReserveItems], held[kReserveItems];
  int cow[kReserveItems], need[kReserveItems], touch[kReserveItems];
  bool cand = false, bad = false;
#pragma unroll
  for (int k = 0; k < kReserveItems; ++k) {
    int i = tid * kReserveItems + k;
    seq[k] = -1; cnt[k] = 0; len[k] = 0; held[k] = 0; cow[k] = 0; need[k] = 0; touch[k] = 0;
    if (i < n_req) {
      int s = desc[i].seq_slot, n = desc[i].count;
      if (s < 0 || s >= d.max_seqs || n < 0) { bad = true; continue; }
      seq[k] = s; cnt[k] = n;
      len[k] = d.seq_len[s];
      held[k] = d.seq_pages[s];
      if (n > 0) {
        int pages_after = (len[k] + n + ps - 1) / ps;
        if (pages_after > d.max_pages_per_seq) { bad = true; continue; }
        if (len[k] % ps != 0) {
          int last = d.block_table[(size_t)s * d.max_pages_per_seq + len[k] / ps];
          if (d.ref_count[last] > 1) { cow[k] = 1; cand = true; }  // tentative
        }
      }
    }
  }
  if (tid == 0) s_any_cow = 0;
  __syncthreads();
  if (cand) s_any_cow = 1;
  if (__syncthreads_or(bad)) {
    if (tid == 0) { d.state[ST_ERR] = B200_ERR_INVALID_BATCH_INDEX; d.state[ST_N_TOUCH] = 0; d.state[ST_N_COW] = 0; }
    return;
  }
  // Copy-on-write decisions depend on earlier requests of the same step sharing the same page
  // (the first writer copies, the last keeps the original), so they are taken serially — only
  // when some candidate exists, which is rare.
  __shared__ unsigned char s_cow_flag[kReserveThreads * kReserveItems];
  if (s_any_cow) {
#pragma unroll
    for (int k = 0; k < kReserveItems; ++k) s_cow_flag[tid * kReserveItems + k] = (unsigned char)cow[k];
    __syncthreads();
    if (tid == 0) {
      for (int i = 0; i < n_req; ++i) {
        if (!s_cow_flag[i]) continue;
        int s = desc[i].seq_slot;
        int last = d.block_table[(size_t)s * d.max_pages_per_seq + d.seq_len[s] / ps];
        if (d.ref_count[last] > 1) d.ref_count[last] -= 1; else s_cow_flag[i] = 0;
      }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kReserveItems; ++k) cow[k] = s_cow_flag[tid * kReserveItems + k];
  }

  int my_need = 0, my_touch = 0, my_cow = 0, my_rows = 0;
#pragma unroll
  for (int k = 0; k < kReserveItems; ++k) {
    if (seq[k] >= 0 && cnt[k] > 0) {
      int pages_after = (len[k] + cnt[k] + ps - 1) / ps;
      int grow = pages_after - held[k];
      need[k] = cow[k] + (grow > 0 ? grow : 0);
      touch[k] = (len[k] + cnt[k] - 1) / ps - len[k] / ps + 1;
    }
    my_need += need[k]; my_touch += touch[k]; my_cow += cow[k]; my_rows += cnt[k];
  }
  int need_off = block_exscan(my_need, &s_total_need, warp_sums);
  int touch_off = block_exscan(my_touch, &s_total_touch, warp_sums);
  int cow_off = block_exscan(my_cow, &s_total_cow, warp_sums);
  int row_off = block_exscan(my_rows, &s_total_rows, warp_sums);

  const int top = d.state[ST_FREE_TOP];
  if (s_total_need > top || s_total_touch > d.max_touch) {
    // All or nothing: undo the tentative ref-count decrements and flag the step.
#pragma unroll
    for (int k = 0; k < kReserveItems; ++k)
      if (cow[k]) {
        int last = d.block_table[(size_t)seq[k] * d.max_pages_per_seq + len[k] / ps];
        atomicAdd(&d.ref_count[last], 1);
      }
    if (tid == 0) {
      d.state[ST_ERR] = s_total_need > top ? B200_ERR_INSUFFICIENT_BLOCKS : B200_ERR_CAPACITY;
      d.state[ST_N_TOUCH] = 0;
      d.state[ST_N_COW] = 0;
    }
    return;
  }

#pragma unroll
  for (int k = 0; k < kReserveItems; ++k) {
    if (seq[k] < 0 || cnt[k] <= 0) { continue; }
    const int s = seq[k];
    int* table = d.block_table + (size_t)s * d.max_pages_per_seq;
    int pop = need_off;
    if (cow[k]) {
      int idx = len[k] / ps;
      int old = table[idx];
      int nw = d.free_stack[top - 1 - pop++];
      d.ref_count[nw] = 1;
      d.tokens_used[nw] = d.tokens_used[old];
      table[idx] = nw;
      d.cow_list[cow_off] = make_int2(old, nw);
      cow_off += 1;
    }
    int pages_after = (len[k] + cnt[k] + ps - 1) / ps;
    for (int p = held[k]; p < pages_after; ++p) {
      int nw = d.free_stack[top - 1 - pop++];
      d.ref_count[nw] = 1;
      d.tokens_used[nw] = 0;
      table[p] = nw;
    }
    int first_page = len[k] / ps, last_page = (len[k] + cnt[k] - 1) / ps;
    for (int p = first_page; p <= last_page; ++p) {
      int tok_lo = max(p * ps, len[k]), tok_hi = min((p + 1) * ps, len[k] + cnt[k]);
      int page = table[p];
      d.tokens_used[page] = tok_hi - p * ps;
      // {page id, first packed row, rows, slot of the first row within the page}
      d.touch_list[touch_off + (p - first_page)] = make_int4(page, row_off + (tok_lo - len[k]), tok_hi - tok_lo, tok_lo - p * ps);
    }
    if (pages_after > held[k]) d.seq_pages[s] = pages_after;
    d.seq_len[s] = len[k] + cnt[k];
    need_off += need[k]; touch_off += touch[k]; row_off += cnt[k];
  }
  __syncthreads();
  if (tid == 0) {
    d.state[ST_FREE_TOP] = top - s_total_need;
    d.state[ST_N_TOUCH] = s_total_touch;
    d.state[ST_N_COW] = s_total_cow;
  }
}

// Copies every queued CoW page (all layers, K and V, scales for FP8 pools).
__global__ void cow_copy_kernel(KvDev d) {
  const int n_cow = d.state[ST_N_COW];
  const size_t page_bytes = (size_t)d.n_kv_heads * d.page_size * d.head_dim * d.elem_bytes;
  const size_t vecs = page_bytes / 16;
  for (int c = blockIdx.x; c < n_cow; c += gridDim.x) {
    int2 pr = d.cow_list[c];
    int layer = blockIdx.y >> 1, is_v = blockIdx.y & 1;
    char* pool = (char*)(is_v ? d.v_pool : d.k_pool);
    const uint4* src = (const uint4*)(pool + ((size_t)layer * d.n_pages + pr.x) * page_bytes);
    uint4* dst = (uint4*)(pool + ((size_t)layer * d.n_pages + pr.y) * page_bytes);
    for (size_t i = threadIdx.x; i < vecs; i += blockDim.x) dst[i] = src[i];
    if (d.elem_bytes == 1 && threadIdx.x < d.n_kv_heads) {
      float* sc = is_v ? d.v_scale : d.k_scale;
      sc[((size_t)layer * d.n_pages + pr.y) * d.n_kv_heads + threadIdx.x] =
          sc[((size_t)layer * d.n_pages + pr.x) * d.n_kv_heads + threadIdx.x];
    }
  }
}

// bf16 append: one CTA per (page touch, kv head) copies rows into the page tile.
__global__ void append_bf16_kernel(KvDev d, int layer, const __nv_bfloat16* __restrict__ k_rows,
                                   const __nv_bfloat16* __restrict__ v_rows, int k_stride, int v_stride) {
  const int n_touch = d.state[ST_N_TOUCH];
  const int head = blockIdx.y, D = d.head_dim, H = d.n_kv_heads;
  const int vec_per_row = D / 8;
  for (int t = blockIdx.x; t < n_touch; t += gridDim.x) {
    int4 tc = d.touch_list[t];  // page, first row, rows, slot
    size_t tile = (((size_t)layer * d.n_pages + tc.x) * H + head) * (size_t)d.page_size * D;
    uint4* kd = (uint4*)((__nv_bfloat16*)d.k_pool + tile + (size_t)tc.w * D);
    uint4* vd = (uint4*)((__nv_bfloat16*)d.v_pool + tile + (size_t)tc.w * D);
    for (int i = threadIdx.x; i < tc.z * vec_per_row; i += blockDim.x) {
      int r = i / vec_per_row, c = i % vec_per_row;
      kd[r * vec_per_row + c] = ((const uint4*)(k_rows + (size_t)(tc.y + r) * k_stride + head * D))[c];
      vd[r * vec_per_row + c] = ((const uint4*)(v_rows + (size_t)(tc.y + r) * v_stride + head * D))[c];
    }
  }
}

// bf16 pools inside the model step: RoPE on q (in place) and k, and the append of the rotated k and
// of v into their pages, in one pass over the fused projection output.  CTA (row, y) takes heads
// 8y..8y+7 of a packed row, one per warp; lane l the rotation pairs (2l, 2l+1) of a head (non-traditional RoPE:
// pair (i, i + D/2) rotates by pos * theta^(-2i/D)), so sin/cos are computed once per thread.
// The page comes from the block table that b200_kv_reserve has just grown.
__global__ void __launch_bounds__(256) rope_append_bf16_kernel(KvDev d, int layer, __nv_bfloat16* __restrict__ q,
                                                               const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                                               int q_stride, int k_stride, int v_stride,
                                                               const int* __restrict__ positions, const int* __restrict__ row_seq, int hq,
                                                               float log2_theta) {
  const int row = blockIdx.x, D = d.head_dim, H = d.n_kv_heads, half = D / 2;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pos = positions[row], seq = row_seq[row];
  const int page_idx = pos / d.page_size, slot = pos - page_idx * d.page_size;
  // a step whose reservation failed has no page for this row: nothing is written (the error word is set)
  const bool have_page = seq >= 0 && seq < d.max_seqs && page_idx < d.seq_pages[seq];
  const int page = have_page ? d.block_table[(size_t)seq * d.max_pages_per_seq + page_idx] : 0;
  const int ppt = half / 32;  // rotation pairs per lane: 1 (D = 64) or 2 (D = 128)
  float sn[2], cs[2];
  for (int j = 0; j < ppt; ++j) {
    const int i = lane * ppt + j;
    sincosf((float)pos * exp2f(-log2_theta * (2.0f * i) / (float)D), &sn[j], &cs[j]);
  }
  for (int h = blockIdx.y * 8 + warp; h < hq + H; h += 8 * gridDim.y) {
    const bool is_q = h < hq;
    const __nv_bfloat16* src = is_q ? q + (size_t)row * q_stride + (size_t)h * D : k + (size_t)row * k_stride + (size_t)(h - hq) * D;
    __nv_bfloat16* dst = nullptr;
    if (is_q) dst = q + (size_t)row * q_stride + (size_t)h * D;
    else if (have_page)
      dst = (__nv_bfloat16*)d.k_pool + ((((size_t)layer * d.n_pages + page) * H + (h - hq)) * d.page_size + slot) * (size_t)D;
    float lo[2], hi[2];
    for (int j = 0; j < ppt; ++j) {
      const int i = lane * ppt + j;
      const float x1 = __bfloat162float(src[i]), x2 = __bfloat162float(src[i + half]);
      lo[j] = x1 * cs[j] - x2 * sn[j];
      hi[j] = x1 * sn[j] + x2 * cs[j];
    }
    if (dst) {
      for (int j = 0; j < ppt; ++j) {
        const int i = lane * ppt + j;
        dst[i] = __float2bfloat16(lo[j]);
        dst[i + half] = __float2bfloat16(hi[j]);
      }
    }
  }
  if (have_page && blockIdx.y == 0) {
    const int vec_per_head = D / 8;
    for (int i = threadIdx.x; i < H * vec_per_head; i += blockDim.x) {
      const int head = i / vec_per_head, c = i - head * vec_per_head;
      uint4* vd = (uint4*)((__nv_bfloat16*)d.v_pool + ((((size_t)layer * d.n_pages + page) * H + head) * d.page_size + slot) * (size_t)D);
      vd[c] = ((const uint4*)(v + (size_t)row * v_stride + (size_t)head * D))[c];
    }
  }
}

__device__ __forceinline__ unsigned char to_e4m3(float x) {
  return (unsigned char)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ float from_e4m3(unsigned char b) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(b, __NV_E4M3);
  return __half2float(__half(h));
}

// FP8 append: per (touch, head, K|V): new scale = max(old, amax(new rows)/448); when it grows the
// rows already in the tile are re-encoded at the new scale; then the new rows are encoded.
__global__ void append_fp8_kernel(KvDev d, int layer, const __nv_bfloat16* __restrict__ k_rows,
                                  const __nv_bfloat16* __restrict__ v_rows, int k_stride, int v_stride) {
  __shared__ float s_red[32];
  __shared__ float s_scale[2];
  const int n_touch = d.state[ST_N_TOUCH];
  const int head = blockIdx.y, D = d.head_dim, H = d.n_kv_heads;
  const int is_v = blockIdx.z;
  const __nv_bfloat16* rows = is_v ? v_rows : k_rows;
  const int stride = is_v ? v_stride : k_stride;
  unsigned char* pool = (unsigned char*)(is_v ? d.v_pool : d.k_pool);
  float* scales = is_v ? d.v_scale : d.k_scale;
  for (int t = blockIdx.x; t < n_touch; t += gridDim.x) {
    int4 tc = d.touch_list[t];
    size_t tile_idx = ((size_t)layer * d.n_pages + tc.x) * H + head;
    unsigned char* tile = pool + tile_idx * (size_t)d.page_size * D;
    float amax = 0.f;
    for (int i = threadIdx.x; i < tc.z * D; i += blockDim.x) {
      int r = i / D, c = i % D;
      amax = fmaxf(amax, fabsf(__bfloat162float(rows[(size_t)(tc.y + r) * stride + head * D + c])));
    }
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
      float m = 0.f;
      for (int w = 0; w < (blockDim.x + 31) / 32; ++w) m = fmaxf(m, s_red[w]);
      m = fmaxf(m, 1e-12f);
      float s_new = m / 448.0f;
      float s_old = tc.w > 0 ? scales[tile_idx] : 0.f;
      s_scale[0] = s_old;
      s_scale[1] = (tc.w > 0 && s_new <= s_old) ? s_old : s_new;
    }
    __syncthreads();
    const float s_old = s_scale[0], s_new = s_scale[1];
    if (tc.w > 0 && s_new > s_old) {
      const float ratio = s_old / s_new;
      for (int i = threadIdx.x; i < tc.w * D; i += blockDim.x) tile[i] = to_e4m3(from_e4m3(tile[i]) * ratio);
    }
    const float inv = 1.0f / s_new;
    for (int i = threadIdx.x; i < tc.z * D; i += blockDim.x) {
      int r = i / D, c = i % D;
      float x = __bfloat162float(rows[(size_t)(tc.y + r) * stride + head * D + c]);
      tile[(size_t)(tc.w + r) * D + c] = to_e4m3(x * inv);
    }
    if (threadIdx.x == 0) scales[tile_idx] = s_new;
    __syncthreads();
  }
}

// Test helper: contiguous [len, H, D] bf16 view of one sequence of one layer.
__global__ void gather_kernel(KvDev d, int layer, int seq, __nv_bfloat16* k_out, __nv_bfloat16* v_out, int cap_rows) {
  const int len = min(d.seq_len[seq], cap_rows);
  const int D = d.head_dim, H = d.n_kv_heads;
  const size_t total = (size_t)len * H * D;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    int c = i % D, h = (i / D) % H, t = i / ((size_t)D * H);
    int page = d.block_table[(size_t)seq * d.max_pages_per_seq + t / d.page_size];
    size_t tile_idx = ((size_t)layer * d.n_pages + page) * H + h;
    size_t off = tile_idx * (size_t)d.page_size * D + (size_t)(t % d.page_size) * D + c;
    if (d.elem_bytes == 2) {
      k_out[i] = ((const __nv_bfloat16*)d.k_pool)[off];
      v_out[i] = ((const __nv_bfloat16*)d.v_pool)[off];
    } else {
      k_out[i] = __float2bfloat16(from_e4m3(((const unsigned char*)d.k_pool)[off]) * d.k_scale[tile_idx]);
      v_out[i] = __float2bfloat16(from_e4m3(((const unsigned char*)d.v_pool)[off]) * d.v_scale[tile_idx]);
    }
  }
}

// ---- administrative operations: one thread, sequential semantics --------------------------------
enum { OP_ALLOC = 0, OP_RELEASE = 1, OP_FORK = 2, OP_ROLLBACK = 3, OP_SET_FREE = 4, OP_SET_LEN = 5 };

__device__ void release_page(KvDev& d, int page) {
  if (d.ref_count[page] > 1) {
    d.ref_count[page] -= 1;
  } else {
    d.ref_count[page] = 0;
    d.tokens_used[page] = 0;
    d.free_stack[d.state[ST_FREE_TOP]++] = page;
  }
}

// args: op-specific; `list` is a device array (sequence slots, or page ids); out: device ints.
__global__ void admin_kernel(KvDev d, int op, int a0, int a1, int a2, const int* list, int* out) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  out[0] = B200_OK;
  switch (op) {
    case OP_ALLOC: {  // a0 = seq, a1 = n  -> out[1..n]
      int s = a0, n = a1;
      if (s < 0 || s >= d.max_seqs) { out[0] = B200_ERR_INVALID_BATCH_INDEX; return; }
      if (d.state[ST_FREE_TOP] < n) { out[0] = B200_ERR_INSUFFICIENT_BLOCKS; return; }
      if (d.seq_pages[s] + n > d.max_pages_per_seq) { out[0] = B200_ERR_CAPACITY; return; }
      for (int i = 0; i < n; ++i) {
        int page = d.free_stack[--d.state[ST_FREE_TOP]];
        d.ref_count[page] = 1;
        d.tokens_used[page] = 0;
        d.block_table[(size_t)s * d.max_pages_per_seq + d.seq_pages[s]++] = page;
        out[1 + i] = page;
      }
      break;
    }
    case OP_RELEASE: {  // a0 = n seqs in list
      for (int i = 0; i < a0; ++i) {
        int s = list[i];
        if (s < 0 || s >= d.max_seqs) { out[0] = B200_ERR_INVALID_BATCH_INDEX; continue; }
        for (int p = 0; p < d.seq_pages[s]; ++p) release_page(d, d.block_table[(size_t)s * d.max_pages_per_seq + p]);
        d.seq_pages[s] = 0;
        d.seq_len[s] = 0;
      }
      break;
    }
    case OP_FORK: {  // a0 = src, a1 = dst, a2 = n_tokens
      int src = a0, dst = a1, nt = a2;
      if (src < 0 || src >= d.max_seqs || dst < 0 || dst >= d.max_seqs || src == dst) { out[0] = B200_ERR_INVALID_BATCH_INDEX; return; }
      if (d.seq_pages[dst] != 0 || nt > d.seq_len[src] || nt < 0) { out[0] = B200_ERR_INVALID_ARGUMENT; return; }
      int np = (nt + d.page_size - 1) / d.page_size;
      for (int p = 0; p < np; ++p) {
        int page = d.block_table[(size_t)src * d.max_pages_per_seq + p];
        d.ref_count[page] += 1;
        d.block_table[(size_t)dst * d.max_pages_per_seq + p] = page;
      }
      d.seq_pages[dst] = np;
      d.seq_len[dst] = nt;
      break;
    }
    case OP_ROLLBACK: {  // a0 = seq, a1 = to_len
      int s = a0;
      if (s < 0 || s >= d.max_seqs) { out[0] = B200_ERR_INVALID_BATCH_INDEX; return; }
      int need = (a1 + d.page_size - 1) / d.page_size;
      while (d.seq_pages[s] > need) release_page(d, d.block_table[(size_t)s * d.max_pages_per_seq + --d.seq_pages[s]]);
      if (d.seq_len[s] > a1) d.seq_len[s] = a1;
      break;
    }
    case OP_SET_LEN: {  // a0 = seq, a1 = tokens now held by the sequence's pages (restored from outside)
      int s = a0, n = a1;
      if (s < 0 || s >= d.max_seqs) { out[0] = B200_ERR_INVALID_BATCH_INDEX; return; }
      if (n < 0 || (n + d.page_size - 1) / d.page_size > d.seq_pages[s]) { out[0] = B200_ERR_INVALID_ARGUMENT; return; }
      d.seq_len[s] = n;
      for (int p = 0; p < d.seq_pages[s]; ++p) {
        int page = d.block_table[(size_t)s * d.max_pages_per_seq + p];
        int used = n - p * d.page_size;
        d.tokens_used[page] = used < 0 ? 0 : (used > d.page_size ? d.page_size : used);
      }
      break;
    }
    case OP_SET_FREE: {  // a0 = n ids in list, popped list[0] first; only on an untouched pool
      if (d.state[ST_FREE_TOP] != d.n_pages || a0 != d.n_pages) { out[0] = B200_ERR_INVALID_ARGUMENT; return; }
      for (int i = 0; i < a0; ++i) d.free_stack[d.n_pages - 1 - i] = list[i];
      break;
    }
  }
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// host API
// ---------------------------------------------------------------------------------------------
static b200_status run_admin(b200_kv* kv, int op, int a0, int a1, int a2, const int* h_list, int n_list,
                             int* h_out, int n_out) {
  if (n_list > kv->admin_cap || n_out + 1 > kv->admin_cap) {
    b200_set_error("admin operation larger than the %d-entry staging buffer", kv->admin_cap);
    return B200_ERR_CAPACITY;
  }
  if (n_list > 0) B200_CUDA_TRY(cudaMemcpy(kv->d_admin_in, h_list, sizeof(int) * n_list, cudaMemcpyHostToDevice));
  admin_kernel<<<1, 32>>>(kv->dev, op, a0, a1, a2, kv->d_admin_in, kv->d_admin_out);
  B200_LAUNCH_CHECK();
  std::vector<int> out(n_out + 1);
  B200_CUDA_TRY(cudaMemcpy(out.data(), kv->d_admin_out, sizeof(int) * (n_out + 1), cudaMemcpyDeviceToHost));
  for (int i = 0; i < n_out; ++i) h_out[i] = out[1 + i];
  if (out[0] != B200_OK) b200_set_error("device pool operation %d failed: %s", op, b200_status_name(out[0]));
  return out[0];
}

extern "C" {

b200_status b200_kv_create(const b200_kv_config* c, b200_kv** out) {
  *out = nullptr;
  b200_status st = b200_require_device();
  if (st != B200_OK) return st;
  if (c->page_size != 32) { b200_set_error("page_size must be 32"); return B200_ERR_INVALID_ARGUMENT; }
  if (c->kv_dtype != B200_KV_BF16 && c->kv_dtype != B200_KV_FP8_E4M3) {
    b200_set_error("kv_dtype %d: only bf16 (0) and FP8-E4M3 (1) pages exist", c->kv_dtype);
    return B200_ERR_INVALID_QUANT_BITS;
  }
  if (c->head_dim != 64 && c->head_dim != 128) { b200_set_error("head_dim must be 64 or 128"); return B200_ERR_INVALID_ARGUMENT; }
  if (c->n_layers <= 0 || c->n_kv_heads <= 0 || c->n_pages <= 0 || c->max_seqs <= 0 || c->max_pages_per_seq <= 0 ||
      c->max_rows <= 0 || c->n_q_heads <= 0 || c->n_q_heads % c->n_kv_heads != 0) {
    b200_set_error("invalid pool configuration");
    return B200_ERR_INVALID_ARGUMENT;
  }
  auto* kv = new b200_kv();
  kv->cfg = *c;
  KvDev& d = kv->dev;
  d.n_layers = c->n_layers; d.n_kv_heads = c->n_kv_heads; d.head_dim = c->head_dim; d.page_size = c->page_size;
  d.n_pages = c->n_pages; d.max_seqs = c->max_seqs; d.max_pages_per_seq = c->max_pages_per_seq;
  d.elem_bytes = c->kv_dtype == B200_KV_BF16 ? 2 : 1;
  d.max_touch = std::max(c->max_rows, c->n_pages + c->max_seqs);  // a bulk fill may touch every page
  size_t pool_bytes = (size_t)c->n_layers * c->n_pages * c->n_kv_heads * c->page_size * c->head_dim * d.elem_bytes;
  size_t n_tiles = (size_t)c->n_layers * c->n_pages * c->n_kv_heads;
#define KV_ALLOC(ptr, bytes)                                            \
  do {                                                                  \
    cudaError_t e_ = cudaMalloc((void**)&(ptr), (bytes));               \
    if (e_ != cudaSuccess) {                                            \
      b200_set_error("cudaMalloc(%zu) failed: %s", (size_t)(bytes), cudaGetErrorString(e_)); \
      b200_kv_destroy(kv);                                              \
      return B200_ERR_CUDA;                                             \
    }                                                                   \
  } while (0)
  KV_ALLOC(d.k_pool, pool_bytes);
  KV_ALLOC(d.v_pool, pool_bytes);
  if (d.elem_bytes == 1) {
    KV_ALLOC(d.k_scale, n_tiles * sizeof(float));
    KV_ALLOC(d.v_scale, n_tiles * sizeof(float));
  }
  KV_ALLOC(d.free_stack, sizeof(int) * c->n_pages);
  KV_ALLOC(d.ref_count, sizeof(int) * c->n_pages);
  KV_ALLOC(d.tokens_used, sizeof(int) * c->n_pages);
  KV_ALLOC(d.block_table, sizeof(int) * (size_t)c->max_seqs * c->max_pages_per_seq);
  KV_ALLOC(d.seq_pages, sizeof(int) * c->max_seqs);
  KV_ALLOC(d.seq_len, sizeof(int) * c->max_seqs);
  KV_ALLOC(d.state, sizeof(int) * 8);
  KV_ALLOC(d.touch_list, sizeof(int4) * d.max_touch);
  KV_ALLOC(d.cow_list, sizeof(int2) * c->max_seqs);
  kv->admin_cap = std::max(c->n_pages, c->max_seqs) + 8;
  KV_ALLOC(kv->d_admin_in, sizeof(int) * kv->admin_cap);
  KV_ALLOC(kv->d_admin_out, sizeof(int) * kv->admin_cap);
  // split-K scratch for the attention kernel
  kv->max_chunks = c->attn_scratch_chunks > 0 ? c->attn_scratch_chunks : c->n_pages / 4 + c->max_rows + 8;
  KV_ALLOC(kv->d_chunk_start, sizeof(int) * (c->max_rows + 2));
  KV_ALLOC(kv->d_groups, sizeof(int) * 3 * (c->max_rows + 2));
  KV_ALLOC(kv->d_part_o, sizeof(float) * (size_t)kv->max_chunks * c->n_q_heads * c->head_dim);
  KV_ALLOC(kv->d_part_ml, sizeof(float) * (size_t)kv->max_chunks * c->n_q_heads * 2);
#undef KV_ALLOC
  cudaMemset(d.block_table, 0, sizeof(int) * (size_t)c->max_seqs * c->max_pages_per_seq);
  // Pages start zeroed so that slots never written hold finite values: attention multiplies
  // masked slots by a zero weight instead of branching around them.
  cudaMemset(d.k_pool, 0, pool_bytes);
  cudaMemset(d.v_pool, 0, pool_bytes);
  if (d.elem_bytes == 2) {
    const uint64_t rows_per_layer = (uint64_t)c->n_pages * c->n_kv_heads * c->page_size;
    const uint64_t dims[3] = {(uint64_t)c->head_dim, rows_per_layer, (uint64_t)c->n_layers};
    const uint64_t strides[2] = {(uint64_t)c->head_dim * 2, rows_per_layer * c->head_dim * 2};
    const uint32_t box[3] = {64, 32, 1};
    st = b200_make_tensor_map(&kv->kmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, d.k_pool, dims, strides, box);
    if (st == B200_OK) st = b200_make_tensor_map(&kv->vmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, d.v_pool, dims, strides, box);
    if (st != B200_OK) { b200_kv_destroy(kv); return st; }
  } else if (c->head_dim == 128) {
    // FP8 pools: a token row of one head is 128 bytes, a page tile one 128 x 32 box
    const uint64_t rows_per_layer = (uint64_t)c->n_pages * c->n_kv_heads * c->page_size;
    const uint64_t dims[3] = {128, rows_per_layer, (uint64_t)c->n_layers};
    const uint64_t strides[2] = {128, rows_per_layer * 128};
    const uint32_t box[3] = {128, 32, 1};
    st = b200_make_tensor_map(&kv->kmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, d.k_pool, dims, strides, box);
    if (st == B200_OK) st = b200_make_tensor_map(&kv->vmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, d.v_pool, dims, strides, box);
    if (st != B200_OK) { b200_kv_destroy(kv); return st; }
  }
  st = b200_kv_reset(kv);
  if (st != B200_OK) { b200_kv_destroy(kv); return st; }
  *out = kv;
  return B200_OK;
}

void b200_kv_destroy(b200_kv* kv) {
  if (!kv) return;
  KvDev& d = kv->dev;
  void* ptrs[] = {d.k_pool, d.v_pool, d.k_scale, d.v_scale, d.free_stack, d.ref_count, d.tokens_used, d.block_table,
                  d.seq_pages, d.seq_len, d.state, d.touch_list, d.cow_list, kv->d_admin_in, kv->d_admin_out,
                  kv->d_chunk_start, kv->d_part_o, kv->d_part_ml, kv->d_groups};
  for (void* p : ptrs) if (p) cudaFree(p);
  delete kv;
}

b200_status b200_kv_dims(const b200_kv* kv, int32_t* n_pages, int32_t* max_seqs) {
  *n_pages = kv->cfg.n_pages;
  *max_seqs = kv->cfg.max_seqs;
  return B200_OK;
}

b200_status b200_kv_limits(const b200_kv* kv, int32_t* max_pages_per_seq, int32_t* page_size) {
  *max_pages_per_seq = kv->cfg.max_pages_per_seq;
  *page_size = kv->cfg.page_size;
  return B200_OK;
}

b200_status b200_kv_reset(b200_kv* kv) {
  int n = std::max(kv->cfg.n_pages, kv->cfg.max_seqs);
  init_pool_kernel<<<(n + 255) / 256, 256>>>(kv->dev);
  B200_LAUNCH_CHECK();
  B200_CUDA_TRY(cudaDeviceSynchronize());
  return B200_OK;
}

b200_status b200_kv_set_free_order(b200_kv* kv, const int32_t* ids, int32_t n) {
  return run_admin(kv, OP_SET_FREE, n, 0, 0, ids, n, nullptr, 0);
}

b200_status b200_kv_free_count(b200_kv* kv, int32_t* out) {
  B200_CUDA_TRY(cudaMemcpy(out, kv->dev.state + ST_FREE_TOP, sizeof(int), cudaMemcpyDeviceToHost));
  return B200_OK;
}

b200_status b200_kv_alloc(b200_kv* kv, int32_t seq, int32_t n, int32_t* out_ids) {
  return run_admin(kv, OP_ALLOC, seq, n, 0, nullptr, 0, out_ids, n);
}
b200_status b200_kv_release(b200_kv* kv, const int32_t* seqs, int32_t n) {
  return run_admin(kv, OP_RELEASE, n, 0, 0, seqs, n, nullptr, 0);
}
b200_status b200_kv_fork(b200_kv* kv, int32_t src, int32_t dst, int32_t n_tokens) {
  return run_admin(kv, OP_FORK, src, dst, n_tokens, nullptr, 0, nullptr, 0);
}
b200_status b200_kv_set_len(b200_kv* kv, int32_t seq, int32_t n_tokens) {
  return run_admin(kv, OP_SET_LEN, seq, n_tokens, 0, nullptr, 0, nullptr, 0);
}
b200_status b200_kv_rollback(b200_kv* kv, int32_t seq, int32_t to_len) {
  return run_admin(kv, OP_ROLLBACK, seq, to_len, 0, nullptr, 0, nullptr, 0);
}
b200_status b200_kv_filter(b200_kv* kv, const int32_t* keep, int32_t n_keep) {
  std::vector<char> kept(kv->cfg.max_seqs, 0);
  for (int i = 0; i < n_keep; ++i) {
    if (keep[i] < 0 || keep[i] >= kv->cfg.max_seqs) {
      b200_set_error("filter: slot %d out of range", keep[i]);
      return B200_ERR_INVALID_BATCH_INDEX;
    }
    kept[keep[i]] = 1;
  }
  std::vector<int> drop;
  for (int s = 0; s < kv->cfg.max_seqs; ++s) if (!kept[s]) drop.push_back(s);
  if (drop.empty()) return B200_OK;
  return b200_kv_release(kv, drop.data(), (int)drop.size());
}

b200_status b200_kv_reserve(b200_kv* kv, const b200_pack_desc* d_desc, int32_t n_req, void* stream) {
  if (n_req < 0 || n_req > kReserveThreads * kReserveItems) {
    b200_set_error("reserve: %d requests in one step (limit %d)", n_req, kReserveThreads * kReserveItems);
    return B200_ERR_INVALID_ARGUMENT;
  }
  cudaStream_t s = (cudaStream_t)stream;
  reserve_kernel<<<1, kReserveThreads, 0, s>>>(kv->dev, d_desc, n_req);
  B200_LAUNCH_CHECK();
  dim3 grid(std::min(kv->cfg.max_seqs, 256), kv->cfg.n_layers * 2);
  cow_copy_kernel<<<grid, 256, 0, s>>>(kv->dev);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

b200_status b200_kv_append(b200_kv* kv, int32_t layer, const void* d_k_rows, const void* d_v_rows,
                           int32_t total_rows, void* stream) {
  const int stride = kv->cfg.n_kv_heads * kv->cfg.head_dim;
  return b200_kv_append_strided(kv, layer, d_k_rows, d_v_rows, stride, stride, total_rows, stream);
}

}  // extern "C"

b200_status b200_kv_append_strided(b200_kv* kv, int32_t layer, const void* d_k_rows, const void* d_v_rows,
                                   int32_t k_stride, int32_t v_stride, int32_t total_rows, void* stream) {
  if (layer < 0 || layer >= kv->cfg.n_layers) { b200_set_error("append: layer %d out of range", layer); return B200_ERR_INVALID_ARGUMENT; }
  if (total_rows <= 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  int gx = std::min(total_rows, 2048);
  if (kv->cfg.kv_dtype == B200_KV_BF16) {
    append_bf16_kernel<<<dim3(gx, kv->cfg.n_kv_heads), 128, 0, s>>>(kv->dev, layer, (const __nv_bfloat16*)d_k_rows,
                                                                    (const __nv_bfloat16*)d_v_rows, k_stride, v_stride);
  } else {
    append_fp8_kernel<<<dim3(gx, kv->cfg.n_kv_heads, 2), 128, 0, s>>>(kv->dev, layer, (const __nv_bfloat16*)d_k_rows,
                                                                      (const __nv_bfloat16*)d_v_rows, k_stride, v_stride);
  }
  B200_LAUNCH_CHECK();
  return B200_OK;
}

// The same on contiguous q [T, n_q_heads, D] and k/v [T, n_kv_heads, D] rows (the exported form).
extern "C" b200_status b200_kv_rope_append(b200_kv* kv, int32_t layer, void* d_q, void* d_k_rows, const void* d_v_rows,
                                           const int32_t* d_positions, const int32_t* d_row_seq, int32_t total_rows,
                                           int32_t n_q_heads, float theta, void* stream) {
  const int q_stride = n_q_heads * kv->cfg.head_dim, kv_stride = kv->cfg.n_kv_heads * kv->cfg.head_dim;
  return b200_kv_rope_append_strided(kv, layer, d_q, d_k_rows, d_v_rows, q_stride, kv_stride, kv_stride, d_positions, d_row_seq,
                                     total_rows, n_q_heads, theta, stream);
}

// RoPE + append fed from the split-K partial sums of the fused q/k/v projection (head_dim 128 = one 128-row weight
// tile per head).  One warp per (row, head): the lane's four columns (two rotation pairs) are summed over the splits
// in split order and rounded to bf16 as the matmul's finish pass would have done, then rotated and stored: q into the
// activation buffer, k and v into the row's page.
__global__ void __launch_bounds__(256) rope_append_partials_bf16_kernel(KvDev d, int layer, b200_qmm_partials p, __nv_bfloat16* __restrict__ q,
                                                                        int q_stride, const int* __restrict__ positions,
                                                                        const int* __restrict__ row_seq, int hq, float log2_theta) {
  constexpr int D = 128, half = 64;
  const int row = blockIdx.x, H = d.n_kv_heads;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pos = positions[row], seq = row_seq[row];
  const int page_idx = pos / d.page_size, slot = pos - page_idx * d.page_size;
  // a step whose reservation failed has no page for this row: nothing is written (the error word is set)
  const bool have_page = seq >= 0 && seq < d.max_seqs && page_idx < d.seq_pages[seq];
  const int page = have_page ? d.block_table[(size_t)seq * d.max_pages_per_seq + page_idx] : 0;
  const int tt = row / p.tn, tr = row - tt * p.tn;
  const size_t split_stride = (size_t)p.tn * 128;
  for (int h = blockIdx.y * 8 + warp; h < hq + 2 * H; h += 8 * gridDim.y) {
    const float* base = p.d_ws + (((size_t)(h * p.tts + tt) * p.splits) * p.tn + tr) * 128;
    if (h < hq + H) {
      // columns 2*lane, 2*lane+1 and their partners 64 further on
      float2 lo = make_float2(0.f, 0.f), hi = make_float2(0.f, 0.f);
      for (int s = 0; s < p.splits; ++s) {
        const float2 a = *reinterpret_cast<const float2*>(base + (size_t)s * split_stride + 2 * lane);
        const float2 b = *reinterpret_cast<const float2*>(base + (size_t)s * split_stride + half + 2 * lane);
        lo.x += a.x; lo.y += a.y; hi.x += b.x; hi.y += b.y;
      }
      const float x1[2] = {__bfloat162float(__float2bfloat16(lo.x)), __bfloat162float(__float2bfloat16(lo.y))};
      const float x2[2] = {__bfloat162float(__float2bfloat16(hi.x)), __bfloat162float(__float2bfloat16(hi.y))};
      __nv_bfloat16* dst = nullptr;
      if (h < hq) dst = q + (size_t)row * q_stride + (size_t)h * D;
      else if (have_page)
        dst = (__nv_bfloat16*)d.k_pool + ((((size_t)layer * d.n_pages + page) * H + (h - hq)) * d.page_size + slot) * (size_t)D;
      float o1[2], o2[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int i = lane * 2 + j;
        float sn, cs;
        sincosf((float)pos * exp2f(-log2_theta * (2.0f * i) / (float)D), &sn, &cs);
        o1[j] = x1[j] * cs - x2[j] * sn;
        o2[j] = x1[j] * sn + x2[j] * cs;
      }
      if (dst) {
        *reinterpret_cast<__nv_bfloat162*>(dst + 2 * lane) = __floats2bfloat162_rn(o1[0], o1[1]);
        *reinterpret_cast<__nv_bfloat162*>(dst + half + 2 * lane) = __floats2bfloat162_rn(o2[0], o2[1]);
      }
    } else {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int s = 0; s < p.splits; ++s) {
        const float4 a = *reinterpret_cast<const float4*>(base + (size_t)s * split_stride + 4 * lane);
        acc.x += a.x; acc.y += a.y; acc.z += a.z; acc.w += a.w;
      }
      if (have_page) {
        __nv_bfloat16* dst = (__nv_bfloat16*)d.v_pool + ((((size_t)layer * d.n_pages + page) * H + (h - hq - H)) * d.page_size + slot) * (size_t)D;
        const __nv_bfloat162 a0 = __floats2bfloat162_rn(acc.x, acc.y), a1 = __floats2bfloat162_rn(acc.z, acc.w);
        *reinterpret_cast<uint2*>(dst + 4 * lane) = make_uint2(*reinterpret_cast<const uint32_t*>(&a0), *reinterpret_cast<const uint32_t*>(&a1));
      }
    }
  }
}

extern "C" b200_status b200_kv_rope_append_partials(b200_kv* kv, int32_t layer, const b200_qmm_partials* parts, void* d_q, int32_t q_stride,
                                                    const int32_t* d_positions, const int32_t* d_row_seq, int32_t total_rows,
                                                    int32_t n_q_heads, float theta, void* stream) {
  const b200_kv_config& c = kv->cfg;
  if (c.kv_dtype != B200_KV_BF16 || c.head_dim != 128) { b200_set_error("rope+append from partial sums: bf16 pools with head_dim 128 only"); return B200_ERR_UNSUPPORTED; }
  if (!parts || !parts->pending || !parts->d_ws || parts->rows != total_rows || parts->n != (n_q_heads + 2 * c.n_kv_heads) * 128 ||
      parts->nt * 128 != parts->n || parts->tn <= 0 || parts->tts != (total_rows + parts->tn - 1) / parts->tn || parts->splits <= 0) {
    b200_set_error("rope+append from partial sums: the partial sums do not describe a q/k/v projection of %d rows", total_rows);
    return B200_ERR_INVALID_ARGUMENT;
  }
  if (layer < 0 || layer >= c.n_layers) { b200_set_error("append: layer %d out of range", layer); return B200_ERR_INVALID_ARGUMENT; }
  if (total_rows <= 0) return B200_OK;
  rope_append_partials_bf16_kernel<<<dim3(total_rows, (n_q_heads + 2 * c.n_kv_heads + 7) / 8), 256, 0, (cudaStream_t)stream>>>(
      kv->dev, layer, *parts, (__nv_bfloat16*)d_q, q_stride, d_positions, d_row_seq, n_q_heads, log2f(theta));
  B200_LAUNCH_CHECK();
  return B200_OK;
}

// RoPE + append for a bf16 pool in one launch (model step); other pools take the two-kernel route.
b200_status b200_kv_rope_append_strided(b200_kv* kv, int32_t layer, void* d_q, const void* d_k_rows, const void* d_v_rows,
                                        int32_t q_stride, int32_t k_stride, int32_t v_stride, const int32_t* d_positions,
                                        const int32_t* d_row_seq, int32_t total_rows, int32_t n_q_heads, float theta, void* stream) {
  const b200_kv_config& c = kv->cfg;
  if (c.kv_dtype != B200_KV_BF16 || (c.head_dim != 64 && c.head_dim != 128)) {
    b200_status st = b200_rope(d_q, const_cast<void*>(d_k_rows), d_positions, total_rows, n_q_heads, c.n_kv_heads, c.head_dim, q_stride,
                               k_stride, theta, stream);
    if (st != B200_OK) return st;
    return b200_kv_append_strided(kv, layer, d_k_rows, d_v_rows, k_stride, v_stride, total_rows, stream);
  }
  if (layer < 0 || layer >= c.n_layers) { b200_set_error("append: layer %d out of range", layer); return B200_ERR_INVALID_ARGUMENT; }
  if (total_rows <= 0) return B200_OK;
  rope_append_bf16_kernel<<<dim3(total_rows, (n_q_heads + c.n_kv_heads + 7) / 8), 256, 0, (cudaStream_t)stream>>>(kv->dev, layer, (__nv_bfloat16*)d_q, (const __nv_bfloat16*)d_k_rows,
                                                                         (const __nv_bfloat16*)d_v_rows, q_stride, k_stride, v_stride,
                                                                         d_positions, d_row_seq, n_q_heads, log2f(theta));
  B200_LAUNCH_CHECK();
  return B200_OK;
}

extern "C" {

b200_status b200_kv_seq_len(b200_kv* kv, int32_t seq, int32_t* out_len) {
  if (seq < 0 || seq >= kv->cfg.max_seqs) { b200_set_error("slot %d out of range", seq); return B200_ERR_INVALID_BATCH_INDEX; }
  B200_CUDA_TRY(cudaMemcpy(out_len, kv->dev.seq_len + seq, sizeof(int), cudaMemcpyDeviceToHost));
  return B200_OK;
}

b200_status b200_kv_current_len(b200_kv* kv, int32_t* out_len) {
  std::vector<int> lens(kv->cfg.max_seqs);
  B200_CUDA_TRY(cudaMemcpy(lens.data(), kv->dev.seq_len, sizeof(int) * lens.size(), cudaMemcpyDeviceToHost));
  int m = 0;
  for (int l : lens) m = std::max(m, l);
  *out_len = m;
  return B200_OK;
}

b200_status b200_kv_block_table(b200_kv* kv, int32_t seq, int32_t* out_ids, int32_t cap, int32_t* out_n_pages) {
  if (seq < 0 || seq >= kv->cfg.max_seqs) { b200_set_error("slot %d out of range", seq); return B200_ERR_INVALID_BATCH_INDEX; }
  int np = 0;
  B200_CUDA_TRY(cudaMemcpy(&np, kv->dev.seq_pages + seq, sizeof(int), cudaMemcpyDeviceToHost));
  *out_n_pages = np;
  if (np > cap) { b200_set_error("block table holds %d pages, out array %d", np, cap); return B200_ERR_CAPACITY; }
  if (np > 0)
    B200_CUDA_TRY(cudaMemcpy(out_ids, kv->dev.block_table + (size_t)seq * kv->cfg.max_pages_per_seq, sizeof(int) * np,
                             cudaMemcpyDeviceToHost));
  return B200_OK;
}

b200_status b200_kv_ref_counts(b200_kv* kv, int32_t* out, int32_t cap) {
  if (cap < kv->cfg.n_pages) { b200_set_error("ref_counts: out array too small"); return B200_ERR_CAPACITY; }
  B200_CUDA_TRY(cudaMemcpy(out, kv->dev.ref_count, sizeof(int) * kv->cfg.n_pages, cudaMemcpyDeviceToHost));
  return B200_OK;
}

b200_status b200_kv_error_word(b200_kv* kv, int32_t* out) {
  int words[4];
  B200_CUDA_TRY(cudaMemcpy(words, kv->dev.state + ST_ERR, sizeof(int) * 4, cudaMemcpyDeviceToHost));
  *out = words[0] != 0 ? words[0] : words[ST_ATTN_ERR - ST_ERR];
  if (words[0] != 0) B200_CUDA_TRY(cudaMemset(kv->dev.state + ST_ERR, 0, sizeof(int)));
  if (words[ST_ATTN_ERR - ST_ERR] != 0) B200_CUDA_TRY(cudaMemset(kv->dev.state + ST_ATTN_ERR, 0, sizeof(int)));
  return B200_OK;
}

b200_status b200_kv_gather(b200_kv* kv, int32_t layer, int32_t seq, void* d_k_out, void* d_v_out, int32_t cap_rows,
                           void* stream) {
  if (layer < 0 || layer >= kv->cfg.n_layers || seq < 0 || seq >= kv->cfg.max_seqs) {
    b200_set_error("gather: layer/slot out of range");
    return B200_ERR_INVALID_BATCH_INDEX;
  }
  gather_kernel<<<296, 256, 0, (cudaStream_t)stream>>>(kv->dev, layer, seq, (__nv_bfloat16*)d_k_out,
                                                       (__nv_bfloat16*)d_v_out, cap_rows);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

b200_status b200_kv_page_load(b200_kv* kv, int32_t layer, int32_t page, const void* h_k, const void* h_v,
                              const float* h_k_scales, const float* h_v_scales) {
  if (layer < 0 || layer >= kv->cfg.n_layers || page < 0 || page >= kv->cfg.n_pages) {
    b200_set_error("page_load: layer/page out of range");
    return B200_ERR_INVALID_BLOCK_ID;
  }
  const KvDev& d = kv->dev;
  if (d.elem_bytes == 1 && (!h_k_scales || !h_v_scales)) { b200_set_error("page_load: FP8 pages need their scales"); return B200_ERR_INVALID_ARGUMENT; }
  size_t page_bytes = (size_t)d.n_kv_heads * d.page_size * d.head_dim * d.elem_bytes;
  size_t off = ((size_t)layer * d.n_pages + page) * page_bytes;
  B200_CUDA_TRY(cudaMemcpy((char*)d.k_pool + off, h_k, page_bytes, cudaMemcpyHostToDevice));
  B200_CUDA_TRY(cudaMemcpy((char*)d.v_pool + off, h_v, page_bytes, cudaMemcpyHostToDevice));
  if (d.elem_bytes == 1) {
    size_t so = ((size_t)layer * d.n_pages + page) * d.n_kv_heads;
    B200_CUDA_TRY(cudaMemcpy(d.k_scale + so, h_k_scales, sizeof(float) * d.n_kv_heads, cudaMemcpyHostToDevice));
    B200_CUDA_TRY(cudaMemcpy(d.v_scale + so, h_v_scales, sizeof(float) * d.n_kv_heads, cudaMemcpyHostToDevice));
  }
  return B200_OK;
}

// extend (src/kvcache/paged.zig:947-1109): a sequence of another pool of the same shape becomes a new
// sequence of this one, with its own copies of the pages.  One launch copies every layer's K and V
// page (and, for FP8 pools, the per-head scales); grid = (pages of the sequence, layers).
__global__ void __launch_bounds__(256) copy_pages_kernel(KvDev src, KvDev dst, const int* __restrict__ src_table,
                                                         const int* __restrict__ dst_table) {
  const int layer = blockIdx.y, sp = src_table[blockIdx.x], dp = dst_table[blockIdx.x];
  if (sp < 0 || sp >= src.n_pages || dp < 0 || dp >= dst.n_pages) return;
  const size_t page_bytes = (size_t)src.n_kv_heads * src.page_size * src.head_dim * src.elem_bytes;  // multiple of 16
  const size_t so = ((size_t)layer * src.n_pages + sp) * page_bytes, dof = ((size_t)layer * dst.n_pages + dp) * page_bytes;
  const uint4* sk = reinterpret_cast<const uint4*>((const char*)src.k_pool + so);
  const uint4* sv = reinterpret_cast<const uint4*>((const char*)src.v_pool + so);
  uint4* dk = reinterpret_cast<uint4*>((char*)dst.k_pool + dof);
  uint4* dv = reinterpret_cast<uint4*>((char*)dst.v_pool + dof);
  for (size_t i = threadIdx.x; i < page_bytes / 16; i += blockDim.x) { dk[i] = sk[i]; dv[i] = sv[i]; }
  if (src.elem_bytes == 1 && threadIdx.x < src.n_kv_heads) {
    const size_t ss = ((size_t)layer * src.n_pages + sp) * src.n_kv_heads + threadIdx.x;
    const size_t ds = ((size_t)layer * dst.n_pages + dp) * dst.n_kv_heads + threadIdx.x;
    dst.k_scale[ds] = src.k_scale[ss];
    dst.v_scale[ds] = src.v_scale[ss];
  }
}

b200_status b200_kv_extend(b200_kv* kv, int32_t dst_seq, b200_kv* src, int32_t src_seq) {
  const b200_kv_config &a = kv->cfg, &b = src->cfg;
  if (a.n_layers != b.n_layers || a.n_kv_heads != b.n_kv_heads || a.head_dim != b.head_dim || a.page_size != b.page_size ||
      a.kv_dtype != b.kv_dtype) {
    b200_set_error("extend: the two pools differ in shape or element type");
    return B200_ERR_INVALID_ARGUMENT;
  }
  if (dst_seq < 0 || dst_seq >= a.max_seqs || src_seq < 0 || src_seq >= b.max_seqs) {
    b200_set_error("extend: slot out of range");
    return B200_ERR_INVALID_BATCH_INDEX;
  }
  int32_t src_len = 0, dst_pages_held = 0, n_src = 0;
  b200_status st = b200_kv_seq_len(src, src_seq, &src_len);
  if (st != B200_OK) return st;
  B200_CUDA_TRY(cudaMemcpy(&dst_pages_held, kv->dev.seq_pages + dst_seq, sizeof(int), cudaMemcpyDeviceToHost));
  if (dst_pages_held != 0) { b200_set_error("extend: destination slot %d is not empty", dst_seq); return B200_ERR_INVALID_ARGUMENT; }
  const int need = (src_len + a.page_size - 1) / a.page_size;
  if (need == 0) return B200_OK;
  if (need > a.max_pages_per_seq) { b200_set_error("extend: %d pages exceed max_pages_per_seq %d", need, a.max_pages_per_seq); return B200_ERR_CAPACITY; }
  std::vector<int32_t> src_ids(b.max_pages_per_seq), dst_ids(need);
  st = b200_kv_block_table(src, src_seq, src_ids.data(), (int32_t)src_ids.size(), &n_src);
  if (st != B200_OK) return st;
  if (n_src < need) { b200_set_error("extend: source holds %d pages for %d tokens", n_src, src_len); return B200_ERR_INVALID_ARGUMENT; }
  st = b200_kv_alloc(kv, dst_seq, need, dst_ids.data());  // InsufficientBlocks when the pool cannot take them
  if (st != B200_OK) return st;
  int* d_ids = nullptr;
  B200_CUDA_TRY(cudaMalloc((void**)&d_ids, sizeof(int) * 2 * need));
  cudaError_t e = cudaMemcpy(d_ids, src_ids.data(), sizeof(int) * need, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(d_ids + need, dst_ids.data(), sizeof(int) * need, cudaMemcpyHostToDevice);
  if (e != cudaSuccess) { cudaFree(d_ids); b200_set_error("extend: %s", cudaGetErrorString(e)); return B200_ERR_CUDA; }
  copy_pages_kernel<<<dim3(need, a.n_layers), 256>>>(src->dev, kv->dev, d_ids, d_ids + need);
  ++g_b200_launch_counter;
  e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  cudaFree(d_ids);
  if (e != cudaSuccess) { b200_set_error("extend: %s", cudaGetErrorString(e)); return B200_ERR_CUDA; }
  return b200_kv_set_len(kv, dst_seq, src_len);
}

b200_status b200_kv_page_raw(b200_kv* kv, int32_t layer, int32_t page, void* h_k, void* h_v, float* h_k_scales,
                             float* h_v_scales) {
  if (layer < 0 || layer >= kv->cfg.n_layers || page < 0 || page >= kv->cfg.n_pages) {
    b200_set_error("page_raw: layer/page out of range");
    return B200_ERR_INVALID_BLOCK_ID;
  }
  const KvDev& d = kv->dev;
  size_t page_bytes = (size_t)d.n_kv_heads * d.page_size * d.head_dim * d.elem_bytes;
  size_t off = ((size_t)layer * d.n_pages + page) * page_bytes;
  B200_CUDA_TRY(cudaMemcpy(h_k, (char*)d.k_pool + off, page_bytes, cudaMemcpyDeviceToHost));
  B200_CUDA_TRY(cudaMemcpy(h_v, (char*)d.v_pool + off, page_bytes, cudaMemcpyDeviceToHost));
  if (d.elem_bytes == 1 && h_k_scales && h_v_scales) {
    size_t so = ((size_t)layer * d.n_pages + page) * d.n_kv_heads;
    B200_CUDA_TRY(cudaMemcpy(h_k_scales, d.k_scale + so, sizeof(float) * d.n_kv_heads, cudaMemcpyDeviceToHost));
    B200_CUDA_TRY(cudaMemcpy(h_v_scales, d.v_scale + so, sizeof(float) * d.n_kv_heads, cudaMemcpyDeviceToHost));
  }
  return B200_OK;
}

}  // extern "C"
