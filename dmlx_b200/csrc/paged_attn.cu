// Split-K GQA paged-attention decode over ragged contexts, reading KV pages in place.
//
// Work decomposition: a row (one query token of one sequence) is cut into chunks of
// `pages_per_chunk` pages; a work item is (chunk, kv head) and serves the 4 query heads of that
// kv head's group.  A persistent grid (a multiple of the SM count) walks the items round-robin.
// Inside a CTA, warp 0 also acts as producer: it stages each page's K tile and V tile
// (32 tokens x head_dim, contiguous in the pool) into shared memory with one bulk-async (TMA)
// copy each, NSTAGE pages ahead across item boundaries, completion signalled on mbarriers.
// The 4 warps split the 32 tokens of a page; within a warp each half-warp owns one token per
// pass and each lane head_dim/16 dims, so a K or V row is read from shared memory as one 16-byte
// (bf16) vector per lane.  Scores are reduced with warp shuffles, softmax is online in base-2
// units, partial (max, sum, out) per item go to a scratch buffer and a second kernel merges the
// chunks of each row.
//
// HBM traffic per item is exactly the K and V tiles of its pages (plus 16 bytes of page ids per
// 4 pages); nothing is re-read.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include <algorithm>

#include "common.h"
#include "kv_pool.cuh"
#include "ptx.cuh"

namespace {

constexpr int kAttnThreads = 128;
constexpr int kStages = 4;
constexpr int kGroup = 4;       // query heads per kv head
constexpr int kMaxChunkPages = 32;

struct AttnArgs {
  KvDev d;
  int layer;
  const __nv_bfloat16* q;
  const int* row_seq;
  const int* row_ctx;
  const int* chunk_start;  // [T+1]
  int total_rows;
  int n_q_heads;
  int pages_per_chunk;
  float* part_o;
  float* part_ml;
  float scale_log2;
};

__global__ void attn_plan_kernel(const int* __restrict__ row_ctx, int total_rows, int page_size, int pages_per_chunk,
                                 int* __restrict__ chunk_start, int max_chunks, int* __restrict__ err) {
  __shared__ int warp_sums[32];
  __shared__ int carry;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) carry = 0;
  __syncthreads();
  for (int base = 0; base < total_rows; base += blockDim.x) {
    int i = base + tid;
    int v = 0;
    if (i < total_rows) {
      int pages = (max(row_ctx[i], 0) + page_size - 1) / page_size;
      v = (pages + pages_per_chunk - 1) / pages_per_chunk;
    }
    int inc = v;
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
    int ex = carry + warp_sums[warp] + inc - v;
    if (i < total_rows) chunk_start[i] = ex;
    __syncthreads();
    if (tid == blockDim.x - 1) carry = ex + v;
    __syncthreads();
  }
  if (tid == 0) {
    // More chunks than the scratch holds: flag the step and leave no work behind.
    if (carry > max_chunks) { *err = B200_ERR_CAPACITY; chunk_start[total_rows] = 0; }
    else chunk_start[total_rows] = carry;
  }
}

struct Item {
  int row, head, seq, ctx, page_begin, page_end, chunk;
};

__device__ __forceinline__ Item decode_item(const AttnArgs& a, int item) {
  Item it;
  const int H = a.d.n_kv_heads;
  it.chunk = item / H;
  it.head = item - it.chunk * H;
  int lo = 0, hi = a.total_rows - 1;  // last row with chunk_start[row] <= chunk
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (a.chunk_start[mid] <= it.chunk) lo = mid; else hi = mid - 1;
  }
  it.row = lo;
  it.seq = a.row_seq[lo];
  it.ctx = a.row_ctx[lo];
  int c = it.chunk - a.chunk_start[lo];
  int npages = (it.ctx + a.d.page_size - 1) / a.d.page_size;
  it.page_begin = c * a.pages_per_chunk;
  it.page_end = min(it.page_begin + a.pages_per_chunk, npages);
  return it;
}

template <int D, bool FP8>
__global__ void __launch_bounds__(kAttnThreads, 3) paged_attn_kernel(AttnArgs a) {
  constexpr int ELEM = FP8 ? 1 : 2;
  constexpr int TILE = 32 * D * ELEM;  // bytes of one (page, kv head) K or V tile
  constexpr int VEC = D / 16;          // dims per lane
  constexpr int DV = D / 32;           // output dims per thread in the item epilogue

  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* tiles = smem;  // [kStages][2][TILE]
  float* red_o = reinterpret_cast<float*>(smem + kStages * 2 * TILE);  // [4 warps][kGroup][D]
  float* red_ml = red_o + 4 * kGroup * D;                              // [4 warps][kGroup][2]
  float* stage_scale = red_ml + 4 * kGroup * 2;                        // [kStages][2]
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(stage_scale + kStages * 2);
  uint64_t* empty_bar = full_bar + kStages;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int half = lane >> 4, l16 = lane & 15;
  const int H = a.d.n_kv_heads;
  const int n_items = a.chunk_start[a.total_rows] * H;
  int* err = a.d.state + ST_ATTN_ERR;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 4);
    }
    ptx::mbar_fence_init();
  }
  __syncthreads();

  // ---- producer state (meaningful in warp 0 only) ----
  int p_item = blockIdx.x;
  int p_page = 0, p_end = 0, p_head = 0;
  int p_pid = 0;           // lane j: physical page id of page (p_begin + j) of the producer's item
  float p_ks = 1.f, p_vs = 1.f;
  int p_begin = 0;
  uint32_t prod_n = 0;
  auto producer_enter_item = [&]() {
    if (p_item < n_items) {
      Item it = decode_item(a, p_item);
      p_begin = it.page_begin; p_page = it.page_begin; p_end = it.page_end; p_head = it.head;
      int pg = it.page_begin + lane;
      if (pg < it.page_end) {
        p_pid = a.d.block_table[(size_t)it.seq * a.d.max_pages_per_seq + pg];
        if (FP8) {
          size_t ti = ((size_t)a.layer * a.d.n_pages + p_pid) * H + it.head;
          p_ks = a.d.k_scale[ti];
          p_vs = a.d.v_scale[ti];
        }
      }
    }
  };
  // Issues the loads of the producer's next page; returns false on a timed-out wait.
  auto produce_one = [&]() -> bool {
    if (p_item >= n_items) return true;
    const int src_lane = p_page - p_begin;
    const int pid = __shfl_sync(0xffffffffu, p_pid, src_lane);
    const float ks = __shfl_sync(0xffffffffu, p_ks, src_lane);
    const float vs = __shfl_sync(0xffffffffu, p_vs, src_lane);
    const uint32_t s = prod_n % kStages;
    bool ok = true;
    if (lane == 0) {
      ok = ptx::mbar_wait(&empty_bar[s], ((prod_n / kStages) & 1u) ^ 1u);
      if (ok) {
        size_t tile_idx = ((size_t)a.layer * a.d.n_pages + pid) * H + p_head;
        const unsigned char* ksrc = (const unsigned char*)a.d.k_pool + tile_idx * TILE;
        const unsigned char* vsrc = (const unsigned char*)a.d.v_pool + tile_idx * TILE;
        if (FP8) { stage_scale[s * 2] = ks; stage_scale[s * 2 + 1] = vs; }
        ptx::mbar_expect_tx(&full_bar[s], 2 * TILE);
        ptx::bulk_g2s(tiles + (size_t)s * 2 * TILE, ksrc, TILE, &full_bar[s]);
        ptx::bulk_g2s(tiles + (size_t)s * 2 * TILE + TILE, vsrc, TILE, &full_bar[s]);
      }
    }
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    prod_n += 1;
    p_page += 1;
    if (p_page >= p_end) {
      p_item += gridDim.x;
      producer_enter_item();
    }
    return ok;
  };

  bool alive = true;
  if (warp == 0) {
    producer_enter_item();
    for (int i = 0; i < kStages - 1 && alive; ++i) alive = produce_one();
  }
  alive = !__syncthreads_or(!alive);

  uint32_t cons_n = 0;
  for (int item = blockIdx.x; item < n_items && alive; item += gridDim.x) {
    const Item it = decode_item(a, item);
    // query fragment: 4 heads x VEC dims, pre-scaled to base-2 logits
    float q[kGroup][VEC];
#pragma unroll
    for (int h = 0; h < kGroup; ++h) {
      const __nv_bfloat16* qp = a.q + ((size_t)it.row * a.n_q_heads + it.head * kGroup + h) * D + l16 * VEC;
#pragma unroll
      for (int i = 0; i < VEC; ++i) q[h][i] = __bfloat162float(qp[i]) * a.scale_log2;
    }
    float m[kGroup], l[kGroup], o[kGroup][VEC];
#pragma unroll
    for (int h = 0; h < kGroup; ++h) {
      m[h] = -1e30f; l[h] = 0.f;
#pragma unroll
      for (int i = 0; i < VEC; ++i) o[h][i] = 0.f;
    }

    for (int pg = it.page_begin; pg < it.page_end; ++pg) {
      if (warp == 0) alive = produce_one();
      const uint32_t s = cons_n % kStages;
      if (alive) alive = ptx::mbar_wait(&full_bar[s], (cons_n / kStages) & 1u);
      if (!alive) break;
      const unsigned char* kt = tiles + (size_t)s * 2 * TILE;
      const unsigned char* vt = kt + TILE;
      float ks = 1.f, vs = 1.f;
      if (FP8) { ks = stage_scale[s * 2]; vs = stage_scale[s * 2 + 1]; }
      const int tok0 = pg * 32;
#pragma unroll
      for (int pass = 0; pass < 4; ++pass) {
        const int tok = warp * 8 + pass * 2 + half;
        float kf[VEC], vf[VEC];
        if constexpr (FP8) {
          // VEC bytes per lane
          const unsigned char* kp = kt + tok * D + l16 * VEC;
          const unsigned char* vp = vt + tok * D + l16 * VEC;
#pragma unroll
          for (int i = 0; i < VEC; i += 2) {
            __half2_raw hk = __nv_cvt_fp8x2_to_halfraw2(*reinterpret_cast<const __nv_fp8x2_storage_t*>(kp + i), __NV_E4M3);
            __half2_raw hv = __nv_cvt_fp8x2_to_halfraw2(*reinterpret_cast<const __nv_fp8x2_storage_t*>(vp + i), __NV_E4M3);
            float2 fk = __half22float2(__half2(hk)), fv = __half22float2(__half2(hv));
            kf[i] = fk.x; kf[i + 1] = fk.y; vf[i] = fv.x; vf[i + 1] = fv.y;
          }
        } else {
          const uint32_t* kp = reinterpret_cast<const uint32_t*>(kt + (tok * D + l16 * VEC) * 2);
          const uint32_t* vp = reinterpret_cast<const uint32_t*>(vt + (tok * D + l16 * VEC) * 2);
          if constexpr (VEC == 8) {
            const uint4 kw = *reinterpret_cast<const uint4*>(kp), vw = *reinterpret_cast<const uint4*>(vp);
            const uint32_t kk[4] = {kw.x, kw.y, kw.z, kw.w}, vv[4] = {vw.x, vw.y, vw.z, vw.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              kf[2 * i] = ptx::bf16_lo(kk[i]); kf[2 * i + 1] = ptx::bf16_hi(kk[i]);
              vf[2 * i] = ptx::bf16_lo(vv[i]); vf[2 * i + 1] = ptx::bf16_hi(vv[i]);
            }
          } else {
            const uint2 kw = *reinterpret_cast<const uint2*>(kp), vw = *reinterpret_cast<const uint2*>(vp);
            kf[0] = ptx::bf16_lo(kw.x); kf[1] = ptx::bf16_hi(kw.x); kf[2] = ptx::bf16_lo(kw.y); kf[3] = ptx::bf16_hi(kw.y);
            vf[0] = ptx::bf16_lo(vw.x); vf[1] = ptx::bf16_hi(vw.x); vf[2] = ptx::bf16_lo(vw.y); vf[3] = ptx::bf16_hi(vw.y);
          }
        }
        float sc[kGroup];
#pragma unroll
        for (int h = 0; h < kGroup; ++h) {
          float acc = 0.f;
#pragma unroll
          for (int i = 0; i < VEC; ++i) acc = fmaf(q[h][i], kf[i], acc);
          sc[h] = acc;
        }
#pragma unroll
        for (int off = 8; off > 0; off >>= 1) {
#pragma unroll
          for (int h = 0; h < kGroup; ++h) sc[h] += __shfl_xor_sync(0xffffffffu, sc[h], off);
        }
        if (tok0 + tok < it.ctx) {  // uniform per half-warp
#pragma unroll
          for (int h = 0; h < kGroup; ++h) {
            const float sv = sc[h] * ks;
            const float m_new = fmaxf(m[h], sv);
            const float corr = exp2f(m[h] - m_new);
            const float p = exp2f(sv - m_new);
            l[h] = l[h] * corr + p;
            m[h] = m_new;
            const float pv = p * vs;
#pragma unroll
            for (int i = 0; i < VEC; ++i) o[h][i] = fmaf(o[h][i], corr, pv * vf[i]);
          }
        }
      }
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&empty_bar[s]);
      cons_n += 1;
    }
    if (__syncthreads_or(!alive)) { alive = false; break; }

    // ---- merge the two half-warps (same dims, different tokens) ----
#pragma unroll
    for (int h = 0; h < kGroup; ++h) {
      const float m_o = __shfl_xor_sync(0xffffffffu, m[h], 16);
      const float l_o = __shfl_xor_sync(0xffffffffu, l[h], 16);
      const float m_new = fmaxf(m[h], m_o);
      const float ca = exp2f(m[h] - m_new), cb = exp2f(m_o - m_new);
      l[h] = l[h] * ca + l_o * cb;
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const float o_o = __shfl_xor_sync(0xffffffffu, o[h][i], 16);
        o[h][i] = o[h][i] * ca + o_o * cb;
      }
      m[h] = m_new;
    }
    if (half == 0) {
#pragma unroll
      for (int h = 0; h < kGroup; ++h) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) red_o[(warp * kGroup + h) * D + l16 * VEC + i] = o[h][i];
        if (l16 == 0) { red_ml[(warp * kGroup + h) * 2] = m[h]; red_ml[(warp * kGroup + h) * 2 + 1] = l[h]; }
      }
    }
    __syncthreads();
    // ---- merge the 4 warps; thread -> (head, DV dims) ----
    {
      const int h = tid / 32, d0 = (tid % 32) * DV;
      float mm = -1e30f;
#pragma unroll
      for (int w = 0; w < 4; ++w) mm = fmaxf(mm, red_ml[(w * kGroup + h) * 2]);
      float ll = 0.f, acc[DV];
#pragma unroll
      for (int i = 0; i < DV; ++i) acc[i] = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float c = exp2f(red_ml[(w * kGroup + h) * 2] - mm);
        ll += red_ml[(w * kGroup + h) * 2 + 1] * c;
#pragma unroll
        for (int i = 0; i < DV; ++i) acc[i] += red_o[(w * kGroup + h) * D + d0 + i] * c;
      }
      const size_t pidx = (size_t)it.chunk * a.n_q_heads + it.head * kGroup + h;
#pragma unroll
      for (int i = 0; i < DV; ++i) a.part_o[pidx * D + d0 + i] = acc[i];
      if ((tid % 32) == 0) { a.part_ml[pidx * 2] = mm; a.part_ml[pidx * 2 + 1] = ll; }
    }
    __syncthreads();
  }
  if (!alive && tid == 0) atomicExch(err, B200_ERR_DEVICE_FLAGGED);
}

// One warp per (row, query head): merge the row's chunks and write bf16.
template <int D>
__global__ void attn_combine_kernel(AttnArgs a, __nv_bfloat16* __restrict__ out) {
  constexpr int DV = D / 32;
  const int warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp_global >= a.total_rows * a.n_q_heads || a.d.state[ST_ATTN_ERR] != 0) return;
  const int row = warp_global / a.n_q_heads, qh = warp_global - row * a.n_q_heads;
  const int c0 = a.chunk_start[row], c1 = a.chunk_start[row + 1];
  float mm = -1e30f;
  for (int c = c0; c < c1; ++c) mm = fmaxf(mm, a.part_ml[((size_t)c * a.n_q_heads + qh) * 2]);
  float ll = 0.f, acc[DV];
#pragma unroll
  for (int i = 0; i < DV; ++i) acc[i] = 0.f;
  for (int c = c0; c < c1; ++c) {
    const size_t pidx = (size_t)c * a.n_q_heads + qh;
    const float w = exp2f(a.part_ml[pidx * 2] - mm);
    ll += a.part_ml[pidx * 2 + 1] * w;
#pragma unroll
    for (int i = 0; i < DV; ++i) acc[i] += a.part_o[pidx * D + lane * DV + i] * w;
  }
  const float inv = ll > 0.f ? 1.0f / ll : 0.f;
#pragma unroll
  for (int i = 0; i < DV; ++i) out[((size_t)row * a.n_q_heads + qh) * D + lane * DV + i] = __float2bfloat16(acc[i] * inv);
}

template <int D, bool FP8>
size_t attn_smem_bytes() {
  size_t tile = 32 * D * (FP8 ? 1 : 2);
  return kStages * 2 * tile + sizeof(float) * (4 * kGroup * D + 4 * kGroup * 2 + kStages * 2) + sizeof(uint64_t) * 2 * kStages;
}

template <int D, bool FP8>
b200_status launch_attn(const AttnArgs& a, void* d_out, int grid, cudaStream_t s) {
  size_t smem = attn_smem_bytes<D, FP8>();
  static bool configured = false;
  if (!configured) {
    B200_CUDA_TRY(cudaFuncSetAttribute(paged_attn_kernel<D, FP8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  paged_attn_kernel<D, FP8><<<grid, kAttnThreads, smem, s>>>(a);
  B200_LAUNCH_CHECK();
  int warps = a.total_rows * a.n_q_heads;
  attn_combine_kernel<D><<<(warps * 32 + 255) / 256, 256, 0, s>>>(a, (__nv_bfloat16*)d_out);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

int g_sm_count = 0;

}  // namespace

// Pages per chunk chosen so that the persistent grid sees several items per CTA without making
// the per-item partials a visible share of the traffic.
int b200_attn_pages_per_chunk = 8;

extern "C" b200_status b200_paged_attn_decode(b200_kv* kv, int32_t layer, const void* d_q, const int32_t* d_row_seq,
                                              const int32_t* d_row_ctx, int32_t total_rows, void* d_out, void* stream) {
  b200_status st = b200_require_device();
  if (st != B200_OK) return st;
  const b200_kv_config& c = kv->cfg;
  if (layer < 0 || layer >= c.n_layers) { b200_set_error("attention: layer %d out of range", layer); return B200_ERR_INVALID_ARGUMENT; }
  if (c.n_q_heads != c.n_kv_heads * kGroup) {
    b200_set_error("attention: only a GQA group of %d query heads per kv head is built (got %d/%d)", kGroup, c.n_q_heads, c.n_kv_heads);
    return B200_ERR_UNSUPPORTED;
  }
  if (total_rows <= 0) return B200_OK;
  if (total_rows > c.max_rows) { b200_set_error("attention: %d rows > max_rows %d", total_rows, c.max_rows); return B200_ERR_CAPACITY; }
  cudaStream_t s = (cudaStream_t)stream;
  if (g_sm_count == 0) {
    int dev = 0;
    B200_CUDA_TRY(cudaGetDevice(&dev));
    B200_CUDA_TRY(cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev));
  }
  int ppc = std::min(std::max(b200_attn_pages_per_chunk, 1), kMaxChunkPages);
  // scratch bound: chunks <= pages/ppc + rows; kv->max_chunks was sized for ppc >= 4
  if (ppc < 4) ppc = 4;
  AttnArgs a;
  a.d = kv->dev; a.layer = layer; a.q = (const __nv_bfloat16*)d_q; a.row_seq = d_row_seq; a.row_ctx = d_row_ctx;
  a.chunk_start = kv->d_chunk_start; a.total_rows = total_rows; a.n_q_heads = c.n_q_heads; a.pages_per_chunk = ppc;
  a.part_o = kv->d_part_o; a.part_ml = kv->d_part_ml;
  a.scale_log2 = 1.4426950408889634f / sqrtf((float)c.head_dim);
  attn_plan_kernel<<<1, 1024, 0, s>>>(d_row_ctx, total_rows, c.page_size, ppc, kv->d_chunk_start, kv->max_chunks,
                                      kv->dev.state + ST_ATTN_ERR);
  B200_LAUNCH_CHECK();
  const int grid = g_sm_count * 3;
  const bool fp8 = c.kv_dtype == B200_KV_FP8_E4M3;
  if (c.head_dim == 128) return fp8 ? launch_attn<128, true>(a, d_out, grid, s) : launch_attn<128, false>(a, d_out, grid, s);
  return fp8 ? launch_attn<64, true>(a, d_out, grid, s) : launch_attn<64, false>(a, d_out, grid, s);
}

// Tuning hook (not part of the reference surface): pages per split-K chunk, 4..32.
extern "C" void b200_set_attn_pages_per_chunk(int32_t n) { b200_attn_pages_per_chunk = n; }
