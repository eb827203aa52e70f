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
#include "tma.cuh"

namespace {

constexpr int kAttnThreads = 128;
constexpr int kStages = 4;
constexpr int kGroup = 4;       // query heads per kv head
constexpr int kMaxChunkPages = 32;

struct AttnArgs {
  KvDev d;
  int layer;
  const __nv_bfloat16* q;
  int q_stride;  // elements between consecutive query rows
  const int* row_seq;
  const int* row_ctx;
  const int* chunk_start;  // [T+1]
  int total_rows;
  int n_q_heads;
  int pages_per_chunk;
  float* part_o;
  float* part_ml;
  float scale_log2;
  // prefill path: rows grouped into runs of consecutive tokens of one sequence
  const int* group_first = nullptr;  // [n_groups + 1] first row of each group
  const int* part_base = nullptr;    // [n_groups] first partial slot of each group (a chunk holds one slot per row)
  const int* row_group = nullptr;    // [T]
  const int* n_groups = nullptr;
  int q_tokens = 1;                  // rows per group at most (16 / GQA group size)
  // prefill path with one chunk per group (a chunk long enough for any context): the kernel normalises and writes
  // the rows itself, no partials and no combine pass
  __nv_bfloat16* direct_out = nullptr;
  // decode path: pages per chunk as the plan kernel chose it for this batch (else pages_per_chunk holds it)
  const int* ppc_dev = nullptr;
};

__device__ __forceinline__ int attn_pages_per_chunk(const AttnArgs& a) { return a.ppc_dev ? *a.ppc_dev : a.pages_per_chunk; }

// pages_per_chunk <= 0: the kernel picks the chunk length from the batch's mean context, 8 pages below 96 pages per
// row, 16 below 192, 32 above.  Short chunks give the persistent grid more items to balance; with long contexts the
// partial sums and the combine pass's walk over a row's chunks cost more than the balance gains (256 requests of
// ~47 pages: 12.8 ms per step at 8 pages per chunk against 13.1 at 16; 64 requests of ~250 pages: 0.338 ms per
// launch at 32 against 0.377 at 8).  The choice is written to *ppc_out for the kernels that follow.
__global__ void attn_plan_kernel(const int* __restrict__ row_ctx, int total_rows, int page_size, int pages_per_chunk,
                                 int* __restrict__ chunk_start, int max_chunks, int* __restrict__ err, int* __restrict__ ppc_out) {
  __shared__ int warp_sums[32];
  __shared__ int carry;
  __shared__ int s_ppc;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) carry = 0;
  if (pages_per_chunk <= 0) {
    long long pages = 0;
    for (int i = tid; i < total_rows; i += blockDim.x) pages += (max(row_ctx[i], 0) + page_size - 1) / page_size;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) pages += __shfl_xor_sync(0xffffffffu, pages, o);
    if (lane == 0) warp_sums[warp] = (int)min(pages, (long long)0x7fffffff / 64);
    __syncthreads();
    if (tid == 0) {
      long long total = 0;
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) total += warp_sums[w];
      const long long mean = total / max(total_rows, 1);
      s_ppc = mean < 96 ? 8 : (mean < 192 ? 16 : 32);
    }
  } else if (tid == 0) {
    s_ppc = pages_per_chunk;
  }
  __syncthreads();
  pages_per_chunk = s_ppc;
  if (tid == 0) *ppc_out = pages_per_chunk;
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
  const int ppc = attn_pages_per_chunk(a);
  it.page_begin = c * ppc;
  it.page_end = min(it.page_begin + ppc, npages);
  return it;
}

// One token row segment of a staged tile -> VEC floats (lane l16 owns dims [l16*VEC, l16*VEC+VEC)).
template <int D, bool FP8>
__device__ __forceinline__ void load_row(const unsigned char* tile, int tok, int l16, float (&f)[D / 16]) {
  constexpr int VEC = D / 16;
  if constexpr (FP8) {
    const unsigned char* p = tile + tok * D + l16 * VEC;
    if constexpr (VEC == 8) {
      const uint2 w = *reinterpret_cast<const uint2*>(p);
      const uint32_t ww[2] = {w.x, w.y};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __nv_fp8x2_storage_t pr = (__nv_fp8x2_storage_t)((ww[i >> 1] >> (16 * (i & 1))) & 0xFFFFu);
        const float2 fv = __half22float2(__half2(__nv_cvt_fp8x2_to_halfraw2(pr, __NV_E4M3)));
        f[2 * i] = fv.x; f[2 * i + 1] = fv.y;
      }
    } else {
      const uint32_t w = *reinterpret_cast<const uint32_t*>(p);
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const __nv_fp8x2_storage_t pr = (__nv_fp8x2_storage_t)((w >> (16 * i)) & 0xFFFFu);
        const float2 fv = __half22float2(__half2(__nv_cvt_fp8x2_to_halfraw2(pr, __NV_E4M3)));
        f[2 * i] = fv.x; f[2 * i + 1] = fv.y;
      }
    }
  } else {
    const unsigned char* p = tile + (tok * D + l16 * VEC) * 2;
    if constexpr (VEC == 8) {
      const uint4 w = *reinterpret_cast<const uint4*>(p);
      const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) { f[2 * i] = ptx::bf16_lo(ww[i]); f[2 * i + 1] = ptx::bf16_hi(ww[i]); }
    } else {
      const uint2 w = *reinterpret_cast<const uint2*>(p);
      f[0] = ptx::bf16_lo(w.x); f[1] = ptx::bf16_hi(w.x); f[2] = ptx::bf16_lo(w.y); f[3] = ptx::bf16_hi(w.y);
    }
  }
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
      const __nv_bfloat16* qp = a.q + (size_t)it.row * a.q_stride + (it.head * kGroup + h) * D + l16 * VEC;
#pragma unroll
      for (int i = 0; i < VEC; ++i) q[h][i] = __bfloat162float(qp[i]) * a.scale_log2;
    }
    // Running softmax state of this lane's own head (head = l16 >> 2; the 4 lanes of a
    // (half-warp, head) group hold the same value); accumulators for all 4 heads x VEC dims.
    const int myh = l16 >> 2;
    const bool b3 = (l16 & 8) != 0, b2 = (l16 & 4) != 0;
    float m_run = -1e30f, l_run = 0.f, o[kGroup][VEC];
#pragma unroll
    for (int h = 0; h < kGroup; ++h) {
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
      const bool partial_page = tok0 + 32 > it.ctx;  // uniform across the CTA

      // ---- phase 1: scores of this warp's 8 tokens (4 passes x 2 half-warps) ----
      float sreg[4];
#pragma unroll
      for (int pass = 0; pass < 4; ++pass) {
        const int tok = warp * 8 + pass * 2 + half;
        float kf[VEC];
        load_row<D, FP8>(kt, tok, l16, kf);
        float part[kGroup];
#pragma unroll
        for (int h = 0; h < kGroup; ++h) {
          float acc = 0.f;
#pragma unroll
          for (int i = 0; i < VEC; ++i) acc = fmaf(q[h][i], kf[i], acc);
          part[h] = acc;
        }
        // Transposed butterfly over the 16 lanes of the half-warp: 5 shuffles leave each lane
        // with the full dot product of head (l16 >> 2).
        const float r0 = __shfl_xor_sync(0xffffffffu, b3 ? part[0] : part[2], 8);
        const float r1 = __shfl_xor_sync(0xffffffffu, b3 ? part[1] : part[3], 8);
        const float a0 = (b3 ? part[2] : part[0]) + r0;
        const float a1 = (b3 ? part[3] : part[1]) + r1;
        float sc = (b2 ? a1 : a0) + __shfl_xor_sync(0xffffffffu, b2 ? a0 : a1, 4);
        sc += __shfl_xor_sync(0xffffffffu, sc, 2);
        sc += __shfl_xor_sync(0xffffffffu, sc, 1);
        sreg[pass] = (tok0 + tok < it.ctx) ? sc * ks : -1e30f;
      }
      // ---- one rescale per page ----
      const float mx = fmaxf(fmaxf(sreg[0], sreg[1]), fmaxf(sreg[2], sreg[3]));
      const float m_new = fmaxf(m_run, mx);
      const float corr = exp2f(m_run - m_new);
      float p[4], psum = 0.f;
#pragma unroll
      for (int pass = 0; pass < 4; ++pass) {
        p[pass] = sreg[pass] > -1e29f ? exp2f(sreg[pass] - m_new) : 0.f;
        psum += p[pass];
      }
      l_run = l_run * corr + psum;
      m_run = m_new;
#pragma unroll
      for (int h = 0; h < kGroup; ++h) {
        const float ch = __shfl_sync(0xffffffffu, corr, (lane & 16) + h * 4);
#pragma unroll
        for (int i = 0; i < VEC; ++i) o[h][i] *= ch;
      }
      // ---- phase 2: o += p * v ----
#pragma unroll
      for (int pass = 0; pass < 4; ++pass) {
        const int tok = warp * 8 + pass * 2 + half;
        float vf[VEC];
        load_row<D, FP8>(vt, tok, l16, vf);
        if (partial_page && tok0 + tok >= it.ctx) {  // unused slots of a page may hold anything
#pragma unroll
          for (int i = 0; i < VEC; ++i) vf[i] = 0.f;
        }
        const float pw = p[pass] * vs;
#pragma unroll
        for (int h = 0; h < kGroup; ++h) {
          const float ph = __shfl_sync(0xffffffffu, pw, (lane & 16) + h * 4);
#pragma unroll
          for (int i = 0; i < VEC; ++i) o[h][i] = fmaf(ph, vf[i], o[h][i]);
        }
      }
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&empty_bar[s]);
      cons_n += 1;
    }
    if (__syncthreads_or(!alive)) { alive = false; break; }

    // ---- merge the two half-warps (same dims, different tokens) ----
    {
      const float m_o = __shfl_xor_sync(0xffffffffu, m_run, 16);
      const float l_o = __shfl_xor_sync(0xffffffffu, l_run, 16);
      const float m_new = fmaxf(m_run, m_o);
      const float ca = exp2f(m_run - m_new), cb = exp2f(m_o - m_new);
      l_run = l_run * ca + l_o * cb;
      m_run = m_new;
#pragma unroll
      for (int h = 0; h < kGroup; ++h) {
        const float cah = __shfl_sync(0xffffffffu, ca, (lane & 16) + h * 4);
        const float cbh = __shfl_sync(0xffffffffu, cb, (lane & 16) + h * 4);
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          const float o_o = __shfl_xor_sync(0xffffffffu, o[h][i], 16);
          o[h][i] = o[h][i] * cah + o_o * cbh;
        }
      }
    }
    if (half == 0) {
#pragma unroll
      for (int h = 0; h < kGroup; ++h) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) red_o[(warp * kGroup + h) * D + l16 * VEC + i] = o[h][i];
      }
      if ((l16 & 3) == 0) { red_ml[(warp * kGroup + myh) * 2] = m_run; red_ml[(warp * kGroup + myh) * 2 + 1] = l_run; }
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


// ---------------------------------------------------------------------------------------------
// bf16 pools: tensor-core variant.
//
// The CUDA-core kernel above is bound by instruction issue, not by HBM (an FP8 pool moves half the
// bytes in the same time).  Here every warp is an independent worker: it owns a private ring of
// kMmaStages page slots, walks its own (chunk, kv head) items, and there is no CTA-wide barrier in
// the main loop.  Lane 0 stages a page's K and V tiles with tiled TMA loads through 3-D tensor
// maps over the pool ([layer][page*head*32 rows][head_dim], box 64 x 32, 128B swizzle), so
// ldmatrix reads them without bank conflicts.  S = Q K^T and O += P V run on mma.sync m16n8k16
// (bf16 in, f32 out) with the group's query heads as the 16-row M dimension (rows >= group size
// are zero), the FlashAttention-2 register reuse turns the score fragments into the P operand,
// and softmax is online per page.  Instructions per staged byte drop by about 8x.
constexpr int kMmaWarps = 4;
constexpr int kMmaStages = 3;

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// D(16x8,f32) += A(16x16,bf16; rows 8..15 are zero: a1 = a3 = 0) * B(16x8,bf16)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  const uint32_t z = 0u;
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(z), "r"(a2), "r"(z), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int D>
__global__ void __launch_bounds__(kMmaWarps * 32, 1)
    paged_attn_mma_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap, AttnArgs a) {
  constexpr int BOXES = D / 64;     // 128-byte wide TMA boxes per tile
  constexpr int TILE = 32 * D * 2;  // bytes of one K or V tile
  constexpr int KS = D / 16;        // k-steps of Q K^T
  constexpr int NO = D / 8;         // n-tiles of the output

  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  unsigned char* my_tiles = smem + (size_t)warp * kMmaStages * 2 * TILE;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)kMmaWarps * kMmaStages * 2 * TILE) + warp * kMmaStages;
  const int H = a.d.n_kv_heads, G = a.n_q_heads / H;
  const int n_items = a.chunk_start[a.total_rows] * H;
  const int worker = blockIdx.x * kMmaWarps + warp, n_workers = gridDim.x * kMmaWarps;

  if (lane == 0) {
    for (int s = 0; s < kMmaStages; ++s) ptx::mbar_init(&full_bar[s], 1);
    ptx::mbar_fence_init();
  }
  __syncwarp();

  // ---- producer cursor (all lanes track it; lane 0 issues) ----
  int p_item = worker, p_page = 0, p_end = 0, p_begin = 0, p_head = 0, p_pid = 0;
  uint32_t prod_n = 0;
  auto producer_enter_item = [&]() {
    if (p_item < n_items) {
      const Item it = decode_item(a, p_item);
      p_begin = it.page_begin; p_page = it.page_begin; p_end = it.page_end; p_head = it.head;
      const int pg = it.page_begin + lane;
      if (pg < it.page_end) p_pid = a.d.block_table[(size_t)it.seq * a.d.max_pages_per_seq + pg];
    }
  };
  auto produce_one = [&]() {
    if (p_item >= n_items) return;
    const int pid = __shfl_sync(0xffffffffu, p_pid, p_page - p_begin);
    const uint32_t s = prod_n % kMmaStages;
    if (lane == 0) {
      ptx::fence_proxy_async_smem();
      unsigned char* kd = my_tiles + (size_t)s * 2 * TILE;
      const int row0 = (pid * H + p_head) * 32;
      ptx::mbar_expect_tx(&full_bar[s], 2 * TILE);
#pragma unroll
      for (int b = 0; b < BOXES; ++b) {
        ptx::tma_load_3d(kd + b * 4096, &kmap, b * 64, row0, a.layer, &full_bar[s]);
        ptx::tma_load_3d(kd + TILE + b * 4096, &vmap, b * 64, row0, a.layer, &full_bar[s]);
      }
    }
    prod_n += 1;
    p_page += 1;
    if (p_page >= p_end) {
      p_item += n_workers;
      producer_enter_item();
    }
  };
  producer_enter_item();
  for (int i = 0; i < kMmaStages; ++i) produce_one();

  bool alive = true;
  uint32_t cons_n = 0;
  // per-lane ldmatrix row/chunk selectors
  const int ld_r = lane & 7, ld_m = lane >> 3;
  for (int item = worker; item < n_items && alive; item += n_workers) {
    const Item it = decode_item(a, item);
    // Q fragments: row g = query head g of the group (zero beyond the group size).
    uint32_t qa0[KS], qa2[KS];
    {
      const uint32_t* qrow = reinterpret_cast<const uint32_t*>(a.q + (size_t)it.row * a.q_stride + (it.head * G + (g < G ? g : 0)) * D);
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        qa0[ks] = g < G ? qrow[ks * 8 + t] : 0u;
        qa2[ks] = g < G ? qrow[ks * 8 + 4 + t] : 0u;
      }
    }
    float o[NO][4];
#pragma unroll
    for (int j = 0; j < NO; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    float m_run = -1e30f, l_run = 0.f;

    for (int pg = it.page_begin; pg < it.page_end; ++pg) {
      const uint32_t s = cons_n % kMmaStages;
      alive = ptx::mbar_wait(&full_bar[s], (cons_n / kMmaStages) & 1u);
      if (!alive) break;
      const uint32_t kbase = ptx::smem_u32(my_tiles + (size_t)s * 2 * TILE), vbase = kbase + TILE;
      // ---- S = Q K^T : 4 n-tiles of 8 tokens ----
      float sc[4][4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) { sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f; }
#pragma unroll
      for (int kk = 0; kk < KS / 2; ++kk) {
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          const int row = nt * 8 + ld_r, cc = 4 * kk + ld_m;  // 16-byte chunk index along head_dim
          uint32_t b[4];
          ldsm_x4(kbase + (cc >> 3) * 4096 + row * 128 + (((cc & 7) ^ (row & 7)) << 4), b);
          mma_bf16_16816(sc[nt], qa0[2 * kk], qa2[2 * kk], b[0], b[1]);
          mma_bf16_16816(sc[nt], qa0[2 * kk + 1], qa2[2 * kk + 1], b[2], b[3]);
        }
      }
      // ---- online softmax on row g (lanes of a quad share the row) ----
      const int tok0 = pg * 32;
      float mx = -1e30f;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const bool valid = tok0 + nt * 8 + 2 * t + e < it.ctx;
          sc[nt][e] = valid ? sc[nt][e] * a.scale_log2 : -1e30f;
          mx = fmaxf(mx, sc[nt][e]);
        }
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run, mx);
      const float corr = exp2f(m_run - m_new);
      float psum = 0.f;
      uint32_t pa0[2], pa2[2];
#pragma unroll
      for (int kt = 0; kt < 2; ++kt) {
        float pv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float sv = sc[2 * kt + (e >> 1)][e & 1];
          pv[e] = sv > -1e29f ? exp2f(sv - m_new) : 0.f;
          psum += pv[e];
        }
        pa0[kt] = pack_bf16(pv[0], pv[1]);
        pa2[kt] = pack_bf16(pv[2], pv[3]);
      }
      l_run = l_run * corr + psum;
      m_run = m_new;
      if (__any_sync(0xffffffffu, corr != 1.f)) {
#pragma unroll
        for (int j = 0; j < NO; ++j) { o[j][0] *= corr; o[j][1] *= corr; }
      }
      // ---- O += P V ----
#pragma unroll
      for (int kt = 0; kt < 2; ++kt) {
#pragma unroll
        for (int jj = 0; jj < NO / 2; ++jj) {
          const int row = kt * 16 + (ld_m & 1) * 8 + ld_r, cc = 2 * jj + (ld_m >> 1);
          uint32_t b[4];
          ldsm_x4_trans(vbase + (cc >> 3) * 4096 + row * 128 + (((cc & 7) ^ (row & 7)) << 4), b);
          mma_bf16_16816(o[2 * jj], pa0[kt], pa2[kt], b[0], b[1]);
          mma_bf16_16816(o[2 * jj + 1], pa0[kt], pa2[kt], b[2], b[3]);
        }
      }
      __syncwarp();
      cons_n += 1;
      produce_one();  // refill the slot just drained: kMmaStages - 1 pages stay in flight while one is computed
    }
    if (!alive) break;
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    if (g < G) {
      const size_t pidx = (size_t)it.chunk * a.n_q_heads + it.head * G + g;
#pragma unroll
      for (int j = 0; j < NO; ++j)
        *reinterpret_cast<float2*>(a.part_o + pidx * D + j * 8 + 2 * t) = make_float2(o[j][0], o[j][1]);
      if (t == 0) { a.part_ml[pidx * 2] = m_run; a.part_ml[pidx * 2 + 1] = l_run; }
    }
  }
  if (!alive && lane == 0) atomicExch(a.d.state + ST_ATTN_ERR, B200_ERR_DEVICE_FLAGGED);
}

// ---------------------------------------------------------------------------------------------
// FP8-E4M3 pools (head_dim 128): tensor-core variant.
//
// Same worker structure as above; a page's K or V tile is 32 tokens x 128 bytes = one 4 KiB TMA box
// (128B swizzle).  The E4M3 codes are widened to f16 in registers (exact) and the products run on
// mma.sync m16n8k16 f16 -> f32, with Q converted bf16 -> f16 once per item.
//   * The MMA's K slots are a free permutation as long as both operands agree: ldmatrix on the
//     byte tile hands lane (g, t) the four consecutive dims 16c+4t..16c+4t+3 of token g, which
//     become the lane's four K slots of step c; Q is loaded with the same dim -> slot map.
//   * For P V, ldmatrix.trans hands the lane two tokens x two adjacent dims; a byte permute sorts
//     them into the B operands of an "even dims" and an "odd dims" output tile.
//   * The per-(page, kv head) scales stay out of the MMAs: the K scale multiplies the f32 scores;
//     the V scale, divided by the largest V scale of the item (so the factor is <= 1), multiplies
//     P before it is rounded to f16, and the item's output is multiplied by that largest scale.
__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  const uint32_t z = 0u;
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(z), "r"(a2), "r"(z), "r"(b0), "r"(b1));
}
// two E4M3 codes (low 16 bits: first code in the low byte) -> f16x2
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint32_t lo16) {
  uint32_t d;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(d) : "h"((unsigned short)lo16));
  return d;
}
__device__ __forceinline__ uint32_t pack_f16(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int STAGES, int MINB>
__global__ void __launch_bounds__(kMmaWarps * 32, MINB)
    paged_attn_mma_fp8_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap, AttnArgs a) {
  constexpr int D = 128;
  constexpr int TILE = 32 * D;  // bytes of one K or V tile
  constexpr int KS = D / 16;    // k-steps of Q K^T = 16-byte chunks of a row
  constexpr int NO = D / 8;     // n-tiles of the output

  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  unsigned char* my_tiles = smem + (size_t)warp * STAGES * 2 * TILE;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)kMmaWarps * STAGES * 2 * TILE) + warp * STAGES;
  const int H = a.d.n_kv_heads, G = a.n_q_heads / H;
  const int n_items = a.chunk_start[a.total_rows] * H;
  const int worker = blockIdx.x * kMmaWarps + warp, n_workers = gridDim.x * kMmaWarps;

  if (lane == 0) {
    for (int s = 0; s < STAGES; ++s) ptx::mbar_init(&full_bar[s], 1);
    ptx::mbar_fence_init();
  }
  __syncwarp();

  int p_item = worker, p_page = 0, p_end = 0, p_begin = 0, p_head = 0, p_pid = 0;
  uint32_t prod_n = 0;
  auto producer_enter_item = [&]() {
    if (p_item < n_items) {
      const Item it = decode_item(a, p_item);
      p_begin = it.page_begin; p_page = it.page_begin; p_end = it.page_end; p_head = it.head;
      const int pg = it.page_begin + lane;
      if (pg < it.page_end) p_pid = a.d.block_table[(size_t)it.seq * a.d.max_pages_per_seq + pg];
    }
  };
  auto produce_one = [&]() {
    if (p_item >= n_items) return;
    const int pid = __shfl_sync(0xffffffffu, p_pid, p_page - p_begin);
    const uint32_t s = prod_n % STAGES;
    if (lane == 0) {
      ptx::fence_proxy_async_smem();
      unsigned char* kd = my_tiles + (size_t)s * 2 * TILE;
      const int row0 = (pid * H + p_head) * 32;
      ptx::mbar_expect_tx(&full_bar[s], 2 * TILE);
      ptx::tma_load_3d(kd, &kmap, 0, row0, a.layer, &full_bar[s]);
      ptx::tma_load_3d(kd + TILE, &vmap, 0, row0, a.layer, &full_bar[s]);
    }
    prod_n += 1;
    p_page += 1;
    if (p_page >= p_end) {
      p_item += n_workers;
      producer_enter_item();
    }
  };
  producer_enter_item();
  for (int i = 0; i < STAGES; ++i) produce_one();

  bool alive = true;
  uint32_t cons_n = 0;
  const int ld_r = lane & 7, ld_m = lane >> 3;
  for (int item = worker; item < n_items && alive; item += n_workers) {
    const Item it = decode_item(a, item);
    // Q fragments (f16): k-step c, slots (2t,2t+1) <- dims 16c+4t+{0,1}; slots (2t+8,2t+9) <- dims 16c+4t+{2,3}
    uint32_t qa0[KS], qa2[KS];
    {
      const __nv_bfloat16* qrow = a.q + (size_t)it.row * a.q_stride + (it.head * G + (g < G ? g : 0)) * D;
#pragma unroll
      for (int c = 0; c < KS; ++c) {
        const uint2 raw = *reinterpret_cast<const uint2*>(qrow + 16 * c + 4 * t);
        qa0[c] = g < G ? pack_f16(ptx::bf16_lo(raw.x), ptx::bf16_hi(raw.x)) : 0u;
        qa2[c] = g < G ? pack_f16(ptx::bf16_lo(raw.y), ptx::bf16_hi(raw.y)) : 0u;
      }
    }
    // scales of this item's pages: lane i holds page page_begin + i
    float my_ks = 0.f, my_vs = 0.f;
    {
      const int pg = it.page_begin + lane;
      if (pg < it.page_end) {
        const int pid = a.d.block_table[(size_t)it.seq * a.d.max_pages_per_seq + pg];
        const size_t si = ((size_t)a.layer * a.d.n_pages + pid) * H + it.head;
        my_ks = a.d.k_scale[si];
        my_vs = a.d.v_scale[si];
      }
    }
    float v_ref = my_vs;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v_ref = fmaxf(v_ref, __shfl_xor_sync(0xffffffffu, v_ref, o));
    const float my_vr = v_ref > 0.f ? my_vs / v_ref : 0.f;

    float o[NO][4];
#pragma unroll
    for (int j = 0; j < NO; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    float m_run = -1e30f, l_run = 0.f;

    for (int pg = it.page_begin; pg < it.page_end; ++pg) {
      const uint32_t s = cons_n % STAGES;
      alive = ptx::mbar_wait(&full_bar[s], (cons_n / STAGES) & 1u);
      if (!alive) break;
      const float ks = __shfl_sync(0xffffffffu, my_ks, pg - it.page_begin) * a.scale_log2;
      const float vr = __shfl_sync(0xffffffffu, my_vr, pg - it.page_begin);
      const uint32_t kbase = ptx::smem_u32(my_tiles + (size_t)s * 2 * TILE), vbase = kbase + TILE;
      // ---- S = Q K^T : 4 n-tiles of 8 tokens; one ldmatrix.x4 = 4 chunks = 4 k-steps ----
      float sc[4][4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) { sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f; }
#pragma unroll
      for (int kk = 0; kk < KS / 4; ++kk) {
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          const int row = nt * 8 + ld_r, cc = 4 * kk + ld_m;
          uint32_t b[4];
          ldsm_x4(kbase + row * 128 + ((cc ^ (row & 7)) << 4), b);
#pragma unroll
          for (int m = 0; m < 4; ++m)
            mma_f16_16816(sc[nt], qa0[4 * kk + m], qa2[4 * kk + m], e4m3x2_to_f16x2(b[m]), e4m3x2_to_f16x2(b[m] >> 16));
        }
      }
      // ---- online softmax on row g ----
      const int tok0 = pg * 32;
      float mx = -1e30f;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const bool valid = tok0 + nt * 8 + 2 * t + e < it.ctx;
          sc[nt][e] = valid ? sc[nt][e] * ks : -1e30f;
          mx = fmaxf(mx, sc[nt][e]);
        }
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run, mx);
      const float corr = exp2f(m_run - m_new);
      float psum = 0.f;
      uint32_t pa0[2], pa2[2];
#pragma unroll
      for (int kt = 0; kt < 2; ++kt) {
        float pv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float sv = sc[2 * kt + (e >> 1)][e & 1];
          pv[e] = sv > -1e29f ? exp2f(sv - m_new) : 0.f;
          psum += pv[e];
        }
        pa0[kt] = pack_f16(pv[0] * vr, pv[1] * vr);
        pa2[kt] = pack_f16(pv[2] * vr, pv[3] * vr);
      }
      l_run = l_run * corr + psum;
      m_run = m_new;
      if (__any_sync(0xffffffffu, corr != 1.f)) {
#pragma unroll
        for (int j = 0; j < NO; ++j) { o[j][0] *= corr; o[j][1] *= corr; }
      }
      // ---- O += P V : output tile 2c holds the even dims of chunk c, tile 2c+1 the odd dims ----
#pragma unroll
      for (int kt = 0; kt < 2; ++kt) {
#pragma unroll
        for (int jj = 0; jj < KS / 2; ++jj) {
          const int row = kt * 16 + (ld_m & 1) * 8 + ld_r, cc = 2 * jj + (ld_m >> 1);
          uint32_t b[4];
          ldsm_x4_trans(vbase + row * 128 + ((cc ^ (row & 7)) << 4), b);
          // bytes (tok 2t, dim 2g), (2t, 2g+1), (2t+1, 2g), (2t+1, 2g+1) -> (even dim pair | odd dim pair)
          const uint32_t p0 = __byte_perm(b[0], 0u, 0x3120), p1 = __byte_perm(b[1], 0u, 0x3120);
          const uint32_t p2 = __byte_perm(b[2], 0u, 0x3120), p3 = __byte_perm(b[3], 0u, 0x3120);
          mma_f16_16816(o[4 * jj], pa0[kt], pa2[kt], e4m3x2_to_f16x2(p0), e4m3x2_to_f16x2(p1));
          mma_f16_16816(o[4 * jj + 1], pa0[kt], pa2[kt], e4m3x2_to_f16x2(p0 >> 16), e4m3x2_to_f16x2(p1 >> 16));
          mma_f16_16816(o[4 * jj + 2], pa0[kt], pa2[kt], e4m3x2_to_f16x2(p2), e4m3x2_to_f16x2(p3));
          mma_f16_16816(o[4 * jj + 3], pa0[kt], pa2[kt], e4m3x2_to_f16x2(p2 >> 16), e4m3x2_to_f16x2(p3 >> 16));
        }
      }
      __syncwarp();
      cons_n += 1;
      produce_one();
    }
    if (!alive) break;
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    if (g < G) {
      const size_t pidx = (size_t)it.chunk * a.n_q_heads + it.head * G + g;
      // chunk c of the row: dims 16c+4t+{0,1,2,3} = (tile 2c col 2t, tile 2c+1 col 2t, tile 2c col 2t+1, tile 2c+1 col 2t+1)
#pragma unroll
      for (int c = 0; c < KS; ++c)
        *reinterpret_cast<float4*>(a.part_o + pidx * D + 16 * c + 4 * t) =
            make_float4(o[2 * c][0] * v_ref, o[2 * c + 1][0] * v_ref, o[2 * c][1] * v_ref, o[2 * c + 1][1] * v_ref);
      if (t == 0) { a.part_ml[pidx * 2] = m_run; a.part_ml[pidx * 2 + 1] = l_run; }
    }
  }
  if (!alive && lane == 0) atomicExch(a.d.state + ST_ATTN_ERR, B200_ERR_DEVICE_FLAGGED);
}

// ---------------------------------------------------------------------------------------------
// Prefill rows (bf16 pools): ragged causal attention of a chunk of new tokens over the paged cache.
//
// Semantics are those of the decode kernels (row r attends to the first row_ctx[r] cached tokens of
// its slot; the rows' own K/V have been appended already), but rows are grouped: up to 16/G
// consecutive rows of one sequence whose contexts grow by one token form a group, and a work item
// is (group, chunk of pages, kv head).  The 16 MMA rows carry (token of the group) x (query head
// of the kv head's GQA group), so a staged K/V page serves every token of the group at once and
// the cache is read once per group instead of once per row.  Causality is a per-MMA-row context
// length.  Groups are found on the device from the row arrays (one CTA, prefix scans).
template <bool MAX>
__device__ __forceinline__ int block_scan_inclusive(int v, int* warp_buf) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc = MAX ? max(inc, t) : inc + t;
  }
  if (lane == 31) warp_buf[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int w = warp_buf[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w = MAX ? max(w, t) : w + t;
    }
    const int ex = __shfl_up_sync(0xffffffffu, w, 1);  // exclusive prefix over the warps
    warp_buf[lane] = lane == 0 ? (MAX ? -1 : 0) : ex;
  }
  __syncthreads();
  const int r = MAX ? max(warp_buf[warp], inc) : warp_buf[warp] + inc;
  __syncthreads();
  return r;
}

__global__ void __launch_bounds__(1024) attn_plan_groups_kernel(const int* __restrict__ row_seq, const int* __restrict__ row_ctx,
                                                                int total_rows, int page_size, int pages_per_chunk, int q_tokens,
                                                                int* __restrict__ chunk_start, int* __restrict__ group_first,
                                                                int* __restrict__ part_base, int* __restrict__ row_group,
                                                                int* __restrict__ n_groups_out, int max_slots, int* __restrict__ err) {
  __shared__ int warp_buf[32];
  __shared__ int carry_start, carry_groups, carry_chunks, carry_slots;
  const int tid = threadIdx.x;
  if (tid == 0) { carry_start = -1; carry_groups = 0; carry_chunks = 0; carry_slots = 0; }
  __syncthreads();
  // pass 1: runs of joinable rows, cut into groups of q_tokens
  for (int base = 0; base < total_rows; base += blockDim.x) {
    const int i = base + tid;
    const bool valid = i < total_rows;
    const bool joinable = valid && i > 0 && row_seq[i] == row_seq[i - 1] && row_ctx[i] == row_ctx[i - 1] + 1;
    const int run_start = max(block_scan_inclusive<true>(valid && !joinable ? i : -1, warp_buf), carry_start);
    const int head = valid && ((i - run_start) % q_tokens == 0) ? 1 : 0;
    const int heads_incl = block_scan_inclusive<false>(head, warp_buf);
    const int gid = carry_groups + heads_incl - 1;
    if (valid) {
      row_group[i] = gid;
      if (head) group_first[gid] = i;
    }
    __syncthreads();
    if (tid == blockDim.x - 1) { carry_start = run_start; carry_groups += heads_incl; }
    __syncthreads();
  }
  const int n_groups = carry_groups;
  if (tid == 0) { group_first[n_groups] = total_rows; *n_groups_out = n_groups; }
  __syncthreads();
  // pass 2: chunks and partial slots per group
  for (int base = 0; base < n_groups; base += blockDim.x) {
    const int gidx = base + tid;
    int chunks = 0, slots = 0;
    if (gidx < n_groups) {
      const int first = group_first[gidx], next = group_first[gidx + 1];
      const int pages = (max(row_ctx[next - 1], 0) + page_size - 1) / page_size;
      chunks = (pages + pages_per_chunk - 1) / pages_per_chunk;
      slots = chunks * (next - first);
    }
    const int c_incl = block_scan_inclusive<false>(chunks, warp_buf);
    const int s_incl = block_scan_inclusive<false>(slots, warp_buf);
    if (gidx < n_groups) {
      chunk_start[gidx] = carry_chunks + c_incl - chunks;
      part_base[gidx] = carry_slots + s_incl - slots;
    }
    __syncthreads();
    if (tid == blockDim.x - 1) { carry_chunks += c_incl; carry_slots += s_incl; }
    __syncthreads();
  }
  if (tid == 0) {
    if (carry_slots > max_slots) { *err = B200_ERR_CAPACITY; chunk_start[n_groups] = 0; }
    else chunk_start[n_groups] = carry_chunks;
  }
}

struct GroupItem {
  int head, seq, first_row, n_rows, ctx0, page_begin, page_end, slot0;
};

__device__ __forceinline__ GroupItem decode_group_item(const AttnArgs& a, int item, int n_groups) {
  GroupItem it;
  const int H = a.d.n_kv_heads;
  const int chunk = item / H;
  it.head = item - chunk * H;
  int lo = 0, hi = n_groups - 1;  // last group with chunk_start[group] <= chunk
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (a.chunk_start[mid] <= chunk) lo = mid; else hi = mid - 1;
  }
  it.first_row = a.group_first[lo];
  it.n_rows = a.group_first[lo + 1] - it.first_row;
  it.seq = a.row_seq[it.first_row];
  it.ctx0 = a.row_ctx[it.first_row];
  const int c = chunk - a.chunk_start[lo];
  const int npages = (it.ctx0 + it.n_rows - 1 + a.d.page_size - 1) / a.d.page_size;
  it.page_begin = c * a.pages_per_chunk;
  it.page_end = min(it.page_begin + a.pages_per_chunk, npages);
  it.slot0 = a.part_base[lo] + c * it.n_rows;
  return it;
}

__device__ __forceinline__ void mma_bf16_16816_full(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                                    uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int D>
__global__ void __launch_bounds__(kMmaWarps * 32, 1)
    paged_attn_prefill_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap, AttnArgs a) {
  constexpr int BOXES = D / 64;
  constexpr int TILE = 32 * D * 2;
  constexpr int KS = D / 16;
  constexpr int NO = D / 8;

  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  unsigned char* my_tiles = smem + (size_t)warp * kMmaStages * 2 * TILE;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)kMmaWarps * kMmaStages * 2 * TILE) + warp * kMmaStages;
  const int H = a.d.n_kv_heads, G = a.n_q_heads / H;
  const int n_groups = *a.n_groups;
  const int n_items = a.chunk_start[n_groups] * H;
  const int worker = blockIdx.x * kMmaWarps + warp, n_workers = gridDim.x * kMmaWarps;

  if (lane == 0) {
    for (int s = 0; s < kMmaStages; ++s) ptx::mbar_init(&full_bar[s], 1);
    ptx::mbar_fence_init();
  }
  __syncwarp();

  // the lanes hold the page ids of a window of 32 pages of the item's chunk (a chunk may be longer: one chunk per
  // group in the direct mode), refilled every 32 pages
  int p_item = worker, p_page = 0, p_end = 0, p_begin = 0, p_head = 0, p_pid = 0, p_seq = 0;
  uint32_t prod_n = 0;
  auto producer_enter_item = [&]() {
    if (p_item < n_items) {
      const GroupItem it = decode_group_item(a, p_item, n_groups);
      p_begin = it.page_begin; p_page = it.page_begin; p_end = it.page_end; p_head = it.head; p_seq = it.seq;
      const int pg = it.page_begin + lane;
      if (pg < it.page_end) p_pid = a.d.block_table[(size_t)it.seq * a.d.max_pages_per_seq + pg];
    }
  };
  auto produce_one = [&]() {
    if (p_item >= n_items) return;
    const int rel = p_page - p_begin;
    if (rel > 0 && (rel & 31) == 0) {
      const int pg = p_page + lane;
      if (pg < p_end) p_pid = a.d.block_table[(size_t)p_seq * a.d.max_pages_per_seq + pg];
    }
    const int pid = __shfl_sync(0xffffffffu, p_pid, rel & 31);
    const uint32_t s = prod_n % kMmaStages;
    if (lane == 0) {
      ptx::fence_proxy_async_smem();
      unsigned char* kd = my_tiles + (size_t)s * 2 * TILE;
      const int row0 = (pid * H + p_head) * 32;
      ptx::mbar_expect_tx(&full_bar[s], 2 * TILE);
#pragma unroll
      for (int b = 0; b < BOXES; ++b) {
        ptx::tma_load_3d(kd + b * 4096, &kmap, b * 64, row0, a.layer, &full_bar[s]);
        ptx::tma_load_3d(kd + TILE + b * 4096, &vmap, b * 64, row0, a.layer, &full_bar[s]);
      }
    }
    prod_n += 1;
    p_page += 1;
    if (p_page >= p_end) {
      p_item += n_workers;
      producer_enter_item();
    }
  };
  producer_enter_item();
  for (int i = 0; i < kMmaStages; ++i) produce_one();

  bool alive = true;
  uint32_t cons_n = 0;
  const int ld_r = lane & 7, ld_m = lane >> 3;
  // MMA rows g and g+8 of this lane: (token of the group, query head within the GQA group)
  const int tokA = g / G, headA = g - tokA * G, tokB = (g + 8) / G, headB = (g + 8) - tokB * G;
  for (int item = worker; item < n_items && alive; item += n_workers) {
    const GroupItem it = decode_group_item(a, item, n_groups);
    const bool onA = tokA < it.n_rows, onB = tokB < it.n_rows;
    const int ctxA = onA ? it.ctx0 + tokA : 0, ctxB = onB ? it.ctx0 + tokB : 0;
    uint32_t qa0[KS], qa1[KS], qa2[KS], qa3[KS];
    {
      const uint32_t* qA = reinterpret_cast<const uint32_t*>(a.q + (size_t)(it.first_row + (onA ? tokA : 0)) * a.q_stride + (it.head * G + headA) * D);
      const uint32_t* qB = reinterpret_cast<const uint32_t*>(a.q + (size_t)(it.first_row + (onB ? tokB : 0)) * a.q_stride + (it.head * G + headB) * D);
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        qa0[ks] = onA ? qA[ks * 8 + t] : 0u;
        qa2[ks] = onA ? qA[ks * 8 + 4 + t] : 0u;
        qa1[ks] = onB ? qB[ks * 8 + t] : 0u;
        qa3[ks] = onB ? qB[ks * 8 + 4 + t] : 0u;
      }
    }
    float o[NO][4];
#pragma unroll
    for (int j = 0; j < NO; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    float mA = -1e30f, lA = 0.f, mB = -1e30f, lB = 0.f;

    for (int pg = it.page_begin; pg < it.page_end; ++pg) {
      const uint32_t s = cons_n % kMmaStages;
      alive = ptx::mbar_wait(&full_bar[s], (cons_n / kMmaStages) & 1u);
      if (!alive) break;
      const uint32_t kbase = ptx::smem_u32(my_tiles + (size_t)s * 2 * TILE), vbase = kbase + TILE;
      float sc[4][4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) { sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f; }
#pragma unroll
      for (int kk = 0; kk < KS / 2; ++kk) {
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          const int row = nt * 8 + ld_r, cc = 4 * kk + ld_m;
          uint32_t b[4];
          ldsm_x4(kbase + (cc >> 3) * 4096 + row * 128 + (((cc & 7) ^ (row & 7)) << 4), b);
          mma_bf16_16816_full(sc[nt], qa0[2 * kk], qa1[2 * kk], qa2[2 * kk], qa3[2 * kk], b[0], b[1]);
          mma_bf16_16816_full(sc[nt], qa0[2 * kk + 1], qa1[2 * kk + 1], qa2[2 * kk + 1], qa3[2 * kk + 1], b[2], b[3]);
        }
      }
      // ---- online softmax on rows g (A) and g+8 (B), each with its own causal context ----
      const int tok0 = pg * 32;
      float mxA = -1e30f, mxB = -1e30f;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int tok = tok0 + nt * 8 + 2 * t + e;
          sc[nt][e] = tok < ctxA ? sc[nt][e] * a.scale_log2 : -1e30f;
          sc[nt][2 + e] = tok < ctxB ? sc[nt][2 + e] * a.scale_log2 : -1e30f;
          mxA = fmaxf(mxA, sc[nt][e]);
          mxB = fmaxf(mxB, sc[nt][2 + e]);
        }
      }
      mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 1));
      mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 2));
      mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 1));
      mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 2));
      const float mA_new = fmaxf(mA, mxA), mB_new = fmaxf(mB, mxB);
      const float corrA = exp2f(mA - mA_new), corrB = exp2f(mB - mB_new);
      float psA = 0.f, psB = 0.f;
      uint32_t pa0[2], pa1[2], pa2[2], pa3[2];
#pragma unroll
      for (int kt = 0; kt < 2; ++kt) {
        float pA[4], pB[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float sa = sc[2 * kt + (e >> 1)][e & 1], sb = sc[2 * kt + (e >> 1)][2 + (e & 1)];
          pA[e] = sa > -1e29f ? exp2f(sa - mA_new) : 0.f;
          pB[e] = sb > -1e29f ? exp2f(sb - mB_new) : 0.f;
          psA += pA[e];
          psB += pB[e];
        }
        pa0[kt] = pack_bf16(pA[0], pA[1]);
        pa2[kt] = pack_bf16(pA[2], pA[3]);
        pa1[kt] = pack_bf16(pB[0], pB[1]);
        pa3[kt] = pack_bf16(pB[2], pB[3]);
      }
      lA = lA * corrA + psA; mA = mA_new;
      lB = lB * corrB + psB; mB = mB_new;
      if (__any_sync(0xffffffffu, corrA != 1.f || corrB != 1.f)) {
#pragma unroll
        for (int j = 0; j < NO; ++j) { o[j][0] *= corrA; o[j][1] *= corrA; o[j][2] *= corrB; o[j][3] *= corrB; }
      }
#pragma unroll
      for (int kt = 0; kt < 2; ++kt) {
#pragma unroll
        for (int jj = 0; jj < NO / 2; ++jj) {
          const int row = kt * 16 + (ld_m & 1) * 8 + ld_r, cc = 2 * jj + (ld_m >> 1);
          uint32_t b[4];
          ldsm_x4_trans(vbase + (cc >> 3) * 4096 + row * 128 + (((cc & 7) ^ (row & 7)) << 4), b);
          mma_bf16_16816_full(o[2 * jj], pa0[kt], pa1[kt], pa2[kt], pa3[kt], b[0], b[1]);
          mma_bf16_16816_full(o[2 * jj + 1], pa0[kt], pa1[kt], pa2[kt], pa3[kt], b[2], b[3]);
        }
      }
      __syncwarp();
      cons_n += 1;
      produce_one();
    }
    if (!alive) break;
    lA += __shfl_xor_sync(0xffffffffu, lA, 1);
    lA += __shfl_xor_sync(0xffffffffu, lA, 2);
    lB += __shfl_xor_sync(0xffffffffu, lB, 1);
    lB += __shfl_xor_sync(0xffffffffu, lB, 2);
    if (a.direct_out) {
      if (onA) {
        const float inv = lA > 0.f ? 1.0f / lA : 0.f;
        __nv_bfloat16* dst = a.direct_out + ((size_t)(it.first_row + tokA) * a.n_q_heads + it.head * G + headA) * D;
#pragma unroll
        for (int j = 0; j < NO; ++j) *reinterpret_cast<__nv_bfloat162*>(dst + j * 8 + 2 * t) = __floats2bfloat162_rn(o[j][0] * inv, o[j][1] * inv);
      }
      if (onB) {
        const float inv = lB > 0.f ? 1.0f / lB : 0.f;
        __nv_bfloat16* dst = a.direct_out + ((size_t)(it.first_row + tokB) * a.n_q_heads + it.head * G + headB) * D;
#pragma unroll
        for (int j = 0; j < NO; ++j) *reinterpret_cast<__nv_bfloat162*>(dst + j * 8 + 2 * t) = __floats2bfloat162_rn(o[j][2] * inv, o[j][3] * inv);
      }
      continue;
    }
    if (onA) {
      const size_t pidx = (size_t)(it.slot0 + tokA) * a.n_q_heads + it.head * G + headA;
#pragma unroll
      for (int j = 0; j < NO; ++j)
        *reinterpret_cast<float2*>(a.part_o + pidx * D + j * 8 + 2 * t) = make_float2(o[j][0], o[j][1]);
      if (t == 0) { a.part_ml[pidx * 2] = mA; a.part_ml[pidx * 2 + 1] = lA; }
    }
    if (onB) {
      const size_t pidx = (size_t)(it.slot0 + tokB) * a.n_q_heads + it.head * G + headB;
#pragma unroll
      for (int j = 0; j < NO; ++j)
        *reinterpret_cast<float2*>(a.part_o + pidx * D + j * 8 + 2 * t) = make_float2(o[j][2], o[j][3]);
      if (t == 0) { a.part_ml[pidx * 2] = mB; a.part_ml[pidx * 2 + 1] = lB; }
    }
  }
  if (!alive && lane == 0) atomicExch(a.d.state + ST_ATTN_ERR, B200_ERR_DEVICE_FLAGGED);
}

__device__ __forceinline__ void mma_f16_16816_full(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                                   uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Prefill rows over an FP8-E4M3 pool (head_dim 128): the row grouping of paged_attn_prefill_kernel
// with the operand handling of paged_attn_mma_fp8_kernel (codes widened to f16 in registers, MMA K
// slots permuted to match ldmatrix on byte tiles, K scale on the scores, relative V scale on P).
__global__ void __launch_bounds__(kMmaWarps * 32, 1)
    paged_attn_prefill_fp8_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap, AttnArgs a) {
  constexpr int D = 128, TILE = 32 * D, KS = D / 16, NO = D / 8, STAGES = kMmaStages;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  unsigned char* my_tiles = smem + (size_t)warp * STAGES * 2 * TILE;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)kMmaWarps * STAGES * 2 * TILE) + warp * STAGES;
  const int H = a.d.n_kv_heads, G = a.n_q_heads / H;
  const int n_groups = *a.n_groups;
  const int n_items = a.chunk_start[n_groups] * H;
  const int worker = blockIdx.x * kMmaWarps + warp, n_workers = gridDim.x * kMmaWarps;

  if (lane == 0) {
    for (int s = 0; s < STAGES; ++s) ptx::mbar_init(&full_bar[s], 1);
    ptx::mbar_fence_init();
  }
  __syncwarp();

  // the lanes hold the page ids of a window of 32 pages of the item's chunk (a chunk may be longer: one chunk per
  // group in the direct mode), refilled every 32 pages
  int p_item = worker, p_page = 0, p_end = 0, p_begin = 0, p_head = 0, p_pid = 0, p_seq = 0;
  uint32_t prod_n = 0;
  auto producer_enter_item = [&]() {
    if (p_item < n_items) {
      const GroupItem it = decode_group_item(a, p_item, n_groups);
      p_begin = it.page_begin; p_page = it.page_begin; p_end = it.page_end; p_head = it.head; p_seq = it.seq;
      const int pg = it.page_begin + lane;
      if (pg < it.page_end) p_pid = a.d.block_table[(size_t)it.seq * a.d.max_pages_per_seq + pg];
    }
  };
  auto produce_one = [&]() {
    if (p_item >= n_items) return;
    const int rel = p_page - p_begin;
    if (rel > 0 && (rel & 31) == 0) {
      const int pg = p_page + lane;
      if (pg < p_end) p_pid = a.d.block_table[(size_t)p_seq * a.d.max_pages_per_seq + pg];
    }
    const int pid = __shfl_sync(0xffffffffu, p_pid, rel & 31);
    const uint32_t s = prod_n % STAGES;
    if (lane == 0) {
      ptx::fence_proxy_async_smem();
      unsigned char* kd = my_tiles + (size_t)s * 2 * TILE;
      const int row0 = (pid * H + p_head) * 32;
      ptx::mbar_expect_tx(&full_bar[s], 2 * TILE);
      ptx::tma_load_3d(kd, &kmap, 0, row0, a.layer, &full_bar[s]);
      ptx::tma_load_3d(kd + TILE, &vmap, 0, row0, a.layer, &full_bar[s]);
    }
    prod_n += 1;
    p_page += 1;
    if (p_page >= p_end) {
      p_item += n_workers;
      producer_enter_item();
    }
  };
  producer_enter_item();
  for (int i = 0; i < STAGES; ++i) produce_one();

  bool alive = true;
  uint32_t cons_n = 0;
  const int ld_r = lane & 7, ld_m = lane >> 3;
  const int tokA = g / G, headA = g - tokA * G, tokB = (g + 8) / G, headB = (g + 8) - tokB * G;
  for (int item = worker; item < n_items && alive; item += n_workers) {
    const GroupItem it = decode_group_item(a, item, n_groups);
    const bool onA = tokA < it.n_rows, onB = tokB < it.n_rows;
    const int ctxA = onA ? it.ctx0 + tokA : 0, ctxB = onB ? it.ctx0 + tokB : 0;
    uint32_t qa0[KS], qa1[KS], qa2[KS], qa3[KS];
    {
      const __nv_bfloat16* qA = a.q + (size_t)(it.first_row + (onA ? tokA : 0)) * a.q_stride + (it.head * G + headA) * D;
      const __nv_bfloat16* qB = a.q + (size_t)(it.first_row + (onB ? tokB : 0)) * a.q_stride + (it.head * G + headB) * D;
#pragma unroll
      for (int c = 0; c < KS; ++c) {
        const uint2 ra = *reinterpret_cast<const uint2*>(qA + 16 * c + 4 * t), rb = *reinterpret_cast<const uint2*>(qB + 16 * c + 4 * t);
        qa0[c] = onA ? pack_f16(ptx::bf16_lo(ra.x), ptx::bf16_hi(ra.x)) : 0u;
        qa2[c] = onA ? pack_f16(ptx::bf16_lo(ra.y), ptx::bf16_hi(ra.y)) : 0u;
        qa1[c] = onB ? pack_f16(ptx::bf16_lo(rb.x), ptx::bf16_hi(rb.x)) : 0u;
        qa3[c] = onB ? pack_f16(ptx::bf16_lo(rb.y), ptx::bf16_hi(rb.y)) : 0u;
      }
    }
    // per-page scales: the lanes hold a window of 32 pages; the reference V scale is the largest of the whole chunk
    float my_ks = 0.f, my_vs = 0.f, v_ref = 0.f;
    for (int base = it.page_begin; base < it.page_end; base += 32) {
      const int pg = base + lane;
      if (pg < it.page_end) {
        const int pid = a.d.block_table[(size_t)it.seq * a.d.max_pages_per_seq + pg];
        const size_t si = ((size_t)a.layer * a.d.n_pages + pid) * H + it.head;
        const float vsc = a.d.v_scale[si];
        v_ref = fmaxf(v_ref, vsc);
        if (base == it.page_begin) { my_ks = a.d.k_scale[si]; my_vs = vsc; }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v_ref = fmaxf(v_ref, __shfl_xor_sync(0xffffffffu, v_ref, o));
    float my_vr = v_ref > 0.f ? my_vs / v_ref : 0.f;

    float o[NO][4];
#pragma unroll
    for (int j = 0; j < NO; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    float mA = -1e30f, lA = 0.f, mB = -1e30f, lB = 0.f;

    for (int pg = it.page_begin; pg < it.page_end; ++pg) {
      const uint32_t s = cons_n % STAGES;
      alive = ptx::mbar_wait(&full_bar[s], (cons_n / STAGES) & 1u);
      if (!alive) break;
      const int rel = pg - it.page_begin;
      if (rel > 0 && (rel & 31) == 0) {  // next window of page scales
        my_ks = 0.f; my_vr = 0.f;
        if (pg + lane < it.page_end) {
          const int pid = a.d.block_table[(size_t)it.seq * a.d.max_pages_per_seq + pg + lane];
          const size_t si = ((size_t)a.layer * a.d.n_pages + pid) * H + it.head;
          my_ks = a.d.k_scale[si];
          my_vr = v_ref > 0.f ? a.d.v_scale[si] / v_ref : 0.f;
        }
      }
      const float ks = __shfl_sync(0xffffffffu, my_ks, rel & 31) * a.scale_log2;
      const float vr = __shfl_sync(0xffffffffu, my_vr, rel & 31);
      const uint32_t kbase = ptx::smem_u32(my_tiles + (size_t)s * 2 * TILE), vbase = kbase + TILE;
      float sc[4][4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) { sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f; }
#pragma unroll
      for (int kk = 0; kk < KS / 4; ++kk) {
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          const int row = nt * 8 + ld_r, cc = 4 * kk + ld_m;
          uint32_t b[4];
          ldsm_x4(kbase + row * 128 + ((cc ^ (row & 7)) << 4), b);
#pragma unroll
          for (int m = 0; m < 4; ++m)
            mma_f16_16816_full(sc[nt], qa0[4 * kk + m], qa1[4 * kk + m], qa2[4 * kk + m], qa3[4 * kk + m], e4m3x2_to_f16x2(b[m]),
                               e4m3x2_to_f16x2(b[m] >> 16));
        }
      }
      const int tok0 = pg * 32;
      float mxA = -1e30f, mxB = -1e30f;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int tok = tok0 + nt * 8 + 2 * t + e;
          sc[nt][e] = tok < ctxA ? sc[nt][e] * ks : -1e30f;
          sc[nt][2 + e] = tok < ctxB ? sc[nt][2 + e] * ks : -1e30f;
          mxA = fmaxf(mxA, sc[nt][e]);
          mxB = fmaxf(mxB, sc[nt][2 + e]);
        }
      }
      mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 1));
      mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 2));
      mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 1));
      mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 2));
      const float mA_new = fmaxf(mA, mxA), mB_new = fmaxf(mB, mxB);
      const float corrA = exp2f(mA - mA_new), corrB = exp2f(mB - mB_new);
      float psA = 0.f, psB = 0.f;
      uint32_t pa0[2], pa1[2], pa2[2], pa3[2];
#pragma unroll
      for (int kt = 0; kt < 2; ++kt) {
        float pA[4], pB[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float sa = sc[2 * kt + (e >> 1)][e & 1], sb = sc[2 * kt + (e >> 1)][2 + (e & 1)];
          pA[e] = sa > -1e29f ? exp2f(sa - mA_new) : 0.f;
          pB[e] = sb > -1e29f ? exp2f(sb - mB_new) : 0.f;
          psA += pA[e];
          psB += pB[e];
        }
        pa0[kt] = pack_f16(pA[0] * vr, pA[1] * vr);
        pa2[kt] = pack_f16(pA[2] * vr, pA[3] * vr);
        pa1[kt] = pack_f16(pB[0] * vr, pB[1] * vr);
        pa3[kt] = pack_f16(pB[2] * vr, pB[3] * vr);
      }
      lA = lA * corrA + psA; mA = mA_new;
      lB = lB * corrB + psB; mB = mB_new;
      if (__any_sync(0xffffffffu, corrA != 1.f || corrB != 1.f)) {
#pragma unroll
        for (int j = 0; j < NO; ++j) { o[j][0] *= corrA; o[j][1] *= corrA; o[j][2] *= corrB; o[j][3] *= corrB; }
      }
#pragma unroll
      for (int kt = 0; kt < 2; ++kt) {
#pragma unroll
        for (int jj = 0; jj < KS / 2; ++jj) {
          const int row = kt * 16 + (ld_m & 1) * 8 + ld_r, cc = 2 * jj + (ld_m >> 1);
          uint32_t b[4];
          ldsm_x4_trans(vbase + row * 128 + ((cc ^ (row & 7)) << 4), b);
          const uint32_t p0 = __byte_perm(b[0], 0u, 0x3120), p1 = __byte_perm(b[1], 0u, 0x3120);
          const uint32_t p2 = __byte_perm(b[2], 0u, 0x3120), p3 = __byte_perm(b[3], 0u, 0x3120);
          mma_f16_16816_full(o[4 * jj], pa0[kt], pa1[kt], pa2[kt], pa3[kt], e4m3x2_to_f16x2(p0), e4m3x2_to_f16x2(p1));
          mma_f16_16816_full(o[4 * jj + 1], pa0[kt], pa1[kt], pa2[kt], pa3[kt], e4m3x2_to_f16x2(p0 >> 16), e4m3x2_to_f16x2(p1 >> 16));
          mma_f16_16816_full(o[4 * jj + 2], pa0[kt], pa1[kt], pa2[kt], pa3[kt], e4m3x2_to_f16x2(p2), e4m3x2_to_f16x2(p3));
          mma_f16_16816_full(o[4 * jj + 3], pa0[kt], pa1[kt], pa2[kt], pa3[kt], e4m3x2_to_f16x2(p2 >> 16), e4m3x2_to_f16x2(p3 >> 16));
        }
      }
      __syncwarp();
      cons_n += 1;
      produce_one();
    }
    if (!alive) break;
    lA += __shfl_xor_sync(0xffffffffu, lA, 1);
    lA += __shfl_xor_sync(0xffffffffu, lA, 2);
    lB += __shfl_xor_sync(0xffffffffu, lB, 1);
    lB += __shfl_xor_sync(0xffffffffu, lB, 2);
    if (a.direct_out) {
      if (onA) {
        const float f = lA > 0.f ? v_ref / lA : 0.f;
        __nv_bfloat16* dst = a.direct_out + ((size_t)(it.first_row + tokA) * a.n_q_heads + it.head * G + headA) * D;
#pragma unroll
        for (int c = 0; c < KS; ++c) {
          const __nv_bfloat162 p0 = __floats2bfloat162_rn(o[2 * c][0] * f, o[2 * c + 1][0] * f), p1 = __floats2bfloat162_rn(o[2 * c][1] * f, o[2 * c + 1][1] * f);
          *reinterpret_cast<uint2*>(dst + 16 * c + 4 * t) = make_uint2(*reinterpret_cast<const uint32_t*>(&p0), *reinterpret_cast<const uint32_t*>(&p1));
        }
      }
      if (onB) {
        const float f = lB > 0.f ? v_ref / lB : 0.f;
        __nv_bfloat16* dst = a.direct_out + ((size_t)(it.first_row + tokB) * a.n_q_heads + it.head * G + headB) * D;
#pragma unroll
        for (int c = 0; c < KS; ++c) {
          const __nv_bfloat162 p0 = __floats2bfloat162_rn(o[2 * c][2] * f, o[2 * c + 1][2] * f), p1 = __floats2bfloat162_rn(o[2 * c][3] * f, o[2 * c + 1][3] * f);
          *reinterpret_cast<uint2*>(dst + 16 * c + 4 * t) = make_uint2(*reinterpret_cast<const uint32_t*>(&p0), *reinterpret_cast<const uint32_t*>(&p1));
        }
      }
      continue;
    }
    if (onA) {
      const size_t pidx = (size_t)(it.slot0 + tokA) * a.n_q_heads + it.head * G + headA;
#pragma unroll
      for (int c = 0; c < KS; ++c)
        *reinterpret_cast<float4*>(a.part_o + pidx * D + 16 * c + 4 * t) =
            make_float4(o[2 * c][0] * v_ref, o[2 * c + 1][0] * v_ref, o[2 * c][1] * v_ref, o[2 * c + 1][1] * v_ref);
      if (t == 0) { a.part_ml[pidx * 2] = mA; a.part_ml[pidx * 2 + 1] = lA; }
    }
    if (onB) {
      const size_t pidx = (size_t)(it.slot0 + tokB) * a.n_q_heads + it.head * G + headB;
#pragma unroll
      for (int c = 0; c < KS; ++c)
        *reinterpret_cast<float4*>(a.part_o + pidx * D + 16 * c + 4 * t) =
            make_float4(o[2 * c][2] * v_ref, o[2 * c + 1][2] * v_ref, o[2 * c][3] * v_ref, o[2 * c + 1][3] * v_ref);
      if (t == 0) { a.part_ml[pidx * 2] = mB; a.part_ml[pidx * 2 + 1] = lB; }
    }
  }
  if (!alive && lane == 0) atomicExch(a.d.state + ST_ATTN_ERR, B200_ERR_DEVICE_FLAGGED);
}

// D threads per (row, query head): merge the partials of the row's group chunks and write bf16.
template <int D>
__global__ void __launch_bounds__(D) attn_combine_groups_kernel(AttnArgs a, __nv_bfloat16* __restrict__ out) {
  const int row = blockIdx.x / a.n_q_heads, qh = blockIdx.x - row * a.n_q_heads, d = threadIdx.x;
  if (a.d.state[ST_ATTN_ERR] != 0) return;
  const int grp = a.row_group[row], first = a.group_first[grp], size = a.group_first[grp + 1] - first;
  const int n_chunks = a.chunk_start[grp + 1] - a.chunk_start[grp];
  const size_t slot0 = (size_t)a.part_base[grp] + (row - first);
  float mm = -1e30f;
  for (int c = 0; c < n_chunks; ++c) mm = fmaxf(mm, a.part_ml[((slot0 + (size_t)c * size) * a.n_q_heads + qh) * 2]);
  float ll = 0.f, acc = 0.f;
#pragma unroll 4
  for (int c = 0; c < n_chunks; ++c) {
    const size_t pidx = (slot0 + (size_t)c * size) * a.n_q_heads + qh;
    const float w = exp2f(a.part_ml[pidx * 2] - mm);
    ll += a.part_ml[pidx * 2 + 1] * w;
    acc += a.part_o[pidx * D + d] * w;
  }
  out[((size_t)row * a.n_q_heads + qh) * D + d] = __float2bfloat16(ll > 0.f ? acc / ll : 0.f);
}

// D threads per (row, query head): merge the row's chunks and write bf16.
template <int D>
__global__ void __launch_bounds__(D) attn_combine_kernel(AttnArgs a, __nv_bfloat16* __restrict__ out) {
  const int row = blockIdx.x / a.n_q_heads, qh = blockIdx.x - row * a.n_q_heads, d = threadIdx.x;
  if (a.d.state[ST_ATTN_ERR] != 0) return;
  const int c0 = a.chunk_start[row], c1 = a.chunk_start[row + 1];
  float mm = -1e30f;
  for (int c = c0; c < c1; ++c) mm = fmaxf(mm, a.part_ml[((size_t)c * a.n_q_heads + qh) * 2]);
  float ll = 0.f, acc = 0.f;
#pragma unroll 4
  for (int c = c0; c < c1; ++c) {
    const size_t pidx = (size_t)c * a.n_q_heads + qh;
    const float w = exp2f(a.part_ml[pidx * 2] - mm);
    ll += a.part_ml[pidx * 2 + 1] * w;
    acc += a.part_o[pidx * D + d] * w;
  }
  out[((size_t)row * a.n_q_heads + qh) * D + d] = __float2bfloat16(ll > 0.f ? acc / ll : 0.f);
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
  attn_combine_kernel<D><<<a.total_rows * a.n_q_heads, D, 0, s>>>(a, (__nv_bfloat16*)d_out);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

template <int D>
b200_status launch_attn_mma(const b200_kv* kv, const AttnArgs& a, void* d_out, int sms, cudaStream_t s) {
  constexpr int TILE = 32 * D * 2;
  const size_t smem = (size_t)kMmaWarps * kMmaStages * 2 * TILE + 1024 + sizeof(uint64_t) * kMmaWarps * kMmaStages;
  static bool configured = false;
  if (!configured) {
    B200_CUDA_TRY(cudaFuncSetAttribute(paged_attn_mma_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  const int ctas_per_sm = smem <= 100 * 1024 ? 2 : 1;
  paged_attn_mma_kernel<D><<<sms * ctas_per_sm, kMmaWarps * 32, smem, s>>>(kv->kmap, kv->vmap, a);
  B200_LAUNCH_CHECK();
  attn_combine_kernel<D><<<a.total_rows * a.n_q_heads, D, 0, s>>>(a, (__nv_bfloat16*)d_out);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

template <int STAGES, int MINB>
b200_status launch_attn_mma_fp8_cfg(const b200_kv* kv, const AttnArgs& a, void* d_out, int sms, cudaStream_t s) {
  constexpr int TILE = 32 * 128;
  const size_t smem = (size_t)kMmaWarps * STAGES * 2 * TILE + 1024 + sizeof(uint64_t) * kMmaWarps * STAGES;
  static bool configured = false;
  if (!configured) {
    B200_CUDA_TRY((cudaFuncSetAttribute(paged_attn_mma_fp8_kernel<STAGES, MINB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)));
    configured = true;
  }
  paged_attn_mma_fp8_kernel<STAGES, MINB><<<sms * MINB, kMmaWarps * 32, smem, s>>>(kv->kmap, kv->vmap, a);
  B200_LAUNCH_CHECK();
  attn_combine_kernel<128><<<a.total_rows * a.n_q_heads, 128, 0, s>>>(a, (__nv_bfloat16*)d_out);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

// Two stages and two CTAs per SM: the kernel is bound by instruction issue (the code widening), not
// by loads in flight; measured 4.22 TB/s against 4.05 (3 stages x 2 CTAs), 4.17 (2 x 3), 2.99 (4 x 1).
b200_status launch_attn_mma_fp8(const b200_kv* kv, const AttnArgs& a, void* d_out, int sms, cudaStream_t s) {
  return launch_attn_mma_fp8_cfg<2, 2>(kv, a, d_out, sms, s);
}

template <int D>
b200_status launch_attn_prefill(const b200_kv* kv, const AttnArgs& a, void* d_out, int sms, cudaStream_t s) {
  constexpr int TILE = 32 * D * 2;
  const size_t smem = (size_t)kMmaWarps * kMmaStages * 2 * TILE + 1024 + sizeof(uint64_t) * kMmaWarps * kMmaStages;
  static bool configured = false;
  if (!configured) {
    B200_CUDA_TRY(cudaFuncSetAttribute(paged_attn_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  const int ctas_per_sm = smem <= 100 * 1024 ? 2 : 1;
  paged_attn_prefill_kernel<D><<<sms * ctas_per_sm, kMmaWarps * 32, smem, s>>>(kv->kmap, kv->vmap, a);
  B200_LAUNCH_CHECK();
  if (a.direct_out) return B200_OK;  // one chunk per group: the kernel wrote the rows itself
  attn_combine_groups_kernel<D><<<a.total_rows * a.n_q_heads, D, 0, s>>>(a, (__nv_bfloat16*)d_out);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

b200_status launch_attn_prefill_fp8(const b200_kv* kv, const AttnArgs& a, void* d_out, int sms, cudaStream_t s) {
  constexpr int TILE = 32 * 128;
  const size_t smem = (size_t)kMmaWarps * kMmaStages * 2 * TILE + 1024 + sizeof(uint64_t) * kMmaWarps * kMmaStages;
  static bool configured = false;
  if (!configured) {
    B200_CUDA_TRY(cudaFuncSetAttribute(paged_attn_prefill_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  paged_attn_prefill_fp8_kernel<<<sms * 2, kMmaWarps * 32, smem, s>>>(kv->kmap, kv->vmap, a);
  B200_LAUNCH_CHECK();
  if (a.direct_out) return B200_OK;  // one chunk per group: the kernel wrote the rows itself
  attn_combine_groups_kernel<128><<<a.total_rows * a.n_q_heads, 128, 0, s>>>(a, (__nv_bfloat16*)d_out);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

int g_sm_count = 0;

}  // namespace

extern int b200_attn_pages_per_chunk;
extern int b200_attn_prefill_direct;
extern int b200_attn_path;

// Pages per chunk: 0 = chosen per batch by the plan kernel (decode rows; 8 for prefill groups below the direct mode),
// so that the persistent grid sees several items per worker without making the per-item partials a visible share of
// the traffic; 4..32 forces a value.
int b200_attn_pages_per_chunk = 0;
int b200_attn_prefill_direct = 1;  // tuning hook for tests: 0 keeps the chunked prefill path at every size
int b200_attn_path = 0;  // 0 = automatic, 1 = CUDA-core kernel, 2 = tensor-core kernel

extern "C" b200_status b200_paged_attn_decode(b200_kv* kv, int32_t layer, const void* d_q, const int32_t* d_row_seq,
                                              const int32_t* d_row_ctx, int32_t total_rows, void* d_out, void* stream) {
  return b200_paged_attn_decode_strided(kv, layer, d_q, kv->cfg.n_q_heads * kv->cfg.head_dim, d_row_seq, d_row_ctx,
                                        total_rows, d_out, stream, 0);
}

b200_status b200_paged_attn_decode_strided(b200_kv* kv, int32_t layer, const void* d_q, int32_t q_stride,
                                           const int32_t* d_row_seq, const int32_t* d_row_ctx, int32_t total_rows,
                                           void* d_out, void* stream, int32_t reuse_plan) {
  b200_status st = b200_require_device();
  if (st != B200_OK) return st;
  const b200_kv_config& c = kv->cfg;
  if (layer < 0 || layer >= c.n_layers) { b200_set_error("attention: layer %d out of range", layer); return B200_ERR_INVALID_ARGUMENT; }
  const bool fp8 = c.kv_dtype == B200_KV_FP8_E4M3;
  // MMA rows 0..7 carry the group's heads; the FP8 tensor-core kernel is built for head_dim 128
  const bool use_mma = b200_attn_path != 1 && c.n_q_heads / c.n_kv_heads <= 8 && (!fp8 || c.head_dim == 128);
  if (!use_mma && c.n_q_heads != c.n_kv_heads * kGroup) {
    b200_set_error("attention: the CUDA-core kernel is built for a GQA group of %d query heads per kv head (got %d/%d)", kGroup, c.n_q_heads, c.n_kv_heads);
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
  // 0 = the plan kernel picks 8, 16 or 32 from the batch's mean context; the tuning hook forces 4..32
  // (scratch bound: chunks <= pages/ppc + rows; kv->max_chunks was sized for ppc >= 4)
  const int ppc = b200_attn_pages_per_chunk <= 0 ? 0 : std::min(std::max(b200_attn_pages_per_chunk, 4), kMaxChunkPages);
  AttnArgs a;
  a.d = kv->dev; a.layer = layer; a.q = (const __nv_bfloat16*)d_q; a.q_stride = q_stride; a.row_seq = d_row_seq; a.row_ctx = d_row_ctx;
  a.chunk_start = kv->d_chunk_start; a.total_rows = total_rows; a.n_q_heads = c.n_q_heads; a.pages_per_chunk = ppc;
  a.part_o = kv->d_part_o; a.part_ml = kv->d_part_ml;
  a.scale_log2 = 1.4426950408889634f / sqrtf((float)c.head_dim);
  a.ppc_dev = kv->d_chunk_start + c.max_rows + 1;  // the last word of the array: the plan kernel's choice
  if (!reuse_plan) {  // the chunk plan depends on the row arrays only: the layers of one step share it
    attn_plan_kernel<<<1, 1024, 0, s>>>(d_row_ctx, total_rows, c.page_size, ppc, kv->d_chunk_start, kv->max_chunks,
                                        kv->dev.state + ST_ATTN_ERR, kv->d_chunk_start + c.max_rows + 1);
    B200_LAUNCH_CHECK();
  }
  if (use_mma && fp8) return launch_attn_mma_fp8(kv, a, d_out, g_sm_count, s);
  if (use_mma) return c.head_dim == 128 ? launch_attn_mma<128>(kv, a, d_out, g_sm_count, s) : launch_attn_mma<64>(kv, a, d_out, g_sm_count, s);
  const int grid = g_sm_count * 3;
  if (c.head_dim == 128) return fp8 ? launch_attn<128, true>(a, d_out, grid, s) : launch_attn<128, false>(a, d_out, grid, s);
  return fp8 ? launch_attn<64, true>(a, d_out, grid, s) : launch_attn<64, false>(a, d_out, grid, s);
}

extern "C" b200_status b200_paged_attn_prefill(b200_kv* kv, int32_t layer, const void* d_q, const int32_t* d_row_seq,
                                               const int32_t* d_row_ctx, int32_t total_rows, void* d_out, void* stream) {
  return b200_paged_attn_prefill_strided(kv, layer, d_q, kv->cfg.n_q_heads * kv->cfg.head_dim, d_row_seq, d_row_ctx,
                                         total_rows, d_out, stream, 0);
}

b200_status b200_paged_attn_prefill_strided(b200_kv* kv, int32_t layer, const void* d_q, int32_t q_stride,
                                            const int32_t* d_row_seq, const int32_t* d_row_ctx, int32_t total_rows,
                                            void* d_out, void* stream, int32_t reuse_plan) {
  const b200_kv_config& c = kv->cfg;
  const int G = c.n_kv_heads > 0 ? c.n_q_heads / c.n_kv_heads : 0;
  // Grouping needs the GQA group to divide the 16 MMA rows, and head_dim 128 for FP8 pools; anything
  // else takes the per-row kernels (same results).
  const bool fp8 = c.kv_dtype == B200_KV_FP8_E4M3;
  if ((fp8 && c.head_dim != 128) || !(G == 1 || G == 2 || G == 4 || G == 8) || b200_attn_path == 1)
    return b200_paged_attn_decode_strided(kv, layer, d_q, q_stride, d_row_seq, d_row_ctx, total_rows, d_out, stream, reuse_plan);
  b200_status st = b200_require_device();
  if (st != B200_OK) return st;
  if (layer < 0 || layer >= c.n_layers) { b200_set_error("attention: layer %d out of range", layer); return B200_ERR_INVALID_ARGUMENT; }
  if (total_rows <= 0) return B200_OK;
  if (total_rows > c.max_rows) { b200_set_error("attention: %d rows > max_rows %d", total_rows, c.max_rows); return B200_ERR_CAPACITY; }
  cudaStream_t s = (cudaStream_t)stream;
  if (g_sm_count == 0) {
    int dev = 0;
    B200_CUDA_TRY(cudaGetDevice(&dev));
    B200_CUDA_TRY(cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev));
  }
  // Prefill batches of 1024 rows and more have rows to spare for parallelism (256 groups x kv heads and up): one chunk
  // per group, as long as its context, and the kernel writes the normalised rows itself: no f32 partials, no combine
  // pass (at 8192 rows of config 5 the partials were 400 MB per layer and the combine pass 7 % of the scenario).
  const bool single_chunk = total_rows >= 1024 && b200_attn_prefill_direct;
  const int ppc = single_chunk ? std::max(c.max_pages_per_seq, 1)
                               : (b200_attn_pages_per_chunk <= 0 ? 8 : std::min(std::max(b200_attn_pages_per_chunk, 4), kMaxChunkPages));
  const int stride = c.max_rows + 2;
  AttnArgs a;
  a.d = kv->dev; a.layer = layer; a.q = (const __nv_bfloat16*)d_q; a.q_stride = q_stride; a.row_seq = d_row_seq; a.row_ctx = d_row_ctx;
  a.chunk_start = kv->d_chunk_start; a.total_rows = total_rows; a.n_q_heads = c.n_q_heads; a.pages_per_chunk = ppc;
  a.part_o = kv->d_part_o; a.part_ml = kv->d_part_ml;
  a.scale_log2 = 1.4426950408889634f / sqrtf((float)c.head_dim);
  a.group_first = kv->d_groups; a.part_base = kv->d_groups + stride; a.row_group = kv->d_groups + 2 * stride;
  a.n_groups = kv->d_groups + 3 * stride - 1;  // last word of the row_group array (never a row index)
  a.q_tokens = 16 / G;
  a.direct_out = single_chunk ? (__nv_bfloat16*)d_out : nullptr;
  if (!reuse_plan) {
    attn_plan_groups_kernel<<<1, 1024, 0, s>>>(d_row_seq, d_row_ctx, total_rows, c.page_size, ppc, a.q_tokens, kv->d_chunk_start,
                                               kv->d_groups, kv->d_groups + stride, kv->d_groups + 2 * stride,
                                               kv->d_groups + 3 * stride - 1, kv->max_chunks, kv->dev.state + ST_ATTN_ERR);
    B200_LAUNCH_CHECK();
  }
  if (fp8) return launch_attn_prefill_fp8(kv, a, d_out, g_sm_count, s);
  return c.head_dim == 128 ? launch_attn_prefill<128>(kv, a, d_out, g_sm_count, s) : launch_attn_prefill<64>(kv, a, d_out, g_sm_count, s);
}

// Tuning hook (not part of the reference surface): pages per split-K chunk, 4..32.
extern "C" void b200_set_attn_pages_per_chunk(int32_t n) { b200_attn_pages_per_chunk = n; }
extern "C" void b200_set_attn_prefill_direct(int32_t on) { b200_attn_prefill_direct = on; }
// Tuning hook: 0 = automatic (tensor-core kernel for bf16 pools), 1 = force the CUDA-core kernel.
extern "C" void b200_set_attn_path(int32_t p) { b200_attn_path = p; }
