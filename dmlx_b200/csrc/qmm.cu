// Dequant-fused quantised matmul  y[T,N] = x[T,K] . dequant(W[N,K])^T  for affine int4 (group 64)
// and MXFP4 (E2M1, one E8M0 scale per 32) weights.
//
// Weight layout in HBM ("blocks"): weights are repacked once into tiles of 128 output rows x 64
// input columns; the block of tile (nt, kc) is contiguous:
//     plane 0: 128 rows x 16 B   (nibbles of columns  0..31 of the chunk)
//     plane 1: 128 rows x 16 B   (nibbles of columns 32..63)
//     affine: 128 bf16 scales, 128 bf16 biases (one group of 64 = one chunk)        -> 4608 B
//     mxfp4 : 128 x 2 E8M0 bytes (one per plane)                                    -> 4352 B
// so a CTA streams its weights as whole blocks (one bulk copy per chunk, or fully coalesced
// 16-byte loads in the GEMV kernel).  Within a 32-bit word holding columns 8w..8w+7, nibble
// position p stores column 2p (p < 4) or 2(p-4)+1, so that (word >> 4i) & 0x000F000F yields the
// adjacent column pair (2i, 2i+1) in the two halves of a bf16x2 register.
//
// The kernels share the layout, the split-K scratch and the epilogue:
//   * qmm_mma_kernel  (up to 16 rows): weight streaming.  Persistent CTAs, a producer warp keeping a
//     ring of raw 4-bit blocks in flight, 8 consumer warps feeding mma.sync from registers.
//   * qmm_tc_kernel   (17..128 rows per token tile, and the grouped MoE launches): "swap-AB" tcgen05
//     GEMM.  The 128 weight rows are the MMA M dimension, the packed tokens (16..256 per tile) the N
//     dimension, so small and large batches both map to dense tensor-core tiles.  Per 64-column
//     chunk: warp 8 issues one bulk copy for the weight block and one 2-D TMA load (128B swizzle)
//     for the activation tile; warps 0-7 dequantise the block to bf16 into a 128B-swizzled K-major
//     tile (one row and one 32-column plane per thread); warp 9 issues 4 tcgen05.mma (M128 x N x
//     K16) accumulating in tensor memory and commits to free the stage.  After the last chunk warps
//     0-3 read the accumulator with tcgen05.ld.
//   * qmm_tc2_kernel  (129..256 rows per token tile): the same with two weight tiles per CTA
//     sharing one activation tile.
//   * qmm_simt_kernel : CUDA-core GEMV kept as a forced path for tests.
// Split-K partials go to an f32 scratch; a finish kernel sums them in split order (deterministic),
// applies the epilogue (residual add, SwiGLU) and writes bf16.  No CTA waits on another.
#include <cuda.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <cstring>
#include <vector>

#include "common.h"
#include "ptx.cuh"
#include "qmm.cuh"
#include "tma.cuh"

namespace {

constexpr int kTileN = 128;
constexpr int kChunkK = 64;
constexpr int kPlaneBytes = kTileN * 16;

__host__ __device__ constexpr int block_bytes(int mode) {
  return mode == B200_Q_AFFINE4_G64 ? 4608 : (mode == B200_Q_MXFP4_G32 ? 4352 : kTileN * 128);
}

// ---- dequantisation of one 32-bit word (8 columns) to 8 bf16 -----------------------------------
template <int MODE>
__device__ __forceinline__ uint4 dequant_word(uint32_t word, __nv_bfloat162 s2, __nv_bfloat162 b2) {
  uint32_t out[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t t = (word >> (4 * i)) & 0x000F000Fu;
    __nv_bfloat162 r;
    if (MODE == B200_Q_AFFINE4_G64) {
      // 0x4300 | q is the bf16 128+q; subtracting 128 leaves q exactly, then one fused q*s+b.
      uint32_t u = t | 0x43004300u;
      const uint32_t c128 = 0x43004300u;
      __nv_bfloat162 q = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&u), *reinterpret_cast<const __nv_bfloat162*>(&c128));
      r = __hfma2(q, s2, b2);
    } else {
      // sign | (e,m) << 6 is the E2M1 value times 2^-126 (exact, subnormals included); two exact
      // power-of-two multiplies bring it to value * 2^(scale-127).
      uint32_t u = ((t & 0x00080008u) << 12) | ((t & 0x00070007u) << 6);
      const uint32_t c64 = 0x5F805F80u;  // 2^64
      r = __hmul2(__hmul2(*reinterpret_cast<__nv_bfloat162*>(&u), *reinterpret_cast<const __nv_bfloat162*>(&c64)), s2);
    }
    out[i] = *reinterpret_cast<uint32_t*>(&r);
  }
  return make_uint4(out[0], out[1], out[2], out[3]);
}

// Per-row dequant parameters for one plane of a block.
template <int MODE>
__device__ __forceinline__ void row_params(const unsigned char* blk, int r, int plane, __nv_bfloat162& s2, __nv_bfloat162& b2) {
  if (MODE == B200_Q_AFFINE4_G64) {
    const __nv_bfloat16* sc = reinterpret_cast<const __nv_bfloat16*>(blk + 2 * kPlaneBytes);
    s2 = __bfloat162bfloat162(sc[r]);
    b2 = __bfloat162bfloat162(sc[kTileN + r]);
  } else {
    uint32_t se = blk[2 * kPlaneBytes + r * 2 + plane];
    se = se > 192u ? 192u : se;
    uint32_t bits = (se + 62u) << 7;  // bf16 2^(se-65)
    bits |= bits << 16;
    s2 = *reinterpret_cast<__nv_bfloat162*>(&bits);
    b2 = s2;
  }
}

// Epilogue of one output quad: columns n..n+3 of row `token` (residual add, SwiGLU over
// interleaved gate/up rows, per-row scale), written as bf16.
__device__ __forceinline__ void finish_store(const QmmArgs& a, int token, int n, float4 acc) {
  const float rs = a.row_scale(token);
  if (a.epilogue == B200_EPI_SWIGLU) {
    float g0 = acc.x, u0 = acc.y, g1 = acc.z, u1 = acc.w;
    if (a.swiglu_limit > 0.f) {
      const float L = a.swiglu_limit;
      g0 = fminf(g0, L); g1 = fminf(g1, L);
      u0 = fminf(fmaxf(u0, -L), L); u1 = fminf(fmaxf(u1, -L), L);
    }
    const float y0 = g0 / (1.0f + __expf(-g0)) * u0 * rs, y1 = g1 / (1.0f + __expf(-g1)) * u1 * rs;
    *reinterpret_cast<__nv_bfloat162*>(a.y + (size_t)a.row_base_out(token) * (a.n / 2) + n / 2) = __floats2bfloat162_rn(y0, y1);
  } else {
    const size_t o = (size_t)a.row_base_out(token) * a.n + n;
    if (a.epilogue == B200_EPI_RESIDUAL) {
      const uint2 rv = *reinterpret_cast<const uint2*>(a.residual + o);
      acc.x += ptx::bf16_lo(rv.x); acc.y += ptx::bf16_hi(rv.x); acc.z += ptx::bf16_lo(rv.y); acc.w += ptx::bf16_hi(rv.y);
    }
    __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x * rs, acc.y * rs), hi = __floats2bfloat162_rn(acc.z * rs, acc.w * rs);
    uint2 ov;
    ov.x = *reinterpret_cast<uint32_t*>(&lo);
    ov.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(a.y + o) = ov;
  }
}

// ---- split-K finish: sums the partial tiles in split order (deterministic), applies the epilogue,
// writes bf16.  One thread per 4 consecutive output columns of one row, so the whole GPU takes
// part and every thread has `splits` independent 16-byte loads in flight.
__global__ void qmm_finish_kernel(QmmArgs a, int splits) {
  const int n4 = a.nt * (kTileN / 4);
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)a.rows * n4) return;
  const int token = (int)(idx / n4), c4 = (int)(idx % n4);
  const int nt = c4 / (kTileN / 4), r = (c4 % (kTileN / 4)) * 4, n = nt * kTileN + r;
  if (n >= a.n) return;
  // Dense launches keep each CTA's partial tile contiguous ([tile][split][tn][128]); grouped
  // launches index by sorted row ([split][row][round_up(N,128)]).
  const float4* p;
  size_t split_stride;  // in float4
  if (a.items) {
    const size_t n_pad = (size_t)a.nt * kTileN;
    p = reinterpret_cast<const float4*>(a.ws + (size_t)token * n_pad + n);
    split_stride = (size_t)a.rows * n_pad / 4;
  } else {
    const int tts = (a.rows + a.tn - 1) / a.tn, tt = token / a.tn, t = token - tt * a.tn;
    p = reinterpret_cast<const float4*>(a.ws + (((size_t)(nt * tts + tt) * splits) * a.tn + t) * kTileN + r);
    split_stride = (size_t)a.tn * kTileN / 4;
  }
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  int s = 0;
  for (; s + 4 <= splits; s += 4) {
    const float4 v0 = p[(size_t)s * split_stride], v1 = p[(size_t)(s + 1) * split_stride];
    const float4 v2 = p[(size_t)(s + 2) * split_stride], v3 = p[(size_t)(s + 3) * split_stride];
    acc.x += v0.x; acc.y += v0.y; acc.z += v0.z; acc.w += v0.w;
    acc.x += v1.x; acc.y += v1.y; acc.z += v1.z; acc.w += v1.w;
    acc.x += v2.x; acc.y += v2.y; acc.z += v2.z; acc.w += v2.w;
    acc.x += v3.x; acc.y += v3.y; acc.z += v3.z; acc.w += v3.w;
  }
  for (; s < splits; ++s) {
    const float4 v = p[(size_t)s * split_stride];
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  finish_store(a, token, n, acc);
}

// ---- split-K finish + RMSNorm ---------------------------------------------------------------------
// The o and down projections end in y = residual + x W^T, and the very next kernel of the layer
// stack normalises y.  One CTA per row sums the partials in split order (the same arithmetic as
// qmm_finish_kernel, so y has the same bits), adds the residual, writes y, and from the bf16 values
// it has just written forms the row's mean square and writes rmsnorm(y) * weight: one launch and one
// pass over y less per projection.  N <= 4 * 4 * blockDim (each thread keeps up to 4 quads).
__global__ void __launch_bounds__(1024) qmm_finish_rmsnorm_kernel(QmmArgs a, int splits) {
  __shared__ float s_part[32];
  const int token = blockIdx.x, n4 = a.n / 4;
  const int tts = (a.rows + a.tn - 1) / a.tn, tt = token / a.tn, t = token - tt * a.tn;
  const size_t split_stride = (size_t)a.tn * kTileN / 4;
  float4 val[4];
  float ss = 0.f;
  int cnt = 0;
  for (int q = threadIdx.x; q < n4; q += blockDim.x, ++cnt) {
    const int n = 4 * q, nt = n / kTileN, r = n - nt * kTileN;
    const float4* p = reinterpret_cast<const float4*>(a.ws + (((size_t)(nt * tts + tt) * splits) * a.tn + t) * kTileN + r);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    int s = 0;
    for (; s + 4 <= splits; s += 4) {
      const float4 v0 = p[(size_t)s * split_stride], v1 = p[(size_t)(s + 1) * split_stride];
      const float4 v2 = p[(size_t)(s + 2) * split_stride], v3 = p[(size_t)(s + 3) * split_stride];
      acc.x += v0.x; acc.y += v0.y; acc.z += v0.z; acc.w += v0.w;
      acc.x += v1.x; acc.y += v1.y; acc.z += v1.z; acc.w += v1.w;
      acc.x += v2.x; acc.y += v2.y; acc.z += v2.z; acc.w += v2.w;
      acc.x += v3.x; acc.y += v3.y; acc.z += v3.z; acc.w += v3.w;
    }
    for (; s < splits; ++s) {
      const float4 v = p[(size_t)s * split_stride];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    const size_t o = (size_t)token * a.n + n;
    const uint2 rv = *reinterpret_cast<const uint2*>(a.residual + o);
    acc.x += ptx::bf16_lo(rv.x); acc.y += ptx::bf16_hi(rv.x); acc.z += ptx::bf16_lo(rv.y); acc.w += ptx::bf16_hi(rv.y);
    __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
    uint2 ov;
    ov.x = *reinterpret_cast<uint32_t*>(&lo);
    ov.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(a.y + o) = ov;
    const float4 rounded = make_float4(ptx::bf16_lo(ov.x), ptx::bf16_hi(ov.x), ptx::bf16_lo(ov.y), ptx::bf16_hi(ov.y));
    val[cnt] = rounded;
    ss += rounded.x * rounded.x + rounded.y * rounded.y + rounded.z * rounded.z + rounded.w * rounded.w;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float tsum = threadIdx.x < (blockDim.x >> 5) ? s_part[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tsum += __shfl_xor_sync(0xffffffffu, tsum, o);
    if (threadIdx.x == 0) s_part[0] = rsqrtf(tsum / (float)a.n + a.norm_eps);
  }
  __syncthreads();
  const float rn = s_part[0];
  cnt = 0;
  for (int q = threadIdx.x; q < n4; q += blockDim.x, ++cnt) {
    const int n = 4 * q;
    const uint2 gw = *reinterpret_cast<const uint2*>(a.norm_w + n);
    const float4 v = val[cnt];
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x * rn * ptx::bf16_lo(gw.x), v.y * rn * ptx::bf16_hi(gw.x));
    __nv_bfloat162 hi = __floats2bfloat162_rn(v.z * rn * ptx::bf16_lo(gw.y), v.w * rn * ptx::bf16_hi(gw.y));
    uint2 ov;
    ov.x = *reinterpret_cast<uint32_t*>(&lo);
    ov.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(a.norm_out + (size_t)token * a.n + n) = ov;
  }
}

// ---- GEMV kernel ---------------------------------------------------------------------------------
template <int MODE, int TT>
__global__ void __launch_bounds__(kTileN) qmm_simt_kernel(QmmArgs a) {
  __shared__ __align__(16) float xs[TT][kChunkK];
  const int nt = blockIdx.x, split = blockIdx.y, tt = blockIdx.z;
  const int r = threadIdx.x, t0 = tt * TT;
  const int kc0 = split * a.chunks_per_split, kc1 = min(kc0 + a.chunks_per_split, a.kc);
  float acc[TT];
#pragma unroll
  for (int t = 0; t < TT; ++t) acc[t] = 0.f;
  constexpr int BB = block_bytes(MODE);
  for (int kc = kc0; kc < kc1; ++kc) {
    __syncthreads();
    for (int idx = threadIdx.x; idx < TT * kChunkK; idx += blockDim.x) {
      const int t = idx / kChunkK, j = idx % kChunkK;
      xs[t][j] = (t0 + t < a.rows) ? __bfloat162float(a.x[(size_t)(t0 + t) * a.k + kc * kChunkK + j]) : 0.f;
    }
    __syncthreads();
    const unsigned char* blk = a.blocks + ((size_t)nt * a.kc + kc) * BB;
    if constexpr (MODE == B200_Q_BF16) {
      // dense bf16 block: row r is 128 bytes, 16-byte chunk c stored at position c ^ (r & 7)
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const uint4 d = *reinterpret_cast<const uint4*>(blk + r * 128 + ((c ^ (r & 7)) << 4));
        const uint32_t dd[4] = {d.x, d.y, d.z, d.w};
        float wf[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) { wf[2 * i] = ptx::bf16_lo(dd[i]); wf[2 * i + 1] = ptx::bf16_hi(dd[i]); }
#pragma unroll
        for (int t = 0; t < TT; ++t) {
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[t] = fmaf(wf[i], xs[t][c * 8 + i], acc[t]);
        }
      }
    } else {
#pragma unroll
    for (int plane = 0; plane < 2; ++plane) {
      const uint4 raw = reinterpret_cast<const uint4*>(blk + plane * kPlaneBytes)[r];
      __nv_bfloat162 s2, b2;
      row_params<MODE>(blk, r, plane, s2, b2);
      const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const uint4 d = dequant_word<MODE>(words[w], s2, b2);
        const uint32_t dd[4] = {d.x, d.y, d.z, d.w};
        float wf[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) { wf[2 * i] = ptx::bf16_lo(dd[i]); wf[2 * i + 1] = ptx::bf16_hi(dd[i]); }
        const int col = plane * 32 + w * 8;
#pragma unroll
        for (int t = 0; t < TT; ++t) {
          const float4 x0 = *reinterpret_cast<const float4*>(&xs[t][col]);
          const float4 x1 = *reinterpret_cast<const float4*>(&xs[t][col + 4]);
          acc[t] = fmaf(wf[0], x0.x, acc[t]); acc[t] = fmaf(wf[1], x0.y, acc[t]);
          acc[t] = fmaf(wf[2], x0.z, acc[t]); acc[t] = fmaf(wf[3], x0.w, acc[t]);
          acc[t] = fmaf(wf[4], x1.x, acc[t]); acc[t] = fmaf(wf[5], x1.y, acc[t]);
          acc[t] = fmaf(wf[6], x1.z, acc[t]); acc[t] = fmaf(wf[7], x1.w, acc[t]);
        }
      }
    }
    }
  }
  float* wsp = a.ws + (((size_t)(nt * gridDim.z + tt) * gridDim.y + split) * a.tn) * kTileN;
#pragma unroll
  for (int t = 0; t < TT; ++t) wsp[(size_t)t * kTileN + r] = acc[t];
}

// ---- tcgen05 kernel ------------------------------------------------------------------------------
constexpr int kTcThreads = 320;  // warps 0-7 dequantise (0-3 also run the epilogue), 8 loads, 9 issues MMAs
constexpr int kRawStride = 5120;  // weight block padded to a multiple of 1024
constexpr int kPrefetchAhead = 12;  // weight blocks requested into L2 ahead of the copy

template <int MODE>
__global__ void __launch_bounds__(kTcThreads, 1) qmm_tc_kernel(const __grid_constant__ CUtensorMap xmap, QmmArgs a) {
  extern __shared__ unsigned char smem_raw[];
  // 1024-byte alignment: the 128B swizzle pattern is a function of the shared-memory address.
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int tn = a.tn, stages = a.stages;
  // [stage][A tile 16 KiB | X tile tn x 128 B] (1024-byte aligned for the 128B swizzle), then the raw
  // weight blocks of all stages (only 16-byte alignment needed), then the barriers.
  constexpr int kRaw = MODE == B200_Q_BF16 ? 0 : ((block_bytes(MODE) + 127) / 128) * 128;
  const int stage_stride = kTileN * 128 + tn * 128;
  auto a_tile = [&](int s) { return smem + (size_t)s * stage_stride; };
  auto x_tile = [&](int s) { return smem + (size_t)s * stage_stride + kTileN * 128; };
  auto raw_blk = [&](int s) { return smem + (size_t)stages * stage_stride + (size_t)s * kRaw; };
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)stages * (stage_stride + kRaw));
  uint64_t* loaded = bars;
  uint64_t* a_ready = bars + stages;
  uint64_t* mma_done = bars + 2 * stages;
  uint64_t* accum_ready = bars + 3 * stages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * stages + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nt = blockIdx.x, split = blockIdx.y;
  // Dense: blockIdx.z is a token tile.  Grouped: blockIdx.z is a work item {expert, first row,
  // rows} of the expert-sorted batch; unused items leave before touching any barrier.
  int t0 = blockIdx.z * tn, rows_here = min(tn, a.rows - t0);
  const unsigned char* blocks = a.blocks;
  if (a.items) {
    if ((int)blockIdx.z >= *a.n_items) return;
    const int4 it = a.items[blockIdx.z];
    blocks += (size_t)it.x * a.expert_stride;
    t0 = it.y;
    rows_here = it.z;
  }
  const int kc0 = split * a.chunks_per_split, kc1 = min(kc0 + a.chunks_per_split, a.kc);
  const int n_chunks = kc1 - kc0;
  constexpr int BB = block_bytes(MODE);
  uint32_t ncols = 32;
  while (ncols < (uint32_t)tn) ncols <<= 1;

  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      ptx::mbar_init(&loaded[s], 1);
      ptx::mbar_init(&a_ready[s], 2 * kTileN / 32);  // one arrival per dequantising warp
      ptx::mbar_init(&mma_done[s], 1);
    }
    ptx::mbar_init(accum_ready, 1);
    ptx::mbar_fence_init();
  }
  if (warp == 9) {
    ptx::tmem_alloc(tmem_slot, ncols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  bool ok = true;

  if (warp == 8) {
    if (lane == 0) {
      // The weight blocks of this CTA are contiguous in HBM: ask for them in L2 well ahead of the
      // stage that will copy them, so that a stage's refill waits for L2, not for HBM.
      const unsigned char* wsrc = blocks + ((size_t)nt * a.kc + kc0) * BB;
      for (int i = 0; i < min(n_chunks, kPrefetchAhead); ++i) ptx::bulk_prefetch_l2(wsrc + (size_t)i * BB, BB);
      int s = 0;
      uint32_t ph = 0;  // stage cursor kept incrementally: no division by the runtime stage count
      for (int i = 0; i < n_chunks && ok; ++i, ph ^= (s + 1 == stages), s = (s + 1 == stages) ? 0 : s + 1) {
        if (i + kPrefetchAhead < n_chunks) ptx::bulk_prefetch_l2(wsrc + (size_t)(i + kPrefetchAhead) * BB, BB);
        ok = ptx::mbar_wait(&mma_done[s], ph ^ 1u);
        if (!ok) break;
        ptx::mbar_expect_tx(&loaded[s], BB + tn * 128);
        // dense bf16 blocks are stored in the swizzled K-major layout and land in the MMA tile directly
        ptx::bulk_g2s(MODE == B200_Q_BF16 ? a_tile(s) : raw_blk(s), blocks + ((size_t)nt * a.kc + kc0 + i) * BB, BB,
                      &loaded[s]);
        ptx::tma_load_2d(x_tile(s), &xmap, (kc0 + i) * kChunkK, a.x_row0 + t0, &loaded[s]);
      }
    }
  } else if (warp == 9) {
    if (lane == 0) {
      const uint32_t idesc = ptx::umma_idesc_bf16(kTileN, tn);
      int s = 0;
      uint32_t ph = 0;  // stage cursor kept incrementally: no division by the runtime stage count
      for (int i = 0; i < n_chunks && ok; ++i, ph ^= (s + 1 == stages), s = (s + 1 == stages) ? 0 : s + 1) {
        ok = ptx::mbar_wait(&loaded[s], ph) && ptx::mbar_wait(&a_ready[s], ph);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        const uint64_t da = ptx::umma_desc_k_sw128(ptx::smem_u32(a_tile(s)));
        const uint64_t db = ptx::umma_desc_k_sw128(ptx::smem_u32(x_tile(s)));
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4)  // 4 x K16 per 64-column chunk; +32 bytes = +2 in 16-byte units
          ptx::umma_bf16(tmem_base, da + 2 * k4, db + 2 * k4, idesc, (i > 0 || k4 > 0) ? 1u : 0u);
        ptx::umma_commit(&mma_done[s]);
      }
      if (ok) ptx::umma_commit(accum_ready);
    }
  } else {
    // ---- dequantise: thread (r, plane) owns one 32-column half of weight row r ----
    const int r = tid & (kTileN - 1), my_plane = tid >> 7;
    int s = 0;
    uint32_t ph = 0;  // stage cursor kept incrementally: no division by the runtime stage count
    for (int i = 0; i < n_chunks && ok; ++i, ph ^= (s + 1 == stages), s = (s + 1 == stages) ? 0 : s + 1) {
      ok = ptx::mbar_wait(&loaded[s], ph);
      if (!ok) break;
      const unsigned char* blk = raw_blk(s);
      unsigned char* arow = a_tile(s) + r * 128;
      if (MODE != B200_Q_BF16) {
        const int plane = my_plane;
        const uint4 raw = reinterpret_cast<const uint4*>(blk + plane * kPlaneBytes)[r];
        __nv_bfloat162 s2, b2;
        row_params<MODE>(blk, r, plane, s2, b2);
        const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          const int chunk16 = plane * 4 + w;  // 16-byte chunk index within the 128-byte row
          *reinterpret_cast<uint4*>(arow + ((chunk16 ^ (r & 7)) << 4)) = dequant_word<MODE>(words[w], s2, b2);
        }
      }
      ptx::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&a_ready[s]);
    }
    // ---- accumulator -> f32 partial tile in scratch ----
    if (ok && warp < 4) ok = ptx::mbar_wait(accum_ready, 0);
    if (ok && warp < 4) {
      ptx::tc_fence_after_sync();
      const int n = nt * kTileN + warp * 32 + lane;
      // One K split and a small token tile: apply the epilogue here and skip the finish kernel.  With
      // large token tiles the strided 64-byte row stores cost more than the extra pass.
      const bool direct = gridDim.y == 1 && tn <= 64;
      const size_t n_pad = a.items ? (size_t)a.nt * kTileN : (size_t)kTileN;  // stride between token rows
      float* wsp = a.items ? a.ws + ((size_t)split * a.rows + t0) * n_pad + n
                           : a.ws + (((size_t)(nt * gridDim.z + blockIdx.z) * gridDim.y + split) * tn) * kTileN + warp * 32 + lane;
      for (int c0 = 0; c0 < rows_here; c0 += 32) {
        uint32_t v[32];
        ptx::tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, v);
        ptx::tmem_ld_wait();
        if (!direct) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (c0 + j < rows_here) wsp[(size_t)(c0 + j) * n_pad] = __uint_as_float(v[j]);
        } else if (a.epilogue == B200_EPI_SWIGLU) {
          // rows 2i / 2i+1 of the tile are gate_i / up_i: neighbouring lanes
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float mine = __uint_as_float(v[j]);
            const float other = __shfl_xor_sync(0xffffffffu, mine, 1);
            if ((lane & 1) == 0 && c0 + j < rows_here && n < a.n) {
              float g = mine, u = other;
              if (a.swiglu_limit > 0.f) { g = fminf(g, a.swiglu_limit); u = fminf(fmaxf(u, -a.swiglu_limit), a.swiglu_limit); }
              const int token = t0 + c0 + j;
              a.y[(size_t)token * (a.n / 2) + n / 2] = __float2bfloat16(g / (1.0f + __expf(-g)) * u * a.row_scale(token));
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (c0 + j < rows_here && n < a.n) {
              const int token = t0 + c0 + j;
              const size_t o = (size_t)token * a.n + n;
              float acc = __uint_as_float(v[j]);
              if (a.epilogue == B200_EPI_RESIDUAL) acc += __bfloat162float(a.residual[o]);
              a.y[o] = __float2bfloat16(acc * a.row_scale(token));
            }
          }
        }
      }
    }
  }
  if (!ok) atomicExch(a.err, B200_ERR_DEVICE_FLAGGED);
  ptx::tc_fence_before_sync();
  const int any_bad = __syncthreads_or(!ok);
  if (warp == 9) ptx::tmem_dealloc(tmem_base, ncols);
  (void)any_bad;
}

// One 32-token batch of accumulators (v[j] = token c0+j, weight row n) to scratch or to the output.
__device__ __forceinline__ void tile_epilogue_store(const QmmArgs& a, const uint32_t (&v)[32], int c0, int rows_here, int t0,
                                                    int n, int lane, bool direct, float* wsp, size_t n_pad) {
  if (!direct) {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (c0 + j < rows_here) wsp[(size_t)(c0 + j) * n_pad] = __uint_as_float(v[j]);
  } else if (a.epilogue == B200_EPI_SWIGLU) {
    // rows 2i / 2i+1 of the tile are gate_i / up_i: neighbouring lanes.  The even lane takes token j,
    // the odd lane token j+1 (one exchange per token pair, no lane idles in the arithmetic).
    const float L = a.swiglu_limit;
    const bool odd = lane & 1;
#pragma unroll
    for (int j = 0; j < 32; j += 2) {
      const float a0 = __uint_as_float(v[j]), a1 = __uint_as_float(v[j + 1]);
      const float got = __shfl_xor_sync(0xffffffffu, odd ? a0 : a1, 1);
      const int tok = c0 + j + (int)odd;
      if (tok < rows_here && n < a.n) {
        float g = odd ? got : a0, u = odd ? a1 : got;
        if (L > 0.f) { g = fminf(g, L); u = fminf(fmaxf(u, -L), L); }
        const int token = t0 + tok;
        a.y[(size_t)token * (a.n / 2) + n / 2] = __float2bfloat16(g / (1.0f + __expf(-g)) * u * a.row_scale(token));
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (c0 + j < rows_here && n < a.n) {
        const int token = t0 + c0 + j;
        const size_t o = (size_t)token * a.n + n;
        float acc = __uint_as_float(v[j]);
        if (a.epilogue == B200_EPI_RESIDUAL) acc += __bfloat162float(a.residual[o]);
        a.y[o] = __float2bfloat16(acc * a.row_scale(token));
      }
    }
  }
}

// ---- tcgen05 kernel with the weight operand in tensor memory -----------------------------------
// In qmm_tc_kernel a stage is one unit: weight block + activation tile + the 16 KiB dequantised
// tile travel together, a stage lives for load + dequantise + MMA and only three of them fit a CTA.
// Here the lifetimes are separated and the dequantised tile leaves shared memory:
//   * raw weight blocks: a ring of PW slots of two consecutive blocks (128 K columns, 9 KiB, one bulk
//     copy).  A slot is released as soon as the dequantising warps hold its words in registers;
//   * activation tiles (two of tn x 128 B per slot, re-read from L2 by every CTA): their own ring of
//     PX slots, released by the MMAs that read them.  Sharing one ring with the weights, as an earlier
//     form of this kernel did, let the activation tiles crowd out the weight bytes in flight;
//   * dequantised weights: warps 0-7 write them straight into tensor memory (tcgen05.st; thread r
//     owns lane r = weight row r, a 64-column chunk is 32 columns of packed bf16 pairs), into a ring
//     of Q slots of 64 columns behind the accumulator, and tcgen05.mma takes its A operand from there.
//     No swizzled shared-memory tile, no proxy fence, and the MMA reads only the activation tile from
//     shared memory.
// Every handshake covers a pair of chunks: with one chunk per handshake a dequantising warp spent about
// 120 of its 186 instructions per chunk on waits, arrivals and ring bookkeeping (instruction counters),
// and the MMA thread 500 cycles per chunk of which the two commits took more than the four MMAs.
constexpr int kTcaThreads = 352;  // warps 0-7 dequantise (0-3 also run the epilogue), 8 loads weights, 9 issues MMAs, 10 loads activations
constexpr int kTcaMaxWeightSlots = 24;

template <int MODE>
__global__ void __launch_bounds__(kTcaThreads, 2) qmm_tca_kernel(const __grid_constant__ CUtensorMap xmap, QmmArgs a) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  constexpr int BB = block_bytes(MODE);
  static_assert(BB % 128 == 0, "two blocks are copied as one run");
  const int tn = a.tn, PW = a.stages, PX = a.x_slots, Q = a.a_slots;
  const uint32_t x_slot_bytes = 2u * (uint32_t)tn * 128u;
  unsigned char* wring = smem + (size_t)PX * x_slot_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(wring + (size_t)PW * 2 * BB);
  // barrier addresses in the shared window (the hot loops keep them as 32-bit integers)
  const uint32_t smem_u = ptx::smem_u32(smem), wring_u = ptx::smem_u32(wring), bars_u = ptx::smem_u32(bars);
  const uint32_t wfull = bars_u;                                  // [PW] a pair of raw blocks has landed
  const uint32_t wfree = wfull + 8u * PW;                         // [PW] every dequantising warp has read it
  const uint32_t xfull = wfree + 8u * PW;                         // [PX] a pair of activation tiles has landed
  const uint32_t xfree = xfull + 8u * PX;                         // [PX] the MMAs reading it are done
  const uint32_t a_ready = xfree + 8u * PX;                       // [Q] a dequantised pair is in tensor memory
  const uint32_t a_free = a_ready + 8u * Q;                       // [Q] the MMAs reading it are done
  uint64_t* accum_ready = bars + 2 * PW + 2 * PX + 2 * Q;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_ready + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nt = blockIdx.x, split = blockIdx.y;
  int t0 = blockIdx.z * tn, rows_here = min(tn, a.rows - t0);
  const unsigned char* blocks = a.blocks;
  if (a.items) {
    if ((int)blockIdx.z >= *a.n_items) return;
    const int4 it = a.items[blockIdx.z];
    blocks += (size_t)it.x * a.expert_stride;
    t0 = it.y;
    rows_here = it.z;
  }
  const int kc0 = split * a.chunks_per_split, kc1 = min(kc0 + a.chunks_per_split, a.kc);
  const int n_chunks = kc1 - kc0, n_pairs = (n_chunks + 1) >> 1;
  uint32_t acc_cols = 32;
  while (acc_cols < (uint32_t)tn) acc_cols <<= 1;
  uint32_t ncols = 32;
  while (ncols < acc_cols + 64u * (uint32_t)Q) ncols <<= 1;

  if (tid == 0) {
    for (int s = 0; s < PW; ++s) {
      ptx::mbar_init(&bars[s], 1);
      ptx::mbar_init(&bars[PW + s], 2 * kTileN / 32);  // one arrival per dequantising warp
    }
    for (int s = 0; s < PX; ++s) {
      ptx::mbar_init(&bars[2 * PW + s], 1);
      ptx::mbar_init(&bars[2 * PW + PX + s], 1);
    }
    for (int q = 0; q < Q; ++q) {
      ptx::mbar_init(&bars[2 * PW + 2 * PX + q], 2 * kTileN / 32);  // one arrival per dequantising warp (256 single arrivals cost ~500 cycles)
      ptx::mbar_init(&bars[2 * PW + 2 * PX + Q + q], 1);
    }
    ptx::mbar_init(accum_ready, 1);
    ptx::mbar_fence_init();
  }
  if (warp == 9) {
    ptx::tmem_alloc(tmem_slot, ncols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t a_col0 = tmem_base + acc_cols;
  bool ok = true;

  if (warp == 8) {
    if (lane == 0) {  // the weight stream
      const unsigned char* wsrc = blocks + ((size_t)nt * a.kc + kc0) * BB;
      int s = 0;
      uint32_t ph = 1;
      for (int p = 0; p < n_pairs; ++p) {
        ok = ptx::mbar_wait_addr(wfree + 8u * s, ph);
        if (!ok) break;
        const uint32_t bytes = (2 * p + 1 < n_chunks) ? 2u * BB : (uint32_t)BB;
        ptx::mbar_expect_tx_addr(wfull + 8u * s, bytes);
        ptx::bulk_g2s_addr(wring_u + (uint32_t)s * 2u * BB, wsrc + (size_t)p * 2 * BB, bytes, wfull + 8u * s);
        if (++s == PW) { s = 0; ph ^= 1u; }
      }
    }
  } else if (warp == 10) {
    if (lane == 0) {  // the activation tiles
      int s = 0;
      uint32_t ph = 1;
      for (int p = 0; p < n_pairs; ++p) {
        ok = ptx::mbar_wait_addr(xfree + 8u * s, ph);
        if (!ok) break;
        const bool two = 2 * p + 1 < n_chunks;
        uint64_t* bar = &bars[2 * PW + s];
        ptx::mbar_expect_tx(bar, two ? x_slot_bytes : x_slot_bytes / 2);
        unsigned char* dst = smem + (size_t)s * x_slot_bytes;
        ptx::tma_load_2d(dst, &xmap, (kc0 + 2 * p) * kChunkK, a.x_row0 + t0, bar);
        if (two) ptx::tma_load_2d(dst + x_slot_bytes / 2, &xmap, (kc0 + 2 * p + 1) * kChunkK, a.x_row0 + t0, bar);
        if (++s == PX) { s = 0; ph ^= 1u; }
      }
    }
  } else if (warp == 9) {
    if (lane == 0) {
      const uint32_t idesc = ptx::umma_idesc_bf16(kTileN, tn);
      int s = 0, q = 0;
      uint32_t ph = 0, qh = 0;
      for (int p = 0; p < n_pairs; ++p) {
        ok = ptx::mbar_wait_addr(xfull + 8u * s, ph) && ptx::mbar_wait_addr(a_ready + 8u * q, qh);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        const uint64_t db = ptx::umma_desc_k_sw128(smem_u + (uint32_t)s * x_slot_bytes);
        const uint64_t db_step = (uint64_t)(x_slot_bytes / 2) >> 4;  // second tile of the pair (descriptor addresses count 16 bytes)
        const uint32_t acol = a_col0 + (uint32_t)(q * 64);
        const int n_here = (2 * p + 1 < n_chunks) ? 2 : 1;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          if (j < n_here) {
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4)
              ptx::umma_bf16_tmem_a(tmem_base, acol + (uint32_t)(j * 32 + k4 * 8), db + j * db_step + 2 * k4, idesc,
                                    (p > 0 || j > 0 || k4 > 0) ? 1u : 0u);
          }
        }
        ptx::umma_commit(&bars[2 * PW + PX + s]);
        ptx::umma_commit(&bars[2 * PW + 2 * PX + Q + q]);
        if (++s == PX) { s = 0; ph ^= 1u; }
        if (++q == Q) { q = 0; qh ^= 1u; }
      }
      if (ok) ptx::umma_commit(accum_ready);
    }
  } else {
    // ---- dequantise: thread (r, plane) owns one 32-column half of weight row r = tensor-memory lane r ----
    const int r = tid & (kTileN - 1), plane = tid >> 7;
    const uint32_t my_taddr = a_col0 + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(plane * 16);
    const unsigned char* my_raw = wring + plane * kPlaneBytes + r * 16;
    int s = 0, q = 0, pending_q = -1;
    uint32_t ph = 0, qh = 1;
    // The stores of pair p into tensor memory are left in flight while pair p+1 is loaded and its first
    // chunk dequantised; they are waited for, and their slot announced, just before the next store.
    for (int p = 0; p < n_pairs; ++p) {
      ok = ptx::mbar_wait_addr(wfull + 8u * s, ph);
      if (!ok) break;
      const bool two = 2 * p + 1 < n_chunks;
      const unsigned char* blk = wring + (size_t)s * 2 * BB;
      const uint4 raw0 = *reinterpret_cast<const uint4*>(my_raw + (size_t)s * 2 * BB);
      uint4 raw1 = make_uint4(0u, 0u, 0u, 0u);
      __nv_bfloat162 s20, b20, s21, b21;
      row_params<MODE>(blk, r, plane, s20, b20);
      s21 = s20; b21 = b20;
      if (two) {
        raw1 = *reinterpret_cast<const uint4*>(my_raw + (size_t)s * 2 * BB + BB);
        row_params<MODE>(blk + BB, r, plane, s21, b21);
      }
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_addr(wfree + 8u * s);  // this warp's share of the pair is in registers
      uint32_t v[16];
      {
        const uint32_t words[4] = {raw0.x, raw0.y, raw0.z, raw0.w};
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          const uint4 d = dequant_word<MODE>(words[w], s20, b20);
          v[4 * w] = d.x; v[4 * w + 1] = d.y; v[4 * w + 2] = d.z; v[4 * w + 3] = d.w;
        }
      }
      if (pending_q >= 0) {
        ptx::tmem_st_wait();
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive_addr(a_ready + 8u * pending_q);
        pending_q = -1;
      }
      ok = ptx::mbar_wait_addr(a_free + 8u * q, qh);
      if (!ok) break;
      ptx::tc_fence_after_sync();
      ptx::tmem_st16(my_taddr + (uint32_t)(q * 64), v);
      if (two) {
        const uint32_t words[4] = {raw1.x, raw1.y, raw1.z, raw1.w};
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          const uint4 d = dequant_word<MODE>(words[w], s21, b21);
          v[4 * w] = d.x; v[4 * w + 1] = d.y; v[4 * w + 2] = d.z; v[4 * w + 3] = d.w;
        }
        ptx::tmem_st16(my_taddr + (uint32_t)(q * 64 + 32), v);
      }
      pending_q = q;
      if (++s == PW) { s = 0; ph ^= 1u; }
      if (++q == Q) { q = 0; qh ^= 1u; }
    }
    if (pending_q >= 0) {
      ptx::tmem_st_wait();
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (ok && lane == 0) ptx::mbar_arrive_addr(a_ready + 8u * pending_q);
    }
    // ---- accumulator -> f32 partial tile in scratch ----
    if (ok && warp < 4) ok = ptx::mbar_wait(accum_ready, 0);
    if (ok && warp < 4) {
      ptx::tc_fence_after_sync();
      const int n = nt * kTileN + warp * 32 + lane;
      const bool direct = gridDim.y == 1 && (tn <= 64 || a.direct_large);
      const size_t n_pad = a.items ? (size_t)a.nt * kTileN : (size_t)kTileN;
      float* wsp = a.items ? a.ws + ((size_t)split * a.rows + t0) * n_pad + n
                           : a.ws + (((size_t)(nt * gridDim.z + blockIdx.z) * gridDim.y + split) * tn) * kTileN + warp * 32 + lane;
      for (int c0 = 0; c0 < rows_here; c0 += 32) {
        uint32_t v[32];
        ptx::tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, v);
        ptx::tmem_ld_wait();
        tile_epilogue_store(a, v, c0, rows_here, t0, n, lane, direct, wsp, n_pad);
      }
    }
  }
  if (!ok) atomicExch(a.err, B200_ERR_DEVICE_FLAGGED);
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) ptx::tmem_dealloc(tmem_base, ncols);
}

// ---- tcgen05 kernel for large batches: two weight tiles per CTA ---------------------------------
// With 129..256 rows per token tile the kernel above moves a 32 KiB activation tile through
// shared memory for every 4.6 KiB weight block, and at one CTA per SM only four such stages fit:
// the load -> dequantise -> MMA -> release chain of a stage is longer than the work the other
// stages hold, and the tensor pipe idles.  Here a CTA owns TWO adjacent 128-row weight tiles and
// multiplies both with the same activation tile (two accumulators, 2 x 256 tensor-memory columns):
// a stage carries twice the MMA work per activation byte, so the same shared memory hides twice
// the latency and the L2 -> SM activation traffic per flop halves.  16 dequant warps (one thread
// per weight row and 32-column plane of either tile), one loader warp, one MMA warp.
constexpr int kTc2Threads = 19 * 32;  // warps 0-15 dequantise, 16 streams the weights, 17 issues MMAs, 18 loads activation tiles
constexpr int kTc2DequantThreads = 16 * 32;

// Quantised weights: the raw 4-bit blocks have a ring of their own (SR slots of two blocks), released as
// soon as the dequantising warps hold the words in registers, so the weight stream runs ahead of the
// stages by the DRAM latency instead of starting when an MMA retires a stage (load 1500 cycles ->
// dequantise 700 -> MMA 1024 per stage of three was longer than the MMAs of the other two stages).
// A stage holds the two dequantised tiles and the activation tile, which comes from L2 while the
// dequantisation runs.  Dense bf16 blocks land in the stage's MMA tiles directly (SR = stages there).
template <int MODE>
__global__ void __launch_bounds__(kTc2Threads, 1) qmm_tc2_kernel(const __grid_constant__ CUtensorMap xmap, QmmArgs a) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  constexpr int BB = block_bytes(MODE);
  constexpr bool kDense = MODE == B200_Q_BF16;
  constexpr int RB = kDense ? 0 : ((BB + 127) / 128) * 128;
  const int tn = a.tn, stages = a.stages, SR = a.x_slots;
  const int stage_stride = 2 * kTileN * 128 + tn * 128;
  auto a_tile = [&](int s, int tile) { return smem + (size_t)s * stage_stride + tile * (kTileN * 128); };
  auto x_tile = [&](int s) { return smem + (size_t)s * stage_stride + 2 * kTileN * 128; };
  auto raw_blk = [&](int sr, int tile) { return smem + (size_t)stages * stage_stride + (size_t)(sr * 2 + tile) * RB; };
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)stages * stage_stride + (size_t)(kDense ? 0 : SR) * 2 * RB);
  uint64_t* x_loaded = bars;                   // [stages] activation tile has landed
  uint64_t* a_ready = bars + stages;           // [stages] both MMA tiles are written (or, dense, have landed)
  uint64_t* mma_done = bars + 2 * stages;      // [stages] the MMAs reading the stage are done
  uint64_t* raw_full = bars + 3 * stages;      // [SR] raw blocks have landed
  uint64_t* raw_free = bars + 3 * stages + SR; // [SR] every dequantising warp has read them
  uint64_t* accum_ready = bars + 3 * stages + 2 * SR;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_ready + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int pair = blockIdx.x, split = blockIdx.y, tt = blockIdx.z;
  const int t0 = tt * tn, rows_here = min(tn, a.rows - t0);
  const int nt0 = 2 * pair;
  const int n_tiles = min(2, a.nt - nt0);  // an odd tile count leaves the last CTA one tile
  const int kc0 = split * a.chunks_per_split, kc1 = min(kc0 + a.chunks_per_split, a.kc);
  const int n_chunks = kc1 - kc0;
  constexpr uint32_t kCols = 512;  // accumulator of tile 0 at column 0, of tile 1 at column 256

  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      ptx::mbar_init(&x_loaded[s], 1);
      ptx::mbar_init(&a_ready[s], kTc2DequantThreads / 32);  // one arrival per dequantising warp
      ptx::mbar_init(&mma_done[s], 1);
    }
    for (int s = 0; s < SR; ++s) {
      ptx::mbar_init(&raw_full[s], 1);
      ptx::mbar_init(&raw_free[s], kTc2DequantThreads / 32);
    }
    ptx::mbar_init(accum_ready, 1);
    ptx::mbar_fence_init();
  }
  if (warp == 17) {
    ptx::tmem_alloc(tmem_slot, kCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  bool ok = true;

  if (warp == 16) {
    if (lane == 0) {  // the weight stream
      int s = 0;
      uint32_t ph = 1;
      for (int i = 0; i < n_chunks; ++i) {
        // dense blocks go into the stage's MMA tiles, so their slot is the stage and frees with its MMAs
        ok = ptx::mbar_wait(kDense ? &mma_done[s] : &raw_free[s], ph);
        if (!ok) break;
        ptx::mbar_expect_tx(&raw_full[s], n_tiles * BB);
        for (int tile = 0; tile < n_tiles; ++tile)
          ptx::bulk_g2s(kDense ? a_tile(s, tile) : raw_blk(s, tile), a.blocks + ((size_t)(nt0 + tile) * a.kc + kc0 + i) * BB, BB,
                        &raw_full[s]);
        if (++s == SR) { s = 0; ph ^= 1u; }
      }
    }
  } else if (warp == 18) {
    if (lane == 0) {  // the activation tiles
      int s = 0;
      uint32_t ph = 1;
      for (int i = 0; i < n_chunks; ++i) {
        ok = ptx::mbar_wait(&mma_done[s], ph);
        if (!ok) break;
        ptx::mbar_expect_tx(&x_loaded[s], tn * 128);
        ptx::tma_load_2d(x_tile(s), &xmap, (kc0 + i) * kChunkK, a.x_row0 + t0, &x_loaded[s]);
        if (++s == stages) { s = 0; ph ^= 1u; }
      }
    }
  } else if (warp == 17) {
    if (lane == 0) {
      const uint32_t idesc = ptx::umma_idesc_bf16(kTileN, tn);
      int s = 0;
      uint32_t ph = 0;
      for (int i = 0; i < n_chunks; ++i) {
        ok = ptx::mbar_wait(&x_loaded[s], ph) && ptx::mbar_wait(&a_ready[s], ph);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        const uint64_t db = ptx::umma_desc_k_sw128(ptx::smem_u32(x_tile(s)));
        for (int tile = 0; tile < n_tiles; ++tile) {
          const uint64_t da = ptx::umma_desc_k_sw128(ptx::smem_u32(a_tile(s, tile)));
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4)
            ptx::umma_bf16(tmem_base + tile * 256, da + 2 * k4, db + 2 * k4, idesc, (i > 0 || k4 > 0) ? 1u : 0u);
        }
        ptx::umma_commit(&mma_done[s]);
        if (++s == stages) { s = 0; ph ^= 1u; }
      }
      if (ok) ptx::umma_commit(accum_ready);
    }
  } else {
    // ---- dequantise: thread (r, plane, tile) owns one 32-column half of weight row r of a tile ----
    const int r = tid & (kTileN - 1), plane = (tid >> 7) & 1, tile = tid >> 8;
    int s = 0, sr = 0;
    uint32_t ph = 0, phr = 0;
    for (int i = 0; i < n_chunks; ++i) {
      ok = ptx::mbar_wait(&raw_full[sr], phr);
      if (!ok) break;
      if (!kDense) {
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        __nv_bfloat162 s2, b2;
        if (tile < n_tiles) {
          const unsigned char* blk = raw_blk(sr, tile);
          raw = reinterpret_cast<const uint4*>(blk + plane * kPlaneBytes)[r];
          row_params<MODE>(blk, r, plane, s2, b2);
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&raw_free[sr]);  // this warp's share of the blocks is in registers
        ok = ptx::mbar_wait(&mma_done[s], ph ^ 1u);     // the stage's MMA tiles may be overwritten
        if (!ok) break;
        if (tile < n_tiles) {
          unsigned char* arow = a_tile(s, tile) + r * 128;
          const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            const int chunk16 = plane * 4 + w;
            *reinterpret_cast<uint4*>(arow + ((chunk16 ^ (r & 7)) << 4)) = dequant_word<MODE>(words[w], s2, b2);
          }
        }
        ptx::fence_proxy_async_smem();
      }
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&a_ready[s]);
      if (++s == stages) { s = 0; ph ^= 1u; }
      if (++sr == SR) { sr = 0; phr ^= 1u; }
    }
    // ---- accumulators: warp w reads lanes 32*(w%4); warps 4g..4g+3 take tile g/2, column half g%2 ----
    if (ok) ok = ptx::mbar_wait(accum_ready, 0);
    const int grp = warp >> 2, etile = grp >> 1, half = grp & 1;
    // SwiGLU written by this kernel (no K split): the outputs go through the idle stage buffers as
    // bf16 [token][tile][64] and leave as 16-byte stores, 256 contiguous bytes per token for the tile
    // pair.  Stores of 64 bytes per token straight from the accumulator layout (one instruction per
    // token and warp) took a quarter of the kernel's time at 256 rows.
    const bool staged = gridDim.y == 1 && a.epilogue == B200_EPI_SWIGLU && a.n % 16 == 0;
    if (staged) {
      uint32_t all_ok;
      asm volatile(
          "{\n\t.reg .pred p, q;\n\t"
          "setp.ne.b32 p, %1, 0;\n\t"
          "bar.red.and.pred q, 1, 512, p;\n\t"
          "selp.u32 %0, 1, 0, q;\n\t}"
          : "=r"(all_ok)
          : "r"((uint32_t)ok)
          : "memory");
      if (all_ok) {
        ptx::tc_fence_after_sync();
        __nv_bfloat16* stage_h = reinterpret_cast<__nv_bfloat16*>(smem);
        const float L = a.swiglu_limit;
        if (etile < n_tiles) {
          const int lq = warp & 3;
          const int ch = ((tn / 2 + 31) / 32) * 32;
          const int c_end = min(rows_here, (half + 1) * ch);
          for (int c0 = half * ch; c0 < c_end; c0 += 32) {
            uint32_t v[32];
            ptx::tmem_ld32(tmem_base + ((uint32_t)(lq * 32) << 16) + (uint32_t)(etile * 256 + c0), v);
            const float rs_mine = c0 + lane < rows_here ? a.row_scale(t0 + c0 + lane) : 0.f;
            ptx::tmem_ld_wait();
            // lanes 2i / 2i+1 hold gate_i / up_i of every token: the even lane takes token j, the odd
            // lane token j+1, one exchange per token pair and no idle lanes in the arithmetic
            const bool odd = lane & 1;
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              const float a0 = __uint_as_float(v[j]), a1 = __uint_as_float(v[j + 1]);
              const float got = __shfl_xor_sync(0xffffffffu, odd ? a0 : a1, 1);
              float g = odd ? got : a0, u = odd ? a1 : got;
              const float rs = __shfl_sync(0xffffffffu, rs_mine, j + (int)odd);
              if (L > 0.f) { g = fminf(g, L); u = fminf(fmaxf(u, -L), L); }
              stage_h[((size_t)(c0 + j + (int)odd) * 2 + etile) * 64 + lq * 16 + (lane >> 1)] =
                  __float2bfloat16(g / (1.0f + __expf(-g)) * u * rs);
            }
          }
        }
        asm volatile("bar.sync 1, 512;" ::: "memory");
        const int n_out = a.n / 2;
        for (int idx = tid; idx < rows_here * 16; idx += kTc2DequantThreads) {
          const int tok = idx >> 4, c16 = idx & 15, tile = c16 >> 3;
          const int col = (nt0 + tile) * 64 + (c16 & 7) * 8;
          if (tile < n_tiles && col < n_out)
            *reinterpret_cast<uint4*>(a.y + (size_t)(t0 + tok) * n_out + col) = *reinterpret_cast<const uint4*>(stage_h + (size_t)idx * 8);
        }
      }
    } else if (ok && etile < n_tiles) {
      ptx::tc_fence_after_sync();
      const int lq = warp & 3;
      const int nt = nt0 + etile, n = nt * kTileN + lq * 32 + lane;
      const bool direct = gridDim.y == 1;
      float* wsp = a.ws + (((size_t)(nt * gridDim.z + tt) * gridDim.y + split) * tn) * kTileN + lq * 32 + lane;
      const int ch = ((tn / 2 + 31) / 32) * 32;
      const int c_end = min(rows_here, (half + 1) * ch);
      for (int c0 = half * ch; c0 < c_end; c0 += 32) {
        uint32_t v[32];
        ptx::tmem_ld32(tmem_base + ((uint32_t)(lq * 32) << 16) + (uint32_t)(etile * 256 + c0), v);
        ptx::tmem_ld_wait();
        tile_epilogue_store(a, v, c0, rows_here, t0, n, lane, direct, wsp, (size_t)kTileN);
      }
    }
  }
  if (!ok) atomicExch(a.err, B200_ERR_DEVICE_FLAGGED);
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 17) ptx::tmem_dealloc(tmem_base, kCols);
}

// ---- small-batch kernel: register dequantisation + mma.sync -------------------------------------
// For a handful of rows the matmul is a weight-streaming problem, and the tcgen05 route above pays
// a long dependent chain per chunk (dequantise into a 16 KiB shared tile -> MMA -> commit -> slot
// free).  Here nothing but the raw 4-bit blocks passes through shared memory: a producer warp
// keeps a deep ring of raw blocks in flight with bulk copies; each of 8 consumer warps owns one
// 16-row slice of the 128-row tile and feeds mma.sync (m16n8k16, bf16) from registers.  Tokens are
// the MMA N dimension: NT8 tiles of 8.  The kernel is bound by instruction issue, so the work per
// block is kept minimal:
//   * The MMA's K slots are a free permutation as long as both operands agree.  Lane t of a quad
//     takes the 8 columns of word t of each plane (columns 8t..8t+7 and 32+8t..32+8t+7): one
//     32-bit load per row and plane yields all four column pairs the lane needs for two K steps,
//     and the matching activations are 16 contiguous bytes of the staged slab.
//   * Affine weights are not dequantised at all: 0x4300 | q is the bf16 value 128 + q, which goes
//     into the MMA as it is.  One block is one quantisation group, so per block
//         y += s * (acc - 128 * sum_x) + b * sum_x = s * acc + (b - 128 s) * sum_x
//     with sum_x (per token and group) computed once per CTA while the slab is staged.
constexpr int kGemvConsumers = 8;
constexpr int kGemvThreads = (kGemvConsumers + 1) * 32;
constexpr int kGemvRawStages = 6;  // ring slots of two blocks each
constexpr int kSlabPad = 64;  // row stride = chunks*128 + 64: the 8 lanes of a 16-byte load phase hit 8 bank groups

__device__ __forceinline__ void mma_bf16_full(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// The same with a zero accumulator input (first K step of a block).
__device__ __forceinline__ void mma_bf16_zero(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
               : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
}

// Column pair i of a word -> MMA operand.  Affine: the raw code as bf16 128+q.  MXFP4: dequantised.
template <int MODE>
__device__ __forceinline__ uint32_t operand_pair(uint32_t word, int i, __nv_bfloat162 s2) {
  const uint32_t t = (word >> (4 * i)) & 0x000F000Fu;
  if (MODE == B200_Q_AFFINE4_G64) return t | 0x43004300u;
  uint32_t u = ((t & 0x00080008u) << 12) | ((t & 0x00070007u) << 6);
  const uint32_t c64 = 0x5F805F80u;  // 2^64
  __nv_bfloat162 r = __hmul2(__hmul2(*reinterpret_cast<__nv_bfloat162*>(&u), *reinterpret_cast<const __nv_bfloat162*>(&c64)), s2);
  return *reinterpret_cast<uint32_t*>(&r);
}

template <int MODE, int NT8>
__global__ void __launch_bounds__(kGemvThreads, NT8 >= 4 ? 1 : 2) qmm_mma_kernel(QmmArgs a) {
  extern __shared__ __align__(128) unsigned char gsm[];
  const int stages = a.stages;
  constexpr int kSlotBytes = 2 * kRawStride;  // a ring slot holds the blocks of two adjacent weight tiles
  uint64_t* raw_full = reinterpret_cast<uint64_t*>(gsm + (size_t)stages * kSlotBytes);
  uint64_t* raw_free = raw_full + stages;
  // Activation slab of this CTA's K range (NT8*8 token rows), then sum_x [chunk][token] (affine).
  unsigned char* slab = reinterpret_cast<unsigned char*>(raw_free + stages);
  constexpr int TILE = NT8 * 8;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  // Persistent CTA: a fixed K split, and every `groups`-th pair of weight tiles starting at pair
  // `grp`.  The activation slab is staged once; the weight ring never drains between pairs.  Both
  // tiles of a pair share the wait, the activation loads and the loop bookkeeping of a chunk.
  const int split = blockIdx.x % a.splits, grp = blockIdx.x / a.splits, groups = gridDim.x / a.splits;
  const int tt = blockIdx.y, t0 = tt * TILE;
  const int kc0 = split * a.chunks_per_split, kc1 = min(kc0 + a.chunks_per_split, a.kc), n_chunks = kc1 - kc0;
  const int n_pairs = (a.nt + 1) / 2;
  const int n_items = grp < n_pairs ? (n_pairs - grp + groups - 1) / groups : 0;
  constexpr int BB = block_bytes(MODE);
  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      ptx::mbar_init(&raw_full[s], 1);
      ptx::mbar_init(&raw_free[s], kGemvConsumers);
    }
    ptx::mbar_fence_init();
  }
  __syncthreads();
  const int slab_stride = a.chunks_per_split * (kChunkK * 2) + kSlabPad;
  float* sum_x = reinterpret_cast<float*>(slab + (size_t)TILE * slab_stride);
  bool ok = true;
  // The producer starts the weight stream at once; the consumer warps meanwhile stage the
  // activations (they meet on named barrier 1, which the producer warp is not part of).
  if (warp == kGemvConsumers) {
    if (lane == 0) {
      int s = 0;
      uint32_t phase = 1;
      for (int item = 0; item < n_items && ok; ++item) {
        const int nt0 = 2 * (grp + item * groups);
        const int tiles = min(2, a.nt - nt0);
        const unsigned char* src = a.blocks + ((size_t)nt0 * a.kc + kc0) * BB;
        for (int i = 0; i < n_chunks; ++i) {
          ok = ptx::mbar_wait(&raw_free[s], phase);
          if (!ok) break;
          ptx::mbar_expect_tx(&raw_full[s], tiles * BB);
          for (int u = 0; u < tiles; ++u)
            ptx::bulk_g2s(gsm + (size_t)s * kSlotBytes + u * kRawStride, src + ((size_t)u * a.kc + i) * BB, BB, &raw_full[s]);
          if (++s == stages) { s = 0; phase ^= 1u; }
        }
      }
    }
  } else {
    const int vec_per_row = n_chunks * (kChunkK * 2 / 16);
    for (int idx = tid; idx < TILE * vec_per_row; idx += kGemvConsumers * 32) {
      const int row = idx / vec_per_row, v = idx - row * vec_per_row;
      uint4 val = make_uint4(0u, 0u, 0u, 0u);
      if (t0 + row < a.rows) val = *reinterpret_cast<const uint4*>(a.x + (size_t)(t0 + row) * a.k + (size_t)kc0 * kChunkK + v * 8);
      *reinterpret_cast<uint4*>(slab + (size_t)row * slab_stride + v * 16) = val;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kGemvConsumers * 32) : "memory");
    if (MODE == B200_Q_AFFINE4_G64) {
      for (int idx = tid; idx < TILE * n_chunks; idx += kGemvConsumers * 32) {
        const int c = idx / TILE, row = idx - c * TILE;
        const uint4* src = reinterpret_cast<const uint4*>(slab + (size_t)row * slab_stride + c * (kChunkK * 2));
        float sum = 0.f;
#pragma unroll
        for (int v = 0; v < 8; ++v) {
          const uint4 q = src[v];
          sum += ptx::bf16_lo(q.x) + ptx::bf16_hi(q.x) + ptx::bf16_lo(q.y) + ptx::bf16_hi(q.y);
          sum += ptx::bf16_lo(q.z) + ptx::bf16_hi(q.z) + ptx::bf16_lo(q.w) + ptx::bf16_hi(q.w);
        }
        sum_x[idx] = sum;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kGemvConsumers * 32) : "memory");
    }
    const int rA = warp * 16 + g, rB = rA + 8;
    const unsigned char* xlane = slab + (size_t)g * slab_stride + 16 * t;  // token g of tile j: + j*8*slab_stride
    // Loop state is kept incremental (slot, phase, pointers): the loop is bound by instruction issue.
    const uint32_t full0 = ptx::smem_u32(raw_full), free0 = ptx::smem_u32(raw_free);
    const uint32_t lane_ofs = (uint32_t)(rA * 16 + 4 * t);
    uint32_t slot = 0, phase = 0;
    for (int item = 0; item < n_items && ok; ++item) {
      const int nt0 = 2 * (grp + item * groups);
      const bool two = nt0 + 1 < a.nt;
      float y[2][NT8][4];
#pragma unroll
      for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int j = 0; j < NT8; ++j) { y[u][j][0] = y[u][j][1] = y[u][j][2] = y[u][j][3] = 0.f; }
      const unsigned char* px = xlane;
      const float* psx = sum_x + 2 * t;
      for (int i = 0; i < n_chunks; ++i) {
        // activations of the chunk first: they do not depend on the weights
        uint4 xv[NT8][2];
#pragma unroll
        for (int j = 0; j < NT8; ++j) {
          xv[j][0] = *reinterpret_cast<const uint4*>(px + (size_t)(j * 8) * slab_stride);
          xv[j][1] = *reinterpret_cast<const uint4*>(px + (size_t)(j * 8) * slab_stride + 64);
        }
        float2 sx[NT8];
        if (MODE == B200_Q_AFFINE4_G64) {
#pragma unroll
          for (int j = 0; j < NT8; ++j) sx[j] = *reinterpret_cast<const float2*>(psx + j * 8);
        }
        ok = ptx::mbar_wait_addr(full0 + 8 * slot, phase);
        if (!ok) break;
        const unsigned char* slot_base = gsm + slot * kSlotBytes;
        uint32_t wa[2][2], wb[2][2];
        float sA[2], bA[2], sB[2], bB[2];
        __nv_bfloat162 mA[2][2], mB[2][2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          if (u == 1 && !two) break;
          const unsigned char* blk = slot_base + u * kRawStride;
#pragma unroll
          for (int plane = 0; plane < 2; ++plane) {
            wa[u][plane] = *reinterpret_cast<const uint32_t*>(blk + lane_ofs + plane * kPlaneBytes);
            wb[u][plane] = *reinterpret_cast<const uint32_t*>(blk + lane_ofs + plane * kPlaneBytes + 8 * 16);
          }
          if (MODE == B200_Q_AFFINE4_G64) {
            const uint16_t* sc = reinterpret_cast<const uint16_t*>(blk + 2 * kPlaneBytes) + rA;
            sA[u] = __uint_as_float((uint32_t)sc[0] << 16); bA[u] = __uint_as_float((uint32_t)sc[kTileN] << 16);
            sB[u] = __uint_as_float((uint32_t)sc[8] << 16); bB[u] = __uint_as_float((uint32_t)sc[kTileN + 8] << 16);
          } else {
            __nv_bfloat162 dummy;
#pragma unroll
            for (int plane = 0; plane < 2; ++plane) {
              row_params<MODE>(blk, rA, plane, mA[u][plane], dummy);
              row_params<MODE>(blk, rB, plane, mB[u][plane], dummy);
            }
          }
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive_addr(free0 + 8 * slot);  // everything this warp needs is in registers
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          if (u == 1 && !two) break;
          if (MODE == B200_Q_AFFINE4_G64) {
            const float cA = fmaf(-128.f, sA[u], bA[u]), cB = fmaf(-128.f, sB[u], bB[u]);
            float acc[NT8][4];
            const __nv_bfloat162 unused = __nv_bfloat162();
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
              const int plane = ks >> 1, p0 = 2 * (ks & 1);
              uint32_t af[4];
              af[0] = operand_pair<MODE>(wa[u][plane], p0, unused);
              af[1] = operand_pair<MODE>(wb[u][plane], p0, unused);
              af[2] = operand_pair<MODE>(wa[u][plane], p0 + 1, unused);
              af[3] = operand_pair<MODE>(wb[u][plane], p0 + 1, unused);
#pragma unroll
              for (int j = 0; j < NT8; ++j) {
                const uint32_t b0 = (ks & 1) ? xv[j][plane].z : xv[j][plane].x, b1 = (ks & 1) ? xv[j][plane].w : xv[j][plane].y;
                if (ks == 0) mma_bf16_zero(acc[j], af, b0, b1);
                else mma_bf16_full(acc[j], af, b0, b1);
              }
            }
#pragma unroll
            for (int j = 0; j < NT8; ++j) {
              y[u][j][0] = fmaf(sA[u], acc[j][0], fmaf(cA, sx[j].x, y[u][j][0]));
              y[u][j][1] = fmaf(sA[u], acc[j][1], fmaf(cA, sx[j].y, y[u][j][1]));
              y[u][j][2] = fmaf(sB[u], acc[j][2], fmaf(cB, sx[j].x, y[u][j][2]));
              y[u][j][3] = fmaf(sB[u], acc[j][3], fmaf(cB, sx[j].y, y[u][j][3]));
            }
          } else {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
              const int plane = ks >> 1, p0 = 2 * (ks & 1);
              uint32_t af[4];
              af[0] = operand_pair<MODE>(wa[u][plane], p0, mA[u][plane]);
              af[1] = operand_pair<MODE>(wb[u][plane], p0, mB[u][plane]);
              af[2] = operand_pair<MODE>(wa[u][plane], p0 + 1, mA[u][plane]);
              af[3] = operand_pair<MODE>(wb[u][plane], p0 + 1, mB[u][plane]);
#pragma unroll
              for (int j = 0; j < NT8; ++j)
                mma_bf16_full(y[u][j], af, (ks & 1) ? xv[j][plane].z : xv[j][plane].x, (ks & 1) ? xv[j][plane].w : xv[j][plane].y);
            }
          }
        }
        px += kChunkK * 2;
        psx += TILE;
        if (++slot == (uint32_t)stages) { slot = 0; phase ^= 1u; }
      }
      if (ok) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          if (u == 1 && !two) break;
          float* wsp = a.ws + (((size_t)((nt0 + u) * gridDim.y + tt) * a.splits + split) * a.tn) * kTileN;
#pragma unroll
          for (int j = 0; j < NT8; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int tl = j * 8 + 2 * t + (e & 1), row = (e & 2) ? rB : rA;
              if (t0 + tl < a.rows) wsp[(size_t)tl * kTileN + row] = y[u][j][e];
            }
          }
        }
      }
    }
  }
  if (!ok) atomicExch(a.err, B200_ERR_DEVICE_FLAGGED);
}

// ---- small-batch kernel, integer variant (affine int4) --------------------------------------------
// The kernel above is bound by the integer pipe: turning a 32-bit word of eight 4-bit codes into four
// bf16x2 MMA operands costs a shift and a logic operation per pair.  An 8-bit integer MMA takes the
// codes almost as they lie: `w & 0x0F0F0F0F` is four operand bytes, `(w >> 4) & 0x0F0F0F0F` the other
// four — three operations per word instead of seven, and m16n8k32 covers a 32-column plane per
// instruction.  The activations of the CTA's K range are quantised once, while the slab is staged, to
// 16-bit fixed point with one scale per token and 64-column group (the weights' quantisation group):
// x = sigma * (128 * hi + lo) with hi in [-127, 127] and lo in [-64, 64], both int8, sigma =
// (largest magnitude of the group) / (127 * 128).  Two integer MMAs per plane (hi, lo) accumulate exactly
// in int32; one chunk is one group, so per chunk and output
//     y += s * sigma * (128 * acc_hi + acc_lo) + b * sum_x,
// with sum_x the group sum of the quantised activations.  The fixed-point error is 2^-14 of the group's
// largest magnitude: an outlier costs precision only among the 63 columns that share its group.
// Byte j of a weight word holds columns (j<2 ? 4j : 4j-7) [low nibble] and that + 2 [high nibble] of the
// word's eight columns, i.e. low nibbles are columns 0,4,1,5 and high nibbles 2,6,3,7: the activation
// slab stores each group of eight columns in the order 0,4,1,5,2,6,3,7, so that a lane's operand is one
// 8-byte load.
__device__ __forceinline__ void mma_s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1, bool zero) {
  if (zero) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0));
  } else {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

// Row stride of the int8 slabs: 32 bytes past a multiple of 128, so that the four token rows a half-warp's
// 8-byte loads touch (8 bytes x 4 lanes per row) fall into four disjoint groups of banks.
__host__ __device__ constexpr int slab8_stride(int chunks) { return (chunks * kChunkK + 127) / 128 * 128 + 32; }

template <int NT8>
__global__ void __launch_bounds__(kGemvThreads, NT8 >= 4 ? 1 : 2) qmm_mma8_kernel(QmmArgs a) {
  extern __shared__ __align__(128) unsigned char gsm[];
  const int stages = a.stages;
  constexpr int kSlotBytes = 2 * kRawStride;
  constexpr int MODE = B200_Q_AFFINE4_G64;
  constexpr int BB = block_bytes(MODE);
  uint64_t* raw_full = reinterpret_cast<uint64_t*>(gsm + (size_t)stages * kSlotBytes);
  uint64_t* raw_free = raw_full + stages;
  constexpr int TILE = NT8 * 8;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int split = blockIdx.x % a.splits, grp = blockIdx.x / a.splits, groups = gridDim.x / a.splits;
  const int tt = blockIdx.y, t0 = tt * TILE;
  const int kc0 = split * a.chunks_per_split, kc1 = min(kc0 + a.chunks_per_split, a.kc), n_chunks = kc1 - kc0;
  const int n_pairs = (a.nt + 1) / 2;
  const int n_items = grp < n_pairs ? (n_pairs - grp + groups - 1) / groups : 0;
  // [hi slab][lo slab] int8, then per chunk and token the group's scale and its sum of activations (f32)
  const int slab_stride = slab8_stride(a.chunks_per_split);
  unsigned char* slab_hi = reinterpret_cast<unsigned char*>(raw_free + stages);
  unsigned char* slab_lo = slab_hi + (size_t)TILE * slab_stride;
  float* sum_x = reinterpret_cast<float*>(slab_lo + (size_t)TILE * slab_stride);
  float* sigma = sum_x + (size_t)TILE * a.chunks_per_split;
  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      ptx::mbar_init(&raw_full[s], 1);
      ptx::mbar_init(&raw_free[s], kGemvConsumers);
    }
    ptx::mbar_fence_init();
  }
  __syncthreads();
  bool ok = true;
  if (warp == kGemvConsumers) {
    if (lane == 0) {
      int s = 0;
      uint32_t phase = 1;
      for (int item = 0; item < n_items && ok; ++item) {
        const int nt0 = 2 * (grp + item * groups);
        const int tiles = min(2, a.nt - nt0);
        const unsigned char* src = a.blocks + ((size_t)nt0 * a.kc + kc0) * BB;
        for (int i = 0; i < n_chunks; ++i) {
          ok = ptx::mbar_wait(&raw_free[s], phase);
          if (!ok) break;
          ptx::mbar_expect_tx(&raw_full[s], tiles * BB);
          for (int u = 0; u < tiles; ++u)
            ptx::bulk_g2s(gsm + (size_t)s * kSlotBytes + u * kRawStride, src + ((size_t)u * a.kc + i) * BB, BB, &raw_full[s]);
          if (++s == stages) { s = 0; phase ^= 1u; }
        }
      }
    }
  } else {
    // ---- stage the activations: 16-bit fixed point with one scale per token and 64-column group ----
    // One thread per 8 columns; the 8 threads of a group (consecutive lanes) agree on the group's scale,
    // quantise, and add up the group's integer sum.  A single pass, one barrier at the end.
    const int vec_per_row = n_chunks * (kChunkK / 8);
    const int total = TILE * vec_per_row;
    for (int base = 0; base < total; base += kGemvConsumers * 32) {
      const int idx = base + tid;
      const bool valid = idx < total;
      const int row = valid ? idx / vec_per_row : 0, v = valid ? idx - row * vec_per_row : 0;
      float xv[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) xv[j] = 0.f;
      if (valid && t0 + row < a.rows) {
        const uint4 q = *reinterpret_cast<const uint4*>(a.x + (size_t)(t0 + row) * a.k + (size_t)kc0 * kChunkK + v * 8);
        const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) { xv[2 * j] = ptx::bf16_lo(w4[j]); xv[2 * j + 1] = ptx::bf16_hi(w4[j]); }
      }
      float m = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(xv[j]));
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
      const float sig = (m > 0.f && m < 3e38f) ? m * (1.0f / (127.0f * 128.0f)) : 1.0f;
      const float inv = 1.0f / (sig * 128.0f);  // 1 / (step of the hi part)
      int h[8], l[8], part = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float hf = rintf(xv[j] * inv);
        h[j] = (int)hf;
        l[j] = (int)rintf((xv[j] * inv - hf) * 128.0f);
        part += h[j] * 128 + l[j];
      }
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
      if (valid) {
        // byte order 0,4,1,5 | 2,6,3,7 (see above)
        auto pack4 = [](int b0, int b1, int b2, int b3) {
          return (uint32_t)(b0 & 0xFF) | ((uint32_t)(b1 & 0xFF) << 8) | ((uint32_t)(b2 & 0xFF) << 16) | ((uint32_t)(b3 & 0xFF) << 24);
        };
        *reinterpret_cast<uint2*>(slab_hi + (size_t)row * slab_stride + v * 8) =
            make_uint2(pack4(h[0], h[4], h[1], h[5]), pack4(h[2], h[6], h[3], h[7]));
        *reinterpret_cast<uint2*>(slab_lo + (size_t)row * slab_stride + v * 8) =
            make_uint2(pack4(l[0], l[4], l[1], l[5]), pack4(l[2], l[6], l[3], l[7]));
        if ((v & 7) == 0) {
          const int c = v >> 3;
          sigma[c * TILE + row] = sig;
          sum_x[c * TILE + row] = (float)part * sig;
        }
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kGemvConsumers * 32) : "memory");

    const int rA = warp * 16 + g;
    const unsigned char* xh_lane = slab_hi + (size_t)g * slab_stride + 8 * t;  // token g of tile j: + j*8*slab_stride
    const unsigned char* xl_lane = slab_lo + (size_t)g * slab_stride + 8 * t;
    const uint32_t full0 = ptx::smem_u32(raw_full), free0 = ptx::smem_u32(raw_free);
    const uint32_t lane_ofs = (uint32_t)(rA * 16 + 4 * t);
    uint32_t slot = 0, phase = 0;
    for (int item = 0; item < n_items && ok; ++item) {
      const int nt0 = 2 * (grp + item * groups);
      const bool two = nt0 + 1 < a.nt;
      float y[2][NT8][4];
#pragma unroll
      for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int j = 0; j < NT8; ++j) { y[u][j][0] = y[u][j][1] = y[u][j][2] = y[u][j][3] = 0.f; }
      int xoff = 0;
      const float* psx = sum_x + 2 * t;
      const float* psg = sigma + 2 * t;
      for (int i = 0; i < n_chunks; ++i) {
        // activations of the chunk first: they do not depend on the weights
        uint2 xh[NT8][2], xl[NT8][2];
        float2 sx[NT8], sg[NT8];
#pragma unroll
        for (int j = 0; j < NT8; ++j) {
#pragma unroll
          for (int plane = 0; plane < 2; ++plane) {
            xh[j][plane] = *reinterpret_cast<const uint2*>(xh_lane + (size_t)(j * 8) * slab_stride + xoff + plane * 32);
            xl[j][plane] = *reinterpret_cast<const uint2*>(xl_lane + (size_t)(j * 8) * slab_stride + xoff + plane * 32);
          }
          sx[j] = *reinterpret_cast<const float2*>(psx + j * 8);
          sg[j] = *reinterpret_cast<const float2*>(psg + j * 8);
        }
        ok = ptx::mbar_wait_addr(full0 + 8 * slot, phase);
        if (!ok) break;
        const unsigned char* slot_base = gsm + slot * kSlotBytes;
        uint32_t wa[2][2], wb[2][2];
        float sA[2], bA[2], sB[2], bB[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          if (u == 1 && !two) break;
          const unsigned char* blk = slot_base + u * kRawStride;
#pragma unroll
          for (int plane = 0; plane < 2; ++plane) {
            wa[u][plane] = *reinterpret_cast<const uint32_t*>(blk + lane_ofs + plane * kPlaneBytes);
            wb[u][plane] = *reinterpret_cast<const uint32_t*>(blk + lane_ofs + plane * kPlaneBytes + 8 * 16);
          }
          const uint16_t* sc = reinterpret_cast<const uint16_t*>(blk + 2 * kPlaneBytes) + rA;
          sA[u] = __uint_as_float((uint32_t)sc[0] << 16); bA[u] = __uint_as_float((uint32_t)sc[kTileN] << 16);
          sB[u] = __uint_as_float((uint32_t)sc[8] << 16); bB[u] = __uint_as_float((uint32_t)sc[kTileN + 8] << 16);
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive_addr(free0 + 8 * slot);  // everything this warp needs is in registers
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          if (u == 1 && !two) break;
          int acc_h[NT8][4], acc_l[NT8][4];
#pragma unroll
          for (int plane = 0; plane < 2; ++plane) {
            uint32_t af[4];
            af[0] = wa[u][plane] & 0x0F0F0F0Fu;
            af[1] = wb[u][plane] & 0x0F0F0F0Fu;
            af[2] = (wa[u][plane] >> 4) & 0x0F0F0F0Fu;
            af[3] = (wb[u][plane] >> 4) & 0x0F0F0F0Fu;
#pragma unroll
            for (int j = 0; j < NT8; ++j) {
              mma_s8(acc_h[j], af, xh[j][plane].x, xh[j][plane].y, plane == 0);
              mma_s8(acc_l[j], af, xl[j][plane].x, xl[j][plane].y, plane == 0);
            }
          }
#pragma unroll
          for (int j = 0; j < NT8; ++j) {
            const float f0 = (float)(acc_h[j][0] * 128 + acc_l[j][0]), f1 = (float)(acc_h[j][1] * 128 + acc_l[j][1]);
            const float f2 = (float)(acc_h[j][2] * 128 + acc_l[j][2]), f3 = (float)(acc_h[j][3] * 128 + acc_l[j][3]);
            y[u][j][0] = fmaf(sA[u] * sg[j].x, f0, fmaf(bA[u], sx[j].x, y[u][j][0]));
            y[u][j][1] = fmaf(sA[u] * sg[j].y, f1, fmaf(bA[u], sx[j].y, y[u][j][1]));
            y[u][j][2] = fmaf(sB[u] * sg[j].x, f2, fmaf(bB[u], sx[j].x, y[u][j][2]));
            y[u][j][3] = fmaf(sB[u] * sg[j].y, f3, fmaf(bB[u], sx[j].y, y[u][j][3]));
          }
        }
        xoff += kChunkK;
        psx += TILE;
        psg += TILE;
        if (++slot == (uint32_t)stages) { slot = 0; phase ^= 1u; }
      }
      if (ok) {
        const int rB = rA + 8;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          if (u == 1 && !two) break;
          float* wsp = a.ws + (((size_t)((nt0 + u) * gridDim.y + tt) * a.splits + split) * a.tn) * kTileN;
#pragma unroll
          for (int j = 0; j < NT8; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int tl = j * 8 + 2 * t + (e & 1), row = (e & 2) ? rB : rA;
              if (t0 + tl < a.rows) wsp[(size_t)tl * kTileN + row] = y[u][j][e];
            }
          }
        }
      }
    }
  }
  if (!ok) atomicExch(a.err, B200_ERR_DEVICE_FLAGGED);
}

// ---- MXFP4 on the block-scaled tensor-core path ---------------------------------------------------
// tcgen05.mma kind::mxf8f6f4 multiplies E2M1 codes by E8M0 block scales in hardware, so MXFP4 weights
// need no dequantisation at all: TMA unpacks the packed codes into the 8-bit containers the MMA reads
// (16 codes -> 16 bytes, tensor-map type 16U4_ALIGN16B), the 128 x 4 scale bytes of a K128 chunk go
// to tensor memory as they are, and the only arithmetic left on the CUDA cores is the epilogue.
// The other operand must be an 8-bit float: the bf16 activations are scaled per row by a power of two
// (largest magnitude in [128, 256)) and split into E4M3 codes plus E4M3 codes of 16x the residual; the two
// halves are two MMAs into the same accumulator with constant block scales 1 and 2^-4, which carries
// the activations to about 2^-9 of the row maximum, i.e. bf16 precision.  The row's scale is undone
// in the epilogue.
//
// One CTA owns two adjacent 128-row weight tiles (they share the activation tiles) and all of K:
// warp 4 loads (per K128 stage: 2 x 16 KiB codes, 2 x 512 B scales, tn x 128 B of each activation
// half), warps 0-3 move the scales to tensor memory (one 16-byte shared-memory read and one
// tcgen05.st per thread and tile; the four 32-lane quarters hold the same words) and later run the
// epilogue, warp 5 issues 2 tiles x 4 K32 steps x 2 halves MMAs per stage.
constexpr int kMxThreads = 6 * 32;
constexpr int kMxpThreads = 10 * 32;  // persistent form: warps 0-3 and 6-9 run the epilogue (one tile each), 4 loads, 5 issues MMAs
constexpr int kMxK = 128;

__device__ __forceinline__ uint32_t mx_f32x2_to_e4m3x2(float lo, float hi) {
  unsigned short d;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(d) : "f"(hi), "f"(lo));
  return d;
}
__device__ __forceinline__ float2 mx_e4m3x2_to_f32x2(uint32_t codes) {
  uint32_t h;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h) : "h"((unsigned short)codes));
  return __half22float2(*reinterpret_cast<const __half2*>(&h));
}

// x [rows, k] bf16 -> hi, lo [rows, k] E4M3 and unscale[rows].  One CTA per row; k % 8 == 0.
__global__ void __launch_bounds__(256) mx_split_activations_kernel(const __nv_bfloat16* __restrict__ x, int k,
                                                                   unsigned char* __restrict__ hi, unsigned char* __restrict__ lo,
                                                                   float* __restrict__ unscale, const int* __restrict__ gather,
                                                                   int gather_div, const int* __restrict__ rows_valid) {
  __shared__ float s_max[8];
  const int row = blockIdx.x;
  if (rows_valid && row >= *rows_valid) return;  // capacity beyond the rows that exist: nothing to read
  const int src_row = gather ? gather[row] / gather_div : row;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)src_row * k);
  float amax = 0.f;
  for (int i = threadIdx.x; i < k / 8; i += blockDim.x) {
    const uint4 q = xr[i];
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) amax = fmaxf(amax, fmaxf(fabsf(ptx::bf16_lo(w[j])), fabsf(ptx::bf16_hi(w[j]))));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = s_max[0];
#pragma unroll
  for (int wv = 1; wv < 8; ++wv) amax = fmaxf(amax, s_max[wv]);
  // amax = m * 2^ex with m in [1, 2): scale by 2^(7 - ex) (zero, vanishing and non-finite rows keep scale 1)
  const int ex = amax >= 1e-30f && amax < 3e38f ? (int)((__float_as_uint(amax) >> 23) & 0xFF) - 127 : 7;
  const float qs = __uint_as_float((uint32_t)(127 + 7 - ex) << 23);
  if (threadIdx.x == 0) unscale[row] = __uint_as_float((uint32_t)(127 + ex - 7) << 23);
  uint2* hr = reinterpret_cast<uint2*>(hi + (size_t)row * k);
  uint2* lr = reinterpret_cast<uint2*>(lo + (size_t)row * k);
  for (int i = threadIdx.x; i < k / 8; i += blockDim.x) {
    const uint4 q = xr[i];
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
    uint32_t h[4], l[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a = ptx::bf16_lo(w[j]) * qs, b = ptx::bf16_hi(w[j]) * qs;
      h[j] = mx_f32x2_to_e4m3x2(a, b);
      const float2 back = mx_e4m3x2_to_f32x2(h[j]);
      l[j] = mx_f32x2_to_e4m3x2((a - back.x) * 16.f, (b - back.y) * 16.f);
    }
    hr[i] = make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16));
    lr[i] = make_uint2(l[0] | (l[1] << 16), l[2] | (l[3] << 16));
  }
}

// Tile-major blocks -> row-major codes + scale atoms (see b200_qweight).  One thread per 32-bit word of a plane.
__global__ void mx_from_blocks_kernel(const unsigned char* __restrict__ blocks, unsigned char* __restrict__ codes,
                                      unsigned char* __restrict__ sf, int nt_total, int kc, int k) {
  constexpr int BB = block_bytes(B200_Q_MXFP4_G32);
  const size_t n_words = (size_t)nt_total * kc * 2 * kTileN * 4;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_words; i += (size_t)gridDim.x * blockDim.x) {
    const int w = (int)(i & 3), r = (int)((i >> 2) & (kTileN - 1)), plane = (int)((i >> 9) & 1);
    const size_t blk_id = i >> 10;
    const int c = (int)(blk_id % kc);
    const size_t tile = blk_id / kc;  // expert * nt + n tile
    const unsigned char* blk = blocks + blk_id * BB;
    const uint32_t word = *reinterpret_cast<const uint32_t*>(blk + plane * kPlaneBytes + r * 16 + w * 4);
    uint32_t out = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t t = (word >> (4 * j)) & 0x000F000Fu;  // columns 2j (low half) and 2j+1 (high half)
      out |= ((t & 0xFu) | (t >> 12)) << (8 * j);
    }
    const size_t row = tile * kTileN + r;
    *reinterpret_cast<uint32_t*>(codes + row * (size_t)(k / 2) + c * 32 + plane * 16 + w * 4) = out;
    if (w == 0) {
      const int kb = c * 2 + plane;  // K32 block of the row
      sf[(tile * (size_t)(k / kMxK) + kb / 4) * 512 + (r & 31) * 16 + (r >> 5) * 4 + (kb & 3)] = blk[2 * kPlaneBytes + r * 2 + plane];
    }
  }
}

// AND of a predicate over the 128 threads of warps 0-3 (named barrier 1; warps 4 and 5 are elsewhere).
__device__ __forceinline__ bool __syncthreads_and_epi(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %1, 0;\n\t"
      "bar.red.and.pred q, 1, 128, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(r)
      : "r"((uint32_t)pred)
      : "memory");
  return r != 0;
}

// The same over the 256 epilogue threads of the persistent kernel (warps 0-3 and 6-9).
__device__ __forceinline__ bool __syncthreads_and_epi8(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %1, 0;\n\t"
      "bar.red.and.pred q, 1, 256, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(r)
      : "r"((uint32_t)pred)
      : "memory");
  return r != 0;
}

// Activation tensor maps with boxes of 32, 64, 96 and 128 rows: a work item loads (and multiplies) only
// as many token rows as it has, rounded up to 32.  The activation tiles are re-read by every CTA of
// an item and are two thirds of the bytes a stage moves.
struct MxActMaps {
  CUtensorMap hi[4];
  CUtensorMap lo[4];
};

__global__ void __launch_bounds__(kMxThreads, 1)
    qmm_mx_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ MxActMaps amaps, QmmArgs a) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int tn = a.tn, P = a.stages;
  constexpr int kATile = kTileN * kMxK;  // 16 KiB: one byte per code
  const int stage_stride = 2 * kATile + 2 * tn * 128 + 1024;
  auto a_tile = [&](int s, int tile) { return smem + (size_t)s * stage_stride + tile * kATile; };
  auto b_tile = [&](int s, int half) { return smem + (size_t)s * stage_stride + 2 * kATile + half * tn * 128; };
  auto sf_tile = [&](int s, int tile) { return smem + (size_t)s * stage_stride + 2 * kATile + 2 * tn * 128 + tile * 512; };
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)P * stage_stride);
  uint64_t* full = bars;            // [P] codes, scales and activations of the stage have landed
  uint64_t* slot_free = bars + P;   // [P] the MMAs of the stage are done (shared memory and scale columns)
  uint64_t* sf_ready = bars + 2 * P;  // [P] the stage's scales are in tensor memory
  uint64_t* accum_ready = bars + 3 * P;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_ready + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nt0 = 2 * blockIdx.x, n_tiles = min(2, a.nt - nt0);
  int t0 = blockIdx.z * tn, rows_here = min(tn, a.rows - t0), expert = 0;
  if (a.items) {
    if ((int)blockIdx.z >= *a.n_items) return;
    const int4 it = a.items[blockIdx.z];
    expert = it.x;
    t0 = it.y;
    rows_here = it.z;
  }
  const int n_chunks = a.kc128;
  const int tn_eff = min(tn, ((rows_here + 31) / 32) * 32), map_idx = (tn_eff + 31) / 32 - 1;  // rows loaded and multiplied
  constexpr uint32_t kCols = 512;  // accumulators at columns 0 and 128, scale words from column 256
  if (tid == 0) {
    for (int s = 0; s < P; ++s) {
      ptx::mbar_init(&full[s], 1);
      ptx::mbar_init(&slot_free[s], 1);
      ptx::mbar_init(&sf_ready[s], 4 * 32);
    }
    ptx::mbar_init(accum_ready, 1);
    ptx::mbar_fence_init();
  }
  if (warp == 5) {
    ptx::tmem_alloc(tmem_slot, kCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t sfa_col0 = tmem_base + 256u, sfb_hi = tmem_base + 256u + 8u * (uint32_t)P, sfb_lo = sfb_hi + 4u;
  bool ok = true;

  if (warp == 4) {
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      const int wrow0 = expert * a.mx_expert_rows + nt0 * kTileN;
      const unsigned char* sf_src = a.mx_sf + ((size_t)(expert * a.nt + nt0) * n_chunks) * 512;
      for (int i = 0; i < n_chunks && ok; ++i, ph ^= (s + 1 == P), s = (s + 1 == P) ? 0 : s + 1) {
        ok = ptx::mbar_wait(&slot_free[s], ph ^ 1u);
        if (!ok) break;
        // the unpacking copy counts the packed bytes it reads, not the containers it writes
        ptx::mbar_expect_tx(&full[s], n_tiles * (kATile / 2 + 512) + 2 * tn_eff * 128);
        for (int tile = 0; tile < n_tiles; ++tile) {
          ptx::tma_load_2d(a_tile(s, tile), &wmap, i * kMxK, wrow0 + tile * kTileN, &full[s]);
          ptx::bulk_g2s(sf_tile(s, tile), sf_src + ((size_t)tile * n_chunks + i) * 512, 512, &full[s]);
        }
        ptx::tma_load_2d(b_tile(s, 0), &amaps.hi[map_idx], i * kMxK, a.x_row0 + t0, &full[s]);
        ptx::tma_load_2d(b_tile(s, 1), &amaps.lo[map_idx], i * kMxK, a.x_row0 + t0, &full[s]);
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      ok = ptx::mbar_wait(&sf_ready[0], 0);  // the constant activation scales are in tensor memory
      for (int i = 0; i < n_chunks && ok; ++i, ph ^= (s + 1 == P), s = (s + 1 == P) ? 0 : s + 1) {
        ok = ptx::mbar_wait(&full[s], ph);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        const uint64_t dh = ptx::umma_desc_k_sw128(ptx::smem_u32(b_tile(s, 0)));
        const uint64_t dl = ptx::umma_desc_k_sw128(ptx::smem_u32(b_tile(s, 1)));
        for (int tile = 0; tile < n_tiles; ++tile) {
          const uint64_t da = ptx::umma_desc_k_sw128(ptx::smem_u32(a_tile(s, tile)));
          const uint32_t sfa = sfa_col0 + (uint32_t)((s * 2 + tile) * 4);
          // the tile's 128 x 4 scale bytes: shared memory -> tensor memory, ahead of the MMAs that read them
          ptx::tmem_cp_32x128b_warpx4(sfa, ptx::umma_desc_k_noswizzle_16B(ptx::smem_u32(sf_tile(s, tile))));
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            const uint32_t idesc = ptx::umma_idesc_mx_e2m1_e4m3(kTileN, tn_eff, k4);
            ptx::umma_mxf8f6f4(tmem_base + tile * 128, da + 2 * k4, dh + 2 * k4, idesc, (i > 0 || k4 > 0) ? 1u : 0u, sfa, sfb_hi);
            ptx::umma_mxf8f6f4(tmem_base + tile * 128, da + 2 * k4, dl + 2 * k4, idesc, 1u, sfa, sfb_lo);
          }
        }
        ptx::umma_commit(&slot_free[s]);
      }
      if (ok) ptx::umma_commit(accum_ready);
    }
  } else {
    // ---- scales: lane l of every warp holds rows l, 32+l, 64+l, 96+l of the tile (4 K32 blocks each) ----
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    ptx::tmem_st4(sfb_hi + lane_base, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu);  // 2^0
    ptx::tmem_st4(sfb_lo + lane_base, 0x7B7B7B7Bu, 0x7B7B7B7Bu, 0x7B7B7B7Bu, 0x7B7B7B7Bu);  // 2^-4
    ptx::tmem_st_wait();
    ptx::tc_fence_before_sync();
    ptx::mbar_arrive(&sf_ready[0]);
    // ---- epilogue ----
    // Warp w holds weight rows 32w..32w+31 of both tiles (one per lane) for every token.  A token's
    // output row wants the 128 (or 64 after SwiGLU) values of a tile side by side, so the accumulators
    // go through the (now idle) stage buffers as f32 [tile][token][128 rows] and leave as 16-byte
    // stores: 64-byte stores straight from the accumulator layout took as long as the whole K loop.
    if (ok) ok = ptx::mbar_wait(accum_ready, 0);
    const bool all_ok = __syncthreads_and_epi(ok);
    if (all_ok) {
      ptx::tc_fence_after_sync();
      float* stage_f = reinterpret_cast<float*>(smem);
      for (int tile = 0; tile < n_tiles; ++tile) {
        for (int c0 = 0; c0 < rows_here; c0 += 32) {
          uint32_t v[32];
          ptx::tmem_ld32(tmem_base + lane_base + (uint32_t)(tile * 128 + c0), v);
          const float us_mine = c0 + lane < rows_here ? a.act_unscale[t0 + c0 + lane] : 0.f;
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float us = __shfl_sync(0xffffffffu, us_mine, j);
            stage_f[((size_t)tile * tn + c0 + j) * kTileN + warp * 32 + lane] = __uint_as_float(v[j]) * us;
          }
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const bool swiglu = a.epilogue == B200_EPI_SWIGLU;
      const int out_per_tile = swiglu ? kTileN / 2 : kTileN, chunks = out_per_tile / 8;
      const int n_out = swiglu ? a.n / 2 : a.n;
      const float L = a.swiglu_limit;
      for (int tile = 0; tile < n_tiles; ++tile) {
        for (int idx = tid; idx < rows_here * chunks; idx += 128) {
          const int tok = idx / chunks, ch = idx - tok * chunks;
          const int token = t0 + tok, col = (nt0 + tile) * out_per_tile + ch * 8;
          if (col >= n_out) continue;
          const float* src = stage_f + ((size_t)tile * tn + tok) * kTileN + ch * (swiglu ? 16 : 8);
          const float rs = a.row_scale(token);
          float o[8];
          if (swiglu) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float4 f = reinterpret_cast<const float4*>(src)[q];  // gate, up, gate, up
              float g0 = f.x, u0 = f.y, g1 = f.z, u1 = f.w;
              if (L > 0.f) { g0 = fminf(g0, L); u0 = fminf(fmaxf(u0, -L), L); g1 = fminf(g1, L); u1 = fminf(fmaxf(u1, -L), L); }
              o[2 * q] = g0 / (1.0f + __expf(-g0)) * u0 * rs;
              o[2 * q + 1] = g1 / (1.0f + __expf(-g1)) * u1 * rs;
            }
          } else {
            const float4 f0 = reinterpret_cast<const float4*>(src)[0], f1 = reinterpret_cast<const float4*>(src)[1];
            o[0] = f0.x; o[1] = f0.y; o[2] = f0.z; o[3] = f0.w; o[4] = f1.x; o[5] = f1.y; o[6] = f1.z; o[7] = f1.w;
            if (a.epilogue == B200_EPI_RESIDUAL) {
              const uint4 r = *reinterpret_cast<const uint4*>(a.residual + (size_t)token * n_out + col);
              const uint32_t rw[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
              for (int q = 0; q < 4; ++q) { o[2 * q] += ptx::bf16_lo(rw[q]); o[2 * q + 1] += ptx::bf16_hi(rw[q]); }
            }
#pragma unroll
            for (int q = 0; q < 8; ++q) o[q] *= rs;
          }
          uint4 out;
          __nv_bfloat162 p0 = __floats2bfloat162_rn(o[0], o[1]), p1 = __floats2bfloat162_rn(o[2], o[3]);
          __nv_bfloat162 p2 = __floats2bfloat162_rn(o[4], o[5]), p3 = __floats2bfloat162_rn(o[6], o[7]);
          out.x = *reinterpret_cast<uint32_t*>(&p0); out.y = *reinterpret_cast<uint32_t*>(&p1);
          out.z = *reinterpret_cast<uint32_t*>(&p2); out.w = *reinterpret_cast<uint32_t*>(&p3);
          *reinterpret_cast<uint4*>(a.y + (size_t)token * n_out + col) = out;
        }
      }
    }
  }
  if (!ok) atomicExch(a.err, B200_ERR_DEVICE_FLAGGED);
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) ptx::tmem_dealloc(tmem_base, kCols);
}

// ---- block-scaled MXFP4, persistent form -----------------------------------------------------------
// The kernel above runs one work item per CTA: a CTA's stage ring drains while its epilogue runs, the
// next CTA starts with an empty ring, and short items (a MoE expert with a few dozen rows, a weight
// stream for a handful of tokens) are mostly ramp-up and tail.  Here a CTA stays on its SM and walks a
// list of work items; the loader warp runs ahead into the next item's weights while the epilogue
// warps drain the accumulators of the current one, so the ring never empties between items.
//   work item   = (tile pair, token tile or expert item, K range); item w of CTA b is b + i * gridDim.x,
//                 tile pair fastest, so that neighbouring CTAs share an item's activation rows in L2.
//   K splits    (dense launches with few tile pairs): partial sums go to the split-K scratch and the
//                 finish kernel, as for the other kernels.
//   epilogue    16 tokens at a time: tensor memory -> registers -> a dedicated 16 KiB f32 staging
//                 tile -> 16-byte stores; the accumulators are handed back to the MMA warp as soon as
//                 the last slab has been read, before it is stored.
constexpr int kMxpStageTokens = 16;

__global__ void __launch_bounds__(kMxpThreads, 1)
    qmm_mxp_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ MxActMaps amaps, QmmArgs a) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int tn = a.tn, P = a.stages;
  constexpr int kATile = kTileN * kMxK;
  const int stage_stride = 2 * kATile + 2 * tn * 128 + 1024;
  auto a_tile = [&](int s, int tile) { return smem + (size_t)s * stage_stride + tile * kATile; };
  auto b_tile = [&](int s, int half) { return smem + (size_t)s * stage_stride + 2 * kATile + half * tn * 128; };
  auto sf_tile = [&](int s, int tile) { return smem + (size_t)s * stage_stride + 2 * kATile + 2 * tn * 128 + tile * 512; };
  float* stage_f = reinterpret_cast<float*>(smem + (size_t)P * stage_stride);  // [2 tiles][16 tokens][128 rows]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)P * stage_stride + 2 * kMxpStageTokens * kTileN * sizeof(float));
  uint64_t* full = bars;
  uint64_t* slot_free = bars + P;
  uint64_t* sf_ready = bars + 2 * P;     // the constant activation scales are in tensor memory (once)
  uint64_t* accum_ready = bars + 2 * P + 1;  // [2] one per accumulator set
  uint64_t* accum_free = bars + 2 * P + 3;   // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * P + 5);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_pairs = (a.nt + 1) / 2;
  const int splits = a.items ? 1 : a.splits;
  const int tts = a.items ? 0 : (a.rows + tn - 1) / tn;
  const int n_work = a.items ? n_pairs * min(*a.n_items, a.max_items) : n_pairs * tts * splits;
  constexpr uint32_t kCols = 512;

  struct Work { int nt0, n_tiles, t0, rows_here, expert, kc0, n_chunks, tn_eff, map_idx, split, tt; };
  auto decode = [&](int w) {
    Work k;
    const int pair = w % n_pairs, rest = w / n_pairs;
    k.nt0 = 2 * pair;
    k.n_tiles = min(2, a.nt - k.nt0);
    k.expert = 0; k.split = 0; k.tt = 0;
    if (a.items) {
      const int4 it = a.items[rest];
      k.expert = it.x; k.t0 = it.y; k.rows_here = it.z;
      k.kc0 = 0; k.n_chunks = a.kc128;
    } else {
      k.tt = rest % tts;
      k.split = rest / tts;
      k.t0 = k.tt * tn;
      k.rows_here = min(tn, a.rows - k.t0);
      k.kc0 = k.split * a.chunks_per_split;
      k.n_chunks = min(a.chunks_per_split, a.kc128 - k.kc0);
    }
    k.tn_eff = min(tn, ((k.rows_here + 31) / 32) * 32);
    if (k.tn_eff < 16) k.tn_eff = 16;
    k.map_idx = (k.tn_eff + 31) / 32 - 1;
    return k;
  };

  if (tid == 0) {
    for (int s = 0; s < P; ++s) {
      ptx::mbar_init(&full[s], 1);
      ptx::mbar_init(&slot_free[s], 1);
    }
    ptx::mbar_init(sf_ready, 4 * 32);
    for (int q = 0; q < 2; ++q) {
      ptx::mbar_init(&accum_ready[q], 1);
      ptx::mbar_init(&accum_free[q], 8);  // one arrival per epilogue warp
    }
    ptx::mbar_fence_init();
  }
  if (warp == 5) {
    ptx::tmem_alloc(tmem_slot, kCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // Tensor-memory columns.  Token tiles of up to 112 rows leave room for TWO sets of accumulators (2 sets x 2 tiles x tn
  // columns + the scales <= 512): work items alternate between them, so that the epilogue of one item drains its set
  // while the MMAs of the next item fill the other.  With one set the next item's first MMA had to wait for the last
  // slab of the epilogue: the MoE stack spent a quarter of its time there (10.7 ms -> 7.9 ms with the epilogue left
  // out, timing only).  Wider tiles keep one set of two 128-column accumulators.
  const bool dual = 4 * tn + 8 * P + 8 <= (int)kCols;
  const uint32_t acc_stride = dual ? (uint32_t)tn : 128u, set_stride = 2u * acc_stride;
  const uint32_t sfa_col0 = tmem_base + (dual ? 2u * set_stride : 256u), sfb_hi = sfa_col0 + 8u * (uint32_t)P, sfb_lo = sfb_hi + 4u;
  bool ok = true;

  if (warp == 4) {
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
        const Work k = decode(w);
        const int wrow0 = k.expert * a.mx_expert_rows + k.nt0 * kTileN;
        const unsigned char* sf_src = a.mx_sf + ((size_t)(k.expert * a.nt + k.nt0) * a.kc128) * 512;
        for (int i = 0; i < k.n_chunks && ok; ++i, ph ^= (s + 1 == P), s = (s + 1 == P) ? 0 : s + 1) {
          ok = ptx::mbar_wait(&slot_free[s], ph ^ 1u);
          if (!ok) break;
          const int kc = k.kc0 + i;
          ptx::mbar_expect_tx(&full[s], k.n_tiles * (kATile / 2 + 512) + 2 * k.tn_eff * 128);
          for (int tile = 0; tile < k.n_tiles; ++tile) {
            ptx::tma_load_2d(a_tile(s, tile), &wmap, kc * kMxK, wrow0 + tile * kTileN, &full[s]);
            ptx::bulk_g2s(sf_tile(s, tile), sf_src + ((size_t)tile * a.kc128 + kc) * 512, 512, &full[s]);
          }
          ptx::tma_load_2d(b_tile(s, 0), &amaps.hi[k.map_idx], kc * kMxK, a.x_row0 + k.t0, &full[s]);
          ptx::tma_load_2d(b_tile(s, 1), &amaps.lo[k.map_idx], kc * kMxK, a.x_row0 + k.t0, &full[s]);
        }
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0, n_done = 0;
      ok = ptx::mbar_wait(sf_ready, 0);
      for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x, ++n_done) {
        const Work k = decode(w);
        // the epilogue of the set's previous item must have read the accumulators out before they are overwritten
        const uint32_t set = dual ? (n_done & 1u) : 0u, uses = dual ? (n_done >> 1) : n_done;
        if (uses > 0) ok = ptx::mbar_wait(&accum_free[set], (uses - 1) & 1u);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        const uint32_t acc0 = tmem_base + set * set_stride;
        for (int i = 0; i < k.n_chunks && ok; ++i, ph ^= (s + 1 == P), s = (s + 1 == P) ? 0 : s + 1) {
          ok = ptx::mbar_wait(&full[s], ph);
          if (!ok) break;
          ptx::tc_fence_after_sync();
          const uint64_t dh = ptx::umma_desc_k_sw128(ptx::smem_u32(b_tile(s, 0)));
          const uint64_t dl = ptx::umma_desc_k_sw128(ptx::smem_u32(b_tile(s, 1)));
          for (int tile = 0; tile < k.n_tiles; ++tile) {
            const uint64_t da = ptx::umma_desc_k_sw128(ptx::smem_u32(a_tile(s, tile)));
            const uint32_t sfa = sfa_col0 + (uint32_t)((s * 2 + tile) * 4);
            ptx::tmem_cp_32x128b_warpx4(sfa, ptx::umma_desc_k_noswizzle_16B(ptx::smem_u32(sf_tile(s, tile))));
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) {
              const uint32_t idesc = ptx::umma_idesc_mx_e2m1_e4m3(kTileN, k.tn_eff, k4);
              ptx::umma_mxf8f6f4(acc0 + tile * acc_stride, da + 2 * k4, dh + 2 * k4, idesc, (i > 0 || k4 > 0) ? 1u : 0u, sfa, sfb_hi);
              ptx::umma_mxf8f6f4(acc0 + tile * acc_stride, da + 2 * k4, dl + 2 * k4, idesc, 1u, sfa, sfb_lo);
            }
          }
          ptx::umma_commit(&slot_free[s]);
        }
        if (ok) ptx::umma_commit(&accum_ready[set]);
      }
    }
  } else {
    // ---- epilogue: warps 0-3 drain tile 0, warps 6-9 tile 1 (a warp reads the tensor-memory lanes 32 * (warp % 4)) ----
    const int etile = warp < 4 ? 0 : 1, etid = warp < 4 ? tid : tid - 64;  // dense index over the 256 epilogue threads
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    if (warp < 4) {
      ptx::tmem_st4(sfb_hi + lane_base, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu);  // 2^0
      ptx::tmem_st4(sfb_lo + lane_base, 0x7B7B7B7Bu, 0x7B7B7B7Bu, 0x7B7B7B7Bu, 0x7B7B7B7Bu);  // 2^-4
      ptx::tmem_st_wait();
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(sf_ready);
    }
    const bool swiglu = a.epilogue == B200_EPI_SWIGLU;
    const int out_per_tile = swiglu ? kTileN / 2 : kTileN, chunks = out_per_tile / 8;
    const int n_out = swiglu ? a.n / 2 : a.n;
    const float L = a.swiglu_limit;
    uint32_t n_done = 0;
    for (int w = blockIdx.x; w < n_work; w += gridDim.x, ++n_done) {
      const Work k = decode(w);
      const uint32_t set = dual ? (n_done & 1u) : 0u, uses = dual ? (n_done >> 1) : n_done;
      const uint32_t acc0 = tmem_base + set * set_stride;
      if (ok) ok = ptx::mbar_wait(&accum_ready[set], uses & 1u);
      const bool all_ok = __syncthreads_and_epi8(ok);
      if (!all_ok) { ok = false; break; }
      ptx::tc_fence_after_sync();
      const bool partial = splits > 1;
      const bool mine = etile < k.n_tiles;
      for (int c0 = 0; c0 < k.rows_here; c0 += kMxpStageTokens) {
        const bool last_slab = c0 + kMxpStageTokens >= k.rows_here;
        const float us_mine = (lane < kMxpStageTokens && c0 + lane < k.rows_here) ? a.act_unscale[k.t0 + c0 + lane] : 0.f;
        if (mine) {
          uint32_t v[16];
          ptx::tmem_ld16(acc0 + lane_base + (uint32_t)etile * acc_stride + (uint32_t)c0, v);
          ptx::tmem_ld_wait();
          if (partial) {
            // [weight tile][token tile][split][tn][128] f32, summed by the finish kernel
            float* wsp = a.ws + (((size_t)((k.nt0 + etile) * tts + k.tt) * splits + k.split) * tn) * kTileN + (warp & 3) * 32 + lane;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float us = __shfl_sync(0xffffffffu, us_mine, j);
              if (c0 + j < k.rows_here) wsp[(size_t)(c0 + j) * kTileN] = __uint_as_float(v[j]) * us;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float us = __shfl_sync(0xffffffffu, us_mine, j);
              stage_f[((size_t)etile * kMxpStageTokens + j) * kTileN + (warp & 3) * 32 + lane] = __uint_as_float(v[j]) * us;
            }
          }
        }
        if (last_slab) {  // everything this warp reads of the item's accumulators has been read
          ptx::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(&accum_free[set]);
        }
        if (partial) continue;
        asm volatile("bar.sync 1, 256;" ::: "memory");
        const int slab_rows = min(kMxpStageTokens, k.rows_here - c0);
        const int per_tile = slab_rows * chunks;
        for (int idx = etid; idx < k.n_tiles * per_tile; idx += 256) {
          const int tile = idx / per_tile, rest = idx - tile * per_tile;
          const int tok = rest / chunks, ch = rest - tok * chunks;
          const int token = k.t0 + c0 + tok, col = (k.nt0 + tile) * out_per_tile + ch * 8;
          if (col >= n_out) continue;
          const float* src = stage_f + ((size_t)tile * kMxpStageTokens + tok) * kTileN + ch * (swiglu ? 16 : 8);
          const float rs = a.row_scale(token);
          float o[8];
          if (swiglu) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float4 f = reinterpret_cast<const float4*>(src)[q];  // gate, up, gate, up
              float g0 = f.x, u0 = f.y, g1 = f.z, u1 = f.w;
              if (L > 0.f) { g0 = fminf(g0, L); u0 = fminf(fmaxf(u0, -L), L); g1 = fminf(g1, L); u1 = fminf(fmaxf(u1, -L), L); }
              o[2 * q] = g0 / (1.0f + __expf(-g0)) * u0 * rs;
              o[2 * q + 1] = g1 / (1.0f + __expf(-g1)) * u1 * rs;
            }
          } else {
            const float4 f0 = reinterpret_cast<const float4*>(src)[0], f1 = reinterpret_cast<const float4*>(src)[1];
            o[0] = f0.x; o[1] = f0.y; o[2] = f0.z; o[3] = f0.w; o[4] = f1.x; o[5] = f1.y; o[6] = f1.z; o[7] = f1.w;
            if (a.epilogue == B200_EPI_RESIDUAL) {
              const uint4 r = *reinterpret_cast<const uint4*>(a.residual + (size_t)token * n_out + col);
              const uint32_t rw[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
              for (int q = 0; q < 4; ++q) { o[2 * q] += ptx::bf16_lo(rw[q]); o[2 * q + 1] += ptx::bf16_hi(rw[q]); }
            }
#pragma unroll
            for (int q = 0; q < 8; ++q) o[q] *= rs;
          }
          uint4 out;
          __nv_bfloat162 p0 = __floats2bfloat162_rn(o[0], o[1]), p1 = __floats2bfloat162_rn(o[2], o[3]);
          __nv_bfloat162 p2 = __floats2bfloat162_rn(o[4], o[5]), p3 = __floats2bfloat162_rn(o[6], o[7]);
          out.x = *reinterpret_cast<uint32_t*>(&p0); out.y = *reinterpret_cast<uint32_t*>(&p1);
          out.z = *reinterpret_cast<uint32_t*>(&p2); out.w = *reinterpret_cast<uint32_t*>(&p3);
          *reinterpret_cast<uint4*>(a.y + (size_t)token * n_out + col) = out;
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");  // the staging tile is free for the next slab
      }
    }
  }
  if (!ok) atomicExch(a.err, B200_ERR_DEVICE_FLAGGED);
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) ptx::tmem_dealloc(tmem_base, kCols);
}

// ---- host-side state -------------------------------------------------------------------------------
// One calling thread and one device per process use the matmul entry points (the library as a whole
// binds to the first device it is used on, see b200_require_device).  The split-K scratch and the
// activation buffers of the block-scaled path grow on demand, but a buffer that has been handed to a
// kernel is never freed: CUDA graphs captured earlier (the decode steps of b200_llama_forward) carry its
// address in their kernel arguments and keep writing their partial sums there.  An outgrown buffer is
// retired (kept until the process exits) and new launches use the larger one; no device-wide
// synchronisation is needed for that.
float* g_ws = nullptr;
size_t g_ws_bytes = 0;
int* g_err = nullptr;
int g_sms = 0;
std::vector<void*> g_retired;  // outgrown scratch buffers, still referenced by captured graphs

b200_status ensure_state(size_t ws_bytes) {
  if (!g_err) {
    B200_CUDA_TRY(cudaMalloc((void**)&g_err, sizeof(int)));
    B200_CUDA_TRY(cudaMemset(g_err, 0, sizeof(int)));
    int dev = 0;
    B200_CUDA_TRY(cudaGetDevice(&dev));
    B200_CUDA_TRY(cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev));
  }
  if (ws_bytes > g_ws_bytes) {
    const size_t want = std::max(ws_bytes + ws_bytes / 4, (size_t)64 << 20);
    float* grown = nullptr;
    B200_CUDA_TRY(cudaMalloc((void**)&grown, want));
    if (g_ws) g_retired.push_back(g_ws);
    g_ws = grown;
    g_ws_bytes = want;
  }
  return B200_OK;
}

b200_status make_x_map(CUtensorMap* map, const void* x, int rows, int k, int box_rows) {
  const uint64_t dims[2] = {(uint64_t)k, (uint64_t)rows};
  const uint64_t strides[1] = {(uint64_t)k * 2};
  const uint32_t box[2] = {(uint32_t)kChunkK, (uint32_t)box_rows};
  return b200_make_tensor_map(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, dims, strides, box);
}

// Number of K splits for `tiles` output tiles with `ctas_per_sm` resident CTAs per SM: the
// smallest count whose grid comes closest to a whole number of waves, each split keeping at
// least 4 chunks.
int pick_splits(int tiles, int kc, int sms, int ctas_per_sm, int fixed_cost = 2) {
  const int slots = sms * ctas_per_sm;
  const int max_s = std::max(1, std::min(16, kc / 4));
  int best = 1;
  double best_eff = 0.0;
  for (int sp = 1; sp <= max_s; ++sp) {
    const int cps = (kc + sp - 1) / sp;
    const int real = (kc + cps - 1) / cps;
    if (real != sp) continue;
    const long long ctas = (long long)tiles * sp;
    const long long waves = (ctas + slots - 1) / slots;
    // useful work / occupied time, with a small penalty per split for its fixed cost
    const double eff = (double)ctas / (double)(waves * slots) * (double)cps / (double)(cps + fixed_cost);
    if (eff > best_eff + 1e-9) { best_eff = eff; best = sp; }
  }
  return best;
}

}  // namespace

// ---- repacking ---------------------------------------------------------------------------------------
static inline int nibble_pos_to_col(int p) { return p < 4 ? 2 * p : 2 * (p - 4) + 1; }

extern "C" b200_status b200_qweight_create(int32_t mode, int32_t n_experts, int32_t n, int32_t k, const void* h_packed,
                                           const void* h_scales, const void* h_biases, b200_qweight** out) {
  *out = nullptr;
  b200_status st = b200_require_device();
  if (st != B200_OK) return st;
  if (mode != B200_Q_AFFINE4_G64 && mode != B200_Q_MXFP4_G32 && mode != B200_Q_BF16) { b200_set_error("unknown quantisation mode %d", mode); return B200_ERR_INVALID_QUANT_BITS; }
  if (n_experts <= 0 || n <= 0 || k <= 0 || k % kChunkK != 0) { b200_set_error("qweight: K must be a positive multiple of 64"); return B200_ERR_INVALID_ARGUMENT; }
  if (mode == B200_Q_AFFINE4_G64 && !h_biases) { b200_set_error("affine weights need biases"); return B200_ERR_INVALID_ARGUMENT; }
  const int nt = (n + kTileN - 1) / kTileN, kc = k / kChunkK, bb = block_bytes(mode);
  const size_t total = (size_t)n_experts * nt * kc * bb;
  std::vector<unsigned char> host(total, 0);
  for (int e = 0; e < n_experts; ++e)
    for (int t = 0; t < nt; ++t)
      for (int c = 0; c < kc; ++c) {
        unsigned char* blk = host.data() + (((size_t)e * nt + t) * kc + c) * bb;
        for (int r = 0; r < kTileN; ++r) {
          const int row = t * kTileN + r;
          if (row >= n) {
            if (mode == B200_Q_MXFP4_G32) { blk[2 * kPlaneBytes + r * 2] = 127; blk[2 * kPlaneBytes + r * 2 + 1] = 127; }
            continue;  // zero nibbles, zero scale/bias (affine) -> zero weights
          }
          const size_t grow = (size_t)e * n + row;
          if (mode == B200_Q_BF16) {
            for (int cc = 0; cc < 8; ++cc)
              std::memcpy(blk + r * 128 + ((cc ^ (r & 7)) << 4), (const uint16_t*)h_packed + grow * k + c * kChunkK + cc * 8, 16);
            continue;
          }
          for (int plane = 0; plane < 2; ++plane)
            for (int w = 0; w < 4; ++w) {
              uint32_t word = 0;
              for (int p = 0; p < 8; ++p) {
                const int col = c * kChunkK + plane * 32 + w * 8 + nibble_pos_to_col(p);
                uint32_t nib;
                if (mode == B200_Q_AFFINE4_G64) {
                  const uint32_t src = ((const uint32_t*)h_packed)[grow * (k / 8) + col / 8];
                  nib = (src >> (4 * (col % 8))) & 0xF;
                } else {
                  const uint8_t src = ((const uint8_t*)h_packed)[grow * (k / 2) + col / 2];
                  nib = (col & 1) ? (src >> 4) & 0xF : src & 0xF;
                }
                word |= nib << (4 * p);
              }
              std::memcpy(blk + plane * kPlaneBytes + r * 16 + w * 4, &word, 4);
            }
          if (mode == B200_Q_AFFINE4_G64) {
            uint16_t* sc = (uint16_t*)(blk + 2 * kPlaneBytes);
            sc[r] = ((const uint16_t*)h_scales)[grow * (k / 64) + c];
            sc[kTileN + r] = ((const uint16_t*)h_biases)[grow * (k / 64) + c];
          } else {
            blk[2 * kPlaneBytes + r * 2] = ((const uint8_t*)h_scales)[grow * (k / 32) + c * 2];
            blk[2 * kPlaneBytes + r * 2 + 1] = ((const uint8_t*)h_scales)[grow * (k / 32) + c * 2 + 1];
          }
        }
      }
  auto* w = new b200_qweight();
  w->mode = mode; w->n_experts = n_experts; w->n = n; w->k = k; w->nt = nt; w->kc = kc; w->block_bytes = bb;
  cudaError_t e = cudaMalloc((void**)&w->d_blocks, total);
  if (e != cudaSuccess) { b200_set_error("cudaMalloc(%zu) failed: %s", total, cudaGetErrorString(e)); delete w; return B200_ERR_CUDA; }
  e = cudaMemcpy(w->d_blocks, host.data(), total, cudaMemcpyHostToDevice);
  if (e != cudaSuccess) { b200_set_error("weight upload failed: %s", cudaGetErrorString(e)); cudaFree(w->d_blocks); delete w; return B200_ERR_CUDA; }
  *out = w;
  return B200_OK;
}

namespace {
__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
  return x;
}
// Fills blocks with pseudo-random codes and plausible scales: affine weights land in about
// [-0.04, 0.035], MXFP4 scales are 2^-6, dense weights are small bf16 values.
__global__ void random_blocks_kernel(unsigned char* blocks, size_t n_blocks, int mode, uint32_t seed) {
  const int bb = block_bytes(mode);
  const size_t words = n_blocks * (size_t)(bb / 4);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < words; i += (size_t)gridDim.x * blockDim.x) {
    const int off = (int)(i % (size_t)(bb / 4)) * 4;
    uint32_t v = mix32((uint32_t)i * 2654435761u + seed) ^ mix32((uint32_t)(i >> 32) + seed * 31u);
    if (mode == B200_Q_AFFINE4_G64) {
      if (off >= 2 * kPlaneBytes) v = off < 2 * kPlaneBytes + 256 ? 0x3BA43BA4u /* 0.005 x2 */ : 0xBD24BD24u /* -0.04 x2 */;
    } else if (mode == B200_Q_MXFP4_G32) {
      if (off >= 2 * kPlaneBytes) v = 0x79797979u;  // E8M0 121 -> 2^-6
    } else {
      v = (v & 0x807F807Fu) | 0x3C003C00u;  // bf16 with exponent 2^-7: |w| in [0.0078, 0.0156)
    }
    reinterpret_cast<uint32_t*>(blocks)[i] = v;
  }
}
}  // namespace

extern "C" b200_status b200_qweight_random(int32_t mode, int32_t n_experts, int32_t n, int32_t k, uint32_t seed,
                                           b200_qweight** out) {
  *out = nullptr;
  b200_status st = b200_require_device();
  if (st != B200_OK) return st;
  if (mode < 0 || mode > B200_Q_BF16) { b200_set_error("unknown quantisation mode %d", mode); return B200_ERR_INVALID_QUANT_BITS; }
  if (n_experts <= 0 || n <= 0 || k <= 0 || k % kChunkK != 0 || n % kTileN != 0) {
    b200_set_error("random weights: N must be a multiple of 128 and K of 64");
    return B200_ERR_INVALID_ARGUMENT;
  }
  auto* w = new b200_qweight();
  w->mode = mode; w->n_experts = n_experts; w->n = n; w->k = k; w->nt = n / kTileN; w->kc = k / kChunkK;
  w->block_bytes = block_bytes(mode);
  const size_t n_blocks = (size_t)n_experts * w->nt * w->kc;
  cudaError_t e = cudaMalloc((void**)&w->d_blocks, n_blocks * w->block_bytes);
  if (e != cudaSuccess) { b200_set_error("cudaMalloc failed: %s", cudaGetErrorString(e)); delete w; return B200_ERR_CUDA; }
  random_blocks_kernel<<<1184, 256>>>(w->d_blocks, n_blocks, mode, seed);
  e = cudaDeviceSynchronize();
  if (e != cudaSuccess) { b200_set_error("random init failed: %s", cudaGetErrorString(e)); cudaFree(w->d_blocks); delete w; return B200_ERR_CUDA; }
  *out = w;
  return B200_OK;
}

// Inverse of b200_qweight_create for one expert: the tile-major blocks go back to the reference's
// layout on the host (checks of weights that were generated on the device).
extern "C" b200_status b200_qweight_export(const b200_qweight* w, int32_t expert, void* h_packed, void* h_scales, void* h_biases) {
  if (expert < 0 || expert >= w->n_experts) { b200_set_error("qweight export: expert %d of %d", expert, w->n_experts); return B200_ERR_INVALID_ARGUMENT; }
  if (w->mode == B200_Q_AFFINE4_G64 && !h_biases) { b200_set_error("qweight export: affine weights have biases"); return B200_ERR_INVALID_ARGUMENT; }
  const int nt = w->nt, kc = w->kc, bb = w->block_bytes, n = w->n, k = w->k;
  const size_t bytes = (size_t)nt * kc * bb;
  std::vector<unsigned char> host(bytes);
  B200_CUDA_TRY(cudaMemcpy(host.data(), w->d_blocks + (size_t)expert * bytes, bytes, cudaMemcpyDeviceToHost));
  const size_t packed_row = w->mode == B200_Q_BF16 ? (size_t)k * 2 : (size_t)k / 2;
  std::memset(h_packed, 0, packed_row * n);
  for (int t = 0; t < nt; ++t)
    for (int c = 0; c < kc; ++c) {
      const unsigned char* blk = host.data() + ((size_t)t * kc + c) * bb;
      for (int r = 0; r < kTileN; ++r) {
        const int row = t * kTileN + r;
        if (row >= n) break;
        if (w->mode == B200_Q_BF16) {
          for (int cc = 0; cc < 8; ++cc)
            std::memcpy((uint16_t*)h_packed + (size_t)row * k + c * kChunkK + cc * 8, blk + r * 128 + ((cc ^ (r & 7)) << 4), 16);
          continue;
        }
        unsigned char* dst = (unsigned char*)h_packed + (size_t)row * (k / 2) + c * (kChunkK / 2);  // 32 bytes of this chunk
        for (int plane = 0; plane < 2; ++plane)
          for (int wd = 0; wd < 4; ++wd) {
            uint32_t word;
            std::memcpy(&word, blk + plane * kPlaneBytes + r * 16 + wd * 4, 4);
            for (int p = 0; p < 8; ++p) {
              const int col = plane * 32 + wd * 8 + nibble_pos_to_col(p);  // column within the chunk
              const uint32_t nib = (word >> (4 * p)) & 0xF;
              dst[col / 2] |= (unsigned char)((col & 1) ? nib << 4 : nib);  // both formats: even column = low nibble
            }
          }
        if (w->mode == B200_Q_AFFINE4_G64) {
          const uint16_t* sc = (const uint16_t*)(blk + 2 * kPlaneBytes);
          ((uint16_t*)h_scales)[(size_t)row * (k / 64) + c] = sc[r];
          ((uint16_t*)h_biases)[(size_t)row * (k / 64) + c] = sc[kTileN + r];
        } else {
          ((uint8_t*)h_scales)[(size_t)row * (k / 32) + c * 2] = blk[2 * kPlaneBytes + r * 2];
          ((uint8_t*)h_scales)[(size_t)row * (k / 32) + c * 2 + 1] = blk[2 * kPlaneBytes + r * 2 + 1];
        }
      }
    }
  return B200_OK;
}

extern "C" void b200_qweight_destroy(b200_qweight* w) {
  if (!w) return;
  if (w->d_blocks) cudaFree(w->d_blocks);
  if (w->d_mx_codes) cudaFree(w->d_mx_codes);
  if (w->d_mx_sf) cudaFree(w->d_mx_sf);
  delete w;
}

// ---- launch -------------------------------------------------------------------------------------------
// Sets a.did_norm when the finish pass also wrote the requested RMSNorm.
static b200_status launch_finish(QmmArgs& a, int splits, cudaStream_t s) {
  if (a.defer && a.epilogue == B200_EPI_NONE && !a.items && !a.row_scales && !a.norm_w) {
    // the caller's next kernel sums the splits (b200_kv_rope_append_partials)
    a.defer->d_ws = a.ws; a.defer->splits = splits; a.defer->tn = a.tn; a.defer->tts = (a.rows + a.tn - 1) / a.tn;
    a.defer->nt = a.nt; a.defer->rows = a.rows; a.defer->n = a.n; a.defer->pending = 1;
    return B200_OK;
  }
  // (decode-sized batches only: one CTA per row does not beat the two separate kernels on prefill chunks)
  if (a.norm_w && a.rows <= 256 && a.epilogue == B200_EPI_RESIDUAL && !a.items && !a.row_scales && a.n % 4 == 0 && a.n <= 16384) {
    int threads = ((a.n / 4 + 31) / 32) * 32;
    while (threads > 1024) threads = (((threads + 1) / 2 + 31) / 32) * 32;
    qmm_finish_rmsnorm_kernel<<<a.rows, threads, 0, s>>>(a, splits);
    B200_LAUNCH_CHECK();
    a.did_norm = 1;
    return B200_OK;
  }
  const long long threads = (long long)a.rows * a.nt * (kTileN / 4);
  qmm_finish_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, s>>>(a, splits);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

template <int MODE>
static b200_status launch_simt(QmmArgs& a, int rows, cudaStream_t s) {
  constexpr int TT = 4;
  a.tn = TT;
  const int tts = (rows + TT - 1) / TT;
  const int tiles = a.nt * tts;
  b200_status st = ensure_state(0);
  if (st != B200_OK) return st;
  const int splits0 = pick_splits(tiles, a.kc, g_sms, 8);
  a.chunks_per_split = (a.kc + splits0 - 1) / splits0;
  const int splits = (a.kc + a.chunks_per_split - 1) / a.chunks_per_split;
  st = ensure_state((size_t)splits * (size_t)tts * TT * a.nt * kTileN * sizeof(float));
  if (st != B200_OK) return st;
  a.ws = g_ws; a.err = g_err;
  qmm_simt_kernel<MODE, TT><<<dim3(a.nt, splits, tts), kTileN, 0, s>>>(a);
  B200_LAUNCH_CHECK();
  return launch_finish(a, splits, s);
}

template <int MODE>
static b200_status launch_tc(QmmArgs& a, int rows, cudaStream_t s) {
  // grouped launches fix the token tile (an expert's rows are cut into tiles of a.tn); dense ones
  // take the whole batch up to 256 rows per tile
  const int tn = a.items ? a.tn : std::min(256, ((rows + 15) / 16) * 16);
  a.tn = tn;
  const int tts = (rows + tn - 1) / tn;
  const int tiles = a.items ? a.nt * a.max_items : a.nt * tts;
  b200_status st = ensure_state(0);
  if (st != B200_OK) return st;
  constexpr int kRaw = MODE == B200_Q_BF16 ? 0 : ((block_bytes(MODE) + 127) / 128) * 128;
  const int stage_stride = kTileN * 128 + tn * 128 + kRaw;
  static int smem_budget[3] = {0, 0, 0};  // opt-in dynamic shared memory available to this kernel
  if (smem_budget[MODE] == 0) {
    int dev = 0, optin = 0;
    B200_CUDA_TRY(cudaGetDevice(&dev));
    B200_CUDA_TRY(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    cudaFuncAttributes fa;
    B200_CUDA_TRY(cudaFuncGetAttributes(&fa, qmm_tc_kernel<MODE>));
    const int budget = optin - (int)fa.sharedSizeBytes;
    B200_CUDA_TRY(cudaFuncSetAttribute(qmm_tc_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, budget));
    smem_budget[MODE] = budget;
  }
  const int fixed = 1024 /*alignment slack*/ + 8 * (3 * 8 + 2) + 16;
  // Small token tiles leave room for two CTAs per SM (more weight bytes in flight); large ones
  // take the whole SM.
  const int per_cta = tn <= 128 ? 113 * 1024 : std::min(smem_budget[MODE], 220 * 1024);
  a.stages = std::max(2, std::min(8, (per_cta - fixed) / stage_stride));
  const int ctas_per_sm = tn <= 128 ? 2 : 1;
  const size_t smem = (size_t)a.stages * stage_stride + fixed;
  if ((int)smem > smem_budget[MODE]) {
    b200_set_error("qmm: %zu bytes of shared memory needed, %d available", smem, smem_budget[MODE]);
    return B200_ERR_CAPACITY;
  }
  // A CTA pays its first load (about 2.3 us measured), set-up and epilogue once: about 12 chunks' worth.
  const int splits0 = a.items ? 1 : pick_splits(tiles, a.kc, g_sms, ctas_per_sm, 12);
  a.chunks_per_split = (a.kc + splits0 - 1) / splits0;
  const int splits = (a.kc + a.chunks_per_split - 1) / a.chunks_per_split;
  st = ensure_state((size_t)splits * (a.items ? (size_t)rows : (size_t)tts * tn) * a.nt * kTileN * sizeof(float));
  if (st != B200_OK) return st;
  a.ws = g_ws; a.err = g_err;
  CUtensorMap xmap;
  st = make_x_map(&xmap, a.x, rows, a.k, tn);
  if (st != B200_OK) return st;
  a.x_row0 = 0;
  qmm_tc_kernel<MODE><<<dim3(a.nt, splits, a.items ? a.max_items : tts), kTcThreads, smem, s>>>(xmap, a);
  B200_LAUNCH_CHECK();
  return (splits == 1 && tn <= 64) ? B200_OK : launch_finish(a, splits, s);  // a single small split writes its output itself
}

// Quantised weights, up to 128 rows per token tile (dense) or grouped work items: dequantised weights
// in tensor memory.
template <int MODE>
static b200_status launch_tca(QmmArgs& a, int rows, cudaStream_t s) {
  const int tn = a.items ? a.tn : std::min(256, ((rows + 15) / 16) * 16);
  a.tn = tn;
  const int tts = (rows + tn - 1) / tn;
  const int tiles = a.items ? a.nt * a.max_items : a.nt * tts;
  b200_status st = ensure_state(0);
  if (st != B200_OK) return st;
  static int smem_budget[3] = {0, 0, 0};
  if (smem_budget[MODE] == 0) {
    int dev = 0, optin = 0;
    B200_CUDA_TRY(cudaGetDevice(&dev));
    B200_CUDA_TRY(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    cudaFuncAttributes fa;
    B200_CUDA_TRY(cudaFuncGetAttributes(&fa, qmm_tca_kernel<MODE>));
    const int budget = optin - (int)fa.sharedSizeBytes;
    B200_CUDA_TRY(cudaFuncSetAttribute(qmm_tca_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, budget));
    smem_budget[MODE] = budget;
  }
  // Two CTAs per SM share the 512 tensor-memory columns: accumulator (tn rounded up to a power of
  // two) + 64 columns per slot of dequantised weights (a pair of chunks), 256 columns per CTA (all
  // 512 above 128 rows).
  const int ctas_per_sm = tn <= 128 ? 2 : 1;
  int acc_cols = 32;
  while (acc_cols < tn) acc_cols <<= 1;
  a.a_slots = std::min(4, ((ctas_per_sm == 2 ? 256 : 512) - acc_cols) / 64);
  // shared memory: two slots of activation-tile pairs, the rest a ring of raw block pairs
  const int per_cta = ctas_per_sm == 2 ? 113 * 1024 : std::min(smem_budget[MODE], 220 * 1024);
  a.x_slots = 2;
  const int fixed = 1024 /*alignment slack*/ + 8 * (2 * kTcaMaxWeightSlots + 2 * 2 + 2 * 4 + 2) + 16;
  a.stages = std::max(2, std::min(kTcaMaxWeightSlots, (per_cta - fixed - a.x_slots * 2 * tn * 128) / (2 * block_bytes(MODE))));
  const size_t smem = (size_t)a.x_slots * 2 * tn * 128 + (size_t)a.stages * 2 * block_bytes(MODE) + fixed;
  if ((int)smem > smem_budget[MODE] || a.a_slots < 2) {
    b200_set_error("qmm: %zu bytes of shared memory needed, %d available", smem, smem_budget[MODE]);
    return B200_ERR_CAPACITY;
  }
  const int splits0 = a.items ? 1 : pick_splits(tiles, a.kc, g_sms, ctas_per_sm, 12);
  a.chunks_per_split = (a.kc + splits0 - 1) / splits0;
  const int splits = (a.kc + a.chunks_per_split - 1) / a.chunks_per_split;
  // Prefill-sized batches (several token tiles, one K split) would need rows x N x 4 bytes of scratch:
  // the kernel writes its output itself instead.
  // ... and so does a single K split of up to 128-row tiles (gate/up at 128 rows 44.9 -> 42.9 us, lm_head 159 -> 147 us;
  // with 256-row tiles at one CTA per SM the longer epilogue costs more than the finish pass: 290 -> 302 us)
  a.direct_large = (!a.items && splits == 1 && (tts >= 4 || tn <= 128)) ? 1 : 0;
  const bool direct = splits == 1 && (tn <= 64 || a.direct_large);
  st = ensure_state(direct ? 0 : (size_t)splits * (a.items ? (size_t)rows : (size_t)tts * tn) * a.nt * kTileN * sizeof(float));
  if (st != B200_OK) return st;
  a.ws = g_ws; a.err = g_err;
  CUtensorMap xmap;
  st = make_x_map(&xmap, a.x, rows, a.k, tn);
  if (st != B200_OK) return st;
  a.x_row0 = 0;
  qmm_tca_kernel<MODE><<<dim3(a.nt, splits, a.items ? a.max_items : tts), kTcaThreads, smem, s>>>(xmap, a);
  B200_LAUNCH_CHECK();
  return direct ? B200_OK : launch_finish(a, splits, s);
}

// ---- block-scaled MXFP4 path: second weight layout, activation split, launch --------------------------
unsigned char* g_mx_act = nullptr;  // [hi: rows x k][lo: rows x k][unscale: rows f32], grown on demand
size_t g_mx_act_bytes = 0;

static b200_status prepare_mx(b200_qweight* w) {
  if (w->d_mx_codes) return B200_OK;
  if (w->mode != B200_Q_MXFP4_G32 || w->k % kMxK != 0) {
    b200_set_error("block-scaled path: MXFP4 weights with K a multiple of 128 only");
    return B200_ERR_UNSUPPORTED;
  }
  const size_t rows = (size_t)w->n_experts * w->nt * kTileN;
  const size_t code_bytes = rows * (size_t)(w->k / 2), sf_bytes = (size_t)w->n_experts * w->nt * (w->k / kMxK) * 512;
  B200_CUDA_TRY(cudaMalloc((void**)&w->d_mx_codes, code_bytes));
  cudaError_t e = cudaMalloc((void**)&w->d_mx_sf, sf_bytes);
  if (e != cudaSuccess) { cudaFree(w->d_mx_codes); w->d_mx_codes = nullptr; b200_set_error("cudaMalloc(%zu) failed: %s", sf_bytes, cudaGetErrorString(e)); return B200_ERR_CUDA; }
  mx_from_blocks_kernel<<<2048, 256>>>(w->d_blocks, w->d_mx_codes, w->d_mx_sf, w->n_experts * w->nt, w->kc, w->k);
  ++g_b200_launch_counter;
  e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  b200_status st = e == cudaSuccess ? B200_OK : B200_ERR_CUDA;
  if (st == B200_OK) {
    const uint64_t dims[2] = {(uint64_t)w->k, (uint64_t)rows};
    const uint64_t strides[1] = {(uint64_t)w->k / 2};
    const uint32_t box[2] = {(uint32_t)kMxK, (uint32_t)kTileN};
    st = b200_make_tensor_map(reinterpret_cast<CUtensorMap*>(w->mx_map), CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 2, w->d_mx_codes,
                              dims, strides, box);
  } else {
    b200_set_error("block-scaled path: layout conversion failed: %s", cudaGetErrorString(e));
  }
  if (st != B200_OK) { cudaFree(w->d_mx_codes); cudaFree(w->d_mx_sf); w->d_mx_codes = nullptr; w->d_mx_sf = nullptr; }
  return st;
}

int b200_qmm_mx_persistent = 1;
extern "C" void b200_set_qmm_mx_persistent(int32_t on) { b200_qmm_mx_persistent = on; }

static b200_status launch_finish(QmmArgs& a, int splits, cudaStream_t s);

static b200_status launch_mx(const b200_qweight* w, QmmArgs& a, int rows, cudaStream_t s) {
  b200_status st = prepare_mx(const_cast<b200_qweight*>(w));  // the handle caches its second layout
  if (st != B200_OK) return st;
  st = ensure_state(0);
  if (st != B200_OK) return st;
  // Dense batches of several token tiles: 112-row tiles keep two accumulator sets in the persistent kernel (gate/up
  // at 512 rows 126 vs 171 us, at 4096 rows 0.90 vs 1.05 ms), unless their grid fills its last wave much worse
  // than 128-row tiles would (16 tile pairs at 1024 rows: 160 items on 148 SMs against 128).
  int tn = a.items ? a.tn : std::min(128, ((rows + 15) / 16) * 16);
  if (!a.items && rows >= 448 && b200_qmm_mx_persistent) {
    const int pairs = (a.nt + 1) / 2;
    auto fill = [&](int t) {
      const long long items = (long long)pairs * ((rows + t - 1) / t);
      return (double)items / (double)(((items + g_sms - 1) / g_sms) * g_sms);
    };
    if (fill(112) * 1.15 >= fill(128)) tn = 112;
  }
  if (a.n % 16 != 0) { b200_set_error("block-scaled path: N must be a multiple of 16 (16-byte output stores)"); return B200_ERR_UNSUPPORTED; }
  if (tn > 128 || tn % 16 != 0) { b200_set_error("block-scaled path: token tiles of 16..128 rows (got %d)", tn); return B200_ERR_INVALID_ARGUMENT; }
  a.tn = tn;
  const int tts = (rows + tn - 1) / tn;
  const size_t act_bytes = 2 * (size_t)rows * a.k + sizeof(float) * (size_t)rows + 256;
  if (act_bytes > g_mx_act_bytes) {  // grown buffers replace, never free (see ensure_state)
    const size_t want = std::max(act_bytes + act_bytes / 4, (size_t)32 << 20);
    unsigned char* grown = nullptr;
    B200_CUDA_TRY(cudaMalloc((void**)&grown, want));
    if (g_mx_act) g_retired.push_back(g_mx_act);
    g_mx_act = grown;
    g_mx_act_bytes = want;
  }
  unsigned char* hi = g_mx_act;
  unsigned char* lo = hi + (size_t)rows * a.k;
  float* unscale = reinterpret_cast<float*>(lo + (((size_t)rows * a.k + 255) / 256) * 256);
  mx_split_activations_kernel<<<rows, 256, 0, s>>>(a.x, a.k, hi, lo, unscale, a.x_gather, a.x_gather_div, a.rows_valid);
  B200_LAUNCH_CHECK();
  MxActMaps amaps;
  std::memset(&amaps, 0, sizeof(amaps));
  const uint64_t dims[2] = {(uint64_t)a.k, (uint64_t)rows};
  const uint64_t strides[1] = {(uint64_t)a.k};
  for (int i = 0; i < 4 && 32 * (i + 1) <= ((tn + 31) / 32) * 32; ++i) {
    const uint32_t box[2] = {(uint32_t)kMxK, (uint32_t)std::min(tn, 32 * (i + 1))};
    st = b200_make_tensor_map(&amaps.hi[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, hi, dims, strides, box);
    if (st == B200_OK) st = b200_make_tensor_map(&amaps.lo[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, lo, dims, strides, box);
    if (st != B200_OK) return st;
  }
  static int smem_budget = 0;
  if (smem_budget == 0) {
    int dev = 0, optin = 0;
    B200_CUDA_TRY(cudaGetDevice(&dev));
    B200_CUDA_TRY(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    cudaFuncAttributes fa, fb;
    B200_CUDA_TRY(cudaFuncGetAttributes(&fa, qmm_mx_kernel));
    B200_CUDA_TRY(cudaFuncGetAttributes(&fb, qmm_mxp_kernel));
    const int budget = optin - (int)std::max(fa.sharedSizeBytes, fb.sharedSizeBytes);
    B200_CUDA_TRY(cudaFuncSetAttribute(qmm_mx_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, budget));
    B200_CUDA_TRY(cudaFuncSetAttribute(qmm_mxp_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, budget));
    smem_budget = budget;
  }
  a.err = g_err;
  a.mx_sf = w->d_mx_sf;
  a.act_unscale = unscale;
  a.mx_expert_rows = w->nt * kTileN;
  a.kc128 = a.k / kMxK;
  a.x_row0 = 0;
  const int stage = 2 * kTileN * kMxK + 2 * tn * 128 + 1024;
  if (b200_qmm_mx_persistent) {
    // persistent form: one CTA per SM walks the work items; dense launches with few tile pairs split K
    const int fixed = 1024 + 2 * kMxpStageTokens * kTileN * (int)sizeof(float) + 8 * (2 * 8 + 6) + 16;
    a.stages = std::max(2, std::min(6, (std::min(smem_budget, 224 * 1024) - fixed) / stage));
    const size_t smem = (size_t)a.stages * stage + fixed;
    if ((int)smem > smem_budget) { b200_set_error("block-scaled path: %zu bytes of shared memory needed, %d available", smem, smem_budget); return B200_ERR_CAPACITY; }
    const int pairs = (a.nt + 1) / 2;
    int splits = 1;
    if (!a.items) {
      // enough work items to give every SM a few chunks of K at a time; each split keeps >= 4 chunks of 128
      const int base = pairs * tts;
      while (base * splits < 2 * g_sms && a.kc128 / (splits * 2) >= 4 && splits < 16) splits *= 2;
    }
    a.splits = splits;
    a.chunks_per_split = (a.kc128 + splits - 1) / splits;
    const int real_splits = (a.kc128 + a.chunks_per_split - 1) / a.chunks_per_split;
    a.splits = real_splits;
    if (real_splits > 1) {
      st = ensure_state((size_t)real_splits * (size_t)tts * tn * a.nt * kTileN * sizeof(float));
      if (st != B200_OK) return st;
      a.ws = g_ws;
    }
    const long long n_work = a.items ? (long long)pairs * a.max_items : (long long)pairs * tts * real_splits;
    const int grid = (int)std::max<long long>(1, std::min<long long>(g_sms, n_work));
    qmm_mxp_kernel<<<grid, kMxpThreads, smem, s>>>(*reinterpret_cast<const CUtensorMap*>(w->mx_map), amaps, a);
    B200_LAUNCH_CHECK();
    return real_splits > 1 ? launch_finish(a, real_splits, s) : B200_OK;
  }
  const int fixed = 1024 + 8 * (3 * 4 + 1) + 16;
  a.stages = std::max(2, std::min(4, (std::min(smem_budget, 220 * 1024) - fixed) / stage));
  a.stages = std::min(a.stages, std::max(2, a.k / kMxK));
  const size_t smem = (size_t)a.stages * stage + fixed;
  if ((int)smem > smem_budget) { b200_set_error("block-scaled path: %zu bytes of shared memory needed, %d available", smem, smem_budget); return B200_ERR_CAPACITY; }
  qmm_mx_kernel<<<dim3((a.nt + 1) / 2, 1, a.items ? a.max_items : tts), kMxThreads, smem, s>>>(
      *reinterpret_cast<const CUtensorMap*>(w->mx_map), amaps, a);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

// Large batches (129..256 rows per token tile): two weight tiles per CTA.
template <int MODE>
static b200_status launch_tc2(QmmArgs& a, int rows, cudaStream_t s) {
  const int tn = std::min(256, ((rows + 15) / 16) * 16);
  a.tn = tn;
  const int tts = (rows + tn - 1) / tn;
  const int pairs = (a.nt + 1) / 2;
  b200_status st = ensure_state(0);
  if (st != B200_OK) return st;
  constexpr int BB = block_bytes(MODE);
  constexpr int RB = MODE == B200_Q_BF16 ? 0 : ((BB + 127) / 128) * 128;
  const int stage_stride = 2 * kTileN * 128 + tn * 128;
  static int smem_budget[3] = {0, 0, 0};
  if (smem_budget[MODE] == 0) {
    int dev = 0, optin = 0;
    B200_CUDA_TRY(cudaGetDevice(&dev));
    B200_CUDA_TRY(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    cudaFuncAttributes fa;
    B200_CUDA_TRY(cudaFuncGetAttributes(&fa, qmm_tc2_kernel<MODE>));
    const int budget = optin - (int)fa.sharedSizeBytes;
    B200_CUDA_TRY(cudaFuncSetAttribute(qmm_tc2_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, budget));
    smem_budget[MODE] = budget;
  }
  // stages of two MMA tiles + one activation tile; quantised weights add a ring of raw block pairs: at least
  // three slots, then whatever the stages leave over
  const int fixed = 1024 /*alignment slack*/ + 8 * (3 * 6 + 2 * 8 + 2) + 16;
  const int raw_min = MODE == B200_Q_BF16 ? 0 : 3 * 2 * RB;
  a.stages = std::min(6, (smem_budget[MODE] - fixed - raw_min) / stage_stride);
  if (a.stages < 2) {
    b200_set_error("qmm: %d bytes of shared memory per stage, %d available", stage_stride, smem_budget[MODE]);
    return B200_ERR_CAPACITY;
  }
  a.x_slots = MODE == B200_Q_BF16 ? a.stages : std::min(8, (smem_budget[MODE] - fixed - a.stages * stage_stride) / (2 * RB));
  const size_t smem = (size_t)a.stages * stage_stride + (MODE == B200_Q_BF16 ? 0 : (size_t)a.x_slots * 2 * RB) + fixed;
  // a K split costs a 128 x tn f32 tile written and read back per weight tile: weigh it as chunks
  const int splits0 = pick_splits(pairs * tts, a.kc, g_sms, 1, 2 + tn / 32);
  a.chunks_per_split = (a.kc + splits0 - 1) / splits0;
  const int splits = (a.kc + a.chunks_per_split - 1) / a.chunks_per_split;
  st = ensure_state(splits > 1 ? (size_t)splits * (size_t)tts * tn * a.nt * kTileN * sizeof(float) : 0);
  if (st != B200_OK) return st;
  a.ws = g_ws; a.err = g_err;
  CUtensorMap xmap;
  st = make_x_map(&xmap, a.x, rows, a.k, tn);
  if (st != B200_OK) return st;
  a.x_row0 = 0;
  qmm_tc2_kernel<MODE><<<dim3(pairs, splits, tts), kTc2Threads, smem, s>>>(xmap, a);
  B200_LAUNCH_CHECK();
  return splits == 1 ? B200_OK : launch_finish(a, splits, s);
}

template <int MODE, int NT8>
static b200_status launch_mma_nt(QmmArgs& a, int rows, cudaStream_t s) {
  const int tile = NT8 * 8;
  a.tn = tile;
  const int tts = (rows + tile - 1) / tile;
  b200_status st = ensure_state(0);
  if (st != B200_OK) return st;
  // Persistent grid: `groups` CTAs per K split, each walking every groups-th weight tile.  Pick the
  // split count whose slab fits 48 KiB and whose critical path (tiles per CTA x (chunks + 1) plus a
  // fixed start-up worth ~8 chunks) is shortest at two CTAs per SM.
  a.stages = kGemvRawStages;
  const size_t base_smem = (size_t)a.stages * 2 * kRawStride + 2 * a.stages * sizeof(uint64_t);
  auto slab_bytes = [&](int cps) { return (size_t)tile * ((size_t)cps * kChunkK * 2 + kSlabPad) + (size_t)tile * cps * sizeof(float); };
  const int slots = std::max(1, g_sms * 2 / tts);
  int best = 0, best_groups = 1;
  long long best_cost = 0;
  for (int sp = 1; sp <= std::min(a.kc, slots); ++sp) {
    const int cps = (a.kc + sp - 1) / sp;
    if ((a.kc + cps - 1) / cps != sp || slab_bytes(cps) > 48 * 1024) continue;
    if (best && cps < 2) break;
    const int pairs = (a.nt + 1) / 2;
    const int groups = std::max(1, std::min(pairs, slots / sp));
    const long long cost = (long long)((pairs + groups - 1) / groups) * (2 * cps + 1) + 8;
    if (!best || cost < best_cost) { best = sp; best_cost = cost; best_groups = groups; }
  }
  if (!best) { b200_set_error("qmm: no K split fits the activation slab"); return B200_ERR_CAPACITY; }
  const int splits = best;
  a.splits = splits;
  a.chunks_per_split = (a.kc + splits - 1) / splits;
  st = ensure_state((size_t)splits * (size_t)tts * tile * a.nt * kTileN * sizeof(float));
  if (st != B200_OK) return st;
  a.ws = g_ws; a.err = g_err;
  a.x_slab = 1;
  const size_t smem = base_smem + slab_bytes(a.chunks_per_split);
  static bool configured = false;
  if (!configured) {
    B200_CUDA_TRY(cudaFuncSetAttribute(qmm_mma_kernel<MODE, NT8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)(base_smem + 48 * 1024)));
    configured = true;
  }
  qmm_mma_kernel<MODE, NT8><<<dim3(best_groups * splits, tts), kGemvThreads, smem, s>>>(a);
  B200_LAUNCH_CHECK();
  return launch_finish(a, splits, s);
}

template <int NT8>
static b200_status launch_mma8_nt(QmmArgs& a, int rows, cudaStream_t s) {
  const int tile = NT8 * 8;
  a.tn = tile;
  const int tts = (rows + tile - 1) / tile;
  b200_status st = ensure_state(0);
  if (st != B200_OK) return st;
  a.stages = kGemvRawStages;
  const size_t base_smem = (size_t)a.stages * 2 * kRawStride + 2 * a.stages * sizeof(uint64_t);
  // two int8 slabs, the group sums, the per-token scales and a little scratch
  auto slab_bytes = [&](int cps) {
    return 2 * (size_t)tile * slab8_stride(cps) + 2 * (size_t)tile * cps * sizeof(float) + 64;
  };
  const int slots = std::max(1, g_sms * 2 / tts);
  int best = 0, best_groups = 1;
  long long best_cost = 0;
  for (int sp = 1; sp <= std::min(a.kc, slots); ++sp) {
    const int cps = (a.kc + sp - 1) / sp;
    if ((a.kc + cps - 1) / cps != sp || slab_bytes(cps) > 48 * 1024) continue;
    if (best && cps < 2) break;
    const int pairs = (a.nt + 1) / 2;
    const int groups = std::max(1, std::min(pairs, slots / sp));
    const long long cost = (long long)((pairs + groups - 1) / groups) * (2 * cps + 1) + 8;
    if (!best || cost < best_cost) { best = sp; best_cost = cost; best_groups = groups; }
  }
  if (!best) { b200_set_error("qmm: no K split fits the activation slab"); return B200_ERR_CAPACITY; }
  const int splits = best;
  a.splits = splits;
  a.chunks_per_split = (a.kc + splits - 1) / splits;
  st = ensure_state((size_t)splits * (size_t)tts * tile * a.nt * kTileN * sizeof(float));
  if (st != B200_OK) return st;
  a.ws = g_ws; a.err = g_err;
  a.x_slab = 1;
  const size_t smem = base_smem + slab_bytes(a.chunks_per_split);
  static bool configured = false;
  if (!configured) {
    B200_CUDA_TRY(cudaFuncSetAttribute(qmm_mma8_kernel<NT8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(base_smem + 48 * 1024)));
    configured = true;
  }
  qmm_mma8_kernel<NT8><<<dim3(best_groups * splits, tts), kGemvThreads, smem, s>>>(a);
  B200_LAUNCH_CHECK();
  return launch_finish(a, splits, s);
}

static b200_status launch_mma8(QmmArgs& a, int rows, cudaStream_t s) {
  if (rows <= 8) return launch_mma8_nt<1>(a, rows, s);
  if (rows <= 16) return launch_mma8_nt<2>(a, rows, s);
  return launch_mma8_nt<4>(a, rows, s);
}

template <int MODE>
static b200_status launch_mma(QmmArgs& a, int rows, cudaStream_t s) {
  if (rows <= 8) return launch_mma_nt<MODE, 1>(a, rows, s);
  if (rows <= 16) return launch_mma_nt<MODE, 2>(a, rows, s);
  return launch_mma_nt<MODE, 4>(a, rows, s);
}

int b200_qmm_grouped_tmem_a = 1;  // measured 15.1 vs 15.8 ms on the 4-layer MoE stack
extern "C" void b200_set_qmm_grouped_tmem_a(int32_t on) { b200_qmm_grouped_tmem_a = on; }
// MXFP4 grouped matmuls on the block-scaled tensor-core path: 13.8 vs 15.3 ms on the 4-layer MoE stack
int b200_qmm_grouped_block_scaled = 1;
extern "C" void b200_set_qmm_grouped_block_scaled(int32_t on) { b200_qmm_grouped_block_scaled = on; }

static b200_status qmm_entry(const b200_qweight* w, const void* d_x, int32_t rows, void* d_y, int32_t epilogue,
                             const void* d_residual, float swiglu_limit, int32_t path, void* stream, const void* d_norm_w,
                             float norm_eps, void* d_norm_out, int* did_norm);

extern "C" b200_status b200_qmm(const b200_qweight* w, const void* d_x, int32_t rows, void* d_y, int32_t epilogue,
                                const void* d_residual, float swiglu_limit, int32_t path, void* stream) {
  return qmm_entry(w, d_x, rows, d_y, epilogue, d_residual, swiglu_limit, path, stream, nullptr, 0.f, nullptr, nullptr);
}

// Set by b200_qmm_deferred around its call of qmm_entry (one calling thread per process uses the matmul entry points).
static b200_qmm_partials* g_defer_target = nullptr;

extern "C" b200_status b200_qmm_deferred(const b200_qweight* w, const void* d_x, int32_t rows, void* d_y, int32_t defer, void* stream,
                                         b200_qmm_partials* out) {
  std::memset(out, 0, sizeof(*out));
  g_defer_target = defer ? out : nullptr;
  const b200_status st = qmm_entry(w, d_x, rows, d_y, B200_EPI_NONE, nullptr, 0.f, B200_QMM_AUTO, stream, nullptr, 0.f, nullptr, nullptr);
  g_defer_target = nullptr;
  return st;
}

extern "C" b200_status b200_rmsnorm(const void* d_x, const void* d_weight, void* d_out, int32_t rows, int32_t hidden, float eps,
                                    void* stream);

extern "C" b200_status b200_qmm_residual_norm(const b200_qweight* w, const void* d_x, int32_t rows, void* d_y,
                                              const void* d_residual, const void* d_norm_weight, float eps, void* d_normed,
                                              void* stream) {
  if (rows <= 0) return B200_OK;
  if (!d_residual || !d_norm_weight || !d_normed || !d_y) { b200_set_error("qmm_residual_norm: null argument"); return B200_ERR_INVALID_ARGUMENT; }
  if (w->n % 8 != 0) { b200_set_error("qmm_residual_norm: N must be a multiple of 8"); return B200_ERR_INVALID_ARGUMENT; }
  int did_norm = 0;
  b200_status st = qmm_entry(w, d_x, rows, d_y, B200_EPI_RESIDUAL, d_residual, 0.f, B200_QMM_AUTO, stream, d_norm_weight, eps, d_normed,
                             &did_norm);
  if (st != B200_OK) return st;
  // kernels that wrote y themselves (no K split) leave the normalisation to the row kernel
  return did_norm ? B200_OK : b200_rmsnorm(d_y, d_norm_weight, d_normed, rows, w->n, eps, stream);
}

static b200_status qmm_entry(const b200_qweight* w, const void* d_x, int32_t rows, void* d_y, int32_t epilogue,
                             const void* d_residual, float swiglu_limit, int32_t path, void* stream, const void* d_norm_w,
                             float norm_eps, void* d_norm_out, int* did_norm) {
  b200_status st = b200_require_device();
  if (st != B200_OK) return st;
  if (rows <= 0) return B200_OK;
  if (w->n_experts != 1) { b200_set_error("qmm: stacked expert weights go through the grouped entry point"); return B200_ERR_INVALID_ARGUMENT; }
  if (epilogue == B200_EPI_RESIDUAL && !d_residual) { b200_set_error("qmm: residual epilogue without a residual"); return B200_ERR_INVALID_ARGUMENT; }
  if (epilogue == B200_EPI_SWIGLU && (w->n % 2) != 0) { b200_set_error("qmm: SwiGLU needs an even N"); return B200_ERR_INVALID_ARGUMENT; }
  // Quantised weights, up to 16 rows: register-dequant mma.sync kernel (pure weight streaming).  More
  // rows: tcgen05 with the dequantised weights in tensor memory; above 128 rows the tile-pair kernel
  // where its grid is one well-filled wave without a K split (gate/up-sized matrices: 74 vs 85 us at
  // 256 rows; elsewhere the tensor-memory kernel measured 3-8 % faster).  Dense bf16 weights: the
  // shared-memory-operand kernels.
  if (path == B200_QMM_AUTO) {
    // MXFP4 at prefill-sized batches: the block-scaled tensor-core path once its grid (tile pairs x
    // 128-row token tiles, no K split) fills most of the GPU: 188 vs 261 us at 4096 x 4096 x 4096,
    // 1.07 vs 1.62 ms at 4096 rows of a 28672 x 4096 matrix; below that the dequantising kernels win.
    if (w->mode == B200_Q_MXFP4_G32 && rows >= 512 && w->k % kMxK == 0 && w->n % 16 == 0 &&
        ((w->nt + 1) / 2) * ((rows + 127) / 128) >= 96)
      path = B200_QMM_MXFP4_BLOCK_SCALED;
    // 16..128 rows of a very wide matrix (lm_head): the persistent block-scaled kernel streams the weights
    // without any conversion work (110 vs 124 us at 16 rows, 125 vs 162 us at 64 rows of 128256 x 4096)
    if (w->mode == B200_Q_MXFP4_G32 && rows >= 16 && rows <= 128 && w->n >= 65536 && w->k % kMxK == 0 && w->n % 16 == 0 &&
        b200_qmm_mx_persistent)
      path = B200_QMM_MXFP4_BLOCK_SCALED;
  }
  if (path == B200_QMM_AUTO) {
    // up to 8 rows of affine int4: the integer small-batch kernel (lm_head 59 vs 80 us, gate/up 20 vs 23 us at
    // one row); 9..16 rows only on the largest matrices, where its longer activation staging is amortised
    if (rows <= 16 && w->mode == B200_Q_AFFINE4_G64 && (rows <= 8 || w->n >= 32768)) path = B200_QMM_MMA_I8;
    else if (rows <= 16 && w->mode != B200_Q_BF16) path = B200_QMM_MMA;
    else if (rows > 128) {
      const int tn = std::min(256, ((rows + 15) / 16) * 16), pair_ctas = ((w->nt + 1) / 2) * ((rows + tn - 1) / tn);
      if (ensure_state(0) != B200_OK) return B200_ERR_CUDA;
      const bool one_wave = pair_ctas <= g_sms && pair_ctas * 2 >= g_sms;
      // more than one 256-row token tile (prefill chunks): the tile-pair kernel is ahead or level on
      // every projection shape (gate/up 122 vs 158 us at 384 rows, 126 vs 172 us at 512, 317 vs 337 us
      // at 1024; down 113 vs 121 us at 1024)
      path = (one_wave || rows > 256 || w->mode == B200_Q_BF16) ? B200_QMM_TCGEN05_X2 : B200_QMM_TCGEN05_TMEM_A;
    } else {
      path = w->mode == B200_Q_BF16 ? B200_QMM_TCGEN05 : B200_QMM_TCGEN05_TMEM_A;
    }
  }
  if (path == B200_QMM_MMA && w->mode == B200_Q_BF16) path = B200_QMM_TCGEN05;
  QmmArgs a{};
  a.blocks = w->d_blocks; a.x = (const __nv_bfloat16*)d_x; a.y = (__nv_bfloat16*)d_y;
  a.residual = (const __nv_bfloat16*)d_residual;
  a.rows = rows; a.n = w->n; a.k = w->k; a.nt = w->nt; a.kc = w->kc; a.epilogue = epilogue; a.swiglu_limit = swiglu_limit;
  a.norm_w = (const __nv_bfloat16*)d_norm_w; a.norm_out = (__nv_bfloat16*)d_norm_out; a.norm_eps = norm_eps;
  a.defer = g_defer_target;
  cudaStream_t s = (cudaStream_t)stream;
  auto dispatch = [&]() -> b200_status {
    if (path == B200_QMM_MXFP4_BLOCK_SCALED) return launch_mx(w, a, rows, s);
    if (path == B200_QMM_MMA_I8) {
      if (w->mode != B200_Q_AFFINE4_G64) { b200_set_error("qmm: the integer small-batch kernel serves affine int4 weights"); return B200_ERR_UNSUPPORTED; }
      return launch_mma8(a, rows, s);
    }
    if (path == B200_QMM_MMA)
      return w->mode == B200_Q_AFFINE4_G64 ? launch_mma<B200_Q_AFFINE4_G64>(a, rows, s) : launch_mma<B200_Q_MXFP4_G32>(a, rows, s);
    if (path == B200_QMM_SIMT) {
      if (w->mode == B200_Q_AFFINE4_G64) return launch_simt<B200_Q_AFFINE4_G64>(a, rows, s);
      if (w->mode == B200_Q_MXFP4_G32) return launch_simt<B200_Q_MXFP4_G32>(a, rows, s);
      return launch_simt<B200_Q_BF16>(a, rows, s);
    }
    if (path == B200_QMM_TCGEN05_TMEM_A && w->mode != B200_Q_BF16)
      return w->mode == B200_Q_AFFINE4_G64 ? launch_tca<B200_Q_AFFINE4_G64>(a, rows, s) : launch_tca<B200_Q_MXFP4_G32>(a, rows, s);
    if (path == B200_QMM_TCGEN05_X2) {
      if (w->mode == B200_Q_AFFINE4_G64) return launch_tc2<B200_Q_AFFINE4_G64>(a, rows, s);
      if (w->mode == B200_Q_MXFP4_G32) return launch_tc2<B200_Q_MXFP4_G32>(a, rows, s);
      return launch_tc2<B200_Q_BF16>(a, rows, s);
    }
    if (w->mode == B200_Q_AFFINE4_G64) return launch_tc<B200_Q_AFFINE4_G64>(a, rows, s);
    if (w->mode == B200_Q_MXFP4_G32) return launch_tc<B200_Q_MXFP4_G32>(a, rows, s);
    return launch_tc<B200_Q_BF16>(a, rows, s);
  };
  st = dispatch();
  if (did_norm) *did_norm = a.did_norm;
  return st;
}

// Grouped matmul over an expert-sorted batch: work item i = {expert, first row, rows}; every
// item multiplies its rows by its expert's weight.  d_items / d_n_items live on the device
// (built by the grouping kernels); max_items bounds the grid.
b200_status b200_qmm_grouped(const b200_qweight* w, const void* d_x, int32_t rows, void* d_y, int32_t epilogue,
                             const float* d_row_scales, float swiglu_limit, const int4* d_items, const int* d_n_items,
                             int32_t max_items, int32_t tile_rows, void* stream) {
  b200_status st = b200_require_device();
  if (st != B200_OK) return st;
  if (rows <= 0) return B200_OK;
  QmmArgs a{};
  a.blocks = w->d_blocks; a.x = (const __nv_bfloat16*)d_x; a.y = (__nv_bfloat16*)d_y; a.residual = nullptr;
  a.row_scales = d_row_scales;
  a.rows = rows; a.n = w->n; a.k = w->k; a.nt = w->nt; a.kc = w->kc; a.epilogue = epilogue; a.swiglu_limit = swiglu_limit;
  a.items = d_items; a.n_items = d_n_items; a.max_items = max_items; a.tn = tile_rows;
  a.expert_stride = (size_t)w->nt * w->kc * w->block_bytes;
  cudaStream_t s = (cudaStream_t)stream;
  if (b200_qmm_grouped_block_scaled && w->mode == B200_Q_MXFP4_G32 && w->k % kMxK == 0 && tile_rows <= 128) return launch_mx(w, a, rows, s);
  if (b200_qmm_grouped_tmem_a && w->mode != B200_Q_BF16)
    return w->mode == B200_Q_AFFINE4_G64 ? launch_tca<B200_Q_AFFINE4_G64>(a, rows, s) : launch_tca<B200_Q_MXFP4_G32>(a, rows, s);
  if (w->mode == B200_Q_AFFINE4_G64) return launch_tc<B200_Q_AFFINE4_G64>(a, rows, s);
  if (w->mode == B200_Q_MXFP4_G32) return launch_tc<B200_Q_MXFP4_G32>(a, rows, s);
  return launch_tc<B200_Q_BF16>(a, rows, s);
}

int b200_qmm_grouped_takes_tokens(const b200_qweight* w, int32_t tile_rows) {
  return b200_qmm_grouped_block_scaled && w->mode == B200_Q_MXFP4_G32 && w->k % kMxK == 0 && w->n % 16 == 0 && tile_rows <= 128 &&
         tile_rows % 16 == 0;
}

b200_status b200_qmm_grouped_from_tokens(const b200_qweight* w, const void* d_tokens, const int* d_order, int32_t top_k,
                                         int32_t rows, void* d_y, int32_t epilogue, const float* d_row_scales,
                                         float swiglu_limit, const int4* d_items, const int* d_n_items, int32_t max_items,
                                         int32_t tile_rows, void* stream, const int* d_rows_valid) {
  b200_status st = b200_require_device();
  if (st != B200_OK) return st;
  if (rows <= 0) return B200_OK;
  if (!b200_qmm_grouped_takes_tokens(w, tile_rows)) { b200_set_error("grouped matmul from tokens: block-scaled MXFP4 path only"); return B200_ERR_UNSUPPORTED; }
  QmmArgs a{};
  a.blocks = w->d_blocks; a.x = (const __nv_bfloat16*)d_tokens; a.y = (__nv_bfloat16*)d_y; a.residual = nullptr;
  a.row_scales = d_row_scales;
  a.rows = rows; a.n = w->n; a.k = w->k; a.nt = w->nt; a.kc = w->kc; a.epilogue = epilogue; a.swiglu_limit = swiglu_limit;
  a.items = d_items; a.n_items = d_n_items; a.max_items = max_items; a.tn = tile_rows;
  a.x_gather = d_order; a.x_gather_div = top_k;
  a.rows_valid = d_rows_valid;
  return launch_mx(w, a, rows, (cudaStream_t)stream);
}

namespace {
constexpr int kMaxDevices = 64;
// Error word of the allocation-free entry point, per device (resolved at that entry point's set-up).
int* g_static_err_ptr[kMaxDevices] = {nullptr};

int* static_err_of_current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  return g_static_err_ptr[dev];
}
}  // namespace

// Reads and clears the matmul kernels' error words (a bounded wait that ran out): the word of the
// kernels launched by b200_qmm / the grouped entry points, and the word of b200_qmm_static_scratch on
// the current device.
extern "C" b200_status b200_qmm_error_word(int32_t* out) {
  *out = 0;
  int32_t dyn = 0, stat = 0;
  if (g_err) {
    B200_CUDA_TRY(cudaMemcpy(&dyn, g_err, sizeof(int), cudaMemcpyDeviceToHost));
    if (dyn != 0) B200_CUDA_TRY(cudaMemset(g_err, 0, sizeof(int)));
  }
  if (int* se = static_err_of_current_device()) {
    B200_CUDA_TRY(cudaMemcpy(&stat, se, sizeof(int), cudaMemcpyDeviceToHost));
    if (stat != 0) B200_CUDA_TRY(cudaMemset(se, 0, sizeof(int)));
  }
  *out = dyn != 0 ? dyn : stat;
  return B200_OK;
}

// Queues copies of both error words into pinned host memory on `stream` (no synchronisation, nothing
// cleared): h_out[0] = b200_qmm's word, h_out[1] = the allocation-free entry point's.
b200_status b200_qmm_error_words_async(int32_t* h_out, void* stream) {
  h_out[0] = h_out[1] = 0;
  if (g_err) B200_CUDA_TRY(cudaMemcpyAsync(h_out, g_err, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  if (int* se = static_err_of_current_device())
    B200_CUDA_TRY(cudaMemcpyAsync(h_out + 1, se, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  return B200_OK;
}

namespace {
// One thread waits, with a short limit, on a barrier that nothing will ever complete: the wait runs
// out, the thread records that in the error word exactly as the matmul kernels do, and the kernel
// returns.  Nothing faults or spins for ever; the context stays usable.
__global__ void wait_runs_out_kernel(int* err, uint32_t polls) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    ptx::mbar_init(&bar, 1);
    ptx::mbar_fence_init();
    const bool ok = ptx::mbar_wait_limit(&bar, 0, polls);
    if (!ok) atomicExch(err, B200_ERR_DEVICE_FLAGGED);
  }
}
}  // namespace

// Test hook (no reference counterpart): runs the kernels' give-up path for real.  A kernel waits at
// most `polls` polls (a fraction of a millisecond for a few thousand) for a barrier nobody arrives on,
// sets the matmul error word and returns; the caller then reads B200_ERR_DEVICE_FLAGGED through
// b200_qmm_error_word and goes on using the library.
extern "C" b200_status b200_qmm_debug_wait_runs_out(int32_t polls, void* stream) {
  b200_status st = b200_require_device();
  if (st != B200_OK) return st;
  if (polls <= 0 || polls > (1 << 20)) { b200_set_error("wait probe: 1..2^20 polls"); return B200_ERR_INVALID_ARGUMENT; }
  st = ensure_state(0);
  if (st != B200_OK) return st;
  wait_runs_out_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(g_err, (uint32_t)polls);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

// Test hook (no reference counterpart): the error word a b200_qmm launch would report through, so that a
// test can check the read-and-clear path without making a kernel time out.
extern "C" b200_status b200_qmm_debug_set_error_word(int32_t value, int32_t static_scratch_word) {
  int* dst = static_scratch_word ? static_err_of_current_device() : g_err;
  if (!dst) { b200_set_error("error word not set up yet (no matmul has run)"); return B200_ERR_INVALID_ARGUMENT; }
  B200_CUDA_TRY(cudaMemcpy(dst, &value, sizeof(int), cudaMemcpyHostToDevice));
  return B200_OK;
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of the tensor-core matmul.
//
// b200_qmm grows its split-K scratch with cudaMalloc the first time a shape needs more room.
// Some hosts cannot take that: an engine that has handed every remaining byte of HBM to its KV
// page pool (a late cudaMalloc then fails in the middle of serving), a step that is being
// recorded into a CUDA graph or runs beside other streams (cudaMalloc synchronises the whole
// device), or an embedding whose rules forbid allocating after start-up.  For them the scratch
// lives in the library image: a fixed device array that every GPU loading the library holds
// until the process exits.
//
//  * Limit: K-splits * round_up(rows, token tile) * round_up(N,128) * 4 bytes must fit in
//    kStaticScratchBytes (32 MiB), the token tile being min(256, round_up(rows,16)) rows (257 rows
//    count as 512); larger problems are refused with B200_ERR_CAPACITY, nothing is launched.
//  * The first call on each device looks up the array's device address (cudaGetSymbolAddress);
//    make that call before any stream capture.
//  * All calls share the one array and it keeps whatever the previous call left there.  Every
//    element a call reads it has written first, so nothing needs clearing, but two calls that
//    overlap on the GPU (different streams, no ordering between them) race on it.
// ---------------------------------------------------------------------------------------------
namespace {
constexpr size_t kStaticScratchBytes = (size_t)32 << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
static __device__ __align__(256) int g_static_err[64];
float* g_static_ws[kMaxDevices] = {nullptr};
int g_static_sms[kMaxDevices] = {0};
int g_static_budget[kMaxDevices][3] = {};  // opt-in dynamic shared memory: a per-device function attribute

template <int MODE>
b200_status launch_tc_static(QmmArgs& a, int rows, int dev, cudaStream_t s) {
  const int tn = std::min(256, ((rows + 15) / 16) * 16);
  a.tn = tn;
  const int tts = (rows + tn - 1) / tn;
  const int tiles = a.nt * tts;
  constexpr int kRaw = MODE == B200_Q_BF16 ? 0 : ((block_bytes(MODE) + 127) / 128) * 128;
  const int stage_stride = kTileN * 128 + tn * 128 + kRaw;
  int* budget = g_static_budget[dev];
  if (budget[MODE] == 0) {
    int optin = 0;
    B200_CUDA_TRY(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    cudaFuncAttributes fa;
    B200_CUDA_TRY(cudaFuncGetAttributes(&fa, qmm_tc_kernel<MODE>));
    const int b = optin - (int)fa.sharedSizeBytes;
    B200_CUDA_TRY(cudaFuncSetAttribute(qmm_tc_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, b));
    budget[MODE] = b;
  }
  const int fixed = 1024 + 8 * (3 * 8 + 2) + 16;
  const int per_cta = tn <= 128 ? 110 * 1024 : std::min(budget[MODE], 220 * 1024);
  a.stages = std::max(2, std::min(8, (per_cta - fixed) / stage_stride));
  const int ctas_per_sm = tn <= 128 ? 2 : 1;
  const size_t smem = (size_t)a.stages * stage_stride + fixed;
  if ((int)smem > budget[MODE]) {
    b200_set_error("qmm (static scratch): %zu bytes of shared memory needed, %d available", smem, budget[MODE]);
    return B200_ERR_CAPACITY;
  }
  const int splits0 = pick_splits(tiles, a.kc, g_static_sms[dev], ctas_per_sm);
  a.chunks_per_split = (a.kc + splits0 - 1) / splits0;
  const int splits = (a.kc + a.chunks_per_split - 1) / a.chunks_per_split;
  const size_t need = (size_t)splits * tts * tn * a.nt * kTileN * sizeof(float);  // token tiles are padded to tn rows
  if (need > kStaticScratchBytes) {
    b200_set_error("qmm (static scratch): %d rows (token tiles of %d) x N=%d in %d K-splits need %zu bytes of scratch, the built-in array holds %zu",
                   rows, tn, a.n, splits, need, kStaticScratchBytes);
    return B200_ERR_CAPACITY;
  }
  a.ws = g_static_ws[dev];
  a.err = g_static_err_ptr[dev];
  CUtensorMap xmap;
  b200_status st = make_x_map(&xmap, a.x, rows, a.k, tn);
  if (st != B200_OK) return st;
  a.x_row0 = 0;
  qmm_tc_kernel<MODE><<<dim3(a.nt, splits, tts), kTcThreads, smem, s>>>(xmap, a);
  B200_LAUNCH_CHECK();
  return (splits == 1 && tn <= 64) ? B200_OK : launch_finish(a, splits, s);
}
}  // namespace

extern "C" b200_status b200_qmm_static_scratch(const b200_qweight* w, const void* d_x, int32_t rows, void* d_y,
                                               int32_t epilogue, const void* d_residual, float swiglu_limit,
                                               void* stream) {
  b200_status st = b200_require_any_device();
  if (st != B200_OK) return st;
  if (rows <= 0) return B200_OK;
  if (w->n_experts != 1) { b200_set_error("qmm (static scratch): single weights only"); return B200_ERR_INVALID_ARGUMENT; }
  if (epilogue == B200_EPI_RESIDUAL && !d_residual) { b200_set_error("qmm (static scratch): residual epilogue without a residual"); return B200_ERR_INVALID_ARGUMENT; }
  if (epilogue == B200_EPI_SWIGLU && (w->n % 2) != 0) { b200_set_error("qmm (static scratch): SwiGLU needs an even N"); return B200_ERR_INVALID_ARGUMENT; }
  int dev = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) { b200_set_error("qmm (static scratch): device ordinal %d not supported", dev); return B200_ERR_INVALID_ARGUMENT; }
  if (!g_static_ws[dev]) {
    // Set-up, once per device, with that device current: the array's name is only a host-side
    // handle here; the kernel needs the address the symbol has on this device.
    void* p = nullptr;
    B200_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
    void* e = nullptr;
    B200_CUDA_TRY(cudaGetSymbolAddress(&e, g_static_err));
    B200_CUDA_TRY(cudaDeviceGetAttribute(&g_static_sms[dev], cudaDevAttrMultiProcessorCount, dev));
    g_static_err_ptr[dev] = (int*)e;
    g_static_ws[dev] = (float*)p;
  }
  QmmArgs a{};
  a.blocks = w->d_blocks; a.x = (const __nv_bfloat16*)d_x; a.y = (__nv_bfloat16*)d_y;
  a.residual = (const __nv_bfloat16*)d_residual;
  a.rows = rows; a.n = w->n; a.k = w->k; a.nt = w->nt; a.kc = w->kc; a.epilogue = epilogue; a.swiglu_limit = swiglu_limit;
  cudaStream_t s = (cudaStream_t)stream;
  if (w->mode == B200_Q_AFFINE4_G64) return launch_tc_static<B200_Q_AFFINE4_G64>(a, rows, dev, s);
  if (w->mode == B200_Q_MXFP4_G32) return launch_tc_static<B200_Q_MXFP4_G32>(a, rows, dev, s);
  return launch_tc_static<B200_Q_BF16>(a, rows, dev, s);
}
