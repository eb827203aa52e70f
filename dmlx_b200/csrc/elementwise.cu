// Row-wise pieces of the layer stack: RMSNorm, RoPE, embedding gather, greedy argmax.
// All activations are bf16 with f32 arithmetic; every kernel is a single pass over its rows.
#include <cuda_bf16.h>

#include "common.h"

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One CTA per row; hidden % 8 == 0.
__global__ void rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                               __nv_bfloat16* __restrict__ out, int hidden, float eps) {
  __shared__ float s_part[32];
  const int row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * hidden);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* orow = reinterpret_cast<uint4*>(out + (size_t)row * hidden);
  const int nvec = hidden / 8;
  float ss = 0.f;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    uint4 v = xr[i];
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __bfloat1622float2(p[j]);
      ss += f.x * f.x + f.y * f.y;
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? s_part[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) s_part[0] = rsqrtf(t / (float)hidden + eps);
  }
  __syncthreads();
  const float r = s_part[0];
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    uint4 v = xr[i], g = wr[i], o;
    const __nv_bfloat162* pv = reinterpret_cast<const __nv_bfloat162*>(&v);
    const __nv_bfloat162* pg = reinterpret_cast<const __nv_bfloat162*>(&g);
    __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __bfloat1622float2(pv[j]), gg = __bfloat1622float2(pg[j]);
      po[j] = __floats2bfloat162_rn(f.x * r * gg.x, f.y * r * gg.y);
    }
    orow[i] = o;
  }
}

// Non-traditional RoPE: pair (i, i + D/2) of every head rotates by pos * theta^(-2i/D).
// One thread per (row, head, i); q heads first, then k heads.
__global__ void rope_kernel(__nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ k,
                            const int* __restrict__ positions, int rows, int hq, int hkv, int D, int q_stride,
                            int k_stride, float log2_theta) {
  const int half = D / 2;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)rows * (hq + hkv) * half;
  if (idx >= total) return;
  const int i = idx % half;
  const int head = (idx / half) % (hq + hkv);
  const int row = idx / ((long long)half * (hq + hkv));
  __nv_bfloat16* base = head < hq ? q + (size_t)row * q_stride + (size_t)head * D
                                  : k + (size_t)row * k_stride + (size_t)(head - hq) * D;
  const float inv_freq = exp2f(-log2_theta * (2.0f * i) / (float)D);
  float s, c;
  sincosf((float)positions[row] * inv_freq, &s, &c);
  const float x1 = __bfloat162float(base[i]), x2 = __bfloat162float(base[i + half]);
  base[i] = __float2bfloat16(x1 * c - x2 * s);
  base[i + half] = __float2bfloat16(x1 * s + x2 * c);
}

__global__ void embed_kernel(const __nv_bfloat16* __restrict__ table, const uint32_t* __restrict__ ids,
                             __nv_bfloat16* __restrict__ out, int hidden) {
  const int row = blockIdx.x;
  const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)ids[row] * hidden);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)row * hidden);
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) dst[i] = src[i];
}

// First strict maximum of each row (ties keep the smaller index).
__global__ void argmax_kernel(const __nv_bfloat16* __restrict__ logits, int vocab, uint32_t* __restrict__ out) {
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  const int row = blockIdx.x;
  const __nv_bfloat16* lr = logits + (size_t)row * vocab;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  // 16-byte loads where the row allows it (row start and length multiples of 8 elements); a thread
  // meets its elements in increasing index order, so a strict > keeps the first maximum it saw.
  const bool vec = (vocab % 8 == 0) && ((reinterpret_cast<uintptr_t>(lr) & 15) == 0);
  if (vec) {
    const uint4* lv = reinterpret_cast<const uint4*>(lr);
    for (int c = threadIdx.x; c < vocab / 8; c += blockDim.x) {
      const uint4 q = lv[c];
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float lo = __uint_as_float(w[j] << 16), hi = __uint_as_float(w[j] & 0xFFFF0000u);
        if (lo > best) { best = lo; bi = c * 8 + 2 * j; }
        if (hi > best) { best = hi; bi = c * 8 + 2 * j + 1; }
      }
    }
  } else {
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      float v = __bfloat162float(lr[i]);
      if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
  }
  auto better = [](float va, int ia, float vb, int ib) { return va > vb || (va == vb && ia < ib); };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { s_val[threadIdx.x >> 5] = best; s_idx[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int nw = blockDim.x >> 5;
    best = threadIdx.x < nw ? s_val[threadIdx.x] : -INFINITY;
    bi = threadIdx.x < nw ? s_idx[threadIdx.x] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, best, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
    }
    if (threadIdx.x == 0) out[row] = bi == 0x7fffffff ? 0u : (uint32_t)bi;
  }
}

__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ idx,
                                   __nv_bfloat16* __restrict__ dst, int hidden) {
  const int row = blockIdx.x;
  const int s = max(idx[row], 0);
  const uint4* sp = reinterpret_cast<const uint4*>(src + (size_t)s * hidden);
  uint4* dp = reinterpret_cast<uint4*>(dst + (size_t)row * hidden);
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) dp[i] = sp[i];
}

// `flags` (optional) points at the pool's state words: a step whose page reservation or attention was
// flagged has computed its tokens from stale pages, so the sequences keep the input token they had
// and the step can be run again once the cause (an exhausted pool) is gone.
__global__ void scatter_tokens_kernel(const uint32_t* __restrict__ next, const b200_pack_desc* __restrict__ desc,
                                      uint32_t* __restrict__ last_token, int n_req, const int* __restrict__ flags,
                                      int flag_a, int flag_b) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (flags && (flags[flag_a] != 0 || flags[flag_b] != 0)) return;
  if (i < n_req && desc[i].count > 0) last_token[desc[i].seq_slot] = next[i];
}

}  // namespace

// Rows idx[r] of src -> row r of dst (the last position of every request, src/generation.zig:124-131).
b200_status b200_gather_rows(const void* d_src, const int32_t* d_idx, void* d_dst, int32_t rows, int32_t hidden, void* stream) {
  if (rows <= 0) return B200_OK;
  gather_rows_kernel<<<rows, 128, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)d_src, d_idx, (__nv_bfloat16*)d_dst, hidden);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

// The sampled token of request i becomes the next decode input of its sequence slot.
b200_status b200_scatter_tokens(const uint32_t* d_next, const b200_pack_desc* d_desc, uint32_t* d_last_token, int32_t n_req,
                                const int* d_flags, int flag_a, int flag_b, void* stream) {
  if (n_req <= 0) return B200_OK;
  scatter_tokens_kernel<<<(n_req + 127) / 128, 128, 0, (cudaStream_t)stream>>>(d_next, d_desc, d_last_token, n_req, d_flags,
                                                                              flag_a, flag_b);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

extern "C" {

b200_status b200_rmsnorm(const void* d_x, const void* d_weight, void* d_out, int32_t rows, int32_t hidden, float eps,
                         void* stream) {
  b200_status st = b200_require_device();
  if (st != B200_OK) return st;
  if (hidden % 8 != 0) { b200_set_error("rmsnorm: hidden must be a multiple of 8"); return B200_ERR_INVALID_ARGUMENT; }
  if (rows <= 0) return B200_OK;
  rmsnorm_kernel<<<rows, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)d_x, (const __nv_bfloat16*)d_weight,
                                                        (__nv_bfloat16*)d_out, hidden, eps);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

b200_status b200_rope(void* d_q, void* d_k, const int32_t* d_positions, int32_t rows, int32_t n_q_heads,
                      int32_t n_kv_heads, int32_t head_dim, int32_t q_stride, int32_t k_stride, float theta,
                      void* stream) {
  b200_status st = b200_require_device();
  if (st != B200_OK) return st;
  if (rows <= 0) return B200_OK;
  long long total = (long long)rows * (n_q_heads + n_kv_heads) * (head_dim / 2);
  rope_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (__nv_bfloat16*)d_q, (__nv_bfloat16*)d_k, d_positions, rows, n_q_heads, n_kv_heads, head_dim, q_stride, k_stride,
      log2f(theta));
  B200_LAUNCH_CHECK();
  return B200_OK;
}

b200_status b200_embed_gather(const void* d_table, const uint32_t* d_ids, void* d_out, int32_t rows, int32_t hidden,
                              void* stream) {
  b200_status st = b200_require_device();
  if (st != B200_OK) return st;
  if (hidden % 8 != 0) { b200_set_error("embed: hidden must be a multiple of 8"); return B200_ERR_INVALID_ARGUMENT; }
  if (rows <= 0) return B200_OK;
  embed_kernel<<<rows, 128, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)d_table, d_ids, (__nv_bfloat16*)d_out, hidden);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

b200_status b200_argmax(const void* d_logits, int32_t rows, int32_t vocab, uint32_t* d_out, void* stream) {
  b200_status st = b200_require_device();
  if (st != B200_OK) return st;
  if (rows <= 0) return B200_OK;
  argmax_kernel<<<rows, 1024, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)d_logits, vocab, d_out);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

}  // extern "C"
