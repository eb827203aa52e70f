// Sampling beyond greedy on the device: temperature, top-k and top-p per row
// (src/sampling.zig:42-72, 175-242, 258-268, 298-322, 328-375), so that only one token id per
// request crosses PCIe for non-greedy requests too.  The uniform variate of each draw is an input.
//
// One CTA of 1024 threads per row.  The row is read from L2 several times (first maximum,
// log-sum-exp, the digit passes of a radix select, one gather pass); nothing of vocabulary size is
// kept on chip.  Ordering follows the reference's stable descending sort: a candidate is the
// 64-bit key (descending score bits << 32 | token id), so equal scores keep index order.  The
// candidates are taken from that order kChunk at a time: one pass over the row bounds the chunk
// (the kChunk-th smallest per-thread minimum), a second gathers the few keys under the bound, a
// bitonic network in shared memory sorts them; a radix select over the key backs this up for rows
// that defeat the bound.  The sums over the sorted prefix (softmax denominator, nucleus cut,
// renormalised draw) run on one thread in the reference's order in f32.
#include <cuda_bf16.h>

#include "common.h"

namespace {

constexpr int kThreads = 1024;
constexpr int kCap = 2048;    // keys held in shared memory
constexpr int kChunk = 512;   // candidates taken from the sorted order at a time

struct Shared {
  unsigned long long key[kCap];
  float e[kChunk];
  int hist[256];
  float red_f[32];
  int red_i[32];
  int sel_digit, sel_below, sel_count, sel_total, count;
  float acc, sum_exp, nucleus, carry;
  int cutoff, done, seg;
  unsigned token, last_idx;
};

template <typename T> struct Row {
  const T* p;
  int V;
  bool vec;  // 16-byte loads: the row starts on a 16-byte boundary and V % 8 == 0
};

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

// Eight consecutive elements starting at i0 (a multiple of 8); returns how many are inside the row.
__device__ __forceinline__ int load8(const Row<__nv_bfloat16>& r, int i0, float (&v)[8]) {
  const int n = min(max(r.V - i0, 0), 8);
  if (r.vec && n == 8) {
    const uint4 q = *reinterpret_cast<const uint4*>(r.p + i0);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[2 * j] = __uint_as_float(w[j] << 16);
      v[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = j < n ? __bfloat162float(r.p[i0 + j]) : 0.f;
  }
  return n;
}
__device__ __forceinline__ int load8(const Row<float>& r, int i0, float (&v)[8]) {
  const int n = min(max(r.V - i0, 0), 8);
  if (r.vec && n == 8) {
    const float4 a = *reinterpret_cast<const float4*>(r.p + i0), b = *reinterpret_cast<const float4*>(r.p + i0 + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = j < n ? r.p[i0 + j] : 0.f;
  }
  return n;
}

// (score descending, token id ascending) as one ascending 64-bit key; -0 is folded into +0 so that
// scores that compare equal share their bits.
__device__ __forceinline__ unsigned long long cand_key(float logit, float temperature, int idx) {
  float s = logit / temperature;
  s += 0.0f;
  unsigned u = __float_as_uint(s);
  u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  return ((unsigned long long)(~u) << 32) | (unsigned)idx;
}
__device__ __forceinline__ float key_score(unsigned long long c) {
  const unsigned u = ~(unsigned)(c >> 32);
  return __uint_as_float((u & 0x80000000u) ? (u ^ 0x80000000u) : ~u);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ float block_sum(float v, Shared& s) {
  __syncthreads();
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) s.red_f[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = warp_sum(s.red_f[threadIdx.x]);
    if (threadIdx.x == 0) s.red_f[0] = t;
  }
  __syncthreads();
  return s.red_f[0];
}

// First strict maximum of the row (src/sampling.zig:22-39): value through *out_max, index returned.
template <typename T> __device__ int block_first_max(const Row<T>& r, Shared& s, float* out_max) {
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int base = 0; base < r.V; base += kThreads * 8) {
    const int i0 = base + threadIdx.x * 8;
    float v[8];
    const int n = load8(r, i0, v);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (j < n && v[j] > best) { best = v[j]; bi = i0 + j; }
  }
  auto better = [](float va, int ia, float vb, int ib) { return va > vb || (va == vb && ia < ib); };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) { s.red_f[threadIdx.x >> 5] = best; s.red_i[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x < 32) {
    best = s.red_f[threadIdx.x];
    bi = s.red_i[threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
    }
    if (threadIdx.x == 0) { s.red_f[0] = best; s.red_i[0] = bi == 0x7fffffff ? 0 : bi; }
  }
  __syncthreads();
  *out_max = s.red_f[0];
  return s.red_i[0];
}

// Ascending bitonic sort of s.key[0, n2), n2 a power of two <= kCap.  All threads call.
__device__ void sort_keys(Shared& s, int n2) {
  for (int k = 2; k <= n2; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = threadIdx.x; i < n2; i += kThreads) {
        const int x = i ^ j;
        if (x > i) {
          const unsigned long long a = s.key[i], c = s.key[x];
          if ((a > c) == ((i & k) == 0)) { s.key[i] = c; s.key[x] = a; }
        }
      }
      __syncthreads();
    }
  }
}

// Largest key of the m smallest keys >= lo_bound (most-significant-digit radix select over the whole
// row); *out_count = how many keys lie in [lo_bound, result] (m, or fewer when the row runs out).
// This is the general path: every element takes part in the first digit passes.
template <typename T>
__device__ unsigned long long radix_threshold(const Row<T>& r, float temperature, unsigned long long lo_bound, int m,
                                              Shared& s, int* out_count) {
  const int tid = threadIdx.x, lane = tid & 31;
  unsigned long long prefix = 0, mask = 0, thr = 0;
  int need = m, taken = 0;
  bool closed = false;
  for (int b = 7; b >= 0 && !closed; --b) {
    // digits of the token id that are zero for every element of the row
    if (b == 3 || (b == 2 && r.V <= (1 << 16)) || (b == 1 && r.V <= (1 << 8))) continue;
    const int shift = 8 * b;
    __syncthreads();
    if (tid < 256) s.hist[tid] = 0;
    __syncthreads();
    for (int base = 0; base < r.V; base += kThreads * 8) {
      const int i0 = base + tid * 8;
      float v[8];
      const int n = load8(r, i0, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        unsigned long long c = 0;
        bool valid = j < n;
        if (valid) {
          c = cand_key(v[j], temperature, i0 + j);
          valid = c >= lo_bound && (c & mask) == prefix;
        }
        if (__any_sync(0xffffffffu, valid)) {
          const unsigned digit = (unsigned)(c >> shift) & 255u;
          // one shared-memory atomic per distinct digit of the warp: the leading digits of a row's
          // scores fall into a handful of bins
          const unsigned peers = __match_any_sync(0xffffffffu, valid ? digit : 256u + lane);
          if (valid && lane == __ffs(peers) - 1) atomicAdd(&s.hist[digit], __popc(peers));
        }
      }
    }
    __syncthreads();
    if (tid < 32) {
      int loc[8], sum = 0;
#pragma unroll
      for (int q = 0; q < 8; ++q) { loc[q] = s.hist[lane * 8 + q]; sum += loc[q]; }
      int incl = sum;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
      }
      const int total = __shfl_sync(0xffffffffu, incl, 31);
      const int want = min(need, total), excl = incl - sum;
      if (total > 0 && excl < want && want <= incl) {
        int run = excl;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          if (run + loc[q] >= want) { s.sel_digit = lane * 8 + q; s.sel_below = run; s.sel_count = loc[q]; break; }
          run += loc[q];
        }
      }
      if (lane == 0) s.sel_total = total;
    }
    __syncthreads();
    if (s.sel_total == 0) { *out_count = 0; return 0; }
    need = min(need, s.sel_total) - s.sel_below;
    taken += s.sel_below;
    prefix |= (unsigned long long)s.sel_digit << shift;
    mask |= 255ull << shift;
    if (s.sel_count == need) {  // the whole bin is taken: no need to look at lower digits
      thr = prefix | (shift ? ((1ull << shift) - 1) : 0ull);
      closed = true;
    }
  }
  if (!closed) thr = prefix;
  *out_count = taken + need;
  return thr;
}

// Appends every key in [lo_bound, hi_bound] to s.key (unordered); returns how many there are, which
// may exceed kCap (only the first kCap are stored).
template <typename T>
__device__ int gather_keys(const Row<T>& r, float temperature, unsigned long long lo_bound, unsigned long long hi_bound,
                           Shared& s) {
  __syncthreads();
  if (threadIdx.x == 0) s.count = 0;
  __syncthreads();
  for (int base = 0; base < r.V; base += kThreads * 8) {
    const int i0 = base + threadIdx.x * 8;
    float v[8];
    const int n = load8(r, i0, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (j < n) {
        const unsigned long long c = cand_key(v[j], temperature, i0 + j);
        if (c >= lo_bound && c <= hi_bound) {
          const int pos = atomicAdd(&s.count, 1);
          if (pos < kCap) s.key[pos] = c;
        }
      }
    }
  }
  __syncthreads();
  return s.count;
}

// The m (<= kChunk) smallest keys >= lo_bound, sorted ascending into s.key[0, m); returns how many
// there were.  Fast path: the m-th smallest of the 1024 per-thread minima bounds the m-th smallest of
// the row from above, and for m <= kChunk only a few more than m keys lie under that bound, so one
// pass finds the bound and a second gathers the candidates.  Rows that defeat the bound (a run of
// equal scores longer than the buffer, or fewer eligible keys than threads) take the radix select.
template <typename T>
__device__ int next_chunk(const Row<T>& r, float temperature, unsigned long long lo_bound, int m, Shared& s) {
  const int tid = threadIdx.x;
  unsigned long long best = ~0ull;
  for (int base = 0; base < r.V; base += kThreads * 8) {
    const int i0 = base + tid * 8;
    float v[8];
    const int n = load8(r, i0, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (j < n) {
        const unsigned long long c = cand_key(v[j], temperature, i0 + j);
        if (c >= lo_bound && c < best) best = c;
      }
    }
  }
  __syncthreads();
  s.key[tid] = best;
  __syncthreads();
  sort_keys(s, kThreads);
  const unsigned long long tau = s.key[m - 1];  // ~0 when fewer than m threads saw an eligible key
  int count = gather_keys(r, temperature, lo_bound, tau, s);
  if (count > kCap) {
    int exact = 0;
    const unsigned long long thr = radix_threshold(r, temperature, lo_bound, m, s, &exact);
    count = exact > 0 ? gather_keys(r, temperature, lo_bound, thr, s) : 0;
  }
  if (count == 0) return 0;
  int n2 = 2;
  while (n2 < count) n2 <<= 1;
  for (int i = count + tid; i < n2; i += kThreads) s.key[i] = ~0ull;
  __syncthreads();
  sort_keys(s, n2);
  return min(count, m);
}

// temperatureSample (src/sampling.zig:42-72): softmax of (logit - max) / T in index order, first
// index whose cumulative probability exceeds u.  Each warp owns a contiguous segment of the row.
template <typename T>
__device__ unsigned sample_full_softmax(const Row<T>& r, float temperature, float gmax, float u, Shared& s) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float part = 0.f;
  for (int base = 0; base < r.V; base += kThreads * 8) {
    float v[8];
    const int n = load8(r, base + tid * 8, v);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (j < n) part += expf((v[j] - gmax) / temperature);
  }
  const float sum = block_sum(part, s);
  const int seg = ((r.V + 31) / 32 + 31) / 32 * 32;
  const int lo = min(warp * seg, r.V), hi = min(lo + seg, r.V);
  float ls = 0.f;
  for (int i = lo + lane; i < hi; i += 32) ls += expf((to_f32(r.p[i]) - gmax) / temperature) / sum;
  ls = warp_sum(ls);
  __syncthreads();
  if (lane == 0) s.red_f[warp] = ls;
  __syncthreads();
  if (tid == 0) {
    float cum = 0.f;
    s.seg = -1;
    for (int w = 0; w < 32; ++w) {
      const float c2 = cum + s.red_f[w];
      if (u < c2) { s.seg = w; s.carry = cum; break; }
      cum = c2;
    }
    s.token = (unsigned)(r.V - 1);  // sampleFromProbs returns n - 1 when u is never exceeded (:267)
  }
  __syncthreads();
  if (s.seg == warp) {
    float carry = s.carry;
    unsigned tok = (unsigned)(hi - 1);
    for (int base = lo; base < hi; base += 32) {
      const int i = base + lane;
      const float p = i < hi ? expf((to_f32(r.p[i]) - gmax) / temperature) / sum : 0.f;
      float incl = p;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
      }
      const unsigned hit = __ballot_sync(0xffffffffu, i < hi && u < carry + incl);
      if (hit) { tok = (unsigned)(base + __ffs(hit) - 1); break; }
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) s.token = tok;
  }
  __syncthreads();
  return s.token;
}

// Sum of exp(score - max_score) over every key <= hi_bound, as a parallel reduction.
template <typename T>
__device__ float sum_exp_below(const Row<T>& r, float temperature, unsigned long long hi_bound, float max_score, Shared& s) {
  float part = 0.f;
  for (int base = 0; base < r.V; base += kThreads * 8) {
    const int i0 = base + threadIdx.x * 8;
    float v[8];
    const int n = load8(r, i0, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (j < n) {
        const unsigned long long c = cand_key(v[j], temperature, i0 + j);
        if (c <= hi_bound) part += expf(key_score(c) - max_score);
      }
    }
  }
  return block_sum(part, s);
}

// topKTopPSampler (src/sampling.zig:175-242).  The sorted order is walked kChunk candidates at a time.
// Up to kChunk candidates (the usual top-k) everything, the softmax denominator included, is summed on
// one thread in sorted order like the reference; above that the denominator is a parallel reduction
// and only the nucleus cut and the draw walk the order, normally inside the first chunk.
template <typename T>
__device__ unsigned sample_top_k_top_p(const Row<T>& r, float temperature, int k_eff, float top_p, float u, float gmax,
                                       Shared& s) {
  const int tid = threadIdx.x;
  const bool single = k_eff <= kChunk;
  bool have_chunk = false;
  int chunk_cnt = 0;
  // the largest score is the largest logit's: division by a positive temperature keeps the order
  const float max_score = gmax / temperature + 0.0f;
  if (!single) {
    unsigned long long hi = ~0ull;
    if (k_eff < r.V) {
      int exact = 0;
      hi = radix_threshold(r, temperature, 0ull, k_eff, s, &exact);
    }
    const float total = sum_exp_below(r, temperature, hi, max_score, s);
    if (tid == 0) s.sum_exp = total;
    __syncthreads();
  }
  for (int pass = single ? 0 : 1; pass < 3; ++pass) {
    // pass 0: softmax denominator over the top k; 1: nucleus cut; 2: the draw inside the nucleus
    unsigned long long lo = 0;
    int taken = 0;
    const int limit = pass == 2 ? s.cutoff : k_eff;
    __syncthreads();
    if (tid == 0) { s.acc = 0.f; s.done = 0; }
    __syncthreads();
    while (taken < limit) {
      int cnt;
      if (single && have_chunk) {
        cnt = chunk_cnt;
      } else {
        cnt = next_chunk(r, temperature, lo, min(kChunk, k_eff - taken), s);
        if (cnt == 0) break;
        for (int i = tid; i < cnt; i += kThreads) s.e[i] = expf(key_score(s.key[i]) - max_score);
        __syncthreads();
        have_chunk = true;
        chunk_cnt = cnt;
      }
      const int use = min(cnt, limit - taken);
      if (tid == 0) {
        float acc = s.acc;
        if (pass == 0) {
          for (int i = 0; i < use; ++i) acc += s.e[i];
        } else if (pass == 1) {
          for (int i = 0; i < use; ++i) {
            acc += s.e[i] / s.sum_exp;
            if (acc > top_p) { s.cutoff = taken + i + 1; s.done = 1; break; }
          }
        } else {
          for (int i = 0; i < use; ++i) {
            acc += (s.e[i] / s.sum_exp) / s.nucleus;
            s.last_idx = (unsigned)s.key[i];
            if (u < acc) { s.token = s.last_idx; s.done = 1; break; }
          }
        }
        s.acc = acc;
      }
      __syncthreads();
      lo = s.key[cnt - 1] + 1;
      taken += cnt;
      const int done = s.done;
      __syncthreads();  // everyone has read the flag and the last key before either is rewritten
      if (done) break;
    }
    __syncthreads();
    if (tid == 0) {
      if (pass == 0) s.sum_exp = s.acc;
      if (pass == 1) { s.nucleus = s.acc; if (!s.done) s.cutoff = min(taken, k_eff); }
      if (pass == 2 && !s.done) s.token = s.last_idx;
    }
    __syncthreads();
  }
  return s.token;
}

template <typename T>
__device__ void sample_row(const Row<T>& r, const b200_sample_params& p, Shared& s, uint32_t* out_token, float* out_logprob) {
  float gmax;
  const int garg = block_first_max(r, s, &gmax);
  unsigned token;
  if (!(p.temperature > 0.0f)) {
    token = (unsigned)garg;
  } else if (p.top_p >= 1.0f && (p.top_k <= 0 || p.top_k >= r.V)) {
    token = sample_full_softmax(r, p.temperature, gmax, p.uniform, s);
  } else {
    const int k_eff = (p.top_k <= 0 || p.top_k > r.V) ? r.V : p.top_k;
    token = sample_top_k_top_p(r, p.temperature, k_eff, p.top_p, p.uniform, gmax, s);
  }
  if (out_logprob != nullptr) {
    float part = 0.f;
    for (int base = 0; base < r.V; base += kThreads * 8) {
      float v[8];
      const int n = load8(r, base + threadIdx.x * 8, v);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j < n) part += expf(v[j] - gmax);
    }
    const float sum = block_sum(part, s);
    if (threadIdx.x == 0) *out_logprob = token < (unsigned)r.V ? to_f32(r.p[token]) - (gmax + logf(sum)) : -INFINITY;
  }
  if (threadIdx.x == 0) *out_token = token;
}

template <typename T>
__global__ void __launch_bounds__(kThreads) sample_rows_kernel(const T* __restrict__ logits, int V,
                                                               const b200_sample_params* __restrict__ params,
                                                               const uint32_t* __restrict__ ctx, const int* __restrict__ ctx_off,
                                                               float* __restrict__ scratch, uint32_t* __restrict__ tokens,
                                                               float* __restrict__ logprobs) {
  __shared__ Shared s;
  const int row = blockIdx.x;
  const b200_sample_params p = params[row];
  const T* x = logits + (size_t)row * V;
  float* lp = logprobs ? logprobs + row : nullptr;
  const int ctx_lo = ctx_off ? ctx_off[row] : 0, ctx_n = ctx_off ? ctx_off[row + 1] - ctx_lo : 0;
  if (p.repetition_penalty > 1.0f && ctx_n > 0 && scratch != nullptr) {
    // applyRepetitionPenalty (src/sampling.zig:328-354): every occurrence of a token divides a positive
    // logit by the penalty or multiplies a non-positive one; occurrences commute, so they may race.
    float* y = scratch + (size_t)row * V;
    for (int i = threadIdx.x; i < V; i += kThreads) y[i] = to_f32(x[i]);
    __syncthreads();
    for (int c = threadIdx.x; c < ctx_n; c += kThreads) {
      const uint32_t tok = ctx[ctx_lo + c];
      if (tok < (uint32_t)V) {
        unsigned* a = reinterpret_cast<unsigned*>(y + tok);
        unsigned old = *a, assumed;
        do {
          assumed = old;
          const float f = __uint_as_float(assumed);
          old = atomicCAS(a, assumed, __float_as_uint(f > 0.f ? f / p.repetition_penalty : f * p.repetition_penalty));
        } while (old != assumed);
      }
    }
    __syncthreads();
    const Row<float> r{y, V, V % 8 == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0};
    sample_row(r, p, s, tokens + row, lp);
  } else {
    const Row<T> r{x, V, V % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0};
    sample_row(r, p, s, tokens + row, lp);
  }
}

}  // namespace

extern "C" {

b200_status b200_sample_rows(const void* d_logits, int32_t logits_f32, int32_t rows, int32_t vocab,
                             const b200_sample_params* d_params, const uint32_t* d_ctx_tokens, const int32_t* d_ctx_offsets,
                             float* d_scratch, uint32_t* d_tokens, float* d_logprobs, void* stream) {
  b200_status st = b200_require_device();
  if (st != B200_OK) return st;
  if (rows <= 0) return B200_OK;
  if (vocab < 1 || vocab > (1 << 24) || d_logits == nullptr || d_params == nullptr || d_tokens == nullptr) {
    b200_set_error("sample_rows: vocab %d outside 1..2^24 or a null argument", vocab);
    return B200_ERR_INVALID_ARGUMENT;
  }
  if ((d_ctx_offsets != nullptr) != (d_ctx_tokens != nullptr) || (d_ctx_offsets != nullptr && d_scratch == nullptr)) {
    b200_set_error("sample_rows: context tokens, their offsets and the f32 scratch go together");
    return B200_ERR_INVALID_ARGUMENT;
  }
  cudaStream_t cs = (cudaStream_t)stream;
  if (logits_f32)
    sample_rows_kernel<float><<<rows, kThreads, 0, cs>>>((const float*)d_logits, vocab, d_params, d_ctx_tokens, d_ctx_offsets,
                                                         d_scratch, d_tokens, d_logprobs);
  else
    sample_rows_kernel<__nv_bfloat16><<<rows, kThreads, 0, cs>>>((const __nv_bfloat16*)d_logits, vocab, d_params, d_ctx_tokens,
                                                                 d_ctx_offsets, d_scratch, d_tokens, d_logprobs);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

}  // extern "C"
