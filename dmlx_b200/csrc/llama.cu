// LLaMA-architecture layer stack driven over a packed ragged batch: one call runs
// pack -> page reservation -> embed -> N x (RMSNorm, fused QKV matmul, RoPE, paged KV append,
// paged attention, output matmul + residual, RMSNorm, gate/up matmul + SwiGLU, down matmul +
// residual) -> last-row gather -> RMSNorm -> lm_head -> greedy argmax, all on one stream.
// Follows LlamaModel.forward / LlamaTransformerBlock.forward / LlamaAttention.forward /
// LlamaMLP.forward (src/models/llama.zig:556-609, 460-481, 138-299, 372-438) and the greedy branch
// of generateBatchStep (src/generation.zig:104-145); per-row positions replace the reference's
// scalar RoPE offset, and attention reads the page pool in place instead of a gathered copy.
#include <cuda_bf16.h>

#include <cstring>
#include <map>
#include <tuple>
#include <vector>

#include "common.h"
#include "kv_pool.cuh"
#include "qmm.cuh"

b200_status b200_gather_rows(const void* d_src, const int32_t* d_idx, void* d_dst, int32_t rows, int32_t hidden, void* stream);
b200_status b200_scatter_tokens(const uint32_t* d_next, const b200_pack_desc* d_desc, uint32_t* d_last_token, int32_t n_req,
                                const int* d_flags, int flag_a, int flag_b, void* stream);

namespace {
struct HostMat {
  int mode = -1, n = 0, k = 0;
  std::vector<unsigned char> packed, scales, biases;
};
size_t packed_row_bytes(int mode, int k) { return mode == B200_Q_AFFINE4_G64 ? (size_t)k / 2 : (mode == B200_Q_MXFP4_G32 ? (size_t)k / 2 : (size_t)k * 2); }
size_t scale_row_bytes(int mode, int k) { return mode == B200_Q_AFFINE4_G64 ? (size_t)k / 64 * 2 : (mode == B200_Q_MXFP4_G32 ? (size_t)k / 32 : 0); }
}  // namespace

struct b200_llama {
  b200_llama_config cfg{};
  std::map<std::pair<int, int>, HostMat> staged;
  bool finalized = false;
  __nv_bfloat16* embed = nullptr;
  std::vector<__nv_bfloat16*> attn_norm, ffn_norm;
  __nv_bfloat16* final_norm = nullptr;
  std::vector<b200_qweight*> wqkv, wo, wgu, wdown;
  b200_qweight* lm_head = nullptr;
  // activations
  __nv_bfloat16 *x = nullptr, *h = nullptr, *qkv = nullptr, *attn = nullptr, *act = nullptr, *last_h = nullptr,
                *last_hn = nullptr, *logits = nullptr;
  // packed batch
  b200_pack_desc* d_desc = nullptr;
  uint32_t *d_prefill = nullptr, *d_tokens = nullptr, *d_next = nullptr, *d_last_token = nullptr;
  int32_t *d_cu = nullptr, *d_pos = nullptr, *d_row_to_req = nullptr, *d_row_seq = nullptr, *d_row_ctx = nullptr,
          *d_last_row = nullptr;
  // pinned staging
  b200_pack_desc* h_desc = nullptr;
  uint32_t *h_prefill = nullptr, *h_next = nullptr;
  int32_t* h_state = nullptr;  // [8] pool state words + [2] matmul error words
  // per-request sampler rows of the coming step (set by b200_llama_set_samplers, used once)
  b200_sample_params *d_samp = nullptr, *h_samp = nullptr;
  float* d_logprobs = nullptr;
  int samp_n = 0;
  bool sampling = false;  // the step in flight samples with d_samp instead of taking the argmax
  int last_n_req = 0;
  long long launches = 0;  // kernels launched by forward calls so far
  // CUDA graphs of decode-only steps, keyed by (requests, device descriptor pointer, stream): the
  // first step of a shape runs eagerly (it may grow scratch buffers), the second is captured,
  // later ones replay the graph.
  bool graphs_on = true;
  bool fuse_qkv_rope = true;  // b200_llama_set_fused_qkv_rope
  struct GraphEntry { int seen = 0; cudaGraphExec_t exec = nullptr; long long kernels = 0; };
  std::map<std::tuple<int, const void*, const void*, void*, bool>, GraphEntry> graphs;
  // optional CUDA-event timing per category: 0 attention, 1 matmuls, 2 rope + KV append, 3 the rest
  bool prof_on = false;
  std::vector<cudaEvent_t> prof_events;  // pairs
  std::vector<int> prof_cat;
  size_t prof_used = 0;
  cudaEvent_t prof_begin(int cat, cudaStream_t s) {
    if (!prof_on) return nullptr;
    if (prof_used + 2 > prof_events.size()) {
      cudaEvent_t a, b;
      cudaEventCreate(&a);
      cudaEventCreate(&b);
      prof_events.push_back(a);
      prof_events.push_back(b);
      prof_cat.push_back(cat);
    }
    prof_cat[prof_used / 2] = cat;
    cudaEventRecord(prof_events[prof_used], s);
    prof_used += 2;
    return prof_events[prof_used - 1];
  }
  void prof_end(cudaEvent_t e, cudaStream_t s) { if (e) cudaEventRecord(e, s); }
};


#define L_ALLOC(ptr, bytes)                                                                            \
  do {                                                                                                 \
    cudaError_t e_ = cudaMalloc((void**)&(ptr), (bytes));                                              \
    if (e_ != cudaSuccess) {                                                                           \
      b200_set_error("cudaMalloc(%zu) failed: %s", (size_t)(bytes), cudaGetErrorString(e_));           \
      b200_llama_destroy(m);                                                                           \
      return B200_ERR_CUDA;                                                                            \
    }                                                                                                  \
  } while (0)

extern "C" {

b200_status b200_llama_create(const b200_llama_config* c, b200_llama** out) {
  *out = nullptr;
  b200_status st = b200_require_device();
  if (st != B200_OK) return st;
  if (c->n_layers <= 0 || c->hidden % 64 != 0 || c->ffn % 64 != 0 || (c->n_heads * c->head_dim) % 64 != 0 ||
      c->n_heads % c->n_kv_heads != 0 || c->max_rows <= 0 || c->max_reqs <= 0 || c->vocab <= 0) {
    b200_set_error("llama: invalid configuration (hidden, ffn and heads*head_dim must be multiples of 64)");
    return B200_ERR_INVALID_ARGUMENT;
  }
  auto* m = new b200_llama();
  m->cfg = *c;
  const int L = c->n_layers, R = c->max_rows, Q = c->max_reqs;
  const size_t qkv_dim = (size_t)(c->n_heads + 2 * c->n_kv_heads) * c->head_dim;
  m->attn_norm.assign(L, nullptr); m->ffn_norm.assign(L, nullptr);
  m->wqkv.assign(L, nullptr); m->wo.assign(L, nullptr); m->wgu.assign(L, nullptr); m->wdown.assign(L, nullptr);
  L_ALLOC(m->embed, (size_t)c->vocab * c->hidden * 2);
  for (int l = 0; l < L; ++l) { L_ALLOC(m->attn_norm[l], (size_t)c->hidden * 2); L_ALLOC(m->ffn_norm[l], (size_t)c->hidden * 2); }
  L_ALLOC(m->final_norm, (size_t)c->hidden * 2);
  L_ALLOC(m->x, (size_t)R * c->hidden * 2);
  L_ALLOC(m->h, (size_t)R * c->hidden * 2);
  L_ALLOC(m->qkv, (size_t)R * qkv_dim * 2);
  L_ALLOC(m->attn, (size_t)R * c->n_heads * c->head_dim * 2);
  L_ALLOC(m->act, (size_t)R * c->ffn * 2);
  L_ALLOC(m->last_h, (size_t)Q * c->hidden * 2);
  L_ALLOC(m->last_hn, (size_t)Q * c->hidden * 2);
  L_ALLOC(m->logits, (size_t)Q * c->vocab * 2);
  L_ALLOC(m->d_desc, sizeof(b200_pack_desc) * Q);
  L_ALLOC(m->d_prefill, sizeof(uint32_t) * R);
  L_ALLOC(m->d_tokens, sizeof(uint32_t) * R);
  L_ALLOC(m->d_next, sizeof(uint32_t) * Q);
  L_ALLOC(m->d_last_token, sizeof(uint32_t) * c->max_seqs);
  L_ALLOC(m->d_cu, sizeof(int32_t) * (Q + 1));
  L_ALLOC(m->d_pos, sizeof(int32_t) * R);
  L_ALLOC(m->d_row_to_req, sizeof(int32_t) * R);
  L_ALLOC(m->d_row_seq, sizeof(int32_t) * R);
  L_ALLOC(m->d_row_ctx, sizeof(int32_t) * R);
  L_ALLOC(m->d_last_row, sizeof(int32_t) * Q);
  L_ALLOC(m->d_samp, sizeof(b200_sample_params) * Q);
  L_ALLOC(m->d_logprobs, sizeof(float) * Q);
  cudaMemset(m->d_last_token, 0, sizeof(uint32_t) * c->max_seqs);
  if (cudaMallocHost((void**)&m->h_desc, sizeof(b200_pack_desc) * Q) != cudaSuccess ||
      cudaMallocHost((void**)&m->h_prefill, sizeof(uint32_t) * R) != cudaSuccess ||
      cudaMallocHost((void**)&m->h_next, sizeof(uint32_t) * Q) != cudaSuccess ||
      cudaMallocHost((void**)&m->h_samp, sizeof(b200_sample_params) * Q) != cudaSuccess ||
      cudaMallocHost((void**)&m->h_state, sizeof(int32_t) * 16) != cudaSuccess) {
    b200_set_error("pinned host allocation failed");
    b200_llama_destroy(m);
    return B200_ERR_CUDA;
  }
  *out = m;
  return B200_OK;
}

void b200_llama_destroy(b200_llama* m) {
  if (!m) return;
  void* dev[] = {m->embed, m->final_norm, m->x, m->h, m->qkv, m->attn, m->act, m->last_h, m->last_hn, m->logits, m->d_desc,
                 m->d_prefill, m->d_tokens, m->d_next, m->d_last_token, m->d_cu, m->d_pos, m->d_row_to_req, m->d_row_seq,
                 m->d_row_ctx, m->d_last_row, m->d_samp, m->d_logprobs};
  for (void* p : dev) if (p) cudaFree(p);
  for (auto* p : m->attn_norm) if (p) cudaFree(p);
  for (auto* p : m->ffn_norm) if (p) cudaFree(p);
  for (auto* w : m->wqkv) b200_qweight_destroy(w);
  for (auto* w : m->wo) b200_qweight_destroy(w);
  for (auto* w : m->wgu) b200_qweight_destroy(w);
  for (auto* w : m->wdown) b200_qweight_destroy(w);
  b200_qweight_destroy(m->lm_head);
  if (m->h_desc) cudaFreeHost(m->h_desc);
  if (m->h_prefill) cudaFreeHost(m->h_prefill);
  if (m->h_next) cudaFreeHost(m->h_next);
  if (m->h_samp) cudaFreeHost(m->h_samp);
  if (m->h_state) cudaFreeHost(m->h_state);
  for (cudaEvent_t e : m->prof_events) cudaEventDestroy(e);
  for (auto& g : m->graphs) if (g.second.exec) cudaGraphExecDestroy(g.second.exec);
  delete m;
}

static bool linear_dims(const b200_llama_config& c, int which, int* n, int* k) {
  const int qd = c.n_heads * c.head_dim, kd = c.n_kv_heads * c.head_dim;
  switch (which) {
    case B200_W_Q: *n = qd; *k = c.hidden; return true;
    case B200_W_K: case B200_W_V: *n = kd; *k = c.hidden; return true;
    case B200_W_O: *n = c.hidden; *k = qd; return true;
    case B200_W_GATE: case B200_W_UP: *n = c.ffn; *k = c.hidden; return true;
    case B200_W_DOWN: *n = c.hidden; *k = c.ffn; return true;
    case B200_W_LM_HEAD: *n = c.vocab; *k = c.hidden; return true;
    default: return false;
  }
}

b200_status b200_llama_set_linear(b200_llama* m, int32_t layer, int32_t which, int32_t mode, const void* h_packed,
                                  const void* h_scales, const void* h_biases) {
  int n = 0, k = 0;
  if (!linear_dims(m->cfg, which, &n, &k) || (which != B200_W_LM_HEAD && (layer < 0 || layer >= m->cfg.n_layers))) {
    b200_set_error("set_linear: bad layer/which (%d/%d)", layer, which);
    return B200_ERR_INVALID_ARGUMENT;
  }
  if (mode < 0 || mode > B200_Q_BF16) { b200_set_error("set_linear: unknown mode %d", mode); return B200_ERR_INVALID_QUANT_BITS; }
  HostMat hm;
  hm.mode = mode; hm.n = n; hm.k = k;
  const size_t pb = packed_row_bytes(mode, k) * n, sb = scale_row_bytes(mode, k) * n;
  hm.packed.assign((const unsigned char*)h_packed, (const unsigned char*)h_packed + pb);
  if (sb) hm.scales.assign((const unsigned char*)h_scales, (const unsigned char*)h_scales + sb);
  if (mode == B200_Q_AFFINE4_G64) hm.biases.assign((const unsigned char*)h_biases, (const unsigned char*)h_biases + sb);
  m->staged[{which == B200_W_LM_HEAD ? -1 : layer, which}] = std::move(hm);
  return B200_OK;
}

b200_status b200_llama_set_embedding(b200_llama* m, const void* h_bf16) {
  B200_CUDA_TRY(cudaMemcpy(m->embed, h_bf16, (size_t)m->cfg.vocab * m->cfg.hidden * 2, cudaMemcpyHostToDevice));
  return B200_OK;
}

b200_status b200_llama_set_norm(b200_llama* m, int32_t layer, int32_t which, const void* h_bf16) {
  __nv_bfloat16* dst = layer < 0 ? m->final_norm : (which == 0 ? m->attn_norm[layer] : m->ffn_norm[layer]);
  if (layer >= m->cfg.n_layers) { b200_set_error("set_norm: layer out of range"); return B200_ERR_INVALID_ARGUMENT; }
  B200_CUDA_TRY(cudaMemcpy(dst, h_bf16, (size_t)m->cfg.hidden * 2, cudaMemcpyHostToDevice));
  return B200_OK;
}

// Row-wise concatenation (and optional interleave) of staged matrices into one weight.
static b200_status fuse(b200_llama* m, int layer, const std::vector<int>& which, bool interleave, b200_qweight** out) {
  std::vector<const HostMat*> parts;
  for (int w : which) {
    auto it = m->staged.find({layer, w});
    if (it == m->staged.end()) { b200_set_error("finalize: weight %d of layer %d was never set", w, layer); return B200_ERR_INVALID_ARGUMENT; }
    parts.push_back(&it->second);
  }
  const int mode = parts[0]->mode, k = parts[0]->k;
  int n = 0;
  for (auto* p : parts) {
    if (p->mode != mode || p->k != k) { b200_set_error("finalize: fused weights must share mode and K"); return B200_ERR_INVALID_ARGUMENT; }
    n += p->n;
  }
  const size_t prb = packed_row_bytes(mode, k), srb = scale_row_bytes(mode, k);
  std::vector<unsigned char> packed(prb * n), scales(srb * n), biases(mode == B200_Q_AFFINE4_G64 ? srb * n : 0);
  int row = 0;
  auto put = [&](const HostMat* p, int r) {
    std::memcpy(&packed[prb * row], &p->packed[prb * r], prb);
    if (srb) std::memcpy(&scales[srb * row], &p->scales[srb * r], srb);
    if (!biases.empty()) std::memcpy(&biases[srb * row], &p->biases[srb * r], srb);
    ++row;
  };
  if (interleave) {
    for (int r = 0; r < parts[0]->n; ++r) for (auto* p : parts) put(p, r);
  } else {
    for (auto* p : parts) for (int r = 0; r < p->n; ++r) put(p, r);
  }
  b200_status st = b200_qweight_create(mode, 1, n, k, packed.data(), scales.empty() ? nullptr : scales.data(),
                                       biases.empty() ? nullptr : biases.data(), out);
  if (st == B200_OK) for (int w : which) m->staged.erase({layer, w});
  return st;
}

b200_status b200_llama_finalize(b200_llama* m) {
  for (int l = 0; l < m->cfg.n_layers; ++l) {
    b200_status st;
    if ((st = fuse(m, l, {B200_W_Q, B200_W_K, B200_W_V}, false, &m->wqkv[l])) != B200_OK) return st;
    if ((st = fuse(m, l, {B200_W_O}, false, &m->wo[l])) != B200_OK) return st;
    if ((st = fuse(m, l, {B200_W_GATE, B200_W_UP}, true, &m->wgu[l])) != B200_OK) return st;
    if ((st = fuse(m, l, {B200_W_DOWN}, false, &m->wdown[l])) != B200_OK) return st;
  }
  b200_status st = fuse(m, -1, {B200_W_LM_HEAD}, false, &m->lm_head);
  if (st != B200_OK) return st;
  m->finalized = true;
  return B200_OK;
}

// Synthetic model for benchmarks: every matrix generated on the device, norm weights 1,
// embedding small random values.
b200_status b200_llama_random_init(b200_llama* m, int32_t mode, uint32_t seed) {
  const b200_llama_config& c = m->cfg;
  const int qkv_n = (c.n_heads + 2 * c.n_kv_heads) * c.head_dim;
  if (qkv_n % 128 || c.hidden % 128 || c.ffn % 64 || c.vocab % 128) {
    b200_set_error("random_init: projection sizes must be multiples of 128");
    return B200_ERR_INVALID_ARGUMENT;
  }
  b200_status st;
  for (int l = 0; l < c.n_layers; ++l) {
    if ((st = b200_qweight_random(mode, 1, qkv_n, c.hidden, seed + 16 * l + 1, &m->wqkv[l])) != B200_OK) return st;
    if ((st = b200_qweight_random(mode, 1, c.hidden, c.n_heads * c.head_dim, seed + 16 * l + 2, &m->wo[l])) != B200_OK) return st;
    if ((st = b200_qweight_random(mode, 1, 2 * c.ffn, c.hidden, seed + 16 * l + 3, &m->wgu[l])) != B200_OK) return st;
    if ((st = b200_qweight_random(mode, 1, c.hidden, c.ffn, seed + 16 * l + 4, &m->wdown[l])) != B200_OK) return st;
  }
  if ((st = b200_qweight_random(mode, 1, c.vocab, c.hidden, seed + 7, &m->lm_head)) != B200_OK) return st;
  std::vector<uint16_t> ones(c.hidden, 0x3F80);
  for (int l = 0; l < c.n_layers; ++l) {
    B200_CUDA_TRY(cudaMemcpy(m->attn_norm[l], ones.data(), c.hidden * 2, cudaMemcpyHostToDevice));
    B200_CUDA_TRY(cudaMemcpy(m->ffn_norm[l], ones.data(), c.hidden * 2, cudaMemcpyHostToDevice));
  }
  B200_CUDA_TRY(cudaMemcpy(m->final_norm, ones.data(), c.hidden * 2, cudaMemcpyHostToDevice));
  b200_qweight* tmp = nullptr;  // reuse the dense random generator for the embedding table
  std::vector<uint16_t> emb((size_t)c.vocab * c.hidden);
  uint32_t s = seed * 2654435761u + 12345u;
  for (auto& e : emb) { s = s * 1664525u + 1013904223u; e = (uint16_t)(((s >> 16) & 0x807F) | 0x3C80); }
  (void)tmp;
  B200_CUDA_TRY(cudaMemcpy(m->embed, emb.data(), emb.size() * 2, cudaMemcpyHostToDevice));
  m->finalized = true;
  return B200_OK;
}

static b200_status llama_forward_eager(b200_llama* m, b200_kv* kv, const b200_pack_desc* d_desc, int32_t n_req,
                                       int32_t total_rows, const uint32_t* d_prefill_tokens, void* stream);

b200_status b200_llama_forward(b200_llama* m, b200_kv* kv, const b200_pack_desc* d_desc, int32_t n_req, int32_t total_rows,
                               const uint32_t* d_prefill_tokens, void* stream) {
  // Decode-only steps (one row per request) are launch-bound at small batch: replay them as a graph.
  // (the legacy default stream cannot be captured)
  if (!m->graphs_on || m->prof_on || total_rows != n_req || n_req <= 0 || !m->finalized || stream == nullptr)
    return llama_forward_eager(m, kv, d_desc, n_req, total_rows, d_prefill_tokens, stream);
  auto& ge = m->graphs[std::make_tuple((int)n_req, (const void*)d_desc, (const void*)kv, stream, m->sampling)];
  ge.seen += 1;
  if (ge.seen == 1) return llama_forward_eager(m, kv, d_desc, n_req, total_rows, d_prefill_tokens, stream);
  cudaStream_t cs = (cudaStream_t)stream;
  if (!ge.exec) {
    if (m->graphs.size() > 64) {  // bounded cache: drop everything else
      for (auto& kvp : m->graphs) if (kvp.second.exec && &kvp.second != &ge) { cudaGraphExecDestroy(kvp.second.exec); kvp.second.exec = nullptr; kvp.second.seen = 0; }
    }
    cudaGraph_t graph = nullptr;
    B200_CUDA_TRY(cudaStreamBeginCapture(cs, cudaStreamCaptureModeThreadLocal));
    const long long before = m->launches;
    b200_status st = llama_forward_eager(m, kv, d_desc, n_req, total_rows, d_prefill_tokens, stream);
    ge.kernels = m->launches - before;  // nodes of the graph
    m->launches = before;
    cudaError_t e = cudaStreamEndCapture(cs, &graph);
    if (st != B200_OK) { if (graph) cudaGraphDestroy(graph); return st; }
    if (e != cudaSuccess) { b200_set_error("graph capture failed: %s", cudaGetErrorString(e)); cudaGetLastError(); return B200_ERR_CUDA; }
    e = cudaGraphInstantiate(&ge.exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) { ge.exec = nullptr; b200_set_error("graph instantiate failed: %s", cudaGetErrorString(e)); return B200_ERR_CUDA; }
  }
  B200_CUDA_TRY(cudaGraphLaunch(ge.exec, cs));
  m->last_n_req = n_req;
  m->launches += ge.kernels;
  return B200_OK;
}

static b200_status llama_forward_eager(b200_llama* m, b200_kv* kv, const b200_pack_desc* d_desc, int32_t n_req,
                                       int32_t total_rows, const uint32_t* d_prefill_tokens, void* stream) {
  if (!m->finalized) { b200_set_error("llama: weights not finalized"); return B200_ERR_INVALID_ARGUMENT; }
  const b200_llama_config& c = m->cfg;
  if (n_req < 0 || n_req > c.max_reqs || total_rows < 0 || total_rows > c.max_rows) {
    b200_set_error("llama: %d requests / %d rows exceed the configured %d / %d", n_req, total_rows, c.max_reqs, c.max_rows);
    return B200_ERR_CAPACITY;
  }
  if (kv->cfg.n_layers != c.n_layers || kv->cfg.n_kv_heads != c.n_kv_heads || kv->cfg.head_dim != c.head_dim ||
      kv->cfg.n_q_heads != c.n_heads) {
    b200_set_error("llama: the page pool was built for a different model shape");
    return B200_ERR_INVALID_ARGUMENT;
  }
  m->last_n_req = n_req;
  if (n_req == 0 || total_rows == 0) return B200_OK;
  const long long launches_before = g_b200_launch_counter;
  const int T = total_rows, qd = c.n_heads * c.head_dim, kd = c.n_kv_heads * c.head_dim, qkv_dim = qd + 2 * kd;
  b200_status st;
  cudaStream_t cs = (cudaStream_t)stream;
#define STEP_CAT(cat, call) do { cudaEvent_t pe_ = m->prof_begin(cat, cs); st = (call); m->prof_end(pe_, cs); if (st != B200_OK) return st; } while (0)
#define STEP(call) STEP_CAT(3, call)
  STEP(b200_pack_batch(d_desc, n_req, d_prefill_tokens, m->d_last_token, m->d_cu, m->d_tokens, m->d_pos, m->d_row_to_req,
                       m->d_row_seq, m->d_row_ctx, m->d_last_row, T, stream));
  STEP(b200_kv_reserve(kv, d_desc, n_req, stream));
  STEP(b200_embed_gather(m->embed, m->d_tokens, m->x, T, c.hidden, stream));
  const int fuse_qkv = (m->fuse_qkv_rope && kv->cfg.kv_dtype == B200_KV_BF16 && c.head_dim == 128) ? 1 : 0;
  // The o and down projections also write the RMSNorm their result feeds (fused into their split-K
  // finish pass), so only the first layer normalises x on its own.
  for (int l = 0; l < c.n_layers; ++l) {
    if (l == 0) STEP(b200_rmsnorm(m->x, m->attn_norm[l], m->h, T, c.hidden, c.rms_eps, stream));
    // When the q/k/v projection splits K, its partial sums go straight to RoPE + append (bf16 pools, head_dim 128):
    // same bits, one launch and one pass over the projection's output less.
    b200_qmm_partials parts;
    STEP_CAT(1, b200_qmm_deferred(m->wqkv[l], m->h, T, m->qkv, fuse_qkv, stream, &parts));
    if (parts.pending) {
      STEP_CAT(2, b200_kv_rope_append_partials(kv, l, &parts, m->qkv, qkv_dim, m->d_pos, m->d_row_seq, T, c.n_heads, c.rope_theta, stream));
    } else {
      STEP_CAT(2, b200_kv_rope_append_strided(kv, l, m->qkv, m->qkv + qd, m->qkv + qd + kd, qkv_dim, qkv_dim, qkv_dim, m->d_pos,
                                              m->d_row_seq, T, c.n_heads, c.rope_theta, stream));
    }
    // batches that hold prefill chunks (more rows than requests) take the grouped kernel
    if (T > n_req) { STEP_CAT(0, b200_paged_attn_prefill_strided(kv, l, m->qkv, qkv_dim, m->d_row_seq, m->d_row_ctx, T, m->attn, stream, l > 0)); }
    else { STEP_CAT(0, b200_paged_attn_decode_strided(kv, l, m->qkv, qkv_dim, m->d_row_seq, m->d_row_ctx, T, m->attn, stream, l > 0)); }
    STEP_CAT(1, b200_qmm_residual_norm(m->wo[l], m->attn, T, m->x, m->x, m->ffn_norm[l], c.rms_eps, m->h, stream));
    STEP_CAT(1, b200_qmm(m->wgu[l], m->h, T, m->act, B200_EPI_SWIGLU, nullptr, 0.f, B200_QMM_AUTO, stream));
    if (l + 1 < c.n_layers) {
      STEP_CAT(1, b200_qmm_residual_norm(m->wdown[l], m->act, T, m->x, m->x, m->attn_norm[l + 1], c.rms_eps, m->h, stream));
    } else {
      STEP_CAT(1, b200_qmm(m->wdown[l], m->act, T, m->x, B200_EPI_RESIDUAL, m->x, 0.f, B200_QMM_AUTO, stream));
    }
  }
  STEP(b200_gather_rows(m->x, m->d_last_row, m->last_h, n_req, c.hidden, stream));
  STEP(b200_rmsnorm(m->last_h, m->final_norm, m->last_hn, n_req, c.hidden, c.rms_eps, stream));
  STEP_CAT(1, b200_qmm(m->lm_head, m->last_hn, n_req, m->logits, B200_EPI_NONE, nullptr, 0.f, B200_QMM_AUTO, stream));
  if (m->sampling) {
    STEP(b200_sample_rows(m->logits, 0, n_req, c.vocab, m->d_samp, nullptr, nullptr, nullptr, m->d_next, m->d_logprobs, stream));
  } else {
    STEP(b200_argmax(m->logits, n_req, c.vocab, m->d_next, stream));
  }
  STEP(b200_scatter_tokens(m->d_next, d_desc, m->d_last_token, n_req, kv->dev.state, ST_ERR, ST_ATTN_ERR, stream));
#undef STEP
#undef STEP_CAT
  m->launches += g_b200_launch_counter - launches_before;
  return B200_OK;
}

b200_status b200_llama_step(b200_llama* m, b200_kv* kv, const b200_pack_desc* h_desc, int32_t n_req,
                            const uint32_t* h_prefill_tokens, int32_t n_prefill_tokens, uint32_t* h_next_tokens,
                            int32_t* out_free_pages, void* stream) {
  const b200_llama_config& c = m->cfg;
  if (n_req < 0 || n_req > c.max_reqs || n_prefill_tokens < 0 || n_prefill_tokens > c.max_rows) {
    b200_set_error("llama step: %d requests / %d prefill tokens exceed the configured limits", n_req, n_prefill_tokens);
    return B200_ERR_CAPACITY;
  }
  cudaStream_t s = (cudaStream_t)stream;
  long long total = 0;
  for (int i = 0; i < n_req; ++i) {
    m->h_desc[i] = h_desc[i];
    total += h_desc[i].count > 0 ? h_desc[i].count : 0;
  }
  if (total > c.max_rows) { b200_set_error("llama step: %lld rows > max_rows %d", total, c.max_rows); return B200_ERR_CAPACITY; }
  if (n_prefill_tokens > 0) std::memcpy(m->h_prefill, h_prefill_tokens, sizeof(uint32_t) * n_prefill_tokens);
  if (n_req > 0) B200_CUDA_TRY(cudaMemcpyAsync(m->d_desc, m->h_desc, sizeof(b200_pack_desc) * n_req, cudaMemcpyHostToDevice, s));
  if (n_prefill_tokens > 0)
    B200_CUDA_TRY(cudaMemcpyAsync(m->d_prefill, m->h_prefill, sizeof(uint32_t) * n_prefill_tokens, cudaMemcpyHostToDevice, s));
  m->sampling = m->samp_n > 0;
  if (m->sampling) {
    if (m->samp_n != n_req) {
      b200_set_error("llama step: %d sampler rows for %d requests", m->samp_n, n_req);
      m->samp_n = 0;
      m->sampling = false;
      return B200_ERR_INVALID_ARGUMENT;
    }
    B200_CUDA_TRY(cudaMemcpyAsync(m->d_samp, m->h_samp, sizeof(b200_sample_params) * n_req, cudaMemcpyHostToDevice, s));
  }
  m->samp_n = 0;
  b200_status st = b200_llama_forward(m, kv, m->d_desc, n_req, (int)total, m->d_prefill, stream);
  m->sampling = false;
  if (st != B200_OK) return st;
  if (n_req > 0) B200_CUDA_TRY(cudaMemcpyAsync(m->h_next, m->d_next, sizeof(uint32_t) * n_req, cudaMemcpyDeviceToHost, s));
  B200_CUDA_TRY(cudaMemcpyAsync(m->h_state, kv->dev.state, sizeof(int32_t) * 8, cudaMemcpyDeviceToHost, s));
  st = b200_qmm_error_words_async(m->h_state + 8, stream);
  if (st != B200_OK) return st;
  B200_CUDA_TRY(cudaStreamSynchronize(s));
  for (int i = 0; i < n_req; ++i) h_next_tokens[i] = m->h_next[i];
  if (out_free_pages) *out_free_pages = m->h_state[ST_FREE_TOP];
  if (m->h_state[8] == 0) m->h_state[8] = m->h_state[9];
  if (m->h_state[ST_ERR] != 0 || m->h_state[ST_ATTN_ERR] != 0 || m->h_state[8] != 0) {
    int32_t word = 0;
    b200_kv_error_word(kv, &word);  // clears the pool's words
    int32_t q = 0;
    b200_qmm_error_word(&q);
    const int code = m->h_state[ST_ERR] ? m->h_state[ST_ERR] : (m->h_state[ST_ATTN_ERR] ? m->h_state[ST_ATTN_ERR] : m->h_state[8]);
    b200_set_error("llama step: a kernel flagged %s", b200_status_name(code));
    return code;
  }
  return B200_OK;
}

b200_status b200_llama_set_samplers(b200_llama* m, const b200_sample_params* h_rows, int32_t n_req) {
  if (n_req < 0 || n_req > m->cfg.max_reqs || (n_req > 0 && h_rows == nullptr)) {
    b200_set_error("set_samplers: %d rows (the model holds %d requests)", n_req, m->cfg.max_reqs);
    return B200_ERR_INVALID_ARGUMENT;
  }
  for (int i = 0; i < n_req; ++i) m->h_samp[i] = h_rows[i];
  m->samp_n = n_req;
  return B200_OK;
}

b200_status b200_llama_last_logprobs(b200_llama* m, float* h_out, int32_t n_req) {
  if (n_req > m->last_n_req) { b200_set_error("last_logprobs: %d rows requested, last step had %d", n_req, m->last_n_req); return B200_ERR_CAPACITY; }
  if (n_req > 0) B200_CUDA_TRY(cudaMemcpy(h_out, m->d_logprobs, sizeof(float) * n_req, cudaMemcpyDeviceToHost));
  return B200_OK;
}

b200_status b200_llama_last_logits(b200_llama* m, void* h_bf16_out, int32_t n_req) {
  if (n_req > m->last_n_req) { b200_set_error("last_logits: %d rows requested, last step had %d", n_req, m->last_n_req); return B200_ERR_CAPACITY; }
  if (n_req > 0) B200_CUDA_TRY(cudaMemcpy(h_bf16_out, m->logits, (size_t)n_req * m->cfg.vocab * 2, cudaMemcpyDeviceToHost));
  return B200_OK;
}

int64_t b200_llama_launch_count(const b200_llama* m) { return m->launches; }
void b200_llama_enable_graphs(b200_llama* m, int32_t on) { m->graphs_on = on != 0; }
void b200_llama_set_fused_qkv_rope(b200_llama* m, int32_t on) {
  m->fuse_qkv_rope = on != 0;
  // graphs captured with the other setting hold the other kernels
  for (auto& g : m->graphs) if (g.second.exec) { cudaGraphExecDestroy(g.second.exec); g.second.exec = nullptr; g.second.seen = 0; }
}

// CUDA-event timing of the step's kernels by category (0 attention, 1 matmuls, 2 rope + KV append,
// 3 the rest).  collect() synchronises the device, adds the elapsed time of every recorded call
// to ms[4] / calls[4] and clears the record.
void b200_llama_profile_enable(b200_llama* m, int32_t on) { m->prof_on = on != 0; m->prof_used = 0; }
b200_status b200_llama_profile_collect(b200_llama* m, double* ms, int64_t* calls) {
  B200_CUDA_TRY(cudaDeviceSynchronize());
  for (int i = 0; i < 4; ++i) { ms[i] = 0; calls[i] = 0; }
  for (size_t i = 0; i + 1 < m->prof_used; i += 2) {
    float t = 0.f;
    B200_CUDA_TRY(cudaEventElapsedTime(&t, m->prof_events[i], m->prof_events[i + 1]));
    ms[m->prof_cat[i / 2]] += t;
    calls[m->prof_cat[i / 2]] += 1;
  }
  m->prof_used = 0;
  return B200_OK;
}

// Device buffers the caller may use for a device-resident step (benchmarks): descriptor array
// [max_reqs], prefill token buffer [max_rows], next-token output [max_reqs].
void b200_llama_device_buffers(b200_llama* m, b200_pack_desc** d_desc, uint32_t** d_prefill, uint32_t** d_next) {
  if (d_desc) *d_desc = m->d_desc;
  if (d_prefill) *d_prefill = m->d_prefill;
  if (d_next) *d_next = m->d_next;
}

}  // extern "C"
