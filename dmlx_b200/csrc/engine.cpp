// Engine step: the caller the reference's framework is missing (its scheduler and batch builder are
// "not wired up" to a forward pass, docs/en/technical/continuous-batching-design.md:187).  One call
// runs schedule() -> ragged batch descriptors -> b200_llama_step -> postprocess(), i.e. the
// Engine_Step loop described at src/scheduler.zig:7-10, with the device page pool behind the
// scheduler's BlockManager (admission takes one page, completion releases the sequence).
//
// Prefill is always chunked here (a prefilling request contributes its current chunk,
// src/scheduler.zig:183-186): the reference's batch builder sends all remaining prompt tokens while
// postprocess advances by one chunk (src/batch_builder.zig:50-66 vs src/scheduler.zig:335-336), which
// would write the same tokens into the KV cache twice.
#include <algorithm>
#include <iterator>
#include <unordered_map>
#include <vector>

#include "common.h"

struct b200_engine {
  b200_llama* model = nullptr;
  b200_kv* kv = nullptr;
  b200_sched_bm* bm = nullptr;
  b200_scheduler* sched = nullptr;
  uint64_t max_prefill = 512;
  std::unordered_map<uint64_t, b200_request*> requests;  // owned
  std::vector<b200_request*> prefill, decode;
  std::vector<b200_pack_desc> descs;
  std::vector<uint32_t> flat, next;
  std::vector<b200_token_output> outs;
  std::vector<uint32_t> scratch;
  int32_t last_free_pages = 0;
  // Prefix sharing (paged.BlockManager.findCachedPrefix, src/kvcache/paged.zig:234-265, applied when a
  // request starts its prefill): live sequence slots with the chained hashes of their prompt blocks.
  bool share_prefix = false;
  uint64_t max_step_tokens = 0;  // 0 = no cap; else prefill chunks beyond the budget wait for a later step
  struct Live { b200_request* req; std::vector<uint64_t> chain; uint64_t parked_tokens = 0; };  // req == nullptr: a parked prefix
  std::unordered_map<int32_t, Live> live;               // by sequence slot
  std::unordered_map<uint64_t, uint64_t> shared_tokens;  // request id -> tokens taken over from a donor
  // Per-request samplers (SamplerConfig, src/sampling.zig:277-296); requests without one are greedy.
  struct Sampler { float temperature; int32_t top_k; float top_p; uint64_t prng[4]; };
  std::unordered_map<uint64_t, Sampler> samplers;
  std::vector<b200_sample_params> samp_rows;
  // Pool pressure: requests left out of a step because their page growth did not fit, and running
  // requests sent back to the waiting queue to make room (their cache is recomputed later).
  uint64_t n_deferred = 0, n_preempted = 0, n_failed = 0;
  bool pressure = false;  // the previous step left a running request out or preempted one: admit nobody new
  int32_t max_pages_per_seq = 0, pool_pages = 0;
  std::vector<b200_request*> running_tmp;
};

namespace {
constexpr uint64_t kPageTokens = 32;

// Chained hashes of the full 32-token blocks of a prompt (hashBlock, src/kvcache/paged.zig:224-230).
std::vector<uint64_t> prompt_chain(const std::vector<uint32_t>& prompt) {
  std::vector<uint64_t> chain;
  uint64_t h = 0;
  for (uint64_t b = 0; (b + 1) * kPageTokens <= prompt.size(); ++b) {
    h = b200_hash_block(h, prompt.data() + b * kPageTokens, kPageTokens);
    chain.push_back(h);
  }
  return chain;
}

// Tokens of a request whose K/V are in the pool.
uint64_t cached_tokens(const b200_request* r) {
  return b200_request_state(r) == B200_REQ_PREFILLING ? b200_request_prefill_offset(r) : b200_request_prompt_len(r);
}

// Pages a request holds before the step (one from admission, then ceil(len / 32), shared ones included)
// and the pages its rows of this step add (page-table growth of src/kvcache/paged.zig:525-531).
uint64_t pages_for(uint64_t tokens) { return (tokens + kPageTokens - 1) / kPageTokens; }
uint64_t pages_held(uint64_t len) { return std::max<uint64_t>(1, pages_for(len)); }
uint64_t pages_needed(uint64_t len, uint64_t count) {
  const uint64_t after = pages_for(len + count), held = pages_held(len);
  return after > held ? after - held : 0;
}

// A request about to run its first prefill chunk takes over the longest run of full prompt blocks
// that a live sequence already holds (same chained hashes, already prefilled): the pages are shared
// by reference count and the request's prefill cursor starts behind them.  At least one prompt
// token is always left to compute (its logits give the first output token).
b200_status try_share_prefix(b200_engine* e, b200_request* r, b200_engine::Live* self, bool* shared) {
  *shared = false;
  const int32_t slot = b200_request_kv_slot(r);
  std::vector<uint32_t> prompt(b200_request_prompt_len(r));
  b200_request_prompt(r, prompt.data(), prompt.size());
  b200_engine::Live me{r, prompt_chain(prompt)};
  uint64_t best = 0;
  int32_t donor = -1;
  for (const auto& kvp : e->live) {
    if (kvp.first == slot) continue;
    const auto& other = kvp.second;
    const uint64_t have = (other.req ? cached_tokens(other.req) : other.parked_tokens) / kPageTokens;
    uint64_t j = 0;
    while (j < me.chain.size() && j < other.chain.size() && j < have && me.chain[j] == other.chain[j]) ++j;
    if (j > best) { best = j; donor = kvp.first; }
  }
  while (best > 0 && best * kPageTokens >= prompt.size()) --best;
  *self = std::move(me);
  if (best == 0) return B200_OK;
  b200_status st = b200_kv_rollback(e->kv, slot, 0);  // give back the page taken at admission
  if (st == B200_OK) st = b200_kv_fork(e->kv, donor, slot, (int32_t)(best * kPageTokens));
  if (st != B200_OK) return st;
  b200_request_force_state(r, B200_REQ_PREFILLING, best * kPageTokens, nullptr, 0);
  e->shared_tokens[b200_request_id(r)] = best * kPageTokens;
  *shared = true;
  return B200_OK;
}
}  // namespace

extern "C" {

b200_engine* b200_engine_create(b200_llama* model, b200_kv* kv, uint64_t max_prefill_tokens) {
  auto* e = new b200_engine();
  e->model = model;
  e->kv = kv;
  e->max_prefill = std::max<uint64_t>(1, max_prefill_tokens);
  e->bm = b200_sched_bm_create_with_kv(kv);
  if (!e->bm) { delete e; return nullptr; }
  int32_t max_seqs = 0, page_size = 0;
  b200_kv_dims(kv, &e->pool_pages, &max_seqs);
  b200_kv_limits(kv, &e->max_pages_per_seq, &page_size);
  e->sched = b200_scheduler_create(e->bm, e->max_prefill);
  return e;
}

void b200_engine_destroy(b200_engine* e) {
  if (!e) return;
  b200_scheduler_destroy(e->sched);
  b200_sched_bm_destroy(e->bm);
  for (auto& kvp : e->requests) b200_request_destroy(kvp.second);
  delete e;
}

b200_status b200_engine_submit(b200_engine* e, uint64_t id, const uint32_t* prompt, uint64_t n_prompt, uint64_t max_tokens,
                               const uint32_t* stop_tokens, uint64_t n_stop) {
  if (e->requests.count(id)) { b200_set_error("engine: request id %llu already exists", (unsigned long long)id); return B200_ERR_INVALID_ARGUMENT; }
  if (n_prompt == 0 || max_tokens == 0) { b200_set_error("engine: empty prompt or max_tokens 0"); return B200_ERR_INVALID_ARGUMENT; }
  // A request whose prompt alone can never fit is refused here instead of blocking the queue for ever.
  const uint64_t most = std::min<uint64_t>((uint64_t)e->max_pages_per_seq, (uint64_t)e->pool_pages) * kPageTokens;
  if (n_prompt + 1 > most) {
    b200_set_error("engine: a prompt of %llu tokens exceeds what one sequence can hold (%llu tokens)", (unsigned long long)n_prompt,
                   (unsigned long long)most);
    return B200_ERR_CAPACITY;
  }
  b200_request* r = b200_request_create(id, prompt, n_prompt, max_tokens, stop_tokens, n_stop);
  e->requests[id] = r;
  return b200_scheduler_add_request(e->sched, r);
}

uint64_t b200_engine_active_count(const b200_engine* e) { return b200_scheduler_active_count(e->sched); }

namespace {
// Ends one request on its own account: out of the scheduler, pages back to the pool, the reason kept
// for b200_engine_request_status (per-request isolation, src/engine/engine_loop.zig:687-754).
b200_status end_request(b200_engine* e, b200_request* r, int32_t reason) {
  const int32_t slot = b200_request_kv_slot(r);
  b200_status st = b200_scheduler_remove(e->sched, r, reason);
  if (st != B200_OK) return st;
  if (slot >= 0) {
    auto it = e->live.find(slot);
    if (it != e->live.end() && it->second.req == r) e->live.erase(it);
  }
  return B200_OK;
}
}  // namespace

b200_status b200_engine_step(b200_engine* e, b200_token_output* out, uint64_t cap, uint64_t* n_out, void* stream) {
  *n_out = 0;
  b200_status st = B200_OK;
  uint64_t np = 0, nd = 0;
  // Up to a few rounds: a round that finds every runnable request blocked on page growth sends the
  // youngest running request back to the waiting queue and schedules again.
  bool pressure_now = false;
  for (int round = 0;; ++round) {
    const uint64_t active = b200_scheduler_active_count(e->sched);
    if (active == 0) return B200_OK;
    // While running requests are short of pages nobody new is admitted: a newcomer would take the page
    // an older request is waiting for (the reference admits on one free block, src/scheduler.zig:291).
    const uint64_t n_running = b200_scheduler_running_count(e->sched);
    b200_scheduler_hold_admission(e->sched, (e->pressure || pressure_now) && n_running > 0);
    // A newcomer is admitted only when its whole prompt fits beside what the running requests are still
    // owed: the prompt pages they have been promised but have not allocated yet (an admitted request
    // holds one page until its chunks run) and one page of growth each.  With nothing running the first
    // request always gets in (it fits the pool, checked at submission).
    {
      const uint64_t free_now = b200_sched_bm_free_count(e->bm);
      uint64_t owed = n_running;
      e->running_tmp.resize(active);
      const uint64_t n_run = b200_scheduler_running(e->sched, e->running_tmp.data(), active);
      for (uint64_t i = 0; i < n_run; ++i) {
        const b200_request* r = e->running_tmp[i];
        if (b200_request_state(r) != B200_REQ_PREFILLING) continue;
        const uint64_t want = pages_for(b200_request_prompt_len(r) + 1), held = pages_held(b200_request_prefill_offset(r));
        if (want > held) owed += want - held;
      }
      b200_scheduler_set_admission_budget(e->sched, n_running == 0 ? (uint64_t)e->pool_pages : (free_now > owed ? free_now - owed : 0));
    }
    e->prefill.resize(active);
    e->decode.resize(active);
    uint64_t need = 0;
    np = nd = 0;
    st = b200_scheduler_schedule(e->sched, e->prefill.data(), &np, e->decode.data(), &nd, active, &need);
    b200_scheduler_hold_admission(e->sched, 0);
    if (st != B200_OK) return st;
    if (np + nd == 0) { e->pressure = false; return B200_OK; }
    // A sequence that has reached the length its page table can hold ends here, alone (CacheOverflow,
    // src/kvcache/quantized.zig:135); the others go on.
    {
      const uint64_t most = (uint64_t)e->max_pages_per_seq * kPageTokens;
      uint64_t kept = 0;
      for (uint64_t i = 0; i < nd; ++i) {
        b200_request* r = e->decode[i];
        if (b200_request_seq_len(r) > most) {
          if ((st = end_request(e, r, B200_ERR_CAPACITY)) != B200_OK) return st;
          e->n_failed += 1;
        } else {
          e->decode[kept++] = r;
        }
      }
      nd = kept;
    }
    // Page budget of the step.  Decode rows come first (oldest request first), then prefill chunks in
    // scheduler order while the step's token budget lasts; a request whose growth does not fit is
    // left out of this step and keeps its cursor (postprocess only advances requests it gets an
    // output for).
    uint64_t free_pages = b200_sched_bm_free_count(e->bm);
    {
      uint64_t kept = 0;
      for (uint64_t i = 0; i < nd; ++i) {
        b200_request* r = e->decode[i];
        const uint64_t grow = pages_needed(b200_request_seq_len(r) - 1, 1);
        if (grow > free_pages) { e->n_deferred += 1; pressure_now = true; continue; }
        free_pages -= grow;
        e->decode[kept++] = r;
      }
      nd = kept;
    }
    {
      uint64_t used = nd, kept = 0;
      for (uint64_t i = 0; i < np; ++i) {
        b200_request* r = e->prefill[i];
        b200_engine::Live self;
        bool fresh = false, shared = false;
        if (e->share_prefix) {
          auto it = e->live.find(b200_request_kv_slot(r));
          fresh = !(it != e->live.end() && it->second.req == r) && b200_request_prefill_offset(r) == 0;
          if (fresh) {
            st = try_share_prefix(e, r, &self, &shared);
            if (st != B200_OK) return st;
            if (shared) {
              e->live[b200_request_kv_slot(r)] = self;  // it holds pages now, whether or not it runs this step
              if ((st = b200_sched_bm_sync(e->bm)) != B200_OK) return st;
              free_pages = std::min<uint64_t>(free_pages, b200_sched_bm_free_count(e->bm));
            }
          }
        }
        const uint64_t len = b200_request_current_prefill_chunk_len(r, e->max_prefill);
        if (e->max_step_tokens > 0 && used + len > e->max_step_tokens && (kept > 0 || nd > 0)) continue;  // tries again next step
        const uint64_t grow = pages_needed(b200_request_prefill_offset(r), len);
        if (grow > free_pages) { e->n_deferred += 1; pressure_now = true; continue; }
        free_pages -= grow;
        if (fresh && !shared) e->live[b200_request_kv_slot(r)] = std::move(self);
        used += len;
        e->prefill[kept++] = r;
      }
      np = kept;
    }
    if (np + nd > 0) break;
    pressure_now = true;
    // Nothing fits: every running request waits for a page nobody will free.  The youngest running
    // request gives its pages back and is prefilled again later; a request that is alone and still
    // does not fit can never run in this pool and fails on its own.
    e->running_tmp.resize(active);
    const uint64_t n_run = b200_scheduler_running(e->sched, e->running_tmp.data(), active);
    if (n_run == 0 || round >= 64) { e->pressure = true; return B200_OK; }
    b200_request* victim = e->running_tmp[n_run - 1];
    if (n_run == 1) {
      if ((st = end_request(e, victim, B200_ERR_INSUFFICIENT_BLOCKS)) != B200_OK) return st;
      e->n_failed += 1;
    } else {
      const int32_t slot = b200_request_kv_slot(victim);
      if ((st = b200_scheduler_preempt(e->sched, victim)) != B200_OK) return st;
      auto it = e->live.find(slot);
      if (it != e->live.end() && it->second.req == victim) e->live.erase(it);
      e->shared_tokens.erase(b200_request_id(victim));
      e->n_preempted += 1;
    }
  }
  // Tokens that will join a request's output this step (every decode row, and a prefill row whose
  // chunk is the last one, src/scheduler.zig:338-349) must fit the caller's array: checked before
  // anything is written to the cache.
  {
    uint64_t joining = nd;
    for (uint64_t i = 0; i < np; ++i) {
      b200_request* r = e->prefill[i];
      if (b200_request_prefill_offset(r) + b200_request_current_prefill_chunk_len(r, e->max_prefill) >= b200_request_prompt_len(r)) joining += 1;
    }
    if (joining > cap) { b200_set_error("engine step: output array holds %llu tokens, %llu needed", (unsigned long long)cap, (unsigned long long)joining); return B200_ERR_CAPACITY; }
  }
  e->descs.clear();
  e->flat.clear();
  for (uint64_t i = 0; i < np; ++i) {  // prefill requests first (src/batch_builder.zig:100-111)
    b200_request* r = e->prefill[i];
    const uint64_t off = b200_request_prefill_offset(r);
    const uint64_t len = b200_request_current_prefill_chunk_len(r, e->max_prefill);
    e->scratch.resize(b200_request_prompt_len(r));
    b200_request_prompt(r, e->scratch.data(), e->scratch.size());
    b200_pack_desc d{b200_request_kv_slot(r), (int32_t)len, (int32_t)off, (int32_t)e->flat.size()};
    e->flat.insert(e->flat.end(), e->scratch.begin() + off, e->scratch.begin() + off + len);
    e->descs.push_back(d);
  }
  for (uint64_t i = 0; i < nd; ++i) {  // decode rows take the token the device sampled last step
    b200_request* r = e->decode[i];
    e->descs.push_back(b200_pack_desc{b200_request_kv_slot(r), 1, (int32_t)(b200_request_seq_len(r) - 1), -1});
  }
  e->next.resize(e->descs.size());
  if (!e->samplers.empty()) {
    // One uniform variate per token that will join a request's output (decode rows and last prefill
    // chunks); the other rows' tokens are dropped, so they stay greedy and draw nothing.
    e->samp_rows.assign(e->descs.size(), b200_sample_params{0.f, 1.f, 1.f, 0.f, 0, 0});
    bool any = false;
    for (uint64_t i = 0; i < np + nd; ++i) {
      b200_request* r = i < np ? e->prefill[i] : e->decode[i - np];
      auto it = e->samplers.find(b200_request_id(r));
      if (it == e->samplers.end() || !(it->second.temperature > 0.f)) continue;
      const bool counts = i >= np || b200_request_prefill_offset(r) + b200_request_current_prefill_chunk_len(r, e->max_prefill) >=
                                         b200_request_prompt_len(r);
      if (!counts) continue;
      auto& sp = it->second;
      e->samp_rows[i] = b200_sample_params{sp.temperature, sp.top_p, 1.f, b200_prng_next_f32(sp.prng), sp.top_k, 0};
      any = true;
    }
    if (any) {
      st = b200_llama_set_samplers(e->model, e->samp_rows.data(), (int32_t)e->samp_rows.size());
      if (st != B200_OK) return st;
    }
  }
  st = b200_llama_step(e->model, e->kv, e->descs.data(), (int32_t)e->descs.size(), e->flat.data(), (int32_t)e->flat.size(),
                       e->next.data(), &e->last_free_pages, stream);
  // A flagged step has changed neither the pool (the reservation is all or nothing) nor any sequence's
  // next input token: the scheduler state is left as it was and the caller may step again.
  if (st != B200_OK) return st;
  b200_sched_bm_note_free(e->bm, (uint64_t)e->last_free_pages);
  e->pressure = pressure_now;
  e->outs.clear();
  for (uint64_t i = 0; i < np + nd; ++i) {
    b200_request* r = i < np ? e->prefill[i] : e->decode[i - np];
    e->outs.push_back(b200_token_output{b200_request_id(r), e->next[i], 0});
  }
  for (uint64_t i = 0; i < np + nd; ++i) {
    b200_request* r = i < np ? e->prefill[i] : e->decode[i - np];
    const bool last_chunk = i < np && b200_request_prefill_offset(r) + b200_request_current_prefill_chunk_len(r, e->max_prefill) >=
                                          b200_request_prompt_len(r);
    if (i >= np || last_chunk) out[(*n_out)++] = e->outs[i];
  }
  st = b200_scheduler_postprocess(e->sched, e->outs.data(), e->outs.size());
  if (e->share_prefix) {  // finished requests have given their slot back
    for (auto it = e->live.begin(); it != e->live.end();)
      it = it->second.req && b200_request_state(it->second.req) == B200_REQ_DONE ? e->live.erase(it) : std::next(it);
  }
  return st;
}

// Cancels a request wherever it is (waiting, mid-prefill or decoding): it leaves the scheduler at once,
// its pages return to the pool and the tokens it has produced stay readable
// (RequestState.cancelled, src/engine/request_state.zig:118,182-189; checked by the engine thread at
// src/engine/engine_loop.zig:240-243).  The engine is single-owner, so this is called between steps.
b200_status b200_engine_cancel(b200_engine* e, uint64_t id) {
  auto it = e->requests.find(id);
  if (it == e->requests.end()) { b200_set_error("engine: unknown request %llu", (unsigned long long)id); return B200_ERR_INVALID_ARGUMENT; }
  if (b200_request_state(it->second) == B200_REQ_DONE) return B200_OK;
  return end_request(e, it->second, B200_ERR_CANCELLED);
}

b200_status b200_engine_request_status(const b200_engine* e, uint64_t id, int32_t* status) {
  auto it = e->requests.find(id);
  if (it == e->requests.end()) { b200_set_error("engine: unknown request %llu", (unsigned long long)id); return B200_ERR_INVALID_ARGUMENT; }
  *status = b200_request_error(it->second);
  return B200_OK;
}

// Request ids of the last step's batch in descriptor order (prefill chunks first, then decode rows):
// row i of b200_llama_last_logits belongs to ids[i].
uint64_t b200_engine_last_batch(const b200_engine* e, uint64_t* ids, uint64_t cap) {
  for (uint64_t i = 0; i < e->outs.size() && i < cap; ++i) ids[i] = e->outs[i].request_id;
  return e->outs.size();
}

void b200_engine_pressure_stats(const b200_engine* e, uint64_t* deferred, uint64_t* preempted, uint64_t* failed) {
  if (deferred) *deferred = e->n_deferred;
  if (preempted) *preempted = e->n_preempted;
  if (failed) *failed = e->n_failed;
}

b200_status b200_engine_park_slot(b200_engine* e, int32_t* out_slot) { return b200_sched_bm_park_slot(e->bm, out_slot); }

b200_status b200_engine_publish_prefix(b200_engine* e, int32_t slot, const uint32_t* token_ids, uint64_t n_tokens) {
  int32_t len = 0;
  b200_status st = b200_kv_seq_len(e->kv, slot, &len);
  if (st != B200_OK) return st;
  if ((uint64_t)len < n_tokens) {
    b200_set_error("publish_prefix: slot %d holds %d tokens, %llu announced", slot, len, (unsigned long long)n_tokens);
    return B200_ERR_INVALID_ARGUMENT;
  }
  b200_engine::Live donor{nullptr, prompt_chain(std::vector<uint32_t>(token_ids, token_ids + n_tokens)), n_tokens};
  e->live[slot] = std::move(donor);
  return b200_sched_bm_sync(e->bm);
}

b200_status b200_engine_drop_prefix(b200_engine* e, int32_t slot) {
  auto it = e->live.find(slot);
  if (it == e->live.end() || it->second.req != nullptr) { b200_set_error("drop_prefix: slot %d holds no parked prefix", slot); return B200_ERR_INVALID_ARGUMENT; }
  e->live.erase(it);
  return b200_sched_bm_unpark_slot(e->bm, slot);
}

int32_t b200_engine_request_slot(const b200_engine* e, uint64_t id) {
  auto it = e->requests.find(id);
  return it == e->requests.end() ? -1 : b200_request_kv_slot(it->second);
}

b200_status b200_engine_set_sampler(b200_engine* e, uint64_t id, float temperature, int32_t top_k, float top_p, uint64_t seed) {
  if (!e->requests.count(id)) { b200_set_error("engine: unknown request %llu", (unsigned long long)id); return B200_ERR_INVALID_ARGUMENT; }
  b200_engine::Sampler sp{temperature, top_k, top_p, {0, 0, 0, 0}};
  b200_prng_seed(seed, sp.prng);
  e->samplers[id] = sp;
  return B200_OK;
}

void b200_engine_set_prefix_sharing(b200_engine* e, int32_t on) { e->share_prefix = on != 0; }
void b200_engine_set_max_step_tokens(b200_engine* e, uint64_t n) { e->max_step_tokens = n; }

uint64_t b200_engine_shared_tokens(const b200_engine* e, uint64_t id) {
  auto it = e->shared_tokens.find(id);
  return it == e->shared_tokens.end() ? 0 : it->second;
}

// Generated tokens of a request so far (and whether it has finished); finished requests stay
// queryable until b200_engine_forget.
b200_status b200_engine_result(const b200_engine* e, uint64_t id, uint32_t* out, uint64_t cap, uint64_t* n, int32_t* done) {
  auto it = e->requests.find(id);
  if (it == e->requests.end()) { b200_set_error("engine: unknown request %llu", (unsigned long long)id); return B200_ERR_INVALID_ARGUMENT; }
  *n = b200_request_generated(it->second, out, cap);
  *done = b200_request_state(it->second) == B200_REQ_DONE;
  return B200_OK;
}

void b200_engine_forget(b200_engine* e, uint64_t id) {
  auto it = e->requests.find(id);
  if (it == e->requests.end() || b200_request_state(it->second) != B200_REQ_DONE) return;
  b200_request_destroy(it->second);
  e->requests.erase(it);
  e->samplers.erase(id);
}

int32_t b200_engine_free_pages(const b200_engine* e) { return (int32_t)b200_sched_bm_free_count(e->bm); }

}  // extern "C"
