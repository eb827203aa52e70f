// Host layer of the continuous-batching path: page/block manager, requests, scheduler and the
// flat batch builder.  Semantics follow the reference's Zig modules (cited per function in
// include/dmlx_b200.h); the data structures are this library's own: flat vectors indexed by block
// id, an open-addressing-free std::unordered_map for the two lookups the reference also hashes.
#include "dmlx_b200.h"

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

#include "common.h"

#include <execinfo.h>
#include <signal.h>
#include <unistd.h>

namespace {
thread_local std::string g_last_error;

// Debugging aid: with DMLX_B200_BACKTRACE=1 in the environment a fatal signal inside the process prints the
// native call stack (module + offset per frame, resolvable with addr2line) before the default action.
void fatal_signal(int sig) {
  void* frames[64];
  const int n = backtrace(frames, 64);
  const char msg[] = "dmlx_b200: fatal signal, native stack:\n";
  if (write(2, msg, sizeof(msg) - 1) < 0) {}
  backtrace_symbols_fd(frames, n, 2);
  signal(sig, SIG_DFL);
  raise(sig);
}
struct BacktraceInstaller {
  BacktraceInstaller() {
    const char* e = getenv("DMLX_B200_BACKTRACE");
    if (e && *e == '1') {
      signal(SIGSEGV, fatal_signal);
      signal(SIGBUS, fatal_signal);
      signal(SIGABRT, fatal_signal);
    }
  }
} g_backtrace_installer;
}
long long g_b200_launch_counter = 0;
extern "C" int64_t b200_launch_count(void) { return (int64_t)g_b200_launch_counter; }

void b200_set_error(const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
}

extern "C" {

const char* b200_last_error(void) { return g_last_error.c_str(); }

const char* b200_status_name(b200_status s) {
  switch (s) {
    case B200_OK: return "OK";
    case B200_ERR_INSUFFICIENT_BLOCKS: return "InsufficientBlocks";
    case B200_ERR_INVALID_BLOCK_ID: return "InvalidBlockId";
    case B200_ERR_PAGE_POOL_EXHAUSTED: return "PagePoolExhausted";
    case B200_ERR_INVALID_QUANT_BITS: return "InvalidQuantBits";
    case B200_ERR_INVALID_BATCH_INDEX: return "InvalidBatchIndex";
    case B200_ERR_INVALID_ARGUMENT: return "InvalidArgument";
    case B200_ERR_CUDA: return "CudaError";
    case B200_ERR_NO_DEVICE: return "NoDevice";
    case B200_ERR_UNSUPPORTED: return "Unsupported";
    case B200_ERR_CAPACITY: return "Capacity";
    case B200_ERR_DEVICE_FLAGGED: return "DeviceFlagged";
    case B200_ERR_CANCELLED: return "Cancelled";
    default: return "Unknown";
  }
}

int32_t b200_version(void) { return 100; }

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// paged.BlockManager
// ---------------------------------------------------------------------------------------------
struct BlockMeta {
  bool used = false;
  uint64_t ref_count = 0;
  bool has_hash = false;
  uint64_t hash = 0;
  uint64_t last_access = 0;
  uint64_t tokens_used = 0;
};

struct b200_block_manager {
  uint64_t total = 0;
  std::vector<uint64_t> free_stack;  // back() is popped next
  std::vector<BlockMeta> pool;
  std::unordered_map<uint64_t, std::vector<uint64_t>> req_to_blocks;
  std::unordered_map<uint64_t, uint64_t> block_hashes;
  uint64_t access_counter = 0;
};

static uint64_t fnv1a64(uint64_t seed, const uint32_t* toks, uint64_t n) {
  uint64_t h = 0xCBF29CE484222325ull;
  auto eat = [&](uint8_t b) {
    h ^= b;
    h *= 0x100000001B3ull;
  };
  for (int i = 0; i < 8; ++i) eat((uint8_t)(seed >> (8 * i)));
  for (uint64_t t = 0; t < n; ++t)
    for (int i = 0; i < 4; ++i) eat((uint8_t)(toks[t] >> (8 * i)));
  return h;
}

extern "C" {

b200_block_manager* b200_bm_create(uint64_t total_blocks) {
  auto* bm = new b200_block_manager();
  bm->total = total_blocks;
  bm->pool.resize(total_blocks);
  bm->free_stack.resize(total_blocks);
  for (uint64_t i = 0; i < total_blocks; ++i) bm->free_stack[i] = total_blocks - 1 - i;
  return bm;
}
void b200_bm_destroy(b200_block_manager* bm) { delete bm; }
int32_t b200_bm_can_allocate(const b200_block_manager* bm, uint64_t n) { return bm->free_stack.size() >= n; }

b200_status b200_bm_allocate_blocks(b200_block_manager* bm, uint64_t req_id, uint64_t n, uint64_t* out_ids) {
  if (bm->free_stack.size() < n) {
    b200_set_error("allocateBlocks: %llu requested, %zu free", (unsigned long long)n, bm->free_stack.size());
    return B200_ERR_INSUFFICIENT_BLOCKS;
  }
  bm->access_counter += 1;
  auto& owned = bm->req_to_blocks[req_id];
  for (uint64_t i = 0; i < n; ++i) {
    uint64_t id = bm->free_stack.back();
    bm->free_stack.pop_back();
    BlockMeta& b = bm->pool[id];
    b.used = true;
    b.ref_count = 1;
    b.last_access = bm->access_counter;
    b.tokens_used = 0;
    b.has_hash = false;
    owned.push_back(id);
    if (out_ids) out_ids[i] = id;
  }
  return B200_OK;
}

void b200_bm_free_blocks(b200_block_manager* bm, uint64_t req_id) {
  auto it = bm->req_to_blocks.find(req_id);
  if (it == bm->req_to_blocks.end()) return;
  for (uint64_t id : it->second) {
    if (id >= bm->pool.size()) continue;
    BlockMeta& b = bm->pool[id];
    if (b.ref_count > 1) {
      b.ref_count -= 1;
    } else {
      b.ref_count = 0;
      b.used = false;
      b.has_hash = false;
      b.tokens_used = 0;
      bm->free_stack.push_back(id);
    }
  }
  bm->req_to_blocks.erase(it);
}

b200_status b200_bm_copy_on_write(b200_block_manager* bm, uint64_t block_id, uint64_t* out_id) {
  if (block_id >= bm->pool.size()) {
    b200_set_error("copyOnWrite: block %llu out of range", (unsigned long long)block_id);
    return B200_ERR_INVALID_BLOCK_ID;
  }
  BlockMeta& b = bm->pool[block_id];
  if (b.ref_count <= 1) {
    *out_id = block_id;
    return B200_OK;
  }
  if (bm->free_stack.empty()) {
    b200_set_error("copyOnWrite: no free block for the copy");
    return B200_ERR_INSUFFICIENT_BLOCKS;
  }
  uint64_t nid = bm->free_stack.back();
  bm->free_stack.pop_back();
  BlockMeta& nb = bm->pool[nid];
  nb.used = true;
  nb.ref_count = 1;
  nb.has_hash = b.has_hash;
  nb.hash = b.hash;
  nb.last_access = bm->access_counter;
  nb.tokens_used = b.tokens_used;
  b.ref_count -= 1;
  *out_id = nid;
  return B200_OK;
}

uint64_t b200_bm_free_count(const b200_block_manager* bm) { return bm->free_stack.size(); }
uint64_t b200_bm_used_count(const b200_block_manager* bm) { return bm->total - bm->free_stack.size(); }
uint64_t b200_bm_total_blocks(const b200_block_manager* bm) { return bm->total; }
uint64_t b200_hash_block(uint64_t prev_hash, const uint32_t* token_ids, uint64_t n) {
  return fnv1a64(prev_hash, token_ids, n);
}

// The generator behind SamplerConfig.prng (src/sampling.zig:284-296): Zig's std.Random.DefaultPrng,
// i.e. xoshiro256++ with its four state words drawn from SplitMix64(seed).
void b200_prng_seed(uint64_t seed, uint64_t state[4]) {
  uint64_t sm = seed;
  for (int i = 0; i < 4; ++i) {
    sm += 0x9E3779B97F4A7C15ull;
    uint64_t z = sm;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    state[i] = z ^ (z >> 31);
  }
}
uint64_t b200_prng_next_u64(uint64_t s[4]) {
  auto rotl = [](uint64_t x, int k) { return (x << k) | (x >> (64 - k)); };
  const uint64_t r = rotl(s[0] + s[3], 23) + s[0];
  const uint64_t t = s[1] << 17;
  s[2] ^= s[0];
  s[3] ^= s[1];
  s[1] ^= s[2];
  s[0] ^= s[3];
  s[2] ^= t;
  s[3] = rotl(s[3], 45);
  return r;
}
// Random.float(f32): the low 23 bits are the mantissa, the number of leading zeros of the 64-bit draw
// lowers the exponent from 2^-1, with more draws when the top 41 bits are all zero.
float b200_prng_next_f32(uint64_t s[4]) {
  auto clz64 = [](uint64_t x) { return x == 0 ? 64u : (uint32_t)__builtin_clzll(x); };
  const uint64_t r = b200_prng_next_u64(s);
  uint32_t lz = clz64(r);
  if (lz >= 41) {
    lz = 41 + clz64(b200_prng_next_u64(s));
    if (lz == 41 + 64) lz += (uint32_t)__builtin_clz((uint32_t)b200_prng_next_u64(s) | 0x7FFu);
  }
  const uint32_t bits = ((126u - lz) << 23) | (uint32_t)(r & 0x7FFFFFu);
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}

b200_status b200_bm_find_cached_prefix(b200_block_manager* bm, const uint32_t* token_ids, uint64_t n_tokens,
                                       uint64_t block_size, uint64_t* out_ids, uint64_t cap, uint64_t* out_n) {
  *out_n = 0;
  if (block_size == 0) return B200_OK;
  uint64_t prev = 0, off = 0;
  while (off + block_size <= n_tokens) {
    uint64_t h = fnv1a64(prev, token_ids + off, block_size);
    auto it = bm->block_hashes.find(h);
    if (it == bm->block_hashes.end()) break;
    BlockMeta& b = bm->pool[it->second];
    if (!(b.used && b.tokens_used == block_size)) break;
    if (*out_n >= cap) {
      b200_set_error("findCachedPrefix: out array holds %llu ids", (unsigned long long)cap);
      return B200_ERR_CAPACITY;
    }
    b.ref_count += 1;
    bm->access_counter += 1;
    b.last_access = bm->access_counter;
    out_ids[(*out_n)++] = it->second;
    prev = h;
    off += block_size;
  }
  return B200_OK;
}

b200_status b200_bm_register_block_hash(b200_block_manager* bm, uint64_t block_id, uint64_t hash) {
  if (block_id >= bm->pool.size()) {
    b200_set_error("registerBlockHash: block %llu out of range", (unsigned long long)block_id);
    return B200_ERR_INVALID_BLOCK_ID;
  }
  bm->pool[block_id].has_hash = true;
  bm->pool[block_id].hash = hash;
  bm->block_hashes[hash] = block_id;
  return B200_OK;
}

uint64_t b200_bm_get_ref(const b200_block_manager* bm, uint64_t id) { return bm->pool[id].ref_count; }
void b200_bm_set_ref(b200_block_manager* bm, uint64_t id, uint64_t n) { bm->pool[id].ref_count = n; }
int32_t b200_bm_is_used(const b200_block_manager* bm, uint64_t id) { return bm->pool[id].used; }
uint64_t b200_bm_get_tokens_used(const b200_block_manager* bm, uint64_t id) { return bm->pool[id].tokens_used; }
void b200_bm_set_tokens_used(b200_block_manager* bm, uint64_t id, uint64_t n) { bm->pool[id].tokens_used = n; }
void b200_bm_share(b200_block_manager* bm, uint64_t req_id, uint64_t id) { bm->req_to_blocks[req_id].push_back(id); }
uint64_t b200_bm_blocks_of(const b200_block_manager* bm, uint64_t req_id, uint64_t* out_ids, uint64_t cap) {
  auto it = bm->req_to_blocks.find(req_id);
  if (it == bm->req_to_blocks.end()) return 0;
  for (uint64_t i = 0; i < it->second.size() && i < cap; ++i) out_ids[i] = it->second[i];
  return it->second.size();
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Request
// ---------------------------------------------------------------------------------------------
struct b200_request {
  uint64_t id = 0;
  std::vector<uint32_t> prompt;
  std::vector<uint32_t> generated;
  int32_t state = B200_REQ_WAITING;
  std::vector<uint64_t> block_ids;
  uint64_t max_tokens = 0;
  std::vector<uint32_t> stop;
  uint64_t prefill_offset = 0;
  int32_t kv_slot = -1;
  // Tokens of `generated` that a preemption appended to `prompt` (their K/V are recomputed by the
  // request's second prefill); they still count as output but no longer as decode positions.
  uint64_t folded = 0;
  int32_t error = B200_OK;  // why the request ended early (cancelled, or failed on its own)
};

extern "C" {

b200_request* b200_request_create(uint64_t id, const uint32_t* prompt, uint64_t n_prompt, uint64_t max_tokens,
                                  const uint32_t* stop_tokens, uint64_t n_stop) {
  auto* r = new b200_request();
  r->id = id;
  r->prompt.assign(prompt, prompt + n_prompt);
  r->max_tokens = max_tokens;
  r->stop.assign(stop_tokens, stop_tokens + n_stop);
  return r;
}
void b200_request_destroy(b200_request* r) { delete r; }
uint64_t b200_request_id(const b200_request* r) { return r->id; }
int32_t b200_request_state(const b200_request* r) { return r->state; }
uint64_t b200_request_prefill_offset(const b200_request* r) { return r->prefill_offset; }
uint64_t b200_request_prompt_len(const b200_request* r) { return r->prompt.size(); }
uint64_t b200_request_seq_len(const b200_request* r) { return r->prefill_offset + r->generated.size() - r->folded; }
int32_t b200_request_error(const b200_request* r) { return r->error; }
int32_t b200_request_is_stop_token(const b200_request* r, uint32_t t) {
  return std::find(r->stop.begin(), r->stop.end(), t) != r->stop.end();
}
int32_t b200_request_has_pending_prefill(const b200_request* r) { return r->prefill_offset < r->prompt.size(); }
uint64_t b200_request_current_prefill_chunk_len(const b200_request* r, uint64_t max_prefill_tokens) {
  return std::min<uint64_t>(r->prompt.size() - r->prefill_offset, max_prefill_tokens);
}
uint64_t b200_request_generated(const b200_request* r, uint32_t* out, uint64_t cap) {
  for (uint64_t i = 0; i < r->generated.size() && i < cap; ++i) out[i] = r->generated[i];
  return r->generated.size();
}
uint64_t b200_request_prompt(const b200_request* r, uint32_t* out, uint64_t cap) {
  for (uint64_t i = 0; i < r->prompt.size() && i < cap; ++i) out[i] = r->prompt[i];
  return r->prompt.size();
}
uint64_t b200_request_block_ids(const b200_request* r, uint64_t* out, uint64_t cap) {
  for (uint64_t i = 0; i < r->block_ids.size() && i < cap; ++i) out[i] = r->block_ids[i];
  return r->block_ids.size();
}
void b200_request_force_state(b200_request* r, int32_t state, uint64_t prefill_offset, const uint32_t* gen,
                              uint64_t n_gen) {
  r->state = state;
  r->prefill_offset = prefill_offset;
  r->generated.assign(gen, gen + n_gen);
}
int32_t b200_request_kv_slot(const b200_request* r) { return r->kv_slot; }

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// scheduler-side BlockManager: bump counter, view of a host BlockManager, or view of the device pool
// ---------------------------------------------------------------------------------------------
struct b200_sched_bm {
  uint64_t total_blocks = 0;
  uint64_t used_blocks = 0;
  b200_block_manager* real = nullptr;
  b200_kv* kv = nullptr;
  std::vector<int32_t> free_slots;  // device pool: sequence slots not bound to a request; back() first
  int32_t kv_free_cached = 0;

  bool can_allocate(uint64_t n) const {
    if (real) return b200_bm_can_allocate(real, n) != 0;
    if (kv) return !free_slots.empty() && (uint64_t)kv_free_cached >= n;
    return total_blocks - used_blocks >= n;
  }
  uint64_t free_count() const {
    if (real) return b200_bm_free_count(real);
    if (kv) return (uint64_t)kv_free_cached;
    return total_blocks - used_blocks;
  }
  b200_status refresh_kv() {
    int32_t fc = 0;
    b200_status st = b200_kv_free_count(kv, &fc);
    if (st != B200_OK) return st;
    kv_free_cached = fc;
    used_blocks = total_blocks - (uint64_t)fc;
    return B200_OK;
  }
  b200_status allocate(b200_request* req, uint64_t n) {
    if (real) {
      std::vector<uint64_t> ids(n);
      b200_status st = b200_bm_allocate_blocks(real, req->id, n, ids.data());
      if (st != B200_OK) return st;
      req->block_ids.insert(req->block_ids.end(), ids.begin(), ids.end());
      used_blocks = b200_bm_used_count(real);
      return B200_OK;
    }
    if (kv) {
      if (free_slots.empty()) {
        b200_set_error("no free sequence slot in the device pool");
        return B200_ERR_INSUFFICIENT_BLOCKS;
      }
      int32_t slot = free_slots.back();
      std::vector<int32_t> ids(n);
      b200_status st = b200_kv_alloc(kv, slot, (int32_t)n, ids.data());
      if (st != B200_OK) {
        // the cached free count was stale (pages taken by decode growth since it was read): refresh it
        // so that the caller sees the pool as it is
        if (st == B200_ERR_INSUFFICIENT_BLOCKS) refresh_kv();
        return st;
      }
      free_slots.pop_back();
      req->kv_slot = slot;
      for (int32_t id : ids) req->block_ids.push_back((uint64_t)id);
      return refresh_kv();
    }
    if (!can_allocate(n)) {
      b200_set_error("allocateBlocks: %llu requested, %llu free", (unsigned long long)n,
                     (unsigned long long)(total_blocks - used_blocks));
      return B200_ERR_INSUFFICIENT_BLOCKS;
    }
    for (uint64_t i = 0; i < n; ++i) req->block_ids.push_back(used_blocks++);
    return B200_OK;
  }
  void release(b200_request* req) {
    if (real) {
      b200_bm_free_blocks(real, req->id);
      used_blocks = b200_bm_used_count(real);
    } else if (kv) {
      if (req->kv_slot >= 0) {
        int32_t s = req->kv_slot;
        b200_kv_release(kv, &s, 1);
        free_slots.push_back(s);
        req->kv_slot = -1;
        refresh_kv();
      }
    } else {
      uint64_t freed = req->block_ids.size();
      used_blocks = freed <= used_blocks ? used_blocks - freed : 0;
    }
    req->block_ids.clear();
  }
};

extern "C" {

b200_sched_bm* b200_sched_bm_create(uint64_t total_blocks) {
  auto* b = new b200_sched_bm();
  b->total_blocks = total_blocks;
  return b;
}
b200_sched_bm* b200_sched_bm_create_with_real(b200_block_manager* real) {
  auto* b = new b200_sched_bm();
  b->real = real;
  b->total_blocks = b200_bm_total_blocks(real);
  b->used_blocks = b200_bm_used_count(real);
  return b;
}
b200_sched_bm* b200_sched_bm_create_with_kv(b200_kv* kv) {
  int32_t n_pages = 0, max_seqs = 0;
  if (b200_kv_dims(kv, &n_pages, &max_seqs) != B200_OK) return nullptr;
  auto* b = new b200_sched_bm();
  b->kv = kv;
  b->total_blocks = (uint64_t)n_pages;
  for (int32_t s = max_seqs - 1; s >= 0; --s) b->free_slots.push_back(s);
  if (b->refresh_kv() != B200_OK) {
    delete b;
    return nullptr;
  }
  return b;
}
void b200_sched_bm_destroy(b200_sched_bm* bm) { delete bm; }
// A sequence slot of the device pool taken out of admission (for pages filled from outside, e.g. a
// prefix restored from disk), and its return; sync re-reads the pool's free count after the caller
// has allocated or released pages behind the scheduler's back.
b200_status b200_sched_bm_park_slot(b200_sched_bm* bm, int32_t* out_slot) {
  if (!bm->kv || bm->free_slots.empty()) {
    b200_set_error("park_slot: no device pool behind this block manager, or no free sequence slot");
    return B200_ERR_INSUFFICIENT_BLOCKS;
  }
  *out_slot = bm->free_slots.back();
  bm->free_slots.pop_back();
  return B200_OK;
}
b200_status b200_sched_bm_unpark_slot(b200_sched_bm* bm, int32_t slot) {
  if (!bm->kv) { b200_set_error("unpark_slot: no device pool behind this block manager"); return B200_ERR_INVALID_ARGUMENT; }
  b200_status st = b200_kv_release(bm->kv, &slot, 1);
  if (st != B200_OK) return st;
  bm->free_slots.push_back(slot);
  return bm->refresh_kv();
}
b200_status b200_sched_bm_sync(b200_sched_bm* bm) { return bm->kv ? bm->refresh_kv() : B200_OK; }
// The same without reading the device: the caller already holds the pool's free count (a model step
// returns it), e.g. after decode growth took pages behind the scheduler's back.
void b200_sched_bm_note_free(b200_sched_bm* bm, uint64_t free_pages) {
  if (!bm->kv) return;
  bm->kv_free_cached = (int32_t)free_pages;
  bm->used_blocks = bm->total_blocks - free_pages;
}
int32_t b200_sched_bm_can_allocate(const b200_sched_bm* bm, uint64_t n) { return bm->can_allocate(n); }
uint64_t b200_sched_bm_free_count(const b200_sched_bm* bm) { return bm->free_count(); }
uint64_t b200_sched_bm_total_blocks(const b200_sched_bm* bm) { return bm->total_blocks; }
uint64_t b200_sched_bm_used_blocks(const b200_sched_bm* bm) { return bm->used_blocks; }

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Scheduler
// ---------------------------------------------------------------------------------------------
struct b200_scheduler {
  std::vector<b200_request*> waiting, running;
  b200_sched_bm* bm = nullptr;
  uint64_t max_prefill_tokens = 0;
  uint64_t blocks_per_request = 1;
  bool hold_admission = false;  // waiting requests stay where they are (set by a caller under pool pressure)
  // Pages the caller is willing to hand to newcomers in one schedule() call (default: no limit, the
  // reference's behaviour).  A waiting request is promoted only while ceil((prompt + 1) / 32) pages are
  // left of it, in arrival order: the first request that does not fit stops the promotions.
  uint64_t admission_budget = ~0ull;
};

extern "C" {

b200_scheduler* b200_scheduler_create(b200_sched_bm* bm, uint64_t max_prefill_tokens) {
  auto* s = new b200_scheduler();
  s->bm = bm;
  s->max_prefill_tokens = max_prefill_tokens;
  return s;
}
void b200_scheduler_destroy(b200_scheduler* s) { delete s; }

b200_status b200_scheduler_add_request(b200_scheduler* s, b200_request* r) {
  r->state = B200_REQ_WAITING;
  s->waiting.push_back(r);
  return B200_OK;
}

b200_status b200_scheduler_schedule(b200_scheduler* s, b200_request** prefill_out, uint64_t* n_prefill,
                                    b200_request** decode_out, uint64_t* n_decode, uint64_t cap,
                                    uint64_t* blocks_needed) {
  *n_prefill = *n_decode = 0;
  *blocks_needed = 0;
  if (s->running.size() + s->waiting.size() > cap) {
    b200_set_error("schedule: out arrays hold %llu requests, %zu active", (unsigned long long)cap,
                   s->running.size() + s->waiting.size());
    return B200_ERR_CAPACITY;
  }
  // Running requests first: mid-prefill ones keep prefilling, the rest decode.
  for (b200_request* r : s->running) {
    if (r->state == B200_REQ_PREFILLING && r->prefill_offset < r->prompt.size())
      prefill_out[(*n_prefill)++] = r;
    else
      decode_out[(*n_decode)++] = r;
  }
  // Promote waiting requests while a block can be had; keep arrival order among those left.
  size_t kept = 0;
  uint64_t budget = s->admission_budget;
  bool closed = s->hold_admission;
  for (size_t i = 0; i < s->waiting.size(); ++i) {
    b200_request* r = s->waiting[i];
    const uint64_t prompt_pages = (r->prompt.size() + 1 + 31) / 32;
    if (!closed && budget != ~0ull && prompt_pages > budget) closed = true;  // arrival order: nobody overtakes it
    if (!closed && s->bm->can_allocate(s->blocks_per_request)) {
      if (budget != ~0ull) budget -= prompt_pages;
      b200_status st = s->bm->allocate(r, s->blocks_per_request);
      if (st == B200_ERR_INSUFFICIENT_BLOCKS && s->bm->kv) {
        // The device pool turned out to be empty (its cached free count was stale): the request keeps
        // waiting, exactly as if canAllocate had said no (src/scheduler.zig:291-293, 306-309).
        *blocks_needed += s->blocks_per_request;
        s->waiting[kept++] = r;
        continue;
      }
      if (st != B200_OK) {
        s->waiting.erase(s->waiting.begin() + kept, s->waiting.begin() + i);
        return st;
      }
      r->state = B200_REQ_PREFILLING;
      prefill_out[(*n_prefill)++] = r;
      s->running.push_back(r);
    } else {
      *blocks_needed += s->blocks_per_request;
      s->waiting[kept++] = r;
    }
  }
  s->waiting.resize(kept);
  return B200_OK;
}

static void note_token(b200_request* r, uint32_t token) {
  r->generated.push_back(token);
  bool stop = std::find(r->stop.begin(), r->stop.end(), token) != r->stop.end();
  if (stop || r->generated.size() >= r->max_tokens) r->state = B200_REQ_DONE;
}

b200_status b200_scheduler_postprocess(b200_scheduler* s, const b200_token_output* outputs, uint64_t n) {
  for (uint64_t i = 0; i < n; ++i) {
    for (b200_request* r : s->running) {
      if (r->id != outputs[i].request_id) continue;
      if (r->state == B200_REQ_PREFILLING) {
        r->prefill_offset += std::min<uint64_t>(r->prompt.size() - r->prefill_offset, s->max_prefill_tokens);
        if (r->prefill_offset >= r->prompt.size()) {
          r->state = B200_REQ_DECODING;
          note_token(r, outputs[i].token);
        }
      } else {
        note_token(r, outputs[i].token);
      }
      break;
    }
  }
  size_t kept = 0;
  for (size_t i = 0; i < s->running.size(); ++i) {
    b200_request* r = s->running[i];
    if (r->state == B200_REQ_DONE)
      s->bm->release(r);
    else
      s->running[kept++] = r;
  }
  s->running.resize(kept);
  return B200_OK;
}

// Take a request out of the scheduler before it has finished (cancellation, or a failure that is its
// own: src/engine/request_state.zig:118,182-189; src/engine/engine_loop.zig:687-754 handleBatchError):
// its blocks go back to the pool, its state becomes done with `error` as the reason, everything else
// keeps running.
b200_status b200_scheduler_remove(b200_scheduler* s, b200_request* r, int32_t error) {
  auto drop = [&](std::vector<b200_request*>& v) {
    auto it = std::find(v.begin(), v.end(), r);
    if (it == v.end()) return false;
    v.erase(it);
    return true;
  };
  const bool was_running = drop(s->running);
  if (!was_running && !drop(s->waiting)) {
    b200_set_error("scheduler: request %llu is not active", (unsigned long long)r->id);
    return B200_ERR_INVALID_ARGUMENT;
  }
  if (was_running) s->bm->release(r);
  r->state = B200_REQ_DONE;
  r->error = error;
  return B200_OK;
}

// Preemption by recomputation (no reference counterpart: the reference admits on one free block and
// has no answer when decode growth finds the pool empty, src/scheduler.zig:242,291-293 vs
// src/kvcache/paged.zig:525-531).  A running request gives all its blocks back and returns to the head
// of the waiting queue; the tokens it has generated so far join its prompt, so that its next prefill
// rebuilds the same cache and its output continues where it stopped.
b200_status b200_scheduler_preempt(b200_scheduler* s, b200_request* r) {
  auto it = std::find(s->running.begin(), s->running.end(), r);
  if (it == s->running.end()) {
    b200_set_error("scheduler: request %llu is not running", (unsigned long long)r->id);
    return B200_ERR_INVALID_ARGUMENT;
  }
  s->running.erase(it);
  s->bm->release(r);
  r->prompt.insert(r->prompt.end(), r->generated.begin() + r->folded, r->generated.end());
  r->folded = r->generated.size();
  r->prefill_offset = 0;
  r->state = B200_REQ_WAITING;
  s->waiting.insert(s->waiting.begin(), r);
  return B200_OK;
}

void b200_scheduler_hold_admission(b200_scheduler* s, int32_t on) { s->hold_admission = on != 0; }
void b200_scheduler_set_admission_budget(b200_scheduler* s, uint64_t pages) { s->admission_budget = pages; }

uint64_t b200_scheduler_running(const b200_scheduler* s, b200_request** out, uint64_t cap) {
  for (uint64_t i = 0; i < s->running.size() && i < cap; ++i) out[i] = s->running[i];
  return s->running.size();
}

uint64_t b200_scheduler_active_count(const b200_scheduler* s) { return s->running.size() + s->waiting.size(); }
uint64_t b200_scheduler_waiting_count(const b200_scheduler* s) { return s->waiting.size(); }
uint64_t b200_scheduler_running_count(const b200_scheduler* s) { return s->running.size(); }

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// batch builder (host)
// ---------------------------------------------------------------------------------------------
// Token span a request contributes to the step: [begin, begin+count) of `src`.
struct Span {
  const uint32_t* src;
  uint64_t count;
  uint64_t base_pos;
};

static Span request_span(const b200_request* r, bool chunked, uint64_t max_prefill) {
  Span sp{nullptr, 0, 0};
  switch (r->state) {
    case B200_REQ_PREFILLING:
    case B200_REQ_WAITING: {
      uint64_t start = r->prefill_offset, end = r->prompt.size();
      sp.base_pos = r->prefill_offset;
      if (start >= end) {
        if (end > 0) {
          sp.src = &r->prompt[end - 1];
          sp.count = 1;
        }
        return sp;
      }
      if (chunked) end = start + std::min<uint64_t>(end - start, max_prefill);
      sp.src = &r->prompt[start];
      sp.count = end - start;
      return sp;
    }
    case B200_REQ_DECODING: {
      if (!r->generated.empty())
        sp.src = &r->generated.back();
      else if (!r->prompt.empty())
        sp.src = &r->prompt.back();
      else
        return sp;
      sp.count = 1;
      uint64_t sl = r->prefill_offset + r->generated.size() - r->folded;
      sp.base_pos = sl > 0 ? sl - sp.count : 0;
      return sp;
    }
    default:
      return sp;
  }
}

extern "C" {

b200_status b200_batch_build(b200_request* const* prefill, uint64_t n_prefill, b200_request* const* decode,
                             uint64_t n_decode, int32_t chunked, uint64_t max_prefill_tokens, uint32_t* tokens,
                             int32_t* positions, int32_t* row_to_req, uint64_t cap_tokens, int32_t* cu_seqlens,
                             uint64_t* total_tokens, uint64_t* num_requests) {
  uint64_t n_req = n_prefill + n_decode, off = 0;
  cu_seqlens[0] = 0;
  for (uint64_t i = 0; i < n_req; ++i) {
    const b200_request* r = i < n_prefill ? prefill[i] : decode[i - n_prefill];
    Span sp = request_span(r, chunked != 0, max_prefill_tokens);
    if (off + sp.count > cap_tokens) {
      b200_set_error("batch build: %llu-token capacity exceeded", (unsigned long long)cap_tokens);
      return B200_ERR_CAPACITY;
    }
    for (uint64_t j = 0; j < sp.count; ++j) {
      tokens[off + j] = sp.src[j];
      positions[off + j] = (int32_t)(sp.base_pos + j);
      row_to_req[off + j] = (int32_t)i;
    }
    off += sp.count;
    cu_seqlens[i + 1] = (int32_t)off;
  }
  *total_tokens = off;
  *num_requests = off == 0 ? 0 : n_req;
  return B200_OK;
}

static int64_t segment_of(const int32_t* cu, uint64_t n_req, uint64_t row) {
  // last i with cu[i] <= row
  uint64_t lo = 0, hi = n_req;
  while (lo < hi) {
    uint64_t mid = (lo + hi + 1) / 2;
    if ((uint64_t)cu[mid] <= row) lo = mid; else hi = mid - 1;
  }
  return (int64_t)lo;
}

int32_t b200_is_attending(const int32_t* cu_seqlens, uint64_t num_requests, uint64_t row, uint64_t col) {
  if (num_requests == 0) return 0;
  uint64_t total = (uint64_t)cu_seqlens[num_requests];
  if (row >= total || col >= total) return 0;
  return segment_of(cu_seqlens, num_requests, row) == segment_of(cu_seqlens, num_requests, col) && col <= row;
}

b200_status b200_batch_mask(const int32_t* cu_seqlens, uint64_t num_requests, float* mask, uint64_t total_tokens) {
  const float ninf = -__builtin_inff();
  for (uint64_t i = 0; i < total_tokens * total_tokens; ++i) mask[i] = ninf;
  for (uint64_t r = 0; r < num_requests; ++r)
    for (uint64_t row = (uint64_t)cu_seqlens[r]; row < (uint64_t)cu_seqlens[r + 1]; ++row)
      for (uint64_t col = (uint64_t)cu_seqlens[r]; col <= row; ++col) mask[row * total_tokens + col] = 0.0f;
  return B200_OK;
}

uint32_t b200_greedy_host(const float* logits, uint64_t n) {
  uint64_t best = 0;
  for (uint64_t i = 1; i < n; ++i)
    if (logits[i] > logits[best]) best = i;
  return (uint32_t)best;
}

}  // extern "C"
