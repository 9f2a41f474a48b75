// Continuous-batching scheduler and paged-KV block manager of the native rollout engine (host C++).
//
// Takes the place of the vLLM engine-core scheduler that the reference drives through
// verl/workers/rollout/vllm_rollout/vllm_async_server.py:391-547. One instance per rollout replica.
//
//  * Block manager: fixed pool of KV pages, free list, reference counts, and a prefix cache keyed
//    by a rolling hash of the full pages of a prompt (the n samples of one prompt share its pages).
//  * Scheduler (FCFS): every step first keeps running sequences decoding (one token each), then admits
//    waiting sequences for (chunked) prefill within the token budget. When pages run out the most
//    recently admitted running sequence is preempted (its pages are released; it is re-prefilled later
//    with the tokens generated so far).
//  * Abort / finish release pages immediately. All state is host memory; the Python side copies the
//    step description (token ids, positions, slot mapping, block tables) into pinned buffers.
//
// C ABI (ctypes). Not thread-safe: one engine loop thread owns an instance.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <deque>
#include <unordered_map>
#include <vector>

namespace {

struct Seq {
  int64_t id;
  std::vector<int32_t> tokens;   // prompt + generated so far
  int prompt_len = 0;
  int max_total = 0;             // prompt_len + max_new_tokens
  int computed = 0;              // tokens whose KV is in the cache
  std::vector<int32_t> blocks;   // page ids
  int num_cached_pages = 0;      // leading pages obtained from the prefix cache
  bool running = false;
  bool finished = false;
  int preempt_count = 0;
  std::vector<uint64_t> page_hashes;  // hash chain of the full prompt pages
};

struct Page {
  int ref = 0;
  uint64_t hash = 0;   // 0 = not registered in the prefix cache
  int64_t last_use = 0;
};

struct Scheduler {
  int num_blocks, block_size, max_num_seqs, max_batched_tokens, max_model_len;
  bool prefix_caching;
  std::vector<Page> pages;
  std::vector<int32_t> free_list;                    // pages with ref == 0 and no cached content
  std::unordered_map<uint64_t, int32_t> cache;        // hash -> page (may have ref == 0: evictable)
  std::deque<int32_t> evictable;                      // cached pages with ref == 0, oldest first
  std::unordered_map<int64_t, Seq> seqs;
  std::deque<int64_t> waiting;
  std::vector<int64_t> running;                       // admission order
  int64_t clock = 0;
  int64_t total_preempted = 0;
  int64_t prefix_hits = 0, prefix_queries = 0;

  // last step description
  std::vector<int64_t> step_seq_ids;     // per scheduled sequence
  std::vector<int32_t> step_num_tokens;  // tokens scheduled for that sequence
  std::vector<int32_t> step_start;       // first position computed this step
  std::vector<int32_t> step_is_prefill;
};

uint64_t mix(uint64_t h, uint64_t v) {
  h ^= v + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
  h *= 0xFF51AFD7ED558CCDull;
  h ^= h >> 33;
  return h ? h : 1;
}

int free_pages(const Scheduler* s) { return (int)s->free_list.size() + (int)s->evictable.size(); }

int32_t take_page(Scheduler* s) {
  if (!s->free_list.empty()) {
    int32_t p = s->free_list.back();
    s->free_list.pop_back();
    return p;
  }
  while (!s->evictable.empty()) {
    int32_t p = s->evictable.front();
    s->evictable.pop_front();
    if (s->pages[p].ref == 0 && s->pages[p].hash != 0) {
      auto it = s->cache.find(s->pages[p].hash);
      if (it != s->cache.end() && it->second == p) s->cache.erase(it);
      s->pages[p].hash = 0;
      return p;
    }
  }
  return -1;
}

void release_page(Scheduler* s, int32_t p) {
  Page& pg = s->pages[p];
  if (--pg.ref > 0) return;
  pg.ref = 0;
  if (pg.hash != 0 && s->prefix_caching) {
    pg.last_use = s->clock;
    s->evictable.push_back(p);
  } else {
    pg.hash = 0;
    s->free_list.push_back(p);
  }
}

void release_seq_pages(Scheduler* s, Seq& q) {
  for (int32_t p : q.blocks) release_page(s, p);
  q.blocks.clear();
  q.computed = 0;
  q.num_cached_pages = 0;
}

void compute_hashes(Scheduler* s, Seq& q) {
  q.page_hashes.clear();
  const int full = q.prompt_len / s->block_size;
  uint64_t h = 0x1234567ull;
  for (int b = 0; b < full; ++b) {
    for (int i = 0; i < s->block_size; ++i) h = mix(h, (uint64_t)(uint32_t)q.tokens[b * s->block_size + i]);
    q.page_hashes.push_back(h);
  }
}

// Try to reuse cached prompt pages for a sequence that owns no pages yet.
void match_prefix(Scheduler* s, Seq& q) {
  if (!s->prefix_caching) return;
  // never cache-hit the whole prompt: the last token must be computed to produce logits
  const int max_pages = (q.prompt_len - 1) / s->block_size;
  int n = 0;
  for (; n < (int)q.page_hashes.size() && n < max_pages; ++n) {
    s->prefix_queries++;
    auto it = s->cache.find(q.page_hashes[n]);
    if (it == s->cache.end()) break;
    s->prefix_hits++;
    int32_t p = it->second;
    if (s->pages[p].ref == 0) {
      // remove from evictable lazily: mark by bumping ref; stale deque entries are skipped in take_page
      auto e = std::find(s->evictable.begin(), s->evictable.end(), p);
      if (e != s->evictable.end()) s->evictable.erase(e);
    }
    s->pages[p].ref++;
    q.blocks.push_back(p);
  }
  q.num_cached_pages = n;
  q.computed = n * s->block_size;
}

bool ensure_pages(Scheduler* s, Seq& q, int upto_tokens) {
  const int need = (upto_tokens + s->block_size - 1) / s->block_size;
  while ((int)q.blocks.size() < need) {
    int32_t p = take_page(s);
    if (p < 0) return false;
    s->pages[p].ref = 1;
    s->pages[p].hash = 0;
    q.blocks.push_back(p);
  }
  return true;
}

// Register prompt pages that became fully computed so later requests can share them.
void publish_pages(Scheduler* s, Seq& q) {
  if (!s->prefix_caching) return;
  const int full_done = std::min(q.computed, q.prompt_len) / s->block_size;
  for (int b = q.num_cached_pages; b < full_done && b < (int)q.page_hashes.size(); ++b) {
    int32_t p = q.blocks[b];
    if (s->pages[p].hash != 0) continue;
    const uint64_t h = q.page_hashes[b];
    if (s->cache.find(h) == s->cache.end()) {
      s->cache[h] = p;
      s->pages[p].hash = h;
    }
  }
}

void preempt(Scheduler* s, int64_t id) {
  Seq& q = s->seqs[id];
  release_seq_pages(s, q);
  q.running = false;
  q.preempt_count++;
  s->total_preempted++;
  s->running.erase(std::find(s->running.begin(), s->running.end(), id));
  s->waiting.push_front(id);
}

}  // namespace

extern "C" {

void* vb_sched_create(int num_blocks, int block_size, int max_num_seqs, int max_batched_tokens, int max_model_len,
                      int prefix_caching) {
  auto* s = new Scheduler();
  s->num_blocks = num_blocks;
  s->block_size = block_size;
  s->max_num_seqs = max_num_seqs;
  s->max_batched_tokens = max_batched_tokens;
  s->max_model_len = max_model_len;
  s->prefix_caching = prefix_caching != 0;
  s->pages.resize(num_blocks);
  for (int i = num_blocks - 1; i >= 0; --i) s->free_list.push_back(i);
  return s;
}

void vb_sched_destroy(void* h) { delete static_cast<Scheduler*>(h); }

// Returns 0, or -1 if the id exists, -2 if the request can never fit.
int vb_sched_add(void* h, int64_t id, const int32_t* tokens, int prompt_len, int max_new_tokens) {
  auto* s = static_cast<Scheduler*>(h);
  if (s->seqs.count(id)) return -1;
  if (prompt_len <= 0 || prompt_len >= s->max_model_len) return -2;
  Seq q;
  q.id = id;
  q.tokens.assign(tokens, tokens + prompt_len);
  q.prompt_len = prompt_len;
  q.max_total = std::min(prompt_len + std::max(max_new_tokens, 0), s->max_model_len);
  if ((q.max_total + s->block_size - 1) / s->block_size > s->num_blocks) return -2;
  compute_hashes(s, q);
  s->seqs.emplace(id, std::move(q));
  s->waiting.push_back(id);
  return 0;
}

// Plan one engine step. Returns the number of scheduled sequences.
int vb_sched_step(void* h) {
  auto* s = static_cast<Scheduler*>(h);
  s->clock++;
  s->step_seq_ids.clear();
  s->step_num_tokens.clear();
  s->step_start.clear();
  s->step_is_prefill.clear();
  int budget = s->max_batched_tokens;

  // 1. running sequences: decode one token each (or continue a chunked prefill)
  for (size_t i = 0; i < s->running.size();) {
    const int64_t id = s->running[i];
    Seq& q = s->seqs[id];
    const int total = (int)q.tokens.size();
    int want = total - q.computed;  // >1 while a chunked prefill is still in flight
    if (want <= 0) { ++i; continue; }
    want = std::min(want, budget);
    if (want <= 0) break;
    bool ok = ensure_pages(s, q, q.computed + want);
    while (!ok && s->running.size() > 1) {
      // free pages by preempting the newest other running sequence
      int64_t victim = s->running.back();
      if (victim == id) {
        if (s->running.size() < 2) break;
        victim = s->running[s->running.size() - 2];
      }
      // un-schedule the victim if it was already planned this step
      for (size_t k = 0; k < s->step_seq_ids.size(); ++k) {
        if (s->step_seq_ids[k] == victim) {
          budget += s->step_num_tokens[k];
          s->step_seq_ids.erase(s->step_seq_ids.begin() + k);
          s->step_num_tokens.erase(s->step_num_tokens.begin() + k);
          s->step_start.erase(s->step_start.begin() + k);
          s->step_is_prefill.erase(s->step_is_prefill.begin() + k);
          break;
        }
      }
      const size_t vpos = std::find(s->running.begin(), s->running.end(), victim) - s->running.begin();
      preempt(s, victim);
      if (vpos < i) --i;
      ok = ensure_pages(s, s->seqs[id], s->seqs[id].computed + want);
    }
    if (!ok) { ++i; continue; }  // alone and still no room: wait for an abort / finish
    Seq& q2 = s->seqs[id];
    s->step_seq_ids.push_back(id);
    s->step_num_tokens.push_back(want);
    s->step_start.push_back(q2.computed);
    s->step_is_prefill.push_back(want > 1 || q2.computed < q2.prompt_len ? 1 : 0);
    budget -= want;
    ++i;
  }

  // 2. admit waiting sequences. A sequence whose first prompt page is being prefilled by another
  //    sequence admitted in this same step is deferred one step so it can hit the prefix cache
  //    (the n samples of one prompt arrive together).
  std::vector<uint64_t> inflight;
  size_t wi = 0;
  while (wi < s->waiting.size() && budget > 0 && (int)s->running.size() < s->max_num_seqs) {
    const int64_t id = s->waiting[wi];
    Seq& q = s->seqs[id];
    if (q.blocks.empty()) match_prefix(s, q);
    if (s->prefix_caching && q.num_cached_pages == 0 && !q.page_hashes.empty() &&
        std::find(inflight.begin(), inflight.end(), q.page_hashes[0]) != inflight.end()) {
      ++wi;
      continue;
    }
    const int total = (int)q.tokens.size();
    int want = std::min(total - q.computed, budget);
    // keep a reserve of one page per running sequence so decoding does not immediately preempt
    const int need_pages = (q.computed + want + s->block_size - 1) / s->block_size - (int)q.blocks.size();
    if (need_pages > free_pages(s) - (int)s->running.size()) {
      release_seq_pages(s, q);  // give matched pages back; retried next step
      break;
    }
    if (!ensure_pages(s, q, q.computed + want)) { release_seq_pages(s, q); break; }
    s->waiting.erase(s->waiting.begin() + wi);
    q.running = true;
    s->running.push_back(id);
    s->step_seq_ids.push_back(id);
    s->step_num_tokens.push_back(want);
    s->step_start.push_back(q.computed);
    s->step_is_prefill.push_back(1);
    budget -= want;
    if ((int)q.page_hashes.size() > q.num_cached_pages) inflight.push_back(q.page_hashes[0]);
  }
  return (int)s->step_seq_ids.size();
}

// Copy the plan of the last step. ``tokens``/``positions``/``slots`` have one entry per scheduled token,
// ``seq_*`` one per scheduled sequence. block tables are written as [num_seqs, max_blocks] (padded with 0).
// Returns the total number of scheduled tokens.
int vb_sched_get_step(void* h, int64_t* seq_ids, int32_t* seq_num_tokens, int32_t* seq_start, int32_t* seq_is_prefill,
                      int32_t* seq_total_len, int64_t* tokens, int64_t* positions, int64_t* slots, int32_t* block_tables,
                      int max_blocks) {
  auto* s = static_cast<Scheduler*>(h);
  int t = 0;
  for (size_t i = 0; i < s->step_seq_ids.size(); ++i) {
    Seq& q = s->seqs[s->step_seq_ids[i]];
    const int n = s->step_num_tokens[i], st = s->step_start[i];
    seq_ids[i] = q.id;
    seq_num_tokens[i] = n;
    seq_start[i] = st;
    // 0 = decode, 1 = prefill chunk that completes the known tokens (a token is sampled), 2 = partial chunk
    seq_is_prefill[i] = s->step_is_prefill[i] ? ((st + n == (int)q.tokens.size()) ? 1 : 2) : 0;
    seq_total_len[i] = st + n;
    for (int j = 0; j < n; ++j, ++t) {
      const int pos = st + j;
      tokens[t] = q.tokens[pos];
      positions[t] = pos;
      slots[t] = (int64_t)q.blocks[pos / s->block_size] * s->block_size + pos % s->block_size;
    }
    if (block_tables) {
      int32_t* row = block_tables + (size_t)i * max_blocks;
      const int nb = std::min((int)q.blocks.size(), max_blocks);
      std::memcpy(row, q.blocks.data(), sizeof(int32_t) * nb);
      for (int b = nb; b < max_blocks; ++b) row[b] = 0;
    }
  }
  return t;
}

// After the model ran the step: mark the scheduled tokens as computed. For sequences whose whole
// context is now computed, ``new_tokens[i]`` is the sampled token (ignored otherwise, pass -1).
// ``finished[i]`` != 0 ends the sequence (EOS / stop criteria decided by the caller); length limits
// are enforced here. Writes 1 to done_out[i] when sequence i ended in this step.
void vb_sched_commit(void* h, const int64_t* new_tokens, const int32_t* finished, int32_t* done_out) {
  auto* s = static_cast<Scheduler*>(h);
  for (size_t i = 0; i < s->step_seq_ids.size(); ++i) {
    const int64_t id = s->step_seq_ids[i];
    auto it = s->seqs.find(id);
    if (it == s->seqs.end()) { if (done_out) done_out[i] = 1; continue; }
    Seq& q = it->second;
    q.computed += s->step_num_tokens[i];
    publish_pages(s, q);
    int done = 0;
    if (q.computed == (int)q.tokens.size()) {
      if (new_tokens[i] >= 0) q.tokens.push_back((int32_t)new_tokens[i]);
      if ((finished && finished[i]) || (int)q.tokens.size() >= q.max_total) done = 1;
    }
    if (done) {
      q.finished = true;
      release_seq_pages(s, q);
      auto r = std::find(s->running.begin(), s->running.end(), id);
      if (r != s->running.end()) s->running.erase(r);
    }
    if (done_out) done_out[i] = done;
  }
}

// Burst decode: after vb_sched_step planned a pure decode step, reserve pages so that up to `k` consecutive decode
// steps of the planned sequences can run on the device without the host (the device advances positions and slots from
// the block tables by itself; a sequence that ends inside the burst just stops advancing). Returns the number of steps
// (1..k) that the reservation covers. 1 when the step contains prefill work, or when a waiting request could be
// admitted at the next step (a burst would delay it).
int vb_sched_reserve_burst(void* h, int k) {
  auto* s = static_cast<Scheduler*>(h);
  if (k <= 1 || s->step_seq_ids.empty()) return 1;
  if (!s->waiting.empty() && (int)s->running.size() < s->max_num_seqs) return 1;
  for (size_t i = 0; i < s->step_seq_ids.size(); ++i)
    if (s->step_is_prefill[i] || s->step_num_tokens[i] != 1) return 1;
  auto need_pages = [&](int kk) {
    long long need = 0;
    for (int64_t id : s->step_seq_ids) {
      const Seq& q = s->seqs[id];
      const int upto = std::min(q.computed + kk, q.max_total);
      const int pages = (upto + s->block_size - 1) / s->block_size;
      need += std::max(0, pages - (int)q.blocks.size());
    }
    return need;
  };
  while (k > 1 && need_pages(k) > free_pages(s)) k /= 2;
  if (k <= 1) return 1;
  for (int64_t id : s->step_seq_ids) {
    Seq& q = s->seqs[id];
    if (!ensure_pages(s, q, std::min(q.computed + k, q.max_total))) return 1;  // cannot happen after the count above
  }
  return k;
}

// Commit a burst of `k` decode steps of the last planned step. toks is [k][n] (n = planned sequences; entries of a
// sequence after its end are ignored), finished_at[i] = 1-based step at which the caller's stop criteria ended
// sequence i (0 = none). Length limits are enforced here. accepted_out[i] = number of tokens taken for sequence i,
// done_out[i] = 1 when it ended.
void vb_sched_commit_burst(void* h, const int64_t* toks, int k, const int32_t* finished_at, int32_t* accepted_out,
                           int32_t* done_out) {
  auto* s = static_cast<Scheduler*>(h);
  const size_t n = s->step_seq_ids.size();
  for (size_t i = 0; i < n; ++i) {
    const int64_t id = s->step_seq_ids[i];
    auto it = s->seqs.find(id);
    if (it == s->seqs.end()) { done_out[i] = 1; accepted_out[i] = 0; continue; }
    Seq& q = it->second;
    int done = 0, acc = 0;
    for (int j = 0; j < k && !done; ++j) {
      q.computed += 1;
      const int64_t t = toks[(size_t)j * n + i];
      if (t >= 0) { q.tokens.push_back((int32_t)t); ++acc; }
      if ((finished_at && finished_at[i] == j + 1) || (int)q.tokens.size() >= q.max_total || t < 0) done = 1;
    }
    publish_pages(s, q);
    if (done) {
      q.finished = true;
      release_seq_pages(s, q);
      auto r = std::find(s->running.begin(), s->running.end(), id);
      if (r != s->running.end()) s->running.erase(r);
    }
    accepted_out[i] = acc;
    done_out[i] = done;
  }
}

// max_total (prompt + allowed new tokens) of the sequences of the last planned step
void vb_sched_step_limits(void* h, int32_t* limits) {
  auto* s = static_cast<Scheduler*>(h);
  for (size_t i = 0; i < s->step_seq_ids.size(); ++i) limits[i] = s->seqs[s->step_seq_ids[i]].max_total;
}

// Number of generated tokens (tokens beyond the prompt) and copy of them.
int vb_sched_output(void* h, int64_t id, int32_t* out, int cap) {
  auto* s = static_cast<Scheduler*>(h);
  auto it = s->seqs.find(id);
  if (it == s->seqs.end()) return -1;
  const Seq& q = it->second;
  const int n = (int)q.tokens.size() - q.prompt_len;
  if (out) std::memcpy(out, q.tokens.data() + q.prompt_len, sizeof(int32_t) * std::min(n, cap));
  return n;
}

int vb_sched_preempt_count(void* h, int64_t id) {
  auto* s = static_cast<Scheduler*>(h);
  auto it = s->seqs.find(id);
  return it == s->seqs.end() ? -1 : it->second.preempt_count;
}

// Remove a sequence (finished, or aborted while waiting / running). Returns 1 if it existed.
int vb_sched_remove(void* h, int64_t id) {
  auto* s = static_cast<Scheduler*>(h);
  auto it = s->seqs.find(id);
  if (it == s->seqs.end()) return 0;
  release_seq_pages(s, it->second);
  auto r = std::find(s->running.begin(), s->running.end(), id);
  if (r != s->running.end()) s->running.erase(r);
  auto w = std::find(s->waiting.begin(), s->waiting.end(), id);
  if (w != s->waiting.end()) s->waiting.erase(w);
  s->seqs.erase(it);
  return 1;
}

void vb_sched_reset_prefix_cache(void* h) {
  auto* s = static_cast<Scheduler*>(h);
  for (int32_t p : s->evictable) {
    if (s->pages[p].ref == 0) {
      s->pages[p].hash = 0;
      s->free_list.push_back(p);
    }
  }
  s->evictable.clear();
  s->cache.clear();
  for (auto& pg : s->pages) pg.hash = 0;
}

// stats: [0] waiting, [1] running, [2] free pages, [3] total preemptions, [4] prefix hits, [5] prefix queries
void vb_sched_stats(void* h, int64_t* out) {
  auto* s = static_cast<Scheduler*>(h);
  out[0] = (int64_t)s->waiting.size();
  out[1] = (int64_t)s->running.size();
  out[2] = free_pages(s);
  out[3] = s->total_preempted;
  out[4] = s->prefix_hits;
  out[5] = s->prefix_queries;
}

}  // extern "C"
