// Randomised stress driver for the continuous-batching scheduler, meant to be built with
// -fsanitize=address,undefined (host only): small page pool so that preemption, prefix-cache eviction, chunked prefill,
// aborts and cache resets all happen, with invariants checked after every step:
//   * a slot (page * block_size + offset) is handed to at most one token of a step,
//   * scheduled tokens stay within the batch budget and the sequence limit,
//   * positions are contiguous per sequence and block-table rows cover them,
//   * every request finishes with exactly the tokens it was given (prompt + committed tokens, in order).
// Prints "SCHED_STRESS_OK <steps>" on success; any sanitizer report or failed check makes the exit code non-zero.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <random>
#include <set>
#include <vector>

extern "C" {
void* vb_sched_create(int, int, int, int, int, int);
void vb_sched_destroy(void*);
int vb_sched_add(void*, int64_t, const int32_t*, int, int);
int vb_sched_step(void*);
int vb_sched_get_step(void*, int64_t*, int32_t*, int32_t*, int32_t*, int32_t*, int64_t*, int64_t*, int64_t*, int32_t*, int);
void vb_sched_commit(void*, const int64_t*, const int32_t*, int32_t*);
int vb_sched_output(void*, int64_t, int32_t*, int);
int vb_sched_remove(void*, int64_t);
void vb_sched_reset_prefix_cache(void*);
void vb_sched_stats(void*, int64_t*);
}

#define CHECK(c)                                                          \
  do {                                                                    \
    if (!(c)) {                                                           \
      std::fprintf(stderr, "check failed: %s (line %d)\n", #c, __LINE__); \
      std::exit(3);                                                       \
    }                                                                     \
  } while (0)

int main(int argc, char** argv) {
  const int seed = argc > 1 ? std::atoi(argv[1]) : 1;
  const int total_requests = argc > 2 ? std::atoi(argv[2]) : 400;
  const int num_blocks = 48, block_size = 4, max_seqs = 12, max_tokens = 40, max_len = 64;
  const int max_blocks = (max_len + block_size - 1) / block_size;
  std::mt19937 rng(seed);
  void* s = vb_sched_create(num_blocks, block_size, max_seqs, max_tokens, max_len, 1);
  CHECK(s != nullptr);
  std::map<int64_t, std::vector<int32_t>> expect;  // id -> prompt + committed tokens
  std::map<int64_t, int> budget;                   // id -> max new tokens
  std::set<int64_t> live;
  int64_t next_id = 0;
  int added = 0, finished = 0, aborted = 0, steps = 0;
  std::vector<int64_t> seq_ids(max_seqs + 8), tokens(max_tokens + max_seqs + 8), positions(tokens.size()), slots(tokens.size());
  std::vector<int32_t> ntok(seq_ids.size()), start(seq_ids.size()), is_prefill(seq_ids.size()), total(seq_ids.size());
  std::vector<int32_t> tables(seq_ids.size() * max_blocks), done(seq_ids.size()), fin(seq_ids.size());
  std::vector<int64_t> new_tok(seq_ids.size());
  while (finished + aborted < total_requests) {
    // arrivals: bursts that share a prefix with an earlier prompt half of the time (prefix cache)
    while (added < total_requests && (int)live.size() < 3 * max_seqs && rng() % 3 != 0) {
      std::vector<int32_t> prompt;
      if (!expect.empty() && rng() % 2 == 0) {
        auto it = expect.begin();
        std::advance(it, rng() % expect.size());
        const int keep = 1 + rng() % std::min<int>(it->second.size(), 24);
        prompt.assign(it->second.begin(), it->second.begin() + keep);
      }
      const int extra = 1 + rng() % 20;
      for (int i = 0; i < extra && (int)prompt.size() < max_len - 2; ++i) prompt.push_back(3 + rng() % 50);
      const int max_new = 1 + rng() % (max_len - (int)prompt.size());
      const int rc = vb_sched_add(s, next_id, prompt.data(), (int)prompt.size(), max_new);
      CHECK(rc == 0);
      expect[next_id] = prompt;
      budget[next_id] = max_new;
      live.insert(next_id);
      ++next_id;
      ++added;
    }
    const int n = vb_sched_step(s);
    CHECK(n >= 0 && n <= max_seqs);
    if (n == 0) {
      CHECK(!live.empty() || added < total_requests);
      if (live.empty()) continue;
      // nothing schedulable although requests are live would be a deadlock
      int64_t st[6];
      vb_sched_stats(s, st);
      CHECK(st[0] + st[1] == 0 || st[2] >= 0);
      if (st[0] + st[1] > 0) CHECK(++steps < 200000);
      continue;
    }
    const int t = vb_sched_get_step(s, seq_ids.data(), ntok.data(), start.data(), is_prefill.data(), total.data(), tokens.data(),
                                    positions.data(), slots.data(), tables.data(), max_blocks);
    CHECK(t > 0 && t <= max_tokens + max_seqs);
    std::set<int64_t> used_slots;
    int cursor = 0;
    for (int i = 0; i < n; ++i) {
      CHECK(live.count(seq_ids[i]) == 1);
      const auto& want = expect[seq_ids[i]];
      CHECK(start[i] + ntok[i] <= (int)want.size() && total[i] == start[i] + ntok[i] && total[i] <= max_len);
      for (int j = 0; j < ntok[i]; ++j, ++cursor) {
        CHECK(positions[cursor] == start[i] + j);
        CHECK(tokens[cursor] == want[start[i] + j]);
        CHECK(slots[cursor] >= 0 && slots[cursor] < (int64_t)num_blocks * block_size);
        CHECK(used_slots.insert(slots[cursor]).second);
        CHECK(tables[i * max_blocks + (start[i] + j) / block_size] == slots[cursor] / block_size);
      }
      const bool samples = is_prefill[i] != 2;
      new_tok[i] = samples ? (int64_t)(3 + rng() % 50) : -1;
      fin[i] = samples && rng() % 23 == 0;
    }
    CHECK(cursor == t);
    vb_sched_commit(s, new_tok.data(), fin.data(), done.data());
    for (int i = 0; i < n; ++i) {
      const int64_t id = seq_ids[i];
      if (new_tok[i] >= 0) expect[id].push_back((int32_t)new_tok[i]);
      if (done[i]) {
        std::vector<int32_t> out(max_len + 4);
        const int got = vb_sched_output(s, id, out.data(), (int)out.size());
        const auto& want = expect[id];
        CHECK(got >= 1 && got <= budget[id]);
        CHECK(got <= (int)want.size());
        for (int j = 0; j < got; ++j) CHECK(out[j] == want[want.size() - got + j]);
        CHECK(vb_sched_remove(s, id) == 1);
        live.erase(id);
        ++finished;
      }
    }
    if (!live.empty() && rng() % 37 == 0) {  // abort a random live request
      auto it = live.begin();
      std::advance(it, rng() % live.size());
      CHECK(vb_sched_remove(s, *it) == 1);
      live.erase(it);
      ++aborted;
    }
    if (rng() % 211 == 0) vb_sched_reset_prefix_cache(s);
    CHECK(++steps < 200000);
  }
  int64_t st[6];
  vb_sched_stats(s, st);
  CHECK(st[0] == 0 && st[1] == 0);
  vb_sched_destroy(s);
  std::printf("SCHED_STRESS_OK %d finished=%d aborted=%d preempted=%lld prefix_hits=%lld\n", steps, finished, aborted,
              (long long)st[3], (long long)st[4]);
  return 0;
}
