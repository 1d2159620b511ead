// Continuous-batching scheduler and paged KV block allocator (host side, C++).
//
// BlockPool: fixed number of KV blocks, a free list, reference counts (a block shared by several sequences
// through a common prompt prefix is freed when the last of them finishes), and a content-hash index that lets a
// new request reuse full blocks of an identical prefix.
// Scheduler: requests wait in arrival order; each step either admits waiting requests for prefill (as many as
// fit the token budget and the free blocks) or advances every running sequence by one token. When a running
// sequence needs a block and none is free, the youngest running sequence is preempted (its blocks are released
// and it re-enters the waiting queue to be recomputed). Queue limit and per-request deadlines mirror the serving
// contracts of the reference (queue limit -> rejection, timeout).
//
// The reference serves one lease per model copy and batches statically (src/Idrak.Abstraction/Serving/EngineModel.cs:181-200,
// src/Idrak/Generation/TextGenerator.cs:569-623); its KV pages (src/Idrak.Abstraction/Generation/KeyValuePages.cs:20-34)
// share prefixes but are copied into a contiguous cache. This scheduler is what replaces both.
#include <cstdint>
#include <cstring>
#include <deque>
#include <mutex>
#include <unordered_map>
#include <vector>

#define IDRAK_API extern "C" __attribute__((visibility("default")))

namespace {

struct BlockPool {
  int num_blocks, block_size;
  std::vector<int> free_list;
  std::vector<int> refs;
  std::vector<uint64_t> hash_of;                       // content hash of a full block (0 = none)
  std::unordered_map<uint64_t, int> by_hash;
  BlockPool(int n, int bs) : num_blocks(n), block_size(bs), refs(n, 0), hash_of(n, 0) {
    free_list.reserve(n);
    for (int i = n - 1; i >= 0; --i) free_list.push_back(i);
  }
  int free_count() const { return int(free_list.size()); }
  int alloc() {
    if (free_list.empty()) return -1;
    int b = free_list.back();
    free_list.pop_back();
    if (hash_of[b]) {
      auto it = by_hash.find(hash_of[b]);
      if (it != by_hash.end() && it->second == b) by_hash.erase(it);
      hash_of[b] = 0;
    }
    refs[b] = 1;
    return b;
  }
  void retain(int b) { ++refs[b]; }
  void release(int b) {
    if (--refs[b] == 0) free_list.push_back(b);        // keeps its hash: may be revived by find() until reused
  }
  int find(uint64_t h) {
    auto it = by_hash.find(h);
    if (it == by_hash.end()) return -1;
    int b = it->second;
    if (refs[b] == 0) {                                 // revive a freed block whose content is still intact
      for (size_t i = 0; i < free_list.size(); ++i)
        if (free_list[i] == b) { free_list.erase(free_list.begin() + long(i)); break; }
      refs[b] = 1;
    } else {
      ++refs[b];
    }
    return b;
  }
  void publish(int b, uint64_t h) {
    if (h == 0) return;
    if (by_hash.find(h) == by_hash.end()) { by_hash[h] = b; hash_of[b] = h; }
  }
};

enum State : int { kWaiting = 0, kRunning = 1, kFinished = 2, kRejected = 3 };

struct Sequence {
  long long id;
  std::vector<int> tokens;        // prompt + generated
  int prompt_len;
  int max_new;
  int computed;                   // tokens whose KV is in the cache
  int cached_prefix;              // prompt tokens served from shared blocks at admission
  std::vector<int> blocks;
  State state;
  long long arrival;
  double deadline;                // absolute seconds, 0 = none
};

uint64_t mix(uint64_t h, uint64_t v) {
  h ^= v + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
  return h;
}

struct Scheduler {
  BlockPool pool;
  int max_batch, max_prefill_tokens, queue_limit;
  bool prefix_sharing;
  long long next_arrival = 0;
  std::unordered_map<long long, Sequence> seqs;
  std::deque<long long> waiting;
  std::vector<long long> running;
  std::mutex mu;
  long long preemptions = 0, rejected = 0, prefix_hits = 0;
  Scheduler(int blocks, int bs, int mb, int mpt, int ql, bool share)
      : pool(blocks, bs), max_batch(mb), max_prefill_tokens(mpt), queue_limit(ql), prefix_sharing(share) {}

  int blocks_for(int tokens) const { return (tokens + pool.block_size - 1) / pool.block_size; }

  void free_seq(Sequence& s) {
    for (int b : s.blocks) pool.release(b);
    s.blocks.clear();
    s.computed = 0;
  }

  // make sure `s` has blocks for `tokens` positions; false when the pool is exhausted
  bool ensure(Sequence& s, int tokens) {
    while (int(s.blocks.size()) < blocks_for(tokens)) {
      int b = pool.alloc();
      if (b < 0) return false;
      s.blocks.push_back(b);
    }
    return true;
  }

  // try to take full prompt blocks from identical prefixes already in the cache
  void share_prefix(Sequence& s) {
    s.cached_prefix = 0;
    if (!prefix_sharing) return;
    uint64_t h = 0x243f6a8885a308d3ull;
    const int bs = pool.block_size;
    // never share the block holding the last prompt token: its logits must be computed
    const int full = (s.prompt_len - 1) / bs;
    for (int i = 0; i < full; ++i) {
      for (int j = 0; j < bs; ++j) h = mix(h, uint64_t(uint32_t(s.tokens[size_t(i) * bs + j])));
      int b = pool.find(h);
      if (b < 0) break;
      s.blocks.push_back(b);
      s.cached_prefix = (i + 1) * bs;
      ++prefix_hits;
    }
  }

  void publish_prompt(Sequence& s) {
    if (!prefix_sharing) return;
    uint64_t h = 0x243f6a8885a308d3ull;
    const int bs = pool.block_size;
    const int full = s.prompt_len / bs;
    for (int i = 0; i < full && i < int(s.blocks.size()); ++i) {
      for (int j = 0; j < bs; ++j) h = mix(h, uint64_t(uint32_t(s.tokens[size_t(i) * bs + j])));
      pool.publish(s.blocks[size_t(i)], h);
    }
  }
};

}  // namespace

IDRAK_API void* idrak_sched_create(int num_blocks, int block_size, int max_batch, int max_prefill_tokens,
                                   int queue_limit, int prefix_sharing) {
  return new Scheduler(num_blocks, block_size, max_batch, max_prefill_tokens, queue_limit, prefix_sharing != 0);
}
IDRAK_API void idrak_sched_destroy(void* h) { delete static_cast<Scheduler*>(h); }

// Returns 0, or -1 when the queue is full (the request is rejected), -2 when it can never fit the cache.
IDRAK_API int idrak_sched_add(void* h, long long id, const int* prompt, int prompt_len, int max_new, double deadline) {
  auto* s = static_cast<Scheduler*>(h);
  std::lock_guard<std::mutex> lock(s->mu);
  if (s->queue_limit > 0 && int(s->waiting.size()) >= s->queue_limit) { ++s->rejected; return -1; }
  if (s->blocks_for(prompt_len + max_new) > s->pool.num_blocks) { ++s->rejected; return -2; }
  Sequence q;
  q.id = id;
  q.tokens.assign(prompt, prompt + prompt_len);
  q.prompt_len = prompt_len;
  q.max_new = max_new;
  q.computed = 0;
  q.cached_prefix = 0;
  q.state = kWaiting;
  q.arrival = s->next_arrival++;
  q.deadline = deadline;
  s->seqs.emplace(id, std::move(q));
  s->waiting.push_back(id);
  return 0;
}

// Plan the next engine step.
//   kind_out: 1 = prefill of the listed sequences (their uncached prompt tokens), 2 = one decode token for each
//   ids_out[max_ids], n_out. Returns the number of sequences in the step (0 = nothing to do).
IDRAK_API int idrak_sched_step(void* h, double now, int* kind_out, long long* ids_out, int max_ids,
                               long long* expired_out, int* n_expired) {
  auto* s = static_cast<Scheduler*>(h);
  std::lock_guard<std::mutex> lock(s->mu);
  int ne = 0;
  // drop requests whose deadline passed while waiting
  for (auto it = s->waiting.begin(); it != s->waiting.end();) {
    Sequence& q = s->seqs[*it];
    if (q.deadline > 0 && now > q.deadline) {
      q.state = kRejected;
      if (expired_out && ne < max_ids) expired_out[ne++] = q.id;
      it = s->waiting.erase(it);
    } else {
      ++it;
    }
  }
  if (n_expired) *n_expired = ne;
  // 1. admit waiting requests (prefill has priority: it shortens time to first token)
  int n = 0, budget = s->max_prefill_tokens;
  while (!s->waiting.empty() && int(s->running.size()) + n < s->max_batch && n < max_ids) {
    Sequence& q = s->seqs[s->waiting.front()];
    if (q.blocks.empty()) s->share_prefix(q);
    const int todo = int(q.tokens.size()) - q.cached_prefix;
    if (n > 0 && todo > budget) break;
    // keep one block per running sequence in reserve so decode can proceed
    const int need = s->blocks_for(int(q.tokens.size()) + 1) - int(q.blocks.size());
    if (need > s->pool.free_count() - int(s->running.size())) {
      if (n == 0 && s->running.empty() && need > s->pool.free_count()) {
        // nothing is running and it still does not fit: shared blocks are all it holds; release and retry later
        s->free_seq(q);
      }
      break;
    }
    s->ensure(q, int(q.tokens.size()) + 1);
    budget -= todo;
    ids_out[n++] = q.id;
    s->waiting.pop_front();
  }
  if (n > 0) {
    for (int i = 0; i < n; ++i) {
      Sequence& q = s->seqs[ids_out[i]];
      q.state = kRunning;
      s->running.push_back(q.id);
    }
    *kind_out = 1;
    return n;
  }
  // 2. decode: every running sequence needs room for one more position
  for (size_t i = 0; i < s->running.size();) {
    Sequence& q = s->seqs[s->running[i]];
    if (!s->ensure(q, int(q.tokens.size()) + 1)) {
      // preempt the youngest running sequence (largest arrival), possibly q itself
      size_t victim = 0;
      for (size_t j = 1; j < s->running.size(); ++j)
        if (s->seqs[s->running[j]].arrival > s->seqs[s->running[victim]].arrival) victim = j;
      Sequence& v = s->seqs[s->running[victim]];
      s->free_seq(v);
      v.state = kWaiting;
      s->waiting.push_front(v.id);
      s->running.erase(s->running.begin() + long(victim));
      ++s->preemptions;
      i = 0;                      // re-check everyone
      continue;
    }
    ++i;
  }
  n = 0;
  for (long long id : s->running)
    if (n < max_ids) ids_out[n++] = id;
  *kind_out = 2;
  return n;
}

// Sequence facts for building the step's tensors.
IDRAK_API int idrak_sched_seq_info(void* h, long long id, int* len, int* computed, int* cached_prefix, int* n_blocks) {
  auto* s = static_cast<Scheduler*>(h);
  std::lock_guard<std::mutex> lock(s->mu);
  auto it = s->seqs.find(id);
  if (it == s->seqs.end()) return -1;
  *len = int(it->second.tokens.size());
  *computed = it->second.computed;
  *cached_prefix = it->second.cached_prefix;
  *n_blocks = int(it->second.blocks.size());
  return int(it->second.state);
}
IDRAK_API int idrak_sched_seq_blocks(void* h, long long id, int* out, int max_out) {
  auto* s = static_cast<Scheduler*>(h);
  std::lock_guard<std::mutex> lock(s->mu);
  auto it = s->seqs.find(id);
  if (it == s->seqs.end()) return -1;
  int n = 0;
  for (int b : it->second.blocks)
    if (n < max_out) out[n++] = b;
  return n;
}
IDRAK_API int idrak_sched_seq_tokens(void* h, long long id, int* out, int max_out) {
  auto* s = static_cast<Scheduler*>(h);
  std::lock_guard<std::mutex> lock(s->mu);
  auto it = s->seqs.find(id);
  if (it == s->seqs.end()) return -1;
  int n = 0;
  for (int t : it->second.tokens)
    if (n < max_out) out[n++] = t;
  return n;
}

// After a prefill: the prompt's KV is in the cache. After any step: append the sampled token.
IDRAK_API int idrak_sched_commit(void* h, long long id, int new_token, int finished) {
  auto* s = static_cast<Scheduler*>(h);
  std::lock_guard<std::mutex> lock(s->mu);
  auto it = s->seqs.find(id);
  if (it == s->seqs.end()) return -1;
  Sequence& q = it->second;
  if (q.computed < q.prompt_len) s->publish_prompt(q);
  q.computed = int(q.tokens.size());
  q.tokens.push_back(new_token);
  const int generated = int(q.tokens.size()) - q.prompt_len;
  if (finished || generated >= q.max_new) {
    s->free_seq(q);
    q.state = kFinished;
    for (size_t i = 0; i < s->running.size(); ++i)
      if (s->running[i] == id) { s->running.erase(s->running.begin() + long(i)); break; }
    return 1;
  }
  return 0;
}

IDRAK_API int idrak_sched_abort(void* h, long long id) {
  auto* s = static_cast<Scheduler*>(h);
  std::lock_guard<std::mutex> lock(s->mu);
  auto it = s->seqs.find(id);
  if (it == s->seqs.end()) return -1;
  s->free_seq(it->second);
  it->second.state = kFinished;
  for (size_t i = 0; i < s->running.size(); ++i)
    if (s->running[i] == id) { s->running.erase(s->running.begin() + long(i)); break; }
  for (auto w = s->waiting.begin(); w != s->waiting.end(); ++w)
    if (*w == id) { s->waiting.erase(w); break; }
  return 0;
}
IDRAK_API void idrak_sched_forget(void* h, long long id) {
  auto* s = static_cast<Scheduler*>(h);
  std::lock_guard<std::mutex> lock(s->mu);
  s->seqs.erase(id);
}
// stats[0..7] = free blocks, total blocks, waiting, running, preemptions, rejected, prefix hits, block size
IDRAK_API void idrak_sched_stats(void* h, long long* stats) {
  auto* s = static_cast<Scheduler*>(h);
  std::lock_guard<std::mutex> lock(s->mu);
  stats[0] = s->pool.free_count();
  stats[1] = s->pool.num_blocks;
  stats[2] = (long long)s->waiting.size();
  stats[3] = (long long)s->running.size();
  stats[4] = s->preemptions;
  stats[5] = s->rejected;
  stats[6] = s->prefix_hits;
  stats[7] = s->pool.block_size;
}
