// Byte-pair-encoding merge engine (host code).
//
// The Python side splits text into pre-tokens; this engine turns each pre-token (a run of initial symbol ids) into
// its final token ids by applying the learned merges in rank order, with a cache of finished words behind a mutex so
// that repeated words cost one hash lookup. A batch of words is encoded in one call.
//
// Reference behaviour: the merge loop of src/Idrak/Models/BpeTokenizer.cs (lowest-rank adjacent pair first, leftmost
// on ties, repeated until no adjacent pair has a rank).
#include <cstdint>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

namespace {

struct Merge {
  int32_t rank;
  int32_t id;
};

struct Bpe {
  std::unordered_map<uint64_t, Merge> merges;
  std::unordered_map<std::string, std::vector<int32_t>> cache;
  std::mutex lock;
  size_t cache_limit = 1u << 20;
};

inline uint64_t key(int32_t a, int32_t b) { return (static_cast<uint64_t>(static_cast<uint32_t>(a)) << 32) | static_cast<uint32_t>(b); }

// Applies merges in place; returns the new length.
int merge_word(const Bpe& bpe, std::vector<int32_t>& w) {
  int n = static_cast<int>(w.size());
  while (n > 1) {
    int best = -1, best_rank = INT32_MAX, best_id = 0;
    for (int i = 0; i + 1 < n; ++i) {
      auto it = bpe.merges.find(key(w[i], w[i + 1]));
      if (it != bpe.merges.end() && it->second.rank < best_rank) {
        best_rank = it->second.rank;
        best = i;
        best_id = it->second.id;
      }
    }
    if (best < 0) break;
    // every non-overlapping occurrence of the winning pair merges in this pass, left to right
    const int32_t a = w[best], b = w[best + 1];
    int out = 0;
    for (int i = 0; i < n;) {
      if (i + 1 < n && w[i] == a && w[i + 1] == b) {
        w[out++] = best_id;
        i += 2;
      } else {
        w[out++] = w[i++];
      }
    }
    n = out;
  }
  w.resize(n);
  return n;
}

}  // namespace

#define IDRAK_API extern "C" __attribute__((visibility("default")))

// left / right / merged: n_merges ids each; the position in the arrays is the rank.
IDRAK_API void* idrak_bpe_create(const int32_t* left, const int32_t* right, const int32_t* merged, int64_t n_merges) {
  auto* bpe = new Bpe();
  bpe->merges.reserve(static_cast<size_t>(n_merges) * 2);
  for (int64_t i = 0; i < n_merges; ++i) {
    // the first (lowest-rank) rule for a pair wins
    bpe->merges.emplace(key(left[i], right[i]), Merge{static_cast<int32_t>(i), merged[i]});
  }
  return bpe;
}

IDRAK_API void idrak_bpe_free(void* handle) { delete static_cast<Bpe*>(handle); }

// symbols: the initial ids of all words back to back; offsets: n_words + 1 positions into it.
// out: room for at least offsets[n_words] ids (merging never lengthens a word); out_offsets: n_words + 1.
// Returns the number of ids written.
IDRAK_API int64_t idrak_bpe_encode(void* handle, const int32_t* symbols, const int64_t* offsets, int64_t n_words, int32_t* out,
                         int64_t* out_offsets) {
  auto* bpe = static_cast<Bpe*>(handle);
  int64_t total = 0;
  std::vector<int32_t> w;
  std::string k;
  out_offsets[0] = 0;
  for (int64_t i = 0; i < n_words; ++i) {
    const int64_t lo = offsets[i], hi = offsets[i + 1];
    const size_t bytes = static_cast<size_t>(hi - lo) * sizeof(int32_t);
    k.assign(reinterpret_cast<const char*>(symbols + lo), bytes);
    bool hit = false;
    {
      std::lock_guard<std::mutex> g(bpe->lock);
      auto it = bpe->cache.find(k);
      if (it != bpe->cache.end()) {
        std::memcpy(out + total, it->second.data(), it->second.size() * sizeof(int32_t));
        total += static_cast<int64_t>(it->second.size());
        hit = true;
      }
    }
    if (!hit) {
      w.assign(symbols + lo, symbols + hi);
      merge_word(*bpe, w);
      std::memcpy(out + total, w.data(), w.size() * sizeof(int32_t));
      total += static_cast<int64_t>(w.size());
      std::lock_guard<std::mutex> g(bpe->lock);
      if (bpe->cache.size() >= bpe->cache_limit) bpe->cache.clear();
      bpe->cache.emplace(k, w);
    }
    out_offsets[i + 1] = total;
  }
  return total;
}

IDRAK_API int64_t idrak_bpe_cache_size(void* handle) {
  auto* bpe = static_cast<Bpe*>(handle);
  std::lock_guard<std::mutex> g(bpe->lock);
  return static_cast<int64_t>(bpe->cache.size());
}

