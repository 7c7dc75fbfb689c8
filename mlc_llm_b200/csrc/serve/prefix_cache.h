// Prefix cache: decides, for a new request, whether its prompt prefix already has KV data that can
// be forked from a live/recycled sequence or whether a finished ("recycling") sequence can be taken
// over outright. Finished sequences are kept in LRU order up to a bound and evicted on memory
// pressure through a removal callback (which frees the KV pages and the internal id).
//
// Behavioural counterpart: cpp/serve/prefix_cache.cc:49-426 (InsertSequence reuse threshold 0.9,
// lazy ExtendSequence + CommitSequenceExtention, RecycleSequence LRU, TryFreeMemory).
#pragma once
#include <cstdint>
#include <functional>
#include <list>
#include <memory>
#include <unordered_map>
#include <unordered_set>
#include <utility>
#include <vector>

#include "radix_tree.h"

namespace mlcb {

struct PrefixMatch {
  int64_t prefilled_offset = 0;            // tokens whose KV is already available
  int64_t forked_seq_id = -1;              // fork the new sequence from this one at the offset
  int64_t reused_seq_id = -1;              // take this recycled sequence over instead
  int64_t reused_seq_pop_last_tokens = 0;  // after popping this many trailing tokens
};

class PrefixCache {
 public:
  using RemoveCallback = std::function<void(int64_t)>;
  // max_recycling < 0: unbounded; enabled == false behaves as "no prefix cache".
  PrefixCache(bool enabled, int64_t max_recycling, RemoveCallback cb);

  bool enabled() const { return enabled_; }
  PrefixMatch InsertSequence(int64_t seq_id, const std::vector<int32_t>& tokens,
                             int sliding_window_size = -1, int attention_sink_size = 0);
  void ExtendSequence(int64_t seq_id, const std::vector<int32_t>& tokens);  // lazy
  void CommitSequenceExtention();
  void RollBackSequence(int64_t seq_id, int64_t num_tokens);
  // lazy == true keeps the sequence (and its KV) for later reuse; false drops it now.
  void RecycleSequence(int64_t seq_id, bool lazy = true);
  void PinSequence(int64_t seq_id) { pinned_.insert(seq_id); }
  bool TryFreeMemory();  // evicts the least recently used recycled sequence
  bool HasSequence(int64_t seq_id) const;
  // Number of tokens recorded for the sequence (pending lazy extensions are applied first).
  int64_t SequenceLength(int64_t seq_id);
  int64_t NumRecycling() const { return static_cast<int64_t>(lru_.size()); }
  void Reset();
  const RadixTree& tree() const { return tree_; }

 private:
  void Evict(int64_t seq_id);
  bool enabled_;
  int64_t max_recycling_;
  RemoveCallback remove_cb_;
  RadixTree tree_;
  std::list<int64_t> lru_;  // front = oldest
  std::unordered_map<int64_t, std::list<int64_t>::iterator> recycling_;
  std::unordered_set<int64_t> pinned_;
  std::unordered_set<int64_t> windowed_;  // sequences created with a sliding window
  std::vector<std::pair<int64_t, std::vector<int32_t>>> pending_extends_;
};

}  // namespace mlcb
