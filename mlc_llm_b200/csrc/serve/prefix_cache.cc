#include "prefix_cache.h"

#include <algorithm>
#include <stdexcept>

namespace mlcb {

PrefixCache::PrefixCache(bool enabled, int64_t max_recycling, RemoveCallback cb)
    : enabled_(enabled), max_recycling_(max_recycling), remove_cb_(std::move(cb)), tree_(1 << 20) {}

void PrefixCache::Reset() {
  tree_.Reset();
  lru_.clear();
  recycling_.clear();
  pinned_.clear();
  windowed_.clear();
  pending_extends_.clear();
}

bool PrefixCache::HasSequence(int64_t seq_id) const { return enabled_ && tree_.Has(seq_id); }

int64_t PrefixCache::SequenceLength(int64_t seq_id) {
  CommitSequenceExtention();
  return tree_.GetLength(seq_id);
}

PrefixMatch PrefixCache::InsertSequence(int64_t seq_id, const std::vector<int32_t>& tokens,
                                        int sliding_window_size, int attention_sink_size) {
  PrefixMatch res;
  if (!enabled_) return res;
  CommitSequenceExtention();
  (void)attention_sink_size;
  const bool windowed = sliding_window_size > 0;
  // the last prompt token is always recomputed so that the model produces logits for it
  std::vector<int32_t> probe(tokens.begin(), tokens.empty() ? tokens.end() : tokens.end() - 1);
  auto [matched, seqs] = tree_.Match(probe);
  if (matched > 0) {
    // 1. a recycled sequence that is (almost) entirely covered can be taken over
    int64_t best = -1, best_len = -1;
    for (int64_t s : seqs) {
      if (!recycling_.count(s) || pinned_.count(s)) continue;
      const int64_t len = tree_.GetLength(s);
      const bool was_windowed = windowed_.count(s) != 0;
      bool ok;
      if (windowed || was_windowed) {
        ok = (windowed && was_windowed && len == matched);  // exact reuse only
      } else {
        ok = static_cast<double>(matched) > 0.9 * static_cast<double>(len);
      }
      if (ok && len > best_len) {
        best = s;
        best_len = len;
      }
    }
    if (best >= 0) {
      lru_.erase(recycling_[best]);
      recycling_.erase(best);
      const int64_t pop = best_len - matched;
      if (pop > 0) tree_.Rollback(best, pop);
      res.prefilled_offset = matched;
      res.reused_seq_id = best;
      res.reused_seq_pop_last_tokens = pop;
      return res;
    }
    // 2. otherwise fork from any non-windowed sequence sharing the prefix
    if (!windowed) {
      for (int64_t s : seqs) {
        if (windowed_.count(s)) continue;
        tree_.Fork(seq_id, s, matched);
        res.prefilled_offset = matched;
        res.forked_seq_id = s;
        // touching a recycled parent refreshes its LRU position
        auto it = recycling_.find(s);
        if (it != recycling_.end()) {
          lru_.erase(it->second);
          lru_.push_back(s);
          it->second = std::prev(lru_.end());
        }
        return res;
      }
    }
  }
  tree_.Add(seq_id);
  if (windowed) windowed_.insert(seq_id);
  return res;
}

void PrefixCache::ExtendSequence(int64_t seq_id, const std::vector<int32_t>& tokens) {
  if (!enabled_ || tokens.empty()) return;
  if (!pending_extends_.empty() && pending_extends_.back().first == seq_id) {
    auto& v = pending_extends_.back().second;
    v.insert(v.end(), tokens.begin(), tokens.end());
  } else {
    pending_extends_.emplace_back(seq_id, tokens);
  }
}

void PrefixCache::CommitSequenceExtention() {
  if (pending_extends_.empty()) return;
  auto pend = std::move(pending_extends_);
  pending_extends_.clear();
  for (auto& pr : pend)
    if (tree_.Has(pr.first)) tree_.Extend(pr.first, pr.second);
}

void PrefixCache::RollBackSequence(int64_t seq_id, int64_t num_tokens) {
  if (!enabled_) return;
  CommitSequenceExtention();
  if (tree_.Has(seq_id)) tree_.Rollback(seq_id, num_tokens);
}

void PrefixCache::Evict(int64_t seq_id) {
  auto it = recycling_.find(seq_id);
  if (it != recycling_.end()) {
    lru_.erase(it->second);
    recycling_.erase(it);
  }
  if (tree_.Has(seq_id)) tree_.Remove(seq_id);
  windowed_.erase(seq_id);
  pinned_.erase(seq_id);
  if (remove_cb_) remove_cb_(seq_id);
}

void PrefixCache::RecycleSequence(int64_t seq_id, bool lazy) {
  if (!enabled_) {
    if (remove_cb_) remove_cb_(seq_id);
    return;
  }
  CommitSequenceExtention();
  if (!tree_.Has(seq_id)) {
    if (remove_cb_) remove_cb_(seq_id);
    return;
  }
  if (!lazy || max_recycling_ == 0) {
    Evict(seq_id);
    return;
  }
  if (recycling_.count(seq_id)) return;
  lru_.push_back(seq_id);
  recycling_[seq_id] = std::prev(lru_.end());
  if (max_recycling_ > 0) {
    while (static_cast<int64_t>(lru_.size()) > max_recycling_) {
      if (!TryFreeMemory()) break;
    }
  }
}

bool PrefixCache::TryFreeMemory() {
  for (auto it = lru_.begin(); it != lru_.end(); ++it) {
    if (pinned_.count(*it)) continue;
    Evict(*it);
    return true;
  }
  return false;
}

}  // namespace mlcb
