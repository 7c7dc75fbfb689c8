#include "kv_manager.h"

#include <algorithm>
#include <string>

namespace mlcb {

KVManager::KVManager(int64_t num_pages, int page_size, int64_t max_num_sequence)
    : num_pages_(num_pages), page_size_(page_size), max_num_sequence_(max_num_sequence) {
  Clear();
}

void KVManager::Clear() {
  seqs_.clear();
  pending_copies_.clear();
  pending_forks_.clear();
  total_len_ = 0;
  refcnt_.assign(static_cast<size_t>(num_pages_), 0);
  free_pages_.clear();
  free_pages_.reserve(static_cast<size_t>(num_pages_));
  for (int64_t p = num_pages_ - 1; p >= 0; --p) free_pages_.push_back(static_cast<int32_t>(p));
}

KVManager::Seq& KVManager::Get(int64_t id) {
  auto it = seqs_.find(id);
  if (it == seqs_.end()) throw std::runtime_error("KVManager: unknown sequence " + std::to_string(id));
  return it->second;
}
const KVManager::Seq& KVManager::Get(int64_t id) const {
  auto it = seqs_.find(id);
  if (it == seqs_.end()) throw std::runtime_error("KVManager: unknown sequence " + std::to_string(id));
  return it->second;
}

int32_t KVManager::AllocPage() {
  if (free_pages_.empty()) throw std::runtime_error("KVManager: out of KV pages");
  int32_t p = free_pages_.back();
  free_pages_.pop_back();
  refcnt_[p] = 1;
  return p;
}

void KVManager::ReleasePage(int32_t p) {
  if (p < 0) return;
  if (--refcnt_[p] != 0) return;
  free_pages_.push_back(p);
  // a copy that was to fill this page is moot now; leaving it queued would let it write into whoever gets the
  // page next
  for (size_t i = 0; i + 1 < pending_copies_.size();) {
    if (pending_copies_[i + 1] == p) {
      const int32_t src = pending_copies_[i];
      pending_copies_.erase(pending_copies_.begin() + i, pending_copies_.begin() + i + 2);
      ReleasePage(src);  // the reference QueueCopy took
      i = 0;             // the recursion may have edited the list
    } else {
      i += 2;
    }
  }
}

// The device runs all queued copies of a plan in ONE launch, so no pair may read a page that another pair writes,
// and a source must keep its content until that launch: a source that is itself waiting to be filled is replaced
// by the page it will be filled from (a fresh copy destination holds nothing else yet), and every source is held
// by a reference of its own until the plan that carries the pair is made.
void KVManager::QueueCopy(int32_t src, int32_t dst) {
  for (bool again = true; again;) {
    again = false;
    for (size_t i = 0; i + 1 < pending_copies_.size(); i += 2)
      if (pending_copies_[i + 1] == src) {
        src = pending_copies_[i];
        again = true;
        break;
      }
  }
  ++refcnt_[src];
  pending_copies_.push_back(src);
  pending_copies_.push_back(dst);
}

void KVManager::AddSequence(int64_t seq_id) {
  if (seqs_.count(seq_id)) throw std::runtime_error("KVManager: sequence exists");
  if (static_cast<int64_t>(seqs_.size()) >= max_num_sequence_)
    throw std::runtime_error("KVManager: too many sequences");
  seqs_[seq_id] = Seq();
}

void KVManager::ForkSequence(int64_t parent_id, int64_t child_id, int64_t fork_pos) {
  if (seqs_.count(child_id)) throw std::runtime_error("KVManager: sequence exists");
  if (static_cast<int64_t>(seqs_.size()) >= max_num_sequence_)
    throw std::runtime_error("KVManager: too many sequences");
  const Seq& parent = Get(parent_id);
  if (fork_pos < 0) fork_pos = parent.len;
  if (fork_pos > parent.len) throw std::runtime_error("KVManager: fork position beyond parent");
  // A windowed parent may have let pages go. The child inherits the window, and its first new token (position
  // fork_pos) sees positions from fork_pos + 1 - window on: the fork is sound when nothing dropped lies there.
  if (parent.window > 0 && parent.dropped_until > 0 &&
      std::max<int64_t>(fork_pos + 1 - parent.window, parent.sink) < parent.dropped_until)
    throw std::runtime_error("KVManager: cannot fork a sequence below what its window already dropped");
  Seq child;
  child.window = parent.window;
  child.sink = parent.sink;
  child.dropped_until = parent.window > 0 ? std::min<int64_t>(parent.dropped_until, fork_pos / page_size_ * page_size_) : 0;
  const int64_t full = fork_pos / page_size_;
  const int64_t rem = fork_pos % page_size_;
  if (rem != 0 && free_pages_.empty()) throw std::runtime_error("KVManager: out of KV pages");
  child.pages.assign(parent.pages.begin(), parent.pages.begin() + full);
  for (int32_t p : child.pages)
    if (p >= 0) ++refcnt_[p];  // -1: a page the window dropped
  if (rem != 0) {
    int32_t np = AllocPage();
    QueueCopy(parent.pages[full], np);
    child.pages.push_back(np);
  }
  child.len = fork_pos;
  total_len_ += fork_pos;
  seqs_[child_id] = std::move(child);
  pending_forks_.push_back(parent_id);
  pending_forks_.push_back(child_id);
}

void KVManager::RequeuePlanSideEffects(const ForwardPlan& plan) {
  std::vector<int32_t> again;
  for (size_t i = 0; i + 1 < plan.page_copies.size(); i += 2) {
    const int32_t src = plan.page_copies[i], dst = plan.page_copies[i + 1];
    if (refcnt_[dst] == 0) continue;  // its owner is gone
    if (refcnt_[src] == 0) {
      // free since the plan was made, untouched because the plan's forward never ran: take it back
      auto it = std::find(free_pages_.begin(), free_pages_.end(), src);
      if (it == free_pages_.end()) continue;  // cannot happen: a page without holders is on the free list
      free_pages_.erase(it);
      refcnt_[src] = 1;
    } else {
      ++refcnt_[src];
    }
    again.push_back(src);
    again.push_back(dst);
  }
  pending_copies_.insert(pending_copies_.begin(), again.begin(), again.end());
  pending_forks_.insert(pending_forks_.begin(), plan.seq_forks.begin(), plan.seq_forks.end());
}

void KVManager::RemoveSequence(int64_t seq_id) {
  Seq& s = Get(seq_id);
  for (int32_t p : s.pages) ReleasePage(p);
  total_len_ -= s.len;
  seqs_.erase(seq_id);
}

void KVManager::PopN(int64_t seq_id, int64_t n) {
  Seq& s = Get(seq_id);
  if (n < 0 || n > s.len) throw std::runtime_error("KVManager: bad popn");
  s.len -= n;
  total_len_ -= n;
  const int64_t need = (s.len + page_size_ - 1) / page_size_;
  while (static_cast<int64_t>(s.pages.size()) > need) {
    ReleasePage(s.pages.back());
    s.pages.pop_back();
  }
  // a shared last page must not be appended into: give the sequence a private copy
  if (!s.pages.empty() && s.len % page_size_ != 0 && s.pages.back() >= 0 &&
      refcnt_[s.pages.back()] > 1) {
    int32_t np = AllocPage();
    QueueCopy(s.pages.back(), np);
    ReleasePage(s.pages.back());
    s.pages.back() = np;
  }
}

void KVManager::EnableSlidingWindow(int64_t seq_id, int32_t window, int32_t sink) {
  Seq& s = Get(seq_id);
  s.window = window;
  s.sink = sink;
}

int64_t KVManager::SequenceLength(int64_t seq_id) const { return Get(seq_id).len; }

std::vector<int32_t> KVManager::SequencePages(int64_t seq_id) const { return Get(seq_id).pages; }

int64_t KVManager::PagesNeeded(int64_t seq_id, int64_t n) const {
  auto it = seqs_.find(seq_id);
  int64_t len = it == seqs_.end() ? 0 : it->second.len;
  int64_t have = it == seqs_.end() ? 0 : static_cast<int64_t>(it->second.pages.size());
  int64_t need = (len + n + page_size_ - 1) / page_size_;
  return std::max<int64_t>(0, need - have);
}

void KVManager::TrimWindow(Seq& s, int64_t first_new_pos) {
  if (s.window <= 0) return;
  // the first token of the chunk being appended still sees `window` positions ending at itself: only what
  // lies below that (and is no sink) is dead for every token of the chunk
  const int64_t first_visible = first_new_pos + 1 - s.window;
  if (first_visible <= s.sink) return;
  const int64_t first_page = (s.sink + page_size_ - 1) / page_size_;
  const int64_t end_page = first_visible / page_size_;  // pages entirely below first_visible
  for (int64_t p = std::max<int64_t>(first_page, s.dropped_until / page_size_); p < end_page; ++p) {
    if (s.pages[p] >= 0) {
      ReleasePage(s.pages[p]);
      s.pages[p] = -1;
    }
  }
  s.dropped_until = std::max<int64_t>(s.dropped_until, end_page * page_size_);
}

ForwardPlan KVManager::BeginForward(const std::vector<int64_t>& seq_ids,
                                    const std::vector<int32_t>& append_lens,
                                    const std::vector<int32_t>* tree_parents) {
  if (seq_ids.size() != append_lens.size()) throw std::runtime_error("KVManager: length mismatch");
  // check capacity first so a failure leaves the state untouched
  int64_t need_pages = 0;
  for (size_t i = 0; i < seq_ids.size(); ++i) need_pages += PagesNeeded(seq_ids[i], append_lens[i]);
  if (need_pages > NumAvailablePages()) throw std::runtime_error("KVManager: out of KV pages");

  ForwardPlan plan;
  plan.seq_ids = seq_ids;
  plan.append_lens = append_lens;
  plan.page_indptr.push_back(0);
  plan.q_indptr.push_back(0);
  plan.page_copies.swap(pending_copies_);
  plan.seq_forks.swap(pending_forks_);
  // the sources stay intact until this plan's copy launch: whatever takes such a page from now on writes to it
  // later in stream order
  for (size_t i = 0; i + 1 < plan.page_copies.size(); i += 2) ReleasePage(plan.page_copies[i]);
  bool any_window = false;
  for (int64_t id : seq_ids) any_window |= Get(id).window > 0;
  size_t tree_off = 0;
  for (size_t i = 0; i < seq_ids.size(); ++i) {
    Seq& s = Get(seq_ids[i]);
    const int32_t n = append_lens[i];
    const int64_t base = s.len;
    const int64_t need = (base + n + page_size_ - 1) / page_size_;
    while (static_cast<int64_t>(s.pages.size()) < need) s.pages.push_back(AllocPage());
    std::vector<int32_t> depth(n, 0);
    if (tree_parents) {
      if (n > 64) throw std::runtime_error("KVManager: token tree larger than 64 nodes");
      for (int32_t j = 0; j < n; ++j) {
        int32_t par = (*tree_parents)[tree_off + j];
        if (par >= j) throw std::runtime_error("KVManager: tree parents must precede children");
        depth[j] = par < 0 ? 0 : depth[par] + 1;
      }
    }
    std::vector<uint64_t> masks(tree_parents ? n : 0, 0);
    for (int32_t j = 0; j < n; ++j) {
      const int64_t slot_pos = base + j;
      const int32_t page = s.pages[slot_pos / page_size_];
      plan.slots.push_back(page * page_size_ + static_cast<int32_t>(slot_pos % page_size_));
      plan.q_seq.push_back(static_cast<int32_t>(i));
      if (tree_parents) {
        int32_t par = (*tree_parents)[tree_off + j];
        masks[j] = (par < 0 ? 0ull : masks[par]) | (1ull << j);
        plan.positions.push_back(static_cast<int32_t>(base + depth[j]));
        plan.q_kvlen.push_back(static_cast<int32_t>(base));
        plan.tree_mask.push_back(masks[j]);
      } else {
        plan.positions.push_back(static_cast<int32_t>(slot_pos));
        plan.q_kvlen.push_back(static_cast<int32_t>(slot_pos + 1));
      }
      if (any_window) {
        int64_t start = s.window > 0 ? std::max<int64_t>(0, slot_pos + 1 - s.window) : 0;
        plan.q_kvstart.push_back(static_cast<int32_t>(start));
      }
    }
    tree_off += n;
    s.len += n;
    total_len_ += n;
    if (!tree_parents) TrimWindow(s, base);
    plan.seq_lens.push_back(static_cast<int32_t>(s.len));
    plan.page_indices.insert(plan.page_indices.end(), s.pages.begin(), s.pages.end());
    plan.page_indptr.push_back(static_cast<int32_t>(plan.page_indices.size()));
    plan.q_indptr.push_back(static_cast<int32_t>(plan.slots.size()));
    plan.max_append = std::max(plan.max_append, n);
    plan.max_seq_len = std::max<int32_t>(plan.max_seq_len, static_cast<int32_t>(s.len));
  }
  return plan;
}

std::vector<int32_t> KVManager::CommitTreeNodes(int64_t seq_id, int32_t num_appended,
                                                const std::vector<int32_t>& accepted) {
  Seq& s = Get(seq_id);
  if (num_appended > s.len || static_cast<int32_t>(accepted.size()) > num_appended)
    throw std::runtime_error("KVManager: bad tree commit");
  const int64_t base = s.len - num_appended;
  std::vector<int32_t> moves;
  for (size_t i = 0; i < accepted.size(); ++i) {
    const int64_t src = base + accepted[i], dst = base + static_cast<int64_t>(i);
    if (accepted[i] < static_cast<int32_t>(i) || accepted[i] >= num_appended)
      throw std::runtime_error("KVManager: accepted nodes must be increasing tree indices");
    if (src != dst) {
      moves.push_back(s.pages[src / page_size_] * page_size_ + static_cast<int32_t>(src % page_size_));
      moves.push_back(s.pages[dst / page_size_] * page_size_ + static_cast<int32_t>(dst % page_size_));
    }
  }
  PopN(seq_id, num_appended - static_cast<int64_t>(accepted.size()));
  return moves;
}

}  // namespace mlcb
