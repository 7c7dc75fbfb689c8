// Host-side manager of the paged KV cache: page table, reference-counted pages shared between
// forked sequences, copy-on-write of a partially filled last page, trailing-token pop, sliding
// window with attention sinks, token-tree append + commit, and the per-step index arrays the
// attention / append kernels consume.
//
// The device memory itself ([layers, pages, 2, kv_heads, page, head_dim]) is owned by the model
// executor; this class only hands out page numbers and lists the device copies the executor must
// perform (page copies for copy-on-write, token moves for tree commit).
//
// Behavioural counterpart: the PagedKVCache of the reference's runtime as driven by
// cpp/serve/model.cc:852-999 (add / fork / remove / popn / begin_forward / commit tree nodes /
// sliding window / available pages / total length).
#pragma once
#include <cstdint>
#include <stdexcept>
#include <unordered_map>
#include <utility>
#include <vector>

namespace mlcb {

struct ForwardPlan {
  // per sequence in the batch
  std::vector<int64_t> seq_ids;
  std::vector<int32_t> append_lens;
  std::vector<int32_t> seq_lens;      // length after the append
  std::vector<int32_t> page_indptr;   // [B+1]
  std::vector<int32_t> page_indices;  // pages of each sequence, -1 for pages dropped by the window
  std::vector<int32_t> q_indptr;      // [B+1] token offsets
  // per appended token
  std::vector<int32_t> positions;
  std::vector<int32_t> slots;         // page * page_size + offset
  std::vector<int32_t> q_seq;         // batch slot
  std::vector<int32_t> q_kvlen;       // causal visibility (positions < q_kvlen are visible)
  std::vector<int32_t> q_kvstart;     // sliding-window start (empty when no sequence uses a window)
  std::vector<uint64_t> tree_mask;    // ancestor bit masks (empty unless a token tree is appended)
  // device copies to run before the forward: (src_page, dst_page) pairs
  std::vector<int32_t> page_copies;
  // (parent id, child id) of every fork since the last plan: models that keep a recurrent state per sequence
  // copy the parent's state to the child before the forward
  std::vector<int64_t> seq_forks;
  int32_t max_append = 0;
  int32_t max_seq_len = 0;
};

class KVManager {
 public:
  KVManager(int64_t num_pages, int page_size, int64_t max_num_sequence);

  void Clear();
  void AddSequence(int64_t seq_id);
  // child shares the first fork_pos tokens of parent (fork_pos < 0: the whole parent).
  void ForkSequence(int64_t parent_id, int64_t child_id, int64_t fork_pos);
  void RemoveSequence(int64_t seq_id);
  void PopN(int64_t seq_id, int64_t n);
  void EnableSlidingWindow(int64_t seq_id, int32_t window, int32_t sink);
  bool Has(int64_t seq_id) const { return seqs_.count(seq_id) != 0; }
  int64_t SequenceLength(int64_t seq_id) const;

  // Reserves room for `append_lens[i]` tokens of sequence i and returns the index arrays.
  // `tree_parents` (optional, concatenated per sequence, -1 = child of the last committed token)
  // turns the append into a token-tree append: positions follow tree depth and visibility inside
  // the appended chunk follows ancestry.
  ForwardPlan BeginForward(const std::vector<int64_t>& seq_ids,
                           const std::vector<int32_t>& append_lens,
                           const std::vector<int32_t>* tree_parents = nullptr);
  // After a tree append of `n` nodes, keep only `accepted` (node indices inside the chunk, in path
  // order). Returns (src_slot, dst_slot) token moves the executor must apply to every layer.
  std::vector<int32_t> CommitTreeNodes(int64_t seq_id, int32_t num_appended,
                                       const std::vector<int32_t>& accepted);

  // Pages needed to append n tokens to the sequence right now.
  int64_t PagesNeeded(int64_t seq_id, int64_t n) const;
  int64_t NumAvailablePages() const { return static_cast<int64_t>(free_pages_.size()); }
  int64_t TotalSequenceLength() const { return total_len_; }
  int64_t NumPages() const { return num_pages_; }
  int PageSize() const { return page_size_; }
  int64_t NumSequences() const { return static_cast<int64_t>(seqs_.size()); }
  // Device copies queued by ForkSequence (copy-on-write), drained by the next BeginForward.
  const std::vector<int32_t>& pending_copies() const { return pending_copies_; }
  // A plan whose forward will not run after all (its appended tokens are popped by the caller): the page copies
  // and forks it carried still have to reach the model with the next plan.
  void RequeuePlanSideEffects(const ForwardPlan& plan);
  // Export / import of a sequence's page list (prefill/decode disaggregation).
  std::vector<int32_t> SequencePages(int64_t seq_id) const;

 private:
  struct Seq {
    std::vector<int32_t> pages;
    int64_t len = 0;
    int32_t window = 0;  // 0 = no sliding window
    int32_t sink = 0;
    int64_t dropped_until = 0;  // positions [sink_pages_end, dropped_until) have been released
  };
  int32_t AllocPage();
  void ReleasePage(int32_t p);
  void QueueCopy(int32_t src, int32_t dst);
  void TrimWindow(Seq& s, int64_t first_new_pos);
  Seq& Get(int64_t id);
  const Seq& Get(int64_t id) const;

  int64_t num_pages_;
  int page_size_;
  int64_t max_num_sequence_;
  std::vector<int32_t> free_pages_;
  std::vector<int32_t> refcnt_;
  std::unordered_map<int64_t, Seq> seqs_;
  std::vector<int32_t> pending_copies_;
  std::vector<int64_t> pending_forks_;
  int64_t total_len_ = 0;
};

}  // namespace mlcb
