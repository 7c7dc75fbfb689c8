// Radix tree over token-id sequences, the index behind the prefix cache.
//
// Every registered sequence id ends exactly at a node boundary; shared prefixes are stored once.
// Storage is accounted in fixed blocks of kBlockTokens tokens drawn from a bounded pool so that
// FreeCapacity() behaves like a paged allocator: removing what was added restores the capacity
// (nodes split by Fork/Extend are merged back when the reason for the split disappears).
//
// Behavioural counterpart: cpp/serve/radix_tree.cc:137-841 (Match / Fork / Extend / RollBack /
// Remove / FreeCapacity), exercised by tests/python/serve/test_radix_tree.py.
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <set>
#include <unordered_map>
#include <utility>
#include <vector>

namespace mlcb {

class RadixTree {
 public:
  static constexpr int kBlockTokens = 64;

  explicit RadixTree(int64_t max_blocks = 1 << 16);
  ~RadixTree();
  RadixTree(const RadixTree&) = delete;
  RadixTree& operator=(const RadixTree&) = delete;

  // Longest prefix of `tokens` present in the tree and the ids of all sequences sharing it.
  std::pair<int64_t, std::vector<int64_t>> Match(const std::vector<int32_t>& tokens) const;
  void Add(int64_t seq_id);
  void Remove(int64_t seq_id);
  void Extend(int64_t seq_id, const std::vector<int32_t>& tokens);
  void Rollback(int64_t seq_id, int64_t num_tokens);
  void Fork(int64_t seq_id, int64_t parent_seq_id, int64_t forked_offset);
  std::vector<int32_t> Get(int64_t seq_id) const;
  int64_t GetLength(int64_t seq_id) const;
  bool Has(int64_t seq_id) const { return seq_node_.count(seq_id) != 0; }
  int64_t FreeCapacity() const { return (max_blocks_ - used_blocks_) * kBlockTokens; }
  void Reset();

 private:
  struct Node {
    std::vector<int32_t> tokens;
    Node* parent = nullptr;
    std::map<int32_t, Node*> children;  // keyed by first token of the child
    std::set<int64_t> seqs;             // sequences ending at the end of this node
    int64_t depth_begin = 0;            // number of tokens on the path before this node
  };
  static int64_t BlocksFor(size_t n) { return static_cast<int64_t>((n + kBlockTokens - 1) / kBlockTokens); }
  void Resize(Node* n, size_t new_len);  // adjusts block accounting (throws when out of capacity)
  Node* SplitAt(Node* n, size_t offset);  // n keeps [0, offset); returns n (the upper part)
  void TryMergeWithChild(Node* n);
  void Cleanup(Node* n);
  void FixDepth(Node* n);
  void CollectSeqs(const Node* n, std::vector<int64_t>* out) const;
  void FreeSubtree(Node* n);

  Node* root_;
  std::unordered_map<int64_t, Node*> seq_node_;
  int64_t max_blocks_;
  int64_t used_blocks_ = 0;
};

}  // namespace mlcb
