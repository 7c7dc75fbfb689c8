#include "radix_tree.h"

#include <algorithm>
#include <stdexcept>
#include <string>

namespace mlcb {

RadixTree::RadixTree(int64_t max_blocks) : root_(new Node()), max_blocks_(max_blocks) {}

RadixTree::~RadixTree() { FreeSubtree(root_); }

void RadixTree::FreeSubtree(Node* n) {
  for (auto& kv : n->children) FreeSubtree(kv.second);
  delete n;
}

void RadixTree::Reset() {
  FreeSubtree(root_);
  root_ = new Node();
  seq_node_.clear();
  used_blocks_ = 0;
}

void RadixTree::Resize(Node* n, size_t new_len) {
  int64_t delta = BlocksFor(new_len) - BlocksFor(n->tokens.size());
  if (used_blocks_ + delta > max_blocks_) throw std::runtime_error("RadixTree: out of capacity");
  used_blocks_ += delta;
}

RadixTree::Node* RadixTree::SplitAt(Node* n, size_t offset) {
  if (offset == 0 || offset >= n->tokens.size()) throw std::runtime_error("RadixTree: bad split");
  Node* lower = new Node();
  lower->tokens.assign(n->tokens.begin() + offset, n->tokens.end());
  lower->parent = n;
  lower->children.swap(n->children);
  for (auto& kv : lower->children) kv.second->parent = lower;
  lower->seqs.swap(n->seqs);
  for (int64_t s : lower->seqs) seq_node_[s] = lower;
  lower->depth_begin = n->depth_begin + static_cast<int64_t>(offset);
  int64_t before = BlocksFor(n->tokens.size());
  int64_t after = BlocksFor(offset) + BlocksFor(lower->tokens.size());
  if (used_blocks_ + after - before > max_blocks_) {
    // undo
    n->children.swap(lower->children);
    for (auto& kv : n->children) kv.second->parent = n;
    n->seqs.swap(lower->seqs);
    for (int64_t s : n->seqs) seq_node_[s] = n;
    delete lower;
    throw std::runtime_error("RadixTree: out of capacity");
  }
  used_blocks_ += after - before;
  n->tokens.resize(offset);
  n->children[lower->tokens[0]] = lower;
  return n;
}

void RadixTree::TryMergeWithChild(Node* n) {
  if (n == root_ || !n->seqs.empty() || n->children.size() != 1) return;
  Node* c = n->children.begin()->second;
  int64_t before = BlocksFor(n->tokens.size()) + BlocksFor(c->tokens.size());
  n->tokens.insert(n->tokens.end(), c->tokens.begin(), c->tokens.end());
  used_blocks_ += BlocksFor(n->tokens.size()) - before;
  n->children.clear();
  n->children.swap(c->children);
  for (auto& kv : n->children) kv.second->parent = n;
  n->seqs.swap(c->seqs);
  for (int64_t s : n->seqs) seq_node_[s] = n;
  delete c;
}

void RadixTree::Cleanup(Node* n) {
  while (n != root_ && n->seqs.empty() && n->children.empty()) {
    Node* parent = n->parent;
    parent->children.erase(n->tokens[0]);
    used_blocks_ -= BlocksFor(n->tokens.size());
    delete n;
    n = parent;
  }
  TryMergeWithChild(n);
}

void RadixTree::CollectSeqs(const Node* n, std::vector<int64_t>* out) const {
  for (int64_t s : n->seqs) out->push_back(s);
  for (auto& kv : n->children) CollectSeqs(kv.second, out);
}

std::pair<int64_t, std::vector<int64_t>> RadixTree::Match(const std::vector<int32_t>& tokens) const {
  const Node* cur = root_;
  size_t i = 0;
  while (i < tokens.size()) {
    auto it = cur->children.find(tokens[i]);
    if (it == cur->children.end()) break;
    const Node* c = it->second;
    size_t common = 0;
    size_t lim = std::min(c->tokens.size(), tokens.size() - i);
    while (common < lim && c->tokens[common] == tokens[i + common]) ++common;
    i += common;
    cur = c;
    if (common < c->tokens.size()) break;
  }
  std::vector<int64_t> seqs;
  if (i > 0) CollectSeqs(cur, &seqs);
  std::sort(seqs.begin(), seqs.end());
  return {static_cast<int64_t>(i), seqs};
}

void RadixTree::Add(int64_t seq_id) {
  if (seq_node_.count(seq_id)) throw std::runtime_error("RadixTree: sequence already exists");
  root_->seqs.insert(seq_id);
  seq_node_[seq_id] = root_;
}

void RadixTree::Remove(int64_t seq_id) {
  auto it = seq_node_.find(seq_id);
  if (it == seq_node_.end()) throw std::runtime_error("RadixTree: unknown sequence");
  Node* n = it->second;
  n->seqs.erase(seq_id);
  seq_node_.erase(it);
  Cleanup(n);
}

void RadixTree::Extend(int64_t seq_id, const std::vector<int32_t>& tokens) {
  auto it = seq_node_.find(seq_id);
  if (it == seq_node_.end()) throw std::runtime_error("RadixTree: unknown sequence");
  if (tokens.empty()) return;
  Node* n = it->second;
  if (n != root_ && n->seqs.size() == 1 && n->children.empty()) {
    Resize(n, n->tokens.size() + tokens.size());
    n->tokens.insert(n->tokens.end(), tokens.begin(), tokens.end());
    return;
  }
  Node* origin = n;
  Node* cur = n;
  size_t i = 0;
  while (i < tokens.size()) {
    auto cit = cur->children.find(tokens[i]);
    if (cit == cur->children.end()) {
      Node* leaf = new Node();
      int64_t need = BlocksFor(tokens.size() - i);
      if (used_blocks_ + need > max_blocks_) {
        delete leaf;
        throw std::runtime_error("RadixTree: out of capacity");
      }
      used_blocks_ += need;
      leaf->tokens.assign(tokens.begin() + i, tokens.end());
      leaf->parent = cur;
      leaf->depth_begin = cur->depth_begin + static_cast<int64_t>(cur->tokens.size());
      cur->children[leaf->tokens[0]] = leaf;
      cur = leaf;
      i = tokens.size();
      break;
    }
    Node* c = cit->second;
    size_t common = 0;
    size_t lim = std::min(c->tokens.size(), tokens.size() - i);
    while (common < lim && c->tokens[common] == tokens[i + common]) ++common;
    if (common < c->tokens.size()) SplitAt(c, common);
    cur = c;
    i += common;
  }
  origin->seqs.erase(seq_id);
  cur->seqs.insert(seq_id);
  seq_node_[seq_id] = cur;
  if (origin != cur) {
    // `origin` is an ancestor of `cur`, so it still has a child and cannot be deleted; it can only
    // have become mergeable with a single child.
    TryMergeWithChild(origin);
  }
}

int64_t RadixTree::GetLength(int64_t seq_id) const {
  auto it = seq_node_.find(seq_id);
  if (it == seq_node_.end()) throw std::runtime_error("RadixTree: unknown sequence");
  return it->second->depth_begin + static_cast<int64_t>(it->second->tokens.size());
}

std::vector<int32_t> RadixTree::Get(int64_t seq_id) const {
  auto it = seq_node_.find(seq_id);
  if (it == seq_node_.end()) throw std::runtime_error("RadixTree: unknown sequence");
  std::vector<const Node*> path;
  for (const Node* n = it->second; n != nullptr; n = n->parent) path.push_back(n);
  std::vector<int32_t> out;
  out.reserve(static_cast<size_t>(GetLength(seq_id)));
  for (auto p = path.rbegin(); p != path.rend(); ++p)
    out.insert(out.end(), (*p)->tokens.begin(), (*p)->tokens.end());
  return out;
}

void RadixTree::Fork(int64_t seq_id, int64_t parent_seq_id, int64_t forked_offset) {
  if (seq_node_.count(seq_id)) throw std::runtime_error("RadixTree: sequence already exists");
  auto it = seq_node_.find(parent_seq_id);
  if (it == seq_node_.end()) throw std::runtime_error("RadixTree: unknown parent sequence");
  int64_t len = GetLength(parent_seq_id);
  if (forked_offset < 0 || forked_offset > len) throw std::runtime_error("RadixTree: bad fork offset");
  Node* n = it->second;
  while (n != root_ && n->depth_begin >= forked_offset) n = n->parent;
  // now n == root (offset 0) or depth_begin < offset <= depth_begin + len(n)
  if (n != root_) {
    size_t off = static_cast<size_t>(forked_offset - n->depth_begin);
    if (off < n->tokens.size()) SplitAt(n, off);
  }
  n->seqs.insert(seq_id);
  seq_node_[seq_id] = n;
}

void RadixTree::Rollback(int64_t seq_id, int64_t num_tokens) {
  auto it = seq_node_.find(seq_id);
  if (it == seq_node_.end()) throw std::runtime_error("RadixTree: unknown sequence");
  if (num_tokens == 0) return;
  int64_t len = GetLength(seq_id);
  if (num_tokens < 0 || num_tokens > len) throw std::runtime_error("RadixTree: bad rollback length");
  int64_t target = len - num_tokens;
  Node* origin = it->second;
  Node* n = origin;
  while (n != root_ && n->depth_begin >= target) n = n->parent;
  origin->seqs.erase(seq_id);
  if (n != root_) {
    size_t off = static_cast<size_t>(target - n->depth_begin);
    if (off < n->tokens.size()) SplitAt(n, off);
  }
  n->seqs.insert(seq_id);
  seq_node_[seq_id] = n;
  // `origin` may have been replaced by the lower half of a split (its seqs moved there); find the
  // deepest node on the old path that is now dead and clean upward from it.
  Node* dead = origin;
  if (origin == n && !n->children.empty()) {
    // split happened on origin itself: the lower half is the single child created by SplitAt
    auto cit = n->children.begin();
    for (; cit != n->children.end(); ++cit)
      if (cit->second->seqs.empty() && cit->second->children.empty()) break;
    if (cit != n->children.end()) dead = cit->second;
  }
  if (dead != n) Cleanup(dead);
}

}  // namespace mlcb
