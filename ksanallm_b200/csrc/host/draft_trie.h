// N-gram trie draft generator for speculative decoding without a draft model.
//
// Same capability as the reference's TrieGenerator
// (src/ksana_llm/runtime/draft_generator/trie_generator.{h,cpp}: frequency trie over the
// request's input and output tokens, bounded depth, suffix match then greedy walk), written as
// an incremental structure: every appended token advances a window of "open" paths, so feeding
// a token costs O(depth) instead of re-inserting all n-grams.
#pragma once
#include <cstdint>
#include <deque>
#include <memory>
#include <unordered_map>
#include <vector>

namespace ksana {

class DraftTrie {
 public:
  explicit DraftTrie(int max_depth = 16, int max_nodes = 1 << 18) : max_depth_(max_depth), max_nodes_(max_nodes) {
    nodes_.emplace_back();
  }

  void Feed(const std::vector<int32_t>& tokens) {
    for (auto t : tokens) FeedOne(t);
  }

  void FeedOne(int32_t tok) {
    history_.push_back(tok);
    if (static_cast<int>(history_.size()) > max_depth_) history_.pop_front();
    // every open path (one per start position within the window) is extended by `tok`
    open_.push_back(0);
    if (static_cast<int>(open_.size()) > max_depth_) open_.pop_front();
    for (auto& n : open_) {
      if (n < 0) continue;
      n = Child(n, tok, true);
    }
  }

  // Longest suffix match of length in [min_match, max_match], then follow the most frequent
  // continuation for up to `num_draft` tokens.
  std::vector<int32_t> Propose(int num_draft, int max_match = 4, int min_match = 1) const {
    std::vector<int32_t> out;
    if (num_draft <= 0) return out;
    int h = static_cast<int>(history_.size());
    for (int m = std::min(max_match, h); m >= min_match; --m) {
      int node = 0;
      bool ok = true;
      for (int i = h - m; i < h; ++i) {
        node = FindChild(node, history_[i]);
        if (node < 0) {
          ok = false;
          break;
        }
      }
      if (!ok || nodes_[node].children.empty()) continue;
      while (static_cast<int>(out.size()) < num_draft) {
        int best = -1, best_freq = 0;
        int32_t best_tok = 0;
        for (auto& kv : nodes_[node].children) {
          int f = nodes_[kv.second].freq;
          if (f > best_freq || (f == best_freq && kv.first < best_tok)) {
            best = kv.second;
            best_freq = f;
            best_tok = kv.first;
          }
        }
        if (best < 0) break;
        out.push_back(best_tok);
        node = best;
      }
      if (!out.empty()) return out;
    }
    return out;
  }

  int num_nodes() const { return static_cast<int>(nodes_.size()); }

 private:
  struct Node {
    int freq = 0;
    std::unordered_map<int32_t, int> children;
  };
  int FindChild(int node, int32_t tok) const {
    auto it = nodes_[node].children.find(tok);
    return it == nodes_[node].children.end() ? -1 : it->second;
  }
  int Child(int node, int32_t tok, bool create) {
    auto it = nodes_[node].children.find(tok);
    if (it != nodes_[node].children.end()) {
      ++nodes_[it->second].freq;
      return it->second;
    }
    if (!create || static_cast<int>(nodes_.size()) >= max_nodes_) return -1;
    int id = static_cast<int>(nodes_.size());
    nodes_.emplace_back();
    nodes_[id].freq = 1;
    nodes_[node].children[tok] = id;
    return id;
  }

  int max_depth_;
  int max_nodes_;
  std::vector<Node> nodes_;
  std::deque<int> open_;
  std::deque<int32_t> history_;
};

}  // namespace ksana
