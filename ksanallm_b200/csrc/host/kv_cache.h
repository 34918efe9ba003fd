// Paged KV block manager with a prefix tree (radix tree over full blocks).
//
// Capability parity with the reference's PrefixCacheManager / DirectCacheManager /
// BlockAllocator (src/ksana_llm/cache_manager/prefix_cache_manager.cpp:109-155, 479-550,
// 607-640, 837-1008; block_allocator/block_allocator.cpp:41-83), redesigned:
//   * blocks are plain integer ids into per-layer device pools [layer][block][...], so the
//     manager never touches device pointers;
//   * a tree node is keyed by (parent node, token ids of one full block); identical blocks
//     committed by two requests are merged (the later request adopts the earlier node);
//   * unreferenced nodes stay cached and are evicted leaf-first in LRU order;
//   * swap-out/in is pure bookkeeping here: the caller receives (device, host) copy pairs and
//     executes them on its copy stream.
#pragma once
#include <algorithm>
#include <cstdint>
#include <deque>
#include <list>
#include <map>
#include <memory>
#include <set>
#include <stdexcept>
#include <unordered_map>
#include <utility>
#include <vector>

namespace ksana {

using BlockId = int32_t;

// Plain free-list allocator with reference counts. One instance per memory tier.
class BlockAllocator {
 public:
  explicit BlockAllocator(int num_blocks) : ref_(num_blocks, 0) {
    for (int i = 0; i < num_blocks; ++i) free_.push_back(i);
  }
  int num_total() const { return static_cast<int>(ref_.size()); }
  int num_free() const { return static_cast<int>(free_.size()); }
  bool Alloc(BlockId* out) {
    if (free_.empty()) return false;
    *out = free_.front();
    free_.pop_front();
    ref_[*out] = 1;
    return true;
  }
  void AddRef(BlockId b) { ++ref_.at(b); }
  int RefCount(BlockId b) const { return ref_.at(b); }
  // Returns true when the block went back to the free list.
  bool Release(BlockId b) {
    int& r = ref_.at(b);
    if (r <= 0) throw std::runtime_error("BlockAllocator: double free of block");
    if (--r == 0) {
      free_.push_back(b);
      return true;
    }
    return false;
  }

 private:
  std::vector<int> ref_;
  std::deque<BlockId> free_;
};

struct PrefixNode {
  PrefixNode* parent = nullptr;
  BlockId block = -1;
  std::vector<int32_t> tokens;  // exactly block_size tokens
  uint64_t key = 0;             // hash(parent key, tokens)
  int active_refs = 0;          // requests currently holding this node
  uint64_t last_use = 0;        // LRU tick
  std::multimap<uint64_t, PrefixNode*> children;  // key -> node (collisions resolved by compare)
};

struct CopyPair {
  BlockId src;
  BlockId dst;
};

// Per-request view of the cache.
struct SeqBlocks {
  std::vector<PrefixNode*> shared;  // leading full blocks that live in the tree
  std::vector<BlockId> own;         // private blocks after the shared ones
  std::vector<BlockId> host;        // host copies while swapped out (own blocks only)
  bool swapped = false;
  bool no_commit = false;  // blocks never enter the prefix tree (token ids do not determine the KV: spliced embeddings)
  int NumBlocks() const { return static_cast<int>(shared.size() + own.size()); }
};

struct CacheStats {
  int64_t prefix_query_tokens = 0;
  int64_t prefix_hit_tokens = 0;
  int64_t evicted_blocks = 0;
  int64_t merged_blocks = 0;
  int64_t swapped_out_blocks = 0;
  int64_t swapped_in_blocks = 0;
  int64_t flexible_hit_tokens = 0;
};

// Result of KVCacheManager::FlexibleReserve: token i of the run has its KV copied from cache slot src_slots[i]
// (written at position src_pos[i]) to slot dst_slots[i] (position dst_begin + i).
struct FlexibleRun {
  int dst_begin = 0;
  std::vector<int32_t> src_slots, dst_slots, src_pos;
  int size() const { return static_cast<int>(src_slots.size()); }
};

class KVCacheManager {
 public:
  KVCacheManager(int num_device_blocks, int num_host_blocks, int block_size, bool enable_prefix)
      : dev_(num_device_blocks), host_(num_host_blocks), block_size_(block_size), prefix_(enable_prefix) {
    root_.key = 0x9E3779B97F4A7C15ull;
  }
  ~KVCacheManager() { FreeSubtree(&root_); }

  int block_size() const { return block_size_; }
  bool prefix_enabled() const { return prefix_; }
  int num_device_blocks() const { return dev_.num_total(); }
  int num_host_blocks() const { return host_.num_total(); }
  int num_free_host_blocks() const { return host_.num_free(); }
  // Blocks obtainable right now: truly free + cached-but-unreferenced (evictable).
  int num_available_blocks() const { return dev_.num_free() + evictable_; }
  int num_free_blocks() const { return dev_.num_free(); }
  int num_cached_blocks() const { return cached_nodes_; }
  const CacheStats& stats() const { return stats_; }

  bool Has(int64_t seq) const { return seqs_.count(seq) != 0; }

  // Longest cached prefix (in tokens, multiple of block_size) for `tokens`, never covering the
  // whole sequence: at least one token is always left to compute so that logits exist.
  int MatchPrefix(const std::vector<int32_t>& tokens) {
    if (!prefix_) return 0;
    int n = 0;
    PrefixNode* cur = &root_;
    const int max_full = (static_cast<int>(tokens.size()) - 1) / block_size_;
    for (int b = 0; b < max_full; ++b) {
      PrefixNode* nxt = FindChild(cur, tokens.data() + b * block_size_);
      if (!nxt) break;
      cur = nxt;
      ++n;
    }
    return n * block_size_;
  }

  // Registers a sequence and pins its cached prefix. Returns number of prefix tokens reused.
  int CreateSeq(int64_t seq, const std::vector<int32_t>& tokens, bool use_prefix = true) {
    if (seqs_.count(seq)) throw std::runtime_error("KVCacheManager: duplicate seq");
    SeqBlocks& sb = seqs_[seq];
    sb.no_commit = !use_prefix;
    stats_.prefix_query_tokens += static_cast<int64_t>(tokens.size());
    if (!prefix_ || !use_prefix) return 0;
    PrefixNode* cur = &root_;
    const int max_full = (static_cast<int>(tokens.size()) - 1) / block_size_;
    for (int b = 0; b < max_full; ++b) {
      PrefixNode* nxt = FindChild(cur, tokens.data() + b * block_size_);
      if (!nxt) break;
      Pin(nxt);
      sb.shared.push_back(nxt);
      cur = nxt;
    }
    int hit = static_cast<int>(sb.shared.size()) * block_size_;
    stats_.prefix_hit_tokens += hit;
    return hit;
  }

  // Makes sure the sequence owns enough blocks for `num_tokens` tokens in total.
  // All-or-nothing: on failure nothing changes and false is returned.
  bool EnsureCapacity(int64_t seq, int num_tokens) {
    SeqBlocks& sb = seqs_.at(seq);
    int need = (num_tokens + block_size_ - 1) / block_size_ - sb.NumBlocks();
    if (need <= 0) return true;
    if (need > num_available_blocks()) return false;
    for (int i = 0; i < need; ++i) {
      BlockId b;
      if (!dev_.Alloc(&b)) {
        if (!EvictOne()) throw std::runtime_error("KVCacheManager: accounting error in eviction");
        if (!dev_.Alloc(&b)) throw std::runtime_error("KVCacheManager: eviction freed no block");
      }
      sb.own.push_back(b);
    }
    return true;
  }

  // After `num_computed` tokens of `tokens` have valid KV, moves newly filled private blocks into
  // the tree (merging with an identical cached block when one exists). Returned pairs are
  // (dropped private block -> adopted cached block): no copy is needed, the block table simply
  // changes; the caller may use them for checksums or tracing.
  std::vector<CopyPair> CommitFilled(int64_t seq, const std::vector<int32_t>& tokens, int num_computed) {
    std::vector<CopyPair> merged;
    if (!prefix_) return merged;
    SeqBlocks& sb = seqs_.at(seq);
    if (sb.no_commit) return merged;
    int full = num_computed / block_size_;
    while (static_cast<int>(sb.shared.size()) < full && !sb.own.empty()) {
      int bidx = static_cast<int>(sb.shared.size());
      PrefixNode* parent = sb.shared.empty() ? &root_ : sb.shared.back();
      const int32_t* tk = tokens.data() + bidx * block_size_;
      PrefixNode* hit = FindChild(parent, tk);
      BlockId mine = sb.own.front();
      if (hit) {
        Pin(hit);
        merged.push_back({mine, hit->block});
        dev_.Release(mine);
        ++stats_.merged_blocks;
        sb.shared.push_back(hit);
      } else {
        auto* node = new PrefixNode();
        node->parent = parent;
        node->block = mine;
        node->tokens.assign(tk, tk + block_size_);
        node->key = HashBlock(parent->key, tk);
        node->active_refs = 1;
        node->last_use = ++tick_;
        parent->children.emplace(node->key, node);
        by_tokens_.emplace(HashBlock(0, tk), node);
        ++cached_nodes_;
        sb.shared.push_back(node);
      }
      sb.own.erase(sb.own.begin());
    }
    return merged;
  }

  // Flexible (non-prefix) reuse, the reference's min_flexible_cache_num feature
  // (cache_manager/prefix_cache_manager.cpp:254-389): after the cached prefix of `shared` tokens, the tokens that
  // follow may already sit in the tree at OTHER positions (a dialogue whose middle changed length). Looks for the
  // longest run of cached full blocks whose tokens equal tokens[shared ...] - the run may start inside a block, up
  // to block_size - 1 tokens late, in which case the tail of that block's parent must match too - and, when it is
  // at least `min_len` tokens long, reserves the sequence's blocks for it and returns the per-token copy list.
  // Keys need their rotary phase moved from src_pos to the new position by the caller. At least one token of the
  // sequence is always left to compute.
  bool FlexibleReserve(int64_t seq, const std::vector<int32_t>& tokens, int shared, int min_len, FlexibleRun* out) {
    if (!prefix_ || min_len <= 0 || shared % block_size_ != 0) return false;
    const int n = static_cast<int>(tokens.size());
    const int bs = block_size_;
    std::vector<PrefixNode*> best;
    int best_len = 0, best_lead = 0;
    for (int lead = 0; lead < bs; ++lead) {
      int offset = shared + lead;
      if (offset + bs >= n) break;
      auto range = by_tokens_.equal_range(HashBlock(0, tokens.data() + offset));
      for (auto it = range.first; it != range.second; ++it) {
        PrefixNode* node = it->second;
        if (!std::equal(node->tokens.begin(), node->tokens.end(), tokens.begin() + offset)) continue;
        std::vector<PrefixNode*> chain;
        if (lead > 0) {
          PrefixNode* par = node->parent;
          if (par == nullptr || par == &root_) continue;
          if (!std::equal(par->tokens.end() - lead, par->tokens.end(), tokens.begin() + shared)) continue;
          chain.push_back(par);
        }
        chain.push_back(node);
        int hit = bs;
        PrefixNode* cur = node;
        while (offset + hit + bs < n) {
          PrefixNode* nxt = FindChild(cur, tokens.data() + offset + hit);
          if (!nxt) break;
          chain.push_back(nxt);
          cur = nxt;
          hit += bs;
        }
        if (lead + hit >= min_len && lead + hit > best_len) {
          best = chain;
          best_len = lead + hit;
          best_lead = lead;
        }
      }
    }
    if (best.empty()) return false;
    // the reservation below must not evict (and hand out) the source blocks; their ancestors are pinned with them,
    // because an unreferenced node above a referenced one counts as obtainable but can never be evicted
    std::vector<PrefixNode*> pinned;
    for (PrefixNode* a = best.front()->parent; a != nullptr && a != &root_; a = a->parent) pinned.push_back(a);
    std::reverse(pinned.begin(), pinned.end());  // root side first: released in the order a sequence would
    pinned.insert(pinned.end(), best.begin(), best.end());
    for (auto* nd : pinned) Pin(nd);
    bool ok = EnsureCapacity(seq, shared + best_len);
    for (auto* nd : pinned) Unpin(nd);
    if (!ok) return false;
    std::vector<BlockId> table = BlockTable(seq);
    int depth = 0;  // position of the first source block
    for (PrefixNode* a = best.front()->parent; a != nullptr && a != &root_; a = a->parent) ++depth;
    int src0 = depth * bs + (best_lead > 0 ? bs - best_lead : 0);
    out->dst_begin = shared;
    for (int i = 0; i < best_len; ++i) {
      int sp = src0 + i, dp = shared + i;
      PrefixNode* nd = best[sp / bs - depth];
      out->src_pos.push_back(sp);
      out->src_slots.push_back(nd->block * bs + sp % bs);
      out->dst_slots.push_back(table[dp / bs] * bs + dp % bs);
    }
    stats_.flexible_hit_tokens += best_len;
    return true;
  }

  // Block table in logical order.
  std::vector<BlockId> BlockTable(int64_t seq) const {
    const SeqBlocks& sb = seqs_.at(seq);
    std::vector<BlockId> out;
    out.reserve(sb.NumBlocks());
    for (auto* n : sb.shared) out.push_back(n->block);
    for (auto b : sb.own) out.push_back(b);
    return out;
  }
  int NumBlocks(int64_t seq) const { return seqs_.at(seq).NumBlocks(); }
  int NumHostBlocks(int64_t seq) const { return static_cast<int>(seqs_.at(seq).host.size()); }

  // Frees everything a sequence holds (cached nodes stay in the tree, unpinned).
  void FreeSeq(int64_t seq) {
    auto it = seqs_.find(seq);
    if (it == seqs_.end()) return;
    SeqBlocks& sb = it->second;
    for (auto* n : sb.shared) Unpin(n);
    for (auto b : sb.own) dev_.Release(b);
    for (auto b : sb.host) host_.Release(b);
    seqs_.erase(it);
  }

  // Drops trailing blocks so that exactly ceil(num_tokens / block_size) remain (used when draft
  // tokens were rejected, and by recompute pre-emption with num_tokens = 0).
  void Truncate(int64_t seq, int num_tokens) {
    SeqBlocks& sb = seqs_.at(seq);
    int keep = (num_tokens + block_size_ - 1) / block_size_;
    while (sb.NumBlocks() > keep) {
      if (!sb.own.empty()) {
        dev_.Release(sb.own.back());
        sb.own.pop_back();
      } else {
        Unpin(sb.shared.back());
        sb.shared.pop_back();
      }
    }
  }

  // Copy-on-write fork: the child shares the parent's tree blocks and gets private copies of the
  // parent's private blocks. Returns false (nothing changed) when there are not enough blocks.
  bool Fork(int64_t parent, int64_t child, std::vector<CopyPair>* copies) {
    if (seqs_.count(child)) throw std::runtime_error("KVCacheManager: duplicate seq in fork");
    const SeqBlocks& p = seqs_.at(parent);
    if (p.swapped) return false;
    if (static_cast<int>(p.own.size()) > num_available_blocks()) return false;
    SeqBlocks c;
    c.no_commit = p.no_commit;
    for (auto* n : p.shared) {
      Pin(n);
      c.shared.push_back(n);
    }
    for (auto b : p.own) {
      BlockId nb;
      if (!dev_.Alloc(&nb)) {
        EvictOne();
        if (!dev_.Alloc(&nb)) throw std::runtime_error("KVCacheManager: fork accounting error");
      }
      c.own.push_back(nb);
      copies->push_back({b, nb});
    }
    seqs_[child] = std::move(c);
    return true;
  }

  // Swap-out: private blocks go to host blocks; tree blocks stay pinned on the device (other
  // requests may share them). Returns false when the host tier is full.
  bool SwapOut(int64_t seq, std::vector<CopyPair>* copies) {
    SeqBlocks& sb = seqs_.at(seq);
    if (sb.swapped) return true;
    if (static_cast<int>(sb.own.size()) > host_.num_free()) return false;
    for (auto b : sb.own) {
      BlockId h;
      host_.Alloc(&h);
      copies->push_back({b, h});
      sb.host.push_back(h);
      dev_.Release(b);
      ++stats_.swapped_out_blocks;
    }
    sb.own.clear();
    sb.swapped = true;
    return true;
  }

  // Swap-in: needs the tree part to still be resident (pinned nodes never leave), then host
  // blocks come back into fresh device blocks. Returns false when memory is short.
  bool SwapIn(int64_t seq, std::vector<CopyPair>* copies) {
    SeqBlocks& sb = seqs_.at(seq);
    if (!sb.swapped) return true;
    if (static_cast<int>(sb.host.size()) > num_available_blocks()) return false;
    for (auto h : sb.host) {
      BlockId b;
      if (!dev_.Alloc(&b)) {
        EvictOne();
        if (!dev_.Alloc(&b)) throw std::runtime_error("KVCacheManager: swap-in accounting error");
      }
      copies->push_back({h, b});
      sb.own.push_back(b);
      host_.Release(h);
      ++stats_.swapped_in_blocks;
    }
    sb.host.clear();
    sb.swapped = false;
    return true;
  }

  // Test hook matching the reference's WITH_CLEAR_CACHE behaviour: drop every unreferenced node.
  int ClearUnreferenced() {
    int n = 0;
    while (EvictOne()) ++n;
    return n;
  }

 private:
  uint64_t HashBlock(uint64_t parent_key, const int32_t* tk) const {
    uint64_t h = parent_key ^ 0xcbf29ce484222325ull;
    for (int i = 0; i < block_size_; ++i) {
      h ^= static_cast<uint32_t>(tk[i]);
      h *= 0x100000001b3ull;
      h ^= h >> 29;
    }
    return h;
  }
  PrefixNode* FindChild(PrefixNode* parent, const int32_t* tk) const {
    uint64_t k = HashBlock(parent->key, tk);
    auto range = parent->children.equal_range(k);
    for (auto it = range.first; it != range.second; ++it) {
      PrefixNode* n = it->second;
      bool same = true;
      for (int i = 0; i < block_size_; ++i)
        if (n->tokens[i] != tk[i]) {
          same = false;
          break;
        }
      if (same) return n;
    }
    return nullptr;
  }
  void Pin(PrefixNode* n) {
    if (n->active_refs == 0) {
      --evictable_;
      lru_.erase({n->last_use, n});
    }
    ++n->active_refs;
    n->last_use = ++tick_;
  }
  void Unpin(PrefixNode* n) {
    if (--n->active_refs == 0) {
      n->last_use = ++tick_;
      ++evictable_;
      lru_.insert({n->last_use, n});
    }
  }
  // Evicts the least recently used unreferenced node that has no children. A parent's last_use is
  // never newer than its pinned descendants', and an unreferenced inner node with unreferenced
  // children is reached after they are gone, so scanning for the first leaf terminates quickly.
  bool EvictOne() {
    for (auto it = lru_.begin(); it != lru_.end(); ++it) {
      PrefixNode* n = it->second;
      if (!n->children.empty()) continue;
      lru_.erase(it);
      --evictable_;
      auto range = n->parent->children.equal_range(n->key);
      for (auto c = range.first; c != range.second; ++c)
        if (c->second == n) {
          n->parent->children.erase(c);
          break;
        }
      dev_.Release(n->block);
      --cached_nodes_;
      ++stats_.evicted_blocks;
      ForgetTokens(n);
      delete n;
      return true;
    }
    return false;
  }
  void ForgetTokens(PrefixNode* n) {
    auto range = by_tokens_.equal_range(HashBlock(0, n->tokens.data()));
    for (auto it = range.first; it != range.second; ++it)
      if (it->second == n) {
        by_tokens_.erase(it);
        return;
      }
  }
  void FreeSubtree(PrefixNode* n) {
    for (auto& kv : n->children) {
      FreeSubtree(kv.second);
      delete kv.second;
    }
    n->children.clear();
  }

  BlockAllocator dev_;
  BlockAllocator host_;
  int block_size_;
  bool prefix_;
  PrefixNode root_;
  std::unordered_map<int64_t, SeqBlocks> seqs_;
  std::set<std::pair<uint64_t, PrefixNode*>> lru_;
  std::unordered_multimap<uint64_t, PrefixNode*> by_tokens_;  // hash of a block's own tokens -> nodes (any depth)
  int evictable_ = 0;
  int cached_nodes_ = 0;
  uint64_t tick_ = 0;
  CacheStats stats_;
};

}  // namespace ksana
