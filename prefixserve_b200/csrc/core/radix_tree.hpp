// Prefix cache over whole cache pages: a tree in which every node stands for
// one full page of tokens and a path from the root spells a cached prefix.
//
// Behaviour follows the reference's tree (csrc/radix_tree.hpp:36-144,
// csrc/radix_tree.cpp:130-290 of PrefixServe):
//  * children are found by hashing all tokens of the page (NH: keyed sums of
//    products of token pairs) together with the parent, and every hit is verified by comparing parent and tokens, so two
//    siblings that start alike are never confused and correctness never rests
//    on the hash;
//  * match_prefix returns the longest cached prefix in whole pages and takes
//    one reference per returned page for the caller;
//  * insert is all-or-nothing, skips pages whose content is already cached
//    (the tree keeps its copy) and takes one reference per adopted page;
//  * evict removes least-recently-used leaves whose page nobody else holds; a
//    parent that loses its last child becomes a candidate in the same call;
//  * the destructor gives the tree's references back.
// Storage is laid out as parallel arrays sized once in the constructor
// (nodes = pages + 1, hash table = next power of two >= twice that), so no call
// allocates afterwards.  The page length in tokens is a run-time parameter.
#pragma once

#include <cstdint>
#include <string>
#include <vector>

#include "block_manager.hpp"

namespace psb200 {

class RadixTree {
 public:
  using Node = int32_t;

  RadixTree(BlockManager& pool, int32_t page_tokens, uint64_t seed);
  ~RadixTree();
  RadixTree(const RadixTree&) = delete;
  RadixTree& operator=(const RadixTree&) = delete;

  static uint64_t fresh_seed();

  // Longest cached prefix of tokens[0, n) in whole pages.  `out` is cleared and
  // receives the page ids; the caller owns one reference on each.  Returns the
  // number of matched tokens.
  int64_t match_prefix(const int32_t* tokens, int64_t n, std::vector<PageId>& out) noexcept;

  // Caches the full pages of tokens[0, n); pages[i] holds tokens
  // [i*page_tokens, (i+1)*page_tokens).  A partial last page is ignored.
  Code insert(const int32_t* tokens, int64_t n, const PageId* pages, int64_t num_pages, int32_t* added) noexcept;

  // Frees up to `want` pages, least recently used first.  Returns how many.
  int32_t evict(int32_t want) noexcept;

  int32_t num_cached_blocks() const noexcept { return capacity_ - 1 - static_cast<int32_t>(spare_.size()); }
  int32_t page_tokens() const noexcept { return page_tokens_; }
  int32_t max_blocks() const noexcept { return pool_.num_blocks(); }
  bool is_cached(PageId id) const noexcept { return pool_.in_range(id) && owned_[static_cast<size_t>(id)] != 0; }
  bool consistent(std::string* why) const;

 private:
  static constexpr Node kRoot = 0;
  static constexpr Node kNone = -1;

  uint64_t edge_hash(Node parent, const int32_t* toks) const noexcept;
  int64_t lookup(Node parent, const int32_t* toks, uint64_t h) const noexcept;
  void table_put(uint64_t h, Node n) noexcept;
  void table_remove(size_t at) noexcept;
  const int32_t* toks_of(Node n) const noexcept { return &tokens_[static_cast<size_t>(n) * static_cast<size_t>(page_tokens_)]; }
  void unlink_leaf(Node leaf) noexcept;

  // indexed binary min-heap of leaves by (stamp, node id)
  bool older(Node a, Node b) const noexcept {
    const uint64_t sa = stamp_[static_cast<size_t>(a)], sb = stamp_[static_cast<size_t>(b)];
    return sa != sb ? sa < sb : a < b;
  }
  void heap_set(size_t at, Node n) noexcept { heap_[at] = n; heap_at_[static_cast<size_t>(n)] = static_cast<int32_t>(at); }
  void heap_up(size_t at) noexcept;
  void heap_down(size_t at) noexcept;
  void heap_add(Node n) noexcept;
  void heap_drop(Node n) noexcept;

  BlockManager& pool_;
  int32_t page_tokens_;
  int32_t capacity_;
  uint64_t seed_;
  uint64_t clock_ = 0;

  // per node
  std::vector<Node> parent_;
  std::vector<PageId> page_;
  std::vector<int32_t> kids_;
  std::vector<int32_t> heap_at_;
  std::vector<uint64_t> stamp_;
  std::vector<uint64_t> hash_;
  std::vector<int32_t> tokens_;

  std::vector<Node> spare_;     // unused node ids
  std::vector<uint64_t> slot_hash_;
  std::vector<Node> slot_node_; // kNone = empty
  size_t mask_ = 0;
  std::vector<Node> heap_;
  std::vector<Node> held_back_; // evict() scratch
  std::vector<uint8_t> owned_;  // per page: a node owns it
  std::vector<uint32_t> keys_;  // per token position: secret key of the page hash
};

}  // namespace psb200
