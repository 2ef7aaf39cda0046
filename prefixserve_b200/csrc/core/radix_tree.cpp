#include "radix_tree.hpp"

#include <cstring>
#include <limits>
#include <random>

namespace psb200 {

namespace {

inline uint64_t scramble(uint64_t x) noexcept {
  x ^= x >> 32;
  x *= 0xd6e8feb86659fd93ULL;
  x ^= x >> 32;
  x *= 0xd6e8feb86659fd93ULL;
  x ^= x >> 32;
  return x;
}

size_t pow2_at_least(size_t v) noexcept {
  size_t p = 16;
  while (p < v) p <<= 1;
  return p;
}

}  // namespace

uint64_t RadixTree::fresh_seed() {
  std::random_device rd;
  return (static_cast<uint64_t>(rd()) << 32) ^ rd();
}

RadixTree::RadixTree(BlockManager& pool, int32_t page_tokens, uint64_t seed)
    : pool_(pool), page_tokens_(page_tokens), capacity_(pool.num_blocks() + 1), seed_(scramble(seed ^ 0x5851f42d4c957f2dULL)) {
  if (page_tokens < 1) throw std::invalid_argument("page_tokens must be >= 1");
  const size_t cap = static_cast<size_t>(capacity_);
  parent_.assign(cap, kNone);
  page_.assign(cap, kNoPage);
  kids_.assign(cap, 0);
  heap_at_.assign(cap, -1);
  stamp_.assign(cap, 0);
  hash_.assign(cap, 0);
  tokens_.assign(cap * static_cast<size_t>(page_tokens), 0);
  spare_.reserve(cap);
  for (Node n = capacity_ - 1; n >= 1; --n) spare_.push_back(n);
  const size_t slots = pow2_at_least(2 * cap);
  slot_hash_.assign(slots, 0);
  slot_node_.assign(slots, kNone);
  mask_ = slots - 1;
  heap_.reserve(cap);
  held_back_.reserve(cap);
  owned_.assign(static_cast<size_t>(pool.num_blocks()), 0);
  // one 32-bit key per token position of a page (an odd page length gets one more for its padding)
  uint64_t state = seed_;
  keys_.resize((static_cast<size_t>(page_tokens) + 1) & ~size_t{1});
  for (uint32_t& k : keys_) {
    state += 0x9e3779b97f4a7c15ULL;
    k = static_cast<uint32_t>(scramble(state));
  }
}

RadixTree::~RadixTree() {
  for (Node n = 1; n < capacity_; ++n) {
    if (page_[static_cast<size_t>(n)] != kNoPage) (void)pool_.drop(page_[static_cast<size_t>(n)]);
  }
}

// The NH construction of the reference's tree (csrc/radix_tree.cpp:65-87 of PrefixServe): with one secret 32-bit key
// per token position, sum over token pairs of (t[i] + k[i]) * (t[i+1] + k[i+1]), the additions wrapping at 32 bits and
// the products and the sum kept in 64; two different pages collide with probability about 2^-32 whatever the
// tokens are, because the keys are drawn from the seed and never shown.  The parent goes into the high half before
// a final scramble, so the same tokens under different parents land in unrelated slots.  An odd page length is
// padded with a zero token.
uint64_t RadixTree::edge_hash(Node parent, const int32_t* toks) const noexcept {
  uint64_t acc = 0;
  int32_t i = 0;
  for (; i + 1 < page_tokens_; i += 2) {
    const uint32_t a = static_cast<uint32_t>(toks[i]) + keys_[static_cast<size_t>(i)];
    const uint32_t b = static_cast<uint32_t>(toks[i + 1]) + keys_[static_cast<size_t>(i) + 1];
    acc += static_cast<uint64_t>(a) * static_cast<uint64_t>(b);
  }
  if (i < page_tokens_) {
    const uint32_t a = static_cast<uint32_t>(toks[i]) + keys_[static_cast<size_t>(i)];
    acc += static_cast<uint64_t>(a) * static_cast<uint64_t>(keys_[static_cast<size_t>(i) + 1]);
  }
  return scramble(acc ^ (static_cast<uint64_t>(static_cast<uint32_t>(parent)) << 32));
}

int64_t RadixTree::lookup(Node parent, const int32_t* toks, uint64_t h) const noexcept {
  const size_t bytes = static_cast<size_t>(page_tokens_) * sizeof(int32_t);
  for (size_t at = static_cast<size_t>(h) & mask_;; at = (at + 1) & mask_) {
    const Node n = slot_node_[at];
    if (n == kNone) return -1;
    if (slot_hash_[at] == h && parent_[static_cast<size_t>(n)] == parent && std::memcmp(toks_of(n), toks, bytes) == 0) {
      return static_cast<int64_t>(at);
    }
  }
}

void RadixTree::table_put(uint64_t h, Node n) noexcept {
  size_t at = static_cast<size_t>(h) & mask_;
  while (slot_node_[at] != kNone) at = (at + 1) & mask_;
  slot_node_[at] = n;
  slot_hash_[at] = h;
}

// Deletion without tombstones: pull later entries of the same probe run back
// over the gap whenever that keeps them reachable from their home slot.
void RadixTree::table_remove(size_t at) noexcept {
  size_t gap = at;
  for (size_t next = (gap + 1) & mask_; slot_node_[next] != kNone; next = (next + 1) & mask_) {
    const size_t home = static_cast<size_t>(slot_hash_[next]) & mask_;
    // distance (mod table) from home to next must be >= distance from gap to next
    const size_t d_home = (next - home) & mask_;
    const size_t d_gap = (next - gap) & mask_;
    if (d_home >= d_gap) {
      slot_node_[gap] = slot_node_[next];
      slot_hash_[gap] = slot_hash_[next];
      gap = next;
    }
  }
  slot_node_[gap] = kNone;
  slot_hash_[gap] = 0;
}

int64_t RadixTree::match_prefix(const int32_t* tokens, int64_t n, std::vector<PageId>& out) noexcept {
  out.clear();
  if (tokens == nullptr || n <= 0) return 0;
  const uint64_t now = ++clock_;
  stamp_[kRoot] = now;
  Node at = kRoot;
  const int64_t whole = n / page_tokens_;
  for (int64_t b = 0; b < whole; ++b) {
    const int32_t* toks = tokens + b * page_tokens_;
    const int64_t slot = lookup(at, toks, edge_hash(at, toks));
    if (slot < 0) break;
    const Node child = slot_node_[static_cast<size_t>(slot)];
    // The tree's own reference makes this succeed; if it ever does not, stop
    // rather than return a page the caller holds no reference on.
    if (pool_.share(page_[static_cast<size_t>(child)]) != Code::ok) break;
    out.push_back(page_[static_cast<size_t>(child)]);
    stamp_[static_cast<size_t>(child)] = now;
    at = child;
  }
  // Only leaves sit in the heap; the deepest matched node may be one and its
  // key has just grown.
  const int32_t pos = heap_at_[static_cast<size_t>(at)];
  if (pos >= 0) heap_down(static_cast<size_t>(pos));
  return static_cast<int64_t>(out.size()) * page_tokens_;
}

Code RadixTree::insert(const int32_t* tokens, int64_t n, const PageId* pages, int64_t num_pages, int32_t* added) noexcept {
  if (added) *added = 0;
  if (n < 0 || num_pages < 0 || (n > 0 && !tokens) || (num_pages > 0 && !pages)) return Code::bad_argument;
  const int64_t whole = n / page_tokens_;
  if (num_pages < whole) return Code::bad_argument;

  // 1. follow what is cached already (reads only)
  Node at = kRoot;
  int64_t depth = 0;
  while (depth < whole) {
    const int32_t* toks = tokens + depth * page_tokens_;
    const int64_t slot = lookup(at, toks, edge_hash(at, toks));
    if (slot < 0) break;
    at = slot_node_[static_cast<size_t>(slot)];
    ++depth;
  }
  const int64_t fresh = whole - depth;
  if (fresh > static_cast<int64_t>(spare_.size())) return Code::no_nodes;

  // 2. vet every page to adopt; marking as we go also catches an id given twice
  for (int64_t i = depth; i < whole; ++i) {
    const PageId id = pages[i];
    Code verdict = Code::ok;
    if (!pool_.in_range(id)) verdict = Code::bad_id;
    else if (pool_.count(id) == 0) verdict = Code::not_held;
    else if (pool_.count(id) == std::numeric_limits<int32_t>::max()) verdict = Code::count_overflow;
    else if (owned_[static_cast<size_t>(id)]) verdict = Code::already_cached;
    if (verdict != Code::ok) {
      for (int64_t j = depth; j < i; ++j) owned_[static_cast<size_t>(pages[j])] = 0;
      return verdict;
    }
    owned_[static_cast<size_t>(id)] = 1;
  }

  // 3. commit; nothing below fails
  const uint64_t now = ++clock_;
  if (fresh > 0 && heap_at_[static_cast<size_t>(at)] >= 0) heap_drop(at);  // gains a child
  for (Node up = at; up != kNone; up = parent_[static_cast<size_t>(up)]) stamp_[static_cast<size_t>(up)] = now;
  if (fresh == 0) {
    const int32_t pos = heap_at_[static_cast<size_t>(at)];
    if (pos >= 0) heap_down(static_cast<size_t>(pos));
    return Code::ok;
  }
  for (int64_t i = depth; i < whole; ++i) {
    const Node child = spare_.back();
    spare_.pop_back();
    const int32_t* toks = tokens + i * page_tokens_;
    const size_t c = static_cast<size_t>(child);
    parent_[c] = at;
    page_[c] = pages[i];
    kids_[c] = 0;
    heap_at_[c] = -1;
    stamp_[c] = now;
    hash_[c] = edge_hash(at, toks);
    std::memcpy(&tokens_[c * static_cast<size_t>(page_tokens_)], toks, static_cast<size_t>(page_tokens_) * sizeof(int32_t));
    table_put(hash_[c], child);
    ++kids_[static_cast<size_t>(at)];
    (void)pool_.share(pages[i]);
    at = child;
  }
  heap_add(at);  // the deepest new node is the only new leaf
  if (added) *added = static_cast<int32_t>(fresh);
  return Code::ok;
}

int32_t RadixTree::evict(int32_t want) noexcept {
  int32_t freed = 0;
  held_back_.clear();
  while (freed < want && !heap_.empty()) {
    const Node leaf = heap_.front();
    heap_drop(leaf);
    if (pool_.count(page_[static_cast<size_t>(leaf)]) > 1) {  // a request still uses it
      held_back_.push_back(leaf);
      continue;
    }
    unlink_leaf(leaf);
    ++freed;
  }
  for (Node n : held_back_) heap_add(n);
  held_back_.clear();
  return freed;
}

void RadixTree::unlink_leaf(Node leaf) noexcept {
  const size_t l = static_cast<size_t>(leaf);
  const Node up = parent_[l];
  const int64_t slot = lookup(up, toks_of(leaf), hash_[l]);
  if (slot >= 0) table_remove(static_cast<size_t>(slot));
  owned_[static_cast<size_t>(page_[l])] = 0;
  (void)pool_.drop(page_[l]);
  parent_[l] = kNone;
  page_[l] = kNoPage;
  kids_[l] = 0;
  stamp_[l] = 0;
  spare_.push_back(leaf);
  if (--kids_[static_cast<size_t>(up)] == 0 && up != kRoot) heap_add(up);
}

void RadixTree::heap_up(size_t at) noexcept {
  const Node n = heap_[at];
  while (at > 0) {
    const size_t up = (at - 1) / 2;
    if (!older(n, heap_[up])) break;
    heap_set(at, heap_[up]);
    at = up;
  }
  heap_set(at, n);
}

void RadixTree::heap_down(size_t at) noexcept {
  const Node n = heap_[at];
  const size_t size = heap_.size();
  for (;;) {
    size_t kid = 2 * at + 1;
    if (kid >= size) break;
    if (kid + 1 < size && older(heap_[kid + 1], heap_[kid])) ++kid;
    if (!older(heap_[kid], n)) break;
    heap_set(at, heap_[kid]);
    at = kid;
  }
  heap_set(at, n);
}

void RadixTree::heap_add(Node n) noexcept {
  heap_.push_back(n);
  heap_at_[static_cast<size_t>(n)] = static_cast<int32_t>(heap_.size() - 1);
  heap_up(heap_.size() - 1);
}

void RadixTree::heap_drop(Node n) noexcept {
  const size_t at = static_cast<size_t>(heap_at_[static_cast<size_t>(n)]);
  const Node last = heap_.back();
  heap_.pop_back();
  heap_at_[static_cast<size_t>(n)] = -1;
  if (last == n) return;
  heap_set(at, last);
  heap_up(at);
  heap_down(static_cast<size_t>(heap_at_[static_cast<size_t>(last)]));
}

bool RadixTree::consistent(std::string* why) const {
  auto fail = [&](std::string m) {
    if (why) *why = std::move(m);
    return false;
  };
  const size_t cap = static_cast<size_t>(capacity_);
  std::vector<int32_t> kid_count(cap, 0);
  std::vector<uint8_t> page_seen(static_cast<size_t>(pool_.num_blocks()), 0);
  std::vector<uint8_t> is_spare(cap, 0);
  for (Node n : spare_) {
    if (n < 1 || n >= capacity_) return fail("spare list holds a bad node id");
    if (is_spare[static_cast<size_t>(n)]++) return fail("node is on the spare list twice");
    if (page_[static_cast<size_t>(n)] != kNoPage) return fail("spare node owns a page");
  }
  int32_t live = 0;
  for (Node n = 1; n < capacity_; ++n) {
    const size_t i = static_cast<size_t>(n);
    if (is_spare[i]) continue;
    ++live;
    const PageId p = page_[i];
    if (!pool_.in_range(p)) return fail("live node owns no valid page");
    if (page_seen[static_cast<size_t>(p)]++) return fail("page " + std::to_string(p) + " is owned by two nodes");
    if (!owned_[static_cast<size_t>(p)]) return fail("owned flag missing for page " + std::to_string(p));
    if (pool_.count(p) < 1) return fail("cached page " + std::to_string(p) + " has no reference");
    const Node up = parent_[i];
    if (up < 0 || up >= capacity_ || (up != kRoot && is_spare[static_cast<size_t>(up)])) return fail("node has a dead parent");
    ++kid_count[static_cast<size_t>(up)];
    if (stamp_[static_cast<size_t>(up)] < stamp_[i]) return fail("parent was touched before its child");
    if (lookup(up, toks_of(n), hash_[i]) < 0) return fail("node is not reachable through the hash table");
    if (hash_[i] != edge_hash(up, toks_of(n))) return fail("stored hash is stale");
  }
  for (size_t p = 0; p < page_seen.size(); ++p) {
    if (owned_[p] && !page_seen[p]) return fail("owned flag set for a page no node owns");
  }
  if (live != num_cached_blocks()) return fail("node count mismatch");
  size_t filled = 0;
  for (Node n : slot_node_) filled += n != kNone;
  if (filled != static_cast<size_t>(live)) return fail("hash table holds " + std::to_string(filled) + " entries for " + std::to_string(live) + " nodes");
  for (Node n = 0; n < capacity_; ++n) {
    const size_t i = static_cast<size_t>(n);
    if (n != kRoot && is_spare[i]) {
      if (heap_at_[i] != -1) return fail("spare node is in the heap");
      continue;
    }
    if (kids_[i] != kid_count[i]) return fail("child count mismatch at node " + std::to_string(n));
    const bool leaf = n != kRoot && kids_[i] == 0;
    if (leaf != (heap_at_[i] >= 0)) return fail("leaf/heap mismatch at node " + std::to_string(n));
    if (heap_at_[i] >= 0 && (static_cast<size_t>(heap_at_[i]) >= heap_.size() || heap_[static_cast<size_t>(heap_at_[i])] != n)) {
      return fail("heap position is stale");
    }
  }
  for (size_t at = 1; at < heap_.size(); ++at) {
    if (older(heap_[at], heap_[(at - 1) / 2])) return fail("heap order broken");
  }
  return true;
}

}  // namespace psb200
